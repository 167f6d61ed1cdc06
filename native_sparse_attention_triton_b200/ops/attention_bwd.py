"""Backward drivers of the two trainable attention operators: allocate outputs and scratch, call the C ABI."""
import torch

from .. import _lib
from ._common import dtype_code, inner_contiguous, ptr, stream_ptr


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


def dense_attention_backward(q, k, v, o, lse, do, cu_q, cu_k, max_seqlen_q, max_seqlen_k, causal, window, stride, sm_scale):
    total_q, num_q_heads, head_dim = q.shape
    total_k, num_kv_heads, _ = k.shape
    batch = cu_q.shape[0] - 1
    dq = torch.empty(total_q, num_q_heads, head_dim, dtype=q.dtype, device=q.device)
    dk = torch.empty(total_k, num_kv_heads, head_dim, dtype=q.dtype, device=q.device)
    dv = torch.empty(total_k, num_kv_heads, head_dim, dtype=q.dtype, device=q.device)
    if total_k == 0:
        return dq.zero_(), dk, dv
    do = inner_contiguous(do)
    lib = _lib.lib()
    nbytes = lib.nsa_varlen_attn_bwd_workspace(total_q, total_k, num_q_heads, num_kv_heads, head_dim)
    ws = _workspace(nbytes, q.device)
    strides = _lib.strides_array(q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                                 o.stride(0), o.stride(1), do.stride(0), do.stride(1), dq.stride(0), dq.stride(1),
                                 dk.stride(0), dk.stride(1), dv.stride(0), dv.stride(1))
    torch.cuda.set_device(q.device)
    rc = lib.nsa_varlen_attn_bwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(cu_q), ptr(cu_k), ptr(dq), ptr(dk),
                                 ptr(dv), ptr(ws), nbytes, total_q, total_k, batch, int(max_seqlen_q), int(max_seqlen_k),
                                 num_q_heads, num_kv_heads, head_dim, int(bool(causal)), int(window), int(stride), strides,
                                 float(sm_scale), dtype_code(q), stream_ptr(q.device))
    _lib.check(rc, "nsa_varlen_attn_bwd")
    return dq, dk, dv


def sparse_attention_backward(q, k, v, o, lse, do, topk_idx, block_size, cu_seqlens, sm_scale):
    total_len, num_q_heads, head_dim = q.shape
    num_kv_heads = k.shape[1]
    batch = cu_seqlens.shape[0] - 1
    topk = topk_idx.shape[-1]
    dq = torch.empty(total_len, num_q_heads, head_dim, dtype=q.dtype, device=q.device)
    dk = torch.empty(total_len, num_kv_heads, head_dim, dtype=q.dtype, device=q.device)
    dv = torch.empty(total_len, num_kv_heads, head_dim, dtype=q.dtype, device=q.device)
    do = inner_contiguous(do)
    # prefix sum of blocks per sequence, on the device (no host sync)
    seqlens = cu_seqlens[1:] - cu_seqlens[:-1]
    cu_blocks = torch.zeros(batch + 1, dtype=torch.int32, device=q.device)
    cu_blocks[1:] = torch.cumsum((seqlens + block_size - 1) // block_size, 0)
    lib = _lib.lib()
    nbytes = lib.nsa_topk_sparse_attn_bwd_workspace(total_len, batch, num_q_heads, num_kv_heads, head_dim, topk, block_size)
    ws = _workspace(nbytes, q.device)
    strides = _lib.strides_array(q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                                 o.stride(0), o.stride(1), do.stride(0), do.stride(1), dq.stride(0), dq.stride(1),
                                 dk.stride(0), dk.stride(1), dv.stride(0), dv.stride(1), *topk_idx.stride())
    torch.cuda.set_device(q.device)
    rc = lib.nsa_topk_sparse_attn_bwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(topk_idx), ptr(cu_seqlens),
                                      ptr(cu_blocks), ptr(dq), ptr(dk), ptr(dv), ptr(ws), nbytes, total_len, batch,
                                      num_q_heads, num_kv_heads, head_dim, topk, int(block_size), strides, float(sm_scale),
                                      dtype_code(q), stream_ptr(q.device))
    _lib.check(rc, "nsa_topk_sparse_attn_bwd")
    return dq, dk, dv
