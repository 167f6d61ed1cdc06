"""Attention over the KV blocks selected per query token (topk_sparse_attention).

Signature follows native_sparse_attention/ops/triton/topk_sparse_attention.py:1182-1217 of the reference.
"""
from typing import Optional

import torch

from .. import _lib
from ._common import default_scale, dtype_code, inner_contiguous, ptr, require_cuda, stream_ptr


def sparse_attention_forward(q, k, v, topk_idx, block_size, cu_seqlens, sm_scale):
    total_len, num_q_heads, head_dim = q.shape
    num_kv_heads = k.shape[1]
    batch = cu_seqlens.shape[0] - 1
    o = torch.empty(total_len, num_q_heads, head_dim, dtype=q.dtype, device=q.device)
    lse = torch.empty(total_len, num_q_heads, dtype=torch.float32, device=q.device)
    strides = _lib.strides_array(q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                                 o.stride(0), o.stride(1), *topk_idx.stride())
    torch.cuda.set_device(q.device)
    rc = _lib.lib().nsa_topk_sparse_attn_fwd(ptr(q), ptr(k), ptr(v), ptr(topk_idx), ptr(cu_seqlens), ptr(o), ptr(lse),
                                             total_len, batch, num_q_heads, num_kv_heads, head_dim, topk_idx.shape[-1],
                                             int(block_size), strides, float(sm_scale), dtype_code(q),
                                             stream_ptr(q.device))
    _lib.check(rc, "nsa_topk_sparse_attn_fwd")
    return o, lse


class TopkSparseAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, topk_idx, block_size, cu_seqlens, sm_scale):
        assert q.dtype == torch.bfloat16 or q.dtype == torch.float16
        assert q.dtype == k.dtype and k.dtype == v.dtype
        assert topk_idx.dtype == torch.int32
        assert cu_seqlens.dtype == torch.int32
        if sm_scale is None:
            sm_scale = default_scale(q.shape[-1])
        q, k, v = inner_contiguous(q), inner_contiguous(k), inner_contiguous(v)
        o, lse = sparse_attention_forward(q, k, v, topk_idx, block_size, cu_seqlens, sm_scale)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens, topk_idx)
        ctx.meta = (sm_scale, block_size)
        return o

    @staticmethod
    def backward(ctx, do, *args):
        from .attention_bwd import sparse_attention_backward
        q, k, v, o, lse, cu_seqlens, topk_idx = ctx.saved_tensors
        sm_scale, block_size = ctx.meta
        dq, dk, dv = sparse_attention_backward(q, k, v, o, lse, do, topk_idx, block_size, cu_seqlens, sm_scale)
        return dq, dk, dv, None, None, None, None


def topk_sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, topk_idx: torch.Tensor, block_size: int,
                          cu_seqlens: torch.Tensor, softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Each query attends, causally, to the keys of its selected blocks.

    Args:
        q: [total_len, num_q_heads, head_dim]
        k, v: [total_len, num_kv_heads, head_dim]
        topk_idx: int32 [num_kv_heads, total_len, topk], valid block ids first, -1 padding
        block_size: keys per block (multiple of 64)
        cu_seqlens: int32 [batch + 1]
        softmax_scale: default 1/sqrt(head_dim)
    Returns:
        attention output [total_len, num_q_heads, head_dim]
    """
    require_cuda(q, k, v, topk_idx, cu_seqlens)
    assert block_size in {32, 64, 128, 256}
    if block_size == 32:
        raise NotImplementedError("block_size 32 is not built: the kernels work on 64-key tiles (use 64, 128 or 256)")
    if topk_idx.shape[-1] * (block_size // 64) > 64:
        raise NotImplementedError("at most 64 tiles of 64 keys per query (topk * block_size / 64 <= 64)")
    assert q.shape[1] % k.shape[1] == 0 and k.shape[1] == v.shape[1] and k.shape[1] == topk_idx.shape[0]
    return TopkSparseAttention.apply(q, k, v, topk_idx, block_size, cu_seqlens, softmax_scale)
