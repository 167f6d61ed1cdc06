"""Sliding-window branch of the NSA layer: causal varlen GQA attention where query t sees keys t - window_size .. t.

The reference has no operator of its own for this branch: its layer calls the third-party
flash_attn.flash_attn_varlen_func(..., causal=True, window_size=(window_size, -1))
(native_sparse_attention/module/native_sparse_attention.py:213-223), which this function replaces with the same
tcgen05 kernels as flash_attention_varlen plus a lower bound on the visible keys.  head_dim 128 only.
"""
from typing import Optional

import torch

from .. import _lib
from ._common import default_scale, dtype_code, inner_contiguous, ptr, require_cuda, stream_ptr
from .attention_bwd import _workspace


class SlidingWindowAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, window_size, sm_scale):
        q, k, v = inner_contiguous(q), inner_contiguous(k), inner_contiguous(v)
        total, num_q_heads, head_dim = q.shape
        num_kv_heads = k.shape[1]
        batch = cu_seqlens.shape[0] - 1
        o = torch.empty_like(q)
        lse = torch.empty(total, num_q_heads, dtype=torch.float32, device=q.device)
        strides = _lib.strides_array(q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                                     o.stride(0), o.stride(1))
        torch.cuda.set_device(q.device)
        rc = _lib.lib().nsa_window_attn_fwd(ptr(q), ptr(k), ptr(v), ptr(cu_seqlens), ptr(o), ptr(lse), total, batch,
                                            int(max_seqlen), num_q_heads, num_kv_heads, head_dim, int(window_size), strides,
                                            float(sm_scale), dtype_code(q), stream_ptr(q.device))
        _lib.check(rc, "nsa_window_attn_fwd")
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens)
        ctx.meta = (sm_scale, max_seqlen, window_size)
        return o

    @staticmethod
    def backward(ctx, do, *args):
        q, k, v, o, lse, cu_seqlens = ctx.saved_tensors
        sm_scale, max_seqlen, window_size = ctx.meta
        total, num_q_heads, head_dim = q.shape
        num_kv_heads = k.shape[1]
        batch = cu_seqlens.shape[0] - 1
        do = inner_contiguous(do)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        lib = _lib.lib()
        nbytes = lib.nsa_varlen_attn_bwd_workspace(total, total, num_q_heads, num_kv_heads, head_dim)
        ws = _workspace(nbytes, q.device)
        strides = _lib.strides_array(q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                                     o.stride(0), o.stride(1), do.stride(0), do.stride(1), dq.stride(0), dq.stride(1),
                                     dk.stride(0), dk.stride(1), dv.stride(0), dv.stride(1))
        torch.cuda.set_device(q.device)
        rc = lib.nsa_window_attn_bwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(cu_seqlens), ptr(dq), ptr(dk),
                                     ptr(dv), ptr(ws), nbytes, total, batch, int(max_seqlen), num_q_heads, num_kv_heads,
                                     head_dim, int(window_size), strides, float(sm_scale), dtype_code(q), stream_ptr(q.device))
        _lib.check(rc, "nsa_window_attn_bwd")
        return dq, dk, dv, None, None, None, None


def sliding_window_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
                             window_size: int, sm_scale: Optional[float] = None) -> torch.Tensor:
    """q [total, Hq, d], k/v [total, Hkv, d] (self-attention: one cu_seqlens); key j is visible to query i of the same
    sequence iff i - window_size <= j <= i, i.e. window_size + 1 keys, as flash_attn's window_size=(window_size, -1) with
    causal=True gives."""
    require_cuda(q, k, v, cu_seqlens)
    assert q.dtype == torch.bfloat16 or q.dtype == torch.float16
    assert k.dtype == q.dtype and v.dtype == q.dtype
    assert cu_seqlens.dtype == torch.int32
    assert q.shape[0] == k.shape[0] == v.shape[0] and q.shape[1] % k.shape[1] == 0 and k.shape[1] == v.shape[1]
    assert q.shape[-1] == 128, "sliding_window_attention supports head_dim 128"
    assert window_size >= 0
    if sm_scale is None:
        sm_scale = default_scale(q.shape[-1])
    return SlidingWindowAttention.apply(q, k, v, cu_seqlens, int(max_seqlen), int(window_size), float(sm_scale))
