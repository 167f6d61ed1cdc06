"""Dense varlen attention (flash_attention_varlen) on the shared strided-causal kernel.

Signature follows native_sparse_attention/ops/triton/flash_attention.py:895-935 of the reference.
`gqa_interleave=True` is rejected: the reference's forward and backward disagree on that head mapping.
"""
from typing import Optional

import torch

from ._common import default_scale, inner_contiguous, require_cuda
from .dense_attention import varlen_attention_backward, varlen_attention_forward


class FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal, sm_scale):
        q, k, v = inner_contiguous(q), inner_contiguous(k), inner_contiguous(v)
        o, lse = varlen_attention_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, causal, 1, 1, sm_scale)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens_q, cu_seqlens_k)
        ctx.meta = (sm_scale, max_seqlen_q, max_seqlen_k, causal)
        return o

    @staticmethod
    def backward(ctx, do, *args):
        q, k, v, o, lse, cu_q, cu_k = ctx.saved_tensors
        sm_scale, max_q, max_k, causal = ctx.meta
        dq, dk, dv = varlen_attention_backward(q, k, v, o, lse, do, cu_q, cu_k, max_q, max_k, causal, 1, 1, sm_scale)
        return dq, dk, dv, None, None, None, None, None, None


def flash_attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                           cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, causal: bool = False,
                           sm_scale: Optional[float] = None, gqa_interleave: bool = False) -> torch.Tensor:
    """Varlen GQA attention; causal means key j is visible to query i iff j <= i within a sequence."""
    require_cuda(q, k, v, cu_seqlens_q, cu_seqlens_k)
    assert q.dtype == torch.bfloat16 or q.dtype == torch.float16
    assert k.dtype == q.dtype and v.dtype == q.dtype
    assert cu_seqlens_q.dtype == torch.int32 and cu_seqlens_k.dtype == torch.int32
    assert q.shape[1] % k.shape[1] == 0 and k.shape[1] == v.shape[1]
    if gqa_interleave:
        raise NotImplementedError("gqa_interleave=True is not supported")
    if sm_scale is None:
        sm_scale = default_scale(q.shape[-1])
    return FlashAttention.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q), int(max_seqlen_k), bool(causal),
                                float(sm_scale))
