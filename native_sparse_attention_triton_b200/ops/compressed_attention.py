"""Attention between queries and compressed keys/values, plus top-k block selection.

Signature and semantics follow native_sparse_attention/ops/triton/compressed_attention.py:1182-1331
of the reference.  The block scores are never materialised: one kernel recomputes QK^T against the
final log-sum-exp, reduces over the query heads of each KV group and selects in shared memory.
"""
import warnings
from typing import Tuple, Union

import torch

from .. import _lib
from ._common import default_scale, dtype_code, host_seqlens, inner_contiguous, ptr, require_cuda, stream_ptr
from .dense_attention import varlen_attention_backward, varlen_attention_forward


class CompressedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, kernel_size, kernel_stride, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, sm_scale):
        assert q.dtype == torch.bfloat16 or q.dtype == torch.float16
        assert q.dtype == k.dtype and k.dtype == v.dtype
        assert cu_seqlens_q.dtype == torch.int32 and cu_seqlens_k.dtype == torch.int32
        if sm_scale is None:
            sm_scale = default_scale(q.shape[-1])
        q, k, v = inner_contiguous(q), inner_contiguous(k), inner_contiguous(v)
        o, lse = varlen_attention_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, True, kernel_size,
                                          kernel_stride, sm_scale)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens_q, cu_seqlens_k)
        ctx.meta = (sm_scale, max_seqlen_q, max_seqlen_k, kernel_size, kernel_stride)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, *args):
        q, k, v, o, lse, cu_q, cu_k = ctx.saved_tensors
        sm_scale, max_q, max_k, kernel_size, kernel_stride = ctx.meta
        dq, dk, dv = varlen_attention_backward(q, k, v, o, lse, do, cu_q, cu_k, max_q, max_k, True, kernel_size,
                                               kernel_stride, sm_scale)
        return dq, dk, dv, None, None, None, None, None, None, None


def select_topk_blocks(q, k, lse, kernel_size, kernel_stride, block_size, topk, cu_seqlens_q, cu_seqlens_k,
                       max_seqlen_q, sm_scale, init_blocks, local_blocks) -> torch.Tensor:
    """topk_idx int32 [num_kv_heads, total_q, min(topk, ceil(max_seqlen_q / block_size))]."""
    total_q, num_q_heads, head_dim = q.shape
    total_k, num_kv_heads, _ = k.shape
    batch = cu_seqlens_q.shape[0] - 1
    max_blocks = (max_seqlen_q + block_size - 1) // block_size
    t_out = min(topk, max_blocks)
    topk_idx = torch.empty(num_kv_heads, total_q, t_out, dtype=torch.int32, device=q.device)
    strides = _lib.strides_array(q.stride(0), q.stride(1), k.stride(0), k.stride(1), *topk_idx.stride())
    rc = _lib.lib().nsa_compressed_attn_topk(
        ptr(q), ptr(k), ptr(lse), ptr(cu_seqlens_q), ptr(cu_seqlens_k), ptr(topk_idx), total_q, total_k, batch,
        max_seqlen_q, num_q_heads, num_kv_heads, head_dim, kernel_size, kernel_stride, block_size, topk, init_blocks,
        local_blocks, strides, sm_scale, dtype_code(q), stream_ptr(q.device))
    _lib.check(rc, "nsa_compressed_attn_topk")
    return topk_idx


def compressed_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    kernel_size: int,
    kernel_stride: int,
    block_size: int,
    topk: int,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int = None,
    max_seqlen_k: int = None,
    sm_scale: float = None,
    init_blocks: int = 1,
    local_blocks: int = 2,
    parallel_topk_compute: Union[str, bool] = "auto",
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention output over compressed K/V and the block ids each query keeps for sparse attention.

    Args:
        q: [total_q_len, num_q_heads, head_dim]
        k, v: [total_kv_len, num_kv_heads, head_dim] (compressed)
        kernel_size, kernel_stride: the compression window and hop that produced k, v
        block_size: selection block size of topk_sparse_attention
        topk: blocks kept per query (<= 0: no selection, topk_idx is None)
        cu_seqlens_q, cu_seqlens_k: int32 [batch + 1]
        max_seqlen_q, max_seqlen_k: optional maxima (computed with one host sync when None)
        sm_scale: softmax scale, default 1/sqrt(head_dim)
        init_blocks, local_blocks: always-selected leading blocks / trailing blocks ending at the query's own
        parallel_topk_compute: accepted for compatibility; selection never materialises scores here
    Returns:
        (attention output like q, topk_idx int32 [num_kv_heads, total_q_len, min(topk, num_blocks)])
    """
    require_cuda(q, k, v, cu_seqlens_q, cu_seqlens_k)
    if max_seqlen_q is None:
        cq = host_seqlens(cu_seqlens_q)
        max_seqlen_q = max(cq[i + 1] - cq[i] for i in range(len(cq) - 1))
    if max_seqlen_k is None:
        ck = host_seqlens(cu_seqlens_k)
        max_seqlen_k = max(ck[i + 1] - ck[i] for i in range(len(ck) - 1))
    max_seqlen_q, max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    assert k.shape[0] == v.shape[0] and q.shape[0] > k.shape[0]
    assert k.shape[1] == v.shape[1] and q.shape[1] % k.shape[1] == 0
    attn_output, lse = CompressedAttention.apply(q, k, v, kernel_size, kernel_stride, cu_seqlens_q, cu_seqlens_k,
                                                 max_seqlen_q, max_seqlen_k, sm_scale)
    if topk <= 0:
        warnings.warn("topk <= 0, returned topk_idx will be None")
        return attn_output, None
    assert topk >= init_blocks + local_blocks
    assert block_size % kernel_stride == 0 and kernel_size % kernel_stride == 0
    with torch.no_grad():
        if sm_scale is None:
            sm_scale = default_scale(q.shape[-1])
        if k.shape[0] == 0:
            # no compressed key anywhere: scores are all zero, only forced blocks and the lowest ids are taken
            k = torch.zeros(1, k.shape[1], k.shape[2], dtype=q.dtype, device=q.device)
        topk_idx = select_topk_blocks(inner_contiguous(q.detach()), inner_contiguous(k.detach()), lse, kernel_size,
                                      kernel_stride, block_size, topk, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                                      sm_scale, init_blocks, local_blocks)
    return attn_output, topk_idx
