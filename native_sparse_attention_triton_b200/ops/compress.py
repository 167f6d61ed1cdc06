"""Key/value compression operators: linear projection, weighted pooling, average pooling.

Signatures, argument meaning and assertion behaviour follow the reference's
native_sparse_attention/ops/triton/linear_compress.py:497-525 and
native_sparse_attention/ops/triton/weighted_pool.py:301-363.  Unlike the reference the
position-embedding bias is folded into the kernel epilogue and its gradient is produced by the same
backward pass.
"""
from typing import Optional, Tuple

import torch

from .. import _lib
from ._common import (compressed_lens, cumsum_tensor, dtype_code, host_seqlens, inner_contiguous, ptr, require_cuda,
                      stream_ptr)

_KERNEL_SIZES = {16, 32, 64, 128}


_layout_cache = {}   # (id(cu_seqlens), kernel_size, kernel_stride) -> (host list it was derived from, y_lens, y_cu, y_cu version)


def _compressed_layout(cu_seqlens, cu, kernel_size, kernel_stride, device):
    """(compressed lengths, their device prefix sum) for a cu_seqlens tensor; remembered per (tensor object, kernel) so
    that repeated calls with the same tensor upload nothing.  `cu` is the host copy host_seqlens returned for it: the
    entry is valid only while that very list is still the cached copy (same object, not written to since)."""
    key = (id(cu_seqlens), kernel_size, kernel_stride)
    hit = _layout_cache.get(key)
    if hit is not None and hit[0] is cu and hit[2]._version == hit[3] and hit[2].device == device:
        return hit[1], hit[2]
    y_lens = compressed_lens(cu, kernel_size, kernel_stride)
    y_cu = cumsum_tensor(y_lens, device)
    if len(_layout_cache) > 64:
        _layout_cache.clear()
    _layout_cache[key] = (cu, y_lens, y_cu, y_cu._version)
    return y_lens, y_cu


class _Compress(torch.autograd.Function):
    """mode: 'linear' | 'weighted' | 'avg'."""

    @staticmethod
    def forward(ctx, x, w, pe, cu_seqlens, kernel_size, kernel_stride, mode):
        require_cuda(x, w, pe, cu_seqlens)
        total_len, num_heads, head_dim = x.shape
        x = inner_contiguous(x)
        cu = host_seqlens(cu_seqlens)
        batch = len(cu) - 1
        y_lens, y_cu = _compressed_layout(cu_seqlens, cu, kernel_size, kernel_stride, x.device)
        total_y, max_y = sum(y_lens), max(y_lens) if y_lens else 0
        y = torch.empty(total_y, num_heads, head_dim, dtype=x.dtype, device=x.device)
        bias = torch.empty(num_heads, head_dim, dtype=x.dtype, device=x.device) if pe is not None else None
        wc = w.contiguous() if w is not None else None
        pec = pe.contiguous() if pe is not None else None
        lib = _lib.lib()
        torch.cuda.set_device(x.device)
        if mode == "linear":
            rc = lib.nsa_linear_compress_fwd(ptr(x), ptr(wc), ptr(pec), ptr(cu_seqlens), ptr(y_cu), ptr(y), ptr(bias),
                                             x.shape[0], batch, total_y, max_y, num_heads, head_dim, kernel_size, kernel_stride,
                                             x.stride(0), x.stride(1), dtype_code(x), stream_ptr(x.device))
            _lib.check(rc, "nsa_linear_compress_fwd")
        else:
            rc = lib.nsa_pool_compress_fwd(ptr(x), ptr(wc), ptr(pec), ptr(cu_seqlens), ptr(y_cu), ptr(y), ptr(bias),
                                           x.shape[0], batch, total_y, max_y, num_heads, head_dim, kernel_size, kernel_stride,
                                           x.stride(0), x.stride(1), dtype_code(x), stream_ptr(x.device))
            _lib.check(rc, "nsa_pool_compress_fwd")
        ctx.save_for_backward(x, wc, pec, cu_seqlens, y_cu)
        ctx.meta = (kernel_size, kernel_stride, mode, batch, total_y, max_y, max(cu[i + 1] - cu[i] for i in range(batch)))
        ctx.mark_non_differentiable(y_cu)
        return y, y_cu

    @staticmethod
    def backward(ctx, dy, _):
        from .compress_bwd import compress_backward
        return compress_backward(ctx, dy)


def _check_common(x, cu_seqlens, kernel_size, kernel_stride, pe):
    assert x.dtype == torch.float16 or x.dtype == torch.bfloat16
    assert cu_seqlens.dtype == torch.int32
    assert kernel_size % kernel_stride == 0
    assert kernel_size in _KERNEL_SIZES
    if pe is not None:
        assert pe.dtype == x.dtype and pe.device == x.device
        assert tuple(pe.shape) == (x.shape[1], kernel_size, x.shape[2])


def linear_compress(x: torch.Tensor, w: torch.Tensor, cu_seqlens: torch.Tensor, kernel_size: int, kernel_stride: int,
                    pe: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Compress keys/values with a per-head linear projection of each window.

    Args:
        x: [total_len, num_heads, head_dim]
        w: [num_heads, kernel_size * head_dim, head_dim]
        cu_seqlens: int32 [batch + 1]
        kernel_size / kernel_stride: window length and hop
        pe: optional intra-block position embedding [num_heads, kernel_size, head_dim]
    Returns:
        (compressed [total_compressed, num_heads, head_dim], y_cu_seqlens int32 [batch + 1])
    """
    _check_common(x, cu_seqlens, kernel_size, kernel_stride, pe)
    assert x.dtype == w.dtype
    total_len, num_heads, head_dim = x.shape
    assert w.shape[0] == num_heads and w.shape[1] == kernel_size * head_dim and w.shape[2] == head_dim
    assert head_dim % 8 == 0
    return _Compress.apply(x, w, pe, cu_seqlens, kernel_size, kernel_stride, "linear")


def weightedpool_compress(x: torch.Tensor, w: torch.Tensor, cu_seqlens: torch.Tensor, kernel_size: int,
                          kernel_stride: int, pe: Optional[torch.Tensor] = None):
    """Compress keys/values with a per-head weighted sum over each window; w is [num_heads, kernel_size]."""
    _check_common(x, cu_seqlens, kernel_size, kernel_stride, pe)
    assert x.dtype == w.dtype
    assert w.shape[0] == x.shape[1] and w.shape[1] == kernel_size
    return _Compress.apply(x, w, pe, cu_seqlens, kernel_size, kernel_stride, "weighted")


def avgpool_compress(x: torch.Tensor, w, cu_seqlens: torch.Tensor, kernel_size: int, kernel_stride: int,
                     pe: Optional[torch.Tensor] = None):
    """Compress keys/values with the mean of each window; w must be None."""
    assert w is None, "don't need additional weight for avgpool"
    _check_common(x, cu_seqlens, kernel_size, kernel_stride, pe)
    return _Compress.apply(x, None, pe, cu_seqlens, kernel_size, kernel_stride, "avg")
