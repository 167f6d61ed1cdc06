"""Backward of the compression operators (called from the autograd Function in compress.py)."""
import torch

from .. import _lib
from ._common import dtype_code, ptr, stream_ptr


def compress_backward(ctx, dy):
    x, w, pe, cu_seqlens, y_cu = ctx.saved_tensors
    kernel_size, kernel_stride, mode, batch, total_y, max_y, max_len = ctx.meta
    total_len, num_heads, head_dim = x.shape
    dy = dy.contiguous()
    dx = torch.empty(total_len, num_heads, head_dim, dtype=x.dtype, device=x.device)
    dpe = torch.empty_like(pe) if pe is not None else None
    dbias = torch.empty(num_heads, head_dim, dtype=torch.float32, device=x.device) if pe is not None else None
    lib = _lib.lib()
    torch.cuda.set_device(x.device)
    if mode == "linear":
        dw = torch.empty_like(w)
        rc = lib.nsa_linear_compress_bwd(ptr(x), ptr(w), ptr(pe), ptr(dy), ptr(cu_seqlens), ptr(y_cu), ptr(dx), ptr(dw),
                                         ptr(dpe), ptr(dbias), total_len, batch, total_y, max_len, num_heads, head_dim,
                                         kernel_size, kernel_stride, x.stride(0), x.stride(1), dtype_code(x),
                                         stream_ptr(x.device))
        _lib.check(rc, "nsa_linear_compress_bwd")
    else:
        dw = torch.empty_like(w) if w is not None else None
        n_ws = lib.nsa_pool_compress_bwd_workspace_floats(total_len, batch, max_len, num_heads, head_dim, kernel_size, kernel_stride)
        ws = torch.empty(n_ws, dtype=torch.float32, device=x.device)   # column sums of dy, then the partial rows of dw
        rc = lib.nsa_pool_compress_bwd(ptr(x), ptr(w), ptr(pe), ptr(dy), ptr(cu_seqlens), ptr(y_cu), ptr(dx), ptr(dw),
                                       ptr(dpe), ptr(ws), n_ws, total_len, batch, total_y, max_len, num_heads, head_dim,
                                       kernel_size, kernel_stride, x.stride(0), x.stride(1), dtype_code(x),
                                       stream_ptr(x.device))
        _lib.check(rc, "nsa_pool_compress_bwd")
    # gradients for (x, w, pe, cu_seqlens, kernel_size, kernel_stride, mode)
    return dx, dw, dpe, None, None, None, None
