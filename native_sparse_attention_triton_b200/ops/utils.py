"""Sequence-length helper with the reference's name and return convention."""
import torch


def get_compressed_seqlens(cu_seqlens: torch.Tensor, kernel_size: int, kernel_stride: int):
    """(y_seqlens, y_cu_seqlens), both int32 on cu_seqlens' device.

    Same contract as native_sparse_attention/ops/triton/utils.py:25-37 of the reference: a sequence
    shorter than kernel_size has no compressed token.
    """
    seqlens = cu_seqlens[1:] - cu_seqlens[:-1]
    y_seqlens = torch.div(seqlens - kernel_size, kernel_stride, rounding_mode="floor").to(torch.int32) + 1
    y_seqlens = torch.where(seqlens < kernel_size, torch.zeros_like(y_seqlens), y_seqlens)
    y_cu_seqlens = torch.zeros(y_seqlens.shape[0] + 1, dtype=torch.int32, device=cu_seqlens.device)
    y_cu_seqlens[1:] = torch.cumsum(y_seqlens, dim=0)
    return y_seqlens, y_cu_seqlens
