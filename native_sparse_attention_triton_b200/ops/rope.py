"""Rotary position embedding of a varlen batch in one kernel (forward and backward).

Mirrors ``RotaryEmbedding.forward(x, cu_seqlens, step=0, stride=1)`` of the reference
(native_sparse_attention/module/rope.py:197-209): ``x * cos + rotate_half(x) * sin`` with the position of every row
derived from ``cu_seqlens`` -- token t of its sequence at ``t * stride`` when ``step == 0``, row b of a decode step at
``(seqlen_b + step - 1) * stride`` otherwise (:158-195).  The frequencies stay the caller's: ``inv_freq`` and
``attention_scaling`` are what the reference obtains from ``ROPE_INIT_FUNCTIONS`` (:88-90); the cos/sin values are
computed from them on the fly (fp32 angle, rounded to the tensor's dtype as the reference's cached tables are), so there
is no table, no Python loop over the batch and no host synchronisation.
"""
import torch

from .. import _lib
from ._common import dtype_code, inner_contiguous, ptr, require_cuda, stream_ptr


def _launch(x, y, inv_freq, cu_seqlens, step, stride, scaling, inverse):
    rows, num_heads, head_dim = x.shape
    torch.cuda.set_device(x.device)
    rc = _lib.lib().nsa_rope(ptr(x), ptr(y), ptr(inv_freq), ptr(cu_seqlens), rows, cu_seqlens.shape[0] - 1, num_heads, head_dim,
                             int(step), int(stride), float(scaling), int(inverse), x.stride(0), x.stride(1), y.stride(0),
                             y.stride(1), dtype_code(x), stream_ptr(x.device))
    _lib.check(rc, "nsa_rope")


class Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, inv_freq, cu_seqlens, step, stride, scaling):
        x = inner_contiguous(x)
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        _launch(x, y, inv_freq, cu_seqlens, step, stride, scaling, 0)
        ctx.save_for_backward(inv_freq, cu_seqlens)
        ctx.meta = (step, stride, scaling)
        return y

    @staticmethod
    def backward(ctx, dy):
        inv_freq, cu_seqlens = ctx.saved_tensors
        step, stride, scaling = ctx.meta
        dy = inner_contiguous(dy)
        dx = torch.empty(dy.shape, dtype=dy.dtype, device=dy.device)
        _launch(dy, dx, inv_freq, cu_seqlens, step, stride, scaling, 1)
        return dx, None, None, None, None, None


def rope(x: torch.Tensor, inv_freq: torch.Tensor, cu_seqlens: torch.Tensor, step: int = 0, stride: int = 1,
         attention_scaling: float = 1.0) -> torch.Tensor:
    """x [rows, heads, d] (d 64 or 128, bf16/fp16), inv_freq fp32 [d / 2], cu_seqlens int32 [batch + 1] -> rotated copy.
    With step > 0, rows == batch (one new token per sequence) and cu_seqlens holds the PREFILL lengths, as in the
    reference's decode loop."""
    require_cuda(x, inv_freq, cu_seqlens)
    assert x.dtype == torch.bfloat16 or x.dtype == torch.float16
    assert x.dim() == 3 and x.shape[-1] in (64, 128), "rope supports head_dim 64 and 128"
    assert inv_freq.dtype == torch.float32 and inv_freq.shape == (x.shape[-1] // 2,) and inv_freq.is_contiguous()
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.dim() == 1 and cu_seqlens.is_contiguous()
    assert step >= 0 and stride >= 1
    if step > 0:
        assert x.shape[0] == cu_seqlens.shape[0] - 1
    return Rope.apply(x, inv_freq, cu_seqlens, int(step), int(stride), float(attention_scaling))
