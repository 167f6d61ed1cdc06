"""Gated sum of the three branch outputs of an NSA layer (compressed, selected, sliding-window).

The reference has no operator for this step: its layer evaluates
    gate[..., 0:1] * compressed_attn_output + gate[..., 1:2] * sparse_attn_output + gate[..., 2:3] * sliding_attn_output
in eager PyTorch (native_sparse_attention/module/native_sparse_attention.py:226-232; the inference path does the same at
native_sparse_attention/infer/nsa_inference.py:146-150).  This function computes the same expression, forward and
backward, in one pass over HBM each, with fp32 arithmetic and a single rounding.
"""
import torch

from .. import _lib
from ._common import dtype_code, inner_contiguous, ptr, require_cuda, stream_ptr


class GateCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, o_cmp, o_sel, o_win):
        gate = gate.contiguous()
        o_cmp, o_sel, o_win = inner_contiguous(o_cmp), inner_contiguous(o_sel), inner_contiguous(o_win)
        total, num_heads, head_dim = o_cmp.shape
        out = torch.empty(total, num_heads, head_dim, dtype=o_cmp.dtype, device=o_cmp.device)
        strides = _lib.strides_array(gate.stride(0), gate.stride(1), o_cmp.stride(0), o_cmp.stride(1), o_sel.stride(0),
                                     o_sel.stride(1), o_win.stride(0), o_win.stride(1), out.stride(0), out.stride(1))
        torch.cuda.set_device(out.device)
        rc = _lib.lib().nsa_gate_combine_fwd(ptr(gate), ptr(o_cmp), ptr(o_sel), ptr(o_win), ptr(out), total, num_heads, head_dim,
                                             strides, dtype_code(out), stream_ptr(out.device))
        _lib.check(rc, "nsa_gate_combine_fwd")
        ctx.save_for_backward(gate, o_cmp, o_sel, o_win)
        return out

    @staticmethod
    def backward(ctx, dout):
        gate, o_cmp, o_sel, o_win = ctx.saved_tensors
        dout = inner_contiguous(dout)
        total, num_heads, head_dim = o_cmp.shape
        d_gate = torch.empty_like(gate)
        d_cmp, d_sel, d_win = (torch.empty(total, num_heads, head_dim, dtype=dout.dtype, device=dout.device) for _ in range(3))
        strides = _lib.strides_array(gate.stride(0), gate.stride(1), o_cmp.stride(0), o_cmp.stride(1), o_sel.stride(0),
                                     o_sel.stride(1), o_win.stride(0), o_win.stride(1), dout.stride(0), dout.stride(1),
                                     d_gate.stride(0), d_gate.stride(1), d_cmp.stride(0), d_cmp.stride(1), d_sel.stride(0),
                                     d_sel.stride(1), d_win.stride(0), d_win.stride(1))
        torch.cuda.set_device(dout.device)
        rc = _lib.lib().nsa_gate_combine_bwd(ptr(gate), ptr(o_cmp), ptr(o_sel), ptr(o_win), ptr(dout), ptr(d_gate), ptr(d_cmp),
                                             ptr(d_sel), ptr(d_win), total, num_heads, head_dim, strides, dtype_code(dout),
                                             stream_ptr(dout.device))
        _lib.check(rc, "nsa_gate_combine_bwd")
        return d_gate, d_cmp, d_sel, d_win


def gate_combine(gate: torch.Tensor, o_cmp: torch.Tensor, o_sel: torch.Tensor, o_win: torch.Tensor) -> torch.Tensor:
    """gate [n, h, 3] (already through the sigmoid), o_* [n, h, d] -> [n, h, d] contiguous, so that the head concat that
    feeds the output projection is a view.  d is 64 or 128; 16-bit inputs of one dtype."""
    require_cuda(gate, o_cmp, o_sel, o_win)
    assert o_cmp.dtype == torch.bfloat16 or o_cmp.dtype == torch.float16
    assert gate.dtype == o_cmp.dtype and o_sel.dtype == o_cmp.dtype and o_win.dtype == o_cmp.dtype
    assert o_cmp.dim() == 3 and o_cmp.shape == o_sel.shape == o_win.shape
    assert gate.shape == (o_cmp.shape[0], o_cmp.shape[1], 3)
    assert o_cmp.shape[-1] in (64, 128), "gate_combine supports head_dim 64 and 128"
    return GateCombine.apply(gate, o_cmp, o_sel, o_win)
