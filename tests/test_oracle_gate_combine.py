"""The oracle's gated sum against a direct per-element evaluation, and the shared library's exports for it."""
import torch

from oracle import nsa_oracle as O


def test_gate_combine_oracle_small_case():
    g = torch.Generator().manual_seed(5)
    gate = torch.rand(7, 3, 3, generator=g)
    outs = [torch.randn(7, 3, 16, generator=g) for _ in range(3)]
    y = O.gate_combine(gate, *outs)
    for n in range(7):
        for h in range(3):
            want = sum(gate[n, h, i] * outs[i][n, h] for i in range(3))
            assert torch.allclose(y[n, h], want, atol=1e-6)


def test_gate_combine_symbols_exported():
    from native_sparse_attention_triton_b200 import _lib
    lib = _lib.lib()
    assert hasattr(lib, "nsa_gate_combine_fwd") and hasattr(lib, "nsa_gate_combine_bwd")
