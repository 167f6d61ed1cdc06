"""The oracle's rotary embedding against an independent formulation (complex multiplication per position), the
positions it derives from cu_seqlens, and the library export."""
import torch

from oracle import nsa_oracle as O


def inv_freq_for(d, theta=10000.0):
    return 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))


def test_rope_oracle_equals_complex_rotation():
    g = torch.Generator().manual_seed(1)
    d, lens, stride = 16, [5, 1, 9], 3
    cu = torch.tensor([0, 5, 6, 15], dtype=torch.int32)
    x = torch.randn(15, 2, d, generator=g)
    y = O.rope(x, inv_freq_for(d), cu, 0, stride)
    n = 0
    for L in lens:
        for t in range(L):
            ang = inv_freq_for(d) * float(t * stride)
            z = torch.complex(x[n, :, :d // 2], x[n, :, d // 2:]) * torch.polar(torch.ones(d // 2), ang)
            assert torch.allclose(y[n, :, :d // 2], z.real, atol=1e-5) and torch.allclose(y[n, :, d // 2:], z.imag, atol=1e-5)
            n += 1


def test_rope_oracle_decode_positions():
    """Row b of decode step s equals the prefill rotation of a token at in-sequence index len_b + s - 1."""
    g = torch.Generator().manual_seed(2)
    d, step, stride = 8, 4, 2
    cu = torch.tensor([0, 3, 10], dtype=torch.int32)
    x = torch.randn(2, 1, d, generator=g)
    y = O.rope(x, inv_freq_for(d), cu, step, stride)
    for b, L in enumerate([3, 7]):
        idx = L + step - 1
        long_cu = torch.tensor([0, idx + 1], dtype=torch.int32)
        xs = x[b:b + 1].expand(idx + 1, 1, d).contiguous()
        assert torch.allclose(O.rope(xs, inv_freq_for(d), long_cu, 0, stride)[idx], y[b], atol=1e-6)


def test_rope_symbol_exported():
    from native_sparse_attention_triton_b200 import _lib
    assert hasattr(_lib.lib(), "nsa_rope")
