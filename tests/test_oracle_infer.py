"""The oracle's decode step (a function of the token history) against the last row of its own prefill on the same
history: they differ only in the sliding window, which is one key shorter in decode."""
import math

import torch

from oracle import nsa_oracle as O


def test_decode_token_equals_last_prefill_row():
    g = torch.Generator().manual_seed(3)
    Hq, Hkv, d, ks, st, bs, topk, W = 4, 2, 16, 8, 4, 16, 3, 12
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    w_k = torch.randn(Hkv, ks * d, d, generator=g) / math.sqrt(ks * d)
    w_v = torch.randn(Hkv, ks * d, d, generator=g) / math.sqrt(ks * d)
    pe = torch.randn(Hkv, ks, d, generator=g) * 0.02
    for n in (1, 5, 8, 13, 50):
        q, k, v = torch.randn(n, Hq, d, generator=g), torch.randn(n, Hkv, d, generator=g), torch.randn(n, Hkv, d, generator=g)
        gate = torch.rand(n, Hq, 3, generator=g)
        cu = torch.tensor([0, n], dtype=torch.int32)
        common = (inv_freq, O.linear_compress, O.linear_compress, w_k, w_v, pe, ks, st, bs, topk, 1, 2)
        row = O.nsa_decode_token(q[-1], k, v, gate[-1], *common, W)
        full = O.nsa_prefill(q, k, v, gate, cu, *common, W - 1)   # a prefill row sees window + 1 keys
        assert torch.allclose(row, full[-1], atol=1e-5), n
