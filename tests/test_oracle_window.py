"""CPU checks of the oracle's sliding-window attention (the branch the reference delegates to flash_attn): against a loop
over single queries, and against the oracle's own causal attention when the window covers all.  The pin against flash_attn's
own output is tests/test_oracle_box_golden.py."""
import math

import torch

from oracle import nsa_oracle as O


def test_window_oracle_against_per_query_loop():
    g = torch.Generator().manual_seed(5)
    seqlens, Hq, Hkv, d, W = [9, 1, 23], 4, 2, 16, 5
    N = sum(seqlens)
    q, k, v = (torch.randn(N, h, d, generator=g) for h in (Hq, Hkv, Hkv))
    cu = torch.tensor([0, 9, 10, 33], dtype=torch.int32)
    o = O.sliding_window_attention(q, k, v, cu, W)
    G = Hq // Hkv
    for b in range(3):
        s, e = int(cu[b]), int(cu[b + 1])
        for i in range(s, e):
            lo = max(s, i - W)
            for h in range(Hq):
                logits = (k[lo:i + 1, h // G] @ q[i, h]) / math.sqrt(d)
                ref = torch.softmax(logits, 0) @ v[lo:i + 1, h // G]
                assert torch.allclose(o[i, h], ref, atol=1e-5), (b, i, h)


def test_window_covering_everything_is_causal_attention():
    g = torch.Generator().manual_seed(6)
    q, k, v = (torch.randn(40, h, 8, generator=g) for h in (4, 2, 2))
    cu = torch.tensor([0, 15, 40], dtype=torch.int32)
    a = O.sliding_window_attention(q, k, v, cu, 1000)
    b = O.flash_attention_varlen(q, k, v, cu, cu, causal=True)
    assert torch.allclose(a, b, atol=1e-6)
