"""Shared helpers for the test-suite: golden fixture loading and seeded input generation."""
import math
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def from_bits(a: np.ndarray) -> torch.Tensor:
    """uint16 bf16 bit patterns -> fp32 tensor."""
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).float()


def bf16_exact(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).float()


def chain_inputs(seed, seqlens, Hq, Hkv, d, ks):
    """Same generator, same draw order as tests/golden/make_golden.py::chain_case."""
    g = torch.Generator().manual_seed(int(seed))
    N = int(sum(seqlens))
    cu = torch.tensor([0] + list(np.cumsum(seqlens)), dtype=torch.int32)
    q = bf16_exact(torch.randn(N, Hq, d, generator=g))
    k = bf16_exact(torch.randn(N, Hkv, d, generator=g))
    v = bf16_exact(torch.randn(N, Hkv, d, generator=g))
    wk = bf16_exact(torch.randn(Hkv, ks * d, d, generator=g) / math.sqrt(ks * d))
    wv = bf16_exact(torch.randn(Hkv, ks * d, d, generator=g) / math.sqrt(ks * d))
    pe = bf16_exact(torch.randn(Hkv, ks, d, generator=g) * 0.02)
    wp = bf16_exact(torch.randn(Hkv, ks, generator=g) / ks)
    return dict(cu=cu, q=q, k=k, v=v, wk=wk, wv=wv, pe=pe, wp=wp)


def load_golden(name):
    """Returns (meta dict, inputs dict, golden dict) for a fixture made by make_golden.py."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    meta = {k: (z[k].tolist() if z[k].ndim else z[k].item()) for k in
            ("seed", "seqlens", "Hq", "Hkv", "d", "ks", "st", "bs", "topk", "init_blocks", "local_blocks",
             "row_step", "q_sum", "k_sum")}
    if "q" in z.files:
        seqlens = meta["seqlens"]
        inp = dict(cu=torch.tensor([0] + list(np.cumsum(seqlens)), dtype=torch.int32))
        for k in ("q", "k", "v", "wk", "wv", "pe", "wp"):
            inp[k] = from_bits(z[k])
    else:
        inp = chain_inputs(meta["seed"], meta["seqlens"], meta["Hq"], meta["Hkv"], meta["d"], meta["ks"])
        # the seeded generator must reproduce the tensors the fixture was made from
        assert abs(float(inp["q"].double().sum()) - meta["q_sum"]) < 1e-6, "RNG stream differs from fixture"
        assert abs(float(inp["k"].double().sum()) - meta["k_sum"]) < 1e-6, "RNG stream differs from fixture"
    gold = {}
    for k in ("lin_k", "lin_v", "pool_k", "avg_k", "dec_o_sel", "dec_o_flash"):
        gold[k] = from_bits(z[k])
    for k in ("o_cmp", "o_sel", "dec_o_cmp"):
        gold[k] = torch.from_numpy(z[k])
    gold["topk_idx"] = torch.from_numpy(z["topk_idx"].astype(np.int32))
    gold["dec_idx"] = torch.from_numpy(z["dec_idx"].astype(np.int32))
    gold["cu_k"] = torch.from_numpy(z["cu_k"]).to(torch.int32)
    return meta, inp, gold


def padded_cache(x, cu, seqlens, pad_to=None):
    """[N, H, d] varlen -> dense [B, Lmax, H, d] cache."""
    B = len(seqlens)
    Lmax = pad_to or max(max(seqlens), 1)
    out = torch.zeros(B, Lmax, x.shape[1], x.shape[2], dtype=x.dtype)
    for b, L in enumerate(seqlens):
        out[b, :L] = x[int(cu[b]):int(cu[b]) + L]
    return out
