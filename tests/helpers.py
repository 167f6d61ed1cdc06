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


def window_case_inputs():
    """Seeded inputs of the sliding-window fixture (tests/golden/box_window.npz)."""
    g = torch.Generator().manual_seed(2024)
    seqlens, Hq, Hkv, d = [37, 300, 700], 8, 2, 128
    N = sum(seqlens)
    cu = torch.tensor([0] + list(np.cumsum(seqlens)), dtype=torch.int32)
    mk = lambda *s: bf16_exact(torch.randn(*s, generator=g))
    return dict(cu=cu, q=mk(N, Hq, d), k=mk(N, Hkv, d), v=mk(N, Hkv, d), do=mk(N, Hq, d))


def rope_case_inputs():
    """Seeded inputs of the rotary-embedding fixture (tests/golden/box_rope.npz): a ragged batch, its compressed counterpart
    (kernel 32, stride 16) and one decode row per sequence.  Values are exact in bf16 and in fp16."""
    g = torch.Generator().manual_seed(77)
    seqlens, H, d = [5, 130, 1000], 2, 128
    clens = [0 if L < 32 else (L - 32) // 16 + 1 for L in seqlens]
    cu = torch.tensor([0] + list(np.cumsum(seqlens)), dtype=torch.int32)
    cu_c = torch.tensor([0] + list(np.cumsum(clens)), dtype=torch.int32)
    mk = lambda *s: (torch.randint(-512, 513, s, generator=g).float() / 128.0)
    return dict(cu=cu, cu_c=cu_c, x=mk(sum(seqlens), H, d), xc=mk(sum(clens), H, d), xd=mk(len(seqlens), H, d))


INFER_PARAMS = dict(HQ=8, HKV=2, D=128, KS=32, ST=16, BS=64, TOPK=4, INIT=1, LOCAL=2, W=64, MAXLEN=512, MAXB=4)


def infer_case_inputs(mode, lens, steps, dtype=torch.bfloat16):
    """Seeded inputs of an inference scenario (prefill of a ragged batch, then `steps` decode steps): used by the GPU
    inference tests and by the fixtures tests/golden/box_infer_*.npz.  All tensors are exact in `dtype`."""
    P = INFER_PARAMS
    HQ, HKV, D, KS = P["HQ"], P["HKV"], P["D"], P["KS"]
    g = torch.Generator().manual_seed(100 + len(lens) + steps)
    B, total = len(lens), sum(lens)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    rd = lambda t: t.to(dtype).float()
    if mode == "linear":
        mk = lambda: rd(torch.randn(HKV, KS * D, D, generator=g) / math.sqrt(KS * D))
        w_k, w_v, pe = mk(), mk(), rd(torch.randn(HKV, KS, D, generator=g) * 0.02)
    elif mode == "weighted":
        mk = lambda: rd(torch.rand(HKV, KS, generator=g) / KS)
        w_k, w_v, pe = mk(), mk(), rd(torch.randn(HKV, KS, D, generator=g) * 0.02)
    else:
        w_k = w_v = pe = None
    rnd = lambda *s: rd(torch.randn(*s, generator=g))
    q, k, v = rnd(total, HQ, D), rnd(total, HKV, D), rnd(total, HKV, D)
    gate = rd(torch.rand(total, HQ, 3, generator=g))
    step_inputs = []
    for _ in range(steps):
        qn, kn, vn = rnd(B, HQ, D), rnd(B, HKV, D), rnd(B, HKV, D)
        step_inputs.append((qn, kn, vn, rd(torch.rand(B, HQ, 3, generator=g))))
    return dict(params=P, cu=cu, w_k=w_k, w_v=w_v, pe=pe, q=q, k=k, v=v, gate=gate, steps=step_inputs)


def from_bits16(a: np.ndarray) -> torch.Tensor:
    """uint16 fp16 bit patterns -> fp32 tensor."""
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.float16).float()


def box_fixture(name):
    """A fixture written by tests/golden/make_golden_on_box.py (outputs of the reference itself on a B200), or None."""
    path = os.path.join(GOLDEN_DIR, name + ".npz")
    return np.load(path) if os.path.exists(path) else None


# ---- the acceptance rule of the hot path, in one place --------------------------------------------------------------
# Results are compared after normalising the tensor to unit variance when its RMS exceeds 1 (outputs of N(0,1) problems
# have RMS <= 1 and are compared in absolute terms; gradients that sum thousands of terms are not): with
# scale = max(1, rms(ref)),
#     max over elements of |test - ref| / max(|ref|, scale) <= MAX_TOL   (an element of magnitude m carries m * 2^-9 of
#                                                                       16-bit rounding by itself)
#     mean |test - ref| / scale                             <= MEAN_TOL
# dK and dV of the two attention operators are sums, over every query row that sees a key, of products of 16-bit P / dS
# values: their worst element is allowed KV_GRAD_MAX_TOL.  On the same seeded inputs the reference's own Triton kernels
# score up to 0.128 there against the fp32 oracle and these kernels 0.074 (BASELINE configurations 1 and 2, measured on a
# B200 by tests/test_gpu_vs_reference.py); every other tensor of either implementation stayed below 1.5e-2, means below
# 1.7e-3.
# Gradients that pass through two operators' backward passes in a row (attention, then compression: dk, dv, dwk, dwv of
# the chain) carry both operators' rounding; their mean bound is CHAIN_GRAD_MEAN_TOL.  The reference's own recorded chain
# (tests/golden/box_triton_*.npz) scores 2.3e-3 .. 2.8e-3 there against the fp32 oracle, these kernels 2.0e-3 .. 2.8e-3.
MAX_TOL, MEAN_TOL, KV_GRAD_MAX_TOL, CHAIN_GRAD_MEAN_TOL = 2e-2, 2e-3, 8e-2, 4e-3


def error_16bit(test, ref):
    """(max error, mean error, scale) of `test` against `ref` under the rule above."""
    t, r = test.detach().float().cpu(), ref.detach().float().cpu()
    if r.numel() == 0:
        return 0.0, 0.0, 1.0
    scale = max(1.0, float(r.pow(2).mean().sqrt()))
    e = (t - r).abs()
    return float((e / r.abs().clamp(min=scale)).max()), float(e.mean()) / scale, scale


def close_16bit(test, ref, max_tol=MAX_TOL, mean_tol=MEAN_TOL):
    """(ok, max error, mean error) under the rule above."""
    mx, mean, _ = error_16bit(test, ref)
    return (mx <= max_tol and mean <= mean_tol), mx, mean


def assert_close_16bit(test, ref, what, max_tol=MAX_TOL, mean_tol=MEAN_TOL):
    assert tuple(test.shape) == tuple(ref.shape), (what, test.shape, ref.shape)
    ok, mx, mean = close_16bit(test, ref, max_tol, mean_tol)
    assert ok, (what, "max", mx, "mean", mean)


def grad_tol(name, chain=False):
    """Worst-element bound of a gradient by its name: dk, dv, dck, dcv are key/value gradients of an attention operator;
    in a chain of operators the compression weights' gradients (dwk, dwv) are sums of those over windows and inherit half
    of their allowance (the reference's recorded chain reaches 2.3e-2 there against the fp32 oracle)."""
    if name in ("dk", "dv", "dck", "dcv"):
        return KV_GRAD_MAX_TOL
    if chain and name in ("dwk", "dwv"):
        return KV_GRAD_MAX_TOL / 2
    if chain and name == "dq":
        return 2 * MAX_TOL   # the sum of two operators' query gradients, each within MAX_TOL (1.5e-2 measured)
    if chain and name == "dgate":
        # an element is the dot product over head_dim of dO with a branch output, which the layer (like the reference's)
        # holds rounded to 16 bits and the oracle in fp32.  For the first tokens of a sequence |o| ~ 1, so the rounding alone
        # has a standard deviation of sqrt(128) * 2^-9 / sqrt(3) = 1.3e-2 per element; the largest of ~1e5 elements sits near
        # 4.5 sigma (2.0e-2 and 4.1e-2 measured on the two layer cases).  Six sigma:
        return KV_GRAD_MAX_TOL
    return MAX_TOL


def rope_tolerance(x, want, ulp, extra=0.0):
    """Elementwise bound on |rotated - want| where `want` comes from the reference's RotaryEmbedding, which rounds both
    products x * cos and rotate_half(x) * sin and their sum to the tensor's dtype (module/rope.py:204-209) while the oracle
    and the kernel round once: half a unit in the last place (`ulp` = 2^-7 for bf16, 2^-10 for fp16: the spacing relative to a value at the bottom of its binade) of each
    product's operand, of the sum and of the compared result; `extra` adds that many units of the operands."""
    half = x.shape[-1] // 2
    mag = x[..., :half].abs() + x[..., half:].abs()
    mag = torch.cat([mag, mag], -1)
    return 0.5 * ulp * (mag * (1.0 + 2.0 * extra) + 2.0 * want.abs()) * 1.001 + 1e-6
