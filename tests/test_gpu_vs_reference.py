"""Same-GPU parity with the reference's own Triton operators (``native_sparse_attention.ops``, imported unmodified from
``baseline/_ref``; skipped where that directory is absent), operator by operator on identical seeded inputs.

Every comparison is made three ways -- these kernels against the reference's Triton kernels, and each of the two against
the fp32 oracle evaluated on the same device -- and written to a JSON report (``REPORT`` below).  The acceptance rule
is the one the hot path is specified with (tests/helpers.py): outputs and gradients within 2e-2 (max) and 2e-3 (mean) of
the reference on unit-variance scale, where an element larger than the scale is allowed the same RELATIVE slack (a 16-bit
result of magnitude m carries m * 2^-9 of rounding alone); ``topk_idx`` identical except where the
reference's own block scores of the differing blocks lie within 1e-3 of the row's selection threshold.  A bound wider
than that is only ever taken from what the reference's kernels themselves score against the oracle on the same inputs
(``SLACK`` times their error).
"""
import json
import math
import os

import pytest
import torch

from tests import refbox
from tests.helpers import MAX_TOL, MEAN_TOL, error_16bit
from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu

SLACK = 1.25
REPORT = os.path.join(refbox.ROOT, os.environ.get("NSA_REPORT_DIR", "gpurun_out"), "parity_vs_triton.json")
_report = {}


@pytest.fixture(scope="module")
def ref():
    r = refbox.load()
    yield r
    os.makedirs(os.path.dirname(REPORT), exist_ok=True)
    old = {}
    if os.path.exists(REPORT):
        try:
            old = json.load(open(REPORT))
        except Exception:
            old = {}
    old.update(_report)
    json.dump(old, open(REPORT, "w"), indent=1, sort_keys=True)
    refbox.unload()


@pytest.fixture(scope="module")
def pkg():
    import native_sparse_attention_triton_b200 as p
    assert torch.cuda.is_available()
    return p


def stats(test, ref_t):
    mx, mean, scale = error_16bit(test, ref_t)
    e = (test.detach().float() - ref_t.detach().float()).abs()
    return dict(max=mx, mean=mean, scale=scale, max_abs=float(e.max()), mean_abs=float(e.mean()),
                ref_max=float(ref_t.detach().float().abs().max()))


def judge(case, name, ours, triton, oracle):
    """Record the three comparisons (errors in the units of tests/helpers.py: after normalising to unit variance where the
    reference's RMS exceeds 1) and apply the acceptance rule to `ours`."""
    a, b, c = stats(ours, triton), stats(triton, oracle), stats(ours, oracle)
    _report[f"{case}/{name}"] = dict(ours_vs_triton=a, triton_vs_oracle=b, ours_vs_oracle=c)
    print(f"{case}/{name}: ours-triton max {a['max']:.4f} mean {a['mean']:.5f} | triton-oracle max {b['max']:.4f} "
          f"mean {b['mean']:.5f} | ours-oracle max {c['max']:.4f} mean {c['mean']:.5f} | scale {a['scale']:.3f} "
          f"largest {a['ref_max']:.2f}")
    # against the fp32 oracle: the stated bound, or no worse than the reference's kernels on the same inputs
    assert c["max"] <= max(MAX_TOL, SLACK * b["max"]), (case, name, c, b)
    assert c["mean"] <= max(MEAN_TOL, SLACK * b["mean"]), (case, name, c, b)
    # against the reference's kernels: two roundings apart at most
    assert a["max"] <= max(MAX_TOL, SLACK * (b["max"] + c["max"])), (case, name, a)
    assert a["mean"] <= max(MEAN_TOL, SLACK * (b["mean"] + c["mean"])), (case, name, a)


def leaf(t):
    return t.detach().clone().requires_grad_(True)


def make_inputs(seed, seqlens, Hq, Hkv, d, ks, dtype, dist):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dev = torch.device("cuda")
    N = sum(seqlens)
    if dist == "normal":
        rnd = lambda *s, scale=1.0: (torch.randn(*s, generator=g, device=dev) * scale).to(dtype)
    else:  # the reference's scripts draw uniformly from (-1, 1)
        rnd = lambda *s, scale=1.0: ((torch.rand(*s, generator=g, device=dev) * 2 - 1) * scale).to(dtype)
    cu = torch.tensor([0] + torch.tensor(seqlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
    return dict(cu=cu, q=rnd(N, Hq, d), k=rnd(N, Hkv, d), v=rnd(N, Hkv, d),
                wk=rnd(Hkv, ks * d, d, scale=1 / math.sqrt(ks * d)), wv=rnd(Hkv, ks * d, d, scale=1 / math.sqrt(ks * d)),
                pe=rnd(Hkv, ks, d, scale=0.02), wp=(torch.rand(Hkv, ks, generator=g, device=dev) / ks).to(dtype),
                do1=rnd(N, Hq, d), do2=rnd(N, Hq, d), g=g)


CASES = {
    # BASELINE configuration 1 (its shapes in 16-bit), configuration 2 at its stated shape, and the shapes of the
    # reference's own parity scripts (test/test_compressed_attention.py:33-70, test/test_topk_sparse_attention.py:90-120)
    # with head_dim 128 in place of 96
    "cfg1": dict(seed=1, seqlens=[256, 768], Hq=16, Hkv=2, d=64, ks=32, st=16, bs=64, topk=4, dtype=torch.bfloat16, dist="normal"),
    "cfg2": dict(seed=2, seqlens=[1024, 7168, 8192], Hq=64, Hkv=4, d=128, ks=32, st=16, bs=64, topk=16, dtype=torch.bfloat16,
                 dist="normal"),
    "script_cmp": dict(seed=3, seqlens=[1000, 4000, 8192], Hq=32, Hkv=8, d=128, ks=32, st=16, bs=64, topk=16, dtype=torch.float16,
                       dist="uniform"),
    "script_sel": dict(seed=4, seqlens=[1000, 2000, 4096], Hq=64, Hkv=8, d=128, ks=32, st=16, bs=64, topk=5, dtype=torch.float16,
                       dist="uniform"),
}


@pytest.mark.parametrize("case", ["cfg1", "cfg2"])
def test_compression_vs_triton(ref, pkg, case):
    from native_sparse_attention.ops import avgpool_compress, weightedpool_compress
    linear_compress, which = refbox.reference_linear_compress()
    _report["linear_compress_reference_implementation"] = which
    c = CASES[case]
    x = make_inputs(c["seed"], c["seqlens"], c["Hq"], c["Hkv"], c["d"], c["ks"], c["dtype"], c["dist"])
    ks, st, cu = c["ks"], c["st"], x["cu"]
    for name, rfn, ofn, orfn, w in (("linear", linear_compress, pkg.ops.linear_compress, O.linear_compress, x["wk"]),
                                    ("weighted", weightedpool_compress, pkg.ops.weightedpool_compress, O.weightedpool_compress, x["wp"]),
                                    ("avg", avgpool_compress, pkg.ops.avgpool_compress, O.avgpool_compress, None)):
        res = []
        for fn, f32 in ((ofn, False), (rfn, False), (orfn, True)):
            cast = (lambda t: leaf(t.float())) if f32 else leaf
            xi, wi, pi = cast(x["k"]), (cast(w) if w is not None else None), cast(x["pe"])
            y, y_cu = fn(xi, wi, cu, ks, st, pi)
            if not res:
                dy = torch.randn(y.shape, generator=x["g"], device=y.device).to(c["dtype"])
            y.backward(dy.to(y.dtype))
            res.append((y, xi.grad, wi.grad if wi is not None else None, pi.grad, y_cu))
        assert torch.equal(res[0][4].cpu(), res[1][4].cpu().to(torch.int32))
        for i, nm in enumerate(("y", "dx", "dw", "dpe")):
            if res[0][i] is not None:
                judge(case, f"{name}_compress/{nm}", res[0][i], res[1][i], res[2][i])
    assert pkg.device_status() == 0


@pytest.mark.parametrize("case", ["cfg1", "cfg2", "script_cmp"])
def test_compressed_attention_vs_triton(ref, pkg, case):
    from native_sparse_attention.ops import compressed_attention
    from native_sparse_attention.ops.triton import compressed_attention as ca
    linear_compress = refbox.reference_linear_compress()[0]
    c = CASES[case]
    x = make_inputs(c["seed"], c["seqlens"], c["Hq"], c["Hkv"], c["d"], c["ks"], c["dtype"], c["dist"])
    ks, st, bs, topk, cu = c["ks"], c["st"], c["bs"], c["topk"], x["cu"]
    with torch.no_grad():   # both implementations see the SAME compressed keys and values (the reference's)
        ck, cu_k = linear_compress(x["k"], x["wk"], cu, ks, st, x["pe"])
        cv, _ = linear_compress(x["v"], x["wv"], cu, ks, st, None)
        if c["dist"] == "uniform":   # the reference's script overwrites them with uniform noise
            ck = torch.empty_like(ck).uniform_(-1, 1, generator=x["g"])
            cv = torch.empty_like(cv).uniform_(-1, 1, generator=x["g"])
    max_q, max_k = max(c["seqlens"]), int((cu_k[1:] - cu_k[:-1]).max())
    res = []
    for which in ("ours", "triton", "oracle"):
        f32 = which == "oracle"
        cast = (lambda t: leaf(t.float())) if f32 else leaf
        q, k, v = cast(x["q"]), cast(ck), cast(cv)
        fn = {"ours": pkg.ops.compressed_attention, "triton": compressed_attention, "oracle": O.compressed_attention}[which]
        o, idx = fn(q, k, v, ks, st, bs, topk, cu, cu_k, max_q, max_k)[:2]
        o.backward(x["do1"].to(o.dtype))
        res.append((o, q.grad, k.grad, v.grad, idx))
    for i, nm in enumerate(("o", "dq", "dk", "dv")):
        judge(case, f"compressed_attention/{nm}", res[0][i], res[1][i], res[2][i])
    # selection: the reference's own block scores decide which differences are ties
    with torch.no_grad():
        _, lse = ca.CompressedAttention.apply(x["q"], ck, cv, ks, st, cu, cu_k, max_q, max_k, None)
        score = ca._get_attention_score(x["q"], ck, lse, ks, st, cu, cu_k, max_q, max_k, None)
        score = ca.transform_score(score, ks, st, bs, cu, cu_k, max_q, max_k, 1, 2)
    bad, differing, rows = O.compare_topk_idx(res[0][4], res[1][4], score.float(), tie_tol=1e-3)
    bad_o, differing_o, _ = O.compare_topk_idx(res[2][4].to(res[1][4].device), res[1][4], score.float(), tie_tol=1e-3)
    _report[f"{case}/topk_idx"] = dict(rows=rows, ours_rows_differing=differing, ours_rows_outside_tie=bad,
                                       oracle_rows_differing=differing_o, oracle_rows_outside_tie=bad_o)
    print(f"{case}/topk_idx: ours vs triton: {differing}/{rows} rows differ, {bad} outside the 1e-3 tie band; fp32 oracle vs "
          f"triton: {differing_o} differ, {bad_o} outside")
    assert bad == 0, (bad, differing, rows)
    assert pkg.device_status() == 0


def random_topk_idx(seqlens, Hkv, bs, topk, g):
    """Left-packed ascending block ids per (head, token), block 0 and the query's own block always present."""
    dev = torch.device("cuda")
    out = []
    for L in seqlens:
        nb = (L + bs - 1) // bs
        bq = torch.arange(L, device=dev) // bs
        sc = torch.rand(Hkv, L, nb, generator=g, device=dev)
        blk = torch.arange(nb, device=dev)
        sc = torch.where(blk[None, None, :] > bq[None, :, None], torch.full_like(sc, -1.0), sc)
        sc = torch.where((blk[None, None, :] == 0) | (blk[None, None, :] == bq[None, :, None]), torch.full_like(sc, 2.0), sc)
        k = min(topk, nb)
        val, idx = sc.topk(k, dim=-1)
        idx = torch.where(val < 0, torch.full_like(idx, 1 << 20), idx).sort(-1).values
        idx = torch.where(idx >= (1 << 20), torch.full_like(idx, -1), idx)
        if k < topk:
            idx = torch.nn.functional.pad(idx, (0, topk - k), value=-1)
        out.append(idx)
    return torch.cat(out, 1).to(torch.int32).contiguous()


@pytest.mark.parametrize("case", ["cfg1", "cfg2", "script_sel"])
def test_topk_sparse_attention_vs_triton(ref, pkg, case):
    from native_sparse_attention.ops import compressed_attention, topk_sparse_attention
    linear_compress = refbox.reference_linear_compress()[0]
    c = CASES[case]
    x = make_inputs(c["seed"], c["seqlens"], c["Hq"], c["Hkv"], c["d"], c["ks"], c["dtype"], c["dist"])
    ks, st, bs, topk, cu = c["ks"], c["st"], c["bs"], c["topk"], x["cu"]
    if case == "script_sel":
        idx = random_topk_idx(c["seqlens"], c["Hkv"], bs, topk, x["g"])
    else:
        with torch.no_grad():   # the reference's own selection, fed to all three
            ck, cu_k = linear_compress(x["k"], x["wk"], cu, ks, st, x["pe"])
            cv, _ = linear_compress(x["v"], x["wv"], cu, ks, st, None)
            idx = compressed_attention(x["q"], ck, cv, ks, st, bs, topk, cu, cu_k)[1]
    res = []
    for which in ("ours", "triton", "oracle"):
        f32 = which == "oracle"
        cast = (lambda t: leaf(t.float())) if f32 else leaf
        q, k, v = cast(x["q"]), cast(x["k"]), cast(x["v"])
        fn = {"ours": pkg.ops.topk_sparse_attention, "triton": topk_sparse_attention, "oracle": O.topk_sparse_attention}[which]
        o = fn(q, k, v, idx, bs, cu)
        o.backward(x["do2"].to(o.dtype))
        res.append((o, q.grad, k.grad, v.grad))
    for i, nm in enumerate(("o", "dq", "dk", "dv")):
        judge(case, f"topk_sparse_attention/{nm}", res[0][i], res[1][i], res[2][i])
    assert pkg.device_status() == 0


def test_decode_ops_vs_triton(ref, pkg):
    """The reference's decode self-test shapes (flash_attention_decode.py:261-282, topk_sparse_attention_decode.py:330-354),
    batch reduced to 12."""
    from native_sparse_attention.ops import compressed_attention_decode, flash_attention_decode, topk_sparse_attention_decode
    dev = torch.device("cuda")
    g = torch.Generator(device="cuda").manual_seed(42)
    B, L, Hq, Hkv, d, bs, topk = 12, 4096, 32, 4, 128, 64, 16
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev).to(torch.bfloat16)
    q, k, v = rnd(B, Hq, d), rnd(B, L, Hkv, d), rnd(B, L, Hkv, d)
    seqlens = (torch.arange(B, device=dev) * 331 + 1).clamp(max=L).to(torch.int32)
    seqlens = seqlens[torch.randperm(B, generator=g, device=dev)]
    a, b = pkg.ops.flash_attention_decode(q, k, v, seqlens), flash_attention_decode(q, k, v, seqlens)
    o = O.flash_attention_decode(q.float(), k.float(), v.float(), seqlens)
    judge("decode", "flash_attention_decode/o", a, b, o)
    clens = torch.where(seqlens < 32, torch.zeros_like(seqlens), (seqlens - 32) // 16 + 1)
    ck, cv = rnd(B, int(clens.max()), Hkv, d), rnd(B, int(clens.max()), Hkv, d)
    a, ia = pkg.ops.compressed_attention_decode(q, ck, cv, seqlens, clens, 32, 16, bs, topk)
    b, ib = compressed_attention_decode(q, ck, cv, seqlens, clens, 32, 16, bs, topk)
    o, io, sc = O.compressed_attention_decode(q.float(), ck.float(), cv.float(), seqlens, clens, 32, 16, bs, topk, return_scores=True)
    judge("decode", "compressed_attention_decode/o", a, b, o)
    bad, differing, rows = O.compare_topk_idx(ia, ib.to(torch.int32), sc, tie_tol=1e-3)
    _report["decode/topk_idx"] = dict(rows=rows, ours_rows_differing=differing, ours_rows_outside_tie=bad)
    assert bad == 0, (bad, differing, rows)
    a, b = pkg.ops.topk_sparse_attention_decode(q, k, v, ib.to(torch.int32), bs, seqlens), topk_sparse_attention_decode(
        q, k, v, ib.to(torch.int32), bs, seqlens)
    o = O.topk_sparse_attention_decode(q.float(), k.float(), v.float(), ib.to(torch.int32), bs, seqlens)
    judge("decode", "topk_sparse_attention_decode/o", a, b, o)
    assert pkg.device_status() == 0
