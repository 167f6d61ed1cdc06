"""The CUDA kernels against outputs of the REFERENCE ITSELF recorded on a B200 (tests/golden/box_*.npz, written by
tests/golden/make_golden_on_box.py): its Triton operators (forward and backward of the chain), flash_attn's
sliding-window call, its RotaryEmbedding, and its nsa_infer + NSACache over a prefill and a run of decode steps.
These run wherever the library runs; the reference does not have to be present."""
import numpy as np
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import (box_fixture, chain_inputs, close_16bit, from_bits, from_bits16, grad_tol, infer_case_inputs,
                           rope_case_inputs, rope_tolerance, window_case_inputs)

pytestmark = pytest.mark.gpu
# gradients of the recorded chain passed through the reference's 16-bit torch linear_compress (its Triton kernel does not
# compile under Triton 3.6, see tests/refbox.py), whose autograd rounds every intermediate: mean error up to 2.8e-3 against fp32
REF_GRAD_MEAN_TOL = 4e-3
DEV = torch.device("cuda")


@pytest.fixture(scope="module")
def pkg():
    import native_sparse_attention_triton_b200 as p
    assert torch.cuda.is_available()
    return p


def need(name):
    z = box_fixture(name)
    if z is None:
        pytest.skip(f"tests/golden/{name}.npz has not been generated")
    return z


@pytest.mark.parametrize("name", ["box_triton_cfg1", "box_triton_g16_d128"])
def test_chain_matches_reference_triton(pkg, name):
    z = need(name)
    m = {k: (z[k].tolist() if z[k].ndim else z[k].item()) for k in ("seed", "seqlens", "Hq", "Hkv", "d", "ks", "st", "bs", "topk",
                                                                    "init_blocks", "local_blocks", "row_step")}
    inp = chain_inputs(m["seed"], m["seqlens"], m["Hq"], m["Hkv"], m["d"], m["ks"])
    g = torch.Generator().manual_seed(m["seed"] + 1000)
    N = sum(m["seqlens"])
    do_cmp = torch.randn(N, m["Hq"], m["d"], generator=g).bfloat16().to(DEV)
    do_sel = torch.randn(N, m["Hq"], m["d"], generator=g).bfloat16().to(DEV)
    t = {n: inp[n].bfloat16().to(DEV).requires_grad_(True) for n in ("q", "k", "v", "wk", "wv", "pe")}
    cu, rs, ops = inp["cu"].to(DEV), m["row_step"], pkg.ops
    ck, cu_k = ops.linear_compress(t["k"], t["wk"], cu, m["ks"], m["st"], t["pe"])
    cv, _ = ops.linear_compress(t["v"], t["wv"], cu, m["ks"], m["st"], None)
    assert torch.equal(cu_k.cpu(), torch.from_numpy(z["cu_k"]).to(torch.int32))
    o_cmp, idx = ops.compressed_attention(t["q"], ck, cv, m["ks"], m["st"], m["bs"], m["topk"], cu, cu_k, max(m["seqlens"]),
                                          None, None, m["init_blocks"], m["local_blocks"])
    ref_idx = torch.from_numpy(z["topk_idx"].astype(np.int32))
    bad, differing, rows = O.compare_topk_idx(idx.cpu(), ref_idx, torch.from_numpy(z["block_score"]), tie_tol=1e-3)
    print(name, "topk_idx rows differing", differing, "outside the tie band", bad, "of", rows)
    assert bad == 0, (bad, differing, rows)
    o_sel = ops.topk_sparse_attention(t["q"], t["k"], t["v"], ref_idx.to(DEV), m["bs"], cu)
    torch.autograd.backward([o_cmp, o_sel], [do_cmp, do_sel])
    checks = [(ck, "lin_k"), (cv, "lin_v"), (o_cmp[::rs], "o_cmp"), (o_sel[::rs], "o_sel"), (t["q"].grad[::rs], "dq"),
              (t["k"].grad, "dk"), (t["v"].grad, "dv"), (t["wk"].grad[:, ::8], "dwk"), (t["wv"].grad[:, ::8], "dwv"),
              ]
    # d(pe) is left out: the bias it produces shifts every compressed key by the same vector, which the softmax cannot see,
    # so its exact gradient is zero and what either implementation returns is rounding noise
    for a, b in checks:
        ok, mx, mean = close_16bit(a, from_bits(z[b]), grad_tol(b, chain=True),
                                   REF_GRAD_MEAN_TOL if b.startswith("d") else 2e-3)
        print(name, b, "max", mx, "mean", mean)
        assert ok, (b, mx, mean)
    assert pkg.device_status() == 0


def test_sliding_window_matches_flash_attn(pkg):
    z = need("box_window")
    for W in (64, 512):
        inp = window_case_inputs()
        q, k, v = (inp[n].bfloat16().to(DEV).requires_grad_(True) for n in ("q", "k", "v"))
        L = int((inp["cu"][1:] - inp["cu"][:-1]).max())
        o = pkg.ops.sliding_window_attention(q, k, v, inp["cu"].to(DEV), L, W)
        o.backward(inp["do"].bfloat16().to(DEV))
        for a, b in ((o[::8], f"o_w{W}"), (q.grad[::8], f"dq_w{W}"), (k.grad[::4], f"dk_w{W}"), (v.grad[::4], f"dv_w{W}")):
            ok, mx, mean = close_16bit(a, from_bits(z[b]), grad_tol(b[:2]))
            print(b, "max", mx, "mean", mean)
            assert ok, (b, mx, mean)
    assert pkg.device_status() == 0


def test_rope_matches_reference_rotary_embedding(pkg):
    z = need("box_rope")
    inp = rope_case_inputs()
    for tag in ("f8", "f4"):
        inv_freq, scaling = torch.from_numpy(z[f"inv_freq_{tag}"]).to(DEV), float(z[f"scaling_{tag}"])
        for dt, dec, dn in ((torch.bfloat16, from_bits, "bf16"), (torch.float16, from_bits16, "fp16")):
            ulp = 2.0 ** (-7 if dn == "bf16" else -10)
            cases = [("prefill", inp["x"], inp["cu"], 0, 1, 4), ("strided", inp["xc"], inp["cu_c"], 0, 16, 1),
                     ("decode3", inp["xd"], inp["cu"], 3, 1, 1), ("decode1s", inp["xd"], inp["cu_c"], 1, 16, 1)]
            for nm, x, cu, step, stride, rs in cases:
                got = pkg.ops.rope(x.to(dt).to(DEV), inv_freq, cu.to(DEV), step, stride, scaling).float().cpu()[::rs]
                want = dec(z[f"{nm}_{tag}_{dn}"])
                # one more unit for the device's cos/sin, which may round to the neighbouring table value
                excess = ((got - want).abs() - rope_tolerance(x.to(dt).float()[::rs], want, ulp, extra=1.0)).max()
                assert float(excess) <= 0, (tag, dn, nm, float(excess))
    assert pkg.device_status() == 0


@pytest.mark.parametrize("name,mode,lens,steps", [("box_infer_weighted", "weighted", [33, 200], 24),
                                                  ("box_infer_linear", "linear", [40, 100, 300], 40)])
def test_inference_matches_reference(pkg, name, mode, lens, steps):
    from native_sparse_attention_triton_b200.infer import RotaryEmbedding, nsa_infer
    from native_sparse_attention_triton_b200.kv_cache import NSACache
    z = need(name)
    c = infer_case_inputs(mode, lens, steps)
    P = c["params"]
    rope = RotaryEmbedding(torch.from_numpy(z["inv_freq"]).to(DEV), float(z["scaling"]))
    cache = NSACache(P["MAXB"], P["MAXLEN"], P["HKV"], P["D"], P["KS"], P["ST"], P["W"], torch.bfloat16, DEV)
    fn = {"linear": pkg.ops.linear_compress, "weighted": pkg.ops.weightedpool_compress}[mode]
    dv = lambda x: None if x is None else x.bfloat16().to(DEV)
    args = dict(rope=rope, cache=cache, compress_weight=(dv(c["w_k"]), dv(c["w_v"])), compress_func=(fn, fn),
                intra_block_pe=dv(c["pe"]), kernel_size=P["KS"], kernel_stride=P["ST"], block_size=P["BS"], topk=P["TOPK"],
                init_blocks=P["INIT"], local_blocks=P["LOCAL"], window_size=P["W"])
    cu = c["cu"].to(DEV)
    out = nsa_infer(cu, 0, dv(c["q"]), dv(c["k"]), dv(c["v"]), dv(c["gate"]), **args)
    ok, mx, mean = close_16bit(out, from_bits(z["prefill"]), 4e-2, 3e-3)
    assert ok, ("prefill", mx, mean)
    dec = from_bits(z["decode"])
    off = 0
    for step in range(1, steps + 1):
        qn, kn, vn, gn = c["steps"][step - 1]
        out = nsa_infer(cu, step, dv(qn), dv(kn), dv(vn), dv(gn), **args)
        for b in range(len(lens)):
            ok, mx, mean = close_16bit(out[b], dec[step - 1, b], 4e-2, 3e-3)
            off += not ok
            assert mx <= 0.5, (step, b, mx, mean)
    assert off <= max(1, steps * len(lens) // 25), off
    B = len(lens)
    assert cache.sparse_kv_len[:B].cpu().tolist() == z["sparse_len"].tolist()
    assert cache.compress_kv_len[:B].cpu().tolist() == z["compress_len"].tolist()
    assert cache.before_compress_kv_len[:B].cpu().tolist() == z["stage_len"].tolist()
    assert torch.clamp(cache.sliding_kv_len[:B], max=P["W"]).cpu().tolist() == np.minimum(z["sliding_len"], P["W"]).tolist()
    assert pkg.device_status() == 0
