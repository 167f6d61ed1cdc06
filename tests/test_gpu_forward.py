"""Forward parity of the CUDA operators (through the C ABI) against the CPU oracle and the golden fixtures."""

import numpy as np
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import chain_inputs, load_golden, padded_cache

pytestmark = pytest.mark.gpu

MAX_TOL, MEAN_TOL = 2e-2, 2e-3  # bf16 tolerance on unit-variance data


@pytest.fixture(scope="module")
def ops():
    import native_sparse_attention_triton_b200 as pkg
    assert torch.cuda.is_available()
    return pkg.ops


def status_ok():
    import native_sparse_attention_triton_b200 as pkg
    return pkg.device_status() == 0


def dev(t, dtype=torch.bfloat16):
    return t.to(dtype).cuda() if t.is_floating_point() else t.cuda()


def close(test, ref, what, mx=MAX_TOL, mean=MEAN_TOL):
    """max |err| <= mx * max(1, |ref|) elementwise (a 16-bit result of magnitude 4..8 carries up to 3e-2 of
    representation error alone), mean |err| <= mean."""
    assert test.shape == ref.shape, (what, test.shape, ref.shape)
    t, r = test.float().cpu(), ref.float().cpu()
    err = (t - r).abs()
    worst = float((err / r.abs().clamp(min=1.0)).max()) if err.numel() else 0.0
    avg = float(err.mean()) if err.numel() else 0.0
    assert worst <= mx and avg <= mean, (what, worst, avg)


GOLDEN = ["mini_ragged", "cfg1", "g16_d128"]


@pytest.mark.parametrize("name", GOLDEN)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_compress_forward(ops, name, dtype):
    meta, x, gold = load_golden(name)
    ks, st = meta["ks"], meta["st"]
    cu = x["cu"].cuda()
    for key, fn, w, pe in (("lin_k", ops.linear_compress, x["wk"], x["pe"]),
                           ("lin_v", ops.linear_compress, x["wv"], None),
                           ("pool_k", ops.weightedpool_compress, x["wp"], x["pe"]),
                           ("avg_k", ops.avgpool_compress, None, x["pe"])):
        src = x["v"] if key == "lin_v" else x["k"]
        y, y_cu = fn(dev(src, dtype), dev(w, dtype) if w is not None else None, cu, ks, st,
                     dev(pe, dtype) if pe is not None else None)
        assert torch.equal(y_cu.cpu(), gold["cu_k"])
        close(y, gold[key], key)
    assert status_ok()


@pytest.mark.parametrize("name", GOLDEN)
def test_attention_chain_forward(ops, name):
    meta, x, gold = load_golden(name)
    ks, st, bs, T = meta["ks"], meta["st"], meta["bs"], meta["topk"]
    step = meta["row_step"]
    cu, cu_k = x["cu"].cuda(), gold["cu_k"].cuda()
    q, ck, cv = dev(x["q"]), dev(gold["lin_k"]), dev(gold["lin_v"])
    o, idx = ops.compressed_attention(q, ck, cv, ks, st, bs, T, cu, cu_k, None, None, None,
                                      meta["init_blocks"], meta["local_blocks"])
    close(o[::step], gold["o_cmp"], "o_cmp")
    _, _, sc = O.compressed_attention(x["q"], gold["lin_k"], gold["lin_v"], ks, st, bs, T, x["cu"], gold["cu_k"],
                                      init_blocks=meta["init_blocks"], local_blocks=meta["local_blocks"],
                                      return_scores=True)
    assert idx.dtype == torch.int32 and idx.shape == gold["topk_idx"].shape
    bad, differing, rows = O.compare_topk_idx(idx.cpu(), gold["topk_idx"], sc, tie_tol=1e-3)
    assert bad == 0, (bad, differing, rows)
    o_sel = ops.topk_sparse_attention(q, dev(x["k"]), dev(x["v"]), gold["topk_idx"].cuda(), bs, cu)
    close(o_sel[::step], gold["o_sel"], "o_sel")
    assert status_ok()


@pytest.mark.parametrize("name", GOLDEN)
def test_decode_forward(ops, name):
    meta, x, gold = load_golden(name)
    ks, st, bs, T = meta["ks"], meta["st"], meta["bs"], meta["topk"]
    seqlens = meta["seqlens"]
    cu = x["cu"]
    y_len, y_cu = O.compressed_seqlens(cu, ks, st)
    q_last = dev(x["q"][(cu[1:] - 1).long()])
    sl = torch.tensor(seqlens, dtype=torch.int32).cuda()
    ckc = dev(padded_cache(gold["lin_k"], y_cu, y_len.tolist(), int(y_len.max())))
    cvc = dev(padded_cache(gold["lin_v"], y_cu, y_len.tolist(), int(y_len.max())))
    o, idx = ops.compressed_attention_decode(q_last, ckc, cvc, sl, y_len.cuda(), ks, st, bs, T,
                                             meta["init_blocks"], meta["local_blocks"])
    close(o, gold["dec_o_cmp"], "dec_o_cmp")
    _, _, sc = O.compressed_attention_decode(x["q"][(cu[1:] - 1).long()], ckc.float().cpu(), cvc.float().cpu(),
                                             sl.cpu(), y_len, ks, st, bs, T, meta["init_blocks"], meta["local_blocks"],
                                             return_scores=True)
    bad, differing, rows = O.compare_topk_idx(idx.cpu(), gold["dec_idx"], sc, tie_tol=1e-3)
    assert bad == 0, (bad, differing, rows)
    kc, vc = dev(padded_cache(x["k"], cu, seqlens)), dev(padded_cache(x["v"], cu, seqlens))
    o_sel = ops.topk_sparse_attention_decode(q_last, kc, vc, gold["dec_idx"].cuda(), bs, sl)
    close(o_sel, gold["dec_o_sel"], "dec_o_sel")
    o_fl = ops.flash_attention_decode(q_last, kc, vc, sl)
    close(o_fl, gold["dec_o_flash"], "dec_o_flash")
    assert status_ok()


@pytest.mark.parametrize("Hq,Hkv,d,seqlens,topk", [
    (8, 2, 64, [70, 513, 31, 1024], 5),      # G = 4, a sequence shorter than the window
    (16, 2, 128, [300, 129], 4),             # G = 8
    (2, 2, 64, [257], 3),                    # G = 1
    (32, 2, 128, [1500, 700], 16),           # G = 16, top-16
])
def test_chain_forward_random(ops, Hq, Hkv, d, seqlens, topk):
    ks, st, bs = 32, 16, 64
    x = chain_inputs(123 + Hq + d, seqlens, Hq, Hkv, d, ks)
    cu = x["cu"].cuda()
    ck, cu_k = ops.linear_compress(dev(x["k"]), dev(x["wk"]), cu, ks, st, dev(x["pe"]))
    cv, _ = ops.linear_compress(dev(x["v"]), dev(x["wv"]), cu, ks, st, None)
    ck_ref, cu_k_ref = O.linear_compress(x["k"], x["wk"], x["cu"], ks, st, x["pe"])
    cv_ref, _ = O.linear_compress(x["v"], x["wv"], x["cu"], ks, st, None)
    assert torch.equal(cu_k.cpu(), cu_k_ref)
    close(ck, ck_ref, "ck")
    close(cv, cv_ref, "cv")
    o, idx = ops.compressed_attention(dev(x["q"]), ck, cv, ks, st, bs, topk, cu, cu_k)
    # oracle on the very tensors the kernel consumed
    o_ref, idx_ref, sc = O.compressed_attention(x["q"], ck.float().cpu(), cv.float().cpu(), ks, st, bs, topk, x["cu"],
                                                cu_k_ref, return_scores=True)
    close(o, o_ref, "o_cmp")
    bad, differing, rows = O.compare_topk_idx(idx.cpu(), idx_ref, sc, tie_tol=1e-3)
    assert bad == 0, (bad, differing, rows)
    o_sel = ops.topk_sparse_attention(dev(x["q"]), dev(x["k"]), dev(x["v"]), idx, bs, cu)
    o_sel_ref = O.topk_sparse_attention(x["q"], x["k"], x["v"], idx.cpu(), bs, x["cu"])
    close(o_sel, o_sel_ref, "o_sel")
    assert status_ok()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("Hq,Hkv,d", [(8, 2, 64), (32, 2, 128), (8, 8, 128)])   # G = 4 / 16 / 1, both head sizes
def test_flash_attention_varlen_forward(ops, causal, Hq, Hkv, d):
    x = chain_inputs(5, [100, 333, 64], Hq, Hkv, d, 32)
    cu = x["cu"].cuda()
    o = ops.flash_attention_varlen(dev(x["q"]), dev(x["k"]), dev(x["v"]), cu, cu, 333, 333, causal)
    o_ref = O.flash_attention_varlen(x["q"], x["k"], x["v"], x["cu"], x["cu"], causal=causal)
    close(o, o_ref, "flash")
    assert status_ok()


def test_decode_bandwidth_shapes(ops):
    """Ragged cache lengths, split-KV path (batch 12, cache 2048, 32q/4kv, d 128)."""
    g = torch.Generator().manual_seed(42)
    B, L, Hq, Hkv, d, bs, T = 12, 2048, 32, 4, 128, 64, 8
    seqlens = torch.clamp(torch.arange(B, dtype=torch.int32) * 190 + 1, max=L)
    q = torch.randn(B, Hq, d, generator=g).bfloat16().float()
    k = torch.randn(B, L, Hkv, d, generator=g).bfloat16().float()
    v = torch.randn(B, L, Hkv, d, generator=g).bfloat16().float()
    o = ops.flash_attention_decode(dev(q), dev(k), dev(v), seqlens.cuda())
    close(o, O.flash_attention_decode(q, k, v, seqlens), "flash_decode")
    nb = (seqlens.long() - 1) // bs + 1
    idx = torch.full((Hkv, B, T), -1, dtype=torch.int32)
    for h in range(Hkv):
        for b in range(B):
            n = int(nb[b])
            pick = torch.randperm(n, generator=g)[: min(T, n)].sort().values
            idx[h, b, : pick.numel()] = pick.int()
    o = ops.topk_sparse_attention_decode(dev(q), dev(k), dev(v), idx.cuda(), bs, seqlens.cuda())
    close(o, O.topk_sparse_attention_decode(q, k, v, idx, bs, seqlens), "sparse_decode")
    assert status_ok()


def test_decode_rows_without_visible_keys_are_zero(ops):
    """A sequence whose cache is still empty (seqlens 0), or whose selection is all padding, gets a zero output row from
    the kernel itself: the wrappers hand it uninitialised memory to write into."""
    g = torch.Generator().manual_seed(43)
    B, L, Hq, Hkv, d, bs, T = 5, 256, 16, 2, 128, 64, 4
    seqlens = torch.tensor([0, 1, 130, 0, 256], dtype=torch.int32)
    q = torch.randn(B, Hq, d, generator=g).bfloat16().float()
    k = torch.randn(B, L, Hkv, d, generator=g).bfloat16().float()
    v = torch.randn(B, L, Hkv, d, generator=g).bfloat16().float()
    live = seqlens > 0
    for _ in range(2):   # the second call writes into memory the first one left non-zero
        o = ops.flash_attention_decode(dev(q), dev(k), dev(v), seqlens.cuda())
        assert float(o[~live.cuda()].float().abs().max()) == 0.0
        close(o[live.cuda()], O.flash_attention_decode(q[live], k[live], v[live], seqlens[live]), "flash_decode")
    idx = torch.full((Hkv, B, T), -1, dtype=torch.int32)
    idx[:, 2, :3] = torch.tensor([0, 1, 2], dtype=torch.int32)
    idx[:, 4, :2] = torch.tensor([1, 3], dtype=torch.int32)
    picked = torch.tensor([False, False, True, False, True])
    for _ in range(2):
        o = ops.topk_sparse_attention_decode(dev(q), dev(k), dev(v), idx.cuda(), bs, seqlens.cuda())
        assert float(o[~picked.cuda()].float().abs().max()) == 0.0
        close(o[picked.cuda()], O.topk_sparse_attention_decode(q[picked], k[picked], v[picked], idx[:, picked], bs, seqlens[picked]),
              "sparse_decode")
    assert status_ok()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("H,seqlens,ks,st", [
    (2, [5000, 37, 2992], 32, 16),     # 8029 tokens: the last windows end in the 13 tokens only the shifted TMA view reaches
    (4, [4103], 64, 16),               # one sequence, four taps per stride group
    (2, [300, 4500], 16, 16),          # windows that do not overlap
    (1, [6000, 129], 32, 8),           # stride 8; a short sequence after a long one
])
def test_linear_compress_tensor_core_path(ops, dtype, H, seqlens, ks, st):
    """head_dim 128 with at least 128 windows in a sequence and enough tokens runs as one tcgen05 GEMM per (sequence, head)
    whose operands TMA fetches through a [token / stride][token % stride] view of x: against the oracle, with and without
    the position embedding, and on a strided view of x (heads sliced out of a wider tensor)."""
    d = 128
    x = chain_inputs(77 + ks + st, seqlens, H, H, d, ks)
    cu = x["cu"].cuda()
    wide = torch.randn(sum(seqlens), H + 2, d, generator=torch.Generator().manual_seed(3)).to(dtype).cuda()
    wide[:, 1:H + 1] = dev(x["k"], dtype)
    for src, w, pe in ((dev(x["k"], dtype), x["wk"], x["pe"]), (wide[:, 1:H + 1], x["wk"], x["pe"]), (dev(x["v"], dtype), x["wv"], None)):
        y, y_cu = ops.linear_compress(src, dev(w, dtype), cu, ks, st, dev(pe, dtype) if pe is not None else None)
        ref_in = x["v"] if pe is None else x["k"]
        y_ref, y_cu_ref = O.linear_compress(ref_in.to(dtype).float(), w.to(dtype).float(), x["cu"], ks, st,
                                            pe.to(dtype).float() if pe is not None else None)
        assert torch.equal(y_cu.cpu(), y_cu_ref.to(torch.int32))
        close(y, y_ref, "linear_compress")
    assert status_ok()


def test_linear_compress_many_waves_of_ctas(ops):
    """A problem of several waves of CTAs: 310 005 tokens, four heads, the last windows ending on the last token (shifted
    TMA view).  The oracle runs on the GPU in fp32."""
    H, d, ks, st = 4, 128, 32, 16
    seqlens = [200005, 110000]
    g = torch.Generator().manual_seed(91)
    N = sum(seqlens)
    x = torch.randn(N, H, d, generator=g).bfloat16()
    w = (torch.randn(H, ks * d, d, generator=g) / (ks * d) ** 0.5).bfloat16()
    pe = (torch.randn(H, ks, d, generator=g) * 0.02).bfloat16()
    cu = torch.tensor([0, seqlens[0], N], dtype=torch.int32).cuda()
    y, y_cu = ops.linear_compress(x.cuda(), w.cuda(), cu, ks, st, pe.cuda())
    y_ref, y_cu_ref = O.linear_compress(x.cuda().float(), w.cuda().float(), cu, ks, st, pe.cuda().float())
    assert torch.equal(y_cu.cpu(), y_cu_ref.cpu().to(torch.int32))
    close(y, y_ref, "linear_compress")
    assert status_ok()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("H,seqlens,ks,st", [
    (4, [150000, 33, 70007], 32, 16),    # 13 748 windows; a sequence without a window in the middle
    (2, [140000], 32, 16),               # two heads per chunk, eight windows at a time
    (3, [135001, 9000], 64, 16),         # three heads: the second head block is half empty; four chunks per window
    (1, [70000, 70000], 16, 16),         # windows that do not overlap
])
def test_pool_compress_streaming_path(ops, dtype, H, seqlens, ks, st):
    """Inputs of 8192 windows or more (head_dim 128) stream through shared memory in TMA chunks: weighted and average pooling,
    with and without the position embedding, and on a view of x whose heads are sliced out of a wider tensor.  The oracle runs
    on the GPU in fp32."""
    d = 128
    g = torch.Generator().manual_seed(200 + H + ks)
    N = sum(seqlens)
    x = torch.randn(N, H, d, generator=g).to(dtype).cuda()
    wide = torch.randn(N, H + 2, d, generator=g).to(dtype).cuda()
    wide[:, 1:H + 1] = x
    w = (torch.rand(H, ks, generator=g) / ks).to(dtype).cuda()
    pe = (torch.randn(H, ks, d, generator=g) * 0.02).to(dtype).cuda()
    cu = torch.tensor([0] + list(np.cumsum(seqlens)), dtype=torch.int32).cuda()
    for src, fn, ofn, wt, pos in ((x, ops.weightedpool_compress, O.weightedpool_compress, w, pe),
                                  (wide[:, 1:H + 1], ops.weightedpool_compress, O.weightedpool_compress, w, None),
                                  (x, ops.avgpool_compress, O.avgpool_compress, None, pe)):
        y, y_cu = fn(src, wt, cu, ks, st, pos)
        if wt is None:
            y_ref, y_cu_ref = ofn(x.float(), None, cu, ks, st, pos.float() if pos is not None else None)
        else:
            y_ref, y_cu_ref = ofn(x.float(), wt.float(), cu, ks, st, pos.float() if pos is not None else None)
        assert torch.equal(y_cu.cpu(), y_cu_ref.cpu().to(torch.int32))
        close(y, y_ref, "pool_compress")
    assert status_ok()
