"""Backward parity of the trainable operators against autograd over the fp32 CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import CHAIN_GRAD_MEAN_TOL, MEAN_TOL, assert_close_16bit, chain_inputs, grad_tol

pytestmark = pytest.mark.gpu



@pytest.fixture(scope="module")
def ops():
    import native_sparse_attention_triton_b200 as pkg
    assert torch.cuda.is_available()
    return pkg.ops


def status_ok():
    import native_sparse_attention_triton_b200 as pkg
    return pkg.device_status() == 0


def close(test, ref, what, chain=False):
    """The acceptance rule of tests/helpers.py; key/value gradients of the attention operators get their own worst-element
    bound, gradients of a chain of operators (chain=True) their own mean bound."""
    assert_close_16bit(test, ref, what, grad_tol(what, chain), CHAIN_GRAD_MEAN_TOL if chain else MEAN_TOL)


def leaf(t, dtype=torch.bfloat16):
    return t.to(dtype).cuda().requires_grad_(True)


def ref_leaf(t):
    return t.clone().requires_grad_(True)


CASES = [
    (8, 2, 64, [70, 513, 31, 300], 5),    # G = 4, a sequence shorter than the window
    (16, 2, 128, [300, 129], 4),          # G = 8
    (32, 2, 128, [700, 260], 16),         # G = 16, top-16
    (2, 2, 64, [257], 3),                 # G = 1
]


@pytest.mark.parametrize("Hq,Hkv,d,seqlens,topk", CASES)
def test_sparse_attention_backward(ops, Hq, Hkv, d, seqlens, topk):
    ks, st, bs = 32, 16, 64
    x = chain_inputs(77 + Hq, seqlens, Hq, Hkv, d, ks)
    g = torch.Generator().manual_seed(5)
    cu = x["cu"]
    # selection from the oracle on average-pooled keys keeps this test independent of the compression kernels
    ck, cu_k = O.avgpool_compress(x["k"], None, cu, ks, st)
    _, idx = O.compressed_attention(x["q"], ck, ck, ks, st, bs, topk, cu, cu_k)
    do = torch.randn(x["q"].shape, generator=g).bfloat16().float()
    q, k, v = leaf(x["q"]), leaf(x["k"]), leaf(x["v"])
    o = ops.topk_sparse_attention(q, k, v, idx.cuda(), bs, cu.cuda())
    o.backward(do.bfloat16().cuda())
    qr, kr, vr = ref_leaf(x["q"]), ref_leaf(x["k"]), ref_leaf(x["v"])
    o_ref = O.topk_sparse_attention(qr, kr, vr, idx, bs, cu)
    o_ref.backward(do)
    close(q.grad, qr.grad, "dq")
    close(k.grad, kr.grad, "dk")
    close(v.grad, vr.grad, "dv")
    assert status_ok()


@pytest.mark.parametrize("Hq,Hkv,d,seqlens,topk", CASES)
def test_compressed_attention_backward(ops, Hq, Hkv, d, seqlens, topk):
    ks, st, bs = 32, 16, 64
    x = chain_inputs(91 + Hq, seqlens, Hq, Hkv, d, ks)
    g = torch.Generator().manual_seed(6)
    cu = x["cu"]
    ck, cu_k = O.avgpool_compress(x["k"], None, cu, ks, st)
    cv, _ = O.avgpool_compress(x["v"], None, cu, ks, st)
    ck, cv = ck.bfloat16().float(), cv.bfloat16().float()
    do = torch.randn(x["q"].shape, generator=g).bfloat16().float()
    q, k, v = leaf(x["q"]), leaf(ck), leaf(cv)
    o, _ = ops.compressed_attention(q, k, v, ks, st, bs, topk, cu.cuda(), cu_k.cuda())
    o.backward(do.bfloat16().cuda())
    qr, kr, vr = ref_leaf(x["q"]), ref_leaf(ck), ref_leaf(cv)
    o_ref, _ = O.compressed_attention(qr, kr, vr, ks, st, bs, topk, cu, cu_k)
    o_ref.backward(do)
    close(q.grad, qr.grad, "dq")
    close(k.grad, kr.grad, "dck")
    close(v.grad, vr.grad, "dcv")
    assert status_ok()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("Hq,Hkv,d", [(8, 2, 64), (32, 2, 128), (8, 8, 128)])   # G = 4 / 16 / 1, both head sizes
def test_flash_attention_backward(ops, causal, Hq, Hkv, d):
    x = chain_inputs(5, [100, 333, 64], Hq, Hkv, d, 32)
    g = torch.Generator().manual_seed(7)
    cu = x["cu"]
    do = torch.randn(x["q"].shape, generator=g).bfloat16().float()
    q, k, v = leaf(x["q"]), leaf(x["k"]), leaf(x["v"])
    o = ops.flash_attention_varlen(q, k, v, cu.cuda(), cu.cuda(), 333, 333, causal)
    o.backward(do.bfloat16().cuda())
    qr, kr, vr = ref_leaf(x["q"]), ref_leaf(x["k"]), ref_leaf(x["v"])
    O.flash_attention_varlen(qr, kr, vr, cu, cu, causal=causal).backward(do)
    close(q.grad, qr.grad, "dq")
    close(k.grad, kr.grad, "dk")
    close(v.grad, vr.grad, "dv")
    assert status_ok()


@pytest.mark.parametrize("H,d,seqlens", [(2, 64, [20, 100, 200]), (4, 128, [12, 1000, 517]), (2, 128, [2048])])
@pytest.mark.parametrize("mode", ["linear", "linear_nope", "weighted", "avg"])
def test_compress_backward(ops, H, d, seqlens, mode):
    ks, st = 32, 16
    x = chain_inputs(31 + d, seqlens, H, H, d, ks)
    g = torch.Generator().manual_seed(8)
    cu = x["cu"]
    xin = x["k"]
    pe = None if mode == "linear_nope" else x["pe"]
    if mode.startswith("linear"):
        w, fn, fn_ref = x["wk"], ops.linear_compress, O.linear_compress
    elif mode == "weighted":
        w, fn, fn_ref = x["wp"], ops.weightedpool_compress, O.weightedpool_compress
    else:
        w, fn, fn_ref = None, ops.avgpool_compress, O.avgpool_compress
    xt = leaf(xin)
    wt = leaf(w) if w is not None else None
    pt = leaf(pe) if pe is not None else None
    y, y_cu = fn(xt, wt, cu.cuda(), ks, st, pt)
    dy = torch.randn(y.shape, generator=g).bfloat16().float()
    y.backward(dy.bfloat16().cuda())
    xr = ref_leaf(xin)
    wr = ref_leaf(w) if w is not None else None
    pr = ref_leaf(pe) if pe is not None else None
    y_ref, _ = fn_ref(xr, wr, cu, ks, st, pr)
    y_ref.backward(dy)
    close(xt.grad, xr.grad, "dx")
    if w is not None:
        close(wt.grad, wr.grad, "dw")
    if pe is not None:
        close(pt.grad, pr.grad, "dpe")
    assert status_ok()


def test_chain_backward_cfg_like(ops):
    """The whole operator chain with gradients flowing into the compression weights (G = 16, d = 128)."""
    Hq, Hkv, d, ks, st, bs, topk = 32, 2, 128, 32, 16, 64, 8
    seqlens = [640, 1100]
    x = chain_inputs(3, seqlens, Hq, Hkv, d, ks)
    g = torch.Generator().manual_seed(9)
    cu = x["cu"]
    do1 = torch.randn(x["q"].shape, generator=g).bfloat16().float()
    do2 = torch.randn(x["q"].shape, generator=g).bfloat16().float()
    names = ["q", "k", "v", "wk", "wv", "pe"]
    t = {n: leaf(x[n]) for n in names}
    ck, cu_k = ops.linear_compress(t["k"], t["wk"], cu.cuda(), ks, st, t["pe"])
    cv, _ = ops.linear_compress(t["v"], t["wv"], cu.cuda(), ks, st, None)
    o1, idx = ops.compressed_attention(t["q"], ck, cv, ks, st, bs, topk, cu.cuda(), cu_k)
    o2 = ops.topk_sparse_attention(t["q"], t["k"], t["v"], idx, bs, cu.cuda())
    ((o1.float() * do1.cuda()).sum() + (o2.float() * do2.cuda()).sum()).backward()
    r = {n: ref_leaf(x[n]) for n in names}
    ck_r, cu_k_r = O.linear_compress(r["k"], r["wk"], cu, ks, st, r["pe"])
    cv_r, _ = O.linear_compress(r["v"], r["wv"], cu, ks, st, None)
    o1_r, _ = O.compressed_attention(r["q"], ck_r, cv_r, ks, st, bs, topk, cu, cu_k_r)
    o2_r = O.topk_sparse_attention(r["q"], r["k"], r["v"], idx.cpu(), bs, cu)
    ((o1_r * do1).sum() + (o2_r * do2).sum()).backward()
    # d(pe) is excluded here: the pe bias shifts every compressed key by the same vector, which the softmax
    # cannot see, so its exact gradient is zero and only rounding noise remains (test_compress_backward covers dpe)
    for n in names[:-1]:
        close(t[n].grad, r[n].grad, "d" + n, chain=True)
    assert status_ok()


@pytest.mark.parametrize("H,seqlens,ks,st", [
    (4, [100000, 20, 45003, 31], 32, 16),   # sequences without a window (their dx is zero), a ragged tail
    (2, [140000], 32, 16),
    (3, [120001, 15000], 16, 16),           # three heads (half-empty second head block); windows that do not overlap
    (4, [135000], 32, 8),                   # stride 8: four windows over every token
])
@pytest.mark.parametrize("mode,dtype", [("weighted", torch.bfloat16), ("avg", torch.bfloat16), ("weighted", torch.float16)])
def test_pool_compress_backward_streaming_path(ops, H, seqlens, ks, st, mode, dtype):
    """Inputs of 131 072 tokens or more (head_dim 128, kernel <= 32) take the one-pass backward: dx written once, x and dy
    read once, dw from per-(CTA, group) partial rows added in a fixed order.  Against autograd through the oracle, run on the
    GPU in fp32; dw is a sum over ~10^7 products, compared relative to its own size."""
    d = 128
    g = torch.Generator().manual_seed(300 + H + ks + st)
    N = sum(seqlens)
    cu = torch.tensor([0] + list(np.cumsum(seqlens)), dtype=torch.int32).cuda()
    xb = torch.randn(N, H, d, generator=g).to(dtype)
    wb = (torch.rand(H, ks, generator=g) / ks).to(dtype)
    peb = (torch.randn(H, ks, d, generator=g) * 0.02).to(dtype)
    x, pe = xb.cuda().requires_grad_(True), peb.cuda().requires_grad_(True)
    w = wb.cuda().requires_grad_(True) if mode == "weighted" else None
    fn = ops.weightedpool_compress if mode == "weighted" else ops.avgpool_compress
    y, _ = fn(x, w, cu, ks, st, pe)
    dy = torch.randn(y.shape, generator=g).to(dtype).cuda()
    y.backward(dy)
    xr, per = xb.cuda().float().requires_grad_(True), peb.cuda().float().requires_grad_(True)
    wr = wb.cuda().float().requires_grad_(True) if mode == "weighted" else None
    ofn = O.weightedpool_compress if mode == "weighted" else O.avgpool_compress
    yr, _ = ofn(xr, wr, cu, ks, st, per)
    yr.backward(dy.float())
    close(x.grad, xr.grad, "dx")
    # tokens no window covers (sequences shorter than the kernel, ragged tails) get exact zeros
    assert float(x.grad[xr.grad == 0].float().abs().max()) == 0.0
    close(pe.grad, per.grad, "dpe")
    if mode == "weighted":
        rel = (w.grad.float() - wr.grad).abs().max() / wr.grad.abs().max()
        assert float(rel) <= 1e-2, float(rel)
    assert status_ok()
