"""Operator chain forward + backward on seeded random configurations (head counts, group sizes 1..16, head_dim 64/128,
kernel sizes / strides / block sizes, ragged batches with sequences shorter than a window, top-k, bf16 / fp16) against
the fp32 CPU oracle.  The fixed cases of the other test files pin known corners; this one walks the space between."""
import math
import random

import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import CHAIN_GRAD_MEAN_TOL, assert_close_16bit, grad_tol

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg():
    import native_sparse_attention_triton_b200 as pkg
    assert torch.cuda.is_available()
    return pkg


def draw(seed):
    rnd = random.Random(seed)
    d = rnd.choice([64, 128, 128])
    Hkv = rnd.choice([1, 2, 4])
    G = rnd.choice([1, 2, 4, 8, 16])
    ks, st, bs = rnd.choice([(32, 16, 64), (16, 8, 64), (64, 16, 128), (32, 32, 64), (16, 16, 64), (64, 32, 128), (32, 8, 64)])
    nseq = rnd.choice([1, 2, 3, 5])
    seqlens = [rnd.choice([rnd.randint(1, 40), rnd.randint(60, 700), rnd.randint(700, 1500)]) for _ in range(nseq)]
    topk = rnd.choice([3, 4, 8, 16])
    dtype = rnd.choice([torch.bfloat16, torch.bfloat16, torch.float16])
    return d, Hkv, Hkv * G, ks, st, bs, seqlens, topk, dtype


def fwd_close(t, r, what):
    assert_close_16bit(t, r, what)


def grad_close(t, r, what):
    """a gradient the oracle's autograd leaves undefined (no compressed key anywhere) must be zero here"""
    r = torch.zeros(t.shape) if r is None else r
    assert_close_16bit(t, r, what, grad_tol(what, chain=True), CHAIN_GRAD_MEAN_TOL)


@pytest.mark.parametrize("seed", range(24))
def test_chain_random_configuration(pkg, seed):
    ops = pkg.ops
    d, Hkv, Hq, ks, st, bs, seqlens, topk, dtype = draw(seed)
    g = torch.Generator().manual_seed(1000 + seed)
    N = sum(seqlens)
    cu = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32)
    rb = lambda t: t.to(dtype).float()   # values exactly representable in the 16-bit type
    q, k, v = (rb(torch.randn(N, h, d, generator=g)) for h in (Hq, Hkv, Hkv))
    wk, wv = (rb(torch.randn(Hkv, ks * d, d, generator=g) / math.sqrt(ks * d)) for _ in range(2))
    pe = rb(torch.randn(Hkv, ks, d, generator=g) * 0.02)
    do1, do2 = (rb(torch.randn(N, Hq, d, generator=g)) for _ in range(2))

    leaf = lambda t: t.to(dtype).cuda().requires_grad_(True)
    qg, kg, vg, wkg, wvg, peg = (leaf(t) for t in (q, k, v, wk, wv, pe))
    cug = cu.cuda()
    ck, cu_k = ops.linear_compress(kg, wkg, cug, ks, st, peg)
    cv, _ = ops.linear_compress(vg, wvg, cug, ks, st, None)
    o1, idx = ops.compressed_attention(qg, ck, cv, ks, st, bs, topk, cug, cu_k, max(seqlens), None, None, 1, 2)
    o2 = ops.topk_sparse_attention(qg, kg, vg, idx, bs, cug)
    torch.autograd.backward([o1, o2], [do1.to(dtype).cuda(), do2.to(dtype).cuda()])

    ref = lambda t: t.clone().requires_grad_(True)
    qr, kr, vr, wkr, wvr, per = (ref(t) for t in (q, k, v, wk, wv, pe))
    ckr, cu_kr = O.linear_compress(kr, wkr, cu, ks, st, per)
    cvr, _ = O.linear_compress(vr, wvr, cu, ks, st, None)
    fwd_close(ck, ckr, "ck")
    fwd_close(cv, cvr, "cv")
    assert torch.equal(cu_k.cpu(), cu_kr)
    # the oracle's attention sees the compressed keys and values the kernels produced (16-bit), so that the selection is
    # compared on identical scores; its gradients still flow into its own compression (straight-through difference)
    ckr = ckr + (ck.detach().float().cpu() - ckr).detach()
    cvr = cvr + (cv.detach().float().cpu() - cvr).detach()
    o1r, idxr, sc = O.compressed_attention(qr, ckr, cvr, ks, st, bs, topk, cu, cu_kr, init_blocks=1, local_blocks=2,
                                           return_scores=True)
    fwd_close(o1, o1r, "o_cmp")
    if idxr is not None:
        bad, differing, rows = O.compare_topk_idx(idx.cpu(), idxr, sc, 1e-3)
        assert bad == 0, (bad, differing, rows)
    o2r = O.topk_sparse_attention(qr, kr, vr, idx.cpu(), bs, cu)
    fwd_close(o2, o2r, "o_sel")
    torch.autograd.backward([o1r, o2r], [do1, do2])
    for name, a_, b_ in (("dq", qg, qr), ("dk", kg, kr), ("dv", vg, vr), ("dwk", wkg, wkr), ("dwv", wvg, wvr)):
        grad_close(a_.grad, b_.grad, name)
    assert pkg.device_status() == 0
