"""BASELINE configurations 2 and 3 at their stated shapes against the fp32 oracle (evaluated on the same device in true
fp32: cuBLAS tensor-float math is off by default for torch matmuls, and the oracle processes one KV head and 1024 query
rows at a time, so an 8192-token sequence of 64 heads needs about 1 GB).  The reference does not have to be present.

  configuration 2: operator chain forward + backward, cu_seqlens = [0, 1024, 8192, 16384], 64q/4kv heads, d = 128,
                   kernel 32 / stride 16, block 64, top-16, bf16.
  configuration 3: topk_sparse_attention forward + backward on one sequence, N = 8192, 64q/4kv heads, d = 128, block 64,
                   top-8, the selection produced by compressed_attention on N(0,1) q/k.
"""
import math

import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import CHAIN_GRAD_MEAN_TOL, assert_close_16bit, grad_tol

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")


@pytest.fixture(scope="module")
def pkg():
    import native_sparse_attention_triton_b200 as p
    assert torch.cuda.is_available()
    return p


def leaf(t, dtype=None):
    t = t.detach().clone() if dtype is None else t.detach().to(dtype)
    return t.requires_grad_(True)


def test_configuration_2_chain_forward_backward(pkg):
    ops = pkg.ops
    seqlens, Hq, Hkv, d, ks, st, bs, topk = [1024, 7168, 8192], 64, 4, 128, 32, 16, 64, 16
    N = sum(seqlens)
    g = torch.Generator(device=DEV).manual_seed(44)
    rnd = lambda *s, scale=1.0: (torch.randn(*s, generator=g, device=DEV) * scale).to(torch.bfloat16)
    x = dict(q=rnd(N, Hq, d), k=rnd(N, Hkv, d), v=rnd(N, Hkv, d), wk=rnd(Hkv, ks * d, d, scale=1 / math.sqrt(ks * d)),
             wv=rnd(Hkv, ks * d, d, scale=1 / math.sqrt(ks * d)), pe=rnd(Hkv, ks, d, scale=0.02))
    do1, do2 = rnd(N, Hq, d), rnd(N, Hq, d)
    cu = torch.tensor([0, 1024, 8192, 16384], dtype=torch.int32, device=DEV)
    t = {n: leaf(v) for n, v in x.items()}
    ck, cu_k = ops.linear_compress(t["k"], t["wk"], cu, ks, st, t["pe"])
    cv, _ = ops.linear_compress(t["v"], t["wv"], cu, ks, st, None)
    o1, idx = ops.compressed_attention(t["q"], ck, cv, ks, st, bs, topk, cu, cu_k)
    o2 = ops.topk_sparse_attention(t["q"], t["k"], t["v"], idx, bs, cu)
    torch.autograd.backward([o1, o2], [do1, do2])

    r = {n: leaf(v, torch.float32) for n, v in x.items()}
    ck_r, cu_k_r = O.linear_compress(r["k"], r["wk"], cu, ks, st, r["pe"])
    cv_r, _ = O.linear_compress(r["v"], r["wv"], cu, ks, st, None)
    assert torch.equal(cu_k.cpu(), cu_k_r.cpu())
    assert_close_16bit(ck, ck_r, "compressed k")
    assert_close_16bit(cv, cv_r, "compressed v")
    # the oracle's attention sees the kernels' 16-bit compressed tensors, so that selection is compared on equal scores
    ck_r = ck_r + (ck.detach().float() - ck_r).detach()
    cv_r = cv_r + (cv.detach().float() - cv_r).detach()
    o1_r, idx_r, sc = O.compressed_attention(r["q"], ck_r, cv_r, ks, st, bs, topk, cu, cu_k_r, return_scores=True)
    bad, differing, rows = O.compare_topk_idx(idx, idx_r, sc, tie_tol=1e-3)
    print("configuration 2: topk_idx rows differing", differing, "outside the tie band", bad, "of", rows)
    assert bad == 0, (bad, differing, rows)
    o2_r = O.topk_sparse_attention(r["q"], r["k"], r["v"], idx, bs, cu)
    assert_close_16bit(o1, o1_r, "o_cmp")
    assert_close_16bit(o2, o2_r, "o_sel")
    torch.autograd.backward([o1_r, o2_r], [do1.float(), do2.float()])
    for n in ("q", "k", "v", "wk", "wv"):
        assert_close_16bit(t[n].grad, r[n].grad, "d" + n, grad_tol("d" + n, chain=True), CHAIN_GRAD_MEAN_TOL)
    assert pkg.device_status() == 0


@pytest.mark.parametrize("N,topk", [(8192, 8), (2048, 16)])
def test_configuration_3_sparse_attention(pkg, N, topk):
    ops = pkg.ops
    Hq, Hkv, d, ks, st, bs = 64, 4, 128, 32, 16, 64
    g = torch.Generator(device=DEV).manual_seed(300 + N)
    q, k, v, do = (torch.randn(N, h, d, generator=g, device=DEV).to(torch.bfloat16) for h in (Hq, Hkv, Hkv, Hq))
    cu = torch.tensor([0, N], dtype=torch.int32, device=DEV)
    with torch.no_grad():
        ck, cu_k = ops.avgpool_compress(k, None, cu, ks, st)
        cv, _ = ops.avgpool_compress(v, None, cu, ks, st)
        idx = ops.compressed_attention(q, ck, cv, ks, st, bs, topk, cu, cu_k, N, ck.shape[0])[1]
    assert idx.shape == (Hkv, N, topk)
    t = [leaf(x) for x in (q, k, v)]
    o = ops.topk_sparse_attention(*t, idx, bs, cu)
    o.backward(do)
    r = [leaf(x, torch.float32) for x in (q, k, v)]
    o_r = O.topk_sparse_attention(*r, idx, bs, cu)
    o_r.backward(do.float())
    assert_close_16bit(o, o_r, "o")
    for name, a, b in zip(("dq", "dk", "dv"), t, r):
        assert_close_16bit(a.grad, b.grad, name, grad_tol(name))
    assert pkg.device_status() == 0
