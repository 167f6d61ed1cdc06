"""Checks at the benchmark's full size (one 65 536-token sequence, 64q/4kv heads, d=128, kernel 32 / stride 16, block 64,
top-16), where the CPU oracle cannot run the whole problem: size-independent properties of attention, and comparisons of
slices that the oracle can afford (the first 2048 tokens, which by causality do not depend on the rest, and a few of the
very last tokens against a direct evaluation of their rows)."""
import math

import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu

N, HQ, HKV, D, KS, ST, BS, TOPK = 65536, 64, 4, 128, 32, 16, 64, 16
G = HQ // HKV


@pytest.fixture(scope="module")
def ops():
    import native_sparse_attention_triton_b200 as pkg
    assert torch.cuda.is_available()
    return pkg.ops


@pytest.fixture(scope="module")
def data(ops):
    g = torch.Generator(device="cuda").manual_seed(2024)
    dev = torch.device("cuda")
    mk = lambda *s, scale=1.0: (torch.randn(*s, generator=g, device=dev) * scale).to(torch.bfloat16)
    x = dict(q=mk(N, HQ, D), k=mk(N, HKV, D), v=mk(N, HKV, D), wk=mk(HKV, KS * D, D, scale=1 / math.sqrt(KS * D)),
             wv=mk(HKV, KS * D, D, scale=1 / math.sqrt(KS * D)), pe=mk(HKV, KS, D, scale=0.02))
    x["cu"] = torch.tensor([0, N], dtype=torch.int32, device=dev)
    with torch.no_grad():
        x["ck"], x["cu_k"] = ops.linear_compress(x["k"], x["wk"], x["cu"], KS, ST, x["pe"])
        x["cv"], _ = ops.linear_compress(x["v"], x["wv"], x["cu"], KS, ST, None)
        x["o_cmp"], x["idx"] = ops.compressed_attention(x["q"], x["ck"], x["cv"], KS, ST, BS, TOPK, x["cu"], x["cu_k"], N,
                                                        x["ck"].shape[0], None, 1, 2)
    return x


def status_ok():
    import native_sparse_attention_triton_b200 as pkg
    return pkg.device_status() == 0


def test_topk_idx_structure(data):
    """Ascending ids in [0, t // block], -1 only at the end, min(topk, t // block + 1) of them, forced blocks present."""
    idx = data["idx"]
    assert idx.shape == (HKV, N, TOPK) and idx.dtype == torch.int32
    t = torch.arange(N, device=idx.device)
    bq = (t // BS)[None, :, None]
    valid = idx >= 0
    assert bool(((idx <= bq) | ~valid).all())
    count = valid.sum(-1)
    assert bool((count == torch.clamp(bq[..., 0] + 1, max=TOPK)).all())
    # valid entries first, strictly ascending
    assert bool((valid[..., 1:] <= valid[..., :-1]).all())
    asc = (idx[..., 1:] > idx[..., :-1]) | ~valid[..., 1:]
    assert bool(asc.all())
    # forced: block 0, the query's own block and the one before it
    has = lambda b: ((idx == b) & valid).any(-1)
    assert bool(has(torch.zeros_like(bq)).all())
    assert bool(has(bq).all())
    assert bool((has(torch.clamp(bq - 1, min=0))).all())
    assert status_ok()


def test_constant_values_give_constant_output_and_zero_key_query_gradients(ops, data):
    """With V == 1 every row that sees a key outputs exactly 1 (softmax rows sum to one), dQ and dK vanish (the output no
    longer depends on the logits), and the key-wise sum of dV equals the row-wise sum of dO of the group's heads."""
    dev = data["q"].device
    g = torch.Generator(device="cuda").manual_seed(7)
    ones_c = torch.ones_like(data["cv"])
    ones_v = torch.ones_like(data["v"])
    do = torch.randn(N, HQ, D, generator=g, device=dev).to(torch.bfloat16)
    # ---- compressed attention ----
    q = data["q"].clone().requires_grad_(True)
    ck = data["ck"].clone().requires_grad_(True)
    cv = ones_c.clone().requires_grad_(True)
    o, _ = ops.compressed_attention(q, ck, cv, KS, ST, BS, TOPK, data["cu"], data["cu_k"], N, ck.shape[0], None, 1, 2)
    sees = torch.arange(N, device=dev) >= KS - 1
    assert float((o.detach()[sees].float() - 1).abs().max()) <= 8e-3      # bf16 rounding of P and of O
    assert float(o.detach()[~sees].float().abs().max()) == 0.0
    o.backward(do)
    # reference magnitudes: the same backward with the real values
    qr = data["q"].clone().requires_grad_(True)
    ckr = data["ck"].clone().requires_grad_(True)
    o_r, _ = ops.compressed_attention(qr, ckr, data["cv"], KS, ST, BS, TOPK, data["cu"], data["cu_k"], N, ck.shape[0], None, 1, 2)
    o_r.backward(do)
    rms = lambda t: float(t.float().pow(2).mean().sqrt())
    # O == 1 only up to its 16-bit rounding, so delta = sum(O * dO) cancels dP to about 2^-8: a few percent at most
    assert rms(q.grad) <= 0.05 * rms(qr.grad) and rms(ck.grad) <= 0.05 * rms(ckr.grad)
    lhs = cv.grad.float().sum(0)                                                   # [Hkv, d]
    rhs = do[sees].float().view(-1, HKV, G, D).sum((0, 2))
    assert float((lhs - rhs).abs().max()) <= 2e-2 * float(rhs.abs().max())
    # ---- top-k sparse attention ----
    q2 = data["q"].clone().requires_grad_(True)
    k2 = data["k"].clone().requires_grad_(True)
    v2 = ones_v.clone().requires_grad_(True)
    o2 = ops.topk_sparse_attention(q2, k2, v2, data["idx"], BS, data["cu"])
    assert float((o2.detach().float() - 1).abs().max()) <= 8e-3
    o2.backward(do)
    q2r = data["q"].clone().requires_grad_(True)
    k2r = data["k"].clone().requires_grad_(True)
    ops.topk_sparse_attention(q2r, k2r, data["v"], data["idx"], BS, data["cu"]).backward(do)
    assert rms(q2.grad) <= 0.05 * rms(q2r.grad) and rms(k2.grad) <= 0.05 * rms(k2r.grad)
    lhs = v2.grad.float().sum(0)
    rhs = do.float().view(N, HKV, G, D).sum((0, 2))
    assert float((lhs - rhs).abs().max()) <= 2e-2 * float(rhs.abs().max())
    assert status_ok()


def test_prefix_matches_oracle(ops, data):
    """Tokens below 2048 depend only on tokens below 2048: their rows of the 65 536-token run must match the CPU oracle run
    on the prefix alone (outputs to the bf16 tolerance of the small-size tests, top-k ids up to score ties)."""
    P = 2048
    cpu = lambda t: t[:P].float().cpu()
    cu = torch.tensor([0, P], dtype=torch.int32)
    ck, cu_k = O.linear_compress(cpu(data["k"]), data["wk"].float().cpu(), cu, KS, ST, data["pe"].float().cpu())
    cv, _ = O.linear_compress(cpu(data["v"]), data["wv"].float().cpu(), cu, KS, ST, None)
    Mp = ck.shape[0]
    err = (data["ck"][:Mp].float().cpu() - ck).abs()
    assert float((err / ck.abs().clamp(min=1.0)).max()) <= 2e-2 and float(err.mean()) <= 2e-3
    # attention and selection are compared on the SAME compressed keys (the GPU's), so that last-bit differences of the
    # compression do not move block scores across the selection threshold
    ck_b, cv_b = data["ck"][:Mp].float().cpu(), data["cv"][:Mp].float().cpu()
    o_ref, idx_ref, scores = O.compressed_attention(cpu(data["q"]), ck_b, cv_b, KS, ST, BS, TOPK, cu, cu_k, init_blocks=1,
                                                    local_blocks=2, return_scores=True)
    err = (data["o_cmp"][:P].float().cpu() - o_ref).abs()
    assert float((err / o_ref.abs().clamp(min=1.0)).max()) <= 2e-2 and float(err.mean()) <= 2e-3
    idx_gpu = data["idx"][:, :P].cpu()
    bad, differing, rows = O.compare_topk_idx(idx_gpu, idx_ref, scores, 1e-3)
    assert bad == 0, (bad, differing, rows)
    o2 = ops.topk_sparse_attention(data["q"], data["k"], data["v"], data["idx"], BS, data["cu"])
    o2_ref = O.topk_sparse_attention(cpu(data["q"]), cpu(data["k"]), cpu(data["v"]), idx_gpu, BS, cu)
    err = (o2[:P].float().cpu() - o2_ref).abs()
    assert float((err / o2_ref.abs().clamp(min=1.0)).max()) <= 2e-2 and float(err.mean()) <= 2e-3
    assert status_ok()


def test_last_tokens_match_direct_evaluation(ops, data):
    """The far end of the sequence: rows of the last tokens, evaluated directly in fp32 on the GPU-computed compressed keys
    (compressed attention over all 4095 keys) and on the rows of their selected blocks (sparse attention)."""
    toks = [N - 1, N - 2, N - 65, N - 300]
    q = data["q"].float()
    sm = 1.0 / math.sqrt(D)
    ck, cv = data["ck"].float(), data["cv"].float()
    o2 = ops.topk_sparse_attention(data["q"], data["k"], data["v"], data["idx"], BS, data["cu"])
    for t in toks:
        nvis = min(ck.shape[0], (t - KS + 1) // ST + 1)
        for h in (0, 17, 63):
            hk = h // G
            p = torch.softmax((ck[:nvis, hk] @ q[t, h]) * sm, 0)
            ref = p @ cv[:nvis, hk]
            assert float((data["o_cmp"][t, h].float() - ref).abs().max()) <= 2e-2
            rows = torch.cat([torch.arange(b * BS, min((b + 1) * BS, t + 1), device=q.device)
                              for b in data["idx"][hk, t].tolist() if b >= 0])
            p = torch.softmax((data["k"][rows, hk].float() @ q[t, h]) * sm, 0)
            ref = p @ data["v"][rows, hk].float()
            assert float((o2[t, h].float() - ref).abs().max()) <= 2e-2
    assert status_ok()
