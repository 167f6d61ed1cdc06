"""The CPU oracle against fixtures produced by the reference's own ops.torch code (no GPU needed)."""
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import load_golden, padded_cache

CASES = ["mini_ragged", "cfg1", "g16_d128"]


@pytest.mark.parametrize("name", CASES)
def test_compress_matches_reference(name):
    meta, x, gold = load_golden(name)
    ks, st = meta["ks"], meta["st"]
    # the reference debug functions run in bf16: compare after rounding, one bf16 ulp of slack
    for key, fn, args in (
        ("lin_k", O.linear_compress, (x["k"], x["wk"], x["cu"], ks, st, x["pe"])),
        ("lin_v", O.linear_compress, (x["v"], x["wv"], x["cu"], ks, st, None)),
        ("pool_k", O.weightedpool_compress, (x["k"], x["wp"], x["cu"], ks, st, x["pe"])),
        ("avg_k", O.avgpool_compress, (x["k"], None, x["cu"], ks, st, x["pe"])),
    ):
        y, y_cu = fn(*args)
        assert torch.equal(y_cu, gold["cu_k"])
        assert y.shape == gold[key].shape
        mx, mean = O.error_stats(y, gold[key])
        assert mx <= 3e-2 and mean <= 3e-3, (key, mx, mean)


@pytest.mark.parametrize("name", CASES)
def test_attention_chain_matches_reference(name):
    meta, x, gold = load_golden(name)
    ks, st, bs, T = meta["ks"], meta["st"], meta["bs"], meta["topk"]
    step = meta["row_step"]
    ck, cv = gold["lin_k"], gold["lin_v"]
    o, idx, sc = O.compressed_attention(x["q"], ck, cv, ks, st, bs, T, x["cu"], gold["cu_k"],
                                        init_blocks=meta["init_blocks"], local_blocks=meta["local_blocks"],
                                        return_scores=True)
    assert torch.allclose(o[::step], gold["o_cmp"], atol=2e-5, rtol=1e-5)
    bad, differing, rows = O.compare_topk_idx(idx, gold["topk_idx"], sc, tie_tol=1e-6)
    assert bad == 0 and differing == 0, (bad, differing, rows)
    o_sel = O.topk_sparse_attention(x["q"], x["k"], x["v"], gold["topk_idx"], bs, x["cu"])
    assert torch.allclose(o_sel[::step], gold["o_sel"], atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("name", CASES)
def test_decode_matches_reference(name):
    meta, x, gold = load_golden(name)
    ks, st, bs, T = meta["ks"], meta["st"], meta["bs"], meta["topk"]
    seqlens = meta["seqlens"]
    cu = x["cu"]
    y_len, y_cu = O.compressed_seqlens(cu, ks, st)
    q_last = x["q"][(cu[1:] - 1).long()]
    sl = torch.tensor(seqlens, dtype=torch.int32)
    ckc = padded_cache(gold["lin_k"], y_cu, y_len.tolist(), int(y_len.max()))
    cvc = padded_cache(gold["lin_v"], y_cu, y_len.tolist(), int(y_len.max()))
    o, idx, sc = O.compressed_attention_decode(q_last, ckc, cvc, sl, y_len, ks, st, bs, T,
                                               meta["init_blocks"], meta["local_blocks"], return_scores=True)
    assert torch.allclose(o, gold["dec_o_cmp"], atol=2e-5, rtol=1e-5)
    bad, differing, _ = O.compare_topk_idx(idx, gold["dec_idx"], sc, tie_tol=1e-6)
    assert bad == 0 and differing == 0
    kc, vc = padded_cache(x["k"], cu, seqlens), padded_cache(x["v"], cu, seqlens)
    o_sel = O.topk_sparse_attention_decode(q_last, kc, vc, gold["dec_idx"], bs, sl)
    mx, mean = O.error_stats(o_sel, gold["dec_o_sel"])  # reference ran in bf16
    assert mx <= 2e-2 and mean <= 2e-3
    o_fl = O.flash_attention_decode(q_last, kc, vc, sl)
    mx, mean = O.error_stats(o_fl, gold["dec_o_flash"])
    assert mx <= 2e-2 and mean <= 2e-3


def test_decode_equals_prefill_last_token():
    """The single-token operator reproduces the last row of the varlen operator (same formulas)."""
    meta, x, gold = load_golden("mini_ragged")
    ks, st, bs, T = meta["ks"], meta["st"], meta["bs"], meta["topk"]
    cu = x["cu"]
    o, idx = O.compressed_attention(x["q"], gold["lin_k"], gold["lin_v"], ks, st, bs, T, cu, gold["cu_k"])
    last = (cu[1:] - 1).long()
    assert torch.allclose(o[last], gold["dec_o_cmp"], atol=2e-5)


def test_block_score_weights():
    assert O.block_score_weights(32, 16, 64) == [1, 2, 2, 2, 1]
    assert O.block_score_weights(16, 16, 64) == [1, 1, 1, 1]
    assert sum(O.block_score_weights(64, 16, 128)) == 4 * 8


def test_flop_model_headline():
    f = O.useful_flops([65536], 64, 4, 128, 32, 16, 64, 16)
    assert abs(f["cmp_fwd"] / 1e12 - 4.395) < 0.01
    assert abs(f["sel_fwd"] / 1e12 - 2.115) < 0.01
    tot = O.total_useful_flops([65536], 64, 4, 128, 32, 16, 64, 16)
    assert abs(tot / 1e12 - 22.89) < 0.05
