"""Sliding-window branch (causal attention over keys t - W .. t): forward and backward parity with the fp32 CPU oracle.

The reference delegates this branch to flash_attn (module/native_sparse_attention.py:213-223); the oracle's restatement of
its mask is pinned by tests/golden/box_window.npz (flash_attn's own output on a B200, tests/test_oracle_box_golden.py), and
tests/test_gpu_box_golden.py compares these kernels with that file directly."""
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import chain_inputs
from tests.test_gpu_backward import close, leaf, ref_leaf, status_ok

pytestmark = pytest.mark.gpu

# (Hq, Hkv, seqlens, window): windows shorter and longer than a 128-key tile, longer than a sequence, and zero;
# sequences that start inside a tile
CASES = [
    (16, 1, [700, 260, 33], 100),   # G = 16
    (8, 2, [1500], 512),            # G = 4, the layer's window
    (16, 2, [300, 129, 1025], 17),  # G = 8, a window inside one tile
    (4, 4, [200, 333], 1000),       # G = 1, window longer than every sequence: plain causal attention
    (16, 1, [260], 0),              # only the diagonal
]


@pytest.fixture(scope="module")
def ops():
    import native_sparse_attention_triton_b200 as pkg
    assert torch.cuda.is_available()
    return pkg.ops


@pytest.mark.parametrize("Hq,Hkv,seqlens,window", CASES)
def test_sliding_window_forward_backward(ops, Hq, Hkv, seqlens, window):
    x = chain_inputs(11, seqlens, Hq, Hkv, 128, 32)
    g = torch.Generator().manual_seed(3)
    cu = x["cu"]
    do = torch.randn(x["q"].shape, generator=g).bfloat16().float()
    q, k, v = leaf(x["q"]), leaf(x["k"]), leaf(x["v"])
    o = ops.sliding_window_attention(q, k, v, cu.cuda(), max(seqlens), window)
    o.backward(do.bfloat16().cuda())
    qr, kr, vr = ref_leaf(x["q"]), ref_leaf(x["k"]), ref_leaf(x["v"])
    o_ref = O.sliding_window_attention(qr, kr, vr, cu, window)
    o_ref.backward(do)
    err = (o.detach().float().cpu() - o_ref.detach()).abs()
    # outputs: max |err| <= 2e-2 * max(1, |ref|), mean |err| <= 2e-3 (bf16 tolerance of the other forward tests)
    assert float((err / o_ref.detach().abs().clamp(min=1.0)).max()) <= 2e-2 and float(err.mean()) <= 2e-3
    close(q.grad, qr.grad, "dq")
    close(k.grad, kr.grad, "dk")
    close(v.grad, vr.grad, "dv")
    assert status_ok()


@pytest.mark.parametrize("seed", range(8))
def test_sliding_window_random_configurations(ops, seed):
    """Seeded random group sizes, ragged batches (sequences that end inside a row tile, so that both the staged and the
    row-by-row output paths of the dQ pass run) and windows."""
    import random
    rnd = random.Random(100 + seed)
    Hkv = rnd.choice([1, 2, 4])
    G = rnd.choice([1, 2, 4, 8, 16])
    seqlens = [rnd.choice([rnd.randint(1, 40), rnd.randint(60, 500), rnd.randint(500, 1200)]) for _ in range(rnd.choice([1, 2, 4]))]
    window = rnd.choice([0, 1, rnd.randint(2, 127), 128, rnd.randint(129, 600), 5000])
    test_sliding_window_forward_backward(ops, Hkv * G, Hkv, seqlens, window)


def test_window_covers_everything_equals_causal(ops):
    """With a window at least as long as the sequences the result is the plain causal attention of flash_attention_varlen."""
    x = chain_inputs(12, [400, 77], 16, 2, 128, 32)
    cu = x["cu"].cuda()
    q, k, v = (x[n].bfloat16().cuda() for n in ("q", "k", "v"))
    a = ops.sliding_window_attention(q, k, v, cu, 400, 4096)
    b = ops.flash_attention_varlen(q, k, v, cu, cu, 400, 400, True)
    assert torch.equal(a, b)
    assert status_ok()
