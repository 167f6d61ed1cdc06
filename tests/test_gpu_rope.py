"""Rotary embedding kernel (through the C interface) against the oracle: prefill positions over a ragged batch, the strided
positions of compressed keys, decode-step positions, large angles, both dtypes and head sizes, strided input, backward."""
import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import native_sparse_attention_triton_b200 as pkg
    assert torch.cuda.is_available()
    return pkg.ops


def inv_freq_for(d, theta=500000.0):
    return 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))


def check(ops, lens, h, d, dtype, step, stride, scaling=1.0, strided=False, seed=0):
    import native_sparse_attention_triton_b200 as pkg
    g = torch.Generator().manual_seed(seed)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    rows = len(lens) if step > 0 else int(cu[-1])
    inv_freq = inv_freq_for(d)
    if strided:
        wide = torch.randn(rows, h + 3, d, generator=g).to(dtype)
        x = wide[:, 2:2 + h]
    else:
        x = torch.randn(rows, h, d, generator=g).to(dtype)
    dy = torch.randn(rows, h, d, generator=g).to(dtype)
    xg = x.cuda().requires_grad_(True)
    y = ops.rope(xg, inv_freq.cuda(), cu.cuda(), step, stride, scaling)
    y.backward(dy.cuda())
    xc = x.float().requires_grad_(True)
    y_ref = rope_ref(xc, inv_freq, cu, step, stride, scaling, dtype)
    y_ref.backward(dy.float())
    tol = 1e-2  # the reference's own comparison tolerance (atol = rtol = 1e-2)
    err = (y.detach().float().cpu() - y_ref.detach()).abs() / y_ref.detach().abs().clamp(min=1.0)
    assert float(err.max()) <= tol, float(err.max())
    err = (xg.grad.float().cpu() - xc.grad).abs() / xc.grad.abs().clamp(min=1.0)
    assert float(err.max()) <= tol, float(err.max())
    assert pkg.device_status() == 0


def rope_ref(x32, inv_freq, cu, step, stride, scaling, dtype):
    """O.rope on fp32 values with tables rounded to `dtype` (differentiable)."""
    half = x32.shape[-1] // 2
    # rotating the unit vector (1, 0) of every pair through the oracle returns its (cos, sin) table, rounded to dtype
    e1 = torch.cat([torch.ones(x32.shape[0], 1, half), torch.zeros(x32.shape[0], 1, half)], -1).to(dtype)
    r = O.rope(e1, inv_freq, cu, step, stride, scaling).float()   # (cos, sin) rounded to dtype
    c, s = r[..., :half], r[..., half:]
    x1, x2 = x32[..., :half], x32[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


@pytest.mark.parametrize("lens,h,d,dtype,step,stride,scaling,strided", [
    ([256, 1, 777], 8, 128, torch.bfloat16, 0, 1, 1.0, False),
    ([15, 47, 300], 4, 128, torch.bfloat16, 0, 16, 1.0, False),      # compressed keys: position = index * kernel_stride
    ([100, 8192, 5], 2, 128, torch.bfloat16, 7, 1, 1.0, False),      # decode step 7: one row per sequence
    ([100, 8192, 5], 2, 64, torch.float16, 1, 16, 1.0, False),
    ([5000], 3, 64, torch.float16, 0, 1, 0.83, True),
    ([70000], 1, 128, torch.bfloat16, 0, 16, 1.0, False),            # angles beyond 1e6 rad
])
def test_rope_matches_oracle(ops, lens, h, d, dtype, step, stride, scaling, strided):
    check(ops, lens, h, d, dtype, step, stride, scaling, strided, seed=len(lens) + h)


def test_rope_in_place_and_argument_checks(ops):
    from native_sparse_attention_triton_b200 import _lib
    from native_sparse_attention_triton_b200.ops._common import ptr, stream_ptr
    x = torch.randn(64, 4, 128).to(torch.bfloat16).cuda()
    inv_freq = inv_freq_for(128).cuda()
    cu = torch.tensor([0, 64], dtype=torch.int32).cuda()
    want = ops.rope(x, inv_freq, cu)
    y = x.clone()
    rc = _lib.lib().nsa_rope(ptr(y), ptr(y), ptr(inv_freq), ptr(cu), 64, 1, 4, 128, 0, 1, 1.0, 0, 512, 128, 512, 128, 0,
                             stream_ptr(x.device))
    assert rc == 0 and torch.equal(y, want)
    # rotating back by the opposite angle restores x up to the two roundings
    back = torch.empty_like(y)
    rc = _lib.lib().nsa_rope(ptr(y), ptr(back), ptr(inv_freq), ptr(cu), 64, 1, 4, 128, 0, 1, 1.0, 1, 512, 128, 512, 128, 0,
                             stream_ptr(x.device))
    assert rc == 0 and float((back.float() - x.float()).abs().max()) <= 5e-2
    assert _lib.lib().nsa_rope(ptr(y), ptr(y), ptr(inv_freq), ptr(cu), 64, 1, 4, 96, 0, 1, 1.0, 0, 384, 96, 384, 96, 0,
                               stream_ptr(x.device)) == -2
    assert _lib.lib().nsa_rope(ptr(y), ptr(y), ptr(inv_freq), ptr(cu), 64, 1, 4, 128, 2, 1, 1.0, 0, 512, 128, 512, 128, 0,
                               stream_ptr(x.device)) == -1    # decode needs rows == batch
    with pytest.raises(AssertionError):
        ops.rope(x.float(), inv_freq, cu)
    with pytest.raises(AssertionError):
        ops.rope(x, inv_freq[:32], cu)


def test_three_decode_rotations_in_one_launch_equal_three_launches(ops):
    from native_sparse_attention_triton_b200.infer import RotaryEmbedding
    g = torch.Generator().manual_seed(8)
    B, Hq, Hkv, d = 5, 16, 2, 128
    rope = RotaryEmbedding(inv_freq_for(d).cuda(), 0.9)
    q = torch.randn(B, Hq, d, generator=g).bfloat16().cuda()
    k = torch.randn(B, Hkv, d, generator=g).bfloat16().cuda()
    ck = torch.randn(B, Hkv, d, generator=g).bfloat16().cuda()
    lens = torch.tensor([0, 5, 8191, 77, 1000], dtype=torch.int32).cuda()
    clens = torch.tensor([0, 0, 510, 3, 61], dtype=torch.int32).cuda()
    yq, yk, yck = rope.decode_at3(q, k, ck, lens, clens, 16)
    assert torch.equal(yq, rope.decode_at(q, lens, 1))
    assert torch.equal(yk, rope.decode_at(k, lens, 1))
    assert torch.equal(yck, rope.decode_at(ck, clens, 16))
    # and a row at a device-side length equals the prefill rotation of the token at that index
    cu = torch.tensor([0, 78], dtype=torch.int32).cuda()
    full = ops.rope(q[3:4].expand(78, Hq, d).contiguous(), rope.inv_freq, cu, 0, 1, 0.9)
    assert torch.equal(full[77], yq[3])
