"""The allocation-free flash-decode entry point, called through the C ABI.

Some callers of the library (a serving process whose memory pool owns the whole device, a loop that
must not risk the synchronisation an allocation can cause) cannot provide scratch memory; for them
`nsa_flash_attn_decode_static` keeps the split-KV scratch inside the library.  Its result has to equal
the regular entry point's, on consecutive calls that reuse the built-in scratch with different data.
This file is collected last on purpose.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, B, L, Hq, Hkv, d):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, d, generator=g).bfloat16().cuda()
    k = torch.randn(B, L, Hkv, d, generator=g).bfloat16().cuda()
    v = torch.randn(B, L, Hkv, d, generator=g).bfloat16().cuda()
    seqlens = torch.randint(1, L + 1, (B,), generator=g, dtype=torch.int32).cuda()
    return q, k, v, seqlens


def _call_static(lib, q, k, v, seqlens, splits, o=None):
    from native_sparse_attention_triton_b200 import _lib

    if o is None:
        o = torch.full_like(q, float("nan"))
    B, Hq, d = q.shape
    L, Hkv = k.shape[1], k.shape[2]
    strides = _lib.strides_array(q.stride(0), q.stride(1), k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1),
                                 v.stride(2), o.stride(0), o.stride(1), 0, 0, 0)
    rc = lib.nsa_flash_attn_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), seqlens.data_ptr(), o.data_ptr(),
                                          splits, B, L, Hq, Hkv, d, strides, 1.0 / d ** 0.5, _lib.DTYPE_BF16,
                                          torch.cuda.current_stream().cuda_stream)
    return rc, o


def test_static_scratch_decode_matches_regular_entry_point_twice():
    import native_sparse_attention_triton_b200 as pkg

    lib = pkg._lib.lib()
    assert lib.nsa_flash_attn_decode_static_capacity() == 2 * 1024 * 1024
    for seed, shape in ((1, (6, 1536, 32, 4, 128)), (2, (3, 700, 16, 2, 64))):   # two calls in a row, different data
        q, k, v, seqlens = _case(seed, *shape)
        ref = pkg.ops.flash_attention_decode(q, k, v, seqlens)      # regular path: caller-provided scratch
        o = torch.full_like(q, float("nan"))                         # the caller owns the output
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc, o = _call_static(lib, q, k, v, seqlens, 0, o)
        assert rc == 0
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, "the entry point must not allocate device memory"
        err = (o.float() - ref.float()).abs()
        assert float(err.max()) <= 2e-2 and float(err.mean()) <= 2e-3, (float(err.max()), float(err.mean()))
    assert pkg.device_status() == 0


def test_static_scratch_rejects_oversized_problems():
    import native_sparse_attention_triton_b200 as pkg

    lib = pkg._lib.lib()
    q, k, v, seqlens = _case(3, 64, 4096, 32, 4, 128)
    # 64 * 4 * 64 splits * 16 * 130 floats = 34 M floats > 2 M: refused with the scratch-too-small code
    rc, _ = _call_static(lib, q, k, v, seqlens, 64)
    assert rc == -3
    rc, o = _call_static(lib, q, k, v, seqlens, 1)   # one split needs no scratch at all
    assert rc == 0
    ref = pkg.ops.flash_attention_decode(q, k, v, seqlens)
    err = (o.float() - ref.float()).abs()
    assert float(err.max()) <= 2e-2 and float(err.mean()) <= 2e-3


def test_static_scratch_default_split_count_always_fits():
    """With num_splits = 0 the library picks the split count itself, so it must pick one whose partial results fit the
    built-in array (batch 64 x 4 KV heads at head_dim 128 would want 4 splits = 2 129 920 floats, 32 768 too many); and an
    explicit request above the 64-split limit is clamped to 64 before its size is judged, as the regular entry point does."""
    import native_sparse_attention_triton_b200 as pkg

    lib = pkg._lib.lib()
    q, k, v, seqlens = _case(4, 64, 1024, 32, 4, 128)
    ref = pkg.ops.flash_attention_decode(q, k, v, seqlens)
    rc, o = _call_static(lib, q, k, v, seqlens, 0)
    assert rc == 0
    err = (o.float() - ref.float()).abs()
    assert float(err.max()) <= 2e-2 and float(err.mean()) <= 2e-3
    q, k, v, seqlens = _case(5, 1, 8192, 16, 1, 128)   # 128 tiles: 200 requested splits run as 64, 133 120 floats
    ref = pkg.ops.flash_attention_decode(q, k, v, seqlens)
    rc, o = _call_static(lib, q, k, v, seqlens, 200)
    assert rc == 0
    err = (o.float() - ref.float()).abs()
    assert float(err.max()) <= 2e-2 and float(err.mean()) <= 2e-3
    assert pkg.device_status() == 0
