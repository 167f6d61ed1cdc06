"""Generate the golden fixtures in this directory from the REFERENCE project itself.

Run once, in a container that holds the reference checkout (read-only):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own ``native_sparse_attention.ops.torch`` debug
implementations (and the in-file torch references of the two Triton decode
operators), runs them on the CPU on seeded inputs and stores inputs (as bf16 bit
patterns) and outputs as ``.npz`` files.  The reference's compression debug
functions hard-code ``device="cuda"`` for one ``torch.zeros`` call and one
decode helper calls ``.cuda()``; the generator redirects exactly those calls to
the CPU and otherwise runs the reference code unmodified.

Nothing in the test-suite or the benchmark needs the reference at run time:
they only read the ``.npz`` files written here.
"""
import math
import os
import sys
from unittest import mock

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NSA_REFERENCE_CHECKOUT", "reference")
sys.path.insert(0, REF)
OUT = __file__.rsplit("/", 1)[0]

from native_sparse_attention.ops.torch.compressed_attention import compressed_attention_torch  # noqa: E402
from native_sparse_attention.ops.torch.topk_sparse_attention import topk_sparse_attention_torch  # noqa: E402
from native_sparse_attention.ops.torch.compressed_attention_decode import compressed_attention_decode  # noqa: E402
from native_sparse_attention.ops.torch import compress_key_value as ref_ckv  # noqa: E402
from native_sparse_attention.ops.triton.flash_attention_decode import torch_attention_decode  # noqa: E402
from native_sparse_attention.ops.triton.topk_sparse_attention_decode import (  # noqa: E402
    torch_topk_sparse_attention_decode,
)
from native_sparse_attention.ops.triton.utils import get_compressed_seqlens  # noqa: E402


def bits(t):  # bf16-exact fp32 tensor -> uint16 bit pattern
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def bf16_exact(t):
    return t.to(torch.bfloat16).float()


_orig_zeros, _orig_arange = torch.zeros, torch.arange


def _cpu_zeros(*a, **k):
    k["device"] = "cpu"
    return _orig_zeros(*a, **k)


def on_cpu(fn, *a, **k):
    """Run a reference function whose only CUDA dependence is a device literal."""
    with mock.patch("torch.zeros", _cpu_zeros), mock.patch.object(torch.Tensor, "cuda", lambda self, *x, **y: self):
        return fn(*a, **k)


def chain_case(name, seed, seqlens, Hq, Hkv, d, ks, st, bs, topk, init_blocks, local_blocks, store_inputs, row_step):
    g = torch.Generator().manual_seed(seed)
    N = sum(seqlens)
    cu = torch.tensor([0] + list(np.cumsum(seqlens)), dtype=torch.int32)
    q = bf16_exact(torch.randn(N, Hq, d, generator=g))
    k = bf16_exact(torch.randn(N, Hkv, d, generator=g))
    v = bf16_exact(torch.randn(N, Hkv, d, generator=g))
    wk = bf16_exact(torch.randn(Hkv, ks * d, d, generator=g) / math.sqrt(ks * d))
    wv = bf16_exact(torch.randn(Hkv, ks * d, d, generator=g) / math.sqrt(ks * d))
    pe = bf16_exact(torch.randn(Hkv, ks, d, generator=g) * 0.02)
    wp = bf16_exact(torch.randn(Hkv, ks, generator=g) / ks)
    out = {}
    # compression through the reference debug functions (bf16 is what they accept)
    bf = torch.bfloat16
    ck_ref, cu_k = on_cpu(ref_ckv.linear_compress_torch, k.to(bf), wk.to(bf), cu, ks, st, pe.to(bf))
    cv_ref, _ = on_cpu(ref_ckv.linear_compress_torch, v.to(bf), wv.to(bf), cu, ks, st, None)
    pk_ref, _ = on_cpu(ref_ckv.weightedpool_compress_torch, k.to(bf), wp.to(bf), cu, ks, st, pe.to(bf))
    ak_ref, _ = on_cpu(ref_ckv.avgpool_compress_torch, k.to(bf), None, cu, ks, st, pe.to(bf))
    y_len, y_cu = get_compressed_seqlens(cu, ks, st)
    assert torch.equal(y_cu, cu_k.to(torch.int32))
    out.update(lin_k=bits(ck_ref), lin_v=bits(cv_ref), pool_k=bits(pk_ref), avg_k=bits(ak_ref), cu_k=cu_k.numpy())
    # attention chain in fp32 on the (bf16-rounded) reference compressed tensors
    ck, cv = ck_ref.float(), cv_ref.float()
    o_cmp, idx = compressed_attention_torch(
        q, ck, cv, ks, st, bs, topk, cu, cu_k.to(torch.int32), max(seqlens), int(y_len.max()), None,
        init_blocks, local_blocks)
    o_sel = topk_sparse_attention_torch(q, k, v, idx, bs, cu)
    out.update(topk_idx=idx.numpy().astype(np.int16), o_cmp=o_cmp[::row_step].numpy(), o_sel=o_sel[::row_step].numpy())
    # decode: the last token of every sequence against its own prefix
    B = len(seqlens)
    Lmax, Lcmax = max(seqlens), int(y_len.max())
    kc = torch.zeros(B, Lmax, Hkv, d)
    vc = torch.zeros(B, Lmax, Hkv, d)
    ckc = torch.zeros(B, Lcmax, Hkv, d)
    cvc = torch.zeros(B, Lcmax, Hkv, d)
    for b, L in enumerate(seqlens):
        kc[b, :L] = k[cu[b]:cu[b + 1]]
        vc[b, :L] = v[cu[b]:cu[b + 1]]
        m = int(y_len[b])
        ckc[b, :m] = ck[cu_k[b]:cu_k[b + 1]]
        cvc[b, :m] = cv[cu_k[b]:cu_k[b + 1]]
    q_last = q[(cu[1:] - 1).long()]
    sl = torch.tensor(seqlens, dtype=torch.int32)
    o_cd, idx_d = compressed_attention_decode(q_last, ckc, cvc, sl, y_len.to(torch.int32), ks, st, bs, topk,
                                              init_blocks, local_blocks)
    o_sd = on_cpu(torch_topk_sparse_attention_decode, q_last.to(bf), kc.to(bf), vc.to(bf), idx_d, bs, sl)
    o_fd = torch_attention_decode(q_last.to(bf), kc.to(bf), vc.to(bf), sl)
    out.update(dec_o_cmp=o_cd.numpy(), dec_idx=idx_d.numpy().astype(np.int16), dec_o_sel=bits(o_sd),
               dec_o_flash=bits(o_fd))
    meta = dict(seed=seed, seqlens=np.array(seqlens), Hq=Hq, Hkv=Hkv, d=d, ks=ks, st=st, bs=bs, topk=topk,
                init_blocks=init_blocks, local_blocks=local_blocks, row_step=row_step,
                q_sum=float(q.double().sum()), k_sum=float(k.double().sum()))
    if store_inputs:
        out.update(q=bits(q), k=bits(k), v=bits(v), wk=bits(wk), wv=bits(wv), pe=bits(pe), wp=bits(wp))
    np.savez_compressed(f"{OUT}/{name}.npz", **out, **meta)
    print(name, {k_: (v_.shape if hasattr(v_, "shape") else v_) for k_, v_ in out.items()})


if __name__ == "__main__":
    # small ragged case, inputs stored (one sequence shorter than the window)
    chain_case("mini_ragged", 7, [20, 100, 200], 4, 2, 64, 32, 16, 64, 4, 1, 2, True, 1)
    # first benchmark configuration (CPU fp32 case); inputs are regenerated from the seed
    chain_case("cfg1", 43, [256, 768], 16, 2, 64, 32, 16, 64, 4, 1, 2, False, 16)
    # a G=16, d=128 case shaped like the headline workload, short
    chain_case("g16_d128", 11, [130, 640], 32, 2, 128, 32, 16, 64, 6, 1, 2, False, 32)
