"""Generate the ``box_*.npz`` fixtures of this directory by RUNNING THE REFERENCE ITSELF on a GPU.

    sh baseline/install_reference.sh /path/to/reference      # once, where the checkout exists
    python tests/golden/make_golden_on_box.py [output dir]   # on a machine with a GPU, Triton and flash_attn

What is run, unmodified, from ``baseline/_ref``:
  * the reference's Triton operators (``native_sparse_attention.ops``: linear_compress, compressed_attention with its
    block scores, topk_sparse_attention) forward and backward on the seeded inputs of the ``cfg1`` and ``g16_d128`` cases
    (where the reference's Triton linear_compress kernel does not compile under the installed Triton, its own torch
    implementation ``ops.torch.compress_key_value.linear_compress_torch`` stands in; the file records which ran);
  * ``flash_attn.flash_attn_varlen_func(causal=True, window_size=(W, -1))``, the call the reference's layer makes for its
    sliding-window branch (module/native_sparse_attention.py:213-223), forward and backward;
  * the reference's ``RotaryEmbedding`` (module/rope.py) in prefill, strided and decode modes;
  * the reference's ``nsa_infer`` with its ``NSACache`` (infer/nsa_inference.py, module/kv_cache.py): a prefill and a run of
    decode steps.
Inputs are regenerated from seeds by the tests (tests/helpers.py); outputs are stored as bf16 bit patterns, large ones
subsampled by rows.  The files written here pin the CPU oracle (tests/test_oracle_box_golden.py) and are compared with
the CUDA kernels (tests/test_gpu_box_golden.py) on machines that do not hold the reference.
"""
import math
import os
import sys
import traceback

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))  # repository root

from tests import refbox  # noqa: E402
from tests.helpers import chain_inputs, infer_case_inputs, rope_case_inputs, window_case_inputs  # noqa: E402

OUT = sys.argv[1] if len(sys.argv) > 1 else HERE
DEV = torch.device("cuda")


def bits(t):
    return t.detach().to(torch.bfloat16).cpu().view(torch.int16).numpy().view(np.uint16)


def bits16(t):  # fp16 bit patterns
    return t.detach().to(torch.float16).cpu().view(torch.int16).numpy().view(np.uint16)


def chain_case(ref, name, seed, seqlens, Hq, Hkv, d, ks, st, bs, topk, init_blocks, local_blocks, row_step):
    from native_sparse_attention.ops import compressed_attention, topk_sparse_attention
    from native_sparse_attention.ops.triton import compressed_attention as ca

    linear_compress, which_linear = refbox.reference_linear_compress()

    inp = chain_inputs(seed, seqlens, Hq, Hkv, d, ks)
    cu = inp["cu"].to(DEV)
    t = {n: inp[n].to(torch.bfloat16).to(DEV).requires_grad_(True) for n in ("q", "k", "v", "wk", "wv", "pe")}
    g = torch.Generator().manual_seed(seed + 1000)
    N = sum(seqlens)
    do_cmp = torch.randn(N, Hq, d, generator=g).to(torch.bfloat16).to(DEV)
    do_sel = torch.randn(N, Hq, d, generator=g).to(torch.bfloat16).to(DEV)
    ck, cu_k = linear_compress(t["k"], t["wk"], cu, ks, st, t["pe"])
    cv, _ = linear_compress(t["v"], t["wv"], cu, ks, st, None)
    max_q, max_k = max(seqlens), int((cu_k[1:] - cu_k[:-1]).max())
    o_cmp, idx = compressed_attention(t["q"], ck, cv, ks, st, bs, topk, cu, cu_k, max_q, max_k, None, init_blocks,
                                      local_blocks)
    # the block scores the reference selected from (forced blocks at +inf), through its own two functions
    with torch.no_grad():
        _, lse = ca.CompressedAttention.apply(t["q"], ck, cv, ks, st, cu, cu_k, max_q, max_k, None)
        score = ca._get_attention_score(t["q"], ck, lse, ks, st, cu, cu_k, max_q, max_k, None)
        score = ca.transform_score(score, ks, st, bs, cu, cu_k, max_q, max_k, init_blocks, local_blocks)
    o_sel = topk_sparse_attention(t["q"], t["k"], t["v"], idx, bs, cu)
    torch.autograd.backward([o_cmp, o_sel], [do_cmp, do_sel])
    out = dict(lin_k=bits(ck), lin_v=bits(cv), cu_k=cu_k.cpu().numpy(), o_cmp=bits(o_cmp[::row_step]),
               o_sel=bits(o_sel[::row_step]), topk_idx=idx.cpu().numpy().astype(np.int16),
               block_score=score.float().cpu().numpy(), dq=bits(t["q"].grad[::row_step]), dk=bits(t["k"].grad),
               dv=bits(t["v"].grad), dwk=bits(t["wk"].grad[:, ::8]), dwv=bits(t["wv"].grad[:, ::8]), dpe=bits(t["pe"].grad))
    meta = dict(seed=seed, seqlens=np.array(seqlens), Hq=Hq, Hkv=Hkv, d=d, ks=ks, st=st, bs=bs, topk=topk,
                init_blocks=init_blocks, local_blocks=local_blocks, row_step=row_step, linear_compress=which_linear,
                q_sum=float(inp["q"].double().sum()), k_sum=float(inp["k"].double().sum()))
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **out, **meta)
    print(name, {k_: getattr(v_, "shape", v_) for k_, v_ in out.items()})


def window_case(name):
    from flash_attn import flash_attn_varlen_func

    out = {}
    for W in (64, 512):
        inp = window_case_inputs()
        cu = inp["cu"].to(DEV)
        q, k, v = (inp[n].to(torch.bfloat16).to(DEV).requires_grad_(True) for n in ("q", "k", "v"))
        L = int((inp["cu"][1:] - inp["cu"][:-1]).max())
        o = flash_attn_varlen_func(q, k, v, cu, cu, L, L, causal=True, window_size=(W, -1))
        o.backward(inp["do"].to(torch.bfloat16).to(DEV))
        out.update({f"o_w{W}": bits(o[::8]), f"dq_w{W}": bits(q.grad[::8]), f"dk_w{W}": bits(k.grad[::4]), f"dv_w{W}": bits(v.grad[::4])})
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **out)
    print(name, {k_: v_.shape for k_, v_ in out.items()})


def rope_case(ref, name):
    from native_sparse_attention.module.rope import RotaryEmbedding

    out = {}
    for tag, factor in (("f8", 8.0), ("f4", 4.0)):
        RotaryEmbedding.cos = RotaryEmbedding.sin = None   # class-level table: rebuild for this configuration
        rope = RotaryEmbedding(refbox.llama3_rope_config(ref, 128, factor), device=DEV)
        out[f"inv_freq_{tag}"] = rope.inv_freq.float().cpu().numpy()
        out[f"scaling_{tag}"] = np.float32(rope.attention_scaling)
        inp = rope_case_inputs()
        cu, cu_c = inp["cu"].to(DEV), inp["cu_c"].to(DEV)
        for dt, enc, dn in ((torch.bfloat16, bits, "bf16"), (torch.float16, bits16, "fp16")):
            RotaryEmbedding.cos = RotaryEmbedding.sin = None   # the table takes the dtype of the first call
            x, xc, xd = (inp[n].to(dt).to(DEV) for n in ("x", "xc", "xd"))
            out[f"prefill_{tag}_{dn}"] = enc(rope(x, cu)[::4])
            out[f"strided_{tag}_{dn}"] = enc(rope(xc, cu_c, stride=16))
            out[f"decode3_{tag}_{dn}"] = enc(rope(xd, cu, step=3))
            out[f"decode1s_{tag}_{dn}"] = enc(rope(xd, cu_c, step=1, stride=16))
    RotaryEmbedding.cos = RotaryEmbedding.sin = None
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **out)
    print(name, sorted(out))


def infer_case(ref, name, mode, lens, steps):
    from native_sparse_attention.infer import nsa_infer
    from native_sparse_attention.module import NSACache
    from native_sparse_attention.module.rope import RotaryEmbedding
    from native_sparse_attention.ops import avgpool_compress, weightedpool_compress

    linear_compress, which_linear = refbox.reference_linear_compress()
    c = infer_case_inputs(mode, lens, steps)
    P = c["params"]
    RotaryEmbedding.cos = RotaryEmbedding.sin = None
    rope = RotaryEmbedding(refbox.llama3_rope_config(ref, P["D"], 8.0), device=DEV)
    cache = NSACache(P["MAXB"], P["MAXLEN"], P["HKV"], P["D"], P["KS"], P["ST"], P["W"], torch.bfloat16, "cuda")
    fn = {"linear": linear_compress, "weighted": weightedpool_compress, "avg": avgpool_compress}[mode]
    dv = lambda x: None if x is None else x.to(torch.bfloat16).to(DEV)
    args = (rope, cache, [dv(c["w_k"]), dv(c["w_v"])], [fn, fn], dv(c["pe"]), P["KS"], P["ST"], P["BS"], P["TOPK"], P["INIT"],
            P["LOCAL"], P["W"])
    cu = c["cu"].to(DEV)
    o0 = nsa_infer(cu, 0, dv(c["q"]), dv(c["k"]), dv(c["v"]), dv(c["gate"]), *args)
    outs = []
    for step in range(1, steps + 1):
        qn, kn, vn, gn = c["steps"][step - 1]
        outs.append(nsa_infer(cu, step, dv(qn), dv(kn), dv(vn), dv(gn), *args))
    B = len(lens)
    out = dict(prefill=bits(o0), decode=bits(torch.stack(outs)), inv_freq=rope.inv_freq.float().cpu().numpy(),
               scaling=np.float32(rope.attention_scaling), sparse_len=cache.sparse_kv_len[:B].cpu().numpy(),
               compress_len=cache.compress_kv_len[:B].cpu().numpy(), sliding_len=cache.sliding_kv_len[:B].cpu().numpy(),
               stage_len=cache.before_compress_kv_len[:B].cpu().numpy(), lens=np.array(lens), steps=steps,
               linear_compress=which_linear)
    RotaryEmbedding.cos = RotaryEmbedding.sin = None
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **out)
    print(name, {k_: getattr(v_, "shape", v_) for k_, v_ in out.items()})


if __name__ == "__main__":
    os.makedirs(OUT, exist_ok=True)
    ref = refbox.load(layers=True)
    jobs = [
        ("box_triton_cfg1", lambda: chain_case(ref, "box_triton_cfg1", 43, [256, 768], 16, 2, 64, 32, 16, 64, 4, 1, 2, 8)),
        ("box_triton_g16_d128", lambda: chain_case(ref, "box_triton_g16_d128", 11, [130, 640], 32, 2, 128, 32, 16, 64, 6, 1, 2, 8)),
        ("box_window", lambda: window_case("box_window")),
        ("box_rope", lambda: rope_case(ref, "box_rope")),
        ("box_infer_linear", lambda: infer_case(ref, "box_infer_linear", "linear", [40, 100, 300], 40)),
        ("box_infer_weighted", lambda: infer_case(ref, "box_infer_weighted", "weighted", [33, 200], 24)),
    ]
    failed = []
    for name, job in jobs:
        try:
            job()
        except Exception:  # keep going: each fixture is independent
            failed.append(name)
            print(f"FAILED {name}\n{traceback.format_exc()}")
    print("failed:", failed)
    sys.exit(1 if failed else 0)
