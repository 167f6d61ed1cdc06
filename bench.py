#!/usr/bin/env python
"""Benchmark of the NSA hot path: linear compression -> compressed attention (+ top-k selection) ->
top-k sparse attention, forward and backward, on one 65536-token sequence per GPU.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...     # the reference's algorithm on the host cores (CPU oracle port)

Rank 0 prints ONE JSON line.  `value` is milliseconds per forward+backward step with inputs resident in
HBM (CUDA events, max over ranks); `e2e` is the same step driven from pinned host buffers with the
host->device copies and the device->host read of the loss inside the timed region.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

# ----------------------------------------------------------------------------------------------------
# workload (the configuration the headline metric is quoted on)
# ----------------------------------------------------------------------------------------------------
WORKLOAD = dict(tokens=65536, Hq=64, Hkv=4, d=128, ks=32, st=16, bs=64, topk=16, init_blocks=1, local_blocks=2)
METRIC = "nsa_fwd_bwd_ms_at_64k_tokens"
CPU_SAMPLE_TOKENS = 2048  # prefix length the CPU baseline is timed on (oracle memory is quadratic in it)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], tc_burst=p["bf16_tflops"], tc_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm=6650.0, tc_burst=1590.0, tc_sustained=1400.0, source="fallback")


def flop_model(tokens):
    from oracle import nsa_oracle as O
    w = WORKLOAD
    f = O.useful_flops([tokens], w["Hq"], w["Hkv"], w["d"], w["ks"], w["st"], w["bs"], w["topk"])
    total = O.total_useful_flops([tokens], w["Hq"], w["Hkv"], w["d"], w["ks"], w["st"], w["bs"], w["topk"])
    return f, total


def make_inputs(tokens, seed, device, pin=False):
    """Seeded synthetic tensors with the shapes and distributions of the workload (q, k, v ~ N(0,1);
    W ~ N(0, 1/(ks*d)); pe ~ N(0, 0.02^2); upstream gradients ~ N(0,1))."""
    w = WORKLOAD
    g = torch.Generator().manual_seed(seed)
    N, Hq, Hkv, d, ks = tokens, w["Hq"], w["Hkv"], w["d"], w["ks"]

    def mk(*shape, scale=1.0):
        t = (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)
        return t.pin_memory() if pin else t

    host = dict(q=mk(N, Hq, d), k=mk(N, Hkv, d), v=mk(N, Hkv, d), wk=mk(Hkv, ks * d, d, scale=1 / math.sqrt(ks * d)),
                wv=mk(Hkv, ks * d, d, scale=1 / math.sqrt(ks * d)), pe=mk(Hkv, ks, d, scale=0.02),
                do1=mk(N, Hq, d), do2=mk(N, Hq, d))
    return host


def chain_step(ops, t, cu, max_q, max_k):
    """One forward+backward pass of the operator chain through the public Python API; returns the loss tensor."""
    w = WORKLOAD
    for n in ("q", "k", "v", "wk", "wv", "pe"):
        t[n].grad = None
    ck, cu_k = ops.linear_compress(t["k"], t["wk"], cu, w["ks"], w["st"], t["pe"])
    cv, _ = ops.linear_compress(t["v"], t["wv"], cu, w["ks"], w["st"], None)
    o1, idx = ops.compressed_attention(t["q"], ck, cv, w["ks"], w["st"], w["bs"], w["topk"], cu, cu_k, max_q, max_k, None,
                                       w["init_blocks"], w["local_blocks"])
    o2 = ops.topk_sparse_attention(t["q"], t["k"], t["v"], idx, w["bs"], cu)
    torch.autograd.backward([o1, o2], [t["do1"], t["do2"]])
    return o1, o2


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "50"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [r.split(", ") for r in open(self.f.name).read().strip().splitlines() if r.strip()]
        os.unlink(self.f.name)
        sm, reasons = [], set()
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                out["sm_max_mhz"] = float(r[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.strip().lower().startswith("active"):
                    reasons.add(name)
        if sm:
            sm.sort()
            out["sm_mhz"] = sm[len(sm) // 2]
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


# ----------------------------------------------------------------------------------------------------
# CPU baseline: the reference's algorithm (CPU oracle port) on a bounded prefix of the workload
# ----------------------------------------------------------------------------------------------------
def cpu_chain_seconds(tokens, repeats=1):
    from oracle import nsa_oracle as O
    w = WORKLOAD
    torch.set_num_threads(os.cpu_count() or 1)
    host = make_inputs(tokens, 1234, "cpu")
    cu = torch.tensor([0, tokens], dtype=torch.int32)
    best = None
    for _ in range(repeats):
        t = {n: host[n].float().requires_grad_(n in ("q", "k", "v", "wk", "wv", "pe")) for n in host}
        t0 = time.perf_counter()
        ck, cu_k = O.linear_compress(t["k"], t["wk"], cu, w["ks"], w["st"], t["pe"])
        cv, _ = O.linear_compress(t["v"], t["wv"], cu, w["ks"], w["st"], None)
        o1, idx = O.compressed_attention(t["q"], ck, cv, w["ks"], w["st"], w["bs"], w["topk"], cu, cu_k,
                                         init_blocks=w["init_blocks"], local_blocks=w["local_blocks"])
        o2 = O.topk_sparse_attention(t["q"], t["k"], t["v"], idx, w["bs"], cu)
        torch.autograd.backward([o1, o2], [t["do1"], t["do2"]])
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def cpu_baseline_record(sample_tokens, seconds):
    """`value` is what was MEASURED: milliseconds of one forward+backward pass of the oracle port over the sample.  The
    full 65536-token workload cannot run on the host at all (the algorithm is quadratic in memory there); an estimate
    scaled by the useful-FLOP ratio is given separately and labelled as such."""
    _, f_full = flop_model(WORKLOAD["tokens"])
    _, f_sample = flop_model(sample_tokens)
    return dict(value=seconds * 1e3, unit="ms", cores=os.cpu_count() or 1, kind="port",
                sample=(f"oracle port (fp32 torch on the host cores), forward+backward of the same operator chain on the first "
                        f"{sample_tokens} tokens of the workload; value = measured ms for that sample"),
                sample_tokens=sample_tokens, useful_tflops=f_sample / 1e12 / seconds,
                estimate_full_workload_ms=seconds * 1e3 * f_full / f_sample,
                estimate_note=f"measured value x useful-FLOP ratio {f_full / f_sample:.1f} (65536 tokens / sample); not a measurement")


def run_reference(args, rank, world):
    """The reference's algorithm on the host cores: the CPU oracle port, timed on a bounded sample of the workload.  The line
    reports the SAMPLE it measured (config.workload says so); nothing is extrapolated into `value`."""
    if rank != 0:
        return
    sample = CPU_SAMPLE_TOKENS
    cpu_chain_seconds(256)   # untimed: thread pool start-up, first-call costs
    for _ in range(min(args.warmup, 1)):
        cpu_chain_seconds(sample)
    times = [cpu_chain_seconds(sample) for _ in range(max(1, args.steps))]
    sec = sum(times) / len(times)
    rec = cpu_baseline_record(sample, sec)
    cfg = config_record()
    cfg["workload"] = (f"BOUNDED SAMPLE of the workload: the first {sample} tokens of the sequence (the host implementation is "
                       f"quadratic in memory and cannot hold 65536) -- " + cfg["workload"].replace(f"{WORKLOAD['tokens']} tokens", f"{sample} tokens"))
    cfg["tokens_per_gpu"] = sample
    line = dict(impl="reference", metric=METRIC, value=rec["value"], unit="ms", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=rec["value"], higher_is_better=False, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic", config=cfg, cpu_baseline=rec,
                e2e=dict(value=rec["value"], unit="ms", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line), flush=True)


def config_record():
    w = WORKLOAD
    return dict(workload=(f"NSA operator chain fwd+bwd (linear_compress k,v -> compressed_attention + top-k -> "
                          f"topk_sparse_attention), one sequence of {w['tokens']} tokens per GPU, {w['Hq']}q/{w['Hkv']}kv heads, "
                          f"d={w['d']}, kernel {w['ks']}/stride {w['st']}, block {w['bs']}, topk {w['topk']}, bf16"),
                tokens_per_gpu=w["tokens"], sharding="one independent sequence per GPU, no data-path collective",
                l2_policy="inputs (q alone is 1.07 GB) exceed the 126 MB L2; no explicit flush")


# kernel -> (bound, algorithmic work per launch as a function of the useful-FLOP model of oracle.nsa_oracle.useful_flops)
# DRAM bytes (read + write) per launch measured by ncu on a 16384-token case.
# These kernels' DRAM traffic is their linear-in-tokens streams (Q, O, dO, dQ rows; K/V re-reads hit L2), so the figure is
# scaled by tokens / 16384 for the workload at hand.
NCU_DRAM_BYTES_16K = {
    "dense_fwd_tc": 0.271e9 + 226.9e6, "score_topk_tc": 0.275e9 + 6.3e6, "sparse_fwd": 0.306e9 + 241.0e6,
    "sparse_dq": 0.851e9 + 259.3e6, "sparse_dkdv_tc": 4.774e9 + 2.758e9, "dense_dq_tc": 0.815e9 + 253.8e6,
    "dense_dkdv_tc": 0.553e9 + 7.3e6,
}


def kernel_work(name, f, fused_dq=True):
    """fused_dq: the sparse dK/dV pass also produces dQ (no separate sparse_dq launch), so it is credited all five
    backward GEMM units of the selected-block attention."""
    cmp_f, sel_f, lin_f = f["cmp_fwd"], f["sel_fwd"], f["lin_fwd"]
    table = {
        "dense_fwd": ("tensor", cmp_f),            # S and PV
        "score_topk": ("tensor", cmp_f / 2),       # S recomputed once for the scores (selection overhead)
        "dense_dq": ("tensor", cmp_f),             # 2 of the 5 backward GEMM units
        "dense_dkdv": ("tensor", 1.5 * cmp_f),     # 3 of the 5 backward GEMM units
        "sparse_fwd": ("tensor", sel_f),
        "sparse_dq": ("tensor", sel_f),
        "sparse_dkdv": ("tensor", (2.5 if fused_dq else 1.5) * sel_f),
        "linear_compress_fwd": ("tensor", lin_f / 2),   # launched once per tensor (k, v)
        "linear_dw": ("tensor", lin_f / 2),
        "linear_dx": ("tensor", lin_f / 2),
    }
    name = name[:-3] if name.endswith("_tc") else name   # tcgen05 variants do the same algorithmic work
    return table.get(name)


def window_microbench(ops, dev, tokens):
    """Sliding-window branch (the third branch of an NSA layer) at the layer's shape: one sequence, 64q/4kv heads, d=128,
    window 512, forward + backward.  Useful FLOPs count unmasked (query, key) pairs only: 2 GEMMs forward, 5 backward."""
    g = torch.Generator().manual_seed(7)
    Hq, Hkv, d, W = WORKLOAD["Hq"], WORKLOAD["Hkv"], WORKLOAD["d"], 512
    q, k, v, do = (torch.randn(tokens, h, d, generator=g).to(torch.bfloat16).to(dev) for h in (Hq, Hkv, Hkv, Hq))
    for x in (q, k, v):
        x.requires_grad_(True)
    cu = torch.tensor([0, tokens], dtype=torch.int32, device=dev)

    def step():
        q.grad = k.grad = v.grad = None
        ops.sliding_window_attention(q, k, v, cu, tokens, W).backward(do)

    for _ in range(3):
        step()
    pkg_lib = sys.modules["native_sparse_attention_triton_b200"]._lib
    pkg_lib.profile(True)
    reps = 5
    for _ in range(reps):
        step()
    torch.cuda.synchronize()
    kern = pkg_lib.profile_collect()
    pkg_lib.profile(False)
    pairs = sum(min(t + 1, W + 1) for t in range(tokens))
    flops = 3.5 * 4 * d * Hq * pairs
    ms = sum(v_[1] for v_ in kern.values()) / reps
    return dict(tokens=tokens, window=W, kernel_ms=ms, useful_tflops=flops / 1e12 / (ms / 1e3),
                per_kernel_ms={k_: v_[1] / reps for k_, v_ in kern.items()})


def gate_combine_microbench(ops, dev, tokens):
    """Gated sum of the three branch outputs at the layer's shape (tokens x 64 heads x 128), forward and backward.  HBM-bound:
    achieved GB/s on the ALGORITHMIC bytes, 4 tensors forward (3 read, 1 written) and 7 backward (4 read, 3 written) plus the
    gates, 2 bytes per element.  The working set (1 GB per tensor at 65 536 tokens) is far larger than L2."""
    g = torch.Generator().manual_seed(9)
    Hq, d = WORKLOAD["Hq"], WORKLOAD["d"]
    outs = [torch.randn(tokens, Hq, d, generator=g).to(torch.bfloat16).to(dev).requires_grad_(True) for _ in range(3)]
    gate = torch.rand(tokens, Hq, 3, generator=g).to(torch.bfloat16).to(dev).requires_grad_(True)
    do = torch.randn(tokens, Hq, d, generator=g).to(torch.bfloat16).to(dev)

    def step():
        gate.grad = None
        for o in outs:
            o.grad = None
        ops.gate_combine(gate, *outs).backward(do)

    for _ in range(3):
        step()
    pkg_lib = sys.modules["native_sparse_attention_triton_b200"]._lib
    pkg_lib.profile(True)
    reps = 5
    for _ in range(reps):
        step()
    torch.cuda.synchronize()
    kern = pkg_lib.profile_collect()
    pkg_lib.profile(False)
    tensor_bytes = 2 * tokens * Hq * d
    gate_bytes = 2 * tokens * Hq * 3
    res = dict(tokens=tokens)
    for name, nbytes in (("gate_combine_fwd", 4 * tensor_bytes + gate_bytes), ("gate_combine_bwd", 7 * tensor_bytes + 2 * gate_bytes)):
        ms = kern[name][1] / reps
        res[name] = dict(ms=ms, bytes=nbytes, gb_per_s=nbytes / 1e9 / (ms / 1e3))
    return res


def rope_microbench(ops, dev, tokens):
    """Rotary embedding of the query tensor at the layer's shape (tokens x 64 heads x 128), forward only (the backward pass
    is the same kernel with the opposite angle).  HBM-bound: one read and one write of the tensor, 2 bytes per element."""
    g = torch.Generator().manual_seed(10)
    Hq, d = WORKLOAD["Hq"], WORKLOAD["d"]
    x = torch.randn(tokens, Hq, d, generator=g).to(torch.bfloat16).to(dev)
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
    cu = torch.tensor([0, tokens], dtype=torch.int32, device=dev)
    for _ in range(3):
        ops.rope(x, inv_freq, cu)
    pkg_lib = sys.modules["native_sparse_attention_triton_b200"]._lib
    pkg_lib.profile(True)
    reps = 5
    for _ in range(reps):
        ops.rope(x, inv_freq, cu)
    torch.cuda.synchronize()
    kern = pkg_lib.profile_collect()
    pkg_lib.profile(False)
    nbytes = 2 * 2 * tokens * Hq * d
    ms = kern["rope"][1] / reps
    return dict(tokens=tokens, ms=ms, bytes=nbytes, gb_per_s=nbytes / 1e9 / (ms / 1e3))


def decode_step_microbench(dev):
    """One whole decode step of an NSA layer's attention (stage + compress + rotary embedding + cache update + three
    attention branches + gated sum) at the shapes of the generation config (batch 4, 8192-token context, 32q/2kv heads,
    d=128, weighted-pool compression, top-8, window 512): launches per step, microseconds per step launched eagerly from
    Python and replayed from a CUDA graph."""
    from native_sparse_attention_triton_b200.infer import DecodeGraph, RotaryEmbedding, nsa_infer
    from native_sparse_attention_triton_b200.kv_cache import NSACache
    pkg = sys.modules["native_sparse_attention_triton_b200"]
    ops = pkg.ops
    B, L, Hq, Hkv, d, ks, st, bs, T, W = 4, 8192, 32, 2, 128, 32, 16, 64, 8, 512
    g = torch.Generator().manual_seed(21)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).to(dev)
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev) * L
    cache = NSACache(B, L + 256, Hkv, d, ks, st, W, torch.bfloat16, dev)
    rope = RotaryEmbedding((1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev))
    wk, wv = (torch.rand(Hkv, ks, generator=g) / ks).to(torch.bfloat16).to(dev), (torch.rand(Hkv, ks, generator=g) / ks).to(torch.bfloat16).to(dev)
    args = dict(rope=rope, cache=cache, compress_weight=(wk, wv), compress_func=(ops.weightedpool_compress, ops.weightedpool_compress),
                intra_block_pe=None, kernel_size=ks, kernel_stride=st, block_size=bs, topk=T, init_blocks=1, local_blocks=2,
                window_size=W)
    nsa_infer(cu, 0, mk(B * L, Hq, d), mk(B * L, Hkv, d), mk(B * L, Hkv, d), torch.rand(B * L, Hq, 3, generator=g).to(torch.bfloat16).to(dev), **args)
    step_in = [mk(B, Hq, d), mk(B, Hkv, d), mk(B, Hkv, d), torch.rand(B, Hq, 3, generator=g).to(torch.bfloat16).to(dev)]
    for s_ in range(1, 4):
        nsa_infer(cu, s_, *step_in, **args)
    n0 = pkg._lib.launch_count()
    nsa_infer(cu, 4, *step_in, **args)
    launches = pkg._lib.launch_count() - n0

    def timed(fn, reps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    reps = 40
    state = {"s": 5}

    def eager():
        nsa_infer(cu, state["s"], *step_in, **args)
        state["s"] += 1

    eager_us = timed(eager, reps)
    graph = DecodeGraph(cu, *step_in, **args)
    for _ in range(3):
        graph(*step_in)
    graph_us = timed(lambda: graph(*step_in), reps)
    return dict(batch=B, context=L, library_launches_per_step=launches, eager_us_per_step=eager_us, graph_us_per_step=graph_us,
                status=pkg.device_status())


def decode_inputs(dev, B, L, Hq, Hkv, T, ragged):
    """Seeded inputs of a decode case: caches [B, L, Hkv, 128], one query row per sequence, lengths, a random selection of
    T blocks per (head, sequence) and the compressed caches (kernel 32, stride 16)."""
    g = torch.Generator().manual_seed(42)
    d, bs, ks, st = 128, 64, 32, 16
    if ragged:
        seqlens = torch.clamp(torch.arange(B, dtype=torch.int32) % 76 * 128 + 1, max=L)
        seqlens = seqlens[torch.randperm(B, generator=g)]
    else:
        seqlens = torch.full((B,), 8192 + 64, dtype=torch.int32)
    q = torch.randn(B, Hq, d, generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn(B, L, Hkv, d, dtype=torch.bfloat16, device=dev)
    v = torch.randn(B, L, Hkv, d, dtype=torch.bfloat16, device=dev)
    Lc = (L - ks) // st + 1
    ck, cv = k[:, :Lc].contiguous(), v[:, :Lc].contiguous()
    clen = torch.clamp((seqlens - ks) // st + 1, min=0).to(torch.int32)
    nb = (seqlens.long() - 1) // bs + 1
    idx = torch.full((Hkv, B, T), -1, dtype=torch.int32)
    for b in range(B):
        n = int(nb[b])
        for h in range(Hkv):
            pick = torch.randperm(n, generator=g)[: min(T, n)].sort().values
            idx[h, b, : pick.numel()] = pick.int()
    return dict(q=q, k=k, v=v, ck=ck, cv=cv, seqlens=seqlens, clen=clen, idx=idx.to(dev), sl=seqlens.to(dev), cl=clen.to(dev),
                d=d, bs=bs, ks=ks, st=st, T=T)


def decode_profile_case(ops, dev):
    """Two rounds of (flash, selected-block, compressed) decode on the bandwidth case: launches 3..5 are the warm ones."""
    x = decode_inputs(dev, 76, 8192, 32, 4, 16, True)
    for _ in range(2):
        ops.flash_attention_decode(x["q"], x["k"], x["v"], x["sl"])
        ops.topk_sparse_attention_decode(x["q"], x["k"], x["v"], x["idx"], x["bs"], x["sl"])
        ops.compressed_attention_decode(x["q"], x["ck"], x["cv"], x["sl"], x["cl"], x["ks"], x["st"], x["bs"], x["T"], max_seqlen=8192)
    torch.cuda.synchronize()
    print(json.dumps(dict(decode_profile="ok")))


def compress_profile_case(ops, dev):
    """The three compression operators on 1 048 576 tokens x 4 heads x 128 (1.07 GB of input: larger than L2, small enough for
    a profiler to replay), a cache-evicting write before each call; two rounds, the second one warm."""
    N, H, d, ks, st = 1048576, WORKLOAD["Hkv"], WORKLOAD["d"], 32, 16
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(N, H, d, generator=g, device=dev).to(torch.bfloat16)
    wl = (torch.randn(H, ks * d, d, generator=g, device=dev) / math.sqrt(ks * d)).to(torch.bfloat16)
    wp = (torch.rand(H, ks, generator=g, device=dev) / ks).to(torch.bfloat16)
    pe = (torch.randn(H, ks, d, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    cu = torch.tensor([0, N], dtype=torch.int32, device=dev)
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device=dev)
    with torch.no_grad():
        for _ in range(2):
            for fn in (lambda: ops.weightedpool_compress(x, wp, cu, ks, st, pe), lambda: ops.linear_compress(x, wl, cu, ks, st, pe)):
                flush.zero_()
                fn()
    torch.cuda.synchronize()
    print(json.dumps(dict(compress_profile="ok")))


def decode_microbench(ops, dev):
    """The three single-token operators on (a) the bandwidth-sized case of the reference's decode self-tests
    (batch 76, cache 8192, 32q/4kv heads, d=128, block 64, top-16, ragged lengths), (b) the same case with four times
    the batch (304 sequences: the selected-block and compressed operators move only 148 MB and 45 MB at batch 76, where the
    9 us a kernel needs before its first tile has arrived is a third of the run) and (c) the shapes of the generation
    config (batch 4, 8192-token context, 32q/2kv heads).  Returns microseconds and achieved GB/s on the ALGORITHMIC bytes
    (K and V rows that must be read, 2 bytes each)."""
    out = {}
    for tag, B, L, Hq, Hkv in (("bandwidth_case", 76, 8192, 32, 4), ("bandwidth_case_batch_304", 304, 8192, 32, 4),
                               ("generation_case", 4, 8192 + 128, 32, 2)):
        T = 16 if tag.startswith("bandwidth_case") else 8
        x = decode_inputs(dev, B, L, Hq, Hkv, T, tag.startswith("bandwidth_case"))
        q, k, v, ck, cv, idx, sl, cl, seqlens, clen = (x[n] for n in ("q", "k", "v", "ck", "cv", "idx", "sl", "cl", "seqlens", "clen"))
        d, bs, ks, st = x["d"], x["bs"], x["ks"], x["st"]
        sel_rows = sum(min(bs, int(seqlens[b]) - int(i) * bs) for b in range(B) for h in range(1) for i in idx[0, b].tolist() if i >= 0)
        work = {
            "flash_attention_decode": (lambda: ops.flash_attention_decode(q, k, v, sl), 4 * int(seqlens.sum()) * Hkv * d),
            "topk_sparse_attention_decode": (lambda: ops.topk_sparse_attention_decode(q, k, v, idx, bs, sl), 4 * sel_rows * Hkv * d),
            "compressed_attention_decode": (lambda: ops.compressed_attention_decode(q, ck, cv, sl, cl, ks, st, bs, T),
                                            4 * int(clen.sum()) * Hkv * d),
        }
        flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device=dev)
        res = {}
        import native_sparse_attention_triton_b200 as pkg
        for name, (fn, nbytes) in work.items():
            for _ in range(3):
                fn()
            times = []
            pkg._lib.profile_collect()
            pkg._lib.profile(True)
            reps = 10
            for _ in range(reps):
                flush.zero_()   # 256 MB write: evicts the caches between timed calls
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            kern = pkg._lib.profile_collect()   # device time of the library's kernels alone (CUDA events around each launch)
            pkg._lib.profile(False)
            kernel_ms = sum(v[1] for v in kern.values()) / reps
            times.sort()
            ms = times[len(times) // 2]
            res[name] = dict(op_us=ms * 1e3, kernel_us=kernel_ms * 1e3, algorithmic_bytes=nbytes,
                             kernel_gb_per_s=nbytes / 1e9 / (kernel_ms / 1e3),
                             frac_of_hbm_peak=nbytes / 1e9 / (kernel_ms / 1e3) / peaks()["hbm"], kernels=sorted(kern))
        out[tag] = res
        del q, k, v, ck, cv
        torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------------------------------
# the unmodified reference project on the same GPU (baseline/_ref, installed by baseline/install_reference.sh)
# ----------------------------------------------------------------------------------------------------
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
_REF_PKG = "native_sparse_attention"


def load_reference(layers=False):
    """Import the reference with ITS OWN Triton operators bound (modules of an earlier import, shimmed or not, are dropped
    first).  None when baseline/_ref is absent.  transformers 5.x wants `rope_parameters` / `standardize_rope_params` on the
    rope config: both are added to the reference's RopeConfig class, outside any arithmetic."""
    if not os.path.isfile(os.path.join(REF_DIR, _REF_PKG, "__init__.py")):
        return None
    for name in [n for n in sys.modules if n == _REF_PKG or n.startswith(_REF_PKG + ".")]:
        del sys.modules[name]
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import native_sparse_attention as ref
    import native_sparse_attention.ops  # noqa: F401
    if layers:
        import native_sparse_attention.module.rope as rope_mod
        cfg = rope_mod.RopeConfig
        if not hasattr(cfg, "standardize_rope_params"):
            cfg.standardize_rope_params = lambda self: None
            cfg.rope_parameters = property(lambda self: dict(self.rope_scaling or {}, rope_theta=self.rope_theta))
        import native_sparse_attention.infer  # noqa: F401
        import native_sparse_attention.model  # noqa: F401
        import native_sparse_attention.module  # noqa: F401
    return ref


def reference_linear_compress():
    """The reference's Triton linear_compress where it compiles, else its own torch implementation of the operator
    (Triton 3.6 fails on linear_compress_fwd_kernel for sm_100: PassManager::run failed in TritonGPUOptimizeDotOperands)."""
    from native_sparse_attention.ops import linear_compress
    from native_sparse_attention.ops.torch.compress_key_value import linear_compress_torch
    try:
        x = torch.zeros(64, 1, 64, dtype=torch.bfloat16, device="cuda")
        w = torch.zeros(1, 32 * 64, 64, dtype=torch.bfloat16, device="cuda")
        linear_compress(x, w, torch.tensor([0, 64], dtype=torch.int32, device="cuda"), 32, 16, None)
        torch.cuda.synchronize()
        return linear_compress, "triton"
    except RuntimeError as e:
        if "PassManager" not in str(e):
            raise
        return linear_compress_torch, "torch (the Triton kernel does not compile under this Triton)"


def time_gpu(fn, warmup=2, reps=3):
    """Median milliseconds of fn() by CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def gpu_reference_chain(t, cu, max_q, max_k):
    """The SAME operator chain, inputs and step as the headline number, through the reference's own operators (Triton JIT
    for sm_100) on the same GPU in the same run; the first call (compilation) is excluded."""
    try:
        if load_reference() is None:
            return dict(unavailable="baseline/_ref is absent (sh baseline/install_reference.sh <reference checkout>)")
        from native_sparse_attention.ops import compressed_attention, topk_sparse_attention
        lin, which = reference_linear_compress()
        w = WORKLOAD

        def step():
            for n in ("q", "k", "v", "wk", "wv", "pe"):
                t[n].grad = None
            ck, cu_k = lin(t["k"], t["wk"], cu, w["ks"], w["st"], t["pe"])
            cv, _ = lin(t["v"], t["wv"], cu, w["ks"], w["st"], None)
            o1, idx = compressed_attention(t["q"], ck, cv, w["ks"], w["st"], w["bs"], w["topk"], cu, cu_k, max_q, max_k, None,
                                           w["init_blocks"], w["local_blocks"])
            o2 = topk_sparse_attention(t["q"], t["k"], t["v"], idx, w["bs"], cu)
            torch.autograd.backward([o1, o2], [t["do1"], t["do2"]])

        ms = time_gpu(step, warmup=2, reps=3)
        import triton
        return dict(ms_per_step=ms, linear_compress=which, triton=triton.__version__,
                    what="reference ops (Triton) on this GPU, same inputs and chain as `value`; median of 3 after 2 warm-up calls")
    except Exception as e:  # the reference failing to run here must not take the benchmark down
        return dict(unavailable=f"{type(e).__name__}: {str(e)[:300]}")
    finally:
        for n in ("q", "k", "v", "wk", "wv", "pe"):
            t[n].grad = None
        torch.cuda.empty_cache()


def config3_sweep(ops, dev, with_reference):
    """BASELINE configuration 3: topk_sparse_attention forward+backward on one sequence of N tokens (64q/4kv heads, d=128,
    block 64), top-k 8 and 16 with the selection produced by compressed_attention on N(0,1) q/k, beside dense causal
    attention at the same shape (this library's flash_attention_varlen; the reference's Triton kernels where present)."""
    Hq, Hkv, d, ks, st, bs = WORKLOAD["Hq"], WORKLOAD["Hkv"], WORKLOAD["d"], 32, 16, 64
    ref_sparse = ref_dense = None
    if with_reference and load_reference() is not None:
        from native_sparse_attention.ops import flash_attention_varlen as ref_dense
        from native_sparse_attention.ops import topk_sparse_attention as ref_sparse
    rows = []
    for N in (2048, 8192, 32768, 65536):
        g = torch.Generator(device=dev).manual_seed(300 + N)
        q, k, v, do = (torch.randn(N, h, d, generator=g, device=dev).to(torch.bfloat16) for h in (Hq, Hkv, Hkv, Hq))
        for x in (q, k, v):
            x.requires_grad_(True)
        cu = torch.tensor([0, N], dtype=torch.int32, device=dev)

        def fwd_bwd(fn):
            def run():
                q.grad = k.grad = v.grad = None
                fn().backward(do)
            return run

        dense_ms = time_gpu(fwd_bwd(lambda: ops.flash_attention_varlen(q, k, v, cu, cu, N, N, causal=True)), 1, 3)
        row = dict(tokens=N, dense_causal_ms=dense_ms, dense_causal_tflops=3.5 * 4 * d * Hq * (N * (N + 1) / 2) / 1e12 / (dense_ms / 1e3))
        try:
            if ref_dense is not None:
                row["reference_dense_causal_ms"] = time_gpu(fwd_bwd(lambda: ref_dense(q, k, v, cu, cu, N, N, causal=True)), 1, 2)
        except Exception as e:
            row["reference_dense_causal_ms"] = f"failed: {type(e).__name__}: {str(e)[:120]}"
        with torch.no_grad():
            ck, cu_k = ops.avgpool_compress(k, None, cu, ks, st)
            cv, _ = ops.avgpool_compress(v, None, cu, ks, st)
        for topk in (8, 16):
            with torch.no_grad():
                idx = ops.compressed_attention(q, ck, cv, ks, st, bs, topk, cu, cu_k, N, ck.shape[0])[1]
            ms = time_gpu(fwd_bwd(lambda: ops.topk_sparse_attention(q, k, v, idx, bs, cu)), 1, 3)
            from oracle import nsa_oracle as O
            pairs = O.visible_pairs_selected([N], bs, topk)
            rec = dict(ms=ms, useful_tflops=3.5 * 4 * d * Hq * pairs / 1e12 / (ms / 1e3), speedup_vs_dense_causal=dense_ms / ms)
            try:
                if ref_sparse is not None:
                    rec["reference_ms"] = time_gpu(fwd_bwd(lambda: ref_sparse(q, k, v, idx, bs, cu)), 1, 2)
            except Exception as e:
                rec["reference_ms"] = f"failed: {type(e).__name__}: {str(e)[:120]}"
            row[f"top{topk}"] = rec
        rows.append(row)
        del q, k, v, do
        torch.cuda.empty_cache()
    return rows


def compression_bandwidth(ops, dev):
    """Compression forward kernels against HBM: 2 097 152 tokens x 4 heads x 128 (2.1 GB of input; at 262 144 tokens the
    pooling kernels last 86 us, a fifth of which is ramp-up: 3.3 TB/s there, 4.7 TB/s at 4 M tokens), kernel 32, stride 16;
    a 256 MB write between timed calls evicts the caches.  Algorithmic bytes: input read once, output written once (plus
    the weights of the linear projection)."""
    pkg = sys.modules["native_sparse_attention_triton_b200"]
    N, H, d, ks, st = 2097152, WORKLOAD["Hkv"], WORKLOAD["d"], 32, 16
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(N, H, d, generator=g, device=dev).to(torch.bfloat16)
    wl = (torch.randn(H, ks * d, d, generator=g, device=dev) / math.sqrt(ks * d)).to(torch.bfloat16)
    wp = (torch.rand(H, ks, generator=g, device=dev) / ks).to(torch.bfloat16)
    pe = (torch.randn(H, ks, d, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    cu = torch.tensor([0, N], dtype=torch.int32, device=dev)
    M = (N - ks) // st + 1
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device=dev)
    io = 2 * (N * H * d + M * H * d)
    work = {"weightedpool_compress": (lambda: ops.weightedpool_compress(x, wp, cu, ks, st, pe), io, "pool_compress_fwd"),
            "avgpool_compress": (lambda: ops.avgpool_compress(x, None, cu, ks, st, pe), io, "pool_compress_fwd"),
            "linear_compress": (lambda: ops.linear_compress(x, wl, cu, ks, st, pe), io + 2 * (H * ks * d * d + H * ks * d), "linear_compress_fwd")}
    out = dict(tokens=N, heads=H)
    # backward of the two pooling modes: dy and x read once, dx written once (average pooling needs no x)
    dy = torch.randn(M, H, d, generator=g, device=dev).to(torch.bfloat16)
    for t_ in (x, wp, pe):
        t_.requires_grad_(True)
    bwd = {"weightedpool_compress_bwd": (lambda: ops.weightedpool_compress(x, wp, cu, ks, st, pe)[0], 2 * (2 * N * H * d + M * H * d)),
           "avgpool_compress_bwd": (lambda: ops.avgpool_compress(x, None, cu, ks, st, pe)[0], 2 * (N * H * d + M * H * d))}
    for name, (fn, nbytes) in bwd.items():
        for _ in range(2):
            fn().backward(dy)
            x.grad = wp.grad = pe.grad = None
        reps, ms = 3, 0.0
        for _ in range(reps):
            y_ = fn()
            flush.zero_()
            pkg._lib.profile_collect()
            pkg._lib.profile(True)
            y_.backward(dy)
            torch.cuda.synchronize()
            kern = pkg._lib.profile_collect()
            pkg._lib.profile(False)
            x.grad = wp.grad = pe.grad = None
            ms += sum(v_[1] for k_, v_ in kern.items() if k_.startswith("pool_dx"))
        ms /= reps
        out[name] = dict(kernels=sorted(k_ for k_ in kern if k_.startswith("pool_d")), main_kernel_ms=ms, algorithmic_bytes=nbytes,
                         gb_per_s=nbytes / 1e9 / (ms / 1e3), frac_of_hbm_peak=nbytes / 1e9 / (ms / 1e3) / peaks()["hbm"],
                         all_kernels_ms={k_: v_[1] for k_, v_ in kern.items()})
    for t_ in (x, wp, pe):
        t_.requires_grad_(False)
    with torch.no_grad():
        for name, (fn, nbytes, kern_name) in work.items():
            for _ in range(2):
                fn()
            pkg._lib.profile_collect()
            pkg._lib.profile(True)
            reps = 5
            for _ in range(reps):
                flush.zero_()
                fn()
            torch.cuda.synchronize()
            kern = pkg._lib.profile_collect()
            pkg._lib.profile(False)
            ms = kern[kern_name][1] / reps
            out[name] = dict(kernel=kern_name, kernel_ms=ms, algorithmic_bytes=nbytes, gb_per_s=nbytes / 1e9 / (ms / 1e3),
                             frac_of_hbm_peak=nbytes / 1e9 / (ms / 1e3) / peaks()["hbm"])
    return out


def config5_generate(dev):
    """BASELINE configuration 5: the reference's OWN ToyNSALlama (8 layers, hidden 4096, ffn 14336, 32q/2kv heads, d=128,
    weighted-pool compression, top-8, window 512, vocab 128256, random weights ~N(0, 0.02)) generating 128 greedy tokens
    for 4 prompts of 8192 uniform-random tokens.  Run twice on identical weights: bound to the reference's Triton
    operators, flash_attn and its NSACache, and -- after shim.install(), install_sliding_window(), install_inference() -- bound
    to this library.  With this library a decode step of the whole model has no host synchronisation, so it is also
    captured in a CUDA graph and replayed.  Decode tokens/s counts the 127 steps after the prefill."""
    try:
        if load_reference(layers=True) is None:
            return dict(unavailable="baseline/_ref is absent: see decode_step for the per-layer attention step measured alone")
        from native_sparse_attention.model import InferenceConfig, ToyNSALlama, ToyNSALlamaConfig
        B, P, NEW = 4, 8192, 128
        cfg = ToyNSALlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=8,
                                num_attention_heads=32, num_key_value_heads=2, head_dim=128, compress_type="weightedpool",
                                kernel_size=32, kernel_stride=16, block_size=64, topk=8, init_blocks=1, local_blocks=2, window_size=512)
        icfg = InferenceConfig(max_batch_size=B, max_length=P + NEW + 64, max_new_tokens=NEW)

        def build():
            with torch.device(dev):
                m = ToyNSALlama(cfg, icfg).bfloat16()
            return m

        g = torch.Generator(device=dev).manual_seed(55)
        model = build()
        with torch.no_grad():
            for prm in model.parameters():
                if prm.dim() > 1:
                    prm.copy_((torch.randn(prm.shape, generator=g, device=dev) * 0.02).to(prm.dtype))
        ids = torch.randint(0, cfg.vocab_size, (B * P,), generator=g, device=dev)
        cu = torch.arange(B + 1, dtype=torch.int32, device=dev) * P
        n_params = sum(prm.numel() for prm in model.parameters())
        weight_bytes = 2 * (n_params - model.embedding.weight.numel())   # a decode step reads every weight but 4 embedding rows

        first_logits = {}

        def generate(m, steps, tag=None):
            """(prefill ms, decode ms for steps-1 steps, tokens [B, steps])"""
            m.kv_cache = None
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            logits = m.inference(ids, cu, 0)
            if tag:
                first_logits[tag] = logits
            tok = logits.argmax(-1)
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            toks = [tok]
            for step in range(1, steps):
                tok = m.inference(tok, cu, step).argmax(-1)
                toks.append(tok)
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            return (t1 - t0) * 1e3, (t2 - t1) * 1e3, torch.stack(toks, 1)

        out = dict(batch=B, prompt_tokens=P, new_tokens=NEW, parameters=n_params, weight_bytes_read_per_step=weight_bytes,
                   weights_only_ceiling_tokens_per_s=B / (weight_bytes / (peaks()["hbm"] * 1e9)))
        try:
            generate(model, 3)   # Triton compilation, allocator warm-up
            pre, dec, toks_ref = generate(model, NEW, "reference")
            out["reference"] = dict(prefill_ms=pre, decode_ms=dec, decode_tokens_per_s=B * (NEW - 1) / (dec / 1e3),
                                    end_to_end_tokens_per_s=B * NEW / ((pre + dec) / 1e3),
                                    what="reference model on its own Triton operators, flash_attn and NSACache (eager)")
        except Exception as e:
            toks_ref = None
            out["reference"] = dict(unavailable=f"{type(e).__name__}: {str(e)[:300]}")
        model.kv_cache = None
        torch.cuda.empty_cache()

        # ---- the same model class and weights on this library ----
        from native_sparse_attention_triton_b200 import shim
        from native_sparse_attention_triton_b200.infer import DecodeGraph
        shim.install(patch_loaded=True)
        shim.install_sliding_window()
        shim.install_inference()
        ours = build()
        ours.load_state_dict(model.state_dict())
        del model
        torch.cuda.empty_cache()
        generate(ours, 3)
        pre, dec, toks = generate(ours, NEW, "ours")
        rec = dict(prefill_ms=pre, decode_ms=dec, decode_tokens_per_s=B * (NEW - 1) / (dec / 1e3),
                   end_to_end_tokens_per_s=B * NEW / ((pre + dec) / 1e3),
                   what="reference model class, unchanged, on libnsa_b200 through the shim (eager Python decode loop)")
        if "reference" in first_logits:
            # Free-running greedy decoding of a random-weight model is chaotic (its logits are noise of RMS 0.6 over 128256
            # classes, so any rounding difference changes the argmax and every later step); what can be compared is the
            # logits both produce for the same input: the prefill's.  tests/test_gpu_reference_layers.py compares every step
            # with the reference's tokens fed to both.
            a, b = first_logits["ours"].float(), first_logits["reference"].float()
            rec["prefill_logits_vs_reference"] = dict(max_abs_diff=float((a - b).abs().max()), mean_abs_diff=float((a - b).abs().mean()),
                                                      reference_rms=float(b.pow(2).mean().sqrt()))
        out["this_library_eager"] = rec

        # ---- the decode step of the whole model replayed from a CUDA graph ----
        ours.kv_cache = None
        tok = ours.inference(ids, cu, 0).argmax(-1)
        tok_static = tok.clone()
        caches = ours.kv_cache
        state = [[x.clone() for x in DecodeGraph._state(c)] for c in caches]
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            ours.inference(tok_static, cu, 1)        # one-time initialisations happen outside the capture
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            logits_static = ours.inference(tok_static, cu, 1)
        for c, st_ in zip(caches, state):            # warm-up and capture advanced the caches: put them back
            for dst, src in zip(DecodeGraph._state(c), st_):
                dst.copy_(src)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        toks_g = [tok]
        for _ in range(1, NEW):
            graph.replay()
            nxt = logits_static.argmax(-1)
            tok_static.copy_(nxt)
            toks_g.append(nxt)
        torch.cuda.synchronize()
        dec_g = (time.perf_counter() - t1) * 1e3
        toks_g = torch.stack(toks_g, 1)
        out["this_library_cuda_graph"] = dict(decode_ms=dec_g, decode_tokens_per_s=B * (NEW - 1) / (dec_g / 1e3),
                                              ms_per_step=dec_g / (NEW - 1),
                                              greedy_tokens_equal_to_eager=f"{int((toks_g == toks).sum())}/{toks.numel()}",
                                              what="one whole-model decode step captured once (no host synchronisation inside), replayed 127 times")
        out["decode_tokens_per_s_per_gpu"] = out["this_library_cuda_graph"]["decode_tokens_per_s"]
        return out
    except Exception as e:
        import traceback
        return dict(unavailable=f"{type(e).__name__}: {str(e)[:300]}", where=traceback.format_exc()[-600:])
    finally:
        for name in [n for n in sys.modules if n == _REF_PKG or n.startswith(_REF_PKG + ".")]:
            del sys.modules[name]
        torch.cuda.empty_cache()


def strong_scaling(ops, dev, rank, world, dist):
    """The two partitionings of the path across the GPUs of one node, with NCCL only to gather the outputs:
    (a) BASELINE configuration 4's batch (8 sequences x 32768 tokens) split by sequence over the ranks;
    (b) configuration 3's single 65536-token sequence split by KV-head group (ranks <= 4 KV heads).
    Each leg: forward+backward of the operator chain on the rank's shard, then all-gather of both attention outputs;
    milliseconds are device time, maximum over ranks."""
    from native_sparse_attention_triton_b200 import dist as nd
    w = WORKLOAD
    Hq, Hkv, d, ks = w["Hq"], w["Hkv"], w["d"], w["ks"]
    out = {}

    def maxed(x):
        tt = torch.tensor([x], device=dev)
        if dist is not None:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    def run_leg(t, cu, max_q, gather):
        max_k = (max_q - ks) // w["st"] + 1

        def compute():
            return chain_step(ops, t, cu, max_q, max_k)

        for _ in range(2):
            o1, o2 = compute()
            gather(o1.detach()), gather(o2.detach())
        res = []
        for _ in range(3):
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            o1, o2 = compute()
            e1.record()
            gather(o1.detach()), gather(o2.detach())
            e2.record()
            torch.cuda.synchronize()
            res.append((maxed(e0.elapsed_time(e2)), maxed(e0.elapsed_time(e1)), maxed(e1.elapsed_time(e2))))
        res.sort()
        return dict(ms=res[1][0], compute_ms=res[1][1], gather_ms=res[1][2], gather_share=res[1][2] / res[1][0])

    def make(seqlens, heads_q, heads_kv, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        n = sum(seqlens)
        mk = lambda *s, scale=1.0: (torch.randn(*s, generator=g, device=dev) * scale).to(torch.bfloat16)
        t = dict(q=mk(n, heads_q, d), k=mk(n, heads_kv, d), v=mk(n, heads_kv, d), wk=mk(heads_kv, ks * d, d, scale=1 / math.sqrt(ks * d)),
                 wv=mk(heads_kv, ks * d, d, scale=1 / math.sqrt(ks * d)), pe=mk(heads_kv, ks, d, scale=0.02), do1=mk(n, heads_q, d),
                 do2=mk(n, heads_q, d))
        for nme in ("q", "k", "v", "wk", "wv", "pe"):
            t[nme].requires_grad_(True)
        return t

    # (a) by sequence
    seqlens = [32768] * 8
    parts = nd.partition_sequences(seqlens, world, kernel_stride=w["st"], block_size=w["bs"], topk=w["topk"])
    mine = [seqlens[i] for i in parts[rank]]
    cu_all = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32, device=dev)
    t = make(mine, Hq, Hkv, 900 + rank)
    cu = torch.tensor([0] + list(torch.tensor(mine).cumsum(0)), dtype=torch.int32, device=dev)
    gather = (lambda o: nd.gather_varlen(o, parts, cu_all)) if dist is not None else (lambda o: o)
    out["by_sequence"] = dict(run_leg(t, cu, 32768, gather), sequences=8, tokens_per_sequence=32768, sequences_per_rank=len(mine),
                              what="configuration 4's batch, operator chain fwd+bwd per rank, outputs all-gathered in token order")
    del t
    torch.cuda.empty_cache()
    # (b) by KV-head group
    if Hkv % world == 0:
        h0, h1 = nd.kv_head_range(rank, world, Hkv)
        G = Hq // Hkv
        t = make([w["tokens"]], (h1 - h0) * G, h1 - h0, 950 + rank)
        cu = torch.tensor([0, w["tokens"]], dtype=torch.int32, device=dev)
        gather = (lambda o: nd.gather_heads(o)) if dist is not None else (lambda o: o)
        out["by_kv_head"] = dict(run_leg(t, cu, w["tokens"], gather), tokens=w["tokens"], kv_heads_per_rank=h1 - h0,
                                 what="configuration 3's sequence, each rank its KV heads and their query heads, outputs all-gathered along heads")
        del t
        torch.cuda.empty_cache()
    else:
        out["by_kv_head"] = dict(skipped=f"{Hkv} KV heads do not divide over {world} ranks")
    return out



def step_timeline(ops, t, cu, max_q, max_k):
    """Device timeline of one step (`--timeline`): every kernel, memset and copy of the middle one of three steps recorded
    by torch.profiler, summarised as the span of the step, the time the device was busy, the idle gaps between activities,
    and how the busy time splits into this library's kernels, memsets and torch's own kernels (autograd's accumulation of
    the two query gradients, index arithmetic).  Taken under a tracer: it explains `ms_per_step`, it is not a bench value."""
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            chain_step(ops, t, cu, max_q, max_k)
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                key=lambda e: e.time_range.start)
    marks = [i for i, e in enumerate(ev) if "linear_bias" in e.name]   # the first launch of a step
    if len(marks) < 3:
        return dict(error="step boundaries not found in the trace")
    step = ev[marks[1]:marks[2]]
    groups = dict(library_kernels=0.0, memsets=0.0, copies=0.0, torch_kernels=0.0)
    other = {}
    busy = gaps = 0.0
    end = step[0].time_range.start
    for e in step:
        dur = e.time_range.end - e.time_range.start
        gaps += max(0.0, e.time_range.start - end)
        end = max(end, e.time_range.end)
        busy += dur
        if "nsa::" in e.name:
            groups["library_kernels"] += dur
        elif e.name.startswith("Memset"):
            groups["memsets"] += dur
        elif e.name.startswith("Memcpy"):
            groups["copies"] += dur
        else:
            groups["torch_kernels"] += dur
            key = e.name.split("<")[0].split("(")[0].replace("void ", "")[:60]
            other[key] = other.get(key, 0.0) + dur
    top_other = sorted(other.items(), key=lambda kv: -kv[1])[:4]
    return dict(span_ms=(ev[marks[2]].time_range.start - step[0].time_range.start) / 1e3, busy_ms=busy / 1e3,
                idle_gaps_ms=gaps / 1e3, activities=len(step), **{k + "_ms": v / 1e3 for k, v in groups.items()},
                largest_torch_kernels_ms={k: v / 1e3 for k, v in top_other},
                what="one step under torch.profiler (CUPTI activity trace); explains ms_per_step, not a bench value")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=None, help="override the sequence length (parity/debug only)")
    ap.add_argument("--topk", type=int, default=None, help="override the number of selected blocks (size sweep only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode-operator micro-benchmark")
    ap.add_argument("--decode-profile", action="store_true",
                    help="only run the three decode operators twice each on the bandwidth case (the input of an ncu capture)")
    ap.add_argument("--compress-profile", action="store_true",
                    help="run only the compression operators on a 1 M-token case (the case the profiler captures)")
    ap.add_argument("--timeline", action="store_true",
                    help="add `step_timeline`: where one step's device time goes (library kernels, memsets, torch kernels, gaps)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the legs beside the headline: reference on the GPU, size sweep, generation, strong scaling")
    args = ap.parse_args()
    if args.tokens:
        WORKLOAD["tokens"] = args.tokens
    if args.topk:
        WORKLOAD["topk"] = args.topk

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import native_sparse_attention_triton_b200 as pkg
    ops = pkg.ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.decode_profile:
        decode_profile_case(ops, dev)
        return
    if args.compress_profile:
        compress_profile_case(ops, dev)
        return
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    w = WORKLOAD
    N = w["tokens"]
    host = make_inputs(N, 42 + rank, dev, pin=True)
    cu = torch.tensor([0, N], dtype=torch.int32, device=dev)
    max_q = N
    max_k = (N - w["ks"]) // w["st"] + 1
    grad_names = ("q", "k", "v", "wk", "wv", "pe")
    t = {n: host[n].to(dev, non_blocking=True) for n in host}
    for n in grad_names:
        t[n].requires_grad_(True)

    for _ in range(max(args.warmup, 3)):
        chain_step(ops, t, cu, max_q, max_k)
    barrier()
    assert pkg.device_status() == 0, "device-side anomaly during warm-up"

    # ---------------- timed region: K steps, inputs resident in HBM ----------------
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = pkg._lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        chain_step(ops, t, cu, max_q, max_k)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    launches = (pkg._lib.launch_count() - launches0)
    clocks = sampler.stop() if sampler else None
    ms_t = torch.tensor([ms], device=dev)
    if dist is not None:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms = float(ms_t.item())

    # ---------------- per-kernel device time (CUDA events inside the library, on the launching stream) ----------------
    pkg._lib.profile(True)
    prof_steps = 2
    for _ in range(prof_steps):
        chain_step(ops, t, cu, max_q, max_k)
    prof = pkg._lib.profile_collect()
    pkg._lib.profile(False)

    timeline = step_timeline(ops, t, cu, max_q, max_k) if (args.timeline and rank == 0) else None

    # ---------------- end to end: host buffers -> device, step, loss back to the host ----------------
    # Two sets of device inputs: the copy of step s+1 (its own stream) runs under the compute of step s, as a training
    # loop with a prefetching loader would do it.  Every step still copies all of its inputs from pinned host memory and
    # reads its loss back; the first copy is not hidden and is inside the timed region.
    e2e_steps = max(4, args.steps)  # as many as the timed region: the first copy cannot hide under a previous step
    h2d_bytes = sum(host[n].numel() * host[n].element_size() for n in host)
    loss_host = torch.empty(e2e_steps, dtype=torch.float32).pin_memory()
    t2 = {n: torch.empty_like(t[n]) for n in t}
    for n in grad_names:
        t2[n].requires_grad_(True)
    sets = (t, t2)
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    copied = [torch.cuda.Event() for _ in range(e2e_steps)]
    freed = [torch.cuda.Event() for _ in range(e2e_steps)]
    barrier()
    e0.record()
    copy_stream.wait_stream(main_stream)

    copy_begin = [torch.cuda.Event(enable_timing=True) for _ in range(e2e_steps)]
    copy_end = [torch.cuda.Event(enable_timing=True) for _ in range(e2e_steps)]

    def enqueue_copy(sidx):
        with torch.cuda.stream(copy_stream), torch.no_grad():
            if sidx >= 2:
                copy_stream.wait_event(freed[sidx - 2])   # the step that used this set has finished with it
            copy_begin[sidx].record(copy_stream)
            for n in host:
                sets[sidx % 2][n].copy_(host[n], non_blocking=True)
            copy_end[sidx].record(copy_stream)
            copied[sidx].record(copy_stream)

    enqueue_copy(0)
    for sidx in range(e2e_steps):
        if sidx + 1 < e2e_steps:
            enqueue_copy(sidx + 1)
        ts = sets[sidx % 2]
        main_stream.wait_event(copied[sidx])
        o1, o2 = chain_step(ops, ts, cu, max_q, max_k)
        loss = torch.dot(o1.flatten(), ts["do1"].flatten()).float() + torch.dot(o2.flatten(), ts["do2"].flatten()).float()
        loss_host[sidx:sidx + 1].copy_(loss.detach().reshape(1), non_blocking=True)
        freed[sidx].record(main_stream)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    # the copies alone, as they ran under the previous step's compute (the first one ran alone)
    e2e_copy_ms = [copy_begin[i].elapsed_time(copy_end[i]) for i in range(e2e_steps)]
    e2e_t = torch.tensor([e2e_ms], device=dev)
    if dist is not None:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_t.item())
    # ---------------- host link: every rank copies its inputs at the same time (what bounds e2e at 4 and 8 GPUs) ----------------
    barrier()
    with torch.no_grad():
        for n in host:
            t2[n].copy_(host[n], non_blocking=True)
        barrier()
        e0.record()
        for n in host:
            t2[n].copy_(host[n], non_blocking=True)
        e1.record()
    barrier()
    h2d = torch.tensor([h2d_bytes / 1e9 / (e0.elapsed_time(e1) / 1e3)], device=dev)
    h2d_all = [torch.zeros_like(h2d) for _ in range(world)]
    if dist is not None:
        dist.all_gather(h2d_all, h2d)
    else:
        h2d_all = [h2d]
    h2d_gbs = [round(float(x.item()), 1) for x in h2d_all]
    status = pkg.device_status()
    del t2, sets
    torch.cuda.empty_cache()
    scaling_legs = None
    if not args.no_extras:
        for n in grad_names:
            t[n].grad = None
        held = t
        del t
        torch.cuda.empty_cache()
        scaling_legs = strong_scaling(ops, dev, rank, world, dist)
        t = held
    decode = window = combine = rope = decode_step = gpu_ref = sweep = generate = compression = None
    if rank == 0 and not args.no_extras:
        gpu_ref = gpu_reference_chain(t, cu, max_q, max_k)
    if rank == 0 and not args.no_decode:
        del t, host
        torch.cuda.empty_cache()
        decode = decode_microbench(ops, dev)
        window = window_microbench(ops, dev, N)
        torch.cuda.empty_cache()
        combine = gate_combine_microbench(ops, dev, N)
        torch.cuda.empty_cache()
        decode_step = decode_step_microbench(dev)
        torch.cuda.empty_cache()
        rope = rope_microbench(ops, dev, N)
        rope["frac_of_hbm_peak"] = rope["gb_per_s"] / peaks()["hbm"]
        for v_ in combine.values():
            if isinstance(v_, dict):
                v_["frac_of_hbm_peak"] = v_["gb_per_s"] / peaks()["hbm"]
        compression = compression_bandwidth(ops, dev)
        torch.cuda.empty_cache()
    if rank == 0 and not args.no_extras:
        t = host = None
        torch.cuda.empty_cache()
        sweep = config3_sweep(ops, dev, with_reference=True)
        generate = config5_generate(dev)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    pk = peaks()
    f, f_total = flop_model(N)
    # dominant kernel and its roofline
    per_kernel = {k: dict(launches=v[0] // prof_steps, ms_per_step=v[1] / prof_steps) for k, v in prof.items()}
    dom = max(per_kernel, key=lambda k: per_kernel[k]["ms_per_step"]) if per_kernel else None
    roofline = None
    if dom:
        work = kernel_work(dom, f, "sparse_dq" not in per_kernel)
        n_launch = max(1, per_kernel[dom]["launches"])
        avg_ms = per_kernel[dom]["ms_per_step"] / n_launch
        if work:
            achieved = work[1] / 1e12 / (avg_ms / 1e3)
            traffic = NCU_DRAM_BYTES_16K.get(dom)
            roofline = dict(kernel=dom, bound=work[0], achieved=achieved, peak=pk["tc_sustained"], unit="TFLOP/s",
                            frac=achieved / pk["tc_sustained"], traffic=None if traffic is None else traffic * N / 16384,
                            traffic_unit="bytes of DRAM read+write per launch (ncu capture at 16384 tokens, scaled by tokens)",
                            launch_ms=avg_ms, peak_source=pk["source"],
                            note="peak = sustained cuBLAS bf16 figure (kernel timed inside a long step)")
        else:
            roofline = dict(kernel=dom, bound="hbm", achieved=None, peak=pk["hbm"], unit="GB/s", frac=None, traffic=None,
                            launch_ms=avg_ms, peak_source=pk["source"])
    # every attention kernel against the tensor roofline: useful flops (what the model credits) and executed flops (the
    # backward passes recompute the logits: dQ executes 3 GEMM units for 2 credited, dK/dV 4 for 3; the score pass 1 for 0)
    executed_over_useful = {"dense_dq": 1.5, "dense_dkdv": 4.0 / 3.0, "sparse_dq": 1.5,
                            "sparse_dkdv": 1.0 if "sparse_dq" not in per_kernel else 4.0 / 3.0}
    kernel_rooflines = {}
    for kname, rec in per_kernel.items():
        work = kernel_work(kname, f, "sparse_dq" not in per_kernel)
        if not work or rec["ms_per_step"] <= 0:
            continue
        base = kname[:-3] if kname.endswith("_tc") else kname
        useful = 0.0 if base == "score_topk" else work[1]
        executed = work[1] * executed_over_useful.get(base, 1.0)
        sec_k = rec["ms_per_step"] / 1e3
        kernel_rooflines[kname] = dict(ms=rec["ms_per_step"], useful_tflops=useful / 1e12 / sec_k,
                                       executed_tflops=executed / 1e12 / sec_k,
                                       executed_frac_of_peak=executed / 1e12 / sec_k / pk["tc_sustained"])
    cpu = None
    if not args.no_cpu_baseline:
        sec = cpu_chain_seconds(CPU_SAMPLE_TOKENS if N >= CPU_SAMPLE_TOKENS else N)
        cpu = cpu_baseline_record(min(N, CPU_SAMPLE_TOKENS), sec)
    useful_tflops = f_total / 1e12 / (ms / 1e3)
    line = dict(metric=METRIC, value=ms, unit="ms", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
                ms_per_step=ms, higher_is_better=False, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
                config=config_record(), clocks=clocks,
                e2e=dict(value=e2e_ms, unit="ms", h2d_bytes_per_step=h2d_bytes, d2h_bytes_per_step=4, steps=e2e_steps,
                         note="host->device copy of step s+1 overlaps the compute of step s (two input sets)",
                         copy_ms_per_step_rank0=[round(x, 2) for x in e2e_copy_ms]),
                gpu_launches=launches, roofline=roofline, cpu_baseline=cpu,
                tokens_per_s=world * N / (ms / 1e3), useful_tflops_per_gpu=useful_tflops,
                frac_of_tc_peak=useful_tflops / pk["tc_sustained"], per_kernel_ms=per_kernel, kernel_rooflines=kernel_rooflines, decode=decode, sliding_window=window, gate_combine=combine, rope=rope, decode_step=decode_step,
                hbm_peak_gb_per_s=pk["hbm"], device_status=status, h2d_gb_per_s_per_rank=h2d_gbs,
                strong_scaling=scaling_legs, gpu_reference=gpu_ref, config3_sweep=sweep, config5_generate=generate,
                compression=compression, step_timeline=timeline,
                decode_tokens_per_s_per_gpu=(generate or {}).get("decode_tokens_per_s_per_gpu"))
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
