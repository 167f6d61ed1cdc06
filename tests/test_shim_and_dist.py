"""Host-side logic that needs no GPU: the drop-in shim and the multi-GPU sharding helpers (gloo, world size 2)."""
import os
import sys
import textwrap

import pytest
import torch
import torch.multiprocessing as mp

from native_sparse_attention_triton_b200 import dist as nsa_dist


def test_shim_routes_reference_imports(tmp_path, monkeypatch):
    # a stand-in for the reference package: its own ops module must never be imported
    pkg = tmp_path / "native_sparse_attention"
    (pkg / "ops").mkdir(parents=True)
    (pkg / "module").mkdir()
    (pkg / "__init__.py").write_text("")
    (pkg / "ops" / "__init__.py").write_text("raise ImportError('the Triton operators must not be imported')")
    (pkg / "module" / "__init__.py").write_text(textwrap.dedent("""
        from native_sparse_attention.ops import linear_compress, compressed_attention, topk_sparse_attention
        from native_sparse_attention.ops import flash_attention_decode, avgpool_compress, weightedpool_compress
        from native_sparse_attention.ops.triton.utils import get_compressed_seqlens
        COMPRESS_TYPE_TO_FUNC = {"avgpool": avgpool_compress, "weightedpool": weightedpool_compress, "linear": linear_compress}
        def flash_attn_varlen_func(*args, **kwargs):   # stands in for the third-party function the layer imports
            return ("third party", args, kwargs)
        def nsa_infer(*args, **kwargs):
            return "reference nsa_infer"
        class NSACache:
            pass
    """))
    monkeypatch.syspath_prepend(str(tmp_path))
    for name in [n for n in sys.modules if n.startswith("native_sparse_attention")]:
        if not name.startswith("native_sparse_attention_triton_b200"):
            monkeypatch.delitem(sys.modules, name)
    from native_sparse_attention_triton_b200 import ops, shim

    shim.install()
    assert shim.installed()
    import native_sparse_attention.module as ref_module

    assert ref_module.linear_compress is ops.linear_compress
    assert ref_module.compressed_attention is ops.compressed_attention
    assert ref_module.get_compressed_seqlens is ops.get_compressed_seqlens
    assert ref_module.COMPRESS_TYPE_TO_FUNC["linear"] is ops.linear_compress
    # patch-after-import path
    ref_module.linear_compress = None
    ref_module.COMPRESS_TYPE_TO_FUNC["linear"] = None
    shim.install(patch_loaded=True)
    assert ref_module.linear_compress is ops.linear_compress
    assert ref_module.COMPRESS_TYPE_TO_FUNC["linear"] is ops.linear_compress
    # opt-in routing of the sliding-window branch: only the layer's own kind of call is taken over
    assert shim.install_sliding_window() == 1 and shim.install_sliding_window() == 0
    x = torch.zeros(4, 2, 64)   # head_dim 64: not ours -> passed on to the function that was there before
    cu = torch.tensor([0, 4], dtype=torch.int32)
    out = ref_module.flash_attn_varlen_func(x, x, x, cu, cu, 4, 4, causal=True, window_size=(2, -1))
    assert out[0] == "third party" and out[2] == {"causal": True, "window_size": (2, -1)}
    with pytest.raises(RuntimeError, match="no CPU path"):   # head_dim 128, causal, windowed: ours (and ours needs CUDA tensors)
        y = torch.zeros(4, 2, 128, dtype=torch.bfloat16)
        ref_module.flash_attn_varlen_func(y, y, y, cu, cu, 4, 4, causal=True, window_size=(2, -1))
    # opt-in routing of the inference step and its cache
    from native_sparse_attention_triton_b200.infer import nsa_infer
    from native_sparse_attention_triton_b200.kv_cache import NSACache
    assert shim.install_inference() == 2 and shim.install_inference() == 0
    assert ref_module.nsa_infer is nsa_infer and ref_module.NSACache is NSACache
    for name in [n for n in sys.modules if n.startswith("native_sparse_attention.") or n == "native_sparse_attention"]:
        monkeypatch.delitem(sys.modules, name)


def test_ops_refuse_cpu_tensors():
    from native_sparse_attention_triton_b200 import ops

    x = torch.zeros(64, 2, 64, dtype=torch.bfloat16)
    cu = torch.tensor([0, 64], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.avgpool_compress(x, None, cu, 32, 16)
    with pytest.raises(AssertionError):
        ops.avgpool_compress(x.float(), None, cu, 32, 16)  # dtype assert, like the reference


def test_get_compressed_seqlens_matches_oracle():
    from native_sparse_attention_triton_b200.ops import get_compressed_seqlens
    from oracle import nsa_oracle as O

    cu = torch.tensor([0, 12, 44, 1044, 1075], dtype=torch.int32)
    y, y_cu = get_compressed_seqlens(cu, 32, 16)
    y_ref, y_cu_ref = O.compressed_seqlens(cu, 32, 16)
    assert y.tolist() == y_ref.tolist() == [0, 1, 61, 0]
    assert y_cu.tolist() == y_cu_ref.tolist()
    assert y.dtype == torch.int32 and y_cu.dtype == torch.int32


def test_partition_is_balanced_and_complete():
    seqlens = [32768] * 8
    parts = nsa_dist.partition_sequences(seqlens, 4)
    assert sorted(i for p in parts for i in p) == list(range(8)) and all(len(p) == 2 for p in parts)
    seqlens = [1024, 7168, 8192, 300, 5000]
    parts = nsa_dist.partition_sequences(seqlens, 2)
    assert sorted(i for p in parts for i in p) == list(range(5))
    cost = [sum(nsa_dist.sequence_cost(seqlens[i]) for i in p) for p in parts]
    assert max(cost) / sum(cost) < 0.6
    assert nsa_dist.kv_head_range(1, 2, 4) == (2, 4)
    with pytest.raises(ValueError):
        nsa_dist.kv_head_range(0, 3, 4)


def _worker(rank, world, port, seqlens, q, ck, cv, cu, cu_k, expected, ret):
    import torch.distributed as dist
    from oracle import nsa_oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        parts = nsa_dist.partition_sequences(seqlens, world)
        q_l, cu_l = nsa_dist.shard_varlen(q, cu, parts[rank])
        ck_l, cu_k_l = nsa_dist.shard_varlen(ck, cu_k, parts[rank])
        cv_l, _ = nsa_dist.shard_varlen(cv, cu_k, parts[rank])
        # the per-rank operator call (the CPU oracle stands in for the CUDA operator in this host-logic test)
        o_l, _ = O.compressed_attention(q_l, ck_l, cv_l, 32, 16, 64, 0, cu_l, cu_k_l)
        o = nsa_dist.gather_varlen(o_l, parts, cu)
        ok = torch.allclose(o, expected, atol=1e-6)
        # head sharding of one tensor
        b, e = nsa_dist.kv_head_range(rank, world, q.shape[1])
        full = nsa_dist.gather_heads(q[:, b:e])
        ok = ok and torch.equal(full, q)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sequence_sharding_round_trip_gloo_world2():
    from oracle import nsa_oracle as O

    g = torch.Generator().manual_seed(0)
    seqlens = [100, 40, 260, 33]
    N = sum(seqlens)
    cu = torch.tensor([0, 100, 140, 400, 433], dtype=torch.int32)
    q = torch.randn(N, 4, 32, generator=g)
    k = torch.randn(N, 2, 32, generator=g)
    ck, cu_k = O.avgpool_compress(k, None, cu, 32, 16)
    cv = ck * 0.5
    expected, _ = O.compressed_attention(q, ck, cv, 32, 16, 64, 0, cu, cu_k)
    port = 29500 + os.getpid() % 2000
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, seqlens, q, ck, cv, cu, cu_k, expected, ret), nprocs=2, join=True)
    assert ret[0] and ret[1]
