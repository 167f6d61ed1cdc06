"""NSA inference step (prefill and decode) on the library's kernels, with a decode step free of host synchronisation.

``nsa_infer`` has the signature and the order of operations of the reference's
native_sparse_attention/infer/nsa_inference.py:24-152 (with its helpers infer/inference_func.py:27-202): stage tokens for
compression, compress, rotary embedding of query / compressed key / key, cache update, the three attention branches, the
gated sum.  Differences, all on the decode path: positions and lengths come from the cache's device counters instead of
the host-side ``step`` number, the staging buffers are compressed through the C interface with precomputed cu_seqlens,
the compressed cache is passed whole (lengths mask it) instead of sliced to ``.max()``, and the sliding-window length is
clamped on the device -- so one decode step is a fixed sequence of launches that ``DecodeGraph`` captures once and replays.
"""
from typing import Callable, Optional, Tuple

import torch

from . import _lib
from . import ops
from .kv_cache import NSACache
from .ops._common import dtype_code, inner_contiguous, ptr, stream_ptr


class RotaryEmbedding:
    """Callable with the reference module's call signature, ``rope(x, cu_seqlens, step=0, stride=1)``
    (native_sparse_attention/module/rope.py:197-209), on ``ops.rope``; the frequencies are the caller's."""

    def __init__(self, inv_freq: torch.Tensor, attention_scaling: float = 1.0):
        assert inv_freq.dtype == torch.float32 and inv_freq.dim() == 1
        self.inv_freq = inv_freq.contiguous()
        self.attention_scaling = float(attention_scaling)

    def __call__(self, x, cu_seqlens, step: int = 0, stride: int = 1):
        return ops.rope(x, self.inv_freq, cu_seqlens, step, stride, self.attention_scaling)

    def decode_at(self, x: torch.Tensor, lengths: torch.Tensor, stride: int = 1) -> torch.Tensor:
        """Row b of x [batch, heads, d] rotated to position lengths[b] * stride, read on the device."""
        x = inner_contiguous(x)
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        batch, num_heads, head_dim = x.shape
        assert lengths.dtype == torch.int32 and lengths.shape[0] >= batch
        torch.cuda.set_device(x.device)
        rc = _lib.lib().nsa_rope_decode(ptr(x), ptr(y), ptr(self.inv_freq), ptr(lengths), batch, num_heads, head_dim, int(stride),
                                        self.attention_scaling, 0, x.stride(0), x.stride(1), y.stride(0), y.stride(1),
                                        dtype_code(x), stream_ptr(x.device))
        _lib.check(rc, "nsa_rope_decode")
        return y

    def decode_at3(self, query, key, compress_key, lengths_qk, lengths_ck, stride_ck: int):
        """The three rotations of a decode step in one launch: query and key at lengths_qk[b], the compressed key at
        lengths_ck[b] * stride_ck."""
        xs = [inner_contiguous(t) for t in (query, key, compress_key)]
        ys = [torch.empty(t.shape, dtype=t.dtype, device=t.device) for t in xs]
        batch, num_q_heads, head_dim = xs[0].shape
        num_kv_heads = xs[1].shape[1]
        assert xs[1].shape == xs[2].shape == (batch, num_kv_heads, head_dim)
        assert lengths_qk.dtype == torch.int32 and lengths_ck.dtype == torch.int32
        strides = _lib.strides_array(*[s for x, y in zip(xs, ys) for s in (x.stride(0), x.stride(1), y.stride(0), y.stride(1))])
        torch.cuda.set_device(xs[0].device)
        rc = _lib.lib().nsa_rope_decode3(ptr(xs[0]), ptr(ys[0]), ptr(xs[1]), ptr(ys[1]), ptr(xs[2]), ptr(ys[2]), ptr(self.inv_freq),
                                         ptr(lengths_qk), ptr(lengths_ck), batch, num_q_heads, num_kv_heads, head_dim,
                                         int(stride_ck), self.attention_scaling, strides, dtype_code(xs[0]),
                                         stream_ptr(xs[0].device))
        _lib.check(rc, "nsa_rope_decode3")
        return ys


def _device_rope_of(rope):
    """A RotaryEmbedding of this module with the frequencies of a foreign rotary-embedding object (the reference's
    module/rope.py:RotaryEmbedding exposes ``inv_freq`` and ``attention_scaling``), made once and kept on that object; None
    when the object has no fixed frequencies (dynamic rope types recompute them from the sequence length).  It lets a decode
    step driven by the reference's own layer read its positions from the cache counters on the device instead of from the
    host-side step number, which is what makes the step free of host synchronisation."""
    mine = getattr(rope, "_nsa_b200_rope", None)
    if mine is not None:
        return mine
    inv_freq, scaling = getattr(rope, "inv_freq", None), getattr(rope, "attention_scaling", None)
    if not torch.is_tensor(inv_freq) or scaling is None or "dynamic" in str(getattr(rope, "rope_type", "")):
        return None
    mine = RotaryEmbedding(inv_freq.detach().float().contiguous(), float(scaling))
    try:
        object.__setattr__(rope, "_nsa_b200_rope", mine)
    except Exception:
        pass
    return mine


def _compress_staged(cache: NSACache, batch: int, which: int, func: Callable, weight, pe):
    """One compressed row per sequence from the staging buffers [batch * kernel_size, heads, d] (the reference runs its
    compress function over them with an arange cu_seqlens, infer/inference_func.py:56-87).  The library's own compress
    functions go through the C interface directly (no host copy of cu_seqlens); any other callable is called as given."""
    x = cache.before_compress_kv_cache[which, :batch].view(batch * cache.kernel_size, cache.num_kv_heads, cache.head_dim)
    cu, ycu = cache.stage_cu_seqlens[:batch + 1], cache.stage_out_cu_seqlens[:batch + 1]
    mode = {ops.linear_compress: "linear", ops.weightedpool_compress: "weighted", ops.avgpool_compress: "avg"}.get(func)
    if mode is None:
        return func(x, weight, cu, cache.kernel_size, cache.kernel_stride, pe)[0]
    y = torch.empty(batch, cache.num_kv_heads, cache.head_dim, dtype=x.dtype, device=x.device)
    bias = torch.empty(cache.num_kv_heads, cache.head_dim, dtype=x.dtype, device=x.device) if pe is not None else None
    w = weight.contiguous() if weight is not None else None
    pec = pe.contiguous() if pe is not None else None
    lib = _lib.lib()
    torch.cuda.set_device(x.device)
    if mode == "linear":
        rc = lib.nsa_linear_compress_fwd(ptr(x), ptr(w), ptr(pec), ptr(cu), ptr(ycu), ptr(y), ptr(bias), x.shape[0], batch, batch, 1,
                                         cache.num_kv_heads, cache.head_dim, cache.kernel_size, cache.kernel_stride, x.stride(0),
                                         x.stride(1), dtype_code(x), stream_ptr(x.device))
        _lib.check(rc, "nsa_linear_compress_fwd")
    else:
        rc = lib.nsa_pool_compress_fwd(ptr(x), ptr(w), ptr(pec), ptr(cu), ptr(ycu), ptr(y), ptr(bias), x.shape[0], batch, batch, 1,
                                       cache.num_kv_heads, cache.head_dim, cache.kernel_size, cache.kernel_stride, x.stride(0),
                                       x.stride(1), dtype_code(x), stream_ptr(x.device))
        _lib.check(rc, "nsa_pool_compress_fwd")
    return y


_pool_bias_cache = {}   # (id(w), id(pe)) -> (weakref w, weakref pe, versions, bias tensor)


def _pool_bias(weight, pe):
    """The position embedding folded through the pooling weights, [H, d]: it changes only when the parameters do, so it is
    computed once per (weight, pe) pair and version, not once per decode step."""
    import weakref

    key = (id(weight), id(pe))
    versions = (weight._version if weight is not None else -1, pe._version)
    hit = _pool_bias_cache.get(key)
    if hit is not None and hit[0]() is weight and hit[1]() is pe and hit[2] == versions:
        return hit[3]
    bias = torch.empty(pe.shape[0], pe.shape[2], dtype=pe.dtype, device=pe.device)
    w = weight.contiguous() if weight is not None else None
    rc = _lib.lib().nsa_pool_bias(ptr(pe.contiguous()), ptr(w), ptr(bias), pe.shape[0], pe.shape[2], pe.shape[1], dtype_code(pe),
                                  stream_ptr(pe.device))
    _lib.check(rc, "nsa_pool_bias")
    if len(_pool_bias_cache) > 256:
        _pool_bias_cache.clear()
    _pool_bias_cache[key] = (weakref.ref(weight) if weight is not None else (lambda: None), weakref.ref(pe), versions, bias)
    return bias


_POOL_FUNCS = (ops.weightedpool_compress, ops.avgpool_compress)


def _compress_staged_pair(cache: NSACache, batch: int, funcs, weights, pe):
    """Both staging buffers pooled in one launch (nsa_pool_compress_decode_pair): one compressed key row and one compressed
    value row per sequence; the key's position-embedding bias comes from the cache above."""
    stage = cache.before_compress_kv_cache
    xk, xv = stage[0, :batch], stage[1, :batch]            # [batch, kernel_size, H, d]
    wk = weights[0].contiguous() if funcs[0] is ops.weightedpool_compress else None
    wv = weights[1].contiguous() if funcs[1] is ops.weightedpool_compress else None
    bias_k = _pool_bias(wk, pe) if pe is not None else None
    yk = torch.empty(batch, cache.num_kv_heads, cache.head_dim, dtype=stage.dtype, device=stage.device)
    yv = torch.empty_like(yk)
    torch.cuda.set_device(stage.device)
    rc = _lib.lib().nsa_pool_compress_decode_pair(ptr(xk), ptr(xv), ptr(wk), ptr(wv), ptr(bias_k), None, ptr(yk), ptr(yv), batch,
                                                  cache.num_kv_heads, cache.head_dim, cache.kernel_size, xk.stride(0), xk.stride(1),
                                                  xk.stride(2), dtype_code(stage), stream_ptr(stage.device))
    _lib.check(rc, "nsa_pool_compress_decode_pair")
    return yk, yv


@torch.no_grad()
def nsa_infer(cu_seqlens: torch.Tensor, step: int, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
              gate_value: torch.Tensor, rope, cache: NSACache, compress_weight: Tuple[torch.Tensor, torch.Tensor],
              compress_func: Tuple[Callable, Callable], intra_block_pe: Optional[torch.Tensor], kernel_size: int,
              kernel_stride: int, block_size: int, topk: int, init_blocks: int, local_blocks: int,
              window_size: int) -> torch.Tensor:
    """Prefill (step == 0; query/key/value [total_len, heads, d]) or one decode step (step > 0; [batch, heads, d]).
    cu_seqlens always describes the PREFILL batch; gate_value is [rows, q_heads, 3].  Returns the gated attention output
    with the shape of query."""
    assert kernel_size == cache.kernel_size and kernel_stride == cache.kernel_stride and window_size == cache.window_size
    batch = cu_seqlens.shape[0] - 1
    if step == 0:
        cache.reset()
        cache.prepare_compress(cu_seqlens, 0, key, value)
        compress_key, compress_cu_seqlens = compress_func[0](key, compress_weight[0], cu_seqlens, kernel_size, kernel_stride,
                                                             intra_block_pe)
        compress_value, _ = compress_func[1](value, compress_weight[1], cu_seqlens, kernel_size, kernel_stride)
        query = rope(query, cu_seqlens, 0)
        compress_key = rope(compress_key, compress_cu_seqlens, 0, stride=kernel_stride)
        key = rope(key, cu_seqlens, 0)
        cache.update_kv(cu_seqlens, 0, compress_key, compress_value, key, value, key, value, compress_cu_seqlens)
        seqlens = cu_seqlens[1:] - cu_seqlens[:-1]
        compress_seqlens = compress_cu_seqlens[1:] - compress_cu_seqlens[:-1]
        max_len, max_comp = int(seqlens.max().item()), int(compress_seqlens.max().item())
        o_cmp, topk_idx = ops.compressed_attention(query, compress_key, compress_value, kernel_size, kernel_stride, block_size,
                                                   topk, cu_seqlens, compress_cu_seqlens, max_len, max_comp, None, init_blocks,
                                                   local_blocks)
        o_sel = ops.topk_sparse_attention(query, key, value, topk_idx, block_size, cu_seqlens)
        o_win = ops.sliding_window_attention(query, key, value, cu_seqlens, max_len, window_size)
        return ops.gate_combine(gate_value, o_cmp, o_sel, o_win)

    # ---- decode: nothing below reads a device value on the host ----
    cache.prepare_compress(cu_seqlens, step, key, value)
    if compress_func[0] in _POOL_FUNCS and compress_func[1] in _POOL_FUNCS:
        compress_key, compress_value = _compress_staged_pair(cache, batch, compress_func, compress_weight, intra_block_pe)
    else:
        compress_key = _compress_staged(cache, batch, 0, compress_func[0], compress_weight[0], intra_block_pe)
        compress_value = _compress_staged(cache, batch, 1, compress_func[1], compress_weight[1], None)
    fast_rope = rope if hasattr(rope, "decode_at3") else _device_rope_of(rope)
    if fast_rope is not None:
        # the new token's index is the number of tokens cached so far; the compressed token's, the compressed count
        query, key, compress_key = fast_rope.decode_at3(query, key, compress_key, cache.sparse_kv_len, cache.compress_kv_len,
                                                         kernel_stride)
    else:
        compress_cu = torch.zeros(batch + 1, dtype=torch.int32, device=key.device)
        compress_cu[1:] = torch.cumsum(cache.compress_kv_len[:batch], 0)
        query = rope(query, cu_seqlens, step)
        compress_key = rope(compress_key, compress_cu, 1, stride=kernel_stride)
        key = rope(key, cu_seqlens, step)
    cache.update_kv(cu_seqlens, step, compress_key, compress_value, key, value, key, value)
    seqlens = cache.sparse_kv_len[:batch]  # counts the new token
    # The sliding-window branch depends on neither of the other two.  While the step is being captured into a CUDA graph
    # it is put on a second stream (fork / join), so that a replay runs it beside the compressed -> selected chain: each of
    # these kernels occupies a dozen SMs.  Launched eagerly the step stays on one stream (the host is the bound there).
    main = torch.cuda.current_stream(query.device)
    fork = torch.cuda.is_current_stream_capturing()
    if fork:
        side = _side_stream(query.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            o_win = ops.flash_attention_decode(query, cache.sliding_kv_cache[0, :batch], cache.sliding_kv_cache[1, :batch],
                                               torch.clamp(cache.sliding_kv_len[:batch], max=window_size))
    o_cmp, topk_idx = ops.compressed_attention_decode(query, cache.compress_kv_cache[0, :batch], cache.compress_kv_cache[1, :batch],
                                                      seqlens, cache.compress_kv_len[:batch], kernel_size, kernel_stride,
                                                      block_size, topk, init_blocks, local_blocks, max_seqlen=cache.max_length)
    o_sel = ops.topk_sparse_attention_decode(query, cache.sparse_kv_cache[0, :batch], cache.sparse_kv_cache[1, :batch], topk_idx,
                                             block_size, seqlens)
    if fork:
        main.wait_stream(side)
    else:
        o_win = ops.flash_attention_decode(query, cache.sliding_kv_cache[0, :batch], cache.sliding_kv_cache[1, :batch],
                                           torch.clamp(cache.sliding_kv_len[:batch], max=window_size))
    return ops.gate_combine(gate_value, o_cmp, o_sel, o_win)


_side_streams = {}


def _side_stream(device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


class DecodeGraph:
    """One decode step of ``nsa_infer`` captured in a CUDA graph: ``graph(query, key, value, gate_value)`` copies the four
    inputs into fixed buffers, replays the launches and returns the (fixed) output tensor.  Capture after prefill; the
    cache object, weights and shapes are fixed at capture."""

    def __init__(self, cu_seqlens, query, key, value, gate_value, **nsa_args):
        self.inputs = [t.clone() for t in (query, key, value, gate_value)]
        self.args = dict(nsa_args)
        self.cu_seqlens = cu_seqlens
        cache: NSACache = nsa_args["cache"]
        # The warm-up step below (which also performs every lazy one-time initialisation of the library outside the capture)
        # and the capture itself both advance the cache: snapshot its state and restore it afterwards.
        state = [t.clone() for t in self._state(cache)]
        side = torch.cuda.Stream(device=query.device)
        side.wait_stream(torch.cuda.current_stream(query.device))
        with torch.cuda.stream(side):
            nsa_infer(cu_seqlens, 1, *self.inputs, **self.args)
        torch.cuda.current_stream(query.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=side):   # the warm-up stream: its decode scratch is reused by the capture
            self.output = nsa_infer(cu_seqlens, 1, *self.inputs, **self.args)
        for dst, src in zip(self._state(cache), state):
            dst.copy_(src)

    @staticmethod
    def _state(cache):
        # what a step overwrites: the counters, the staging buffers (shifted) and the ring (a live slot once it is full);
        # rows appended to the two large caches lie beyond the restored counters and are rewritten by the next real step
        return (cache.sparse_kv_len, cache.compress_kv_len, cache.before_compress_kv_cache, cache.before_compress_kv_len,
                cache.sliding_kv_cache, cache.sliding_kv_len)

    def __call__(self, query, key, value, gate_value):
        srcs = [query, key, value, gate_value]
        if all(s.dtype == d.dtype and s.device == d.device and s.shape == d.shape for s, d in zip(srcs, self.inputs)):
            torch._foreach_copy_(self.inputs, srcs)   # one launch for the four inputs
        else:
            for dst, src in zip(self.inputs, srcs):
                dst.copy_(src)
        self.graph.replay()
        return self.output
