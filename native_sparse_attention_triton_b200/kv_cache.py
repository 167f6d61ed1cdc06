"""KV cache of NSA inference with device-side bookkeeping.

Same constructor, attributes and methods as the reference's ``NSACache``
(native_sparse_attention/module/kv_cache.py:128-449): four ``[2, max_batch, rows, kv_heads, head_dim]`` tensors (keys and
values of the selected-block branch, of the compressed branch, the staging buffer of tokens not yet compressed, the
sliding-window ring) with one int32 row counter each.  The reference fills them with a Triton kernel sized by
``.max().item()`` and updates them, per decode step, with ``torch.where`` and advanced-index assignments; here prefill is
one copy kernel per cache and a decode step is two launches, all reading the counters on the device, so nothing
synchronises with the host and a decode step can be replayed from a CUDA graph.
"""
from typing import Union

import torch

from . import _lib
from .ops._common import inner_contiguous, ptr, require_cuda, stream_ptr


class NSACache:
    def __init__(self, max_batch_size: int, max_length: int, num_kv_heads: int, head_dim: int, kernel_size: int,
                 kernel_stride: int, window_size: int, dtype: torch.dtype, device: Union[str, torch.device] = "cuda"):
        assert dtype in (torch.bfloat16, torch.float16)
        assert kernel_size % kernel_stride == 0 and head_dim % 8 == 0
        self.max_batch_size = max_batch_size
        self.max_length = max_length
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.kernel_size = kernel_size
        self.kernel_stride = kernel_stride
        self.window_size = window_size
        self.dtype = dtype
        self.device = torch.device(device)
        self.max_comp_length = (max_length - kernel_size) // kernel_stride + 1

        def alloc(rows):
            cache = torch.zeros(2, max_batch_size, rows, num_kv_heads, head_dim, dtype=dtype, device=self.device)
            return cache, torch.zeros(max_batch_size, dtype=torch.int32, device=self.device)

        self.sparse_kv_cache, self.sparse_kv_len = alloc(max_length)
        self.compress_kv_cache, self.compress_kv_len = alloc(self.max_comp_length)
        self.before_compress_kv_cache, self.before_compress_kv_len = alloc(kernel_size)
        self.sliding_kv_cache, self.sliding_kv_len = alloc(window_size)
        self.device = self.sparse_kv_cache.device  # with its index
        # cu_seqlens of the staging buffers seen as a varlen batch (every sequence kernel_size rows, one compressed row)
        self.stage_cu_seqlens = torch.arange(max_batch_size + 1, dtype=torch.int32, device=self.device) * kernel_size
        self.stage_out_cu_seqlens = torch.arange(max_batch_size + 1, dtype=torch.int32, device=self.device)

    def reset(self):
        for t in (self.compress_kv_cache, self.compress_kv_len, self.before_compress_kv_cache, self.before_compress_kv_len,
                  self.sparse_kv_cache, self.sparse_kv_len, self.sliding_kv_cache, self.sliding_kv_len):
            t.zero_()

    # ------------------------------------------------------------------ helpers
    def _fill(self, cache, length, key, value, cu_seqlens, mode, window, hop):
        require_cuda(key, value, cu_seqlens)
        assert key.shape == value.shape and key.dtype == self.dtype and value.dtype == self.dtype
        assert key.shape[1:] == (self.num_kv_heads, self.head_dim)
        assert cu_seqlens.dtype == torch.int32
        batch = cu_seqlens.shape[0] - 1
        assert batch <= self.max_batch_size
        key, value = inner_contiguous(key), inner_contiguous(value)
        strides = _lib.strides_array(cache.stride(0), cache.stride(1), cache.stride(2), cache.stride(3), key.stride(0),
                                     key.stride(1), value.stride(0), value.stride(1))
        torch.cuda.set_device(cache.device)
        rc = _lib.lib().nsa_kv_cache_fill(ptr(cache), ptr(length), ptr(key), ptr(value), ptr(cu_seqlens), mode, window, hop,
                                          key.shape[0], batch, cache.shape[2], self.num_kv_heads, self.head_dim, strides,
                                          stream_ptr(cache.device))
        _lib.check(rc, "nsa_kv_cache_fill")

    # ------------------------------------------------------------------ the reference's interface
    def prepare_compress(self, cu_seqlens: torch.Tensor, step: int, key: torch.Tensor, value: torch.Tensor):
        """Stage the tokens the next compressed token will need (before rotary embedding).  Prefill: the tail of every
        sequence after its last full compression hop; decode: shift full buffers by kernel_stride and append the new row."""
        if step == 0:
            self._fill(self.before_compress_kv_cache, self.before_compress_kv_len, key, value, cu_seqlens, 2, self.kernel_size,
                       self.kernel_stride)
            return
        require_cuda(key, value)
        batch, num_heads, head_dim = key.shape
        assert key.shape == value.shape and num_heads == self.num_kv_heads and head_dim == self.head_dim
        assert batch == cu_seqlens.shape[0] - 1 and batch <= self.max_batch_size
        key, value = inner_contiguous(key), inner_contiguous(value)
        c = self.before_compress_kv_cache
        strides = _lib.strides_array(c.stride(0), c.stride(1), c.stride(2), c.stride(3), key.stride(0), key.stride(1),
                                     value.stride(0), value.stride(1))
        torch.cuda.set_device(c.device)
        rc = _lib.lib().nsa_kv_cache_stage_decode(ptr(c), ptr(self.before_compress_kv_len), ptr(key), ptr(value), batch,
                                                  self.kernel_size, self.kernel_stride, num_heads, head_dim, strides,
                                                  stream_ptr(c.device))
        _lib.check(rc, "nsa_kv_cache_stage_decode")

    def update_kv(self, cu_seqlens: torch.Tensor, step: int, compress_key: torch.Tensor, compress_value: torch.Tensor,
                  sparse_key: torch.Tensor, sparse_value: torch.Tensor, sliding_key: torch.Tensor, sliding_value: torch.Tensor,
                  compress_cu_seqlens: torch.Tensor = None):
        """Prefill: fill the three caches from the varlen tensors (compress_cu_seqlens = the compressed tokens' cu_seqlens;
        derived from cu_seqlens when not given).  Decode: append one row per sequence to each cache; the compressed row is
        kept only for sequences whose staging buffer is full."""
        if step == 0:
            if compress_cu_seqlens is None:
                from .ops.utils import get_compressed_seqlens
                _, compress_cu_seqlens = get_compressed_seqlens(cu_seqlens, self.kernel_size, self.kernel_stride)
            self._fill(self.compress_kv_cache, self.compress_kv_len, compress_key, compress_value, compress_cu_seqlens, 0, 0, 0)
            self._fill(self.sparse_kv_cache, self.sparse_kv_len, sparse_key, sparse_value, cu_seqlens, 0, 0, 0)
            self._fill(self.sliding_kv_cache, self.sliding_kv_len, sliding_key, sliding_value, cu_seqlens, 1, self.window_size, 0)
            return
        tensors = [compress_key, compress_value, sparse_key, sparse_value, sliding_key, sliding_value]
        require_cuda(*tensors)
        batch = sparse_key.shape[0]
        for t in tensors:
            assert t.shape == (batch, self.num_kv_heads, self.head_dim) and t.dtype == self.dtype
        assert batch == cu_seqlens.shape[0] - 1 and batch <= self.max_batch_size
        tensors = [inner_contiguous(t) for t in tensors]
        caches = (self.compress_kv_cache, self.sparse_kv_cache, self.sliding_kv_cache)
        flat = [s for c in caches for s in c.stride()[:4]] + [s for t in tensors for s in t.stride()[:2]]
        torch.cuda.set_device(self.device)
        rc = _lib.lib().nsa_kv_cache_append_decode(
            ptr(self.compress_kv_cache), ptr(self.compress_kv_len), ptr(self.sparse_kv_cache), ptr(self.sparse_kv_len),
            ptr(self.sliding_kv_cache), ptr(self.sliding_kv_len), ptr(self.before_compress_kv_len), *[ptr(t) for t in tensors],
            batch, self.kernel_size, self.max_comp_length, self.max_length, self.window_size, self.num_kv_heads, self.head_dim,
            _lib.strides_array(*flat), stream_ptr(self.device))
        _lib.check(rc, "nsa_kv_cache_append_decode")
