"""Single-token (decode) operators against dense KV caches.

Signatures follow the reference:
  flash_attention_decode        native_sparse_attention/ops/triton/flash_attention_decode.py:142-217
  compressed_attention_decode   native_sparse_attention/ops/torch/compressed_attention_decode.py:65-153
  topk_sparse_attention_decode  native_sparse_attention/ops/triton/topk_sparse_attention_decode.py:151-237
Cache tensors may be strided views ([batch, len, kv_heads, d] slices of a larger cache).
"""
from typing import Optional, Tuple

import torch

from .. import _lib
from ._common import default_scale, dtype_code, inner_contiguous, ptr, require_cuda, stream_ptr


def _decode_strides(q, k, v, o, topk_idx=None):
    t = topk_idx.stride() if topk_idx is not None else (0, 0, 0)
    return _lib.strides_array(q.stride(0), q.stride(1), k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1),
                              v.stride(2), o.stride(0), o.stride(1), *t)


_scratch_cache = {}   # (device index, stream handle) -> float32 tensor whose control words are zero between calls


def _scratch(batch, num_kv_heads, head_dim, max_tiles, device, compressed_cache_len=None):
    """(splits, scratch tensor or None, its size in floats) for one decode call: the split count the library asks for and
    the scratch that count needs (control words, partial results, and the logits of the compressed operator).

    The kernels leave the control words at zero when they finish, so a buffer zeroed once serves every later call that is
    ordered after it: one buffer is kept per (device, stream) -- calls on one stream cannot overlap -- and regrown (and
    zeroed again) when a call needs more.  A CUDA-graph capture uses the buffer of its capture stream when a warm-up call on
    that stream has made one (DecodeGraph does), else a fresh zeroed buffer from the graph's pool."""
    lib = _lib.lib()
    splits = lib.nsa_decode_num_splits(batch, num_kv_heads, max_tiles)
    if compressed_cache_len is None:
        n = lib.nsa_decode_scratch_floats(batch, num_kv_heads, head_dim, splits)
    else:
        n = lib.nsa_compressed_decode_scratch_floats(batch, num_kv_heads, head_dim, splits, compressed_cache_len)
    if n <= 0:
        return splits, None, 0
    ctrl = (batch * num_kv_heads + 1 + 63) // 64 * 64

    def fresh(size):
        buf = torch.empty(size, dtype=torch.float32, device=device)
        buf[:ctrl].zero_()
        return buf

    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_ptr(device))
    buf = _scratch_cache.get(key)
    if torch.cuda.is_current_stream_capturing() and (buf is None or buf.numel() < n or buf._nsa_ctrl < ctrl):
        return splits, fresh(n), n   # from the graph's own pool, zeroed by a captured kernel at every replay
    if buf is None or buf.numel() < n:
        buf = fresh(max(n, 0 if buf is None else buf.numel()))
        _scratch_cache[key] = buf
    elif buf._nsa_ctrl < ctrl:
        # the control region grows with batch * kv_heads; beyond the previous call's region lie that call's partial results
        buf[:ctrl].zero_()
    buf._nsa_ctrl = ctrl
    return splits, buf, n


def _drop_scratch(device):
    """Forget the stream's scratch after a failed call: its control words may not have returned to zero."""
    _scratch_cache.pop((device.index if device.index is not None else torch.cuda.current_device(), stream_ptr(device)), None)


def _check_decode(q, k, v, seqlens):
    require_cuda(q, k, v, seqlens)
    assert q.dtype == torch.bfloat16 or q.dtype == torch.float16
    assert k.dtype == q.dtype and v.dtype == q.dtype
    assert seqlens.dtype == torch.int32
    batch_size, num_q_heads, head_dim = q.shape
    assert k.shape[1] == v.shape[1] and batch_size == seqlens.shape[0]
    assert k.shape[2] == v.shape[2] and num_q_heads % k.shape[2] == 0


def flash_attention_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seqlens: torch.Tensor,
                           sm_scale: Optional[float] = None) -> torch.Tensor:
    """One query token per sequence attends to the first seqlens[b] rows of its cache.

    q [batch, num_q_heads, d]; k, v [batch, cache_len, num_kv_heads, d]; seqlens int32 [batch].
    """
    _check_decode(q, k, v, seqlens)
    q, k, v = inner_contiguous(q), inner_contiguous(k), inner_contiguous(v)
    batch, num_q_heads, head_dim = q.shape
    cache_len, num_kv_heads = k.shape[1], k.shape[2]
    if sm_scale is None:
        sm_scale = default_scale(head_dim)
    if cache_len == 0:
        return torch.zeros_like(q)
    o = torch.empty_like(q)   # every row is written: a sequence without visible rows gets zeros from the kernel
    splits, scratch, n = _scratch(batch, num_kv_heads, head_dim, (cache_len + 63) // 64, q.device)
    torch.cuda.set_device(q.device)
    rc = _lib.lib().nsa_flash_attn_decode(ptr(q), ptr(k), ptr(v), ptr(seqlens), ptr(o), ptr(scratch), n, splits, batch,
                                          cache_len, num_q_heads, num_kv_heads, head_dim, _decode_strides(q, k, v, o),
                                          float(sm_scale), dtype_code(q), stream_ptr(q.device))
    if rc:
        _drop_scratch(q.device)
    _lib.check(rc, "nsa_flash_attn_decode")
    return o


def topk_sparse_attention_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, topk_idx: torch.Tensor,
                                 block_size: int, seqlens: torch.Tensor, sm_scale: Optional[float] = None) -> torch.Tensor:
    """One query token per sequence attends to the rows of its selected blocks below seqlens[b].

    topk_idx int32 [num_kv_heads, batch, topk], -1 padding.
    """
    _check_decode(q, k, v, seqlens)
    assert k.shape[2] == topk_idx.shape[0] and q.shape[0] == topk_idx.shape[1]
    q, k, v = inner_contiguous(q), inner_contiguous(k), inner_contiguous(v)
    if topk_idx.dtype != torch.int32:
        topk_idx = topk_idx.to(torch.int32)
    batch, num_q_heads, head_dim = q.shape
    cache_len, num_kv_heads = k.shape[1], k.shape[2]
    topk = topk_idx.shape[-1]
    if sm_scale is None:
        sm_scale = default_scale(head_dim)
    if cache_len == 0:
        return torch.zeros_like(q)
    o = torch.empty_like(q)   # every row is written: a sequence without visible rows gets zeros from the kernel
    splits, scratch, n = _scratch(batch, num_kv_heads, head_dim, topk * max(1, block_size // 64), q.device)
    torch.cuda.set_device(q.device)
    rc = _lib.lib().nsa_topk_sparse_attn_decode(ptr(q), ptr(k), ptr(v), ptr(topk_idx), ptr(seqlens), ptr(o),
                                                ptr(scratch), n, splits, batch, cache_len, num_q_heads, num_kv_heads,
                                                head_dim, topk, int(block_size), _decode_strides(q, k, v, o, topk_idx),
                                                float(sm_scale), dtype_code(q), stream_ptr(q.device))
    if rc:
        _drop_scratch(q.device)
    _lib.check(rc, "nsa_topk_sparse_attn_decode")
    return o


def compressed_attention_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seqlens: torch.Tensor,
                                compress_seqlens: torch.Tensor, kernel_size: int, kernel_stride: int, block_size: int,
                                topk: int, init_blocks: int = 1, local_blocks: int = 2,
                                sm_scale: Optional[float] = None, max_seqlen: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Single-token attention over the compressed cache and block selection for the current token.

    seqlens counts the current token; compress_seqlens is the number of valid compressed rows.
    Returns (o [batch, num_q_heads, d], topk_idx int32 [num_kv_heads, batch, min(topk, num_blocks)]).
    num_blocks = ceil(max(seqlens) / block_size) as in the reference, which costs a device-to-host copy; a caller that must
    not synchronise passes max_seqlen (an upper bound, e.g. the cache capacity): the width of topk_idx then follows the
    bound and the entries beyond a sequence's blocks are -1.
    """
    assert block_size % kernel_size == 0 and kernel_size % kernel_stride == 0
    require_cuda(q, k, v, seqlens, compress_seqlens)
    batch, num_q_heads, head_dim = q.shape
    cache_len, num_kv_heads = k.shape[1], k.shape[2]
    if cache_len == 0:  # input is too short to have a compressed block
        return torch.zeros_like(q), torch.zeros(num_kv_heads, batch, 1, device=q.device, dtype=torch.int32)
    q, k, v = inner_contiguous(q), inner_contiguous(k), inner_contiguous(v)
    seqlens = seqlens.to(torch.int32)
    compress_seqlens = compress_seqlens.to(torch.int32)
    if sm_scale is None:
        sm_scale = default_scale(head_dim)
    if max_seqlen is None:
        max_seqlen = int(seqlens.max().item())
    max_blocks = (max_seqlen + block_size - 1) // block_size
    t_out = min(topk, max_blocks)
    o = torch.empty_like(q)
    topk_idx = torch.empty(num_kv_heads, batch, t_out, dtype=torch.int32, device=q.device)
    splits, scratch, n = _scratch(batch, num_kv_heads, head_dim, (cache_len + 63) // 64, q.device, cache_len)
    torch.cuda.set_device(q.device)
    rc = _lib.lib().nsa_compressed_attn_decode(ptr(q), ptr(k), ptr(v), ptr(seqlens), ptr(compress_seqlens), ptr(o),
                                               ptr(topk_idx), ptr(scratch), n, splits, batch, cache_len, max_seqlen,
                                               num_q_heads, num_kv_heads, head_dim, kernel_size, kernel_stride, block_size,
                                               topk, init_blocks, local_blocks, _decode_strides(q, k, v, o, topk_idx),
                                               float(sm_scale), dtype_code(q), stream_ptr(q.device))
    if rc:
        _drop_scratch(q.device)
    _lib.check(rc, "nsa_compressed_attn_decode")
    return o, topk_idx
