"""Helpers shared by the operator wrappers: argument plumbing between torch tensors and the C ABI."""
import math
import weakref
from typing import List

import torch

from .. import _lib


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.DTYPE_BF16
    if t.dtype == torch.float16:
        return _lib.DTYPE_FP16
    raise AssertionError("only bfloat16 and float16 tensors are supported")


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("native_sparse_attention_triton_b200 ops run on CUDA tensors only (no CPU path)")


def inner_contiguous(t: torch.Tensor) -> torch.Tensor:
    """Kernels need a unit innermost stride, 16-byte aligned rows; copy only when that does not hold."""
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


_host_seqlens_cache = {}   # id(tensor) -> (weak reference, tensor version, list)


def host_seqlens(cu_seqlens: torch.Tensor) -> List[int]:
    """cu_seqlens -> python list.  Costs one device-to-host copy (a synchronisation) the first time a tensor object is
    seen; the result is remembered for as long as that same object lives and is not written to (its version counter),
    so a training loop that passes the same cu_seqlens tensor every step does not synchronise every step."""
    key = id(cu_seqlens)
    hit = _host_seqlens_cache.get(key)
    if hit is not None and hit[0]() is cu_seqlens and hit[1] == cu_seqlens._version:
        return hit[2]
    out = cu_seqlens.tolist()
    if len(_host_seqlens_cache) > 64:
        for k in [k for k, v in _host_seqlens_cache.items() if v[0]() is None]:
            del _host_seqlens_cache[k]
        if len(_host_seqlens_cache) > 64:
            _host_seqlens_cache.clear()
    _host_seqlens_cache[key] = (weakref.ref(cu_seqlens), cu_seqlens._version, out)
    return out


def compressed_lens(cu: List[int], kernel_size: int, kernel_stride: int) -> List[int]:
    out = []
    for i in range(len(cu) - 1):
        L = cu[i + 1] - cu[i]
        out.append(0 if L < kernel_size else (L - kernel_size) // kernel_stride + 1)
    return out


def cumsum_tensor(lens: List[int], device) -> torch.Tensor:
    cu = [0]
    for x in lens:
        cu.append(cu[-1] + x)
    return torch.tensor(cu, dtype=torch.int32, device=device)


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
