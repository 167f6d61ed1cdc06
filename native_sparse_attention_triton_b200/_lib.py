"""ctypes binding of libnsa_b200.so, the C-ABI library that holds every CUDA kernel.

The library is built in-tree by ``make -C csrc`` (see ``build``); there is no CPU fallback:
if the shared object is missing or a call fails, a RuntimeError is raised.
"""
import ctypes
import os
import subprocess
from ctypes import c_float, c_int, c_longlong, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnsa_b200.so")
_lib = None

DTYPE_BF16, DTYPE_FP16 = 0, 1

_I, _L, _F, _P = c_int, c_longlong, c_float, c_void_p

# name -> argument types (all functions return int)
_SIGNATURES = {
    "nsa_version": [],
    "nsa_last_device_status": [_P],
    "nsa_profile_enable": [_I],
    "nsa_profile_collect": [ctypes.c_char_p, _I],
    "nsa_topk_sparse_attn_fwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _F, _I, _P],
    "nsa_varlen_attn_fwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _F, _I, _P],
    "nsa_window_attn_fwd": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _F, _I, _P],
    "nsa_compressed_attn_topk": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _F,
                                 _I, _P],
    "nsa_linear_compress_fwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _L, _L, _I, _P],
    "nsa_pool_compress_fwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _L, _L, _I, _P],
    "nsa_varlen_attn_bwd": [_P] * 12 + [_L] + [_I] * 11 + [_P, _F, _I, _P],
    "nsa_window_attn_bwd": [_P] * 11 + [_L] + [_I] * 7 + [_P, _F, _I, _P],
    "nsa_topk_sparse_attn_bwd": [_P] * 13 + [_L] + [_I] * 7 + [_P, _F, _I, _P],
    "nsa_linear_compress_bwd": [_P] * 10 + [_I] * 8 + [_L, _L, _I, _P],
    "nsa_pool_compress_bwd": [_P] * 10 + [_L] + [_I] * 8 + [_L, _L, _I, _P],
    "nsa_gate_combine_fwd": [_P] * 5 + [_I, _I, _I, _P, _I, _P],
    "nsa_gate_combine_bwd": [_P] * 9 + [_I, _I, _I, _P, _I, _P],
    "nsa_rope": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _L, _L, _L, _L, _I, _P],
    "nsa_rope_decode": [_P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _L, _L, _L, _L, _I, _P],
    "nsa_rope_decode3": [_P] * 9 + [_I, _I, _I, _I, _I, _F, _P, _I, _P],
    "nsa_kv_cache_fill": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "nsa_kv_cache_stage_decode": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "nsa_kv_cache_append_decode": [_P] * 13 + [_I] * 7 + [_P, _P],
    "nsa_pool_compress_decode_pair": [_P] * 8 + [_I, _I, _I, _I, _L, _L, _L, _I, _P],
    "nsa_pool_bias": [_P, _P, _P, _I, _I, _I, _I, _P],
    "nsa_decode_num_splits": [_I, _I, _I],
    "nsa_flash_attn_decode": [_P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _P, _F, _I, _P],
    "nsa_flash_attn_decode_static": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _F, _I, _P],
    "nsa_topk_sparse_attn_decode": [_P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _I, _I, _P, _F, _I, _P],
    "nsa_compressed_attn_decode": [_P, _P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I,
                                   _I, _P, _F, _I, _P],
}


# functions that return a byte count (long long)
_SIZE_QUERIES = {
    "nsa_pool_compress_bwd_workspace_floats": [_I] * 7,
    "nsa_varlen_attn_bwd_workspace": [_I, _I, _I, _I, _I],
    "nsa_topk_sparse_attn_bwd_workspace": [_I, _I, _I, _I, _I, _I, _I],
    "nsa_launch_count": [],
    "nsa_flash_attn_decode_static_capacity": [],
    "nsa_decode_scratch_floats": [_I, _I, _I, _I],
    "nsa_compressed_decode_scratch_floats": [_I, _I, _I, _I, _I],
}


def build(verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a into libnsa_b200.so (nvcc cross-compiles without a GPU)."""
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), "-j", str(min(8, os.cpu_count() or 1))]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode:
        print(res.stdout)
    if res.returncode:
        raise RuntimeError("building libnsa_b200.so failed")
    return LIB_PATH


def lib() -> ctypes.CDLL:
    """The loaded library; raises when it has not been built (there is no fallback path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                "or `make -C native_sparse_attention_triton_b200/csrc`"
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here means header and library disagree
            fn.argtypes = argtypes
            fn.restype = c_int
        for name, argtypes in _SIZE_QUERIES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = c_longlong
        _lib = handle
    return _lib


def exported_symbols():
    return sorted(list(_SIGNATURES) + list(_SIZE_QUERIES))


_ERRORS = {-1: "invalid argument", -2: "unsupported configuration", -3: "scratch buffer too small",
           -4: "device status raised"}


def check(rc: int, name: str) -> None:
    if rc != 0:
        why = _ERRORS.get(rc, f"CUDA error {rc - 1000}" if rc >= 1000 else "unknown")
        raise RuntimeError(f"{name} failed: code {rc} ({why})")


def strides_array(*values):
    return (c_longlong * len(values))(*values)


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib().nsa_launch_count())


def profile(enable: bool) -> None:
    check(lib().nsa_profile_enable(1 if enable else 0), "nsa_profile_enable")


def profile_collect():
    """{kernel: (launches, total_ms)} for the launches recorded since the last call (synchronises)."""
    buf = ctypes.create_string_buffer(1 << 16)
    lib().nsa_profile_collect(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split()
        out[name] = (int(n), float(ms))
    return out
