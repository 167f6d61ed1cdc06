"""Drop-in installation: make the reference project's own modules bind to these operators.

The reference's callers import the operators by name at import time:
  native_sparse_attention/module/native_sparse_attention.py:16-22 (and the dict COMPRESS_TYPE_TO_FUNC, :28-32)
  native_sparse_attention/infer/inference_func.py:17-24
  native_sparse_attention/module/self_attention.py:19
  native_sparse_attention/module/kv_cache.py:18 (get_compressed_seqlens from ops.triton.utils)

`install()` registers this package's operator namespace in ``sys.modules`` under the names
``native_sparse_attention.ops``, ``native_sparse_attention.ops.triton`` and
``native_sparse_attention.ops.triton.utils`` so that a later ``import native_sparse_attention.module`` binds to
the CUDA kernels of libnsa_b200.so and the reference's Triton sources are never imported.  When the reference
has already been imported, the binding sites listed above are rewritten in place as well.
"""
import sys
import types

from . import ops as _ops

_OP_NAMES = [
    "avgpool_compress", "weightedpool_compress", "linear_compress", "flash_attention_varlen", "compressed_attention",
    "topk_sparse_attention", "flash_attention_decode", "compressed_attention_decode", "topk_sparse_attention_decode",
]
_PKG = "native_sparse_attention"


def _module(name, is_pkg, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    if is_pkg:
        m.__path__ = []  # a package without files: submodules must be pre-registered
    m.__nsa_b200_shim__ = True
    return m


def install(patch_loaded: bool = True):
    """Route ``native_sparse_attention.ops`` (and ``.ops.triton.utils``) to this package.  Returns the ops module."""
    fns = {n: getattr(_ops, n) for n in _OP_NAMES}
    ops_mod = _module(f"{_PKG}.ops", True, __all__=list(_OP_NAMES), **fns)
    triton_mod = _module(f"{_PKG}.ops.triton", True)
    utils_mod = _module(f"{_PKG}.ops.triton.utils", False, get_compressed_seqlens=_ops.get_compressed_seqlens,
                        is_hopper_gpu=lambda: False)
    ops_mod.triton = triton_mod
    triton_mod.utils = utils_mod
    sys.modules[f"{_PKG}.ops"] = ops_mod
    sys.modules[f"{_PKG}.ops.triton"] = triton_mod
    sys.modules[f"{_PKG}.ops.triton.utils"] = utils_mod
    parent = sys.modules.get(_PKG)
    if parent is not None:
        parent.ops = ops_mod
    if patch_loaded:
        _patch_loaded_modules(fns)
    return ops_mod


def _patch_loaded_modules(fns):
    """Rewrite names that already-imported reference modules captured."""
    for name, mod in list(sys.modules.items()):
        if mod is None or not name.startswith(_PKG + ".") or name.startswith(_PKG + ".ops"):
            continue
        for fn_name, fn in fns.items():
            if hasattr(mod, fn_name):
                setattr(mod, fn_name, fn)
        if hasattr(mod, "get_compressed_seqlens"):
            mod.get_compressed_seqlens = _ops.get_compressed_seqlens
        table = getattr(mod, "COMPRESS_TYPE_TO_FUNC", None)
        if isinstance(table, dict):
            for key, fn_name in (("avgpool", "avgpool_compress"), ("weightedpool", "weightedpool_compress"),
                                 ("linear", "linear_compress")):
                if key in table:
                    table[key] = fns[fn_name]


def window_attention_adapter(fallback):
    """A function with flash_attn.flash_attn_varlen_func's calling convention that runs the sliding-window branch of the
    NSA layer (causal self-attention, ``window_size=(W, -1)``, head_dim 128, no other option) on this package's kernels
    and passes every other call on to ``fallback`` (the function it replaces)."""
    def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, *args, causal=False,
                               window_size=(-1, -1), **kwargs):
        ours = (not args and not kwargs and causal and window_size[0] >= 0 and window_size[1] in (-1, 0)
                and cu_seqlens_q is cu_seqlens_k and q.shape[-1] == 128 and q.shape[0] == k.shape[0])
        if ours:
            return _ops.sliding_window_attention(q, k, v, cu_seqlens_q.to(_int32()), max_seqlen_q, window_size[0])
        if fallback is None:
            raise NotImplementedError("only the sliding-window call of the NSA layer is implemented")
        return fallback(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, *args, causal=causal,
                        window_size=window_size, **kwargs)
    return flash_attn_varlen_func


def _int32():
    import torch
    return torch.int32


def install_sliding_window():
    """Opt-in: also route the NSA layer's sliding-window branch, which the reference sends to the third-party flash_attn
    package (native_sparse_attention/module/native_sparse_attention.py:15,213-223), to this package.  Only the layer
    module is touched, and only its call with ``causal=True, window_size=(W, -1)`` is taken over.  Call after the
    reference's module package has been imported.  Returns the number of modules patched."""
    patched = 0
    for name, mod in list(sys.modules.items()):
        if mod is None or not name.startswith(_PKG + ".module"):
            continue
        fn = getattr(mod, "flash_attn_varlen_func", None)
        if fn is not None and hasattr(mod, "topk_sparse_attention") and not getattr(fn, "__nsa_b200_shim__", False):
            adapter = window_attention_adapter(fn)
            adapter.__nsa_b200_shim__ = True
            mod.flash_attn_varlen_func = adapter
            patched += 1
    return patched


def install_inference():
    """Opt-in: bind the reference's names ``nsa_infer`` and ``NSACache`` (native_sparse_attention/infer/nsa_inference.py:24,
    module/kv_cache.py:128), wherever its already-imported modules hold them, to this package's device-side cache and
    host-sync-free decode step.  A cache must then be constructed after this call (the two implementations do not share
    objects).  Returns the number of bindings replaced."""
    from .infer import nsa_infer
    from .kv_cache import NSACache
    mine = {"nsa_infer": nsa_infer, "NSACache": NSACache}
    patched = 0
    for name, mod in list(sys.modules.items()):
        if mod is None or not (name == _PKG or name.startswith(_PKG + ".")):
            continue
        for attr, obj in mine.items():
            cur = getattr(mod, attr, None)
            if cur is not None and cur is not obj and not isinstance(cur, type(sys)):
                setattr(mod, attr, obj)
                patched += 1
    return patched


def installed() -> bool:
    return getattr(sys.modules.get(f"{_PKG}.ops"), "__nsa_b200_shim__", False)
