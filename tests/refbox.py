"""Loader of the UNMODIFIED reference project for tests that run beside it on one GPU.

The reference (XunhaoLai/native-sparse-attention-triton) is installed by ``baseline/install_reference.sh`` into the
git-ignored directory ``baseline/_ref``; where that directory is absent the tests that need it are skipped.  Nothing of
the product imports this module.

Two environment differences from the versions the reference pins are bridged here, outside the operators and without
touching reference arithmetic:
  * transformers 5.x computes rotary frequencies from ``config.rope_parameters`` after calling
    ``config.standardize_rope_params()``; the reference's ``RopeConfig`` dataclass (module/rope.py:27-47) has neither, so
    both are added to the class (``rope_parameters`` = its ``rope_scaling`` dict plus ``rope_theta``).
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
_PKG = "native_sparse_attention"


def available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, _PKG, "__init__.py"))


def _purge():
    for name in [n for n in sys.modules if n == _PKG or n.startswith(_PKG + ".")]:
        del sys.modules[name]


def _rope_config_compat(rope_mod):
    cfg = rope_mod.RopeConfig
    if not hasattr(cfg, "standardize_rope_params"):
        cfg.standardize_rope_params = lambda self: None
        cfg.rope_parameters = property(lambda self: dict(self.rope_scaling or {}, rope_theta=self.rope_theta))


def load(layers: bool = False):
    """Import the reference with its own Triton operators bound (any earlier shim of this repository is removed first).
    Returns the ``native_sparse_attention`` package; with ``layers`` its ``module``, ``infer`` and ``model`` subpackages
    are imported too (they need a GPU and flash_attn at import time)."""
    if not available():
        pytest.skip("baseline/_ref is absent: run `sh baseline/install_reference.sh <reference checkout>`")
    ops_mod = sys.modules.get(_PKG + ".ops")
    if ops_mod is not None and getattr(ops_mod, "__nsa_b200_shim__", False):
        _purge()
    pkg = sys.modules.get(_PKG)
    if pkg is not None and not os.path.abspath(getattr(pkg, "__file__", "") or "").startswith(REF_DIR):
        _purge()
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import native_sparse_attention as ref
    import native_sparse_attention.ops  # noqa: F401  (the Triton operators)
    import native_sparse_attention.ops.triton.compressed_attention  # noqa: F401
    assert os.path.abspath(ref.__file__).startswith(REF_DIR), ref.__file__
    if layers:
        import native_sparse_attention.module.rope as rope_mod
        _rope_config_compat(rope_mod)
        import native_sparse_attention.infer  # noqa: F401
        import native_sparse_attention.model  # noqa: F401
        import native_sparse_attention.module  # noqa: F401
    return ref


_linear = None


def reference_linear_compress():
    """(function, "triton" | "torch"): the reference's Triton ``linear_compress`` when its kernel compiles under the
    installed Triton, else the reference's own torch implementation of the same operator
    (ops/torch/compress_key_value.py:156-231, differentiable, 16-bit inputs, CUDA only).  Triton 3.6 fails to compile
    ``linear_compress_fwd_kernel`` for sm_100 (``PassManager::run failed`` in ``TritonGPUOptimizeDotOperands``); the
    reference pins Triton 3.0."""
    global _linear
    if _linear is None:
        import torch
        from native_sparse_attention.ops import linear_compress
        from native_sparse_attention.ops.torch.compress_key_value import linear_compress_torch
        try:
            x = torch.zeros(64, 1, 64, dtype=torch.bfloat16, device="cuda")
            w = torch.zeros(1, 32 * 64, 64, dtype=torch.bfloat16, device="cuda")
            linear_compress(x, w, torch.tensor([0, 64], dtype=torch.int32, device="cuda"), 32, 16, None)
            torch.cuda.synchronize()
            _linear = (linear_compress, "triton")
        except RuntimeError as e:
            if "PassManager" not in str(e):
                raise
            _linear = (linear_compress_torch, "torch")
    return _linear


def unload():
    """Forget the reference (and any shim installed over it) so that later tests start clean."""
    global _linear
    _linear = None
    _purge()


def llama3_rope_config(ref, head_dim=128, factor=8.0, theta=500000.0):
    from native_sparse_attention.module.rope import RopeConfig
    return RopeConfig(max_position_embeddings=131072, head_dim=head_dim, rope_theta=theta,
                      rope_scaling={"factor": factor, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                                    "original_max_position_embeddings": 8192, "rope_type": "llama3"})
