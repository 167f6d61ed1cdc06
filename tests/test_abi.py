"""The C-ABI library loads on a machine without a GPU and exports every symbol the public header declares."""
import os
import re

from native_sparse_attention_triton_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    """Every function declared by the headers under include/ (the operator interface and the measurement hooks)."""
    names = set()
    for header in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not header.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(nsa_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    handle = _lib.lib()
    declared = header_functions()
    assert len(declared) >= 17
    for name in declared:
        assert hasattr(handle, name), f"{name} is declared under include/ but not exported"
    # and the Python binding knows the argument types of every one of them
    assert sorted(_lib.exported_symbols()) == declared


def test_version_and_argument_checks_without_gpu():
    handle = _lib.lib()
    assert handle.nsa_version() >= 1
    # null pointers are rejected before anything touches a device
    assert handle.nsa_decode_num_splits(4, 2, 128) >= 1
    assert handle.nsa_decode_num_splits(4, 2, 1) == 1
    nbytes = handle.nsa_topk_sparse_attn_bwd_workspace(1024, 2, 16, 2, 64, 4, 64)
    assert nbytes > 1024 * 2 * 64 * 4 * 2
