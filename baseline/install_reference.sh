#!/bin/sh
# Installs the UNMODIFIED reference project (XunhaoLai/native-sparse-attention-triton) into baseline/_ref/, which is
# git-ignored: the reference never enters this repository's history, but the directory travels with a working copy to
# a GPU machine, where the same-box parity tests (tests/test_gpu_vs_reference*.py), tests/golden/make_golden_on_box.py
# and bench.py's "gpu_reference" block import it.  Offline: no index is contacted and no dependency is resolved (torch,
# triton, einops, flash_attn and transformers come from the environment).
#
#   sh baseline/install_reference.sh /path/to/reference/checkout
set -e
SRC="${1:?usage: install_reference.sh /path/to/reference/checkout}"
HERE="$(cd "$(dirname "$0")" && pwd)"
TMP="$(mktemp -d)"
cp -r "$SRC" "$TMP/ref"          # the build writes into the source tree; the checkout may be read-only
chmod -R u+w "$TMP/ref"
rm -rf "$HERE/_ref"
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
    --target "$HERE/_ref" "$TMP/ref"
rm -rf "$TMP"
ls "$HERE/_ref"
