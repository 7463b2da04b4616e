#!/usr/bin/env bash
# Compiles the native module in-tree for sm_100a (nvcc + g++, about 20 s cold, cached by content hash).
set -euo pipefail
cd "$(dirname "$0")"
python -c "import __graft_entry__ as g; g.build()"
python -c "import flexkv_b200; from flexkv_b200 import _native; print('flexkv_b200', flexkv_b200.__git_commit__ or '', 'native module:', _native.C.__file__)"
