"""Replacement for ``custom_models.hybrid_modules.sparse_ops_loader``.

The reference JIT-compiles a TORCH_LIBRARY extension or loads ``SPARSE_OPS_PREBUILT``
(custom_models/hybrid_modules/sparse_ops_loader.py:50-94).  Here the operators are
registered from Python (``sparse_ops.register_ops``) on top of the prebuilt C-ABI
library, so there is nothing to compile at import time.  ``SPARSE_OPS_PREBUILT``, when
set, names the C-ABI library to load instead of the in-tree one.
"""
from __future__ import annotations

import os
from pathlib import Path

from . import _lib, sparse_ops

_BASE_DIR = Path(__file__).resolve().parent
_EXT_NAME = "sparse_ops"
_loaded = False


def load_sparse_ops(verbose: bool = False):
    """Registers ``torch.ops.sparse_ops`` / ``sparse_ops_config`` / ``sparse_ops_perf``.
    Idempotent.  Raises if the CUDA library is missing (no fallback)."""
    global _loaded
    if _loaded:
        return
    prebuilt = os.environ.get("SPARSE_OPS_PREBUILT")
    if prebuilt:
        _lib._LIB = _lib.load_library(prebuilt)
    else:
        _lib.load_library()
    sparse_ops.register_ops()
    if verbose:
        print(f"[sparse_ops] registered on top of {prebuilt or _lib.LIB_PATH}")
    _loaded = True
