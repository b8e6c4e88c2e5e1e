"""Make the reference's own scripts use these kernels without editing them.

The reference imports its kernels under two module names:

* ``custom_models.twell_modules.twell`` (custom_models/sparse_testing_utils.py:7,
  benchmark_inference.py:28), and
* ``custom_models.hybrid_modules.sparse_ops_loader``
  (custom_models/sparse_models.py:313-316).

``install()`` registers this package's modules under those names in
``sys.modules`` before the reference is imported, so
``model.replace_mlp_modules(convert_sparse_mlp_to_twell_fused)`` and
``benchmark_inference.py`` pick up the sm_100a kernels.  The reference checkout
must be importable (on ``sys.path``) for its remaining modules.
"""
from __future__ import annotations

import importlib
import sys
import types

TWELL_NAME = "custom_models.twell_modules.twell"
LOADER_NAME = "custom_models.hybrid_modules.sparse_ops_loader"


def _ensure_parent(name: str) -> None:
    """Register an empty namespace package for ``name`` if it cannot be imported."""
    if name in sys.modules:
        return
    try:
        importlib.import_module(name)
    except Exception:
        mod = types.ModuleType(name)
        mod.__path__ = []  # mark as package
        sys.modules[name] = mod


def install(twell: bool = True, sparse_ops: bool = True) -> None:
    """Register the replacements under the reference's module names (idempotent)."""
    _ensure_parent("custom_models")
    if twell:
        from . import twell as twell_mod
        _ensure_parent("custom_models.twell_modules")
        sys.modules[TWELL_NAME] = twell_mod
        setattr(sys.modules["custom_models.twell_modules"], "twell", twell_mod)
    if sparse_ops:
        try:
            from . import sparse_ops_loader as loader_mod
        except ImportError:
            loader_mod = None
        if loader_mod is not None:
            _ensure_parent("custom_models.hybrid_modules")
            sys.modules[LOADER_NAME] = loader_mod
            setattr(sys.modules["custom_models.hybrid_modules"], "sparse_ops_loader", loader_mod)


def uninstall() -> None:
    for name in (TWELL_NAME, LOADER_NAME):
        sys.modules.pop(name, None)
