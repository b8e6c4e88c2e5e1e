"""Stage the reference's own Python callers of the sparse-FFN path under ``oracle/_ref/``.

Test infrastructure, not product code: ``oracle/_ref/`` is git-ignored, it travels with the
working tree to a GPU machine that has no checkout of the reference, and only ``tests/`` and
``bench.py``'s CPU legs import from it.  The files are taken unmodified from a read-only
checkout (default: the directory ``reference`` next to this repository, or
``SPARSER_REFERENCE_ROOT``):

* ``custom_models/sparse_models.py``      SparseMLP (the torch path that defines the function),
                                          SparsityTracker, SparseLlamaForCausalLM,
                                          replace_mlp_modules
* ``custom_models/sparse_testing_utils.py``  convert_sparse_mlp_to_twell_fused, state-dict keys
* ``benchmark_inference.py``, ``benchmark_base.py``, ``energy_utils.py``  the inference benchmark

The reference's kernel modules (``twell_modules/twell.py``, ``hybrid_modules/*``) are NOT
staged: ``sparser_faster_llms_b200.dropin.install()`` registers this repository's modules
under those names.  ``python oracle/make_ref.py`` is idempotent; it prints what it did and
exits 0 when no checkout is present (the tests that need the files skip).
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
FILES = (
    "custom_models/__init__.py",
    "custom_models/sparse_models.py",
    "custom_models/sparse_testing_utils.py",
    "benchmark_inference.py",
    "benchmark_base.py",
    "energy_utils.py",
)


def reference_root() -> Path:
    return Path(os.environ.get("SPARSER_REFERENCE_ROOT", HERE.parent.parent / "reference"))


def stage(verbose: bool = True) -> bool:
    """Copy the caller files; True when ``oracle/_ref`` is complete afterwards."""
    root = reference_root()
    if not (root / "custom_models" / "sparse_models.py").exists():
        if verbose:
            print(f"oracle/make_ref: no reference checkout at {root}; nothing staged")
        return available()
    for rel in FILES:
        src, dst = root / rel, REF_DIR / rel
        if not src.exists():
            continue
        dst.parent.mkdir(parents=True, exist_ok=True)
        if not dst.exists() or dst.read_bytes() != src.read_bytes():
            shutil.copyfile(src, dst)
    if verbose:
        print(f"oracle/make_ref: staged {len(FILES)} files under {REF_DIR}")
    return available()


def available() -> bool:
    return all((REF_DIR / rel).exists() for rel in FILES if rel != "custom_models/__init__.py")


def import_path() -> str:
    """Directory to put on ``sys.path`` (after ``dropin.install()``) to import the callers."""
    return str(REF_DIR)


if __name__ == "__main__":
    sys.exit(0 if stage() or True else 1)
