"""In-tree build of the C-ABI CUDA library (sm_100a only).

``python -m sparser_faster_llms_b200.build`` compiles every ``csrc/*.cu`` into
``sparser_faster_llms_b200/libb200_sparse_ffn.so`` with plain nvcc: no torch
headers, no pybind, static cudart, so the result is a stable C ABI that loads
with ``ctypes`` on a machine without a GPU driver.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_NAME = "libb200_sparse_ffn.so"
LIB_PATH = PKG_DIR / LIB_NAME
GENCODE = "arch=compute_100a,code=sm_100a"


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc")
    if nvcc is None:
        cand = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
        if cand.exists():
            nvcc = str(cand)
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
    return nvcc


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [
        PKG_DIR.parent / "include" / "b200_sparse_ffn.h"]
    return any(p.stat().st_mtime > built for p in deps)


def build_library(force: bool = False, verbose: bool = False, extra_flags=()) -> Path:
    """Compile the library if it is missing or older than its sources."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = find_nvcc()
    objs = []
    obj_dir = PKG_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    common = [nvcc, "-gencode", GENCODE, "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", *extra_flags]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        objs.append(obj)
        procs.append((src, subprocess.Popen(
            common + ["-c", str(src), "-o", str(obj)],
            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose and out:
            print(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
    tmp = LIB_PATH.with_suffix(".so.tmp")
    link = [nvcc, "-gencode", GENCODE, "-shared", "-o", str(tmp), *map(str, objs)]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc link failed:\n{res.stdout}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
