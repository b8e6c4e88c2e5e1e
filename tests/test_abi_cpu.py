"""C-ABI library: loads without a GPU, exports every declared symbol, validates arguments
before touching CUDA."""
import ctypes
import re
from pathlib import Path

import pytest

from sparser_faster_llms_b200 import _lib, build

REPO = Path(__file__).resolve().parent.parent
HEADER = REPO / "include" / "b200_sparse_ffn.h"


@pytest.fixture(scope="module")
def lib():
    build.build_library()
    return _lib.load_library()


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_functions()
    assert len(names) >= 8
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(names) == set(_lib.exported_names())


def test_version_and_arch(lib):
    assert lib.b200_version() >= 100
    assert lib.b200_built_for_sm() == 100


def test_argument_validation_happens_before_any_cuda_call(lib):
    buf = (ctypes.c_char * 64)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    # bad compression factor
    assert lib.b200_twell_pack(p16, p16, None, p16, 4, 256, 256, 3, None) == -1
    assert b"compression_factor" in lib.b200_last_error()
    # unsupported dims
    assert lib.b200_twell_pack(p16, p16, None, p16, 4, 100, 256, 8, None) == -4
    assert lib.b200_twell_pack(p16, p16, None, p16, 4, 256, 300, 8, None) == -4
    assert lib.b200_twell_pack(p16, p16, None, p16, -1, 256, 256, 8, None) == -1
    # null and misaligned pointers
    assert lib.b200_twell_pack(None, p16, None, p16, 4, 256, 256, 8, None) == -2
    assert lib.b200_twell_pack(p16 + 2, p16, None, p16, 4, 256, 256, 8, None) == -3
    assert lib.b200_twell_gated_t2d(p16, p16, None, p16, p16, 4, 256, 256, 8, 0, None, 0, None) == -2
    assert lib.b200_twell_gated_t2d(p16, p16, p16, p16, p16, 4, 256, 256, 8, 0x80, None, 0, None) == -1
    assert lib.b200_twell_t2d(p16, p16, p16, 4, 256, 256, 8, 3, None, 0, None) == -1
    # M == 0 is a successful no-op and needs no pointers
    assert lib.b200_twell_pack(None, None, None, None, 0, 256, 256, 8, None) == 0
    assert lib.b200_twell_gated_mlp(None, None, None, None, None, None, None, 0, 256, 256, 8, 0,
                                    None, 0, None) == 0
    assert lib.b200_twell_mlp(None, None, None, None, None, 0, 256, 256, 8, 2, None, 0, None) == 0
    assert lib.b200_workspace_bytes() >= 1 << 20


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load_library(tmp_path / "nope.so")
