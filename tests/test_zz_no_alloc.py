"""The allocation-free gated contraction entry point, through the C ABI.

``b200_twell_gated_t2d_noalloc`` serves hosts that are not allowed to call the CUDA
allocator from a plugin (a server with a pre-planned memory map, a pool owned by another
framework): its scratch lives in a fixed array inside the library.  This file is named so
that pytest collects it last; it must pass alone in a fresh process and after every other
test, because the built-in array is shared by all calls of the process.
"""
import numpy as np
import pytest
import torch

from oracle import ffn_oracle as fo
from sparser_faster_llms_b200 import _lib, synthetic, twell

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")

# Same bound the other GPU tests use for two contraction runs on one slab: only the fp32
# summation grouping may differ.
REL_L2_SAME_SLAB = 2e-3


def _call_noalloc(lib, x, packed, up, down, out, flags=0):
    m, d = x.shape
    h = up.shape[0]
    with torch.cuda.device(DEV):
        return lib.b200_twell_gated_t2d_noalloc(
            x.data_ptr(), packed.data_ptr(), up.data_ptr(), down.data_ptr(), out.data_ptr(),
            m, d, h, 8, flags, torch.cuda.current_stream(DEV).cuda_stream)


@pytest.mark.parametrize("m,hp", [(1, False), (8, False), (32, True)])
def test_noalloc_matches_existing_entry_point_twice_in_a_row(m, hp):
    lib = _lib.load_library()
    d, h = 2048, 8192
    ffn = synthetic.make_ffn(d, h, seed=70, density=0.02, skew_sigma=1.0, device=DEV)
    x = synthetic.make_tokens(m, d, seed=71, device=DEV)
    packed = twell.matmul_sparse(x, ffn.gate)
    ref = twell.matmul_gated_t2d(x, packed, ffn.up, ffn.down, highest_precision=hp).float()
    torch.cuda.synchronize()
    outs = []
    for _ in range(2):  # second call sees the scratch the first one left behind
        y = torch.full_like(x, float("nan"))
        rc = _call_noalloc(lib, x, packed, ffn.up, ffn.down, y, 1 if hp else 0)
        assert rc == 0, lib.b200_last_error()
        torch.cuda.synchronize()
        outs.append(y.float())
    for y in outs:
        assert torch.isfinite(y).all()
        rel = ((y - ref).norm() / ref.norm()).item()
        assert rel < REL_L2_SAME_SLAB, rel
    assert torch.equal(outs[0], outs[1])
    # and against the CPU oracle fed the same slab (a prefix of rows: the loop oracle is slow)
    mo = min(m, 4)
    slab = packed[:mo].cpu().view(torch.int32).numpy().view(np.uint32)
    want = fo.gated_t2d(x[:mo].cpu(), slab, ffn.up.cpu(), ffn.down.cpu(), highest_precision=hp)
    _, rel = fo.max_abs_and_rel_l2(outs[0][:mo].cpu(), want)
    assert rel < REL_L2_SAME_SLAB, rel


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    lib = _lib.load_library()
    buf = torch.zeros(1024, dtype=torch.uint8, device=DEV)
    p = buf.data_ptr()
    # D = 2048: at most 63 tokens fit; nothing is launched for a rejected call
    rc = lib.b200_twell_gated_t2d_noalloc(p, p, p, p, p, 64, 2048, 8192, 8, 0, None)
    assert rc == -6
    assert b"exceeds the built-in scratch" in lib.b200_last_error()
    assert lib.b200_twell_gated_t2d_noalloc(p, p, p, p, p, 513, 256, 256, 8, 0, None) == -6
    assert lib.b200_twell_gated_t2d_noalloc(p, p, p, p, p, 4, 2048, 8192, 3, 0, None) == -1
    assert lib.b200_twell_gated_t2d_noalloc(None, p, p, p, p, 4, 2048, 8192, 8, 0, None) == -2
    assert lib.b200_twell_gated_t2d_noalloc(p, p, p, p, p, 0, 2048, 8192, 8, 0, None) == 0
    torch.cuda.synchronize()
