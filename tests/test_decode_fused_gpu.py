"""GPU parity of the one-kernel decode layer (b200_twell_gated_mlp_decode) through the C ABI:
slab words bit-exact, outputs against the CPU oracle fed the same slab and against the
two-kernel path, workspace re-use, in-place, flex widths, the non-gated form and the
automatic choice inside b200_twell_gated_mlp.
"""
import numpy as np
import pytest
import torch

from oracle import ffn_oracle as fo
from oracle import twell_format as tf
from sparser_faster_llms_b200 import _lib, synthetic, twell

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")

REL_L2_MIXED = 1.2e-2     # vs the fp32 dense formula on the same bf16 inputs
REL_L2_HP = 4e-3
REL_L2_SAME_SLAB = 2e-3   # vs the oracle fed the same slab (summation order only)


def to_np_u32(t):
    return t.cpu().view(torch.int32).numpy().view(np.uint32)


def decode_ws(m, d, h):
    n = int(_lib.load_library().b200_twell_decode_workspace_bytes(m, d, h))
    return n, (torch.zeros(max(n, 16), dtype=torch.uint8, device=DEV) if n else None)


def fused(x, gate, up, down, cf=8, flags=0, ws=None, out=None, bias=None):
    m, d = x.shape
    h = gate.shape[0]
    packed = twell.allocate_packed_output(m, h, device=x.device, compression_factor=cf)
    out = torch.empty_like(x) if out is None else out
    if ws is None:
        _, ws = decode_ws(m, d, h)
    _lib.call("b200_twell_gated_mlp_decode", DEV, x.data_ptr(), gate.data_ptr(), _lib.ptr(bias),
              up.data_ptr(), down.data_ptr(), packed.data_ptr(), out.data_ptr(), m, d, h, cf,
              flags, ws.data_ptr(), ws.numel(), None, 0)
    torch.cuda.synchronize()
    return packed, out


SHAPES = [(1, 2048, 8192), (8, 2048, 8192), (32, 2048, 8192), (7, 1024, 4096),
          (17, 512, 1024), (3, 256, 256), (8, 4096, 2048), (5, 2048, 8448),
          (16, 2048, 8192), (12, 4096, 2048), (5, 2048, 16384), (20, 4096, 2048)]


@pytest.mark.parametrize("m,d,h", SHAPES)
def test_exact_arithmetic_slab_is_bit_exact(m, d, h):
    x, gate, up, down = synthetic.dyadic_case(m, d, h, seed=m + d + h)
    want = tf.pack_preactivations(fo.gate_preactivation(x, gate).numpy(), 8)
    packed, _ = fused(x.to(DEV), gate.to(DEV), up.to(DEV), down.to(DEV))
    assert np.array_equal(to_np_u32(packed), want)
    assert _lib.load_library().b200_twell_decode_status() == 0


@pytest.mark.parametrize("m,d,h", SHAPES)
@pytest.mark.parametrize("hp", [False, True])
def test_output_matches_oracle_on_the_kernels_own_slab(m, d, h, hp):
    ffn = synthetic.make_ffn(d, h, seed=11, density=0.02, skew_sigma=1.0)
    x = synthetic.make_tokens(m, d, seed=12)
    flags = _lib.FLAG_HIGH_PRECISION if hp else 0
    xg, gg = x.to(DEV), ffn.gate.to(DEV)
    packed, out = fused(xg, gg, ffn.up.to(DEV), ffn.down.to(DEV), flags=flags)
    slab = to_np_u32(packed)
    # the slab is what the pack kernel with the same summation order writes for the same call:
    # the mma.sync kernel (1) where the small-batch form serves, else tcgen05 split-k (3 / 5)
    ref = twell.allocate_packed_output(m, h, device=DEV)
    split8 = h // 256 <= 8 and d % 512 == 0
    small = m <= 16 and d in (2048, 4096)
    _lib.call("b200_twell_pack_select", DEV, xg.data_ptr(), gg.data_ptr(), None, ref.data_ptr(),
              m, d, h, 8, 1 if small else 5 if split8 else 3)
    torch.cuda.synchronize()
    assert np.array_equal(slab, to_np_u32(ref))
    mo = min(m, 10)
    want = fo.gated_t2d(x[:mo], slab[:mo], ffn.up, ffn.down, highest_precision=hp)
    got = out.float().cpu()
    _, rel_same = fo.max_abs_and_rel_l2(got[:mo], want)
    assert rel_same < REL_L2_SAME_SLAB, rel_same
    dense = fo.dense_ffn(x, ffn.gate, ffn.up, ffn.down)
    max_abs, rel = fo.max_abs_and_rel_l2(got, dense)
    assert rel < (REL_L2_HP if hp else REL_L2_MIXED), (max_abs, rel)
    assert _lib.load_library().b200_twell_decode_status() == 0


@pytest.mark.parametrize("cf", [4, 2])
def test_flex_widths(cf):
    m, d, h = 12, 1024, 2048
    ffn = synthetic.make_ffn(d, h, seed=13, density=0.05, skew_sigma=1.0)
    x = synthetic.make_tokens(m, d, seed=14)
    packed, out = fused(x.to(DEV), ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV), cf=cf)
    slab = to_np_u32(packed)
    want = fo.gated_t2d(x, slab, ffn.up, ffn.down, compression_factor=cf)
    _, rel = fo.max_abs_and_rel_l2(out.float().cpu(), want)
    assert rel < REL_L2_SAME_SLAB, rel


def test_slab_overflow_drops_the_same_entries_as_the_two_kernel_path():
    """Above a slab's capacity (31 entries at cf = 8) both forms use the stored prefix only."""
    m, d, h = 16, 1024, 2048
    ffn = synthetic.make_ffn(d, h, seed=15, density=0.2, skew_sigma=0.5)
    x = synthetic.make_tokens(m, d, seed=16)
    xg, g, u, dn = x.to(DEV), ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV)
    packed, out = fused(xg, g, u, dn)
    assert (tf.slab_counts(to_np_u32(packed), 8) > 31).any()
    want = twell.matmul_gated_t2d(xg, packed, u, dn)
    torch.cuda.synchronize()
    _, rel = fo.max_abs_and_rel_l2(out.float().cpu(), want.float().cpu())
    assert rel < REL_L2_SAME_SLAB, rel


def test_in_place_bias_and_workspace_shared_with_the_two_kernel_path():
    m, d, h = 32, 2048, 4096
    ffn = synthetic.make_ffn(d, h, seed=17, density=0.03, skew_sigma=1.0, fold_bias=False)
    x = synthetic.make_tokens(m, d, seed=18, fold_bias=False)
    xg, g, u, dn = x.to(DEV), ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV)
    bias = ffn.gate_bias.to(DEV)
    n, ws = decode_ws(m, d, h)
    assert n >= int(_lib.load_library().b200_workspace_bytes())
    _, first = fused(xg, g, u, dn, ws=ws, bias=bias)
    # the same buffer serves the multi-cluster contraction (few tokens) in between ...
    packed1 = twell.allocate_packed_output(1, h, device=DEV)
    y1 = torch.empty(1, d, device=DEV, dtype=torch.bfloat16)
    _lib.call("b200_twell_pack", DEV, xg.data_ptr(), g.data_ptr(), bias.data_ptr(),
              packed1.data_ptr(), 1, d, h, 8)
    _lib.call("b200_twell_gated_t2d", DEV, xg.data_ptr(), packed1.data_ptr(), u.data_ptr(),
              dn.data_ptr(), y1.data_ptr(), 1, d, h, 8, 0, ws.data_ptr(), ws.numel())
    # ... and the fused kernel again, this time over its own input
    buf = xg.clone()
    _, second = fused(buf, g, u, dn, ws=ws, out=buf, bias=bias)
    assert torch.equal(first, second)
    assert torch.equal(first[:1], y1) or fo.max_abs_and_rel_l2(
        y1.float().cpu(), first[:1].float().cpu())[1] < REL_L2_SAME_SLAB
    dense = fo.dense_ffn(x, ffn.gate, ffn.up, ffn.down, ffn.gate_bias)
    _, rel = fo.max_abs_and_rel_l2(first.float().cpu(), dense)
    assert rel < REL_L2_MIXED, rel
    assert _lib.load_library().b200_twell_decode_status() == 0


def test_gated_mlp_and_the_fused_form_agree():
    """b200_twell_gated_mlp (two kernels unless B200_DECODE_FUSED=1 is set) against the
    one-kernel entry point on the same call."""
    m, d, h = 24, 2048, 8192
    ffn = synthetic.make_ffn(d, h, seed=19, density=0.02, skew_sigma=1.0)
    x = synthetic.make_tokens(m, d, seed=20)
    xg, g, u, dn = x.to(DEV), ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV)
    n, ws = decode_ws(m, d, h)
    _, want = fused(xg, g, u, dn, ws=ws)
    packed = twell.allocate_packed_output(m, h, device=DEV)
    out = torch.empty_like(xg)
    _lib.call("b200_twell_gated_mlp", DEV, xg.data_ptr(), g.data_ptr(), None, u.data_ptr(),
              dn.data_ptr(), packed.data_ptr(), out.data_ptr(), m, d, h, 8, 0, ws.data_ptr(),
              ws.numel())
    torch.cuda.synchronize()
    _, rel = fo.max_abs_and_rel_l2(out.float().cpu(), want.float().cpu())
    assert rel < REL_L2_SAME_SLAB, rel
    small = torch.zeros(int(_lib.load_library().b200_workspace_bytes()), dtype=torch.uint8,
                        device=DEV)
    out2 = torch.empty_like(xg)
    _lib.call("b200_twell_gated_mlp", DEV, xg.data_ptr(), g.data_ptr(), None, u.data_ptr(),
              dn.data_ptr(), packed.data_ptr(), out2.data_ptr(), m, d, h, 8, 0, small.data_ptr(),
              small.numel())
    torch.cuda.synchronize()
    _, rel = fo.max_abs_and_rel_l2(out2.float().cpu(), want.float().cpu())
    assert rel < REL_L2_SAME_SLAB, rel  # the two-kernel form: another summation order


def test_non_gated_form_matches_the_two_kernel_path():
    m, d, h = 9, 1024, 4096
    ffn = synthetic.make_ffn(d, h, seed=21, density=0.02, skew_sigma=1.0)
    x = synthetic.make_tokens(m, d, seed=22)
    xg, u, dn = x.to(DEV), ffn.gate.to(DEV), ffn.down.to(DEV)
    n, ws = decode_ws(m, d, h)
    small = torch.zeros(int(_lib.load_library().b200_workspace_bytes()), dtype=torch.uint8,
                        device=DEV)
    outs = []
    for w in (ws, small):
        packed = twell.allocate_packed_output(m, h, device=DEV)
        out = torch.empty_like(xg)
        _lib.call("b200_twell_mlp", DEV, xg.data_ptr(), u.data_ptr(), dn.data_ptr(),
                  packed.data_ptr(), out.data_ptr(), m, d, h, 8, 2, w.data_ptr(), w.numel())
        torch.cuda.synchronize()
        outs.append(out.float().cpu())
    want = fo.t2d(to_np_u32(packed), ffn.down)
    assert fo.max_abs_and_rel_l2(outs[0], want)[1] < REL_L2_SAME_SLAB
    assert fo.max_abs_and_rel_l2(outs[1], want)[1] < REL_L2_SAME_SLAB


def test_shapes_the_fused_kernel_does_not_serve_are_refused():
    lib = _lib.load_library()
    assert lib.b200_twell_decode_workspace_bytes(33, 2048, 8192) == 0     # more than 32 tokens
    assert lib.b200_twell_decode_workspace_bytes(32, 4096, 16384) == 0    # accumulator too large
    assert lib.b200_twell_decode_workspace_bytes(0, 2048, 8192) == 0
    m, d, h = 20, 2048, 16384   # tcgen05 form: 64 clusters of 4 CTAs cannot be resident at once
    ffn = synthetic.make_ffn(d, h, seed=23, density=0.02)
    x = synthetic.make_tokens(m, d, seed=24).to(DEV)
    gg, ug, dg = ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV)
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device=DEV)
    packed = twell.allocate_packed_output(m, h, device=DEV)
    out = torch.empty_like(x)
    with pytest.raises(ValueError, match="resident"):
        _lib.call("b200_twell_gated_mlp_decode", DEV, x.data_ptr(), gg.data_ptr(), None,
                  ug.data_ptr(), dg.data_ptr(), packed.data_ptr(), out.data_ptr(), m, d, h, 8, 0,
                  ws.data_ptr(), ws.numel(), None, 0)
    with pytest.raises(ValueError, match="workspace"):
        _lib.call("b200_twell_gated_mlp_decode", DEV, x.data_ptr(), gg.data_ptr(), None,
                  ug.data_ptr(), dg.data_ptr(), packed.data_ptr(), out.data_ptr(), m, d, 8192, 8,
                  0, ws.data_ptr(), 4096, None, 0)
    with pytest.raises(ValueError, match="workspace"):   # the small-batch form as well
        _lib.call("b200_twell_gated_mlp_decode", DEV, x.data_ptr(), gg.data_ptr(), None,
                  ug.data_ptr(), dg.data_ptr(), packed.data_ptr(), out.data_ptr(), 4, d, 8192, 8,
                  0, ws.data_ptr(), 4096, None, 0)


def test_l2_prefetch_is_a_harmless_hint():
    w = torch.randn(1 << 20, device=DEV)
    _lib.call("b200_l2_prefetch", DEV, w.data_ptr(), w.numel() * 4)
    _lib.call("b200_l2_prefetch", DEV, w.data_ptr(), 0)
    torch.cuda.synchronize()
    with pytest.raises(ValueError):
        _lib.call("b200_l2_prefetch", DEV, w.data_ptr() + 4, 64)
