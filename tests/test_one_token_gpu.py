"""GPU parity of the one-token form (GEMV pack kernel, kernel id 6 of b200_twell_pack_select,
and the whole layer inside it through b200_twell_gated_mlp / b200_twell_mlp at M = 1):
slab words bit-exact on exact-arithmetic inputs, outputs against the CPU oracle fed the
kernel's own slab and against the dense formula, overflowing slabs, bias, in-place,
workspace re-use next to the contraction kernel, and the refusals.
"""
import numpy as np
import pytest
import torch

from oracle import ffn_oracle as fo
from oracle import twell_format as tf
from sparser_faster_llms_b200 import _lib, synthetic, twell

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")

REL_L2_MIXED = 1.2e-2
REL_L2_HP = 4e-3
REL_L2_SAME_SLAB = 2e-3

SHAPES = [(2048, 8192), (2048, 256), (4096, 2048), (2048, 5632), (4096, 16384),
          (2048, 11008)]


def to_np_u32(t):
    return t.cpu().view(torch.int32).numpy().view(np.uint32)


def workspace(d, h):
    return torch.zeros(4096 * 4 + (h // 256) * d * 4, dtype=torch.uint8, device=DEV)


def pack6(x, w, cf=8, bias=None):
    h = w.shape[0]
    packed = twell.allocate_packed_output(1, h, device=DEV, compression_factor=cf)
    packed.zero_()
    _lib.call("b200_twell_pack_select", DEV, x.data_ptr(), w.data_ptr(), _lib.ptr(bias),
              packed.data_ptr(), 1, x.shape[1], h, cf, 6)
    torch.cuda.synchronize()
    return packed


def layer(x, gate, up, down, cf=8, flags=0, ws=None, out=None, bias=None):
    d, h = x.shape[1], gate.shape[0]
    packed = twell.allocate_packed_output(1, h, device=DEV, compression_factor=cf)
    packed.zero_()
    out = torch.empty_like(x) if out is None else out
    ws = workspace(d, h) if ws is None else ws
    _lib.call("b200_twell_gated_mlp", DEV, x.data_ptr(), gate.data_ptr(), _lib.ptr(bias),
              up.data_ptr(), down.data_ptr(), packed.data_ptr(), out.data_ptr(), 1, d, h, cf,
              flags, ws.data_ptr(), ws.numel())
    torch.cuda.synchronize()
    return packed, out


@pytest.mark.parametrize("d,h", SHAPES)
@pytest.mark.parametrize("cf", [8, 2])
def test_exact_arithmetic_slab_is_bit_exact(d, h, cf):
    x, gate, up, down = synthetic.dyadic_case(1, d, h, seed=d + h)
    want = tf.pack_preactivations(fo.gate_preactivation(x, gate).numpy(), cf)
    assert np.array_equal(to_np_u32(pack6(x.to(DEV), gate.to(DEV), cf)), want)
    packed, _ = layer(x.to(DEV), gate.to(DEV), up.to(DEV), down.to(DEV), cf=cf)
    assert np.array_equal(to_np_u32(packed), want)


@pytest.mark.parametrize("d,h", SHAPES)
@pytest.mark.parametrize("hp", [False, True])
def test_output_matches_oracle_on_the_kernels_own_slab(d, h, hp):
    ffn = synthetic.make_ffn(d, h, seed=31, density=0.03, skew_sigma=1.0)
    x = synthetic.make_tokens(1, d, seed=32)
    flags = _lib.FLAG_HIGH_PRECISION if hp else 0
    xg, gg = x.to(DEV), ffn.gate.to(DEV)
    packed, out = layer(xg, gg, ffn.up.to(DEV), ffn.down.to(DEV), flags=flags)
    slab = to_np_u32(packed)
    assert np.array_equal(slab, to_np_u32(pack6(xg, gg)))      # both forms: the same kernel code
    # against the few-token pack kernel: another summation order, so equal outside a sign band
    ref = twell.allocate_packed_output(1, h, device=DEV)
    ref.zero_()
    _lib.call("b200_twell_pack_select", DEV, xg.data_ptr(), gg.data_ptr(), None, ref.data_ptr(),
              1, d, h, 8, 1)
    torch.cuda.synchronize()
    a = tf.unpack_to_dense(slab, h, 8, strict=False)
    b = tf.unpack_to_dense(to_np_u32(ref), h, 8, strict=False)
    amb, _ = fo.ambiguity_mask(x, ffn.gate, rel=4e-6)
    sure = ~amb.numpy()
    assert np.array_equal((a > 0)[sure], (b > 0)[sure])
    want = fo.gated_t2d(x, slab, ffn.up, ffn.down, highest_precision=hp)
    got = out.float().cpu()
    assert fo.max_abs_and_rel_l2(got, want)[1] < REL_L2_SAME_SLAB
    dense = fo.dense_ffn(x, ffn.gate, ffn.up, ffn.down)
    assert fo.max_abs_and_rel_l2(got, dense)[1] < (REL_L2_HP if hp else REL_L2_MIXED)


@pytest.mark.parametrize("cf", [8, 4])
def test_overflowing_slabs_keep_the_stored_prefix_like_the_two_kernel_path(cf):
    d, h = 2048, 2048
    ffn = synthetic.make_ffn(d, h, seed=33, density=0.3, skew_sigma=0.5)
    x = synthetic.make_tokens(1, d, seed=34)
    xg, g, u, dn = x.to(DEV), ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV)
    packed, out = layer(xg, g, u, dn, cf=cf)
    slab = to_np_u32(packed)
    assert (tf.slab_counts(slab, cf) > 256 // cf - 1).any()
    want = fo.gated_t2d(x, slab, ffn.up, ffn.down, compression_factor=cf)
    assert fo.max_abs_and_rel_l2(out.float().cpu(), want)[1] < REL_L2_SAME_SLAB
    two = twell.matmul_gated_t2d(xg, packed, u, dn, compression_factor=cf, flex_kernels=True)
    torch.cuda.synchronize()
    assert fo.max_abs_and_rel_l2(out.float().cpu(), two.float().cpu())[1] < REL_L2_SAME_SLAB


def test_bias_in_place_and_workspace_shared_with_the_contraction_kernel():
    d, h = 2048, 4096
    ffn = synthetic.make_ffn(d, h, seed=35, density=0.03, skew_sigma=1.0, fold_bias=False)
    x = synthetic.make_tokens(4, d, seed=36, fold_bias=False)
    xg, g, u, dn = x.to(DEV), ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV)
    bias = ffn.gate_bias.to(DEV)
    ws = workspace(d, h)
    _, first = layer(xg[:1], g, u, dn, ws=ws, bias=bias)
    # the same buffer serves the multi-cluster contraction of a 4-token call in between
    packed4 = twell.allocate_packed_output(4, h, device=DEV)
    y4 = torch.empty(4, d, device=DEV, dtype=torch.bfloat16)
    _lib.call("b200_twell_gated_mlp", DEV, xg.data_ptr(), g.data_ptr(), bias.data_ptr(),
              u.data_ptr(), dn.data_ptr(), packed4.data_ptr(), y4.data_ptr(), 4, d, h, 8, 0,
              ws.data_ptr(), ws.numel())
    buf = xg[:1].clone()
    _, second = layer(buf, g, u, dn, ws=ws, out=buf, bias=bias)
    assert torch.equal(first, second)
    assert fo.max_abs_and_rel_l2(y4[:1].float().cpu(), first.float().cpu())[1] < REL_L2_SAME_SLAB
    dense = fo.dense_ffn(x[:1], ffn.gate, ffn.up, ffn.down, ffn.gate_bias)
    assert fo.max_abs_and_rel_l2(first.float().cpu(), dense)[1] < REL_L2_MIXED
    # many launches back to back leave the counters at zero every time
    outs = [layer(xg[:1], g, u, dn, ws=ws, bias=bias)[1] for _ in range(5)]
    assert all(torch.equal(o, first) for o in outs)


def test_non_gated_form_matches_the_oracle():
    d, h = 2048, 4096
    ffn = synthetic.make_ffn(d, h, seed=37, density=0.02, skew_sigma=1.0)
    x = synthetic.make_tokens(1, d, seed=38)
    xg, u, dn = x.to(DEV), ffn.gate.to(DEV), ffn.down.to(DEV)
    ws = workspace(d, h)
    packed = twell.allocate_packed_output(1, h, device=DEV)
    packed.zero_()
    out = torch.empty_like(xg)
    _lib.call("b200_twell_mlp", DEV, xg.data_ptr(), u.data_ptr(), dn.data_ptr(),
              packed.data_ptr(), out.data_ptr(), 1, d, h, 8, 2, ws.data_ptr(), ws.numel())
    torch.cuda.synchronize()
    want = fo.t2d(to_np_u32(packed), ffn.down)
    assert fo.max_abs_and_rel_l2(out.float().cpu(), want)[1] < REL_L2_SAME_SLAB


def test_empty_slabs_give_a_zero_row():
    d, h = 2048, 1024
    x = torch.ones(1, d, dtype=torch.bfloat16, device=DEV)
    gate = -torch.ones(h, d, dtype=torch.bfloat16, device=DEV)
    up = torch.ones(h, d, dtype=torch.bfloat16, device=DEV)
    packed, out = layer(x, gate, up, up.clone())
    assert int(to_np_u32(packed).sum()) == 0 and float(out.float().abs().sum()) == 0.0


def test_refusals():
    lib = _lib.load_library()
    d, h = 1024, 1024          # d_model not served by the one-token kernel
    x = torch.zeros(1, d, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(h, d, dtype=torch.bfloat16, device=DEV)
    packed = twell.allocate_packed_output(1, h, device=DEV)
    rc = lib.b200_twell_pack_select(x.data_ptr(), w.data_ptr(), None, packed.data_ptr(), 1, d, h,
                                    8, 6, None)
    assert rc == -4 and b"not served" in lib.b200_last_error()
    x2 = torch.zeros(2, 2048, dtype=torch.bfloat16, device=DEV)
    w2 = torch.zeros(256, 2048, dtype=torch.bfloat16, device=DEV)
    p2 = twell.allocate_packed_output(2, 256, device=DEV)
    rc = lib.b200_twell_pack_select(x2.data_ptr(), w2.data_ptr(), None, p2.data_ptr(), 2, 2048,
                                    256, 8, 6, None)
    assert rc == -4 and b"one token" in lib.b200_last_error()
    rc = lib.b200_twell_pack_select(x2.data_ptr(), w2.data_ptr(), None, p2.data_ptr(), 2, 2048,
                                    256, 8, 10, None)
    assert rc == -1
