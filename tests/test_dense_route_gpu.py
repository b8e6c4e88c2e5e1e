"""Hybrid contraction: dense-enough / overflowed token rows on the tcgen05 dense route, the
rest on the gather kernel.  Checked against the fp32 dense formula (the oracle) row by row,
and against the gather-only path bit for bit on the rows that were not routed."""
import pytest
import torch

from oracle import ffn_oracle as fo
from sparser_faster_llms_b200 import _lib, synthetic, twell

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# Relative L2 per row against the fp32 dense formula on the same bf16 inputs.  The dense
# route rounds g, u, h and y to bf16 once each (fp32 tensor-core sums in between).
REL_L2_ROW = 1.5e-2


def row_rel_l2(y, ref):
    y, ref = y.float().cpu(), ref.float().cpu()
    return (y - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-20)


def make_case(m, d, h, seed, base_density=0.02):
    ffn = synthetic.make_ffn(d, h, seed=seed, density=base_density, skew_sigma=0.0)
    x, rho = synthetic.make_tokens_mixed_density(m, d, base_density=base_density, seed=seed + 1)
    ref = fo.dense_ffn(x, ffn.gate, ffn.up, ffn.down)
    return ffn, x, rho, ref


def slab_counts(x, gate, cf=8):
    packed = twell.matmul_sparse(x, gate, compression_factor=cf)
    w = 256 // cf
    return packed.view(torch.int32)[:, ::w].cpu().long()


def modules(layer, ffn, **route):
    args = [ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV)]
    sparse = twell.TwELLGatedMLP(layer, *args)
    hybrid = twell.TwELLGatedMLP(layer + 1, *args)
    hybrid.enable_dense_route(**route)
    return sparse, hybrid


@pytest.mark.parametrize("m,d,h", [(1024, 1024, 4096), (300, 2048, 11008)])
def test_hybrid_rows_match_dense_formula(m, d, h):
    ffn, x, rho, ref = make_case(m, d, h, seed=300 + m)
    xg = x.to(DEV)
    sparse, hybrid = modules(7000, ffn, nnz_threshold=h // 16, dense_cap=m, min_tokens=128)
    y_sparse = sparse(xg)
    y_hybrid = hybrid(xg)
    torch.cuda.synchronize()
    assert _lib.load_library().b200_twell_hybrid_status() == 0

    counts = slab_counts(xg, ffn.gate.to(DEV))
    qualifies = (counts.sum(1) > h // 16) | (counts > 31).any(1)
    overflowed = (counts > 31).any(1)
    assert qualifies.sum() >= 8 and overflowed.sum() >= 4, "the case must exercise the route"
    c = hybrid.dense_route_counters()
    assert c == {"dense_rows": int(qualifies.sum()), "lossy_rows_left_sparse": 0,
                 "qualified_rows": int(qualifies.sum())}

    err_h = row_rel_l2(y_hybrid, ref)
    err_s = row_rel_l2(y_sparse, ref)
    assert err_h.max() < REL_L2_ROW, (int(err_h.argmax()), float(err_h.max()))
    # the gather-only path loses the entries beyond a slab's capacity on overflowed rows
    assert err_s[overflowed].max() > 5 * REL_L2_ROW
    # rows that were not routed come from the same kernel: identical bits
    keep = ~qualifies
    assert torch.equal(y_hybrid.cpu()[keep], y_sparse.cpu()[keep])
    sparse.destroy()
    hybrid.destroy()


def test_hybrid_with_wider_slabs_cf4():
    """cf = 4: 63 entries per tile, so only rows above ~25 % in some tile overflow; routing reads
    the capacity from the slab width."""
    m, d, h, cf = 384, 1024, 4096, 4
    ffn, x, rho, ref = make_case(m, d, h, seed=905)
    xg = x.to(DEV)
    args = [ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV)]
    kw = dict(compression_factor=cf, flex_kernels=True)
    sparse = twell.TwELLGatedMLP(7040, *args, **kw)
    hybrid = twell.TwELLGatedMLP(7041, *args, **kw)
    hybrid.enable_dense_route(nnz_threshold=h // 8, dense_cap=m, min_tokens=128)
    y_sparse, y_hybrid = sparse(xg), hybrid(xg)
    torch.cuda.synchronize()
    counts = slab_counts(xg, ffn.gate.to(DEV), cf=cf)
    qualifies = (counts.sum(1) > h // 8) | (counts > 63).any(1)
    assert qualifies.sum() >= 4
    assert hybrid.dense_route_counters()["dense_rows"] == int(qualifies.sum())
    assert row_rel_l2(y_hybrid, ref).max() < REL_L2_ROW
    assert torch.equal(y_hybrid.cpu()[~qualifies], y_sparse.cpu()[~qualifies])
    sparse.destroy()
    hybrid.destroy()


def test_dense_cap_exhausted_leaves_later_rows_on_gather_path():
    m, d, h = 512, 1024, 4096
    ffn, x, rho, ref = make_case(m, d, h, seed=411)
    xg = x.to(DEV)
    cap = 128
    sparse, hybrid = modules(7010, ffn, nnz_threshold=h // 64, dense_cap=cap, min_tokens=128)
    y_sparse, y_hybrid = sparse(xg), hybrid(xg)
    torch.cuda.synchronize()
    counts = slab_counts(xg, ffn.gate.to(DEV))
    qualifies = (counts.sum(1) > h // 64) | (counts > 31).any(1)
    overflowed = (counts > 31).any(1)
    q_rows = torch.nonzero(qualifies).flatten()
    assert len(q_rows) > cap
    routed = torch.zeros(m, dtype=torch.bool)
    routed[q_rows[:cap]] = True
    c = hybrid.dense_route_counters()
    assert c["dense_rows"] == cap and c["qualified_rows"] == len(q_rows)
    assert c["lossy_rows_left_sparse"] == int((overflowed & ~routed).sum())
    assert row_rel_l2(y_hybrid, ref)[routed].max() < REL_L2_ROW
    assert torch.equal(y_hybrid.cpu()[~routed], y_sparse.cpu()[~routed])
    sparse.destroy()
    hybrid.destroy()


def test_small_calls_keep_the_gather_kernel():
    m, d, h = 64, 1024, 4096
    ffn, x, rho, ref = make_case(m, d, h, seed=77)
    xg = x.to(DEV)
    sparse, hybrid = modules(7020, ffn, min_tokens=256)
    assert torch.equal(sparse(xg).cpu(), hybrid(xg).cpu())
    assert hybrid.dense_route_counters() is None
    sparse.destroy()
    hybrid.destroy()


@pytest.mark.parametrize("m", [40, 128, 200, 512, 1024])   # up to 512 rows: the split-k GEMMs
def test_all_rows_dense_with_gate_bias(m):
    """dense_all_tokens: no slab at all; also covers the explicit (not folded) gate bias and a
    token count that is not a multiple of the 128-token tile."""
    d, h = 1024, 4096
    ffn = synthetic.make_ffn(d, h, seed=500 + m, density=0.05, fold_bias=False)
    x = synthetic.make_tokens(m, d, seed=501, fold_bias=False)
    ref = fo.dense_ffn(x, ffn.gate, ffn.up, ffn.down, gate_bias=ffn.gate_bias)
    mod = twell.TwELLGatedMLP(7030, ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV))
    mod.set_gate_bias(ffn.gate_bias)
    mod.enable_dense_route(dense_all_tokens=32)
    y = mod(x.to(DEV))
    torch.cuda.synchronize()
    assert _lib.load_library().b200_twell_hybrid_status() == 0
    assert row_rel_l2(y, ref).max() < REL_L2_ROW
    # switching the route off returns to the slab path (reference behaviour)
    mod.disable_dense_route()
    y2 = mod(x.to(DEV))
    assert row_rel_l2(y2, ref).max() < 3e-2
    mod.destroy()


def test_hybrid_entry_point_rejects_bad_arguments():
    lib = _lib.load_library()
    m, d, h = 256, 1024, 4096
    need = lib.b200_twell_hybrid_workspace_bytes(m, d, h, 128)
    assert need > 128 * (d + h) * 2
    t = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    p = t.data_ptr()
    # workspace too small
    rc = lib.b200_twell_gated_t2d_hybrid(p, p, p, None, p, p, p, p, m, d, h, 8, 0, 100, 128,
                                         p, 4096, None, 0, None)
    assert rc == -6
    # NULL transposed down projection
    rc = lib.b200_twell_gated_t2d_hybrid(p, p, p, None, p, p, None, p, m, d, h, 8, 0, 100, 128,
                                         p, need, None, 0, None)
    assert rc == -2
    rc = lib.b200_twell_gated_t2d_hybrid(p, p, p, None, p, p, p, p, m, d, h, 8, 0, 100, 0,
                                         p, need, None, 0, None)
    assert rc == -1


def test_all_rows_dense_on_256_token_tiles_for_both_products():
    """4096 tokens at D 2048 / d_ff 1024: both GEMMs of the all-dense route have 128 tiles of
    256 tokens, i.e. both run the one-CTA-per-SM form with sixteen epilogue warps."""
    m, d, h = 4096, 2048, 1024
    ffn = synthetic.make_ffn(d, h, seed=900, density=0.05)
    x = synthetic.make_tokens(m, d, seed=901)
    ref = fo.dense_ffn(x, ffn.gate, ffn.up, ffn.down)
    mod = twell.TwELLGatedMLP(7040, ffn.gate.to(DEV), ffn.up.to(DEV), ffn.down.to(DEV))
    mod.enable_dense_route(dense_all_tokens=1024)
    y = mod(x.to(DEV))
    torch.cuda.synchronize()
    assert _lib.load_library().b200_twell_hybrid_status() == 0
    assert row_rel_l2(y, ref).max() < REL_L2_ROW
    mod.destroy()
