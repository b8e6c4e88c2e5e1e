"""Hybrid training operator on the GPU: forward outputs, l0 / l1 and all four gradients
against fp32 autograd of the dense formula (the oracle; its agreement with the reference's
SparseMLP training branch is pinned in tests/test_oracle_golden.py) and against the
gradients the reference itself produced (tests/golden/training_gated.npz).
"""
import numpy as np
import pytest
import torch

from oracle import ffn_oracle as fo
from sparser_faster_llms_b200 import sparse_ops, synthetic
from sparser_faster_llms_b200.sparse_ops_loader import load_sparse_ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# bf16 storage of R, T, dT, dR, dU and of the outputs; fp32 accumulation inside each product
REL_OUT = 1.2e-2
REL_GRAD = 2.5e-2


def rel_l2(a, b):
    a, b = a.double().flatten().cpu(), b.double().flatten().cpu()
    return ((a - b).norm() / b.norm()).item()


def dense_reference(x, gate, up, down, gout, coeff):
    """fp32 autograd through out = (relu(X G^T) * (X K^T)) V and l1 = mean_rows sum |T|."""
    x = x.float().clone().requires_grad_(True)
    g, k, v = (t.float().clone().requires_grad_(True) for t in (gate, up, down))
    xf = x.reshape(-1, x.shape[-1])
    hid = torch.relu(xf @ g.T) * (xf @ k.T)
    out = (hid @ v).reshape(x.shape)
    l0, l1 = fo.l0_l1(hid.abs())
    ((out * gout.float()).sum() + coeff * l1).backward()
    return out.detach(), l0.detach(), l1.detach(), x.grad, g.grad, k.grad, v.grad


@pytest.fixture(scope="module", autouse=True)
def ops():
    load_sparse_ops()
    load_sparse_ops()  # idempotent
    yield
    torch.ops.sparse_ops_config.set_ell_width_regular(128)


@pytest.fixture(params=["sparse", "dense"])
def wgrad_mode(request):
    """Both forms of the weight-gradient products: column lists + transposed SpMM, and
    scatter + tcgen05 GEMM (the automatic choice depends on the token count)."""
    sparse_ops.set_weight_gradient_mode(request.param)
    yield request.param
    sparse_ops.set_weight_gradient_mode("auto")


@pytest.mark.parametrize("b,s,d,h,density", [(2, 12, 256, 512, 0.06), (2, 64, 1024, 4096, 0.02),
                                            (1, 33, 512, 1024, 0.10), (4, 640, 512, 2048, 0.03)])
def test_forward_and_backward_match_dense_autograd(b, s, d, h, density, wgrad_mode):
    ffn = synthetic.make_ffn(d, h, seed=21, density=density, skew_sigma=0.5)
    x = synthetic.make_tokens(b * s, d, seed=22).reshape(b, s, d)
    gout = synthetic.make_tokens(b * s, d, seed=23, fold_bias=False).reshape(b, s, d)
    coeff = 0.05
    ref = dense_reference(x, ffn.gate, ffn.up, ffn.down, gout, coeff)

    X = x.to(DEV).requires_grad_(True)
    G, K, V = (t.to(DEV).requires_grad_(True) for t in (ffn.gate, ffn.up, ffn.down))
    out, l0, l1, P, R, T = torch.ops.sparse_ops.ff_forward_gated(X, G, K, V)
    assert out.shape == X.shape and out.dtype == torch.bfloat16
    assert P.dtype == torch.int32 and P.shape == R.shape == T.shape
    ((out.float() * gout.to(DEV).float()).sum() + coeff * l1).backward()
    torch.cuda.synchronize()

    assert rel_l2(out, ref[0]) < REL_OUT
    assert abs(l0.item() - ref[1].item()) <= 0.02 * ref[1].item() + 0.05
    assert abs(l1.item() - ref[2].item()) <= 1e-2 * abs(ref[2].item())
    for got, want, name in ((X.grad, ref[3], "dX"), (G.grad, ref[4], "dG"),
                            (K.grad, ref[5], "dK"), (V.grad, ref[6], "dV")):
        assert got is not None and got.shape == want.shape, name
        assert rel_l2(got, want) < REL_GRAD, (name, rel_l2(got, want))
    cnt = torch.ops.sparse_ops_config.get_last_transpose_overflow_count()
    assert int(cnt.item()) == 0


def test_against_gradients_produced_by_the_reference(golden_dir, wgrad_mode):
    g = np.load(golden_dir / "training_gated.npz")
    b, s, d, h = (int(g[k]) for k in ("b", "s", "d", "h"))
    ffn = synthetic.make_ffn(d, h, seed=int(g["seed_ffn"]), density=0.06, skew_sigma=0.5)
    x = synthetic.make_tokens(b * s, d, seed=int(g["seed_x"])).reshape(b, s, d)
    gout = synthetic.make_tokens(b * s, d, seed=int(g["seed_gout"]), fold_bias=False)
    X = x.to(DEV).requires_grad_(True)
    G, K, V = (t.to(DEV).requires_grad_(True) for t in (ffn.gate, ffn.up, ffn.down))
    out, l0, l1, *_ = torch.ops.sparse_ops.ff_forward_gated(X, G, K, V)
    ((out.float().reshape(-1, d) * gout.to(DEV).float()).sum() + float(g["coeff"]) * l1).backward()
    assert rel_l2(out, torch.from_numpy(g["y"])) < REL_OUT
    assert abs(l1.item() - float(g["l1"])) < 1e-2 * abs(float(g["l1"]))
    assert abs(l0.item() - float(g["l0"])) < 0.05
    for got, key in ((X.grad, "dx"), (G.grad, "dgate"), (K.grad, "dup"), (V.grad, "ddown")):
        assert rel_l2(got, torch.from_numpy(g[key])) < REL_GRAD, key


def test_autocast_and_fp32_master_weights():
    """The caller holds fp32 parameters and runs under autocast, as SparseMLP.forward does
    (custom_models/sparse_models.py:380-388)."""
    d, h = 512, 1024
    ffn = synthetic.make_ffn(d, h, seed=31, density=0.05, dtype=torch.float32)
    x = synthetic.make_tokens(40, d, seed=32, dtype=torch.float32).reshape(2, 20, d)
    X = x.to(DEV).requires_grad_(True)
    G, K, V = (t.to(DEV).requires_grad_(True) for t in (ffn.gate, ffn.up, ffn.down))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        outs, l0, l1, _, _, _ = torch.ops.sparse_ops.ff_forward_gated(X, G, K, V)
    (outs.float().square().sum() + 1e-3 * l1).backward()
    assert outs.dtype == torch.bfloat16
    assert G.grad.dtype == torch.float32 and G.grad.shape == G.shape
    assert torch.isfinite(X.grad).all() and X.grad.abs().sum() > 0


def test_direct_api_returns_hybrid_containers_and_knobs_change_slab_width():
    d, h = 256, 1024
    ffn = synthetic.make_ffn(d, h, seed=33, density=0.05, device=DEV)
    x = synthetic.make_tokens(16, d, seed=34, device=DEV).reshape(1, 16, d)
    out, l0, l1, P, R, T = sparse_ops.ff_forward_gated(x, ffn.gate, ffn.up, ffn.down)
    assert isinstance(P, sparse_ops.HybridSp) and P.cf == 4 and P.slab.shape == (16, 4 * 64)
    assert int(P.overflow_count_tensor().item()) == 0
    torch.ops.sparse_ops_config.set_ell_width_regular(512)   # 127 entries per tile
    out2, *_rest = sparse_ops.ff_forward_gated(x, ffn.gate, ffn.up, ffn.down)
    assert _rest[2].cf == 2 and _rest[2].slab.shape == (16, 4 * 128)
    assert torch.equal(out, out2)
    torch.ops.sparse_ops_config.set_ell_width_regular(128)
    torch.ops.sparse_ops_perf.reset_stats()
    torch.ops.sparse_ops_perf.print_report()


def test_ell_spmm_raw_matches_torch():
    m, k, n, stride = 37, 300, 256, 24
    gen = torch.Generator().manual_seed(5)
    counts = torch.randint(0, stride + 1, (m,), generator=gen, dtype=torch.int32)
    counts[3] = 0
    cols = torch.randint(0, k, (m, stride), generator=gen).to(torch.int16)
    vals = torch.randn(m, stride, generator=gen).to(torch.bfloat16)
    B = torch.randn(k, n, generator=gen).to(torch.bfloat16)
    thr = 20
    ref = torch.zeros(m, n)
    for r in range(m):
        c = int(counts[r])
        if 0 < c <= thr:
            ref[r] = (vals[r, :c].float()[:, None] * B[cols[r, :c].long()].float()).sum(0)
    got = torch.ops.sparse_ops.ell_spmm_raw(vals.to(DEV), cols.to(DEV), counts.to(DEV), B.to(DEV),
                                            m, k, n, stride, thr)
    assert got.shape == (m, n)
    assert torch.allclose(got.float().cpu(), ref, rtol=2e-2, atol=2e-2)
    assert got[3].abs().sum() == 0


def test_bad_inputs_raise():
    d, h = 256, 512
    x = torch.zeros(1, 4, d, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(h, d, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(Exception):
        torch.ops.sparse_ops.ff_forward_gated(x.float(), w, w, w)
    with pytest.raises(Exception):
        torch.ops.sparse_ops.ff_forward_gated(x[0], w, w, w)
    with pytest.raises(Exception):
        torch.ops.sparse_ops.ff_forward_gated(x, w, w[:256], w)


def _mixed_density_case(b, s, d, h, dense_fraction=0.05):
    """Tokens at about 3 % gate density, ``dense_fraction`` of them at 20-40 % (their feature
    0, which carries the gate shift, is scaled down): the prefill mix of the kernel-3 route."""
    ffn = synthetic.make_ffn(d, h, seed=41, density=0.03, skew_sigma=0.5)
    x = synthetic.make_tokens(b * s, d, seed=42)
    gen = torch.Generator().manual_seed(43)
    dense_rows = torch.rand(b * s, generator=gen) < dense_fraction
    dense_rows[0] = True
    scale = 0.12 + 0.28 * torch.rand(b * s, generator=gen)
    x[dense_rows, 0] = (x[dense_rows, 0].float() * scale[dense_rows]).to(x.dtype)
    gout = synthetic.make_tokens(b * s, d, seed=44, fold_bias=False).reshape(b, s, d)
    return ffn, x.reshape(b, s, d), gout, dense_rows


@pytest.mark.parametrize("adaptive", [False, True])
def test_dense_tail_keeps_overflowed_rows_exact(wgrad_mode, adaptive):
    """5 % of the tokens fire 20-40 % of the neurons: far more than a slab holds.  With the
    dense tail (discard_overflow = 0, the default) nothing is dropped and outputs, l0, l1 and
    all four gradients meet the usual tolerances against fp32 autograd
    (custom_op.cpp:79-116, hybrid_sp.cu:811-952, :1358-1383)."""
    b, s, d, h = 2, 320, 512, 2048
    ffn, x, gout, dense_rows = _mixed_density_case(b, s, d, h)
    coeff = 0.05
    ref = dense_reference(x, ffn.gate, ffn.up, ffn.down, gout, coeff)
    sparse_ops.set_tail_rows_adaptive(adaptive)
    try:
        for step in range(3 if adaptive else 1):  # adaptive: later calls size the tail from earlier ones
            X = x.to(DEV).requires_grad_(True)
            G, K, V = (t.to(DEV).requires_grad_(True) for t in (ffn.gate, ffn.up, ffn.down))
            if step:
                torch.cuda.synchronize()  # let the count read-back of the previous call land
            out, l0, l1, P, R, T = torch.ops.sparse_ops.ff_forward_gated(X, G, K, V)
            ((out.float() * gout.to(DEV).float()).sum() + coeff * l1).backward()
            torch.cuda.synchronize()
            with torch.no_grad():
                direct = sparse_ops.ff_forward_gated(X.detach(), G.detach(), K.detach(), V.detach())
            assert int(direct[3].overflow_count_tensor().item()) == 0
            flagged = (P.view(b * s, h // 256, -1)[:, :, 0] < 0).any(dim=1).cpu()
            assert flagged.sum() >= dense_rows.sum() * 0.9 and flagged.sum() < 0.2 * b * s
            assert rel_l2(out, ref[0]) < REL_OUT
            assert abs(l0.item() - ref[1].item()) <= 0.02 * ref[1].item() + 0.05
            assert abs(l1.item() - ref[2].item()) <= 1e-2 * abs(ref[2].item())
            for got, want, name in ((X.grad, ref[3], "dX"), (G.grad, ref[4], "dG"),
                                    (K.grad, ref[5], "dK"), (V.grad, ref[6], "dV")):
                assert rel_l2(got, want) < REL_GRAD, (name, step, rel_l2(got, want))
    finally:
        sparse_ops.set_tail_rows_adaptive(False)


def test_discard_mode_drops_and_counts_what_the_tail_would_keep():
    """set_discard_overflow(1) (custom_op.cpp:92-97): no tail, entries past a tile's capacity
    are lost and counted; set_tail_rows_regular(0) behaves the same; a capacity below the
    number of overflowed rows keeps the first rows exact and counts the rest."""
    b, s, d, h = 2, 320, 512, 2048
    ffn, x, gout, dense_rows = _mixed_density_case(b, s, d, h)
    ref_out = dense_reference(x, ffn.gate, ffn.up, ffn.down, gout, 0.0)[0]
    X, G, K, V = (t.to(DEV) for t in (x, ffn.gate, ffn.up, ffn.down))
    cfg = torch.ops.sparse_ops_config
    try:
        out, *_, P, _, _ = sparse_ops.ff_forward_gated(X, G, K, V)
        assert int(P.overflow_count_tensor().item()) == 0 and rel_l2(out, ref_out) < REL_OUT
        cfg.set_discard_overflow(1)
        out, *_, P, _, _ = sparse_ops.ff_forward_gated(X, G, K, V)
        dropped_all = int(P.overflow_count_tensor().item())
        assert dropped_all > 0 and rel_l2(out, ref_out) > 5 * REL_OUT
        assert not bool((P.slab.view(b * s, h // 256, -1)[:, :, 0] < 0).any())
        cfg.set_discard_overflow(0)
        cfg.set_tail_rows_regular(0)
        out, *_, P, _, _ = sparse_ops.ff_forward_gated(X, G, K, V)
        assert int(P.overflow_count_tensor().item()) == dropped_all
        cfg.set_tail_rows_regular(8)  # fewer rows than overflowed
        out, *_, P, _, _ = sparse_ops.ff_forward_gated(X, G, K, V)
        some = int(P.overflow_count_tensor().item())
        assert 0 < some < dropped_all
    finally:
        cfg.set_discard_overflow(0)
        cfg.set_tail_rows_regular(2048)


def test_adaptive_tail_costs_nothing_until_overflow_appears_then_catches_up():
    """Adaptive sizing: while no call has seen an overflowed row there is no tail; the first
    call that meets overflow rows leaves them on their slab prefix (counted), the next one has
    a tail and is exact again."""
    b, s, d, h = 2, 320, 512, 2048
    ffn, x_mixed, gout, _ = _mixed_density_case(b, s, d, h)
    x_sparse = synthetic.make_tokens(b * s, d, seed=45).reshape(b, s, d)   # ~3 % everywhere
    ref_mixed = dense_reference(x_mixed, ffn.gate, ffn.up, ffn.down, gout, 0.0)[0]
    G, K, V = (t.to(DEV) for t in (ffn.gate, ffn.up, ffn.down))   # one gate tensor = one history
    sparse_ops.set_tail_rows_adaptive(True)
    try:
        for _ in range(3):
            out, *_, P, _, _ = sparse_ops.ff_forward_gated(x_sparse.to(DEV), G, K, V)
            torch.cuda.synchronize()
            assert int(P.overflow_count_tensor().item()) == 0
        assert not bool((P.slab.view(b * s, h // 256, -1)[:, :, 0] < 0).any())
        out, *_, P, _, _ = sparse_ops.ff_forward_gated(x_mixed.to(DEV), G, K, V)
        torch.cuda.synchronize()
        assert int(P.overflow_count_tensor().item()) > 0          # the one lossy call
        out, *_, P, _, _ = sparse_ops.ff_forward_gated(x_mixed.to(DEV), G, K, V)
        torch.cuda.synchronize()
        assert int(P.overflow_count_tensor().item()) == 0 and rel_l2(out, ref_mixed) < REL_OUT
    finally:
        sparse_ops.set_tail_rows_adaptive(False)
