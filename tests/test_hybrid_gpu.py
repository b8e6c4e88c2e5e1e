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
