"""Dead-neuron bookkeeping of the fused operator on the GPU: the per-neuron activity kernel
against the oracle's count over the same slabs (bit-exact), and the tracker's
``record_pattern`` against ``record_activations`` on the dense activation."""
import numpy as np
import pytest
import torch

from oracle import ffn_oracle as fo
from oracle import twell_format as tf
from sparser_faster_llms_b200 import _lib, sparse_ops, synthetic, tracking
from sparser_faster_llms_b200.sparse_ops_loader import load_sparse_ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def ops():
    load_sparse_ops()
    yield
    torch.ops.sparse_ops_config.set_ell_width_regular(128)


def forward(b, s, d, h, density, seed, dead=(), zero_up=()):
    ffn = synthetic.make_ffn(d, h, seed=seed, density=density, skew_sigma=0.5)
    gate, up = ffn.gate.clone(), ffn.up.clone()
    for j in dead:
        gate[j] = 0                 # relu(0) = 0: never in the pattern
    for j in zero_up:
        up[j] = 0                   # in the pattern, but h = relu(gate) * 0 = 0
    x = synthetic.make_tokens(b * s, d, seed=seed + 1).reshape(b, s, d)
    out = torch.ops.sparse_ops.ff_forward_gated(x.to(DEV), gate.to(DEV), up.to(DEV),
                                                ffn.down.to(DEV))
    return out


@pytest.mark.parametrize("width", [64, 128, 256])      # slab compression factor 8, 4, 2
@pytest.mark.parametrize("b,s,d,h,density", [(2, 12, 256, 512, 0.06), (4, 160, 512, 2048, 0.03),
                                            (1, 33, 512, 1024, 0.10)])
def test_activity_matches_the_oracle_on_the_same_slabs(b, s, d, h, density, width):
    torch.ops.sparse_ops_config.set_ell_width_regular(width)
    cf = sparse_ops.compression_factor()
    dead, zero_up = range(0, 40), range(300, 340)
    _, l0, _, P, _, T = forward(b, s, d, h, density, 31, dead, zero_up)
    m = b * s
    p_np, t_np = P.cpu().numpy().view(np.uint32), T.cpu().numpy().view(np.uint32)
    for vals, vals_np in ((T, t_np), (None, None)):
        want = fo.slab_active_rows(p_np, vals_np, h, cf)
        last = torch.arange(h, dtype=torch.int64, device=DEV)
        got = sparse_ops.neuron_activity(P, vals, last_activated=last, microbatch_tokens=m)
        assert got.dtype == torch.int32 and np.array_equal(got.cpu().numpy(), want)
        want_last = np.where(want > 0, 0, np.arange(h) + m)
        assert np.array_equal(last.cpu().numpy(), want_last)
    act = sparse_ops.neuron_activity(P, T).cpu().numpy()
    assert act[:40].sum() == 0 and act[300:340].sum() == 0
    pat = sparse_ops.neuron_activity(P).cpu().numpy()
    assert pat[300:340].sum() > 0                      # in the pattern, zero in T
    # the forward's l0 counts pattern entries per token; so does the activity of P
    counts = tf.slab_counts(p_np, cf)
    counts = np.where(counts >= 2 ** 31, 0, counts)    # rows the dense tail took: sign bit set
    stored = counts.clip(max=256 // cf - 1).sum()
    assert pat.sum() == stored


def test_record_pattern_equals_record_activations_on_the_dense_activation(ref_models):
    torch.ops.sparse_ops_config.set_ell_width_regular(128)
    cf = sparse_ops.compression_factor()
    b, s, d, h = 2, 64, 512, 1024
    make = lambda: ref_models.SparsityTracker(train_batch_size=8, max_seq_len=s,  # noqa: E731
                                              per_device_train_batch_size=b,
                                              tokens_until_dead=2 * b * s)
    fused, dense = make(), make()
    for step in range(4):
        # from step 1 on, neurons 0..199 stop firing and die two steps later
        _, l0, l1, P, _, T = forward(b, s, d, h, 0.04, 50 + step,
                                     dead=range(200) if step else ())
        h_abs = torch.from_numpy(np.abs(tf.unpack_to_dense(
            T.cpu().numpy().view(np.uint32), h, cf))).reshape(b, s, h)
        fused.start_forward_pass()
        dense.start_forward_pass()
        tracking.record_pattern(fused, 0, l0, l1, P, T)
        dense.record_activations(0, h_abs.to(DEV))
        l1_f, stats_f = fused.finalize_forward_pass()
        l1_d, stats_d = dense.finalize_forward_pass()
        assert torch.equal(fused._last_activated[0], dense._last_activated[0])
        assert torch.equal(fused.get_alive_neurons()[0], dense.get_alive_neurons()[0])
        assert float(stats_f["activation_alive/mean"]) == float(stats_d["activation_alive/mean"])
        assert float(l1_f) == pytest.approx(float(l1_d), rel=2e-2)
    assert int(fused.get_alive_neurons()[0][:200].sum()) == 0
    assert int(fused.get_alive_neurons()[0].sum()) > 0


def test_patched_module_keeps_counters_live_through_forward_and_backward(ref_models):
    """A module with the reference SparseMLP's attributes (kernel-layout weights, tracker,
    layer_idx; custom_models/sparse_models.py:262-395), patched: the fused training branch
    runs under autograd and ages / revives the counters."""
    torch.ops.sparse_ops_config.set_ell_width_regular(128)
    d, h, b, s = 256, 512, 2, 32
    ffn = synthetic.make_ffn(d, h, seed=9, density=0.05)

    class Mlp(torch.nn.Module):
        def __init__(self, tracker):
            super().__init__()
            lin = lambda w: torch.nn.Linear(w.shape[1], w.shape[0], bias=False)  # noqa: E731
            self.gate_proj, self.up_proj, self.down_proj = lin(ffn.gate), lin(ffn.up), lin(ffn.down)
            for m, w in ((self.gate_proj, ffn.gate), (self.up_proj, ffn.up), (self.down_proj, ffn.down)):
                m.weight.data = w.clone()
            with torch.no_grad():
                self.gate_proj.weight[:50] = 0                  # neurons 0..49 never fire
            self.tracker, self.layer_idx, self.intermediate_size = tracker, 0, h
            self._training_mode, self._use_fast, self.gated = True, True, True

        def forward(self, x):
            raise AssertionError("the fused branch must not reach the module's own forward")

    tr = ref_models.SparsityTracker(train_batch_size=b, max_seq_len=s,
                                    per_device_train_batch_size=b, tokens_until_dead=b * s)
    mlp = Mlp(tr).to(DEV).to(torch.bfloat16)
    tracking.enable_live_dead_neuron_tracking(mlp)
    for step in range(2):
        x = synthetic.make_tokens(b * s, d, seed=60 + step).reshape(b, s, d).to(DEV).requires_grad_(True)
        tr.start_forward_pass()
        out = mlp(x)
        l1, stats = tr.finalize_forward_pass()
        (out.float().sum() + 0.01 * l1).backward()
        assert x.grad is not None and mlp.gate_proj.weight.grad is not None
        assert int(tr._last_activated[0][:50].min()) == (step + 1) * b * s
    alive = tr.get_alive_neurons()[0]
    assert int(alive[:50].sum()) == 0 and int(alive.sum()) > 0
    assert float(stats["activation_l0/mean"]) > 0


def test_hybridsp_wrappers_empty_input_and_argument_errors():
    torch.ops.sparse_ops_config.set_ell_width_regular(128)
    ffn = synthetic.make_ffn(256, 512, seed=3, density=0.05)
    x = synthetic.make_tokens(16, 256, seed=4).reshape(1, 16, 256)
    _, _, _, P, _, T = sparse_ops.ff_forward_gated(x.to(DEV), ffn.gate.to(DEV), ffn.up.to(DEV),
                                                   ffn.down.to(DEV))
    a = sparse_ops.neuron_activity(P, T)
    assert torch.equal(a, sparse_ops.neuron_activity(P.slab, T.slab))
    empty = torch.empty((0, P.slab.shape[1]), dtype=torch.int32, device=DEV)
    last = torch.full((512,), 7, dtype=torch.int64, device=DEV)
    z = sparse_ops.neuron_activity(empty, None, last_activated=last, microbatch_tokens=5, width=512)
    assert int(z.sum()) == 0 and bool((last == 12).all())
    with pytest.raises(ValueError, match="last_activated"):
        sparse_ops.neuron_activity(P, T, last_activated=last.to(torch.int32))
    with pytest.raises(ValueError, match="shape"):
        sparse_ops.neuron_activity(P.slab, T.slab[:, :-1])
    with pytest.raises(RuntimeError, match="CUDA"):
        sparse_ops.neuron_activity(P.slab.cpu())
    lib = _lib.load_library()
    rc = lib.b200_hybrid_neuron_activity(P.slab.data_ptr(), None, 16, 500, 4, 0,
                                         a.data_ptr(), None, None)
    assert rc == -4 and b"multiple of 256" in lib.b200_last_error()
    rc = lib.b200_hybrid_neuron_activity(P.slab.data_ptr(), None, 16, 512, 4, 0, None, None, None)
    assert rc == -2
