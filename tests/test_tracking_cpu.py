"""Sparsity bookkeeping on CPU: the oracle's l0 / l1 / dead-neuron update (and the staged
reference SparsityTracker itself) against vectors generated from the reference's tracker
(custom_models/sparse_models.py:95-256; generator: tests/golden/make_golden.py
--only-tracker), the patch helpers, and the oracle's slab-level activity count against the
dense definition."""
import contextlib
import importlib.util
import io
import json
import os
import sys
import types
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import ffn_oracle as fo
from oracle import twell_format as tf
from sparser_faster_llms_b200 import tracking

GOLDEN = Path(__file__).resolve().parent / "golden"


def _generator():
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    return gen


def test_oracle_and_reference_tracker_reproduce_the_golden_vectors(monkeypatch, ref_models):
    monkeypatch.delenv("WORLD_SIZE", raising=False)
    gen = _generator()
    golden = json.loads((GOLDEN / "sparsity_tracker.json").read_text())
    with contextlib.redirect_stdout(io.StringIO()):
        tr = ref_models.SparsityTracker(**gen.TRACKER_ARGS)
    shadow = None
    for layers, want in zip(gen.tracker_inputs(), golden, strict=True):
        if shadow is None:
            shadow = [torch.zeros(h.shape[-1], dtype=torch.int64) for h in layers]
        tr.start_forward_pass()
        l1s = []
        for i, h in enumerate(layers):
            tr.record_activations(layer_idx=i, absolute_activations=h)
            _, shadow[i] = fo.last_activated_update(h, shadow[i], tr._microbatch_tokens)
            l1s.append(fo.l0_l1(h)[1])
        l1, stats = tr.finalize_forward_pass()
        assert float(l1) == pytest.approx(want["l1"], rel=1e-6)
        assert float(torch.stack(l1s).mean()) == pytest.approx(want["l1"], rel=1e-6)
        assert {k: float(v) for k, v in stats.items()} == pytest.approx(want["stats"], rel=1e-6)
        for i in range(len(layers)):
            assert tr._last_activated[i].tolist() == want["last_activated"][i]
            assert shadow[i].tolist() == want["last_activated"][i]  # the oracle agrees too
        assert [int(a.sum()) for a in tr.get_alive_neurons()] == want["alive"]


class _FakeSparseMLP(torch.nn.Module):
    """The attributes of the reference's SparseMLP that the patch reads
    (custom_models/sparse_models.py:262-395)."""

    def __init__(self):
        super().__init__()
        self._training_mode, self._use_fast, self.gated = True, True, True
        self.calls = []

    def forward(self, hidden_states):
        self.calls.append("own")
        return hidden_states + 1


def test_live_tracking_patch_routes_only_the_fused_training_branch(monkeypatch):
    seen = []
    monkeypatch.setattr(tracking, "fused_training_forward",
                        lambda mlp, x: (seen.append(mlp), x * 2)[1])
    mlp = _FakeSparseMLP()
    x = torch.ones(2)
    tracking.enable_live_dead_neuron_tracking(mlp)
    tracking.enable_live_dead_neuron_tracking(mlp)          # idempotent
    assert torch.equal(mlp(x), x * 2) and seen == [mlp] and mlp.calls == []
    for attr in ("_use_fast", "_training_mode", "gated"):
        setattr(mlp, attr, False)
        assert torch.equal(mlp(x), x + 1)                   # the module's own forward
        setattr(mlp, attr, True)
    assert mlp.calls == ["own"] * 3 and len(seen) == 1
    tracking.disable_live_dead_neuron_tracking(mlp)
    tracking.disable_live_dead_neuron_tracking(mlp)
    assert torch.equal(mlp(x), x + 1) and "forward" not in mlp.__dict__


REFERENCE = Path(os.environ.get("SPARSER_REFERENCE_ROOT",
                                Path(__file__).resolve().parents[2] / "reference"))


@pytest.mark.skipif(not (REFERENCE / "custom_models").exists(),
                    reason="reference checkout not present on this machine")
def test_patch_fits_the_reference_sparse_mlp(monkeypatch):
    """The reference's own SparseMLP (custom_models/sparse_models.py:259-410), built with
    use_hybrid_kernel=True over this package's operator loader: the patch takes over the
    fused training branch and leaves the einsum branch to the module."""
    from sparser_faster_llms_b200 import dropin
    saved = {k: v for k, v in sys.modules.items() if k.startswith("custom_models")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, str(REFERENCE))
    try:
        dropin.install()
        from transformers import LlamaConfig
        from custom_models import sparse_models as ref
        with contextlib.redirect_stdout(io.StringIO()):
            tr = ref.SparsityTracker(train_batch_size=2, max_seq_len=8,
                                     per_device_train_batch_size=2, gated=True)
        cfg = LlamaConfig(hidden_size=256, intermediate_size=512, mlp_bias=False)
        mlp = ref.SparseMLP(layer_idx=0, config=cfg, gated=True, tracker=tr,
                            execution_logic="training", use_hybrid_kernel=True)
        assert mlp.down_proj.weight.shape == (512, 256)       # kernel layout [H, D]
        seen = []
        monkeypatch.setattr(tracking, "fused_training_forward",
                            lambda m, x: (seen.append(m), x)[1])
        tracking.enable_live_dead_neuron_tracking(mlp)
        x = torch.randn(2, 8, 256)
        mlp.enable_fast(True)
        assert mlp(x) is x and seen == [mlp]
        mlp.enable_fast(False)                                # einsum branch, reference code
        tr.start_forward_pass()
        y = mlp(x)
        assert y.shape == x.shape and len(seen) == 1 and len(tr._l0_per_layer) == 1
        # the module-level record_pattern accepts the reference's tracker object as it is
        for field in ("active", "register_layer", "_l0_per_layer", "_l1_per_layer",
                      "_last_activated", "_microbatch_tokens"):
            assert hasattr(tr, field), field
        tracking.disable_live_dead_neuron_tracking(mlp)
        assert "forward" not in mlp.__dict__
    finally:
        sys.path.remove(str(REFERENCE))
        dropin.uninstall()
        for k in [k for k in sys.modules if k.startswith("custom_models")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_record_pattern_function_falls_back_for_trackers_without_counters():
    calls = []

    class Plain:
        def record_l0_l1(self, **kw):
            calls.append(kw)

    tracking.record_pattern(Plain(), 3, 1.0, 2.0, P=None, T=None, width=256)
    assert calls == [{"layer_idx": 3, "l0": 1.0, "l1": 2.0, "width": 256}]
    # a tracker with the reference's fields, inactive while grad is enabled: ignored
    tr = types.SimpleNamespace(active=False, _l1_per_layer=[], _l0_per_layer=[],
                               _last_activated={}, _microbatch_tokens=8,
                               register_layer=lambda *a, **k: None)
    tracking.record_pattern(tr, 0, None, None, P=torch.zeros(2, 64, dtype=torch.int32))
    assert tr._l1_per_layer == [] and tr._last_activated == {}


def test_select_fast_layers():
    l0 = [torch.tensor(10.0), torch.tensor(200.0), 99.9]
    assert tracking.select_fast_layers(l0, 100) == [True, False, True]
    assert tracking.select_fast_layers(l0, -1) == [True, True, True]


@pytest.mark.parametrize("cf", [8, 4])
def test_slab_activity_matches_the_dense_definition(cf):
    rng = np.random.default_rng(5)
    m, h = 37, 768
    z = rng.standard_normal((m, h)).astype(np.float32)
    z[rng.random((m, h)) > 0.05] = -1.0          # ~5 % positive: no slab overflows
    z[:, 10:20] = -1.0
    packed = tf.pack_preactivations(z, cf)
    dense = tf.unpack_to_dense(packed, h, cf)
    want = (dense > 0).sum(0).astype(np.int32)
    got = fo.slab_active_rows(packed, None, h, cf)
    assert np.array_equal(got, want) and got[10:20].sum() == 0
    # a values slab with zeros in some stored entries: those entries stop counting
    vals = packed.copy().reshape(m, h // 256, 256 // cf)
    vals[:, :, 1::2] &= 0xFFFF                   # odd slots: value bits cleared (+0)
    vals[:, :, 2::4] = (vals[:, :, 2::4] & 0xFFFF) | (0x8000 << 16)   # -0 is zero as well
    p3 = packed.reshape(vals.shape)
    cnt = np.clip(p3[:, :, 0].astype(np.int64), 0, 256 // cf - 1)
    want2 = np.zeros(h, dtype=np.int32)
    for r in range(m):
        for t in range(h // 256):
            for s in range(1, cnt[r, t] + 1):
                if s % 2 == 0 and s % 4 != 2:
                    want2[p3[r, t, s] & 0xFFFF] += 1
    got2 = fo.slab_active_rows(packed, vals.reshape(packed.shape), h, cf)
    assert np.array_equal(got2, want2)
