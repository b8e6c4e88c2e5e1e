"""The CPU oracle against fixtures produced by the reference's torch path
(tests/golden/make_golden.py).  Runs without a GPU."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import ffn_oracle as fo
from oracle import twell_format as tf
from sparser_faster_llms_b200 import synthetic


def from_bits(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def sha(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.to(torch.bfloat16).view(torch.int16).numpy().tobytes())
    return h.hexdigest()


@pytest.fixture(scope="module")
def small(golden_dir):
    g = np.load(golden_dir / "small_gated.npz")
    return {k: g[k] for k in g.files}


def test_dense_oracle_matches_reference_sparse_mlp(small):
    x, gate, up, down = (from_bits(small[k]) for k in ("x", "gate", "up", "down"))
    y = fo.dense_ffn(x, gate, up, down)
    ref = torch.from_numpy(small["y_fp32"])
    max_abs, rel = fo.max_abs_and_rel_l2(y, ref)
    assert rel < 1e-6, (max_abs, rel)


@pytest.mark.parametrize("cf", [8, 4, 2])
def test_pack_decodes_like_reference_packed_to_dense(small, cf):
    x, gate = from_bits(small["x"]), from_bits(small["gate"])
    h = gate.shape[0]
    packed = fo.pack_gate(x, gate, None, cf)
    if int(small[f"ref_raises_cf{cf}"]):
        with pytest.raises(ValueError):
            tf.unpack_to_dense(packed, h, cf)
        return
    ours = tf.f32_to_bf16_bits(tf.unpack_to_dense(packed, h, cf))
    assert np.array_equal(ours, small[f"ref_dense_cf{cf}"])
    # and the decoded slab is relu(z) rounded to bf16
    z = fo.gate_preactivation(x, gate)
    want = tf.f32_to_bf16_bits(torch.relu(z).numpy())
    assert np.array_equal(ours, want)


@pytest.mark.parametrize("hp", [False, True])
def test_contraction_oracle_close_to_reference(small, hp):
    x, gate, up, down = (from_bits(small[k]) for k in ("x", "gate", "up", "down"))
    y, packed = fo.gated_mlp(x, gate, up, down, highest_precision=hp, compression_factor=2)
    ref = torch.from_numpy(small["y_fp32"])
    max_abs, rel = fo.max_abs_and_rel_l2(y, ref)
    # mixed mode rounds every product and h to bf16: relative L2 ~ 2^-8
    assert rel < (3e-3 if hp else 1.2e-2), (max_abs, rel)
    # the reference's own bf16 torch run is no closer to fp32 than that
    _, rel_torch = fo.max_abs_and_rel_l2(torch.from_numpy(small["y_bf16_torch"]), ref)
    assert rel_torch < 2e-2


def test_training_statistics_and_gradients(golden_dir):
    g = np.load(golden_dir / "training_gated.npz")
    b, s, d, h = (int(g[k]) for k in ("b", "s", "d", "h"))
    ffn = synthetic.make_ffn(d, h, seed=int(g["seed_ffn"]), density=0.06, skew_sigma=0.5)
    x = synthetic.make_tokens(b * s, d, seed=int(g["seed_x"])).float()
    gout = synthetic.make_tokens(b * s, d, seed=int(g["seed_gout"]), fold_bias=False).float()
    assert sha(x, ffn.gate, ffn.up, ffn.down) == str(g["input_sha"])
    gate, up, down = (t.float().requires_grad_(True) for t in (ffn.gate, ffn.up, ffn.down))
    x = x.requires_grad_(True)
    hid = torch.relu(x @ gate.T) * (x @ up.T)
    y = hid @ down
    l0, l1 = fo.l0_l1(hid.abs())
    (((y * gout).sum()) + float(g["coeff"]) * l1).backward()
    assert torch.allclose(y.detach(), torch.from_numpy(g["y"]).reshape(-1, d), rtol=1e-5, atol=1e-6)
    assert abs(float(l1) - float(g["l1"])) < 1e-5 * max(1.0, abs(float(g["l1"])))
    assert abs(float(l0) - float(g["l0"])) < 1e-4
    for ours, key in ((x.grad, "dx"), (gate.grad, "dgate"), (up.grad, "dup"), (down.grad, "ddown")):
        ref = torch.from_numpy(g[key]).reshape(ours.shape)
        assert torch.allclose(ours, ref, rtol=1e-4, atol=1e-6), key


def test_config1_outputs_and_counts(golden_dir):
    g = np.load(golden_dir / "config1_gated.npz")
    m, d, h = int(g["m"]), int(g["d"]), int(g["h"])
    gen = torch.Generator().manual_seed(int(g["seed"]))
    x = torch.randn(m, d, generator=gen)
    gate = (torch.randn(h, d, generator=gen) * 0.02).to(torch.bfloat16)
    up = (torch.randn(h, d, generator=gen) * 0.02).to(torch.bfloat16)
    down = (torch.randn(h, d, generator=gen) * 0.02).to(torch.bfloat16)
    x = x.to(torch.bfloat16)
    assert sha(x, gate, up, down) == str(g["input_sha"])
    bias = torch.full((h,), float(g["shift"]))
    y = fo.dense_ffn(x, gate, up, down, bias)
    assert torch.allclose(y[:32], torch.from_numpy(g["y_rows"]), rtol=1e-4, atol=1e-6)
    assert abs(float(y.double().norm()) - float(g["y_norm"])) < 1e-4 * float(g["y_norm"])
    packed = fo.pack_gate(x, gate, bias, 2)
    assert np.array_equal(tf.slab_counts(packed, 2), g["counts"].astype(np.int64))
    assert 0.015 < float(g["density"]) < 0.025
