"""State-dict conversions against fixtures produced by the reference's own functions
(custom_models/sparse_testing_utils.py:182-207; generator: tests/golden/make_golden.py
--only-state-dicts), plus the d_ff shard slicing."""
import importlib.util
import json
from pathlib import Path

import pytest
import torch

from sparser_faster_llms_b200 import checkpoint, sharded

GOLDEN = Path(__file__).parent / "golden"


def _generator_module():
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_conversions_match_the_reference_outputs():
    gen = _generator_module()
    golden = json.loads((GOLDEN / "state_dict_conversions.json").read_text())
    digest = lambda sd: {k: [list(v.shape), gen.sha(v)] for k, v in sd.items()}  # noqa: E731
    for name, (sd, gated) in gen.state_dict_inputs().items():
        assert digest(checkpoint.sparse_to_hf_state_dict(sd, gated=gated)) == golden[name]["hf"], name
        assert digest(checkpoint.sparse_to_twell_state_dict(sd, gated=gated)) == golden[name]["twell"], name
        assert digest(checkpoint.sparse_to_hf_state_dict(sd, drop_auxiliary=False, gated=gated)) \
            == golden[name]["hf_keep_aux"], name


def test_gate_keys_are_rejected_when_not_gated():
    sd = {"mlp.gate_proj.weight": torch.zeros(4, 2)}
    with pytest.raises(ValueError):
        checkpoint.sparse_to_twell_state_dict(sd, gated=False)
    with pytest.raises(ValueError):
        checkpoint.sparse_to_hf_state_dict({"mlp.GATE": torch.zeros(4, 2)}, gated=False)


def test_round_trip_hf_twell_hf_is_exact():
    gen = _generator_module()
    sd, _ = gen.state_dict_inputs()["gated_hf"]
    hf = checkpoint.sparse_to_hf_state_dict(sd)
    back = checkpoint.sparse_to_hf_state_dict(checkpoint.sparse_to_twell_state_dict(hf))
    assert back.keys() == hf.keys()
    for k in hf:
        assert torch.equal(back[k], hf[k])


@pytest.mark.parametrize("world", [2, 3, 8])
def test_shard_and_merge_twell_state_dict(world):
    g = torch.Generator().manual_seed(5)
    h, d = 11008, 8
    sd = {"l0.mlp.GATE": torch.randn(h, d, generator=g), "l0.mlp.UP": torch.randn(h, d, generator=g),
          "l0.mlp.DOWN": torch.randn(h, d, generator=g), "l0.norm.weight": torch.randn(d, generator=g)}
    shards = [checkpoint.shard_twell_state_dict(sd, r, world) for r in range(world)]
    for r, s in enumerate(shards):
        h0, h1 = sharded.shard_range(h, r, world)
        assert s["l0.mlp.GATE"].shape == (h1 - h0, d) and (h1 - h0) % 256 == 0
        assert torch.equal(s["l0.mlp.DOWN"], sd["l0.mlp.DOWN"][h0:h1])
        assert s["l0.norm.weight"] is sd["l0.norm.weight"]
    merged = checkpoint.merge_twell_shards(shards)
    for k in sd:
        assert torch.equal(merged[k], sd[k])


def test_hybrid_down_proj_is_retransposed_once():
    from types import SimpleNamespace
    from torch import nn
    d, h = 4, 12

    def layer():
        mlp = nn.Module()
        mlp.down_proj = nn.Linear(h, d, bias=False)   # HF layout: weight [D, H]
        return SimpleNamespace(mlp=mlp)

    model = SimpleNamespace(config=SimpleNamespace(sparsity_use_hybrid_kernel=True, hidden_size=d),
                            model=SimpleNamespace(layers=[layer(), layer()]))
    before = [l.mlp.down_proj.weight.data.clone() for l in model.model.layers]
    assert checkpoint.retranspose_hybrid_down_proj(model) == 2
    for l, w in zip(model.model.layers, before):
        assert torch.equal(l.mlp.down_proj.weight.data, w.t())
    assert checkpoint.retranspose_hybrid_down_proj(model) == 0  # already [H, D]
    model.config.sparsity_use_hybrid_kernel = False
    assert checkpoint.retranspose_hybrid_down_proj(model) == 0
