"""Reference-compatible Python surface: names, parameters, defaults, error rules (CPU)."""
import inspect
import json
import os
import sys
from pathlib import Path

import pytest
import torch

from sparser_faster_llms_b200 import dropin, twell

GOLDEN = Path(__file__).resolve().parent / "golden" / "twell_signatures.json"
# A checkout of the reference next to this repository (or named by SPARSER_REFERENCE_ROOT);
# the tests that run the reference's own code are skipped where it is absent.
REFERENCE = Path(os.environ.get("SPARSER_REFERENCE_ROOT",
                                Path(__file__).resolve().parents[2] / "reference"))


def test_public_api_matches_reference_signatures():
    sigs = json.loads(GOLDEN.read_text())
    assert twell.sparse_algorithms() == sigs.pop("sparse_algorithms()")
    for name, want in sigs.items():
        if name.endswith(".methods"):
            cls = getattr(twell, name[:-len(".methods")])
            have = {m for m in dir(cls) if not m.startswith("__")}
            # the public methods are the contract; the reference's private dispatch helpers
            # (_forward_shared, _select_forward_impl, ...) are its own implementation detail
            missing = [m for m in want if m not in have and not m.startswith("_")]
            assert not missing, (name, missing)
            continue
        obj = getattr(twell, name)
        target = obj.__init__ if inspect.isclass(obj) else obj
        have = [[p.name, p.kind.name,
                 None if p.default is inspect.Parameter.empty else repr(p.default)]
                for p in inspect.signature(target).parameters.values() if p.name != "self"]
        assert have == want, name


def test_attributes_the_reference_benchmark_pokes_exist():
    for attr in ("CUDA_HOME", "load", "_BASE_DIR", "_DEFAULT_EXT_NAME", "_EXT_CACHE",
                 "ALGORITHM_SPECS", "_validate_algorithms", "_resolve_algorithms_with_deps"):
        assert hasattr(twell, attr), attr
    assert twell._resolve_algorithms_with_deps(["twell_mlp"])[-1] == "twell_mlp"
    with pytest.raises(ValueError):
        twell._validate_algorithms(["nope"])


def test_validation_rules_of_the_reference_wrappers():
    w = torch.zeros(256, 256, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="compression_factor must be one of"):
        twell.TwELLGatedMLP(0, w, w, w, compression_factor=3)
    with pytest.raises(ValueError, match="requires flex_kernels=True"):
        twell.TwELLGatedMLP(0, w, w, w, compression_factor=4)
    with pytest.raises(ValueError, match="Only compression_factor=8"):
        twell.TwELLMLP(0, w, w, compression_factor=4)
    with pytest.raises(ValueError, match="Only compression_factor=8"):
        twell.T2DLinear(w, compression_factor=2)
    with pytest.raises(ValueError):
        twell.GatedT2DLinear(w, w, compression_factor=2)
    twell.GatedT2DLinear(w, w, compression_factor=2, flex_kernels=True)


def test_module_built_on_cpu_registers_buffers_and_defers_cuda_state():
    g = torch.randn(512, 256)
    mod = twell.TwELLGatedMLP(layer_number=3, GATE=g, UP=g.clone(), DOWN=g.clone())
    assert mod.layer is None
    assert set(mod.state_dict()) == {"GATE", "UP", "DOWN"}
    with pytest.raises(RuntimeError, match="must be moved to CUDA"):
        mod(torch.zeros(2, 256))
    mod.destroy()


def test_dropin_registers_module_names():
    dropin.install(sparse_ops=False)
    assert sys.modules[dropin.TWELL_NAME] is twell
    import importlib
    assert importlib.import_module("custom_models.twell_modules.twell") is twell
    dropin.uninstall()


@pytest.mark.skipif(not (REFERENCE / "custom_models").exists(),
                    reason="reference checkout not present on this machine")
def test_reference_swap_hook_builds_our_modules():
    """The reference's own replace_mlp_modules(convert_sparse_mlp_to_twell_fused), unchanged."""
    saved = {k: v for k, v in sys.modules.items() if k.startswith("custom_models")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, str(REFERENCE))
    try:
        dropin.install(sparse_ops=False)
        from custom_models.sparse_models import SparseLlamaConfig, SparseLlamaForCausalLM
        from custom_models.sparse_testing_utils import (convert_sparse_mlp_to_twell_fused,
                                                        sparse_to_twell_state_dict)
        cfg = SparseLlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                num_attention_heads=4, num_key_value_heads=4, vocab_size=128,
                                max_position_embeddings=64)
        model = SparseLlamaForCausalLM(cfg)
        sd = sparse_to_twell_state_dict(model.state_dict())
        model.replace_mlp_modules(convert_sparse_mlp_to_twell_fused)
        mlps = [layer.mlp for layer in model.model.layers]
        assert all(isinstance(m, twell.TwELLGatedMLP) for m in mlps)
        assert mlps[0].DOWN.shape == (512, 256)
        keys = set(model.state_dict())
        assert "model.layers.0.mlp.GATE" in keys and "model.layers.1.mlp.DOWN" in keys
        model.load_state_dict(sd, strict=False)
    finally:
        sys.path.remove(str(REFERENCE))
        dropin.uninstall()
        for k in [k for k in sys.modules if k.startswith("custom_models")]:
            del sys.modules[k]
        sys.modules.update(saved)
