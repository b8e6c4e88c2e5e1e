"""The reference's own callers, unmodified, running on the GPU through this repository's
modules: the MLP swap hook on a SparseLlamaForCausalLM, SparseMLP's fused training branch, and
benchmark_inference.benchmark_model.

The reference's Python files are staged under ``oracle/_ref`` by ``oracle/make_ref.py`` (run
by ``__graft_entry__.build()`` where a checkout of the reference is present); the tests skip
where they are absent.  ``dropin.install()`` registers this repository's ``twell`` module and
operator loader under the names the reference imports.
"""
import sys
import types

import pytest
import torch

from oracle import make_ref
from sparser_faster_llms_b200 import dropin, twell

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not make_ref.available(),
                                 reason="reference callers not staged under oracle/_ref")]
DEV = "cuda:0"


@pytest.fixture()
def reference():
    """Import context: reference callers from oracle/_ref on top of the drop-in modules."""
    saved = {k: v for k, v in sys.modules.items()
             if k.startswith("custom_models") or k in ("benchmark_inference", "benchmark_base",
                                                       "energy_utils")}
    for k in saved:
        del sys.modules[k]
    stubbed = []
    for name in ("matplotlib", "matplotlib.pyplot"):  # energy_utils imports it for a plot helper
        if name not in sys.modules:
            try:
                __import__(name)
            except Exception:
                sys.modules[name] = types.ModuleType(name)
                stubbed.append(name)
    if "matplotlib" in stubbed:
        sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
        sys.modules["matplotlib"].use = lambda *a, **k: None
    sys.path.insert(0, make_ref.import_path())
    dropin.install()
    try:
        yield
    finally:
        sys.path.remove(make_ref.import_path())
        dropin.uninstall()
        for k in [k for k in sys.modules
                  if k.startswith("custom_models") or k in ("benchmark_inference",
                                                            "benchmark_base", "energy_utils")]:
            del sys.modules[k]
        for name in stubbed:
            sys.modules.pop(name, None)
        sys.modules.update(saved)
        twell.destroy_all_d2t_layers()


def tiny_sparse_llama(d=256, h=1024, layers=2, logic="inference", seed=0):
    """Random-init SparseLlamaForCausalLM whose gates fire on about 2 % of the neurons:
    positive embeddings and a small negative mean on the gate weights."""
    from custom_models.sparse_models import SparseLlamaConfig, SparseLlamaForCausalLM
    torch.manual_seed(seed)
    cfg = SparseLlamaConfig(hidden_size=d, intermediate_size=h, num_hidden_layers=layers,
                            num_attention_heads=4, num_key_value_heads=4, vocab_size=128,
                            max_position_embeddings=512, sparsity_mlp_execution_logic=logic,
                            sparsity_train_batch_size=2, sparsity_per_device_train_batch_size=2,
                            sparsity_max_seq_len=128)
    cfg.use_cache = False
    model = SparseLlamaForCausalLM(cfg)
    with torch.no_grad():
        model.model.embed_tokens.weight.copy_(torch.randn(128, d).abs())
        for layer in model.model.layers:
            layer.mlp.gate_proj.weight.copy_(torch.randn(h, d) * 0.02 - 0.82 / d)
    return model


def test_swapped_model_matches_the_reference_torch_path(reference):
    """replace_mlp_modules(convert_sparse_mlp_to_twell_fused) on a tiny model
    (custom_models/sparse_models.py:552-614, sparse_testing_utils.py:10-43): logits of the
    swapped model against the same model on SparseMLP's torch path."""
    import copy

    from custom_models.sparse_testing_utils import convert_sparse_mlp_to_twell_fused
    model = tiny_sparse_llama().eval()
    swapped = copy.deepcopy(model)
    swapped.replace_mlp_modules(convert_sparse_mlp_to_twell_fused)
    assert all(isinstance(l.mlp, twell.TwELLGatedMLP) for l in swapped.model.layers)
    model = model.to(DEV).to(torch.bfloat16)
    swapped = swapped.to(DEV).to(torch.bfloat16)
    gen = torch.Generator().manual_seed(1)
    for shape in ((2, 128), (1, 5)):  # a prefill-sized and a decode-sized call
        ids = torch.randint(0, 128, shape, generator=gen).to(DEV)
        with torch.inference_mode():
            want = model(input_ids=ids).logits.float()
            got = swapped(input_ids=ids).logits.float()
        rel = float((got - want).norm() / want.norm())
        assert rel < 2e-2, (shape, rel)
    # the hidden width of a swapped layer comes from the reference's own linears
    assert swapped.model.layers[0].mlp.DOWN.shape == (1024, 256)


def test_sparse_mlp_fast_branch_trains_one_step(reference):
    """SparseMLP(use_hybrid_kernel=True).enable_fast(True) (sparse_models.py:380-395): output,
    the tracker's l0 / l1 and the four gradients against the module's own einsum branch."""
    from custom_models.sparse_models import SparseLlamaConfig, SparseMLP, SparsityTracker
    d, h, b, s = 512, 2048, 2, 64
    torch.manual_seed(3)
    cfg = SparseLlamaConfig(hidden_size=d, intermediate_size=h, num_hidden_layers=1,
                            num_attention_heads=4, num_key_value_heads=4, vocab_size=64)

    def tracker():
        return SparsityTracker(train_batch_size=b, max_seq_len=s,
                               per_device_train_batch_size=b, tokens_until_dead=10 * b * s)

    def run(fast):
        tr = tracker()
        torch.manual_seed(4)
        mlp = SparseMLP(layer_idx=0, config=cfg, gated=True, tracker=tr,
                        execution_logic="training", use_hybrid_kernel=True)
        with torch.no_grad():
            mlp.gate_proj.weight.normal_(0, 0.02)
            mlp.gate_proj.weight[:, 0] = -0.9  # x[..., 0] = 1: about 2-3 % of the gates fire
            mlp.up_proj.weight.normal_(0, 0.02)
            mlp.down_proj.weight.normal_(0, 0.02)
        mlp = mlp.to(DEV).to(torch.bfloat16)
        mlp.enable_fast(fast)
        gen = torch.Generator().manual_seed(5)
        x = torch.randn(b, s, d, generator=gen)
        x[..., 0] = 1.0
        x = x.to(DEV).to(torch.bfloat16).requires_grad_(True)
        tr.start_forward_pass()
        out = mlp(x)
        l1, stats = tr.finalize_forward_pass()
        w = torch.randn(b, s, d, generator=gen).to(DEV)
        loss = (out.float() * w).sum() + 0.05 * l1.float()
        loss.backward()
        grads = [x.grad, mlp.gate_proj.weight.grad, mlp.up_proj.weight.grad,
                 mlp.down_proj.weight.grad]
        return out.detach().float(), float(l1), stats, [g.float() for g in grads]

    out_f, l1_f, stats_f, g_f = run(True)
    out_e, l1_e, stats_e, g_e = run(False)
    rel = lambda a, b_: float((a - b_).norm() / (b_.norm() + 1e-12))  # noqa: E731
    assert rel(out_f, out_e) < 1.5e-2
    assert l1_f == pytest.approx(l1_e, rel=2e-2)
    assert float(stats_f["activation_l0/mean"]) == pytest.approx(
        float(stats_e["activation_l0/mean"]), rel=3e-2)
    for name, a, b_ in zip(("dX", "dG", "dK", "dV"), g_f, g_e):
        assert rel(a, b_) < 4e-2, name  # both sides are bf16 computations


def test_reference_benchmark_model_runs_on_the_swapped_model(reference):
    """benchmark_inference.benchmark_model (benchmark_inference.py:268-343) on a random-init
    model built the way load_twell_model builds it (:237-265), minus the checkpoint file."""
    import benchmark_inference as bi
    from custom_models.sparse_testing_utils import convert_sparse_mlp_to_twell_fused
    model = tiny_sparse_llama()
    model.replace_mlp_modules(convert_sparse_mlp_to_twell_fused)
    model = bi.finalize_model(model, device=torch.device(DEV), dtype=torch.bfloat16)
    ids, mask = bi.build_inputs(model.config, batch_size=2, seq_len=128, device=torch.device(DEV))
    bi.validate_twell_shape(2, 128)
    res = bi.benchmark_model(model, ids, mask, reps=2, warmup_reps=1,
                             implementation_name="twell")
    assert res["avg_total_ms"] > 0
    with torch.inference_mode():
        hidden = bi.get_core_model(model)(input_ids=ids, attention_mask=mask).last_hidden_state
    assert torch.isfinite(hidden.float()).all()
