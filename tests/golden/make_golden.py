"""Generate the golden fixtures from the reference's own torch implementation.

Run in a container where the reference checkout is importable:

    python tests/golden/make_golden.py --reference /path/to/sparser-faster-llms

Writes ``tests/golden/*.npz``.  Sources of truth used (reference paths):

* ``custom_models/sparse_models.py`` ``SparseMLP`` - inference logic (:343-351)
  and training branch with the ``SparsityTracker`` l0 / l1 statistics
  (:397-410, :148-181), plus autograd gradients of
  ``sum(out * gout) + coeff * l1``;
* ``custom_models/twell_modules/twell.py`` ``packed_to_dense`` (:215-264) - the
  executable spec of the TwELL slab format.

Weights are bf16-representable so that the CUDA kernels (bf16 storage) see
exactly the same numbers as the fp32 reference run.
"""
from __future__ import annotations

import argparse
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

from oracle import twell_format as tf  # noqa: E402
from sparser_faster_llms_b200 import synthetic  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).copy()


def sha(*tensors: torch.Tensor) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(bits(t).tobytes())
    return h.hexdigest()


def build_sparse_mlp(ref, d, h, gate, up, down, bias, execution_logic):
    from transformers import LlamaConfig
    cfg = LlamaConfig(hidden_size=d, intermediate_size=h, mlp_bias=bias is not None)
    tracker = ref.SparsityTracker(train_batch_size=1, max_seq_len=1,
                                  per_device_train_batch_size=1, gated=True)
    mlp = ref.SparseMLP(layer_idx=0, config=cfg, gated=True, tracker=tracker,
                        execution_logic=execution_logic)
    with torch.no_grad():
        mlp.gate_proj.weight.copy_(gate.float())
        mlp.up_proj.weight.copy_(up.float())
        mlp.down_proj.weight.copy_(down.float().T)
        if bias is not None:
            mlp.gate_proj.bias.copy_(bias)
            mlp.up_proj.bias.zero_()
            mlp.down_proj.bias.zero_()
    return mlp, tracker


def case_small(ref, twell_ref, out: Path):
    """Inputs stored in full: M=16, D=256, H=512."""
    m, d, h = 16, 256, 512
    ffn = synthetic.make_ffn(d, h, seed=11, density=0.05, skew_sigma=1.0)
    x = synthetic.make_tokens(m, d, seed=12)
    mlp, _ = build_sparse_mlp(ref, d, h, ffn.gate, ffn.up, ffn.down, None, "inference")
    with torch.no_grad():
        y32 = mlp(x.float()[None])[0]
        y_bf16 = mlp.to(torch.bfloat16)(x[None])[0].float()
    z = x.float() @ ffn.gate.float().T
    fixtures = {"x": bits(x), "gate": bits(ffn.gate), "up": bits(ffn.up), "down": bits(ffn.down),
                "y_fp32": y32.numpy(), "y_bf16_torch": y_bf16.numpy()}
    for cf in (8, 4, 2):
        packed = tf.pack_preactivations(z.numpy(), cf)
        try:
            dense = twell_ref.packed_to_dense(
                torch.from_numpy(packed.view(np.int32)).view(torch.uint32), h,
                compression_factor=cf)
            fixtures[f"ref_dense_cf{cf}"] = bits(dense)
            fixtures[f"ref_raises_cf{cf}"] = np.array(0)
        except ValueError:
            fixtures[f"ref_raises_cf{cf}"] = np.array(1)
    np.savez_compressed(out / "small_gated.npz", **fixtures)


def case_training(ref, out: Path):
    """Training branch: l0 / l1 statistics and gradients. M=2x12, D=256, H=512."""
    b, s, d, h = 2, 12, 256, 512
    ffn = synthetic.make_ffn(d, h, seed=21, density=0.06, skew_sigma=0.5)
    x = synthetic.make_tokens(b * s, d, seed=22).float().reshape(b, s, d)
    gout = synthetic.make_tokens(b * s, d, seed=23, fold_bias=False).float().reshape(b, s, d)
    coeff = 0.05
    mlp, tracker = build_sparse_mlp(ref, d, h, ffn.gate, ffn.up, ffn.down, None, "training")
    x = x.clone().requires_grad_(True)
    tracker.start_forward_pass()
    y = mlp(x)
    l1, stats = tracker.finalize_forward_pass()
    loss = (y * gout).sum() + coeff * l1
    loss.backward()
    np.savez_compressed(
        out / "training_gated.npz",
        seed_ffn=21, seed_x=22, seed_gout=23, coeff=coeff, b=b, s=s, d=d, h=h,
        input_sha=np.array(sha(x.detach().reshape(-1, d), ffn.gate, ffn.up, ffn.down)),
        y=y.detach().numpy(), l1=float(l1),
        l0=float(stats["activation_l0/mean"]) if "activation_l0/mean" in stats else
        float(list(v for k, v in stats.items() if k.startswith("activation_l0"))[0]),
        dx=x.grad.numpy(), dgate=mlp.gate_proj.weight.grad.numpy(),
        dup=mlp.up_proj.weight.grad.numpy(), ddown=mlp.down_proj.weight.grad.T.numpy().copy())


def case_config1(ref, out: Path):
    """Single-layer configuration: x [256, 1024] fp32 ~N(0,1), weights ~N(0, 0.02),
    constant gate bias for about 2 % density.  Only outputs and an input hash are stored."""
    m, d, h = 256, 1024, 4096
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(m, d, generator=gen)
    gate = (torch.randn(h, d, generator=gen) * 0.02).to(torch.bfloat16)
    up = (torch.randn(h, d, generator=gen) * 0.02).to(torch.bfloat16)
    down = (torch.randn(h, d, generator=gen) * 0.02).to(torch.bfloat16)
    x = x.to(torch.bfloat16)
    z0 = x.float() @ gate.float().T
    shift = -float(torch.quantile(z0.flatten()[:: 7].float(), 0.98))
    bias = torch.full((h,), shift)
    mlp, _ = build_sparse_mlp(ref, d, h, gate, up, down, bias, "inference")
    with torch.no_grad():
        y = mlp(x.float()[None])[0]
    z = z0 + shift
    counts = tf.slab_counts(tf.pack_preactivations(z.numpy(), 2), 2)
    np.savez_compressed(
        out / "config1_gated.npz", m=m, d=d, h=h, seed=0, shift=shift,
        input_sha=np.array(sha(x, gate, up, down)),
        y_rows=y[:32].numpy(), y_norm=float(y.double().norm()),
        counts=counts.astype(np.int16), density=float((z > 0).float().mean()))


PUBLIC_NAMES = [
    "packed_width", "allocate_packed_output", "packed_to_dense", "matmul_sparse",
    "matmul_sparse_out", "matmul_t2d", "matmul_t2d_out", "matmul_gated_t2d",
    "matmul_gated_t2d_out", "create_d2t_layer", "run_d2t_layer", "ensure_d2t_layer_shape",
    "run_mlp_layer", "run_gated_mlp_layer", "_run_mlp_layer_with_hidden_states",
    "_run_gated_mlp_layer_with_hidden_states", "run_mlp_layer_inplace",
    "run_gated_mlp_layer_inplace", "_run_mlp_layer_inplace_with_hidden_states",
    "_run_gated_mlp_layer_inplace_with_hidden_states", "destroy_d2t_layer",
    "destroy_all_d2t_layers", "load_ext", "get_ext", "sparse_algorithms",
    "D2TLayer", "D2TLinear", "T2DLinear", "GatedT2DLinear", "TwELLMLP", "TwELLGatedMLP",
]


def case_signatures(twell_ref, out: Path):
    """Parameter names, order and defaults of the reference's public TwELL API."""
    import inspect
    import json
    sigs = {}
    for name in PUBLIC_NAMES:
        obj = getattr(twell_ref, name)
        target = obj.__init__ if inspect.isclass(obj) else obj
        params = []
        for p in inspect.signature(target).parameters.values():
            if p.name == "self":
                continue
            default = None if p.default is inspect.Parameter.empty else repr(p.default)
            params.append([p.name, p.kind.name, default])
        sigs[name] = params
        if inspect.isclass(obj):
            sigs[name + ".methods"] = sorted(
                m for m in vars(obj) if not m.startswith("__") and callable(getattr(obj, m)))
    sigs["sparse_algorithms()"] = twell_ref.sparse_algorithms()
    (out / "twell_signatures.json").write_text(json.dumps(sigs, indent=1, sort_keys=True))


def state_dict_inputs():
    """Small seeded state dicts in the three layouts the reference converts between
    (HF linears, raw parameters, TwELL buffers), gated and not, with auxiliary keys."""
    gen = torch.Generator().manual_seed(2024)
    d, h = 6, 10
    r = lambda *s: torch.randn(*s, generator=gen)  # noqa: E731
    gated_hf = {"model.embed.weight": r(7, d), "tracker.count": r(3),
                "model.layers.0.mlp.metrics_accumulator.x": r(2)}
    gated_raw, gated_twell, plain_raw = {"lm_head.weight": r(7, d)}, {"norm.weight": r(d)}, {}
    for l in range(2):
        p = f"model.layers.{l}.mlp."
        gated_hf.update({p + "gate_proj.weight": r(h, d), p + "up_proj.weight": r(h, d),
                         p + "down_proj.weight": r(d, h), p + "tracker.last": r(h)})
        gated_raw.update({p + "gate_weight": r(d, h), p + "up_weight": r(h, d),
                          p + "down_weight": r(h, d)})
        gated_twell.update({p + "GATE": r(h, d), p + "UP": r(h, d), p + "DOWN": r(h, d)})
        plain_raw.update({p + "up_weight": r(d, h), p + "down_weight": r(h, d)})
    return {"gated_hf": (gated_hf, True), "gated_raw": (gated_raw, True),
            "gated_twell": (gated_twell, True), "plain_raw": (plain_raw, False)}


def case_state_dicts(reference_root: str, out: Path):
    """Outputs of the reference's sparse_to_hf_state_dict / sparse_to_twell_state_dict
    (custom_models/sparse_testing_utils.py:182-207): key -> [shape, sha256 of the bytes]."""
    import importlib.util
    import json
    import types
    # sparse_testing_utils imports the TwELL module classes only to build modules; give it
    # the file-loaded reference twell module under the package name it expects.
    spec = importlib.util.spec_from_file_location(
        "custom_models.twell_modules.twell",
        Path(reference_root) / "custom_models/twell_modules/twell.py")
    tw = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tw)
    sys.modules.setdefault("custom_models.twell_modules", types.ModuleType("custom_models.twell_modules"))
    sys.modules["custom_models.twell_modules.twell"] = tw
    spec = importlib.util.spec_from_file_location(
        "ref_sparse_testing_utils", Path(reference_root) / "custom_models/sparse_testing_utils.py")
    stu = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(stu)
    digest = lambda sd: {k: [list(v.shape), sha(v)] for k, v in sd.items()}  # noqa: E731
    golden = {}
    for name, (sd, gated) in state_dict_inputs().items():
        golden[name] = {"hf": digest(stu.sparse_to_hf_state_dict(sd, gated=gated)),
                        "twell": digest(stu.sparse_to_twell_state_dict(sd, gated=gated)),
                        "hf_keep_aux": digest(stu.sparse_to_hf_state_dict(
                            sd, drop_auxiliary=False, gated=gated))}
    (out / "state_dict_conversions.json").write_text(json.dumps(golden, indent=1, sort_keys=True))


TRACKER_ARGS = dict(train_batch_size=8, max_seq_len=16, per_device_train_batch_size=2,
                    tokens_until_dead=96, gated=True)


def tracker_inputs():
    """Seeded ``|h|`` micro-batches ``[step][layer] -> [2, 16, 512]`` fp32 for the tracker
    case: ~3 % dense, with neurons 0..63 of layer 0 never firing and neurons 64..127 firing
    only in step 0, so some counters cross ``tokens_until_dead``."""
    gen = torch.Generator().manual_seed(77)
    steps = []
    for step in range(5):
        layers = []
        for layer in range(2):
            h = torch.rand(2, 16, 512, generator=gen)
            h = torch.where(torch.rand(2, 16, 512, generator=gen) < 0.03, h, torch.zeros(()))
            if layer == 0:
                h[..., :64] = 0
                if step > 0:
                    h[..., 64:128] = 0
            layers.append(h)
        steps.append(layers)
    return steps


def case_tracker(ref, out: Path):
    """The reference's SparsityTracker (custom_models/sparse_models.py:95-256) driven over
    ``tracker_inputs()`` through record_activations: per step the ``_last_activated``
    counters, alive masks, L1 loss and logged statistics."""
    import contextlib
    import io
    import json
    with contextlib.redirect_stdout(io.StringIO()):
        tr = ref.SparsityTracker(**TRACKER_ARGS)
    golden = []
    for layers in tracker_inputs():
        tr.start_forward_pass()
        for i, h in enumerate(layers):
            tr.record_activations(layer_idx=i, absolute_activations=h)
        l1, stats = tr.finalize_forward_pass()
        golden.append({
            "l1": float(l1),
            "stats": {k: float(v) for k, v in stats.items()},
            "last_activated": [tr._last_activated[i].tolist() for i in range(len(layers))],
            "alive": [int(a.sum()) for a in tr.get_alive_neurons()],
        })
    (out / "sparsity_tracker.json").write_text(json.dumps(golden, sort_keys=True))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=str(REPO.parent / "reference"),
                    help="checkout of the reference (default: a sibling of this repository)")
    ap.add_argument("--only-state-dicts", action="store_true")
    ap.add_argument("--only-tracker", action="store_true")
    args = ap.parse_args()
    if args.only_state_dicts:
        case_state_dicts(args.reference, HERE)
        return
    sys.path.insert(0, args.reference)
    from custom_models import sparse_models as ref
    if args.only_tracker:
        case_tracker(ref, HERE)
        return
    import importlib.util
    # twell.py imports torch.utils.cpp_extension only; it is safe to import on CPU.
    spec = importlib.util.spec_from_file_location(
        "ref_twell", Path(args.reference) / "custom_models/twell_modules/twell.py")
    twell_ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(twell_ref)
    torch.manual_seed(0)
    case_signatures(twell_ref, HERE)
    case_small(ref, twell_ref, HERE)
    case_training(ref, HERE)
    case_config1(ref, HERE)
    case_tracker(ref, HERE)
    for p in sorted(HERE.glob("*.npz")):
        print(p.name, p.stat().st_size)


if __name__ == "__main__":
    main()
