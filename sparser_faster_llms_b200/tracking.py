"""Live dead-neuron counters for the fused training operator.

The reference's ``SparsityTracker`` (custom_models/sparse_models.py:95-256) keeps, per layer,
``_last_activated`` - for each neuron the number of tokens since it last fired - from which
``get_alive_neurons`` derives the alive masks.  It updates the counters only on the einsum
path (``record_activations``, :148-181); ``record_l0_l1`` (:183-208) documents that the hybrid
kernel leaves them stale because the per-neuron mask is never materialised.  Here the forward
keeps the activation as a slab (``T``), so :func:`record_pattern` brings the counters of the
reference's own tracker object up to date with one extra pass over the slabs
(``sparse_ops.neuron_activity``) - no dense ``[M, H]`` mask, no host synchronisation.  The
tracker class itself is the reference's and is not restated here.

``select_fast_layers`` is the adaptive switch of ``SparseLlamaForCausalLM.forward``
(:631-643): layers whose last measured L0 is under the cutoff run the fused operator.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


def record_pattern(tracker, layer_idx: int, l0: torch.Tensor, l1: torch.Tensor, P, T=None,
                   width: Optional[int] = None) -> None:
    """``record_l0_l1`` with the dead-neuron counters kept live, for a tracker that has the
    fields of the reference's ``SparsityTracker`` (``active``, ``register_layer``,
    ``_l0_per_layer``, ``_l1_per_layer``, ``_last_activated``, ``_microbatch_tokens``).
    Trackers without those fields (the reference's ``NullTracker``) get the plain
    ``record_l0_l1`` call."""
    from . import sparse_ops

    if not hasattr(tracker, "_last_activated"):
        tracker.record_l0_l1(layer_idx=layer_idx, l0=l0, l1=l1, width=width)
        return
    if (not tracker.active) and torch.is_grad_enabled():
        return
    slab = P.slab if isinstance(P, sparse_ops.HybridSp) else P
    if width is None:
        width = (P.n if isinstance(P, sparse_ops.HybridSp)
                 else slab.shape[1] // (sparse_ops.TILE // sparse_ops.compression_factor())
                 * sparse_ops.TILE)
    tracker.register_layer(layer_idx, width, slab.device)
    tracker._l1_per_layer.append(l1)
    if not tracker.active:
        return
    assert layer_idx == len(tracker._l0_per_layer)
    tracker._l0_per_layer.append(l0)
    sparse_ops.neuron_activity(P, T, last_activated=tracker._last_activated[layer_idx],
                               microbatch_tokens=tracker._microbatch_tokens, width=width)


def fused_training_forward(mlp, hidden_states: torch.Tensor) -> torch.Tensor:
    """The fused branch of ``SparseMLP.forward`` (sparse_models.py:378-395) with
    ``record_pattern`` in place of ``record_l0_l1``.  ``mlp`` is a reference ``SparseMLP``
    (or anything with ``gate_proj`` / ``up_proj`` / ``down_proj`` weights in the kernel
    layout, ``tracker``, ``layer_idx``, ``intermediate_size``)."""
    outs, l0, l1, P, _, T = torch.ops.sparse_ops.ff_forward_gated(
        hidden_states, mlp.gate_proj.weight, mlp.up_proj.weight, mlp.down_proj.weight)
    record_pattern(mlp.tracker, mlp.layer_idx, l0, l1, P, T, width=mlp.intermediate_size)
    return outs


def enable_live_dead_neuron_tracking(mlp) -> None:
    """Patch one ``SparseMLP`` instance so that its fused training branch keeps the
    dead-neuron counters current; every other branch (einsum training path, inference
    logic) runs the module's own ``forward`` unchanged.  Idempotent; undo with
    :func:`disable_live_dead_neuron_tracking`."""
    if "_forward_without_live_tracking" in mlp.__dict__:
        return
    original = mlp.forward

    def forward(hidden_states):
        if (getattr(mlp, "_training_mode", False) and getattr(mlp, "_use_fast", False)
                and getattr(mlp, "gated", False)):
            return fused_training_forward(mlp, hidden_states)
        return original(hidden_states)

    mlp.__dict__["_forward_without_live_tracking"] = original
    mlp.forward = forward


def disable_live_dead_neuron_tracking(mlp) -> None:
    original = mlp.__dict__.pop("_forward_without_live_tracking", None)
    if original is not None:
        del mlp.forward


def select_fast_layers(l0_per_layer: Sequence, l0_cutoff: float) -> List[bool]:
    """Which layers run the fused operator: those whose last measured L0 is below
    ``l0_cutoff`` (sparse_models.py:636-643; a non-positive cutoff disables the switch and
    keeps every layer on the fused path)."""
    if l0_cutoff <= 0:
        return [True] * len(l0_per_layer)
    return [float(v) < l0_cutoff for v in l0_per_layer]
