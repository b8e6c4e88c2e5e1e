"""Sparsity bookkeeping of the training path, with live dead-neuron counters on the fused
operator.

Mirror of ``SparsityTracker`` / ``NullTracker`` (custom_models/sparse_models.py:51-256): the
per-layer L0 / L1 lists, the auxiliary L1 loss, and ``_last_activated`` - for each neuron the
number of tokens since it last fired, from which ``get_alive_neurons`` derives the alive
masks.  The reference updates ``_last_activated`` only on the einsum path
(``record_activations``, :148-181); ``record_l0_l1`` (:183-208) documents that the hybrid
kernel leaves it stale because the per-neuron mask is never materialised.  Here the forward
keeps the activation as a slab (``T``), so ``record_pattern`` brings the counters up to date
with one extra pass over the slabs (``sparse_ops.neuron_activity``) - no dense ``[M, H]``
mask, no host synchronisation.

``select_fast_layers`` is the adaptive switch of ``SparseLlamaForCausalLM.forward``
(:631-643): layers whose last measured L0 is under the cutoff run the fused operator.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch


def get_tensor_stats_for_logging(prefix: str, t) -> Dict[str, torch.Tensor]:
    """min / max / mean / std of a tensor or list of scalars (sparse_models.py:36-48)."""
    if not isinstance(t, torch.Tensor) and isinstance(t, list):
        t = torch.stack([ti.detach() for ti in t], dim=0)
    flat = t.detach().reshape(-1)
    return {f"{prefix}/min": flat.min(), f"{prefix}/max": flat.max(),
            f"{prefix}/mean": flat.mean(), f"{prefix}/std": flat.std()}


class NullTracker:
    """No-op tracker for baseline or inference-only flows (sparse_models.py:51-92)."""

    def __init__(self, train_batch_size: int = 0, max_seq_len: int = 0,
                 tokens_until_dead: Optional[int] = None) -> None:
        pass

    def register_layer(self, layer_idx: int, width: int, device: torch.device) -> None:
        pass

    def start_forward_pass(self) -> None:
        pass

    def record_activations(self, layer_idx: int, **kwargs) -> None:
        pass

    def record_l0_l1(self, layer_idx: int, l0, l1, width: int) -> None:
        pass

    def record_pattern(self, layer_idx: int, l0, l1, P, T=None, width: Optional[int] = None) -> None:
        pass

    def finalize_forward_pass(self) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        return torch.tensor(0.0), {}


class SparsityTracker:
    """Activation-sparsity statistics and the auxiliary L1 signal (sparse_models.py:95-256).

    ``total_devices`` (default: ``WORLD_SIZE`` from the environment, else 1, which is what
    the reference's ``get_total_devices()`` returns, :30-34) divides the global batch."""

    def __init__(self, train_batch_size: int, max_seq_len: int,
                 per_device_train_batch_size: int, tokens_until_dead: Optional[int] = None,
                 gated: bool = False, total_devices: Optional[int] = None) -> None:
        self._last_activated: Dict[int, torch.Tensor] = {}
        self._l1_per_layer: List[torch.Tensor] = []
        self._l0_per_layer: List[torch.Tensor] = []
        if total_devices is None:
            total_devices = int(os.environ.get("WORLD_SIZE", 1))
        self._batch_tokens = int((train_batch_size * max_seq_len) // max(1, int(total_devices)))
        self._microbatch_tokens = int(per_device_train_batch_size * max_seq_len)
        if tokens_until_dead is None:
            tokens_until_dead = self._batch_tokens
        self._tokens_until_dead = int(tokens_until_dead)
        self._number_of_layers: Optional[int] = None
        self._gated = gated
        self.active = False

    def register_layer(self, layer_idx: int, width: int, device: torch.device) -> None:
        if layer_idx in self._last_activated:
            return
        self._last_activated[layer_idx] = torch.zeros(int(width), dtype=torch.int64, device=device)

    def start_forward_pass(self) -> None:
        self.active = True
        self._l1_per_layer.clear()
        self._l0_per_layer.clear()

    def record_activations(self, layer_idx: int, absolute_activations: torch.Tensor) -> None:
        """Einsum path: statistics from the dense ``|h|`` (sparse_models.py:148-181)."""
        if (not self.active) and torch.is_grad_enabled():
            return
        self.register_layer(layer_idx, absolute_activations.shape[-1],
                            absolute_activations.device)
        self._l1_per_layer.append(absolute_activations.sum(dim=-1).mean())
        if not self.active:
            return
        is_active = absolute_activations.detach() > 0
        l0_per_neuron = is_active.float().mean(dim=tuple(range(is_active.dim() - 1)))
        self._l0_per_layer.append(l0_per_neuron.sum(-1))
        last = self._last_activated[layer_idx]
        self._last_activated[layer_idx] = torch.where(
            l0_per_neuron > 0, torch.zeros_like(last), last + self._microbatch_tokens)

    def record_l0_l1(self, layer_idx: int, l0: torch.Tensor, l1: torch.Tensor,
                     width: int) -> None:
        """Fused path, scalars only: ``_last_activated`` stays stale, as in the reference
        (sparse_models.py:183-208).  Prefer :meth:`record_pattern`."""
        if (not self.active) and torch.is_grad_enabled():
            return
        self.register_layer(layer_idx, width, l0.device)
        self._l1_per_layer.append(l1)
        if not self.active:
            return
        assert layer_idx == len(self._l0_per_layer)
        self._l0_per_layer.append(l0)

    def record_pattern(self, layer_idx: int, l0: torch.Tensor, l1: torch.Tensor, P, T=None,
                       width: Optional[int] = None) -> None:
        """Fused path with live dead-neuron counters: ``record_l0_l1`` plus the
        ``_last_activated`` update computed on the device from the forward's slabs ``P``
        (pattern) and ``T`` (``relu(gate)*up`` values)."""
        record_pattern(self, layer_idx, l0, l1, P, T, width)

    def get_alive_neurons(self) -> List[torch.Tensor]:
        if self._number_of_layers is None:
            raise ValueError("Must call finalize_forward_pass before get_alive_neurons")
        return [(self._last_activated[i] < self._tokens_until_dead).to(torch.float32)
                for i in range(self._number_of_layers)]

    def finalize_forward_pass(self) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        stats: Dict[str, torch.Tensor] = {}
        if self._number_of_layers is None:
            self._number_of_layers = len(self._last_activated)
        if not self._l1_per_layer:
            return 0.0, stats
        l1_loss = torch.mean(torch.stack(self._l1_per_layer))
        if not self.active:
            return l1_loss, stats
        self.active = False
        stats.update(get_tensor_stats_for_logging("activation_l0", self._l0_per_layer))
        stats.update(get_tensor_stats_for_logging("activation_l1", self._l1_per_layer))
        alive = [mask.mean() for mask in self.get_alive_neurons()]
        stats.update(get_tensor_stats_for_logging("activation_alive", alive))
        return l1_loss, stats


def record_pattern(tracker, layer_idx: int, l0: torch.Tensor, l1: torch.Tensor, P, T=None,
                   width: Optional[int] = None) -> None:
    """``record_l0_l1`` with the dead-neuron counters kept live, for any tracker that has
    the reference's fields (``active``, ``register_layer``, ``_l0_per_layer``,
    ``_l1_per_layer``, ``_last_activated``, ``_microbatch_tokens``) - this module's
    :class:`SparsityTracker` or the reference's own.  Trackers without those fields
    (``NullTracker``) get the plain ``record_l0_l1`` call."""
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
