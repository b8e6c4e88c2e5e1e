"""State-dict conversions around the sparse FFN: HF layout <-> TwELL buffers, d_ff shards.

Mirrors custom_models/sparse_testing_utils.py:78-207 (``sparse_to_hf_state_dict``,
``sparse_to_twell_state_dict``: same key rules, same transposes) and adds what the d_ff-sharded
modules need: slicing a TwELL state dict to one rank's rows and merging shards back.

Weight layouts (``D`` = hidden size, ``H`` = d_ff):

=====================  ==============================  =========================
key suffix             tensor                           meaning
=====================  ==============================  =========================
``gate_proj.weight``   ``[H, D]``                       HF linear
``up_proj.weight``     ``[H, D]``                       HF linear
``down_proj.weight``   ``[D, H]``                       HF linear
``GATE`` / ``UP``      ``[H, D]``                       TwELL module buffers
``DOWN``               ``[H, D]`` = ``down_proj.weight.T``
``gate_weight``        ``[D, H]``                       raw-parameter checkpoints
``up_weight``          ``[H, D]`` gated, ``[D, H]`` not
``down_weight``        ``[H, D]``
=====================  ==============================  =========================
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .sharded import shard_range

_AUX_MARKERS = ("tracker.", "metrics_accumulator.")

# (key suffix, only valid for gated checkpoints, name and transpose in the HF dict, name and
# transpose in the TwELL dict); first match wins, in the reference's order.
_RULES = (
    # suffix            gated_only  hf_name              hf_T   twell_name  twell_T
    ("gate_proj.weight", True,      "gate_proj.weight",  False, "GATE",     False),
    ("up_proj.weight",   False,     "up_proj.weight",    False, "UP",       False),
    ("down_proj.weight", False,     "down_proj.weight",  False, "DOWN",     True),
    ("gate_weight",      True,      "gate_proj.weight",  True,  "GATE",     True),
    ("up_weight",        False,     "up_proj.weight",    None,  "UP",       None),   # see below
    ("down_weight",      False,     "down_proj.weight",  True,  "DOWN",     False),
    ("GATE",             True,      "gate_proj.weight",  False, "GATE",     False),
    ("UP",               False,     "up_proj.weight",    False, "UP",       False),
    ("DOWN",             False,     "down_proj.weight",  True,  "DOWN",     False),
)


def _is_auxiliary(key: str) -> bool:
    return any(key.startswith(m) or ("." + m) in key for m in _AUX_MARKERS)


def _convert(state_dict: Mapping[str, torch.Tensor], target: str, gated: bool,
             drop_auxiliary: bool) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for key, value in state_dict.items():
        if drop_auxiliary and _is_auxiliary(key):
            continue
        for suffix, gated_only, hf_name, hf_t, tw_name, tw_t in _RULES:
            if not key.endswith(suffix):
                continue
            if gated_only and not gated:
                raise ValueError(f"Attempting to convert {suffix} but gated is False")
            prefix = key[: -len(suffix)]
            name, transpose = (hf_name, hf_t) if target == "hf" else (tw_name, tw_t)
            if transpose is None:  # up_weight is [H, D] in gated checkpoints, [D, H] otherwise
                transpose = not gated
            out[prefix + name] = (value.T if transpose else value).contiguous()
            break
        else:
            out[key] = value
    return out


def sparse_to_hf_state_dict(state_dict: Mapping[str, torch.Tensor], drop_auxiliary: bool = True,
                            gated: bool = True) -> Dict[str, torch.Tensor]:
    """Any of the three sparse layouts -> HF ``*_proj.weight`` keys (sparse_testing_utils.py:182-193)."""
    return _convert(state_dict, "hf", gated, drop_auxiliary)


def sparse_to_twell_state_dict(state_dict: Mapping[str, torch.Tensor],
                               gated: bool = True) -> Dict[str, torch.Tensor]:
    """Any of the three sparse layouts -> ``GATE / UP / DOWN`` buffers, all ``[H, D]``
    (sparse_testing_utils.py:196-207)."""
    return _convert(state_dict, "twell", gated, True)


_TWELL_SUFFIXES = ("GATE", "UP", "DOWN")


def shard_twell_state_dict(state_dict: Mapping[str, torch.Tensor], rank: int,
                           world_size: int) -> Dict[str, torch.Tensor]:
    """This rank's rows ``[h0, h1)`` of every ``GATE / UP / DOWN`` buffer (tile-granular,
    :func:`sharded.shard_range`); every other entry is passed through.  Feed the result to
    ``ShardedTwELLGatedMLP(..., presharded=True)``."""
    out: Dict[str, torch.Tensor] = {}
    for key, value in state_dict.items():
        if key.endswith(_TWELL_SUFFIXES) and value.dim() == 2:
            h0, h1 = shard_range(value.shape[0], rank, world_size)
            out[key] = value[h0:h1].contiguous()
        else:
            out[key] = value
    return out


def merge_twell_shards(shards: list[Mapping[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    """Inverse of :func:`shard_twell_state_dict` over all ranks, in rank order."""
    if not shards:
        raise ValueError("need at least one shard")
    out: Dict[str, torch.Tensor] = {}
    for key, value in shards[0].items():
        if key.endswith(_TWELL_SUFFIXES) and value.dim() == 2:
            out[key] = torch.cat([s[key] for s in shards], dim=0).contiguous()
        else:
            out[key] = value
    return out


def retranspose_hybrid_down_proj(model) -> int:
    """Re-applies the ``[H, D]`` layout of ``down_proj.weight`` that the hybrid training path
    expects after a checkpoint in HF layout ``[D, H]`` was loaded over it
    (hydra_utils.py:69-80).  Only weights still in HF layout are touched, so calling it twice
    is harmless when ``H != D``.  Returns the number of layers changed."""
    cfg = getattr(model, "config", None)
    if not getattr(cfg, "sparsity_use_hybrid_kernel", False):
        return 0
    inner = getattr(model, "model", model)
    changed = 0
    for layer in getattr(inner, "layers", []):
        mlp = getattr(layer, "mlp", None)
        down = getattr(mlp, "down_proj", None) if mlp is not None else None
        if down is None:
            continue
        w = down.weight.data
        hidden = getattr(cfg, "hidden_size", None)
        if hidden is not None and w.shape[0] == hidden and w.shape[1] != hidden:
            down.weight.data = w.t().contiguous()
            changed += 1
    return changed
