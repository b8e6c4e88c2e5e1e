"""CPU restatement of the sparse gated-FFN arithmetic (test infrastructure only).

Three layers of truth, from loosest to tightest coupling with the kernels:

* ``dense_ffn`` - the function itself, ``relu(x Wg^T + b) * (x Wu^T)) Wd`` in
  fp32 or fp64, exactly what ``SparseMLP._forward_mlp_inference_logic`` computes
  (custom_models/sparse_models.py:343-351) with TwELL-layout weights
  (GATE/UP/DOWN all ``[H, D]``, custom_models/sparse_testing_utils.py:23-34).
* ``gate_preactivation`` + ``oracle.twell_format.pack_preactivations`` - the
  pack kernel's contract (custom_models/twell_modules/matmul_d2t.cu:614-704).
* ``gated_t2d`` / ``t2d`` - the contraction kernels with the reference's
  rounding points reproduced (custom_models/twell_modules/matmul_gated_t2d.cu:
  17-169 mixed precision, :330-461 high precision; matmul_t2d.cu:15-113).

All inputs are torch CPU tensors.  bf16 rounding is torch's round-to-nearest-even
conversion, the same as ``__float2bfloat16_rn`` / ``__hmul2`` on the device.
"""
from __future__ import annotations

import numpy as np
import torch

from . import twell_format as tf

TILE_N = tf.TILE_N


def bf16r(x: torch.Tensor) -> torch.Tensor:
    """Round an fp32 tensor to bf16 and return it as fp32."""
    return x.to(torch.float32).to(torch.bfloat16).to(torch.float32)


# --------------------------------------------------------------------------
# dense truth
# --------------------------------------------------------------------------
def dense_ffn(x, gate, up, down, gate_bias=None, dtype=torch.float32):
    """``(relu(x gate^T + b) * (x up^T)) @ down`` with ``[H, D]`` weights.

    Restates SparseMLP._forward_mlp_inference_logic (sparse_models.py:343-351):
    ``gate_proj.weight == gate``, ``up_proj.weight == up``,
    ``down_proj.weight == down.T``.
    """
    x = x.to(dtype)
    g = x @ gate.to(dtype).T
    if gate_bias is not None:
        g = g + gate_bias.to(dtype)
    u = x @ up.to(dtype).T
    h = torch.relu(g) * u
    return h @ down.to(dtype)


def dense_mlp(x, up, down, dtype=torch.float32):
    """Non-gated variant ``relu(x up^T) @ down`` (sparse_models.py:349-351)."""
    x = x.to(dtype)
    return torch.relu(x @ up.to(dtype).T) @ down.to(dtype)


def gate_preactivation(x, gate, gate_bias=None, dtype=torch.float32):
    """Pre-activation ``z = x gate^T (+ b)``; the pack kernel keeps ``z > 0``."""
    z = x.to(dtype) @ gate.to(dtype).T
    if gate_bias is not None:
        z = z + gate_bias.to(dtype)
    return z


def pack_gate(x, gate, gate_bias=None, compression_factor=8):
    """TwELL slabs of ``relu(x gate^T + b)`` from an fp32 pre-activation."""
    z = gate_preactivation(x, gate, gate_bias, torch.float32)
    return tf.pack_preactivations(z.numpy(), compression_factor)


def ambiguity_mask(x, gate, gate_bias=None, rel=2e-6):
    """Entries whose sign an fp32 accumulation in another order may flip.

    ``|z64| <= rel * sum_k |x_k w_k|``: the fp32 rounding-error bound of a
    length-D dot product is about ``D * 2^-24`` relative to the sum of absolute
    products, so ``rel`` defaults to a small multiple of that for D <= 4096...
    callers scale ``rel`` with D when needed.
    """
    x64 = x.to(torch.float64)
    g64 = gate.to(torch.float64)
    z = x64 @ g64.T
    if gate_bias is not None:
        z = z + gate_bias.to(torch.float64)
    mag = x64.abs() @ g64.abs().T
    if gate_bias is not None:
        mag = mag + gate_bias.to(torch.float64).abs()
    return (z.abs() <= rel * mag), z


# --------------------------------------------------------------------------
# contraction kernels, with the reference's rounding points
# --------------------------------------------------------------------------
def _warp_order_dot(prod: torch.Tensor) -> torch.Tensor:
    """fp32 sum of ``prod[..., D]`` in the reference warp order.

    Lane ``l`` owns elements ``iter*256 + l*8 + e`` and adds them sequentially
    (iter outer, e inner; matmul_gated_t2d.cu:77-105), then an xor butterfly
    with strides 16,8,4,2,1 combines the lanes (:108-111).
    """
    d = prod.shape[-1]
    iters = d // 256
    p = prod.reshape(*prod.shape[:-1], iters, 32, 8)
    acc = torch.zeros(*prod.shape[:-1], 32, dtype=torch.float32)
    for it in range(iters):
        for e in range(8):
            acc = acc + p[..., it, :, e]
    lanes = torch.arange(32)
    for stride in (16, 8, 4, 2, 1):
        acc = acc + acc[..., lanes ^ stride]
    return acc[..., 0]


def _row_entries(packed_row: np.ndarray, w: int):
    cols, bits = [], []
    for t in range(packed_row.shape[0] // w):
        slab = packed_row[t * w:(t + 1) * w]
        n = min(int(slab[0]), w - 1)
        cols.extend((slab[1:1 + n] & 0xFFFF).tolist())
        bits.extend((slab[1:1 + n] >> 16).tolist())
    return cols, bits


def gated_t2d(x, packed, up, down, highest_precision=False,
              compression_factor=8):
    """Gated TwELL -> dense contraction with the reference's rounding points.

    mixed (matmul_gated_t2d.cu:74-149): ``u = sum_k fp32(bf16(x_k * UP[j,k]))``,
    ``h = bf16(bf16(g) * bf16(u))``, ``y_c += fp32(bf16(h * DOWN[j,c]))``.
    high precision (:389-441): fp32 fma everywhere, ``h = g * u`` kept in fp32.
    Entries are consumed in stored order; y is rounded to bf16 at the end.
    Returns fp32 holding bf16-representable values.
    """
    x = bf16r(x)
    up = bf16r(up)
    down = bf16r(down)
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    w = tf.slab_words(compression_factor)
    m, d = x.shape
    y = torch.zeros(m, d, dtype=torch.float32)
    for r in range(m):
        cols, bits = _row_entries(packed[r], w)
        if not cols:
            continue
        idx = torch.tensor(cols, dtype=torch.int64)
        g = torch.from_numpy(
            tf.bf16_bits_to_f32(np.asarray(bits, dtype=np.uint16)).copy())
        up_rows = up[idx]                      # [nnz, D]
        down_rows = down[idx]
        if highest_precision:
            # fp32 fma chain; a float64 product-sum rounded once per step is not
            # reproducible cheaply, so evaluate in the same lane order in fp64
            # and round the final dot to fp32: differences are below 1 ulp of
            # fp32 and far inside the stated tolerances.
            u = (x[r].double()[None, :] * up_rows.double()).sum(-1).float()
            h = g * u
            acc = torch.zeros(d, dtype=torch.float64)
            for k in range(idx.numel()):
                acc = acc + (h[k].double() * down_rows[k].double())
            y[r] = acc.float()
        else:
            prod = bf16r(x[r][None, :] * up_rows)
            u = _warp_order_dot(prod)
            h = bf16r(g * bf16r(u))
            acc = torch.zeros(d, dtype=torch.float32)
            for k in range(idx.numel()):
                acc = acc + bf16r(h[k] * down_rows[k])
            y[r] = acc
    return bf16r(y)


def t2d(packed, down, compression_factor=8):
    """Non-gated TwELL -> dense: ``y_c += fp32(bf16(v * DOWN[j,c]))``.

    matmul_t2d.cu:50-96; output rounded to bf16 (:97-112).
    """
    down = bf16r(down)
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    w = tf.slab_words(compression_factor)
    m = packed.shape[0]
    d = down.shape[1]
    y = torch.zeros(m, d, dtype=torch.float32)
    for r in range(m):
        cols, bits = _row_entries(packed[r], w)
        if not cols:
            continue
        idx = torch.tensor(cols, dtype=torch.int64)
        v = torch.from_numpy(
            tf.bf16_bits_to_f32(np.asarray(bits, dtype=np.uint16)).copy())
        rows = down[idx]
        acc = torch.zeros(d, dtype=torch.float32)
        for k in range(idx.numel()):
            acc = acc + bf16r(v[k] * rows[k])
        y[r] = acc
    return bf16r(y)


def gated_mlp(x, gate, up, down, gate_bias=None, highest_precision=False,
              compression_factor=8):
    """Pack then contract: what ``run_gated_mlp_layer`` computes
    (custom_models/twell_modules/mlp_twell.cu:126-152)."""
    packed = pack_gate(bf16r(x), bf16r(gate), gate_bias, compression_factor)
    return gated_t2d(x, packed, up, down, highest_precision, compression_factor), packed


def mlp(x, up, down, compression_factor=8):
    """Non-gated fused MLP (mlp_twell.cu:73-98)."""
    packed = pack_gate(bf16r(x), bf16r(up), None, compression_factor)
    return t2d(packed, down, compression_factor), packed


# --------------------------------------------------------------------------
# sparsity statistics (SparsityTracker.record_activations, sparse_models.py:148-181)
# --------------------------------------------------------------------------
def l0_l1(h_abs: torch.Tensor):
    """``l1 = mean_tokens sum_neurons |h|``; ``l0 = sum_neurons mean_tokens(h>0)``."""
    h_abs = h_abs.reshape(-1, h_abs.shape[-1])
    l1 = h_abs.sum(-1).mean()
    l0 = (h_abs > 0).float().mean(0).sum()
    return l0, l1


def last_activated_update(h_abs: torch.Tensor, last_activated: torch.Tensor,
                          microbatch_tokens: int):
    """Dead-neuron counter update from the dense activation (sparse_models.py:170-181):
    a neuron active for any token restarts at 0, the others age by ``microbatch_tokens``.
    Returns ``(active_rows int32 [H], new last_activated int64 [H])``."""
    h_abs = h_abs.reshape(-1, h_abs.shape[-1])
    active_rows = (h_abs > 0).sum(0).to(torch.int32)
    new = torch.where(active_rows > 0, torch.zeros_like(last_activated),
                      last_activated + int(microbatch_tokens))
    return active_rows, new


def slab_active_rows(p_slab: np.ndarray, vals_slab: np.ndarray | None, output_n: int,
                     compression_factor: int = 8) -> np.ndarray:
    """Per-neuron count of rows whose stored value is not +-0, read from slab arrays (the
    pattern ``p_slab`` gives the columns, ``vals_slab`` the values when given).  Entries a
    slab dropped on overflow are not seen, as on the device; neither are rows whose count
    words carry the sign bit (the training operator's mark for "this row went to the dense
    tail": every kernel reads such a count as zero)."""
    w = tf.slab_words(compression_factor)
    tiles = output_n // TILE_N
    p = np.ascontiguousarray(p_slab).view(np.uint32).reshape(-1, tiles, w)
    v = p if vals_slab is None else np.ascontiguousarray(vals_slab).view(np.uint32).reshape(p.shape)
    cnt = np.clip(p[:, :, 0].view(np.int32).astype(np.int64), 0, w - 1)
    stored = np.arange(1, w)[None, None, :] <= cnt[:, :, None]
    nonzero = ((v[:, :, 1:] >> 16) & 0x7FFF) != 0
    cols = (p[:, :, 1:] & 0xFFFF)[stored & nonzero]
    return np.bincount(cols, minlength=output_n).astype(np.int32)


# --------------------------------------------------------------------------
# error metrics
# --------------------------------------------------------------------------
def max_abs_and_rel_l2(y, y_ref):
    y = y.double().reshape(-1)
    y_ref = y_ref.double().reshape(-1)
    diff = (y - y_ref)
    max_abs = diff.abs().max().item() if diff.numel() else 0.0
    denom = y_ref.norm().item()
    rel = diff.norm().item() / denom if denom > 0 else diff.norm().item()
    return max_abs, rel
