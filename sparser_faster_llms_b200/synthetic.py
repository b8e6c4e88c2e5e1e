"""Seeded synthetic sparse-FFN workloads (weights, tokens, gate density control).

There are no checkpoints or datasets offline, so every measurement and parity
test uses random-init weights ~N(0, 0.02) (the reference's initializer_range,
custom_models/sparse_models.py:571-577) and Gaussian tokens.  The gate density
is set by a per-neuron shift ``b_j`` of the gate pre-activation chosen from the
Gaussian quantile of the target firing rate; per-neuron rates are either uniform
or log-normal skewed (a few hot neurons).

The reference's kernels take no bias, so by default the shift is *folded into
the weights*: token feature 0 is the constant 1 and ``gate[:, 0] = b_j``.  The
same tensors then drive the reference module surface unchanged.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass
class SparseFFN:
    gate: torch.Tensor  # [H, D]
    up: torch.Tensor    # [H, D]
    down: torch.Tensor  # [H, D]  (= down_proj.weight.T)
    gate_bias: torch.Tensor | None  # [H] fp32, only when fold_bias=False
    rates: torch.Tensor  # [H] target firing rate per neuron (fp32, CPU)
    fold_bias: bool


def neuron_rates(h: int, density: float, skew_sigma: float, gen: torch.Generator) -> torch.Tensor:
    """Per-neuron firing rates with mean ``density``; log-normal when ``skew_sigma > 0``."""
    if skew_sigma <= 0:
        return torch.full((h,), float(density), dtype=torch.float64)
    n = torch.randn(h, generator=gen, dtype=torch.float64)
    r = torch.exp(skew_sigma * n - 0.5 * skew_sigma ** 2) * density
    for _ in range(8):  # clip then renormalise so the mean stays at the target
        r = r.clamp(1e-6, 0.5)
        r = r * (density / r.mean())
    return r.clamp(1e-6, 0.5)


def make_ffn(d_model: int, d_ff: int, *, seed: int = 0, density: float = 0.02,
             skew_sigma: float = 0.0, fold_bias: bool = True, std: float = 0.02,
             dtype: torch.dtype = torch.bfloat16, device="cpu") -> SparseFFN:
    gen = torch.Generator().manual_seed(seed)
    gate = torch.randn(d_ff, d_model, generator=gen) * std
    up = torch.randn(d_ff, d_model, generator=gen) * std
    down = torch.randn(d_ff, d_model, generator=gen) * std
    rates = neuron_rates(d_ff, density, skew_sigma, gen)
    k_eff = d_model - 1 if fold_bias else d_model
    sigma = std * math.sqrt(k_eff)  # std of the pre-activation for x ~ N(0, 1)
    shift = (sigma * torch.special.ndtri(rates)).to(torch.float32)
    bias = None
    if fold_bias:
        gate[:, 0] = shift
    else:
        bias = shift.to(device)
    return SparseFFN(gate.to(dtype).to(device), up.to(dtype).to(device),
                     down.to(dtype).to(device), bias, rates.float(), fold_bias)


def make_tokens(m: int, d_model: int, *, seed: int = 1, fold_bias: bool = True,
                dtype: torch.dtype = torch.bfloat16, device="cpu") -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(m, d_model, generator=gen)
    if fold_bias:
        x[:, 0] = 1.0
    return x.to(dtype).to(device)


def dyadic_case(m: int, d_model: int, d_ff: int, *, seed: int = 0, device="cpu"):
    """Inputs on a coarse dyadic grid: every fp32 partial sum of x.w is exact.

    x in {-2..2}/2, w in {-4..4}/64 (both exactly representable in bf16) and
    |sum| < 2^24 ulp-units, so any summation order gives the same fp32 result and
    TwELL counts / indices / values must match an oracle bit for bit.
    """
    gen = torch.Generator().manual_seed(seed)
    x = torch.randint(-2, 3, (m, d_model), generator=gen).float() / 2
    gate = torch.randint(-4, 5, (d_ff, d_model), generator=gen).float() / 64
    # shift towards sparsity: most pre-activations negative
    # feature 0 carries a negative shift of about two standard deviations of the
    # remaining sum (a multiple of 1/2, exactly representable)
    sigma = math.sqrt((d_model - 1) * 0.5 * (60.0 / 9.0) / 4096.0)
    gate[:, 0] = -max(0.5, round(4.0 * sigma) / 2.0)
    x[:, 0] = 1.0
    up = torch.randint(-4, 5, (d_ff, d_model), generator=gen).float() / 64
    down = torch.randint(-4, 5, (d_ff, d_model), generator=gen).float() / 64
    bf = torch.bfloat16
    return (x.to(bf).to(device), gate.to(bf).to(device), up.to(bf).to(device),
            down.to(bf).to(device))
