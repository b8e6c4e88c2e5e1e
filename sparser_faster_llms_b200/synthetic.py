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
             dtype: torch.dtype = torch.bfloat16, device="cpu",
             generate_on_device: bool = False) -> SparseFFN:
    """``generate_on_device`` draws the three matrices with the device's own generator (much
    faster for model-sized stacks; another random stream than the CPU one, same statistics)."""
    gen = torch.Generator().manual_seed(seed)
    if generate_on_device and torch.device(device).type == "cuda":
        dgen = torch.Generator(device=device).manual_seed(seed)
        gate, up, down = (torch.randn(d_ff, d_model, generator=dgen, device=device) * std
                          for _ in range(3))
    else:
        gate = torch.randn(d_ff, d_model, generator=gen) * std
        up = torch.randn(d_ff, d_model, generator=gen) * std
        down = torch.randn(d_ff, d_model, generator=gen) * std
    rates = neuron_rates(d_ff, density, skew_sigma, gen)
    k_eff = d_model - 1 if fold_bias else d_model
    sigma = std * math.sqrt(k_eff)  # std of the pre-activation for x ~ N(0, 1)
    shift = (sigma * torch.special.ndtri(rates)).to(torch.float32)
    bias = None
    if fold_bias:
        gate[:, 0] = shift.to(gate.device)
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


def make_tokens_mixed_density(m: int, d_model: int, *, base_density: float, seed: int = 1,
                              beta: tuple[float, float] = (2.0, 60.0),
                              dense_fraction: float = 0.05,
                              dense_range: tuple[float, float] = (0.2, 0.4),
                              dtype: torch.dtype = torch.bfloat16, device="cpu"):
    """Tokens whose gate density differs per token (prefill-like mix): most tokens draw their
    density from ``Beta(*beta)``, a ``dense_fraction`` of them from ``U(*dense_range)``.

    Works with a bias-folded FFN built for ``base_density`` (uniform neuron rates): the
    per-neuron shift lives in ``gate[:, 0]`` and is multiplied by token feature 0, so feature 0
    of token t is set to ``q(rho_t) / q(base_density)`` with ``q`` the Gaussian upper quantile.
    Returns ``(x, rho)`` with ``rho`` the target density per token (fp32, CPU).
    """
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(m, d_model, generator=gen)
    a = torch.distributions.Gamma(torch.tensor(beta[0]), torch.tensor(1.0))
    b = torch.distributions.Gamma(torch.tensor(beta[1]), torch.tensor(1.0))
    torch.manual_seed(seed + 7919)  # the Gamma sampler has no generator argument
    ga, gb = a.sample((m,)), b.sample((m,))
    rho = (ga / (ga + gb)).double()
    dense = torch.rand(m, generator=gen) < dense_fraction
    lo, hi = dense_range
    rho = torch.where(dense, lo + (hi - lo) * torch.rand(m, generator=gen).double(), rho)
    rho = rho.clamp(1e-4, 0.49)
    q = torch.special.ndtri(1.0 - rho) / torch.special.ndtri(torch.tensor(1.0 - base_density,
                                                                          dtype=torch.float64))
    x[:, 0] = q.float()
    return x.to(dtype).to(device), rho.float()


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
