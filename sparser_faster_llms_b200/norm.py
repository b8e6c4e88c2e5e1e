"""Residual add + RMSNorm around the sparse FFN, as one kernel for decode-sized calls.

``residual_rmsnorm(x, delta, weight, eps)`` returns ``(x + delta, rmsnorm(x + delta) * weight)``
from one launch of ``b200_residual_rmsnorm`` (``delta=None``: the norm alone).  In a decoder
layer these are the steps between the attention block and the FFN and between the FFN and the
next layer; in eager torch each is a launch of its own, which at decode sizes costs as much as
the FFN kernels themselves.  bf16 CUDA tensors ``[..., D]``; there is no CPU implementation
(:func:`reference` is the same function in plain torch, for tests and CPU callers).
"""
from __future__ import annotations

import torch

from . import _lib


def reference(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float):
    """The same function in plain torch (fp32 inside, bf16-rounded sum first)."""
    s = x if delta is None else (x.float() + delta.float()).to(x.dtype)
    f = s.float()
    n = (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
    return s, (n.float() * weight.float()).to(x.dtype)


def residual_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor,
                     eps: float, *, inplace: bool = False):
    """``(x_out, h)`` with ``x_out = x + delta`` (written into ``x`` when ``inplace``) and
    ``h = rmsnorm(x_out) * weight``."""
    if not x.is_cuda:
        raise RuntimeError("residual_rmsnorm needs CUDA tensors (use norm.reference on CPU)")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise RuntimeError("residual_rmsnorm: x and weight must be bfloat16")
    d = x.shape[-1]
    if weight.shape != (d,):
        raise ValueError(f"weight must have shape [{d}]")
    if delta is not None and (delta.shape != x.shape or delta.dtype != x.dtype):
        raise ValueError("delta must have x's shape and dtype")
    xc = x if x.is_contiguous() else x.contiguous()
    dc = None if delta is None else (delta if delta.is_contiguous() else delta.contiguous())
    h = torch.empty_like(xc)
    if delta is None:
        x_out = xc
        out_ptr = None
    else:
        x_out = xc if inplace and xc is x else torch.empty_like(xc)
        out_ptr = x_out.data_ptr()
    _lib.call("b200_residual_rmsnorm", x.device, xc.data_ptr(), _lib.ptr(dc),
              weight.contiguous().data_ptr(), float(eps), out_ptr, h.data_ptr(),
              xc.numel() // d, d)
    return x_out, h
