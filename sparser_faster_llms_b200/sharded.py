"""d_ff-sharded sparse gated FFN: one process per GPU, one all-reduce on the output.

In the TwELL layout all three weights are ``[H, D]`` (reference:
custom_models/sparse_testing_utils.py:26-28), so a d_ff shard is the same
contiguous row range ``[h0, h1)`` of GATE, UP and DOWN.  Shard boundaries are
multiples of 256 neurons (one TwELL tile); shards may be uneven (11008 = 43 tiles).
Every rank packs and contracts its own shard with *local* column indices and
produces a partial ``y_r [M, D]``; the partials are summed with a single
all-reduce.  The reference has no tensor parallelism (data parallel only), so
this module has no counterpart there.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist
from torch import nn

TILE = 256


def shard_range(d_ff: int, rank: int, world_size: int) -> tuple[int, int]:
    """Row range ``[h0, h1)`` of ``rank``: tile-granular, contiguous, sizes differ by at most
    one tile, earlier ranks take the larger shards."""
    if d_ff % TILE:
        raise ValueError(f"d_ff must be a multiple of {TILE}")
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside 0..{world_size - 1}")
    tiles = d_ff // TILE
    if tiles < world_size:
        raise ValueError(f"d_ff={d_ff} has {tiles} tiles, fewer than world_size={world_size}")
    base, rem = divmod(tiles, world_size)
    start = rank * base + min(rank, rem)
    n = base + (1 if rank < rem else 0)
    return start * TILE, (start + n) * TILE


def shard_weights(GATE: torch.Tensor, UP: torch.Tensor, DOWN: torch.Tensor, rank: int,
                  world_size: int):
    """This rank's contiguous copies of the three ``[H, D]`` weights."""
    h = UP.shape[0]
    if DOWN.shape[0] != h or (GATE is not None and GATE.shape[0] != h):
        raise ValueError("GATE / UP / DOWN must all be [H, D] (DOWN = down_proj.weight.T)")
    h0, h1 = shard_range(h, rank, world_size)
    g = None if GATE is None else GATE[h0:h1].contiguous()
    return g, UP[h0:h1].contiguous(), DOWN[h0:h1].contiguous()


class _CopyToShards(torch.autograd.Function):
    """Identity in forward (x is replicated); sums the ranks' input gradients in backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        acc = g.float() if g.dtype != torch.float32 else g.clone()
        dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=ctx.group)
        return acc.to(g.dtype), None


class _ReduceFromShards(torch.autograd.Function):
    """Sums the ranks' partial results in forward; the gradient passes through unchanged
    (every rank holds the same upstream gradient of the replicated sum)."""

    @staticmethod
    def forward(ctx, y, group):
        y = y.contiguous()
        acc = y.float() if y.dtype != torch.float32 else y.clone()
        dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=group)
        return acc.to(y.dtype)

    @staticmethod
    def backward(ctx, g):
        return g, None


def sharded_ff_gated(X: torch.Tensor, G: torch.Tensor, K: torch.Tensor, V: torch.Tensor, *,
                     process_group=None, local_op: Callable | None = None):
    """Training forward of the hybrid operator over a d_ff shard; differentiable.

    ``G/K/V`` are this rank's ``[H_local, D]`` rows (see :func:`shard_weights`), ``X [B,S,D]`` is
    replicated.  Returns ``(out, l0, l1)`` equal on every rank: ``out`` and the two sparsity
    statistics are sums over neurons, hence additive across shards (l0 = sum over neurons of
    the firing rate, l1 = mean over tokens of sum |T|; custom_op.cpp:120-133), so the forward
    needs one all-reduce of ``out`` and one of each scalar, the backward one all-reduce of
    ``dX``; weight gradients stay shard-local.  ``local_op(X, G, K, V)`` returns at least
    ``(out, l0, l1)`` and defaults to ``torch.ops.sparse_ops.ff_forward_gated``.  The
    reference trains data-parallel only and has no counterpart.
    """
    if local_op is None:
        from .sparse_ops import register_ops
        register_ops()
        local_op = torch.ops.sparse_ops.ff_forward_gated
    single = not dist.is_initialized() or dist.get_world_size(process_group) == 1
    Xs = X if single else _CopyToShards.apply(X, process_group)
    out, l0, l1 = local_op(Xs, G, K, V)[:3]
    if single:
        return out, l0, l1
    return (_ReduceFromShards.apply(out, process_group),
            _ReduceFromShards.apply(l0, process_group),
            _ReduceFromShards.apply(l1, process_group))


class ShardedTwELLGatedMLP(nn.Module):
    """``TwELLGatedMLP`` over a d_ff shard plus the all-reduce of the FFN output.

    ``GATE/UP/DOWN`` are the FULL ``[H, D]`` weights unless ``presharded=True``.
    ``local_factory(layer_number, GATE, UP, DOWN, **kwargs)`` builds the per-rank module; it
    defaults to :class:`sparser_faster_llms_b200.twell.TwELLGatedMLP` (CUDA only).
    """

    def __init__(self, layer_number: int, GATE: torch.Tensor, UP: torch.Tensor,
                 DOWN: torch.Tensor, *, process_group=None, rank: int | None = None,
                 world_size: int | None = None, presharded: bool = False,
                 reduce_dtype: torch.dtype | None = None, peer_allreduce=None,
                 fused_allreduce=None,
                 local_factory: Callable[..., nn.Module] | None = None, **twell_kwargs):
        super().__init__()
        self.process_group = process_group
        # optional sparser_faster_llms_b200.peer_allreduce.FusedShardAllReduce shared by all
        # layers: decode-sized calls sum the shards inside the contraction kernel; other calls
        # fall back to peer_allreduce / NCCL below
        self.fused_allreduce = fused_allreduce
        # optional sparser_faster_llms_b200.peer_allreduce.PeerAllReduce shared by all layers:
        # one peer-memory kernel instead of an NCCL all-reduce (bf16 sum, rank order)
        self.peer_allreduce = peer_allreduce
        if world_size is None:
            world_size = dist.get_world_size(process_group) if dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.rank, self.world_size = int(rank), int(world_size)
        self.d_ff = int(UP.shape[0]) if not presharded else None
        if presharded:
            g, u, d = GATE.contiguous(), UP.contiguous(), DOWN.contiguous()
            self.h_range = None
        else:
            g, u, d = shard_weights(GATE, UP, DOWN, self.rank, self.world_size)
            self.h_range = shard_range(UP.shape[0], self.rank, self.world_size)
        if local_factory is None:
            from .twell import TwELLGatedMLP
            local_factory = TwELLGatedMLP
        self.local = local_factory(layer_number, g, u, d, **twell_kwargs)
        self.reduce_dtype = reduce_dtype
        self.last_route = None  # how the last forward summed the shards: fused / peer / nccl

    def _fused_ready(self, A: torch.Tensor) -> bool:
        """Attach the fused all-reduce to the local layer's cached state (created on the first
        forward, re-created when the module is moved) and say whether it serves this call."""
        far = self.fused_allreduce
        if far is None or self.world_size == 1:
            return False
        tokens = A.numel() // A.shape[-1]
        if not far.serves(tokens, A.shape[-1]):
            return False
        from . import twell
        entry = twell._D2T_LAYERS.get(int(getattr(self.local, "layer_number", -1)))
        if entry is None:
            return False  # first forward: the layer state does not exist yet
        entry["fused_allreduce"] = far
        return True

    def forward(self, A: torch.Tensor) -> torch.Tensor:
        if self._fused_ready(A):
            try:
                self.last_route = "fused"
                return self.local(A)  # the contraction's epilogue has already summed the shards
            except ValueError as exc:
                # the library refuses a fused call whose grid is not resident at once (the same
                # decision on every rank: identical GPUs); such calls take the unfused route
                if "fused all-reduce" not in str(exc):
                    raise
        if self.fused_allreduce is not None:
            from . import twell
            entry = twell._D2T_LAYERS.get(int(getattr(self.local, "layer_number", -1)))
            if entry is not None:
                entry.pop("fused_allreduce", None)  # a call the fused form does not serve
        y = self.local(A)
        par = self.peer_allreduce
        if (self.world_size > 1 and par is not None
                and y.numel() * y.element_size() <= getattr(par, "max_bytes", float("inf"))):
            self.last_route = "peer"
            return par.all_reduce(y.contiguous())  # larger outputs (prefill) go through NCCL
        self.last_route = "nccl" if self.world_size > 1 else "local"
        if self.world_size > 1:
            if self.reduce_dtype is not None and self.reduce_dtype != y.dtype:
                acc = y.to(self.reduce_dtype)
                dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.process_group)
                y = acc.to(y.dtype)
            else:
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.process_group)
        return y

    def check_status(self) -> int:
        """Error words of the peer-memory all-reduces this module uses: 0, or ``0x100 + peer``
        if a bounded wait for that peer gave up since the last check (the sums of such a call
        are invalid).  Reads and clears the words and synchronises the device, so call it once
        per step, not per layer.  After a non-zero status the module stops using the peer
        kernels and sums through the process group (NCCL) from the next call on."""
        status = 0
        for obj in (self.fused_allreduce, self.peer_allreduce):
            if obj is not None and getattr(obj, "block", None) is not None:
                status = status or int(obj.status())
        if status:
            self.fused_allreduce = None
            self.peer_allreduce = None
            from . import twell
            entry = twell._D2T_LAYERS.get(int(getattr(self.local, "layer_number", -1)))
            if entry is not None:
                entry.pop("fused_allreduce", None)
        return status

    def destroy(self) -> None:
        if hasattr(self.local, "destroy"):
            self.local.destroy()
