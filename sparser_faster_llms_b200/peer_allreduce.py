"""Low-latency sum all-reduce over peer-mapped memory for the d_ff-sharded FFN output.

``PeerAllReduce`` owns one symmetric block per rank (torch symmetric memory provides the
peer mapping) and launches ``b200_peer_allreduce_bf16``: one kernel per rank that pushes
the local partial into every peer's inbox, flags, waits (bounded) and sums in rank order.
At decode sizes (4..128 KB) this replaces an NCCL all-reduce whose latency is larger than
the sharded FFN itself.  One object serves every layer of a model: its inbox is
double-buffered by a device-side epoch, and the launch is safe to capture in a CUDA graph.

The kernels use plain peer stores and local loads only.  torch's symmetric-memory
rendezvous would by default also bind the block to an NVLink multicast object on NVSwitch
machines; that binding buys these kernels nothing and a rank that exits while bound can
raise NVLink faults on its peers, so ``_disable_symm_mem_multicast()`` switches it off
(``TORCH_SYMM_MEM_DISABLE_MULTICAST=1``) before the first symmetric allocation of the
process.  ``NCCL_NVLS_ENABLE`` only governs NCCL's own collectives.  Call ``close()`` on
these objects (then synchronise) before the process leaves, so no mapping of a peer's
memory is still held at exit.  A missing peer shows up as a non-zero ``status()``; the
error word is sticky: after it is set, later waits give up after a short spin until
``status()`` has read and cleared it.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib


def _disable_symm_mem_multicast() -> None:
    """Keep torch symmetric memory from binding blocks to an NVLink multicast object."""
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


class FusedShardAllReduce:
    """Peer blocks for the contraction that sums the d_ff shards in its own epilogue
    (``b200_twell_gated_mlp_allreduce``): one kernel per rank computes the shard's FFN output,
    exchanges bf16 pairs with the peers and stores the sum.  Decode-sized calls only
    (``max_tokens`` <= 256 and a single wave of CTAs); attach it to a layer with
    :func:`sparser_faster_llms_b200.twell.set_d2t_layer_fused_allreduce` or pass it to
    :class:`sparser_faster_llms_b200.sharded.ShardedTwELLGatedMLP`.  One object serves all
    layers of a model; keep it separate from any :class:`PeerAllReduce` (own epochs, own inbox).
    """

    def __init__(self, max_tokens: int, d_model: int, *, group=None,
                 device: torch.device | None = None):
        _disable_symm_mem_multicast()
        import torch.distributed._symmetric_memory as symm_mem
        if not dist.is_initialized():
            raise RuntimeError("FusedShardAllReduce needs an initialised process group")
        if not 0 < max_tokens <= 256:
            raise ValueError("max_tokens must be in 1..256")
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("FusedShardAllReduce supports at most 8 ranks (one node)")
        self.device = device if device is not None else torch.device("cuda",
                                                                     torch.cuda.current_device())
        self.max_tokens, self.d_model = int(max_tokens), int(d_model)
        lib = _lib.load_library()
        self.block_bytes = int(lib.b200_fused_allreduce_block_bytes(self.max_tokens, self.d_model))
        self.block = symm_mem.empty(self.block_bytes, dtype=torch.uint8, device=self.device)
        self.block.zero_()
        self.handle = symm_mem.rendezvous(self.block, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != self.world:
            raise RuntimeError("symmetric memory returned an unexpected number of peers")
        self.ptr_array = (ctypes.c_void_p * self.world)(*ptrs)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every block is zeroed before anyone may push into it

    def serves(self, tokens: int, d_model: int) -> bool:
        return (self.block is not None and tokens <= self.max_tokens
                and d_model == self.d_model)

    def close(self) -> None:
        """Release the symmetric block and the peer mappings (idempotent).  Call on every
        rank between steps, with no kernel of this object in flight."""
        if self.block is not None:
            torch.cuda.synchronize(self.device)
        self.handle = None
        self.block = None
        self.ptr_array = None

    def status(self) -> int:
        """0, or ``0x100 + peer`` if a wait for that peer gave up.  Synchronises the device."""
        with torch.cuda.device(self.device):
            return int(_lib.load_library().b200_fused_allreduce_status(self.block.data_ptr()))


class PeerAllReduce:
    def __init__(self, max_bytes: int, *, group=None, device: torch.device | None = None):
        _disable_symm_mem_multicast()
        import torch.distributed._symmetric_memory as symm_mem
        if not dist.is_initialized():
            raise RuntimeError("PeerAllReduce needs an initialised process group")
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("PeerAllReduce supports at most 8 ranks (one node)")
        self.device = device if device is not None else torch.device("cuda",
                                                                     torch.cuda.current_device())
        lib = _lib.load_library()
        self.max_bytes = int(max_bytes)
        self.block_bytes = int(lib.b200_peer_allreduce_block_bytes(self.max_bytes))
        self.block = symm_mem.empty(self.block_bytes, dtype=torch.uint8, device=self.device)
        self.block.zero_()
        self.handle = symm_mem.rendezvous(self.block, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != self.world:
            raise RuntimeError("symmetric memory returned an unexpected number of peers")
        self._ptr_array = (ctypes.c_void_p * self.world)(*ptrs)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every block is zeroed before anyone may push into it

    def all_reduce(self, local_in: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``out = sum over ranks of local_in`` (bf16, contiguous, numel % 8 == 0).
        ``out`` must not alias ``local_in``."""
        if local_in.dtype != torch.bfloat16 or not local_in.is_contiguous():
            raise ValueError("local_in must be a contiguous bfloat16 tensor")
        if out is None:
            out = torch.empty_like(local_in)
        elif out.data_ptr() == local_in.data_ptr():
            raise ValueError("out must not alias local_in")
        n = local_in.numel()
        if n * 2 > self.max_bytes:
            raise ValueError(f"{n * 2} bytes exceed this PeerAllReduce's max_bytes={self.max_bytes}")
        _lib.call("b200_peer_allreduce_bf16", self.device, local_in.data_ptr(), out.data_ptr(), n,
                  self._ptr_array, self.rank, self.world, self.block_bytes)
        return out

    def status(self) -> int:
        """0, or ``0x100 + peer`` if a wait for that peer gave up.  Synchronises the device."""
        with torch.cuda.device(self.device):
            return int(_lib.load_library().b200_peer_allreduce_status(self.block.data_ptr()))

    def close(self) -> None:
        """Release the symmetric block and the peer mappings (idempotent).  Call on every
        rank between steps, with no kernel of this object in flight."""
        if self.block is not None:
            torch.cuda.synchronize(self.device)
        fused = getattr(self, "fused", None)
        if fused is not None:
            fused.close()
        self.handle = None
        self.block = None
        self._ptr_array = None
