"""Run a list of sparse FFN modules as one CUDA graph (decode serving helper).

At decode batch sizes one sparse FFN layer takes 10-30 microseconds on a B200, less than
the host needs to issue its two launches from Python.  ``GraphedFFNStack`` captures
"host input -> device, every layer's fused gated MLP, result -> host" once and replays it,
so a step costs one graph launch.  The modules are ordinary
:class:`sparser_faster_llms_b200.twell.TwELLGatedMLP` objects (the reference's module
surface); nothing about them changes.

This helper has no counterpart in the reference, whose benchmark launches eagerly
(benchmark_inference.py:295-326).
"""
from __future__ import annotations

import torch

from . import _lib


class GraphedFFNStack:
    """``y[l] = mlps[l](x[l])`` for all layers, replayed as a single CUDA graph.

    ``run(x_host)`` takes a pinned host tensor ``[L, B, D]`` (bf16) and returns a pinned
    host tensor: all layer outputs ``[L, B, D]`` or, with ``return_last_only``, the last
    layer's ``[B, D]``.  The returned tensor is reused by the next call.
    """

    def __init__(self, mlps, batch: int, *, return_last_only: bool = False,
                 device: torch.device | str | None = None, copy_chunk: int = 4):
        self.mlps = list(mlps)
        if not self.mlps:
            raise ValueError("need at least one module")
        first = getattr(self.mlps[0], "local", self.mlps[0])  # d_ff-sharded modules wrap one
        dev = torch.device(device) if device is not None else first.GATE.device
        if dev.type != "cuda":
            raise RuntimeError("GraphedFFNStack needs CUDA modules (there is no CPU path)")
        self.device = dev
        self.layers = len(self.mlps)
        self.batch = int(batch)
        self.d_model = int(first.GATE.shape[1])
        self.return_last_only = bool(return_last_only)
        shape = (self.layers, self.batch, self.d_model)
        self.x_dev = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        self.y_dev = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        self.x_host = torch.zeros(shape, dtype=torch.bfloat16).pin_memory()
        out_shape = shape[1:] if self.return_last_only else shape
        self.y_host = torch.zeros(out_shape, dtype=torch.bfloat16).pin_memory()
        self.stream = torch.cuda.Stream(dev)
        self.copy_stream = torch.cuda.Stream(dev)
        self.copy_chunk = max(1, int(copy_chunk))
        self.graph: torch.cuda.CUDAGraph | None = None
        self._capture()

    def _body(self) -> None:
        # The host -> device copies run on a second stream in chunks of a few layers, each
        # chunk followed by an event the compute stream waits on: layer l starts as soon as
        # its own input has arrived, and the rest of the transfer hides under the kernels.
        # The first chunk is a single layer, so the compute stream starts after one small copy.
        main = torch.cuda.current_stream(self.device)
        self.copy_stream.wait_stream(main)
        bounds = [0, 1] + list(range(1 + self.copy_chunk, self.layers, self.copy_chunk))
        bounds = [b for b in bounds if b < self.layers] + [self.layers]
        ready = {}
        with torch.cuda.stream(self.copy_stream):
            for l0, l1 in zip(bounds[:-1], bounds[1:]):
                self.x_dev[l0:l1].copy_(self.x_host[l0:l1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
                ready[l0] = ev
        for l, mlp in enumerate(self.mlps):
            if l in ready:
                main.wait_event(ready[l])
            y = mlp(self.x_dev[l])
            # only what is returned is gathered: with return_last_only the last layer's
            # output goes to the host straight from the module's own tensor
            if not self.return_last_only and y.data_ptr() != self.y_dev[l].data_ptr():
                self.y_dev[l].copy_(y)
        main.wait_stream(self.copy_stream)
        src = y.view(self.batch, self.d_model) if self.return_last_only else self.y_dev
        self.y_host.copy_(src, non_blocking=True)

    def _capture(self) -> None:
        with torch.cuda.device(self.device):
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                _lib.workspace(self.device)  # create this stream's workspace outside capture
                for _ in range(2):           # lazy per-layer state, allocator warm-up
                    self._body()
            self.stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream):
                self._body()
            self.graph = graph

    def run(self, x_host: torch.Tensor | None = None) -> torch.Tensor:
        """Copy ``x_host`` into the pinned staging buffer (unless it *is* the staging buffer or
        None), replay the graph, wait for the result."""
        if x_host is not None and x_host.data_ptr() != self.x_host.data_ptr():
            if tuple(x_host.shape) != tuple(self.x_host.shape) or x_host.dtype != torch.bfloat16:
                raise ValueError(f"x_host must be bf16 of shape {tuple(self.x_host.shape)}")
            self.x_host.copy_(x_host)
        with torch.cuda.stream(self.stream):
            self.graph.replay()
        self.stream.synchronize()
        return self.y_host
