"""Latency of the shard-sum kernels under CUDA-graph replay (torchrun, N ranks of one node).

``python -m torch.distributed.run --nproc-per-node N -m sparser_faster_llms_b200.allreduce_bench``
prints one JSON line per message size (rank 0): microseconds per call of

* ``peer_us``   ``b200_peer_allreduce_bf16`` (one-shot push into every peer's inbox),
* ``nccl_us``   ``torch.distributed.all_reduce`` (NCCL) on the same tensor,
* ``fused_contraction_us`` / ``contraction_plus_peer_us``  (sizes of at most 256 tokens of
  d_model 2048) the gated contraction of a d_ff shard with the shard sum in its epilogue
  (``b200_twell_gated_t2d_allreduce``) against the plain contraction followed by the peer
  all-reduce,

and the bytes a rank pushes over NVLink per call: ``2 * (N - 1) * payload`` (every 4-byte
payload word travels with a 4-byte epoch word).  Each figure is the maximum over ranks of a
CUDA-event time over 5 replays of a graph holding 200 calls.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

from . import _lib, peer_allreduce, synthetic, twell


def _graph_us(fn, dev, calls: int = 200, replays: int = 5) -> float:
    s = torch.cuda.Stream(dev)
    s.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(s):
        for _ in range(3):
            fn()
    torch.cuda.current_stream(dev).wait_stream(s)
    torch.cuda.synchronize(dev)
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(calls):
            fn()
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize(dev)
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([e0.elapsed_time(e1) / (replays * calls) * 1e3], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    d, h_full = 2048, 8192
    par = peer_allreduce.PeerAllReduce(512 * 1024, device=dev)
    far = peer_allreduce.FusedShardAllReduce(32, d, device=dev)
    lib = _lib.load_library()
    hs = h_full // world
    ffn = synthetic.make_ffn(d, hs, seed=3 + rank, density=0.02, skew_sigma=1.0)
    up, down, gate = ffn.up.to(dev), ffn.down.to(dev), ffn.gate.to(dev)
    ws = torch.zeros(int(lib.b200_workspace_bytes()), dtype=torch.uint8, device=dev)
    for tokens in (1, 8, 32, 128):
        n = tokens * d
        x = torch.randn(n, device=dev).to(torch.bfloat16)
        y = torch.empty_like(x)
        z = x.clone()
        rec = {"n_gpus": world, "payload_bytes": n * 2,
               "nvlink_bytes_pushed_per_rank": 2 * (world - 1) * n * 2,
               "peer_us": _graph_us(lambda: par.all_reduce(x, y), dev),
               "nccl_us": _graph_us(lambda: dist.all_reduce(z), dev)}
        if far.serves(tokens, d):
            xt = synthetic.make_tokens(tokens, d, seed=9).to(dev)
            packed = twell.matmul_sparse(xt, gate)
            out = torch.empty_like(xt)
            part = torch.empty_like(xt)

            def fused():
                _lib.call("b200_twell_gated_t2d_allreduce", dev, xt.data_ptr(), packed.data_ptr(),
                          up.data_ptr(), down.data_ptr(), out.data_ptr(), tokens, d, hs, 8, 0,
                          ws.data_ptr(), ws.numel(), far.ptr_array, far.rank, far.world,
                          far.block_bytes)

            def two():
                _lib.call("b200_twell_gated_t2d", dev, xt.data_ptr(), packed.data_ptr(),
                          up.data_ptr(), down.data_ptr(), part.data_ptr(), tokens, d, hs, 8, 0,
                          ws.data_ptr(), ws.numel())
                par.all_reduce(part, out)

            rec["fused_contraction_us"] = _graph_us(fused, dev)
            rec["contraction_plus_peer_us"] = _graph_us(two, dev)
        rec["status"] = [par.status(), far.status()]
        if rank == 0:
            print(json.dumps(rec), flush=True)
    par.fused = far
    par.close()
    torch.cuda.synchronize(dev)
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
