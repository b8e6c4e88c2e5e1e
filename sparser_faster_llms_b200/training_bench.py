"""Hybrid sparse FFN training step (forward + backward) of one 0.5B-shape layer, optionally
d_ff-sharded over the ranks of a torchrun launch.

``python -m sparser_faster_llms_b200.training_bench`` (1 GPU) or
``python -m torch.distributed.run --nproc-per-node N -m sparser_faster_llms_b200.training_bench``
prints one JSON line (rank 0): milliseconds for forward, backward and both of

* ``sparse``  ``torch.ops.sparse_ops.ff_forward_gated`` + its backward (this package's
  kernels; with N > 1 through :func:`sharded.sharded_ff_gated`: all-reduce of out / l0 / l1
  forward and of dX backward), loss = ``sum(out * W) + l1_coeff * l1``;
* ``dense``   the same function through torch autograd and cuBLAS bf16 on one GPU (the
  unsharded layer), as the comparison point.

Layer: D = 1024, d_ff = 4096, 8 x 2048 tokens (the 24-layer 0.5B configuration's FFN),
weights ~N(0, 0.02), gate density set by the folded shift of :mod:`synthetic` (default 1 %,
about the L0 of 41 at which the reference switches a layer to the hybrid kernel,
cfgs/run_cfg/sparsity_gated_hybrid_0p5b.yaml:56-61).  CUDA events, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from . import sharded, sparse_ops, synthetic


def _time(fn, reps: int, warmup: int, device) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) / reps


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--d-model", type=int, default=1024)
    ap.add_argument("--d-ff", type=int, default=4096)
    ap.add_argument("--density", type=float, default=0.01)
    ap.add_argument("--l1-coeff", type=float, default=3e-4)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--adaptive-tail", type=int, default=1,
                    help="1: size the dense tail from the overflow rows seen on earlier calls "
                         "(sparse_ops.set_tail_rows_adaptive); 0: always tail_rows_regular rows")
    ap.add_argument("--tail-rows", type=int, default=2048)
    ap.add_argument("--wgrad", default="auto", choices=["auto", "sparse", "dense"],
                    help="weight-gradient form (sparse_ops.set_weight_gradient_mode)")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sparse_ops.register_ops()
    sparse_ops.set_tail_rows_adaptive(bool(args.adaptive_tail))
    sparse_ops.set_weight_gradient_mode(args.wgrad)
    torch.ops.sparse_ops_config.set_tail_rows_regular(args.tail_rows)
    b, s, d, h = args.batch, args.seq, args.d_model, args.d_ff
    ffn = synthetic.make_ffn(d, h, seed=21, density=args.density, skew_sigma=1.0)
    x = synthetic.make_tokens(b * s, d, seed=22).view(b, s, d).to(dev).requires_grad_(True)
    w = torch.randn(b, s, d, generator=torch.Generator().manual_seed(23)).to(torch.bfloat16).to(dev)
    g_full, k_full, v_full = ffn.gate.to(dev), ffn.up.to(dev), ffn.down.to(dev)
    g, k, v = (t.clone().requires_grad_(True)
               for t in sharded.shard_weights(g_full, k_full, v_full, rank, world))

    def sparse_forward():
        out, l0, l1 = sharded.sharded_ff_gated(x, g, k, v)
        return (out.float() * w.float()).sum() + args.l1_coeff * l1, l0

    def sparse_step():
        loss, _ = sparse_forward()
        loss.backward()
        for t in (x, g, k, v):
            t.grad = None

    gd, kd, vd = (t.clone().requires_grad_(True) for t in (g_full, k_full, v_full))

    def dense_forward():
        gate = torch.relu(x @ gd.T)
        t = gate * (x @ kd.T)
        return ((t @ vd).float() * w.float()).sum() + args.l1_coeff * t.float().abs().sum() / (b * s)

    def dense_step():
        dense_forward().backward()
        for t in (x, gd, kd, vd):
            t.grad = None

    res = {}
    for name, fwd, step in (("sparse", lambda: sparse_forward()[0], sparse_step),
                            ("dense", dense_forward, dense_step)):
        if name == "dense" and rank != 0:
            continue  # the comparison point is the unsharded layer on one GPU
        with torch.no_grad():
            t_f = _time(fwd, args.reps, args.warmup, dev)
        t_fb = _time(step, args.reps, args.warmup, dev)
        res[name] = {"forward_ms": t_f, "forward_backward_ms": t_fb, "backward_ms": t_fb - t_f}
    _, l0 = sparse_forward()
    # dead-neuron bookkeeping of this rank's neuron shard (shard-local: no exchange needed)
    with torch.no_grad():
        _, _, _, p_slab, _, t_slab = torch.ops.sparse_ops.ff_forward_gated(x.detach(), g, k, v)
        last = torch.zeros(g.shape[0], dtype=torch.int64, device=dev)
        res["sparse"]["dead_neuron_bookkeeping_ms"] = _time(
            lambda: sparse_ops.neuron_activity(p_slab, t_slab, last, b * s),
            args.reps, args.warmup, dev)
    if world > 1:
        t = torch.tensor([res["sparse"]["forward_ms"], res["sparse"]["forward_backward_ms"]],
                         device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res["sparse"]["forward_ms"], res["sparse"]["forward_backward_ms"] = t.tolist()
        res["sparse"]["backward_ms"] = res["sparse"]["forward_backward_ms"] - res["sparse"]["forward_ms"]
    if rank == 0:
        tokens = b * s
        print(json.dumps({
            "n_gpus": world, "tokens": tokens, "d_model": d, "d_ff": h, "l0_per_token": float(l0),
            "dtype": "bf16", "data": "synthetic", "adaptive_tail": bool(args.adaptive_tail),
            "tail_rows": args.tail_rows, **res,
            "sparse_tokens_per_s": tokens / (res["sparse"]["forward_backward_ms"] * 1e-3),
            "dense_tokens_per_s": tokens / (res["dense"]["forward_backward_ms"] * 1e-3)}), flush=True)
    if world > 1:
        torch.cuda.synchronize(dev)
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
