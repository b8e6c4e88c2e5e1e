"""Kernel sweep on one sparse FFN layer: token count x gate density x neuron-rate skew.

``python -m sparser_faster_llms_b200.sweep_bench [--d-model 4096] [--d-ff 16384]
[--tokens 1,16,128,1024,16384] [--densities 0.005,0.01,0.02,0.05,0.1,0.3] [--skews 0,1]``
prints one JSON line per point with the time of

* ``pack``      gate projection + ReLU + TwELL pack,
* ``sparse``    pack + gather contraction (the TwELL path),
* ``routed``    pack + hybrid contraction (rows over ``d_ff/64`` positives or with an
  overflowed tile on the dense tcgen05 route; only from 128 tokens on),
* ``dense_all`` both dense tcgen05 GEMMs, no slab (only from 128 tokens on),
* ``cublas``    the dense bf16 formula through torch / cuBLAS,

the fastest of them, the pack kernel's HBM or tensor roofline fraction (bytes ``2 D H`` or
flops ``2 M D H`` against the peaks given on the command line) and each path's relative L2
error against the cuBLAS result.  Weights ~N(0, 0.02), Gaussian tokens, the density set by a
per-neuron shift folded into feature 0; log-normal neuron rates when skew > 0.  With cf = 8 a
slab holds 31 of 256 neurons, so from about 10 % density on the gather path drops entries
(visible in its error) and only the routed / dense paths stay exact.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import synthetic, twell


def _time(fn, reps: int, warmup: int = 2) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3  # microseconds


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--d-ff", type=int, default=16384)
    ap.add_argument("--tokens", default="1,16,128,1024,16384")
    ap.add_argument("--densities", default="0.005,0.01,0.02,0.05,0.1,0.3")
    ap.add_argument("--skews", default="0,1")
    ap.add_argument("--hbm-gbs", type=float, default=6552.6)
    ap.add_argument("--bf16-tflops", type=float, default=1620.9)
    args = ap.parse_args()
    import os
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        return sharded_sweep(args)
    dev = torch.device("cuda", torch.cuda.current_device())
    d, h = args.d_model, args.d_ff
    for skew in [float(s) for s in args.skews.split(",")]:
        for rho in [float(s) for s in args.densities.split(",")]:
            ffn = synthetic.make_ffn(d, h, seed=11, density=rho, skew_sigma=skew)
            g, u, dn = ffn.gate.to(dev), ffn.up.to(dev), ffn.down.to(dev)
            sparse = twell.TwELLGatedMLP(5000, g, u, dn)
            routed = twell.TwELLGatedMLP(5001, g, u, dn)
            routed.enable_dense_route(nnz_threshold=h // 64, min_tokens=128, dense_cap=1 << 30)
            dense = twell.TwELLGatedMLP(5002, g, u, dn)
            dense.enable_dense_route(dense_all_tokens=128)
            for m in [int(s) for s in args.tokens.split(",")]:
                x = synthetic.make_tokens(m, d, seed=12).to(dev)
                reps = 20 if m <= 1024 else 5
                packed = twell.allocate_packed_output(m, h, device=dev)

                def cublas():
                    return (torch.relu(x @ g.T) * (x @ u.T)) @ dn

                ref = cublas().float()
                rel = lambda y: float((y.float() - ref).norm() / ref.norm())  # noqa: E731
                rec = {"tokens": m, "density": rho, "skew": skew, "d_model": d, "d_ff": h}
                t_pack = _time(lambda: twell.matmul_sparse_out(x, g, packed), reps)
                rec["pack_us"] = t_pack
                cnt = packed.view(torch.int32)[:, ::32].long()
                rec["measured_density"] = cnt.sum().item() / (m * h)
                rec["overflowed_rows"] = int((cnt > 31).any(1).sum())
                if m <= 32:
                    rec["pack_roofline"] = {"bound": "hbm", "frac": 2 * d * h / (t_pack * 1e-6) / 1e9
                                            / args.hbm_gbs}
                else:
                    rec["pack_roofline"] = {"bound": "tensor", "frac": 2 * m * d * h / (t_pack * 1e-6)
                                            / 1e12 / args.bf16_tflops}
                times = {"sparse": _time(lambda: sparse(x), reps),
                         "cublas": _time(cublas, reps)}
                errs = {"sparse": rel(sparse(x))}
                if m >= 128:
                    times["routed"] = _time(lambda: routed(x), reps)
                    errs["routed"] = rel(routed(x))
                    rec["routed_dense_rows"] = routed.dense_route_counters()["dense_rows"]
                    times["dense_all"] = _time(lambda: dense(x), reps)
                    errs["dense_all"] = rel(dense(x))
                rec["us"] = times
                rec["rel_l2_vs_cublas"] = errs
                ours = {k: v for k, v in times.items() if k != "cublas"}
                # only paths that lose nothing count as candidates for "best"
                exact = {k: v for k, v in ours.items() if errs[k] < 2e-2}
                rec["best_exact_path"] = min(exact, key=exact.get) if exact else None
                rec["speedup_vs_cublas"] = (times["cublas"] / min(exact.values())) if exact else None
                print(json.dumps(rec), flush=True)
            for mod in (sparse, routed, dense):
                mod.destroy()


def sharded_sweep(args) -> None:
    """Under torchrun: the TwELL path with d_ff sharded over the ranks (pack + contraction on
    each shard, shard sum inside the contraction kernel up to 256 tokens, through NCCL beyond)
    against the unsharded cuBLAS formula on rank 0's GPU.  Time = max over ranks."""
    import os
    import sys

    import torch.distributed as dist

    from . import peer_allreduce, sharded
    world, rank = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    d, h = args.d_model, args.d_ff
    tokens = [int(s) for s in args.tokens.split(",")]
    small = [m for m in tokens if m <= 256]
    far = par = None
    if small:
        par = peer_allreduce.PeerAllReduce(max(small) * d * 2, device=dev)
        far = peer_allreduce.FusedShardAllReduce(max(small), d, device=dev)
    for skew in [float(s) for s in args.skews.split(",")]:
        for rho in [float(s) for s in args.densities.split(",")]:
            ffn = synthetic.make_ffn(d, h, seed=11, density=rho, skew_sigma=skew)
            g, u, dn = ffn.gate.to(dev), ffn.up.to(dev), ffn.down.to(dev)
            mod = sharded.ShardedTwELLGatedMLP(5100, g, u, dn, rank=rank, world_size=world,
                                               peer_allreduce=par, fused_allreduce=far)
            for m in tokens:
                x = synthetic.make_tokens(m, d, seed=12).to(dev)
                reps = 20 if m <= 1024 else 5
                mod(x)
                torch.cuda.synchronize(dev)
                dist.barrier()
                t = torch.tensor([_time(lambda: mod(x), reps)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                rec = {"tokens": m, "density": rho, "skew": skew, "d_model": d, "d_ff": h,
                       "n_gpus": world, "sharded_sparse_us": float(t.item()),
                       "shard_sum": mod.last_route}
                if rank == 0:
                    def cublas():
                        return (torch.relu(x @ g.T) * (x @ u.T)) @ dn
                    ref = cublas().float()
                    rec["cublas_unsharded_us"] = _time(cublas, reps)
                    rec["rel_l2_vs_cublas"] = float((mod_out(mod, x) - ref).norm() / ref.norm())
                else:
                    mod_out(mod, x)
                if rank == 0:
                    print(json.dumps(rec), flush=True)
                torch.cuda.synchronize(dev)
                dist.barrier()
            mod.destroy()
    if par is not None:
        par.fused = far
        par.close()
    torch.cuda.synchronize(dev)
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


def mod_out(mod, x):
    """One more (collective) forward on every rank, as fp32."""
    y = mod(x).float()
    torch.cuda.synchronize()
    return y


if __name__ == "__main__":
    main()
