"""Prefill-sized sparse FFN layer with a per-token density mix: gather-only, routed and
all-dense contraction next to dense cuBLAS.

``python -m sparser_faster_llms_b200.prefill_bench [--tokens 16384] [--d-model 2048]
[--d-ff 11008] [--modes gather,routed,dense_all,cublas]`` prints one JSON line per mode.
The workload stands in for the 2B-shape prefill configuration: one layer, tokens whose gate
density is drawn from Beta(2, 60) (mean about 3 %) with 5 % of the tokens at 20-40 %, weights
~N(0, 0.02), all seeded (:func:`synthetic.make_tokens_mixed_density`).  Times are CUDA events
around ``reps`` calls after ``warmup`` calls on the current stream; every mode reports its
relative L2 error against the fp32 dense formula evaluated by cuBLAS on the same inputs.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import _lib, synthetic, twell


def _time(fn, reps: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--d-ff", type=int, default=11008)
    ap.add_argument("--base-density", type=float, default=0.03)
    ap.add_argument("--nnz-threshold", type=int, default=None, help="default d_ff // 64")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--modes", default="gather,routed,dense_all,cublas")
    args = ap.parse_args()
    dev = torch.device("cuda", torch.cuda.current_device())
    m, d, h = args.tokens, args.d_model, args.d_ff
    ffn = synthetic.make_ffn(d, h, seed=5, density=args.base_density, skew_sigma=0.0)
    g, u, dn = ffn.gate.to(dev), ffn.up.to(dev), ffn.down.to(dev)
    x, rho = synthetic.make_tokens_mixed_density(m, d, base_density=args.base_density, seed=9)
    x = x.to(dev)
    thr = args.nnz_threshold if args.nnz_threshold is not None else h // 64

    def cublas():
        return (torch.relu(x @ g.T) * (x @ u.T)) @ dn

    ref = cublas().float()
    flops = 3 * 2 * m * d * h
    common = {"tokens": m, "d_model": d, "d_ff": h, "mean_target_density": float(rho.mean()),
              "reps": args.reps}
    for mode in args.modes.split(","):
        rec = dict(common, mode=mode)
        if mode == "cublas":
            ms = _time(cublas, args.reps, args.warmup)
            y = cublas()
        else:
            mod = twell.TwELLGatedMLP(4242, g, u, dn)
            if mode == "routed":
                mod.enable_dense_route(nnz_threshold=thr, dense_cap=m, min_tokens=128)
            elif mode == "dense_all":
                mod.enable_dense_route(dense_all_tokens=1)
            elif mode != "gather":
                raise SystemExit(f"unknown mode {mode}")
            ms = _time(lambda: mod(x), args.reps, args.warmup)
            y = mod(x)
            if mode == "routed":
                rec.update(mod.dense_route_counters(), nnz_threshold=thr)
            lib = _lib.load_library()
            rec["wait_status"] = [int(lib.b200_twell_pack_tc_status()),
                                  int(lib.b200_twell_hybrid_status())]
            mod.destroy()
        rec["ms"] = ms
        rec["tokens_per_s"] = m / (ms * 1e-3)
        rec["dense_equivalent_tflops"] = flops / (ms * 1e-3) / 1e12
        rec["rel_l2_vs_dense_formula"] = float((y.float() - ref).norm() / ref.norm())
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
