#!/usr/bin/env python
"""Benchmark of the sparse gated-FFN hot path at the 1.5B decode shape.

Workload (``config.workload``): the FFN stack of a random-init 1.5B-shape sparse
decoder - 28 layers, d_model 2048, d_ff 8192, bf16 weights ~N(0, 0.02), gate
density about 2 % with log-normal(sigma=1) per-neuron firing rates - at a decode
batch of B tokens (default 32).  One step = one pass of all 28 sparse FFN layers
over one batch of synthetic activations; ``value`` = B / step time (tokens/s).
The 2.8 GB of weights exceed the 126 MB L2, so every step streams them from HBM
(no L2 flush needed).

Legs printed in ONE JSON line by rank 0:
  value        device-resident inputs, the step replayed as a CUDA graph
  e2e          the same stack through the public ``TwELLGatedMLP`` modules with
               pinned-host inputs and outputs (H2D + D2H inside the timed region)
  roofline     the dominant kernel (gate GEMV + TwELL pack) timed alone
  cpu_baseline the dense torch formula on the host cores (bounded sample)

``--impl reference`` times the reference's torch CPU formulation
(SparseMLP._forward_mlp_inference_logic) on the host cores instead.
With ``--gpus N`` (torchrun) d_ff is sharded over the ranks and the partial FFN
outputs are summed with one NCCL all-reduce per layer (strong scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

LAYERS, D_MODEL, D_FF = 28, 2048, 8192
DENSITY, SKEW = 0.02, 1.0
NCU_DRAM_OVER_ALGORITHMIC = 33.73 / 33.71
METRIC = "sparse_ffn_decode_tokens_per_s"
UNIT = "tokens/s"


def workload_name(args) -> str:
    return (f"1.5B-shape sparse FFN stack decode: {args.layers} layers, d_model {args.d_model}, "
            f"d_ff {args.d_ff}, batch {args.batch}, gate density ~{DENSITY:.0%} "
            f"log-normal sigma {SKEW}")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--d-model", type=int, default=D_MODEL)
    ap.add_argument("--d-ff", type=int, default=D_FF)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-decode-model", action="store_true",
                    help="skip the end-to-end decode ms/token of the full 1.5B-shape model")
    ap.add_argument("--no-energy", action="store_true",
                    help="skip the energy-per-step measurement (single GPU only)")
    ap.add_argument("--energy-seconds", type=float, default=1.5,
                    help="length of each energy window (sparse stack, dense stack)")
    ap.add_argument("--eager-collectives", action="store_true",
                    help="multi-rank: launch the step eagerly instead of as one CUDA graph")
    ap.add_argument("--collective", default="fused", choices=["fused", "peer", "nccl"],
                    help="multi-rank: sum the partial outputs inside the contraction kernel "
                         "(default), with the library's peer-memory all-reduce kernel, or with NCCL")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch eagerly instead of replaying a CUDA graph (for profilers)")
    return ap.parse_args()


def measured_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        j = json.loads(p.read_text())
        return float(j["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ----------------------------------------------------------------------------
# clocks sampling
# ----------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------
# workload
# ----------------------------------------------------------------------------
def shard_range(h: int, rank: int, world: int):
    """Tile-granular (256-neuron) contiguous split of d_ff; uneven shards allowed."""
    tiles = h // 256
    base, rem = divmod(tiles, world)
    start = rank * base + min(rank, rem)
    n = base + (1 if rank < rem else 0)
    return start * 256, (start + n) * 256


def full_layer_weights(args, device, l):
    """fp32 [3, d_ff, d_model] (gate, up, down) of layer ``l``, the same on every rank."""
    from sparser_faster_llms_b200 import synthetic
    d, h = args.d_model, args.d_ff
    gen = torch.Generator(device=device).manual_seed(1000 + l)
    w = torch.randn(3, h, d, generator=gen, device=device, dtype=torch.float32) * 0.02
    cg = torch.Generator().manual_seed(2000 + l)
    rates = synthetic.neuron_rates(h, DENSITY, SKEW, cg)
    shift = (0.02 * (d - 1) ** 0.5 * torch.special.ndtri(rates)).float().to(device)
    w[0, :, 0] = shift  # bias folded into feature 0 (tokens carry x[:, 0] = 1)
    return w


def build_layers(args, device, rank, world):
    from sparser_faster_llms_b200 import synthetic
    d, h = args.d_model, args.d_ff
    h0, h1 = shard_range(h, rank, world)
    layers = []
    for l in range(args.layers):
        w = full_layer_weights(args, device, l)
        wb = w[:, h0:h1].to(torch.bfloat16).contiguous()
        layers.append((wb[0], wb[1], wb[2]))
        del w
    gen = torch.Generator(device=device).manual_seed(7)
    x = torch.randn(args.layers, args.batch, d, generator=gen, device=device)
    x[:, :, 0] = 1.0
    return layers, x.to(torch.bfloat16).contiguous(), (h0, h1)


def capture(fn, device):
    """Warm up ``fn`` on a side stream, then capture it into a CUDA graph."""
    s = torch.cuda.Stream(device)
    s.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(s):
        for _ in range(2):
            fn()
    torch.cuda.current_stream(device).wait_stream(s)
    torch.cuda.synchronize(device)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


def time_replays(run, steps, warmup, device, dist_on):
    import torch.distributed as dist
    for _ in range(warmup):
        run()
    torch.cuda.synchronize(device)
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize(device)
    if dist_on:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist_on:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def make_peer_allreduce(args, device, dist_on):
    """(PeerAllReduce or None, description).  Every rank takes the same branch: the outcome of
    the symmetric-memory set-up is agreed with a MIN all-reduce before anyone uses it."""
    if not dist_on:
        return None, "none"
    if args.collective == "nccl":
        return None, "nccl all-reduce"
    import torch.distributed as dist
    from sparser_faster_llms_b200 import peer_allreduce
    par, far, why = None, None, ""
    try:
        par = peer_allreduce.PeerAllReduce(args.batch * args.d_model * 2, device=device)
        if args.collective == "fused" and args.batch <= 256:
            far = peer_allreduce.FusedShardAllReduce(args.batch, args.d_model, device=device)
    except Exception as exc:  # symmetric memory not available on this machine
        why = f"{type(exc).__name__}: {exc}"[:160]
        par = far = None
    ok = torch.tensor([1 if par is not None else 0], device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 1:
        par.fused = far
        if far is not None:
            return par, ("contraction fused with the shard all-reduce over peer memory "
                         "(b200_twell_gated_mlp_allreduce)")
        return par, "peer-memory all-reduce kernel (b200_peer_allreduce_bf16)"
    return None, f"nccl all-reduce (peer all-reduce unavailable: {why or 'on another rank'})"


def one_token_layer(B: int, d: int, hl: int, par) -> bool:
    """Whether b200_twell_gated_mlp serves the call with the one-token kernel (one launch):
    a single token, d_model 2048 / 4096, a tile count that fits clusters of four (33 on
    B200), the 1 MiB workspace large enough for the partial rows, no d_ff sharding."""
    tiles = hl // 256
    return (par is None and B == 1 and d in (2048, 4096) and tiles <= 33
            and 4096 * 4 + tiles * d * 4 <= (1 << 20)
            and os.environ.get("B200_ONE_TOKEN", "2") == "2")


def pack_kernel_name(B: int, d: int, hl: int) -> str:
    """The kernel b200_twell_pack launches for this call (csrc/c_api.cu)."""
    tiles = hl // 256
    if B == 1 and d in (2048, 4096):
        return "twell_gemv_kernel"
    if B <= 16:
        return "twell_pack_kernel"
    if B <= 32:
        return "twell_pack_tc_splitk_wide_kernel"
    if B <= 256 and tiles * 2 * -(-B // 128) <= 148:
        return "twell_pack_tc_splitk_mid_kernel"
    return "twell_pack_tc_wide_kernel" if B > 64 else "twell_pack_tc_kernel"


def run_ours(args):
    import torch.distributed as dist
    from sparser_faster_llms_b200 import _lib, twell

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist_on = world > 1
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if dist_on:
        dist.init_process_group("nccl", device_id=device)
    _lib.load_library()

    layers, x, (h0, h1) = build_layers(args, device, rank, world)
    hl = h1 - h0
    L, B, d = args.layers, args.batch, args.d_model
    packed = torch.zeros(B, twell.packed_width(hl), device=device, dtype=torch.uint32)
    out = torch.empty(L, B, d, device=device, dtype=torch.bfloat16)

    ws_buf = torch.zeros(int(_lib.load_library().b200_workspace_bytes()), dtype=torch.uint8,
                         device=device)
    ws = (ws_buf.data_ptr(), ws_buf.numel())

    par, collective = make_peer_allreduce(args, device, dist_on)
    far = getattr(par, "fused", None)
    part = torch.empty(B, d, device=device, dtype=torch.bfloat16) if par is not None else None

    def step():
        for l, (g, u, dn) in enumerate(layers):
            if far is not None:  # one pack kernel + one contraction-and-all-reduce kernel
                _lib.call("b200_twell_gated_mlp_allreduce", device, x[l].data_ptr(), g.data_ptr(),
                          None, u.data_ptr(), dn.data_ptr(), packed.data_ptr(),
                          out[l].data_ptr(), B, d, hl, 8, 0, *ws, far.ptr_array, far.rank,
                          far.world, far.block_bytes)
                continue
            y = out[l] if par is None else part
            _lib.call("b200_twell_gated_mlp", device, x[l].data_ptr(), g.data_ptr(), None,
                      u.data_ptr(), dn.data_ptr(), packed.data_ptr(), y.data_ptr(),
                      B, d, hl, 8, 0, *ws)
            if par is not None:
                par.all_reduce(part, out[l])
            elif dist_on:
                dist.all_reduce(out[l])

    def pack_only():
        for l, (g, u, dn) in enumerate(layers):
            _lib.call("b200_twell_pack", device, x[l].data_ptr(), g.data_ptr(), None,
                      packed.data_ptr(), B, d, hl, 8)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # Multi-rank steps are captured with their NCCL all-reduces inside the graph
    # (--eager-collectives launches them eagerly instead).
    graphed = not args.no_graph and (not dist_on or not args.eager_collectives)
    if dist_on:
        # the peer kernels wait (bounded) for one another: start the first step together
        torch.cuda.synchronize(device)
        dist.barrier()
    run_step = capture(step, device).replay if graphed else step
    ms_step = time_replays(run_step, args.steps, args.warmup, device, dist_on)
    clocks = sampler.stop() if rank == 0 else None

    # dense GPU baseline: the same stack as three cuBLAS bf16 matmuls per layer (a reported
    # comparison point, not part of the product path)
    def dense_step():
        for l, (g, u, dn) in enumerate(layers):
            h = torch.relu(x[l] @ g.T) * (x[l] @ u.T)
            torch.matmul(h, dn, out=out[l])

    ms_dense = None
    if not dist_on:
        run_dense = dense_step if args.no_graph else capture(dense_step, device).replay
        ms_dense = time_replays(run_dense, max(10, args.steps // 2), 3, device, False)

    # energy per step (the reference benchmark's --measure-energy figure, energy per forward:
    # benchmark_inference.py:280-343), after the timed region, sparse and dense stacks alike
    energy_row = None
    if not dist_on and not args.no_energy:
        try:
            from sparser_faster_llms_b200 import energy as energy_mod
            e_s = energy_mod.measure_replays(run_step, device, min_seconds=args.energy_seconds)
            e_d = energy_mod.measure_replays(run_dense, device, min_seconds=args.energy_seconds)
            if e_s is not None:
                energy_row = {"j_per_step": e_s["energy_per_forward_j"],
                              "j_per_token": e_s["energy_per_forward_j"] / B,
                              "avg_power_w": e_s["avg_power_w"], "steps": e_s["reps"],
                              "window_s": e_s["energy_duration_s"],
                              "backend": e_s["energy_backend"]}
                if e_d is not None:
                    energy_row["dense_cublas_bf16_j_per_step"] = e_d["energy_per_forward_j"]
                    energy_row["dense_cublas_bf16_avg_power_w"] = e_d["avg_power_w"]
        except Exception as exc:  # a power query must never cost the benchmark line
            energy_row = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}

    # dominant kernel alone (per-launch time, CUDA events on the launching stream)
    run_pack = pack_only if args.no_graph else capture(pack_only, device).replay
    ms_pack = time_replays(run_pack, max(10, args.steps // 2), 3, device, False) / L
    # statistics of the last slab for the byte model
    torch.cuda.synchronize(device)
    counts = packed.view(torch.int32)[:, ::32].long()
    nnz_per_token = counts.sum().item() / B
    act = twell.packed_to_dense(packed, hl)
    union = int((act != 0).any(dim=0).sum().item())

    # algorithmic bytes per launch of the pack kernel: all of W_gate + x + slab words written
    slab_bytes = 4 * (counts.clamp(max=31).sum().item() + counts.numel())
    pack_bytes = 2 * d * hl + 2 * B * d + slab_bytes
    peak, peak_kind = measured_peaks()
    achieved = pack_bytes / (ms_pack * 1e-3) / 1e9
    # whole-FFN algorithmic bytes (gate + active up/down rows + x, y + slab write/read)
    ffn_bytes = 2 * d * hl + 2 * 2 * d * union + 2 * 2 * B * d + 2 * slab_bytes

    result = {
        "metric": METRIC, "value": B / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args),
                   "layers": L, "d_model": d, "d_ff": args.d_ff, "batch": B,
                   "d_ff_shard": [h0, h1], "parallelism": f"dff_shard{world}",
                   "l2": "weights (2.8 GB) exceed L2; no flush needed",
                   "cuda_graph": graphed, "collective": collective,
                   "nnz_per_token_last_layer": nnz_per_token,
                   "active_union_last_layer": union,
                   "ms_per_layer": ms_step / L,
                   "dense_cublas_bf16_ms_per_step": ms_dense,
                   "ffn_algorithmic_gbs": ffn_bytes / (ms_step / L * 1e-3) / 1e9},
        "roofline": {"bound": "hbm",
                     "kernel": pack_kernel_name(B, d, hl),
                     "achieved": achieved,
                     "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": achieved / peak,
                     # DRAM bytes per launch: one ncu capture of this kernel at this shape read
                     # 33.73 MB for 33.71 MB of algorithmic bytes; scaled to this launch
                     "traffic": float(pack_bytes) * NCU_DRAM_OVER_ALGORITHMIC,
                     "us_per_launch": ms_pack * 1e3, "algorithmic_bytes": pack_bytes},
        # one token on one GPU: pack and contraction are ONE launch (the GEMV kernel)
        "gpu_launches": args.steps * L * (3 if (par is not None and far is None) else
                                          1 if one_token_layer(B, d, hl, par) else 2),
        "clocks": clocks,
        "energy": energy_row,
    }

    # the other decode batch sizes of the configuration, measured the same way (shorter)
    if not dist_on and not args.no_graph:
        others = {}
        for b2 in (1, 8):
            if b2 >= B:
                continue
            xb = x[:, :b2].contiguous()

            def step_b():
                for l, (g, u, dn) in enumerate(layers):
                    _lib.call("b200_twell_gated_mlp", device, xb[l].data_ptr(), g.data_ptr(), None,
                              u.data_ptr(), dn.data_ptr(), packed.data_ptr(), out[l].data_ptr(),
                              b2, d, hl, 8, 0, *ws)

            def dense_b():
                for l, (g, u, dn) in enumerate(layers):
                    h = torch.relu(xb[l] @ g.T) * (xb[l] @ u.T)
                    torch.matmul(h, dn, out=out[l, :b2])

            ms_b = time_replays(capture(step_b, device).replay, max(10, args.steps // 2), 3,
                                device, False)
            ms_db = time_replays(capture(dense_b, device).replay, max(10, args.steps // 2), 3,
                                 device, False)
            others[str(b2)] = {"ms_per_step": ms_b, "tokens_per_s": b2 / (ms_b * 1e-3),
                               "dense_cublas_bf16_ms_per_step": ms_db}
        result["config"]["other_batches"] = others

    if not args.no_e2e:
        result["e2e"] = run_e2e(args, layers, x, device, dist_on, par)
    if (not dist_on and not args.no_decode_model and not args.no_graph
            and (args.layers, args.d_model, args.d_ff) == (LAYERS, D_MODEL, D_FF)):
        result["config"]["decode_ms_per_token"] = decode_model_ms_per_token()
    if dist_on and rank == 0:
        # self-check of the sharded sum: layer 0 recomputed on this rank alone over all of d_ff
        wf = full_layer_weights(args, device, 0).to(torch.bfloat16).contiguous()
        packed_f = torch.zeros(B, twell.packed_width(args.d_ff), device=device,
                               dtype=torch.uint32)
        y_f = torch.empty(B, d, device=device, dtype=torch.bfloat16)
        _lib.call("b200_twell_gated_mlp", device, x[0].data_ptr(), wf[0].data_ptr(), None,
                  wf[1].data_ptr(), wf[2].data_ptr(), packed_f.data_ptr(), y_f.data_ptr(),
                  B, d, args.d_ff, 8, 0, *ws)
        torch.cuda.synchronize(device)
        diff = out[0].float() - y_f.float()
        result["config"]["max_abs_vs_unsharded"] = float(diff.abs().max())
        result["config"]["rel_l2_vs_unsharded"] = float(diff.norm() / y_f.float().norm())
        del wf
    if par is not None:
        # non-zero: a bounded wait on a peer gave up somewhere in the run (results invalid)
        result["config"]["peer_allreduce_status"] = par.status()
        if far is not None:
            result["config"]["fused_allreduce_status"] = far.status()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline(args, sample_layers=2, reps=3)
    if rank == 0:
        print(json.dumps(result))
    if dist_on:
        torch.cuda.synchronize(device)
        dist.barrier()
        if par is not None:
            par.close()  # no peer mapping is held when the process leaves
            torch.cuda.synchronize(device)
            dist.barrier()
        # Tearing the NCCL communicator down while captured graphs still hold its kernels
        # stalled on this stack: every rank has finished and flushed, so leave without the
        # collective teardown.
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def decode_model_ms_per_token():
    """End-to-end decode of the full random-init 1.5B-shape model (attention, norms, LM head
    around the FFN; decode_model.py): ms per token with the TwELL FFN and with the dense cuBLAS
    FFN on the same weights, prompt 512, 64 timed steps of one CUDA graph each."""
    from sparser_faster_llms_b200 import decode_model as dm
    cfg = dm.DecoderConfig(max_seq=640)
    out = {}
    for b in (1, 8, 32):
        try:
            tw = dm.time_decode(cfg, b, 512, 72, "twell", reps=1)
            de = dm.time_decode(cfg, b, 512, 72, "dense", reps=1)
            out[str(b)] = {"twell_ffn": tw["ms_per_token"], "dense_cublas_ffn": de["ms_per_token"],
                           "ratio": de["ms_per_token"] / tw["ms_per_token"]}
        except Exception as exc:  # the model leg must never cost the benchmark line
            out[str(b)] = {"unavailable": f"{type(exc).__name__}: {exc}"[:160]}
    return out


def run_e2e(args, layers, x, device, dist_on, par=None):
    """The same stack through the public modules (TwELLGatedMLP, or the d_ff-sharded module
    on several ranks) run by GraphedFFNStack: every step copies the inputs from pinned host
    memory, runs all layers and reads the last layer's output back to the host."""
    import torch.distributed as dist
    from sparser_faster_llms_b200 import sharded, stack, twell
    L, B, d = args.layers, args.batch, args.d_model
    if dist_on:
        mods = [sharded.ShardedTwELLGatedMLP(1000 + l, g, u, dn, presharded=True,
                                             peer_allreduce=par,
                                             fused_allreduce=getattr(par, "fused", None),
                                             preallocate_shared_hidden_state=True)
                for l, (g, u, dn) in enumerate(layers)]
    else:
        mods = [twell.TwELLGatedMLP(1000 + l, g, u, dn, preallocate_shared_hidden_state=True)
                for l, (g, u, dn) in enumerate(layers)]
    if dist_on:
        torch.cuda.synchronize(device)
        dist.barrier()  # the warm-up steps inside the constructor exchange with the peers
    runner = stack.GraphedFFNStack(mods, B, return_last_only=True, device=device)
    runner.x_host.copy_(x.cpu())
    for _ in range(3):
        runner.run()
    steps = max(5, args.steps // 2)
    torch.cuda.synchronize(device)
    if dist_on:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        y = runner.run()
    torch.cuda.synchronize(device)
    ms = (time.perf_counter() - t0) * 1e3 / steps
    if dist_on:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    checksum = float(y.float().abs().sum())
    for m in mods:
        m.destroy()
    return {"value": B / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms,
            "h2d_bytes_per_step": L * B * d * 2, "d2h_bytes_per_step": B * d * 2,
            "result_checksum": checksum,
            "api": "GraphedFFNStack.run over TwELLGatedMLP modules: pinned host input, one CUDA "
                   "graph (H2D, 28 fused gated MLPs, D2H of the last layer's output), host wall "
                   "clock"}


# ----------------------------------------------------------------------------
# CPU legs
# ----------------------------------------------------------------------------
def reference_sparse_mlp(d, h):
    """The reference's own SparseMLP (custom_models/sparse_models.py:259-412) on its torch
    inference path, from the files staged under oracle/_ref; None where they are absent."""
    try:
        from oracle import make_ref
        if not make_ref.available():
            return None
        if make_ref.import_path() not in sys.path:
            sys.path.insert(0, make_ref.import_path())
        from custom_models.sparse_models import NullTracker, SparseLlamaConfig, SparseMLP
        cfg = SparseLlamaConfig(hidden_size=d, intermediate_size=h, num_hidden_layers=1,
                                num_attention_heads=16, num_key_value_heads=16, vocab_size=64)
        return SparseMLP(layer_idx=0, config=cfg, gated=True, tracker=NullTracker(1, 1),
                         execution_logic="inference").eval()
    except Exception:
        return None


def cpu_baseline(args, sample_layers, reps):
    """The FFN stack on the host cores: the reference's SparseMLP torch path
    (SparseMLP._forward_mlp_inference_logic, sparse_models.py:343-351) where its files are
    staged (kind "reference"), else the oracle's dense restatement of it (kind "port").
    fp32, every host thread, bounded sample scaled to the full stack."""
    from oracle import ffn_oracle as fo
    from sparser_faster_llms_b200 import synthetic
    d, h, B = args.d_model, args.d_ff, args.batch
    torch.set_num_threads(os.cpu_count() or 1)  # torchrun sets OMP_NUM_THREADS=1
    threads = torch.get_num_threads()
    ffns = [synthetic.make_ffn(d, h, seed=50 + i, density=DENSITY, skew_sigma=SKEW)
            for i in range(sample_layers)]
    x = synthetic.make_tokens(B, d, seed=60)
    mlp = reference_sparse_mlp(d, h)
    if mlp is not None:
        mods = []
        import copy
        for f in ffns:
            m = copy.deepcopy(mlp)
            with torch.no_grad():
                m.gate_proj.weight.copy_(f.gate.float())
                m.up_proj.weight.copy_(f.up.float())
                m.down_proj.weight.copy_(f.down.float().T)
            mods.append(m)
        xs = x.float().unsqueeze(0)

        def run_layers():
            with torch.inference_mode():
                for m in mods:
                    m(xs)
        kind = "reference"
        what = "the reference's SparseMLP torch inference path"
    else:
        ws = [(f.gate.float(), f.up.float(), f.down.float()) for f in ffns]

        def run_layers():
            for g, u, dn in ws:
                fo.dense_ffn(x, g, u, dn)
        kind = "port"
        what = "fp32 torch dense formula (oracle restatement)"
    times = []
    for r in range(reps + 1):
        t0 = time.perf_counter()
        run_layers()
        times.append(time.perf_counter() - t0)
    per_layer = statistics.median(times[1:]) / sample_layers
    return {"value": B / (per_layer * args.layers), "unit": UNIT, "cores": threads,
            "kind": kind, "ms_per_step": per_layer * args.layers * 1e3,
            "sample": f"{sample_layers} of {args.layers} layers at batch {B}, {what}, fp32, "
                      f"median of {reps} reps, scaled to {args.layers} layers"}


def run_reference(args):
    """Reference arm: the reference's CPU torch formulation on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_layers = 4
    reps = max(3, min(args.steps, 10))
    base = cpu_baseline(args, sample_layers=sample_layers, reps=reps)
    result = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_name(args),
                   "note": "reference CUDA kernels are sm_90a-only (WGMMA) and cannot run on "
                           "sm_100; this arm times the reference's torch CPU formulation"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(result))


def main():
    args = parse()
    watchdog = int(os.environ.get("B200_BENCH_WATCHDOG_S", "0"))
    if watchdog > 0:  # dump every thread's stack and exit instead of hanging silently
        import faulthandler
        faulthandler.dump_traceback_later(watchdog, exit=True)
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); "
                         "use --impl reference for the CPU arm")
    run_ours(args)


if __name__ == "__main__":
    main()
