"""Per-layer timing of the decode-sized sparse FFN through the C ABI (one GPU).

``python -m sparser_faster_llms_b200.decode_layer_bench [--d-model 2048] [--d-ff 8192]
[--layers 28] [--batch 1,8,32]`` prints one JSON line per batch size:

* ``two_kernels_us``      b200_twell_pack + b200_twell_gated_t2d per layer (also with a
  b200_l2_prefetch of the next layer's gate matrix between the two),
* ``pack_us`` / ``pack_narrow_epilogue_us``  the pack kernel alone, with sixteen and (in a
  child process started with ``B200_PACK_WIDE=0``) with four epilogue warps,
* ``one_kernel_us``       b200_twell_gated_mlp_decode per layer, also with the next layer's
  gate matrix as its L2 prefetch range,
* slab / output agreement of the two forms on the same inputs, the status word, and - when the
  library was built with ``-DB200_TRACE`` - the phase time stamps of the one-kernel form.

Every timing replays a CUDA graph of all layers (distinct weights per layer, larger than L2
together) and divides by the layer count.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys

import torch

from . import _lib, synthetic, twell


def _graph_us(fn, layers: int, reps: int = 20) -> float:
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * layers)


def _layers(d: int, h: int, n: int, dev):
    out = []
    for l in range(n):
        f = synthetic.make_ffn(d, h, seed=100 + l, density=0.02, skew_sigma=1.0)
        out.append((f.gate.to(dev), f.up.to(dev), f.down.to(dev)))
    return out


def run_batch(b: int, d: int, h: int, layers, dev) -> dict:
    lib = _lib.load_library()
    L = len(layers)
    x = synthetic.make_tokens(b, d, seed=7).to(dev)
    packed = twell.allocate_packed_output(b, h, device=dev)
    packed2 = twell.allocate_packed_output(b, h, device=dev)
    y = torch.empty(L, b, d, device=dev, dtype=torch.bfloat16)
    y2 = torch.empty_like(y)
    small = torch.zeros(int(lib.b200_workspace_bytes()), dtype=torch.uint8, device=dev)
    need = int(lib.b200_twell_decode_workspace_bytes(b, d, h))
    big = torch.zeros(max(need, 16), dtype=torch.uint8, device=dev)
    wbytes = h * d * 2

    def two(l):
        g, u, dn = layers[l]
        _lib.call("b200_twell_pack", dev, x.data_ptr(), g.data_ptr(), None, packed.data_ptr(),
                  b, d, h, 8)
        _lib.call("b200_twell_gated_t2d", dev, x.data_ptr(), packed.data_ptr(), u.data_ptr(),
                  dn.data_ptr(), y[l].data_ptr(), b, d, h, 8, 0, small.data_ptr(), small.numel())

    def two_prefetch(l):
        g, u, dn = layers[l]
        _lib.call("b200_twell_pack", dev, x.data_ptr(), g.data_ptr(), None, packed.data_ptr(),
                  b, d, h, 8)
        _lib.call("b200_l2_prefetch", dev, layers[(l + 1) % L][0].data_ptr(), wbytes)
        _lib.call("b200_twell_gated_t2d", dev, x.data_ptr(), packed.data_ptr(), u.data_ptr(),
                  dn.data_ptr(), y[l].data_ptr(), b, d, h, 8, 0, small.data_ptr(), small.numel())

    def pack_only(l):
        _lib.call("b200_twell_pack", dev, x.data_ptr(), layers[l][0].data_ptr(), None,
                  packed.data_ptr(), b, d, h, 8)

    def one(l, prefetch=False):
        g, u, dn = layers[l]
        nxt = layers[(l + 1) % L][0]
        _lib.call("b200_twell_gated_mlp_decode", dev, x.data_ptr(), g.data_ptr(), None,
                  u.data_ptr(), dn.data_ptr(), packed2.data_ptr(), y2[l].data_ptr(), b, d, h, 8,
                  0, big.data_ptr(), big.numel(), nxt.data_ptr() if prefetch else None,
                  wbytes if prefetch else 0)

    def pack_mma(l):
        _lib.call("b200_twell_pack_select", dev, x.data_ptr(), layers[l][0].data_ptr(), None,
                  packed.data_ptr(), b, d, h, 8, 1)

    def two_mma(l):
        g, u, dn = layers[l]
        pack_mma(l)
        _lib.call("b200_twell_gated_t2d", dev, x.data_ptr(), packed.data_ptr(), u.data_ptr(),
                  dn.data_ptr(), y[l].data_ptr(), b, d, h, 8, 0, small.data_ptr(), small.numel())

    def layer_call(l):
        g, u, dn = layers[l]
        _lib.call("b200_twell_gated_mlp", dev, x.data_ptr(), g.data_ptr(), None, u.data_ptr(),
                  dn.data_ptr(), packed2.data_ptr(), y2[l].data_ptr(), b, d, h, 8, 0,
                  one_ws.data_ptr(), one_ws.numel())

    rec = {"batch": b, "d_model": d, "d_ff": h, "layers": L}
    if b == 1 and d in (2048, 4096):
        # one token: GEMV pack kernel (automatic) against the mma.sync kernel, and the whole
        # layer in the GEMV kernel (b200_twell_gated_mlp with a workspace for its partial rows)
        one_ws = torch.zeros(4096 * 4 + (h // 256) * d * 4, dtype=torch.uint8, device=dev)
        rec["pack_mma_sync_us"] = _graph_us(lambda: [pack_mma(l) for l in range(L)], L)
        rec["two_kernels_mma_sync_pack_us"] = _graph_us(lambda: [two_mma(l) for l in range(L)], L)
        rec["one_token_layer_us"] = _graph_us(lambda: [layer_call(l) for l in range(L)], L)
        two(0)
        layer_call(0)
        torch.cuda.synchronize()
        diff = y[0].float() - y2[0].float()
        rec["one_token_rel_l2_vs_two_kernels"] = float(diff.norm() / y[0].float().norm())
    rec["two_kernels_us"] = _graph_us(lambda: [two(l) for l in range(L)], L)
    rec["two_kernels_with_l2_prefetch_us"] = _graph_us(
        lambda: [two_prefetch(l) for l in range(L)], L)
    rec["pack_us"] = _graph_us(lambda: [pack_only(l) for l in range(L)], L)
    if need:
        packed.zero_()   # words past a slab's count are left untouched by the kernels
        packed2.zero_()
        two(0)
        one(0)
        torch.cuda.synchronize()
        a, c = packed.view(torch.int32), packed2.view(torch.int32)
        rec["slab_words_differing"] = int((a != c).sum())
        diff = y[0].float() - y2[0].float()
        rec["out_rel_l2_vs_two_kernels"] = float(diff.norm() / y[0].float().norm())
        rec["one_kernel_us"] = _graph_us(lambda: [one(l) for l in range(L)], L)
        rec["one_kernel_with_l2_prefetch_us"] = _graph_us(
            lambda: [one(l, True) for l in range(L)], L)
        rec["decode_status"] = int(lib.b200_twell_decode_status())
        if hasattr(lib, "b200_debug_trace_decode"):
            stamps = (ctypes.c_ulonglong * 16)()
            one(0)
            torch.cuda.synchronize()
            lib.b200_debug_trace_decode(stamps)
            rec["phase_stamps_ns"] = {str(i): int(stamps[i]) - int(stamps[0])
                                      for i in (1, 2, 8, 9, 10, 3, 4, 5, 6, 7)}
    else:
        rec["one_kernel_us"] = None
    return rec


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--d-ff", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--batch", default="1,8,32")
    ap.add_argument("--pack-only", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    layers = _layers(args.d_model, args.d_ff, args.layers, dev)
    for b in (int(s) for s in args.batch.split(",")):
        if args.pack_only:  # child process: the pack kernel under another environment
            lib = _lib.load_library()
            x = synthetic.make_tokens(b, args.d_model, seed=7).to(dev)
            packed = twell.allocate_packed_output(b, args.d_ff, device=dev)
            us = _graph_us(lambda: [_lib.call("b200_twell_pack", dev, x.data_ptr(),
                                              layers[l][0].data_ptr(), None, packed.data_ptr(),
                                              b, args.d_model, args.d_ff, 8)
                                    for l in range(len(layers))], len(layers))
            print(json.dumps({"batch": b, "pack_us": us}), flush=True)
            del lib
            continue
        rec = run_batch(b, args.d_model, args.d_ff, layers, dev)
        if os.environ.get("B200_PACK_WIDE") != "0" and b > 16:
            child = subprocess.run(
                [sys.executable, "-m", "sparser_faster_llms_b200.decode_layer_bench", "--pack-only",
                 "--d-model", str(args.d_model), "--d-ff", str(args.d_ff), "--layers",
                 str(args.layers), "--batch", str(b)],
                env={**os.environ, "B200_PACK_WIDE": "0"}, capture_output=True, text=True)
            try:
                rec["pack_narrow_epilogue_us"] = json.loads(child.stdout.strip().splitlines()[-1])[
                    "pack_us"]
            except (ValueError, IndexError, KeyError):
                rec["pack_narrow_epilogue_us"] = None
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
