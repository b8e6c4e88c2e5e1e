"""Peer-memory all-reduce on 2 GPUs (skipped with fewer): repeated calls, changing sizes,
graph replay, and the sharded FFN using it.  NVLS is switched off; the kernel uses plain
peer stores only."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    from sparser_faster_llms_b200 import peer_allreduce, sharded, synthetic
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok = True
    try:
        par = peer_allreduce.PeerAllReduce(256 * 1024, device=dev)
        gen = torch.Generator(device=dev).manual_seed(100 + rank)
        # eager calls, sizes change between calls, many in a row
        for it, n in enumerate([2048, 65536, 8, 131072, 4096, 65536, 65536, 2048 * 32]):
            x = torch.randn(n, generator=gen, device=dev).to(torch.bfloat16)
            got = par.all_reduce(x)
            ref = x.float()
            dist.all_reduce(ref)          # fp32 NCCL sum of the same bf16 inputs
            err = (got.float() - ref).abs().max().item()
            tol = 2e-2 * max(1.0, ref.abs().max().item())
            ok = ok and err <= tol
        # graph replay: the device-side epoch must advance on every replay
        x = torch.randn(32 * 2048, generator=gen, device=dev).to(torch.bfloat16)
        y = torch.empty_like(x)
        s = torch.cuda.Stream(dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            par.all_reduce(x, y)
        torch.cuda.current_stream(dev).wait_stream(s)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(3):
                par.all_reduce(x, y)
        ref = x.float()
        dist.all_reduce(ref)
        for _ in range(5):
            y.zero_()
            g.replay()
            torch.cuda.synchronize(dev)
            ok = ok and (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
        ok = ok and par.status() == 0
        # the sharded FFN with the peer all-reduce against the NCCL one
        d, h, m = 2048, 8192, 32
        ffn = synthetic.make_ffn(d, h, seed=95, density=0.02, skew_sigma=1.0)
        xs = synthetic.make_tokens(m, d, seed=96).to(dev)
        args = (ffn.gate.to(dev), ffn.up.to(dev), ffn.down.to(dev))
        a = sharded.ShardedTwELLGatedMLP(0, *args, peer_allreduce=par)
        b = sharded.ShardedTwELLGatedMLP(1, *args, reduce_dtype=torch.float32)
        ya, yb = a(xs), b(xs)
        torch.cuda.synchronize(dev)
        rel = ((ya.float() - yb.float()).norm() / yb.float().norm()).item()
        ok = ok and rel < 1e-2 and par.status() == 0
        # contraction fused with the all-reduce: identical bits to contraction + peer all-reduce
        # (same rounding points, same rank order), for the few-token multi-cluster shape
        # (batch 1, 8) and the one-cluster shape (batch 32), repeated calls, graph replay
        far = peer_allreduce.FusedShardAllReduce(32, d, device=dev)
        c = sharded.ShardedTwELLGatedMLP(2, *args, fused_allreduce=far)
        for m_f in (1, 8, 32, 8, 32):
            xf = synthetic.make_tokens(m_f, d, seed=200 + m_f).to(dev)
            yf, yp = c(xf), a(xf)
            torch.cuda.synchronize(dev)
            ok = ok and torch.equal(yf, yp)
        xf = synthetic.make_tokens(32, d, seed=300).to(dev)
        yp = a(xf).clone()
        sg = torch.cuda.Stream(dev)
        sg.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(sg):
            c(xf)
        torch.cuda.current_stream(dev).wait_stream(sg)
        torch.cuda.synchronize(dev)
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=sg):
            yg = c(xf)
        for _ in range(4):
            yg.zero_()
            g2.replay()
            torch.cuda.synchronize(dev)
            ok = ok and torch.equal(yg, yp)
        ok = ok and far.status() == 0 and par.status() == 0
        with open(os.path.join(out_dir, f"ok{rank}"), "w") as f:
            f.write(f"{int(ok)} {rel}")
        a.destroy()
        b.destroy()
        c.destroy()
        torch.cuda.synchronize(dev)
        dist.barrier()
    finally:
        os._exit(0)  # captured graphs hold communicator state: skip the collective teardown


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_peer_allreduce_two_ranks(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    for r in range(2):
        flag, rel = (tmp_path / f"ok{r}").read_text().split()
        assert flag == "1", (r, rel)
