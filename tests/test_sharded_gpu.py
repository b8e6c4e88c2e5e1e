"""d_ff-sharded module on 2 GPUs with NCCL (skipped when fewer than 2 GPUs are visible)."""
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
    from sparser_faster_llms_b200 import sharded, synthetic
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        d, h, m = 2048, 11008, 16   # 43 tiles: uneven shards
        ffn = synthetic.make_ffn(d, h, seed=95, density=0.02, skew_sigma=1.0)
        x = synthetic.make_tokens(m, d, seed=96)
        dev = torch.device("cuda", rank)
        mod = sharded.ShardedTwELLGatedMLP(0, ffn.gate.to(dev), ffn.up.to(dev),
                                           ffn.down.to(dev), reduce_dtype=torch.float32)
        y = mod(x.to(dev))
        torch.cuda.synchronize()
        if rank == 0:
            torch.save(y.cpu(), os.path.join(out_dir, "y.pt"))
        mod.destroy()
    finally:
        dist.destroy_process_group()


def _training_case(dev):
    from sparser_faster_llms_b200 import synthetic
    b, s, d, h = 2, 64, 1024, 4096
    ffn = synthetic.make_ffn(d, h, seed=140, density=0.02)
    x = synthetic.make_tokens(b * s, d, seed=141).view(b, s, d)
    w = torch.randn(b, s, d, generator=torch.Generator().manual_seed(142)).to(torch.bfloat16)
    return [t.to(dev) for t in (x, ffn.gate, ffn.up, ffn.down, w)]


def _training_worker(rank, world, port, out_dir):
    from sparser_faster_llms_b200 import sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        x, g, k, v, w = _training_case(dev)
        gl, kl, vl = sharded.shard_weights(g, k, v, rank, world)
        x.requires_grad_(True)
        gl, kl, vl = (t.clone().requires_grad_(True) for t in (gl, kl, vl))
        out, l0, l1 = sharded.sharded_ff_gated(x, gl, kl, vl)
        ((out.float() * w.float()).sum() + 0.5 * l1).backward()
        torch.cuda.synchronize()
        h0, h1 = sharded.shard_range(g.shape[0], rank, world)
        torch.save({"out": out.detach().cpu(), "l0": l0.item(), "l1": l1.item(),
                    "dX": x.grad.cpu(), "dG": gl.grad.cpu(), "dK": kl.grad.cpu(),
                    "dV": vl.grad.cpu(), "h": (h0, h1)}, os.path.join(out_dir, f"t{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_rank_sharded_training_op_matches_single_gpu(tmp_path):
    """Forward + backward of the hybrid operator over two d_ff shards against the same
    operator unsharded on one GPU (bf16 results: shard sums differ only by rounding)."""
    from sparser_faster_llms_b200 import sparse_ops
    mp.spawn(_training_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    sparse_ops.register_ops()
    dev = torch.device("cuda", 0)
    x, g, k, v, w = _training_case(dev)
    for t in (x, g, k, v):
        t.requires_grad_(True)
    out, l0, l1 = torch.ops.sparse_ops.ff_forward_gated(x, g, k, v)[:3]
    ((out.float() * w.float()).sum() + 0.5 * l1).backward()

    def rel(a, b):
        a, b = a.float().cpu(), b.float().cpu()
        return ((a - b).norm() / b.norm()).item()

    parts = [torch.load(tmp_path / f"t{r}.pt") for r in range(2)]
    for p in parts:
        assert rel(p["out"], out.detach()) < 1e-2
        assert abs(p["l0"] - l0.item()) < 1e-3 * l0.item()
        assert abs(p["l1"] - l1.item()) < 1e-3 * abs(l1.item())
        assert rel(p["dX"], x.grad) < 1.5e-2
        h0, h1 = p["h"]
        assert rel(p["dG"], g.grad[h0:h1]) < 1e-2
        assert rel(p["dK"], k.grad[h0:h1]) < 1e-2
        assert rel(p["dV"], v.grad[h0:h1]) < 1e-2
    assert torch.equal(parts[0]["out"], parts[1]["out"])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_rank_sharded_ffn_matches_dense(tmp_path):
    from oracle import ffn_oracle as fo
    from sparser_faster_llms_b200 import synthetic
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    d, h, m = 2048, 11008, 16
    ffn = synthetic.make_ffn(d, h, seed=95, density=0.02, skew_sigma=1.0)
    x = synthetic.make_tokens(m, d, seed=96)
    ref = fo.dense_ffn(x, ffn.gate, ffn.up, ffn.down)
    y = torch.load(tmp_path / "y.pt")
    _, rel = fo.max_abs_and_rel_l2(y.float(), ref)
    assert rel < 1.2e-2, rel
