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
