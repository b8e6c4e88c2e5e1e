"""d_ff sharding: host-side logic with world_size-2 (and 3) gloo ranks on CPU.

The per-rank compute is replaced by the CPU oracle through ``local_factory`` (the product's
default local module needs CUDA); what is tested here is the partition, the weight slicing,
the all-reduce plumbing and the per-shard slab indices.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from oracle import ffn_oracle as fo
from oracle import twell_format as tf
from sparser_faster_llms_b200 import sharded, synthetic


def test_shard_ranges_cover_d_ff_tile_granular_and_uneven():
    for h, world in ((8192, 2), (8192, 8), (11008, 2), (11008, 4), (11008, 8), (4096, 3)):
        ranges = [sharded.shard_range(h, r, world) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == h
        for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
            assert a1 == b0
        sizes = [(b - a) // 256 for a, b in ranges]
        assert all((b - a) % 256 == 0 for a, b in ranges)
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    assert [sharded.shard_range(11008, r, 8)[1] - sharded.shard_range(11008, r, 8)[0]
            for r in range(8)] == [1536, 1536, 1536, 1280, 1280, 1280, 1280, 1280]
    with pytest.raises(ValueError):
        sharded.shard_range(512, 0, 4)
    with pytest.raises(ValueError):
        sharded.shard_range(1000, 0, 2)


class OracleLocal(nn.Module):
    """Stand-in for the CUDA module: the CPU oracle on this rank's shard."""

    def __init__(self, layer_number, GATE, UP, DOWN, **kw):
        super().__init__()
        self.g, self.u, self.d = GATE, UP, DOWN

    def forward(self, A):
        y, self.packed = fo.gated_mlp(A, self.g, self.u, self.d)
        return y


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, h, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d, m = 256, 6
        ffn = synthetic.make_ffn(d, h, seed=90, density=0.03, skew_sigma=1.0)
        x = synthetic.make_tokens(m, d, seed=91)
        mod = sharded.ShardedTwELLGatedMLP(0, ffn.gate, ffn.up, ffn.down,
                                           local_factory=OracleLocal,
                                           reduce_dtype=torch.float32)
        y = mod(x)
        h0, h1 = mod.h_range
        np.savez(os.path.join(out_dir, f"r{rank}.npz"), y=y.numpy(), packed=mod.local.packed,
                 h0=h0, h1=h1)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,h", [(2, 1024), (3, 1280)])
def test_sharded_module_equals_unsharded(tmp_path, world, h):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, h, str(tmp_path)), nprocs=world, join=True)
    d, m = 256, 6
    ffn = synthetic.make_ffn(d, h, seed=90, density=0.03, skew_sigma=1.0)
    x = synthetic.make_tokens(m, d, seed=91)
    ref = fo.dense_ffn(x, ffn.gate, ffn.up, ffn.down)
    full_packed = fo.pack_gate(x, ffn.gate)
    outs = [np.load(tmp_path / f"r{r}.npz") for r in range(world)]
    for o in outs[1:]:
        assert np.array_equal(o["y"], outs[0]["y"])  # every rank holds the reduced output
    _, rel = fo.max_abs_and_rel_l2(torch.from_numpy(outs[0]["y"]), ref)
    assert rel < 1.5e-2
    # per-shard slabs carry local column indices; rebased and concatenated they are the full slab
    parts = []
    for o in outs:
        slabs = o["packed"].reshape(m, -1, 32).copy()
        cnt = np.minimum(slabs[:, :, 0], 31)
        valid = np.arange(31)[None, None, :] < cnt[:, :, None]
        slabs[:, :, 1:][valid] += int(o["h0"])
        parts.append(slabs.reshape(m, -1))
    assert np.array_equal(tf.canonicalize(np.concatenate(parts, 1)), tf.canonicalize(full_packed))


def _early_exit_worker(rank, world, port):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        os._exit(0)  # leaves between steps, with nothing in flight
    t = torch.ones(4)
    try:
        dist.all_reduce(t)
    except Exception:
        os._exit(17)  # the survivor learns of it on the host as an error, not a hang
    os._exit(3)


def test_rank_that_leaves_is_detected_on_the_host():
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_early_exit_worker, args=(r, 2, port)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert procs[1].exitcode == 0
    assert procs[0].exitcode == 17
