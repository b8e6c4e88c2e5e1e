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


def _dense_training_op(X, G, K, V):
    """Dense fp32 formula of the hybrid operator (out, l0, l1); autograd does the backward."""
    m = X.shape[0] * X.shape[1]
    g = torch.relu(X @ G.T)
    t = g * (X @ K.T)
    return t @ V, (g > 0).float().sum() / m, t.abs().sum() / m


def _training_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        X, G, K, V, W = _training_case()
        Gl, Kl, Vl = sharded.shard_weights(G, K, V, rank, world)
        X = X.clone().requires_grad_(True)
        Gl, Kl, Vl = (t.clone().requires_grad_(True) for t in (Gl, Kl, Vl))
        out, l0, l1 = sharded.sharded_ff_gated(X, Gl, Kl, Vl, local_op=_dense_training_op)
        loss = (out * W).sum() + 0.3 * l1
        loss.backward()
        h0, h1 = sharded.shard_range(G.shape[0], rank, world)
        np.savez(os.path.join(out_dir, f"t{rank}.npz"), out=out.detach().numpy(),
                 l0=l0.item(), l1=l1.item(), dX=X.grad.numpy(), dG=Gl.grad.numpy(),
                 dK=Kl.grad.numpy(), dV=Vl.grad.numpy(), h0=h0, h1=h1)
    finally:
        dist.destroy_process_group()


def _training_case():
    gen = torch.Generator().manual_seed(123)
    b, s, d, h = 2, 5, 64, 768
    X = torch.randn(b, s, d, generator=gen)
    G = torch.randn(h, d, generator=gen) * 0.1
    K = torch.randn(h, d, generator=gen) * 0.1
    V = torch.randn(h, d, generator=gen) * 0.1
    W = torch.randn(b, s, d, generator=gen)
    return X, G, K, V, W


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_training_forward_backward_equals_unsharded(tmp_path, world):
    port = _free_port()
    mp.spawn(_training_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    X, G, K, V, W = _training_case()
    X.requires_grad_(True)
    G.requires_grad_(True)
    K.requires_grad_(True)
    V.requires_grad_(True)
    out, l0, l1 = _dense_training_op(X, G, K, V)
    ((out * W).sum() + 0.3 * l1).backward()
    outs = [np.load(tmp_path / f"t{r}.npz") for r in range(world)]
    for o in outs:
        assert np.allclose(o["out"], out.detach().numpy(), rtol=1e-4, atol=1e-5)
        assert abs(o["l0"] - l0.item()) < 1e-3 and abs(o["l1"] - l1.item()) < 1e-4
        assert np.allclose(o["dX"], X.grad.numpy(), rtol=1e-4, atol=1e-5)
        h0, h1 = int(o["h0"]), int(o["h1"])
        assert np.allclose(o["dG"], G.grad.numpy()[h0:h1], rtol=1e-4, atol=1e-5)
        assert np.allclose(o["dK"], K.grad.numpy()[h0:h1], rtol=1e-4, atol=1e-5)
        assert np.allclose(o["dV"], V.grad.numpy()[h0:h1], rtol=1e-4, atol=1e-5)


def test_fused_allreduce_is_attached_only_to_calls_it_serves():
    """Host logic of the sharded module's fused path, with fakes: a call the fused form serves
    attaches it to the layer's cached state and returns the local module's (already reduced)
    output; any other call detaches it and goes through the separate all-reduce."""
    from sparser_faster_llms_b200 import twell

    class FakeLocal(nn.Module):
        layer_number = 4711

        def __init__(self, layer_number, GATE, UP, DOWN, **kw):
            super().__init__()
            twell._D2T_LAYERS[self.layer_number] = {"B": GATE, "cf": 8, "bias": None, "m": None}

        def forward(self, A):
            fused = "fused_allreduce" in twell._D2T_LAYERS[self.layer_number]
            return A + (100.0 if fused else 1.0)

    class FakeFused:
        def serves(self, tokens, d_model):
            return tokens <= 4

    class FakePeer:
        def all_reduce(self, y):
            return y * 2

    w = torch.zeros(512, 8)
    mod = sharded.ShardedTwELLGatedMLP(0, w, w, w, rank=0, world_size=2, presharded=True,
                                       local_factory=FakeLocal, fused_allreduce=FakeFused(),
                                       peer_allreduce=FakePeer())
    try:
        small, large = torch.zeros(2, 2, 8), torch.zeros(3, 5, 8)   # 4 and 15 tokens
        assert torch.equal(mod(small), small + 100.0)
        assert "fused_allreduce" in twell._D2T_LAYERS[4711]
        assert torch.equal(mod(large), (large + 1.0) * 2)
        assert "fused_allreduce" not in twell._D2T_LAYERS[4711]
        assert torch.equal(mod(small), small + 100.0)
    finally:
        twell._D2T_LAYERS.pop(4711, None)


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
