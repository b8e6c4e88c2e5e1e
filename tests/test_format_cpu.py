"""TwELL slab format properties (CPU): the oracle's writer/reader and the package's
``packed_to_dense`` agree, counts are true counts, entries are ascending and in-tile."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from oracle import twell_format as tf
from sparser_faster_llms_b200 import twell


def as_u32_tensor(a):
    return torch.from_numpy(a.view(np.int32)).view(torch.uint32)


@settings(max_examples=40, deadline=None)
@given(m=st.integers(1, 6), tiles=st.integers(1, 4), cf=st.sampled_from([2, 4, 8]),
       density=st.floats(0.0, 0.6), seed=st.integers(0, 10_000))
def test_pack_properties(m, tiles, cf, density, seed):
    rng = np.random.default_rng(seed)
    h = tiles * 256
    z = rng.standard_normal((m, h)).astype(np.float32)
    z = np.where(rng.random((m, h)) < density, np.abs(z), -np.abs(z)).astype(np.float32)
    z[0, 0] = 0.0  # exactly zero is not kept (strict > 0)
    packed = tf.pack_preactivations(z, cf)
    w = tf.slab_words(cf)
    assert packed.shape == (m, tf.packed_width(h, cf)) == (m, twell.packed_width(h, compression_factor=cf))
    counts = tf.slab_counts(packed, cf)
    assert np.array_equal(counts, (z > 0).reshape(m, tiles, 256).sum(-1))
    for r, ent in enumerate(tf.slab_entries(packed, cf)):
        cols = [c for c, _ in ent]
        assert cols == sorted(set(cols))
        assert all(z[r, c] > 0 for c in cols)
    overflow = (counts > w - 1).any()
    if overflow:
        with pytest.raises(ValueError):
            tf.unpack_to_dense(packed, h, cf)
        with pytest.raises(ValueError):
            twell.packed_to_dense(as_u32_tensor(packed), h, compression_factor=cf)
    else:
        dense = tf.unpack_to_dense(packed, h, cf)
        assert np.array_equal(dense, tf.bf16_round(np.maximum(z, 0)))
        ours = twell.packed_to_dense(as_u32_tensor(packed), h, compression_factor=cf)
        assert np.array_equal(ours.float().numpy(), dense)
    # canonical form is insensitive to entry order and unused-word contents
    shuffled = packed.copy().reshape(m, tiles, w)
    for r in range(m):
        for t in range(tiles):
            n = min(int(shuffled[r, t, 0]), w - 1)
            shuffled[r, t, 1:1 + n] = rng.permutation(shuffled[r, t, 1:1 + n])
            shuffled[r, t, 1 + n:] = rng.integers(0, 2**32, w - 1 - n, dtype=np.uint64).astype(np.uint32)
    assert np.array_equal(tf.canonicalize(shuffled.reshape(m, -1), cf), tf.canonicalize(packed, cf))


def test_bf16_rounding_matches_torch():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(100000).astype(np.float32) * rng.choice([1e-3, 1.0, 1e3], 100000).astype(np.float32)
    ours = tf.f32_to_bf16_bits(x)
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ours, ref)


def test_d_ff_shards_concatenate_to_unsharded_slab():
    rng = np.random.default_rng(1)
    m, h = 5, 1024
    z = np.where(rng.random((m, h)) < 0.05, 1.0, -1.0).astype(np.float32) * rng.random((m, h)).astype(np.float32)
    full = tf.pack_preactivations(z, 8)
    parts = []
    for h0, h1 in ((0, 512), (512, 1024)):
        p = tf.pack_preactivations(z[:, h0:h1], 8)  # local column indices
        slabs = p.reshape(m, -1, 32).copy()
        cnt = np.minimum(slabs[:, :, 0], 31)
        valid = np.arange(31)[None, None, :] < cnt[:, :, None]
        slabs[:, :, 1:][valid] += h0  # rebase
        parts.append(slabs.reshape(m, -1))
    assert np.array_equal(np.concatenate(parts, axis=1), full)


def test_width_and_cf_validation():
    with pytest.raises(ValueError):
        twell.packed_width(300)
    with pytest.raises(ValueError):
        twell.packed_width(256, compression_factor=3)
    assert twell.packed_width(8192) == 1024
    assert twell.packed_width(11008, compression_factor=2) == 43 * 128
    out = twell.allocate_packed_output(3, 512, device="cpu")
    assert out.dtype == torch.uint32 and out.shape == (3, 64) and int(out.view(torch.int32).abs().sum()) == 0
