"""TwELL packed-slab format: CPU restatement (test infrastructure only).

Format (reference writer: custom_models/twell_modules/matmul_d2t.cu:614-704;
reference reader/spec: custom_models/twell_modules/twell.py:152-264):

* ``packed[M, (H/256) * W]`` uint32, ``W = 256 / compression_factor``.
* Tile ``t`` of row ``r`` occupies words ``[t*W, (t+1)*W)``.
* Word 0 of a tile is the number of strictly positive pre-activations among
  that tile's 256 columns (the true count, which can exceed the capacity).
* Words ``1..min(count, W-1)`` hold ``col | bf16_bits(value) << 16`` where
  ``col`` is the column index relative to the weight matrix handed to the
  kernel (< 65536).  Remaining words are unspecified.

The reference kernel appends entries in whatever order its shared-memory
atomics resolve (matmul_d2t.cu:646-651); this restatement, like the CUDA
kernels of this repository, uses ascending column order, so comparisons
against a reference-produced slab must sort each slab first.
"""
from __future__ import annotations

import numpy as np

TILE_N = 256
SUPPORTED_CF = (2, 4, 8)


def slab_words(compression_factor: int) -> int:
    """Words per (row, 256-column tile) slab.  twell.py:152-159."""
    if int(compression_factor) not in SUPPORTED_CF:
        raise ValueError("compression_factor must be one of {8, 4, 2}")
    return TILE_N // int(compression_factor)


def packed_width(output_n: int, compression_factor: int = 8) -> int:
    """Total uint32 words per row.  twell.py:152-159."""
    if output_n % TILE_N != 0:
        raise ValueError(f"output_n must be divisible by {TILE_N}")
    return (output_n // TILE_N) * slab_words(compression_factor)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16).

    Same rounding as ``__float2bfloat16`` used by the reference pack epilogue
    (matmul_d2t.cu:660-662).  NaN is not expected on this path.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounding = ((u >> 16) & 1) + 0x7FFF
    return ((u + rounding) >> 16).astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    return (bits.astype(np.uint32) << 16).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 values rounded to the nearest bf16, returned as fp32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def pack_preactivations(z: np.ndarray, compression_factor: int = 8,
                        fill: int = 0) -> np.ndarray:
    """Pack fp32 gate pre-activations ``z[M, H]`` into TwELL slabs.

    Keeps ``z > 0`` (fp32 test, matmul_d2t.cu:643), value = RN bf16 of ``z``.
    Entries are in ascending column order; at most ``W-1`` are stored while the
    count word keeps the true count.  Unused words are ``fill``.
    """
    z = np.ascontiguousarray(z, dtype=np.float32)
    m, h = z.shape
    w = slab_words(compression_factor)
    tiles = h // TILE_N
    if h % TILE_N:
        raise ValueError("H must be a multiple of 256")
    if h > 65536:
        raise ValueError("column indices are 16-bit: H must be <= 65536")
    out = np.full((m, tiles * w), fill, dtype=np.uint32)
    bits = f32_to_bf16_bits(z).astype(np.uint32)
    cols = np.arange(h, dtype=np.uint32)
    words = cols[None, :] | (bits << 16)
    pos = z > 0
    for t in range(tiles):
        p = pos[:, t * TILE_N:(t + 1) * TILE_N]
        cnt = p.sum(axis=1)
        out[:, t * w] = cnt.astype(np.uint32)
        # rank of each positive inside its slab (ascending column order)
        rank = np.cumsum(p, axis=1) - 1
        keep = p & (rank < (w - 1))
        r_idx, c_idx = np.nonzero(keep)
        out[r_idx, t * w + 1 + rank[r_idx, c_idx]] = words[r_idx, t * TILE_N + c_idx]
    return out


def slab_counts(packed: np.ndarray, compression_factor: int = 8) -> np.ndarray:
    """Count words ``[M, H/256]`` (int64)."""
    w = slab_words(compression_factor)
    return packed[:, ::w].astype(np.int64)


def unpack_to_dense(packed: np.ndarray, output_n: int,
                    compression_factor: int = 8, strict: bool = True):
    """Decode slabs to a dense fp32 matrix of bf16-representable values.

    Independent restatement of twell.py:215-264.  With ``strict`` a count above
    the capacity raises ``ValueError`` exactly like the reference; otherwise the
    stored ``W-1`` entries are decoded.
    """
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    w = slab_words(compression_factor)
    tiles = output_n // TILE_N
    m = packed.shape[0]
    if packed.shape[1] != tiles * w:
        raise ValueError(
            f"packed width mismatch: got {packed.shape[1]}, expected {tiles * w}")
    out = np.zeros((m, output_n), dtype=np.float32)
    slots = np.arange(w - 1)[None, :]
    for t in range(tiles):
        slab = packed[:, t * w:(t + 1) * w]
        cnt = slab[:, 0].astype(np.int64)
        if strict and (cnt > w - 1).any():
            raise ValueError(
                f"Embedded count exceeds payload slots in tile {t}: "
                f"max={int(cnt.max())}, max_allowed={w - 1}")
        valid = slots < np.minimum(cnt, w - 1)[:, None]
        payload = slab[:, 1:]
        r_idx, s_idx = np.nonzero(valid)
        col = (payload[r_idx, s_idx] & 0xFFFF).astype(np.int64)
        val = bf16_bits_to_f32((payload[r_idx, s_idx] >> 16).astype(np.uint16))
        out[r_idx, col] = val
    return out


def slab_entries(packed: np.ndarray, compression_factor: int = 8):
    """Per-row list of ``(col, bf16_bits)`` in stored order (valid slots only)."""
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    w = slab_words(compression_factor)
    tiles = packed.shape[1] // w
    rows = []
    for r in range(packed.shape[0]):
        ent = []
        for t in range(tiles):
            slab = packed[r, t * w:(t + 1) * w]
            n = min(int(slab[0]), w - 1)
            for s in range(1, n + 1):
                ent.append((int(slab[s]) & 0xFFFF, int(slab[s]) >> 16))
        rows.append(ent)
    return rows


def canonicalize(packed: np.ndarray, compression_factor: int = 8) -> np.ndarray:
    """Zero the unspecified words and sort every slab's entries by column.

    Gives a byte-comparable form of a slab buffer whatever order its writer
    used and whatever the unused words contain.
    """
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    w = slab_words(compression_factor)
    m, width = packed.shape
    tiles = width // w
    slabs = packed.reshape(m, tiles, w)
    cnt = slabs[:, :, 0].astype(np.int64)
    nvalid = np.minimum(cnt, w - 1)
    payload = slabs[:, :, 1:].copy()
    slot = np.arange(w - 1)[None, None, :]
    invalid = slot >= nvalid[:, :, None]
    key = (payload & 0xFFFF).astype(np.int64)
    key[invalid] = 1 << 20  # sorts after every real column
    order = np.argsort(key, axis=2, kind="stable")
    payload = np.take_along_axis(payload, order, axis=2)
    payload[np.take_along_axis(invalid, order, axis=2)] = 0
    out = np.empty_like(slabs)
    out[:, :, 0] = slabs[:, :, 0]
    out[:, :, 1:] = payload
    return out.reshape(m, width)
