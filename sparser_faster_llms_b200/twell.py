"""Drop-in replacement for the reference module ``custom_models.twell_modules.twell``.

Same public names, argument order, defaults and error behaviour as the reference
(custom_models/twell_modules/twell.py:40-1097); the bodies call the sm_100a
kernels of ``libb200_sparse_ffn.so`` through ctypes instead of a JIT-built
pybind extension.  Differences a caller can observe:

* any ``M >= 1``, ``d_model`` in 256..4096 (multiple of 256) and ``d_ff`` up to
  65536 (multiple of 256) are accepted; the reference accepts only
  ``d_model == 2048``, ``d_ff`` in {5632, 8192} and ``M % 256 == 0``
  (matmul_gated_t2d.cu:617-654);
* slab entries are in ascending column order (the reference's order depends on
  shared-memory atomics, matmul_d2t.cu:646-651);
* kernels run on torch's current stream (the reference uses stream 0,
  twell.cpp:442);
* ``flex_kernels`` selects nothing: one kernel reads every slab width;
* there is no CPU path: CUDA tensors are required and a missing library raises.

``ext=`` arguments are accepted and ignored.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from types import SimpleNamespace
from typing import Final

import torch
from torch import nn

from . import _lib

# Attributes the reference module exposes and the reference benchmark pokes at
# (benchmark_inference.py:55-117).  There is no JIT build here; they exist so that
# code written against the reference module keeps working.
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
_BASE_DIR = Path(__file__).resolve().parent
_DEFAULT_EXT_NAME = "twell_prod_ext"
_SHARED_PACKED_HIDDEN_STATE: torch.Tensor | None = None
_SHARED_PACKED_HIDDEN_STATE_SPEC: tuple[str, int, int, int, int] | None = None
_SUPPORTED_COMPRESSION_FACTORS: Final[set[int]] = {2, 4, 8}

ALGORITHM_SPECS = {
    "twell_d2t": {"source": "csrc/twell_pack.cu", "deps": []},
    "twell_t2d": {"source": "csrc/twell_t2d.cu", "deps": []},
    "twell_gated_t2d": {"source": "csrc/twell_t2d.cu", "deps": []},
    "twell_mlp": {"source": "csrc/c_api.cu",
                  "deps": ["twell_d2t", "twell_t2d", "twell_gated_t2d"]},
}


def sparse_algorithms() -> list[str]:
    """Returns the supported sparse algorithm keys."""
    return sorted(ALGORITHM_SPECS.keys())


def _validate_algorithms(algorithms: list[str]) -> list[str]:
    selected = [a.strip().lower() for a in algorithms if a.strip()]
    if not selected:
        raise ValueError("No algorithms selected")
    unknown = [a for a in selected if a not in ALGORITHM_SPECS]
    if unknown:
        raise ValueError(
            f"Unknown algorithm(s): {unknown}. Available: {', '.join(sparse_algorithms())}")
    return selected


def _resolve_algorithms_with_deps(selected: list[str]) -> list[str]:
    resolved: list[str] = []
    seen: set[str] = set()

    def visit(key: str) -> None:
        if key in seen:
            return
        for dep in ALGORITHM_SPECS[key].get("deps", []):
            visit(dep)
        seen.add(key)
        resolved.append(key)

    for key in selected:
        visit(key)
    return resolved


def load(*args, **kwargs):
    """Stand-in for ``torch.utils.cpp_extension.load``: the kernels are prebuilt."""
    return _native_namespace()


_EXT_CACHE: dict[tuple[str, ...], object] = {}


def load_ext(name: str = _DEFAULT_EXT_NAME, algorithms: list[str] | None = None,
             verbose: bool = False):
    """Returns the native namespace after validating the algorithm keys."""
    _resolve_algorithms_with_deps(_validate_algorithms(algorithms or ["twell_d2t"]))
    return _native_namespace()


def get_ext(algorithms: list[str] | None = None, verbose: bool = False):
    """Returns a cached handle for the requested algorithms (loads the library)."""
    selected = _resolve_algorithms_with_deps(
        _validate_algorithms(algorithms or ["twell_d2t"]))
    key = tuple(selected)
    module = _EXT_CACHE.get(key)
    if module is None:
        module = load_ext(algorithms=selected, verbose=verbose)
        _EXT_CACHE[key] = module
    return module


def _module_for(ext, *, algorithms: list[str]):
    return ext if ext is not None else get_ext(algorithms=algorithms)


def _validate_compression_factor(compression_factor: int) -> int:
    compression_factor = int(compression_factor)
    if compression_factor not in _SUPPORTED_COMPRESSION_FACTORS:
        raise ValueError("compression_factor must be one of {8, 4, 2}")
    return compression_factor


# --------------------------------------------------------------------------
# TwELL format helpers (reference: twell.py:152-264)
# --------------------------------------------------------------------------
def packed_width(output_n: int, tile_n: int = 256, compression_factor: int = 8) -> int:
    """Returns the packed width used by TwELL sparse outputs."""
    compression_factor = _validate_compression_factor(compression_factor)
    if output_n % tile_n != 0:
        raise ValueError(f"output_n must be divisible by {tile_n}")
    if tile_n % compression_factor != 0:
        raise ValueError("tile_n must be divisible by compression_factor")
    return (output_n // tile_n) * (tile_n // compression_factor)


def allocate_packed_output(m: int, n: int, *, device: torch.device | str, tile_n: int = 256,
                           compression_factor: int = 8) -> torch.Tensor:
    """Allocates a zeroed packed sparse output buffer."""
    return torch.zeros(
        (m, packed_width(n, tile_n=tile_n, compression_factor=compression_factor)),
        device=device, dtype=torch.uint32)


def _shared_packed_hidden_state(m: int, n: int, *, device: torch.device,
                                compression_factor: int = 8) -> torch.Tensor:
    """One process-wide slab buffer shared by every layer (reference: twell.py:178-204).

    Safe only because layers run one after another on one stream.
    """
    global _SHARED_PACKED_HIDDEN_STATE, _SHARED_PACKED_HIDDEN_STATE_SPEC
    compression_factor = _validate_compression_factor(compression_factor)
    device_index: Final[int] = -1 if device.index is None else int(device.index)
    key = (device.type, device_index, int(m), int(n), compression_factor)
    if (_SHARED_PACKED_HIDDEN_STATE is None or _SHARED_PACKED_HIDDEN_STATE_SPEC != key
            or _SHARED_PACKED_HIDDEN_STATE.device != device):
        _SHARED_PACKED_HIDDEN_STATE = allocate_packed_output(
            m, n, device=device, compression_factor=compression_factor)
        _SHARED_PACKED_HIDDEN_STATE_SPEC = key
    return _SHARED_PACKED_HIDDEN_STATE


def _clear_shared_packed_hidden_state() -> None:
    global _SHARED_PACKED_HIDDEN_STATE, _SHARED_PACKED_HIDDEN_STATE_SPEC
    _SHARED_PACKED_HIDDEN_STATE = None
    _SHARED_PACKED_HIDDEN_STATE_SPEC = None


def packed_to_dense(packed: torch.Tensor, output_n: int, tile_n: int = 256,
                    compression_factor: int = 8) -> torch.Tensor:
    """Converts a packed TwELL tensor back to a dense bf16 tensor (any device)."""
    compression_factor = _validate_compression_factor(compression_factor)
    m, compressed_n = packed.shape
    expected = packed_width(output_n, tile_n=tile_n, compression_factor=compression_factor)
    if packed.dtype != torch.uint32:
        raise ValueError(f"packed tensor must be uint32, got {packed.dtype}")
    if compressed_n != expected:
        raise ValueError(f"packed width mismatch: got {compressed_n}, expected {expected}")
    w = tile_n // compression_factor
    tiles = output_n // tile_n
    slabs = packed.view(torch.int32).to(torch.int64).bitwise_and(0xFFFFFFFF).view(m, tiles, w)
    counts = slabs[:, :, 0]
    if bool((counts > w - 1).any()):
        bad = int((counts > w - 1).any(dim=0).nonzero()[0])
        raise ValueError(
            f"Embedded count exceeds payload slots in tile {bad}: "
            f"max={int(counts[:, bad].max().item())}, max_allowed={w - 1}")
    payload = slabs[:, :, 1:]
    valid = torch.arange(w - 1, device=packed.device)[None, None, :] < counts[:, :, None]
    rows = torch.arange(m, device=packed.device)[:, None, None].expand_as(payload)[valid]
    cols = (payload % 65536)[valid]
    vals = (payload // 65536)[valid].to(torch.uint16).view(torch.bfloat16)
    out = torch.zeros((m, output_n), device=packed.device, dtype=torch.bfloat16)
    out[rows, cols] = vals
    return out


# --------------------------------------------------------------------------
# argument checks shared by the functional wrappers
# --------------------------------------------------------------------------
def _need(t: torch.Tensor, name: str, dtype: torch.dtype, ndim: int = 2) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if t.dtype != dtype:
        raise RuntimeError(f"{name}: expected scalar type {dtype} but found {t.dtype}")
    if t.dim() != ndim:
        raise ValueError(f"{name} must be {ndim}-D, got shape {tuple(t.shape)}")
    if not t.is_cuda:
        raise RuntimeError(
            f"{name} must be a CUDA tensor: the TwELL kernels have no CPU implementation")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def _same_device(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors[1:]:
        if t is not None and t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def _check_packed(packed: torch.Tensor, m: int, h: int, cf: int, name: str) -> None:
    _need(packed, name, torch.uint32)
    want = packed_width(h, compression_factor=cf)
    if packed.shape[0] != m or packed.shape[1] != want:
        raise ValueError(
            f"{name} must have shape ({m}, {want}) for N={h}, compression_factor={cf}; "
            f"got {tuple(packed.shape)}")


# --------------------------------------------------------------------------
# native calls
# --------------------------------------------------------------------------
def _native_pack(A, B, C_packed, cf, bias=None) -> None:
    _need(A, "A", torch.bfloat16)
    _need(B, "B", torch.bfloat16)
    m, d = A.shape
    h = B.shape[0]
    if B.shape[1] != d:
        raise ValueError(f"A is [M, {d}] but B is {tuple(B.shape)}; expected [N, {d}]")
    _check_packed(C_packed, m, h, cf, "C_packed")
    if bias is not None:
        if bias.dtype != torch.float32 or bias.shape != (h,) or not bias.is_contiguous():
            raise ValueError("gate bias must be a contiguous float32 tensor of shape [N]")
    dev = _same_device(A, B, C_packed, bias)
    _lib.call("b200_twell_pack", dev, A.data_ptr(), B.data_ptr(), _lib.ptr(bias),
              C_packed.data_ptr(), m, d, h, cf)


def _native_gated_t2d(IN_dense, GATE_packed, UP, DOWN, OUT, highest_precision, cf) -> None:
    _need(IN_dense, "IN_dense", torch.bfloat16)
    _need(UP, "UP", torch.bfloat16)
    _need(DOWN, "DOWN", torch.bfloat16)
    _need(OUT, "OUT", torch.bfloat16)
    m, d = IN_dense.shape
    h = UP.shape[0]
    if UP.shape != (h, d) or DOWN.shape != (h, d):
        raise ValueError(
            f"UP and DOWN must both be [{h}, {d}]; got {tuple(UP.shape)} and {tuple(DOWN.shape)}")
    if OUT.shape != (m, d):
        raise ValueError(f"OUT must be [{m}, {d}], got {tuple(OUT.shape)}")
    _check_packed(GATE_packed, m, h, cf, "GATE_packed")
    dev = _same_device(IN_dense, GATE_packed, UP, DOWN, OUT)
    flags = _lib.FLAG_HIGH_PRECISION if highest_precision else 0
    _lib.call("b200_twell_gated_t2d", dev, IN_dense.data_ptr(), GATE_packed.data_ptr(),
              UP.data_ptr(), DOWN.data_ptr(), OUT.data_ptr(), m, d, h, cf, flags,
              *_lib.workspace(dev))


def _native_t2d(IN_packed, DOWN, OUT, num_splits, cf=8) -> None:
    _need(DOWN, "DOWN", torch.bfloat16)
    _need(OUT, "OUT", torch.bfloat16)
    h, d = DOWN.shape
    m = IN_packed.shape[0]
    if OUT.shape != (m, d):
        raise ValueError(f"OUT must be [{m}, {d}], got {tuple(OUT.shape)}")
    _check_packed(IN_packed, m, h, cf, "IN_packed")
    dev = _same_device(IN_packed, DOWN, OUT)
    _lib.call("b200_twell_t2d", dev, IN_packed.data_ptr(), DOWN.data_ptr(), OUT.data_ptr(),
              m, d, h, cf, int(num_splits), *_lib.workspace(dev))


# layer_number -> {"B": weight, "cf": int, "bias": tensor | None, "m": int | None}
_D2T_LAYERS: dict[int, dict] = {}


def _layer(layer_number: int) -> dict:
    try:
        return _D2T_LAYERS[int(layer_number)]
    except KeyError:
        raise RuntimeError(
            f"D2T layer {int(layer_number)} does not exist: call create_d2t_layer first") from None


def _native_namespace():
    """Object with the attribute names of the reference's pybind module
    (custom_models/twell_modules/twell.cpp:871-896); loading it loads the library."""
    _lib.load_library()
    return SimpleNamespace(
        matmul_sparse=lambda A, B, algorithm="twell_d2t", cf=8: matmul_sparse(
            A, B, algorithm, cf),
        matmul_sparse_out=lambda A, B, C, algorithm="twell_d2t", cf=8: matmul_sparse_out(
            A, B, C, algorithm, cf),
        matmul_t2d=matmul_t2d, matmul_t2d_out=matmul_t2d_out,
        matmul_gated_t2d=matmul_gated_t2d, matmul_gated_t2d_out=matmul_gated_t2d_out,
        create_d2t_layer=create_d2t_layer, run_d2t_layer=run_d2t_layer,
        ensure_d2t_layer_shape=ensure_d2t_layer_shape,
        run_mlp_layer=run_mlp_layer, run_gated_mlp_layer=run_gated_mlp_layer,
        run_mlp_layer_inplace=run_mlp_layer_inplace,
        run_gated_mlp_layer_inplace=run_gated_mlp_layer_inplace,
        destroy_d2t_layer=destroy_d2t_layer, destroy_all_d2t_layers=destroy_all_d2t_layers,
    )


# --------------------------------------------------------------------------
# functional API (reference: twell.py:267-578)
# --------------------------------------------------------------------------
def matmul_sparse(A: torch.Tensor, B: torch.Tensor, algorithm: str = "twell_d2t",
                  compression_factor: int = 8, ext=None) -> torch.Tensor:
    """Runs packed sparse matmul and returns the packed output."""
    compression_factor = _validate_compression_factor(compression_factor)
    _validate_algorithms([algorithm])
    C_packed = allocate_packed_output(A.size(0), B.size(0), device=A.device,
                                      compression_factor=compression_factor)
    matmul_sparse_out(A, B, C_packed, algorithm, compression_factor)
    return C_packed


def matmul_sparse_out(A: torch.Tensor, B: torch.Tensor, C_packed: torch.Tensor,
                      algorithm: str = "twell_d2t", compression_factor: int = 8,
                      ext=None) -> None:
    """Runs packed sparse matmul into a caller-provided packed output tensor."""
    compression_factor = _validate_compression_factor(compression_factor)
    if algorithm != "twell_d2t":
        _validate_algorithms([algorithm])
        raise ValueError(f"algorithm {algorithm!r} is not a packed matmul; use 'twell_d2t'")
    _native_pack(A, B, C_packed, compression_factor)


def matmul_t2d(IN_packed: torch.Tensor, DOWN: torch.Tensor, num_splits: int = 2,
               ext=None) -> torch.Tensor:
    """Runs packed-to-dense downprojection and returns the dense output."""
    OUT = torch.empty((IN_packed.size(0), DOWN.size(1)), device=DOWN.device, dtype=DOWN.dtype)
    matmul_t2d_out(IN_packed, DOWN, OUT, num_splits)
    return OUT


def matmul_t2d_out(IN_packed: torch.Tensor, DOWN: torch.Tensor, OUT: torch.Tensor,
                   num_splits: int = 2, ext=None) -> None:
    """Runs packed-to-dense downprojection into a caller-provided output tensor."""
    _native_t2d(IN_packed, DOWN, OUT, int(num_splits))


def matmul_gated_t2d(IN_dense: torch.Tensor, GATE_packed: torch.Tensor, UP: torch.Tensor,
                     DOWN: torch.Tensor, highest_precision: bool = False,
                     compression_factor: int = 8, flex_kernels: bool = False,
                     ext=None) -> torch.Tensor:
    """Runs gated packed-to-dense projection and returns the dense output."""
    compression_factor = _validate_compression_factor(compression_factor)
    if not flex_kernels and compression_factor != 8:
        raise ValueError("compression_factor != 8 requires flex_kernels=True")
    OUT = torch.empty_like(IN_dense)
    _native_gated_t2d(IN_dense, GATE_packed, UP, DOWN, OUT, bool(highest_precision),
                      compression_factor)
    return OUT


def matmul_gated_t2d_out(IN_dense: torch.Tensor, GATE_packed: torch.Tensor, UP: torch.Tensor,
                         DOWN: torch.Tensor, OUT: torch.Tensor, highest_precision: bool = False,
                         compression_factor: int = 8, flex_kernels: bool = False,
                         ext=None) -> None:
    """Runs gated packed-to-dense projection into a caller-provided output tensor."""
    compression_factor = _validate_compression_factor(compression_factor)
    if not flex_kernels and compression_factor != 8:
        raise ValueError("compression_factor != 8 requires flex_kernels=True")
    _native_gated_t2d(IN_dense, GATE_packed, UP, DOWN, OUT, bool(highest_precision),
                      compression_factor)


def create_d2t_layer(layer_number: int, B: torch.Tensor, compression_factor: int = 8,
                     ext=None) -> None:
    """Creates or refreshes cached D2T state for one layer id."""
    compression_factor = _validate_compression_factor(compression_factor)
    _need(B, "B", torch.bfloat16)
    _lib.load_library()
    prev = _D2T_LAYERS.get(int(layer_number))
    _D2T_LAYERS[int(layer_number)] = {
        "B": B, "cf": compression_factor, "m": None,
        "bias": prev["bias"] if prev and prev["B"].shape[0] == B.shape[0] else None}


def set_d2t_layer_bias(layer_number: int, bias: torch.Tensor | None) -> None:
    """Extension: add a per-neuron fp32 bias before the ReLU of one cached layer.

    The reference kernels take no bias; the default (``None``) keeps their
    behaviour.  Used to induce a target gate density with random weights.
    """
    entry = _layer(layer_number)
    if bias is not None:
        bias = bias.detach().to(device=entry["B"].device, dtype=torch.float32).contiguous()
        if bias.shape != (entry["B"].shape[0],):
            raise ValueError(f"bias must have shape [{entry['B'].shape[0]}]")
    entry["bias"] = bias


def run_d2t_layer(layer_number: int, A: torch.Tensor, C_packed: torch.Tensor, ext=None) -> None:
    """Runs one cached D2T layer into a packed output tensor."""
    entry = _layer(layer_number)
    _native_pack(A, entry["B"], C_packed, entry["cf"], entry["bias"])
    entry["m"] = int(A.size(0))


def ensure_d2t_layer_shape(layer_number: int, M: int, ext=None) -> None:
    """Ensures cached D2T state is ready for the requested row count."""
    if int(M) < 0:
        raise ValueError("M must be >= 0")
    _layer(layer_number)["m"] = int(M)


def _gated_mlp(layer_number, A, UP, DOWN, C_packed, OUT, highest_precision, cf) -> None:
    entry = _layer(layer_number)
    if entry["cf"] != cf:
        raise ValueError(
            f"layer {int(layer_number)} was created with compression_factor={entry['cf']}, "
            f"called with {cf}")
    GATE = entry["B"]
    _need(A, "A", torch.bfloat16)
    _need(UP, "UP", torch.bfloat16)
    _need(DOWN, "DOWN", torch.bfloat16)
    m, d = A.shape
    h = GATE.shape[0]
    if GATE.shape != (h, d) or UP.shape != (h, d) or DOWN.shape != (h, d):
        raise ValueError(
            f"GATE/UP/DOWN must all be [{h}, {d}]; got {tuple(GATE.shape)}, "
            f"{tuple(UP.shape)}, {tuple(DOWN.shape)}")
    _check_packed(C_packed, m, h, cf, "C_packed")
    dev = _same_device(A, GATE, UP, DOWN, C_packed, OUT)
    flags = _lib.FLAG_HIGH_PRECISION if highest_precision else 0
    route = entry.get("dense_route")
    far = entry.get("fused_allreduce")
    if far is not None and far.serves(m, d):
        # d_ff shard: the contraction sums the shards in its own epilogue (one kernel per rank)
        _lib.call("b200_twell_gated_mlp_allreduce", dev, A.data_ptr(), GATE.data_ptr(),
                  _lib.ptr(entry["bias"]), UP.data_ptr(), DOWN.data_ptr(), C_packed.data_ptr(),
                  OUT.data_ptr(), m, d, h, cf, flags, *_lib.workspace(dev), far.ptr_array,
                  far.rank, far.world, far.block_bytes)
    elif (route is not None and route["dense_all_tokens"] is not None
            and m >= route["dense_all_tokens"]):
        # so many tokens that every row is cheaper as dense GEMMs: no slab is produced
        ws_ptr, _ = _hybrid_workspace(dev, m, d, h, 0)
        _lib.call("b200_dense_gated_mlp", dev, A.data_ptr(), GATE.data_ptr(),
                  _lib.ptr(entry["bias"]), UP.data_ptr(), route["DOWN_T"].data_ptr(), ws_ptr,
                  OUT.data_ptr(), m, d, h)
        route["last"] = None
    elif route is not None and m >= route["min_tokens"]:
        cap = route["dense_cap"]
        cap = min(m, (max(128, m // 4) + 127) // 128 * 128) if cap is None else min(m, int(cap))
        thr = route["nnz_threshold"]
        thr = h // 16 if thr is None else int(thr)
        ws_ptr, ws_bytes = _hybrid_workspace(dev, m, d, h, cap)
        _lib.call("b200_twell_gated_mlp_hybrid", dev, A.data_ptr(), GATE.data_ptr(),
                  _lib.ptr(entry["bias"]), UP.data_ptr(), DOWN.data_ptr(),
                  route["DOWN_T"].data_ptr(), C_packed.data_ptr(), OUT.data_ptr(), m, d, h, cf,
                  flags, thr, cap, ws_ptr, ws_bytes, *_lib.workspace(dev))
        route["last"] = (m, d, h, cap)
    else:
        _lib.call("b200_twell_gated_mlp", dev, A.data_ptr(), GATE.data_ptr(),
                  _lib.ptr(entry["bias"]), UP.data_ptr(), DOWN.data_ptr(), C_packed.data_ptr(),
                  OUT.data_ptr(), m, d, h, cf, flags, *_lib.workspace(dev))
    entry["m"] = m


# One growing scratch buffer per device for the dense-row route (calls on a stream are
# serialised, so all layers share it).
_HYBRID_WS: dict[int, torch.Tensor] = {}


def _hybrid_workspace(dev: torch.device, m: int, d: int, h: int, cap: int) -> tuple[int, int]:
    if cap > 0:
        need = int(_lib.load_library().b200_twell_hybrid_workspace_bytes(m, d, h, cap))
    else:  # all rows dense: only the [M, H] bf16 hidden state
        need = m * h * 2
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    buf = _HYBRID_WS.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.empty(need, dtype=torch.uint8, device=dev)
        _HYBRID_WS[key] = buf
    return buf.data_ptr(), buf.numel()


def set_d2t_layer_dense_route(layer_number: int, DOWN_T: torch.Tensor | None, *,
                              dense_cap: int | None = None, nnz_threshold: int | None = None,
                              min_tokens: int = 256,
                              dense_all_tokens: int | None = None) -> None:
    """Extension: route dense-enough token rows of one cached gated layer to tensor-core GEMMs.

    ``DOWN_T`` is ``down_proj.weight`` itself, ``[D, H]`` bf16 contiguous (``None`` switches the
    route off = reference behaviour).  Rows with more than ``nnz_threshold`` gate positives
    (default ``H // 16``) or with an overflowed slab tile are computed densely, at most
    ``dense_cap`` of them per call (default a quarter of the rows); calls with fewer than
    ``min_tokens`` rows keep the gather kernel for every row.  Calls with at least
    ``dense_all_tokens`` rows (default: never) skip the slab altogether and run every row
    through the dense GEMMs.  The reference's TwELL path has no such route and drops
    overflowed entries; its hybrid format has the dense tail (hybrid_sp.cu:516-576).
    """
    entry = _layer(layer_number)
    if DOWN_T is None:
        entry.pop("dense_route", None)
        return
    _need(DOWN_T, "DOWN_T", torch.bfloat16)
    h, d = entry["B"].shape
    if DOWN_T.shape != (d, h):
        raise ValueError(f"DOWN_T must be [{d}, {h}], got {tuple(DOWN_T.shape)}")
    entry["dense_route"] = {"DOWN_T": DOWN_T, "dense_cap": dense_cap,
                            "nnz_threshold": nnz_threshold, "min_tokens": int(min_tokens),
                            "dense_all_tokens": dense_all_tokens, "last": None}


def set_d2t_layer_fused_allreduce(layer_number: int, fused) -> None:
    """Extension for d_ff-sharded layers: ``fused`` is a
    :class:`sparser_faster_llms_b200.peer_allreduce.FusedShardAllReduce` (or None to detach).
    Gated calls it serves (decode-sized token counts) then return the sum over all ranks'
    shards; every rank must make the same calls.  No reference counterpart."""
    entry = _layer(layer_number)
    if fused is None:
        entry.pop("fused_allreduce", None)
    else:
        entry["fused_allreduce"] = fused


def d2t_layer_dense_route_counters(layer_number: int) -> dict | None:
    """``{"dense_rows", "lossy_rows_left_sparse", "qualified_rows"}`` of the last routed call
    of this layer, or None if it has not run one.  Synchronises the device; valid only until
    another layer's routed call reuses the shared scratch buffer."""
    route = _layer(layer_number).get("dense_route")
    if route is None or route["last"] is None:
        return None
    m, d, h, cap = route["last"]
    dev = route["DOWN_T"].device
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    out = (ctypes.c_int * 3)()
    with torch.cuda.device(dev):
        _lib.check("b200_twell_hybrid_counters",
                   _lib.load_library().b200_twell_hybrid_counters(
                       _HYBRID_WS[key].data_ptr(), m, d, h, cap, out))
    return {"dense_rows": out[0], "lossy_rows_left_sparse": out[1], "qualified_rows": out[2]}


def _plain_mlp(layer_number, A, DOWN, C_packed, OUT, num_splits) -> None:
    entry = _layer(layer_number)
    UP = entry["B"]
    _need(A, "A", torch.bfloat16)
    _need(DOWN, "DOWN", torch.bfloat16)
    m, d = A.shape
    h = UP.shape[0]
    if UP.shape != (h, d) or DOWN.shape != (h, d):
        raise ValueError(f"UP/DOWN must both be [{h}, {d}]")
    _check_packed(C_packed, m, h, entry["cf"], "C_packed")
    dev = _same_device(A, UP, DOWN, C_packed, OUT)
    _lib.call("b200_twell_mlp", dev, A.data_ptr(), UP.data_ptr(), DOWN.data_ptr(),
              C_packed.data_ptr(), OUT.data_ptr(), m, d, h, entry["cf"], int(num_splits),
              *_lib.workspace(dev))
    entry["m"] = m


def _temp_packed(layer_number: int, A: torch.Tensor) -> torch.Tensor:
    entry = _layer(layer_number)
    return torch.empty(
        (A.size(0), packed_width(entry["B"].shape[0], compression_factor=entry["cf"])),
        device=A.device, dtype=torch.uint32)


def run_mlp_layer(layer_number: int, A: torch.Tensor, DOWN: torch.Tensor, num_splits: int = 2,
                  ext=None) -> torch.Tensor:
    """Runs the fused non-gated TwELL MLP."""
    OUT = torch.empty_like(A)
    _plain_mlp(layer_number, A, DOWN, _temp_packed(layer_number, A), OUT, num_splits)
    return OUT


def run_gated_mlp_layer(layer_number: int, A: torch.Tensor, UP: torch.Tensor, DOWN: torch.Tensor,
                        highest_precision: bool = False, compression_factor: int = 8,
                        flex_kernels: bool = False, ext=None) -> torch.Tensor:
    """Runs the fused gated TwELL MLP."""
    compression_factor = _validate_compression_factor(compression_factor)
    if not flex_kernels and compression_factor != 8:
        raise ValueError("compression_factor != 8 requires flex_kernels=True")
    OUT = torch.empty_like(A)
    _gated_mlp(layer_number, A, UP, DOWN, _temp_packed(layer_number, A), OUT,
               bool(highest_precision), compression_factor)
    return OUT


def _run_mlp_layer_with_hidden_states(layer_number: int, A: torch.Tensor, DOWN: torch.Tensor,
                                      C_packed: torch.Tensor, num_splits: int = 2,
                                      ext=None) -> torch.Tensor:
    """Runs the fused non-gated TwELL MLP with caller-provided packed hidden states."""
    OUT = torch.empty_like(A)
    _plain_mlp(layer_number, A, DOWN, C_packed, OUT, num_splits)
    return OUT


def _run_gated_mlp_layer_with_hidden_states(layer_number: int, A: torch.Tensor, UP: torch.Tensor,
                                            DOWN: torch.Tensor, C_packed: torch.Tensor,
                                            highest_precision: bool = False,
                                            compression_factor: int = 8,
                                            flex_kernels: bool = False, ext=None) -> torch.Tensor:
    """Runs the fused gated TwELL MLP with caller-provided packed hidden states."""
    compression_factor = _validate_compression_factor(compression_factor)
    if not flex_kernels and compression_factor != 8:
        raise ValueError("compression_factor != 8 requires flex_kernels=True")
    OUT = torch.empty_like(A)
    _gated_mlp(layer_number, A, UP, DOWN, C_packed, OUT, bool(highest_precision),
               compression_factor)
    return OUT


def run_mlp_layer_inplace(layer_number: int, A: torch.Tensor, DOWN: torch.Tensor,
                          num_splits: int = 2, ext=None) -> None:
    """Runs the fused non-gated TwELL MLP in place."""
    _plain_mlp(layer_number, A, DOWN, _temp_packed(layer_number, A), A, num_splits)


def run_gated_mlp_layer_inplace(layer_number: int, A: torch.Tensor, UP: torch.Tensor,
                                DOWN: torch.Tensor, highest_precision: bool = False,
                                compression_factor: int = 8, flex_kernels: bool = False,
                                ext=None) -> None:
    """Runs the fused gated TwELL MLP in place."""
    compression_factor = _validate_compression_factor(compression_factor)
    if not flex_kernels and compression_factor != 8:
        raise ValueError("compression_factor != 8 requires flex_kernels=True")
    _gated_mlp(layer_number, A, UP, DOWN, _temp_packed(layer_number, A), A,
               bool(highest_precision), compression_factor)


def _run_mlp_layer_inplace_with_hidden_states(layer_number: int, A: torch.Tensor,
                                              DOWN: torch.Tensor, C_packed: torch.Tensor,
                                              num_splits: int = 2, ext=None) -> None:
    """Runs the fused non-gated TwELL MLP in place with caller-provided packed hidden states."""
    _plain_mlp(layer_number, A, DOWN, C_packed, A, num_splits)


def _run_gated_mlp_layer_inplace_with_hidden_states(layer_number: int, A: torch.Tensor,
                                                    UP: torch.Tensor, DOWN: torch.Tensor,
                                                    C_packed: torch.Tensor,
                                                    highest_precision: bool = False,
                                                    compression_factor: int = 8,
                                                    flex_kernels: bool = False, ext=None) -> None:
    """Runs the fused gated TwELL MLP in place with caller-provided packed hidden states."""
    compression_factor = _validate_compression_factor(compression_factor)
    if not flex_kernels and compression_factor != 8:
        raise ValueError("compression_factor != 8 requires flex_kernels=True")
    _gated_mlp(layer_number, A, UP, DOWN, C_packed, A, bool(highest_precision),
               compression_factor)


def destroy_d2t_layer(layer_number: int, ext=None) -> None:
    """Destroys one cached D2T layer entry."""
    _D2T_LAYERS.pop(int(layer_number), None)


def destroy_all_d2t_layers(ext=None) -> None:
    """Destroys all cached D2T layer entries."""
    _D2T_LAYERS.clear()


# --------------------------------------------------------------------------
# object API (reference: twell.py:581-1097)
# --------------------------------------------------------------------------
class D2TLayer:
    """Caches and runs one D2T layer configuration."""

    def __init__(self, layer_number: int, B: torch.Tensor, compression_factor: int = 8,
                 ext=None):
        self.layer_number = int(layer_number)
        self.ext = _module_for(ext, algorithms=["twell_d2t"])
        self.m: int | None = None
        self.n = int(B.size(0))
        self.compression_factor = _validate_compression_factor(compression_factor)
        self.c_packed: torch.Tensor | None = None
        create_d2t_layer(self.layer_number, B, compression_factor=self.compression_factor,
                         ext=self.ext)

    def prepare(self, A: torch.Tensor, C_packed: torch.Tensor | None = None) -> torch.Tensor:
        m = int(A.size(0))
        if self.m != m:
            ensure_d2t_layer_shape(self.layer_number, m, ext=self.ext)
            self.m = m
            self.c_packed = None
        if C_packed is not None:
            return C_packed
        if (self.c_packed is None or self.c_packed.size(0) != A.size(0)
                or self.c_packed.device != A.device):
            self.c_packed = allocate_packed_output(
                A.size(0), self.n, device=A.device, compression_factor=self.compression_factor)
        return self.c_packed

    def prepare_shared_hidden_state(self, A: torch.Tensor) -> torch.Tensor:
        m = int(A.size(0))
        if self.m != m:
            ensure_d2t_layer_shape(self.layer_number, m, ext=self.ext)
            self.m = m
        return _shared_packed_hidden_state(m, self.n, device=A.device,
                                           compression_factor=self.compression_factor)

    def run(self, A: torch.Tensor, C_packed: torch.Tensor | None = None) -> torch.Tensor:
        packed = self.prepare(A, C_packed=C_packed)
        run_d2t_layer(self.layer_number, A, packed, ext=self.ext)
        return packed

    def destroy(self) -> None:
        destroy_d2t_layer(self.layer_number, ext=self.ext)
        self.m = None
        self.c_packed = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class D2TLinear(nn.Module):
    """nn.Module wrapper around one cached D2T layer."""

    def __init__(self, layer_number: int, B: torch.Tensor, compression_factor: int = 8,
                 ext=None):
        super().__init__()
        self.register_buffer("B", B.contiguous())
        self.layer = D2TLayer(layer_number=layer_number, B=self.B,
                              compression_factor=compression_factor, ext=ext)

    def forward(self, A: torch.Tensor, C_packed: torch.Tensor | None = None) -> torch.Tensor:
        return self.layer.run(A, C_packed=C_packed)

    def destroy(self) -> None:
        self.layer.destroy()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class T2DLinear(nn.Module):
    """nn.Module wrapper around the packed-to-dense downprojection."""

    def __init__(self, DOWN: torch.Tensor, num_splits: int = 2, compression_factor: int = 8,
                 ext=None):
        super().__init__()
        if compression_factor != 8:
            raise ValueError("Only compression_factor=8 is currently supported for T2DLinear")
        self.register_buffer("DOWN", DOWN.contiguous())
        self.num_splits = int(num_splits)
        self.ext = _module_for(ext, algorithms=["twell_t2d"])
        self._out: torch.Tensor | None = None

    def forward(self, IN_packed: torch.Tensor, OUT: torch.Tensor | None = None) -> torch.Tensor:
        if OUT is None:
            if (self._out is None or self._out.size(0) != IN_packed.size(0)
                    or self._out.device != IN_packed.device):
                self._out = torch.empty((IN_packed.size(0), self.DOWN.size(1)),
                                        device=IN_packed.device, dtype=self.DOWN.dtype)
            OUT = self._out
        matmul_t2d_out(IN_packed, self.DOWN, OUT, num_splits=self.num_splits, ext=self.ext)
        return OUT


class GatedT2DLinear(nn.Module):
    """nn.Module wrapper around the gated packed-to-dense projection."""

    def __init__(self, UP: torch.Tensor, DOWN: torch.Tensor, highest_precision: bool = False,
                 compression_factor: int = 8, flex_kernels: bool = False, ext=None):
        super().__init__()
        compression_factor = _validate_compression_factor(compression_factor)
        if compression_factor != 8 and not flex_kernels:
            raise ValueError(
                "Only compression_factor=8 is currently supported for "
                "GatedT2DLinear without flex kernels, please set flex_kernels=True")
        self.register_buffer("UP", UP.contiguous())
        self.register_buffer("DOWN", DOWN.contiguous())
        self.ext = _module_for(ext, algorithms=["twell_gated_t2d"])
        self.highest_precision = bool(highest_precision)
        self.compression_factor = compression_factor
        self.flex_kernels = bool(flex_kernels)
        self._out: torch.Tensor | None = None

    def forward(self, IN_dense: torch.Tensor, GATE_packed: torch.Tensor,
                OUT: torch.Tensor | None = None,
                highest_precision: bool | None = None) -> torch.Tensor:
        use_hp = self.highest_precision if highest_precision is None else bool(highest_precision)
        if OUT is None:
            if (self._out is None or self._out.size(0) != IN_dense.size(0)
                    or self._out.device != IN_dense.device):
                self._out = torch.empty((IN_dense.size(0), IN_dense.size(1)),
                                        device=IN_dense.device, dtype=IN_dense.dtype)
            OUT = self._out
        matmul_gated_t2d_out(IN_dense, GATE_packed, self.UP, self.DOWN, OUT,
                             highest_precision=use_hp,
                             compression_factor=self.compression_factor,
                             flex_kernels=self.flex_kernels, ext=self.ext)
        return OUT


class _BaseTwELLMLP(nn.Module):
    """What the two fused MLP modules share: weight buffers, lazily created per-layer state,
    and one forward that picks the functional entry point from (shared slab, in place).

    The modules are built on CPU and moved with ``.to(device).to(dtype)``
    (benchmark_inference.py:208-213), so the cached layer - which holds a reference to the
    first-projection weight - is created at the first forward and re-created whenever that
    buffer has been moved or cast since.  Subclasses name the first-projection buffer
    (``_first``), their four functional entry points (``_entry``) and the arguments those take
    between ``A`` and the packed buffer (``_call_args``).
    """

    _first: str = ""
    _entry: dict = {}

    def __init__(self, layer_number: int, *, inplace: bool, preallocate_shared_hidden_state: bool,
                 compression_factor: int, ext=None):
        super().__init__()
        self.layer_number = int(layer_number)
        self.ext = ext
        self.inplace = bool(inplace)
        self.preallocate_shared_hidden_state = bool(preallocate_shared_hidden_state)
        self.compression_factor = _validate_compression_factor(compression_factor)
        self._gate_bias: torch.Tensor | None = None
        self.layer: D2TLayer | None = None

    def _call_args(self) -> tuple[tuple, dict]:
        raise NotImplementedError

    def _apply_dense_route(self) -> None:  # gated modules override
        pass

    def _ensure_layer(self) -> None:
        weight = getattr(self, self._first)
        entry = _D2T_LAYERS.get(self.layer_number)
        if (self.layer is not None and entry is not None
                and entry["B"].data_ptr() == weight.data_ptr()):
            return
        if not weight.is_cuda:
            raise RuntimeError("TwELL MLP weights must be moved to CUDA before first forward")
        self.layer = D2TLayer(layer_number=self.layer_number, B=weight,
                              compression_factor=self.compression_factor, ext=self.ext)
        if self._gate_bias is not None:
            set_d2t_layer_bias(self.layer_number, self._gate_bias)
        self._apply_dense_route()

    def set_gate_bias(self, bias: torch.Tensor | None) -> None:
        """Extension: per-neuron bias added before the ReLU (None = reference behaviour)."""
        self._gate_bias = None if bias is None else bias.detach().float().contiguous()
        if self.layer is not None:
            set_d2t_layer_bias(self.layer_number, self._gate_bias)

    def forward(self, A: torch.Tensor) -> torch.Tensor:
        shape = A.shape
        rows = A.view(-1, shape[-1])
        self._ensure_layer()
        shared = self.preallocate_shared_hidden_state
        args, kwargs = self._call_args()
        if shared:  # one slab for all layers of the process (they run one after another)
            args = args + (self.layer.prepare_shared_hidden_state(rows),)
        out = self._entry[(shared, self.inplace)](self.layer_number, rows, *args, ext=self.ext,
                                                  **kwargs)
        return A if self.inplace else out.view(shape)

    def destroy(self) -> None:
        if self.layer is not None:
            self.layer.destroy()
            self.layer = None
        if self.preallocate_shared_hidden_state:
            _clear_shared_packed_hidden_state()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class TwELLMLP(_BaseTwELLMLP):
    """Fused non-gated TwELL MLP wrapper."""

    _first = "UP"
    _entry = {(False, False): run_mlp_layer, (False, True): run_mlp_layer_inplace,
              (True, False): _run_mlp_layer_with_hidden_states,
              (True, True): _run_mlp_layer_inplace_with_hidden_states}

    def __init__(self, layer_number: int, UP: torch.Tensor, DOWN: torch.Tensor,
                 num_splits: int = 2, inplace: bool = False,
                 preallocate_shared_hidden_state: bool = False, compression_factor: int = 8,
                 ext=None):
        if _validate_compression_factor(compression_factor) != 8:
            raise ValueError("Only compression_factor=8 is currently supported for TwELLMLP")
        super().__init__(layer_number, inplace=inplace,
                         preallocate_shared_hidden_state=preallocate_shared_hidden_state,
                         compression_factor=compression_factor, ext=ext)
        self.register_buffer("UP", UP.contiguous())
        self.register_buffer("DOWN", DOWN.contiguous())
        self.num_splits = int(num_splits)

    def _call_args(self):
        return (self.DOWN,), {"num_splits": self.num_splits}


class TwELLGatedMLP(_BaseTwELLMLP):
    """Fused gated TwELL MLP wrapper."""

    _first = "GATE"
    _entry = {(False, False): run_gated_mlp_layer, (False, True): run_gated_mlp_layer_inplace,
              (True, False): _run_gated_mlp_layer_with_hidden_states,
              (True, True): _run_gated_mlp_layer_inplace_with_hidden_states}

    def __init__(self, layer_number: int, GATE: torch.Tensor, UP: torch.Tensor,
                 DOWN: torch.Tensor, inplace: bool = False,
                 preallocate_shared_hidden_state: bool = False, highest_precision: bool = False,
                 compression_factor: int = 8, flex_kernels: bool = False, ext=None):
        if _validate_compression_factor(compression_factor) != 8 and not flex_kernels:
            raise ValueError("compression_factor != 8 requires flex_kernels=True")
        super().__init__(layer_number, inplace=inplace,
                         preallocate_shared_hidden_state=preallocate_shared_hidden_state,
                         compression_factor=compression_factor, ext=ext)
        self.highest_precision = bool(highest_precision)
        self.flex_kernels = bool(flex_kernels)
        self.register_buffer("GATE", GATE.contiguous())
        self.register_buffer("UP", UP.contiguous())
        self.register_buffer("DOWN", DOWN.contiguous())
        self._dense_route: dict | None = None
        self._down_t: torch.Tensor | None = None

    def _call_args(self):
        return (self.UP, self.DOWN), {"highest_precision": self.highest_precision,
                                      "compression_factor": self.compression_factor,
                                      "flex_kernels": self.flex_kernels}

    def enable_dense_route(self, dense_cap: int | None = None, nnz_threshold: int | None = None,
                           min_tokens: int = 256, dense_all_tokens: int | None = None) -> None:
        """Extension (off by default = reference behaviour): for calls with at least
        ``min_tokens`` rows, compute dense-enough or overflowed token rows as tensor-core GEMMs
        instead of per-entry gathers (see :func:`set_d2t_layer_dense_route`).  Keeps a
        ``[D, H]`` copy of the down projection."""
        self._dense_route = {"dense_cap": dense_cap, "nnz_threshold": nnz_threshold,
                             "min_tokens": min_tokens, "dense_all_tokens": dense_all_tokens}
        if self.layer is not None:
            self._apply_dense_route()

    def disable_dense_route(self) -> None:
        self._dense_route = None
        self._down_t = None
        if self.layer is not None:
            set_d2t_layer_dense_route(self.layer_number, None)

    def dense_route_counters(self) -> dict | None:
        return d2t_layer_dense_route_counters(self.layer_number) if self.layer is not None else None

    def _apply_dense_route(self) -> None:
        if self._dense_route is None:
            return
        if self._down_t is None or self._down_t.device != self.DOWN.device:
            self._down_t = self.DOWN.t().contiguous()
        set_d2t_layer_dense_route(self.layer_number, self._down_t, **self._dense_route)
