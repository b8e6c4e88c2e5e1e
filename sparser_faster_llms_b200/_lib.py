"""ctypes binding of ``libb200_sparse_ffn.so`` (declared in include/b200_sparse_ffn.h).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  Tensors are passed as raw device pointers, the stream is torch's
current CUDA stream.
"""
from __future__ import annotations

import ctypes
import warnings
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_uint32, c_void_p
from pathlib import Path

import torch

_PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = _PKG_DIR / "libb200_sparse_ffn.so"

OK = 0
FLAG_HIGH_PRECISION = 1

_ERRORS = {
    -1: "invalid argument",
    -2: "null pointer",
    -3: "misaligned pointer",
    -4: "unsupported shape",
    -5: "CUDA error",
    -6: "workspace too small",
}

# name -> (restype, argtypes); mirrors include/b200_sparse_ffn.h
_PROTOTYPES = {
    "b200_version": (c_int, []),
    "b200_built_for_sm": (c_int, []),
    "b200_last_error": (c_char_p, []),
    "b200_workspace_bytes": (c_size_t, []),
    "b200_twell_pack": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                c_int64, c_int, c_void_p]),
    "b200_twell_pack_select": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                       c_int64, c_int, c_int, c_void_p]),
    "b200_twell_pack_tc_status": (c_int, []),
    "b200_twell_gated_t2d": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                     c_int64, c_int64, c_int, c_uint32, c_void_p, c_size_t,
                                     c_void_p]),
    "b200_twell_t2d": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                               c_int, c_void_p, c_size_t, c_void_p]),
    "b200_hybrid_sddmm_fwd": (c_int, [c_void_p] * 8 + [c_int64, c_int64, c_int64, c_int, c_void_p]),
    "b200_hybrid_sddmm_bwd": (c_int, [c_void_p] * 7 + [c_int64, c_int64, c_int64, c_int,
                                                       c_void_p]),
    "b200_hybrid_spmm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                 c_void_p, c_size_t, c_void_p]),
    "b200_hybrid_csc_build": (c_int, [c_void_p] * 6 + [c_int64, c_void_p, c_int64, c_int64, c_int,
                                                       c_void_p]),
    "b200_hybrid_spmm_t": (c_int, [c_void_p] * 5 + [c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                                    c_int64, c_void_p]),
    "b200_hybrid_wgrad_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "b200_hybrid_wgrad_dense": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                        c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "b200_hybrid_ell_spmm_raw": (c_int, [c_void_p] * 5 + [c_int64] * 5 + [c_void_p]),
    # p_slab, vals_slab, M, H, cf, microbatch_tokens, active_rows, last_activated, stream
    "b200_hybrid_neuron_activity": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64,
                                            c_void_p, c_void_p, c_void_p]),
    "b200_twell_hybrid_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64]),
    # x, packed, gate, gate_bias, up, down, down_t, out, M, D, H, cf, flags, nnz_threshold,
    # dense_cap, hybrid_ws, hybrid_ws_bytes, workspace, workspace_bytes, stream
    "b200_twell_gated_t2d_hybrid": (c_int, [c_void_p] * 8 + [c_int64, c_int64, c_int64, c_int,
                                            c_uint32, c_int64, c_int64, c_void_p, c_size_t,
                                            c_void_p, c_size_t, c_void_p]),
    # x, gate, gate_bias, up, down, down_t, packed, out, then as above
    "b200_twell_gated_mlp_hybrid": (c_int, [c_void_p] * 8 + [c_int64, c_int64, c_int64, c_int,
                                            c_uint32, c_int64, c_int64, c_void_p, c_size_t,
                                            c_void_p, c_size_t, c_void_p]),
    "b200_dense_gated_mlp": (c_int, [c_void_p] * 7 + [c_int64, c_int64, c_int64, c_void_p]),
    "b200_twell_hybrid_counters": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64,
                                           ctypes.POINTER(c_int)]),
    "b200_twell_hybrid_status": (c_int, []),
    "b200_fused_allreduce_block_bytes": (c_size_t, [c_int64, c_int64]),
    # x, packed, up, down, out, M, D, H, cf, flags, ws, ws_bytes, peer_blocks, rank, world,
    # block_bytes, stream
    "b200_twell_gated_t2d_allreduce": (c_int, [c_void_p] * 5 + [c_int64, c_int64, c_int64, c_int,
                                               c_uint32, c_void_p, c_size_t, c_void_p, c_int,
                                               c_int, c_int64, c_void_p]),
    # x, gate, gate_bias, up, down, packed, out, then as above
    "b200_twell_gated_mlp_allreduce": (c_int, [c_void_p] * 7 + [c_int64, c_int64, c_int64, c_int,
                                               c_uint32, c_void_p, c_size_t, c_void_p, c_int,
                                               c_int, c_int64, c_void_p]),
    "b200_fused_allreduce_status": (c_int, [c_void_p]),
    "b200_peer_allreduce_block_bytes": (c_size_t, [c_int64]),
    "b200_peer_allreduce_bf16": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int,
                                         c_int64, c_void_p]),
    "b200_peer_allreduce_status": (c_int, [c_void_p]),
    "b200_twell_gated_t2d_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_int64, c_int64, c_int64, c_int, c_uint32,
                                             c_void_p]),
    "b200_twell_gated_mlp": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_int64, c_int64, c_int64, c_int, c_uint32,
                                     c_void_p, c_size_t, c_void_p]),
    "b200_twell_decode_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    # x, gate, gate_bias, up, down, packed, out, M, D, H, cf, flags, ws, ws_bytes, prefetch,
    # prefetch_bytes, stream
    "b200_twell_gated_mlp_decode": (c_int, [c_void_p] * 7 + [c_int64, c_int64, c_int64, c_int,
                                            c_uint32, c_void_p, c_size_t, c_void_p, c_int64,
                                            c_void_p]),
    "b200_twell_decode_status": (c_int, []),
    "b200_l2_prefetch": (c_int, [c_void_p, c_int64, c_void_p]),
    # x, delta, weight, eps, x_out, h_out, M, D, stream
    "b200_residual_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                      c_int64, c_int64, c_void_p]),
    "b200_twell_mlp": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                               c_int64, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p]),
}

_LIB = None


class B200Error(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, fn: str, code: int, text: str):
        self.fn, self.code, self.text = fn, code, text
        kind = _ERRORS.get(code, f"error {code}")
        super().__init__(f"{fn} failed ({kind}): {text}")


def load_library(path: str | Path | None = None) -> ctypes.CDLL:
    """Load the shared library (once) and attach prototypes.  Raises if absent."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    lib_path = Path(path) if path is not None else LIB_PATH
    if not lib_path.exists():
        raise RuntimeError(
            f"{lib_path} is missing: the sm_100a CUDA library has not been built. "
            "Run `python -m sparser_faster_llms_b200.build` (needs nvcc). "
            "There is no CPU or PyTorch fallback for these operators.")
    lib = ctypes.CDLL(str(lib_path))
    for name, (restype, argtypes) in _PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    if path is None:
        _LIB = lib
    return lib


def exported_names() -> list[str]:
    return sorted(_PROTOTYPES)


def last_error() -> str:
    return load_library().b200_last_error().decode("utf-8", "replace")


def check(fn_name: str, status: int) -> None:
    if status != OK:
        code = int(status)
        if code in (-1, -2, -3, -4):
            raise ValueError(str(B200Error(fn_name, code, last_error())))
        raise B200Error(fn_name, code, last_error())


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def current_stream_handle(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}
_WARNED_CAPTURE = False


def workspace(device: torch.device) -> tuple[int | None, int]:
    """(pointer, bytes) of the zero-initialised contraction workspace of ``device``'s current
    stream, created on first use.  During CUDA-graph capture no new workspace is created:
    ``(None, 0)`` is returned and the kernels use their workspace-free shape."""
    stream = torch.cuda.current_stream(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           stream.cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            global _WARNED_CAPTURE
            if not _WARNED_CAPTURE:
                _WARNED_CAPTURE = True
                warnings.warn(
                    "sparser_faster_llms_b200: a contraction is being captured on a stream that "
                    "has no workspace yet, so it runs without the few-token multi-cluster shape. "
                    "Run the step once on the capture stream before capturing "
                    "(torch.cuda.graph(g, stream=s) with the warm-up on s).", stacklevel=3)
            return None, 0
        nbytes = int(load_library().b200_workspace_bytes())
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws.data_ptr(), ws.numel()


def call(fn_name: str, device: torch.device, *args) -> None:
    """Invoke ``fn_name(*args, stream)`` on ``device``'s current stream and raise on error."""
    lib = load_library()
    fn = getattr(lib, fn_name)
    with torch.cuda.device(device):
        status = fn(*args, current_stream_handle(device))
    check(fn_name, status)
