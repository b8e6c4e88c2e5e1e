"""Hybrid sparse training operator: ``torch.ops.sparse_ops.ff_forward_gated`` and friends.

Python/torch host side of the reference's ``custom_models/hybrid_modules/custom_op.cpp``.
The math is

    P = relu(X G^T)           (pattern + values, TwELL slabs from the pack kernel)
    R = (X K^T) on P's pattern,   T = R * P
    out = T V,   l0 = mean_rows nnz(P),   l1 = mean_rows sum |T|

and its backward (custom_op.cpp:139-282).  Every sparse operand is a slab-shaped
``uint32`` tensor aligned with P (see ``csrc/hybrid_ops.cu``); the reference's
row-ELL + dense-tail container ``hybrid_sp_t`` and its conversion / transpose
kernels have no equivalent here because nothing is converted.

Registered operators (same names and argument order as custom_op.cpp:308-342, :424-427):

    sparse_ops::ff_forward_gated(X, G, K, V) -> (out, l0, l1, P, R, T)
    sparse_ops::ff_backward_gated(X, G, K, V, P, R, T, gR, gl0, gl1) -> (dX, dG, dK, dV)
    sparse_ops::ell_spmm_raw(ell_vals, ell_cols, row_counts, B, M, K, N, ell_stride, thr)
    sparse_ops_config::set_ell_width_regular / set_ell_width_transpose /
        set_tail_rows_regular / set_tail_rows_transpose / set_discard_overflow /
        get_last_transpose_overflow_count
    sparse_ops_perf::print_report / reset_stats

P, R, T are returned as int32 tensors (a Python-registered operator cannot return a
TorchScript custom class); :class:`HybridSp` wraps one of them for callers that want
``overflow_count_tensor()``.  There is no CPU implementation.

Dense tail (custom_op.cpp:79-116, hybrid_sp.cu:516-576, :811-952, :1358-1383).  A token row
with more positives in some 256-neuron tile than a slab holds cannot be represented by the
slabs alone.  With ``discard_overflow == 0`` (the default, as in the reference) up to
``tail_rows_regular`` such rows are taken out of the sparse kernels - the sign bit of their
count words is set, which every kernel reads as "no entries" while the true counts stay in
the low bits - and computed exactly as dense bf16 GEMMs over the gathered rows, forward and
backward, the way the reference multiplies its ``tail_dense`` rows with ``torch::matmul``.
The row list is rebuilt from the flags in backward, so nothing but P carries it; no host
synchronisation is involved (the reference waits on an event per backward).  Rows beyond the
capacity keep the slab prefix and are counted in ``dropped``.  ``discard_overflow == 1`` keeps
every row on the slabs: entries past a tile's capacity are dropped and counted.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass

import torch

from . import _lib

TILE = 256

# ----------------------------------------------------------------------------
# knobs (reference: hybrid_sp.cu:634-646, KNOBS.md)
# ----------------------------------------------------------------------------
_CONFIG = {
    # entries kept per 256-column tile of a row: 31 / 63 / 127 (slab width 32 / 64 / 128 words).
    # The reference's "ELL width" (entries per row, default 128) maps onto the slab width.
    "ell_width_regular": 128,
    "ell_width_transpose": 256,
    "tail_rows_regular": 2048,
    "tail_rows_transpose": 2048,
    "discard_overflow": 0,
    # average stored entries per row the column lists are sized for
    "csc_entries_per_row": 512,
    # weight gradients dK / dG / dV: "sparse" = column lists + transposed SpMM, "dense" =
    # scatter to a K-major matrix + tcgen05 GEMM, "auto" = dense from 2048 tokens on
    "weight_gradient_mode": "auto",
    # size the tail from the overflow count observed on earlier calls instead of always
    # computing tail_rows_regular rows (see set_tail_rows_adaptive)
    "tail_rows_adaptive": 0,
}
_LAST_TRANSPOSE_OVERFLOW: torch.Tensor | None = None
_PERF: dict[str, list[float]] = {}
_PERF_ENABLED = os.environ.get("SPARSE_ENABLE_PERF_PROFILING", "0") not in ("0", "", "false", "False")


def set_weight_gradient_mode(mode: str) -> None:
    """``"sparse"``, ``"dense"`` or ``"auto"`` (default: dense from 2048 tokens on).  The three
    weight gradients reduce over all tokens and are dense ``[H, D]`` matrices, so they can run
    as tensor-core GEMMs over a scattered K-major copy of the slab instead of gathers along
    column lists.  Measured on B200 (16384 tokens, D = 1024, H = 4096, 41 positives per token)
    the two forms take the same time (0.79 ms for the three products against 0.78 ms including
    the lists: the GEMM has only 128 tiles and is bound by the operand stream into each SM);
    the dense form is deterministic, whereas the order inside a column list follows atomic
    arrival.  No reference counterpart: the reference always transposes the hybrid container
    and runs its SpMM (custom_op.cpp:247-269)."""
    if mode not in ("sparse", "dense", "auto"):
        raise ValueError("mode must be 'sparse', 'dense' or 'auto'")
    _CONFIG["weight_gradient_mode"] = mode


def _dense_weight_gradients(m: int) -> bool:
    mode = _CONFIG["weight_gradient_mode"]
    return mode == "dense" or (mode == "auto" and m >= 2048)


_WGRAD_WS: dict[int, torch.Tensor] = {}


def _wgrad_workspace(dev: torch.device, m: int, d: int, h: int) -> torch.Tensor:
    need = int(_lib.load_library().b200_hybrid_wgrad_workspace_bytes(m, d, h))
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    buf = _WGRAD_WS.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.empty(need, dtype=torch.uint8, device=dev)
        _WGRAD_WS[key] = buf
    return buf


def set_tail_rows_adaptive(on: bool) -> None:
    """Size the dense tail from the overflow-row count seen on earlier calls with the same
    gate matrix (read back asynchronously, never waited for): twice the last count rounded up
    to 128 rows, at most ``tail_rows_regular`` - and no tail at all while the last count is
    zero (the call then only counts its overflow rows, so that the next one has a tail).  Off
    (the default) the tail always spans ``min(tail_rows_regular, tokens)`` rows, which is what
    the reference's forward computes (custom_op.cpp:125-127 sets the active rows to the
    capacity).  The price of the adaptive form: the first call in which overflow rows appear,
    or more than doubles, leaves the excess rows on their slab prefix for that one call
    (counted in ``dropped``).  No reference counterpart."""
    _CONFIG["tail_rows_adaptive"] = 1 if on else 0


_INT_MIN = -(2 ** 31)
_TAIL_SEEN: dict[tuple, dict] = {}


def _tail_state(key: tuple) -> dict:
    st = _TAIL_SEEN.get(key)
    if st is None:
        if len(_TAIL_SEEN) > 512:
            _TAIL_SEEN.clear()
        st = {"host": torch.zeros((), dtype=torch.int64).pin_memory(),
              "event": None, "last": None, "cap_fwd": None}
        _TAIL_SEEN[key] = st
    return st


def _tail_capacity(key: tuple, m: int) -> int:
    """Rows the forward's dense tail spans for this call (0 = no tail)."""
    cap = min(int(_CONFIG["tail_rows_regular"]), m)
    if cap <= 0 or _CONFIG["discard_overflow"]:
        return 0
    if not _CONFIG["tail_rows_adaptive"]:
        return cap
    st = _tail_state(key)
    if st["event"] is not None and st["event"].query():
        st["last"] = int(st["host"].item())
    if st["last"] is not None:
        cap = 0 if st["last"] == 0 else min(cap, (2 * st["last"] + 127) // 128 * 128)
    # the backward must span at least the rows of every forward since the last backward
    st["cap_fwd"] = cap if st["cap_fwd"] is None else max(st["cap_fwd"], cap)
    return cap


def _tail_observe(key: tuple, n_over: torch.Tensor) -> None:
    """Start an asynchronous read-back of this call's overflow-row count (never waited for)."""
    st = _tail_state(key)
    if st["event"] is not None and not st["event"].query():
        return  # the previous read-back is still in flight: keep it
    st["host"].copy_(n_over, non_blocking=True)
    st["event"] = torch.cuda.Event()
    st["event"].record()


def _count_view(P: torch.Tensor, m: int, h: int, cf: int) -> torch.Tensor:
    """Strided int32 view ``[m, tiles]`` of the count words of a slab array."""
    return P.view(m, h // TILE, TILE // cf)[:, :, 0]


def _tail_index(in_tail: torch.Tensor, cap: int, m: int):
    """(idx [cap] clamped to valid rows, valid [cap] bool, scatter index with m = padding)."""
    raw = torch.nonzero_static(in_tail, size=cap, fill_value=m).reshape(cap)
    valid = raw < m
    return raw.clamp(max=max(m - 1, 0)), valid, raw


def compression_factor() -> int:
    """Slab compression factor implied by ``ell_width_regular``: the per-tile capacity is
    the smallest of 31 / 63 / 127 that is >= ell_width / 4 (a row of 4096 neurons has 16
    tiles, so the default 128 entries per row never overflows a 63-entry tile on average)."""
    per_tile = max(1, _CONFIG["ell_width_regular"] // 4)
    if per_tile <= 31:
        return 8
    if per_tile <= 63:
        return 4
    return 2


@dataclass
class HybridSp:
    """Slab-shaped sparse operand (pattern P, or values aligned with P)."""
    slab: torch.Tensor          # int32 [M, tiles * W]
    m: int
    n: int
    cf: int
    dropped: torch.Tensor | None = None  # int32 scalar: entries lost to slab overflow

    def overflow_count_tensor(self) -> torch.Tensor:
        if self.dropped is None:
            return torch.zeros((), dtype=torch.int32, device=self.slab.device)
        return self.dropped


class _Timer:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _PERF_ENABLED:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e1 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if _PERF_ENABLED:
            self.e1.record()
            self.e1.synchronize()
            _PERF.setdefault(self.name, []).append(self.e0.elapsed_time(self.e1))
        return False


def _check_inputs(X, G, K, V):
    for name, t in (("X", X), ("G", G), ("K", K), ("V", V)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor: sparse_ops has no CPU implementation")
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name}: Expected a bfloat16 tensor but got {t.dtype}")
    if X.dim() != 3:
        raise ValueError(f"X must be [B, S, D], got {tuple(X.shape)}")
    h, d = K.shape
    if G.shape != (h, d) or V.shape != (h, d) or X.shape[-1] != d:
        raise ValueError(
            f"G, K, V must all be [H, D] with D = X.shape[-1]; got {tuple(G.shape)}, "
            f"{tuple(K.shape)}, {tuple(V.shape)}, X {tuple(X.shape)}")
    return h, d


def _slab_shape(m: int, h: int, cf: int) -> tuple[int, int]:
    if h % TILE:
        raise ValueError(f"H must be a multiple of {TILE}")
    return m, (h // TILE) * (TILE // cf)


def _spmm(vals: torch.Tensor, B: torch.Tensor, m: int, d: int, h: int, cf: int,
          pad_rows: int = 0) -> torch.Tensor:
    """Row product ``out[r,:] = sum value * B[col,:]`` (fp32 fma, bf16 store).  ``pad_rows``
    extra rows are allocated behind the result (scatter target of the tail's padding index)."""
    out = torch.empty((m + pad_rows, d), dtype=torch.bfloat16, device=vals.device)
    _lib.call("b200_hybrid_spmm", vals.device, vals.data_ptr(), B.data_ptr(), out.data_ptr(),
              m, d, h, cf, *_lib.workspace(vals.device))
    return out


def ff_forward_impl(X: torch.Tensor, G: torch.Tensor, K: torch.Tensor, V: torch.Tensor):
    """Forward of the hybrid operator (custom_op.cpp:40-137).  Returns
    ``(out [B,S,D] bf16, l0 [], l1 [], P, R, T, dropped)`` with P/R/T int32 slab tensors."""
    h, d = _check_inputs(X, G, K, V)
    m = X.shape[0] * X.shape[1]
    cf = compression_factor()
    dev = X.device
    Xf = X.reshape(m, d).contiguous()
    G, K, V = G.contiguous(), K.contiguous(), V.contiguous()
    shape = _slab_shape(m, h, cf)
    tail_key = (dev.index, G.data_ptr(), m, h)
    cap = _tail_capacity(tail_key, m) if m > 0 else 0
    with _Timer("ff_forward_gated_total"):
        P = torch.empty(shape, dtype=torch.int32, device=dev)
        with _Timer("gate_gemm_pack"):
            _lib.call("b200_twell_pack", dev, Xf.data_ptr(), G.data_ptr(), None, P.data_ptr(),
                      m, d, h, cf)
        inv_m = 1.0 / max(m, 1)
        tail = None
        adaptive = bool(_CONFIG["tail_rows_adaptive"]) and m > 0 and \
            not _CONFIG["discard_overflow"] and _CONFIG["tail_rows_regular"] > 0
        if cap > 0 or adaptive:
            cnt = _count_view(P, m, h, cf)
            over = (cnt > TILE // cf - 1).any(dim=1)
            if adaptive:
                _tail_observe(tail_key, over.sum())
        if cap > 0:
            # rows with an overflowed tile leave the slabs: flag their count words
            in_tail = over & (over.cumsum(0) <= cap) if cap < m else over
            l0 = cnt.sum(dtype=torch.float32) * inv_m
            cnt.bitwise_or_(in_tail.to(torch.int32).mul_(_INT_MIN).unsqueeze(1))
            tail = _tail_index(in_tail, cap, m)
        R = torch.empty_like(P)
        T = torch.empty_like(P)
        row_l1 = torch.empty(m, dtype=torch.float32, device=dev)
        row_nnz = torch.empty(m, dtype=torch.int32, device=dev)
        row_drop = torch.empty(m, dtype=torch.int32, device=dev)
        with _Timer("sddmm_R_T"):
            _lib.call("b200_hybrid_sddmm_fwd", dev, Xf.data_ptr(), K.data_ptr(), P.data_ptr(),
                      R.data_ptr(), T.data_ptr(), row_l1.data_ptr(), row_nnz.data_ptr(),
                      row_drop.data_ptr(), m, d, h, cf)
        with _Timer("spmm_out"):
            out = _spmm(T, V, m, d, h, cf, pad_rows=1 if tail is not None else 0)
        l1 = row_l1.sum()
        if tail is None:
            l0 = row_nnz.sum(dtype=torch.float32) * inv_m
        else:
            with _Timer("dense_tail_forward"):
                idx, valid, scatter = tail
                Xt = Xf[idx] * valid.unsqueeze(1)
                Pt = torch.relu(Xt @ G.t())
                Tt = (Xt @ K.t()) * Pt
                out.index_copy_(0, scatter, Tt @ V)
                l1 = l1 + Tt.abs().sum(dtype=torch.float32)
            out = out[:m]
        l1 = l1 * inv_m
        dropped = row_drop.sum(dtype=torch.int32)
    return out.reshape(X.shape), l0, l1, P, R, T, dropped


_CSC_SCRATCH: dict[tuple, dict[str, torch.Tensor]] = {}


def _csc_scratch(dev: torch.device, m: int, h: int) -> dict[str, torch.Tensor]:
    cap = int(min(m * _CONFIG["csc_entries_per_row"], 2**31 - 1))
    key = (dev.index, m, h, cap)
    buf = _CSC_SCRATCH.get(key)
    if buf is None:
        _CSC_SCRATCH.clear()  # one shape at a time: the lists are rebuilt by every backward
        i32 = dict(dtype=torch.int32, device=dev)
        buf = {"count": torch.empty(h, **i32), "start": torch.empty(h + 1, **i32),
               "cursor": torch.empty(h, **i32), "row": torch.empty(max(cap, 1), **i32),
               "pos": torch.empty(max(cap, 1), **i32), "cap": cap}
        _CSC_SCRATCH[key] = buf
    return buf


def ff_backward_impl(X, G, K, V, P, R, T, gR, gl0, gl1):
    """Backward of the hybrid operator (custom_op.cpp:139-282).  ``gl0`` is ignored, as in
    the reference.  Returns ``(dX [B,S,D], dG, dK, dV [H,D])`` in bf16."""
    global _LAST_TRANSPOSE_OVERFLOW
    h, d = _check_inputs(X, G, K, V)
    m = X.shape[0] * X.shape[1]
    cf = compression_factor()
    dev = X.device
    if tuple(P.shape) != _slab_shape(m, h, cf):
        raise ValueError("P does not match the current slab width: the ELL-width knob changed "
                         "between forward and backward")
    if gR.dtype != torch.bfloat16:
        raise RuntimeError(f"gR: Expected a bfloat16 tensor but got {gR.dtype}")
    Xf = X.reshape(m, d).contiguous()
    gRf = gR.reshape(m, d).contiguous()
    G, K, V = G.contiguous(), K.contiguous(), V.contiguous()
    gl1_dev = None
    if gl1 is not None:
        gl1_dev = gl1.detach().to(device=dev, dtype=torch.float32).reshape(1).contiguous()
    # tail rows: flagged count words (sign bit) in P, set by the forward
    tail = None
    if m > 0 and not _CONFIG["discard_overflow"] and _CONFIG["tail_rows_regular"] > 0:
        cap = min(int(_CONFIG["tail_rows_regular"]), m)
        if _CONFIG["tail_rows_adaptive"]:
            st = _TAIL_SEEN.get((dev.index, G.data_ptr(), m, h))
            if st is not None and st["cap_fwd"] is not None:
                cap = min(cap, st["cap_fwd"])  # what the forward(s) since the last backward used
                st["cap_fwd"] = None
        if cap > 0:
            flagged = (_count_view(P, m, h, cf) < 0).any(dim=1)
            tail = _tail_index(flagged, cap, m)
    pad = 1 if tail is not None else 0
    with _Timer("ff_backward_gated_total"):
        dR = torch.empty_like(P)
        dU = torch.empty_like(P)
        with _Timer("sddmm_dT_dR_dU"):
            _lib.call("b200_hybrid_sddmm_bwd", dev, gRf.data_ptr(), V.data_ptr(), P.data_ptr(),
                      R.data_ptr(), dR.data_ptr(), dU.data_ptr(), _lib.ptr(gl1_dev), m, d, h, cf)
        with _Timer("spmm_dX"):
            dX = _spmm(dR, K, m, d, h, cf, pad) + _spmm(dU, G, m, d, h, cf, pad)
        dK = torch.empty((h, d), dtype=torch.bfloat16, device=dev)
        dG = torch.empty_like(dK)
        dV = torch.empty_like(dK)
        if _dense_weight_gradients(m):
            ws = _wgrad_workspace(dev, m, d, h)
            with _Timer("wgrad_dense_dK_dG"):
                _lib.call("b200_hybrid_wgrad_dense", dev, dR.data_ptr(), Xf.data_ptr(),
                          dK.data_ptr(), m, d, h, cf, 0, ws.data_ptr(), ws.numel())
                _lib.call("b200_hybrid_wgrad_dense", dev, dU.data_ptr(), Xf.data_ptr(),
                          dG.data_ptr(), m, d, h, cf, 1, ws.data_ptr(), ws.numel())
            with _Timer("wgrad_dense_dV"):
                _lib.call("b200_hybrid_wgrad_dense", dev, T.data_ptr(), gRf.data_ptr(),
                          dV.data_ptr(), m, d, h, cf, 0, ws.data_ptr(), ws.numel())
            _LAST_TRANSPOSE_OVERFLOW = torch.zeros((), dtype=torch.int32, device=dev)
        else:
            sc = _csc_scratch(dev, m, h)
            overflow = torch.empty(1, dtype=torch.int32, device=dev)
            with _Timer("column_lists"):
                _lib.call("b200_hybrid_csc_build", dev, P.data_ptr(), sc["count"].data_ptr(),
                          sc["start"].data_ptr(), sc["cursor"].data_ptr(), sc["row"].data_ptr(),
                          sc["pos"].data_ptr(), sc["cap"], overflow.data_ptr(), m, h, cf)
            with _Timer("spmm_t_dK_dG"):
                _lib.call("b200_hybrid_spmm_t", dev, dR.data_ptr(), dU.data_ptr(),
                          sc["start"].data_ptr(), sc["row"].data_ptr(), sc["pos"].data_ptr(),
                          sc["cap"], Xf.data_ptr(), dK.data_ptr(), dG.data_ptr(), h, d)
            with _Timer("spmm_t_dV"):
                _lib.call("b200_hybrid_spmm_t", dev, T.data_ptr(), None, sc["start"].data_ptr(),
                          sc["row"].data_ptr(), sc["pos"].data_ptr(), sc["cap"], gRf.data_ptr(),
                          dV.data_ptr(), None, h, d)
            _LAST_TRANSPOSE_OVERFLOW = overflow.reshape(())
        if tail is not None:
            # the flagged rows, dense (gate, up and the pattern recomputed from X)
            with _Timer("dense_tail_backward"):
                idx, valid, scatter = tail
                keep = valid.unsqueeze(1)
                Xt = Xf[idx] * keep
                gRt = gRf[idx] * keep
                Pt = torch.relu(Xt @ G.t())
                Rt = Xt @ K.t()
                dTt = gRt @ V.t()
                if gl1_dev is not None:
                    dTt = dTt + (gl1_dev * (1.0 / m)).to(torch.bfloat16) * torch.sign(Rt)
                dTt = dTt * (Pt > 0)
                dRt = dTt * Pt
                dUt = dTt * Rt
                dX.index_copy_(0, scatter, dRt @ K + dUt @ G)
                dK = (dK.float() + (dRt.t() @ Xt).float()).to(torch.bfloat16)
                dG = (dG.float() + (dUt.t() @ Xt).float()).to(torch.bfloat16)
                dV = (dV.float() + ((Rt * Pt).t() @ gRt).float()).to(torch.bfloat16)
            dX = dX[:m]
    return dX.reshape(X.shape), dG, dK, dV


def ell_spmm_raw_impl(ell_vals, ell_cols, row_counts, B, M, K, N, ell_stride,
                      overflow_threshold):
    """Row-ELL x dense (custom_op.cpp:313): bf16 values, 16-bit columns, int32 counts."""
    if ell_vals.dtype != torch.bfloat16 or B.dtype != torch.bfloat16:
        raise RuntimeError("ell_spmm_raw: ell_vals and B must be bfloat16")
    if ell_cols.dtype not in (torch.int16, torch.uint16):
        raise RuntimeError("ell_spmm_raw: ell_cols must be a 16-bit integer tensor")
    if row_counts.dtype != torch.int32:
        raise RuntimeError("ell_spmm_raw: row_counts must be int32")
    dev = B.device
    C = torch.empty((int(M), int(N)), dtype=torch.bfloat16, device=dev)
    _lib.call("b200_hybrid_ell_spmm_raw", dev, ell_vals.contiguous().data_ptr(),
              ell_cols.contiguous().data_ptr(), row_counts.contiguous().data_ptr(),
              B.contiguous().data_ptr(), C.data_ptr(), int(M), int(K), int(N), int(ell_stride),
              int(overflow_threshold))
    return C


# ----------------------------------------------------------------------------
# operator registration
# ----------------------------------------------------------------------------
_REGISTERED = False
_LIBS: list = []  # keeps the torch.library.Library objects alive

_FWD = "sparse_ops::ff_forward_gated"
_BWD = "sparse_ops::ff_backward_gated"


def _fake_forward(X, G, K, V):
    m = X.shape[0] * X.shape[1]
    shape = _slab_shape(m, K.shape[0], compression_factor())
    slab = lambda: torch.empty(shape, dtype=torch.int32, device=X.device)  # noqa: E731
    scalar = lambda: torch.empty((), dtype=torch.float32, device=X.device)  # noqa: E731
    return (torch.empty(X.shape, dtype=torch.bfloat16, device=X.device), scalar(), scalar(),
            slab(), slab(), slab())


def _fake_backward(X, G, K, V, P, R, T, gR, gl0, gl1):
    e = lambda t: torch.empty(t.shape, dtype=torch.bfloat16, device=t.device)  # noqa: E731
    return e(X), e(G), e(K), e(V)


def _setup_context(ctx, inputs, output):
    X, G, K, V = inputs
    _, _, _, P, R, T = output
    ctx.save_for_backward(X, G, K, V, P, R, T)
    ctx.set_materialize_grads(False)


def _autograd_backward(ctx, g_out, g_l0, g_l1, g_p, g_r, g_t):
    X, G, K, V, P, R, T = ctx.saved_tensors
    if g_out is None:
        g_out = torch.zeros_like(X)
    zero = torch.zeros((), dtype=torch.float32, device=X.device)
    dX, dG, dK, dV = torch.ops.sparse_ops.ff_backward_gated(
        X, G, K, V, P, R, T, g_out.to(torch.bfloat16), zero if g_l0 is None else g_l0,
        zero if g_l1 is None else g_l1)
    return dX, dG, dK, dV


def register_ops() -> None:
    """Define and implement the operators (idempotent)."""
    global _REGISTERED
    if _REGISTERED:
        return
    lib = torch.library.Library("sparse_ops", "DEF")
    lib.define("ff_forward_gated(Tensor X, Tensor G, Tensor K, Tensor V) -> "
               "(Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")
    lib.define("ff_backward_gated(Tensor X, Tensor G, Tensor K, Tensor V, Tensor P, Tensor R, "
               "Tensor T, Tensor gR, Tensor gl0, Tensor gl1) -> (Tensor, Tensor, Tensor, Tensor)")
    lib.define("ell_spmm_raw(Tensor ell_vals, Tensor ell_cols, Tensor row_counts, Tensor B, int M, "
               "int K, int N, int ell_stride, int overflow_threshold) -> Tensor")
    lib.impl("ff_forward_gated", lambda X, G, K, V: ff_forward_impl(X, G, K, V)[:6], "CUDA")
    lib.impl("ff_backward_gated", ff_backward_impl, "CUDA")
    lib.impl("ell_spmm_raw", ell_spmm_raw_impl, "CUDA")
    torch.library.register_fake(_FWD, _fake_forward, lib=lib)
    torch.library.register_fake(_BWD, _fake_backward, lib=lib)
    torch.library.register_autograd(_FWD, _autograd_backward, setup_context=_setup_context,
                                    lib=lib)
    torch.library.register_autocast(_FWD, "cuda", torch.bfloat16, lib=lib)
    _LIBS.append(lib)

    cfg = torch.library.Library("sparse_ops_config", "DEF")
    for name in ("set_ell_width_regular", "set_ell_width_transpose", "set_tail_rows_regular",
                 "set_tail_rows_transpose", "set_discard_overflow"):
        cfg.define(f"{name}(int v) -> ()")
        cfg.impl(name, (lambda key: lambda v: _set_knob(key, v))(name[4:]),
                 "CompositeExplicitAutograd")
    cfg.define("get_last_transpose_overflow_count() -> Tensor")
    cfg.impl("get_last_transpose_overflow_count", _get_last_transpose_overflow,
             "CompositeExplicitAutograd")
    _LIBS.append(cfg)

    perf = torch.library.Library("sparse_ops_perf", "DEF")
    perf.define("print_report() -> ()")
    perf.define("reset_stats() -> ()")
    perf.impl("print_report", print_report, "CompositeExplicitAutograd")
    perf.impl("reset_stats", reset_stats, "CompositeExplicitAutograd")
    _LIBS.append(perf)
    _REGISTERED = True


def _set_knob(key: str, v: int) -> None:
    v = int(v)
    if v < 0:
        raise ValueError(f"{key} must be >= 0")
    _CONFIG[key] = v


def _get_last_transpose_overflow() -> torch.Tensor:
    if _LAST_TRANSPOSE_OVERFLOW is None:
        raise RuntimeError("No backward pass has been run yet")
    return _LAST_TRANSPOSE_OVERFLOW


def print_report() -> None:
    """Per-section CUDA-event timings (enabled by SPARSE_ENABLE_PERF_PROFILING=1);
    reference: perf_instrumentation.h:86-216."""
    if not _PERF:
        print("[sparse_ops_perf] no samples (set SPARSE_ENABLE_PERF_PROFILING=1)")
        return
    print(f"[sparse_ops_perf] {time.strftime('%H:%M:%S')}")
    for name, xs in sorted(_PERF.items()):
        s = sorted(xs)
        mean = sum(xs) / len(xs)
        print(f"  {name:28s} n={len(xs):5d} mean={mean:8.3f} ms min={s[0]:8.3f} "
              f"p50={s[len(s) // 2]:8.3f} max={s[-1]:8.3f}")


def reset_stats() -> None:
    _PERF.clear()


def neuron_activity(P, T=None, last_activated: torch.Tensor | None = None,
                    microbatch_tokens: int = 0, width: int | None = None) -> torch.Tensor:
    """Per-neuron activity of one forward: ``active_rows`` int32 ``[H]`` = number of tokens
    with a non-zero stored value for the neuron (values from ``T``, the forward's
    ``relu(gate)*up`` slab, else from the pattern ``P``).  With ``last_activated`` (int64
    ``[H]``, updated in place) active neurons restart at 0 and the others age by
    ``microbatch_tokens``: the update SparsityTracker.record_activations applies from the
    dense activation (custom_models/sparse_models.py:170-181), which the reference's fused
    path leaves stale (:183-208).  ``P`` / ``T`` are the int32 slab tensors the forward
    returns, or :class:`HybridSp` wrappers."""
    if isinstance(P, HybridSp):
        width = P.n if width is None else width
        cf, P = P.cf, P.slab
    else:
        cf = compression_factor()
    if isinstance(T, HybridSp):
        T = T.slab
    if width is None:
        width = P.shape[1] // (TILE // cf) * TILE
    if not P.is_cuda:
        raise RuntimeError("P must be a CUDA tensor: sparse_ops has no CPU implementation")
    m = P.shape[0]
    if tuple(P.shape) != _slab_shape(m, width, cf):
        raise ValueError(f"P {tuple(P.shape)} is not a slab array of width {width} at cf {cf}")
    if T is not None and (T.shape != P.shape or T.device != P.device):
        raise ValueError("T must have P's shape and device")
    dev = P.device
    if last_activated is not None:
        if (last_activated.dtype != torch.int64 or last_activated.shape != (width,)
                or last_activated.device != dev or not last_activated.is_contiguous()):
            raise ValueError(f"last_activated must be a contiguous int64 [{width}] tensor on {dev}")
    active_rows = torch.empty(width, dtype=torch.int32, device=dev)
    P = P.contiguous()
    T = None if T is None else T.contiguous()
    _lib.call("b200_hybrid_neuron_activity", dev, P.data_ptr(), _lib.ptr(T), m, width, cf,
              int(microbatch_tokens), active_rows.data_ptr(), _lib.ptr(last_activated))
    return active_rows


def ff_forward_gated(X, G, K, V):
    """Direct (non-dispatcher) forward returning :class:`HybridSp` objects like the
    reference's CUDA implementation (custom_op.cpp:40-137)."""
    out, l0, l1, P, R, T, dropped = ff_forward_impl(X, G, K, V)
    m, h, cf = X.shape[0] * X.shape[1], K.shape[0], compression_factor()
    wrap = lambda t: HybridSp(t, m, h, cf, dropped)  # noqa: E731
    return out, l0, l1, wrap(P), wrap(R), wrap(T)
