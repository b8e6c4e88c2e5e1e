/*
 * b200_sparse_ffn.h - C ABI of the B200 (sm_100a) activation-sparse gated-FFN kernels.
 *
 * Every entry point takes raw device pointers, 64-bit sizes and a CUDA stream
 * handle (a cudaStream_t passed as void*; NULL = the legacy default stream).
 * No entry point allocates device memory, synchronises the host with the
 * device, or keeps a pointer after it returns, unless its comment says so.
 * All return 0 on success or a negative B200_E* code; the text of the last
 * failure on the calling thread is available from b200_last_error().
 *
 * Layout conventions (TwELL layout of the reference, all row-major, bf16):
 *   x     [M, D]   activations
 *   gate, up, down [H, D]   (down = down_proj.weight transposed;
 *                            reference: custom_models/sparse_testing_utils.py:23-34)
 *   packed [M, (H/256) * (256/cf)] uint32 TwELL slabs
 *          (reference spec: custom_models/twell_modules/twell.py:152-264)
 * Constraints: D % 256 == 0, 256 <= D <= 8192; H % 256 == 0, H <= 65536;
 * cf in {2,4,8}; pointers 16-byte aligned.  M >= 0 is unrestricted.
 */
#ifndef B200_SPARSE_FFN_H_
#define B200_SPARSE_FFN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_EINVAL (-1)      /* bad size / flag / compression factor          */
#define B200_ENULL (-2)       /* a required pointer is NULL                    */
#define B200_EALIGN (-3)      /* a pointer is not 16-byte aligned              */
#define B200_EUNSUPPORTED (-4)/* shape outside the compiled range              */
#define B200_ECUDA (-5)       /* CUDA runtime reported an error at launch      */
#define B200_EWORKSPACE (-6)  /* caller-provided workspace is too small        */

/* flags for the contraction entry points */
#define B200_FLAG_HIGH_PRECISION 1u /* fp32 fma everywhere, h kept in fp32     */

/* Library version (major*10000 + minor*100 + patch) and the sm arch it was built for. */
int b200_version(void);
int b200_built_for_sm(void);
/* Text of the last error raised on the calling thread ("" if none). */
const char* b200_last_error(void);

/*
 * Optional workspace of the contraction entry points.  With few tokens (decode)
 * the contraction spreads one token over the whole GPU and combines partial
 * sums through global memory; that needs a caller-owned device buffer of at
 * least b200_workspace_bytes() bytes, 16-byte aligned, zero-filled ONCE before
 * its first use (the kernels leave it zeroed where it matters).  Calls that may
 * overlap on the GPU (different streams) need different workspaces.  Passing
 * NULL / 0 is always valid: one thread-block cluster per token is used instead.
 */
size_t b200_workspace_bytes(void);

/*
 * Gate projection + ReLU + TwELL pack:  packed = pack(relu(x @ w^T + bias)).
 * Replaces matmul_sparse_out / run_d2t_layer
 * (custom_models/twell_modules/twell.cpp:423-444, :583-601; kernel
 * custom_models/twell_modules/matmul_d2t.cu:287-709).  `bias` ([H] fp32) may be
 * NULL.  Each slab's word 0 receives the true count of positive
 * pre-activations; words 1..min(count, 256/cf-1) receive col | bf16(value)<<16
 * in ascending column order; the remaining words are left untouched.
 */
int b200_twell_pack(const void* x, const void* w, const float* bias, void* packed,
                    int64_t M, int64_t D, int64_t H, int cf, void* stream);

/*
 * Same as b200_twell_pack with the kernel family chosen by the caller:
 *   kernel 0 = automatic (M == 1: kernel 6 where it serves; M <= 16: split-k cluster kernel on mma.sync;
 *              33..256: kernel 8 / 9 while one wave; 17..32: tcgen05
 *              split-k cluster kernel; M > 32: tcgen05 / TMEM / TMA tile kernel),
 *   kernel 1 = mma.sync split-k cluster kernel (any M),
 *   kernel 2 = tcgen05 tile kernel (64 tokens per CTA tile up to 64 tokens, kernel 7 above;
 *              with B200_PACK_TILE=128: 128-token tiles, two co-resident CTAs per SM from
 *              1024 tokens on),
 *   kernel 3 = tcgen05 split-k cluster kernel (32 tokens per tile, D split 4 ways),
 *   kernel 4 = tcgen05 tile kernel, two co-resident 128-token CTAs per SM at any M,
 *   kernel 5 = tcgen05 split-k cluster kernel with D split 8 ways (D % 512 == 0; chosen
 *              automatically for 17..32 tokens when H <= 2048, e.g. a narrow d_ff shard),
 *   kernel 6 = one-token GEMV kernel (M == 1, D 2048 or 4096): each warp reduces whole
 *              weight rows against the token held in registers, no split-k exchange; chosen
 *              automatically for such calls unless B200_ONE_TOKEN=0,
 *   kernel 7 = tcgen05 tile kernel with 256-token tiles, one CTA per SM and sixteen epilogue
 *              warps (what kernels 0 and 2 run above 64 tokens unless B200_PACK_TILE=128),
 *   kernel 8 / 9 = tcgen05 split-k cluster kernel with 128-token tiles, D split 4 / 2 ways
 *              (chosen automatically for 33..256 tokens while its grid is a single wave).
 * All produce identical slab bytes on exact-arithmetic inputs.  No reference
 * counterpart (the reference has one WGMMA kernel, matmul_d2t.cu:287-709).
 */
int b200_twell_pack_select(const void* x, const void* w, const float* bias, void* packed,
                           int64_t M, int64_t D, int64_t H, int cf, int kernel, void* stream);

/*
 * Error word of the tcgen05 kernel: 0, or the role (1 producer, 2 mma, 3 epilogue) whose
 * bounded mbarrier wait gave up; -1 if it cannot be read.  Reads and clears the word;
 * synchronises the device (a diagnostic, not part of the hot path).
 */
int b200_twell_pack_tc_status(void);

/*
 * Gated TwELL -> dense contraction:
 *   out[r,:] = sum over stored (j, g) of row r:  (g * (x[r,:] . up[j,:])) * down[j,:]
 * Replaces matmul_gated_t2d_out and its flex / high-precision / in-place
 * variants (custom_models/twell_modules/twell.cpp:499-539; kernels
 * custom_models/twell_modules/matmul_gated_t2d.cu:17-594, :972-1541).
 * `out` may alias `x` (in-place).  flags: B200_FLAG_HIGH_PRECISION.
 */
int b200_twell_gated_t2d(const void* x, const void* packed, const void* up,
                         const void* down, void* out, int64_t M, int64_t D,
                         int64_t H, int cf, uint32_t flags, void* workspace,
                         size_t workspace_bytes, void* stream);

/*
 * Non-gated TwELL -> dense down projection: out[r,:] = sum (v * down[j,:]).
 * Replaces matmul_t2d_out (custom_models/twell_modules/twell.cpp:463-483;
 * kernel custom_models/twell_modules/matmul_t2d.cu:15-113).  `num_splits` is
 * accepted for signature compatibility (1, 2, 4 or 8) and does not change the
 * result.
 */
int b200_twell_t2d(const void* packed, const void* down, void* out, int64_t M,
                   int64_t D, int64_t H, int cf, int num_splits, void* workspace,
                   size_t workspace_bytes, void* stream);

/*
 * Fused gated MLP: pack(relu(x @ gate^T + bias)) into `packed`, then the gated
 * contraction into `out` (may alias x).  Replaces TWELL_MLP::run_gated_mlp_layer*
 * (custom_models/twell_modules/mlp_twell.cu:100-232).
 */
int b200_twell_gated_mlp(const void* x, const void* gate, const float* gate_bias,
                         const void* up, const void* down, void* packed, void* out,
                         int64_t M, int64_t D, int64_t H, int cf, uint32_t flags,
                         void* workspace, size_t workspace_bytes, void* stream);

/*
 * The fused gated MLP as ONE kernel for decode-sized calls (1 <= M <= 32): a thread-block
 * cluster per 256-neuron tile computes its slice of the gate, writes the slab words (same
 * bytes as b200_twell_pack) and at once contracts its own active neurons, and the tiles'
 * partial sums meet in the workspace.  Two forms: up to 16 tokens at D = 2048 or 4096 the
 * mma.sync pack kernel with the contraction appended (each finalising CTA gathers the rows of
 * its token's active neurons with 128-bit loads; the last tile of a token to arrive sums the
 * tiles' rows, so no CTA waits for another and any H is served); otherwise the tcgen05 form
 * (every active up / down row is fetched once per call, staged in shared memory by
 * cp.async.bulk, however many tokens fire it; its CTAs meet at a bounded barrier).  Replaces the
 * reference's two launches per layer (custom_models/twell_modules/mlp_twell.cu:126-152:
 * matmul_d2t.cu:287-709 followed by matmul_gated_t2d.cu:17-169).
 *   workspace: at least b200_twell_decode_workspace_bytes(M, D, H) bytes (0 = this shape is
 *     not served), 16-byte aligned, zero-filled once before its first use; it may be the
 *     same buffer that the other contraction entry points use.  Calls that can overlap on
 *     the GPU need different workspaces.
 *   prefetch / prefetch_bytes: optional range of this GPU's memory (16-byte aligned) that the
 *     kernel asks L2 to prefetch while it runs, e.g. the next layer's gate matrix, which does
 *     not depend on this layer's result; NULL / 0 = none.
 * In the tcgen05 form the CTAs of the grid wait for one another (bounded): the call needs the
 * GPU to itself while it runs; the host checks with cudaOccupancyMaxActiveClusters that the
 * grid is resident at once.  Returns B200_EUNSUPPORTED when the shape, the workspace or the
 * residency check rules the kernel out.  b200_twell_gated_mlp / b200_twell_mlp take this path
 * by themselves only when the environment variable B200_DECODE_FUSED is 1 (every call a form
 * serves) or 2 (the mma.sync form only) and their workspace argument is large enough:
 * measured on B200 at D = 2048, H = 8192 the two-kernel form is the faster one - 16.7 / 20.2 /
 * 23.9 / 24.8 us per layer at 1 / 8 / 16 / 32 tokens against 20.2 / 23.1 / 33.6 us (mma.sync
 * form, 1 / 8 / 16 tokens) and 44.1 us (tcgen05 form, 32 tokens) - because each serial phase
 * of a one-kernel form costs 0.3-4 us of latency that the launch it saves does not pay for.
 */
size_t b200_twell_decode_workspace_bytes(int64_t M, int64_t D, int64_t H);

int b200_twell_gated_mlp_decode(const void* x, const void* gate, const float* gate_bias,
                                const void* up, const void* down, void* packed, void* out,
                                int64_t M, int64_t D, int64_t H, int cf, uint32_t flags,
                                void* workspace, size_t workspace_bytes, const void* prefetch,
                                int64_t prefetch_bytes, void* stream);

/* Error word of the fused decode kernel: 0, or the wait that gave up (1 producer, 2 mma,
 * 3 accumulator, 4 up rows, 5 down rows, 6 cross-tile barrier); -1 if it cannot be read.
 * Reads and clears the word; synchronises the device. */
int b200_twell_decode_status(void);

/* Asks L2 to prefetch [ptr, ptr + bytes) of this GPU's memory (cp.async.bulk.prefetch.L2,
 * one small kernel on `stream`).  A hint: no result depends on it.  No reference counterpart. */
int b200_l2_prefetch(const void* ptr, int64_t bytes, void* stream);

/*
 * Fused non-gated MLP: pack(relu(x @ up^T)) then the down projection.
 * Replaces TWELL_MLP::run_mlp_layer* (custom_models/twell_modules/mlp_twell.cu:73-98).
 */
int b200_twell_mlp(const void* x, const void* up, const void* down, void* packed,
                   void* out, int64_t M, int64_t D, int64_t H, int cf,
                   int num_splits, void* workspace, size_t workspace_bytes,
                   void* stream);

/* ------------------------------------------------------------------------
 * Hybrid sparse training operator (custom_models/hybrid_modules).
 * Every sparse operand is a slab-shaped uint32 array with the layout of `packed`:
 * word (row, tile, slot) = col | bf16(value) << 16 for the same entry as the
 * pattern P produced by b200_twell_pack; count words are copied from P.
 * ------------------------------------------------------------------------ */

/*
 * Forward: R = (x k_w^T) sampled at P's pattern (bf16), T = R * P (bf16 multiply),
 * row_l1[r] = sum |T[r,:]| (fp32), row_nnz[r] = true positive count of the row,
 * row_drop[r] = entries of the row lost to slab overflow.  Replaces
 * new_product_as_sparse_sma + sparse_elementwise of ff_forward_cuda_gated
 * (custom_models/hybrid_modules/custom_op.cpp:131-132; kernels hybrid_sp.cu:711-805,
 * :1480-1587).
 */
int b200_hybrid_sddmm_fwd(const void* x, const void* k_w, const void* p_slab, void* r_slab,
                          void* t_slab, float* row_l1, int* row_nnz, int* row_drop,
                          int64_t M, int64_t D, int64_t H, int cf, void* stream);

/*
 * Backward: dT = (g_out v_w^T) at the pattern (bf16) + (*l1_grad / M) * sign(R) (bf16),
 * dR = dT * P, dU = dT * R.  Replaces the dT / L1-shift / dR / dU steps of
 * ff_backward_cuda_gated (custom_op.cpp:203-222; hybrid_sp.cu:711-805, :1754-1779,
 * :1480-1664).  l1_grad: device pointer to the fp32 gradient of l1 (NULL = 0); it is
 * read on the device, so the host never waits for it.
 */
int b200_hybrid_sddmm_bwd(const void* g_out, const void* v_w, const void* p_slab,
                          const void* r_slab, void* dr_slab, void* du_slab,
                          const float* l1_grad, int64_t M, int64_t D, int64_t H, int cf,
                          void* stream);

/*
 * Row product: out[r,:] = sum over row r's entries of value * b_rows[col,:], fp32 fma,
 * bf16 store.  Replaces sparse_dense_gemm_hybrid_dense (custom_op.cpp:133, :239-245;
 * hybrid_sp.cu:222-301, :1320-1396).  Workspace as for b200_twell_gated_t2d.
 */
int b200_hybrid_spmm(const void* vals_slab, const void* b_rows, void* out, int64_t M,
                     int64_t D, int64_t H, int cf, void* workspace, size_t workspace_bytes,
                     void* stream);

/*
 * Column lists of the pattern: col_start[H+1] (exclusive scan of per-column counts) and,
 * for list position i, csc_row[i] = row and csc_pos[i] = word index into a slab array.
 * col_count[H], cursor[H], overflow[1] are scratch / status (overflow = entries beyond
 * `capacity`).  Order inside a column follows atomic arrival (as the reference's scatter
 * transpose does).  Replaces transpose_hybrid_dense (custom_op.cpp:182-237;
 * hybrid_sp.cu:1042-1214).
 */
int b200_hybrid_csc_build(const void* p_slab, int* col_count, int* col_start, int* cursor,
                          int* csc_row, int* csc_pos, int64_t capacity, int* overflow,
                          int64_t M, int64_t H, int cf, void* stream);

/*
 * Transposed product(s): out0[j,:] = sum over column j's list of value(vals0) * b_rows[row,:]
 * (and out1 from vals1 over the same rows when vals1 != NULL).  fp32 fma, bf16 store,
 * out [H, D].  Replaces the three sparse_dense_gemm_hybrid_dense calls on transposed
 * operands (custom_op.cpp:261-269).
 */
int b200_hybrid_spmm_t(const void* vals0, const void* vals1, const int* col_start,
                       const int* csc_row, const int* csc_pos, int64_t capacity,
                       const void* b_rows, void* out0, void* out1, int64_t H, int64_t D,
                       void* stream);

/*
 * Weight-gradient product on the tensor cores: out[H, D] = vals^T . rows, with vals a
 * slab-shaped sparse [M, H] operand (dR, dU or T) and rows a dense [M, D] bf16 matrix (X or
 * the output gradient).  The reduction runs over all M tokens and the result is dense, so
 * for training-sized M this is a GEMM: the slab is scattered into a zero-filled K-major
 * [H, M] matrix, rows is transposed once (reuse_rows_t = 1 reuses the transposed copy left
 * in ws by the previous call with the same rows) and a tcgen05 GEMM does the rest.  Same
 * result as b200_hybrid_csc_build + b200_hybrid_spmm_t (fp32 accumulation, bf16 store;
 * the summation order differs), which remain the path for small M.  Replaces
 * sparse_dense_gemm_hybrid_dense on transposed operands (custom_op.cpp:261-269).
 * ws: b200_hybrid_wgrad_workspace_bytes(M, D, H) bytes, 256-byte aligned.
 */
size_t b200_hybrid_wgrad_workspace_bytes(int64_t M, int64_t D, int64_t H);
int b200_hybrid_wgrad_dense(const void* vals_slab, const void* rows, void* out, int64_t M,
                            int64_t D, int64_t H, int cf, int reuse_rows_t, void* ws,
                            size_t ws_bytes, void* stream);

/*
 * Dead-neuron bookkeeping for the hybrid path.  active_rows[j] (int32 [H], overwritten) =
 * number of token rows whose stored value for neuron j is non-zero; the values are read
 * from vals_slab (the forward's T = relu(gate)*up slab), or from p_slab itself when
 * vals_slab is NULL.  When last_activated (int64 [H]) is not NULL it is updated in place:
 * 0 for a neuron with active_rows > 0, else + microbatch_tokens.  Entries a slab dropped on
 * overflow are not seen.  Supplies what SparsityTracker.record_activations computes from the
 * dense activation (custom_models/sparse_models.py:148-181) and record_l0_l1 leaves stale
 * on the fused path (:183-208).
 */
int b200_hybrid_neuron_activity(const void* p_slab, const void* vals_slab, int64_t M, int64_t H,
                                int cf, int64_t microbatch_tokens, int* active_rows,
                                int64_t* last_activated, void* stream);

/*
 * Row-ELL x dense: C[r,:] = sum_k vals[r,k] * B[cols[r,k],:] for rows with
 * 0 < row_counts[r] <= overflow_threshold, zeros otherwise.  vals bf16 / cols uint16
 * [M, ell_stride], B [K, N] bf16, C [M, N] bf16.  Replaces ell_spmm_raw
 * (custom_op.cpp:313; hybrid_sp.cu:222-301).
 */
int b200_hybrid_ell_spmm_raw(const void* ell_vals, const void* ell_cols, const int* row_counts,
                             const void* b, void* c, int64_t M, int64_t K, int64_t N,
                             int64_t ell_stride, int64_t overflow_threshold, void* stream);

/* ------------------------------------------------------------------------
 * Hybrid contraction for large token counts: rows whose gate has more than
 * nnz_threshold positives, or whose slab overflowed in some tile, are computed
 * as dense tcgen05 GEMMs (gate and up recomputed densely, so nothing is lost to
 * slab capacity); all other rows run on the gather kernel of b200_twell_gated_t2d.
 * At most dense_cap rows (ascending row order) take the dense route.
 * Replaces the dense tail of the reference's hybrid format (hybrid_sp.cu:516-576:
 * rows beyond the ELL width go to tail_dense and through torch::matmul); the
 * reference's TwELL inference kernels have no such route and drop overflowed
 * entries (matmul_gated_t2d.cu:17-169).
 *   gate, up, down [H, D] bf16 as elsewhere; down_t [D, H] bf16 = a K-major copy of
 *   the down projection (down_proj.weight itself) kept by the caller;
 *   hybrid_ws: b200_twell_hybrid_workspace_bytes(M, D, H, dense_cap) bytes,
 *   256-byte aligned, contents need not be initialised; workspace as in
 *   b200_twell_gated_t2d.  No host synchronisation.
 * ------------------------------------------------------------------------ */
size_t b200_twell_hybrid_workspace_bytes(int64_t M, int64_t D, int64_t H, int64_t dense_cap);

int b200_twell_gated_t2d_hybrid(const void* x, const void* packed, const void* gate,
                                const float* gate_bias, const void* up, const void* down,
                                const void* down_t, void* out, int64_t M, int64_t D, int64_t H,
                                int cf, uint32_t flags, int64_t nnz_threshold, int64_t dense_cap,
                                void* hybrid_ws, size_t hybrid_ws_bytes, void* workspace,
                                size_t workspace_bytes, void* stream);

/* b200_twell_pack followed by b200_twell_gated_t2d_hybrid. */
int b200_twell_gated_mlp_hybrid(const void* x, const void* gate, const float* gate_bias,
                                const void* up, const void* down, const void* down_t,
                                void* packed, void* out, int64_t M, int64_t D, int64_t H, int cf,
                                uint32_t flags, int64_t nnz_threshold, int64_t dense_cap,
                                void* hybrid_ws, size_t hybrid_ws_bytes, void* workspace,
                                size_t workspace_bytes, void* stream);

/*
 * Every row on the dense route, with no slab, routing or gather: for token counts so
 * large that the weights are amortised and the per-entry gather cannot win.
 *   h_ws [M, H] bf16 = relu(x gate^T + gate_bias) * (x up^T)   (caller scratch)
 *   out  [M, D] bf16 = h_ws . down,  down_t [D, H] bf16 as above.
 * The function of SparseMLP's dense inference path (sparse_models.py:343-351) on
 * tcgen05; the reference runs it through torch matmuls.
 */
int b200_dense_gated_mlp(const void* x, const void* gate, const float* gate_bias, const void* up,
                         const void* down_t, void* h_ws, void* out, int64_t M, int64_t D,
                         int64_t H, void* stream);

/* counters_out[0] = rows the last call on this workspace routed to the dense path,
 * [1] = overflowed rows left on the sparse path because dense_cap was exhausted,
 * [2] = rows that qualified.  Synchronises the device. */
int b200_twell_hybrid_counters(const void* hybrid_ws, int64_t M, int64_t D, int64_t H,
                               int64_t dense_cap, int* counters_out);

/* 0, or the stage (1 producer, 2 mma, 3 epilogue) of a bounded wait that gave up in the
 * dense GEMMs; reads and clears the word; synchronises the device. */
int b200_twell_hybrid_status(void);

/* ------------------------------------------------------------------------
 * Sum all-reduce of the d_ff-sharded FFN output over peer-mapped memory (no reference
 * counterpart: the reference is data parallel only).  Every rank owns one symmetric
 * block of b200_peer_allreduce_block_bytes(max_bytes) bytes, zero-filled once, and
 * knows the device address of every rank's block (peer-mapped: CUDA IPC, VMM or
 * torch symmetric memory).  One call = one kernel per rank: push the local bf16
 * tensor into every peer's inbox as 8-byte {payload, call epoch} words (no fence, no
 * separate flag), poll the own inbox with a bounded wait, sum in rank order into `out`
 * (identical bits on every rank).  All ranks must issue the same sequence of calls
 * (same n_elems) on their streams; the launch may be captured in a CUDA graph.
 * ------------------------------------------------------------------------ */
size_t b200_peer_allreduce_block_bytes(int64_t max_bytes);

/* peer_blocks: host array of `world` device pointers (entry `rank` = this rank's block).
 * n_elems: multiple of 8, n_elems*2 <= max_bytes.  world <= 8. */
int b200_peer_allreduce_bf16(const void* local_in, void* out, int64_t n_elems,
                             void* const* peer_blocks, int rank, int world,
                             int64_t block_bytes, void* stream);

/* 0, or 0x100 + peer rank if a wait for that peer gave up; -1 if unreadable.  Reads and
 * clears the word; synchronises the device. */
int b200_peer_allreduce_status(void* my_block);

/* ------------------------------------------------------------------------
 * Gated contraction fused with the d_ff-shard all-reduce (no reference counterpart).
 * The CTA that holds the final sums of a (token, column slice) rounds them to bf16, sends
 * them to every peer as 8-byte {bf16 pair, call epoch} words, polls - bounded - its own
 * inbox for the peers' words, adds the `world` contributions in rank order and stores:
 * the same result as b200_twell_gated_t2d + b200_peer_allreduce_bf16 in one kernel.
 * Decode-sized calls only: every CTA must be resident while it waits (M * clusters <= 2 x SMs)
 * and M <= 256; larger calls return B200_EUNSUPPORTED (use the two-kernel form).
 * peer_blocks: `world` device pointers to symmetric, peer-mapped blocks of
 * b200_fused_allreduce_block_bytes(max_tokens, D) bytes, zero-filled once, used by this
 * entry point only.  All ranks issue the same sequence of calls.  Capturable.
 * world == 1 degenerates to b200_twell_gated_t2d.
 * ------------------------------------------------------------------------ */
size_t b200_fused_allreduce_block_bytes(int64_t max_tokens, int64_t D);

int b200_twell_gated_t2d_allreduce(const void* x, const void* packed, const void* up,
                                   const void* down, void* out, int64_t M, int64_t D, int64_t H,
                                   int cf, uint32_t flags, void* workspace, size_t workspace_bytes,
                                   void* const* peer_blocks, int rank, int world,
                                   int64_t block_bytes, void* stream);

/* b200_twell_pack followed by b200_twell_gated_t2d_allreduce. */
int b200_twell_gated_mlp_allreduce(const void* x, const void* gate, const float* gate_bias,
                                   const void* up, const void* down, void* packed, void* out,
                                   int64_t M, int64_t D, int64_t H, int cf, uint32_t flags,
                                   void* workspace, size_t workspace_bytes,
                                   void* const* peer_blocks, int rank, int world,
                                   int64_t block_bytes, void* stream);

/* 0, or 0x100 + peer rank if a wait for that peer gave up; -1 if unreadable.  Reads and
 * clears the word; synchronises the device. */
int b200_fused_allreduce_status(void* my_block);

/*
 * Residual add + RMSNorm of a few token rows in one kernel (the element-wise steps around the
 * FFN of a decoder layer; no counterpart in the reference, whose models run them as separate
 * torch modules around the MLP swap point, custom_models/sparse_models.py:552-614):
 *   x_out[r,:] = x[r,:] + delta[r,:]            (delta may be NULL; x_out may alias x or be NULL)
 *   h_out[r,:] = x_out[r,:] * rsqrt(mean(x_out[r,:]^2) + eps) * weight[:]
 * bf16 in and out, fp32 inside; D % 8 == 0, D <= 8192; h_out must not alias the others.
 */
int b200_residual_rmsnorm(const void* x, const void* delta, const void* weight, float eps,
                          void* x_out, void* h_out, int64_t M, int64_t D, void* stream);

/*
 * Gated contraction for hosts that may not allocate device memory (no counterpart
 * in the reference).  Same arguments and result as b200_twell_gated_t2d, minus the
 * workspace: the scratch for the few-token shape is a 1 MiB array built into the
 * library image (resident on every GPU that loads the library until exit), so the
 * call makes no cudaMalloc / cudaFree and needs no caller buffer.
 *   - Limit: M <= min(512, 129024 / D) tokens (63 at D = 2048, 31 at D = 4096);
 *     larger M returns B200_EWORKSPACE - use b200_twell_gated_t2d there.
 *   - The first call on each device resolves the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call
 *     before starting any stream capture.
 *   - All calls on a device share the one array; the arrival counters in it are
 *     cleared at every call.  Calls that can overlap on the GPU (two streams, two
 *     host threads) race on it: issue them on one stream, or serialise them.
 */
int b200_twell_gated_t2d_noalloc(const void* x, const void* packed, const void* up,
                                 const void* down, void* out, int64_t M, int64_t D,
                                 int64_t H, int cf, uint32_t flags, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_SPARSE_FFN_H_ */
