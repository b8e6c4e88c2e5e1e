// Hybrid contraction for large token counts: dense-enough token rows leave the gather path
// and run as dense tensor-core GEMMs; the remaining rows stay on the TwELL gather kernel.
//
// A token whose gate row has more positives than a threshold, or whose slab overflowed in
// some 256-neuron tile (count > capacity, entries lost), costs more as a per-entry gather
// of W_up / W_down rows through L2 than as three dense products.  The path is
//   1. route:   per row, nnz and overflow from the slab count words -> flag; a single-CTA
//               scan turns the flags into an ascending list of dense rows (at most
//               `dense_cap`; later rows stay sparse and are counted if they were lossy),
//   2. sparse:  the gather kernel skips flagged rows,
//   3. gather:  Xd[i, :] = x[dense_rows[i], :],
//   4. GEMM 1:  Hd = relu(Xd Wg^T + b) * (Xd Wu^T)   tcgen05, two TMEM accumulators per CTA
//               (gate and up of the same 128 neurons x 128 tokens), bf16 store,
//   5. GEMM 2:  y[dense_rows[i], :] = Hd Wd          tcgen05, K = H, A operand = Wd^T [D, H]
//               (a K-major copy of the down projection kept by the caller), scattered store.
// Dense rows are computed from the dense gate product, not from the slab, so rows that
// overflowed the slab lose nothing.  The dense-row count lives on the device: grids are
// sized for `dense_cap` and CTAs beyond the count return at once; no host synchronisation.
//
// Reference counterpart: the hybrid format's dense tail (hybrid_sp.cu:516-576: rows whose
// count exceeds the ELL width go to `tail_dense` and are multiplied with torch::matmul);
// the TwELL inference kernels themselves have no such route
// (custom_models/twell_modules/matmul_gated_t2d.cu:17-169 drops overflowed entries).
#include <cooperative_groups.h>

#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace b200 {

int twell_t2d_launch(bool gated, bool hp, const void* x, const void* packed, const void* up,
                     const void* down, void* out, int64_t M, int64_t D, int64_t H, int cf,
                     void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream,
                     const unsigned char* skip_rows, const FusedAr* fused_ar);
int sm_count();

namespace {

__device__ int g_dense_error = 0;

// Tile shape of the dense GEMMs: tokens per CTA, shared-memory stages, CTAs per SM.
// Two co-resident CTAs of 128 tokens (2 x 256 TMEM columns, 2 x 2 stages of 48 KB) let one
// CTA's epilogue run under the other's MMAs.  Measured on B200 for all three products at
// M = 16384, D = 2048, H = 11008: 1100 TFLOP/s, against 841 for one CTA with four stages and
// 1044 for one CTA of 256 tokens with three (cuBLAS bf16: 1394).
#ifndef B200_DENSE_TOK
#define B200_DENSE_TOK 128
#endif
#ifndef B200_DENSE_STAGES
#define B200_DENSE_STAGES 2
#endif
#ifndef B200_DENSE_MINB
#define B200_DENSE_MINB 2
#endif
// 1 / 0 force the persistent / the one-tile form of the GEMM; -1 chooses per call.
#ifndef B200_DENSE_PERSISTENT
#define B200_DENSE_PERSISTENT (-1)
#endif
#ifndef B200_DENSE_KS
#define B200_DENSE_KS 64
#endif
constexpr int kDenseTok = B200_DENSE_TOK;
constexpr int kDenseStages = B200_DENSE_STAGES;

// ---- routing ----------------------------------------------------------------
// One warp per row: flag bit 0 = nnz above the threshold, bit 1 = some tile overflowed.
__global__ void __launch_bounds__(256)
route_flags_kernel(const uint32_t* __restrict__ packed, int M, int tiles, int slab_w,
                   int nnz_threshold, unsigned char* __restrict__ flags) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const uint32_t* prow = packed + (size_t)row * tiles * slab_w;
  int nnz = 0, over = 0;
  for (int t = lane; t < tiles; t += 32) {
    const int c = (int)prow[(size_t)t * slab_w];
    nnz += max(c, 0);
    over |= (c > slab_w - 1) ? 1 : 0;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    nnz += __shfl_xor_sync(0xffffffffu, nnz, o);
    over |= __shfl_xor_sync(0xffffffffu, over, o);
  }
  if (lane == 0) flags[row] = (unsigned char)((nnz > nnz_threshold ? 1 : 0) | (over ? 2 : 0));
}

// One CTA: ascending list of flagged rows, at most `cap`; rows beyond it return to the
// sparse path.  counters[0] = dense rows, [1] = overflowed rows left on the (lossy) sparse
// path, [2] = rows that qualified.
__global__ void __launch_bounds__(1024)
route_compact_kernel(unsigned char* __restrict__ flags, int M, int cap, int* __restrict__ rows,
                     int* __restrict__ counters) {
  __shared__ int warp_sum[32];
  __shared__ int lossy_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (M + 1023) / 1024;
  const int r0 = tid * per, r1 = min(M, r0 + per);
  if (tid == 0) lossy_s = 0;
  int mine = 0;
  for (int r = r0; r < r1; ++r) mine += flags[r] != 0;
  int inc = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += v;
  }
  if (lane == 31) warp_sum[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sum[lane], winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += v;
    }
    warp_sum[lane] = winc - w;  // exclusive prefix of the warp totals
    if (lane == 31) counters[2] = winc;
    if (lane == 31) counters[0] = min(winc, cap);
  }
  __syncthreads();
  int pos = warp_sum[warp] + inc - mine;
  int lossy = 0;
  for (int r = r0; r < r1; ++r) {
    const unsigned char f = flags[r];
    if (f == 0) continue;
    if (pos < cap) {
      rows[pos] = r;
    } else {
      flags[r] = 0;  // stays on the gather path
      lossy += (f & 2) ? 1 : 0;
    }
    ++pos;
  }
  if (lossy) atomicAdd(&lossy_s, lossy);
  __syncthreads();
  if (tid == 0) counters[1] = lossy_s;
}

__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ rows,
                   const int* __restrict__ counters, uint4* __restrict__ xd, int vec_per_row) {
  const int i = blockIdx.x;
  if (i >= counters[0]) return;
  const uint4* src = x + (size_t)rows[i] * vec_per_row;
  uint4* dst = xd + (size_t)i * vec_per_row;
  for (int v = threadIdx.x; v < vec_per_row; v += 256) dst[v] = __ldg(src + v);
}

// ---- dense GEMMs --------------------------------------------------------------
// acc0[128, NTOK] = A0 tile . B^T, acc1[128, NTOK] = A1 tile . B^T over K, both in TMEM
// (lane = output feature, column = token).
//   DUAL:  A0 = W_gate rows, A1 = W_up rows of the same 128 neurons (grid.x = H / 128);
//          epilogue h = relu(g + bias) * u -> out[token, neuron] (ld_out = H).
//   !DUAL: A0 / A1 = rows [256 t, +128) and [256 t + 128, +128) of one matrix
//          (grid.x = N_out / 256); epilogue out[row_ids[token], feature] = acc (ld_out = N_out).
// grid.y = token tiles of the capacity; tiles at or beyond *n_rows_ptr return at once.
template <int NTOK, int STAGES, bool DUAL, int KS>
__global__ void __launch_bounds__(kThreadsTc, B200_DENSE_MINB)
dense_rows_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a0,
                       const __grid_constant__ CUtensorMap tmap_a1,
                       const __grid_constant__ CUtensorMap tmap_b, const float* __restrict__ bias,
                       __nv_bfloat16* __restrict__ out, const int* __restrict__ row_ids,
                       const int* __restrict__ n_rows_ptr, int n_rows_host, int K, int ld_out,
                       int group) {
  // KS k-values per stage: 64 (128-byte rows, 128-byte swizzle) or 32 (64-byte rows and swizzle)
  constexpr int kATile = 128 * KS * 2;
  constexpr int kBTileBytes = NTOK * KS * 2;
  constexpr int kStageBytes = 2 * kATile + kBTileBytes;
  constexpr uint32_t kTmemCols = 2 * NTOK;
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);

  // row count: on the device when routing decided it, else given by the host
  const int n_rows = n_rows_ptr != nullptr ? *n_rows_ptr : n_rows_host;
  int tile, mblk;
  raster_remap(group, tile, mblk);
  const int m0 = mblk * NTOK;
  if (m0 >= n_rows) return;  // uniform for the CTA: nothing allocated yet

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ksteps = K / KS;
  const int a0_row = DUAL ? tile * 128 : tile * 256;
  const int a1_row = DUAL ? tile * 128 : tile * 256 + 128;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
          abort_s = 1;
          atomicExch(&g_dense_error, 1);
          break;
        }
        unsigned char* st = smem + (size_t)s * kStageBytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)kStageBytes);
        tma_load_2d(st, &tmap_a0, k * KS, a0_row, &full_bar[s]);
        tma_load_2d(st + kATile, DUAL ? &tmap_a1 : &tmap_a0, k * KS, a1_row,
                    &full_bar[s]);
        tma_load_2d(st + 2 * kATile, &tmap_b, k * KS, m0, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) {
          abort_s = 1;
          atomicExch(&g_dense_error, 2);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a0 = smem_u32(smem + (size_t)s * kStageBytes);
        const uint64_t da0 = KS == 64 ? umma_desc(a0) : umma_desc_sw64(a0),
                       da1 = KS == 64 ? umma_desc(a0 + kATile) : umma_desc_sw64(a0 + kATile),
                       db = KS == 64 ? umma_desc(a0 + 2 * kATile) : umma_desc_sw64(a0 + 2 * kATile);
#pragma unroll
        for (int kk = 0; kk < KS / 16; ++kk) {
          const uint32_t acc = (k > 0 || kk > 0) ? 1u : 0u;
          umma_bf16(tmem_base, da0 + 2 * kk, db + 2 * kk, kIdesc, acc);
          umma_bf16(tmem_base + NTOK, da1 + 2 * kk, db + 2 * kk, kIdesc, acc);
        }
        umma_commit(&empty_bar[s]);
      }
      if (!abort_s) umma_commit(&acc_bar);
    }
  } else {
    // ---- epilogue: warps 2..5 own TMEM lane quarters 2, 3, 0, 1 ----
    const int q = warp & 3;
    bool ok = mbar_wait(&acc_bar, 0u);
    if (!ok) {
      abort_s = 1;
      atomicExch(&g_dense_error, 3);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const int f0 = a0_row + q * 32 + lane;  // output feature of accumulator 0
    const float b0 = (DUAL && bias != nullptr) ? bias[f0] : 0.f;
    for (int tb = 0; tb < NTOK / 32 && ok; ++tb) {
      if (m0 + tb * 32 >= n_rows) break;
      float v0[32], v1[32];
      tmem_ld32(lane_addr + (uint32_t)(tb * 32), v0);
      tmem_ld32(lane_addr + (uint32_t)(NTOK + tb * 32), v1);
      if (DUAL) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int tok = m0 + tb * 32 + c;
          if (tok >= n_rows) break;
          const float g = v0[c] + b0;
          float h = 0.f;
          if (g > 0.f)
            h = __bfloat162float(__float2bfloat16_rn(g)) * __bfloat162float(__float2bfloat16_rn(v1[c]));
          out[(size_t)tok * ld_out + f0] = __float2bfloat16_rn(h);
        }
      } else {
        const int t_mine = m0 + tb * 32 + lane;
        const int rid = t_mine < n_rows ? (row_ids != nullptr ? row_ids[t_mine] : t_mine) : -1;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int r = __shfl_sync(0xffffffffu, rid, c);
          if (r < 0) continue;
          __nv_bfloat16* orow = out + (size_t)r * ld_out;
          orow[f0] = __float2bfloat16_rn(v0[c]);
          orow[f0 + 128] = __float2bfloat16_rn(v1[c]);
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

// The same GEMM as ONE CTA per SM on 256-token tiles with sixteen epilogue warps: the two
// accumulators fill all 512 TMEM columns, a 64-k stage is 32 KB of A rows + 32 KB of token rows
// (131 flop per staged byte against 87 for the 128-token tile, which is what the L2 -> SM
// operand stream limits), and the epilogue is spread over four groups of four warps that take
// every fourth 32-token block.  Used when the host knows the row count and the grid fills the GPU.
constexpr int kThreadsDenseWide = 64 + 512;

template <int STAGES, bool DUAL>
__global__ void __launch_bounds__(kThreadsDenseWide, 1)
dense_rows_gemm_wide_kernel(const __grid_constant__ CUtensorMap tmap_a0,
                            const __grid_constant__ CUtensorMap tmap_a1,
                            const __grid_constant__ CUtensorMap tmap_b,
                            const float* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ row_ids, int n_rows, int K, int ld_out,
                            int group) {
  constexpr int NTOK = 256;
  constexpr int kBTileBytes = NTOK * 128;
  constexpr int kStageBytes = 2 * kATileBytes + kBTileBytes;
  constexpr uint32_t kTmemCols = 2 * NTOK;
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);

  int tile, mblk;
  raster_remap(group, tile, mblk);
  const int m0 = mblk * NTOK;
  if (m0 >= n_rows) return;  // uniform for the CTA: nothing allocated yet

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ksteps = K / kStageK;
  const int a0_row = DUAL ? tile * 128 : tile * 256;
  const int a1_row = DUAL ? tile * 128 : tile * 256 + 128;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
          abort_s = 1;
          atomicExch(&g_dense_error, 1);
          break;
        }
        unsigned char* st = smem + (size_t)s * kStageBytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)kStageBytes);
        tma_load_2d(st, &tmap_a0, k * kStageK, a0_row, &full_bar[s]);
        tma_load_2d(st + kATileBytes, DUAL ? &tmap_a1 : &tmap_a0, k * kStageK, a1_row,
                    &full_bar[s]);
        tma_load_2d(st + 2 * kATileBytes, &tmap_b, k * kStageK, m0, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) {
          abort_s = 1;
          atomicExch(&g_dense_error, 2);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a0 = smem_u32(smem + (size_t)s * kStageBytes);
        const uint64_t da0 = umma_desc(a0), da1 = umma_desc(a0 + kATileBytes),
                       db = umma_desc(a0 + 2 * kATileBytes);
#pragma unroll
        for (int kk = 0; kk < kStageK / 16; ++kk) {
          const uint32_t acc = (k > 0 || kk > 0) ? 1u : 0u;
          umma_bf16(tmem_base, da0 + 2 * kk, db + 2 * kk, kIdesc, acc);
          umma_bf16(tmem_base + NTOK, da1 + 2 * kk, db + 2 * kk, kIdesc, acc);
        }
        umma_commit(&empty_bar[s]);
      }
      if (!abort_s) umma_commit(&acc_bar);
    }
  } else {
    // ---- epilogue: group g = (warp - 2) / 4 takes token blocks g, g + 4; quarter = warp % 4 ----
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;
    bool ok = mbar_wait(&acc_bar, 0u);
    if (!ok) {
      abort_s = 1;
      atomicExch(&g_dense_error, 3);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const int f0 = a0_row + q * 32 + lane;  // output feature of accumulator 0
    const float b0 = (DUAL && bias != nullptr) ? bias[f0] : 0.f;
    for (int tb = grp; tb < NTOK / 32 && ok; tb += 4) {
      if (m0 + tb * 32 >= n_rows) break;
      float v0[32], v1[32];
      tmem_ld32(lane_addr + (uint32_t)(tb * 32), v0);
      tmem_ld32(lane_addr + (uint32_t)(NTOK + tb * 32), v1);
      if (DUAL) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int tok = m0 + tb * 32 + c;
          if (tok >= n_rows) break;
          const float g = v0[c] + b0;
          float h = 0.f;
          if (g > 0.f)
            h = __bfloat162float(__float2bfloat16_rn(g)) * __bfloat162float(__float2bfloat16_rn(v1[c]));
          out[(size_t)tok * ld_out + f0] = __float2bfloat16_rn(h);
        }
      } else {
        const int t_mine = m0 + tb * 32 + lane;
        const int rid = t_mine < n_rows ? (row_ids != nullptr ? row_ids[t_mine] : t_mine) : -1;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int r = __shfl_sync(0xffffffffu, rid, c);
          if (r < 0) continue;
          __nv_bfloat16* orow = out + (size_t)r * ld_out;
          orow[f0] = __float2bfloat16_rn(v0[c]);
          orow[f0 + 128] = __float2bfloat16_rn(v1[c]);
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

// Split-k form of the same GEMM for at most a few hundred rows, where a (feature tile, token
// block) grid is a handful of CTAs that each walk a long, latency-bound k-loop (the down
// projection of 128 rows at D 2048 is 8 tiles of K = d_ff).  A cluster of CL CTAs owns a tile of
// 128 features (DUAL: 128 gate + 128 up rows, two accumulators) x 128 rows and splits K; the
// fp32 partial tiles are pushed into the operand rings once every CTA of the cluster is past its
// last MMA (cluster barrier), CTA r then finalises rows [r * 128 / CL, (r + 1) * 128 / CL).
// 576 threads: warp 0 producer, warp 1 mma, warps 2..17 epilogue (four groups of 32 rows).
// grid = (a_rows / 128 * CL, ceil(rows / 128)), cluster = CL.
template <int CL, int STAGES, bool DUAL>
__global__ void __launch_bounds__(kThreadsDenseWide, 1)
dense_rows_gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a0,
                              const __grid_constant__ CUtensorMap tmap_a1,
                              const __grid_constant__ CUtensorMap tmap_b,
                              const float* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                              const int* __restrict__ row_ids, int n_rows, int K, int ld_out) {
  constexpr int NTOK = 128;
  constexpr int NACC = DUAL ? 2 : 1;
  constexpr int TOK = NTOK / CL;  // rows finalised per CTA
  constexpr int kBTileBytes = NTOK * 128;
  constexpr int kStageBytes = NACC * kATileBytes + kBTileBytes;
  constexpr uint32_t kTmemCols = NACC * NTOK;
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);
  constexpr int kStride = NACC * 128 + 4;    // floats per (source rank, row) of the exchange
  constexpr int EPT = TOK * 128 / 512;       // outputs per epilogue thread in the final pass
  static_assert(CL == 2 || CL == 4 || CL == 8, "cluster size");
  static_assert((size_t)NTOK * kStride * sizeof(float) <= (size_t)STAGES * kStageBytes,
                "the partial sums must fit into the operand ring");

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* part = reinterpret_cast<float*>(smem);  // [CL x TOK][kStride], once the ring is free
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_s;

  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / CL;
  const int m0 = blockIdx.y * NTOK;
  const int kc = K / CL;
  const int ksteps = kc / kStageK;
  const int k_base = crank * kc;
  const int a_row = tile * 128;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;

  bool ok = true;
  if (warp == 0) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
          abort_s = 1;
          atomicExch(&g_dense_error, 1);
          break;
        }
        unsigned char* st = smem + (size_t)s * kStageBytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)kStageBytes);
        const int kcoord = k_base + k * kStageK;
        tma_load_2d(st, &tmap_a0, kcoord, a_row, &full_bar[s]);
        if (DUAL) tma_load_2d(st + kATileBytes, &tmap_a1, kcoord, a_row, &full_bar[s]);
        tma_load_2d(st + NACC * kATileBytes, &tmap_b, kcoord, m0, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) {
          abort_s = 1;
          atomicExch(&g_dense_error, 2);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a0 = smem_u32(smem + (size_t)s * kStageBytes);
        const uint64_t da0 = umma_desc(a0), da1 = umma_desc(a0 + kATileBytes),
                       db = umma_desc(a0 + NACC * kATileBytes);
#pragma unroll
        for (int kk = 0; kk < kStageK / 16; ++kk) {
          const uint32_t acc = (k > 0 || kk > 0) ? 1u : 0u;
          umma_bf16(tmem_base, da0 + 2 * kk, db + 2 * kk, kIdesc, acc);
          if (DUAL) umma_bf16(tmem_base + NTOK, da1 + 2 * kk, db + 2 * kk, kIdesc, acc);
        }
        umma_commit(&empty_bar[s]);
      }
      if (!abort_s) umma_commit(&acc_bar);
    }
  } else {
    ok = mbar_wait(&acc_bar, 0u);  // every MMA of this CTA has read its operands
    if (!ok) {
      abort_s = 1;
      atomicExch(&g_dense_error, 3);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  cluster.sync();  // every CTA of the cluster is past its last MMA: the rings are free

  if (warp >= 2 && ok) {
    // ---- TMEM -> registers -> the owner's ring memory ----
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;  // rows [32 grp, 32 grp + 32) of the block
    const int nl = q * 32 + lane;     // feature inside the tile
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(grp * 32);
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      float v[32];
      tmem_ld32(lane_addr + (uint32_t)(a * NTOK), v);
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int t = grp * 32 + c, owner = t / TOK, tl = t % TOK;
        cluster.map_shared_rank(part, owner)[(size_t)(crank * TOK + tl) * kStride + a * 128 + nl] =
            v[c];
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster.sync();  // all partials delivered
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
  if (warp < 2 || abort_s) return;

  // ---- final pass: this CTA owns rows [crank * TOK, (crank + 1) * TOK) of the block ----
  const int et = threadIdx.x - 64;  // 0..511
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = et + i * 512;
    const int tl = e / 128, nl = e % 128;
    const int tok = m0 + crank * TOK + tl;
    if (tok >= n_rows) continue;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int r = 0; r < CL; ++r) {
      s0 += part[(size_t)(r * TOK + tl) * kStride + nl];
      if (DUAL) s1 += part[(size_t)(r * TOK + tl) * kStride + 128 + nl];
    }
    const int f = a_row + nl;
    if (DUAL) {
      const float g = s0 + (bias != nullptr ? bias[f] : 0.f);
      float h = 0.f;
      if (g > 0.f)
        h = __bfloat162float(__float2bfloat16_rn(g)) * __bfloat162float(__float2bfloat16_rn(s1));
      out[(size_t)tok * ld_out + f] = __float2bfloat16_rn(h);
    } else {
      const int rid = row_ids != nullptr ? row_ids[tok] : tok;
      out[(size_t)rid * ld_out + f] = __float2bfloat16_rn(s0);
    }
  }
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Persistent form of the same GEMM: one CTA per SM walks the (feature tile, token tile) list
// with a stride of the grid, feature tile fastest, so the CTAs of a wave share one token tile.
// TMEM holds two accumulator pairs (4 x NTOK columns): while the epilogue warps drain pair a
// of tile i, the MMA thread already fills pair a^1 with tile i + 1, and the producer keeps
// the shared-memory ring full across tile boundaries (one running stage counter).
//   full / empty      : ring stages, as in the one-tile kernel;
//   tfull[a]          : tcgen05.commit after the last k-step of a tile -> epilogue may read pair a;
//   tempty[a]         : one epilogue thread arrives after all four warps have read pair a.
// The grid is sized by the host for the capacity; the token-tile count comes from the
// device-side row count, so no CTA is launched per empty tile.
template <int NTOK, int STAGES, int NBUF, bool DUAL>
__global__ void __launch_bounds__(kThreadsTc, NBUF == 1 ? 2 : 1)
dense_rows_gemm_persistent_kernel(const __grid_constant__ CUtensorMap tmap_a0,
                                  const __grid_constant__ CUtensorMap tmap_a1,
                                  const __grid_constant__ CUtensorMap tmap_b,
                                  const float* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                  const int* __restrict__ row_ids,
                                  const int* __restrict__ n_rows_ptr, int n_rows_host, int K,
                                  int ld_out, int feature_tiles) {
  constexpr int kBTileBytes = NTOK * 128;
  constexpr int kStageBytes = 2 * kATileBytes + kBTileBytes;
  constexpr uint32_t kTmemCols = 2 * NTOK * NBUF;  // NBUF accumulator pairs
  static_assert(kTmemCols <= 512, "TMEM has 512 columns");
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);

  const int n_rows = n_rows_ptr != nullptr ? *n_rows_ptr : n_rows_host;
  const int token_tiles = (n_rows + NTOK - 1) / NTOK;
  const int total = feature_tiles * token_tiles;
  if ((int)blockIdx.x >= total) return;  // uniform for the CTA: nothing allocated yet

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ksteps = K / kStageK;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 1);
    }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      uint32_t it = 0;  // ring position, running across tiles
      for (int t = blockIdx.x; t < total && !abort_s; t += gridDim.x) {
        const int ft = t % feature_tiles, m0 = (t / feature_tiles) * NTOK;
        const int a0_row = DUAL ? ft * 128 : ft * 256;
        const int a1_row = DUAL ? ft * 128 : ft * 256 + 128;
        for (int k = 0; k < ksteps; ++k, ++it) {
          const int s = (int)(it % STAGES);
          const uint32_t phase = (it / STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
            abort_s = 1;
            atomicExch(&g_dense_error, 1);
            break;
          }
          unsigned char* st = smem + (size_t)s * kStageBytes;
          mbar_expect_tx(&full_bar[s], (uint32_t)kStageBytes);
          tma_load_2d(st, &tmap_a0, k * kStageK, a0_row, &full_bar[s]);
          tma_load_2d(st + kATileBytes, DUAL ? &tmap_a1 : &tmap_a0, k * kStageK, a1_row,
                      &full_bar[s]);
          tma_load_2d(st + 2 * kATileBytes, &tmap_b, k * kStageK, m0, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      uint32_t it = 0;
      int i = 0;
      for (int t = blockIdx.x; t < total && !abort_s; t += gridDim.x, ++i) {
        const int a = i % NBUF;
        const uint32_t use = (uint32_t)(i / NBUF);
        if (!mbar_wait(&tempty_bar[a], (use & 1u) ^ 1u)) {  // epilogue has drained this pair
          abort_s = 1;
          atomicExch(&g_dense_error, 4);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc0 = tmem_base + (uint32_t)(a * 2 * NTOK);
        for (int k = 0; k < ksteps; ++k, ++it) {
          const int s = (int)(it % STAGES);
          const uint32_t phase = (it / STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], phase)) {
            abort_s = 1;
            atomicExch(&g_dense_error, 2);
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes);
          const uint64_t da0 = umma_desc(sa), da1 = umma_desc(sa + kATileBytes),
                         db = umma_desc(sa + 2 * kATileBytes);
#pragma unroll
          for (int kk = 0; kk < kStageK / 16; ++kk) {
            const uint32_t acc = (k > 0 || kk > 0) ? 1u : 0u;
            umma_bf16(acc0, da0 + 2 * kk, db + 2 * kk, kIdesc, acc);
            umma_bf16(acc0 + NTOK, da1 + 2 * kk, db + 2 * kk, kIdesc, acc);
          }
          umma_commit(&empty_bar[s]);
        }
        if (abort_s) break;
        umma_commit(&tfull_bar[a]);  // both accumulators of this tile are complete
      }
    }
  } else {
    // ---- epilogue: warps 2..5 own TMEM lane quarters 2, 3, 0, 1 ----
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    int i = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x, ++i) {
      const int a = i % NBUF;
      const uint32_t use = (uint32_t)(i / NBUF);
      const int ft = t % feature_tiles, m0 = (t / feature_tiles) * NTOK;
      bool ok = mbar_wait(&tfull_bar[a], use & 1u);
      if (!ok) {
        abort_s = 1;
        atomicExch(&g_dense_error, 3);
      }
      if (!epi_barrier_and(ok)) break;  // the same decision in all 128 epilogue threads
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_addr =
          tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * 2 * NTOK);
      const int f0 = (DUAL ? ft * 128 : ft * 256) + q * 32 + lane;
      const float b0 = (DUAL && bias != nullptr) ? bias[f0] : 0.f;
      for (int tb = 0; tb < NTOK / 32; ++tb) {
        if (m0 + tb * 32 >= n_rows) break;
        float v0[32], v1[32];
        tmem_ld32(lane_addr + (uint32_t)(tb * 32), v0);
        tmem_ld32(lane_addr + (uint32_t)(NTOK + tb * 32), v1);
        if (DUAL) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int tok = m0 + tb * 32 + c;
            if (tok >= n_rows) break;
            const float g = v0[c] + b0;
            float h = 0.f;
            if (g > 0.f)
              h = __bfloat162float(__float2bfloat16_rn(g)) * __bfloat162float(__float2bfloat16_rn(v1[c]));
            out[(size_t)tok * ld_out + f0] = __float2bfloat16_rn(h);
          }
        } else {
          const int t_mine = m0 + tb * 32 + lane;
          const int rid = t_mine < n_rows ? (row_ids != nullptr ? row_ids[t_mine] : t_mine) : -1;
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int r = __shfl_sync(0xffffffffu, rid, c);
            if (r < 0) continue;
            __nv_bfloat16* orow = out + (size_t)r * ld_out;
            orow[f0] = __float2bfloat16_rn(v0[c]);
            orow[f0 + 128] = __float2bfloat16_rn(v1[c]);
          }
        }
      }
      // all four warps have read the pair: hand it back to the MMA thread
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      epi_barrier();
      if (et == 0) mbar_arrive(&tempty_bar[a]);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

// ---- workspace ------------------------------------------------------------------
struct DenseWs {
  unsigned char* flags;  // [M]
  int* rows;             // [cap]
  int* counters;         // [4]
  __nv_bfloat16* xd;     // [cap_pad, D]
  __nv_bfloat16* hd;     // [cap_pad, H]
  size_t total;
};

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

DenseWs dense_ws_layout(void* base, int64_t M, int64_t D, int64_t H, int64_t cap) {
  const int64_t cap_pad = (cap + kDenseTok - 1) / kDenseTok * kDenseTok;
  unsigned char* p = static_cast<unsigned char*>(base);
  DenseWs w;
  size_t off = 0;
  w.flags = p + off;
  off += align256((size_t)M);
  w.rows = reinterpret_cast<int*>(p + off);
  off += align256((size_t)cap * 4);
  w.counters = reinterpret_cast<int*>(p + off);
  off += 256;
  w.xd = reinterpret_cast<__nv_bfloat16*>(p + off);
  off += align256((size_t)cap_pad * D * 2);
  w.hd = reinterpret_cast<__nv_bfloat16*>(p + off);
  off += align256((size_t)cap_pad * H * 2);
  w.total = off;
  return w;
}

// Persistent form: NBUF accumulator pairs per CTA; one CTA per SM with two pairs and a deep
// ring, or two CTAs per SM with one pair and two stages each.
template <int STAGES, int NBUF, bool DUAL>
int launch_persistent(const CUtensorMap& map_a0, const CUtensorMap& map_a1, const CUtensorMap& map_b,
                      const float* bias, void* out, const int* row_ids, const int* n_rows_ptr,
                      int64_t cap, int64_t K, int64_t ld_out, int feature_tiles, int64_t tiles_max,
                      cudaStream_t stream) {
  const size_t smem = (size_t)STAGES * (2 * kATileBytes + kDenseTok * 128) + 1024;
  auto kern = dense_rows_gemm_persistent_kernel<kDenseTok, STAGES, NBUF, DUAL>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_gated_t2d_hybrid")) return rc;
  const int64_t slots = (int64_t)sm_count() * (NBUF == 1 ? 2 : 1);
  const int ctas = (int)(tiles_max < slots ? tiles_max : slots);
  kern<<<ctas, kThreadsTc, smem, stream>>>(map_a0, map_a1, map_b, bias,
                                           static_cast<__nv_bfloat16*>(out), row_ids, n_rows_ptr,
                                           (int)cap, (int)K, (int)ld_out, feature_tiles);
  return check_launch("b200_twell_gated_t2d_hybrid (dense rows, persistent)");
}

template <int CL, bool DUAL>
int launch_dense_splitk_cl(const void* a0, const void* a1, int64_t a_rows, const void* b,
                           int64_t b_rows, int64_t K, const float* bias, void* out,
                           const int* row_ids, int64_t ld_out, int64_t cap, cudaStream_t stream) {
  constexpr int STAGES = DUAL ? 4 : 5;
  CUtensorMap map_a0, map_a1, map_b;
  if (int rc = make_map(&map_a0, a0, a_rows, K, 128)) return rc;
  if (int rc = make_map(&map_a1, a1, a_rows, K, 128)) return rc;
  if (int rc = make_map(&map_b, b, b_rows, K, 128)) return rc;
  const size_t smem = (size_t)STAGES * ((DUAL ? 2 : 1) * kATileBytes + 128 * 128) + 1024;
  auto kern = dense_rows_gemm_splitk_kernel<CL, STAGES, DUAL>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_gated_t2d_hybrid")) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(a_rows / 128 * CL), (unsigned)((cap + 127) / 128), 1);
  cfg.blockDim = dim3(kThreadsDenseWide, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (CL == 8) {  // clusters of 8 of a 160-190 KB CTA: only a limited number is resident at once
    static int fit[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (fit[dev] == 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = -1;
      }
      fit[dev] = n;
    }
    if ((int64_t)cfg.gridDim.x / CL * cfg.gridDim.y > fit[dev])
      return fail(B200_EUNSUPPORTED, "dense rows (split-k): clusters of 8 do not fit one wave");
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_a0, map_a1, map_b, bias,
                                     static_cast<__nv_bfloat16*>(out), row_ids, (int)cap, (int)K,
                                     (int)ld_out);
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "b200_twell_gated_t2d_hybrid (dense rows, split-k): launch: %s",
                cudaGetErrorString(e));
  return B200_OK;
}

template <bool DUAL>
int launch_dense_splitk(int cl, const void* a0, const void* a1, int64_t a_rows, const void* b,
                        int64_t b_rows, int64_t K, const float* bias, void* out,
                        const int* row_ids, int64_t ld_out, int64_t cap, cudaStream_t stream) {
  if (cl == 8) {
    const int rc = launch_dense_splitk_cl<8, DUAL>(a0, a1, a_rows, b, b_rows, K, bias, out,
                                                   row_ids, ld_out, cap, stream);
    if (rc != B200_EUNSUPPORTED) return rc;
    cl = 4;
  }
  if (cl == 4)
    return launch_dense_splitk_cl<4, DUAL>(a0, a1, a_rows, b, b_rows, K, bias, out, row_ids,
                                           ld_out, cap, stream);
  return launch_dense_splitk_cl<2, DUAL>(a0, a1, a_rows, b, b_rows, K, bias, out, row_ids, ld_out,
                                         cap, stream);
}

template <bool DUAL>
int launch_dense_gemm(const void* a0, const void* a1, int64_t a_rows, const void* b,
                      int64_t b_rows, int64_t K, const float* bias, void* out, const int* row_ids,
                      const int* n_rows_ptr, int64_t ld_out, int64_t cap, cudaStream_t stream) {
  // cap: rows the grid covers; without a device-side count (n_rows_ptr == NULL) all of them
  CUtensorMap map_a0, map_a1, map_b;
  if (int rc = make_map(&map_a0, a0, a_rows, K, 128)) return rc;
  if (int rc = make_map(&map_a1, a1, a_rows, K, 128)) return rc;
  if (int rc = make_map(&map_b, b, b_rows, K, kDenseTok)) return rc;
  // Which form.  Measured on B200, all three products, TFLOP/s at (M, D, H) =
  // (2048, 2048, 11008) / (16384, 2048, 11008) / (2048, 4096, 16384) / (16384, 4096, 16384):
  //   one-tile CTAs, two per SM              858 / 1118 / 1148 / 1108
  //   persistent, two accumulator pairs      921 / 1042 /  896 /  893   (one CTA per SM)
  //   persistent, one pair, two CTAs per SM  852 / 1041 / 1127 / 1069
  // All are bound by the L2 -> SM operand stream, which is latency-bound (about 1.3 us times
  // the bytes in flight per SM: 49 GB/s per SM with 64 KB in flight, 94-112 GB/s with 128 KB),
  // and two CTAs per SM keep more loads in flight than one ring.  The one-tile form is used when
  // the host knows the row count; when the count lives on the device (routing) the
  // persistent two-CTA form is used, because it launches no CTA per empty tile.
  const int feature_tiles = (int)(a_rows / (DUAL ? 128 : 256));
  const int64_t tiles_max = (int64_t)feature_tiles * ((cap + kDenseTok - 1) / kDenseTok);
  int form = B200_DENSE_PERSISTENT;  // 0 one-tile CTAs, 1 persistent x 2 accumulator pairs,
                                     // 2 persistent x 1 pair, two CTAs per SM
  if (form < 0) form = (n_rows_ptr != nullptr) ? 2 : 0;
  if (form == 1)
    return launch_persistent<4, 2, DUAL>(map_a0, map_a1, map_b, bias, out, row_ids, n_rows_ptr, cap,
                                         K, ld_out, feature_tiles, tiles_max, stream);
  if (form == 2)
    return launch_persistent<2, 1, DUAL>(map_a0, map_a1, map_b, bias, out, row_ids, n_rows_ptr, cap,
                                         K, ld_out, feature_tiles, tiles_max, stream);
  // Stage depth in K of the one-tile form: 64 k-values x 2 stages, or (B200_DENSE_KS=32)
  // 32 x 4 in the same shared memory with 64-byte swizzle.  The finer stages keep more bytes
  // in flight but double the barrier round trips of the single MMA-issuing thread: measured
  // 861 vs 1107 TFLOP/s at M = 16384, D = 2048, H = 11008, so 64 stays the default.
  constexpr int KS = B200_DENSE_KS;
  constexpr int STAGES = kDenseStages * (64 / KS);
  if (KS != 64) {
    if (int rc = make_map(&map_a0, a0, a_rows, K, 128, KS)) return rc;
    if (int rc = make_map(&map_a1, a1, a_rows, K, 128, KS)) return rc;
    if (int rc = make_map(&map_b, b, b_rows, K, kDenseTok, KS)) return rc;
  }
  // Host-known row count of at most 512: split-k over a cluster, 128 features x 128 rows per
  // tile (B200_DENSE_SPLITK=0 switches it off).  The largest cluster whose grid is one wave;
  // two CTAs per tile are also taken when that needs two waves.
  static const bool splitk_on = [] {
    const char* e = getenv("B200_DENSE_SPLITK");
    return e == nullptr || atoi(e) != 0;
  }();
  if (KS == 64 && splitk_on && n_rows_ptr == nullptr && cap <= 512) {
    const int64_t tiles128 = a_rows / 128, blocks = (cap + 127) / 128;
    const int sms = sm_count();
    int cl = 0;
    for (int c : {8, 4, 2})
      if (cl == 0 && tiles128 * c * blocks <= sms && K % (c * 64) == 0 && K / c >= 256) cl = c;
    if (cl == 0 && tiles128 * 2 * blocks <= 2 * sms && K % 128 == 0 && K >= 512) cl = 2;
    if (cl != 0) {
      const int rc = launch_dense_splitk<DUAL>(cl, a0, a1, a_rows, b, b_rows, K, bias, out, row_ids,
                                               ld_out, cap, stream);
      if (rc != B200_EUNSUPPORTED) return rc;
    }
  }
  // Host-known row count and enough 256-token tiles to fill the GPU: one CTA per SM on
  // 256-token tiles with sixteen epilogue warps (B200_DENSE_WIDE=0 keeps the 128-token tiles).
  static const bool wide_on = [] {
    const char* e = getenv("B200_DENSE_WIDE");
    return e == nullptr || atoi(e) != 0;
  }();
  const int64_t wide_ctas = (int64_t)feature_tiles * ((cap + 255) / 256);
  if (KS == 64 && wide_on && n_rows_ptr == nullptr && wide_ctas * 5 >= (int64_t)sm_count() * 4) {
    CUtensorMap map_b256;
    if (int rc = make_map(&map_b256, b, b_rows, K, 256)) return rc;
    constexpr int WST = 3;
    const size_t smem_w = (size_t)WST * (2 * kATileBytes + 256 * 128) + 1024;
    auto wide = dense_rows_gemm_wide_kernel<WST, DUAL>;
    static size_t granted_w[64] = {0};
    if (int rc = ensure_dynamic_smem(wide, smem_w, granted_w, "b200_twell_gated_t2d_hybrid"))
      return rc;
    dim3 wgrid((unsigned)feature_tiles, (unsigned)((cap + 255) / 256), 1);
    wide<<<wgrid, kThreadsDenseWide, smem_w, stream>>>(
        map_a0, map_a1, map_b256, bias, static_cast<__nv_bfloat16*>(out), row_ids, (int)cap,
        (int)K, (int)ld_out,
        raster_group((DUAL ? 2 : 1) * a_rows * K * 2, (int64_t)256 * K * 2));
    return check_launch("b200_twell_gated_t2d_hybrid (dense rows, 256-token tiles)");
  }
  dim3 grid((unsigned)(a_rows / (DUAL ? 128 : 256)), (unsigned)((cap + kDenseTok - 1) / kDenseTok), 1);
  // A grid of at most one CTA per SM (the weight-gradient products at d_model 1024: 128
  // tiles with K = all tokens) gets a ring twice as deep: the second co-resident CTA that
  // would otherwise double the bytes in flight does not exist there.
  static const bool deep_ring = [] {
    const char* e = getenv("B200_DENSE_DEEP_RING");
    return e == nullptr || atoi(e) != 0;
  }();
  if (KS == 64 && deep_ring && (int64_t)grid.x * grid.y <= (int64_t)sm_count()) {
    constexpr int DEEP = 2 * kDenseStages;
    const size_t smem_deep = (size_t)DEEP * (2 * 128 * 64 * 2 + kDenseTok * 64 * 2) + 1024;
    auto deep = dense_rows_gemm_kernel<kDenseTok, DEEP, DUAL, 64>;
    static size_t granted_deep[64] = {0};
    if (int rc = ensure_dynamic_smem(deep, smem_deep, granted_deep, "b200_twell_gated_t2d_hybrid"))
      return rc;
    deep<<<grid, kThreadsTc, smem_deep, stream>>>(map_a0, map_a1, map_b, bias,
                                                  static_cast<__nv_bfloat16*>(out), row_ids,
                                                  n_rows_ptr, (int)cap, (int)K, (int)ld_out, 1);
    return check_launch("b200_twell_gated_t2d_hybrid (dense rows, deep ring)");
  }
  const size_t smem = (size_t)STAGES * (2 * 128 * KS * 2 + kDenseTok * KS * 2) + 1024;
  auto kern = dense_rows_gemm_kernel<kDenseTok, STAGES, DUAL, KS>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_gated_t2d_hybrid")) return rc;
  kern<<<grid, kThreadsTc, smem, stream>>>(map_a0, map_a1, map_b, bias,
                                           static_cast<__nv_bfloat16*>(out), row_ids, n_rows_ptr,
                                           (int)cap, (int)K, (int)ld_out,
                                           raster_group((DUAL ? 2 : 1) * a_rows * K * 2,
                                                        (int64_t)kDenseTok * K * 2));
  return check_launch("b200_twell_gated_t2d_hybrid (dense rows)");
}

// ---- weight-gradient products of the training operator on the tensor cores ------------
// out[H, D] = vals^T . rows, with vals a slab-shaped sparse [M, H] operand and rows a dense
// [M, D] matrix: a reduction over all M tokens with a dense result, i.e. GEMM-shaped.  The
// slab is scattered into a zero-filled K-major matrix vals_T [H, Mp], rows is transposed to
// rows_T [D, Mp], and the one-tile GEMM above computes out[h, d] = sum_m rows_T[d, m] *
// vals_T[h, m] (features = D on the TMEM lanes, "tokens" = H on the columns).

// rows [M, D] -> rows_T [D, Mp], columns M..Mp-1 zero.  32 x 32 tiles through shared memory.
__global__ void __launch_bounds__(256)
transpose_pad_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int M,
                     int D, int Mp) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int m0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
  for (int r = ty; r < 32; r += 8) {
    const int m = m0 + r;
    tile[r][tx] = (m < M) ? in[(size_t)m * D + d0 + tx] : __float2bfloat16(0.f);
  }
  __syncthreads();
#pragma unroll
  for (int r = ty; r < 32; r += 8) {
    const int m = m0 + tx;
    if (m < Mp) out[(size_t)(d0 + r) * Mp + m] = tile[tx][r];
  }
}

// One warp per token row: vals_T[col, row] = value for every stored entry of the row.
__global__ void __launch_bounds__(256)
scatter_slab_transposed_kernel(const uint32_t* __restrict__ slab, __nv_bfloat16* __restrict__ vals_t,
                               int M, int tiles, int slab_w, int Mp) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const uint32_t* prow = slab + (size_t)row * tiles * slab_w;
  for (int t = 0; t < tiles; ++t) {
    const uint32_t* s = prow + (size_t)t * slab_w;
    const int n = min(max((int)s[0], 0), slab_w - 1);
    for (int e = lane; e < n; e += 32) {
      const uint32_t w = s[1 + e];
      vals_t[(size_t)(w & 0xFFFFu) * Mp + row] = __ushort_as_bfloat16((unsigned short)(w >> 16));
    }
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_hybrid_wgrad_workspace_bytes(int64_t M, int64_t D, int64_t H) {
  if (M <= 0 || D <= 0 || H <= 0) return 0;
  const int64_t Mp = (M + 63) / 64 * 64;
  return align256((size_t)D * Mp * 2) + align256((size_t)H * Mp * 2);
}

int b200_hybrid_wgrad_dense(const void* vals_slab, const void* rows, void* out, int64_t M,
                            int64_t D, int64_t H, int cf, int reuse_rows_t, void* ws,
                            size_t ws_bytes, void* stream) {
  const char* fn = "b200_hybrid_wgrad_dense";
  if (int rc = check_dims(fn, M, D, H, cf)) return rc;
  if (M == 0) return fail(B200_EINVAL, "%s: M must be > 0", fn);
  if (M > (int64_t)1 << 22) return fail(B200_EUNSUPPORTED, "%s: M > 2^22 rows", fn);
  const void* ptrs[4] = {vals_slab, rows, out, ws};
  const char* names[4] = {"vals_slab", "rows", "out", "ws"};
  for (int i = 0; i < 4; ++i) {
    if (ptrs[i] == nullptr) return fail(B200_ENULL, "%s: %s is NULL", fn, names[i]);
    if (!aligned16(ptrs[i])) return fail(B200_EALIGN, "%s: %s is not 16-byte aligned", fn, names[i]);
  }
  if (reinterpret_cast<uintptr_t>(ws) & 255u)
    return fail(B200_EALIGN, "%s: ws is not 256-byte aligned", fn);
  if (ws_bytes < b200_hybrid_wgrad_workspace_bytes(M, D, H))
    return fail(B200_EWORKSPACE, "%s: ws holds %zu bytes, %zu needed", fn, ws_bytes,
                b200_hybrid_wgrad_workspace_bytes(M, D, H));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t Mp = (M + 63) / 64 * 64;
  __nv_bfloat16* rows_t = static_cast<__nv_bfloat16*>(ws);
  __nv_bfloat16* vals_t = reinterpret_cast<__nv_bfloat16*>(static_cast<unsigned char*>(ws) +
                                                          align256((size_t)D * Mp * 2));
  if (!reuse_rows_t) {
    dim3 grid((unsigned)((Mp + 31) / 32), (unsigned)(D / 32), 1);
    transpose_pad_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(rows), rows_t,
                                               (int)M, (int)D, (int)Mp);
  }
  cudaError_t e = cudaMemsetAsync(vals_t, 0, (size_t)H * Mp * 2, st);
  if (e != cudaSuccess) return fail(B200_ECUDA, "%s: cudaMemsetAsync: %s", fn, cudaGetErrorString(e));
  scatter_slab_transposed_kernel<<<(unsigned)((M + 7) / 8), 256, 0, st>>>(
      static_cast<const uint32_t*>(vals_slab), vals_t, (int)M, (int)(H / kTileN), kTileN / cf,
      (int)Mp);
  if (int rc = check_launch(fn)) return rc;
  return launch_dense_gemm<false>(rows_t, rows_t, D, vals_t, H, Mp, nullptr, out, nullptr, nullptr,
                                  D, H, st);
}

size_t b200_twell_hybrid_workspace_bytes(int64_t M, int64_t D, int64_t H, int64_t dense_cap) {
  if (M <= 0 || D <= 0 || H <= 0 || dense_cap <= 0) return 0;
  return dense_ws_layout(nullptr, M, D, H, dense_cap).total;
}

int b200_twell_gated_t2d_hybrid(const void* x, const void* packed, const void* gate,
                                const float* gate_bias, const void* up, const void* down,
                                const void* down_t, void* out, int64_t M, int64_t D, int64_t H,
                                int cf, uint32_t flags, int64_t nnz_threshold, int64_t dense_cap,
                                void* hybrid_ws, size_t hybrid_ws_bytes, void* workspace,
                                size_t workspace_bytes, void* stream) {
  const char* fn = "b200_twell_gated_t2d_hybrid";
  if (int rc = check_dims(fn, M, D, H, cf)) return rc;
  if (flags & ~B200_FLAG_HIGH_PRECISION) return fail(B200_EINVAL, "%s: unknown flags 0x%x", fn, flags);
  if (dense_cap <= 0 || nnz_threshold < 0)
    return fail(B200_EINVAL, "%s: need dense_cap > 0 and nnz_threshold >= 0", fn);
  if (M == 0) return B200_OK;
  if (M > (int64_t)1 << 20) return fail(B200_EUNSUPPORTED, "%s: M > 2^20 rows", fn);
  if (dense_cap > M) dense_cap = M;
  const void* ptrs[8] = {x, packed, gate, up, down, down_t, out, hybrid_ws};
  const char* names[8] = {"x", "packed", "gate", "up", "down", "down_t", "out", "hybrid_ws"};
  for (int i = 0; i < 8; ++i) {
    if (ptrs[i] == nullptr) return fail(B200_ENULL, "%s: %s is NULL", fn, names[i]);
    if (!aligned16(ptrs[i])) return fail(B200_EALIGN, "%s: %s is not 16-byte aligned", fn, names[i]);
  }
  if (reinterpret_cast<uintptr_t>(hybrid_ws) & 255u)
    return fail(B200_EALIGN, "%s: hybrid_ws is not 256-byte aligned", fn);
  DenseWs w = dense_ws_layout(hybrid_ws, M, D, H, dense_cap);
  if (hybrid_ws_bytes < w.total)
    return fail(B200_EWORKSPACE, "%s: hybrid_ws holds %zu bytes, %zu needed", fn, hybrid_ws_bytes,
                w.total);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int tiles = (int)(H / kTileN), slab_w = kTileN / cf;
  const int64_t cap_pad = (dense_cap + kDenseTok - 1) / kDenseTok * kDenseTok;

  route_flags_kernel<<<(unsigned)((M + 7) / 8), 256, 0, st>>>(
      static_cast<const uint32_t*>(packed), (int)M, tiles, slab_w,
      (int)(nnz_threshold > 0x7fffffff ? 0x7fffffff : nnz_threshold), w.flags);
  route_compact_kernel<<<1, 1024, 0, st>>>(w.flags, (int)M, (int)dense_cap, w.rows, w.counters);
  if (int rc = check_launch(fn)) return rc;
  if (int rc = twell_t2d_launch(true, (flags & B200_FLAG_HIGH_PRECISION) != 0, x, packed, up, down,
                                out, M, D, H, cf, workspace, workspace_bytes, sm_count(), st,
                                w.flags, nullptr))
    return rc;
  gather_rows_kernel<<<(unsigned)dense_cap, 256, 0, st>>>(
      static_cast<const uint4*>(x), w.rows, w.counters, reinterpret_cast<uint4*>(w.xd),
      (int)(D / 8));
  if (int rc = check_launch(fn)) return rc;
  if (int rc = launch_dense_gemm<true>(gate, up, H, w.xd, cap_pad, D, gate_bias, w.hd, nullptr,
                                       w.counters, H, dense_cap, st))
    return rc;
  return launch_dense_gemm<false>(down_t, down_t, D, w.hd, cap_pad, H, nullptr, out, w.rows,
                                  w.counters, D, dense_cap, st);
}

int b200_twell_gated_mlp_hybrid(const void* x, const void* gate, const float* gate_bias,
                                const void* up, const void* down, const void* down_t,
                                void* packed, void* out, int64_t M, int64_t D, int64_t H, int cf,
                                uint32_t flags, int64_t nnz_threshold, int64_t dense_cap,
                                void* hybrid_ws, size_t hybrid_ws_bytes, void* workspace,
                                size_t workspace_bytes, void* stream) {
  if (int rc = b200_twell_pack(x, gate, gate_bias, packed, M, D, H, cf, stream)) return rc;
  return b200_twell_gated_t2d_hybrid(x, packed, gate, gate_bias, up, down, down_t, out, M, D, H,
                                     cf, flags, nnz_threshold, dense_cap, hybrid_ws,
                                     hybrid_ws_bytes, workspace, workspace_bytes, stream);
}

/* Every row on the dense route, without slab, routing or gather: Hd = relu(x Wg^T + b) *
 * (x Wu^T) into h_ws [M, H] bf16 (caller scratch), then out = Hd Wd via down_t [D, H]. */
int b200_dense_gated_mlp(const void* x, const void* gate, const float* gate_bias, const void* up,
                         const void* down_t, void* h_ws, void* out, int64_t M, int64_t D,
                         int64_t H, void* stream) {
  const char* fn = "b200_dense_gated_mlp";
  if (int rc = check_dims(fn, M, D, H, 8)) return rc;
  if (M == 0) return B200_OK;
  if (M > (int64_t)1 << 20) return fail(B200_EUNSUPPORTED, "%s: M > 2^20 rows", fn);
  const void* ptrs[6] = {x, gate, up, down_t, h_ws, out};
  const char* names[6] = {"x", "gate", "up", "down_t", "h_ws", "out"};
  for (int i = 0; i < 6; ++i) {
    if (ptrs[i] == nullptr) return fail(B200_ENULL, "%s: %s is NULL", fn, names[i]);
    if (!aligned16(ptrs[i])) return fail(B200_EALIGN, "%s: %s is not 16-byte aligned", fn, names[i]);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Token tiles past M read zero-filled TMA rows and store nothing.
  if (int rc = launch_dense_gemm<true>(gate, up, H, x, M, D, gate_bias, h_ws, nullptr, nullptr, H,
                                       M, st))
    return rc;
  return launch_dense_gemm<false>(down_t, down_t, D, h_ws, M, H, nullptr, out, nullptr, nullptr, D,
                                  M, st);
}

/* counters_out[0] = rows routed to the dense path by the last call on this workspace,
 * [1] = overflowed rows left on the sparse path (capacity exhausted), [2] = rows that
 * qualified.  Synchronises the device. */
int b200_twell_hybrid_counters(const void* hybrid_ws, int64_t M, int64_t D, int64_t H,
                               int64_t dense_cap, int* counters_out) {
  if (hybrid_ws == nullptr || counters_out == nullptr || M <= 0 || dense_cap <= 0) return B200_EINVAL;
  if (dense_cap > M) dense_cap = M;
  DenseWs w = dense_ws_layout(const_cast<void*>(hybrid_ws), M, D, H, dense_cap);
  if (cudaMemcpy(counters_out, w.counters, 3 * sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return fail(B200_ECUDA, "b200_twell_hybrid_counters: copy failed");
  return B200_OK;
}

/* Error word raised by a bounded wait that gave up in the dense GEMMs (0 = none).  Reads and
 * clears it; synchronises the device. */
int b200_twell_hybrid_status(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_dense_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_dense_error, &zero, sizeof(int));
  return v;
}

}  // extern "C"
