// Gate projection + ReLU + TwELL pack on the 5th-generation tensor cores.
//
// Kernels of this file, by token count: twell_pack_tc_splitk_(wide_)kernel (17..32 tokens, D
// split over a cluster), twell_pack_tc_splitk_mid_kernel (33..256, 128-token tiles, D split),
// twell_pack_tc_wide_kernel (256-token tiles, one CTA per SM, sixteen epilogue warps: the
// default above that) and twell_pack_tc_kernel, described first (64- / 128-token tiles, four
// epilogue warps).
//
// CTA tile: one 256-neuron TwELL tile x NTOK tokens (64 or 128) x all of D.
// Neurons ride the MMA M axis as two 128-row accumulators, tokens the N axis:
//   D0[128, NTOK] = W[tile*256      .. +128, :] . X[tok0 .. +NTOK, :]^T
//   D1[128, NTOK] = W[tile*256 + 128 .. +128, :] . X[tok0 .. +NTOK, :]^T
// Operands are K-major bf16 tiles of 64 k-values (128 bytes per row), brought in by
// TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) into a ring of shared
// memory stages; one elected thread issues tcgen05.mma (kind::f16, fp32 accumulate
// in TMEM); tcgen05.commit releases a stage back to the producer and, after the
// last k step, hands the accumulators to four epilogue warps.
//
// In TMEM a lane is a neuron and a column is a token, so after tcgen05.ld the 32
// lanes of an epilogue warp hold 32 consecutive neurons of one token per register:
// __ballot_sync gives the tile's positives in ascending neuron order, __popc the
// slot.  Eight (accumulator, warp) chunks per token are stitched by an exclusive
// prefix in shared memory.  Deterministic; same slab bytes as the small-M kernel.
//
// Every mbarrier wait is bounded: when a wait gives up, the CTA raises an error word
// (read with b200_twell_pack_tc_status), skips the rest of its work, frees its TMEM
// and returns.
//
// Replaces mm_wgmma_nt_kernel (custom_models/twell_modules/matmul_d2t.cu:287-709):
// wgmma -> tcgen05.mma, register accumulators -> TMEM, multicast TMA -> per-CTA TMA,
// shared-memory atomics in the epilogue -> ballot/popc.
#include <cooperative_groups.h>

#include <cstdlib>

#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

__device__ int g_tc_error = 0;

// grid = (H / 256, ceil(M / NTOK)).  Dynamic shared memory: STAGES x (A0 | A1 | B), 1024-aligned.
template <int NTOK, int STAGES, int MINB>
__global__ void __launch_bounds__(kThreadsTc, MINB)
twell_pack_tc_kernel(const __grid_constant__ CUtensorMap tmap_w,
                     const __grid_constant__ CUtensorMap tmap_x, const float* __restrict__ bias,
                     uint32_t* __restrict__ packed, int M, int D, int slab_w, int row_words,
                     int group) {
  constexpr int kBTileBytes = NTOK * 128;
  constexpr int kStageBytes = 2 * kATileBytes + kBTileBytes;
  constexpr uint32_t kTmemCols = 2 * NTOK;  // 128 or 256: a power of two >= 32
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_s;
  __shared__ uint32_t masks_s[32][8];
  __shared__ int prefix_s[32][8];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int tile, mblk;
  raster_remap(group, tile, mblk);
  const int m0 = mblk * NTOK;
  const int ksteps = D / kStageK;

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
    // ---- TMA producer ----
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
          abort_s = 1;
          atomicExch(&g_tc_error, 1);
          break;
        }
        unsigned char* st = smem + (size_t)s * kStageBytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)kStageBytes);
        tma_load_2d(st, &tmap_w, k * kStageK, tile * kTileN, &full_bar[s]);
        tma_load_2d(st + kATileBytes, &tmap_w, k * kStageK, tile * kTileN + 128, &full_bar[s]);
        tma_load_2d(st + 2 * kATileBytes, &tmap_x, k * kStageK, m0, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) {
          abort_s = 1;
          atomicExch(&g_tc_error, 2);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a0 = smem_u32(smem + (size_t)s * kStageBytes);
        const uint64_t da0 = umma_desc(a0), da1 = umma_desc(a0 + kATileBytes),
                       db = umma_desc(a0 + 2 * kATileBytes);
#pragma unroll
        for (int kk = 0; kk < kStageK / 16; ++kk) {
          const uint32_t acc = (k > 0 || kk > 0) ? 1u : 0u;
          // +32 bytes per 16 k-values inside the 128-byte swizzled row (encoded >> 4)
          umma_bf16(tmem_base, da0 + 2 * kk, db + 2 * kk, kIdesc, acc);
          umma_bf16(tmem_base + NTOK, da1 + 2 * kk, db + 2 * kk, kIdesc, acc);
        }
        umma_commit(&empty_bar[s]);  // stage reusable once these MMAs have read it
      }
      if (!abort_s) umma_commit(&acc_bar);  // accumulators complete
    }
  } else {
    // ---- epilogue: warps 2..5 own TMEM lane quarters 2, 3, 0, 1 ----
    const int q = warp & 3;
    const int et = threadIdx.x - 64;  // 0..127
    bool ok = mbar_wait(&acc_bar, 0u);
    if (!ok) {
      abort_s = 1;
      atomicExch(&g_tc_error, 3);
    }
    ok = epi_barrier_and(ok);  // the same decision in all 128 epilogue threads
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int n_lo = tile * kTileN + q * 32 + lane;  // neuron of accumulator 0; +128 for 1
    const float b_lo = bias != nullptr ? bias[n_lo] : 0.f;
    const float b_hi = bias != nullptr ? bias[n_lo + 128] : 0.f;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    for (int tb = 0; tb < NTOK / 32 && ok; ++tb) {
      float v0[32], v1[32];
      tmem_ld32(lane_addr + (uint32_t)(tb * 32), v0);
      tmem_ld32(lane_addr + (uint32_t)(NTOK + tb * 32), v1);
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const bool valid = m0 + tb * 32 + c < M;
        v0[c] += b_lo;
        v1[c] += b_hi;
        const uint32_t k0 = __ballot_sync(0xffffffffu, valid && v0[c] > 0.f);
        const uint32_t k1 = __ballot_sync(0xffffffffu, valid && v1[c] > 0.f);
        if (lane == 0) {
          masks_s[c][q] = k0;
          masks_s[c][4 + q] = k1;
        }
      }
      epi_barrier();
      if (et < 32) {
        const int tok = m0 + tb * 32 + et;
        int run = 0;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          prefix_s[et][ch] = run;
          run += __popc(masks_s[et][ch]);
        }
        if (tok < M) packed[(size_t)tok * row_words + (size_t)tile * slab_w] = (uint32_t)run;
      }
      epi_barrier();
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int tok = m0 + tb * 32 + c;
        uint32_t* slab = packed + (size_t)tok * row_words + (size_t)tile * slab_w;
        const uint32_t k0 = masks_s[c][q], k1 = masks_s[c][4 + q];
        if ((k0 >> lane) & 1u) {
          const int slot = prefix_s[c][q] + __popc(k0 & lanemask_lt());
          if (slot < slab_w - 1) slab[1 + slot] = (uint32_t)n_lo | (bf16_bits(v0[c]) << 16);
        }
        if ((k1 >> lane) & 1u) {
          const int slot = prefix_s[c][4 + q] + __popc(k1 & lanemask_lt());
          if (slot < slab_w - 1) slab[1 + slot] = (uint32_t)(n_lo + 128) | (bf16_bits(v1[c]) << 16);
        }
      }
      epi_barrier();  // masks_s / prefix_s are rewritten by the next token block
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

// ---------------------------------------------------------------------------
// Decode variant (M <= 32): the same TMA -> tcgen05 pipeline, with the reduction
// dimension split over a cluster of CL CTAs so that (H/256)*CL CTAs stream W_gate
// concurrently.  CTA `crank` multiplies all 256 neurons of the tile by its slice of D for
// up to 32 tokens; the partial accumulators leave TMEM through registers and are pushed
// (distributed shared memory) to the CTA that finalises each token, which adds the CL
// partials in rank order and compacts with ballot / popc.
// grid = ((H/256) * CL, ceil(M / 32)), cluster = CL.
// Dynamic shared memory: STAGES x (A0 | A1 | B) | partial sums [32][kPartStrideTc] fp32.
// ---------------------------------------------------------------------------
constexpr int kTokDecode = 32;
constexpr int kPartStrideTc = kTileN + 4;

template <int CL, int STAGES>
__global__ void __launch_bounds__(kThreadsTc, CL >= 8 ? 2 : 1)
twell_pack_tc_splitk_kernel(const __grid_constant__ CUtensorMap tmap_w,
                            const __grid_constant__ CUtensorMap tmap_x,
                            const float* __restrict__ bias, uint32_t* __restrict__ packed, int M,
                            int D, int slab_w, int row_words) {
  constexpr int NTOK = kTokDecode;
  constexpr int TOK = NTOK / CL;  // tokens finalised by this CTA
  constexpr int kBTileBytes = NTOK * 128;
  constexpr int kStageBytes = 2 * kATileBytes + kBTileBytes;
  constexpr uint32_t kTmemCols = 2 * NTOK;
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);
  constexpr int EPT = TOK * kTileN / 128;  // elements per epilogue thread in the final pass

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* part = reinterpret_cast<float*>(smem + (size_t)STAGES * kStageBytes);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_s;
  __shared__ int cnt_chunk[TOK][8];

  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  cluster.barrier_arrive();  // matched by barrier_wait() before the first remote store

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / CL;
  const int m0 = blockIdx.y * NTOK;
  const int kc = D / CL;
  const int ksteps = kc / kStageK;
  const int k_base = crank * kc;

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
  // Barriers, TMEM and the cluster hand-shake are set up; from here on the kernel reads x and
  // writes the slab, so the predecessor in the stream must have completed.
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
          abort_s = 1;
          atomicExch(&g_tc_error, 1);
          break;
        }
        unsigned char* st = smem + (size_t)s * kStageBytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)kStageBytes);
        const int kcoord = k_base + k * kStageK;
        // one copy for the tile's 256 weight rows (A0 | A1 are contiguous): a copy costs the
        // producer thread about 160 ns whatever its size
        tma_load_2d(st, &tmap_w, kcoord, tile * kTileN, &full_bar[s]);
        tma_load_2d(st + 2 * kATileBytes, &tmap_x, kcoord, m0, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) {
          abort_s = 1;
          atomicExch(&g_tc_error, 2);
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
    // ---- epilogue part 1: TMEM -> registers -> owner CTA's shared memory ----
    const int q = warp & 3;
    bool ok = mbar_wait(&acc_bar, 0u);
    if (!ok) {
      abort_s = 1;
      atomicExch(&g_tc_error, 3);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    cluster.barrier_wait();  // every CTA of the cluster is running
    if (ok) {
      const int nl = q * 32 + lane;  // neuron inside the tile (accumulator 0); +128 for 1
      const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
      float v0[32], v1[32];
      tmem_ld32(lane_addr, v0);
      tmem_ld32(lane_addr + (uint32_t)NTOK, v1);
#pragma unroll
      for (int c = 0; c < NTOK; ++c) {
        const int owner = c / TOK, tl = c % TOK;
        float* dst = cluster.map_shared_rank(part, owner) +
                     (size_t)(crank * TOK + tl) * kPartStrideTc + nl;
        dst[0] = v0[c];
        dst[128] = v1[c];
      }
    }
  }
  if (warp < 2) cluster.barrier_wait();  // pair the early arrive for the non-epilogue warps

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster.sync();  // all partials delivered (every thread of every CTA takes part)
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
  if (warp < 2 || abort_s) return;

  // ---- epilogue part 2: this CTA finalises tokens [crank*TOK, (crank+1)*TOK) ----
  const int et = threadIdx.x - 64;
  const int neuron0 = tile * kTileN;
  float z[EPT];
  uint32_t mask[EPT];
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = et + i * 128;
    const int tl = e / kTileN, nl = e % kTileN;
    const int tok = crank * TOK + tl;
    float v = 0.f;
#pragma unroll
    for (int r = 0; r < CL; ++r) v += part[(size_t)(r * TOK + tl) * kPartStrideTc + nl];
    if (bias != nullptr) v += bias[neuron0 + nl];
    const bool keep = (v > 0.f) && (m0 + tok < M);
    z[i] = v;
    mask[i] = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) cnt_chunk[tl][nl / 32] = __popc(mask[i]);
  }
  epi_barrier();
  if (et < TOK) {  // counts -> exclusive prefix over the 8 chunks of this token, count word
    int run = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int v = cnt_chunk[et][c];
      cnt_chunk[et][c] = run;
      run += v;
    }
    const int tok = m0 + crank * TOK + et;
    if (tok < M) packed[(size_t)tok * row_words + (size_t)tile * slab_w] = (uint32_t)run;
  }
  epi_barrier();
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = et + i * 128;
    const int tl = e / kTileN, nl = e % kTileN;
    const int tok = crank * TOK + tl;
    if (m0 + tok >= M) continue;
    uint32_t* slab = packed + (size_t)(m0 + tok) * row_words + (size_t)tile * slab_w;
    const int slot = cnt_chunk[tl][nl / 32] + __popc(mask[i] & lanemask_lt());
    if (((mask[i] >> lane) & 1u) && slot < slab_w - 1)
      slab[1 + slot] = (uint32_t)(neuron0 + nl) | (bf16_bits(z[i]) << 16);
  }
}

// ---------------------------------------------------------------------------
// Large-M kernel with sixteen epilogue warps: ONE CTA per SM computes 256 neurons x 256 tokens
// (two 128-lane accumulators of 256 columns = all of TMEM; a stage of 64 k-values is 32 KB of
// weights + 32 KB of tokens, i.e. 131 flop per staged byte against 87 for the 128-token tile),
// and the pack epilogue - which four warps need about 2 us per 32-token block for - is spread
// over four groups of four warps that each take every fourth token block.  The epilogue
// reads the accumulators twice (signs first, values again when the slots are known) so that a
// thread holds 32 instead of 64 of them.
// Threads: warp 0 producer, warp 1 mma, warps 2..17 epilogue (group = (warp - 2) / 4, TMEM
// lane quarter = warp % 4).  grid = (H / 256, ceil(M / 256)).
// ---------------------------------------------------------------------------
constexpr int kThreadsTcWideM = 64 + 512;

template <int STAGES>
__global__ void __launch_bounds__(kThreadsTcWideM, 1)
twell_pack_tc_wide_kernel(const __grid_constant__ CUtensorMap tmap_w,
                          const __grid_constant__ CUtensorMap tmap_x,
                          const float* __restrict__ bias, uint32_t* __restrict__ packed, int M,
                          int D, int slab_w, int row_words, int group) {
  constexpr int NTOK = 256;
  constexpr int kBTileBytes = NTOK * 128;
  constexpr int kStageBytes = 2 * kATileBytes + kBTileBytes;
  constexpr uint32_t kTmemCols = 2 * NTOK;
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_s;
  __shared__ uint32_t masks_s[4][32][8];
  __shared__ int prefix_s[4][32][8];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int tile, mblk;
  raster_remap(group, tile, mblk);
  const int m0 = mblk * NTOK;
  const int ksteps = D / kStageK;

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
          atomicExch(&g_tc_error, 1);
          break;
        }
        unsigned char* st = smem + (size_t)s * kStageBytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)kStageBytes);
        tma_load_2d(st, &tmap_w, k * kStageK, tile * kTileN, &full_bar[s]);  // 256 rows: A0 | A1
        tma_load_2d(st + 2 * kATileBytes, &tmap_x, k * kStageK, m0, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) {
          abort_s = 1;
          atomicExch(&g_tc_error, 2);
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
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;              // 0..3
    const int gt = (int)threadIdx.x - 64 - grp * 128;  // 0..127 inside the group
    const int bar_id = 2 + grp;
    bool ok = mbar_wait(&acc_bar, 0u);
    if (!ok) {
      abort_s = 1;
      atomicExch(&g_tc_error, 3);
    }
    ok = named_barrier_and(1, 512, ok);  // the same decision in all 512 epilogue threads
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int n_lo = tile * kTileN + q * 32 + lane;  // neuron of accumulator 0; +128 for 1
    const float b_lo = bias != nullptr ? bias[n_lo] : 0.f;
    const float b_hi = bias != nullptr ? bias[n_lo + 128] : 0.f;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t (*masks)[8] = masks_s[grp];
    int (*prefix)[8] = prefix_s[grp];
    for (int tb = grp; tb < NTOK / 32 && ok; tb += 4) {
      if (m0 + tb * 32 >= M) break;  // the same in every thread of the group
      float v[32];
      // signs
      tmem_ld32(lane_addr + (uint32_t)(tb * 32), v);
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const uint32_t k = __ballot_sync(0xffffffffu, m0 + tb * 32 + c < M && v[c] + b_lo > 0.f);
        if (lane == 0) masks[c][q] = k;
      }
      tmem_ld32(lane_addr + (uint32_t)(NTOK + tb * 32), v);
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const uint32_t k = __ballot_sync(0xffffffffu, m0 + tb * 32 + c < M && v[c] + b_hi > 0.f);
        if (lane == 0) masks[c][4 + q] = k;
      }
      named_barrier(bar_id, 128);
      if (gt < 32) {
        const int tok = m0 + tb * 32 + gt;
        int run = 0;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          prefix[gt][ch] = run;
          run += __popc(masks[gt][ch]);
        }
        if (tok < M) packed[(size_t)tok * row_words + (size_t)tile * slab_w] = (uint32_t)run;
      }
      named_barrier(bar_id, 128);
      // values (accumulator 1 is still in v; accumulator 0 is read again)
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const uint32_t k = masks[c][4 + q];
        if ((k >> lane) & 1u) {
          const int slot = prefix[c][4 + q] + __popc(k & lanemask_lt());
          if (slot < slab_w - 1)
            packed[(size_t)(m0 + tb * 32 + c) * row_words + (size_t)tile * slab_w + 1 + slot] =
                (uint32_t)(n_lo + 128) | (bf16_bits(v[c] + b_hi) << 16);
        }
      }
      tmem_ld32(lane_addr + (uint32_t)(tb * 32), v);
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const uint32_t k = masks[c][q];
        if ((k >> lane) & 1u) {
          const int slot = prefix[c][q] + __popc(k & lanemask_lt());
          if (slot < slab_w - 1)
            packed[(size_t)(m0 + tb * 32 + c) * row_words + (size_t)tile * slab_w + 1 + slot] =
                (uint32_t)n_lo | (bf16_bits(v[c] + b_lo) << 16);
        }
      }
      named_barrier(bar_id, 128);  // masks / prefix are rewritten by the group's next block
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

// ---------------------------------------------------------------------------
// The same split-k kernel with sixteen epilogue warps instead of four.  The epilogue of the
// four-warp form is a latency chain on one warp per scheduler (TMEM read, 64 remote stores
// per thread, then 16 elements per thread to sum, ballot and store).  Here four groups of
// four warps each read 8 token columns of their TMEM lane quarter (tcgen05.ld ...x8) and push
// 16 values per thread, and all 512 epilogue threads take part in the final pass (4 elements
// per thread for a 4-CTA cluster).  Same arithmetic, same slab bytes.
// Threads: warp 0 producer, warp 1 mma, warps 2..17 epilogue (group = (warp - 2) / 4, TMEM
// lane quarter = warp % 4).
// ---------------------------------------------------------------------------
constexpr int kThreadsTcWide = 64 + 512;

template <int CL, int STAGES>
__global__ void __launch_bounds__(kThreadsTcWide, 1)
twell_pack_tc_splitk_wide_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                 const __grid_constant__ CUtensorMap tmap_x,
                                 const float* __restrict__ bias, uint32_t* __restrict__ packed,
                                 int M, int D, int slab_w, int row_words) {
  constexpr int NTOK = kTokDecode;
  constexpr int TOK = NTOK / CL;
  constexpr int kBTileBytes = NTOK * 128;
  constexpr int kStageBytes = 2 * kATileBytes + kBTileBytes;
  constexpr uint32_t kTmemCols = 2 * NTOK;
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);
  constexpr int EPT = TOK * kTileN / 512;  // elements per epilogue thread in the final pass
  static_assert(EPT >= 1, "the final pass needs at least one element per thread");

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* part = reinterpret_cast<float*>(smem + (size_t)STAGES * kStageBytes);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_s;
  __shared__ int cnt_chunk[TOK][8];

  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  cluster.barrier_arrive();  // matched by barrier_wait() before the first remote store

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / CL;
  const int m0 = blockIdx.y * NTOK;
  const int kc = D / CL;
  const int ksteps = kc / kStageK;
  const int k_base = crank * kc;

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
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
          abort_s = 1;
          atomicExch(&g_tc_error, 1);
          break;
        }
        unsigned char* st = smem + (size_t)s * kStageBytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)kStageBytes);
        const int kcoord = k_base + k * kStageK;
        // one copy for the tile's 256 weight rows (A0 | A1 are contiguous): a copy costs the
        // producer thread about 160 ns whatever its size
        tma_load_2d(st, &tmap_w, kcoord, tile * kTileN, &full_bar[s]);
        tma_load_2d(st + 2 * kATileBytes, &tmap_x, kcoord, m0, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) {
          abort_s = 1;
          atomicExch(&g_tc_error, 2);
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
    // ---- epilogue part 1: TMEM -> registers -> owner CTA's shared memory ----
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;  // token columns [8 * grp, 8 * grp + 8)
    bool ok = mbar_wait(&acc_bar, 0u);
    if (!ok) {
      abort_s = 1;
      atomicExch(&g_tc_error, 3);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    cluster.barrier_wait();  // every CTA of the cluster is running
    if (ok) {
      const int nl = q * 32 + lane;  // neuron inside the tile (accumulator 0); +128 for 1
      const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(grp * 8);
      float v0[8], v1[8];
      tmem_ld8(lane_addr, v0);
      tmem_ld8(lane_addr + (uint32_t)NTOK, v1);
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        const int c = grp * 8 + c8;
        const int owner = c / TOK, tl = c % TOK;
        float* dst = cluster.map_shared_rank(part, owner) +
                     (size_t)(crank * TOK + tl) * kPartStrideTc + nl;
        dst[0] = v0[c8];
        dst[128] = v1[c8];
      }
    }
  }
  if (warp < 2) cluster.barrier_wait();  // pair the early arrive for the non-epilogue warps

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster.sync();  // all partials delivered (every thread of every CTA takes part)
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
  if (warp < 2 || abort_s) return;

  // ---- epilogue part 2: this CTA finalises tokens [crank*TOK, (crank+1)*TOK) ----
  const int et = threadIdx.x - 64;  // 0..511
  const int neuron0 = tile * kTileN;
  float z[EPT];
  uint32_t mask[EPT];
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = et + i * 512;
    const int tl = e / kTileN, nl = e % kTileN;
    const int tok = crank * TOK + tl;
    float v = 0.f;
#pragma unroll
    for (int r = 0; r < CL; ++r) v += part[(size_t)(r * TOK + tl) * kPartStrideTc + nl];
    if (bias != nullptr) v += bias[neuron0 + nl];
    const bool keep = (v > 0.f) && (m0 + tok < M);
    z[i] = v;
    mask[i] = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) cnt_chunk[tl][nl / 32] = __popc(mask[i]);
  }
  named_barrier2(512);
  if (et < TOK) {  // counts -> exclusive prefix over the 8 chunks of this token, count word
    int run = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int v = cnt_chunk[et][c];
      cnt_chunk[et][c] = run;
      run += v;
    }
    const int tok = m0 + crank * TOK + et;
    if (tok < M) packed[(size_t)tok * row_words + (size_t)tile * slab_w] = (uint32_t)run;
  }
  named_barrier2(512);
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = et + i * 512;
    const int tl = e / kTileN, nl = e % kTileN;
    const int tok = crank * TOK + tl;
    if (m0 + tok >= M) continue;
    uint32_t* slab = packed + (size_t)(m0 + tok) * row_words + (size_t)tile * slab_w;
    const int slot = cnt_chunk[tl][nl / 32] + __popc(mask[i] & lanemask_lt());
    if (((mask[i] >> lane) & 1u) && slot < slab_w - 1)
      slab[1 + slot] = (uint32_t)(neuron0 + nl) | (bf16_bits(z[i]) << 16);
  }
}

// ---------------------------------------------------------------------------
// Split-k kernel for 33..256 tokens: the decode kernel above with 128-token tiles.  A tile of
// 256 neurons x 128 tokens has only H / 256 CTAs to itself when d_model is not split (32 at
// d_ff 8192: 32 SMs walking 32 latency-bound k-steps, 31-36 us per call whatever the token
// count); split four ways over a cluster every SM streams a quarter of the weight rows.
// The fp32 partial tile of a CTA (128 KB) does not fit next to the operand ring, so the
// partial sums land in the ring itself: a cluster barrier after every CTA's last MMA (instead
// of the early arrive of the decode kernel) makes the ring free, then the TMEM -> DSMEM push,
// a second cluster barrier and the same final pass (CTA r owns 128 / CL tokens).
// grid = ((H/256) * CL, ceil(M / 128)), cluster = CL (4, or 2 when four CTAs per tile would not
// fit one wave), 576 threads.
// ---------------------------------------------------------------------------
constexpr int kTokMid = 128;

template <int CL, int STAGES>
__global__ void __launch_bounds__(kThreadsTcWide, 1)
twell_pack_tc_splitk_mid_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                const __grid_constant__ CUtensorMap tmap_x,
                                const float* __restrict__ bias, uint32_t* __restrict__ packed,
                                int M, int D, int slab_w, int row_words) {
  constexpr int NTOK = kTokMid;
  constexpr int TOK = NTOK / CL;  // tokens finalised per CTA: 32 (CL 4) or 64 (CL 2)
  static_assert(CL == 2 || CL == 4, "cluster size");
  constexpr int kBTileBytes = NTOK * 128;
  constexpr int kStageBytes = 2 * kATileBytes + kBTileBytes;
  constexpr uint32_t kTmemCols = 2 * NTOK;
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);
  constexpr int EPT = TOK * kTileN / 512;  // elements per epilogue thread in the final pass
  static_assert((size_t)NTOK * kPartStrideTc * sizeof(float) <= (size_t)STAGES * kStageBytes,
                "the partial sums must fit into the operand ring");

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* part = reinterpret_cast<float*>(smem);  // [CL source ranks x TOK][kPartStrideTc], after the ring is free
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_s;
  __shared__ int cnt_chunk[TOK][8];

  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / CL;
  const int m0 = blockIdx.y * NTOK;
  const int kc = D / CL;
  const int ksteps = kc / kStageK;
  const int k_base = crank * kc;

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
  pdl_wait();

  bool ok = true;
  if (warp == 0) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
          abort_s = 1;
          atomicExch(&g_tc_error, 1);
          break;
        }
        unsigned char* st = smem + (size_t)s * kStageBytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)kStageBytes);
        const int kcoord = k_base + k * kStageK;
        tma_load_2d(st, &tmap_w, kcoord, tile * kTileN, &full_bar[s]);  // 256 rows: A0 | A1
        tma_load_2d(st + 2 * kATileBytes, &tmap_x, kcoord, m0, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int k = 0; k < ksteps && !abort_s; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) {
          abort_s = 1;
          atomicExch(&g_tc_error, 2);
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
    // every MMA of this CTA has read its operands once the accumulators are published
    ok = mbar_wait(&acc_bar, 0u);
    if (!ok) {
      abort_s = 1;
      atomicExch(&g_tc_error, 3);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  // Every CTA of the cluster is past its last MMA (or has given up): the rings are free.
  cluster.sync();

  if (warp >= 2 && ok) {
    // ---- epilogue part 1: TMEM -> registers -> the owner's ring memory ----
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;  // token columns [32 grp, 32 grp + 32)
    const int owner = grp * 32 / TOK, tl0 = grp * 32 % TOK;
    const int nl = q * 32 + lane;     // neuron inside the tile (accumulator 0); +128 for 1
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(grp * 32);
    float* dst0 = cluster.map_shared_rank(part, owner) +
                  (size_t)(crank * TOK + tl0) * kPartStrideTc + nl;
    float v[32];
    tmem_ld32(lane_addr, v);
#pragma unroll
    for (int c = 0; c < 32; ++c) dst0[(size_t)c * kPartStrideTc] = v[c];
    tmem_ld32(lane_addr + (uint32_t)NTOK, v);
#pragma unroll
    for (int c = 0; c < 32; ++c) dst0[(size_t)c * kPartStrideTc + 128] = v[c];
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster.sync();  // all partials delivered (every thread of every CTA takes part)
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
  if (warp < 2 || abort_s) return;

  // ---- epilogue part 2: this CTA finalises tokens [crank*TOK, (crank+1)*TOK) ----
  const int et = threadIdx.x - 64;  // 0..511
  const int neuron0 = tile * kTileN;
  float z[EPT];
  uint32_t mask[EPT];
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = et + i * 512;
    const int tl = e / kTileN, nl = e % kTileN;
    const int tok = crank * TOK + tl;
    float v = 0.f;
#pragma unroll
    for (int r = 0; r < CL; ++r) v += part[(size_t)(r * TOK + tl) * kPartStrideTc + nl];
    if (bias != nullptr) v += bias[neuron0 + nl];
    const bool keep = (v > 0.f) && (m0 + tok < M);
    z[i] = v;
    mask[i] = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) cnt_chunk[tl][nl / 32] = __popc(mask[i]);
  }
  named_barrier2(512);
  if (et < TOK) {  // counts -> exclusive prefix over the 8 chunks of this token, count word
    int run = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int v = cnt_chunk[et][c];
      cnt_chunk[et][c] = run;
      run += v;
    }
    const int tok = m0 + crank * TOK + et;
    if (tok < M) packed[(size_t)tok * row_words + (size_t)tile * slab_w] = (uint32_t)run;
  }
  named_barrier2(512);
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = et + i * 512;
    const int tl = e / kTileN, nl = e % kTileN;
    const int tok = crank * TOK + tl;
    if (m0 + tok >= M) continue;
    uint32_t* slab = packed + (size_t)(m0 + tok) * row_words + (size_t)tile * slab_w;
    const int slot = cnt_chunk[tl][nl / 32] + __popc(mask[i] & lanemask_lt());
    if (((mask[i] >> lane) & 1u) && slot < slab_w - 1)
      slab[1 + slot] = (uint32_t)(neuron0 + nl) | (bf16_bits(z[i]) << 16);
  }
}

// ---- host side -------------------------------------------------------------
template <int NTOK, int STAGES, int MINB = 1>
int launch_tc(const void* x, const void* w, const float* bias, void* packed, int64_t M, int64_t D,
              int64_t H, int cf, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  if (int rc = make_map(&map_w, w, H, D, 128)) return rc;
  if (int rc = make_map(&map_x, x, M, D, NTOK)) return rc;
  const size_t smem = (size_t)STAGES * (2 * kATileBytes + NTOK * 128) + 1024;
  auto kern = twell_pack_tc_kernel<NTOK, STAGES, MINB>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_pack")) return rc;
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  dim3 grid((unsigned)tiles, (unsigned)((M + NTOK - 1) / NTOK), 1);
  kern<<<grid, kThreadsTc, smem, stream>>>(map_w, map_x, bias, static_cast<uint32_t*>(packed),
                                           (int)M, (int)D, slab_w, tiles * slab_w,
                                           raster_group(H * D * 2, (int64_t)NTOK * D * 2));
  return check_launch("b200_twell_pack (tcgen05)");
}

template <int STAGES>
int launch_tc_wide(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                   int64_t D, int64_t H, int cf, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  if (int rc = make_map(&map_w, w, H, D, 256)) return rc;
  if (int rc = make_map(&map_x, x, M, D, 256)) return rc;
  const size_t smem = (size_t)STAGES * (2 * kATileBytes + 256 * 128) + 1024;
  auto kern = twell_pack_tc_wide_kernel<STAGES>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_pack")) return rc;
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  dim3 grid((unsigned)tiles, (unsigned)((M + 255) / 256), 1);
  kern<<<grid, kThreadsTcWideM, smem, stream>>>(map_w, map_x, bias,
                                                static_cast<uint32_t*>(packed), (int)M, (int)D,
                                                slab_w, tiles * slab_w,
                                                raster_group(H * D * 2, (int64_t)256 * D * 2));
  return check_launch("b200_twell_pack (tcgen05, 256-token tiles)");
}

template <int CL, int STAGES>
int launch_tc_splitk_mid(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                         int64_t D, int64_t H, int cf, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  if (int rc = make_map(&map_w, w, H, D, 256)) return rc;
  if (int rc = make_map(&map_x, x, M, D, kTokMid)) return rc;
  const size_t smem = (size_t)STAGES * (2 * kATileBytes + kTokMid * 128) + 1024;
  auto kern = twell_pack_tc_splitk_mid_kernel<CL, STAGES>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_pack")) return rc;
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * CL), (unsigned)((M + kTokMid - 1) / kTokMid), 1);
  cfg.blockDim = dim3(kThreadsTcWide, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = add_pdl_attribute(attr, 1, 1);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_w, map_x, bias,
                                     static_cast<uint32_t*>(packed), (int)M, (int)D, slab_w,
                                     tiles * slab_w);
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "b200_twell_pack (tcgen05 split-k, 128-token tiles): launch: %s",
                cudaGetErrorString(e));
  return B200_OK;
}

// Epilogue form of the split-k kernel: sixteen epilogue warps unless B200_PACK_WIDE=0.
bool pack_wide_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("B200_PACK_WIDE");
    on = (e != nullptr && atoi(e) == 0) ? 0 : 1;
  }
  return on != 0;
}

template <int CL, int STAGES, bool WIDE>
int launch_tc_splitk_form(const void* x, const void* w, const float* bias, void* packed,
                          int64_t M, int64_t D, int64_t H, int cf, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  if (int rc = make_map(&map_w, w, H, D, 256)) return rc;
  if (int rc = make_map(&map_x, x, M, D, kTokDecode)) return rc;
  const size_t smem = (size_t)STAGES * (2 * kATileBytes + kTokDecode * 128) +
                      (size_t)kTokDecode * kPartStrideTc * sizeof(float) + 1024;
  auto kern = WIDE ? twell_pack_tc_splitk_wide_kernel<CL, STAGES>
                   : twell_pack_tc_splitk_kernel<CL, STAGES>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_pack")) return rc;
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * CL), (unsigned)((M + kTokDecode - 1) / kTokDecode), 1);
  cfg.blockDim = dim3(WIDE ? kThreadsTcWide : kThreadsTc, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = add_pdl_attribute(attr, 1, 1);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_w, map_x, bias,
                                     static_cast<uint32_t*>(packed), (int)M, (int)D, slab_w,
                                     tiles * slab_w);
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "b200_twell_pack (tcgen05 split-k): launch: %s",
                cudaGetErrorString(e));
  return B200_OK;
}

template <int CL, int STAGES>
int launch_tc_splitk(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                     int64_t D, int64_t H, int cf, cudaStream_t stream) {
  return pack_wide_enabled()
             ? launch_tc_splitk_form<CL, STAGES, true>(x, w, bias, packed, M, D, H, cf, stream)
             : launch_tc_splitk_form<CL, STAGES, false>(x, w, bias, packed, M, D, H, cf, stream);
}

}  // namespace

// Decode path on the tensor cores: split-k over a cluster of 4 CTAs.
int twell_pack_tc_splitk(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                         int64_t D, int64_t H, int cf, cudaStream_t stream) {
  return launch_tc_splitk<4, 5>(x, w, bias, packed, M, D, H, cf, stream);
}

// The same with D split 8 ways: twice the CTAs for narrow d_ff (a d_ff shard of 2048..4096
// neurons has only 8..16 tiles).  Needs D % 512 == 0.
int twell_pack_tc_splitk8(const void* x, const void* w, const float* bias, void* packed,
                          int64_t M, int64_t D, int64_t H, int cf, cudaStream_t stream) {
  if (D % 512) return fail(B200_EUNSUPPORTED, "b200_twell_pack: 8-way split needs D %% 512 == 0");
  return launch_tc_splitk<8, 4>(x, w, bias, packed, M, D, H, cf, stream);
}

// Large-M path.  Needs D % 64 == 0 (guaranteed by D % 256 == 0).
int twell_pack_tc(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                  int64_t D, int64_t H, int cf, cudaStream_t stream) {
  // Above 64 tokens: one CTA per SM on 256-token tiles with sixteen epilogue warps.  Measured
  // on B200 against two co-resident 128-token CTAs per SM (four epilogue warps each) and
  // cuBLAS matmul + relu, TFLOP/s at (M, D, H): (2048, 2048, 8192) 996 / 826 / 1063;
  // (16384, 2048, 8192) 1222 / 995 / 1273; (16384, 2048, 11008) 1221 / 1002 / 1260;
  // (2048, 4096, 16384) 1299 / 1102 / 1363; (16384, 4096, 16384) 1288 / 1222 / 1391;
  // (16384, 1024, 4096) 855 / 681 / 994; at 100 tokens (D 2048, H 8192) 30.4 against 34.6 us
  // for one 128-token tile per CTA.  B200_PACK_TILE=128 keeps the 128-token forms.
  static const int tile_tokens = [] {
    const char* e = getenv("B200_PACK_TILE");
    return e != nullptr ? atoi(e) : 256;
  }();
  if (M > 64 && tile_tokens != 128) return launch_tc_wide<3>(x, w, bias, packed, M, D, H, cf, stream);
  if (M >= 1024) return launch_tc<128, 2, 2>(x, w, bias, packed, M, D, H, cf, stream);
  if (M > 64) return launch_tc<128, 4>(x, w, bias, packed, M, D, H, cf, stream);
  return launch_tc<64, 4>(x, w, bias, packed, M, D, H, cf, stream);
}

// (A 2-way split - 64 CTAs streaming 512 KB each at H = 8192 - was measured at 16.8 us against
// 12.8 us for the 4-way split: one SM pulls about 64 GB/s through TMA, so the weight stream
// needs well over 100 CTAs to reach the HBM rate.)

// Two co-resident CTAs of 128 tokens per SM (2 x 256 TMEM columns, 2 x 2 stages): one CTA's
// pack epilogue runs under the other's MMAs.
int twell_pack_tc_pair(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                       int64_t D, int64_t H, int cf, cudaStream_t stream) {
  return launch_tc<128, 2, 2>(x, w, bias, packed, M, D, H, cf, stream);
}

// 33..256 tokens: split-k over a cluster of `split` (4 or 2) CTAs with 128-token tiles.
int twell_pack_tc_splitk_mid(const void* x, const void* w, const float* bias, void* packed,
                             int64_t M, int64_t D, int64_t H, int cf, int split,
                             cudaStream_t stream) {
  if (split == 2) return launch_tc_splitk_mid<2, 4>(x, w, bias, packed, M, D, H, cf, stream);
  return launch_tc_splitk_mid<4, 4>(x, w, bias, packed, M, D, H, cf, stream);
}

// Cluster size for the 128-token split-k kernel: the largest of 4 and 2 whose grid is one
// wave (one CTA per SM); 0 when neither is.  Measured on B200 (D 2048, d_ff 8192): 17.0 us
// at 33..128 tokens against 27.4-29.5 us for unsplit tiles; at D 4096, d_ff 16384 and 128
// tokens the four-way split needs two waves (45.6 against 50.2 us).
int twell_pack_mid_split(int64_t M, int64_t H, int sm_count) {
  const int64_t tiles = H / kTileN, blocks = (M + kTokMid - 1) / kTokMid;
  if (tiles * 4 * blocks <= sm_count) return 4;
  if (tiles * 2 * blocks <= sm_count) return 2;
  return 0;
}

// One CTA per SM, 256 neurons x 256 tokens per tile, sixteen epilogue warps.
int twell_pack_tc_wide(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                       int64_t D, int64_t H, int cf, cudaStream_t stream) {
  return launch_tc_wide<3>(x, w, bias, packed, M, D, H, cf, stream);
}

// Error word raised by a bounded wait that gave up (0 = none).  Reads and clears it;
// synchronises the device.
int twell_pack_tc_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
  return v;
}

}  // namespace b200
