// Gate projection + ReLU + TwELL pack on the 5th-generation tensor cores (large M).
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
#include <cuda.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kStageK = 64;                 // k-values per stage (128 bytes per row)
constexpr int kATileBytes = 128 * 128;      // 128 rows x 128 bytes
constexpr int kThreadsTc = 192;             // warp 0 producer, warp 1 mma, warps 2..5 epilogue
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ int g_tc_error = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

// Bounded wait on a phase parity.  false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address
  d |= (uint64_t)1 << 16;                     // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                     // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                     // SWIZZLE_128B
  return d;
}

// Instruction descriptor, kind::f16: fp32 accumulate, bf16 x bf16, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void epi_barrier() {  // the 128 epilogue threads only
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// grid = (H / 256, ceil(M / NTOK)).  Dynamic shared memory: STAGES x (A0 | A1 | B), 1024-aligned.
template <int NTOK, int STAGES>
__global__ void __launch_bounds__(kThreadsTc, 1)
twell_pack_tc_kernel(const __grid_constant__ CUtensorMap tmap_w,
                     const __grid_constant__ CUtensorMap tmap_x, const float* __restrict__ bias,
                     uint32_t* __restrict__ packed, int M, int D, int slab_w, int row_words) {
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
  const int tile = blockIdx.x;
  const int m0 = blockIdx.y * NTOK;
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
        tma_load_2d(st, &tmap_w, kcoord, tile * kTileN, &full_bar[s]);
        tma_load_2d(st + kATileBytes, &tmap_w, kcoord, tile * kTileN + 128, &full_bar[s]);
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

// ---- host side -------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is resolved through the runtime, so the library carries no
// link-time dependency on libcuda and still loads on a machine without a driver.
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [rows, D] bf16 row-major; box = 64 k-values x box_rows rows, 128-byte swizzle, zero fill.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t D, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(B200_ECUDA, "b200_twell_pack: cuTensorMapEncodeTiled unavailable");
  const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kStageK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B200_ECUDA, "b200_twell_pack: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return B200_OK;
}

template <int NTOK, int STAGES>
int launch_tc(const void* x, const void* w, const float* bias, void* packed, int64_t M, int64_t D,
              int64_t H, int cf, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  if (int rc = make_map(&map_w, w, H, D, 128)) return rc;
  if (int rc = make_map(&map_x, x, M, D, NTOK)) return rc;
  const size_t smem = (size_t)STAGES * (2 * kATileBytes + NTOK * 128) + 1024;
  auto kern = twell_pack_tc_kernel<NTOK, STAGES>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_pack")) return rc;
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  dim3 grid((unsigned)tiles, (unsigned)((M + NTOK - 1) / NTOK), 1);
  kern<<<grid, kThreadsTc, smem, stream>>>(map_w, map_x, bias, static_cast<uint32_t*>(packed),
                                           (int)M, (int)D, slab_w, tiles * slab_w);
  return check_launch("b200_twell_pack (tcgen05)");
}

template <int CL, int STAGES>
int launch_tc_splitk(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                     int64_t D, int64_t H, int cf, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  if (int rc = make_map(&map_w, w, H, D, 128)) return rc;
  if (int rc = make_map(&map_x, x, M, D, kTokDecode)) return rc;
  const size_t smem = (size_t)STAGES * (2 * kATileBytes + kTokDecode * 128) +
                      (size_t)kTokDecode * kPartStrideTc * sizeof(float) + 1024;
  auto kern = twell_pack_tc_splitk_kernel<CL, STAGES>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_pack")) return rc;
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * CL), (unsigned)((M + kTokDecode - 1) / kTokDecode), 1);
  cfg.blockDim = dim3(kThreadsTc, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_w, map_x, bias,
                                     static_cast<uint32_t*>(packed), (int)M, (int)D, slab_w,
                                     tiles * slab_w);
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "b200_twell_pack (tcgen05 split-k): launch: %s",
                cudaGetErrorString(e));
  return B200_OK;
}

}  // namespace

// Decode path on the tensor cores: split-k over a cluster of 4 CTAs.
int twell_pack_tc_splitk(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                         int64_t D, int64_t H, int cf, cudaStream_t stream) {
  return launch_tc_splitk<4, 5>(x, w, bias, packed, M, D, H, cf, stream);
}

// Large-M path.  Needs D % 64 == 0 (guaranteed by D % 256 == 0).
int twell_pack_tc(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                  int64_t D, int64_t H, int cf, cudaStream_t stream) {
  // 256-token tiles raise the flops per byte staged through shared memory (the 128-token
  // tile is bound by L2 -> SM bandwidth); they use all 512 TMEM columns.
  if (M >= 1024) return launch_tc<256, 3>(x, w, bias, packed, M, D, H, cf, stream);
  if (M > 64) return launch_tc<128, 4>(x, w, bias, packed, M, D, H, cf, stream);
  return launch_tc<64, 4>(x, w, bias, packed, M, D, H, cf, stream);
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
