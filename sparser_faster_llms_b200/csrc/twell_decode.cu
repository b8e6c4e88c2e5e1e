// One kernel per sparse FFN layer for decode-sized calls (1..32 tokens):
// gate projection + ReLU + TwELL pack + gated up/down contraction, no slab round trip.
//
// Decomposition: a thread-block cluster of CL CTAs owns one 256-neuron TwELL tile; CTA r of
// the cluster owns column slice r of d_model ([r*kc, (r+1)*kc), kc = D / CL) in every phase.
//
//   1. gate GEMM, split-k: CTA r multiplies the tile's 256 gate rows by slice r of the
//      tokens (TMA -> shared-memory ring -> tcgen05.mma, fp32 accumulators in TMEM).  The
//      x slice stays in shared memory for phase 4.
//   2. the partial accumulators leave TMEM through registers and are pushed (distributed
//      shared memory) to the CTA that finalises each token; it adds the CL partials in rank
//      order, applies bias and ReLU, compacts with ballot / popc and writes the slab words
//      (same bytes as b200_twell_pack), and all-gathers the surviving gate values as a
//      [32 tokens][256 neurons] bf16 tile into every CTA of the cluster.
//   3. every CTA derives the same lists from that tile: the active neurons of the tile (the
//      union over the tokens), a token mask per active neuron, and the (neuron, token) pairs.
//   4. neuron-major contraction: each active neuron's slice of its up row and of its down
//      row is fetched ONCE per call with cp.async.bulk (1 KB pieces at D = 2048, completion
//      on an mbarrier) into shared memory, however many tokens fire it.  Pass A dots the x
//      slice with the up slice for every pair (one warp per pair); the CL slice sums of a
//      pair meet through distributed shared memory and give u, h = g * u; pass B adds
//      h * down slice into this CTA's [tokens][kc] fp32 accumulator in shared memory.
//   5. cross-tile sum: every CTA writes its accumulator to the workspace; the CTAs of one
//      column slice meet at a bounded spin barrier in global memory (all CTAs of the grid are
//      co-resident: the host checks cudaOccupancyMaxActiveClusters), then each of them sums a
//      share of the slice over the tiles in tile order and stores bf16.  Fixed order
//      everywhere: deterministic.
//
// Optionally every CTA first asks L2 to prefetch its share of a caller-named byte range
// (cp.async.bulk.prefetch.L2 on this GPU's own memory): the next layer's gate matrix does not
// depend on this layer's result, so its HBM stream overlaps this layer's latency-bound phases.
//
// Numerics follow the reference kernels as twell_t2d.cu does: mixed mode rounds every product
// and h to bf16 (custom_models/twell_modules/matmul_gated_t2d.cu:74-149), high precision is
// fp32 fma throughout (:389-441).  Entries beyond a slab's capacity are dropped as in the
// two-kernel path.  Replaces the reference's two launches per layer,
// TWELL_MLP::run_gated_mlp_layer* (custom_models/twell_modules/mlp_twell.cu:126-152).
//
// Every wait is bounded.  A wait that gives up raises an error word
// (b200_twell_decode_status) and the kernel carries on with whatever it has - control flow
// never depends on a wait's outcome, so every barrier is still attended - frees its TMEM and
// returns.
#include <cooperative_groups.h>

#include <cstdlib>

#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

__device__ int g_dec_error = 0;

#ifdef B200_TRACE
// Phase time stamps (globaltimer, ns) of CTA 0: a debugging aid compiled in on request.
__device__ unsigned long long g_dec_trace[16];
__device__ __forceinline__ void dec_stamp(int i) {
  if (blockIdx.x == 0 && threadIdx.x == 64) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_dec_trace[i] = t;
  }
}
#else
__device__ __forceinline__ void dec_stamp(int) {}
#endif

constexpr int kDecThreads = 256;  // warp 0 producer, 1 mma, 2..5 epilogue, 6..7 join from phase 3
constexpr int kDecWarps = kDecThreads / 32;
static_assert(kDecThreads == kTileN, "phase 3 maps one thread to one neuron of the tile");
constexpr int kDecTok = 32;                   // token rows of the MMA tile (padded)
constexpr int kDecPartStride = kTileN + 4;    // floats per row of the partial-sum inbox
constexpr int kDecRingStageBytes = 2 * kATileBytes;  // two 128-neuron halves of a k step
constexpr int kDecPartBytes = kDecTok * kDecPartStride * 4;
constexpr int kDecGtileBytes = kDecTok * kTileN * 2;
constexpr int kDecMaxStageRows = 64;          // active neurons staged per round, at most
constexpr uint32_t kDecSpinLimit = 1u << 22;

// Workspace words used by the cross-tile barrier (see twell_t2d.cu for the whole layout).
constexpr size_t kDecCounterWords = 4096;
constexpr size_t kDecSyncWord0 = kDecCounterWords - 64;  // + 2 * crank: arrivals, + 1: release

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

__device__ __forceinline__ void dec_fail(int code) { atomicExch(&g_dec_error, code); }

// Shared-memory layout of the lists that replace the partial-sum inbox after phase 2.
template <int CL>
struct DecLists {
  static constexpr int kPairMax = 4096 / CL;  // (neuron, token) pairs per round
  float uin[CL][kPairMax];                    // slice sums of u, one row per source CTA
  float h[kPairMax];
  unsigned char ptok[kPairMax];               // token of a pair
  unsigned char prow[kPairMax];               // staged row (slot - round start) of a pair
  uint32_t mlist[kTileN];                     // token mask of active neuron `slot`
  int poff[kTileN + 1];                       // exclusive prefix of popc(mlist)
  unsigned short nlist[kTileN];               // neuron (inside the tile) of active slot
};
static_assert(sizeof(DecLists<4>) <= kDecPartBytes, "lists must fit the inbox they replace");
static_assert(sizeof(DecLists<8>) <= kDecPartBytes, "lists must fit the inbox they replace");

// grid.x = tiles * CL, cluster = CL.  Dynamic shared memory (1024-aligned):
//   ring   STAGES x 32 KB (gate tiles; after phase 2: y accumulator + staged up / down slices)
//   xs     (kc / 64) x 4 KB  x slice, 128-byte swizzled K-major tiles of 64 columns
//   part   33280 B       partial-sum inbox, then DecLists
//   gtile  16 KB         gate values [32][256] bf16, 0 = inactive
template <int CL, int STAGES, bool GATED, bool HP>
__global__ void __launch_bounds__(kDecThreads, 1)
twell_decode_kernel(const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_x, const float* __restrict__ bias,
                    uint32_t* __restrict__ packed, const __nv_bfloat16* __restrict__ up,
                    const __nv_bfloat16* __restrict__ down, __nv_bfloat16* out, int M, int D,
                    int slab_w, int row_words, int stage_rows, float* ws_part,
                    unsigned int* ws_sync, const unsigned char* pf_ptr, long long pf_bytes) {
  constexpr int NTOK = kDecTok;
  constexpr int TOK = NTOK / CL;  // tokens finalised by this CTA
  constexpr uint32_t kTmemCols = 2 * NTOK;
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);
  constexpr int EPT = TOK * kTileN / 128;
  constexpr int PMAX = DecLists<CL>::kPairMax;
  constexpr uint32_t FULL = 0xffffffffu;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar, up_bar, dn_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int cnt_chunk[TOK][8];
  __shared__ int warp_cnt[kDecWarps];
  __shared__ uint32_t release0_s;

  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  cluster.barrier_arrive();  // B0: matched by barrier_wait() before the first remote store

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x / CL;
  const int tiles = gridDim.x / CL;
  const int kc = D / CL;
  const int ksteps = kc / kStageK;
  const int k_base = crank * kc;

  unsigned char* ring = smem;
  unsigned char* xs = ring + (size_t)STAGES * kDecRingStageBytes;
  float* part = reinterpret_cast<float*>(xs + (size_t)ksteps * 4096);
  unsigned short* gtile = reinterpret_cast<unsigned short*>(
      reinterpret_cast<unsigned char*>(part) + kDecPartBytes);
  DecLists<CL>& L = *reinterpret_cast<DecLists<CL>*>(part);
  // after phase 2 the ring holds the accumulator and the staged weight slices
  float* yacc = reinterpret_cast<float*>(ring);
  unsigned char* up_s = ring + (((size_t)M * kc * 4 + 1023) & ~(size_t)1023);
  unsigned char* dn_s = up_s + (size_t)stage_rows * kc * 2;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    mbar_init(&up_bar, 1);
    mbar_init(&dn_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    release0_s = reinterpret_cast<volatile unsigned int*>(ws_sync)[2 * crank + 1];
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
  dec_stamp(0);

  // ---- phase 1: gate GEMM over this CTA's k slice --------------------------------------
  if (warp == 0) {
    if (lane == 0) {
      for (int k = 0; k < ksteps; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], phase ^ 1u)) dec_fail(1);
        unsigned char* st = ring + (size_t)s * kDecRingStageBytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)(kDecRingStageBytes + NTOK * 128));
        const int kcoord = k_base + k * kStageK;
        tma_load_2d(st, &tmap_w, kcoord, tile * kTileN, &full_bar[s]);
        tma_load_2d(st + kATileBytes, &tmap_w, kcoord, tile * kTileN + 128, &full_bar[s]);
        tma_load_2d(xs + (size_t)k * 4096, &tmap_x, kcoord, 0, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int k = 0; k < ksteps; ++k) {
        const int s = k % STAGES;
        const uint32_t phase = (uint32_t)(k / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) dec_fail(2);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a0 = smem_u32(ring + (size_t)s * kDecRingStageBytes);
        const uint64_t da0 = umma_desc(a0), da1 = umma_desc(a0 + kATileBytes),
                       db = umma_desc(smem_u32(xs + (size_t)k * 4096));
#pragma unroll
        for (int kk = 0; kk < kStageK / 16; ++kk) {
          const uint32_t acc = (k > 0 || kk > 0) ? 1u : 0u;
          umma_bf16(tmem_base, da0 + 2 * kk, db + 2 * kk, kIdesc, acc);
          umma_bf16(tmem_base + NTOK, da1 + 2 * kk, db + 2 * kk, kIdesc, acc);
        }
        umma_commit(&empty_bar[s]);
      }
      umma_commit(&acc_bar);
    }
  } else if (warp == 6) {
    // L2 prefetch of the caller's range (the next layer's gate matrix): this CTA's share
    if (pf_ptr != nullptr && pf_bytes > 0) {
      const long long piece = 16384;
      const long long pieces = (pf_bytes + piece - 1) / piece;
      const long long per = (pieces + gridDim.x - 1) / gridDim.x;
      const long long p0 = (long long)blockIdx.x * per;
      for (long long p = p0 + lane; p < p0 + per && p < pieces; p += 32) {
        const long long off = p * piece;
        const long long n = (pf_bytes - off < piece ? pf_bytes - off : piece) & ~15ll;
        if (n > 0) l2_prefetch(pf_ptr + off, (uint32_t)n);
      }
    }
  }
  if (warp >= 2 && warp < 6) {
    // ---- phase 2a: TMEM -> registers -> owner CTA's inbox ----
    const int q = warp & 3;
    if (!mbar_wait(&acc_bar, 0u)) dec_fail(3);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    dec_stamp(1);
    cluster.barrier_wait();  // B0: every CTA of the cluster is running
    const int nl = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    float v0[32], v1[32];
    tmem_ld32(lane_addr, v0);
    tmem_ld32(lane_addr + (uint32_t)NTOK, v1);
#pragma unroll
    for (int c = 0; c < NTOK; ++c) {
      const int owner = c / TOK, tl = c % TOK;
      float* dst = cluster.map_shared_rank(part, owner) +
                   (size_t)(crank * TOK + tl) * kDecPartStride + nl;
      dst[0] = v0[c];
      dst[128] = v1[c];
    }
  } else {
    cluster.barrier_wait();  // B0 for the other warps
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster.sync();  // B1: all partials delivered; every CTA's MMAs are complete
  dec_stamp(2);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }

  if (warp >= 2 && warp < 6) {
    // ---- phase 2b: finalise tokens [crank*TOK, (crank+1)*TOK), slab + gate tile ----
    const int et = tid - 64;
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
      for (int r = 0; r < CL; ++r) v += part[(size_t)(r * TOK + tl) * kDecPartStride + nl];
      if (bias != nullptr) v += bias[neuron0 + nl];
      const bool keep = (v > 0.f) && (tok < M);
      z[i] = v;
      mask[i] = __ballot_sync(FULL, keep);
      if (lane == 0) cnt_chunk[tl][nl / 32] = __popc(mask[i]);
    }
    epi_barrier();
    if (et < TOK) {
      int run = 0;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int v = cnt_chunk[et][c];
        cnt_chunk[et][c] = run;
        run += v;
      }
      const int tok = crank * TOK + et;
      if (tok < M) packed[(size_t)tok * row_words + (size_t)tile * slab_w] = (uint32_t)run;
    }
    epi_barrier();
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const int e = et + i * 128;
      const int tl = e / kTileN, nl = e % kTileN;
      const int tok = crank * TOK + tl;
      const int slot = cnt_chunk[tl][nl / 32] + __popc(mask[i] & lanemask_lt());
      const bool stored = ((mask[i] >> lane) & 1u) && slot < slab_w - 1;
      const uint32_t bits = bf16_bits(z[i]);
      if (stored)
        packed[(size_t)tok * row_words + (size_t)tile * slab_w + 1 + slot] =
            (uint32_t)(neuron0 + nl) | (bits << 16);
      gtile[tok * kTileN + nl] = stored ? (unsigned short)bits : (unsigned short)0;
    }
    epi_barrier();
    // all-gather: this CTA's TOK rows of the gate tile go to the other CTAs of the cluster
    {
      const uint4* src = reinterpret_cast<const uint4*>(gtile + crank * TOK * kTileN);
      constexpr int kVec = TOK * kTileN * 2 / 16;
      for (int r = 1; r < CL; ++r) {
        const int dstrank = (crank + r) % CL;
        uint4* dst = reinterpret_cast<uint4*>(cluster.map_shared_rank(gtile, dstrank) +
                                              crank * TOK * kTileN);
        for (int i = et; i < kVec; i += 128) dst[i] = src[i];
      }
    }
  } else {
    // the ring is free (B1): clear the accumulator while the epilogue warps finalise
    const int n4 = M * kc / 4;
    const int t4 = (warp < 2 ? warp : warp - 4) * 32 + lane;  // 0..127 over warps 0, 1, 6, 7
    for (int i = t4; i < n4; i += 128)
      reinterpret_cast<float4*>(yacc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  cluster.sync();  // B2: gate tile complete in every CTA; inbox no longer read
  dec_stamp(3);

  // ---- phase 3: lists (identical in every CTA of the cluster) --------------------------
  {
    uint32_t tmask = 0;
#pragma unroll 8
    for (int t = 0; t < NTOK; ++t)
      if (gtile[t * kTileN + tid] != 0) tmask |= 1u << t;
    const bool act = tmask != 0;
    const uint32_t ball = __ballot_sync(FULL, act);
    if (lane == 0) warp_cnt[warp] = __popc(ball);
    __syncthreads();
    int base = 0, n_act = 0;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const int c = warp_cnt[w];
      if (w < warp) base += c;
      n_act += c;
    }
    const int slot = base + __popc(ball & lanemask_lt());
    if (act) {
      L.nlist[slot] = (unsigned short)tid;
      L.mlist[slot] = tmask;
    }
    __syncthreads();
    // exclusive prefix of the pair counts over the slots (thread = slot)
    const int c = tid < n_act ? __popc(L.mlist[tid]) : 0;
    int inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(FULL, inc, o);
      if (lane >= o) inc += v;
    }
    if (lane == 31) warp_cnt[warp] = inc;  // all threads have read warp_cnt above
    __syncthreads();
    int wbase = 0;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w)
      if (w < warp) wbase += warp_cnt[w];
    L.poff[tid] = wbase + inc - c;
    if (tid == kDecThreads - 1) L.poff[kTileN] = wbase + inc;
    __syncthreads();

    // ---- phase 4: contraction, rounds of at most stage_rows active neurons ----
    const int nrounds = (n_act + stage_rows - 1) / stage_rows;
    const int row_bytes = kc * 2;
    const size_t w_row0 = (size_t)tile * kTileN * D + (size_t)k_base;  // element offset
    auto issue = [&](const __nv_bfloat16* w, unsigned char* dst, uint64_t* bar, int s0, int s1) {
      // warp 0: one bulk copy per staged row
      if (warp == 0) {
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)((s1 - s0) * row_bytes));
        __syncwarp();
        for (int s = s0 + lane; s < s1; s += 32)
          bulk_g2s(dst + (size_t)(s - s0) * row_bytes, w + w_row0 + (size_t)L.nlist[s] * D,
                   (uint32_t)row_bytes, bar);
      }
    };
    if (nrounds > 0) {
      const int s1 = min(n_act, stage_rows);
      if (GATED) issue(up, up_s, &up_bar, 0, s1);
      issue(down, dn_s, &dn_bar, 0, s1);
    }
    dec_stamp(4);
    for (int rd = 0; rd < nrounds; ++rd) {
      const int s0 = rd * stage_rows, s1 = min(n_act, s0 + stage_rows);
      const int p0 = L.poff[s0], np = L.poff[s1] - p0;
      const uint32_t par = (uint32_t)rd & 1u;
      // pair list of the round (thread = staged row)
      if (tid < s1 - s0) {
        uint32_t m = L.mlist[s0 + tid];
        int p = L.poff[s0 + tid] - p0;
        while (m) {
          const int t = __ffs(m) - 1;
          m &= m - 1;
          L.ptok[p] = (unsigned char)t;
          L.prow[p] = (unsigned char)tid;
          ++p;
        }
      }
      __syncthreads();
      if (GATED) {
        if (!mbar_wait(&up_bar, par)) dec_fail(4);
        if (rd > 0) cluster.barrier_wait();  // Bb: every CTA has read the previous round's uin
        // pass A: one warp per pair, this CTA's slice of the dot product
        for (int p = warp; p < np; p += kDecWarps) {
          const int t = L.ptok[p];
          const unsigned char* wrow = up_s + (size_t)L.prow[p] * row_bytes;
          float s = 0.f;
          for (int qv = lane; qv < kc / 8; qv += 32) {
            const uint4 xv = *reinterpret_cast<const uint4*>(
                xs + (size_t)(qv >> 3) * 4096 + t * 128 + (((qv & 7) ^ (t & 7)) << 4));
            const uint4 wv = *reinterpret_cast<const uint4*>(wrow + qv * 16);
            const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (HP) {
                const float2 wf = __bfloat1622float2(w2[e]), xf = __bfloat1622float2(x2[e]);
                s = __fmaf_rn(wf.x, xf.x, s);
                s = __fmaf_rn(wf.y, xf.y, s);
              } else {
                const float2 pf = __bfloat1622float2(__hmul2(x2[e], w2[e]));
                s += pf.x;
                s += pf.y;
              }
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FULL, s, o);
          if (lane < CL) cluster.map_shared_rank(&L.uin[0][0], lane)[crank * PMAX + p] = s;
        }
        cluster.sync();  // Ba: the round's slice sums are in every CTA; up_s is free
        if (rd + 1 < nrounds) issue(up, up_s, &up_bar, s1, min(n_act, s1 + stage_rows));
      }
      // h of every pair of the round
      for (int p = tid; p < np; p += kDecThreads) {
        const int t = L.ptok[p];
        const int n = L.nlist[s0 + L.prow[p]];
        const __nv_bfloat16 g = __ushort_as_bfloat16(gtile[t * kTileN + n]);
        float hv;
        if (GATED) {
          float u = 0.f;
#pragma unroll
          for (int r = 0; r < CL; ++r) u += L.uin[r][p];
          hv = HP ? __bfloat162float(g) * u
                  : __bfloat162float(__hmul(g, __float2bfloat16_rn(u)));
        } else {
          hv = __bfloat162float(g);
        }
        L.h[p] = hv;
      }
      __syncthreads();
      if (GATED && rd + 1 < nrounds) cluster.barrier_arrive();  // Bb: uin of this round is read
      if (!mbar_wait(&dn_bar, par)) dec_fail(5);
      // pass B: y[t, slice] += h * down[n, slice]; a thread owns fixed column pairs
      for (int p = 0; p < np; ++p) {
        const int t = L.ptok[p];
        const float hv = L.h[p];
        const __nv_bfloat162* drow =
            reinterpret_cast<const __nv_bfloat162*>(dn_s + (size_t)L.prow[p] * row_bytes);
        float2* yrow = reinterpret_cast<float2*>(yacc + (size_t)t * kc);
        const __nv_bfloat162 hb2 = __float2bfloat162_rn(hv);
        for (int c2 = tid; c2 < kc / 2; c2 += kDecThreads) {
          float2 y = yrow[c2];
          if (HP) {
            const float2 wf = __bfloat1622float2(drow[c2]);
            y.x = __fmaf_rn(wf.x, hv, y.x);
            y.y = __fmaf_rn(wf.y, hv, y.y);
          } else {
            const float2 pf = __bfloat1622float2(__hmul2(hb2, drow[c2]));
            y.x += pf.x;
            y.y += pf.y;
          }
          yrow[c2] = y;
        }
      }
      __syncthreads();  // dn_s and the pair list are free
      if (rd + 1 < nrounds) issue(down, dn_s, &dn_bar, s1, min(n_act, s1 + stage_rows));
    }
  }
  dec_stamp(5);

  // ---- phase 5: cross-tile sum over the workspace ----------------------------------------
  {
    const int n4 = M * kc / 4, kc4 = kc / 4;
    for (int i = tid; i < n4; i += kDecThreads) {
      const int t = i / kc4, c4 = i - t * kc4;
      __stcg(reinterpret_cast<float4*>(ws_part + ((size_t)tile * M + t) * D + k_base) + c4,
             reinterpret_cast<const float4*>(yacc)[i]);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      unsigned int* cnt = ws_sync + 2 * crank;
      volatile unsigned int* rel = ws_sync + 2 * crank + 1;
      const unsigned int old = atomicAdd(cnt, 1u);
      if (old == (unsigned int)tiles - 1u) {
        *cnt = 0u;  // ready for the next launch
        __threadfence();
        *rel = release0_s + 1u;
      } else {
        uint32_t spins = 0;
        while (*rel == release0_s && ++spins < kDecSpinLimit) {
        }
        if (*rel == release0_s) dec_fail(6);
      }
      __threadfence();
    }
    __syncthreads();
    dec_stamp(6);
    const int n2 = M * kc / 2, kc2 = kc / 2;
    const int per = (n2 + tiles - 1) / tiles;
    const int lo = tile * per, hi = min(n2, lo + per);
    for (int i = lo + tid; i < hi; i += kDecThreads) {
      const int t = i / kc2, c2 = i - t * kc2;
      const float* src = ws_part + (size_t)t * D + k_base + 2 * c2;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
      for (int q = 0; q < tiles; ++q) {
        const float2 v = __ldcg(reinterpret_cast<const float2*>(src + (size_t)q * M * D));
        s0 += v.x;
        s1 += v.y;
      }
      *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * D + k_base + 2 * c2) =
          __floats2bfloat162_rn(s0, s1);
    }
  }
  dec_stamp(7);
}

// L2 prefetch of an arbitrary byte range (one bulk prefetch per 16 KB piece).
__global__ void l2_prefetch_kernel(const unsigned char* p, long long bytes) {
  const long long piece = 16384;
  const long long pieces = (bytes + piece - 1) / piece;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < pieces;
       i += (long long)gridDim.x * blockDim.x) {
    const long long off = i * piece;
    const long long n = (bytes - off < piece ? bytes - off : piece) & ~15ll;
    if (n > 0) l2_prefetch(p + off, (uint32_t)n);
  }
}

// ---- host side -------------------------------------------------------------------------
struct DecShape {
  int cl, stages, stage_rows;
  size_t smem;
};

constexpr int kDecStages = 4;

// Shape of a call, or false when the fused kernel does not serve it.
bool dec_shape(int64_t M, int64_t D, int64_t H, DecShape* s) {
  if (M < 1 || M > kDecTok || D < 256 || D > 8192 || D % 256 || H < 256 || H % 256) return false;
  const int tiles = (int)(H / kTileN);
  if (tiles < 1 || tiles > 255) return false;
  int cl = 4;
  if (tiles <= 16 && D % 512 == 0) cl = 8;  // a narrow d_ff shard: more CTAs per tile
  if (D % (cl * kStageK)) return false;
  const int kc = (int)(D / cl);
  const size_t ring = (size_t)kDecStages * kDecRingStageBytes;
  const size_t yacc = ((size_t)M * kc * 4 + 1023) & ~(size_t)1023;
  if (yacc + 4 * (size_t)kc * 4 > ring) return false;
  int rows = (int)((ring - yacc) / ((size_t)kc * 4));  // up slice + down slice per row
  const int by_pairs = (4096 / cl) / (int)M;
  if (rows > by_pairs) rows = by_pairs;
  if (rows > kDecMaxStageRows) rows = kDecMaxStageRows;
  if (rows < 4) return false;
  s->cl = cl;
  s->stages = kDecStages;
  s->stage_rows = rows;
  s->smem = ring + (size_t)(kc / kStageK) * 4096 + kDecPartBytes + kDecGtileBytes + 1024;
  return s->smem <= 227 * 1024;
}

template <int CL, bool GATED, bool HP>
int launch_decode(const DecShape& shp, const void* x, const void* gate, const float* bias,
                  const void* up, const void* down, void* packed, void* out, int64_t M, int64_t D,
                  int64_t H, int cf, void* workspace, const void* pf_ptr, int64_t pf_bytes,
                  cudaStream_t stream, bool probe_only) {
  auto kern = twell_decode_kernel<CL, kDecStages, GATED, HP>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, shp.smem, granted, "b200_twell_gated_mlp (decode)"))
    return rc;
  const int tiles = (int)(H / kTileN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * CL), 1, 1);
  cfg.blockDim = dim3(kDecThreads, 1, 1);
  cfg.dynamicSmemBytes = shp.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // The CTAs of a column slice wait for one another: the whole grid must be resident at once.
  static int max_clusters[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (max_clusters[dev] == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = -1;
    }
    max_clusters[dev] = n > 0 ? n : -1;
  }
  if (max_clusters[dev] < tiles)
    return fail(B200_EUNSUPPORTED,
                "b200_twell_gated_mlp (decode): %d clusters of %d CTAs are not resident at once "
                "(limit %d)", tiles, CL, max_clusters[dev]);
  if (probe_only) return B200_OK;
  CUtensorMap map_w, map_x;
  if (int rc = make_map(&map_w, gate, H, D, 128)) return rc;
  if (int rc = make_map(&map_x, x, M, D, kDecTok)) return rc;
  const int slab_w = kTileN / cf;
  unsigned int* words = reinterpret_cast<unsigned int*>(workspace);
  float* ws_part = reinterpret_cast<float*>(words + kDecCounterWords);
  cudaError_t e = cudaLaunchKernelEx(
      &cfg, kern, map_w, map_x, bias, static_cast<uint32_t*>(packed),
      reinterpret_cast<const __nv_bfloat16*>(up), reinterpret_cast<const __nv_bfloat16*>(down),
      reinterpret_cast<__nv_bfloat16*>(out), (int)M, (int)D, slab_w, tiles * slab_w,
      shp.stage_rows, ws_part, words + kDecSyncWord0,
      static_cast<const unsigned char*>(pf_ptr), (long long)pf_bytes);
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "b200_twell_gated_mlp (decode): launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

}  // namespace

// Bytes of workspace the fused decode kernel needs for a call (0 = the shape is not served).
size_t twell_decode_workspace_bytes(int64_t M, int64_t D, int64_t H) {
  DecShape s;
  if (!dec_shape(M, D, H, &s)) return 0;
  return kDecCounterWords * 4 + (size_t)(H / kTileN) * (size_t)M * (size_t)D * 4;
}

// B200_OK, B200_EUNSUPPORTED (shape / residency / workspace: use the two-kernel path) or an
// error.  probe_only: decide without launching.
int twell_decode_launch(bool gated, bool hp, const void* x, const void* gate, const float* bias,
                        const void* up, const void* down, void* packed, void* out, int64_t M,
                        int64_t D, int64_t H, int cf, void* workspace, size_t workspace_bytes,
                        const void* pf_ptr, int64_t pf_bytes, cudaStream_t stream,
                        bool probe_only) {
  DecShape s;
  if (!dec_shape(M, D, H, &s))
    return fail(B200_EUNSUPPORTED, "b200_twell_gated_mlp (decode): shape M=%lld D=%lld H=%lld "
                "is not served by the fused kernel", (long long)M, (long long)D, (long long)H);
  const size_t need = twell_decode_workspace_bytes(M, D, H);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(B200_EUNSUPPORTED, "b200_twell_gated_mlp (decode): workspace of %zu bytes needed",
                need);
#define B200_DEC(CLV)                                                                         \
  if (s.cl == CLV) {                                                                          \
    if (gated)                                                                                \
      return hp ? launch_decode<CLV, true, true>(s, x, gate, bias, up, down, packed, out, M, D, \
                                                 H, cf, workspace, pf_ptr, pf_bytes, stream,  \
                                                 probe_only)                                  \
                : launch_decode<CLV, true, false>(s, x, gate, bias, up, down, packed, out, M, \
                                                  D, H, cf, workspace, pf_ptr, pf_bytes,      \
                                                  stream, probe_only);                        \
    return launch_decode<CLV, false, false>(s, x, gate, bias, up, down, packed, out, M, D, H, \
                                            cf, workspace, pf_ptr, pf_bytes, stream,          \
                                            probe_only);                                      \
  }
  B200_DEC(4)
  B200_DEC(8)
#undef B200_DEC
  return fail(B200_EUNSUPPORTED, "b200_twell_gated_mlp (decode): cluster size %d", s.cl);
}

int l2_prefetch_launch(const void* p, int64_t bytes, cudaStream_t stream) {
  if (bytes <= 0) return B200_OK;
  const long long pieces = (bytes + 16383) / 16384;
  const int threads = 128;
  long long blocks = (pieces + threads - 1) / threads;
  if (blocks > 296) blocks = 296;
  l2_prefetch_kernel<<<(unsigned)blocks, threads, 0, stream>>>(
      static_cast<const unsigned char*>(p), (long long)bytes);
  return check_launch("b200_l2_prefetch");
}

int twell_decode_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_dec_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_dec_error, &zero, sizeof(int));
  return v;
}

#ifdef B200_TRACE
void twell_decode_trace(unsigned long long* out16) {
  cudaMemcpyFromSymbol(out16, g_dec_trace, sizeof(unsigned long long) * 16);
}
#endif

}  // namespace b200
