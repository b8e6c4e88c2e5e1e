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

constexpr int kDecThreads = 512;  // warp 0 producer, 1 mma, 2..5 epilogue; all 16 from phase 3
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kDecTok = 32;                   // token rows of the MMA tile (padded)
constexpr int kDecPartStride = kTileN + 4;    // floats per row of the partial-sum inbox
constexpr int kDecRingStageBytes = 2 * kATileBytes;  // two 128-neuron halves of a k step
constexpr int kDecPartBytes = kDecTok * kDecPartStride * 4;
constexpr int kDecGtileBytes = kDecTok * kTileN * 2;
constexpr int kDecMaxBufs = 4;                // staging buffers for up / down row slices
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
  static constexpr int kPairMax = 4096 / CL;  // (neuron, token) pairs per exchange of u
  static constexpr int kChunkRows = kPairMax / 32 < 32 ? kPairMax / 32 : 32;  // rows per chunk
  static constexpr int kChunks = kTileN / kChunkRows;
  float uin[CL][kPairMax];                    // slice sums of u, one row per source CTA
  float h[kPairMax];
  unsigned char ptok[kPairMax];               // token of a pair
  unsigned char pslot[kPairMax];              // active slot of a pair - first slot of the exchange
  uint32_t mlist[kTileN];                     // token mask of active slot
  int poff[kTileN + 1];                       // exclusive prefix of popc(mlist)
  unsigned short nlist[kTileN];               // neuron (inside the tile) of active slot
  uint32_t rowmask[kChunks][32];              // per chunk and token: rows of the chunk it fires
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
                    int slab_w, int row_words, int nbuf, float* ws_part,
                    unsigned int* ws_sync, const unsigned char* pf_ptr, long long pf_bytes) {
  constexpr int NTOK = kDecTok;
  constexpr int TOK = NTOK / CL;  // tokens finalised by this CTA
  constexpr uint32_t kTmemCols = 2 * NTOK;
  constexpr uint32_t kIdesc = umma_idesc(128, NTOK);
  constexpr int EPT = TOK * kTileN / 128;
  constexpr int PMAX = DecLists<CL>::kPairMax;
  constexpr int CH = DecLists<CL>::kChunkRows;
  constexpr uint32_t FULL = 0xffffffffu;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar,
      buf_bar[kDecMaxBufs];
  __shared__ uint32_t tmem_slot;
  __shared__ int cnt_chunk[TOK][8];
  __shared__ int warp_cnt[8];
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
  const int row_bytes = kc * 2;
  const int buf_bytes = CH * row_bytes;
  unsigned char* stage0 = ring + (((size_t)M * kc * 4 + 1023) & ~(size_t)1023);

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
#pragma unroll
    for (int b = 0; b < kDecMaxBufs; ++b) mbar_init(&buf_bar[b], 1);
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
    // L2 prefetch of the caller's range (e.g. the next layer's gate matrix): this CTA's share
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
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float v[32];
      tmem_ld32(lane_addr + (uint32_t)(half * NTOK), v);
#pragma unroll
      for (int c = 0; c < NTOK; ++c) {
        const int owner = c / TOK, tl = c % TOK;
        float* dst = cluster.map_shared_rank(part, owner) +
                     (size_t)(crank * TOK + tl) * kDecPartStride + nl + half * 128;
        dst[0] = v[c];
      }
    }
  } else {
    cluster.barrier_wait();  // B0 for the other warps
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster.sync();  // B1: all partials delivered; every CTA's MMAs are complete
  dec_stamp(2);

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
    dec_stamp(8);
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
    dec_stamp(9);
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
    dec_stamp(10);
  } else {
    // the ring is free (B1): clear the accumulator while the epilogue warps finalise
    const int n4 = M * kc / 4;
    const int t4 = (warp < 2 ? warp : warp - 4) * 32 + lane;  // 0..383 over the other 12 warps
    for (int i = t4; i < n4; i += kDecThreads - 128)
      reinterpret_cast<float4*>(yacc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  cluster.sync();  // B2: gate tile complete in every CTA; inbox no longer read
  dec_stamp(3);

  // ---- phase 3: lists (identical in every CTA of the cluster) --------------------------
  int n_act = 0;
  {
    uint32_t tmask = 0;
    uint32_t ball = 0;
    if (tid < kTileN) {
#pragma unroll 8
      for (int t = 0; t < NTOK; ++t)
        if (gtile[t * kTileN + tid] != 0) tmask |= 1u << t;
      ball = __ballot_sync(FULL, tmask != 0);
      if (lane == 0) warp_cnt[warp] = __popc(ball);
    }
    __syncthreads();
    int base = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int c = warp_cnt[w];
      if (w < warp) base += c;
      n_act += c;
    }
    if (tid < kTileN && tmask != 0) {
      const int slot = base + __popc(ball & lanemask_lt());
      L.nlist[slot] = (unsigned short)tid;
      L.mlist[slot] = tmask;
    }
    __syncthreads();
    // exclusive prefix of the pair counts over the slots (thread = slot)
    int c = 0, inc = 0;
    if (tid < kTileN) {
      c = tid < n_act ? __popc(L.mlist[tid]) : 0;
      inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(FULL, inc, o);
        if (lane >= o) inc += v;
      }
    }
    __syncthreads();  // every thread has read warp_cnt
    if (tid < kTileN && lane == 31) warp_cnt[warp] = inc;
    __syncthreads();
    if (tid < kTileN) {
      int wbase = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w)
        if (w < warp) wbase += warp_cnt[w];
      L.poff[tid] = wbase + inc - c;
      if (tid == kTileN - 1) L.poff[kTileN] = wbase + inc;
    }
    // per chunk and token: which rows of the chunk the token fires (one warp per chunk)
    const int nch_all = (n_act + CH - 1) / CH;
    for (int ch = warp; ch < nch_all; ch += kDecWarps) {
      const int s = ch * CH + lane;
      const uint32_t m = (lane < CH && s < n_act) ? L.mlist[s] : 0u;
      uint32_t mine = 0;
#pragma unroll
      for (int t = 0; t < 32; ++t) {
        const uint32_t b = __ballot_sync(FULL, (m >> t) & 1u);
        if (lane == t) mine = b;
      }
      L.rowmask[ch][lane] = mine;
    }
    __syncthreads();
  }
  dec_stamp(4);

  // ---- phase 4: contraction ----------------------------------------------------------------
  // The active rows are walked in chunks of CH.  An "exchange" is a run of chunks whose pairs
  // fit the u inbox (normally the whole tile): its up chunks stream through the staging
  // buffers for pass A, one cluster barrier publishes the slice sums, then its down chunks
  // stream through the same buffers for pass B.
  {
    const int nch = (n_act + CH - 1) / CH;
    const size_t w_row0 = (size_t)tile * kTileN * D + (size_t)k_base;  // element offset
    int item_g = 0;   // items issued / consumed so far: buffer = item % nbuf
    int c0 = 0;
    bool first_exchange = true;
    while (c0 < nch) {
      const int pbase = L.poff[c0 * CH];
      int c1 = c0 + 1;
      while (c1 < nch && L.poff[min(n_act, (c1 + 1) * CH)] - pbase <= PMAX) ++c1;
      const int sA = c0 * CH, sB = min(n_act, c1 * CH);
      const int np = L.poff[sB] - pbase;
      const int ncs = c1 - c0;
      const int nitems = GATED ? 2 * ncs : ncs;
      // item i of this exchange: up chunk c0 + i (i < ncs, gated) else down chunk
      auto issue = [&](int i) {
        if (warp == 0) {
          const bool is_up = GATED && i < ncs;
          const int ch = c0 + (is_up ? i : i - (GATED ? ncs : 0));
          const int s0 = ch * CH, s1 = min(n_act, s0 + CH);
          const int b = (item_g + i) % nbuf;
          const __nv_bfloat16* w = is_up ? up : down;
          unsigned char* dst = stage0 + (size_t)b * buf_bytes;
          if (lane == 0) mbar_expect_tx(&buf_bar[b], (uint32_t)((s1 - s0) * row_bytes));
          __syncwarp();
          for (int s = s0 + lane; s < s1; s += 32)
            bulk_g2s(dst + (size_t)(s - s0) * row_bytes, w + w_row0 + (size_t)L.nlist[s] * D,
                     (uint32_t)row_bytes, &buf_bar[b]);
        }
      };
      for (int i = 0; i < nbuf && i < nitems; ++i) issue(i);
      // pair list of the exchange (thread = slot)
      for (int s = sA + tid; s < sB; s += kDecThreads) {
        uint32_t m = L.mlist[s];
        int p = L.poff[s] - pbase;
        while (m) {
          const int t = __ffs(m) - 1;
          m &= m - 1;
          L.ptok[p] = (unsigned char)t;
          L.pslot[p] = (unsigned char)(s - sA);
          ++p;
        }
      }
      __syncthreads();
      if (!GATED) {  // plain down projection: h is the stored value itself
        for (int p = tid; p < np; p += kDecThreads) {
          const int t = L.ptok[p];
          const int n = L.nlist[sA + L.pslot[p]];
          L.h[p] = __bfloat162float(__ushort_as_bfloat16(gtile[t * kTileN + n]));
        }
        __syncthreads();
      }
      for (int i = 0; i < nitems; ++i) {
        const int gi = item_g + i;
        const int b = gi % nbuf;
        const bool is_up = GATED && i < ncs;
        const int ch = c0 + (is_up ? i : i - (GATED ? ncs : 0));
        const int s0 = ch * CH, s1 = min(n_act, s0 + CH);
        const unsigned char* buf = stage0 + (size_t)b * buf_bytes;
        if (!mbar_wait(&buf_bar[b], (uint32_t)(gi / nbuf) & 1u)) dec_fail(4);
        if (is_up) {
          if (i == 0 && !first_exchange) cluster.barrier_wait();  // Bb: previous uin is read
          // pass A: 8 lanes per pair, 4 pairs per warp; this CTA's slice of the dot product
          const int pa = L.poff[s0] - pbase, pb = L.poff[s1] - pbase;
          const int sub = lane & 7;
          for (int pw = pa + warp * 4; pw < pb; pw += kDecWarps * 4) {
            const int p = pw + (lane >> 3);
            const bool valid = p < pb;
            const int t = valid ? L.ptok[p] : 0;
            const int r = valid ? (int)L.pslot[p] - (s0 - sA) : 0;
            const unsigned char* wrow = buf + (size_t)r * row_bytes + sub * 16;
            const unsigned char* xrow = xs + t * 128 + ((sub ^ (t & 7)) << 4);
            float sa = 0.f, sb = 0.f;
            for (int j = 0; j < ksteps; ++j) {
              const uint4 xv = *reinterpret_cast<const uint4*>(xrow + (size_t)j * 4096);
              const uint4 wv = *reinterpret_cast<const uint4*>(wrow + j * 128);
              const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
              const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (HP) {
                  const float2 wf = __bfloat1622float2(w2[e]), xf = __bfloat1622float2(x2[e]);
                  sa = __fmaf_rn(wf.x, xf.x, sa);
                  sb = __fmaf_rn(wf.y, xf.y, sb);
                } else {
                  const float2 pf = __bfloat1622float2(__hmul2(x2[e], w2[e]));
                  sa += pf.x;
                  sb += pf.y;
                }
              }
            }
            float sum = sa + sb;
            sum += __shfl_xor_sync(FULL, sum, 4);
            sum += __shfl_xor_sync(FULL, sum, 2);
            sum += __shfl_xor_sync(FULL, sum, 1);
            if (valid && sub < CL)
              cluster.map_shared_rank(&L.uin[0][0], sub)[crank * PMAX + p] = sum;
          }
        } else {
          // pass B: token-major inside the chunk.  A group of kc / 8 threads owns one token at
          // a time (thread = 8 columns): y[t, cols] += h * down[row, cols] for the rows the
          // token fires, then the next token of the group.
          const int tpg = kc / 8;                    // threads per group
          const int groups = kDecThreads / tpg;
          const int g = tid / tpg, cl8 = (tid - g * tpg) * 8;
          if (g < groups) {
            for (int t = g; t < M; t += groups) {
              uint32_t m = L.rowmask[ch][t];
              if (m == 0) continue;
              float* yrow = yacc + (size_t)t * kc + cl8;
              float4 y0 = *reinterpret_cast<const float4*>(yrow);
              float4 y1 = *reinterpret_cast<const float4*>(yrow + 4);
              const uint32_t below = (1u << t) - 1u;
              while (m) {
                const int r = __ffs(m) - 1;
                m &= m - 1;
                const int s = s0 + r;
                const int p = L.poff[s] - pbase + __popc(L.mlist[s] & below);
                const float hv = L.h[p];
                const uint4 wv = *reinterpret_cast<const uint4*>(buf + (size_t)r * row_bytes +
                                                                 cl8 * 2);
                const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
                if (HP) {
                  const float2 a = __bfloat1622float2(w2[0]), bq = __bfloat1622float2(w2[1]),
                               cq = __bfloat1622float2(w2[2]), dq = __bfloat1622float2(w2[3]);
                  y0.x = __fmaf_rn(a.x, hv, y0.x);
                  y0.y = __fmaf_rn(a.y, hv, y0.y);
                  y0.z = __fmaf_rn(bq.x, hv, y0.z);
                  y0.w = __fmaf_rn(bq.y, hv, y0.w);
                  y1.x = __fmaf_rn(cq.x, hv, y1.x);
                  y1.y = __fmaf_rn(cq.y, hv, y1.y);
                  y1.z = __fmaf_rn(dq.x, hv, y1.z);
                  y1.w = __fmaf_rn(dq.y, hv, y1.w);
                } else {
                  const __nv_bfloat162 hb2 = __float2bfloat162_rn(hv);  // h is bf16-representable
                  const float2 a = __bfloat1622float2(__hmul2(hb2, w2[0])),
                               bq = __bfloat1622float2(__hmul2(hb2, w2[1])),
                               cq = __bfloat1622float2(__hmul2(hb2, w2[2])),
                               dq = __bfloat1622float2(__hmul2(hb2, w2[3]));
                  y0.x += a.x;
                  y0.y += a.y;
                  y0.z += bq.x;
                  y0.w += bq.y;
                  y1.x += cq.x;
                  y1.y += cq.y;
                  y1.z += dq.x;
                  y1.w += dq.y;
                }
              }
              *reinterpret_cast<float4*>(yrow) = y0;
              *reinterpret_cast<float4*>(yrow + 4) = y1;
            }
          }
        }
        __syncthreads();  // the buffer is free
        if (i + nbuf < nitems) issue(i + nbuf);
        if (GATED && i == ncs - 1) {
          cluster.sync();  // Ba: the slice sums of the exchange are in every CTA
          for (int p = tid; p < np; p += kDecThreads) {
            const int t = L.ptok[p];
            const int n = L.nlist[sA + L.pslot[p]];
            const __nv_bfloat16 gv = __ushort_as_bfloat16(gtile[t * kTileN + n]);
            float u = 0.f;
#pragma unroll
            for (int r = 0; r < CL; ++r) u += L.uin[r][p];
            L.h[p] = HP ? __bfloat162float(gv) * u
                        : __bfloat162float(__hmul(gv, __float2bfloat16_rn(u)));
          }
          __syncthreads();
          if (c1 < nch) cluster.barrier_arrive();  // Bb: this exchange's uin has been read
        }
      }
      item_g += nitems;
      c0 = c1;
      first_exchange = false;
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
    const int per = (n4 + tiles - 1) / tiles;
    const int lo = tile * per, hi = min(n4, lo + per);
    for (int i = lo + tid; i < hi; i += kDecThreads) {
      const int t = i / kc4, c4 = i - t * kc4;
      const float4* src = reinterpret_cast<const float4*>(ws_part + (size_t)t * D + k_base) + c4;
      const size_t qstride = (size_t)M * D / 4;
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      int q = 0;
      for (; q + 16 <= tiles; q += 16) {
        float4 v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __ldcg(src + (size_t)(q + j) * qstride);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          s.x += v[j].x;
          s.y += v[j].y;
          s.z += v[j].z;
          s.w += v[j].w;
        }
      }
      for (; q < tiles; ++q) {
        const float4 v = __ldcg(src + (size_t)q * qstride);
        s.x += v.x;
        s.y += v.y;
        s.z += v.z;
        s.w += v.w;
      }
      __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * D + k_base + 4 * c4);
      o[0] = __floats2bfloat162_rn(s.x, s.y);
      o[1] = __floats2bfloat162_rn(s.z, s.w);
    }
  }
  dec_stamp(7);
  // TMEM is released last: nothing above waits for it.
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
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
  int cl, stages, nbuf;
  size_t smem;
};

constexpr int kDecStages = 4;

// Shape of a call, or false when the fused kernel does not serve it.
bool dec_shape(int64_t M, int64_t D, int64_t H, DecShape* s) {
  if (M < 1 || M > kDecTok || D < 256 || D > 8192 || D % 256 || H < 256 || H % 256) return false;
  const int tiles = (int)(H / kTileN);
  if (tiles < 1 || tiles > 255) return false;
  int cl = 4;
  if (tiles <= 8 && D % 512 == 0) cl = 8;  // a narrow d_ff shard: more CTAs per tile
  if (D % (cl * kStageK)) return false;
  const int kc = (int)(D / cl);
  if (kDecThreads % (kc / 8)) return false;  // pass B: groups of kc / 8 threads
  const int chunk_rows = (4096 / cl) / 32 < 32 ? (4096 / cl) / 32 : 32;
  const size_t ring = (size_t)kDecStages * kDecRingStageBytes;
  const size_t yacc = ((size_t)M * kc * 4 + 1023) & ~(size_t)1023;
  const size_t buf = (size_t)chunk_rows * kc * 2;
  if (yacc + 2 * buf > ring) return false;
  int nbuf = (int)((ring - yacc) / buf);
  if (nbuf > kDecMaxBufs) nbuf = kDecMaxBufs;
  s->cl = cl;
  s->stages = kDecStages;
  s->nbuf = nbuf;
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
      shp.nbuf, ws_part, words + kDecSyncWord0,
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
