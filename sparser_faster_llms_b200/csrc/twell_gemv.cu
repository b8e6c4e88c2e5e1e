// One-token sparse FFN layer (sm_100a): gate projection as a CUDA-core GEMV with every
// neuron's dot product finished inside ONE warp, TwELL slab, and - in the fused form - the
// gathered up / down contraction of the stored entries in the same kernel.
//
// Why a separate form for one token.  The split-k pack kernels (mma.sync for up to 16 tokens,
// tcgen05 above) split d_model over a cluster and exchange fp32 partial tiles through
// distributed shared memory before a neuron's sign is known: two cluster barriers and a
// shared-memory pass after the weight stream has ended.  With a single token a warp can keep
// the token in registers and reduce a whole weight row by shuffles, so a neuron is decided
// 5 shuffles after its row arrived and the only exchange left is four counts per tile.
//
// grid = (H / 256) * CL CTAs of 256 threads in clusters of CL = 2, 4 or 8 (the largest whose
// clusters are all resident at once): a cluster owns one 256-neuron tile, a CTA 256 / CL
// neurons of it, a warp 32 / CL rows.  Phases:
//   1  weight rows -> registers (two rows per batch, next batch requested before the current
//      one is reduced), fp32 fma against the token, shuffle reduction, bias, sign;
//   2  the CTAs of a tile exchange their counts (one DSMEM word each, one cluster barrier),
//      slab words are written in ascending neuron order, the true count by rank 0;
//   3  (fused) for the CTA's stored entries, eight at a time: every warp requests its
//      d_model/8 column slice of the eight down rows, warp q also the whole up row of entry q
//      (the first batch already before the count exchange of phase 2 has completed);
//      u = x . up, h = z * u with the contraction kernel's roundings, then
//      acc[columns] += h * down: one memory round trip per eight entries;
//   4  (fused) each rank sums d_model / CL columns of the cluster's CTAs through DSMEM, the
//      tile's partial row goes to the workspace, and the last tile to arrive for a column
//      range (a counter per rank) adds the partial rows in tile order and writes the bf16 output.
// No spin waits: cluster barriers and last-arrival counters only.
//
// Replaces, for one token, TWELL_MLP::run_gated_mlp_layer* / run_mlp_layer*
// (custom_models/twell_modules/mlp_twell.cu:73-232) and the pack kernel alone
// (custom_models/twell_modules/matmul_d2t.cu:287-709, which needs M % 256 == 0).
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kGemvThreads = 256;
constexpr int kGemvCounterWord = 4064;                  // + cluster rank (0..7)
constexpr size_t kGemvCounterBlock = 4096;              // words before the partial rows

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p));
  return v;
}

__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// fp32 dot product of this lane's DI 16-byte chunks (exact bf16 products, two chains).
template <int DI>
__device__ __forceinline__ float dot_chunks(const uint4 (&w)[DI], const uint4 (&x)[DI]) {
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int it = 0; it < DI; ++it) {
    s0 = __fmaf_rn(bf_lo(w[it].x), bf_lo(x[it].x), s0);
    s1 = __fmaf_rn(bf_hi(w[it].x), bf_hi(x[it].x), s1);
    s0 = __fmaf_rn(bf_lo(w[it].y), bf_lo(x[it].y), s0);
    s1 = __fmaf_rn(bf_hi(w[it].y), bf_hi(x[it].y), s1);
    s0 = __fmaf_rn(bf_lo(w[it].z), bf_lo(x[it].z), s0);
    s1 = __fmaf_rn(bf_hi(w[it].z), bf_hi(x[it].z), s1);
    s0 = __fmaf_rn(bf_lo(w[it].w), bf_lo(x[it].w), s0);
    s1 = __fmaf_rn(bf_hi(w[it].w), bf_hi(x[it].w), s1);
  }
  return s0 + s1;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// The contraction kernel's u = x . up_row: per 256-column chunk a lane sums its 8 products
// (rounded to bf16 first unless HP), the chunk is reduced by shuffles, chunks add in order.
template <int DI, bool HP>
__device__ __forceinline__ float dot_up(const uint4 (&w)[DI], const uint4 (&x)[DI]) {
  float u = 0.f;
#pragma unroll
  for (int it = 0; it < DI; ++it) {
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&w[it]);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x[it]);
    float s = 0.f;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      if (HP) {
        const float2 wf = __bfloat1622float2(w2[p]), xf = __bfloat1622float2(x2[p]);
        s = __fmaf_rn(wf.x, xf.x, s);
        s = __fmaf_rn(wf.y, xf.y, s);
      } else {
        const float2 pf = __bfloat1622float2(__hmul2(x2[p], w2[p]));
        s += pf.x;
        s += pf.y;
      }
    }
    u += warp_sum(s);
  }
  return u;
}

// DI = d_model / 256 (8 or 16), CL = CTAs per cluster.  FUSED: phases 3 and 4 as well.  GATED
// only matters when FUSED (h = z * (x . up) against h = z).
template <int DI, int CL, bool GATED, bool HP, bool FUSED>
__global__ void __launch_bounds__(kGemvThreads, 1)
twell_gemv_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                  const float* __restrict__ bias, uint32_t* __restrict__ packed,
                  const __nv_bfloat16* __restrict__ up, const __nv_bfloat16* __restrict__ down,
                  __nv_bfloat16* __restrict__ out, int slab_w, int tiles,
                  float* __restrict__ ws_part, unsigned int* __restrict__ ws_words) {
  constexpr int D = DI * 256;
  constexpr int ROWS = kTileN / CL;          // neurons of this CTA: 128, 64 or 32
  constexpr int RPW = ROWS / 8;              // rows per warp
  constexpr int RB = DI == 8 ? 2 : 1;        // rows per register batch
  constexpr int NB = RPW / RB;               // batches per warp
  constexpr int NS = DI / 8;                 // 16-byte chunks of a warp's column slice
  constexpr int QCOLS = D / CL;              // columns a cluster rank owns in phase 4
  constexpr int NBAL = ROWS / 32;            // ballots that cover the CTA's neurons

  __shared__ float zs[ROWS];
  __shared__ int cnt_s[CL];
  __shared__ uint32_t ent_s[ROWS];
  __shared__ int n_ent_s;
  __shared__ float hs[8];
  __shared__ int is_last_s;
  __shared__ __align__(16) float red_s[FUSED ? CL * QCOLS : 4];  // [source rank][QCOLS]

  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  cluster.barrier_arrive();  // matched by barrier_wait() before the first remote store
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = (int)blockIdx.x / CL;
  const int nb = tile * kTileN + crank * ROWS;  // first neuron of this CTA
  const uint4* wrow = reinterpret_cast<const uint4*>(w + (size_t)(nb + warp * RPW) * D) + lane;

  // ---- phase 1 ---------------------------------------------------------------------
  uint4 buf[2][RB][DI];
  auto request = [&](uint4 (&b)[RB][DI], int row0) {
#pragma unroll
    for (int r = 0; r < RB; ++r)
#pragma unroll
      for (int it = 0; it < DI; ++it)
        b[r][it] = ldg_stream(wrow + (size_t)(row0 + r) * (D / 8) + it * 32);
  };
  pdl_wait();  // before any global read: the predecessor may have written the weights too
  request(buf[0], 0);
  uint4 xv[DI];
#pragma unroll
  for (int it = 0; it < DI; ++it)
    xv[it] = *(reinterpret_cast<const uint4*>(x) + it * 32 + lane);
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    if (b + 1 < NB) request(buf[(b + 1) & 1], (b + 1) * RB);
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      float z = warp_sum(dot_chunks<DI>(buf[b & 1][r], xv));
      const int i = b * RB + r;
      if (lane == 0) {
        if (bias != nullptr) z += bias[nb + warp * RPW + i];
        zs[warp * RPW + i] = z;
      }
    }
  }
  __syncthreads();

  // ---- phase 2 ---------------------------------------------------------------------
  cluster.barrier_wait();  // every CTA of the cluster is running
  uint32_t mask[NBAL];
  float zv[NBAL];
  int mine = 0;
  const int cap = slab_w - 1;
  if (warp == 0) {
#pragma unroll
    for (int b = 0; b < NBAL; ++b) {
      zv[b] = zs[b * 32 + lane];
      mask[b] = __ballot_sync(0xffffffffu, zv[b] > 0.f);
      mine += __popc(mask[b]);
    }
    if (lane < CL) cluster.map_shared_rank(cnt_s, lane)[crank] = mine;
    if (FUSED) {
      // Tentative entry list: this CTA's first `cap` positives.  The entries the slab keeps
      // are a prefix of it (entry k is stored iff prefix + k < cap), so their rows can be
      // requested before the counts have crossed the cluster.
      int before = 0;
#pragma unroll
      for (int b = 0; b < NBAL; ++b) {
        const int k = before + __popc(mask[b] & lanemask_lt());
        if (((mask[b] >> lane) & 1u) && k < cap)
          ent_s[k] = (uint32_t)(nb + b * 32 + lane) | (bf16_bits(zv[b]) << 16);
        before += __popc(mask[b]);
      }
      if (lane == 0) n_ent_s = min(mine, cap);
    }
  }

  // ---- phase 3, first half: row requests of a batch of eight entries ---------------------
  const uint4* up_lane = reinterpret_cast<const uint4*>(up) + lane;
  const uint4* down_slice = reinterpret_cast<const uint4*>(down) + warp * (D / 64) + lane;
  // Every warp: its column slice of the batch's down rows; warp q: the whole up row of entry q.
  auto request_rows = [&](int e0, int limit, uint4 (&dv)[8][NS], uint4 (&uv)[GATED ? DI : 1]) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const bool live = e0 + q < limit;
      const size_t roff = live ? (size_t)(ent_s[e0 + q] & 0xFFFFu) * (D / 8) : 0;
#pragma unroll
      for (int j = 0; j < NS; ++j)
        dv[q][j] = live ? ldg_stream(down_slice + roff + j * 32) : make_uint4(0u, 0u, 0u, 0u);
    }
    if (GATED && e0 + warp < limit) {  // the same decision in all lanes
      const size_t roff = (size_t)(ent_s[e0 + warp] & 0xFFFFu) * (D / 8);
#pragma unroll
      for (int it = 0; it < (GATED ? DI : 1); ++it) uv[it] = ldg_stream(up_lane + roff + it * 32);
    }
  };
  uint4 dv0[8][NS];
  uint4 uv0[GATED ? DI : 1];
  if (FUSED) {
    __syncthreads();  // tentative list visible
    request_rows(0, n_ent_s, dv0, uv0);
  }

  cluster.sync();  // counts delivered
  if (warp == 0) {
    int prefix = 0, total = 0;
#pragma unroll
    for (int q = 0; q < CL; ++q) {
      const int c = cnt_s[q];
      if (q < crank) prefix += c;
      total += c;
    }
    uint32_t* slab = packed + (size_t)tile * slab_w;
    if (crank == 0 && lane == 0) slab[0] = (uint32_t)total;
    int before = 0;  // positives of this CTA in lower ballots
#pragma unroll
    for (int b = 0; b < NBAL; ++b) {
      const int k = before + __popc(mask[b] & lanemask_lt());
      if (((mask[b] >> lane) & 1u) && prefix + k < cap)
        slab[1 + prefix + k] = (uint32_t)(nb + b * 32 + lane) | (bf16_bits(zv[b]) << 16);
      before += __popc(mask[b]);
    }
    if (lane == 0) n_ent_s = max(0, min(mine, cap - prefix));  // entries the slab keeps
  }
  if (!FUSED) return;
  __syncthreads();

  // ---- phase 3, second half ------------------------------------------------------------
  const int n = n_ent_s;
  float acc[NS * 8];
#pragma unroll
  for (int c = 0; c < NS * 8; ++c) acc[c] = 0.f;
  auto consume_rows = [&](int e0, uint4 (&dv)[8][NS], uint4 (&uv)[GATED ? DI : 1]) {
    float h = 0.f;
    if (e0 + warp < n) {  // the same decision in all lanes
      const uint32_t word = ent_s[e0 + warp];
      const __nv_bfloat16 gval = __ushort_as_bfloat16((unsigned short)(word >> 16));
      if (GATED) {
        const float u = dot_up<DI, HP>(reinterpret_cast<uint4 (&)[DI]>(uv), xv);
        h = HP ? __bfloat162float(gval) * u
               : __bfloat162float(__hmul(gval, __float2bfloat16_rn(u)));
      } else {
        h = __bfloat162float(gval);
      }
    }
    if (lane == 0) hs[warp] = h;
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float hq = hs[q];  // 0 for a padding entry or one the slab dropped
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&dv[q][j]);
        if (HP) {
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const float2 wf = __bfloat1622float2(w2[p]);
            acc[j * 8 + 2 * p] = __fmaf_rn(wf.x, hq, acc[j * 8 + 2 * p]);
            acc[j * 8 + 2 * p + 1] = __fmaf_rn(wf.y, hq, acc[j * 8 + 2 * p + 1]);
          }
        } else {
          const __nv_bfloat162 hb2 = __float2bfloat162_rn(hq);  // hq is bf16-representable
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const float2 pf = __bfloat1622float2(__hmul2(hb2, w2[p]));
            acc[j * 8 + 2 * p] += pf.x;
            acc[j * 8 + 2 * p + 1] += pf.y;
          }
        }
      }
    }
    __syncthreads();  // hs is rewritten by the next batch
  };
  if (n > 0) consume_rows(0, dv0, uv0);
  for (int e0 = 8; e0 < n; e0 += 8) {
    uint4 dv[8][NS];
    uint4 uv[GATED ? DI : 1];
    request_rows(e0, n, dv, uv);
    consume_rows(e0, dv, uv);
  }

  // ---- phase 4 ---------------------------------------------------------------------
  {
    constexpr int WPO = 8 / CL;  // warps per owner when CL <= 8 warps' slices divide evenly
    static_assert(CL == 2 || CL == 4 || CL == 8, "cluster size");
    const int owner = warp / WPO;  // the rank that owns this warp's columns
    float* dst = cluster.map_shared_rank(red_s, owner) + crank * QCOLS + (warp % WPO) * (D / 8) +
                 lane * 8;
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      *reinterpret_cast<float4*>(dst + j * 256) =
          make_float4(acc[j * 8], acc[j * 8 + 1], acc[j * 8 + 2], acc[j * 8 + 3]);
      *reinterpret_cast<float4*>(dst + j * 256 + 4) =
          make_float4(acc[j * 8 + 4], acc[j * 8 + 5], acc[j * 8 + 6], acc[j * 8 + 7]);
    }
  }
  cluster.sync();
  // column pairs of this rank's range: pair p covers columns 2p, 2p + 1
  constexpr int PAIRS = QCOLS / 2;
  constexpr int PPT = (PAIRS + kGemvThreads - 1) / kGemvThreads;  // pairs per thread: 1..4
  float2 sum[PPT];
#pragma unroll
  for (int i = 0; i < PPT; ++i) {
    sum[i] = make_float2(0.f, 0.f);
    const int p = tid + i * kGemvThreads;
    if (p < PAIRS) {
#pragma unroll
      for (int s = 0; s < CL; ++s) {
        const float2 v = *reinterpret_cast<const float2*>(red_s + s * QCOLS + 2 * p);
        sum[i].x += v.x;
        sum[i].y += v.y;
      }
    }
  }
  const int col0 = crank * QCOLS;
  unsigned int* counter = ws_words + kGemvCounterWord + crank;
  if (tiles > 1) {
#pragma unroll
    for (int i = 0; i < PPT; ++i) {
      const int p = tid + i * kGemvThreads;
      if (p < PAIRS)
        __stcg(reinterpret_cast<float2*>(ws_part + (size_t)tile * D + col0 + 2 * p), sum[i]);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last_s = atomicAdd(counter, 1u) == (unsigned)(tiles - 1);
    __syncthreads();
    if (!is_last_s) return;
    __threadfence();
#pragma unroll
    for (int i = 0; i < PPT; ++i) sum[i] = make_float2(0.f, 0.f);
    constexpr int kRowsInFlight = 32 / PPT;  // partial rows whose loads are in flight together
#pragma unroll kRowsInFlight
    for (int t = 0; t < tiles; ++t) {
#pragma unroll
      for (int i = 0; i < PPT; ++i) {
        const int p = tid + i * kGemvThreads;
        if (p < PAIRS) {
          const float2 v =
              __ldcg(reinterpret_cast<const float2*>(ws_part + (size_t)t * D + col0 + 2 * p));
          sum[i].x += v.x;
          sum[i].y += v.y;
        }
      }
    }
    if (tid == 0) *counter = 0u;  // ready for the next launch
  }
#pragma unroll
  for (int i = 0; i < PPT; ++i) {
    const int p = tid + i * kGemvThreads;
    if (p < PAIRS)
      *reinterpret_cast<uint32_t*>(out + col0 + 2 * p) =
          bf16_bits(sum[i].x) | (bf16_bits(sum[i].y) << 16);
  }
}

template <int CL>
void gemv_launch_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int tiles,
                        cudaStream_t stream) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3((unsigned)(tiles * CL), 1, 1);
  cfg->blockDim = dim3(kGemvThreads, 1, 1);
  cfg->dynamicSmemBytes = 0;
  cfg->stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
}

// Clusters of CL CTAs of this kernel that can be resident at once (cached per device).
template <int DI, int CL, bool GATED, bool HP, bool FUSED>
int gemv_resident_clusters() {
  static int cache[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (cache[dev] == 0) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    gemv_launch_config<CL>(&cfg, attr, 1, nullptr);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, twell_gemv_kernel<DI, CL, GATED, HP, FUSED>, &cfg) !=
            cudaSuccess ||
        n <= 0) {
      cudaGetLastError();
      n = -1;  // unknown: treated as "does not fit"
    }
    cache[dev] = n;
  }
  return cache[dev];
}

template <int DI, int CL, bool GATED, bool HP, bool FUSED>
int launch_gemv(const void* x, const void* w, const float* bias, void* packed, const void* up,
                const void* down, void* out, int64_t H, int cf, void* workspace,
                cudaStream_t stream) {
  const int tiles = (int)(H / kTileN);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  gemv_launch_config<CL>(&cfg, attr, tiles, stream);
  cfg.numAttrs = add_pdl_attribute(attr, 1, 1);
  unsigned int* words = reinterpret_cast<unsigned int*>(workspace);
  float* ws_part = FUSED ? reinterpret_cast<float*>(words + kGemvCounterBlock) : nullptr;
  cudaError_t e = cudaLaunchKernelEx(
      &cfg, twell_gemv_kernel<DI, CL, GATED, HP, FUSED>,
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w), bias,
      reinterpret_cast<uint32_t*>(packed), reinterpret_cast<const __nv_bfloat16*>(up),
      reinterpret_cast<const __nv_bfloat16*>(down), reinterpret_cast<__nv_bfloat16*>(out),
      kTileN / cf, tiles, ws_part, words);
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "b200_twell (one-token form): launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

// The largest cluster size whose clusters are all resident in one wave; 2 when none is (the
// grid then runs in more than one wave, which every cluster size would).
template <int DI, bool GATED, bool HP, bool FUSED>
int launch_gemv_any(const void* x, const void* w, const float* bias, void* packed,
                    const void* up, const void* down, void* out, int64_t H, int cf,
                    void* workspace, cudaStream_t stream) {
  const int tiles = (int)(H / kTileN);
  static const int forced = [] {
    const char* e = getenv("B200_ONE_TOKEN_CLUSTER");
    return e != nullptr ? atoi(e) : 0;
  }();
#define B200_GEMV_CL(C) \
  launch_gemv<DI, C, GATED, HP, FUSED>(x, w, bias, packed, up, down, out, H, cf, workspace, stream)
  if (forced == 8) return B200_GEMV_CL(8);
  if (forced == 4) return B200_GEMV_CL(4);
  if (forced == 2) return B200_GEMV_CL(2);
  if (tiles <= gemv_resident_clusters<DI, 8, GATED, HP, FUSED>()) return B200_GEMV_CL(8);
  if (tiles <= gemv_resident_clusters<DI, 4, GATED, HP, FUSED>()) return B200_GEMV_CL(4);
  return B200_GEMV_CL(2);
#undef B200_GEMV_CL
}

template <int DI>
int dispatch_gemv(bool fused, bool gated, bool hp, const void* x, const void* w,
                  const float* bias, void* packed, const void* up, const void* down, void* out,
                  int64_t H, int cf, void* workspace, cudaStream_t stream) {
#define B200_GEMV(G, P, F) \
  launch_gemv_any<DI, G, P, F>(x, w, bias, packed, up, down, out, H, cf, workspace, stream)
  if (!fused) return B200_GEMV(false, false, false);
  if (!gated) return hp ? B200_GEMV(false, true, true) : B200_GEMV(false, false, true);
  return hp ? B200_GEMV(true, true, true) : B200_GEMV(true, false, true);
#undef B200_GEMV
}

}  // namespace

// One token, d_model 2048 or 4096.
bool twell_gemv_serves(int64_t M, int64_t D, int64_t H) {
  return M == 1 && (D == 2048 || D == 4096) && H >= 256 && H % 256 == 0;
}

// Fused form: the 4096-word block (words 4064..4071 are the per-rank counters) followed by
// [tiles][D] fp32 partial rows.
size_t twell_gemv_workspace_bytes(int64_t D, int64_t H) {
  return kGemvCounterBlock * 4 + (size_t)(H / kTileN) * (size_t)D * 4;
}

// Slab only.
int twell_gemv_pack(const void* x, const void* w, const float* bias, void* packed, int64_t D,
                    int64_t H, int cf, cudaStream_t stream) {
  if (!twell_gemv_serves(1, D, H))
    return fail(B200_EUNSUPPORTED, "b200_twell_pack (one-token form): shape not served");
  return D == 2048 ? dispatch_gemv<8>(false, false, false, x, w, bias, packed, nullptr, nullptr,
                                      nullptr, H, cf, nullptr, stream)
                   : dispatch_gemv<16>(false, false, false, x, w, bias, packed, nullptr, nullptr,
                                       nullptr, H, cf, nullptr, stream);
}

// Slab and output.  gated = false: w is the up projection and h = relu(x . w).
int twell_gemv_layer(bool gated, bool hp, const void* x, const void* w, const float* bias,
                     const void* up, const void* down, void* packed, void* out, int64_t D,
                     int64_t H, int cf, void* workspace, size_t workspace_bytes,
                     cudaStream_t stream) {
  if (!twell_gemv_serves(1, D, H))
    return fail(B200_EUNSUPPORTED, "b200_twell_gated_mlp (one-token form): shape not served");
  if (workspace == nullptr || workspace_bytes < twell_gemv_workspace_bytes(D, H))
    return fail(B200_EUNSUPPORTED,
                "b200_twell_gated_mlp (one-token form): workspace of %zu bytes needed",
                twell_gemv_workspace_bytes(D, H));
  // With more tiles than clusters of 4 can be resident the kernel would run clusters of 2,
  // whose two ranks then add all partial rows by themselves: measured slower than the pack
  // form followed by the contraction kernel (D 4096, H 16384: 35.9 against 34.8 us).
  const int fit4 = D == 2048 ? gemv_resident_clusters<8, 4, true, false, true>()
                             : gemv_resident_clusters<16, 4, true, false, true>();
  if (H / kTileN > fit4)
    return fail(B200_EUNSUPPORTED,
                "b200_twell_gated_mlp (one-token form): %lld tiles exceed the %d resident "
                "clusters of 4",
                (long long)(H / kTileN), fit4);
  return D == 2048 ? dispatch_gemv<8>(true, gated, hp, x, w, bias, packed, up, down, out, H, cf,
                                      workspace, stream)
                   : dispatch_gemv<16>(true, gated, hp, x, w, bias, packed, up, down, out, H, cf,
                                       workspace, stream);
}

}  // namespace b200
