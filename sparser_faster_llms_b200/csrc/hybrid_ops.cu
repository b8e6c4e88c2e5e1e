// Kernels of the hybrid sparse training operator (forward and backward).
//
// The reference keeps the gate pattern in a row-ELL container with a dense tail
// for overflow rows (hybrid_sp_t, custom_models/hybrid_modules/hybrid_sp.h:32-60)
// and converts to it from the TwELL slabs (wgmma_gemm.cu:40-140).  Here every
// sparse operand of the operator stays in TwELL slab layout: the pattern P is
// the pack kernel's output, and R, T, dR, dU are slab-shaped arrays whose word
// (row, tile, slot) holds  col | bf16(value) << 16  for the same entry as P.
// One layout means no conversion kernels, no tail bookkeeping and no host
// synchronisation; row products reuse the TwELL contraction kernel.
//
//   hyb_sddmm_kernel<false>  R = (X K^T) on P's pattern, T = R*P, per-row l1 / nnz
//                            (reference: dense_ab_as_sparse_hybrid_unified_optimized,
//                             hybrid_sp.cu:711-805; sparse_elementwise_product, :1480-1587)
//   hyb_sddmm_kernel<true>   dT = (gR V^T) on the pattern (+ L1 shift), dR = dT*P, dU = dT*R
//                            (hybrid_sp.cu:711-805, :1754-1779, :1480-1587, :1590-1664)
//   hyb_count / hyb_scan / hyb_fill   column lists of the pattern (replaces the atomic
//                            scatter transpose, hybrid_sp.cu:1042-1214)
//   hyb_spmm_t_kernel        out[j,:] = sum over rows of value(row, j) * B[row,:]
//                            (the transposed products dK, dG, dV of custom_op.cpp:261-269)
//   hyb_ell_spmm_raw_kernel  row-ELL x dense (ell_spmm_raw, custom_op.cpp:313)
#include <cooperative_groups.h>

#include <initializer_list>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kSddmmThreads = 256;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float bf16_hi(uint32_t word) {
  return __uint_as_float(word & 0xFFFF0000u);
}

__device__ __forceinline__ float bf16_mul(float a, float b) {  // __hmul on bf16 operands
  return __bfloat162float(__hmul(__float2bfloat16_rn(a), __float2bfloat16_rn(b)));
}

// One CTA per row.  A row (D bf16) sits in shared memory; warp w takes tiles w, w+8, ...
// and, entry by entry, dots the row with Bm[col, :] (fp32 fma, butterfly sum).
template <bool BWD>
__global__ void __launch_bounds__(kSddmmThreads)
hyb_sddmm_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ Bm,
                 const uint32_t* __restrict__ P, const uint32_t* __restrict__ Rin,
                 uint32_t* __restrict__ out1, uint32_t* __restrict__ out2,
                 float* __restrict__ row_l1, int* __restrict__ row_nnz, int* __restrict__ row_drop,
                 const float* __restrict__ l1_grad, float inv_m, int D, int tiles, int W) {
  const float shift = (BWD && l1_grad != nullptr) ? __ldg(l1_grad) * inv_m : 0.f;
  extern __shared__ __align__(16) unsigned char smem[];
  __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(smem);
  __shared__ float l1_warp[kSddmmThreads / 32];
  __shared__ int nnz_warp[kSddmmThreads / 32], drop_warp[kSddmmThreads / 32];

  const int row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t rw = (size_t)tiles * W;
  const uint32_t* prow = P + (size_t)row * rw;

  for (int i = tid; i < D / 8; i += kSddmmThreads)
    reinterpret_cast<uint4*>(a_s)[i] = __ldg(reinterpret_cast<const uint4*>(A + (size_t)row * D) + i);
  __syncthreads();

  float l1 = 0.f;
  int nnz = 0, drop = 0;
  for (int t = warp; t < tiles; t += kSddmmThreads / 32) {
    const int raw = (int)prow[(size_t)t * W];
    const int cnt = min(max(raw, 0), W - 1);
    if (lane == 0) {
      out1[(size_t)row * rw + (size_t)t * W] = (uint32_t)raw;
      out2[(size_t)row * rw + (size_t)t * W] = (uint32_t)raw;
    }
    nnz += max(raw, 0);
    drop += max(raw, 0) - cnt;
    for (int s = 0; s < cnt; ++s) {
      const size_t pos = (size_t)row * rw + (size_t)t * W + 1 + s;
      const uint32_t pw = P[pos];
      const uint32_t col = pw & 0xFFFFu;
      const __nv_bfloat16* brow = Bm + (size_t)col * D;
      float acc = 0.f;
      for (int c = lane * 8; c < D; c += 256) {
        const uint4 av = *reinterpret_cast<const uint4*>(a_s + c);
        const uint4 bv = __ldg(reinterpret_cast<const uint4*>(brow + c));
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float2 af = __bfloat1622float2(a2[p]), bf = __bfloat1622float2(b2[p]);
          acc = fmaf(af.x, bf.x, acc);
          acc = fmaf(af.y, bf.y, acc);
        }
      }
      acc = warp_sum_f(acc);
      if (lane == 0) {
        const float pval = bf16_hi(pw);
        if (!BWD) {
          const uint32_t rb = bf16_bits(acc);                 // R
          const float tval = bf16_mul(__uint_as_float(rb << 16), pval);  // T = R * P
          out1[pos] = col | (rb << 16);
          out2[pos] = col | (bf16_bits(tval) << 16);
          l1 += fabsf(tval);
        } else {
          const float r = bf16_hi(Rin[pos]);
          float dt = __uint_as_float(bf16_bits(acc) << 16);   // dT rounded to bf16
          const float sgn = (r > 0.f) ? 1.f : (r < 0.f ? -1.f : 0.f);
          dt = __uint_as_float(bf16_bits(dt + shift * sgn) << 16);
          out1[pos] = col | (bf16_bits(bf16_mul(dt, pval)) << 16);  // dR = dT * P
          out2[pos] = col | (bf16_bits(bf16_mul(dt, r)) << 16);     // dU = dT * R
        }
      }
    }
  }
  if (!BWD) {
    if (lane == 0) {
      l1_warp[warp] = l1;
      nnz_warp[warp] = nnz;
      drop_warp[warp] = drop;
    }
    __syncthreads();
    if (tid == 0) {
      float s = 0.f;
      int n = 0, dr = 0;
      for (int w = 0; w < kSddmmThreads / 32; ++w) {
        s += l1_warp[w];
        n += nnz_warp[w];
        dr += drop_warp[w];
      }
      row_l1[row] = s;
      row_nnz[row] = n;
      row_drop[row] = dr;
    }
  }
}

// ---- column lists ---------------------------------------------------------
__global__ void hyb_count_kernel(const uint32_t* __restrict__ P, int M, int tiles, int W,
                                 int* __restrict__ col_count) {
  const int64_t slab = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (slab >= (int64_t)M * tiles) return;
  const int lane = threadIdx.x & 31;
  const uint32_t* s = P + slab * W;
  const int cnt = min(max((int)s[0], 0), W - 1);
  for (int i = lane; i < cnt; i += 32) atomicAdd(&col_count[s[1 + i] & 0xFFFFu], 1);
}

// Exclusive scan of H counts by one CTA; start[H] = total.  Also clears the cursors.
__global__ void hyb_scan_kernel(const int* __restrict__ col_count, int* __restrict__ col_start,
                                int* __restrict__ cursor, int H) {
  __shared__ int warp_tot[32];
  __shared__ int carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < H; base += blockDim.x) {
    const int i = base + tid;
    const int v = i < H ? col_count[i] : 0;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += u;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      int w = lane < (int)(blockDim.x >> 5) ? warp_tot[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += u;
      }
      warp_tot[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const int before = carry_s + (warp > 0 ? warp_tot[warp - 1] : 0) + inc - v;
    if (i < H) {
      col_start[i] = before;
      cursor[i] = 0;
    }
    __syncthreads();
    if (tid == 0) carry_s += warp_tot[(blockDim.x >> 5) - 1];
    __syncthreads();
  }
  if (tid == 0) col_start[H] = carry_s;
}

__global__ void hyb_fill_kernel(const uint32_t* __restrict__ P, int M, int tiles, int W,
                                const int* __restrict__ col_start, int* __restrict__ cursor,
                                int* __restrict__ csc_row, int* __restrict__ csc_pos, int cap,
                                int* __restrict__ overflow) {
  const int64_t slab = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (slab >= (int64_t)M * tiles) return;
  const int lane = threadIdx.x & 31;
  const uint32_t* s = P + slab * W;
  const int cnt = min(max((int)s[0], 0), W - 1);
  const int row = (int)(slab / tiles);
  for (int i = lane; i < cnt; i += 32) {
    const int col = (int)(s[1 + i] & 0xFFFFu);
    const int idx = col_start[col] + atomicAdd(&cursor[col], 1);
    if (idx < cap) {
      csc_row[idx] = row;
      csc_pos[idx] = (int)(slab * W + 1 + i);
    } else {
      atomicAdd(overflow, 1);
    }
  }
}

// ---- per-neuron activity (dead-neuron bookkeeping) ---------------------------
// The reference tracker marks a neuron active in a micro-batch when |h| > 0 for some token
// (SparsityTracker.record_activations, custom_models/sparse_models.py:148-181) but cannot
// do so on the hybrid path, which never materialises h (record_l0_l1, :183-208).  Here h
// is the slab T of the forward, so the mask costs one pass over P and T, counting per neuron
// the rows whose stored value is not +-0.  Eight lanes per (row, tile) slab: they fetch the
// slab's first 32-byte sector (count word + 7 entries) in one round trip, which covers most
// slabs at training densities, and only longer slabs loop on.
// A CTA owns one 256-neuron tile over kActivityRows rows and counts into shared memory, so
// a neuron that fires in many rows costs one global atomic per CTA instead of one per row
// (with skewed firing rates the per-row form serialises on the hot neurons' addresses).
constexpr int kActivityLanes = 8;
constexpr int kActivityRows = 64;
__global__ void __launch_bounds__(256)
hyb_activity_count_kernel(const uint32_t* __restrict__ P, const uint32_t* __restrict__ vals,
                          int M, int tiles, int W, int* __restrict__ active_rows) {
  __shared__ int hist[kTileN];
  const int t = blockIdx.x, r0 = blockIdx.y * kActivityRows;
  const int r1 = min(r0 + kActivityRows, M);
  const int g = threadIdx.x % kActivityLanes, lane = threadIdx.x & 31;
  hist[threadIdx.x] = 0;
  __syncthreads();
  // every group runs the same number of iterations: the shuffle needs all lanes
  for (int rb = r0; rb < r1; rb += 256 / kActivityLanes) {
    const int r = rb + threadIdx.x / kActivityLanes;
    const bool live = r < r1;
    const size_t off = ((size_t)(live ? r : r0) * tiles + t) * W;
    const uint32_t* s = P + off;
    const uint32_t* v = vals != nullptr ? vals + off : s;
    uint32_t pw = s[g];                          // W >= 32: the first 8 words always exist
    uint32_t vw = vals != nullptr ? v[g] : pw;
    int cnt = __shfl_sync(0xffffffffu, (int)pw, lane - g);
    cnt = live ? min(max(cnt, 0), W - 1) : 0;
    if (g >= 1 && g <= cnt && ((vw >> 16) & 0x7FFFu) != 0u) atomicAdd(&hist[pw & (kTileN - 1)], 1);
    for (int i = kActivityLanes + g; i <= cnt; i += kActivityLanes) {
      pw = s[i];
      vw = vals != nullptr ? v[i] : pw;
      if (((vw >> 16) & 0x7FFFu) != 0u) atomicAdd(&hist[pw & (kTileN - 1)], 1);
    }
  }
  __syncthreads();
  const int n = hist[threadIdx.x];
  if (n > 0) atomicAdd(&active_rows[t * kTileN + threadIdx.x], n);
}

// last_activated[j] = 0 for a neuron seen active, else + microbatch_tokens (:175-181).
__global__ void hyb_activity_update_kernel(const int* __restrict__ active_rows,
                                           long long* __restrict__ last_activated,
                                           long long microbatch_tokens, int H) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j < H) last_activated[j] = active_rows[j] > 0 ? 0ll : last_activated[j] + microbatch_tokens;
}

// ---- transposed products ----------------------------------------------------
// One cluster of kSplitT CTAs per column j, one warp per 256-column slice of D.  The
// cluster's CTAs take the column's entry batches round-robin (a hot neuron's long list
// is spread over kSplitT SMs); lane q of each warp fetches entry q of a batch, values
// are broadcast by shuffle.  Column sums are pushed to the CTA that owns that slice of D
// through distributed shared memory and added in rank order.  NSRC value arrays share
// one pass over B's rows.
constexpr int kSplitT = 8;

template <int NI, int NSRC>
__global__ void __launch_bounds__(NI * 32)
hyb_spmm_t_kernel(const uint32_t* __restrict__ V0, const uint32_t* __restrict__ V1,
                  const int* __restrict__ col_start, const int* __restrict__ csc_row,
                  const int* __restrict__ csc_pos, const __nv_bfloat16* __restrict__ Bm,
                  __nv_bfloat16* __restrict__ out0, __nv_bfloat16* __restrict__ out1, int cap) {
  constexpr int D = NI * 256;
  constexpr int BATCH = 8;
  constexpr int COLS = D / kSplitT;  // columns finished by each CTA of the cluster
  __shared__ __align__(16) float inbox[NSRC][kSplitT][COLS];
  cg::cluster_group cluster = cg::this_cluster();
  const int j = blockIdx.x / kSplitT;
  const int crank = blockIdx.x % kSplitT;
  cluster.barrier_arrive();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int beg = col_start[j], end = min(col_start[j + 1], cap);
  float acc0[8], acc1[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc0[e] = acc1[e] = 0.f;
  const __nv_bfloat16* b_lane = Bm + warp * 256 + lane * 8;

  for (int e0 = beg + crank * BATCH; e0 < end; e0 += kSplitT * BATCH) {
    int my_row = 0;
    float my_v0 = 0.f, my_v1 = 0.f;
    if (lane < BATCH && e0 + lane < end) {
      my_row = csc_row[e0 + lane];
      const int pos = csc_pos[e0 + lane];
      my_v0 = bf16_hi(V0[pos]);
      if (NSRC == 2) my_v1 = bf16_hi(V1[pos]);
    }
    uint4 bv[BATCH];
#pragma unroll
    for (int q = 0; q < BATCH; ++q) {
      const int r = __shfl_sync(0xffffffffu, my_row, q);
      bv[q] = (e0 + q < end) ? __ldg(reinterpret_cast<const uint4*>(b_lane + (size_t)r * D))
                             : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int q = 0; q < BATCH; ++q) {
      const float v0 = __shfl_sync(0xffffffffu, my_v0, q);
      const float v1 = __shfl_sync(0xffffffffu, my_v1, q);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv[q]);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 bf = __bfloat1622float2(b2[p]);
        acc0[2 * p] = fmaf(v0, bf.x, acc0[2 * p]);
        acc0[2 * p + 1] = fmaf(v0, bf.y, acc0[2 * p + 1]);
        if (NSRC == 2) {
          acc1[2 * p] = fmaf(v1, bf.x, acc1[2 * p]);
          acc1[2 * p + 1] = fmaf(v1, bf.y, acc1[2 * p + 1]);
        }
      }
    }
  }

  cluster.barrier_wait();  // every CTA of the cluster is running: remote stores are safe
  {
    const int c = warp * 256 + lane * 8;
    const int owner = c / COLS, off = c - owner * COLS;
    float* d0 = cluster.map_shared_rank(&inbox[0][crank][off], owner);
    *reinterpret_cast<float4*>(d0) = make_float4(acc0[0], acc0[1], acc0[2], acc0[3]);
    *reinterpret_cast<float4*>(d0 + 4) = make_float4(acc0[4], acc0[5], acc0[6], acc0[7]);
    if (NSRC == 2) {
      float* d1 = cluster.map_shared_rank(&inbox[NSRC - 1][crank][off], owner);
      *reinterpret_cast<float4*>(d1) = make_float4(acc1[0], acc1[1], acc1[2], acc1[3]);
      *reinterpret_cast<float4*>(d1 + 4) = make_float4(acc1[4], acc1[5], acc1[6], acc1[7]);
    }
  }
  cluster.sync();
  for (int c = threadIdx.x * 2; c < COLS; c += NI * 32 * 2) {
#pragma unroll
    for (int sI = 0; sI < NSRC; ++sI) {
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int r = 0; r < kSplitT; ++r) {
        s0 += inbox[sI][r][c];
        s1 += inbox[sI][r][c + 1];
      }
      __nv_bfloat16* o = (sI == 0 ? out0 : out1) + (size_t)j * D + crank * COLS + c;
      *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(s0, s1);
    }
  }
}

// Row-ELL (u16 columns, bf16 values, per-row counts) x dense B[K_rows, N]; rows whose
// count exceeds overflow_threshold (or is zero) produce zeros.  One CTA per row.
__global__ void __launch_bounds__(256)
hyb_ell_spmm_raw_kernel(const __nv_bfloat16* __restrict__ vals, const uint16_t* __restrict__ cols,
                        const int* __restrict__ row_counts, const __nv_bfloat16* __restrict__ Bm,
                        __nv_bfloat16* __restrict__ C, int N, int ell_stride,
                        int overflow_threshold) {
  const int row = blockIdx.x;
  int nnz = row_counts[row];
  if (nnz < 0 || nnz > overflow_threshold) nnz = 0;
  for (int n0 = threadIdx.x * 8; n0 < N; n0 += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int k = 0; k < nnz; ++k) {
      const float a = __bfloat162float(vals[(size_t)row * ell_stride + k]);
      const int col = cols[(size_t)row * ell_stride + k];
      const uint4 bv = __ldg(reinterpret_cast<const uint4*>(Bm + (size_t)col * N + n0));
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 bf = __bfloat1622float2(b2[p]);
        acc[2 * p] = fmaf(a, bf.x, acc[2 * p]);
        acc[2 * p + 1] = fmaf(a, bf.y, acc[2 * p + 1]);
      }
    }
    __nv_bfloat162 o[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) o[p] = __floats2bfloat162_rn(acc[2 * p], acc[2 * p + 1]);
    *reinterpret_cast<uint4*>(C + (size_t)row * N + n0) = *reinterpret_cast<uint4*>(o);
  }
}

template <int NSRC>
int spmm_t_dispatch(int ni, int H, const uint32_t* v0, const uint32_t* v1, const int* col_start,
                    const int* csc_row, const int* csc_pos, const __nv_bfloat16* Bm,
                    __nv_bfloat16* o0, __nv_bfloat16* o1, int cap, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)H * kSplitT, 1, 1);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kSplitT;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaSuccess;
  switch (ni) {
#define B200_CASE(N)                                                                         \
  case N:                                                                                    \
    cfg.blockDim = dim3(N * 32, 1, 1);                                                       \
    e = cudaLaunchKernelEx(&cfg, hyb_spmm_t_kernel<N, NSRC>, v0, v1, col_start, csc_row,     \
                           csc_pos, Bm, o0, o1, cap);                                        \
    break;
    B200_CASE(1) B200_CASE(2) B200_CASE(3) B200_CASE(4) B200_CASE(5) B200_CASE(6) B200_CASE(7)
    B200_CASE(8) B200_CASE(9) B200_CASE(10) B200_CASE(11) B200_CASE(12) B200_CASE(13)
    B200_CASE(14) B200_CASE(15) B200_CASE(16)
#undef B200_CASE
    default:
      return fail(B200_EUNSUPPORTED, "b200_hybrid_spmm_t: D = %d is not compiled (256..4096)",
                  ni * 256);
  }
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "b200_hybrid_spmm_t: launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

int check_all(const char* fn, std::initializer_list<const void*> ptrs) {
  for (const void* p : ptrs) {
    if (p == nullptr) return fail(B200_ENULL, "%s: a required pointer is NULL", fn);
    if (!aligned16(p)) return fail(B200_EALIGN, "%s: a pointer is not 16-byte aligned", fn);
  }
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_hybrid_sddmm_fwd(const void* x, const void* k_w, const void* p_slab, void* r_slab,
                          void* t_slab, float* row_l1, int* row_nnz, int* row_drop, int64_t M,
                          int64_t D, int64_t H, int cf, void* stream) {
  const char* fn = "b200_hybrid_sddmm_fwd";
  if (int rc = check_dims(fn, M, D, H, cf)) return rc;
  if (M == 0) return B200_OK;
  if (int rc = check_all(fn, {x, k_w, p_slab, r_slab, t_slab, row_l1, row_nnz, row_drop})) return rc;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(hyb_sddmm_kernel<false>, (size_t)D * 2, granted, fn)) return rc;
  hyb_sddmm_kernel<false><<<(unsigned)M, kSddmmThreads, (size_t)D * 2,
                            static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(k_w),
      static_cast<const uint32_t*>(p_slab), nullptr, static_cast<uint32_t*>(r_slab),
      static_cast<uint32_t*>(t_slab), row_l1, row_nnz, row_drop, nullptr, 0.f, (int)D,
      (int)(H / kTileN), kTileN / cf);
  return check_launch(fn);
}

int b200_hybrid_sddmm_bwd(const void* g_out, const void* v_w, const void* p_slab,
                          const void* r_slab, void* dr_slab, void* du_slab,
                          const float* l1_grad, int64_t M, int64_t D, int64_t H, int cf,
                          void* stream) {
  const char* fn = "b200_hybrid_sddmm_bwd";
  if (int rc = check_dims(fn, M, D, H, cf)) return rc;
  if (M == 0) return B200_OK;
  if (int rc = check_all(fn, {g_out, v_w, p_slab, r_slab, dr_slab, du_slab})) return rc;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(hyb_sddmm_kernel<true>, (size_t)D * 2, granted, fn)) return rc;
  hyb_sddmm_kernel<true><<<(unsigned)M, kSddmmThreads, (size_t)D * 2,
                           static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(g_out), static_cast<const __nv_bfloat16*>(v_w),
      static_cast<const uint32_t*>(p_slab), static_cast<const uint32_t*>(r_slab),
      static_cast<uint32_t*>(dr_slab), static_cast<uint32_t*>(du_slab), nullptr, nullptr, nullptr,
      l1_grad, 1.0f / (float)M, (int)D, (int)(H / kTileN), kTileN / cf);
  return check_launch(fn);
}

int b200_hybrid_csc_build(const void* p_slab, int* col_count, int* col_start, int* cursor,
                          int* csc_row, int* csc_pos, int64_t capacity, int* overflow, int64_t M,
                          int64_t H, int cf, void* stream) {
  const char* fn = "b200_hybrid_csc_build";
  if (int rc = check_dims(fn, M, 256, H, cf)) return rc;
  if (capacity < 0 || capacity > 0x7fffffffLL) return fail(B200_EINVAL, "%s: bad capacity", fn);
  if (p_slab == nullptr || col_count == nullptr || col_start == nullptr || cursor == nullptr ||
      csc_row == nullptr || csc_pos == nullptr || overflow == nullptr)
    return fail(B200_ENULL, "%s: a required pointer is NULL", fn);
  if ((int64_t)M * (H / kTileN) * (kTileN / cf) > 0x7fffffffLL)
    return fail(B200_EUNSUPPORTED, "%s: slab array exceeds 2^31 words", fn);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(col_count, 0, sizeof(int) * (size_t)H, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(overflow, 0, sizeof(int), st);
  if (e != cudaSuccess) return fail(B200_ECUDA, "%s: memset: %s", fn, cudaGetErrorString(e));
  const int tiles = (int)(H / kTileN), W = kTileN / cf;
  if (M > 0) {
    const int64_t slabs = M * tiles;
    const unsigned blocks = (unsigned)((slabs + 7) / 8);
    hyb_count_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint32_t*>(p_slab), (int)M, tiles, W,
                                             col_count);
    hyb_scan_kernel<<<1, 1024, 0, st>>>(col_count, col_start, cursor, (int)H);
    hyb_fill_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint32_t*>(p_slab), (int)M, tiles, W,
                                            col_start, cursor, csc_row, csc_pos, (int)capacity,
                                            overflow);
  } else {
    hyb_scan_kernel<<<1, 1024, 0, st>>>(col_count, col_start, cursor, (int)H);
  }
  return check_launch(fn);
}

int b200_hybrid_neuron_activity(const void* p_slab, const void* vals_slab, int64_t M, int64_t H,
                                int cf, int64_t microbatch_tokens, int* active_rows,
                                int64_t* last_activated, void* stream) {
  const char* fn = "b200_hybrid_neuron_activity";
  if (M < 0 || H <= 0 || H % kTileN || H > 65536)
    return fail(B200_EUNSUPPORTED, "%s: H must be a multiple of 256, at most 65536", fn);
  if (cf != 2 && cf != 4 && cf != 8) return fail(B200_EUNSUPPORTED, "%s: cf must be 2, 4 or 8", fn);
  if (microbatch_tokens < 0) return fail(B200_EINVAL, "%s: microbatch_tokens is negative", fn);
  if (active_rows == nullptr) return fail(B200_ENULL, "%s: active_rows is NULL", fn);
  if (M > 0 && p_slab == nullptr) return fail(B200_ENULL, "%s: p_slab is NULL", fn);
  if ((int64_t)M * (H / kTileN) * (kTileN / cf) > 0x7fffffffLL)
    return fail(B200_EUNSUPPORTED, "%s: slab array exceeds 2^31 words", fn);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(active_rows, 0, sizeof(int) * (size_t)H, st);
  if (e != cudaSuccess) return fail(B200_ECUDA, "%s: memset: %s", fn, cudaGetErrorString(e));
  const int tiles = (int)(H / kTileN), W = kTileN / cf;
  if (M > 0) {
    const dim3 grid((unsigned)tiles, (unsigned)((M + kActivityRows - 1) / kActivityRows));
    hyb_activity_count_kernel<<<grid, 256, 0, st>>>(
        static_cast<const uint32_t*>(p_slab), static_cast<const uint32_t*>(vals_slab), (int)M,
        tiles, W, active_rows);
  }
  if (last_activated != nullptr) {
    hyb_activity_update_kernel<<<(unsigned)((H + 255) / 256), 256, 0, st>>>(
        active_rows, reinterpret_cast<long long*>(last_activated), (long long)microbatch_tokens,
        (int)H);
  }
  return check_launch(fn);
}

int b200_hybrid_spmm_t(const void* vals0, const void* vals1, const int* col_start,
                       const int* csc_row, const int* csc_pos, int64_t capacity, const void* b_rows,
                       void* out0, void* out1, int64_t H, int64_t D, void* stream) {
  const char* fn = "b200_hybrid_spmm_t";
  if (H <= 0 || H > 65536) return fail(B200_EUNSUPPORTED, "%s: bad H", fn);
  if (D < 256 || D > 4096 || D % 256) return fail(B200_EUNSUPPORTED, "%s: D must be 256..4096", fn);
  if (int rc = check_all(fn, {vals0, b_rows, out0})) return rc;
  if (col_start == nullptr || csc_row == nullptr || csc_pos == nullptr)
    return fail(B200_ENULL, "%s: column lists are NULL", fn);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (vals1 != nullptr) {
    if (int rc = check_all(fn, {vals1, out1})) return rc;
    return spmm_t_dispatch<2>((int)(D / 256), (int)H, static_cast<const uint32_t*>(vals0),
                              static_cast<const uint32_t*>(vals1), col_start, csc_row, csc_pos,
                              static_cast<const __nv_bfloat16*>(b_rows),
                              static_cast<__nv_bfloat16*>(out0), static_cast<__nv_bfloat16*>(out1),
                              (int)capacity, st);
  }
  return spmm_t_dispatch<1>((int)(D / 256), (int)H, static_cast<const uint32_t*>(vals0), nullptr,
                            col_start, csc_row, csc_pos, static_cast<const __nv_bfloat16*>(b_rows),
                            static_cast<__nv_bfloat16*>(out0), nullptr, (int)capacity, st);
}

int b200_hybrid_ell_spmm_raw(const void* ell_vals, const void* ell_cols, const int* row_counts,
                             const void* b, void* c, int64_t M, int64_t K, int64_t N,
                             int64_t ell_stride, int64_t overflow_threshold, void* stream) {
  const char* fn = "b200_hybrid_ell_spmm_raw";
  if (M < 0 || K <= 0 || K > 65536 || N <= 0 || N % 8 || ell_stride <= 0)
    return fail(B200_EINVAL, "%s: bad sizes (N must be a multiple of 8, K <= 65536)", fn);
  if (M == 0) return B200_OK;
  if (ell_vals == nullptr || ell_cols == nullptr || row_counts == nullptr || b == nullptr ||
      c == nullptr)
    return fail(B200_ENULL, "%s: a required pointer is NULL", fn);
  if (!aligned16(b) || !aligned16(c)) return fail(B200_EALIGN, "%s: B / C not 16-byte aligned", fn);
  hyb_ell_spmm_raw_kernel<<<(unsigned)M, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(ell_vals), static_cast<const uint16_t*>(ell_cols),
      row_counts, static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(c), (int)N,
      (int)ell_stride, (int)overflow_threshold);
  return check_launch(fn);
}

}  // extern "C"
