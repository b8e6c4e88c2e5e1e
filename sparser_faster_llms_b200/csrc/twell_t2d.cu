// TwELL -> dense contraction (gated up/down and plain down projection).
//
// One thread-block cluster per token.  The token's stored entries (over all
// slabs) are numbered 0..n-1 and divided evenly over the cluster's CTAs and,
// inside a CTA, over its warps.  For each entry (j, g) a warp
//   * dots the token's x row (held in registers) with up[j, :]   (gated only),
//   * forms h = g * u,
//   * adds h * down[j, :] to a register accumulator spanning all D columns,
// with 128-bit loads of the two weight rows.  Warp accumulators are summed in a
// fixed order through shared memory, CTA sums through distributed shared memory,
// so the result is deterministic.  At decode (M <= 32) the cluster spreads one
// token over several SMs; at prefill one CTA per token keeps weight rows hot in L2.
//
// Numerics follow the reference kernels: mixed mode rounds every product to
// bf16 before the fp32 add and rounds h to bf16
// (custom_models/twell_modules/matmul_gated_t2d.cu:74-149, matmul_t2d.cu:56-95);
// high-precision mode uses fp32 fma throughout (matmul_gated_t2d.cu:389-441).
// The reference's flex variants (:174-324, :466-594) differ only in how the slab
// is read; this kernel reads any slab width.  The output row may alias the
// input row (in-place variants, :972-1541): x is cached in registers before the
// cluster barrier that precedes the first store.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxTiles = 256;  // H <= 65536

__device__ __forceinline__ uint4 ldg_nc(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// NI = D / 256.  Shared memory: entries[cap] | partial[kWarps][D] fp32.
template <int NI, bool GATED, bool HP>
__global__ void __launch_bounds__(kThreads)
twell_t2d_kernel(const __nv_bfloat16* x, const uint32_t* __restrict__ packed,
                 const __nv_bfloat16* __restrict__ up, const __nv_bfloat16* __restrict__ down,
                 __nv_bfloat16* out, int M, int tiles, int slab_w, int cs, int ent_cap) {
  constexpr int D = NI * 256;
  extern __shared__ __align__(16) unsigned char smem[];
  uint32_t* entries = reinterpret_cast<uint32_t*>(smem);
  float* partial = reinterpret_cast<float*>(smem + (size_t)ent_cap * sizeof(uint32_t));
  __shared__ int tile_off[kMaxTiles + 1];

  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x / cs;
  const int crank = blockIdx.x % cs;
  const uint32_t* prow = packed + (size_t)row * tiles * slab_w;

  // x row -> registers (lane owns columns it*256 + lane*8 .. +7).
  uint4 xr[GATED ? NI : 1];
  if (GATED) {
#pragma unroll
    for (int it = 0; it < NI; ++it)
      xr[it] = *reinterpret_cast<const uint4*>(x + (size_t)row * D + it * 256 + lane * 8);
  }

  // Exclusive prefix of the per-slab entry counts (warp 0).
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < tiles; base += 32) {
      const int tI = base + lane;
      int c = 0;
      if (tI < tiles) {
        c = (int)prow[(size_t)tI * slab_w];
        c = min(max(c, 0), slab_w - 1);
      }
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
      }
      if (tI < tiles) tile_off[tI] = carry + inc - c;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) tile_off[tiles] = carry;
  }
  __syncthreads();
  const int n_total = tile_off[tiles];
  const int per = (n_total + cs - 1) / cs;
  const int lo = crank * per;
  const int hi = min(n_total, lo + per);
  const int n_mine = max(hi - lo, 0);

  // Gather this CTA's share of the entries.
  for (int tI = warp; tI < tiles; tI += kWarps) {
    const int o = tile_off[tI], c = tile_off[tI + 1] - o;
    if (o + c <= lo || o >= hi) continue;
    for (int s = lane; s < c; s += 32) {
      const int k = o + s;
      if (k >= lo && k < hi) entries[k - lo] = prow[(size_t)tI * slab_w + 1 + s];
    }
  }
  __syncthreads();

  float acc[NI][8];
#pragma unroll
  for (int it = 0; it < NI; ++it)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[it][e] = 0.f;

  for (int k = warp; k < n_mine; k += kWarps) {
    const uint32_t word = entries[k];
    const uint32_t j = word & 0xFFFFu;
    const __nv_bfloat16 gval = __ushort_as_bfloat16((unsigned short)(word >> 16));
    const __nv_bfloat16* drow = down + (size_t)j * D + lane * 8;
    // The down row does not depend on u: fetch it before the dot product when
    // the registers allow, so both rows are in flight together.
    constexpr bool kPreload = NI <= 8;
    uint4 dv[kPreload ? NI : 1];
    if (kPreload) {
#pragma unroll
      for (int it = 0; it < NI; ++it) dv[it] = ldg_nc(drow + it * 256);
    }

    float hf;              // h as fp32 (high precision)
    __nv_bfloat162 hb2;    // h as bf16 pair (mixed)
    if (GATED) {
      const __nv_bfloat16* urow = up + (size_t)j * D + lane * 8;
      float u = 0.f;
#pragma unroll
      for (int it = 0; it < NI; ++it) {
        const uint4 uv = ldg_nc(urow + it * 256);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xr[it]);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          if (HP) {
            const float2 wf = __bfloat1622float2(w2[p]), xf = __bfloat1622float2(x2[p]);
            u = __fmaf_rn(wf.x, xf.x, u);
            u = __fmaf_rn(wf.y, xf.y, u);
          } else {
            const float2 pf = __bfloat1622float2(__hmul2(x2[p], w2[p]));
            u += pf.x;
            u += pf.y;
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) u += __shfl_xor_sync(0xffffffffu, u, o);
      if (HP) {
        hf = __bfloat162float(gval) * u;
      } else {
        hb2 = __bfloat162bfloat162(__hmul(gval, __float2bfloat16_rn(u)));
      }
    } else {
      hf = __bfloat162float(gval);
      hb2 = __bfloat162bfloat162(gval);
    }

#pragma unroll
    for (int it = 0; it < NI; ++it) {
      uint4 dcur;
      if (kPreload) dcur = dv[it]; else dcur = ldg_nc(drow + it * 256);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&dcur);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        if (HP) {
          const float2 wf = __bfloat1622float2(w2[p]);
          acc[it][2 * p] = __fmaf_rn(wf.x, hf, acc[it][2 * p]);
          acc[it][2 * p + 1] = __fmaf_rn(wf.y, hf, acc[it][2 * p + 1]);
        } else {
          const float2 pf = __bfloat1622float2(__hmul2(hb2, w2[p]));
          acc[it][2 * p] += pf.x;
          acc[it][2 * p + 1] += pf.y;
        }
      }
    }
  }

  // Warp accumulators -> shared memory, fixed-order sum over warps.
#pragma unroll
  for (int it = 0; it < NI; ++it) {
    float* p = partial + (size_t)warp * D + it * 256 + lane * 8;
    *reinterpret_cast<float4*>(p) = make_float4(acc[it][0], acc[it][1], acc[it][2], acc[it][3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(acc[it][4], acc[it][5], acc[it][6], acc[it][7]);
  }
  __syncthreads();
  for (int c = tid; c < D; c += kThreads) {
    float s = partial[c];
#pragma unroll
    for (int wI = 1; wI < kWarps; ++wI) s += partial[(size_t)wI * D + c];
    partial[c] = s;  // column c is read and written by this thread only
  }
  cluster.sync();

  // Cluster reduction: CTA r finishes columns [r*D/cs, (r+1)*D/cs).
  const int cols = D / cs;
  for (int c = tid * 2; c < cols; c += kThreads * 2) {
    const int col = crank * cols + c;
    float s0 = 0.f, s1 = 0.f;
    for (int r = 0; r < cs; ++r) {
      const float* peer = cluster.map_shared_rank(partial, r);
      const float2 v = *reinterpret_cast<const float2*>(peer + col);
      s0 += v.x;
      s1 += v.y;
    }
    *reinterpret_cast<__nv_bfloat162*>(out + (size_t)row * D + col) = __floats2bfloat162_rn(s0, s1);
  }
  cluster.sync();  // keep shared memory alive until every peer has read it
}

template <int NI, bool GATED, bool HP>
int launch_t2d(const void* x, const void* packed, const void* up, const void* down, void* out,
               int64_t M, int64_t H, int cf, int cs, cudaStream_t stream) {
  constexpr int D = NI * 256;
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  // Worst-case entries one CTA may hold: its share of a row that is full everywhere.
  const int64_t full = (int64_t)tiles * (slab_w - 1);
  const int ent_cap = (int)(((full + cs - 1) / cs + 3) & ~(int64_t)3);
  const size_t smem = (size_t)ent_cap * 4 + (size_t)kWarps * D * sizeof(float);
  auto kern = twell_t2d_kernel<NI, GATED, HP>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(B200_ECUDA, "twell_t2d: smem attribute (%zu B): %s", smem, cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(M * cs), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, reinterpret_cast<const __nv_bfloat16*>(x),
                         reinterpret_cast<const uint32_t*>(packed),
                         reinterpret_cast<const __nv_bfloat16*>(up),
                         reinterpret_cast<const __nv_bfloat16*>(down),
                         reinterpret_cast<__nv_bfloat16*>(out), (int)M, tiles, slab_w, cs, ent_cap);
  if (e != cudaSuccess) return fail(B200_ECUDA, "twell_t2d: launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

template <bool GATED, bool HP>
int dispatch_ni(int ni, const void* x, const void* packed, const void* up, const void* down,
                void* out, int64_t M, int64_t H, int cf, int cs, cudaStream_t stream) {
  switch (ni) {
#define B200_CASE(N) \
  case N: return launch_t2d<N, GATED, HP>(x, packed, up, down, out, M, H, cf, cs, stream);
    B200_CASE(1) B200_CASE(2) B200_CASE(3) B200_CASE(4) B200_CASE(5) B200_CASE(6) B200_CASE(7)
    B200_CASE(8) B200_CASE(10) B200_CASE(12) B200_CASE(14) B200_CASE(16)
#undef B200_CASE
    default:
      return fail(B200_EUNSUPPORTED,
                  "twell_t2d: D = %d is not compiled (supported: 256*k for k in 1..8,10,12,14,16)",
                  ni * 256);
  }
}

}  // namespace

// Cluster size: spread a token over several SMs while there are fewer tokens
// than SMs, keeping D divisible by 2*cs.
int t2d_cluster_size(int64_t M, int64_t D, int sm_count) {
  int cs = 1;
  while (cs < 8 && M * cs * 2 <= (int64_t)sm_count * 2 && (D / (cs * 2)) % 2 == 0) cs *= 2;
  return cs;
}

int twell_t2d_launch(bool gated, bool hp, const void* x, const void* packed, const void* up,
                     const void* down, void* out, int64_t M, int64_t D, int64_t H, int cf, int cs,
                     cudaStream_t stream) {
  const int ni = (int)(D / 256);
  if (gated) {
    return hp ? dispatch_ni<true, true>(ni, x, packed, up, down, out, M, H, cf, cs, stream)
              : dispatch_ni<true, false>(ni, x, packed, up, down, out, M, H, cf, cs, stream);
  }
  return dispatch_ni<false, false>(ni, x, packed, up, down, out, M, H, cf, cs, stream);
}

}  // namespace b200
