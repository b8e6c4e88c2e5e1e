// Gate projection + ReLU + TwELL pack for small and medium token counts.
//
// The weight matrix w[H, D] is streamed from HBM exactly once per 32-token tile;
// the activations x[M, D] sit in shared memory.  Neurons ride the M axis of the
// tensor-core instruction (mma.sync m16n8k16, bf16 -> fp32) and tokens the N
// axis, so a decode batch of 1..32 tokens costs one pass over w.  A 256-neuron
// TwELL tile is owned by a thread-block cluster: each CTA computes NPC = 64 (or
// 32) neurons for all tokens of the tile, the CTAs exchange per-token counts
// through distributed shared memory, and every CTA then writes its entries at
// the right offset of the slab - ascending column order, no atomics, so the
// slab bytes are reproducible run to run.
//
// Replaces the reference's WGMMA kernel mm_wgmma_nt_kernel
// (custom_models/twell_modules/matmul_d2t.cu:287-709) for M below the
// tensor-core GEMM crossover.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kKSplit = 4;    // warps that share one 16-neuron strip, each a quarter of D
constexpr int kXPadBytes = 64;  // row padding of the x tile: conflict-free 128-bit reads
constexpr int kPrefetch = 4;  // 32-wide k steps held in registers ahead of the math

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// TM tokens per tile (multiple of 8), NPC neurons per CTA (32 or 64).
// Cluster = 256 / NPC CTAs along x; grid.x = (H/256) * cluster, grid.y = ceil(M / TM).
template <int TM, int NPC>
__global__ void __launch_bounds__((NPC / 16) * kKSplit * 32, 1)
twell_pack_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                  const float* __restrict__ bias, uint32_t* __restrict__ packed, int M, int D,
                  int slab_w, int row_words) {
  constexpr int MT = NPC / 16;          // 16-neuron strips per CTA
  constexpr int NWARPS = MT * kKSplit;
  constexpr int NTHREADS = NWARPS * 32;
  constexpr int NT = TM / 8;            // 8-token column blocks
  constexpr int CL = kTileN / NPC;      // cluster size
  constexpr int RS = NPC + 4;           // row stride of the partial-sum buffer (floats)
  constexpr int EPT = TM * NPC / NTHREADS;
  constexpr int CHUNKS = NPC / 32;

  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int cnt_chunk[TM][CHUNKS];
  __shared__ int cta_total[TM];   // read by the peer CTAs of the cluster
  __shared__ int cta_base[TM];

  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  const int tile = blockIdx.x / CL;
  const int m0 = blockIdx.y * TM;

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int mt = warp % MT, kq = warp / MT;

  const int xs_stride = D * 2 + kXPadBytes;
  const int kspan = D / kKSplit;        // k range of this warp
  const int ksteps = kspan / 32;

  const int neuron_cta0 = tile * kTileN + crank * NPC;
  const __nv_bfloat16* w_lo = w + (size_t)(neuron_cta0 + mt * 16 + g) * D + kq * kspan + t * 8;
  const __nv_bfloat16* w_hi = w_lo + (size_t)8 * D;

  // Weight loads do not depend on shared memory: put the first chunk in flight
  // before staging x.
  uint4 a0_lo[kPrefetch], a0_hi[kPrefetch], a1_lo[kPrefetch], a1_hi[kPrefetch];
  auto load_chunk = [&](uint4 (&lo)[kPrefetch], uint4 (&hi)[kPrefetch], int s_base) {
#pragma unroll
    for (int u = 0; u < kPrefetch; ++u) {
      if (s_base + u < ksteps) {
        lo[u] = ldg_stream(w_lo + (s_base + u) * 32);
        hi[u] = ldg_stream(w_hi + (s_base + u) * 32);
      }
    }
  };
  load_chunk(a0_lo, a0_hi, 0);

  // Stage the x tile (rows past M are zero).
  {
    const int vec_per_row = D / 8;
    for (int i = tid; i < TM * vec_per_row; i += NTHREADS) {
      const int r = i / vec_per_row, c = i - r * vec_per_row;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (m0 + r < M) v = *reinterpret_cast<const uint4*>(x + (size_t)(m0 + r) * D + c * 8);
      *reinterpret_cast<uint4*>(smem + (size_t)r * xs_stride + c * 16) = v;
    }
  }
  __syncthreads();

  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

  const unsigned char* xs_thread = smem + (size_t)g * xs_stride + (kq * kspan + t * 8) * 2;

  auto compute_chunk = [&](const uint4 (&lo)[kPrefetch], const uint4 (&hi)[kPrefetch],
                           int s_base) {
#pragma unroll
    for (int u = 0; u < kPrefetch; ++u) {
      const int s = s_base + u;
      if (s < ksteps) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const uint4 b = *reinterpret_cast<const uint4*>(xs_thread + (size_t)n * 8 * xs_stride +
                                                          s * 64);
          mma_bf16_16816(acc[n], lo[u].x, hi[u].x, lo[u].y, hi[u].y, b.x, b.y);
          mma_bf16_16816(acc[n], lo[u].z, hi[u].z, lo[u].w, hi[u].w, b.z, b.w);
        }
      }
    }
  };
  for (int s0 = 0; s0 < ksteps; s0 += 2 * kPrefetch) {
    load_chunk(a1_lo, a1_hi, s0 + kPrefetch);
    compute_chunk(a0_lo, a0_hi, s0);
    load_chunk(a0_lo, a0_hi, s0 + 2 * kPrefetch);
    compute_chunk(a1_lo, a1_hi, s0 + kPrefetch);
  }
  __syncthreads();  // x tile no longer needed: its storage becomes the partial-sum buffer

  float* red = reinterpret_cast<float*>(smem);  // [kKSplit][TM][RS]
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int tok = n * 8 + 2 * t;
    const int nl = mt * 16 + g;
    float* base = red + ((size_t)kq * TM + tok) * RS + nl;
    base[0] = acc[n][0];
    base[RS] = acc[n][1];
    base[8] = acc[n][2];
    base[RS + 8] = acc[n][3];
  }
  __syncthreads();

  // Pass 1: final pre-activation, ballot per (token, 32-neuron chunk).
  float z[EPT];
  uint32_t mask[EPT];
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = tid + i * NTHREADS;
    const int tok = e / NPC, nl = e % NPC;
    float v = 0.f;
#pragma unroll
    for (int q = 0; q < kKSplit; ++q) v += red[((size_t)q * TM + tok) * RS + nl];
    if (bias != nullptr) v += bias[neuron_cta0 + nl];
    const bool keep = (v > 0.f) && (m0 + tok < M);
    z[i] = v;
    mask[i] = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) cnt_chunk[tok][nl / 32] = __popc(mask[i]);
  }
  __syncthreads();
  if (tid < TM) {
    int s = 0;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) s += cnt_chunk[tid][c];
    cta_total[tid] = s;
  }
  cluster.sync();
  if (tid < TM) {
    int before = 0, total = 0;
#pragma unroll
    for (int r = 0; r < CL; ++r) {
      const int* peer = cluster.map_shared_rank(cta_total, r);
      const int c = peer[tid];
      if (r < crank) before += c;
      total += c;
    }
    cta_base[tid] = before;
    if (crank == 0 && m0 + tid < M)
      packed[(size_t)(m0 + tid) * row_words + (size_t)tile * slab_w] = (uint32_t)total;
  }
  __syncthreads();

  // Pass 2: scatter the kept entries.
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = tid + i * NTHREADS;
    const int tok = e / NPC, nl = e % NPC;
    const bool keep = (mask[i] >> lane) & 1u;
    int slot = cta_base[tok] + __popc(mask[i] & lanemask_lt());
    for (int c = 0; c < nl / 32; ++c) slot += cnt_chunk[tok][c];
    if (keep && slot < slab_w - 1) {
      packed[(size_t)(m0 + tok) * row_words + (size_t)tile * slab_w + 1 + slot] =
          (uint32_t)(neuron_cta0 + nl) | (bf16_bits(z[i]) << 16);
    }
  }
  cluster.sync();  // peers may still be reading cta_total
}

template <int TM, int NPC>
int launch_pack(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                int64_t D, int64_t H, int cf, cudaStream_t stream) {
  constexpr int NTHREADS = (NPC / 16) * kKSplit * 32;
  constexpr int CL = kTileN / NPC;
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  const size_t xs_bytes = (size_t)TM * (D * 2 + kXPadBytes);
  const size_t red_bytes = (size_t)kKSplit * TM * (NPC + 4) * sizeof(float);
  const size_t smem = xs_bytes > red_bytes ? xs_bytes : red_bytes;

  auto kern = twell_pack_kernel<TM, NPC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(B200_ECUDA, "b200_twell_pack: smem attribute: %s", cudaGetErrorString(e));

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * CL), (unsigned)((M + TM - 1) / TM), 1);
  cfg.blockDim = dim3(NTHREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, reinterpret_cast<const __nv_bfloat16*>(x),
                         reinterpret_cast<const __nv_bfloat16*>(w), bias,
                         reinterpret_cast<uint32_t*>(packed), (int)M, (int)D, slab_w,
                         tiles * slab_w);
  if (e != cudaSuccess) return fail(B200_ECUDA, "b200_twell_pack: launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

}  // namespace

int twell_pack_small(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                     int64_t D, int64_t H, int cf, cudaStream_t stream) {
  // Token-tile height: the largest of 32/16/8 whose x tile fits beside the
  // static shared memory, and no larger than M needs.
  const size_t budget = 200 * 1024;
  int tm = 32;
  while (tm > 8 && ((size_t)tm * (D * 2 + kXPadBytes) > budget || tm / 2 >= M)) tm /= 2;
  switch (tm) {
    case 32: return launch_pack<32, 64>(x, w, bias, packed, M, D, H, cf, stream);
    case 16: return launch_pack<16, 64>(x, w, bias, packed, M, D, H, cf, stream);
    default: return launch_pack<8, 64>(x, w, bias, packed, M, D, H, cf, stream);
  }
}

}  // namespace b200
