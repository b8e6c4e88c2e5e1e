// Gate projection + ReLU + TwELL pack for small and medium token counts.
//
// The weight matrix w[H, D] is streamed from HBM exactly once per 32-token tile.
// Neurons ride the M axis of the tensor-core instruction (mma.sync m16n8k16,
// bf16 -> fp32) and tokens the N axis, so a decode batch of 1..32 tokens costs
// one pass over w.  A 256-neuron TwELL tile is owned by a thread-block cluster
// that splits the reduction dimension: CTA q of the cluster multiplies all 256
// neurons by the q-th slice of D (its slice of x sits in shared memory, its
// slice of every weight row is 128-bit-loaded straight into mma fragments).
// The partial sums meet in distributed shared memory: each CTA owns a share of
// the tokens, receives the cluster's partials for them (remote stores, one
// cluster barrier), adds them in a fixed order, and compacts each of its
// tokens' 256 pre-activations with warp ballot / popc into the slab - ascending
// column order, no atomics, so the slab bytes are reproducible run to run.
//
// Replaces the reference's WGMMA kernel mm_wgmma_nt_kernel
// (custom_models/twell_modules/matmul_d2t.cu:287-709) for M below the
// tensor-core GEMM crossover.
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kXPadBytes = 64;           // row padding of the x slice: conflict-free 128-bit reads
constexpr int kPartStride = kTileN + 4;  // floats per token row of the partial-sum buffer

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

// 16-byte asynchronous global -> shared copy; src_bytes = 0 zero-fills.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int src_bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc),
               "r"(src_bytes));
}

// TM     tokens per tile (8, 16 or 32)
// CL     cluster size = number of k slices
// WARPS  warps per CTA; each warp owns STRIPS strips of 16 neurons (WARPS*STRIPS = 16)
// PF     32-wide k steps of weights each thread keeps in flight per strip
// grid.x = (H/256) * CL, grid.y = ceil(M / TM).
// Dynamic shared memory: x slice [TM][KC*2 + pad] bytes | partial sums [TM][kPartStride] fp32.
template <int TM, int CL, int WARPS, int STRIPS, int PF, int MINB>
__global__ void __launch_bounds__(WARPS * 32, MINB)
twell_pack_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                  const float* __restrict__ bias, uint32_t* __restrict__ packed, int M, int D,
                  int slab_w, int row_words) {
  constexpr int NTHREADS = WARPS * 32;
  constexpr int NT = TM / 8;          // 8-token column blocks of the mma
  constexpr int TOK = TM / CL;        // tokens finalised by this CTA
  constexpr int EPT = TOK * kTileN / NTHREADS;
  static_assert(WARPS * STRIPS * 16 == kTileN, "a CTA covers one 256-neuron tile");
  static_assert(TM % CL == 0 && EPT >= 1, "token tile must split evenly over the cluster");

  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int cnt_chunk[TOK][8];

  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  const int tile = blockIdx.x / CL;
  const int m0 = blockIdx.y * TM;
  cluster.barrier_arrive();  // matched by barrier_wait() before the first remote store
  pdl_wait();                // nothing is read or written before the predecessor has completed

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  const int kc = D / CL;              // k slice of this CTA
  const int ksteps = kc / 32;
  const int xs_stride = kc * 2 + kXPadBytes;
  unsigned char* xs = smem;
  float* part = reinterpret_cast<float*>(smem + (size_t)TM * xs_stride);

  const int neuron0 = tile * kTileN;
  const __nv_bfloat16* w_lo =
      w + (size_t)(neuron0 + warp * STRIPS * 16 + g) * D + crank * kc + t * 8;
  const size_t strip_elems = (size_t)16 * D, half_elems = (size_t)8 * D;

  // Weight loads do not depend on shared memory: put the first steps in flight
  // before staging x.
  uint4 a_lo[STRIPS][PF], a_hi[STRIPS][PF];
#pragma unroll
  for (int u = 0; u < PF; ++u) {
    if (u < ksteps) {
#pragma unroll
      for (int i = 0; i < STRIPS; ++i) {
        a_lo[i][u] = ldg_stream(w_lo + i * strip_elems + u * 32);
        a_hi[i][u] = ldg_stream(w_lo + i * strip_elems + half_elems + u * 32);
      }
    }
  }

  // Stage this CTA's slice of the x tile (rows past M are zero-filled).
  {
    const int vec_per_row = kc / 8;
    for (int i = tid; i < TM * vec_per_row; i += NTHREADS) {
      const int r = i / vec_per_row, c = i - r * vec_per_row;
      const bool ok = m0 + r < M;
      const __nv_bfloat16* src = x + (size_t)(ok ? m0 + r : 0) * D + crank * kc + c * 8;
      cp_async16(xs + (size_t)r * xs_stride + c * 16, src, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
  }
  __syncthreads();

  float acc[STRIPS][NT][4];
#pragma unroll
  for (int i = 0; i < STRIPS; ++i)
#pragma unroll
    for (int n = 0; n < NT; ++n) acc[i][n][0] = acc[i][n][1] = acc[i][n][2] = acc[i][n][3] = 0.f;

  const unsigned char* xs_thread = xs + (size_t)g * xs_stride + t * 16;
  // Each register buffer is refilled (step s + PF) right after its last use.
  for (int s0 = 0; s0 < ksteps; s0 += PF) {
#pragma unroll
    for (int u = 0; u < PF; ++u) {
      const int s = s0 + u;
      if (s < ksteps) {
        uint4 lo[STRIPS], hi[STRIPS];
#pragma unroll
        for (int i = 0; i < STRIPS; ++i) {
          lo[i] = a_lo[i][u];
          hi[i] = a_hi[i][u];
        }
        if (s + PF < ksteps) {
#pragma unroll
          for (int i = 0; i < STRIPS; ++i) {
            a_lo[i][u] = ldg_stream(w_lo + i * strip_elems + (s + PF) * 32);
            a_hi[i][u] = ldg_stream(w_lo + i * strip_elems + half_elems + (s + PF) * 32);
          }
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const uint4 b = *reinterpret_cast<const uint4*>(xs_thread + (size_t)n * 8 * xs_stride +
                                                          s * 64);
#pragma unroll
          for (int i = 0; i < STRIPS; ++i) {
            mma_bf16_16816(acc[i][n], lo[i].x, hi[i].x, lo[i].y, hi[i].y, b.x, b.y);
            mma_bf16_16816(acc[i][n], lo[i].z, hi[i].z, lo[i].w, hi[i].w, b.z, b.w);
          }
        }
      }
    }
  }

  // Push the partial pre-activations to the CTA that finalises each token:
  // owner r receives rank q's values in part[(q*TOK + local token)][neuron].
  cluster.barrier_wait();  // every CTA of the cluster is running (arrived at kernel start)
#pragma unroll
  for (int n = 0; n < NT; ++n) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int tok = n * 8 + 2 * t + j;
      const int owner = tok / TOK, tl = tok % TOK;
      float* dst = cluster.map_shared_rank(part, owner) +
                   (size_t)(crank * TOK + tl) * kPartStride + warp * STRIPS * 16 + g;
#pragma unroll
      for (int i = 0; i < STRIPS; ++i) {
        dst[i * 16] = acc[i][n][j];
        dst[i * 16 + 8] = acc[i][n][2 + j];
      }
    }
  }
  cluster.sync();

  // This CTA finalises tokens [crank*TOK, (crank+1)*TOK): sum the cluster's
  // partials in rank order, then ballot per (token, 32-neuron chunk).
  float z[EPT];
  uint32_t mask[EPT];
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = tid + i * NTHREADS;
    const int tl = e / kTileN, nl = e % kTileN;
    const int tok = crank * TOK + tl;
    float v = 0.f;
#pragma unroll
    for (int r = 0; r < CL; ++r) v += part[(size_t)(r * TOK + tl) * kPartStride + nl];
    if (bias != nullptr) v += bias[neuron0 + nl];
    const bool keep = (v > 0.f) && (m0 + tok < M);
    z[i] = v;
    mask[i] = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) cnt_chunk[tl][nl / 32] = __popc(mask[i]);
  }
  __syncthreads();

#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = tid + i * NTHREADS;
    const int tl = e / kTileN, nl = e % kTileN;
    const int tok = crank * TOK + tl;
    if (m0 + tok >= M) continue;
    uint32_t* slab = packed + (size_t)(m0 + tok) * row_words + (size_t)tile * slab_w;
    int before = 0, total = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int v = cnt_chunk[tl][c];
      if (c < nl / 32) before += v;
      total += v;
    }
    if (nl == 0) slab[0] = (uint32_t)total;
    const int slot = before + __popc(mask[i] & lanemask_lt());
    if (((mask[i] >> lane) & 1u) && slot < slab_w - 1)
      slab[1 + slot] = (uint32_t)(neuron0 + nl) | (bf16_bits(z[i]) << 16);
  }
}

template <int TM, int CL, int WARPS, int STRIPS, int PF, int MINB>
int launch_pack(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                int64_t D, int64_t H, int cf, cudaStream_t stream) {
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  const int kc = (int)(D / CL);
  const size_t smem = (size_t)TM * (kc * 2 + kXPadBytes) + (size_t)TM * kPartStride * sizeof(float);

  auto kern = twell_pack_kernel<TM, CL, WARPS, STRIPS, PF, MINB>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_pack")) return rc;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * CL), (unsigned)((M + TM - 1) / TM), 1);
  cfg.blockDim = dim3(WARPS * 32, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = add_pdl_attribute(attr, 1, 1);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, reinterpret_cast<const __nv_bfloat16*>(x),
                                     reinterpret_cast<const __nv_bfloat16*>(w), bias,
                                     reinterpret_cast<uint32_t*>(packed), (int)M, (int)D, slab_w,
                                     tiles * slab_w);
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "b200_twell_pack: launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

}  // namespace

int twell_pack_small(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                     int64_t D, int64_t H, int cf, cudaStream_t stream) {
  // Token-tile height: no larger than M needs.
  int tm = 32;
  while (tm > 8 && tm / 2 >= M) tm /= 2;
  // Measured on B200 (d_model 2048, d_ff 8192): up to 16 tokens, 8 k slices with two
  // 256-thread CTAs per SM win (one CTA's epilogue overlaps the other's streaming);
  // at 32 tokens the mma work per CTA favours 4 k slices with one 512-thread CTA.
  switch (tm) {
    case 32: return launch_pack<32, 4, 16, 1, 8, 1>(x, w, bias, packed, M, D, H, cf, stream);
    case 16: return launch_pack<16, 8, 8, 2, 4, 2>(x, w, bias, packed, M, D, H, cf, stream);
    default: return launch_pack<8, 8, 8, 2, 4, 2>(x, w, bias, packed, M, D, H, cf, stream);
  }
}

}  // namespace b200
