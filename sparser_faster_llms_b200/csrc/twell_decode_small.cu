// One kernel per sparse FFN layer for 1..16 tokens: the mma.sync split-k pack kernel of
// twell_pack.cu with the gated up/down contraction appended to it.
//
// Pack phase (unchanged): a cluster of CL CTAs owns a 256-neuron tile and splits d_model; the
// partial pre-activations meet in distributed shared memory and CTA q of the cluster finalises
// the tile for its TOK = TM / CL tokens (sum in rank order, ReLU, ballot / popc, slab words -
// the same bytes as b200_twell_pack).
//
// Contraction phase (new): the finalising CTA knows, for each of its tokens, the active
// neurons of the tile (about 5 of 256 at 2 % density) and their gate values.  With a thread
// owning 8 columns per 2048 of d_model it loads the token's x row once, then for every stored
// neuron - in ascending order, four at a time - the up row and the down row (one 128-bit load
// per thread and row, all loads of a batch in flight together), forms u = x . up (warp
// shuffles, then the eight warp sums added in warp order), h = g * u, and adds h * down into
// its 8 accumulators.  The (token, tile) partial row goes to the workspace; the last tile of a
// token to arrive (one counter per token) adds the tiles' rows in tile order and stores bf16.
// No CTA ever waits for another one, so the grid need not be resident at once, and every sum
// has a fixed order: deterministic.
//
// Numerics as in twell_t2d.cu: mixed mode rounds every product and h to bf16
// (custom_models/twell_modules/matmul_gated_t2d.cu:74-149), high precision is fp32 fma
// throughout (:389-441); entries beyond a slab's capacity are dropped, as the two-kernel path
// does.  Replaces the two launches of TWELL_MLP::run_gated_mlp_layer*
// (custom_models/twell_modules/mlp_twell.cu:126-152) for decode-sized calls.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kXPadBytes = 64;
constexpr int kPartStride = kTileN + 4;
constexpr int kSmallBatch = 4;  // neurons whose rows are in flight together

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

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int src_bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc),
               "r"(src_bytes));
}

// TM tokens per tile (8 or 16), CL k slices, 8 warps of STRIPS strips of 16 neurons
// (8 * STRIPS * 16 == 256), PF weight steps in flight, NCH = D / 2048 column chunks per thread.
// grid.x = (H / 256) * CL.  Dynamic shared memory as in twell_pack_kernel.
// ws_counter: one word per token, zero between launches; ws_part: [M][tiles][D] fp32.
template <int TM, int CL, int STRIPS, int PF, int NCH, bool GATED, bool HP>
__global__ void __launch_bounds__(256, 2)
twell_decode_small_kernel(const __nv_bfloat16* x, const __nv_bfloat16* __restrict__ w,
                          const float* __restrict__ bias, uint32_t* __restrict__ packed,
                          const __nv_bfloat16* __restrict__ up,
                          const __nv_bfloat16* __restrict__ down, __nv_bfloat16* out, int M, int D,
                          int slab_w, int row_words, float* ws_part, unsigned int* ws_counter) {
  constexpr int NTHREADS = 256, WARPS = 8;
  constexpr int NT = TM / 8;
  constexpr int TOK = TM / CL;
  static_assert(WARPS * STRIPS * 16 == kTileN, "a CTA covers one 256-neuron tile");
  static_assert(TOK >= 1 && TOK * kTileN % NTHREADS == 0, "one neuron per thread and token");
  constexpr uint32_t FULL = 0xffffffffu;

  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int cnt_chunk[TOK][8];
  __shared__ uint32_t bal_s[TOK][8];
  __shared__ unsigned short gz_s[TOK][kTileN];
  __shared__ float red_s[kSmallBatch][WARPS];
  __shared__ int is_last_s;

  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  const int tile = blockIdx.x / CL;
  const int tiles = gridDim.x / CL;
  cluster.barrier_arrive();

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  const int kc = D / CL;
  const int ksteps = kc / 32;
  const int xs_stride = kc * 2 + kXPadBytes;
  unsigned char* xs = smem;
  float* part = reinterpret_cast<float*>(smem + (size_t)TM * xs_stride);

  const int neuron0 = tile * kTileN;
  const __nv_bfloat16* w_lo =
      w + (size_t)(neuron0 + warp * STRIPS * 16 + g) * D + crank * kc + t * 8;
  const size_t strip_elems = (size_t)16 * D, half_elems = (size_t)8 * D;

  // ---- pack phase: as twell_pack_kernel ----
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
  {
    const int vec_per_row = kc / 8;
    for (int i = tid; i < TM * vec_per_row; i += NTHREADS) {
      const int r = i / vec_per_row, c = i - r * vec_per_row;
      const bool ok = r < M;
      const __nv_bfloat16* src = x + (size_t)(ok ? r : 0) * D + crank * kc + c * 8;
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

  cluster.barrier_wait();
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
  // From here on the CTA works alone (no remote shared memory is touched again).

  // ---- finalise: thread = neuron `tid` of the tile, for each of this CTA's tokens ----
#pragma unroll
  for (int tl = 0; tl < TOK; ++tl) {
    const int tok = crank * TOK + tl;
    float v = 0.f;
#pragma unroll
    for (int r = 0; r < CL; ++r) v += part[(size_t)(r * TOK + tl) * kPartStride + tid];
    if (bias != nullptr) v += bias[neuron0 + tid];
    const bool keep = (v > 0.f) && (tok < M);
    const uint32_t m = __ballot_sync(FULL, keep);
    gz_s[tl][tid] = (unsigned short)bf16_bits(v);
    if (lane == 0) {
      bal_s[tl][warp] = m;
      cnt_chunk[tl][warp] = __popc(m);
    }
  }
  __syncthreads();
#pragma unroll
  for (int tl = 0; tl < TOK; ++tl) {
    const int tok = crank * TOK + tl;
    if (tok >= M) continue;
    uint32_t* slab = packed + (size_t)tok * row_words + (size_t)tile * slab_w;
    int before = 0, total = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int cv = cnt_chunk[tl][c];
      if (c < warp) before += cv;
      total += cv;
    }
    if (tid == 0) slab[0] = (uint32_t)total;
    const uint32_t m = bal_s[tl][warp];
    const int slot = before + __popc(m & lanemask_lt());
    if (((m >> lane) & 1u) && slot < slab_w - 1)
      slab[1 + slot] = (uint32_t)(neuron0 + tid) | ((uint32_t)gz_s[tl][tid] << 16);
  }

  // ---- contraction of this CTA's (token, tile) pairs ----
  const int col0 = tid * 8;  // + c * 2048 for chunk c
#pragma unroll 1
  for (int tl = 0; tl < TOK; ++tl) {
    const int tok = crank * TOK + tl;
    if (tok >= M) continue;  // uniform over the CTA
    uint4 xv[NCH];
    if (GATED) {
#pragma unroll
      for (int c = 0; c < NCH; ++c)
        xv[c] = *reinterpret_cast<const uint4*>(x + (size_t)tok * D + c * 2048 + col0);
    }
    float y[NCH][8];
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int e = 0; e < 8; ++e) y[c][e] = 0.f;

    // walk the stored neurons in ascending order, kSmallBatch at a time
    int word = 0, stored = 0;
    uint32_t bits = bal_s[tl][0];
    const int cap = slab_w - 1;
    bool more = true;
    while (more) {
      int nb = 0;
      int nid[kSmallBatch];
#pragma unroll
      for (int q = 0; q < kSmallBatch; ++q) nid[q] = -1;
#pragma unroll
      for (int q = 0; q < kSmallBatch; ++q) {
        while (bits == 0u && word < 7) bits = bal_s[tl][++word];
        if (bits != 0u && stored < cap) {
          const int b = __ffs(bits) - 1;
          bits &= bits - 1u;
          nid[q] = word * 32 + b;
          ++stored;
          ++nb;
        }
      }
      if (nb == 0) break;
      more = (nb == kSmallBatch);
      uint4 uv[GATED ? kSmallBatch : 1][NCH], dv[kSmallBatch][NCH];
#pragma unroll
      for (int q = 0; q < kSmallBatch; ++q) {
        if (nid[q] >= 0) {
          const size_t roff = (size_t)(neuron0 + nid[q]) * D + col0;
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            if (GATED) uv[q][c] = __ldg(reinterpret_cast<const uint4*>(up + roff + c * 2048));
            dv[q][c] = __ldg(reinterpret_cast<const uint4*>(down + roff + c * 2048));
          }
        }
      }
      float hq[kSmallBatch];
      if (GATED) {
        float s[kSmallBatch];
#pragma unroll
        for (int q = 0; q < kSmallBatch; ++q) {
          s[q] = 0.f;
          if (nid[q] >= 0) {
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
              const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv[c]);
              const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&uv[q][c]);
#pragma unroll
              for (int p = 0; p < 4; ++p) {
                if (HP) {
                  const float2 wf = __bfloat1622float2(w2[p]), xf = __bfloat1622float2(x2[p]);
                  s[q] = __fmaf_rn(wf.x, xf.x, s[q]);
                  s[q] = __fmaf_rn(wf.y, xf.y, s[q]);
                } else {
                  const float2 pf = __bfloat1622float2(__hmul2(x2[p], w2[p]));
                  s[q] += pf.x;
                  s[q] += pf.y;
                }
              }
            }
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
          for (int q = 0; q < kSmallBatch; ++q) s[q] += __shfl_xor_sync(FULL, s[q], o);
        }
        if (lane == 0) {
#pragma unroll
          for (int q = 0; q < kSmallBatch; ++q) red_s[q][warp] = s[q];
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < kSmallBatch; ++q) {
          float u = 0.f;
#pragma unroll
          for (int wv = 0; wv < WARPS; ++wv) u += red_s[q][wv];
          const __nv_bfloat16 gv =
              __ushort_as_bfloat16(nid[q] >= 0 ? gz_s[tl][nid[q]] : (unsigned short)0);
          hq[q] = HP ? __bfloat162float(gv) * u
                     : __bfloat162float(__hmul(gv, __float2bfloat16_rn(u)));
        }
        __syncthreads();  // red_s is rewritten by the next batch
      } else {
#pragma unroll
        for (int q = 0; q < kSmallBatch; ++q)
          hq[q] = nid[q] >= 0 ? __bfloat162float(__ushort_as_bfloat16(gz_s[tl][nid[q]])) : 0.f;
      }
#pragma unroll
      for (int q = 0; q < kSmallBatch; ++q) {
        if (nid[q] < 0) continue;
        const __nv_bfloat162 hb2 = __float2bfloat162_rn(hq[q]);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&dv[q][c]);
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            if (HP) {
              const float2 wf = __bfloat1622float2(w2[p]);
              y[c][2 * p] = __fmaf_rn(wf.x, hq[q], y[c][2 * p]);
              y[c][2 * p + 1] = __fmaf_rn(wf.y, hq[q], y[c][2 * p + 1]);
            } else {
              const float2 pf = __bfloat1622float2(__hmul2(hb2, w2[p]));
              y[c][2 * p] += pf.x;
              y[c][2 * p + 1] += pf.y;
            }
          }
        }
      }
    }

    // publish the (token, tile) row; the last tile of the token to arrive finishes it
    float* mine = ws_part + ((size_t)tok * tiles + tile) * D + col0;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      __stcg(reinterpret_cast<float4*>(mine + c * 2048),
             make_float4(y[c][0], y[c][1], y[c][2], y[c][3]));
      __stcg(reinterpret_cast<float4*>(mine + c * 2048 + 4),
             make_float4(y[c][4], y[c][5], y[c][6], y[c][7]));
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned int old = atomicAdd(&ws_counter[tok], 1u);
      is_last_s = (old == (unsigned int)tiles - 1u);
    }
    __syncthreads();
    if (is_last_s) {
      __threadfence();
      const float* rows = ws_part + (size_t)tok * tiles * D + col0;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        float sum[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) sum[e] = 0.f;
#pragma unroll 4
        for (int q = 0; q < tiles; ++q) {
          const float4 a = __ldcg(reinterpret_cast<const float4*>(rows + (size_t)q * D + c * 2048));
          const float4 b =
              __ldcg(reinterpret_cast<const float4*>(rows + (size_t)q * D + c * 2048 + 4));
          sum[0] += a.x;
          sum[1] += a.y;
          sum[2] += a.z;
          sum[3] += a.w;
          sum[4] += b.x;
          sum[5] += b.y;
          sum[6] += b.z;
          sum[7] += b.w;
        }
        uint4 o;
        o.x = bf16_bits(sum[0]) | (bf16_bits(sum[1]) << 16);
        o.y = bf16_bits(sum[2]) | (bf16_bits(sum[3]) << 16);
        o.z = bf16_bits(sum[4]) | (bf16_bits(sum[5]) << 16);
        o.w = bf16_bits(sum[6]) | (bf16_bits(sum[7]) << 16);
        *reinterpret_cast<uint4*>(out + (size_t)tok * D + c * 2048 + col0) = o;
      }
      if (tid == 0) ws_counter[tok] = 0u;  // ready for the next launch
    }
    __syncthreads();  // is_last_s and red_s are reused by the next token
  }
}

template <int TM, int CL, int STRIPS, int PF, int NCH, bool GATED, bool HP>
int launch_small(const void* x, const void* w, const float* bias, const void* up,
                 const void* down, void* packed, void* out, int64_t M, int64_t D, int64_t H,
                 int cf, void* workspace, cudaStream_t stream) {
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  const int kc = (int)(D / CL);
  const size_t smem =
      (size_t)TM * (kc * 2 + kXPadBytes) + (size_t)TM * kPartStride * sizeof(float);
  auto kern = twell_decode_small_kernel<TM, CL, STRIPS, PF, NCH, GATED, HP>;
  static size_t granted[64] = {0};
  if (int rc = ensure_dynamic_smem(kern, smem, granted, "b200_twell_gated_mlp (decode)")) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * CL), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  unsigned int* words = reinterpret_cast<unsigned int*>(workspace);
  float* ws_part = reinterpret_cast<float*>(words + 4096);
  cudaError_t e = cudaLaunchKernelEx(
      &cfg, kern, reinterpret_cast<const __nv_bfloat16*>(x),
      reinterpret_cast<const __nv_bfloat16*>(w), bias, reinterpret_cast<uint32_t*>(packed),
      reinterpret_cast<const __nv_bfloat16*>(up), reinterpret_cast<const __nv_bfloat16*>(down),
      reinterpret_cast<__nv_bfloat16*>(out), (int)M, (int)D, slab_w, tiles * slab_w, ws_part, words);
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "b200_twell_gated_mlp (decode, small): launch: %s",
                cudaGetErrorString(e));
  return B200_OK;
}

template <int TM, int NCH>
int dispatch_small(bool gated, bool hp, const void* x, const void* w, const float* bias,
                   const void* up, const void* down, void* packed, void* out, int64_t M,
                   int64_t D, int64_t H, int cf, void* workspace, cudaStream_t stream) {
  if (!gated)
    return launch_small<TM, 8, 2, 4, NCH, false, false>(x, w, bias, up, down, packed, out, M, D,
                                                        H, cf, workspace, stream);
  return hp ? launch_small<TM, 8, 2, 4, NCH, true, true>(x, w, bias, up, down, packed, out, M, D,
                                                         H, cf, workspace, stream)
            : launch_small<TM, 8, 2, 4, NCH, true, false>(x, w, bias, up, down, packed, out, M, D,
                                                          H, cf, workspace, stream);
}

}  // namespace

// Whether the small-batch one-kernel form serves a call: 1..16 tokens, d_model 2048 or 4096.
bool twell_decode_small_serves(int64_t M, int64_t D, int64_t H) {
  return M >= 1 && M <= 16 && (D == 2048 || D == 4096) && H >= 256 && H % 256 == 0 &&
         H / 256 <= 255;
}

// Workspace: the 4096-word block (word `token` is that token's arrival counter) followed by
// [M][tiles][D] fp32 partial rows.
size_t twell_decode_small_workspace_bytes(int64_t M, int64_t D, int64_t H) {
  if (!twell_decode_small_serves(M, D, H)) return 0;
  return (size_t)4096 * 4 + (size_t)M * (size_t)(H / kTileN) * (size_t)D * 4;
}

int twell_decode_small_launch(bool gated, bool hp, const void* x, const void* w,
                              const float* bias, const void* up, const void* down, void* packed,
                              void* out, int64_t M, int64_t D, int64_t H, int cf, void* workspace,
                              size_t workspace_bytes, cudaStream_t stream) {
  if (!twell_decode_small_serves(M, D, H))
    return fail(B200_EUNSUPPORTED, "b200_twell_gated_mlp (decode, small): shape not served");
  if (workspace == nullptr || workspace_bytes < twell_decode_small_workspace_bytes(M, D, H))
    return fail(B200_EUNSUPPORTED,
                "b200_twell_gated_mlp (decode, small): workspace of %zu bytes needed",
                twell_decode_small_workspace_bytes(M, D, H));
  const bool two = D == 4096;
  if (M <= 8)
    return two ? dispatch_small<8, 2>(gated, hp, x, w, bias, up, down, packed, out, M, D, H, cf,
                                      workspace, stream)
               : dispatch_small<8, 1>(gated, hp, x, w, bias, up, down, packed, out, M, D, H, cf,
                                      workspace, stream);
  return two ? dispatch_small<16, 2>(gated, hp, x, w, bias, up, down, packed, out, M, D, H, cf,
                                     workspace, stream)
             : dispatch_small<16, 1>(gated, hp, x, w, bias, up, down, packed, out, M, D, H, cf,
                                     workspace, stream);
}

}  // namespace b200
