// TwELL -> dense contraction (gated up/down and plain down projection).
//
// A token's stored entries (over all slabs) are numbered 0..n-1 and divided
// evenly over nc thread-block clusters of cs CTAs.  A CTA has one warp per
// 256-column slice of d_model.  Entries are processed in batches; the up and
// down rows of a whole batch are requested together (128-bit loads), so a batch
// costs one memory round trip:
//   pass A (gated only): warp s dots its slice of the token's x row (8 values per
//           lane, in registers) with the same slice of up[j, :];
//           slice sums meet in shared memory and give u, then h = g * u;
//   pass B: warp s adds h * down[j, slice s] into 8 accumulators per lane - each
//           warp owns its output columns, so no reduction inside the CTA.
// The CTA pushes its column sums into the owning CTA of its cluster through
// distributed shared memory; after one cluster barrier the owner adds the
// cluster's contributions in rank order.  With one cluster per token it stores
// bf16 directly.  With several (few tokens: spread one token over the whole
// GPU) each owner writes its fp32 column sums to the workspace and bumps a
// counter; the last owner to arrive adds the nc partial sums in cluster order,
// stores bf16 and resets the counter.  Every sum has a fixed order: the result
// is deterministic.
//
// Numerics follow the reference kernels: mixed mode rounds every product to
// bf16 before the fp32 add and rounds h to bf16
// (custom_models/twell_modules/matmul_gated_t2d.cu:74-149, matmul_t2d.cu:56-95);
// high-precision mode uses fp32 fma throughout (matmul_gated_t2d.cu:389-441).
// The reference's flex variants (:174-324, :466-594) differ only in how the slab
// is read; this kernel reads any slab width.  The output row may alias the
// input row (in-place variants, :972-1541): every CTA reads x before the
// barrier / counter that precedes the first store.
#include <cooperative_groups.h>

#include <atomic>
#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kMaxTiles = 256;  // H <= 65536
constexpr int kChunk = 256;     // entries staged in shared memory at a time
#ifndef B200_T2D_DEPTH
#define B200_T2D_DEPTH 8
#endif
constexpr int kDepth = B200_T2D_DEPTH;  // entries per batch (row loads in flight per lane: 2x gated)
constexpr int kStageWords = 4096;  // slab rows up to this many words are staged in shared memory

__device__ __forceinline__ uint4 ldg_nc(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// ---- contraction fused with the d_ff-shard all-reduce ------------------------------
// With world > 1 the CTA that holds the final sums of a (token, column slice) does not store
// them: it rounds them to bf16 (exactly what the unfused path would have stored), sends each
// bf16 pair to every peer GPU as one 8-byte word {pair, call epoch} (plain peer stores into
// the peers' inboxes; no fence, no TMA, no multicast), polls its own inbox - bounded - for
// the peers' words of the same pairs, adds the world contributions in rank order in fp32 and
// only then stores bf16.  Same result as contraction + b200_peer_allreduce_bf16, one kernel
// and one pass over `out` less.  Block layout per rank (symmetric):
//   word 0 epoch of the last finished call, word 1 finished (token, slice) groups of the
//   running call, word 2 error word; from 1 KB on inbox[parity][source rank][pair] of uint2,
//   pair = (token * D + column) / 2 - independent of how the call is cut into CTAs.
// The inbox is double-buffered by the epoch's parity (a pair is rewritten two calls later,
// which a peer can reach only after this rank has finished the call in between).
constexpr uint32_t kFarSpinLimit = 1u << 22;
constexpr uint32_t kFarShortSpinLimit = 1u << 10;  // once the error word is set (sticky)

__device__ __forceinline__ uint32_t bf162_bits(__nv_bfloat162 v) {
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void far_push(const FusedAr& ar, size_t inbox_off, size_t pair,
                                         uint32_t payload, uint32_t e) {
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    if (p >= ar.world || p == ar.rank) continue;
    uint2* dst = reinterpret_cast<uint2*>(ar.block[p] + inbox_off +
                                          (size_t)ar.rank * (size_t)ar.slot_bytes) + pair;
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(payload), "r"(e)
                 : "memory");
  }
}

// Sum over ranks, in rank order, of the bf16 pairs of one position; `mine` is this rank's.
__device__ __forceinline__ float2 far_gather(const FusedAr& ar, const unsigned char* my_inbox,
                                             size_t pair, uint32_t mine, uint32_t e,
                                             uint32_t* err, uint32_t& limit) {
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    if (p >= ar.world) continue;
    uint32_t payload = mine;
    if (p != ar.rank) {
      const uint2* src = reinterpret_cast<const uint2*>(my_inbox + (size_t)p * (size_t)ar.slot_bytes) + pair;
      uint32_t flag = 0, spins = 0;
      do {
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];"
                     : "=r"(payload), "=r"(flag)
                     : "l"(src)
                     : "memory");
      } while (flag != e && ++spins < limit);
      if (flag != e) {
        atomicExch(err, 0x100u + (uint32_t)p);  // this peer never arrived
        limit = kFarShortSpinLimit;             // the remaining waits of this thread drain fast
      }
    }
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&payload));
    s0 += f.x;
    s1 += f.y;
  }
  return make_float2(s0, s1);
}

// NI = D / 256 = warps per CTA.
// grid.x = M * nc * cs, cluster = cs.  ws_partial: [M][nc][D] fp32, ws_counter: [M][8] (nc > 1).
template <int NI, bool GATED, bool HP>
__global__ void __launch_bounds__(NI * 32)
twell_t2d_kernel(const __nv_bfloat16* x, const uint32_t* __restrict__ packed,
                 const __nv_bfloat16* __restrict__ up, const __nv_bfloat16* __restrict__ down,
                 __nv_bfloat16* out, int M, int tiles, int slab_w, int cs, int nc,
                 float* ws_partial, unsigned int* ws_counter,
                 const unsigned char* __restrict__ skip_rows,
                 const __grid_constant__ FusedAr ar) {
  constexpr int D = NI * 256;
  constexpr int NTHREADS = NI * 32;
  __shared__ int tile_off[kMaxTiles + 1];
  __shared__ uint32_t entries[kChunk];
  __shared__ float usum[2][GATED ? kDepth : 1][GATED ? NI : 1];  // double-buffered per batch
  __shared__ __align__(16) float inbox[D];  // [cs][D / cs]: column sums pushed by the cluster
  __shared__ int is_last;
  __shared__ uint32_t epoch_s, far_limit_s;
  __shared__ __align__(16) uint32_t slab_s[kStageWords];

  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int crank = blockIdx.x % cs;
  const int cidx = (blockIdx.x / cs) % nc;
  const int row = blockIdx.x / (cs * nc);
  // Nothing of the predecessor's output (slab, routing flags) is read before it has completed.
  pdl_wait();
  // Rows routed to the dense tensor-core path: every CTA of every cluster of the row leaves
  // (the row is uniform per cluster, so no cluster barrier is left half-attended).
  if (skip_rows != nullptr && skip_rows[row]) return;
  // Fused all-reduce: every CTA reads the call epoch now (the round trip hides under the slab
  // load).  It is advanced by the last (token, slice) group to finish, which cannot happen
  // before every CTA of the grid has contributed its partial sums, i.e. has started.
  const bool fused = ar.world > 1;
  unsigned char* my_block = nullptr;
#pragma unroll
  for (int p = 0; p < 8; ++p)
    if (p == ar.rank) my_block = ar.block[p];
  if (fused && tid == 0) {
    epoch_s = reinterpret_cast<volatile uint32_t*>(my_block)[kFarEpochWord] + 1u;
    // The error word stays set until the host reads it: after one peer failed to arrive,
    // later waits (this call and the following ones) give up after a short spin.
    far_limit_s = reinterpret_cast<volatile uint32_t*>(my_block)[kFarErrorWord] != 0u
                      ? kFarShortSpinLimit
                      : kFarSpinLimit;
  }
  const uint32_t* prow = packed + (size_t)row * tiles * slab_w;
  // Remote shared memory may only be touched once every CTA of the cluster runs:
  // arrive now, wait right before the first remote store.
  cluster.barrier_arrive();

  // This lane's 8 values of the x row (columns warp*256 + lane*8 .. +7).
  uint4 xv = make_uint4(0u, 0u, 0u, 0u);
  if (GATED) xv = *reinterpret_cast<const uint4*>(x + (size_t)row * D + warp * 256 + lane * 8);

  // One round trip brings the token's whole slab row on chip when it fits; the
  // count words and entry words are then read from shared memory.
  const int row_words = tiles * slab_w;
  const bool staged = row_words <= kStageWords;
  if (staged) {
    for (int i = tid; i < row_words / 4; i += NTHREADS)
      reinterpret_cast<uint4*>(slab_s)[i] = __ldg(reinterpret_cast<const uint4*>(prow) + i);
    __syncthreads();
  }
  const uint32_t* src = staged ? slab_s : prow;

  // Exclusive prefix of the per-slab entry counts (warp 0).
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < tiles; base += 32) {
      const int tI = base + lane;
      int c = 0;
      if (tI < tiles) {
        c = (int)src[(size_t)tI * slab_w];
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
  const int parts = cs * nc;
  const int per = (n_total + parts - 1) / parts;
  const int lo = (cidx * cs + crank) * per;
  const int hi = min(n_total, lo + per);

  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  int buf = 0;

  const __nv_bfloat16* up_lane = up + warp * 256 + lane * 8;
  const __nv_bfloat16* down_lane = down + warp * 256 + lane * 8;
  const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);

  for (int c0 = lo; c0 < hi; c0 += kChunk) {
    const int n = min(kChunk, hi - c0);
    // Gather this chunk's entry words: thread i finds entry c0 + i by binary search.
    for (int i = tid; i < n; i += NTHREADS) {
      const int k = c0 + i;
      int a = 0, b = tiles;  // largest tile with tile_off[tile] <= k
      while (b - a > 1) {
        const int mid = (a + b) >> 1;
        if (tile_off[mid] <= k) a = mid; else b = mid;
      }
      const uint32_t word = src[(size_t)a * slab_w + 1 + (k - tile_off[a])];
      entries[i] = word;
    }
    __syncthreads();

    // Row loads of a batch: kDepth entries, this lane's 16 bytes of the up and the down row.
    auto fetch = [&](int e0, uint4 (&uv)[GATED ? kDepth : 1], uint4 (&dv)[kDepth]) {
#pragma unroll
      for (int q = 0; q < kDepth; ++q) {
        if (e0 + q < n) {
          const size_t roff = (size_t)(entries[e0 + q] & 0xFFFFu) * D;
          if (GATED) uv[q] = ldg_nc(up_lane + roff);
          dv[q] = ldg_nc(down_lane + roff);
        } else {
          if (GATED) uv[q] = make_uint4(0u, 0u, 0u, 0u);
          dv[q] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    };
    auto consume = [&](int e0, uint4 (&uv)[GATED ? kDepth : 1], uint4 (&dv)[kDepth]) {
      if (GATED) {
        // pass A: this warp's slice of the kDepth dot products (independent chains)
        float u[kDepth];
#pragma unroll
        for (int q = 0; q < kDepth; ++q) {
          const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&uv[q]);
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
          u[q] = s;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
          for (int q = 0; q < kDepth; ++q) u[q] += __shfl_xor_sync(0xffffffffu, u[q], o);
        }
        if (lane == 0) {
#pragma unroll
          for (int q = 0; q < kDepth; ++q) usum[buf][q][warp] = u[q];
        }
        __syncthreads();
      }
      // h of entry e0 + lane (fixed-order sum over the slices), then broadcast.
      float h_lane = 0.f;
      if (lane < kDepth && e0 + lane < n) {
        const __nv_bfloat16 gval = __ushort_as_bfloat16((unsigned short)(entries[e0 + lane] >> 16));
        if (GATED) {
          float s = 0.f;
#pragma unroll
          for (int sI = 0; sI < NI; ++sI) s += usum[buf][lane][sI];
          h_lane = HP ? __bfloat162float(gval) * s
                      : __bfloat162float(__hmul(gval, __float2bfloat16_rn(s)));
        } else {
          h_lane = __bfloat162float(gval);
        }
      }
      // pass B: column-sliced down projection (padding entries have h = 0, row = 0)
#pragma unroll
      for (int q = 0; q < kDepth; ++q) {
        const float h = __shfl_sync(0xffffffffu, h_lane, q);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&dv[q]);
        if (HP) {
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const float2 wf = __bfloat1622float2(w2[p]);
            acc[2 * p] = __fmaf_rn(wf.x, h, acc[2 * p]);
            acc[2 * p + 1] = __fmaf_rn(wf.y, h, acc[2 * p + 1]);
          }
        } else {
          const __nv_bfloat162 hb2 = __float2bfloat162_rn(h);  // h is bf16-representable
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const float2 pf = __bfloat1622float2(__hmul2(hb2, w2[p]));
            acc[2 * p] += pf.x;
            acc[2 * p + 1] += pf.y;
          }
        }
      }
      buf ^= 1;
    };
    // One batch at a time.  Requesting batch b + 1 before batch b is reduced (two register
    // buffers) was measured and does not pay: with 4 entries per buffer 13.97 vs 12.32 us per
    // launch at batch 32, and 6 or 8 per buffer push the kernel past 128 registers and halve
    // its occupancy (23.9 / 25.5 us).
    for (int e0 = 0; e0 < n; e0 += kDepth) {
      uint4 uv[GATED ? kDepth : 1], dv[kDepth];
      fetch(e0, uv, dv);
      consume(e0, uv, dv);
    }
    __syncthreads();  // entries are rewritten by the next chunk
  }

  // Push this CTA's column sums to the owners: CTA r owns columns [r*cols, (r+1)*cols)
  // and receives rank q's contribution in inbox[q*cols .. (q+1)*cols).
  const int cols = D / cs;
  cluster.barrier_wait();
  {
    const int c = warp * 256 + lane * 8;  // first of this lane's 8 columns
    const int owner = c / cols, off = c - owner * cols;
    float* dst = cluster.map_shared_rank(inbox, owner) + (size_t)crank * cols + off;
    *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  cluster.sync();

  __nv_bfloat16* orow = out + (size_t)row * D + crank * cols;
  // Final sums of a column pair: stored, or (fused all-reduce) sent to the peers and kept.
  // A thread finishes at most 4 pairs (cols <= D = 8 * NTHREADS), pair k at column
  // c = 2 * (tid + k * NTHREADS).
  const uint32_t e = fused ? epoch_s : 0u;
  const size_t inbox_off = kFarControlBytes + (size_t)(e & 1u) * 8 * (size_t)ar.slot_bytes;
  const size_t pair0 = ((size_t)row * D + (size_t)crank * cols) >> 1;
  __nv_bfloat162 mine[4];
  auto emit = [&](int k, int c, float s0, float s1) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(s0, s1);
    if (!fused) {
      *reinterpret_cast<__nv_bfloat162*>(orow + c) = v;
    } else {
      mine[k] = v;
      far_push(ar, inbox_off, pair0 + (c >> 1), bf162_bits(v), e);
    }
  };
  // Fused: wait for the peers' pairs, add in rank order, store.  The last of the M * cs
  // finishing CTAs of the call advances the call epoch.
  auto collect = [&]() {
    if (!fused) return;
    uint32_t* ctl = reinterpret_cast<uint32_t*>(my_block);
    uint32_t limit = far_limit_s;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = 2 * (tid + k * NTHREADS);
      if (c >= cols) break;
      const float2 s = far_gather(ar, my_block + inbox_off, pair0 + (c >> 1), bf162_bits(mine[k]),
                                  e, ctl + kFarErrorWord, limit);
      *reinterpret_cast<__nv_bfloat162*>(orow + c) = __floats2bfloat162_rn(s.x, s.y);
    }
    __syncthreads();
    if (tid == 0) {
      const uint32_t done = atomicAdd(ctl + kFarDoneWord, 1u);
      if (done == (uint32_t)(M * cs) - 1u) {
        ctl[kFarDoneWord] = 0u;
        __threadfence();
        reinterpret_cast<volatile uint32_t*>(ctl)[kFarEpochWord] = e;
      }
    }
  };
  if (nc == 1) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = 2 * (tid + k * NTHREADS);
      if (c >= cols) break;
      float s0 = 0.f, s1 = 0.f;
      for (int q = 0; q < cs; ++q) {
        const float2 v = *reinterpret_cast<const float2*>(inbox + (size_t)q * cols + c);
        s0 += v.x;
        s1 += v.y;
      }
      emit(k, c, s0, s1);
    }
    collect();
    return;
  }

  // Several clusters per token: publish this cluster's column sums, last arrival finishes.
  float* my_part = ws_partial + ((size_t)row * nc + cidx) * D + crank * cols;
  for (int c = tid * 2; c < cols; c += NTHREADS * 2) {
    float s0 = 0.f, s1 = 0.f;
    for (int q = 0; q < cs; ++q) {
      const float2 v = *reinterpret_cast<const float2*>(inbox + (size_t)q * cols + c);
      s0 += v.x;
      s1 += v.y;
    }
    __stcg(reinterpret_cast<float2*>(my_part + c), make_float2(s0, s1));
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int old = atomicAdd(&ws_counter[row * 8 + crank], 1u);
    is_last = (old == (unsigned int)(nc - 1));
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const float* tok_part = ws_partial + (size_t)row * nc * D + crank * cols;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = 2 * (tid + k * NTHREADS);
    if (c >= cols) break;
    float s0 = 0.f, s1 = 0.f;
    for (int q = 0; q < nc; ++q) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(tok_part + (size_t)q * D + c));
      s0 += v.x;
      s1 += v.y;
    }
    emit(k, c, s0, s1);
  }
  if (tid == 0) ws_counter[row * 8 + crank] = 0u;  // ready for the next launch
  collect();
}

template <int NI, bool GATED, bool HP>
int launch_t2d(const void* x, const void* packed, const void* up, const void* down, void* out,
               int64_t M, int64_t H, int cf, int cs, int nc, float* ws_partial,
               unsigned int* ws_counter, const unsigned char* skip_rows, const FusedAr& ar,
               cudaStream_t stream) {
  const int slab_w = kTileN / cf;
  const int tiles = (int)(H / kTileN);
  auto kern = twell_t2d_kernel<NI, GATED, HP>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(M * nc * cs), 1, 1);
  cfg.blockDim = dim3(NI * 32, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (ar.world > 1) {
    // A CTA of the fused form waits for remote data, and its peers wait for the data of every
    // CTA of this grid: all clusters must be resident at once.  Ask the occupancy calculator
    // for this kernel, block size and cluster size (cached per device and cluster size).
    static int max_clusters[64][4] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    const int slot = cs == 1 ? 0 : cs == 2 ? 1 : cs == 4 ? 2 : 3;
    if (max_clusters[dev][slot] == 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = -1;
      }
      max_clusters[dev][slot] = n;
    }
    if (M * nc > (int64_t)max_clusters[dev][slot]) {
      // fewer clusters per token until the grid fits one wave
      nc = (int)((int64_t)max_clusters[dev][slot] / M);
      if (nc < 1)
        return fail(B200_EUNSUPPORTED,
                    "twell_t2d: the fused all-reduce needs all %lld clusters of %d CTAs resident "
                    "at once (limit %d)", (long long)M, cs, max_clusters[dev][slot]);
      cfg.gridDim = dim3((unsigned)(M * nc * cs), 1, 1);
    }
  }
  cfg.numAttrs = add_pdl_attribute(attr, 1, 2);
  cudaError_t e = cudaLaunchKernelEx(
      &cfg, kern, reinterpret_cast<const __nv_bfloat16*>(x),
      reinterpret_cast<const uint32_t*>(packed), reinterpret_cast<const __nv_bfloat16*>(up),
      reinterpret_cast<const __nv_bfloat16*>(down), reinterpret_cast<__nv_bfloat16*>(out), (int)M,
      tiles, slab_w, cs, nc, ws_partial, ws_counter, skip_rows, ar);
  if (e != cudaSuccess) return fail(B200_ECUDA, "twell_t2d: launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

template <bool GATED, bool HP>
int dispatch_ni(int ni, const void* x, const void* packed, const void* up, const void* down,
                void* out, int64_t M, int64_t H, int cf, int cs, int nc, float* ws_partial,
                unsigned int* ws_counter, const unsigned char* skip_rows, const FusedAr& ar,
                cudaStream_t stream) {
  switch (ni) {
#define B200_CASE(N)                                                                           \
  case N:                                                                                      \
    return launch_t2d<N, GATED, HP>(x, packed, up, down, out, M, H, cf, cs, nc, ws_partial,   \
                                    ws_counter, skip_rows, ar, stream);
    B200_CASE(1) B200_CASE(2) B200_CASE(3) B200_CASE(4) B200_CASE(5) B200_CASE(6) B200_CASE(7)
    B200_CASE(8) B200_CASE(9) B200_CASE(10) B200_CASE(11) B200_CASE(12) B200_CASE(13)
    B200_CASE(14) B200_CASE(15) B200_CASE(16)
#undef B200_CASE
    default:
      return fail(B200_EUNSUPPORTED, "twell_t2d: D = %d is not compiled (supported: 256..4096)",
                  ni * 256);
  }
}

}  // namespace

// Workspace layout: [kCounterWords words][fp32 partial sums].  The first kT2dCounterWords
// words are this kernel's arrival counters; the last 64 words of the block belong to the
// cross-tile barrier of the fused decode kernel (twell_decode.cu).
constexpr size_t kCounterWords = 4096;
constexpr size_t kT2dCounterWords = kCounterWords - 64;

// Launch shape.  cs: CTAs per cluster (D / cs must stay a multiple of 8 columns).
// nc: clusters per token - more than one only when there are few tokens and the
// caller's workspace can hold the partial sums.
void t2d_shape(int64_t M, int64_t D, int sm_count, size_t workspace_bytes, int* cs_out,
               int* nc_out) {
  int cs = 1;
  while (cs < 8 && M * cs * 2 <= (int64_t)sm_count * 2 && (D / (cs * 2)) % 8 == 0) cs *= 2;
  int nc = 1;
  if (workspace_bytes > kCounterWords * 4 && M * 8 <= (int64_t)kT2dCounterWords) {
    const int64_t cap_floats = (int64_t)((workspace_bytes - kCounterWords * 4) / 4);
    int64_t want = ((int64_t)sm_count * 2) / (M * cs);  // about two CTAs per SM in total
    // Clusters per token are capped: every extra cluster adds a partial sum to the final
    // reduction.  Measured at one token (D 2048, H 8192, 28 layers): 0.479 ms per step with a
    // cap of 4..8, 0.483 with 16, 0.515 with 32, 0.514 with 1.  B200_T2D_MAX_NC overrides.
    static const int max_nc = [] {
      const char* e = getenv("B200_T2D_MAX_NC");
      const int v = e != nullptr ? atoi(e) : 8;
      return v >= 1 && v <= 32 ? v : 8;
    }();
    if (want > max_nc) want = max_nc;
    while (want > 1 && M * want * D > cap_floats) --want;
    if (want > 1) nc = (int)want;
  }
  *cs_out = cs;
  *nc_out = nc;
}

int twell_t2d_launch(bool gated, bool hp, const void* x, const void* packed, const void* up,
                     const void* down, void* out, int64_t M, int64_t D, int64_t H, int cf,
                     void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream,
                     const unsigned char* skip_rows = nullptr,
                     const FusedAr* fused_ar = nullptr) {
  int cs = 1, nc = 1;
  t2d_shape(M, D, sm_count, workspace != nullptr ? workspace_bytes : 0, &cs, &nc);
  FusedAr far = {};
  if (fused_ar != nullptr && fused_ar->world > 1) {
    // Every CTA must be resident while it waits for the peers (the exact residency check
    // is made against the occupancy calculator at launch).
    if (M * nc * cs > 2 * (int64_t)sm_count || M > kFarMaxTokens)
      return fail(B200_EUNSUPPORTED,
                  "twell_t2d: the fused all-reduce serves at most %d tokens in one wave (M = %lld)",
                  kFarMaxTokens, (long long)M);
    if ((int64_t)M * D * 4 > fused_ar->slot_bytes)
      return fail(B200_EWORKSPACE, "twell_t2d: %lld tokens do not fit the peer blocks' slots",
                  (long long)M);
    far = *fused_ar;
  }
  unsigned int* counters = reinterpret_cast<unsigned int*>(workspace);
  float* partial = workspace ? reinterpret_cast<float*>(counters + kCounterWords) : nullptr;
  const int ni = (int)(D / 256);
  auto run = [&](int cs_, int nc_) {
    if (gated) {
      return hp ? dispatch_ni<true, true>(ni, x, packed, up, down, out, M, H, cf, cs_, nc_, partial,
                                          counters, skip_rows, far, stream)
                : dispatch_ni<true, false>(ni, x, packed, up, down, out, M, H, cf, cs_, nc_,
                                           partial, counters, skip_rows, far, stream);
    }
    return hp ? dispatch_ni<false, true>(ni, x, packed, up, down, out, M, H, cf, cs_, nc_, partial,
                                         counters, skip_rows, far, stream)
              : dispatch_ni<false, false>(ni, x, packed, up, down, out, M, H, cf, cs_, nc_,
                                          partial, counters, skip_rows, far, stream);
  };
  int rc = run(cs, nc);
  // A fused call whose clusters are not all resident at once is retried with smaller clusters
  // (one cluster per token): wide d_model means 512-thread CTAs, one per SM.
  while (rc == B200_EUNSUPPORTED && far.world > 1 && cs > 1) {
    cs /= 2;
    rc = run(cs, 1);
  }
  return rc;
}

int sm_count();  // c_api.cu

}  // namespace b200

// ---------------------------------------------------------------------------
// Gated contraction for callers that must not allocate device memory.
//
// Some hosts hand a plugin a fixed set of buffers and forbid it to touch the
// allocator: an inference server that planned all of its device memory up front,
// a process whose pool belongs to another framework, a latency-critical loop in
// which cudaMalloc's implicit device synchronisation is not acceptable.  Such a
// caller still wants the few-token shape of the contraction (one token spread
// over many clusters), which needs scratch memory for partial sums and arrival
// counters.  Here that scratch is a fixed array inside the library image:
// every GPU that loads the library holds these bytes until the process exits.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = (size_t)1 << 20;  // counters + fp32 partial sums

// Device-side storage.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is never passed to a kernel directly.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch per device ordinal, resolved on first use.  Atomic:
// two host threads may make their first call on a device at the same time (both store the
// same address).
std::atomic<void*> g_static_scratch_ptr[64];

int static_scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess)
    return b200::fail(B200_ECUDA, "b200_twell_gated_t2d_noalloc: cudaGetDevice: %s",
                      cudaGetErrorString(e));
  if (dev < 0 || dev >= 64)
    return b200::fail(B200_EUNSUPPORTED,
                      "b200_twell_gated_t2d_noalloc: device ordinal %d is outside 0..63", dev);
  void* p = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    e = cudaGetSymbolAddress(&p, g_static_scratch);  // address on the CURRENT device
    if (e != cudaSuccess || p == nullptr)
      return b200::fail(B200_ECUDA, "b200_twell_gated_t2d_noalloc: cudaGetSymbolAddress: %s",
                        cudaGetErrorString(e));
    g_static_scratch_ptr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return B200_OK;
}

// Largest token count the built-in scratch serves: two clusters per token must fit
// their fp32 partial sums, and every token needs 8 arrival counters.
int noalloc_max_tokens(int64_t D) {
  const int64_t cap_floats = (int64_t)((kStaticScratchBytes - b200::kCounterWords * 4) / 4);
  const int64_t by_partials = cap_floats / (2 * D);
  const int64_t by_counters = (int64_t)b200::kT2dCounterWords / 8;
  return (int)(by_partials < by_counters ? by_partials : by_counters);
}

}  // namespace

extern "C" int b200_twell_gated_t2d_noalloc(const void* x, const void* packed, const void* up,
                                            const void* down, void* out, int64_t M, int64_t D,
                                            int64_t H, int cf, uint32_t flags, void* stream) {
  const char* fn = "b200_twell_gated_t2d_noalloc";
  if (int rc = b200::check_dims(fn, M, D, H, cf)) return rc;
  if (flags & ~B200_FLAG_HIGH_PRECISION)
    return b200::fail(B200_EINVAL, "%s: unknown flags 0x%x", fn, flags);
  const int max_tokens = noalloc_max_tokens(D);
  if (M > max_tokens)
    return b200::fail(B200_EWORKSPACE,
                      "%s: M = %lld exceeds the built-in scratch (%zu bytes hold at most %d tokens "
                      "at D = %lld); use b200_twell_gated_t2d with a caller workspace",
                      fn, (long long)M, kStaticScratchBytes, max_tokens, (long long)D);
  if (M == 0) return B200_OK;
  const void* ptrs[5] = {x, packed, up, down, out};
  const char* names[5] = {"x", "packed", "up", "down", "out"};
  for (int i = 0; i < 5; ++i) {
    if (ptrs[i] == nullptr) return b200::fail(B200_ENULL, "%s: %s is NULL", fn, names[i]);
    if (!b200::aligned16(ptrs[i]))
      return b200::fail(B200_EALIGN, "%s: %s is not 16-byte aligned", fn, names[i]);
  }
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left behind: the arrival counters
  // must start at zero (the partial sums are fully overwritten before they are read).
  cudaError_t e = cudaMemsetAsync(scratch, 0, b200::kT2dCounterWords * sizeof(unsigned int), st);
  if (e != cudaSuccess)
    return b200::fail(B200_ECUDA,
                      "%s: cudaMemsetAsync: %s (the stream must belong to the current device, "
                      "whose copy of the scratch array this call uses)", fn,
                      cudaGetErrorString(e));
  b200::pdl_suppressed() = true;  // the predecessor of this launch is the memset above
  const int rc = b200::twell_t2d_launch(true, (flags & B200_FLAG_HIGH_PRECISION) != 0, x, packed,
                                        up, down, out, M, D, H, cf, scratch, kStaticScratchBytes,
                                        b200::sm_count(), st);
  b200::pdl_suppressed() = false;
  return rc;
}
