// Building blocks shared by the tcgen05 kernels: mbarrier waits with an iteration limit,
// 2-D TMA loads (no multicast), shared-memory / instruction descriptors for K-major bf16
// tiles with 128-byte swizzle, tcgen05.mma / commit / ld wrappers and the host-side tensor
// map encoder.  Everything here is file-local to the including translation unit.
#pragma once

#include <cstdlib>
#include <cuda.h>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kStageK = 64;                 // k-values per stage (128 bytes per row)
constexpr int kATileBytes = 128 * 128;      // 128 rows x 128 bytes
constexpr int kThreadsTc = 192;             // warp 0 producer, warp 1 mma, warps 2..5 epilogue
constexpr uint32_t kSpinLimit = 1u << 22;

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

// The same for tiles of 32 k-values (64 bytes per row): 64-byte swizzle, 8-row groups 512 B apart.
__device__ __forceinline__ uint64_t umma_desc_sw64(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;                     // SWIZZLE_64B
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

// 8 consecutive accumulator columns of this warp's 32 TMEM lanes.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// Barrier 2 for `count` threads (count a multiple of 32).
__device__ __forceinline__ void named_barrier2(int count) {
  asm volatile("bar.sync 2, %0;" ::"r"(count) : "memory");
}

__device__ __forceinline__ void epi_barrier() {  // the 128 epilogue threads only
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// Barrier of the 128 epilogue threads that also ANDs a flag over them, so that a decision
// taken after a bounded wait (carry on / give up) is the same in every epilogue thread and
// no thread is left alone at a later epi_barrier().
__device__ __forceinline__ bool epi_barrier_and(bool v) {
  uint32_t r;
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\n"
      "bar.red.and.pred p, 1, 128, q;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(r)
      : "r"((uint32_t)v)
      : "memory");
  return r != 0;
}

// Named barrier `id` (1..15) for `count` threads (a multiple of 32).
__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Barrier `id` over `count` threads that also ANDs a flag over them.
__device__ __forceinline__ bool named_barrier_and(int id, int count, bool v) {
  uint32_t r;
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.u32 q, %3, 0;\n"
      "bar.red.and.pred p, %1, %2, q;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(r)
      : "r"(id), "r"(count), "r"((uint32_t)v)
      : "memory");
  return r != 0;
}

// Launch order of a (feature tiles, token blocks) grid.  CTAs start in the order of their linear
// index; walking that index down `group` token blocks before moving on to the next feature
// tile keeps the token rows of one group in L2 while the weight matrix streams past once per
// group instead of once per resident wave.  group <= 1 leaves (blockIdx.x, blockIdx.y) as is.
__device__ __forceinline__ void raster_remap(int group, int& tile, int& mblk) {
  tile = (int)blockIdx.x;
  mblk = (int)blockIdx.y;
  if (group <= 1) return;
  const int pid = (int)(blockIdx.y * gridDim.x + blockIdx.x);
  const int per_group = group * (int)gridDim.x;
  const int first = (pid / per_group) * group;
  const int rows = min(group, (int)gridDim.y - first);
  const int in_group = pid - (pid / per_group) * per_group;
  mblk = first + in_group % rows;
  tile = in_group / rows;
}

// ---- host side -------------------------------------------------------------
// Token blocks per raster group: none while the weight operand (weight_bytes) stays resident in
// L2 by itself; otherwise as many blocks as put about 32 MB of token rows (block_bytes each)
// into one group.  B200_TC_RASTER=<n> forces a group size (1 = off).
inline int raster_group(int64_t weight_bytes, int64_t block_bytes) {
  static int forced = -2;
  if (forced == -2) {
    const char* e = getenv("B200_TC_RASTER");
    forced = e != nullptr ? atoi(e) : -1;
  }
  if (forced >= 1) return forced;
  if (weight_bytes <= (int64_t)48 << 20) return 1;
  const int64_t g = ((int64_t)32 << 20) / (block_bytes > 0 ? block_bytes : 1);
  return (int)(g < 4 ? 4 : g > 64 ? 64 : g);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is resolved through the runtime, so the library carries no
// link-time dependency on libcuda and still loads on a machine without a driver.
inline EncodeTiledFn encode_fn() {
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

// [rows, K] bf16 row-major; box = box_k (64 or 32) k-values x box_rows rows with the 128- or
// 64-byte swizzle that matches the row length, zero fill.
inline int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int box_rows,
                    int box_k = kStageK) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(B200_ECUDA, "tensor map: cuTensorMapEncodeTiled unavailable");
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_k, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  box_k == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B200_ECUDA, "tensor map: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return B200_OK;
}

}  // namespace
}  // namespace b200
