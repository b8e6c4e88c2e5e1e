// Shared helpers for the sm_100a sparse-FFN kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/b200_sparse_ffn.h"

namespace b200 {

constexpr int kTileN = 256;  // TwELL tile width in neurons (reference: twell.py:152)

// Thread-local text of the last failure, returned by b200_last_error().
char* last_error_buffer();
int fail(int code, const char* fmt, ...);

inline bool aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ECUDA, "%s: %s", what, cudaGetErrorString(e));
  return B200_OK;
}

// Validates the dimensions every entry point shares.
inline int check_dims(const char* fn, int64_t M, int64_t D, int64_t H, int cf) {
  if (cf != 2 && cf != 4 && cf != 8)
    return fail(B200_EINVAL, "%s: compression_factor must be one of {8, 4, 2} (got %d)", fn, cf);
  if (M < 0) return fail(B200_EINVAL, "%s: M must be >= 0 (got %lld)", fn, (long long)M);
  if (M > (int64_t)1 << 30) return fail(B200_EUNSUPPORTED, "%s: M too large (%lld)", fn, (long long)M);
  if (D < 256 || D > 8192 || D % 256)
    return fail(B200_EUNSUPPORTED, "%s: D must be a multiple of 256 in [256, 8192] (got %lld)", fn,
                (long long)D);
  if (H < 256 || H > 65536 || H % 256)
    return fail(B200_EUNSUPPORTED, "%s: H must be a multiple of 256 in [256, 65536] (got %lld)", fn,
                (long long)H);
  return B200_OK;
}

// Raises a kernel's dynamic shared-memory limit once per device and size.
template <typename Kernel>
inline int ensure_dynamic_smem(Kernel kern, size_t bytes, size_t (&granted)[64], const char* what) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (bytes <= granted[dev]) return B200_OK;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "%s: cannot reserve %zu bytes of shared memory: %s", what, bytes,
                cudaGetErrorString(e));
  granted[dev] = bytes;
  return B200_OK;
}

// Programmatic dependent launch.  A kernel launched with the attribute below is set up by the
// driver while its predecessor in the stream still runs; it must execute pdl_wait() before
// its first global read of data the predecessor may write and before its first global write
// (the wait returns once the predecessor grid has completed and its memory is visible).
// No kernel here issues griddepcontrol.launch_dependents: with an explicit early trigger the
// successor's CTAs become resident under the predecessor's tail and take shared memory and L1
// from it (measured on B200, decode stack at batch 32: 0.79-0.83 ms per step against 0.70
// without the attribute), whereas the implicit trigger at grid exit only removes the launch
// latency between the two kernels (0.677 ms).  pdl_wait() is a no-op in a kernel launched
// without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Whether the decode kernels are launched with programmatic stream serialisation
// (environment variable B200_PDL: "0" switches it off, anything else or unset keeps the
// built-in default).
bool pdl_enabled();

// Per-thread switch for launches whose predecessor in the stream is not a kernel (a memset).
inline bool& pdl_suppressed() {
  static thread_local bool suppressed = false;
  return suppressed;
}

// Which launches take the attribute: bit 0 the pack kernels (successors of a contraction),
// bit 1 the contraction kernel (successor of a pack kernel).  B200_PDL = 1 or 3 sets both,
// 2 only the contraction.
int pdl_mask();

// Appends the attribute to attrs[n] when enabled for this kind of launch (1 pack,
// 2 contraction); returns the new count.
inline unsigned add_pdl_attribute(cudaLaunchAttribute* attrs, unsigned n, int kind = 3) {
  if (!pdl_enabled() || pdl_suppressed() || !(pdl_mask() & kind)) return n;
  attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[n].val.programmaticStreamSerializationAllowed = 1;
  return n + 1;
}

// Peer blocks of the contraction fused with the d_ff-shard all-reduce (twell_t2d.cu).
// world <= 1 means "not fused".
struct FusedAr {
  unsigned char* block[8];
  int rank, world;
  long long slot_bytes;  // bytes of one (parity, source rank) inbox slot: 8 per bf16 pair
};
constexpr int kFarEpochWord = 0;            // epoch of the last finished call
constexpr int kFarDoneWord = 1;             // (token, slice) groups of the running call that finished
constexpr int kFarErrorWord = 2;            // set when a wait for a peer gave up
constexpr size_t kFarControlBytes = 1024;   // control words, padding; the inbox follows
constexpr int kFarMaxTokens = 256;

__device__ __forceinline__ uint32_t bf16_bits(float v) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}

__device__ __forceinline__ uint32_t lanemask_lt() {
  uint32_t m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

}  // namespace b200
