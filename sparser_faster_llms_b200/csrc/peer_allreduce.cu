// One-shot sum all-reduce of a small bf16 tensor over peer-mapped memory (NVLink / NVSwitch).
//
// The d_ff-sharded FFN ends with a sum of the ranks' partial outputs [M, D].  At decode that
// is 4..128 KB: a latency problem, not a bandwidth one, so the exchange is a single one-way
// trip with no fence and no separate flag.  Each rank owns a symmetric block (same layout on
// every GPU, every rank holds a pointer to every peer's block):
//
//   control | inbox parity 0: world slots | inbox parity 1: world slots
//
// A slot holds "flagged words": every 8 bytes are 4 bytes of payload followed by the 4-byte
// epoch of the call that wrote them.  An aligned 8-byte store is never torn, so a reader
// that sees the epoch in the upper half also sees the payload in the lower half.
// Per call (epoch e, parity e & 1) the thread that owns 16-byte vector i of the tensor
//   1. stores vector i of the local input, as two 16-byte flagged stores, into slot `rank`
//      of every peer's inbox (plain peer stores over NVLink; no TMA, no multicast),
//   2. polls - bounded - the same two words in every peer's slot of its own inbox until
//      all four flags read e,
//   3. sums in rank order (its own share comes from the local input) and stores bf16.
// Every rank adds the same values in the same order, so all ranks hold identical results.
// Slots are double-buffered by the parity of a device-side epoch, so a slot is rewritten
// only two calls later, which a peer can reach only after this rank has finished the call
// in between: no trailing barrier is needed, in eager launches or graph replays.  The
// epoch lives in device memory (one word per CTA, advanced by that CTA), so a captured
// launch advances it on every replay; the grid is always kArCtas CTAs for that reason.
// A wait that gives up records an error word (b200_peer_allreduce_status) and the thread
// continues with whatever arrived; it never spins forever.
//
// The reference has no counterpart (it is data parallel only; its collectives are
// DeepSpeed's NCCL calls, launch.sh:20-46).
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kArCtas = 32;
constexpr int kArThreads = 256;
constexpr uint32_t kArSpinLimit = 1u << 22;
constexpr uint32_t kArShortSpinLimit = 1u << 10;  // once the error word is set
// control block (uint32 words): epoch of the last finished call per CTA, then the error word
constexpr int kEpochOff = 0;
constexpr int kErrorOff = kArCtas;
constexpr size_t kControlBytes = 1024;
static_assert((kErrorOff + 1) * 4 <= (int)kControlBytes, "control block too small");

struct PeerBlocks {
  unsigned char* block[kMaxWorld];
};

__device__ __forceinline__ void st_flagged(uint4* p, uint32_t a, uint32_t b, uint32_t e) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(e), "r"(b),
               "r"(e)
               : "memory");
}

__device__ __forceinline__ uint4 ld_flagged(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ void add_pair(float& lo, float& hi, uint32_t packed) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&packed));
  lo += f.x;
  hi += f.y;
}

__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(kArThreads)
peer_allreduce_kernel(const __grid_constant__ PeerBlocks peers, const uint4* __restrict__ local_in, uint4* __restrict__ out,
                      int rank, int world, int64_t n_vec, int64_t slot_bytes) {
  __shared__ uint32_t epoch_s, limit_s;
  const int tid = threadIdx.x;
  unsigned char* my_block = nullptr;  // unrolled select: no runtime index into the parameter
#pragma unroll
  for (int p = 0; p < kMaxWorld; ++p)
    if (p == rank) my_block = peers.block[p];
  uint32_t* ctl = reinterpret_cast<uint32_t*>(my_block);
  const int64_t stride = (int64_t)kArCtas * kArThreads;
  const int64_t first = (int64_t)blockIdx.x * kArThreads + tid;
  uint4 mine = make_uint4(0u, 0u, 0u, 0u);
  if (first < n_vec) mine = local_in[first];  // in flight while the epoch is read
  if (tid == 0) {
    epoch_s = *reinterpret_cast<volatile uint32_t*>(ctl + kEpochOff + blockIdx.x) + 1u;
    // The error word is sticky until the host reads it: once a peer has failed to arrive,
    // every later wait (of this call and of the following calls) gives up after a short
    // spin, so a dead or late rank costs microseconds per call instead of seconds.
    limit_s = *reinterpret_cast<volatile uint32_t*>(ctl + kErrorOff) != 0u ? kArShortSpinLimit
                                                                             : kArSpinLimit;
  }
  __syncthreads();
  const uint32_t e = epoch_s;
  uint32_t limit = limit_s;
  // flagged slots are twice the payload: 2 * slot_bytes per (parity, source rank)
  const size_t inbox_off = kControlBytes + (size_t)(e & 1u) * kMaxWorld * 2 * (size_t)slot_bytes;

  // 1. push my vectors into slot `rank` of every peer's inbox
  for (int64_t i = first; i < n_vec; i += stride) {
    const uint4 v = (i == first) ? mine : local_in[i];
#pragma unroll
    for (int p = 0; p < kMaxWorld; ++p) {
      if (p >= world || p == rank) continue;
      uint4* dst = reinterpret_cast<uint4*>(peers.block[p] + inbox_off +
                                            (size_t)rank * 2 * (size_t)slot_bytes) + 2 * i;
      st_flagged(dst, v.x, v.y, e);
      st_flagged(dst + 1, v.z, v.w, e);
    }
  }
  // 2 + 3. wait for the peers' copies of my vectors, sum in rank order, store
  const unsigned char* inbox = my_block + inbox_off;
  for (int64_t i = first; i < n_vec; i += stride) {
    uint4 lo[kMaxWorld], hi[kMaxWorld];
    uint32_t pending = 0;
#pragma unroll
    for (int p = 0; p < kMaxWorld; ++p)
      if (p < world && p != rank) pending |= 1u << p;
    uint32_t spins = 0;
    while (pending) {
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p) {
        if (!((pending >> p) & 1u)) continue;
        const uint4* src = reinterpret_cast<const uint4*>(inbox + (size_t)p * 2 * (size_t)slot_bytes) +
                           2 * i;
        lo[p] = ld_flagged(src);
        hi[p] = ld_flagged(src + 1);
      }
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p) {
        if (!((pending >> p) & 1u)) continue;
        if (lo[p].y == e && lo[p].w == e && hi[p].y == e && hi[p].w == e) pending &= ~(1u << p);
      }
      if (pending && ++spins >= limit) {
        atomicExch(ctl + kErrorOff, 0x100u + (uint32_t)(__ffs(pending) - 1));  // who is missing
        limit = kArShortSpinLimit;
        break;
      }
    }
    const uint4 own = (i == first) ? mine : local_in[i];
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
    for (int p = 0; p < kMaxWorld; ++p) {
      if (p >= world) continue;
      if (p == rank) {
        add_pair(acc[0], acc[1], own.x);
        add_pair(acc[2], acc[3], own.y);
        add_pair(acc[4], acc[5], own.z);
        add_pair(acc[6], acc[7], own.w);
      } else {
        add_pair(acc[0], acc[1], lo[p].x);
        add_pair(acc[2], acc[3], lo[p].z);
        add_pair(acc[4], acc[5], hi[p].x);
        add_pair(acc[6], acc[7], hi[p].z);
      }
    }
    uint4 o;
    o.x = pack_pair(acc[0], acc[1]);
    o.y = pack_pair(acc[2], acc[3]);
    o.z = pack_pair(acc[4], acc[5]);
    o.w = pack_pair(acc[6], acc[7]);
    out[i] = o;
  }
  __syncthreads();
  if (tid == 0) *reinterpret_cast<volatile uint32_t*>(ctl + kEpochOff + blockIdx.x) = e;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_peer_allreduce_block_bytes(int64_t max_bytes) {
  if (max_bytes <= 0) return 0;
  const size_t slot = ((size_t)max_bytes + 255) & ~(size_t)255;
  return kControlBytes + 2 * (size_t)kMaxWorld * 2 * slot;
}

int b200_peer_allreduce_bf16(const void* local_in, void* out, int64_t n_elems,
                             void* const* peer_blocks, int rank, int world, int64_t block_bytes,
                             void* stream) {
  const char* fn = "b200_peer_allreduce_bf16";
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
    return fail(B200_EINVAL, "%s: need 1 <= world <= %d and 0 <= rank < world", fn, kMaxWorld);
  if (n_elems < 0 || n_elems % 8) return fail(B200_EINVAL, "%s: n_elems must be a multiple of 8", fn);
  if (n_elems == 0) return B200_OK;
  if (local_in == nullptr || out == nullptr || peer_blocks == nullptr)
    return fail(B200_ENULL, "%s: a required pointer is NULL", fn);
  if (!aligned16(local_in) || !aligned16(out))
    return fail(B200_EALIGN, "%s: local_in / out not 16-byte aligned", fn);
  if (block_bytes < (int64_t)kControlBytes + 4 * kMaxWorld * 256)
    return fail(B200_EWORKSPACE, "%s: block_bytes too small", fn);
  const int64_t slot_bytes = ((block_bytes - (int64_t)kControlBytes) / (4 * kMaxWorld)) & ~(int64_t)255;
  if (n_elems * 2 > slot_bytes)
    return fail(B200_EWORKSPACE, "%s: %lld bytes do not fit a %lld-byte slot", fn,
                (long long)(n_elems * 2), (long long)slot_bytes);
  PeerBlocks pb;
  for (int r = 0; r < kMaxWorld; ++r) pb.block[r] = nullptr;
  for (int r = 0; r < world; ++r) {
    if (peer_blocks[r] == nullptr) return fail(B200_ENULL, "%s: peer block %d is NULL", fn, r);
    if (!aligned16(peer_blocks[r])) return fail(B200_EALIGN, "%s: peer block %d misaligned", fn, r);
    pb.block[r] = static_cast<unsigned char*>(peer_blocks[r]);
  }
  peer_allreduce_kernel<<<kArCtas, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      pb, static_cast<const uint4*>(local_in), static_cast<uint4*>(out), rank, world, n_elems / 8,
      slot_bytes);
  return check_launch(fn);
}

/* Reads and clears the error word of this rank's block (0 = no wait ever gave up).
 * Synchronises the device. */
int b200_peer_allreduce_status(void* my_block) {
  if (my_block == nullptr) return -1;
  uint32_t v = 0, zero = 0;
  uint32_t* p = static_cast<uint32_t*>(my_block) + kErrorOff;
  if (cudaMemcpy(&v, p, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpy(p, &zero, 4, cudaMemcpyHostToDevice);
  return (int)v;
}

}  // extern "C"
