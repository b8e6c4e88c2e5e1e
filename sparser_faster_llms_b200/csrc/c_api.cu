// extern "C" surface of the library: argument validation and dispatch.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

// Built-in default of the programmatic-dependent-launch switch (B200_PDL overrides it).
#ifndef B200_PDL_DEFAULT
#define B200_PDL_DEFAULT 3
#endif

namespace b200 {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int twell_pack_small(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                     int64_t D, int64_t H, int cf, cudaStream_t stream);
int twell_pack_tc(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                  int64_t D, int64_t H, int cf, cudaStream_t stream);
int twell_pack_tc_splitk(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                         int64_t D, int64_t H, int cf, cudaStream_t stream);
int twell_pack_tc_pair(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                       int64_t D, int64_t H, int cf, cudaStream_t stream);
int twell_pack_tc_splitk8(const void* x, const void* w, const float* bias, void* packed,
                          int64_t M, int64_t D, int64_t H, int cf, cudaStream_t stream);
int twell_pack_tc_splitk_mid(const void* x, const void* w, const float* bias, void* packed,
                             int64_t M, int64_t D, int64_t H, int cf, int split,
                             cudaStream_t stream);
int twell_pack_mid_split(int64_t M, int64_t H, int sm_count);
int twell_pack_tc_wide(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                       int64_t D, int64_t H, int cf, cudaStream_t stream);
int twell_pack_tc_status();
int twell_t2d_launch(bool gated, bool hp, const void* x, const void* packed, const void* up,
                     const void* down, void* out, int64_t M, int64_t D, int64_t H, int cf,
                     void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream,
                     const unsigned char* skip_rows = nullptr, const FusedAr* fused_ar = nullptr);

size_t twell_decode_workspace_bytes(int64_t M, int64_t D, int64_t H);
int twell_decode_launch(bool gated, bool hp, const void* x, const void* gate, const float* bias,
                        const void* up, const void* down, void* packed, void* out, int64_t M,
                        int64_t D, int64_t H, int cf, void* workspace, size_t workspace_bytes,
                        const void* pf_ptr, int64_t pf_bytes, cudaStream_t stream,
                        bool probe_only);
bool twell_decode_small_serves(int64_t M, int64_t D, int64_t H);
size_t twell_decode_small_workspace_bytes(int64_t M, int64_t D, int64_t H);
int twell_decode_small_launch(bool gated, bool hp, const void* x, const void* w,
                              const float* bias, const void* up, const void* down, void* packed,
                              void* out, int64_t M, int64_t D, int64_t H, int cf, void* workspace,
                              size_t workspace_bytes, cudaStream_t stream);
int l2_prefetch_launch(const void* p, int64_t bytes, cudaStream_t stream);
bool twell_gemv_serves(int64_t M, int64_t D, int64_t H);
size_t twell_gemv_workspace_bytes(int64_t D, int64_t H);
int twell_gemv_pack(const void* x, const void* w, const float* bias, void* packed, int64_t D,
                    int64_t H, int cf, cudaStream_t stream);
int twell_gemv_layer(bool gated, bool hp, const void* x, const void* w, const float* bias,
                     const void* up, const void* down, void* packed, void* out, int64_t D,
                     int64_t H, int cf, void* workspace, size_t workspace_bytes,
                     cudaStream_t stream);
int twell_decode_status();
#ifdef B200_TRACE
void twell_decode_trace(unsigned long long* out16);
#endif

// Which calls b200_twell_gated_mlp / b200_twell_mlp hand to a one-kernel decode form when the
// caller's workspace is large enough (environment variable B200_DECODE_FUSED):
//   0  none (always pack + contraction),
//   2  the mma.sync form for up to 16 tokens only,
//   1  every call a one-kernel form serves (the tcgen05 form for 17..32 tokens as well).
// Measured on B200 (D 2048, H 8192, 28 layers under graph replay) the tcgen05 form takes
// 44 us per layer at 32 tokens against 25 us for pack + contraction - its serial phases
// (split-k exchange, finalise, lists, row staging, cross-tile barrier, sum) each cost 0.3-4 us of
// latency on one resident CTA per SM, more than the launch and slab round trip they save - so
// it is never the default.
#ifndef B200_DECODE_FUSED_DEFAULT
#define B200_DECODE_FUSED_DEFAULT 0
#endif
int decode_fused_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("B200_DECODE_FUSED");
    const int v = e != nullptr ? atoi(e) : B200_DECODE_FUSED_DEFAULT;
    mode = (v == 1 || v == 2) ? v : 0;
  }
  return mode;
}

// One-token calls (environment variable B200_ONE_TOKEN): 0 the few-token kernels as for any
// other small batch, 1 the GEMV pack kernel, 2 (default) also the whole layer in that kernel when
// b200_twell_gated_mlp / b200_twell_mlp get a workspace that holds its partial rows.
#ifndef B200_ONE_TOKEN_DEFAULT
#define B200_ONE_TOKEN_DEFAULT 2
#endif
int one_token_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("B200_ONE_TOKEN");
    const int v = e != nullptr ? atoi(e) : B200_ONE_TOKEN_DEFAULT;
    mode = (v >= 0 && v <= 2) ? v : B200_ONE_TOKEN_DEFAULT;
  }
  return mode;
}

int pdl_mask() {
  static int mask = -1;
  if (mask < 0) {
    const char* e = getenv("B200_PDL");
    int v = (e != nullptr) ? atoi(e) : B200_PDL_DEFAULT;
    if (v == 1) v = 3;
    mask = v & 3;
  }
  return mask;
}

bool pdl_enabled() { return pdl_mask() != 0; }

// Number of SMs of the current device (cached per device ordinal).
int sm_count() {
  static int cache[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cache[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cache[dev] = n;
  }
  return cache[dev];
}

namespace {
int check_ptr(const char* fn, const char* name, const void* p) {
  if (p == nullptr) return fail(B200_ENULL, "%s: %s is NULL", fn, name);
  if (!aligned16(p)) return fail(B200_EALIGN, "%s: %s is not 16-byte aligned", fn, name);
  return B200_OK;
}
int check_workspace(const char* fn, const void* ws) {
  if (ws != nullptr && !aligned16(ws))
    return fail(B200_EALIGN, "%s: workspace is not 16-byte aligned", fn);
  return B200_OK;
}
}  // namespace

}  // namespace b200

using namespace b200;

#define B200_TRY(expr)        \
  do {                        \
    int rc__ = (expr);        \
    if (rc__ != B200_OK) return rc__; \
  } while (0)

extern "C" {

int b200_version(void) { return 100; }

int b200_built_for_sm(void) { return 100; }

const char* b200_last_error(void) { return last_error_buffer(); }

size_t b200_workspace_bytes(void) { return (size_t)1 << 20; }

int b200_twell_pack_select(const void* x, const void* w, const float* bias, void* packed,
                           int64_t M, int64_t D, int64_t H, int cf, int kernel, void* stream) {
  const char* fn = "b200_twell_pack";
  B200_TRY(check_dims(fn, M, D, H, cf));
  if (kernel < 0 || kernel > 9) return fail(B200_EINVAL, "%s: kernel must be 0..9", fn);
  if (M == 0) return B200_OK;
  B200_TRY(check_ptr(fn, "x", x));
  B200_TRY(check_ptr(fn, "w", w));
  B200_TRY(check_ptr(fn, "packed", packed));
  if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 3u))
    return fail(B200_EALIGN, "%s: bias is not 4-byte aligned", fn);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Up to one 32-token tile the weight stream is read once and the split-k kernels are
  // HBM-bound; 33..256 tokens take 128-token tiles, still split over a cluster while that grid
  // is one wave; beyond that the tcgen05 tile kernel reuses each weight tile for 256 tokens.
  // Measured on B200 (D 2048, H 8192): up to 16 tokens the mma.sync cluster kernel is
  // fastest (9.6-9.9 us vs 11.7-12.4); at 17..32 tokens its mma work per CTA grows and the
  // tcgen05 split-k kernel wins (12.5 vs 13.9 us).
  // A d_ff shard of at most 8 tiles (2048 neurons) fills too few SMs with a 4-way split:
  // the 8-way split takes 8.5 us against 11.0 us there, but loses from 16 tiles on
  // (15.9 against 11.2 us at 4096 neurons), where its 8-CTA clusters no longer fit one wave.
  // One token: a warp reduces a whole weight row by itself (no split-k exchange).
  if (kernel == 6 || (kernel == 0 && one_token_mode() >= 1 && twell_gemv_serves(M, D, H))) {
    if (M != 1) return fail(B200_EUNSUPPORTED, "%s: kernel 6 serves one token", fn);
    return twell_gemv_pack(x, w, bias, packed, D, H, cf, st);
  }
  if (kernel == 0 && M > 16 && M <= 32 && H <= 8 * kTileN && D % 512 == 0)
    return twell_pack_tc_splitk8(x, w, bias, packed, M, D, H, cf, st);
  if (kernel == 3 || (kernel == 0 && M > 16 && M <= 32))
    return twell_pack_tc_splitk(x, w, bias, packed, M, D, H, cf, st);
  if (kernel == 4) return twell_pack_tc_pair(x, w, bias, packed, M, D, H, cf, st);
  if (kernel == 5) return twell_pack_tc_splitk8(x, w, bias, packed, M, D, H, cf, st);
  if (kernel == 7) return twell_pack_tc_wide(x, w, bias, packed, M, D, H, cf, st);
  if (kernel == 8) return twell_pack_tc_splitk_mid(x, w, bias, packed, M, D, H, cf, 4, st);
  if (kernel == 9) return twell_pack_tc_splitk_mid(x, w, bias, packed, M, D, H, cf, 2, st);
  // 33..256 tokens: 128-token tiles with d_model split over a cluster while that grid is one wave.
  if (kernel == 0 && M > 32 && M <= 256) {
    const int split = twell_pack_mid_split(M, H, sm_count());
    if (split != 0) return twell_pack_tc_splitk_mid(x, w, bias, packed, M, D, H, cf, split, st);
  }
  const bool use_tc = kernel == 2 || (kernel == 0 && M > 32);
  return use_tc ? twell_pack_tc(x, w, bias, packed, M, D, H, cf, st)
                : twell_pack_small(x, w, bias, packed, M, D, H, cf, st);
}

int b200_twell_pack(const void* x, const void* w, const float* bias, void* packed, int64_t M,
                    int64_t D, int64_t H, int cf, void* stream) {
  return b200_twell_pack_select(x, w, bias, packed, M, D, H, cf, 0, stream);
}

int b200_twell_pack_tc_status(void) { return twell_pack_tc_status(); }

int b200_twell_gated_t2d(const void* x, const void* packed, const void* up, const void* down,
                         void* out, int64_t M, int64_t D, int64_t H, int cf, uint32_t flags,
                         void* workspace, size_t workspace_bytes, void* stream) {
  const char* fn = "b200_twell_gated_t2d";
  B200_TRY(check_dims(fn, M, D, H, cf));
  if (flags & ~B200_FLAG_HIGH_PRECISION) return fail(B200_EINVAL, "%s: unknown flags 0x%x", fn, flags);
  if (M == 0) return B200_OK;
  B200_TRY(check_ptr(fn, "x", x));
  B200_TRY(check_ptr(fn, "packed", packed));
  B200_TRY(check_ptr(fn, "up", up));
  B200_TRY(check_ptr(fn, "down", down));
  B200_TRY(check_ptr(fn, "out", out));
  B200_TRY(check_workspace(fn, workspace));
  return twell_t2d_launch(true, (flags & B200_FLAG_HIGH_PRECISION) != 0, x, packed, up, down, out,
                          M, D, H, cf, workspace, workspace_bytes, sm_count(),
                          static_cast<cudaStream_t>(stream));
}

int b200_twell_t2d(const void* packed, const void* down, void* out, int64_t M, int64_t D,
                   int64_t H, int cf, int num_splits, void* workspace, size_t workspace_bytes,
                   void* stream) {
  const char* fn = "b200_twell_t2d";
  B200_TRY(check_dims(fn, M, D, H, cf));
  if (num_splits != 1 && num_splits != 2 && num_splits != 4 && num_splits != 8)
    return fail(B200_EINVAL, "%s: unsupported num_splits=%d (supported: 1/2/4/8)", fn, num_splits);
  if (M == 0) return B200_OK;
  B200_TRY(check_ptr(fn, "packed", packed));
  B200_TRY(check_ptr(fn, "down", down));
  B200_TRY(check_ptr(fn, "out", out));
  B200_TRY(check_workspace(fn, workspace));
  return twell_t2d_launch(false, false, nullptr, packed, nullptr, down, out, M, D, H, cf,
                          workspace, workspace_bytes, sm_count(),
                          static_cast<cudaStream_t>(stream));
}

int b200_hybrid_spmm(const void* vals_slab, const void* b_rows, void* out, int64_t M, int64_t D,
                     int64_t H, int cf, void* workspace, size_t workspace_bytes, void* stream) {
  const char* fn = "b200_hybrid_spmm";
  B200_TRY(check_dims(fn, M, D, H, cf));
  if (M == 0) return B200_OK;
  B200_TRY(check_ptr(fn, "vals_slab", vals_slab));
  B200_TRY(check_ptr(fn, "b_rows", b_rows));
  B200_TRY(check_ptr(fn, "out", out));
  B200_TRY(check_workspace(fn, workspace));
  return twell_t2d_launch(false, true, nullptr, vals_slab, nullptr, b_rows, out, M, D, H, cf,
                          workspace, workspace_bytes, sm_count(),
                          static_cast<cudaStream_t>(stream));
}

size_t b200_twell_decode_workspace_bytes(int64_t M, int64_t D, int64_t H) {
  if (M < 0 || D <= 0 || H <= 0 || D % 256 || H % 256) return 0;
  if (twell_decode_small_serves(M, D, H)) return twell_decode_small_workspace_bytes(M, D, H);
  return twell_decode_workspace_bytes(M, D, H);
}

namespace {
// The one-kernel decode forms: the mma.sync form for up to 16 tokens (d_model 2048 / 4096), the
// tcgen05 form otherwise.  A prefetch range is only taken by the tcgen05 form.
bool decode_wanted(int64_t M, int64_t D, int64_t H, const void* workspace,
                   size_t workspace_bytes) {
  const int mode = decode_fused_mode();
  if (mode == 0 || workspace == nullptr || M < 1 || M > 32) return false;
  if (D < 256 || D % 256 || H < 256 || H % 256) return false;
  const bool small = twell_decode_small_serves(M, D, H);
  if (mode == 2 && !small) return false;
  const size_t need = small ? twell_decode_small_workspace_bytes(M, D, H)
                            : twell_decode_workspace_bytes(M, D, H);
  return need > 0 && workspace_bytes >= need;
}

bool one_token_wanted(int64_t M, int64_t D, int64_t H, const void* workspace,
                      size_t workspace_bytes) {
  return one_token_mode() == 2 && workspace != nullptr && twell_gemv_serves(M, D, H) &&
         workspace_bytes >= twell_gemv_workspace_bytes(D, H);
}

int decode_dispatch(bool gated, bool hp, const void* x, const void* gate, const float* bias,
                    const void* up, const void* down, void* packed, void* out, int64_t M,
                    int64_t D, int64_t H, int cf, void* workspace, size_t workspace_bytes,
                    const void* pf, int64_t pf_bytes, cudaStream_t stream) {
  if (twell_decode_small_serves(M, D, H))
    return twell_decode_small_launch(gated, hp, x, gate, bias, up, down, packed, out, M, D, H, cf,
                                     workspace, workspace_bytes, stream);
  return twell_decode_launch(gated, hp, x, gate, bias, up, down, packed, out, M, D, H, cf,
                             workspace, workspace_bytes, pf, pf_bytes, stream, false);
}
}  // namespace

int b200_twell_decode_status(void) { return twell_decode_status(); }

#ifdef B200_TRACE
void b200_debug_trace_decode(unsigned long long* out16) { twell_decode_trace(out16); }
#endif

int b200_l2_prefetch(const void* ptr, int64_t bytes, void* stream) {
  const char* fn = "b200_l2_prefetch";
  if (bytes < 0) return fail(B200_EINVAL, "%s: bytes must be >= 0", fn);
  if (bytes == 0) return B200_OK;
  B200_TRY(check_ptr(fn, "ptr", ptr));
  return l2_prefetch_launch(ptr, bytes, static_cast<cudaStream_t>(stream));
}

namespace {
// Argument checks shared by the fused decode entry points.
int check_decode_args(const char* fn, const void* x, const void* gate, const float* gate_bias,
                      const void* up, const void* down, const void* packed, const void* out,
                      int64_t M, int64_t D, int64_t H, int cf, uint32_t flags, const void* ws,
                      bool gated) {
  B200_TRY(check_dims(fn, M, D, H, cf));
  if (flags & ~B200_FLAG_HIGH_PRECISION) return fail(B200_EINVAL, "%s: unknown flags 0x%x", fn, flags);
  if (M == 0) return B200_OK;
  B200_TRY(check_ptr(fn, "x", x));
  B200_TRY(check_ptr(fn, gated ? "gate" : "up", gate));
  if (gated) B200_TRY(check_ptr(fn, "up", up));
  B200_TRY(check_ptr(fn, "down", down));
  B200_TRY(check_ptr(fn, "packed", packed));
  B200_TRY(check_ptr(fn, "out", out));
  B200_TRY(check_workspace(fn, ws));
  if (gate_bias != nullptr && (reinterpret_cast<uintptr_t>(gate_bias) & 3u))
    return fail(B200_EALIGN, "%s: bias is not 4-byte aligned", fn);
  return B200_OK;
}
}  // namespace

int b200_twell_gated_mlp_decode(const void* x, const void* gate, const float* gate_bias,
                                const void* up, const void* down, void* packed, void* out,
                                int64_t M, int64_t D, int64_t H, int cf, uint32_t flags,
                                void* workspace, size_t workspace_bytes, const void* prefetch,
                                int64_t prefetch_bytes, void* stream) {
  const char* fn = "b200_twell_gated_mlp_decode";
  B200_TRY(check_decode_args(fn, x, gate, gate_bias, up, down, packed, out, M, D, H, cf, flags,
                             workspace, true));
  if (M == 0) return B200_OK;
  if (prefetch != nullptr && (!aligned16(prefetch) || prefetch_bytes < 0))
    return fail(B200_EALIGN, "%s: prefetch range must be 16-byte aligned and non-negative", fn);
  return decode_dispatch(true, (flags & B200_FLAG_HIGH_PRECISION) != 0, x, gate, gate_bias, up,
                         down, packed, out, M, D, H, cf, workspace, workspace_bytes, prefetch,
                         prefetch != nullptr ? prefetch_bytes : 0,
                         static_cast<cudaStream_t>(stream));
}

int b200_twell_gated_mlp(const void* x, const void* gate, const float* gate_bias, const void* up,
                         const void* down, void* packed, void* out, int64_t M, int64_t D,
                         int64_t H, int cf, uint32_t flags, void* workspace,
                         size_t workspace_bytes, void* stream) {
  if (decode_wanted(M, D, H, workspace, workspace_bytes)) {
    B200_TRY(check_decode_args("b200_twell_gated_mlp", x, gate, gate_bias, up, down, packed, out,
                               M, D, H, cf, flags, workspace, true));
    const int rc = decode_dispatch(true, (flags & B200_FLAG_HIGH_PRECISION) != 0, x, gate,
                                   gate_bias, up, down, packed, out, M, D, H, cf, workspace,
                                   workspace_bytes, nullptr, 0, static_cast<cudaStream_t>(stream));
    if (rc != B200_EUNSUPPORTED) return rc;  // served (or failed for good)
  }
  if (one_token_wanted(M, D, H, workspace, workspace_bytes)) {
    B200_TRY(check_decode_args("b200_twell_gated_mlp", x, gate, gate_bias, up, down, packed, out,
                               M, D, H, cf, flags, workspace, true));
    const int rc = twell_gemv_layer(true, (flags & B200_FLAG_HIGH_PRECISION) != 0, x, gate,
                                    gate_bias, up, down, packed, out, D, H, cf, workspace,
                                    workspace_bytes, static_cast<cudaStream_t>(stream));
    if (rc != B200_EUNSUPPORTED) return rc;  // served (or failed for good)
  }
  B200_TRY(b200_twell_pack(x, gate, gate_bias, packed, M, D, H, cf, stream));
  return b200_twell_gated_t2d(x, packed, up, down, out, M, D, H, cf, flags, workspace,
                              workspace_bytes, stream);
}

size_t b200_fused_allreduce_block_bytes(int64_t max_tokens, int64_t D) {
  if (max_tokens <= 0 || D <= 0) return 0;
  const size_t slot = ((size_t)max_tokens * (size_t)D * 4 + 255) & ~(size_t)255;
  return kFarControlBytes + 2 * 8 * slot;
}

int b200_twell_gated_t2d_allreduce(const void* x, const void* packed, const void* up,
                                   const void* down, void* out, int64_t M, int64_t D, int64_t H,
                                   int cf, uint32_t flags, void* workspace, size_t workspace_bytes,
                                   void* const* peer_blocks, int rank, int world,
                                   int64_t block_bytes, void* stream) {
  const char* fn = "b200_twell_gated_t2d_allreduce";
  B200_TRY(check_dims(fn, M, D, H, cf));
  if (flags & ~B200_FLAG_HIGH_PRECISION) return fail(B200_EINVAL, "%s: unknown flags 0x%x", fn, flags);
  if (world < 1 || world > 8 || rank < 0 || rank >= world)
    return fail(B200_EINVAL, "%s: need 1 <= world <= 8 and 0 <= rank < world", fn);
  if (M == 0) return B200_OK;
  B200_TRY(check_ptr(fn, "x", x));
  B200_TRY(check_ptr(fn, "packed", packed));
  B200_TRY(check_ptr(fn, "up", up));
  B200_TRY(check_ptr(fn, "down", down));
  B200_TRY(check_ptr(fn, "out", out));
  B200_TRY(check_workspace(fn, workspace));
  FusedAr ar = {};
  ar.rank = rank;
  ar.world = world;
  if (world > 1) {
    if (peer_blocks == nullptr) return fail(B200_ENULL, "%s: peer_blocks is NULL", fn);
    if (block_bytes <= (int64_t)kFarControlBytes)
      return fail(B200_EWORKSPACE, "%s: block_bytes too small", fn);
    ar.slot_bytes = ((block_bytes - (int64_t)kFarControlBytes) / 16) & ~(int64_t)255;
    for (int r = 0; r < world; ++r) {
      B200_TRY(check_ptr(fn, "peer block", peer_blocks[r]));
      ar.block[r] = static_cast<unsigned char*>(peer_blocks[r]);
    }
  }
  return twell_t2d_launch(true, (flags & B200_FLAG_HIGH_PRECISION) != 0, x, packed, up, down, out,
                          M, D, H, cf, workspace, workspace_bytes, sm_count(),
                          static_cast<cudaStream_t>(stream), nullptr, &ar);
}

int b200_twell_gated_mlp_allreduce(const void* x, const void* gate, const float* gate_bias,
                                   const void* up, const void* down, void* packed, void* out,
                                   int64_t M, int64_t D, int64_t H, int cf, uint32_t flags,
                                   void* workspace, size_t workspace_bytes,
                                   void* const* peer_blocks, int rank, int world,
                                   int64_t block_bytes, void* stream) {
  B200_TRY(b200_twell_pack(x, gate, gate_bias, packed, M, D, H, cf, stream));
  return b200_twell_gated_t2d_allreduce(x, packed, up, down, out, M, D, H, cf, flags, workspace,
                                        workspace_bytes, peer_blocks, rank, world, block_bytes,
                                        stream);
}

/* Reads and clears the error word of this rank's fused all-reduce block (0 = no wait ever
 * gave up, else 0x100 + the peer that did not arrive).  Synchronises the device. */
int b200_fused_allreduce_status(void* my_block) {
  if (my_block == nullptr) return -1;
  uint32_t v = 0, zero = 0;
  uint32_t* p = static_cast<uint32_t*>(my_block) + kFarErrorWord;
  if (cudaMemcpy(&v, p, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpy(p, &zero, 4, cudaMemcpyHostToDevice);
  return (int)v;
}

int b200_twell_mlp(const void* x, const void* up, const void* down, void* packed, void* out,
                   int64_t M, int64_t D, int64_t H, int cf, int num_splits, void* workspace,
                   size_t workspace_bytes, void* stream) {
  if ((num_splits == 1 || num_splits == 2 || num_splits == 4 || num_splits == 8) &&
      decode_wanted(M, D, H, workspace, workspace_bytes)) {
    B200_TRY(check_decode_args("b200_twell_mlp", x, up, nullptr, nullptr, down, packed, out, M, D,
                               H, cf, 0, workspace, false));
    const int rc = decode_dispatch(false, false, x, up, nullptr, nullptr, down, packed, out, M, D,
                                   H, cf, workspace, workspace_bytes, nullptr, 0,
                                   static_cast<cudaStream_t>(stream));
    if (rc != B200_EUNSUPPORTED) return rc;
  }
  if ((num_splits == 1 || num_splits == 2 || num_splits == 4 || num_splits == 8) &&
      one_token_wanted(M, D, H, workspace, workspace_bytes)) {
    B200_TRY(check_decode_args("b200_twell_mlp", x, up, nullptr, nullptr, down, packed, out, M, D,
                               H, cf, 0, workspace, false));
    const int rc = twell_gemv_layer(false, false, x, up, nullptr, nullptr, down, packed, out, D,
                                    H, cf, workspace, workspace_bytes,
                                    static_cast<cudaStream_t>(stream));
    if (rc != B200_EUNSUPPORTED) return rc;
  }
  B200_TRY(b200_twell_pack(x, up, nullptr, packed, M, D, H, cf, stream));
  return b200_twell_t2d(packed, down, out, M, D, H, cf, num_splits, workspace, workspace_bytes,
                        stream);
}

}  // extern "C"
