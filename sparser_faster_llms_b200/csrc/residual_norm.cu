// Residual add + RMSNorm in one pass over a few token rows: the two element-wise steps that sit
// between the attention block and the sparse FFN of a decoder layer (and between the FFN and
// the next layer's attention).  For decode-sized calls each of them is a launch of its own in
// eager torch; here one CTA per token row does both.
//   x_out[r, :] = x[r, :] + delta[r, :]                      (bf16, delta may be NULL)
//   h_out[r, :] = x_out[r, :] * rsqrt(mean(x_out[r, :]^2) + eps) * weight[:]
// The sum of squares and the normalisation run in fp32 on the bf16-rounded x_out, which is what
// a separate add followed by an fp32 RMSNorm computes (the function of LlamaRMSNorm around the
// reference's MLP swap point, custom_models/sparse_models.py:552-614).
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kNormThreads = 256;

__global__ void __launch_bounds__(kNormThreads)
residual_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                        const __nv_bfloat16* __restrict__ weight, float eps,
                        __nv_bfloat16* x_out, __nv_bfloat16* __restrict__ h_out, int D) {
  __shared__ float warp_sum[kNormThreads / 32];
  __shared__ float scale_s;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t base = (size_t)row * D;
  const int nvec = D / 8;  // 16-byte vectors per row; at most 4 per thread (D <= 8192)
  uint4 v[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int vi = tid + i * kNormThreads;
    if (vi < nvec) {
      uint4 a = *reinterpret_cast<const uint4*>(x + base + (size_t)vi * 8);
      if (delta != nullptr) {
        const uint4 b = *reinterpret_cast<const uint4*>(delta + base + (size_t)vi * 8);
        __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&a);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float2 af = __bfloat1622float2(a2[p]), bf = __bfloat1622float2(b2[p]);
          a2[p] = __floats2bfloat162_rn(af.x + bf.x, af.y + bf.y);
        }
        if (x_out != nullptr) *reinterpret_cast<uint4*>(x_out + base + (size_t)vi * 8) = a;
      } else if (x_out != nullptr && x_out != x) {
        *reinterpret_cast<uint4*>(x_out + base + (size_t)vi * 8) = a;
      }
      v[i] = a;
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 f = __bfloat1622float2(a2[p]);
        ss = __fmaf_rn(f.x, f.x, ss);
        ss = __fmaf_rn(f.y, f.y, ss);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) warp_sum[warp] = ss;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) t += warp_sum[w];
    scale_s = rsqrtf(t / (float)D + eps);
  }
  __syncthreads();
  const float scale = scale_s;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int vi = tid + i * kNormThreads;
    if (vi < nvec) {
      const uint4 wv = *reinterpret_cast<const uint4*>(weight + (size_t)vi * 8);
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 f = __bfloat1622float2(a2[p]), wf = __bfloat1622float2(w2[p]);
        // normalised value rounded to bf16, then the weight product (the order of a bf16
        // RMSNorm module: cast back, then scale)
        const __nv_bfloat162 n = __floats2bfloat162_rn(f.x * scale, f.y * scale);
        const float2 nf = __bfloat1622float2(n);
        o2[p] = __floats2bfloat162_rn(nf.x * wf.x, nf.y * wf.y);
      }
      *reinterpret_cast<uint4*>(h_out + base + (size_t)vi * 8) = o;
    }
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_residual_rmsnorm(const void* x, const void* delta, const void* weight,
                                     float eps, void* x_out, void* h_out, int64_t M, int64_t D,
                                     void* stream) {
  const char* fn = "b200_residual_rmsnorm";
  if (M < 0 || M > (int64_t)1 << 30) return fail(B200_EINVAL, "%s: bad M", fn);
  if (D < 8 || D > 8192 || D % 8)
    return fail(B200_EUNSUPPORTED, "%s: D must be a multiple of 8 in [8, 8192] (got %lld)", fn,
                (long long)D);
  if (!(eps >= 0.f)) return fail(B200_EINVAL, "%s: eps must be >= 0", fn);
  if (M == 0) return B200_OK;
  if (x == nullptr || weight == nullptr || h_out == nullptr)
    return fail(B200_ENULL, "%s: x, weight and h_out are required", fn);
  const void* ptrs[5] = {x, delta, weight, x_out, h_out};
  for (const void* p : ptrs)
    if (p != nullptr && !aligned16(p)) return fail(B200_EALIGN, "%s: a pointer is not 16-byte aligned", fn);
  if (h_out == x || h_out == x_out || (delta != nullptr && h_out == delta))
    return fail(B200_EINVAL, "%s: h_out must not alias x, delta or x_out", fn);
  residual_rmsnorm_kernel<<<(unsigned)M, kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta),
      static_cast<const __nv_bfloat16*>(weight), eps, static_cast<__nv_bfloat16*>(x_out),
      static_cast<__nv_bfloat16*>(h_out), (int)D);
  return check_launch(fn);
}
