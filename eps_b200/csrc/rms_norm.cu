// RMS normalisation of bf16 rows: out = (x * rsqrt(mean(x^2) + eps)) * scale, fp32 arithmetic.
//
// The reference's rms_norm (src/utils/rms_norm.cu:103-140; torch op utils.rms_norm_op,
// src/utils/bindings/th_rms_norm.cu:13-35) reads every row twice.  Here one CTA of 256 threads keeps its row in
// registers (16-byte loads, up to 16384 columns), so the row crosses HBM once each way; longer rows take the
// two-pass kernel.  The operation order per element is the reference's ((x * inv_rms) * scale, one rounding to bf16);
// the sum of squares is accumulated in another order, so inv_rms can differ in the last place.
#include "common.cuh"

namespace epsb {

namespace {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = lane < kNormThreads / 32 ? smem[lane] : 0.0f;
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
  return __shfl_sync(0xffffffffu, t, 0);
}

__device__ __forceinline__ float inv_rms(float sum_sq, int n, float eps) {
  // the reference's expression, on its half-width column count (rms_norm.cu:118-121)
  return rsqrtf(0.5f * sum_sq / (float)(n / 2) + eps);
}

// n % 8 == 0, n <= kNormThreads * 8 * kChunks: thread t holds the 16-byte chunks t, t + 256, ...
template <int kChunks>
__global__ void __launch_bounds__(kNormThreads)
rms_norm_rows_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ in,
                     const __nv_bfloat16* __restrict__ scale, float eps, int n) {
  __shared__ float red[kNormThreads / 32];
  const int64_t row = blockIdx.x;
  const int chunks = n / 8;
  const uint4* src = reinterpret_cast<const uint4*>(in + row * n);
  uint4 v[kChunks];
  float acc = 0.0f;
#pragma unroll
  for (int c = 0; c < kChunks; c++) {
    const int i = threadIdx.x + c * kNormThreads;
    v[c] = i < chunks ? ld_nc_16(src + i) : make_uint4(0, 0, 0, 0);
    const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float a = bf16_lo(w[j]), b = bf16_hi(w[j]);
      acc += a * a;
      acc += b * b;
    }
  }
  const float inv = inv_rms(block_sum(acc, red), n, eps);
  const uint4* sc = reinterpret_cast<const uint4*>(scale);
  uint4* dst = reinterpret_cast<uint4*>(out + row * n);
#pragma unroll
  for (int c = 0; c < kChunks; c++) {
    const int i = threadIdx.x + c * kNormThreads;
    if (i < chunks) {
      const uint4 s = __ldg(sc + i);
      const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
      const uint32_t q[4] = {s.x, s.y, s.z, s.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; j++)
        o[j] = pack_bf16x2(bf16_lo(w[j]) * inv * bf16_lo(q[j]), bf16_hi(w[j]) * inv * bf16_hi(q[j]));
      st_16(dst + i, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

// any even n: two passes over the row, two columns at a time
__global__ void __launch_bounds__(kNormThreads)
rms_norm_two_pass_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ in,
                         const __nv_bfloat16* __restrict__ scale, float eps, int n) {
  __shared__ float red[kNormThreads / 32];
  const int64_t row = blockIdx.x;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(in + row * n);
  float acc = 0.0f;
  for (int i = threadIdx.x; i < n / 2; i += kNormThreads) {
    const uint32_t w = src[i];
    acc += bf16_lo(w) * bf16_lo(w);
    acc += bf16_hi(w) * bf16_hi(w);
  }
  const float inv = inv_rms(block_sum(acc, red), n, eps);
  const uint32_t* sc = reinterpret_cast<const uint32_t*>(scale);
  uint32_t* dst = reinterpret_cast<uint32_t*>(out + row * n);
  for (int i = threadIdx.x; i < n / 2; i += kNormThreads) {
    const uint32_t w = src[i], q = sc[i];
    dst[i] = pack_bf16x2(bf16_lo(w) * inv * bf16_lo(q), bf16_hi(w) * inv * bf16_hi(q));
  }
}

}  // namespace

}  // namespace epsb

using namespace epsb;

extern "C" int epsb_rms_norm(void* out, const void* input, const void* scale, float eps, int64_t m, int64_t n,
                             void* stream) {
  EPSB_REQUIRE(m >= 0 && n > 0, EPSB_ERR_INVALID, "bad sizes m=%lld n=%lld", (long long)m, (long long)n);
  EPSB_REQUIRE(n % 2 == 0, EPSB_ERR_INVALID, "dim %lld is not divisible by 2.", (long long)n);
  EPSB_REQUIRE(m < (1ll << 31) && n < (1ll << 31), EPSB_ERR_INVALID, "tensor too large");
  if (m == 0) return EPSB_OK;
  auto st = static_cast<cudaStream_t>(stream);
  auto* o = static_cast<__nv_bfloat16*>(out);
  auto* x = static_cast<const __nv_bfloat16*>(input);
  auto* s = static_cast<const __nv_bfloat16*>(scale);
  const bool vec = n % 8 == 0 && (((uintptr_t)out | (uintptr_t)input | (uintptr_t)scale) & 15) == 0;
  const int64_t chunks = n / 8;
  if (vec && chunks <= kNormThreads * 1)
    rms_norm_rows_kernel<1><<<(int)m, kNormThreads, 0, st>>>(o, x, s, eps, (int)n);
  else if (vec && chunks <= kNormThreads * 2)
    rms_norm_rows_kernel<2><<<(int)m, kNormThreads, 0, st>>>(o, x, s, eps, (int)n);
  else if (vec && chunks <= kNormThreads * 4)
    rms_norm_rows_kernel<4><<<(int)m, kNormThreads, 0, st>>>(o, x, s, eps, (int)n);
  else if (vec && chunks <= kNormThreads * 8)
    rms_norm_rows_kernel<8><<<(int)m, kNormThreads, 0, st>>>(o, x, s, eps, (int)n);
  else
    rms_norm_two_pass_kernel<<<(int)m, kNormThreads, 0, st>>>(o, x, s, eps, (int)n);
  return check_launch("rms_norm");
}
