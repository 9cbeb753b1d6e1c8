// Shared helpers for the eps_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/eps_b200.h"

namespace epsb {

// Thread-local text of the last failure; read through epsb_last_error().
char* last_error_buffer();
int fail(int code, const char* fmt, ...);

#define EPSB_REQUIRE(cond, code, ...) \
  do {                                \
    if (!(cond)) return ::epsb::fail((code), __VA_ARGS__); \
  } while (0)

// Checks the launch that was just made on `stream` (launch-time errors only; no sync).
inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return EPSB_OK;
}

// CTAs a persistent GEMM launch may use: every SM, or the caller's sm_count when that is in (0, all).
int gemm_cta_limit(int sm_count_arg);

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

constexpr float kFp8Max = 448.0f;
constexpr int kZcMark = 1000000;  // fast_ep marker for zero-computation slots (fast_ep_kernels.cu:16)

struct alignas(16) Vec16 {
  uint4 v;
};

__device__ __forceinline__ uint4 ld_nc_16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ void st_16(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Two floats -> two e4m3 codes (round to nearest even, saturate to +-448); lo in bits 0..7.
__device__ __forceinline__ uint16_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// The quantisation step shared by every producer of FP8 rows: clamp(x*inv, +-448) -> code.
// fminf/fmaxf drop a NaN operand (0*inf for an all-zero group), as the reference relies on.
__device__ __forceinline__ float quant_clamp(float x, float inv) { return fmaxf(-kFp8Max, fminf(x * inv, kFp8Max)); }

template <bool kDivFull>
__device__ __forceinline__ float scale_of_amax(float amax) {
  if constexpr (kDivFull) {
    float s;
    asm("div.full.f32 %0, %1, %2;" : "=f"(s) : "f"(amax), "f"(kFp8Max));
    return s;
  } else {
    return __fdiv_rn(amax, kFp8Max);
  }
}

}  // namespace epsb
