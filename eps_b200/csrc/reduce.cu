// Weighted row reductions of the combine path and the unfused SwiGLU (sm_100a).
//
// A warp owns an output row; each lane walks the row in 16-byte vectors (8 bf16)
// and issues the loads of all summands of a vector before accumulating, so k
// (or W) independent 16-byte loads per lane are in flight.  Two arithmetic
// families are provided: "_ref" reproduces the reference kernels' bf16
// multiply/accumulate order; the others accumulate in fp32 and round once.
#include "common.cuh"

namespace epsb {

namespace {

constexpr int kRedThreads = 256;
constexpr int kRedWarps = kRedThreads / 32;
constexpr int kMaxSlots = 16;  // largest top-k / world size a register-resident kernel takes
// Kernels are instantiated for 4, 8, 12 and 16 summands: fewer registers -> more resident warps -> more loads in flight.

union BfVec {
  uint4 u;
  __nv_bfloat162 h[4];
};

__device__ __forceinline__ void acc_f32(float (&a)[8], uint4 v) {
  a[0] += bf16_lo(v.x); a[1] += bf16_hi(v.x);
  a[2] += bf16_lo(v.y); a[3] += bf16_hi(v.y);
  a[4] += bf16_lo(v.z); a[5] += bf16_hi(v.z);
  a[6] += bf16_lo(v.w); a[7] += bf16_hi(v.w);
}

__device__ __forceinline__ void fma_f32(float (&a)[8], uint4 v, float w) {
  a[0] = fmaf(bf16_lo(v.x), w, a[0]); a[1] = fmaf(bf16_hi(v.x), w, a[1]);
  a[2] = fmaf(bf16_lo(v.y), w, a[2]); a[3] = fmaf(bf16_hi(v.y), w, a[3]);
  a[4] = fmaf(bf16_lo(v.z), w, a[4]); a[5] = fmaf(bf16_hi(v.z), w, a[5]);
  a[6] = fmaf(bf16_lo(v.w), w, a[6]); a[7] = fmaf(bf16_hi(v.w), w, a[7]);
}

__device__ __forceinline__ uint4 pack8(const float (&a)[8]) {
  uint4 o;
  o.x = pack_bf16x2(a[0], a[1]);
  o.y = pack_bf16x2(a[2], a[3]);
  o.z = pack_bf16x2(a[4], a[5]);
  o.w = pack_bf16x2(a[6], a[7]);
  return o;
}

// Maps the warp's running row counter onto the stage windows of every source
// rank: window d is [incl[d*S+stage-1] (0 for the very first), incl[d*S+stage]).
// stage < 0 selects the single window [0, incl[W*S-1]).
struct StageWindows {
  const int32_t* incl;
  int W, S, stage;
  __device__ int count() const { return stage < 0 ? 1 : W; }
  __device__ void window(int d, int64_t& b, int64_t& e) const {
    if (stage < 0) {
      b = 0;
      e = incl[W * S - 1];
    } else {
      const int i = d * S + stage;
      b = i == 0 ? 0 : incl[i - 1];
      e = incl[i];
    }
  }
};

// ---------------------------------------------------------------- local reduce (expert rank)

template <bool kRefArith, int kSlots>
__global__ void __launch_bounds__(kRedThreads)
local_reduce_kernel(const uint8_t* __restrict__ y, const float* __restrict__ w_recv,
                    const int32_t* __restrict__ scale_map, const int32_t* __restrict__ red_map, StageWindows win,
                    int k, int64_t H, uint8_t* __restrict__ send) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kRedWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kRedWarps;
  const int vecs = (int)(H >> 3);
  const int64_t row_bytes = H * 2;
  const int64_t sentinel = (int64_t)win.incl[win.W * win.S - 1] * k;
  int64_t seen = 0;
  for (int d = 0; d < win.count(); d++) {
    int64_t b, e;
    win.window(d, b, e);
    const int64_t first = (warp - seen % n_warps + n_warps) % n_warps;
    for (int64_t q = b + first; q < e; q += n_warps) {
      int32_t rows[kSlots];
      float wts[kSlots];
#pragma unroll
      for (int j = 0; j < kSlots; j++) {
        rows[j] = -1;
        wts[j] = 0.0f;
        if (j < k) {
          const int32_t r = __ldg(red_map + q * k + j);
          if (r < sentinel) {
            rows[j] = r;
            if constexpr (kRefArith) wts[j] = __ldg(w_recv + (int64_t)__ldg(scale_map + q) * k + j);
          }
        }
      }
      for (int v = lane; v < vecs; v += 32) {
        uint4 in[kSlots];
#pragma unroll
        for (int j = 0; j < kSlots; j++)
          if (j < k && rows[j] >= 0) in[j] = ld_nc_16(y + (int64_t)rows[j] * row_bytes + (int64_t)v * 16);
        uint4 out;
        if constexpr (kRefArith) {
          // reference: thread_result += (thread_value * scale) with bf16 operators
          // (local_reducer.cu:137, cuda_utils.cuh:123-126,166-213); the fp32 weight is rounded to bf16 first.
          BfVec acc;
          acc.u = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int j = 0; j < kSlots; j++)
            if (j < k && rows[j] >= 0) {
              BfVec t;
              t.u = in[j];
              const __nv_bfloat16 s = __float2bfloat16_rn(wts[j]);
#pragma unroll
              for (int c = 0; c < 4; c++) {
                __nv_bfloat162 prod = __nv_bfloat162{t.h[c].x * s, t.h[c].y * s};
                acc.h[c] += prod;
              }
            }
          out = acc.u;
        } else {
          float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
          for (int j = 0; j < kSlots; j++)
            if (j < k && rows[j] >= 0) acc_f32(a, in[j]);
          out = pack8(a);
        }
        st_16(send + q * row_bytes + (int64_t)v * 16, out);
      }
    }
    seen += e - b;
  }
}

// ---------------------------------------------------------------- world of one: local + global reduce in one pass

// out[t,:] = bf16( sum_j float(y[red_map[q,j],:]) + shared[t,:] + x[t,:] * zero_scale[t] ), q = glob_map[t]
// (the return row of token t; with one rank the return buffer IS the collect buffer).  fp32 accumulation in
// slot order, one rounding.  Replaces local_reduce -> (no-op exchange) -> global_reduce for ep_world_size 1.
template <int kSlots>
__global__ void __launch_bounds__(kRedThreads)
reduce_ep1_kernel(const uint8_t* __restrict__ y, const int32_t* __restrict__ red_map,
                  const int32_t* __restrict__ glob_map, const int32_t* __restrict__ ret_incl, int S,
                  const uint8_t* __restrict__ shared, const uint8_t* __restrict__ x,
                  const float* __restrict__ zero_scale, int T, int k, int64_t H, uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kRedWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kRedWarps;
  const int vecs = (int)(H >> 3);
  const int64_t row_bytes = H * 2;
  const int64_t sentinel = (int64_t)ret_incl[S - 1] * k;
  for (int64_t t = warp; t < T; t += n_warps) {
    const int32_t q = __ldg(glob_map + t);
    int32_t rows[kSlots];
#pragma unroll
    for (int j = 0; j < kSlots; j++) {
      rows[j] = -1;
      if (j < k && q < T) {
        const int32_t r = __ldg(red_map + (int64_t)q * k + j);
        if (r < sentinel) rows[j] = r;
      }
    }
    const float zs = zero_scale != nullptr ? __ldg(zero_scale + t) : 0.0f;
    for (int v = lane; v < vecs; v += 32) {
      const int64_t off = t * row_bytes + (int64_t)v * 16;
      uint4 in[kSlots];
#pragma unroll
      for (int j = 0; j < kSlots; j++)
        if (j < k && rows[j] >= 0) in[j] = ld_nc_16(y + (int64_t)rows[j] * row_bytes + (int64_t)v * 16);
      uint4 sh = make_uint4(0, 0, 0, 0), xin = make_uint4(0, 0, 0, 0);
      if (shared != nullptr) sh = ld_nc_16(shared + off);
      const bool has_zero = zero_scale != nullptr && zs != 0.0f;  // tokens without identity experts skip the x row
      if (has_zero) xin = ld_nc_16(x + off);
      float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int j = 0; j < kSlots; j++)
        if (j < k && rows[j] >= 0) acc_f32(a, in[j]);
      if (shared != nullptr) acc_f32(a, sh);
      if (has_zero) fma_f32(a, xin, zs);
      st_16(out + off, pack8(a));
    }
  }
}

// ---------------------------------------------------------------- global reduce (source rank)

template <bool kRefArith, int kSlots>
__global__ void __launch_bounds__(kRedThreads)
global_reduce_kernel(const uint8_t* __restrict__ recv, const int32_t* __restrict__ glob_map,
                     const uint8_t* __restrict__ shared, const uint8_t* __restrict__ x,
                     const float* __restrict__ zero_scale, int T, int W, int64_t H, uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kRedWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kRedWarps;
  const int vecs = (int)(H >> 3);
  const int64_t row_bytes = H * 2;
  const int32_t sentinel = T * W;
  for (int64_t t = warp; t < T; t += n_warps) {
    int32_t rows[kSlots];
#pragma unroll
    for (int j = 0; j < kSlots; j++) {
      rows[j] = -1;
      if (j < W) {
        const int32_t r = __ldg(glob_map + t * W + j);
        if (r < sentinel) rows[j] = r;
      }
    }
    const float zs = zero_scale != nullptr ? __ldg(zero_scale + t) : 0.0f;
    for (int v = lane; v < vecs; v += 32) {
      const int64_t off = t * row_bytes + (int64_t)v * 16;
      uint4 in[kSlots];
#pragma unroll
      for (int j = 0; j < kSlots; j++)
        if (j < W && rows[j] >= 0) in[j] = ld_nc_16(recv + (int64_t)rows[j] * row_bytes + (int64_t)v * 16);
      uint4 sh = make_uint4(0, 0, 0, 0), xin = make_uint4(0, 0, 0, 0);
      if (shared != nullptr) sh = ld_nc_16(shared + off);
      if (zero_scale != nullptr) xin = ld_nc_16(x + off);
      uint4 o;
      if constexpr (kRefArith) {
        // reference: bf16 adds over ranks, then shared + result (global_reducer.cu:138-180), then
        // out += bf16(float(x) * zero_scale) as a separate pass (zero_reducer.cu:34-42).
        BfVec acc;
        acc.u = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < kSlots; j++)
          if (j < W && rows[j] >= 0) {
            BfVec tv;
            tv.u = in[j];
#pragma unroll
            for (int c = 0; c < 4; c++) acc.h[c] += tv.h[c];
          }
        if (shared != nullptr) {
          BfVec s;
          s.u = sh;
#pragma unroll
          for (int c = 0; c < 4; c++) acc.h[c] = s.h[c] + acc.h[c];
        }
        if (zero_scale != nullptr) {
          BfVec xv;
          xv.u = xin;
#pragma unroll
          for (int c = 0; c < 4; c++) {
            acc.h[c].x += __float2bfloat16_rn(__bfloat162float(xv.h[c].x) * zs);
            acc.h[c].y += __float2bfloat16_rn(__bfloat162float(xv.h[c].y) * zs);
          }
        }
        o = acc.u;
      } else {
        float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < kSlots; j++)
          if (j < W && rows[j] >= 0) acc_f32(a, in[j]);
        if (shared != nullptr) acc_f32(a, sh);
        if (zero_scale != nullptr) fma_f32(a, xin, zs);
        o = pack8(a);
      }
      st_16(out + off, o);
    }
  }
}

// General world size (W > kMaxSlots): same arithmetic, summands streamed one at a time.
template <bool kRefArith>
__global__ void __launch_bounds__(kRedThreads)
global_reduce_wide_kernel(const uint8_t* __restrict__ recv, const int32_t* __restrict__ glob_map,
                          const uint8_t* __restrict__ shared, const uint8_t* __restrict__ x,
                          const float* __restrict__ zero_scale, int T, int W, int64_t H, uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kRedWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kRedWarps;
  const int vecs = (int)(H >> 3);
  const int64_t row_bytes = H * 2;
  const int32_t sentinel = T * W;
  for (int64_t t = warp; t < T; t += n_warps) {
    const float zs = zero_scale != nullptr ? __ldg(zero_scale + t) : 0.0f;
    for (int v = lane; v < vecs; v += 32) {
      const int64_t off = t * row_bytes + (int64_t)v * 16;
      BfVec acc;
      acc.u = make_uint4(0, 0, 0, 0);
      float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = 0; j < W; j++) {
        const int32_t r = __ldg(glob_map + t * W + j);
        if (r >= sentinel) continue;
        BfVec tv;
        tv.u = ld_nc_16(recv + (int64_t)r * row_bytes + (int64_t)v * 16);
        if constexpr (kRefArith) {
#pragma unroll
          for (int c = 0; c < 4; c++) acc.h[c] += tv.h[c];
        } else {
          acc_f32(a, tv.u);
        }
      }
      if (shared != nullptr) {
        BfVec s;
        s.u = ld_nc_16(shared + off);
        if constexpr (kRefArith) {
#pragma unroll
          for (int c = 0; c < 4; c++) acc.h[c] = s.h[c] + acc.h[c];
        } else {
          acc_f32(a, s.u);
        }
      }
      if (zero_scale != nullptr) {
        BfVec xv;
        xv.u = ld_nc_16(x + off);
        if constexpr (kRefArith) {
#pragma unroll
          for (int c = 0; c < 4; c++) {
            acc.h[c].x += __float2bfloat16_rn(__bfloat162float(xv.h[c].x) * zs);
            acc.h[c].y += __float2bfloat16_rn(__bfloat162float(xv.h[c].y) * zs);
          }
        } else {
          fma_f32(a, xv.u, zs);
        }
      }
      st_16(out + off, kRefArith ? acc.u : pack8(a));
    }
  }
}

// ---------------------------------------------------------------- fast_ep combine

template <int kSlots>
__global__ void __launch_bounds__(kRedThreads)
fastep_reduce_kernel(const uint8_t* __restrict__ rows_in, const uint8_t* __restrict__ raw,
                     const uint8_t* __restrict__ shared, const float* __restrict__ w,
                     const int32_t* __restrict__ mapping, int T, int k, int64_t H, uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kRedWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kRedWarps;
  const int vecs = (int)(H >> 3);
  const int64_t row_bytes = H * 2;
  for (int64_t t = warp; t < T; t += n_warps) {
    const uint8_t* srcs[kSlots];
    float wts[kSlots];
#pragma unroll
    for (int j = 0; j < kSlots; j++) {
      srcs[j] = nullptr;
      wts[j] = 0.0f;
      if (j < k) {
        const int32_t m = __ldg(mapping + t * k + j);
        srcs[j] = m >= kZcMark ? raw + (int64_t)(m - kZcMark) * row_bytes : rows_in + (int64_t)m * row_bytes;
        wts[j] = __ldg(w + t * k + j);
      }
    }
    for (int v = lane; v < vecs; v += 32) {
      uint4 in[kSlots];
#pragma unroll
      for (int j = 0; j < kSlots; j++)
        if (j < k) in[j] = ld_nc_16(srcs[j] + (int64_t)v * 16);
      float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int j = 0; j < kSlots; j++)
        if (j < k) fma_f32(a, in[j], wts[j]);
      const int64_t off = t * row_bytes + (int64_t)v * 16;
      if (shared != nullptr) acc_f32(a, ld_nc_16(shared + off));
      st_16(out + off, pack8(a));
    }
  }
}

// ---------------------------------------------------------------- SwiGLU (bf16 in, bf16 out)

__global__ void __launch_bounds__(kRedThreads)
silu_kernel(const uint8_t* __restrict__ gate_up, uint8_t* __restrict__ act, const int32_t* __restrict__ bounds,
            int num_experts, int64_t rows, int64_t I) {
  int64_t begin = 0, end = rows;
  if (bounds != nullptr) {
    begin = bounds[0];
    end = bounds[num_experts];
  }
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kRedWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kRedWarps;
  const int vecs = (int)(I >> 3);
  for (int64_t r = begin + warp; r < end; r += n_warps) {
    const uint8_t* g = gate_up + r * I * 4;
    const uint8_t* u = g + I * 2;
    for (int v = lane; v < vecs; v += 32) {
      const uint4 gv = ld_nc_16(g + (int64_t)v * 16), uv = ld_nc_16(u + (int64_t)v * 16);
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
      uint32_t ow[4];
#pragma unroll
      for (int c = 0; c < 4; c++) {
        // silu(x) = x / (1 + __expf(-x)) in fp32, times up in fp32, one bf16 rounding
        // (reference common/cuda_utils.cuh:71-90, executor/activations.cu:35-36)
        const float g0 = bf16_lo(gw[c]), g1 = bf16_hi(gw[c]);
        const float s0 = g0 / (1.0f + __expf(-g0)), s1 = g1 / (1.0f + __expf(-g1));
        ow[c] = pack_bf16x2(s0 * bf16_lo(uw[c]), s1 * bf16_hi(uw[c]));
      }
      st_16(act + r * I * 2 + (int64_t)v * 16, make_uint4(ow[0], ow[1], ow[2], ow[3]));
    }
  }
}

// Picks the instantiation with the smallest slot capacity >= n.
#define EPSB_SLOT_SWITCH(n, ...)            \
  do {                                      \
    if ((n) <= 4) { constexpr int kS = 4; __VA_ARGS__; }        \
    else if ((n) <= 8) { constexpr int kS = 8; __VA_ARGS__; }   \
    else if ((n) <= 12) { constexpr int kS = 12; __VA_ARGS__; } \
    else { constexpr int kS = 16; __VA_ARGS__; }                \
  } while (0)

int red_grid(int64_t rows) {
  int64_t want = (rows + kRedWarps - 1) / kRedWarps;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return (int)want;
}

int check_h(int64_t H) {
  EPSB_REQUIRE(H > 0 && H % 8 == 0, EPSB_ERR_INVALID, "hidden size %lld is not a multiple of 8", (long long)H);
  return EPSB_OK;
}

}  // namespace

}  // namespace epsb

using namespace epsb;

extern "C" int epsb_local_reduce_ref(const void* y, const float* w_recv, const int32_t* scale_map,
                                     const int32_t* red_map, const int32_t* ret_incl, int k, int W, int S, int stage,
                                     int64_t max_rows, int64_t H, void* send, void* stream) {
  int rc = check_h(H);
  if (rc) return rc;
  EPSB_REQUIRE(k > 0 && k <= kMaxSlots, EPSB_ERR_INVALID, "topk %d exceeds %d", k, kMaxSlots);
  EPSB_REQUIRE(stage >= -1 && stage < S, EPSB_ERR_INVALID, "stage %d out of range for %d stages", stage, S);
  if (max_rows <= 0) return EPSB_OK;
  StageWindows win{ret_incl, W, S, stage};
  EPSB_SLOT_SWITCH(k, (local_reduce_kernel<true, kS><<<red_grid(max_rows), kRedThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)y, w_recv, scale_map, red_map, win, k, H, (uint8_t*)send)));
  return check_launch("local_reduce_ref");
}

extern "C" int epsb_local_reduce(const void* y, const int32_t* red_map, const int32_t* ret_incl, int k, int W, int S,
                                 int stage, int64_t max_rows, int64_t H, void* send, void* stream) {
  int rc = check_h(H);
  if (rc) return rc;
  EPSB_REQUIRE(k > 0 && k <= kMaxSlots, EPSB_ERR_INVALID, "topk %d exceeds %d", k, kMaxSlots);
  EPSB_REQUIRE(stage >= -1 && stage < S, EPSB_ERR_INVALID, "stage %d out of range for %d stages", stage, S);
  if (max_rows <= 0) return EPSB_OK;
  StageWindows win{ret_incl, W, S, stage};
  EPSB_SLOT_SWITCH(k, (local_reduce_kernel<false, kS><<<red_grid(max_rows), kRedThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)y, nullptr, nullptr, red_map, win, k, H, (uint8_t*)send)));
  return check_launch("local_reduce");
}

template <bool kRef>
static int launch_global_reduce(const void* recv, const int32_t* glob_map, const void* shared, const void* x,
                                const float* zero_scale, int T, int W, int64_t H, void* out, void* stream) {
  int rc = check_h(H);
  if (rc) return rc;
  EPSB_REQUIRE(W > 0, EPSB_ERR_INVALID, "world size %d", W);
  EPSB_REQUIRE(zero_scale == nullptr || x != nullptr, EPSB_ERR_INVALID, "zero_scale needs the raw input x");
  if (T <= 0) return EPSB_OK;
  auto st = static_cast<cudaStream_t>(stream);
  if (W <= kMaxSlots)
    EPSB_SLOT_SWITCH(W, (global_reduce_kernel<kRef, kS><<<red_grid(T), kRedThreads, 0, st>>>(
        (const uint8_t*)recv, glob_map, (const uint8_t*)shared, (const uint8_t*)x, zero_scale, T, W, H, (uint8_t*)out)));
  else
    global_reduce_wide_kernel<kRef><<<red_grid(T), kRedThreads, 0, st>>>((const uint8_t*)recv, glob_map,
                                                                         (const uint8_t*)shared, (const uint8_t*)x,
                                                                         zero_scale, T, W, H, (uint8_t*)out);
  return check_launch("global_reduce");
}

extern "C" int epsb_global_reduce_ref(const void* recv, const int32_t* glob_map, const void* shared, const void* x,
                                      const float* zero_scale, int T, int W, int64_t H, void* out, void* stream) {
  return launch_global_reduce<true>(recv, glob_map, shared, x, zero_scale, T, W, H, out, stream);
}

extern "C" int epsb_global_reduce(const void* recv, const int32_t* glob_map, const void* shared, const void* x,
                                  const float* zero_scale, int T, int W, int64_t H, void* out, void* stream) {
  return launch_global_reduce<false>(recv, glob_map, shared, x, zero_scale, T, W, H, out, stream);
}

extern "C" int epsb_reduce_ep1(const void* y, const int32_t* red_map, const int32_t* glob_map, const int32_t* ret_incl,
                               int S, const void* shared, const void* x, const float* zero_scale, int T, int k,
                               int64_t H, void* out, void* stream) {
  int rc = check_h(H);
  if (rc) return rc;
  EPSB_REQUIRE(k > 0 && k <= kMaxSlots, EPSB_ERR_INVALID, "topk %d exceeds %d", k, kMaxSlots);
  EPSB_REQUIRE(S > 0, EPSB_ERR_INVALID, "num_stages %d", S);
  EPSB_REQUIRE(zero_scale == nullptr || x != nullptr, EPSB_ERR_INVALID, "zero_scale needs the raw input x");
  if (T <= 0) return EPSB_OK;
  EPSB_SLOT_SWITCH(k, (reduce_ep1_kernel<kS><<<red_grid(T), kRedThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)y, red_map, glob_map, ret_incl, S, (const uint8_t*)shared, (const uint8_t*)x, zero_scale, T, k, H,
      (uint8_t*)out)));
  return check_launch("reduce_ep1");
}

extern "C" int epsb_fastep_reduce(const void* rows, const void* raw, const void* shared, const float* w,
                                  const int32_t* mapping, int T, int k, int64_t H, void* out, void* stream) {
  int rc = check_h(H);
  if (rc) return rc;
  EPSB_REQUIRE(k > 0 && k <= kMaxSlots, EPSB_ERR_INVALID, "topk %d exceeds %d", k, kMaxSlots);
  if (T <= 0) return EPSB_OK;
  EPSB_SLOT_SWITCH(k, (fastep_reduce_kernel<kS><<<red_grid(T), kRedThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)rows, (const uint8_t*)raw, (const uint8_t*)shared, w, mapping, T, k, H, (uint8_t*)out)));
  return check_launch("fastep_reduce");
}

extern "C" int epsb_silu_run(const void* gate_up, void* act, const int32_t* exclusive_sum, int num_experts,
                             int64_t rows, int64_t inter_size, void* stream) {
  EPSB_REQUIRE(inter_size > 0 && inter_size % 8 == 0, EPSB_ERR_INVALID, "Unsupported inter_size: %lld",
               (long long)inter_size);
  if (rows <= 0) return EPSB_OK;
  silu_kernel<<<red_grid(rows), kRedThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)gate_up, (uint8_t*)act, exclusive_sum, num_experts, rows, inter_size);
  return check_launch("silu_run");
}
