// Router: group-limited top-k over sigmoid scores, the step that produces expert_indices / expert_scales.
//
// Semantics of the reference's topk_sigmoid (src/utils/topk_sigmoid.cu:158-262), which it instantiates for
// 256 experts / 8 groups / top-8 only; here for any expert count that is a multiple of 32 up to 1024, any
// group count that divides it, any k <= 32:
//   score  = 1 / (1 + expf(-logit))                      (fp32; or, not in the reference, softmax over the token's logits)
//   biased = score + bias[e]
//   group score = sum of the two largest biased scores of the group        (topk_sigmoid.cu:65-102)
//   the topk_groups groups with the largest group score stay               (:104-118)
//   k times: the largest biased score among the experts of those groups    (:120-156)
//   weight = score of the chosen expert * route_scale / sum of the chosen scores (unbiased)   (:236-244)
// Ties go to the lower group / expert id (the reference's strict `>` in its shuffle tree does the same for its
// power-of-two tile sizes).  Outputs are in selection order.  Ids >= num_ffn_experts can be mapped to the
// negative ids the scheduler reads as identity experts (-1 - (id - num_ffn_experts)).
//
// One warp per token; lane r holds experts [r*E/32, (r+1)*E/32) in registers (the kernel is instantiated per
// E/32); every reduction is an arg-max on (score, lowest index), over the warp, or over lane segments for all
// groups at once when a group is a power-of-two number of whole lanes.
#include <cfloat>

#include "common.cuh"

namespace epsb {

namespace {

constexpr int kMaxPerLane = 32;   // experts per lane: E <= 1024
constexpr int kRouterThreads = 256;

struct Best {
  float score;
  int index;
};

// (higher score, then lower index) over the warp; every lane gets the winner.
__device__ __forceinline__ Best warp_argmax(Best b) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float s = __shfl_xor_sync(0xffffffffu, b.score, off);
    const int i = __shfl_xor_sync(0xffffffffu, b.index, off);
    if (s > b.score || (s == b.score && i < b.index)) {
      b.score = s;
      b.index = i;
    }
  }
  return b;
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// (higher score, then lower index) over aligned segments of `width` lanes (a power of two); every lane of a
// segment gets its segment's winner.
__device__ __forceinline__ Best segment_argmax(Best b, int width) {
  for (int off = width >> 1; off > 0; off >>= 1) {
    const float s = __shfl_xor_sync(0xffffffffu, b.score, off);
    const int i = __shfl_xor_sync(0xffffffffu, b.index, off);
    if (s > b.score || (s == b.score && i < b.index)) {
      b.score = s;
      b.index = i;
    }
  }
  return b;
}

// kEpt = experts per lane (E / 32), a compile-time bound so that the scores stay in registers.
template <typename T, int kEpt>
__global__ void __launch_bounds__(kRouterThreads)
router_topk_sigmoid_kernel(const T* __restrict__ logits, const float* __restrict__ bias, int num_tokens, int n_groups,
                           int topk_groups, int k, float route_scale, int num_ffn_experts, int softmax,
                           int32_t* __restrict__ out_idx, float* __restrict__ out_w) {
  constexpr int E = 32 * kEpt;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = kRouterThreads / 32;
  const int gsize = E / n_groups;    // experts per group
  const int e0 = lane * kEpt;
  // Groups made of whole lanes, a power of two of them: all groups are reduced at once inside lane segments.
  const int lanes_per_group = gsize / kEpt;
  const bool segmented = gsize % kEpt == 0 && lanes_per_group >= 1 && (lanes_per_group & (lanes_per_group - 1)) == 0;
  float bias_r[kEpt];
#pragma unroll
  for (int i = 0; i < kEpt; i++) bias_r[i] = bias != nullptr ? bias[e0 + i] : 0.0f;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < num_tokens; t += gridDim.x * warps_per_block) {
    float orig[kEpt], biased[kEpt];
    if (softmax) {   // warp-uniform: score = softmax over all experts of the token
      float mx = -FLT_MAX;
#pragma unroll
      for (int i = 0; i < kEpt; i++) {
        orig[i] = to_float(logits[(size_t)t * E + e0 + i]);
        mx = fmaxf(mx, orig[i]);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      float den = 0.0f;
#pragma unroll
      for (int i = 0; i < kEpt; i++) {
        orig[i] = expf(orig[i] - mx);
        den += orig[i];
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) den += __shfl_xor_sync(0xffffffffu, den, off);
#pragma unroll
      for (int i = 0; i < kEpt; i++) {
        orig[i] = orig[i] / den;
        biased[i] = orig[i] + bias_r[i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < kEpt; i++) {
        const float x = to_float(logits[(size_t)t * E + e0 + i]);
        const float s = 1.0f / (1.0f + expf(-x));
        orig[i] = s;
        biased[i] = s + bias_r[i];
      }
    }
    // ---- group scores: lane g ends up holding the score of group g
    float my_group_score = -FLT_MAX;
    if (segmented) {
      Best first{-FLT_MAX, INT32_MAX};
#pragma unroll
      for (int i = 0; i < kEpt; i++)
        if (biased[i] > first.score) first = Best{biased[i], e0 + i};
      first = segment_argmax(first, lanes_per_group);
      Best second{-FLT_MAX, INT32_MAX};
#pragma unroll
      for (int i = 0; i < kEpt; i++)
        if (e0 + i != first.index && biased[i] > second.score) second = Best{biased[i], e0 + i};
      second = segment_argmax(second, lanes_per_group);
      const float gs = first.score + second.score;        // held by every lane of group lane / lanes_per_group
      my_group_score = __shfl_sync(0xffffffffu, gs, (lane * lanes_per_group) & 31);
    } else {
      for (int g = 0; g < n_groups; g++) {
        const int lo = g * gsize, hi = lo + gsize;
        Best first{-FLT_MAX, INT32_MAX};
#pragma unroll
        for (int i = 0; i < kEpt; i++) {
          const int e = e0 + i;
          if (e >= lo && e < hi && biased[i] > first.score) first = Best{biased[i], e};
        }
        first = warp_argmax(first);
        Best second{-FLT_MAX, INT32_MAX};
#pragma unroll
        for (int i = 0; i < kEpt; i++) {
          const int e = e0 + i;
          if (e >= lo && e < hi && e != first.index && biased[i] > second.score) second = Best{biased[i], e};
        }
        second = warp_argmax(second);
        if (lane == g) my_group_score = first.score + second.score;
      }
    }
    // ---- the topk_groups best groups (n_groups <= 32: one per lane)
    uint32_t group_mask = 0;
    for (int r = 0; r < topk_groups; r++) {
      const bool open = lane < n_groups && !((group_mask >> lane) & 1u);
      Best b{open ? my_group_score : -FLT_MAX, open ? lane : INT32_MAX};
      b = warp_argmax(b);
      if (b.index < n_groups) group_mask |= 1u << b.index;
    }
    // experts outside the kept groups leave the contest
#pragma unroll
    for (int i = 0; i < kEpt; i++)
      if (!((group_mask >> ((e0 + i) / gsize)) & 1u)) biased[i] = -FLT_MAX;
    // ---- k experts among the kept groups
    float sum = 0.0f;
    float my_w = 0.0f;   // lane j keeps the j-th selected expert
    int my_e = 0;
    for (int j = 0; j < k; j++) {
      Best b{-FLT_MAX, INT32_MAX};
#pragma unroll
      for (int i = 0; i < kEpt; i++)
        if (biased[i] > b.score) b = Best{biased[i], e0 + i};
      b = warp_argmax(b);
      float o = 0.0f;
#pragma unroll
      for (int i = 0; i < kEpt; i++)
        if (e0 + i == b.index) {
          o = orig[i];
          biased[i] = -FLT_MAX;
        }
      // the owner lane holds the unbiased score: hand it to everybody
      o = __shfl_sync(0xffffffffu, o, b.index != INT32_MAX ? b.index / kEpt : 0);
      sum += o;
      if (lane == j) {
        my_w = o;
        my_e = b.index;
      }
    }
    const float rescale = route_scale / sum;
    if (lane < k) {
      int e = my_e;
      if (e >= num_ffn_experts) e = -1 - (e - num_ffn_experts);
      out_idx[(size_t)t * k + lane] = e;
      out_w[(size_t)t * k + lane] = my_w * rescale;
    }
  }
}

template <typename T>
int launch_router(int ept, int blocks, cudaStream_t st, const T* logits, const float* bias, int num_tokens, int n_groups,
                  int topk_groups, int k, float route_scale, int num_ffn, int softmax, int32_t* out_idx, float* out_w) {
#define EPSB_ROUTER_CASE(N)                                                                                          \
  case N:                                                                                                             \
    router_topk_sigmoid_kernel<T, N><<<blocks, kRouterThreads, 0, st>>>(logits, bias, num_tokens, n_groups,           \
                                                                          topk_groups, k, route_scale, num_ffn,       \
                                                                          softmax, out_idx, out_w);                   \
    break;
  switch (ept) {
    EPSB_ROUTER_CASE(1) EPSB_ROUTER_CASE(2) EPSB_ROUTER_CASE(3) EPSB_ROUTER_CASE(4) EPSB_ROUTER_CASE(5)
    EPSB_ROUTER_CASE(6) EPSB_ROUTER_CASE(7) EPSB_ROUTER_CASE(8) EPSB_ROUTER_CASE(9) EPSB_ROUTER_CASE(10)
    EPSB_ROUTER_CASE(11) EPSB_ROUTER_CASE(12) EPSB_ROUTER_CASE(13) EPSB_ROUTER_CASE(14) EPSB_ROUTER_CASE(15)
    EPSB_ROUTER_CASE(16) EPSB_ROUTER_CASE(17) EPSB_ROUTER_CASE(18) EPSB_ROUTER_CASE(19) EPSB_ROUTER_CASE(20)
    EPSB_ROUTER_CASE(21) EPSB_ROUTER_CASE(22) EPSB_ROUTER_CASE(23) EPSB_ROUTER_CASE(24) EPSB_ROUTER_CASE(25)
    EPSB_ROUTER_CASE(26) EPSB_ROUTER_CASE(27) EPSB_ROUTER_CASE(28) EPSB_ROUTER_CASE(29) EPSB_ROUTER_CASE(30)
    EPSB_ROUTER_CASE(31) EPSB_ROUTER_CASE(32)
    default:
      return fail(EPSB_ERR_INVALID, "Not supported num_experts: %d", ept * 32);
  }
#undef EPSB_ROUTER_CASE
  return check_launch("router_topk_sigmoid");
}

}  // namespace

}  // namespace epsb

using namespace epsb;

extern "C" int epsb_router_topk(int score_func, const void* logits, int logits_are_bf16, const float* bias,
                                int num_tokens, int num_experts, int num_expert_groups, int topk_groups, int topk,
                                float route_scale, int num_ffn_experts, int32_t* expert_indices, float* expert_scales,
                                void* stream) {
  EPSB_REQUIRE(score_func == EPSB_ROUTER_SIGMOID || score_func == EPSB_ROUTER_SOFTMAX, EPSB_ERR_INVALID,
               "unknown score function %d", score_func);
  EPSB_REQUIRE(num_tokens >= 0, EPSB_ERR_INVALID, "num_tokens %d is negative", num_tokens);
  EPSB_REQUIRE(num_experts > 0 && num_experts % 32 == 0 && num_experts <= 32 * kMaxPerLane, EPSB_ERR_INVALID,
               "Not supported num_experts: %d (a multiple of 32 up to %d)", num_experts, 32 * kMaxPerLane);
  EPSB_REQUIRE(num_expert_groups > 0 && num_expert_groups <= 32 && num_experts % num_expert_groups == 0,
               EPSB_ERR_INVALID, "Not supported num_expert_groups: %d for num_experts: %d", num_expert_groups,
               num_experts);
  EPSB_REQUIRE(topk_groups > 0 && topk_groups <= num_expert_groups, EPSB_ERR_INVALID,
               "topk_groups %d out of range for %d groups", topk_groups, num_expert_groups);
  EPSB_REQUIRE(topk > 0 && topk <= 32 && topk <= topk_groups * (num_experts / num_expert_groups), EPSB_ERR_INVALID,
               "Not supported topk: %d", topk);
  EPSB_REQUIRE(num_ffn_experts > 0 && num_ffn_experts <= num_experts, EPSB_ERR_INVALID,
               "num_ffn_experts %d out of range", num_ffn_experts);
  if (num_tokens == 0) return EPSB_OK;
  const int warps_per_block = kRouterThreads / 32;
  int64_t blocks = ((int64_t)num_tokens + warps_per_block - 1) / warps_per_block;
  if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
  auto st = static_cast<cudaStream_t>(stream);
  if (logits_are_bf16)
    return launch_router(num_experts / 32, (int)blocks, st, static_cast<const __nv_bfloat16*>(logits), bias, num_tokens,
                         num_expert_groups, topk_groups, topk, route_scale, num_ffn_experts, score_func,
                         expert_indices, expert_scales);
  return launch_router(num_experts / 32, (int)blocks, st, static_cast<const float*>(logits), bias, num_tokens,
                       num_expert_groups, topk_groups, topk, route_scale, num_ffn_experts, score_func, expert_indices,
                       expert_scales);
}

extern "C" int epsb_router_topk_sigmoid(const void* logits, int logits_are_bf16, const float* bias, int num_tokens,
                                        int num_experts, int num_expert_groups, int topk_groups, int topk,
                                        float route_scale, int num_ffn_experts, int32_t* expert_indices,
                                        float* expert_scales, void* stream) {
  return epsb_router_topk(EPSB_ROUTER_SIGMOID, logits, logits_are_bf16, bias, num_tokens, num_experts,
                          num_expert_groups, topk_groups, topk, route_scale, num_ffn_experts, expert_indices,
                          expert_scales, stream);
}
