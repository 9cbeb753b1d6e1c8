// Router: group-limited top-k over sigmoid scores, the step that produces expert_indices / expert_scales.
//
// Semantics of the reference's topk_sigmoid (src/utils/topk_sigmoid.cu:158-262), which it instantiates for
// 256 experts / 8 groups / top-8 only; here for any expert count that is a multiple of 32 up to 1024, any
// group count that divides it, any k <= 32:
//   score  = 1 / (1 + expf(-logit))                      (fp32)
//   biased = score + bias[e]
//   group score = sum of the two largest biased scores of the group        (topk_sigmoid.cu:65-102)
//   the topk_groups groups with the largest group score stay               (:104-118)
//   k times: the largest biased score among the experts of those groups    (:120-156)
//   weight = score of the chosen expert * route_scale / sum of the chosen scores (unbiased)   (:236-244)
// Ties go to the lower group / expert id (the reference's strict `>` in its shuffle tree does the same for its
// power-of-two tile sizes).  Outputs are in selection order.  Ids >= num_ffn_experts can be mapped to the
// negative ids the scheduler reads as identity experts (-1 - (id - num_ffn_experts)).
//
// One warp per token; lane r holds experts [r*E/32, (r+1)*E/32) in registers; every reduction is a warp
// arg-max on (score, lowest index).
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

template <typename T>
__global__ void __launch_bounds__(kRouterThreads)
router_topk_sigmoid_kernel(const T* __restrict__ logits, const float* __restrict__ bias, int num_tokens, int E,
                           int n_groups, int topk_groups, int k, float route_scale, int num_ffn_experts,
                           int32_t* __restrict__ out_idx, float* __restrict__ out_w) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = kRouterThreads / 32;
  const int ept = E / 32;            // experts per lane
  const int gsize = E / n_groups;    // experts per group
  const int e0 = lane * ept;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < num_tokens; t += gridDim.x * warps_per_block) {
    float orig[kMaxPerLane], biased[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; i++) {
      if (i < ept) {
        const float x = to_float(logits[(size_t)t * E + e0 + i]);
        const float s = 1.0f / (1.0f + expf(-x));
        orig[i] = s;
        biased[i] = s + (bias != nullptr ? bias[e0 + i] : 0.0f);
      } else {
        orig[i] = 0.0f;
        biased[i] = -FLT_MAX;
      }
    }
    // ---- group scores: lane g ends up holding the score of group g
    float my_group_score = -FLT_MAX;
    for (int g = 0; g < n_groups; g++) {
      const int lo = g * gsize, hi = lo + gsize;
      Best first{-FLT_MAX, INT32_MAX};
#pragma unroll
      for (int i = 0; i < kMaxPerLane; i++) {
        const int e = e0 + i;
        if (i < ept && e >= lo && e < hi && biased[i] > first.score) first = Best{biased[i], e};
      }
      first = warp_argmax(first);
      Best second{-FLT_MAX, INT32_MAX};
#pragma unroll
      for (int i = 0; i < kMaxPerLane; i++) {
        const int e = e0 + i;
        if (i < ept && e >= lo && e < hi && e != first.index && biased[i] > second.score) second = Best{biased[i], e};
      }
      second = warp_argmax(second);
      const float gs = first.score + second.score;
      if (lane == g) my_group_score = gs;
    }
    // ---- the topk_groups best groups (n_groups <= 32: one per lane)
    uint32_t group_mask = 0;
    for (int r = 0; r < topk_groups; r++) {
      Best b{(lane < n_groups && !((group_mask >> lane) & 1u)) ? my_group_score : -FLT_MAX,
             (lane < n_groups && !((group_mask >> lane) & 1u)) ? lane : INT32_MAX};
      b = warp_argmax(b);
      if (b.index < n_groups) group_mask |= 1u << b.index;
    }
    // ---- k experts among the selected groups
    float sum = 0.0f;
    float my_w = 0.0f;   // lane j keeps the j-th selected expert
    int my_e = 0;
    for (int j = 0; j < k; j++) {
      Best b{-FLT_MAX, INT32_MAX};
#pragma unroll
      for (int i = 0; i < kMaxPerLane; i++) {
        const int e = e0 + i;
        if (i < ept && ((group_mask >> (e / gsize)) & 1u) && biased[i] > b.score) b = Best{biased[i], e};
      }
      b = warp_argmax(b);
      float o = 0.0f;
      if (b.index != INT32_MAX && b.index >= e0 && b.index < e0 + ept) {
#pragma unroll
        for (int i = 0; i < kMaxPerLane; i++)
          if (i == b.index - e0) {
            o = orig[i];
            biased[i] = -FLT_MAX;
          }
      }
      // the owner lane holds the unbiased score: hand it to everybody
      const int owner = b.index != INT32_MAX ? b.index / ept : 0;
      o = __shfl_sync(0xffffffffu, o, owner);
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

}  // namespace

}  // namespace epsb

using namespace epsb;

extern "C" int epsb_router_topk_sigmoid(const void* logits, int logits_are_bf16, const float* bias, int num_tokens,
                                        int num_experts, int num_expert_groups, int topk_groups, int topk,
                                        float route_scale, int num_ffn_experts, int32_t* expert_indices,
                                        float* expert_scales, void* stream) {
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
    router_topk_sigmoid_kernel<__nv_bfloat16><<<(int)blocks, kRouterThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), bias, num_tokens, num_experts, num_expert_groups, topk_groups, topk,
        route_scale, num_ffn_experts, expert_indices, expert_scales);
  else
    router_topk_sigmoid_kernel<float><<<(int)blocks, kRouterThreads, 0, st>>>(
        static_cast<const float*>(logits), bias, num_tokens, num_experts, num_expert_groups, topk_groups, topk,
        route_scale, num_ffn_experts, expert_indices, expert_scales);
  return check_launch("router_topk_sigmoid");
}
