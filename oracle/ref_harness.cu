// extern "C" launchers around the REFERENCE's own arch-agnostic CUDA kernels.
//
// TEST INFRASTRUCTURE ONLY.  This file contains no reference code: it includes the reference's
// headers from where they lie and calls the reference's launchers, so that the kernels the
// reference ships can run on a B200 as a second witness for the CPU oracle and for this
// repository's kernels.  oracle/build_ref.py compiles it together with the reference's .cu
// files (in place, never copied) into oracle/_ref/libeps_ref.so.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "src/executor/activations.cuh"
#include "src/fast_ep/all_to_all/fast_ep_kernels.cuh"
#include "src/quant/fp8.cuh"
#include "src/scheduler/comm_expander.cuh"
#include "src/scheduler/gemm_expander.cuh"
#include "src/scheduler/global_reducer.cuh"
#include "src/scheduler/local_reducer.cuh"
#include "src/scheduler/zero_reducer.cuh"
#include "src/utils/rms_norm.cuh"
#include "src/utils/topk_sigmoid.cuh"

using bf16 = __nv_bfloat16;

extern "C" {

int ref_sync() { return (int)cudaDeviceSynchronize(); }

// scheduler/comm_expander_ver2.cu:174
void ref_comm_plan(const int* idx, int* leading_ws, int* mapping, int* incl, int T, int k, int E, int S, int W) {
  eps::ExpandForCommPlanKernelParams p{};
  p.expert_indices = idx;
  p.sorted_leading_experts = leading_ws;
  p.expand_plan = eps::ExpandForCommPlan{mapping, incl};
  p.num_tokens = T;
  p.topk = k;
  p.num_experts = E;
  p.num_stages = S;
  p.ep_world_size = W;
  p.tile_states = nullptr;
  eps::getExpandForCommPlan_ver2(p, 0);
}

// scheduler/gemm_expander_ver2.cu:180
void ref_gemm_plan(int* ridx, const int* recv_incl, int* mapping, int* excl, int lo, int hi, int E, int S, int k,
                   int W, long long max_tok) {
  eps::ExpandForGemmPlanKernelParams p{};
  p.expert_indices = ridx;
  p.sorted_expert_indices = nullptr;
  p.inclusive_sum = recv_incl;
  p.expand_plan = eps::ExpandForGemmPlan{mapping, excl};
  p.local_expert_begin = lo;
  p.local_expert_end = hi;
  p.num_experts = E;
  p.num_stages = S;
  p.topk = k;
  p.ep_world_size = W;
  p.max_num_tokens_per_gpu = max_tok;
  eps::getExpandForGemmPlan_ver2(p, 0);
}

// scheduler/local_reducer_ver2.cu:471
void ref_local_reduce_plan(const int* ridx, int* tail_ws, int* sorted_tail_ws, const int* recv_incl, int* red_map,
                           int* scale_map, int* ret_incl, int* gemm_map, int* excl, int lo, int hi, int E, int S,
                           int k, int W, long long max_tok, int num_global_tokens) {
  eps::LocalReducePlanKernelParams p{};
  p.expert_indices = ridx;
  p.tailing_experts = tail_ws;
  p.sorted_tailing_experts = sorted_tail_ws;
  p.inclusive_sum = recv_incl;
  p.mapping = nullptr;
  p.reduce_plan = eps::LocalReducePlan{red_map, scale_map, ret_incl};
  p.expand_plan = eps::ExpandForGemmPlan{gemm_map, excl};
  p.local_expert_begin = lo;
  p.local_expert_end = hi;
  p.num_experts = E;
  p.num_stages = S;
  p.topk = k;
  p.ep_world_size = W;
  p.max_num_tokens_per_gpu = max_tok;
  eps::getLocalReducePlan_ver2(p, 0, num_global_tokens);
}

// scheduler/global_reducer_ver2.cu:206
void ref_global_reduce_plan(const int* idx, int* tail_ws, int* glob_map, int* coll_incl, int* send_map,
                            int* send_incl, int T, int E, int S, int k, int W) {
  eps::GlobalReducePlanKernelParams p{};
  p.expert_indices = idx;
  p.tailing_experts = tail_ws;
  p.sorted_tailing_experts = nullptr;
  p.reduce_plan = eps::GlobalReducePlan{glob_map, coll_incl};
  p.expand_plan = eps::ExpandForCommPlan{send_map, send_incl};
  p.num_tokens = T;
  p.num_experts = E;
  p.num_stages = S;
  p.topk = k;
  p.ep_world_size = W;
  eps::getGlobalReducePlan_ver2(p, 0);
}

// scheduler/zero_reducer.cu:27,44
void ref_zero_plan(const int* idx, const float* w, int T, int k, float* zero_scale) {
  eps::ZeroReducePlanKernelParams<bf16, float> p{};
  p.expert_indices = idx;
  p.expert_scales = w;
  p.num_local_tokens = T;
  p.topk = k;
  p.zero_reduce_plan.zero_reduce_scales = zero_scale;
  eps::getZeroReducePlan(p, 0);
}
void ref_zero_reduce(float* zero_scale, int T, long long H, const void* x, void* out) {
  eps::ZeroReduceKernelParams<bf16, bf16, float> p{};
  p.zero_reduce_scales = zero_scale;
  p.num_local_tokens = T;
  p.hidden_size = H;
  p.raw_input = (const bf16*)x;
  p.output = (bf16*)out;
  eps::zeroReduce(p, 0);
}

// scheduler/local_reducer.cu:193 (bf16 rows, fp32 gate weights)
void ref_local_reduce(int* red_map, int* scale_map, int* ret_incl, int S, int k, int W, long long H, const void* y,
                      void* send, const float* w_recv, long long hint, int stage) {
  eps::LocalReduceKernelParams<bf16, float> p{};
  p.reduce_plan = eps::LocalReducePlan{red_map, scale_map, ret_incl};
  p.num_stages = S;
  p.topk = k;
  p.ep_world_size = W;
  p.hidden_size = H;
  p.src = (const bf16*)y;
  p.dst = (bf16*)send;
  p.expert_scales = w_recv;
  p.num_tokens_hint = hint;
  eps::localReduce(p, stage, 0);
}

// scheduler/global_reducer.cu:183
void ref_global_reduce(int* glob_map, int T, int W, long long H, const void* recv, void* out, const void* shared) {
  eps::GlobalReduceKernelParams<bf16> p{};
  p.reduce_plan = eps::GlobalReducePlan{glob_map, nullptr};
  p.num_tokens = T;
  p.ep_world_size = W;
  p.hidden_size = H;
  p.src = (const bf16*)recv;
  p.dst = (bf16*)out;
  p.shared = (const bf16*)shared;
  eps::globalReduce(p, 0);
}

// quant/fp8.cu:362 (dense form)
void ref_quant_1x128(void* x, long long rows, long long cols, void* q, float* scales) {
  eps::PerTokenGroupQuantFP8DenseParams<bf16> p{};
  p.quanted = (eps::FP8_TYPE*)q;
  p.origin = (bf16*)x;
  p.scales = scales;
  p.cols = cols;
  p.group_size = 128;
  p.num_tokens = rows;
  p.dequant = false;
  eps::per_token_group_quant_fp8<bf16, eps::PerTokenGroupQuantFP8DenseParams>(p, 0);
}

// executor/activations.cu (ragged form)
void ref_silu(const void* gate_up, void* act, const int* excl, int num_experts, int inter_x2, int hint) {
  eps::silu_activate<bf16>((const bf16*)gate_up, (bf16*)act, excl, num_experts, inter_x2, hint, 0);
}

// utils/topk_sigmoid.cu:264-286 (throws for anything but 256 experts / 8 groups / top-8)
int ref_topk_sigmoid_f32(const float* scores, const float* bias, float* expert_scales, int* expert_indices, int T, int E,
                         int n_groups, int topk_groups, int topk, float route_scale) {
  eps::TopkSigmoidParams<float, float, int> p{};
  p.scores = scores;
  p.bias = bias;
  p.expert_scales = expert_scales;
  p.expert_indices = expert_indices;
  p.num_tokens = T;
  p.num_experts = E;
  p.num_expert_groups = n_groups;
  p.topk_groups = topk_groups;
  p.topk = topk;
  p.route_scale = route_scale;
  try {
    eps::topk_sigmoid(p, 0);
  } catch (...) {
    return 1;
  }
  return 0;
}

int ref_topk_sigmoid_bf16(const bf16* scores, const float* bias, float* expert_scales, int* expert_indices, int T, int E,
                          int n_groups, int topk_groups, int topk, float route_scale) {
  eps::TopkSigmoidParams<bf16, float, int> p{};
  p.scores = scores;
  p.bias = bias;
  p.expert_scales = expert_scales;
  p.expert_indices = expert_indices;
  p.num_tokens = T;
  p.num_experts = E;
  p.num_expert_groups = n_groups;
  p.topk_groups = topk_groups;
  p.topk = topk;
  p.route_scale = route_scale;
  try {
    eps::topk_sigmoid(p, 0);
  } catch (...) {
    return 1;
  }
  return 0;
}

// utils/rms_norm.cu:128-140
int ref_rms_norm_bf16(bf16* out, const bf16* input, const bf16* scale, float eps, int m, int n) {
  try {
    eps::rms_norm<bf16>(out, input, scale, eps, m, n, 0);
  } catch (...) {
    return 1;
  }
  return 0;
}

// fast_ep/all_to_all/fast_ep_kernels.cu:158 (expandPlanKernel<E> for E in {512, 256, 128, 32}, blockExpandPlanKernel else)
void ref_fastep_expand_plan(const int* idx, int* excl, int* mapping, long long T, long long k, long long E) {
  fast_ep::ExpandPlan p{T, k, E, idx, excl, mapping};
  fast_ep::expandPlan(p, 0);
}

// fast_ep_kernels.cu:202 (cols must be one of the reference's HIDDEN_SIZE_SWITCH values)
int ref_fastep_expand(const bf16* src, bf16* dst, long long cols, const int* idx, int* excl, int* mapping, long long T,
                      long long k, long long E) {
  fast_ep::ExpandParams<bf16> p{src, dst, cols, fast_ep::ExpandPlan{T, k, E, idx, excl, mapping}};
  try {
    fast_ep::expand<bf16>(p, 0);
  } catch (...) {
    return 1;
  }
  return 0;
}

// fast_ep_kernels.cu:321
int ref_fastep_reduce(const bf16* src, bf16* dst, const bf16* shared, const bf16* raw, const float* scales,
                      long long cols, const int* idx, int* excl, int* mapping, long long T, long long k, long long E) {
  fast_ep::ReduceParams<bf16, float> p{src, dst, shared, raw, scales, cols, fast_ep::ExpandPlan{T, k, E, idx, excl, mapping}};
  try {
    fast_ep::reduce<bf16, float>(p, 0);
  } catch (...) {
    return 1;
  }
  return 0;
}

// fast_ep_kernels.cu:591.  The channel calls of the all-gather kernel are no-ops here: the caller passes the table
// `all_gathered` [W][E+1] already filled, and the plan kernels derive everything else from it.
void ref_fastep_plan(int* all_gathered, long long my_rank, long long W, long long E, int* remote_recv, int* local_send,
                     int* gemm_plan, int* arr_src, int* arr_rows, int* arr_dst) {
  eps::CommBuffHost<int> host(0, 0, my_rank, W);
  fast_ep::AllGatheredPlan p{my_rank, W, W, E, all_gathered, remote_recv, local_send, gemm_plan,
                             fast_ep::ArrangePlan{arr_src, arr_rows, arr_dst}, eps::CommBuff<int>(host)};
  fast_ep::allGatherPlan(p, 0);
}

// fast_ep_kernels.cu:679
int ref_fastep_arrange(const bf16* src, bf16* dst, long long W, long long E, long long cols, int* arr_src, int* arr_rows,
                       int* arr_dst, long long num_tokens_hint) {
  fast_ep::ArrangeParams<bf16> p{W, E, cols, src, dst, fast_ep::ArrangePlan{arr_src, arr_rows, arr_dst}, num_tokens_hint};
  try {
    fast_ep::arrange<bf16>(p, 0);
  } catch (...) {
    return 1;
  }
  return 0;
}

}  // extern "C"
