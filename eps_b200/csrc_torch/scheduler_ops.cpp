// libscheduler_.so: the scheduler operators, registered under `scheduler` (what python/eps/scheduler/ops.py:11 reads)
// and under `eps` (what the reference's src/scheduler/bindings/bindings.cpp:6 registers), with the reference's
// names and argument lists (src/scheduler/bindings/scheduler_ops.cu:18-224).  Handles are raw pointers to the
// C++ objects of scheduler.hpp.  The ops after `eps_epilogue` are additions for the FP8 path (no counterpart in
// the reference): FP8 hidden rows, rows that carry their gate weight out of the down GEMM, the single-rank fused
// reduce, and a rendezvous that does not read the row count on the host.
#include "scheduler.hpp"

namespace {

using namespace epsb_host;

Scheduler* sched(fptr_t p) {
  TORCH_CHECK(p != 0, "scheduler handle is null");
  return reinterpret_cast<Scheduler*>(p);
}
Scheduler::Context& ctx(fptr_t p) {
  TORCH_CHECK(p != 0, "context handle is null");
  return *reinterpret_cast<Scheduler::Context*>(p);
}

fptr_t create_impl(int64_t topk, int64_t num_experts, int64_t hidden_size, int64_t input_scales_dim,
                   int64_t max_num_tokens_per_gpu, fptr_t comm, int64_t max_num_stages, bool fp8_hidden) {
  return reinterpret_cast<fptr_t>(new Scheduler(Scheduler::Params{(int)topk, (int)num_experts, hidden_size,
                                                                  (int)input_scales_dim, max_num_tokens_per_gpu,
                                                                  reinterpret_cast<Communicator*>(comm),
                                                                  (int)max_num_stages, fp8_hidden}));
}

fptr_t create(int64_t topk, int64_t num_experts, int64_t hidden_size, int64_t input_scales_dim,
              int64_t max_num_tokens_per_gpu, fptr_t comm, int64_t max_num_stages) {
  return create_impl(topk, num_experts, hidden_size, input_scales_dim, max_num_tokens_per_gpu, comm, max_num_stages,
                     false);
}
fptr_t create_fp8(int64_t topk, int64_t num_experts, int64_t hidden_size, int64_t input_scales_dim,
                  int64_t max_num_tokens_per_gpu, fptr_t comm, int64_t max_num_stages) {
  return create_impl(topk, num_experts, hidden_size, input_scales_dim, max_num_tokens_per_gpu, comm, max_num_stages,
                     true);
}

void destroy(fptr_t ptr) { delete reinterpret_cast<Scheduler*>(ptr); }

fptr_t get_context(fptr_t ptr, int64_t num_tokens, int64_t num_global_tokens, int64_t num_stages, bool input_quanted) {
  return reinterpret_cast<fptr_t>(
      sched(ptr)->getContext((int)num_tokens, (int)num_global_tokens, (int)num_stages, input_quanted));
}
void destroy_context(fptr_t ptr) { delete reinterpret_cast<Scheduler::Context*>(ptr); }
int64_t get_workspace_size_context(fptr_t ptr) { return (int64_t)Scheduler::workspaceSize(ctx(ptr)); }
void set_ws_context(fptr_t ptr, at::Tensor& ws) {
  TORCH_CHECK(ws.is_cuda() && ws.is_contiguous(), "ws must be a contiguous CUDA tensor");
  TORCH_CHECK((size_t)ws.numel() * ws.element_size() >= ctx(ptr).ws_bytes, "ws is smaller than the context needs");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(ws.data_ptr()) & 15) == 0, "ws must be 16-byte aligned");
  // only the address is remembered here: the buffers are carved by the scheduler (whose sizes the layout needs)
  // when rendezvous starts the call
  ctx(ptr).ws = static_cast<char*>(ws.data_ptr());
}

int64_t rendezvous(fptr_t ptr, const at::Tensor& expert_indices, fptr_t context) {
  check(expert_indices, 2, "expert_indices");
  TORCH_CHECK(expert_indices.scalar_type() == at::kInt, "expert_indices must be int32");
  auto& c = ctx(context);
  TORCH_CHECK(expert_indices.size(0) == c.num_tokens, "expert_indices has ", expert_indices.size(0),
              " rows, the context was made for ", c.num_tokens);
  sched(ptr)->setWorkspace(c, c.ws);
  return sched(ptr)->rendezvous(expert_indices.data_ptr<int32_t>(), c, current_stream());
}

int64_t rendezvous_async(fptr_t ptr, const at::Tensor& expert_indices, fptr_t context, int64_t max_cluster) {
  check(expert_indices, 2, "expert_indices");
  TORCH_CHECK(expert_indices.scalar_type() == at::kInt, "expert_indices must be int32");
  auto& c = ctx(context);
  TORCH_CHECK(expert_indices.size(0) == c.num_tokens, "expert_indices has ", expert_indices.size(0),
              " rows, the context was made for ", c.num_tokens);
  sched(ptr)->setWorkspace(c, c.ws);
  return sched(ptr)->rendezvous(expert_indices.data_ptr<int32_t>(), c, current_stream(), true, (int)max_cluster);
}

void plan(fptr_t ptr, const at::Tensor& expert_indices, const at::Tensor& expert_scales,
          const at::Tensor& exclusive_sum, fptr_t context) {
  check(expert_indices, 2, "expert_indices");
  check(expert_scales, 2, "expert_scales");
  check(exclusive_sum, 1, "exclusive_sum");
  TORCH_CHECK(expert_scales.scalar_type() == at::kFloat, "expert_scales must be float32");
  TORCH_CHECK(exclusive_sum.scalar_type() == at::kInt && exclusive_sum.numel() == sched(ptr)->localNumExperts() + 1,
              "exclusive_sum must be int32 [local_num_experts + 1]");
  sched(ptr)->plan(expert_indices.data_ptr<int32_t>(), expert_scales.data_ptr<float>(),
                   exclusive_sum.data_ptr<int32_t>(), ctx(context), current_stream());
}

void plan_fp8(fptr_t ptr, const at::Tensor& expert_indices, const at::Tensor& expert_scales,
              const at::Tensor& exclusive_sum, fptr_t context, const std::optional<at::Tensor>& payload_hidden,
              const std::optional<at::Tensor>& payload_scales, int64_t max_cluster) {
  check(expert_indices, 2, "expert_indices");
  check(expert_scales, 2, "expert_scales");
  check(exclusive_sum, 1, "exclusive_sum");
  TORCH_CHECK(exclusive_sum.scalar_type() == at::kInt && exclusive_sum.numel() == sched(ptr)->localNumExperts() + 1,
              "exclusive_sum must be int32 [local_num_experts + 1]");
  sched(ptr)->plan(expert_indices.data_ptr<int32_t>(), expert_scales.data_ptr<float>(),
                   exclusive_sum.data_ptr<int32_t>(), ctx(context), current_stream(),
                   payload_hidden.has_value() ? payload_hidden->data_ptr() : nullptr,
                   payload_scales.has_value() ? payload_scales->data_ptr<float>() : nullptr, (int)max_cluster);
}

void prologue(fptr_t ptr, const at::Tensor& expert_scales, const at::Tensor& hidden_states,
              const std::optional<at::Tensor>& input_scales, const std::optional<at::Tensor>& recv_input_scales,
              fptr_t context) {
  check(expert_scales, 2, "expert_scales");
  check(hidden_states, 2, "hidden_states");
  sched(ptr)->prologue(expert_scales.data_ptr<float>(), hidden_states.data_ptr(),
                       input_scales.has_value() ? input_scales->data_ptr<float>() : nullptr,
                       recv_input_scales.has_value() ? recv_input_scales->data_ptr<float>() : nullptr, ctx(context),
                       current_stream());
}

void prologue_fp8(fptr_t ptr, const at::Tensor& expert_scales, const at::Tensor& hidden_codes,
                  const at::Tensor& input_scales, at::Tensor& recv_input_scales, const at::Tensor& raw_input,
                  fptr_t context) {
  check(expert_scales, 2, "expert_scales");
  check(hidden_codes, 2, "hidden_states");
  check(raw_input, 2, "raw_input");
  TORCH_CHECK(is_fp8_codes(hidden_codes), "hidden_states must hold e4m3 codes (uint8 or float8_e4m3fn)");
  TORCH_CHECK(raw_input.scalar_type() == at::kBFloat16, "raw_input must be bfloat16");
  sched(ptr)->prologue(expert_scales.data_ptr<float>(), hidden_codes.data_ptr(), input_scales.data_ptr<float>(),
                       recv_input_scales.data_ptr<float>(), ctx(context), current_stream(), raw_input.data_ptr(),
                       /*direct=*/sched(ptr)->worldSize() == 1);
}

void dispatch(fptr_t ptr, fptr_t context, int64_t stage_idx) {
  sched(ptr)->dispatch(ctx(context), (int)stage_idx, current_stream());
}

void gemm_expand(fptr_t ptr, at::Tensor& gemm_input, fptr_t context, int64_t stage_idx) {
  check(gemm_input, 2, "gemm_input");
  sched(ptr)->gemmExpand(gemm_input.data_ptr(), ctx(context), (int)stage_idx, current_stream());
}

void local_reduce(fptr_t ptr, const at::Tensor& gemm_output, fptr_t context, int64_t stage_idx) {
  check(gemm_output, 2, "gemm_output");
  TORCH_CHECK(gemm_output.scalar_type() == at::kBFloat16, "gemm_output must be bfloat16");
  sched(ptr)->localReduce(gemm_output.data_ptr(), ctx(context), (int)stage_idx, current_stream(), false);
}

void local_reduce_weighted(fptr_t ptr, const at::Tensor& gemm_output, fptr_t context, int64_t stage_idx) {
  check(gemm_output, 2, "gemm_output");
  TORCH_CHECK(gemm_output.scalar_type() == at::kBFloat16, "gemm_output must be bfloat16");
  sched(ptr)->localReduce(gemm_output.data_ptr(), ctx(context), (int)stage_idx, current_stream(), true);
}

void combine(fptr_t ptr, fptr_t context, int64_t stage_idx) {
  sched(ptr)->combine(ctx(context), (int)stage_idx, current_stream());
}

void epilogue(fptr_t ptr, at::Tensor& output, fptr_t context) {
  check(output, 2, "output");
  TORCH_CHECK(output.scalar_type() == at::kBFloat16, "output must be bfloat16");
  sched(ptr)->epilogue(output.data_ptr(), ctx(context), current_stream());
}

void epilogue_fused(fptr_t ptr, at::Tensor& output, const std::optional<at::Tensor>& shared, fptr_t context) {
  check(output, 2, "output");
  TORCH_CHECK(output.scalar_type() == at::kBFloat16, "output must be bfloat16");
  sched(ptr)->epilogue(output.data_ptr(), ctx(context), current_stream(),
                       shared.has_value() ? shared->data_ptr() : nullptr, false);
}

void reduce_single_rank(fptr_t ptr, const at::Tensor& gemm_output, at::Tensor& output,
                        const std::optional<at::Tensor>& shared, fptr_t context) {
  check(gemm_output, 2, "gemm_output");
  check(output, 2, "output");
  sched(ptr)->reduceSingleRank(gemm_output.data_ptr(), output.data_ptr(),
                               shared.has_value() ? shared->data_ptr() : nullptr, ctx(context), current_stream());
}

// fp32 [gemm rows] gate weight of every GEMM row (a view into the context's workspace: valid until the context goes)
at::Tensor gemm_row_weights(fptr_t ptr, fptr_t context) {
  auto& c = ctx(context);
  float* w = sched(ptr)->gemmRowWeights(c, current_stream());
  const int64_t n = std::max<int64_t>(sched(ptr)->gemm_bound(c), 1);
  return at::from_blob(w, {n}, at::TensorOptions().device(at::kCUDA, at::cuda::current_device()).dtype(at::kFloat));
}

void check_status(fptr_t ptr, fptr_t context) { sched(ptr)->checkStatus(ctx(context), current_stream()); }

void register_scheduler_ops(torch::Library& m) {
  m.def("eps_create", &create);
  m.def("eps_destroy", &destroy);
  m.def("eps_get_context", &get_context);
  m.def("eps_destroy_context", &destroy_context);
  m.def("eps_get_workspace_size_context", &get_workspace_size_context);
  m.def("eps_set_ws_context", &set_ws_context);
  m.def("eps_rendezvous", &rendezvous);
  m.def("eps_plan", &plan);
  m.def("eps_prologue", &prologue);
  m.def("eps_dispatch", &dispatch);
  m.def("eps_gemm_expand", &gemm_expand);
  m.def("eps_local_reduce", &local_reduce);
  m.def("eps_combine", &combine);
  m.def("eps_epilogue", &epilogue);
  // additions for the FP8 path
  m.def("eps_create_fp8", &create_fp8);
  m.def("eps_rendezvous_async", &rendezvous_async);
  m.def("eps_plan_fp8", &plan_fp8);
  m.def("eps_prologue_fp8", &prologue_fp8);
  m.def("eps_local_reduce_weighted", &local_reduce_weighted);
  m.def("eps_epilogue_fused", &epilogue_fused);
  m.def("eps_reduce_single_rank", &reduce_single_rank);
  m.def("eps_gemm_row_weights", &gemm_row_weights);
  m.def("eps_check_status", &check_status);
}

}  // namespace

TORCH_LIBRARY(scheduler, m) { register_scheduler_ops(m); }
TORCH_LIBRARY(eps, m) { register_scheduler_ops(m); }

EPSB_REGISTER_EXTENSION(libscheduler_)
