// torch op registration of the executor operators (and the router of the utils library) over the eps_b200 C ABI.
//
// Mirrors the reference's src/executor/bindings/{bindings.cpp,aok_grouped_gemm_ops.cu,silu_ops.cu}: the same
// namespace (`executor`), op names and argument lists, registered with TORCH_LIBRARY and loadable with
// torch.ops.load_library(), plus a PyInit stub like the reference's REGISTER_EXTENSION (src/registration.h:19-26).
// The FP8 entry points are additions; `aok_run` (bf16 x bf16, sm_90a in the reference) reports that it is not
// part of this build.
#include <Python.h>

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <torch/library.h>

#include <stdexcept>

#include "../../include/eps_b200.h"

namespace {

using fptr_t = int64_t;

struct GemmHandle {
  int num_local_experts;
  int sm_count;
};

void check(const at::Tensor& t, int64_t dim, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.dim() == dim, name, " must have ", dim, " dimensions");
}

void raise_if(int rc) {
  if (rc != EPSB_OK) throw std::runtime_error(epsb_last_error());
}

fptr_t aok_create(int64_t num_local_experts, int64_t sm_count) {
  return reinterpret_cast<fptr_t>(new GemmHandle{(int)num_local_experts, (int)sm_count});
}

void aok_destroy(fptr_t ptr) { delete reinterpret_cast<GemmHandle*>(ptr); }

int64_t aok_get_workspace_size(fptr_t, int64_t, int64_t) { return 0; }  // the tile list is built inside the kernel

void aok_run(fptr_t, const at::Tensor&, const at::Tensor&, at::Tensor&, const at::Tensor&, int64_t, int64_t, at::Tensor&) {
  throw std::runtime_error(
      "aok_run: the bf16 x bf16 grouped GEMM of the reference is not part of this build; use aok_run_fp8 with e4m3 "
      "operands and their 1x128 / 128x128 scales");
}

void aok_run_fp8(fptr_t ptr, const at::Tensor& A, const at::Tensor& A_scale, const at::Tensor& B,
                 const at::Tensor& B_scale, at::Tensor& C, const at::Tensor& exclusive_sum, int64_t /*num_tokens_hint*/,
                 int64_t max_num_tokens, at::Tensor& /*ws*/) {
  check(A, 2, "A");
  check(B, 3, "B");
  check(C, 2, "C");
  check(A_scale, 2, "A_scale");
  check(B_scale, 3, "B_scale");
  check(exclusive_sum, 1, "exclusive_sum");
  TORCH_CHECK(exclusive_sum.scalar_type() == at::kInt, "exclusive_sum must be of type kInt32");
  TORCH_CHECK(C.scalar_type() == at::kBFloat16, "C must be bfloat16");
  auto* h = reinterpret_cast<GemmHandle*>(ptr);
  TORCH_CHECK(h == nullptr || h->num_local_experts == B.size(0), "B holds ", B.size(0), " experts, executor has ",
              h ? h->num_local_experts : 0);
  raise_if(epsb_grouped_gemm_fp8(EPSB_GEMM_PLAIN, A.data_ptr(), A_scale.data_ptr<float>(), B.data_ptr(),
                                 B_scale.data_ptr<float>(), exclusive_sum.data_ptr<int32_t>(), (int)B.size(0),
                                 max_num_tokens, B.size(1), B.size(2), C.data_ptr(), nullptr, nullptr, nullptr,
                                 h != nullptr ? h->sm_count : 0,  // the executor's sm_count, as in the reference
                                 at::cuda::getCurrentCUDAStream().stream()));
}

void silu_run(const at::Tensor& gate_up, at::Tensor& result, const at::Tensor& exclusive_sum, int64_t /*num_tokens_hint*/) {
  check(gate_up, 2, "gate_up");
  check(result, 2, "result");
  check(exclusive_sum, 1, "exclusive_sum");
  TORCH_CHECK(exclusive_sum.scalar_type() == at::kInt, "exclusive_sum must be of type kInt32");
  TORCH_CHECK(gate_up.scalar_type() == at::kBFloat16, "gate_up must be bfloat16");
  raise_if(epsb_silu_run(gate_up.data_ptr(), result.data_ptr(), exclusive_sum.data_ptr<int32_t>(),
                         (int)exclusive_sum.size(0) - 1, gate_up.size(0), gate_up.size(1) / 2,
                         at::cuda::getCurrentCUDAStream().stream()));
}

// per_token_group_quant_fp8 (reference: C++ only, src/quant/fp8.cuh:71-72), dense form.
void per_token_group_quant_fp8(const at::Tensor& x, at::Tensor& q, at::Tensor& scales, int64_t div_mode) {
  check(x, 2, "x");
  check(q, 2, "q");
  check(scales, 2, "scales");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16, "x must be bfloat16");
  raise_if(epsb_quant_1x128(x.data_ptr(), x.size(0), x.size(1), q.data_ptr(), scales.data_ptr<float>(), (int)div_mode,
                            at::cuda::getCurrentCUDAStream().stream()));
}

// utils.topk_sigmoid with the reference's argument list (src/utils/bindings/th_topk_sigmoid.cu:13-62): bf16 scores,
// fp32 bias and scales, int32 indices.  int64 indices (which the reference also takes) are not part of this build.
void topk_sigmoid_op(at::Tensor scores, at::Tensor bias, at::Tensor expert_scales, at::Tensor expert_indices,
                     int64_t num_tokens, int64_t num_experts, int64_t num_expert_groups, int64_t topk_groups,
                     int64_t topk, double route_scale) {
  check(scores, 2, "scores");
  check(bias, 1, "bias");
  check(expert_scales, 2, "expert_scales");
  check(expert_indices, 2, "expert_indices");
  TORCH_CHECK(scores.scalar_type() == at::kBFloat16, "scores must be bfloat16");
  TORCH_CHECK(bias.scalar_type() == at::kFloat, "bias must be float32");
  TORCH_CHECK(expert_scales.scalar_type() == at::kFloat, "expert_scales must be float32");
  if (expert_indices.scalar_type() != at::kInt) throw std::runtime_error("Not supported expert_indices data type.");
  raise_if(epsb_router_topk_sigmoid(scores.data_ptr(), 1, bias.data_ptr<float>(), (int)num_tokens, (int)num_experts,
                                    (int)num_expert_groups, (int)topk_groups, (int)topk, (float)route_scale,
                                    (int)num_experts, expert_indices.data_ptr<int32_t>(),
                                    expert_scales.data_ptr<float>(), at::cuda::getCurrentCUDAStream().stream()));
}

// utils.rms_norm_op with the reference's argument list (src/utils/bindings/th_rms_norm.cu:13-35)
void rms_norm_op(at::Tensor output, at::Tensor input, at::Tensor scale, double eps) {
  if (output.dim() != 2 || input.dim() != 2)
    throw std::runtime_error("output and input dim must be 2 but got " + std::to_string(output.dim()) + " and " +
                             std::to_string(input.dim()));
  check(output, 2, "output");
  check(input, 2, "input");
  check(scale, 1, "scale");
  TORCH_CHECK(output.scalar_type() == at::kBFloat16 && input.scalar_type() == at::kBFloat16 &&
                  scale.scalar_type() == at::kBFloat16,
              "output, input and scale must be bfloat16");
  raise_if(epsb_rms_norm(output.data_ptr(), input.data_ptr(), scale.data_ptr(), (float)eps, input.size(0),
                         input.size(1), at::cuda::getCurrentCUDAStream().stream()));
}

}  // namespace

TORCH_LIBRARY(utils, m) {
  m.def("topk_sigmoid", &topk_sigmoid_op);
  m.def("rms_norm_op", &rms_norm_op);
}

TORCH_LIBRARY(executor, m) {
  m.def("aok_create", &aok_create);
  m.def("aok_get_workspace_size", &aok_get_workspace_size);
  m.def("aok_run", &aok_run);
  m.def("aok_run_fp8", &aok_run_fp8);
  m.def("aok_destroy", &aok_destroy);
  m.def("silu_run", &silu_run);
  m.def("per_token_group_quant_fp8", &per_token_group_quant_fp8);
}

PyMODINIT_FUNC PyInit_libexecutor_() {
  static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, "libexecutor_", nullptr, 0, nullptr};
  return PyModule_Create(&module);
}
