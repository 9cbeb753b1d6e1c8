// libutils_.so: `utils.topk_sigmoid` and `utils.rms_norm_op` with the reference's argument lists
// (src/utils/bindings/th_topk_sigmoid.cu:13-67, th_rms_norm.cu:13-40).
#include "host_common.hpp"

namespace {

using namespace epsb_host;

// bf16 scores, fp32 bias and scales, int32 indices (the reference also takes int64 indices; not part of this build)
void topk_sigmoid_op(at::Tensor scores, at::Tensor bias, at::Tensor expert_scales, at::Tensor expert_indices,
                     int64_t num_tokens, int64_t num_experts, int64_t num_expert_groups, int64_t topk_groups,
                     int64_t topk, double route_scale) {
  check(scores, 2, "scores");
  check(bias, 1, "bias");
  check(expert_scales, 2, "expert_scales");
  check(expert_indices, 2, "expert_indices");
  TORCH_CHECK(scores.scalar_type() == at::kBFloat16 || scores.scalar_type() == at::kFloat,
              "scores must be bfloat16 or float32");
  TORCH_CHECK(bias.scalar_type() == at::kFloat, "bias must be float32");
  TORCH_CHECK(expert_scales.scalar_type() == at::kFloat, "expert_scales must be float32");
  if (expert_indices.scalar_type() != at::kInt) throw std::runtime_error("Not supported expert_indices data type.");
  TORCH_CHECK(scores.size(0) >= num_tokens && scores.size(1) == num_experts && bias.numel() == num_experts,
              "scores must be [num_tokens, num_experts] and bias [num_experts]");
  TORCH_CHECK(expert_scales.size(0) >= num_tokens && expert_scales.size(1) == topk &&
                  expert_indices.size(0) >= num_tokens && expert_indices.size(1) == topk,
              "expert_scales and expert_indices must be [num_tokens, topk]");
  raise_if(epsb_router_topk_sigmoid(scores.data_ptr(), scores.scalar_type() == at::kBFloat16, bias.data_ptr<float>(),
                                    (int)num_tokens, (int)num_experts, (int)num_expert_groups, (int)topk_groups,
                                    (int)topk, (float)route_scale, (int)num_experts,
                                    expert_indices.data_ptr<int32_t>(), expert_scales.data_ptr<float>(),
                                    current_stream()));
}

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
  TORCH_CHECK(output.sizes() == input.sizes() && scale.numel() == input.size(1), "shapes of output / input / scale differ");
  raise_if(epsb_rms_norm(output.data_ptr(), input.data_ptr(), scale.data_ptr(), (float)eps, input.size(0), input.size(1),
                         current_stream()));
}

}  // namespace

TORCH_LIBRARY(utils, m) {
  m.def("topk_sigmoid", &topk_sigmoid_op);
  m.def("rms_norm_op", &rms_norm_op);
}

EPSB_REGISTER_EXTENSION(libutils_)
