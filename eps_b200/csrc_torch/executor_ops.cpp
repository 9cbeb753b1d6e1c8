// libexecutor_.so: the executor operators under namespace `executor`, with the reference's names and argument lists
// (src/executor/bindings/aok_grouped_gemm_ops.cu:18-86, silu_ops.cu:14-43).  `aok_run` is the reference's bf16 x bf16
// grouped GEMM; the *_fp8 ops and per_token_group_quant_fp8 are additions for the FP8 path (no counterpart among the
// reference's ops; its FP8 quantiser is C++ only, src/quant/fp8.cuh:71-72).
#include "executor.hpp"
#include "host_common.hpp"

namespace {

using namespace epsb_host;

struct GemmHandle {
  AokGroupedGemm bf16;
  Fp8GroupedGemm fp8;
  GemmHandle(int n, int sm) : bf16(n, sm), fp8(n, sm) {}
};

GemmHandle* handle(fptr_t p) {
  TORCH_CHECK(p != 0, "executor handle is null");
  return reinterpret_cast<GemmHandle*>(p);
}

fptr_t aok_create(int64_t num_local_experts, int64_t sm_count) {
  // the reference passes the device's SM count; any count >= the device's means "all"
  return reinterpret_cast<fptr_t>(new GemmHandle((int)num_local_experts, (int)sm_count));
}
void aok_destroy(fptr_t ptr) { delete reinterpret_cast<GemmHandle*>(ptr); }
int64_t aok_get_workspace_size(fptr_t ptr, int64_t cols, int64_t max_num_tokens) {
  return (int64_t)handle(ptr)->bf16.getWorkspaceSize(cols, max_num_tokens, handle(ptr)->bf16.num_local_experts());
}

void check_gemm_shapes(const GemmHandle* h, const at::Tensor& A, const at::Tensor& B, const at::Tensor& C,
                       const at::Tensor& exclusive_sum, int64_t max_num_tokens, int64_t c_cols) {
  check(A, 2, "A");
  check(B, 3, "B");
  check(C, 2, "C");
  check(exclusive_sum, 1, "exclusive_sum");
  TORCH_CHECK(exclusive_sum.scalar_type() == at::kInt, "exclusive_sum must be of type kInt32");
  TORCH_CHECK(B.size(0) == h->bf16.num_local_experts(), "B holds ", B.size(0), " experts, the executor was created for ",
              h->bf16.num_local_experts());
  TORCH_CHECK(exclusive_sum.numel() == B.size(0) + 1, "exclusive_sum must have num_local_experts + 1 entries");
  TORCH_CHECK(A.size(1) == B.size(2), "A has K = ", A.size(1), " but B has K = ", B.size(2));
  TORCH_CHECK(C.size(1) == c_cols, "C has ", C.size(1), " columns, expected ", c_cols);
  TORCH_CHECK(max_num_tokens >= 0 && max_num_tokens <= A.size(0) && max_num_tokens <= C.size(0), "max_num_tokens ",
              max_num_tokens, " exceeds the rows of A (", A.size(0), ") or C (", C.size(0), ")");
}

void check_fp8_scales(const at::Tensor& A, const at::Tensor& A_scale, const at::Tensor& B, const at::Tensor& B_scale) {
  check(A_scale, 2, "A_scale");
  check(B_scale, 3, "B_scale");
  TORCH_CHECK(is_fp8_codes(A) && is_fp8_codes(B), "A and B must hold e4m3 codes (uint8 or float8_e4m3fn)");
  TORCH_CHECK(A_scale.scalar_type() == at::kFloat && B_scale.scalar_type() == at::kFloat, "scales must be float32");
  TORCH_CHECK(A.size(1) % 128 == 0 && B.size(1) % 128 == 0, "K and N must be multiples of 128");
  TORCH_CHECK(A_scale.size(0) >= A.size(0) && A_scale.size(1) == A.size(1) / 128, "A_scale must be [rows, K/128]");
  TORCH_CHECK(B_scale.size(0) == B.size(0) && B_scale.size(1) == B.size(1) / 128 && B_scale.size(2) == B.size(2) / 128,
              "B_scale must be [experts, N/128, K/128]");
}

void aok_run(fptr_t ptr, const at::Tensor& A, const at::Tensor& B, at::Tensor& C, const at::Tensor& exclusive_sum,
             int64_t num_tokens_hint, int64_t max_num_tokens, at::Tensor& /*ws*/) {
  auto* h = handle(ptr);
  check_gemm_shapes(h, A, B, C, exclusive_sum, max_num_tokens, B.size(1));
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16 && C.scalar_type() == at::kBFloat16,
              "A, B and C must be bfloat16");
  GemmInterface::RunParams p{};
  p.A = A.data_ptr();
  p.B = B.data_ptr();
  p.C = C.data_ptr();
  p.total_rows_before_expert = exclusive_sum.data_ptr<int32_t>();
  p.gemm_n = B.size(1);
  p.gemm_k = B.size(2);
  p.num_experts_per_stage = (int)B.size(0);
  p.max_num_tokens = max_num_tokens;
  p.total_rows = num_tokens_hint;
  h->bf16.run(p, current_stream());
}

void run_fp8(int mode, fptr_t ptr, const at::Tensor& A, const at::Tensor& A_scale, const at::Tensor& B,
             const at::Tensor& B_scale, at::Tensor& C, const std::optional<at::Tensor>& C_scale,
             const std::optional<at::Tensor>& row_weights, const at::Tensor& exclusive_sum, int64_t max_num_tokens,
             const std::optional<at::Tensor>& status) {
  auto* h = handle(ptr);
  const int64_t N = B.size(1);
  check_gemm_shapes(h, A, B, C, exclusive_sum, max_num_tokens, mode == EPSB_GEMM_GATEUP ? N / 2 : N);
  check_fp8_scales(A, A_scale, B, B_scale);
  float* c_s = nullptr;
  if (mode == EPSB_GEMM_GATEUP) {
    TORCH_CHECK(C_scale.has_value(), "the gate/up mode needs C_scale");
    TORCH_CHECK(is_fp8_codes(C), "C must hold e4m3 codes in the gate/up mode");
    TORCH_CHECK(C_scale->scalar_type() == at::kFloat && C_scale->size(0) >= max_num_tokens &&
                    C_scale->size(1) == N / 256,
                "C_scale must be float32 [rows, I/128]");
    c_s = C_scale->data_ptr<float>();
  } else {
    TORCH_CHECK(C.scalar_type() == at::kBFloat16, "C must be bfloat16");
  }
  const float* rw = nullptr;
  if (row_weights.has_value()) {
    TORCH_CHECK(row_weights->scalar_type() == at::kFloat && row_weights->numel() >= max_num_tokens,
                "row_weights must be float32 [rows]");
    rw = row_weights->data_ptr<float>();
  }
  raise_if(epsb_grouped_gemm_fp8(mode, A.data_ptr(), A_scale.data_ptr<float>(), B.data_ptr(), B_scale.data_ptr<float>(),
                                 exclusive_sum.data_ptr<int32_t>(), (int)B.size(0), max_num_tokens, N, B.size(2),
                                 C.data_ptr(), c_s, rw, status.has_value() ? status->data_ptr<int32_t>() : nullptr,
                                 h->fp8.sm_count(),  // the executor's sm_count, as in the reference
                                 current_stream()));
}

void aok_run_fp8(fptr_t ptr, const at::Tensor& A, const at::Tensor& A_scale, const at::Tensor& B,
                 const at::Tensor& B_scale, at::Tensor& C, const at::Tensor& exclusive_sum, int64_t /*num_tokens_hint*/,
                 int64_t max_num_tokens, at::Tensor& /*ws*/) {
  run_fp8(EPSB_GEMM_PLAIN, ptr, A, A_scale, B, B_scale, C, std::nullopt, std::nullopt, exclusive_sum, max_num_tokens,
          std::nullopt);
}

// gate/up GEMM + SwiGLU + 1x128 requantisation: C e4m3 [rows, I], C_scale fp32 [rows, I/128]
void aok_run_gate_up_fp8(fptr_t ptr, const at::Tensor& A, const at::Tensor& A_scale, const at::Tensor& B,
                         const at::Tensor& B_scale, at::Tensor& C, at::Tensor& C_scale, const at::Tensor& exclusive_sum,
                         int64_t max_num_tokens, const std::optional<at::Tensor>& status) {
  run_fp8(EPSB_GEMM_GATEUP, ptr, A, A_scale, B, B_scale, C, C_scale, std::nullopt, exclusive_sum, max_num_tokens, status);
}

// down GEMM whose rows leave multiplied by their gate weight (fp32): C bf16 [rows, N]
void aok_run_down_fp8(fptr_t ptr, const at::Tensor& A, const at::Tensor& A_scale, const at::Tensor& B,
                      const at::Tensor& B_scale, at::Tensor& C, const std::optional<at::Tensor>& row_weights,
                      const at::Tensor& exclusive_sum, int64_t max_num_tokens, const std::optional<at::Tensor>& status) {
  run_fp8(EPSB_GEMM_DOWN, ptr, A, A_scale, B, B_scale, C, std::nullopt, row_weights, exclusive_sum, max_num_tokens,
          status);
}

void silu_run(const at::Tensor& gate_up, at::Tensor& result, const at::Tensor& exclusive_sum,
              int64_t /*num_tokens_hint*/) {
  check(gate_up, 2, "gate_up");
  check(result, 2, "result");
  check(exclusive_sum, 1, "exclusive_sum");
  TORCH_CHECK(exclusive_sum.scalar_type() == at::kInt, "exclusive_sum must be of type kInt32");
  TORCH_CHECK(gate_up.scalar_type() == at::kBFloat16, "gate_up must be bfloat16");
  TORCH_CHECK(result.size(0) >= gate_up.size(0) && result.size(1) * 2 == gate_up.size(1), "result must be [rows, I]");
  raise_if(epsb_silu_run(gate_up.data_ptr(), result.data_ptr(), exclusive_sum.data_ptr<int32_t>(),
                         (int)exclusive_sum.size(0) - 1, gate_up.size(0), gate_up.size(1) / 2, current_stream()));
}

void per_token_group_quant_fp8(const at::Tensor& x, at::Tensor& q, at::Tensor& scales, int64_t div_mode) {
  check(x, 2, "x");
  check(q, 2, "q");
  check(scales, 2, "scales");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16, "x must be bfloat16");
  TORCH_CHECK(is_fp8_codes(q) && q.size(0) == x.size(0) && q.size(1) == x.size(1), "q must be e4m3 codes like x");
  TORCH_CHECK(scales.scalar_type() == at::kFloat && scales.size(0) == x.size(0) && scales.size(1) * 128 == x.size(1),
              "scales must be float32 [rows, cols/128]");
  raise_if(epsb_quant_1x128(x.data_ptr(), x.size(0), x.size(1), q.data_ptr(), scales.data_ptr<float>(), (int)div_mode,
                            current_stream()));
}

}  // namespace

TORCH_LIBRARY(executor, m) {
  m.def("aok_create", &aok_create);
  m.def("aok_get_workspace_size", &aok_get_workspace_size);
  m.def("aok_run", &aok_run);
  m.def("aok_destroy", &aok_destroy);
  m.def("silu_run", &silu_run);
  // additions for the FP8 path
  m.def("aok_run_fp8", &aok_run_fp8);
  m.def("aok_run_gate_up_fp8", &aok_run_gate_up_fp8);
  m.def("aok_run_down_fp8", &aok_run_down_fp8);
  m.def("per_token_group_quant_fp8", &per_token_group_quant_fp8);
}

EPSB_REGISTER_EXTENSION(libexecutor_)
