// libexecutor_.so: the executor operators under namespace `executor`, with the reference's names and argument lists
// (src/executor/bindings/aok_grouped_gemm_ops.cu:18-86, silu_ops.cu:14-43).  `aok_run` is the reference's bf16 x bf16
// grouped GEMM; the *_fp8 ops and per_token_group_quant_fp8 are additions for the FP8 path (no counterpart among the
// reference's ops; its FP8 quantiser is C++ only, src/quant/fp8.cuh:71-72).
#include <memory>

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

// ---- the FFN executors over the contract types GemmExecutorInterface / SharedExpertsInterface / DenseGemmInterface /
// BatchedGemmInterface / DenseActivationInterface (no ops for them exist in the reference, which only declares the types)
struct FfnHandle {
  at::Tensor wgu, wgu_s, wd, wd_s;   // keeps the weights alive
  at::Tensor status;
  std::unique_ptr<Fp8GemmExecutor> routed;
  std::unique_ptr<Fp8SharedExperts> shared;
};

Fp8FfnWeights ffn_weights(const at::Tensor& wgu, const at::Tensor& wgu_s, const at::Tensor& wd, const at::Tensor& wd_s) {
  check(wgu, 3, "gate_up_weights");
  check(wgu_s, 3, "gate_up_scales");
  check(wd, 3, "down_weights");
  check(wd_s, 3, "down_scales");
  TORCH_CHECK(is_fp8_codes(wgu) && is_fp8_codes(wd), "weights must hold e4m3 codes (uint8 or float8_e4m3fn)");
  TORCH_CHECK(wgu_s.scalar_type() == at::kFloat && wd_s.scalar_type() == at::kFloat, "weight scales must be float32");
  const int64_t E = wgu.size(0), I2 = wgu.size(1), H = wgu.size(2);
  TORCH_CHECK(I2 % 256 == 0 && H % 128 == 0, "gate_up_weights must be [E, 2I, H] with I and H multiples of 128");
  TORCH_CHECK(wd.size(0) == E && wd.size(1) == H && wd.size(2) == I2 / 2, "down_weights must be [E, H, I]");
  TORCH_CHECK(wgu_s.size(0) == E && wgu_s.size(1) == I2 / 128 && wgu_s.size(2) == H / 128,
              "gate_up_scales must be [E, 2I/128, H/128]");
  TORCH_CHECK(wd_s.size(0) == E && wd_s.size(1) == H / 128 && wd_s.size(2) == I2 / 256,
              "down_scales must be [E, H/128, I/128]");
  return Fp8FfnWeights{wgu.data_ptr(), wgu_s.data_ptr<float>(), wd.data_ptr(), wd_s.data_ptr<float>(), H, I2 / 2, (int)E};
}

FfnHandle* ffn(fptr_t p) {
  TORCH_CHECK(p != 0, "FFN executor handle is null");
  return reinterpret_cast<FfnHandle*>(p);
}

fptr_t make_ffn(const at::Tensor& wgu, const at::Tensor& wgu_s, const at::Tensor& wd, const at::Tensor& wd_s,
                int64_t sm_count, bool shared) {
  auto h = std::make_unique<FfnHandle>();
  const Fp8FfnWeights w = ffn_weights(wgu, wgu_s, wd, wd_s);
  h->wgu = wgu, h->wgu_s = wgu_s, h->wd = wd, h->wd_s = wd_s;
  h->status = at::zeros({4}, wgu_s.options().dtype(at::kInt));
  if (shared) {
    h->shared = std::make_unique<Fp8SharedExperts>(w, (int)sm_count);
    h->shared->set_status(h->status.data_ptr<int32_t>());
  } else {
    h->routed = std::make_unique<Fp8GemmExecutor>(w, (int)sm_count);
    h->routed->set_status(h->status.data_ptr<int32_t>());
  }
  return reinterpret_cast<fptr_t>(h.release());
}

fptr_t gemm_executor_create(const at::Tensor& wgu, const at::Tensor& wgu_s, const at::Tensor& wd, const at::Tensor& wd_s,
                            int64_t sm_count) {
  return make_ffn(wgu, wgu_s, wd, wd_s, sm_count, false);
}
fptr_t shared_experts_create(const at::Tensor& wgu, const at::Tensor& wgu_s, const at::Tensor& wd,
                             const at::Tensor& wd_s, int64_t sm_count) {
  return make_ffn(wgu, wgu_s, wd, wd_s, sm_count, true);
}
void ffn_destroy(fptr_t p) { delete reinterpret_cast<FfnHandle*>(p); }
at::Tensor ffn_status(fptr_t p) { return ffn(p)->status; }

int64_t gemm_executor_get_workspace_size(fptr_t p, int64_t max_num_tokens) {
  TORCH_CHECK(ffn(p)->routed, "not a routed-experts executor");
  return (int64_t)ffn(p)->routed->getWorkspaceSize(max_num_tokens);
}
int64_t shared_experts_get_workspace_size(fptr_t p, int64_t num_tokens) {
  TORCH_CHECK(ffn(p)->shared, "not a shared-experts executor");
  return (int64_t)ffn(p)->shared->getWorkspaceSize((int)num_tokens);
}

void check_ffn_io(const FfnHandle* h, const at::Tensor& input, const at::Tensor& input_scales, const at::Tensor& output,
                  const at::Tensor& ws, int64_t rows, size_t need) {
  check(input, 2, "input");
  check(input_scales, 2, "input_scales");
  check(output, 2, "output");
  TORCH_CHECK(ws.is_cuda() && ws.is_contiguous(), "ws must be a contiguous CUDA tensor");
  const int64_t H = h->wgu.size(2);
  TORCH_CHECK(is_fp8_codes(input) && input.size(1) == H && input.size(0) >= rows, "input must be e4m3 codes [rows, H]");
  TORCH_CHECK(input_scales.scalar_type() == at::kFloat && input_scales.size(0) >= rows &&
                  input_scales.size(1) == H / 128,
              "input_scales must be float32 [rows, H/128]");
  TORCH_CHECK(output.scalar_type() == at::kBFloat16 && output.size(0) >= rows && output.size(1) == H,
              "output must be bfloat16 [rows, H]");
  TORCH_CHECK((size_t)ws.nbytes() >= need, "workspace holds ", ws.nbytes(), " bytes, ", need, " are needed");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(ws.data_ptr()) % 256 == 0, "the workspace must be 256-byte aligned");
}

void gemm_executor_run(fptr_t p, const at::Tensor& input, const at::Tensor& input_scales, at::Tensor& output,
                       const at::Tensor& exclusive_sum, int64_t num_stages, int64_t stage_idx, int64_t num_tokens_hint,
                       int64_t max_num_tokens, const std::optional<at::Tensor>& row_weights, at::Tensor& ws) {
  auto* h = ffn(p);
  TORCH_CHECK(h->routed, "not a routed-experts executor");
  check(exclusive_sum, 1, "exclusive_sum");
  TORCH_CHECK(exclusive_sum.scalar_type() == at::kInt && exclusive_sum.numel() == h->wgu.size(0) + 1,
              "exclusive_sum must be int32 [num_local_experts + 1]");
  check_ffn_io(h, input, input_scales, output, ws, max_num_tokens, h->routed->getWorkspaceSize(max_num_tokens));
  const float* rw = nullptr;
  if (row_weights.has_value()) {
    TORCH_CHECK(row_weights->scalar_type() == at::kFloat && row_weights->numel() >= max_num_tokens,
                "row_weights must be float32 [rows]");
    rw = row_weights->data_ptr<float>();
  }
  h->routed->set_row_weights(rw);
  GemmExecutorInterface::RunParams rp{input.data_ptr(), input_scales.data_ptr<float>(), output.data_ptr(),
                                      exclusive_sum.data_ptr<int32_t>(), (int)num_stages, num_tokens_hint, max_num_tokens};
  GemmExecutorInterface* ex = h->routed.get();   // through the contract type, as a caller of the reference would
  ex->run(rp, (int)stage_idx, ws.data_ptr(), current_stream());
}

void shared_experts_run(fptr_t p, const at::Tensor& input, const at::Tensor& input_scales, at::Tensor& output,
                        int64_t num_tokens, at::Tensor& ws) {
  auto* h = ffn(p);
  TORCH_CHECK(h->shared, "not a shared-experts executor");
  check_ffn_io(h, input, input_scales, output, ws, num_tokens, h->shared->getWorkspaceSize((int)num_tokens));
  SharedExpertsInterface::RunParams rp{input.data_ptr(), input_scales.data_ptr(), output.data_ptr(), (int)num_tokens};
  SharedExpertsInterface* ex = h->shared.get();
  ex->run(rp, ws.data_ptr(), current_stream());
}

void dense_gemm_fp8(const at::Tensor& A, const at::Tensor& A_scale, const at::Tensor& B, const at::Tensor& B_scale,
                    at::Tensor& C, int64_t sm_count) {
  check(A, 2, "A");
  check(B, 2, "B");
  check(C, 2, "C");
  check(A_scale, 2, "A_scale");
  check(B_scale, 2, "B_scale");
  TORCH_CHECK(is_fp8_codes(A) && is_fp8_codes(B), "A and B must hold e4m3 codes");
  TORCH_CHECK(A.size(1) == B.size(1) && A.size(1) % 128 == 0 && B.size(0) % 128 == 0, "A [M, K], B [N, K], K and N % 128 == 0");
  TORCH_CHECK(A_scale.scalar_type() == at::kFloat && A_scale.size(0) == A.size(0) && A_scale.size(1) == A.size(1) / 128,
              "A_scale must be float32 [M, K/128]");
  TORCH_CHECK(B_scale.scalar_type() == at::kFloat && B_scale.size(0) == B.size(0) / 128 && B_scale.size(1) == B.size(1) / 128,
              "B_scale must be float32 [N/128, K/128]");
  TORCH_CHECK(C.scalar_type() == at::kBFloat16 && C.size(0) == A.size(0) && C.size(1) == B.size(0), "C must be bfloat16 [M, N]");
  Fp8DenseGemm gemm((int)sm_count);
  DenseGemmInterface::RunParams rp{A.data_ptr(), A_scale.data_ptr(), B.data_ptr(), B_scale.data_ptr(), C.data_ptr(),
                                   B.size(0), B.size(1), nullptr, A.size(0)};
  DenseGemmInterface* g = &gemm;
  g->run(rp, current_stream());
  cuda_ok(cudaStreamSynchronize(current_stream()), "dense_gemm_fp8");   // the row bounds die with `gemm`
}

void batched_gemm_fp8(const at::Tensor& A, const at::Tensor& A_scale, const at::Tensor& B, const at::Tensor& B_scale,
                      at::Tensor& C, int64_t sm_count) {
  check(A, 3, "A");
  check(B, 3, "B");
  check(C, 3, "C");
  check(A_scale, 3, "A_scale");
  check(B_scale, 3, "B_scale");
  TORCH_CHECK(is_fp8_codes(A) && is_fp8_codes(B), "A and B must hold e4m3 codes");
  const int64_t G = A.size(0), M = A.size(1), K = A.size(2), N = B.size(1);
  TORCH_CHECK(B.size(0) == G && B.size(2) == K && K % 128 == 0 && N % 128 == 0, "A [G, M, K], B [G, N, K], K and N % 128 == 0");
  TORCH_CHECK(A_scale.scalar_type() == at::kFloat && A_scale.size(0) == G && A_scale.size(1) == M && A_scale.size(2) == K / 128,
              "A_scale must be float32 [G, M, K/128]");
  TORCH_CHECK(B_scale.scalar_type() == at::kFloat && B_scale.size(0) == G && B_scale.size(1) == N / 128 && B_scale.size(2) == K / 128,
              "B_scale must be float32 [G, N/128, K/128]");
  TORCH_CHECK(C.scalar_type() == at::kBFloat16 && C.size(0) == G && C.size(1) == M && C.size(2) == N, "C must be bfloat16 [G, M, N]");
  Fp8BatchedGemm gemm((int)sm_count);
  BatchedGemmInterface::RunParams rp{A.data_ptr(), A_scale.data_ptr(), B.data_ptr(), B_scale.data_ptr(), C.data_ptr(),
                                     M, N, K, M * K, N * K, M * N, K, K, N, (int)G, nullptr};
  BatchedGemmInterface* g = &gemm;
  g->run(rp, current_stream());
  cuda_ok(cudaStreamSynchronize(current_stream()), "batched_gemm_fp8");
}

void dense_silu_run(const at::Tensor& gate_up, at::Tensor& result) {
  check(gate_up, 2, "gate_up");
  check(result, 2, "result");
  TORCH_CHECK(gate_up.scalar_type() == at::kBFloat16 && result.scalar_type() == at::kBFloat16, "bfloat16 tensors");
  TORCH_CHECK(result.size(0) == gate_up.size(0) && result.size(1) * 2 == gate_up.size(1), "result must be [rows, I]");
  DenseSiluActivation act;
  DenseActivationInterface::RunParams rp{result.data_ptr(), gate_up.data_ptr(), gate_up.size(1), gate_up.size(0)};
  DenseActivationInterface* a = &act;
  a->run(rp, current_stream());
  cuda_ok(cudaStreamSynchronize(current_stream()), "dense_silu_run");
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
  // the FFN executors behind the reference's contract types (gemm_executor_interface.cuh:50-151)
  m.def("gemm_executor_create", &gemm_executor_create);
  m.def("gemm_executor_get_workspace_size", &gemm_executor_get_workspace_size);
  m.def("gemm_executor_run", &gemm_executor_run);
  m.def("shared_experts_create", &shared_experts_create);
  m.def("shared_experts_get_workspace_size", &shared_experts_get_workspace_size);
  m.def("shared_experts_run", &shared_experts_run);
  m.def("ffn_destroy", &ffn_destroy);
  m.def("ffn_status", &ffn_status);
  m.def("dense_gemm_fp8", &dense_gemm_fp8);
  m.def("batched_gemm_fp8", &batched_gemm_fp8);
  m.def("dense_silu_run", &dense_silu_run);
}

EPSB_REGISTER_EXTENSION(libexecutor_)
