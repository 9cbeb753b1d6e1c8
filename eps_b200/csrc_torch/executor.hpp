// The executor contract types and their implementations over the eps_b200 C ABI.
//
// GemmInterface / ActivationInterface have the shape of the reference's contract types
// (src/scheduler/gemm_executor_interface.cuh:3-48): the same RunParams fields in the same order and the same virtual
// methods, so that code written against `GemmInterface* g; g->run(params, stream)` compiles and links against these
// classes unchanged.  AokGroupedGemm is the reference's executor of that name (src/executor/aok_grouped_gemm.cu:12-37:
// bf16 x bf16 -> bf16, fp32 accumulate); Fp8GroupedGemm fills the A_scales / weight_scales slots the contract already
// has with the FP8 block-scaled path.  Errors are std::runtime_error, as in the reference.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/eps_b200.h"

namespace epsb_host {

class GemmInterface {
 public:
  struct RunParams {
    const void* A;
    const void* A_scales;
    const void* B;
    const void* weight_scales;
    const void* biases;
    void* C;
    const int* total_rows_before_expert;
    int64_t total_rows;
    int64_t gemm_n;
    int64_t gemm_k;
    int num_experts_per_stage;
    int expert_begin;
    char* ws;
    int64_t max_num_tokens;
  };
  virtual void run(RunParams p, cudaStream_t stream) = 0;
  virtual size_t output_type_bytes() = 0;
  virtual size_t getWorkspaceSize(int64_t cols, int64_t max_num_tokens, int64_t local_num_experts) = 0;
  virtual ~GemmInterface() = default;
};

class ActivationInterface {
 public:
  struct RunParams {
    void* activation;
    void* gate_up;
    const int* exclusive_sum;
    int num_experts_per_stage;
    int64_t inter_size_x2;
    void* gate;
    void* up;
    int64_t inter_size;
    int64_t num_tokens_hint;
  };
  virtual void run(RunParams p, cudaStream_t stream) = 0;
  virtual ~ActivationInterface() = default;
};

inline void executor_raise_if(int rc) {
  if (rc != EPSB_OK) throw std::runtime_error(epsb_last_error());
}

// The tile list is built inside the kernels from total_rows_before_expert: no workspace, nothing read on the host.
class GroupedGemmBase : public GemmInterface {
 public:
  GroupedGemmBase(int num_local_experts, int sm_count) : num_local_experts_(num_local_experts), sm_count_(sm_count) {
    if (num_local_experts <= 0) throw std::runtime_error("num_local_experts must be positive");
    if (sm_count < 0) throw std::runtime_error("sm_count must not be negative");
  }
  size_t output_type_bytes() override { return 2; }
  size_t getWorkspaceSize(int64_t, int64_t, int64_t) override { return 0; }
  int num_local_experts() const { return num_local_experts_; }
  int sm_count() const { return sm_count_; }
  // device int32[4]; word 0 becomes non-zero if a bounded wait inside a kernel gave up
  void set_status(int32_t* status) { status_ = status; }

 protected:
  const int* window(const RunParams& p) const { return p.total_rows_before_expert + p.expert_begin; }
  int num_local_experts_, sm_count_;
  int32_t* status_ = nullptr;
};

// bf16 x bf16 -> bf16: for expert e of the stage, C[rows of e] = A[rows of e] * B[e]^T (B is [E, N, K], K contiguous).
class AokGroupedGemm : public GroupedGemmBase {
 public:
  using GroupedGemmBase::GroupedGemmBase;
  void run(RunParams p, cudaStream_t stream) override {
    if (p.biases != nullptr) throw std::runtime_error("biases are not supported");
    const char* B = static_cast<const char*>(p.B) + (int64_t)p.expert_begin * p.gemm_n * p.gemm_k * 2;
    executor_raise_if(epsb_grouped_gemm_bf16(p.A, B, window(p), p.num_experts_per_stage, p.max_num_tokens,
                                             p.total_rows > 0 ? p.total_rows : 0, p.gemm_n, p.gemm_k, p.C, status_,
                                             sm_count_, stream));
  }
};

// e4m3 x e4m3 with 1x128 (A_scales [rows, K/128]) and 128x128 (weight_scales [E, N/128, K/128]) fp32 scales -> bf16.
class Fp8GroupedGemm : public GroupedGemmBase {
 public:
  using GroupedGemmBase::GroupedGemmBase;
  void run(RunParams p, cudaStream_t stream) override {
    if (p.biases != nullptr) throw std::runtime_error("biases are not supported");
    if (p.A_scales == nullptr || p.weight_scales == nullptr)
      throw std::runtime_error("the FP8 grouped GEMM needs A_scales and weight_scales");
    const int64_t nb = p.gemm_n / 128, kb = p.gemm_k / 128;
    const char* B = static_cast<const char*>(p.B) + (int64_t)p.expert_begin * p.gemm_n * p.gemm_k;
    const float* bs = static_cast<const float*>(p.weight_scales) + (int64_t)p.expert_begin * nb * kb;
    executor_raise_if(epsb_grouped_gemm_fp8(EPSB_GEMM_PLAIN, p.A, static_cast<const float*>(p.A_scales), B, bs, window(p),
                                            p.num_experts_per_stage, p.max_num_tokens, p.gemm_n, p.gemm_k, p.C, nullptr,
                                            nullptr, status_, sm_count_, stream));
  }
};

// silu(gate) * up on ragged rows (reference Activation<T>, src/executor/activations.cu:173-205).
class SiluActivation : public ActivationInterface {
 public:
  void run(RunParams p, cudaStream_t stream) override {
    if (p.gate_up == nullptr) throw std::runtime_error("separate gate / up buffers are not supported: pass gate_up");
    executor_raise_if(epsb_silu_run(p.gate_up, p.activation, p.exclusive_sum, p.num_experts_per_stage, p.num_tokens_hint,
                                    p.inter_size_x2 / 2, stream));
  }
};

}  // namespace epsb_host
