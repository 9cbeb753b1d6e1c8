// The executor contract types and their implementations over the eps_b200 C ABI.
//
// GemmInterface / ActivationInterface have the shape of the reference's contract types
// (src/scheduler/gemm_executor_interface.cuh:3-48): the same RunParams fields in the same order and the same virtual
// methods, so that code written against `GemmInterface* g; g->run(params, stream)` compiles and links against these
// classes unchanged.  AokGroupedGemm is the reference's executor of that name (src/executor/aok_grouped_gemm.cu:12-37:
// bf16 x bf16 -> bf16, fp32 accumulate); Fp8GroupedGemm fills the A_scales / weight_scales slots the contract already
// has with the FP8 block-scaled path.  The other contract types of that header (GemmExecutorInterface,
// SharedExpertsInterface, DenseGemmInterface, BatchedGemmInterface, DenseActivationInterface), which the reference
// declares without an implementation, are implemented here on the FP8 kernels.  Errors are std::runtime_error, as in
// the reference.
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

// The remaining contract types of the reference's header (src/scheduler/gemm_executor_interface.cuh:50-151), field for
// field: the reference declares them and ships no implementation; the FP8 engine below implements each.
class DenseActivationInterface {
 public:
  struct RunParams {
    void* activation;
    void* gate_up;
    int64_t inter_size_x2;
    int64_t num_tokens;
  };
  virtual void run(RunParams p, cudaStream_t stream) = 0;
  virtual ~DenseActivationInterface() = default;
};

class GemmExecutorInterface {
 public:
  struct RunParams {
    const void* input;
    const float* input_scales;
    void* output;
    const int* exclusive_sum; /*[local_expert_end - local_expert_begin + 1]*/
    int num_stages;
    int64_t num_tokens_hint;
    int64_t max_num_tokens;
  };
  virtual size_t getWorkspaceSize(int64_t max_num_tokens) = 0;
  virtual void run(RunParams rp, int stage_idx, void* ws, cudaStream_t stream) = 0;
  virtual ~GemmExecutorInterface() = default;
};

class DenseGemmInterface {
 public:
  struct RunParams {
    const void* A;
    const void* A_scales;
    const void* B;
    const void* weight_scales;
    void* C;
    int64_t gemm_n;
    int64_t gemm_k;
    char* ws;
    int64_t num_tokens;
  };
  virtual void run(RunParams p, cudaStream_t stream) = 0;
  virtual size_t output_type_bytes() = 0;
  virtual size_t getWorkspaceSize(int64_t cols, int64_t num_tokens) = 0;
  virtual ~DenseGemmInterface() = default;
};

class SharedExpertsInterface {
 public:
  struct RunParams {
    const void* input;
    const void* input_scales;
    void* output;
    int num_tokens;
  };
  virtual size_t getWorkspaceSize(int num_tokens) = 0;
  virtual void run(RunParams rp, void* ws, cudaStream_t stream) = 0;
  virtual ~SharedExpertsInterface() = default;
};

class BatchedGemmInterface {
 public:
  struct RunParams {
    const void* A;
    const void* A_scales;
    const void* B;
    const void* weight_scales;
    void* C;
    int64_t M;         // per gemm
    int64_t N;         // per gemm
    int64_t K;         // per gemm
    int64_t A_stride;  // A move to next gemm
    int64_t B_stride;  // B move to next gemm
    int64_t C_stride;  // C move to next gemm
    int64_t lda;       // A move to next row
    int64_t ldb;       // B move to next row
    int64_t ldc;       // C move to next row
    int num_gemms;
    char* ws;
  };
  virtual void run(RunParams rp, cudaStream_t stream) = 0;
  virtual size_t output_type_bytes() = 0;
  virtual size_t getWorkspaceSize(RunParams rp) = 0;
  virtual ~BatchedGemmInterface() = default;
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

// Row bounds [0, n, 2n, ...] on the device for the dense and batched forms: the grouped kernels read every row range
// from device memory, so a dense problem is one "expert" whose range the host writes here (an 8-byte copy on the
// stream; the host vector is pageable, so the copy is staged before the call returns).
class DeviceRowBounds {
 public:
  explicit DeviceRowBounds(int max_entries) : cap_(max_entries) {
    if (cudaMalloc(&dev_, sizeof(int) * (size_t)max_entries) != cudaSuccess)
      throw std::runtime_error("cudaMalloc of the row bounds failed");
  }
  DeviceRowBounds(const DeviceRowBounds&) = delete;
  DeviceRowBounds& operator=(const DeviceRowBounds&) = delete;
  ~DeviceRowBounds() { cudaFree(dev_); }
  // bounds[i] = i * rows for i in [0, parts]
  const int* uniform(int parts, int64_t rows, cudaStream_t stream) {
    if (parts + 1 > cap_) throw std::runtime_error("too many row ranges");
    if (rows < 0 || rows * parts > 0x7fffffffll) throw std::runtime_error("row count out of range");
    int host[kMaxParts + 1];
    if (parts > kMaxParts) throw std::runtime_error("too many row ranges");
    for (int i = 0; i <= parts; i++) host[i] = (int)(rows * i);
    if (cudaMemcpyAsync(dev_, host, sizeof(int) * (size_t)(parts + 1), cudaMemcpyHostToDevice, stream) != cudaSuccess)
      throw std::runtime_error("copy of the row bounds failed");
    return dev_;
  }
  static constexpr int kMaxParts = 1024;

 private:
  int* dev_ = nullptr;
  int cap_;
};

inline size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

// One expert's (or one stage of experts') FFN on FP8 rows: gate/up GEMM + SwiGLU + 1x128 requantisation into the
// workspace, then the down GEMM (optionally x the row's gate weight) -> bf16.  Weights: gate_up [E, 2I, H] e4m3 (gate
// rows first) with scales [E, 2I/128, H/128]; down [E, H, I] with scales [E, H/128, I/128].
struct Fp8FfnWeights {
  const void* gate_up;
  const float* gate_up_scales;
  const void* down;
  const float* down_scales;
  int64_t hidden, inter;
  int num_experts;
};

inline size_t fp8_ffn_workspace(int64_t rows, int64_t inter) {
  return align256((size_t)rows * (size_t)inter) + align256((size_t)rows * (size_t)(inter / 128) * sizeof(float));
}

inline void fp8_ffn_run(const Fp8FfnWeights& w, int expert_begin, int num_experts, const void* input,
                        const float* input_scales, const int* bounds, int64_t max_rows, void* ws, void* output,
                        const float* row_weights, int32_t* status, int sm_count, cudaStream_t stream) {
  if (w.hidden % 128 != 0 || w.inter % 128 != 0) throw std::runtime_error("hidden and inter must be multiples of 128");
  if (ws == nullptr && max_rows > 0) throw std::runtime_error("the FFN needs its workspace");
  char* act = static_cast<char*>(ws);
  float* act_s = reinterpret_cast<float*>(act + align256((size_t)max_rows * (size_t)w.inter));
  const int64_t gu = 2 * w.inter * w.hidden, gus = (2 * w.inter / 128) * (w.hidden / 128);
  const int64_t dn = w.hidden * w.inter, dns = (w.hidden / 128) * (w.inter / 128);
  executor_raise_if(epsb_grouped_gemm_fp8(
      EPSB_GEMM_GATEUP, input, input_scales, static_cast<const char*>(w.gate_up) + expert_begin * gu,
      w.gate_up_scales + expert_begin * gus, bounds, num_experts, max_rows, 2 * w.inter, w.hidden, act, act_s, nullptr,
      status, sm_count, stream));
  executor_raise_if(epsb_grouped_gemm_fp8(EPSB_GEMM_DOWN, act, act_s, static_cast<const char*>(w.down) + expert_begin * dn,
                                          w.down_scales + expert_begin * dns, bounds, num_experts, max_rows, w.hidden,
                                          w.inter, output, nullptr, row_weights, status, sm_count, stream));
}

// The routed experts of a rank, stage by stage (reference contract GemmExecutorInterface; the scheduler hands it the
// rows in expert order and their exclusive_sum): stage s computes experts [s * E/S, (s+1) * E/S).
class Fp8GemmExecutor : public GemmExecutorInterface {
 public:
  Fp8GemmExecutor(Fp8FfnWeights w, int sm_count) : w_(w), sm_count_(sm_count) {
    if (w.num_experts <= 0) throw std::runtime_error("num_experts must be positive");
    if (sm_count < 0) throw std::runtime_error("sm_count must not be negative");
  }
  size_t getWorkspaceSize(int64_t max_num_tokens) override { return fp8_ffn_workspace(max_num_tokens, w_.inter); }
  void run(RunParams rp, int stage_idx, void* ws, cudaStream_t stream) override {
    if (rp.num_stages <= 0 || w_.num_experts % rp.num_stages != 0 || stage_idx < 0 || stage_idx >= rp.num_stages)
      throw std::runtime_error("Invalid num_stages: " + std::to_string(rp.num_stages) +
                               " for local_num_experts: " + std::to_string(w_.num_experts));
    const int per = w_.num_experts / rp.num_stages;
    fp8_ffn_run(w_, stage_idx * per, per, rp.input, rp.input_scales, rp.exclusive_sum + stage_idx * per,
                rp.max_num_tokens, ws, rp.output, row_weights_, status_, sm_count_, stream);
  }
  // fp32 [rows]: every output row leaves multiplied by its gate weight (nullptr: not)
  void set_row_weights(const float* w) { row_weights_ = w; }
  void set_status(int32_t* status) { status_ = status; }

 private:
  Fp8FfnWeights w_;
  int sm_count_;
  const float* row_weights_ = nullptr;
  int32_t* status_ = nullptr;
};

// The shared expert: the same FFN on all of a rank's tokens (one "expert" whose rows are [0, num_tokens)).
class Fp8SharedExperts : public SharedExpertsInterface {
 public:
  Fp8SharedExperts(Fp8FfnWeights w, int sm_count) : w_(w), sm_count_(sm_count), bounds_(2) {
    if (w.num_experts != 1) throw std::runtime_error("the shared expert is one FFN");
  }
  size_t getWorkspaceSize(int num_tokens) override { return fp8_ffn_workspace(num_tokens, w_.inter); }
  void run(RunParams rp, void* ws, cudaStream_t stream) override {
    if (rp.num_tokens <= 0) return;
    fp8_ffn_run(w_, 0, 1, rp.input, static_cast<const float*>(rp.input_scales), bounds_.uniform(1, rp.num_tokens, stream),
                rp.num_tokens, ws, rp.output, nullptr, status_, sm_count_, stream);
  }
  void set_status(int32_t* status) { status_ = status; }

 private:
  Fp8FfnWeights w_;
  int sm_count_;
  DeviceRowBounds bounds_;
  int32_t* status_ = nullptr;
};

// C[num_tokens, N] = A[num_tokens, K] * B[N, K]^T on e4m3 codes with 1x128 / 128x128 scales -> bf16.
class Fp8DenseGemm : public DenseGemmInterface {
 public:
  explicit Fp8DenseGemm(int sm_count) : sm_count_(sm_count), bounds_(2) {}
  size_t output_type_bytes() override { return 2; }
  size_t getWorkspaceSize(int64_t, int64_t) override { return 0; }
  void run(RunParams p, cudaStream_t stream) override {
    if (p.num_tokens <= 0) return;
    if (p.A_scales == nullptr || p.weight_scales == nullptr)
      throw std::runtime_error("the FP8 dense GEMM needs A_scales and weight_scales");
    executor_raise_if(epsb_grouped_gemm_fp8(EPSB_GEMM_PLAIN, p.A, static_cast<const float*>(p.A_scales), p.B,
                                            static_cast<const float*>(p.weight_scales),
                                            bounds_.uniform(1, p.num_tokens, stream), 1, p.num_tokens, p.gemm_n, p.gemm_k,
                                            p.C, nullptr, nullptr, status_, sm_count_, stream));
  }
  void set_status(int32_t* status) { status_ = status; }

 private:
  int sm_count_;
  DeviceRowBounds bounds_;
  int32_t* status_ = nullptr;
};

// num_gemms independent GEMMs of one shape, packed back to back: C[g] = A[g] * B[g]^T.  Only the dense packing is
// supported (lda = K, ldb = K, ldc = N, strides = the matrices' sizes): the TMA descriptors of the grouped kernel
// describe one [rows, K] matrix.
class Fp8BatchedGemm : public BatchedGemmInterface {
 public:
  explicit Fp8BatchedGemm(int sm_count) : sm_count_(sm_count), bounds_(DeviceRowBounds::kMaxParts + 1) {}
  size_t output_type_bytes() override { return 2; }
  size_t getWorkspaceSize(RunParams) override { return 0; }
  void run(RunParams rp, cudaStream_t stream) override {
    if (rp.num_gemms <= 0 || rp.M <= 0) return;
    if (rp.lda != rp.K || rp.ldb != rp.K || rp.ldc != rp.N || rp.A_stride != rp.M * rp.K ||
        rp.B_stride != rp.N * rp.K || rp.C_stride != rp.M * rp.N)
      throw std::runtime_error("the batched GEMM supports densely packed operands only");
    if (rp.A_scales == nullptr || rp.weight_scales == nullptr)
      throw std::runtime_error("the FP8 batched GEMM needs A_scales and weight_scales");
    executor_raise_if(epsb_grouped_gemm_fp8(EPSB_GEMM_PLAIN, rp.A, static_cast<const float*>(rp.A_scales), rp.B,
                                            static_cast<const float*>(rp.weight_scales),
                                            bounds_.uniform(rp.num_gemms, rp.M, stream), rp.num_gemms,
                                            rp.M * rp.num_gemms, rp.N, rp.K, rp.C, nullptr, nullptr, status_, sm_count_,
                                            stream));
  }
  void set_status(int32_t* status) { status_ = status; }

 private:
  int sm_count_;
  DeviceRowBounds bounds_;
  int32_t* status_ = nullptr;
};

// silu(gate) * up on dense rows (reference contract DenseActivationInterface).
class DenseSiluActivation : public DenseActivationInterface {
 public:
  DenseSiluActivation() : bounds_(2) {}
  void run(RunParams p, cudaStream_t stream) override {
    if (p.num_tokens <= 0) return;
    executor_raise_if(epsb_silu_run(p.gate_up, p.activation, bounds_.uniform(1, p.num_tokens, stream), 1, p.num_tokens,
                                    p.inter_size_x2 / 2, stream));
  }

 private:
  DeviceRowBounds bounds_;
};

}  // namespace epsb_host
