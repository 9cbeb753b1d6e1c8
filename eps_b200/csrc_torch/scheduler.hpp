// The staged EPS scheduler as a C++ object over the eps_b200 C ABI: what libscheduler_.so hands out as the
// `eps_create` handle.
//
// Same constructor arguments, methods, stage semantics and index layouts as the reference's
// eps::Scheduler<Traits> (src/scheduler/scheduler.cuh, scheduler.cu:30-353) and its Context
// (src/scheduler/context.cu): rendezvous -> plan -> prologue -> per stage {dispatch, gemm_expand, <GEMMs>,
// local_reduce, combine} -> epilogue.  Underneath: plans from two single-launch cluster kernels, row movement by
// grid-filling gathers, and for ep_world_size > 1 the device-side exchange over peer memory (no NCCL on the data
// path, no host read of the plans except the row count `rendezvous` has to return).
// The per-call plan buffers live in the caller's workspace (eps_get_workspace_size_context / eps_set_ws_context),
// like the reference's; nothing is allocated per call.
#pragma once

#include <memory>
#include <vector>

#include "communicator.hpp"

namespace epsb_host {

class Scheduler {
 public:
  struct Params {
    int topk;
    int num_experts;
    int64_t hidden_size;
    int input_scales_dim;
    int64_t max_num_tokens_per_gpu;
    Communicator* comm;   // may be NULL: a world of one
    int max_num_stages;
    bool fp8_hidden;      // hidden rows are e4m3 codes (FP8 path) instead of bf16
  };

  // Per-call state (reference Scheduler::Context).  Plan buffers are carved from the caller's workspace.
  struct Context {
    int num_tokens, num_global_tokens, num_stages;
    bool input_quanted;
    int64_t rows_bound = 0;   // upper bound of received rows known on the host
    char* ws = nullptr;
    // carved pointers
    int32_t *send_map = nullptr, *send_bounds = nullptr, *send_incl = nullptr, *glob_map = nullptr, *coll_incl = nullptr;
    int32_t *recv_incl = nullptr, *gemm_map = nullptr, *inv_gemm = nullptr, *scale_map = nullptr, *red_map = nullptr;
    int32_t *ret_incl = nullptr, *status = nullptr;
    const int32_t* excl = nullptr;  // the caller's exclusive_sum tensor
    float *zero_scale = nullptr, *row_w = nullptr;
    int32_t* a_rows = nullptr;   // source row of every GEMM row (direct sources)
    // what prologue recorded
    const void* raw_input = nullptr;
    const void* src_hidden = nullptr;
    const float* src_scales = nullptr;
    float* scales_out = nullptr;
    const float* src_weights = nullptr;
    bool direct = false;          // world of one, FP8 path: nothing is staged, GEMM rows are read from the caller's tensors
    bool sources_ready = false;   // a_rows / row_w of this call have been composed
    bool eager = false;
    bool have_zero = false;   // zero_scale was computed (plan got the gate weights)
    size_t ws_bytes = 0;
  };

  explicit Scheduler(Params p) : p_(p) {
    W_ = p.comm != nullptr ? p.comm->getWorldSize() : 1;
    rank_ = p.comm != nullptr ? p.comm->getRank() : 0;
    if (p.num_experts % W_ != 0)
      throw std::runtime_error("num_experts " + std::to_string(p.num_experts) + " is not divisible by ep_world_size " +
                               std::to_string(W_));
    EL_ = p.num_experts / W_;
    lo_ = rank_ * EL_;
    hi_ = lo_ + EL_;
    rows_ = std::max<int64_t>(1, p.max_num_tokens_per_gpu * W_);  // reference arena sizing (msccl_comm.cu:191-199)
    hidden_elem_ = p.fp8_hidden ? 1 : 2;
    auto dev = at::TensorOptions().device(at::kCUDA, at::cuda::current_device());
    if (W_ > 1) {
      const int S_max = std::max(1, std::min(p.max_num_stages, EL_));
      int64_t bytes = 0;
      raise_if(epsb_exchange_region_bytes(W_, (int)p.max_num_tokens_per_gpu, S_max, p.topk, p.hidden_size, hidden_elem_,
                                          p.input_scales_dim, &bytes));
      std::vector<void*> peers;
      region_ = p.comm->symm_alloc(bytes, peers);
      raise_if(epsb_exchange_create(rank_, W_, (int)p.max_num_tokens_per_gpu, S_max, p.topk, p.hidden_size, hidden_elem_,
                                    p.input_scales_dim, peers.data(), &x_));
      S_max_ = S_max;
    } else {
      // a world of one: the receive side IS the send side
      idx_ = at::empty({rows_, p.topk}, dev.dtype(at::kInt));
      wts_ = at::empty({rows_, p.topk}, dev.dtype(at::kFloat));
      hidden_ = at::empty({rows_, p.hidden_size * hidden_elem_}, dev.dtype(at::kByte));
      out_ = at::empty({rows_, p.hidden_size}, dev.dtype(at::kBFloat16));
      if (p.input_scales_dim > 0) scales_ = at::empty({rows_, p.input_scales_dim}, dev.dtype(at::kFloat));
    }
  }

  ~Scheduler() {
    if (x_ != nullptr) {
      p_.comm->symm_free(region_);
      epsb_exchange_destroy(x_);
    }
  }

  Context* getContext(int num_tokens, int num_global_tokens, int num_stages, bool input_quanted) {
    if (num_stages <= 0 || EL_ % num_stages != 0 || (W_ > 1 && num_stages > S_max_))
      throw std::runtime_error("Invalid num_stages: " + std::to_string(num_stages) +
                               " for local_num_experts: " + std::to_string(EL_));
    if (num_tokens > p_.max_num_tokens_per_gpu)
      throw std::runtime_error("num_tokens " + std::to_string(num_tokens) + " exceeds max_num_tokens_per_gpu " +
                               std::to_string(p_.max_num_tokens_per_gpu));
    auto* c = new Context();
    c->num_tokens = num_tokens;
    c->num_global_tokens = num_global_tokens;
    c->num_stages = num_stages;
    c->input_quanted = input_quanted;
    c->ws_bytes = layout(*c, nullptr);
    return c;
  }

  static size_t workspaceSize(const Context& c) { return c.ws_bytes; }

  void setWorkspace(Context& c, char* ws) {
    c.ws = ws;
    layout(c, ws);
  }

  // Dispatch plan (+ collect plan), plan exchange; returns the number of unique rows this rank receives.  Blocks
  // the host on that one number, as the reference does (scheduler.cu:274-278); no_host_read skips the read and
  // returns the arena size (every later step reads its bounds on the device).
  int64_t rendezvous(const int32_t* idx, Context& c, cudaStream_t st, bool no_host_read = false, int max_cluster = 0) {
    need_ws(c);
    const int T = c.num_tokens, S = c.num_stages;
    cuda_ok(cudaMemsetAsync(c.send_bounds, 0, 4, st), "memset");
    cuda_ok(cudaMemsetAsync(c.status, 0, 16, st), "memset");
    raise_if(epsb_source_plans(idx, nullptr, T, p_.topk, p_.num_experts, W_, S, c.send_map, c.send_incl, c.glob_map,
                               c.coll_incl, nullptr, max_cluster, st));
    const int32_t* count_at;
    if (W_ == 1) {
      c.recv_incl = c.send_incl;
      count_at = c.send_incl + S - 1;
    } else {
      raise_if(epsb_exchange_begin(x_, &epoch_));
      raise_if(epsb_exchange_publish_plans(x_, c.send_incl, c.coll_incl, S, st));
      raise_if(epsb_exchange_recv_plans(x_, S, c.recv_incl, c.status, 0, st));
      count_at = c.recv_incl + W_ * S - 1;
    }
    if (no_host_read) {
      c.rows_bound = W_ == 1 ? T : rows_;
      return c.rows_bound;
    }
    int32_t n = 0;
    cuda_ok(cudaMemcpyAsync(&n, count_at, 4, cudaMemcpyDeviceToHost, st), "row count");
    cuda_ok(cudaStreamSynchronize(st), "rendezvous");
    if (n > rows_) throw std::runtime_error("received rows exceed the arena");
    c.rows_bound = n;
    return n;
  }

  // Moves the expert ids (and gate weights) to the expert ranks, then the expert-side plans; exclusive_sum is the
  // caller's [EL+1] tensor.  payload_hidden/payload_scales (FP8 path, one stage): the rows travel in the same launch.
  void plan(const int32_t* idx, const float* scales, int32_t* exclusive_sum, Context& c, cudaStream_t st,
            const void* payload_hidden = nullptr, const float* payload_scales = nullptr, int max_cluster = 0) {
    need_ws(c);
    const int T = c.num_tokens, S = c.num_stages, k = p_.topk;
    c.excl = exclusive_sum;
    c.have_zero = scales != nullptr;
    if (scales != nullptr) raise_if(epsb_zero_plan(idx, scales, T, k, c.zero_scale, st));
    if (W_ == 1) {
      if (T > 0)
        raise_if(epsb_gather_rows(idx, idx_arena(), c.send_map, 1, T, c.send_bounds, 0, W_ * S, 0, send_bound(T),
                                  (int64_t)k * 4, st));
    } else {
      int mask = EPSB_PUT_META;
      c.eager = payload_hidden != nullptr;
      if (c.eager) mask |= EPSB_PUT_HIDDEN | (payload_scales != nullptr ? EPSB_PUT_SCALES : 0);
      raise_if(epsb_exchange_put(x_, EPSB_FLAG_META, -1, mask, idx, scales, payload_hidden, payload_scales, c.send_map,
                                 c.send_incl, T, S, st));
      raise_if(epsb_exchange_wait(x_, EPSB_FLAG_META, c.status, 0, st));
    }
    raise_if(epsb_expert_plans(idx_arena(), c.recv_incl, k, lo_, hi_, W_, S, (int)p_.max_num_tokens_per_gpu,
                               std::max<int64_t>(c.rows_bound, 0), exclusive_sum, c.gemm_map, c.inv_gemm, c.scale_map,
                               c.red_map, c.ret_incl, c.status + 2, max_cluster, st));
  }

  // direct (a world of one): in a world of one the receive order IS the send order, so the GEMM rows can be read
  // straight from the caller's tensors through the composed plans (gemmExpand) and nothing is staged here.
  void prologue(const float* expert_scales, const void* hidden, const float* input_scales, float* recv_input_scales,
                Context& c, cudaStream_t st, const void* raw_input = nullptr, bool direct = false) {
    need_ws(c);
    const int T = c.num_tokens, S = c.num_stages, k = p_.topk;
    c.direct = false;
    c.sources_ready = false;
    // the identity-expert term reads the raw bf16 tokens: an FP8 caller passes them as raw_input
    c.raw_input = raw_input != nullptr ? raw_input : (p_.fp8_hidden ? nullptr : hidden);
    if (c.input_quanted && (input_scales == nullptr || recv_input_scales == nullptr || p_.input_scales_dim == 0))
      throw std::runtime_error("input_quanted needs input_scales, recv_input_scales and input_scales_dim > 0");
    if (W_ > 1) {  // rows are read through the dispatch plan when they are sent: nothing to stage
      c.src_hidden = hidden;
      c.src_scales = c.input_quanted ? input_scales : nullptr;
      c.scales_out = c.input_quanted ? recv_input_scales : nullptr;
      return;
    }
    if (T == 0) return;
    if (direct) {
      c.direct = true;
      c.src_hidden = hidden;
      c.src_scales = c.input_quanted ? input_scales : nullptr;
      c.scales_out = c.input_quanted ? recv_input_scales : nullptr;
      c.src_weights = expert_scales;
      return;
    }
    const int64_t bound = send_bound(T);
    raise_if(epsb_gather_rows(expert_scales, wts_.data_ptr(), c.send_map, 1, T, c.send_bounds, 0, S, 0, bound,
                              (int64_t)k * 4, st));
    raise_if(epsb_gather_rows(hidden, hidden_.data_ptr(), c.send_map, 1, T, c.send_bounds, 0, S, 0, bound,
                              p_.hidden_size * hidden_elem_, st));
    if (c.input_quanted) {
      raise_if(epsb_gather_rows(input_scales, scales_.data_ptr(), c.send_map, 1, T, c.send_bounds, 0, S, 0, bound,
                                (int64_t)p_.input_scales_dim * 4, st));
      raise_if(epsb_gather_rows(scales_.data_ptr(), recv_input_scales, c.gemm_map, k, INT32_MAX, c.excl, 0, EL_, 0,
                                gemm_bound(c), (int64_t)p_.input_scales_dim * 4, st));
    }
  }

  void dispatch(Context& c, int stage, cudaStream_t st) {
    if (W_ == 1 || c.eager) return;
    int mask = EPSB_PUT_HIDDEN | (c.src_scales != nullptr ? EPSB_PUT_SCALES : 0);
    const int slot = EPSB_FLAG_DISPATCH(std::max(stage, 0));
    raise_if(epsb_exchange_put(x_, slot, stage, mask, nullptr, nullptr, c.src_hidden, c.src_scales, c.send_map,
                               c.send_incl, c.num_tokens, c.num_stages, st));
    raise_if(epsb_exchange_wait(x_, slot, c.status, 0, st));
  }

  // a_rows[d] = the token whose row GEMM row d is, row_w[d] = its gate weight for that expert (one kernel per call)
  void composeSources(Context& c, cudaStream_t st) {
    if (c.sources_ready) return;
    raise_if(epsb_gemm_row_sources(c.gemm_map, c.excl, EL_, p_.topk, c.send_map, c.num_tokens, c.src_weights,
                                   gemm_bound(c), c.a_rows, c.row_w, st));
    c.sources_ready = true;
  }

  void gemmExpand(void* gemm_input, Context& c, int stage, cudaStream_t st) {
    const int eps = EL_ / c.num_stages;
    const int b0 = stage < 0 ? 0 : eps * stage, b1 = stage < 0 ? EL_ : eps * (stage + 1);
    if (c.direct) {
      composeSources(c, st);
      raise_if(epsb_gather_rows(c.src_hidden, gemm_input, c.a_rows, 1, INT32_MAX, c.excl, b0, b1, 0, gemm_bound(c),
                                p_.hidden_size * hidden_elem_, st));
      if (c.scales_out != nullptr)
        raise_if(epsb_gather_rows(c.src_scales, c.scales_out, c.a_rows, 1, INT32_MAX, c.excl, b0, b1, 0, gemm_bound(c),
                                  (int64_t)p_.input_scales_dim * 4, st));
      return;
    }
    raise_if(epsb_gather_rows(hidden_arena(), gemm_input, c.gemm_map, p_.topk, INT32_MAX, c.excl, b0, b1, 0,
                              gemm_bound(c), p_.hidden_size * hidden_elem_, st));
    if (W_ > 1 && c.scales_out != nullptr)
      raise_if(epsb_gather_rows(scales_arena(), c.scales_out, c.gemm_map, p_.topk, INT32_MAX, c.excl, b0, b1, 0,
                                gemm_bound(c), (int64_t)p_.input_scales_dim * 4, st));
  }

  // pre_weighted = false: the reference's arithmetic (bf16(weight) * row, bf16 accumulate); world of one only when the
  // device-side exchange is in use.  pre_weighted = true: rows already carry their gate weight, fp32 accumulation.
  void localReduce(const void* gemm_output, Context& c, int stage, cudaStream_t st, bool pre_weighted) {
    const int64_t mr = std::max<int64_t>(c.rows_bound, 0);
    if (W_ > 1) {
      if (!pre_weighted)
        throw std::runtime_error("with ep_world_size > 1 the return rows must be pre-weighted (eps_local_reduce_weighted)");
      raise_if(epsb_exchange_local_reduce_put(x_, EPSB_FLAG_COMBINE(S_max_, std::max(stage, 0)), gemm_output, c.red_map,
                                              c.ret_incl, c.num_stages, stage, mr, st));
      return;
    }
    if (!pre_weighted && c.direct)
      throw std::runtime_error("the reference-arithmetic local reduce reads the staged gate weights: use eps_prologue, or "
                               "eps_local_reduce_weighted on rows that carry their weight");
    if (pre_weighted)
      raise_if(epsb_local_reduce(gemm_output, c.red_map, c.ret_incl, p_.topk, W_, c.num_stages, stage, mr,
                                 p_.hidden_size, out_.data_ptr(), st));
    else
      raise_if(epsb_local_reduce_ref(gemm_output, wts_.data_ptr<float>(), c.scale_map, c.red_map, c.ret_incl, p_.topk,
                                     W_, c.num_stages, stage, mr, p_.hidden_size, out_.data_ptr(), st));
  }

  void combine(Context& c, int stage, cudaStream_t st) {
    if (W_ == 1) return;
    raise_if(epsb_exchange_wait(x_, EPSB_FLAG_COMBINE(S_max_, std::max(stage, 0)), c.status, 0, st));
  }

  // ref_arith: reference bf16 adds (globalReduce + zeroReduce, scheduler.cu:205-228); otherwise one fp32 sum.
  void epilogue(void* output, Context& c, cudaStream_t st, const void* shared = nullptr, bool ref_arith = true) {
    const bool zero = c.raw_input != nullptr && c.have_zero;
    const void* x = zero ? c.raw_input : nullptr;
    const float* zs = zero ? c.zero_scale : nullptr;
    if (ref_arith)
      raise_if(epsb_global_reduce_ref(out_arena(), c.glob_map, shared, x, zs, c.num_tokens, W_, p_.hidden_size, output, st));
    else
      raise_if(epsb_global_reduce(out_arena(), c.glob_map, shared, x, zs, c.num_tokens, W_, p_.hidden_size, output, st));
  }

  // ep_world_size == 1: local reduce + (empty) exchange + global reduce in one pass over pre-weighted rows.
  void reduceSingleRank(const void* gemm_output, void* output, const void* shared, Context& c, cudaStream_t st) {
    if (W_ != 1) throw std::runtime_error("reduce_single_rank needs ep_world_size == 1");
    const bool zero = c.raw_input != nullptr && c.have_zero;
    raise_if(epsb_reduce_ep1(gemm_output, c.red_map, c.glob_map, c.ret_incl, c.num_stages, shared,
                             zero ? c.raw_input : nullptr, zero ? c.zero_scale : nullptr, c.num_tokens, p_.topk,
                             p_.hidden_size, output, st));
  }

  // row_w[d] = gate weight of GEMM row d (for the down GEMM's fused weighting); lives in the workspace.
  float* gemmRowWeights(Context& c, cudaStream_t st) {
    if (c.direct) {
      composeSources(c, st);
      return c.row_w;
    }
    raise_if(epsb_gather_row_weights(wts_arena(), c.gemm_map, c.excl, EL_, gemm_bound(c), c.row_w, st));
    return c.row_w;
  }

  void checkStatus(Context& c, cudaStream_t st) {
    int32_t s[4];
    cuda_ok(cudaMemcpyAsync(s, c.status, 16, cudaMemcpyDeviceToHost, st), "status");
    cuda_ok(cudaStreamSynchronize(st), "status");
    if (s[0] != 0) throw std::runtime_error("expert-parallel exchange failed (code " + std::to_string(s[0]) + ")");
    if (s[2] != 0) throw std::runtime_error("expert plans refused the received row count " + std::to_string(s[3]));
  }

  int localNumExperts() const { return EL_; }
  int worldSize() const { return W_; }
  int64_t gemm_bound(const Context& c) const { return std::max<int64_t>(c.rows_bound, 0) * std::min(p_.topk, EL_); }

 private:
  void need_ws(const Context& c) const {
    if (c.ws == nullptr) throw std::runtime_error("the context has no workspace: call eps_set_ws_context first");
  }
  int64_t send_bound(int T) const { return std::min<int64_t>((int64_t)T * std::min(W_, p_.topk), rows_); }

  // this rank's receive arena of the current call (the dispatch arenas alternate with the exchange's epoch)
  void* arena(int which) const {
    void* p = nullptr;
    raise_if(epsb_exchange_arena(x_, which, epoch_ & 1, &p));
    return p;
  }
  int32_t* idx_arena() const { return W_ == 1 ? idx_.data_ptr<int32_t>() : static_cast<int32_t*>(arena(EPSB_ARENA_IDX)); }
  float* wts_arena() const { return W_ == 1 ? wts_.data_ptr<float>() : static_cast<float*>(arena(EPSB_ARENA_WEIGHTS)); }
  void* hidden_arena() const { return W_ == 1 ? hidden_.data_ptr() : arena(EPSB_ARENA_HIDDEN); }
  void* scales_arena() const { return W_ == 1 ? scales_.data_ptr() : arena(EPSB_ARENA_SCALES); }
  void* out_arena() const { return W_ == 1 ? out_.data_ptr() : arena(EPSB_ARENA_OUT); }

  // Carves the plan buffers out of `ws` (or only sizes them when ws == nullptr).
  size_t layout(Context& c, char* ws) const {
    size_t off = 0;
    auto take = [&](size_t bytes) {
      char* p = ws != nullptr ? ws + off : nullptr;
      off = (off + bytes + 255) & ~(size_t)255;
      return p;
    };
    const int64_t T = std::max(c.num_tokens, 1), n = (int64_t)W_ * c.num_stages, k = p_.topk;
    const int64_t R = W_ == 1 ? T : rows_;
    c.send_map = (int32_t*)take(T * W_ * 4);
    c.send_bounds = (int32_t*)take((n + 1) * 4);
    c.send_incl = c.send_bounds != nullptr ? c.send_bounds + 1 : nullptr;
    c.glob_map = (int32_t*)take(T * W_ * 4);
    c.coll_incl = (int32_t*)take(n * 4);
    c.zero_scale = (float*)take(T * 4);
    c.recv_incl = (int32_t*)take(n * 4);
    c.gemm_map = (int32_t*)take(R * k * 4);
    c.inv_gemm = (int32_t*)take(R * k * 4);
    c.scale_map = (int32_t*)take(R * 4);
    c.red_map = (int32_t*)take(R * k * 4);
    c.ret_incl = (int32_t*)take(n * 4);
    c.row_w = (float*)take(R * std::min<int64_t>(k, EL_) * 4);
    c.a_rows = (int32_t*)take(R * std::min<int64_t>(k, EL_) * 4);
    c.status = (int32_t*)take(16);
    return off;
  }

  Params p_;
  int epoch_ = 0;
  int W_ = 1, rank_ = 0, EL_ = 0, lo_ = 0, hi_ = 0, hidden_elem_ = 2, S_max_ = 1;
  int64_t rows_ = 1;
  void* region_ = nullptr;
  epsb_exchange_t* x_ = nullptr;
  at::Tensor idx_, wts_, hidden_, scales_, out_;
};

}  // namespace epsb_host
