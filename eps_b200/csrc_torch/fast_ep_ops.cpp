// libfast_ep.so: the non-staged expert-parallel dispatch / combine (`fast_ep.all_to_all_*`), with the reference's op
// names and argument lists (src/fast_ep/bindings/all_to_all_ops.cu:17-95) over FastEP<T>::dispatch / combine
// (src/fast_ep/all_to_all/fast_ep.cu:63-215).
//
// dispatch: count-sort the (token, slot) pairs by GLOBAL expert (rows of one expert in descending pair order, the
// reference's order, fast_ep_kernels.cu:146-155), scatter the token rows into send order, all-gather the counts,
// exchange the rows, regroup [source][expert] -> [expert][source].  combine: the inverse regroup and exchange, then
// the fp32-accumulated weighted sum over the k slots, where a zero-computation slot reads the raw input token.
// With ep_world_size > 1 the rows travel as one grouped NCCL send/recv per direction, sized from one host read of
// the all-gathered counts (the reference spins on a mapped integer at the same point).
#include "communicator.hpp"

namespace {

using namespace epsb_host;

class FastEP {
 public:
  FastEP(int64_t topk, int64_t num_experts, int64_t hidden, int64_t max_num_global_tokens, Communicator* comm)
      : k_((int)topk), E_((int)num_experts), H_(hidden), comm_(comm) {
    W_ = comm != nullptr ? comm->getWorldSize() : 1;
    rank_ = comm != nullptr ? comm->getRank() : 0;
    if (E_ % W_ != 0)
      throw std::runtime_error("num_experts " + std::to_string(E_) + " is not divisible by ep_world_size " +
                               std::to_string(W_));
    EL_ = E_ / W_;
    rows_ = std::max<int64_t>(1, max_num_global_tokens * topk);  // reference arena: every pair may land on one rank
    auto dev = at::TensorOptions().device(at::kCUDA, at::cuda::current_device());
    send_ = at::empty({rows_, H_}, dev.dtype(at::kBFloat16));
    recv_ = W_ == 1 ? send_ : at::empty({rows_, H_}, dev.dtype(at::kBFloat16));
    excl_ = at::empty({E_ + 1}, dev.dtype(at::kInt));
    mapping_ = at::empty({rows_}, dev.dtype(at::kInt));
    ag_ = at::empty({W_, E_ + 1}, dev.dtype(at::kInt));
    plan_ = at::empty({5, std::max(EL_ * W_, W_ + 1)}, dev.dtype(at::kInt));
  }

  void dispatch(int32_t* out_exclusive_sum, void* out_expert_x, int64_t out_rows, const void* dp_x,
                const int32_t* indices, int64_t T, cudaStream_t st) {
    if (T * k_ > rows_) throw std::runtime_error("tokens exceed max_num_global_tokens");
    raise_if(epsb_fastep_expand_plan(indices, (int)T, k_, E_, excl_.data_ptr<int32_t>(), mapping_.data_ptr<int32_t>(), st));
    if (T > 0) raise_if(epsb_scatter_rows(dp_x, send_.data_ptr(), mapping_.data_ptr<int32_t>(), k_, T * k_, H_ * 2, st));
    if (W_ == 1) {
      cuda_ok(cudaMemcpyAsync(ag_.data_ptr(), excl_.data_ptr(), (size_t)(E_ + 1) * 4, cudaMemcpyDeviceToDevice, st), "copy");
    } else {
      nccl_ok(ncclAllGather(excl_.data_ptr(), ag_.data_ptr(), (size_t)E_ + 1, ncclInt32, comm_->nccl(), st),
              "ncclAllGather(counts)");
    }
    int32_t* pl = plan_.data_ptr<int32_t>();
    const int64_t pitch = plan_.size(1);
    raise_if(epsb_fastep_plan(ag_.data_ptr<int32_t>(), rank_, W_, E_, pl, pl + pitch, out_exclusive_sum, pl + 2 * pitch,
                              pl + 3 * pitch, pl + 4 * pitch, st));
    if (W_ > 1) {
      host_.resize((size_t)W_ * (E_ + 1));
      cuda_ok(cudaMemcpyAsync(host_.data(), ag_.data_ptr(), host_.size() * 4, cudaMemcpyDeviceToHost, st), "counts");
      cuda_ok(cudaStreamSynchronize(st), "counts");   // the one host read
      windows();
      if (recv_end_.back() > rows_ || recv_end_.back() > out_rows) throw std::runtime_error("received rows exceed the buffers");
      exchange(send_, send_begin_, send_end_, recv_, recv_begin_, recv_end_, st);
    }
    raise_if(epsb_arrange_rows(recv_.data_ptr(), out_expert_x, pl + 2 * pitch, pl + 3 * pitch, pl + 4 * pitch, EL_ * W_,
                               out_rows, H_ * 2, st));
    dp_x_ = dp_x;
    T_ = T;
    dispatched_ = true;
  }

  void combine(void* out_tokens, const float* weights, const void* expert_y, int64_t y_rows, const void* shared,
               cudaStream_t st) {
    if (!dispatched_) throw std::runtime_error("combine called before dispatch");
    int32_t* pl = plan_.data_ptr<int32_t>();
    const int64_t pitch = plan_.size(1);
    // inverse regroup: [expert][source] -> [source][expert] in the receive buffer of dispatch
    raise_if(epsb_arrange_rows(expert_y, recv_.data_ptr(), pl + 4 * pitch, pl + 3 * pitch, pl + 2 * pitch, EL_ * W_,
                               y_rows, H_ * 2, st));
    // what I received from p goes back to p and lands where p sent it from
    if (W_ > 1) exchange(recv_, recv_begin_, recv_end_, send_, send_begin_, send_end_, st);
    raise_if(epsb_fastep_reduce(send_.data_ptr(), dp_x_, shared, weights, mapping_.data_ptr<int32_t>(), (int)T_, k_, H_,
                                out_tokens, st));
  }

 private:
  void windows() {
    send_begin_.assign(W_, 0); send_end_.assign(W_, 0); recv_begin_.assign(W_, 0); recv_end_.assign(W_, 0);
    const int64_t* dummy = nullptr;
    (void)dummy;
    int64_t acc = 0;
    for (int p = 0; p < W_; p++) {
      send_begin_[p] = host_[(size_t)rank_ * (E_ + 1) + (size_t)p * EL_];
      send_end_[p] = host_[(size_t)rank_ * (E_ + 1) + (size_t)(p + 1) * EL_];
      const int64_t cnt = host_[(size_t)p * (E_ + 1) + (size_t)(rank_ + 1) * EL_] -
                          host_[(size_t)p * (E_ + 1) + (size_t)rank_ * EL_];   // rows source p sends me
      recv_begin_[p] = acc;
      acc += cnt;
      recv_end_[p] = acc;
    }
  }

  void exchange(const at::Tensor& src, const std::vector<int64_t>& sb, const std::vector<int64_t>& se,
                const at::Tensor& dst, const std::vector<int64_t>& rb, const std::vector<int64_t>& re, cudaStream_t st) {
    const char* s = static_cast<const char*>(src.data_ptr());
    char* d = static_cast<char*>(dst.data_ptr());
    const int64_t row = H_ * 2;
    if (se[rank_] > sb[rank_])
      cuda_ok(cudaMemcpyAsync(d + rb[rank_] * row, s + sb[rank_] * row, (size_t)((se[rank_] - sb[rank_]) * row),
                              cudaMemcpyDeviceToDevice, st), "local rows");
    nccl_ok(ncclGroupStart(), "ncclGroupStart");
    for (int step = 1; step < W_; step++) {
      const int to = (rank_ + step) % W_, from = (rank_ - step + W_) % W_;
      if (se[to] > sb[to])
        nccl_ok(ncclSend(s + sb[to] * row, (size_t)((se[to] - sb[to]) * H_), ncclBfloat16, to, comm_->nccl(), st), "ncclSend");
      if (re[from] > rb[from])
        nccl_ok(ncclRecv(d + rb[from] * row, (size_t)((re[from] - rb[from]) * H_), ncclBfloat16, from, comm_->nccl(), st),
                "ncclRecv");
    }
    nccl_ok(ncclGroupEnd(), "ncclGroupEnd");
  }

  int k_, E_, EL_ = 0, W_ = 1, rank_ = 0;
  int64_t H_, rows_ = 1, T_ = 0;
  Communicator* comm_;
  at::Tensor send_, recv_, excl_, mapping_, ag_, plan_;
  std::vector<int32_t> host_;
  std::vector<int64_t> send_begin_, send_end_, recv_begin_, recv_end_;
  const void* dp_x_ = nullptr;
  bool dispatched_ = false;
};

FastEP* fe(fptr_t p) {
  TORCH_CHECK(p != 0, "fast_ep handle is null");
  return reinterpret_cast<FastEP*>(p);
}

fptr_t create(int64_t topk, int64_t num_experts, int64_t hidden_size, int64_t max_num_global_tokens, fptr_t comm) {
  return reinterpret_cast<fptr_t>(
      new FastEP(topk, num_experts, hidden_size, max_num_global_tokens, reinterpret_cast<Communicator*>(comm)));
}
void destroy(fptr_t ptr) { delete reinterpret_cast<FastEP*>(ptr); }

void dispatch(fptr_t ptr, at::Tensor& outExclusiveSum, at::Tensor& outExpertX, const at::Tensor& dpX,
              const at::Tensor& indices, int64_t /*num_global_tokens*/) {
  check(outExpertX, 2, "outExpertX");
  check(dpX, 2, "dpX");
  check(indices, 2, "indices");
  TORCH_CHECK(indices.scalar_type() == at::kInt, "indices must be of type kInt32");
  TORCH_CHECK(outExclusiveSum.scalar_type() == at::kInt, "outExclusiveSum must be of type kInt32");
  TORCH_CHECK(dpX.scalar_type() == at::kBFloat16 && outExpertX.scalar_type() == at::kBFloat16, "rows must be bfloat16");
  fe(ptr)->dispatch(outExclusiveSum.data_ptr<int32_t>(), outExpertX.data_ptr(), outExpertX.size(0), dpX.data_ptr(),
                    indices.data_ptr<int32_t>(), indices.size(0), current_stream());
}

void combine(fptr_t ptr, at::Tensor& outTokens, const at::Tensor& weights, const at::Tensor& expertY,
             int64_t /*num_global_tokens*/) {
  check(outTokens, 2, "outTokens");
  TORCH_CHECK(outTokens.scalar_type() == at::kBFloat16, "outTokens must be of type BFloat16");
  check(weights, 2, "weights");
  TORCH_CHECK(weights.scalar_type() == at::kFloat, "weights must be of type Float32");
  check(expertY, 2, "expertY");
  fe(ptr)->combine(outTokens.data_ptr(), weights.data_ptr<float>(), expertY.data_ptr(), expertY.size(0), nullptr,
                   current_stream());
}

}  // namespace

TORCH_LIBRARY(fast_ep, m) {
  m.def("all_to_all_create", &create);
  m.def("all_to_all_destroy", &destroy);
  m.def("all_to_all_dispatch", &dispatch);
  m.def("all_to_all_combine", &combine);
}

EPSB_REGISTER_EXTENSION(libfast_ep)
