// libcommunication_.so: the communicator and TP<->DP convertor operators under namespace `communication`, with the
// reference's names and argument lists (src/communication/bindings/communication_ops.cu:21-204).
#include "communicator.hpp"

namespace {

using namespace epsb_host;

at::Tensor comm_create_unique_id() {
  auto out = at::empty({(int64_t)Communicator::kUniqueIdBytes}, at::TensorOptions().dtype(at::kByte).device(at::kCPU));
  Communicator::make_unique_id(out.data_ptr<uint8_t>());
  return out;
}

fptr_t comm_create(const at::Tensor& unique_id, int64_t rank, int64_t ep_world_size, int64_t num_ranks_per_node) {
  TORCH_CHECK(unique_id.device().is_cpu(), "unique_id must be a CPU tensor");
  TORCH_CHECK(unique_id.scalar_type() == at::kByte, "unique_id must be uint8");
  TORCH_CHECK(unique_id.is_contiguous(), "unique_id must be contiguous");
  TORCH_CHECK(unique_id.numel() == (int64_t)Communicator::kUniqueIdBytes, "unique_id must hold ",
              Communicator::kUniqueIdBytes, " bytes");
  return reinterpret_cast<fptr_t>(
      new Communicator(unique_id.data_ptr<uint8_t>(), (int)rank, (int)ep_world_size, (int)num_ranks_per_node));
}

void comm_destroy(fptr_t ptr) { delete reinterpret_cast<Communicator*>(ptr); }

void comm_barrier(fptr_t ptr) {
  TORCH_CHECK(ptr != 0, "communicator handle is null");
  reinterpret_cast<Communicator*>(ptr)->barrier();
}

// the reference's syncAndCheckEps (src/common/debug.cu): device-wide synchronise, then report the last error
void sync_check_cuda_error_eps_wrap() {
  cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  cuda_ok(cudaGetLastError(), "CUDA");
}

// TP <-> DP conversion inside groups of attn_tp_size consecutive ranks (reference TPDPConvertor<__nv_bfloat16>).
class TPDPConvertor {
 public:
  TPDPConvertor(int global_rank, int64_t tp_max_num_tokens, int attn_tp_size, int64_t hidden, Communicator* comm)
      : rank_(global_rank), tp_(attn_tp_size), hidden_(hidden), comm_(comm) {
    const int world = comm != nullptr ? comm->getWorldSize() : 1;
    if (attn_tp_size < 1 || world % attn_tp_size != 0 || attn_tp_size > EPSB_MAX_PEERS)
      throw std::runtime_error("attn_tp_size " + std::to_string(attn_tp_size) + " does not divide the world of " +
                               std::to_string(world));
    if (comm != nullptr && comm->getRank() != global_rank) throw std::runtime_error("global_rank differs from the communicator's");
    rows_ = std::max<int64_t>(1, (int64_t)attn_tp_size * tp_max_num_tokens);   // reference getMaxNumElems
    int64_t bytes = 0;
    raise_if(epsb_tpdp_region_bytes(rows_, hidden, &bytes));
    std::vector<void*> peers;
    if (comm != nullptr) {
      local_ = comm->symm_alloc(bytes, peers);
    } else {
      uint8_t handle[EPSB_IPC_HANDLE_BYTES];
      raise_if(epsb_symm_alloc(bytes, &local_, handle));
      peers.assign(1, local_);
    }
    const int base = attn_tp_size * (global_rank / attn_tp_size);   // first rank of my group
    for (int j = 0; j < attn_tp_size; j++) group_.push_back(peers[base + j]);
    tp_rank_ = global_rank - base;
    cuda_ok(cudaMalloc(reinterpret_cast<void**>(&status_), 16), "cudaMalloc(status)");
    cuda_ok(cudaMemset(status_, 0, 16), "cudaMemset(status)");
  }

  ~TPDPConvertor() {
    if (comm_ != nullptr) comm_->symm_free(local_);
    else epsb_symm_free(local_);
    cudaFree(status_);
  }

  void split(int64_t tp_num_tokens, int64_t& n, int64_t& off) const {
    const int64_t q = tp_num_tokens / tp_, rem = tp_num_tokens % tp_;
    n = q + (tp_rank_ < rem ? 1 : 0);
    off = q * tp_rank_ + std::min<int64_t>(tp_rank_, rem);
  }

  at::Tensor view(int64_t row0, int64_t rows, int64_t cols) const {
    auto opt = at::TensorOptions().device(at::kCUDA, at::cuda::current_device()).dtype(at::kBFloat16);
    return at::from_blob(static_cast<char*>(local_) + row0 * cols * 2, {rows, cols}, {cols, 1}, opt);
  }

  void check_hidden(int64_t hidden) const {
    if (hidden > hidden_)
      throw std::runtime_error(std::to_string(hidden) + " should be smaller than or equal to" + std::to_string(hidden_));
  }
  void check_tokens(int64_t tokens, int64_t hidden) const {
    if (tokens < 0 || tokens * hidden > rows_ * hidden_) throw std::runtime_error("tp_num_tokens exceeds the buffer");
  }

  void all_gather(int64_t tp_num_tokens, int64_t hidden, cudaStream_t st) {
    check_hidden(hidden);
    check_tokens(tp_num_tokens, hidden);
    const int e = ++epoch_;
    raise_if(epsb_tpdp_signal(group_.data(), tp_rank_, tp_, rows_, hidden_, 0, e, st));
    raise_if(epsb_tpdp_wait(local_, tp_, rows_, hidden_, 0, e, status_, 0, st));
    raise_if(epsb_tpdp_all_gather_put(group_.data(), tp_rank_, tp_, rows_, tp_num_tokens, hidden, hidden_, 1, e, st));
    raise_if(epsb_tpdp_wait(local_, tp_, rows_, hidden_, 1, e, status_, 0, st));
  }

  void reduce_scatter(int64_t tp_num_tokens, cudaStream_t st) {
    check_tokens(tp_num_tokens, hidden_);
    const int e = ++epoch_;
    raise_if(epsb_tpdp_signal(group_.data(), tp_rank_, tp_, rows_, hidden_, 2, e, st));
    raise_if(epsb_tpdp_wait(local_, tp_, rows_, hidden_, 2, e, status_, 0, st));
    raise_if(epsb_tpdp_reduce_scatter_sum(group_.data(), tp_rank_, tp_, rows_, tp_num_tokens, hidden_, hidden_, 3, e, st));
    raise_if(epsb_tpdp_wait(local_, tp_, rows_, hidden_, 3, e, status_, 0, st));
  }

  int64_t hidden() const { return hidden_; }

 private:
  int rank_, tp_, tp_rank_ = 0, epoch_ = 0;
  int64_t hidden_, rows_ = 1;
  Communicator* comm_;
  void* local_ = nullptr;
  std::vector<void*> group_;
  int32_t* status_ = nullptr;
};

TPDPConvertor* tpdp(fptr_t p) {
  TORCH_CHECK(p != 0, "tpdp handle is null");
  return reinterpret_cast<TPDPConvertor*>(p);
}

fptr_t tpdp_create(int64_t global_rank, int64_t tp_max_num_tokens, int64_t attn_tp_size, int64_t hidden_size, fptr_t comm) {
  return reinterpret_cast<fptr_t>(new TPDPConvertor((int)global_rank, tp_max_num_tokens, (int)attn_tp_size, hidden_size,
                                                    reinterpret_cast<Communicator*>(comm)));
}
void tpdp_destroy(fptr_t ptr) { delete reinterpret_cast<TPDPConvertor*>(ptr); }

// reduce-scatter: input = all tp_num_tokens rows of my buffer (my partial sums), output = my slice, in place
at::Tensor tpdp_get_reduce_scatter_input(fptr_t ptr, int64_t tp_num_tokens, int64_t /*num_blocks*/) {
  return tpdp(ptr)->view(0, tp_num_tokens, tpdp(ptr)->hidden());
}
at::Tensor tpdp_get_reduce_scatter_output(fptr_t ptr, int64_t tp_num_tokens, int64_t /*num_blocks*/) {
  int64_t n, off;
  tpdp(ptr)->split(tp_num_tokens, n, off);
  return tpdp(ptr)->view(off, n, tpdp(ptr)->hidden());
}
int64_t tpdp_get_reduce_scatter_output_row_offset(fptr_t ptr, int64_t tp_num_tokens, int64_t /*num_blocks*/) {
  int64_t n, off;
  tpdp(ptr)->split(tp_num_tokens, n, off);
  return off;
}
void tpdp_reduce_scatter(fptr_t ptr, int64_t tp_num_tokens, int64_t /*num_blocks*/, int64_t stream) {
  tpdp(ptr)->reduce_scatter(tp_num_tokens, reinterpret_cast<cudaStream_t>(stream));
}

// all-gather: input = my slice (rows of hidden_size columns), output = all tp_num_tokens rows
at::Tensor tpdp_get_all_gather_input(fptr_t ptr, int64_t tp_num_tokens, int64_t hidden_size, int64_t /*num_blocks*/) {
  tpdp(ptr)->check_hidden(hidden_size);
  int64_t n, off;
  tpdp(ptr)->split(tp_num_tokens, n, off);
  return tpdp(ptr)->view(off, n, hidden_size);
}
at::Tensor tpdp_get_all_gather_output(fptr_t ptr, int64_t tp_num_tokens, int64_t hidden_size, int64_t /*num_blocks*/) {
  tpdp(ptr)->check_hidden(hidden_size);
  return tpdp(ptr)->view(0, tp_num_tokens, hidden_size);
}
int64_t tpdp_get_all_gather_input_row_offset(fptr_t ptr, int64_t tp_num_tokens, int64_t hidden_size,
                                             int64_t /*num_blocks*/) {
  tpdp(ptr)->check_hidden(hidden_size);
  int64_t n, off;
  tpdp(ptr)->split(tp_num_tokens, n, off);
  return off;
}
void tpdp_all_gather(fptr_t ptr, int64_t tp_num_tokens, int64_t hidden_size, int64_t /*num_blocks*/, int64_t stream) {
  tpdp(ptr)->all_gather(tp_num_tokens, hidden_size, reinterpret_cast<cudaStream_t>(stream));
}

}  // namespace

TORCH_LIBRARY(communication, m) {
  m.def("eps_comm_create_unique_id", &comm_create_unique_id);
  m.def("eps_comm_create", &comm_create);
  m.def("eps_comm_destroy", &comm_destroy);
  m.def("eps_comm_barrier", &comm_barrier);
  m.def("sync_check_cuda_error_eps", &sync_check_cuda_error_eps_wrap);
  m.def("eps_tpdp_create", &tpdp_create);
  m.def("eps_tpdp_destroy", &tpdp_destroy);
  m.def("eps_tpdp_get_reduce_scatter_input", &tpdp_get_reduce_scatter_input);
  m.def("eps_tpdp_get_reduce_scatter_output", &tpdp_get_reduce_scatter_output);
  m.def("eps_tpdp_get_reduce_scatter_output_row_offset", &tpdp_get_reduce_scatter_output_row_offset);
  m.def("eps_tpdp_reduce_scatter", &tpdp_reduce_scatter);
  m.def("eps_tpdp_get_all_gather_input", &tpdp_get_all_gather_input);
  m.def("eps_tpdp_get_all_gather_output", &tpdp_get_all_gather_output);
  m.def("eps_tpdp_get_all_gather_input_row_offset", &tpdp_get_all_gather_input_row_offset);
  m.def("eps_tpdp_all_gather", &tpdp_all_gather);
}

EPSB_REGISTER_EXTENSION(libcommunication_)
