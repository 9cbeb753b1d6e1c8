// libfast_oep.so: lookups in an embedding table sharded over the ranks (`fast_oep.all_to_all_*`), with the
// reference's op names and argument lists (src/fast_oep/bindings/all_to_all_ops.cu:17-82) over
// FastOEP<T>::dispatch / combine (src/fast_oep/all_to_all/fast_oep.cu:52-151).
//
// dispatch(ids): the ids are grouped by owner rank (id / size_per_rank), the counts are exchanged device-side and
// every id is stored into its owner's id arena.  combine(out, ...): every owner answers the ids it received with the
// rows of its table shard, stored straight into the asking rank's row arena at the id's position in that rank's
// grouped order; the asking rank then scatters the rows to out[i] (or to the n-gram-major position).  Negative ids
// are skipped (their rows of `out` are left untouched), as in the reference.
// The transport is the library's peer-store exchange; a world of one runs the same kernels on its own region.
#include "communicator.hpp"

namespace {

using namespace epsb_host;

class FastOEP {
 public:
  FastOEP(int64_t embed_dim, int64_t size_per_rank, int64_t max_num_global_tokens, Communicator* comm)
      : D_(embed_dim), size_per_rank_(size_per_rank), comm_(comm) {
    W_ = comm != nullptr ? comm->getWorldSize() : 1;
    rank_ = comm != nullptr ? comm->getRank() : 0;
    if (embed_dim <= 0 || embed_dim % 8 != 0) throw std::runtime_error("Not supported embed_dim: " + std::to_string(embed_dim));
    max_ids_ = std::max<int64_t>(1, max_num_global_tokens);
    // arenas of max_tok * W rows: every id of the group may have this rank as its owner
    const int max_tok = (int)((max_ids_ + W_ - 1) / W_);
    int64_t bytes = 0;
    raise_if(epsb_exchange_region_bytes(W_, max_tok, 1, 1, D_, 0, 0, &bytes));
    std::vector<void*> peers;
    if (comm != nullptr) {
      region_ = comm->symm_alloc(bytes, peers);
    } else {
      uint8_t handle[EPSB_IPC_HANDLE_BYTES];
      raise_if(epsb_symm_alloc(bytes, &region_, handle));
      peers.assign(1, region_);
    }
    raise_if(epsb_exchange_create(rank_, W_, max_tok, 1, 1, D_, 0, 0, peers.data(), &x_));
    rows_ = (int64_t)max_tok * W_;
    auto dev = at::TensorOptions().device(at::kCUDA, at::cuda::current_device()).dtype(at::kInt);
    mapping_ = at::empty({max_ids_}, dev);
    send_map_ = at::empty({max_ids_}, dev);
    plan_ = at::zeros({W_ + 4}, dev);   // send_incl [W], then status [4]
  }

  ~FastOEP() {
    epsb_exchange_destroy(x_);
    if (comm_ != nullptr) comm_->symm_free(region_);
    else epsb_symm_free(region_);
  }

  void dispatch(const int32_t* ids, int64_t n, cudaStream_t st) {
    if (n > max_ids_ || n > rows_) throw std::runtime_error("ids exceed max_num_global_tokens");
    int32_t* send_incl = plan_.data_ptr<int32_t>();
    raise_if(epsb_oep_arrange_plan(ids, n, size_per_rank_, W_, send_incl, mapping_.data_ptr<int32_t>(),
                                   send_map_.data_ptr<int32_t>(), st));
    raise_if(epsb_exchange_begin(x_, nullptr));
    raise_if(epsb_exchange_publish_plans(x_, send_incl, send_incl, 1, st));
    raise_if(epsb_exchange_recv_plans(x_, 1, nullptr, send_incl + W_, 0, st));
    raise_if(epsb_exchange_put_ids(x_, EPSB_FLAG_META, ids, send_map_.data_ptr<int32_t>(), send_incl, n, st));
    raise_if(epsb_exchange_wait(x_, EPSB_FLAG_META, send_incl + W_, 0, st));
    n_ = n;
    dispatched_ = true;
  }

  void combine(void* out, int64_t n_grams, bool do_permute, const void* embed_table, cudaStream_t st) {
    if (!dispatched_) throw std::runtime_error("combine called before dispatch");
    int32_t* status = plan_.data_ptr<int32_t>() + W_;
    const int slot = EPSB_FLAG_COMBINE(1, 0);
    raise_if(epsb_exchange_lookup_put(x_, slot, embed_table, size_per_rank_, rows_, st));
    raise_if(epsb_exchange_wait(x_, slot, status, 0, st));
    void* rows = nullptr;
    raise_if(epsb_exchange_arena(x_, EPSB_ARENA_OUT, 0, &rows));
    raise_if(epsb_oep_scatter(rows, mapping_.data_ptr<int32_t>(), n_, D_ * 2, n_grams, do_permute ? 1 : 0, out, st));
  }

  int64_t embed_dim() const { return D_; }
  int64_t size_per_rank() const { return size_per_rank_; }
  int64_t num_ids() const { return n_; }

 private:
  int64_t D_, size_per_rank_, max_ids_ = 1, rows_ = 1, n_ = 0;
  int W_ = 1, rank_ = 0;
  Communicator* comm_;
  void* region_ = nullptr;
  epsb_exchange_t* x_ = nullptr;
  at::Tensor mapping_, send_map_, plan_;
  bool dispatched_ = false;
};

FastOEP* oep(fptr_t p) {
  TORCH_CHECK(p != 0, "fast_oep handle is null");
  return reinterpret_cast<FastOEP*>(p);
}

fptr_t create(int64_t embed_dim, int64_t size_per_rank, int64_t max_num_global_tokens, fptr_t comm) {
  return reinterpret_cast<fptr_t>(
      new FastOEP(embed_dim, size_per_rank, max_num_global_tokens, reinterpret_cast<Communicator*>(comm)));
}
void destroy(fptr_t ptr) { delete reinterpret_cast<FastOEP*>(ptr); }

void dispatch(fptr_t ptr, const at::Tensor& ids) {
  TORCH_CHECK(ids.is_cuda() && ids.is_contiguous(), "ids must be a contiguous CUDA tensor");
  TORCH_CHECK(ids.scalar_type() == at::kInt, "ids must be of type kInt32");
  oep(ptr)->dispatch(ids.data_ptr<int32_t>(), ids.numel(), current_stream());
}

void combine(fptr_t ptr, at::Tensor& out, int64_t /*num_global_tokens*/, int64_t n_grams, bool do_permute,
             const at::Tensor& embed_table) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && embed_table.is_cuda() && embed_table.is_contiguous(),
              "out and embed_table must be contiguous CUDA tensors");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && embed_table.scalar_type() == at::kBFloat16,
              "out and embed_table must be bfloat16");
  check(embed_table, 2, "embed_table");
  TORCH_CHECK(embed_table.size(0) == oep(ptr)->size_per_rank() && embed_table.size(1) == oep(ptr)->embed_dim(),
              "embed_table must be [size_per_rank, embed_dim]");
  TORCH_CHECK(out.numel() == oep(ptr)->num_ids() * oep(ptr)->embed_dim(), "out must hold one row per dispatched id");
  oep(ptr)->combine(out.data_ptr(), n_grams, do_permute, embed_table.data_ptr(), current_stream());
}

}  // namespace

TORCH_LIBRARY(fast_oep, m) {
  m.def("all_to_all_create", &create);
  m.def("all_to_all_destroy", &destroy);
  m.def("all_to_all_dispatch", &dispatch);
  m.def("all_to_all_combine", &combine);
}

EPSB_REGISTER_EXTENSION(libfast_oep)
