// The expert-parallel communicator behind the `communication` ops: one NVSwitch box, W <= 8 ranks.
//
// Takes the place of the reference's MscclppCommunicator (src/communication/msccl_comm.cuh:14-120,
// msccl_comm.cu:20-120): created from a unique id + (rank, world, ranks per node), offers a barrier and is handed
// to Scheduler / FastEP / TPDPConvertor as a raw pointer.  The reference bootstraps over TCP and registers memory
// with mscclpp; here the unique id is an NCCL id, the NCCL communicator carries the set-up traffic (the 64-byte
// CUDA IPC handles of the symmetric regions) and the barrier, and the data path is this library's own peer-store
// kernels (include/eps_b200.h, "Expert-parallel exchange over peer memory").
#pragma once

#include <nccl.h>

#include <cstring>
#include <vector>

#include "host_common.hpp"

namespace epsb_host {

inline void nccl_ok(ncclResult_t r, const char* what) {
  if (r != ncclSuccess) throw std::runtime_error(std::string(what) + ": " + ncclGetErrorString(r));
}

class Communicator {
 public:
  static constexpr int kUniqueIdBytes = (int)sizeof(ncclUniqueId);

  static void make_unique_id(uint8_t* out) {
    ncclUniqueId id;
    nccl_ok(ncclGetUniqueId(&id), "ncclGetUniqueId");
    std::memcpy(out, &id, sizeof(id));
  }

  Communicator(const uint8_t* unique_id, int rank, int world, int ranks_per_node)
      : rank_(rank), world_(world), ranks_per_node_(ranks_per_node) {
    if (world < 1 || rank < 0 || rank >= world) throw std::runtime_error("bad rank / ep_world_size");
    if (world > EPSB_MAX_PEERS)
      throw std::runtime_error("ep_world_size " + std::to_string(world) + " exceeds " + std::to_string(EPSB_MAX_PEERS));
    if (world != ranks_per_node)
      throw std::runtime_error("multi-node expert parallelism is not supported: one NVSwitch box only");
    cuda_ok(cudaGetDevice(&device_), "cudaGetDevice");
    if (world > 1) {
      ncclUniqueId id;
      std::memcpy(&id, unique_id, sizeof(id));
      nccl_ok(ncclCommInitRank(&nccl_, world, id, rank), "ncclCommInitRank");
      cuda_ok(cudaMalloc(&scratch_, (size_t)(world + 1) * EPSB_IPC_HANDLE_BYTES), "cudaMalloc(comm scratch)");
    }
  }

  ~Communicator() {
    for (auto& r : regions_) release(r);
    if (scratch_ != nullptr) cudaFree(scratch_);
    if (nccl_ != nullptr) ncclCommDestroy(nccl_);
  }

  int getRank() const { return rank_; }
  int getWorldSize() const { return world_; }
  int getNumRanksPerNode() const { return ranks_per_node_; }
  ncclComm_t nccl() const { return nccl_; }

  void barrier() {
    if (world_ == 1) return;
    cudaStream_t st = current_stream();
    nccl_ok(ncclAllReduce(scratch_, scratch_, 1, ncclInt32, ncclSum, nccl_, st), "ncclAllReduce(barrier)");
    cuda_ok(cudaStreamSynchronize(st), "barrier");
  }

  // Collective.  Zeroed device memory on every rank, mapped into every process: peers[r] = rank r's block here.
  void* symm_alloc(int64_t bytes, std::vector<void*>& peers) {
    Region reg;
    uint8_t handle[EPSB_IPC_HANDLE_BYTES];
    raise_if(epsb_symm_alloc(bytes, &reg.local, handle));
    reg.peers.assign(world_, reg.local);
    if (world_ > 1) {
      cudaStream_t st = current_stream();
      uint8_t* mine = static_cast<uint8_t*>(scratch_);
      uint8_t* all = mine + EPSB_IPC_HANDLE_BYTES;
      cuda_ok(cudaMemcpyAsync(mine, handle, sizeof(handle), cudaMemcpyHostToDevice, st), "handle upload");
      nccl_ok(ncclAllGather(mine, all, EPSB_IPC_HANDLE_BYTES, ncclUint8, nccl_, st), "ncclAllGather(handles)");
      std::vector<uint8_t> host((size_t)world_ * EPSB_IPC_HANDLE_BYTES);
      cuda_ok(cudaMemcpyAsync(host.data(), all, host.size(), cudaMemcpyDeviceToHost, st), "handle download");
      cuda_ok(cudaStreamSynchronize(st), "handle exchange");
      for (int r = 0; r < world_; r++) {
        if (r == rank_) continue;
        raise_if(epsb_symm_open(host.data() + (size_t)r * EPSB_IPC_HANDLE_BYTES, &reg.peers[r]));
      }
      barrier();
    }
    peers = reg.peers;
    regions_.push_back(reg);
    return reg.local;
  }

  // Collective.  No rank may still be writing into the block.
  void symm_free(void* local) {
    for (size_t i = 0; i < regions_.size(); i++)
      if (regions_[i].local == local) {
        if (world_ > 1) {
          cuda_ok(cudaDeviceSynchronize(), "symm_free");
          barrier();
        }
        release(regions_[i]);
        regions_.erase(regions_.begin() + (long)i);
        if (world_ > 1) barrier();
        return;
      }
  }

 private:
  struct Region {
    void* local = nullptr;
    std::vector<void*> peers;
  };
  void release(Region& r) {
    for (int p = 0; p < (int)r.peers.size(); p++)
      if (p != rank_ && r.peers[p] != nullptr && r.peers[p] != r.local) epsb_symm_close(r.peers[p]);
    if (r.local != nullptr) epsb_symm_free(r.local);
    r.local = nullptr;
    r.peers.clear();
  }

  int rank_, world_, ranks_per_node_, device_ = 0;
  ncclComm_t nccl_ = nullptr;
  void* scratch_ = nullptr;
  std::vector<Region> regions_;
};

}  // namespace epsb_host
