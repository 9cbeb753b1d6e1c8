// Stand-in for the mscclpp header of this name.  The reference's quant/fp8.cuh and fast_ep_kernels.cuh include it
// only to NAME types (channel handles in parameter structs, the communicator class); its fast_ep kernels call put /
// signal / wait on the handles, which here do nothing (the test harness fills the tables those calls would fill).
// Declarations only, written for the witness build; test infrastructure, not product code.
#pragma once
#include "core.hpp"
namespace mscclpp {
struct SmChannel {};
template <> struct DeviceHandle<SmChannel> {
  template <int A> __device__ void put(uint64_t, uint64_t, uint64_t, uint32_t, uint32_t) {}
  __device__ void wait(int64_t) {}
  __device__ void signal() {}
};
}
