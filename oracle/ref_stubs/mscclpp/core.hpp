// Stand-in for the mscclpp header of this name.  The reference's quant/fp8.cuh and fast_ep_kernels.cuh include it
// only to NAME types (channel handles in parameter structs, the communicator class); its fast_ep kernels call put /
// signal / wait on the handles, which here do nothing (the test harness fills the tables those calls would fill).
// Declarations only, written for the witness build; test infrastructure, not product code.
#pragma once
#include <cstdint>
#include <memory>
#include <vector>
#include <unordered_map>
#include <tuple>
#include <string>
namespace mscclpp {
template <typename T> struct DeviceHandle {};
struct UniqueId { char bytes[128]; };
struct TcpBootstrap { static UniqueId createUniqueId() { return UniqueId{}; } };
enum class Transport { Unknown };
struct Bootstrap { void barrier() {} };
class Communicator { public: std::shared_ptr<Bootstrap> bootstrap() { return nullptr; } };
class Connection {};
class ProxyService {};
class SmDevice2DeviceSemaphore {};
template <typename T> struct CudaDeleter { void operator()(void*) const {} };
}
