// Stand-in for the mscclpp header that the reference's quant/fp8.cuh includes only to name one
// pointer type in a parameter struct (quant/fp8.cuh:26-33).  Test infrastructure; not product code.
#pragma once
namespace mscclpp {
template <typename T>
struct DeviceHandle {};
struct SmChannel {};
}  // namespace mscclpp
