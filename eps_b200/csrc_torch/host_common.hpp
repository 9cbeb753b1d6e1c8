// Shared pieces of the torch-op libraries (libscheduler_.so, libexecutor_.so, libfast_ep.so, libfast_oep.so,
// libcommunication_.so, libutils_.so): tensor checks in the style of the reference's src/common/torch_utils.h:39-44,
// error translation from the C ABI (the reference throws std::runtime_error), and the PyInit stub of
// src/registration.h:19-26 that lets `import` load the library.
#pragma once

#include <Python.h>

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <cuda_runtime.h>
#include <torch/library.h>

#include <stdexcept>
#include <string>

#include "../../include/eps_b200.h"

namespace epsb_host {

using fptr_t = int64_t;

inline void check(const at::Tensor& t, int64_t dim, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.dim() == dim, name, " must have ", dim, " dimensions");
}

inline void raise_if(int rc) {
  if (rc != EPSB_OK) throw std::runtime_error(epsb_last_error());
}

inline void cuda_ok(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

inline cudaStream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline bool is_fp8_codes(const at::Tensor& t) {
  return t.scalar_type() == at::kByte || t.scalar_type() == at::kFloat8_e4m3fn;
}

}  // namespace epsb_host

#define EPSB_REGISTER_EXTENSION(NAME)                                                             \
  PyMODINIT_FUNC PyInit_##NAME() {                                                                \
    static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, #NAME, nullptr, 0, nullptr};       \
    return PyModule_Create(&module);                                                              \
  }
