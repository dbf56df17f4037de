// Error plumbing between CUDA / the kernel library and C++ exceptions.
#pragma once

#include <cuda_runtime.h>

namespace dl::cuda {

/// Throws std::runtime_error("<action>: <cudaGetErrorString>") unless `status` is cudaSuccess.
/// Same contract as fast_dl's dl::cuda::check (src/core/CudaUtils.cpp:8-13).
void check(cudaError_t status, const char* action);

/// Same for a status returned by the C ABI of the kernel library (fdl_* functions):
/// message "<action>: <fdl_error_string(status)>".
void check_fdl(int status, const char* action);

/// Makes `device_index` current both in this library's CUDA runtime and in the kernel
/// library's (they may be separate runtime instances when linked statically).
void set_device(int device_index);

/// Number of visible CUDA devices (0 when there is no driver).
int device_count();

/// Blocks until all work enqueued on the current device has finished.
void synchronize();

}  // namespace dl::cuda
