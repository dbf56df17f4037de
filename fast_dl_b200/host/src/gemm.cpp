// dl::kernels::gemm -- out of the bandwidth path; a plain cuBLAS SGEMM so that matmul and
// linear keep working.  One handle per device for the life of the process (the reference
// creates and destroys one per call, src/kernels/cuda/gemm.cu:166-177).
#include <dl/kernels/kernels.hpp>

#include <cublas_v2.h>
#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>

namespace dl::kernels {

namespace {
std::mutex g_mutex;
cublasHandle_t g_handle[64] = {};

cublasHandle_t handle_for_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        throw std::runtime_error("gemm: no current CUDA device");
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_handle[dev] == nullptr) {
        if (cublasCreate(&g_handle[dev]) != CUBLAS_STATUS_SUCCESS) {
            throw std::runtime_error("cublasCreate failed");
        }
        // fp32 multiply-add, no TF32: the reference's pedantic mode.
        cublasSetMathMode(g_handle[dev], CUBLAS_PEDANTIC_MATH);
    }
    return g_handle[dev];
}
}  // namespace

void gemm(const float* a, const float* b, float* c, int m, int n, int k, GemmAlgo) {
    if (m <= 0 || n <= 0) return;
    cublasHandle_t h = handle_for_current_device();
    cublasSetStream(h, nullptr);
    const float one = 1.0f, zero = 0.0f;
    // Row-major C[m,n] = A[m,k] B[k,n] is column-major C^T = B^T A^T.
    if (cublasSgemm(h, CUBLAS_OP_N, CUBLAS_OP_N, n, m, k, &one, b, n, a, k, &zero, c, n) !=
        CUBLAS_STATUS_SUCCESS) {
        throw std::runtime_error("cublasSgemm failed");
    }
}

}  // namespace dl::kernels
