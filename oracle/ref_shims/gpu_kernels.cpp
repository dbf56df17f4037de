// C ABI over the reference's own CUDA kernel launchers (dl::kernels::*), which are compiled
// in place for sm_100a into the same shared object.  Used on a GPU box as the same-device
// parity oracle and speed bar.  Test infrastructure only.
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include <dl/kernels/kernels.hpp>

namespace k = dl::kernels;

extern "C" {

int ref_gpu_set_device(int dev) { return static_cast<int>(cudaSetDevice(dev)); }
int ref_gpu_sync() { return static_cast<int>(cudaDeviceSynchronize()); }

int ref_gpu_elementwise(const float* a, const float* b, float* c, int n, int op) {
    k::elementwise(a, b, c, n, static_cast<k::ElementwiseOp>(op));
    return static_cast<int>(cudaGetLastError());
}
int ref_gpu_activation(const float* x, float* y, int n, int op, float alpha) {
    k::activation(x, y, n, static_cast<k::ActivationOp>(op), alpha);
    return static_cast<int>(cudaGetLastError());
}
int ref_gpu_vector_add(const float* a, const float* b, float* c, std::size_t n) {
    k::vector_add(a, b, c, n, k::VectorAddAlgo::Naive);
    return static_cast<int>(cudaGetLastError());
}
int ref_gpu_add_row_bias(float* out, const float* bias, int rows, int cols) {
    k::add_row_bias(out, bias, rows, cols);
    return static_cast<int>(cudaGetLastError());
}
int ref_gpu_reduction(const float* x, float* out, std::size_t n, int algo) {
    k::reduction(x, out, n, static_cast<k::ReductionAlgo>(algo));
    return static_cast<int>(cudaGetLastError());
}
int ref_gpu_softmax(const float* x, float* y, std::size_t rows, std::size_t cols, int algo) {
    k::softmax(x, y, rows, cols, static_cast<k::SoftmaxAlgo>(algo));
    return static_cast<int>(cudaGetLastError());
}
int ref_gpu_layernorm(const float* x, float* y, int rows, int cols, float eps) {
    k::layernorm(x, y, rows, cols, eps);
    return static_cast<int>(cudaGetLastError());
}

int ref_gpu_cross_entropy(const float* logits, const long long* labels, float* loss, int batch, int classes) {
    // as dl::ops::cross_entropy does (src/ops/CrossEntropy.cpp): the kernel accumulates into *loss
    cudaMemset(loss, 0, sizeof(float));
    k::cross_entropy(logits, reinterpret_cast<const int64_t*>(labels), loss, batch, classes);
    return static_cast<int>(cudaGetLastError());
}
int ref_gpu_transpose(const float* in, float* out, std::size_t n, int algo) {
    k::transpose(in, out, n, static_cast<k::TransposeAlgo>(algo));
    return static_cast<int>(cudaGetLastError());
}
int ref_gpu_uniform(float* data, long long n, float low, float high, unsigned long long seed) {
    k::uniform_float32(data, n, low, high, seed);
    return static_cast<int>(cudaGetLastError());
}
int ref_gpu_normal(float* data, long long n, float mean, float stddev, unsigned long long seed) {
    k::normal_float32(data, n, mean, stddev, seed);
    return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
