// dl::kernels -- the kernel-level interface fast_dl's ops are written against
// (include/dl/kernels/*.hpp).  Signatures, enums and default arguments are the reference's;
// the bodies (src/kernels_shim.cpp) forward to the C ABI of the sm_100a kernel library
// (include/fdl_kernels.h) on the legacy default stream.
//
// Conventions kept from the reference: raw device pointers borrowed for the call, the
// caller has selected the device, functions return void.  A failed launch throws
// std::runtime_error here (the reference leaves it to the caller's cudaGetLastError).
// The `...Algo` selectors of the reference's teaching kernels are accepted and, except for
// the two reduction tree orders, all map to the single sm_100a implementation.
#pragma once

#include <cstddef>
#include <cstdint>

namespace dl::kernels {

// ---- elementwise (elementwise.hpp, vector_add.hpp) ----
enum class ElementwiseOp { Add, Sub, Mul, Div };
const char* to_string(ElementwiseOp op);
void elementwise(const float* a, const float* b, float* c, int n, ElementwiseOp op);

enum class VectorAddAlgo { Naive };
const char* to_string(VectorAddAlgo algo);
void vector_add(const float* a, const float* b, float* c, std::size_t size,
                VectorAddAlgo algo = VectorAddAlgo::Naive);

// ---- activations (activation.hpp) ----
enum class ActivationOp { ReLU, LeakyReLU, GELU, Sigmoid, Tanh };
const char* to_string(ActivationOp op);
void activation(const float* a, float* b, int n, ActivationOp op, float alpha = 0.01f);

// ---- row bias (bias.hpp) ----
void add_row_bias(float* output, const float* bias, int rows, int cols);

// ---- 1024-element block sums (reduction.hpp) ----
enum class ReductionAlgo { Interleave, Address };
const char* to_string(ReductionAlgo algo);
void reduction(const float* input, float* output, std::size_t size,
               ReductionAlgo algo = ReductionAlgo::Address);

// ---- row softmax (softmax.hpp) ----
enum class SoftmaxAlgo { Naive, SharedMemory, WarpShuffleRegCache };
const char* to_string(SoftmaxAlgo algo);
void softmax(const float* input, float* output, std::size_t rows, std::size_t cols,
             SoftmaxAlgo algo = SoftmaxAlgo::Naive);

// ---- row layernorm (layernorm.hpp) ----
void layernorm(const float* input, float* output, int rows, int cols, float eps);

// ---- neighbours of the path ----
void cross_entropy(const float* logits, const int64_t* labels, float* loss, int batch, int classes);

enum class TransposeAlgo { Naive, Shared, Padding };
const char* to_string(TransposeAlgo algo);
void transpose(const float* input, float* output, std::size_t size,
               TransposeAlgo algo = TransposeAlgo::Padding);

void uniform_float32(float* data, int64_t n, float low, float high, uint64_t seed);
void normal_float32(float* data, int64_t n, float mean, float stddev, uint64_t seed);

enum class GemmAlgo { Naive, Tiled, Register, Cublas };
const char* to_string(GemmAlgo algo);
/// Row-major C[m,n] = A[m,k] B[k,n]; every algo value runs cuBLAS SGEMM (fp32, no TF32).
void gemm(const float* a, const float* b, float* c, int m, int n, int k,
          GemmAlgo algo = GemmAlgo::Cublas);

// ---- additions (no counterpart in fast_dl) ----
/// out = max(0, a*b + c) with a*b rounded before the add (what mul, add, relu give).
void mul_add_relu(const float* a, const float* b, const float* c, float* out, int64_t n);
/// In place: out[r,c] = max(0, out[r,c] + bias[c]).
void add_row_bias_relu(float* output, const float* bias, int rows, int cols);
/// gamma / beta may be null.
void layernorm_affine(const float* input, const float* gamma, const float* beta, float* output,
                      int rows, int cols, float eps);

}  // namespace dl::kernels
