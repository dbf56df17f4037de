// dl::ops -- tensor-level operations.  Names, argument meaning, defaults and error strings
// follow fast_dl's include/dl/ops/*.hpp; each op validates, allocates the result, selects the
// device, calls dl::kernels / the C ABI and checks the launch, in the order of
// run_elementwise (src/ops/Elementwise.cpp:36-50).
//
// Extensions, all API-compatible with what was there:
//   * add/sub/mul/div (and operators) accept NumPy-broadcastable shapes; equal shapes behave
//     exactly as before, non-broadcastable ones raise the reference's
//     "... tensors must have the same shape" error;
//   * sum / mean / max / argmax along an axis, full sum (fast_dl has none, FUTURE_WORK.md:84-92
//     gives the pattern new ops should follow);
//   * layernorm with gamma and beta; mul_add_relu; linear with a fused ReLU epilogue.
#pragma once

#include <cstdint>

#include <dl/tensor/Tensor.hpp>

namespace dl::ops {

// ---- Elementwise.hpp ----
Tensor add(const Tensor& a, const Tensor& b);
Tensor sub(const Tensor& a, const Tensor& b);
Tensor mul(const Tensor& a, const Tensor& b);
Tensor div(const Tensor& a, const Tensor& b);
/// relu(a*b + c) in one pass, bit-identical to relu(add(mul(a, b), c)).
Tensor mul_add_relu(const Tensor& a, const Tensor& b, const Tensor& c);

// ---- Activation.hpp ----
Tensor relu(const Tensor& a);
Tensor leaky_relu(const Tensor& a, float alpha = 0.01f);
Tensor gelu(const Tensor& a);
Tensor sigmoid(const Tensor& a);
Tensor tanh(const Tensor& a);

// ---- Softmax.hpp / LayerNorm.hpp (rank-2 inputs, along the last axis) ----
Tensor softmax(const Tensor& input);
Tensor layernorm(const Tensor& input, float eps = 1.0e-5f);
/// (x - mean) * rstd * gamma + beta; gamma and beta have shape [cols].
Tensor layernorm(const Tensor& input, const Tensor& gamma, const Tensor& beta, float eps = 1.0e-5f);

// ---- reductions (new).  `axis` may be negative; the reduced axis is removed. ----
/// Sum of all elements, shape {1} (fast_dl has no rank-0 tensors: src/core/Shape.cpp:17-20).
Tensor sum(const Tensor& input);
Tensor sum(const Tensor& input, int axis);
Tensor mean(const Tensor& input, int axis);
Tensor max(const Tensor& input, int axis);
/// Int64 indices of the maximum along the LAST axis; ties go to the lowest index.
Tensor argmax(const Tensor& input, int axis);

// ---- Matmul.hpp / Linear.hpp / CrossEntropy.hpp ----
Tensor matmul(const Tensor& a, const Tensor& b);
Tensor linear(const Tensor& input, const Tensor& weight, const Tensor& bias);
/// relu(linear(...)) with bias add and ReLU fused into one pass over the GEMM output.
Tensor linear_relu(const Tensor& input, const Tensor& weight, const Tensor& bias);
Tensor cross_entropy(const Tensor& logits, const Tensor& labels);

}  // namespace dl::ops

namespace dl {
Tensor operator+(const Tensor& a, const Tensor& b);
Tensor operator-(const Tensor& a, const Tensor& b);
Tensor operator*(const Tensor& a, const Tensor& b);
Tensor operator/(const Tensor& a, const Tensor& b);
}  // namespace dl
