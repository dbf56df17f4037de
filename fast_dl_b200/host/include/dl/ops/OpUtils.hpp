// Argument checks shared by the ops.  Each throws std::runtime_error with the message
// "<op>: <tensor name> tensor ..." that fast_dl's checks produce (src/ops/OpUtils.cpp:20-101),
// so callers and tests that match on the text keep working.
#pragma once

#include <cstdint>
#include <vector>

#include <dl/tensor/Tensor.hpp>

namespace dl::ops {

void check_defined(const Tensor& t, const char* op, const char* name = "input");
void check_rank(const Tensor& t, int64_t rank, const char* op, const char* name = "input");
void check_cuda(const Tensor& t, const char* op, const char* name = "input");
void check_dtype(const Tensor& t, DType dtype, const char* op, const char* name = "input");
void check_float32(const Tensor& t, const char* op, const char* name = "input");
void check_same_device(const Tensor& a, const Tensor& b, const char* op,
                       const char* a_name = "left", const char* b_name = "right");
void check_same_dtype(const Tensor& a, const Tensor& b, const char* op,
                      const char* a_name = "left", const char* b_name = "right");
void check_same_shape(const Tensor& a, const Tensor& b, const char* op,
                      const char* a_name = "left", const char* b_name = "right");
/// defined, same shape, same dtype, Float32, CUDA, same device -- in the reference's order.
void check_binary_float_cuda_op(const Tensor& a, const Tensor& b, const char* op);

/// NumPy broadcast of two shapes.  Returns false when they do not broadcast.  On success
/// fills the output shape and per-dimension element strides (0 in broadcast dimensions).
bool broadcast_shapes(const Shape& a, const Shape& b, std::vector<int64_t>* out,
                      std::vector<int64_t>* a_strides, std::vector<int64_t>* b_strides);

}  // namespace dl::ops
