// dl::kernels -- functions this library adds beside the reference's (declared in this
// repository's include/dl/kernels/kernels.hpp only): the fused chain, the bias + ReLU
// epilogue and layernorm with gamma / beta.  Same forwarding convention as kernels_shim.cpp.
#include <dl/kernels/kernels.hpp>

#include <dl/core/CudaUtils.hpp>

#include <fdl_kernels.h>

namespace dl::kernels {

namespace {
using dl::cuda::check_fdl;
constexpr void* kLegacyStream = nullptr;
}  // namespace

void add_row_bias_relu(float* output, const float* bias, int rows, int cols) {
    check_fdl(fdl_add_row_bias_relu_f32(output, bias, rows, cols, kLegacyStream), "add_row_bias_relu kernel");
}

void layernorm_affine(const float* input, const float* gamma, const float* beta, float* output, int rows,
                      int cols, float eps) {
    check_fdl(fdl_layernorm_rows_f32(input, gamma, beta, output, nullptr, nullptr, rows, cols, eps,
                                     kLegacyStream),
              "layernorm kernel");
}

void mul_add_relu(const float* a, const float* b, const float* c, float* out, int64_t n) {
    check_fdl(fdl_mul_add_relu_f32(a, b, c, out, n, kLegacyStream), "mul_add_relu kernel");
}

}  // namespace dl::kernels
