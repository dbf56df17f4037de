// dl::kernels -- the reference's kernel-level functions as forwards into the C ABI.
//
// This file defines exactly the functions that fast_dl's include/dl/kernels/*.hpp declare and
// depends on nothing else of the host library, so the same source compiles against
// fast_dl's own headers: there it is the "forwarding source" that replaces the seven
// hot-path .cu files of dl_cuda_kernels behind an unmodified dl_core (CMakeLists.txt:44-56, 75).
// A signature that drifts from the reference's header is then a compile or link error.
// Functions this library adds to the namespace live in kernels_ext.cpp.
#include <dl/kernels/kernels.hpp>

#include <fdl_kernels.h>

#include <stdexcept>
#include <string>

namespace dl::kernels {

namespace {
constexpr void* kLegacyStream = nullptr;  // what the reference launches on

// The reference's kernel functions return void and its callers ask cudaGetLastError; a
// failure reported by the C ABI surfaces as std::runtime_error("<action>: <text>"), the
// form of dl::cuda::check (src/core/CudaUtils.cpp:8-13).
void check_fdl(int status, const char* action) {
    if (status != FDL_OK) throw std::runtime_error(std::string(action) + ": " + fdl_error_string(status));
}
}  // namespace

const char* to_string(ElementwiseOp op) {
    static const char* const names[] = {"add", "sub", "mul", "div"};
    const int i = static_cast<int>(op);
    return i >= 0 && i < 4 ? names[i] : "unknown";
}
const char* to_string(VectorAddAlgo algo) { return algo == VectorAddAlgo::Naive ? "naive" : "unknown"; }
const char* to_string(ActivationOp op) {
    static const char* const names[] = {"relu", "leaky_relu", "gelu", "sigmoid", "tanh"};
    const int i = static_cast<int>(op);
    return i >= 0 && i < 5 ? names[i] : "unknown";
}
const char* to_string(ReductionAlgo algo) {
    return algo == ReductionAlgo::Interleave ? "interleave" : algo == ReductionAlgo::Address ? "address" : "unknown";
}
const char* to_string(SoftmaxAlgo algo) {
    static const char* const names[] = {"naive", "shared_memory", "warp_shuffle_reg_cache"};
    const int i = static_cast<int>(algo);
    return i >= 0 && i < 3 ? names[i] : "unknown";
}
const char* to_string(TransposeAlgo algo) {
    static const char* const names[] = {"naive", "shared", "padding"};
    const int i = static_cast<int>(algo);
    return i >= 0 && i < 3 ? names[i] : "unknown";
}
const char* to_string(GemmAlgo algo) {
    static const char* const names[] = {"naive", "tiled", "register", "cublas"};
    const int i = static_cast<int>(algo);
    return i >= 0 && i < 4 ? names[i] : "unknown";
}

void elementwise(const float* a, const float* b, float* c, int n, ElementwiseOp op) {
    check_fdl(fdl_binary_f32(a, b, c, n, static_cast<int>(op), kLegacyStream), "elementwise kernel");
}

void vector_add(const float* a, const float* b, float* c, std::size_t size, VectorAddAlgo) {
    check_fdl(fdl_binary_f32(a, b, c, static_cast<int64_t>(size), FDL_ADD, kLegacyStream), "vector_add kernel");
}

void activation(const float* a, float* b, int n, ActivationOp op, float alpha) {
    const int code = static_cast<int>(op);
    if (code < FDL_RELU || code > FDL_TANH) throw std::runtime_error("Unsupported activation type");
    check_fdl(fdl_unary_f32(a, b, n, code, alpha, kLegacyStream), "activation kernel");
}

void add_row_bias(float* output, const float* bias, int rows, int cols) {
    check_fdl(fdl_add_row_bias_f32(output, bias, rows, cols, kLegacyStream), "add_row_bias kernel");
}

void reduction(const float* input, float* output, std::size_t size, ReductionAlgo algo) {
    check_fdl(fdl_block_reduce_1024_f32(input, output, static_cast<int64_t>(size), static_cast<int>(algo),
                                        kLegacyStream),
              "reduction kernel");
}

void softmax(const float* input, float* output, std::size_t rows, std::size_t cols, SoftmaxAlgo) {
    check_fdl(fdl_softmax_rows_f32(input, output, static_cast<int64_t>(rows), static_cast<int64_t>(cols),
                                   kLegacyStream),
              "softmax kernel");
}

void layernorm(const float* input, float* output, int rows, int cols, float eps) {
    check_fdl(fdl_layernorm_rows_f32(input, nullptr, nullptr, output, nullptr, nullptr, rows, cols, eps,
                                     kLegacyStream),
              "layernorm kernel");
}

void cross_entropy(const float* logits, const int64_t* labels, float* loss, int batch, int classes) {
    check_fdl(fdl_cross_entropy_f32(logits, labels, loss, batch, classes, kLegacyStream), "cross_entropy kernel");
}

void transpose(const float* input, float* output, std::size_t size, TransposeAlgo) {
    check_fdl(fdl_transpose_f32(input, output, static_cast<int64_t>(size), kLegacyStream), "transpose kernel");
}

void uniform_float32(float* data, int64_t n, float low, float high, uint64_t seed) {
    check_fdl(fdl_uniform_f32(data, n, low, high, seed, kLegacyStream), "uniform kernel");
}

void normal_float32(float* data, int64_t n, float mean, float stddev, uint64_t seed) {
    check_fdl(fdl_normal_f32(data, n, mean, stddev, seed, kLegacyStream), "normal kernel");
}

}  // namespace dl::kernels
