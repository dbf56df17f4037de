// Exposes the CPU check functions of the reference's activation test through a C ABI.
// The reference file is compiled IN PLACE (include path = reference root); nothing of it
// is copied here.  Its main() becomes an unused static function and is discarded.
// Test infrastructure only.
#include <cstddef>
#include <cstring>
#include <vector>

#define main static ref_activation_test_main_unused
#include "tests/tensor/activation_tensor_test.cpp"
#undef main

namespace {
template <class Fn>
void run_chunked(const float* x, float* out, std::size_t n, Fn fn) {
    const std::vector<float> in(x, x + n);
    const std::vector<float> res = fn(in);
    std::memcpy(out, res.data(), n * sizeof(float));
}
}  // namespace

// op codes follow dl::kernels::ActivationOp: 0 relu, 1 leaky_relu, 2 gelu, 3 sigmoid, 4 tanh.
extern "C" int ref_cpu_activation(const float* x, float* out, std::size_t n, int op, float alpha) {
    switch (op) {
        case 0: run_chunked(x, out, n, [](const std::vector<float>& v) { return relu_cpu(v); }); return 0;
        case 1: run_chunked(x, out, n, [alpha](const std::vector<float>& v) { return leaky_relu_cpu(v, alpha); }); return 0;
        case 2: run_chunked(x, out, n, [](const std::vector<float>& v) { return gelu_cpu(v); }); return 0;
        case 3: run_chunked(x, out, n, [](const std::vector<float>& v) { return sigmoid_cpu(v); }); return 0;
        case 4: run_chunked(x, out, n, [](const std::vector<float>& v) { return tanh_cpu(v); }); return 0;
        default: return -1;
    }
}
