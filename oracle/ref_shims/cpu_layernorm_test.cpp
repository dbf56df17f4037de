// C ABI over layernorm_cpu of the reference's layernorm tensor test, compiled in place.
// Test infrastructure only.
#include <cstddef>
#include <cstring>
#include <vector>

#define main static ref_layernorm_test_main_unused
#include "tests/tensor/layernorm_tensor_test.cpp"
#undef main

extern "C" int ref_cpu_layernorm(const float* x, float* out, std::size_t rows, std::size_t cols, float eps) {
    const std::vector<float> in(x, x + rows * cols);
    const std::vector<float> res = layernorm_cpu(in, rows, cols, eps);
    std::memcpy(out, res.data(), rows * cols * sizeof(float));
    return 0;
}
