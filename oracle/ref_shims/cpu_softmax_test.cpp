// C ABI over softmax_cpu of the reference's softmax tensor test, compiled in place.
// Test infrastructure only.
#include <cstddef>
#include <cstring>
#include <vector>

#define main static ref_softmax_test_main_unused
#include "tests/tensor/softmax_tensor_test.cpp"
#undef main

extern "C" int ref_cpu_softmax_test(const float* x, float* out, std::size_t rows, std::size_t cols) {
    const std::vector<float> in(x, x + rows * cols);
    const std::vector<float> res = softmax_cpu(in, rows, cols);
    std::memcpy(out, res.data(), rows * cols * sizeof(float));
    return 0;
}
