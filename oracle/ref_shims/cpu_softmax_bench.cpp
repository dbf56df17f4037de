// C ABI over softmax_cpu of the reference's softmax benchmark, compiled in place
// (host-only translation unit; built with g++ -x c++).  Test infrastructure only.
#include <cstddef>

#include "tests/benchmarks/softmax/softmax_benchmark.cu"

extern "C" int ref_cpu_softmax_bench(const float* x, float* out, std::size_t rows, std::size_t cols) {
    softmax_cpu(x, out, rows, cols);
    return 0;
}
