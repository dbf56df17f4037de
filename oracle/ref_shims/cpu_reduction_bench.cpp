// C ABI over the two tree-order CPU sums of the reference's reduction benchmark, compiled
// in place (host-only translation unit; built with g++ -x c++).  Test infrastructure only.
#include <cstddef>

#include "tests/benchmarks/reduction/reduction_benchmark.cu"

// tree: 0 interleave, 1 sequential ("address").
extern "C" int ref_cpu_block_reduce(const float* x, float* out, std::size_t n, int tree) {
    if (tree == 0) reduction_interleave_cpu(x, out, n);
    else reduction_sequential_cpu(x, out, n);
    return 0;
}
