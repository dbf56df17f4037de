// C ABI over vector_add_cpu of the reference's vector_add benchmark, compiled in place
// (host-only translation unit; built with g++ -x c++).  Test infrastructure only.
#include <cstddef>

#include "tests/benchmarks/vector_add/vector_add_benchmark.cu"

extern "C" int ref_cpu_vector_add(const float* a, const float* b, float* c, std::size_t n) {
    vector_add_cpu(a, b, c, n);
    return 0;
}
