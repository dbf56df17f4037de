// Runs the reference's CPU functions over row/element ranges on several host threads, for
// the timed CPU baseline.  Each thread calls the unmodified reference function on its own
// contiguous slice, so results equal the single-threaded ones for these row- and
// element-independent operations.  Test infrastructure only.
#include <algorithm>
#include <cstddef>
#include <thread>
#include <vector>

extern "C" {
int ref_cpu_activation(const float*, float*, std::size_t, int, float);
int ref_cpu_vector_add(const float*, const float*, float*, std::size_t);
int ref_cpu_softmax_bench(const float*, float*, std::size_t, std::size_t);
int ref_cpu_layernorm(const float*, float*, std::size_t, std::size_t, float);
int ref_cpu_block_reduce(const float*, float*, std::size_t, int);
}

namespace {
template <class Fn>
void parallel_ranges(std::size_t n, std::size_t granule, int threads, Fn fn) {
    if (threads < 1) threads = 1;
    const std::size_t units = (n + granule - 1) / granule;
    const std::size_t per = (units + threads - 1) / threads;
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) {
        const std::size_t b = std::min(n, t * per * granule);
        const std::size_t e = std::min(n, (t + 1) * per * granule);
        if (b >= e) break;
        pool.emplace_back([=] { fn(b, e); });
    }
    for (auto& th : pool) th.join();
}
}  // namespace

extern "C" {

int ref_cpu_hardware_threads() { return static_cast<int>(std::thread::hardware_concurrency()); }

int ref_cpu_vector_add_mt(const float* a, const float* b, float* c, std::size_t n, int threads) {
    parallel_ranges(n, 4096, threads, [=](std::size_t lo, std::size_t hi) {
        ref_cpu_vector_add(a + lo, b + lo, c + lo, hi - lo);
    });
    return 0;
}

int ref_cpu_activation_mt(const float* x, float* y, std::size_t n, int op, float alpha, int threads) {
    parallel_ranges(n, 4096, threads, [=](std::size_t lo, std::size_t hi) {
        ref_cpu_activation(x + lo, y + lo, hi - lo, op, alpha);
    });
    return 0;
}

int ref_cpu_softmax_mt(const float* x, float* y, std::size_t rows, std::size_t cols, int threads) {
    parallel_ranges(rows, 1, threads, [=](std::size_t lo, std::size_t hi) {
        ref_cpu_softmax_bench(x + lo * cols, y + lo * cols, hi - lo, cols);
    });
    return 0;
}

int ref_cpu_layernorm_mt(const float* x, float* y, std::size_t rows, std::size_t cols, float eps,
                         int threads) {
    parallel_ranges(rows, 1, threads, [=](std::size_t lo, std::size_t hi) {
        ref_cpu_layernorm(x + lo * cols, y + lo * cols, hi - lo, cols, eps);
    });
    return 0;
}

int ref_cpu_block_reduce_mt(const float* x, float* out, std::size_t n, int tree, int threads) {
    const std::size_t blocks = n / 1024;
    parallel_ranges(blocks, 1, threads, [=](std::size_t lo, std::size_t hi) {
        ref_cpu_block_reduce(x + lo * 1024, out + lo, (hi - lo) * 1024, tree);
    });
    return 0;
}

}  // extern "C"
