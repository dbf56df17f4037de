// What a call through the public dl::ops API costs, allocation included, with the caching
// allocator on (this library) and off (one cudaMalloc / cudaFree per tensor, which is what
// the reference does in TensorImpl).  Prints microseconds per call; not a pass/fail test.
#include <dl/core/CudaUtils.hpp>
#include <dl/dl.hpp>
#include <dl/tensor/Allocator.hpp>

#include <chrono>
#include <cstdio>
#include <functional>
#include <vector>

namespace {

double time_us(const std::function<void()>& fn, int iters) {
    for (int i = 0; i < 3; ++i) fn();
    dl::cuda::synchronize();
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < iters; ++i) fn();
    dl::cuda::synchronize();
    const auto t1 = std::chrono::steady_clock::now();
    return std::chrono::duration<double, std::micro>(t1 - t0).count() / iters;
}

void line(const char* name, const std::function<void()>& fn, int iters) {
    dl::allocator::set_caching(true);
    const double cached = time_us(fn, iters);
    dl::allocator::set_caching(false);
    const double uncached = time_us(fn, iters);
    dl::allocator::set_caching(true);
    std::printf("%-46s cached %9.1f us   cudaMalloc/cudaFree per tensor %9.1f us   x%.2f\n", name, cached, uncached,
                uncached / cached);
}

}  // namespace

int main() {
    const dl::Device dev(dl::DeviceType::CUDA, 0);
    auto uniform = [&](dl::Shape s, uint64_t seed) {
        return dl::Tensor::uniform(s, dl::DType::Float32, dev, -1.0f, 1.0f, seed);
    };
    {
        const dl::Tensor a = uniform(dl::Shape({1 << 20}), 1), b = uniform(dl::Shape({1 << 20}), 2),
                         c = uniform(dl::Shape({1 << 20}), 3);
        line("C1 relu(a*b+c), three ops (2^20 elements)", [&] { dl::Tensor y = dl::ops::relu(a * b + c); }, 200);
        line("C1 mul_add_relu, one op", [&] { dl::Tensor y = dl::ops::mul_add_relu(a, b, c); }, 200);
    }
    {
        const dl::Tensor A = uniform(dl::Shape({4096, 4096}), 4), row = uniform(dl::Shape({1, 4096}), 5),
                         col = uniform(dl::Shape({4096, 1}), 6);
        line("C2 (A + b[1,4096]) * s[4096,1]", [&] { dl::Tensor y = (A + row) * col; }, 100);
    }
    {
        const dl::Tensor X = uniform(dl::Shape({8192, 8192}), 7);
        line("C3 sum axis 1 + argmax axis 1 + full sum", [&] {
            dl::Tensor s = dl::ops::sum(X, 1);
            dl::Tensor m = dl::ops::argmax(X, 1);
            dl::Tensor t = dl::ops::sum(X);
        }, 50);
    }
    {
        const dl::Tensor L = uniform(dl::Shape({65536, 1024}), 8);
        line("C4 softmax [65536,1024]", [&] { dl::Tensor y = dl::ops::softmax(L); }, 50);
        line("C4 layernorm [65536,1024]", [&] { dl::Tensor y = dl::ops::layernorm(L); }, 50);
    }
    return 0;
}
