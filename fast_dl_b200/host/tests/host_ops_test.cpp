// Tests of the host library's additions to the fast_dl API, in the style of the reference's
// own tests: one main(), CPU loops in this file as the expectation, "<name> : passed|not
// passed" per check, exit code 0 only if all pass.  Needs a GPU (device 0).
#include <dl/dl.hpp>
#include <dl/ops/OpUtils.hpp>
#include <dl/tensor/Allocator.hpp>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <iostream>
#include <random>
#include <string>
#include <vector>

namespace {

int g_failed = 0;

void report(const char* name, bool ok) {
    std::cout << name << " : " << (ok ? "passed" : "not passed") << "\n";
    if (!ok) ++g_failed;
}

bool same_bits(const std::vector<float>& a, const std::vector<float>& b) {
    return a.size() == b.size() && std::memcmp(a.data(), b.data(), a.size() * sizeof(float)) == 0;
}

bool close(const std::vector<float>& a, const std::vector<float>& b, float tol) {
    if (a.size() != b.size()) return false;
    for (std::size_t i = 0; i < a.size(); ++i) {
        if (std::fabs(a[i] - b[i]) > tol * std::max(1.0f, std::fabs(b[i]))) return false;
    }
    return true;
}

std::vector<float> randoms(std::size_t n, unsigned seed, float lo, float hi) {
    std::mt19937 gen(seed);
    std::uniform_real_distribution<float> dist(lo, hi);
    std::vector<float> v(n);
    for (float& x : v) x = dist(gen);
    return v;
}

template <class Fn>
bool throws_with(Fn fn, const std::string& text) {
    try {
        fn();
    } catch (const std::runtime_error& e) {
        return std::string(e.what()).find(text) != std::string::npos;
    }
    return false;
}

}  // namespace

int main() {
    const dl::Device dev(dl::DeviceType::CUDA, 0);
    const int64_t R = 37, C = 52;
    const auto a = randoms(R * C, 1, -1, 1), row = randoms(C, 2, -1, 1), col = randoms(R, 3, 0.5f, 2);
    dl::Tensor ta = dl::Tensor::from_host<float>(a, dl::Shape({R, C}), dev);
    dl::Tensor trow = dl::Tensor::from_host<float>(row, dl::Shape({1, C}), dev);
    dl::Tensor tcol = dl::Tensor::from_host<float>(col, dl::Shape({R, 1}), dev);
    dl::Tensor tvec = dl::Tensor::from_host<float>(row, dl::Shape({C}), dev);

    {   // broadcasting binary ops: bit-exact against the expanded loops
        std::vector<float> e_add(R * C), e_mul(R * C), e_outer(R * C), e_div(R * C);
        for (int64_t r = 0; r < R; ++r) {
            for (int64_t c = 0; c < C; ++c) {
                e_add[r * C + c] = a[r * C + c] + row[c];
                e_mul[r * C + c] = a[r * C + c] * col[r];
                e_outer[r * C + c] = col[r] - row[c];
                e_div[r * C + c] = a[r * C + c] / col[r];
            }
        }
        report("broadcast add [R,C]+[1,C]", same_bits((ta + trow).to_host<float>(), e_add));
        report("broadcast add [R,C]+[C]", same_bits(dl::ops::add(ta, tvec).to_host<float>(), e_add));
        report("broadcast mul [R,C]*[R,1]", same_bits((ta * tcol).to_host<float>(), e_mul));
        report("broadcast div [R,C]/[R,1]", same_bits((ta / tcol).to_host<float>(), e_div));
        dl::Tensor outer = tcol - trow;
        report("broadcast sub [R,1]-[1,C]", outer.shape()[0] == R && outer.shape()[1] == C &&
                                                same_bits(outer.to_host<float>(), e_outer));
        dl::Tensor bad = dl::Tensor::zeros(dl::Shape({R, C + 1}), dl::DType::Float32, dev);
        report("non-broadcastable shapes keep the reference's message",
               throws_with([&] { dl::ops::add(ta, bad); }, "add: left and right tensors must have the same shape"));
        report("undefined operand message",
               throws_with([&] { dl::ops::mul(dl::Tensor(), ta); }, "mul: left tensor is not defined"));
    }

    {   // fused chain == three ops
        const auto b = randoms(R * C, 4, -1, 1), c = randoms(R * C, 5, -1, 1);
        dl::Tensor tb = dl::Tensor::from_host<float>(b, dl::Shape({R, C}), dev);
        dl::Tensor tc = dl::Tensor::from_host<float>(c, dl::Shape({R, C}), dev);
        const auto fused = dl::ops::mul_add_relu(ta, tb, tc).to_host<float>();
        const auto chain = dl::ops::relu(ta * tb + tc).to_host<float>();
        std::vector<float> expect(R * C);
        for (int64_t i = 0; i < R * C; ++i) {
            volatile float p = a[i] * b[i];
            expect[i] = std::max(0.0f, p + c[i]);
        }
        report("mul_add_relu equals relu(a*b+c) bit for bit", same_bits(fused, chain) && same_bits(fused, expect));
    }

    {   // reductions
        std::vector<float> s1(R), mx1(R), m0(C);
        std::vector<int64_t> am(R);
        double total = 0;
        for (int64_t r = 0; r < R; ++r) {
            double s = 0;
            float m = a[r * C];
            int64_t arg = 0;
            for (int64_t c = 0; c < C; ++c) {
                s += a[r * C + c];
                if (a[r * C + c] > m) { m = a[r * C + c]; arg = c; }
            }
            s1[r] = static_cast<float>(s); mx1[r] = m; am[r] = arg; total += s;
        }
        for (int64_t c = 0; c < C; ++c) {
            double s = 0;
            for (int64_t r = 0; r < R; ++r) s += a[r * C + c];
            m0[c] = static_cast<float>(s / R);
        }
        report("sum axis 1", close(dl::ops::sum(ta, 1).to_host<float>(), s1, 1e-5f));
        report("sum axis -1", close(dl::ops::sum(ta, -1).to_host<float>(), s1, 1e-5f));
        report("max axis 1", same_bits(dl::ops::max(ta, 1).to_host<float>(), mx1));
        report("mean axis 0", close(dl::ops::mean(ta, 0).to_host<float>(), m0, 1e-5f));
        dl::Tensor arg = dl::ops::argmax(ta, 1);
        report("argmax axis 1 is int64 and exact", arg.dtype() == dl::DType::Int64 && arg.to_host<int64_t>() == am);
        const auto full = dl::ops::sum(ta).to_host<float>();
        report("full sum has shape {1}", full.size() == 1 && std::fabs(full[0] - total) <= 1e-5 * std::max(1.0, std::fabs(total)));
        dl::Tensor t3 = ta.reshaped(dl::Shape({R, 4, 13}));
        std::vector<float> mid(R * 13, 0.0f);
        for (int64_t r = 0; r < R; ++r)
            for (int64_t j = 0; j < 4; ++j)
                for (int64_t k = 0; k < 13; ++k) mid[r * 13 + k] += a[(r * 4 + j) * 13 + k];
        dl::Tensor red = dl::ops::sum(t3, 1);
        report("sum over the middle axis of a rank-3 view",
               red.shape().rank() == 2 && red.shape()[0] == R && red.shape()[1] == 13 &&
                   close(red.to_host<float>(), mid, 1e-5f));
        report("axis out of range", throws_with([&] { dl::ops::sum(ta, 2); }, "sum: axis is out of range"));
    }

    {   // affine layernorm = plain layernorm * gamma + beta
        const auto g = randoms(C, 6, 0.9f, 1.1f), b = randoms(C, 7, -0.1f, 0.1f);
        dl::Tensor tg = dl::Tensor::from_host<float>(g, dl::Shape({C}), dev);
        dl::Tensor tb = dl::Tensor::from_host<float>(b, dl::Shape({C}), dev);
        const auto plain = dl::ops::layernorm(ta).to_host<float>();
        std::vector<float> expect(R * C);
        for (int64_t i = 0; i < R * C; ++i) expect[i] = plain[i] * g[i % C] + b[i % C];
        report("layernorm with gamma and beta", close(dl::ops::layernorm(ta, tg, tb, 1e-5f).to_host<float>(), expect, 1e-5f));
    }

    {   // linear with fused ReLU epilogue == relu(linear)
        dl::Tensor w = dl::Tensor::uniform(dl::Shape({C, 24}), dl::DType::Float32, dev, -1, 1, 9);
        dl::Tensor bias = dl::Tensor::uniform(dl::Shape({24}), dl::DType::Float32, dev, -1, 1, 10);
        report("linear_relu equals relu(linear)",
               same_bits(dl::ops::linear_relu(ta, w, bias).to_host<float>(),
                         dl::ops::relu(dl::ops::linear(ta, w, bias)).to_host<float>()));
    }

    {   // shapes that take the other kernels: short rows, a few very long rows, a handful of rows
        struct Case { int64_t rows, cols; };
        const Case cases[] = {{5000, 16}, {300, 128}, {3, 400000}, {4, 40000}, {2, 262144}};
        bool ok_red = true, ok_norm = true;
        for (const Case& k : cases) {
            const auto x = randoms(k.rows * k.cols, 11, -3, 3);
            dl::Tensor tx = dl::Tensor::from_host<float>(x, dl::Shape({k.rows, k.cols}), dev);
            std::vector<float> rs(k.rows), cm(k.cols), sm(k.rows * k.cols), ln(k.rows * k.cols);
            std::vector<int64_t> am(k.rows);
            std::vector<double> colsum(k.cols, 0.0);
            for (int64_t r = 0; r < k.rows; ++r) {
                const float* xr = x.data() + r * k.cols;
                double s = 0, e = 0, q = 0;
                float m = xr[0];
                int64_t arg = 0;
                for (int64_t c = 0; c < k.cols; ++c) {
                    s += xr[c];
                    colsum[c] += xr[c];
                    if (xr[c] > m) { m = xr[c]; arg = c; }
                }
                const double mean = s / k.cols;
                for (int64_t c = 0; c < k.cols; ++c) {
                    e += std::exp(static_cast<double>(xr[c]) - m);
                    q += (xr[c] - mean) * (xr[c] - mean);
                }
                const double rstd = 1.0 / std::sqrt(q / k.cols + 1e-5);
                for (int64_t c = 0; c < k.cols; ++c) {
                    sm[r * k.cols + c] = static_cast<float>(std::exp(static_cast<double>(xr[c]) - m) / e);
                    ln[r * k.cols + c] = static_cast<float>((xr[c] - mean) * rstd);
                }
                rs[r] = static_cast<float>(s);
                am[r] = arg;
            }
            for (int64_t c = 0; c < k.cols; ++c) cm[c] = static_cast<float>(colsum[c] / k.rows);
            // sums of n terms of size <= 3: allow 1e-5 of the terms' scale, not of a sum that may be near zero
            const float sum_tol = 1e-5f * 3.0f * std::sqrt(static_cast<float>(k.cols));
            const auto got_rs = dl::ops::sum(tx, 1).to_host<float>();
            for (int64_t r = 0; r < k.rows; ++r) ok_red = ok_red && std::fabs(got_rs[r] - rs[r]) <= sum_tol;
            ok_red = ok_red && dl::ops::argmax(tx, 1).to_host<int64_t>() == am;
            ok_red = ok_red && close(dl::ops::mean(tx, 0).to_host<float>(), cm, 1e-5f);
            ok_norm = ok_norm && close(dl::ops::softmax(tx).to_host<float>(), sm, 1e-5f);
            ok_norm = ok_norm && close(dl::ops::layernorm(tx).to_host<float>(), ln, 1e-5f);
        }
        report("reductions on short rows, a few long rows and a handful of rows", ok_red);
        report("softmax and layernorm on rows of 16 ... 262144 floats", ok_norm);
    }

    {   // the allocator hands blocks back out instead of calling cudaMalloc again
        const auto before = dl::allocator::stats();
        for (int i = 0; i < 50; ++i) dl::Tensor tmp = ta + ta;
        const auto after = dl::allocator::stats();
        report("temporaries reuse cached blocks",
               after.cuda_malloc_calls - before.cuda_malloc_calls <= 1 && after.cache_hits - before.cache_hits >= 49);
        dl::allocator::set_caching(false);
        const auto u0 = dl::allocator::stats();
        for (int i = 0; i < 5; ++i) dl::Tensor tmp = ta + ta;
        const auto u1 = dl::allocator::stats();
        dl::allocator::set_caching(true);
        report("caching can be switched off", u1.cuda_malloc_calls - u0.cuda_malloc_calls == 5);
    }

    std::cout << "host_ops_test : " << (g_failed == 0 ? "passed" : "not passed") << "\n";
    return g_failed == 0 ? 0 : 1;
}
