// Row-sharded tensors: every op on the shards must equal the op on the whole tensor.
// Uses all visible GPUs (at most 8); on a single-GPU box the three shards share device 0,
// which exercises the same splitting, broadcasting and combining code.
#include <dl/dist/Sharded.hpp>
#include <dl/dl.hpp>

#include <dl/core/CudaUtils.hpp>

#include <cmath>
#include <cstring>
#include <iostream>
#include <random>
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
std::vector<float> randoms(std::size_t n, unsigned seed, float lo, float hi) {
    std::mt19937 gen(seed);
    std::uniform_real_distribution<float> dist(lo, hi);
    std::vector<float> v(n);
    for (float& x : v) x = dist(gen);
    return v;
}
}  // namespace

int main() {
    const int ngpu = dl::cuda::device_count();
    std::vector<int> devices;
    if (ngpu >= 2) {
        for (int i = 0; i < ngpu && i < 8; ++i) devices.push_back(i);
    } else {
        devices = {0, 0, 0};
    }
    std::cout << "shards: " << devices.size() << " over " << ngpu << " GPU(s)\n";

    const int64_t R = 1003, C = 256;  // 1003 rows: uneven split
    const dl::Device d0(dl::DeviceType::CUDA, 0);
    const auto a = randoms(R * C, 1, -1, 1), b = randoms(R * C, 2, -1, 1), c = randoms(R * C, 3, -1, 1);
    const auto row = randoms(C, 4, -1, 1), col = randoms(R, 5, 0.5f, 2), g = randoms(C, 6, 0.9f, 1.1f),
               be = randoms(C, 7, -0.1f, 0.1f);
    dl::Tensor wa = dl::Tensor::from_host<float>(a, dl::Shape({R, C}), d0);
    dl::Tensor wb = dl::Tensor::from_host<float>(b, dl::Shape({R, C}), d0);
    dl::Tensor wc = dl::Tensor::from_host<float>(c, dl::Shape({R, C}), d0);
    dl::Tensor wrow = dl::Tensor::from_host<float>(row, dl::Shape({1, C}), d0);
    dl::Tensor wcol = dl::Tensor::from_host<float>(col, dl::Shape({R, 1}), d0);
    dl::Tensor wg = dl::Tensor::from_host<float>(g, dl::Shape({C}), d0);
    dl::Tensor wbe = dl::Tensor::from_host<float>(be, dl::Shape({C}), d0);

    namespace ds = dl::dist;
    ds::ShardedTensor sa = ds::ShardedTensor::scatter(a, dl::Shape({R, C}), devices);
    ds::ShardedTensor sb = ds::ShardedTensor::scatter(b, dl::Shape({R, C}), devices);
    ds::ShardedTensor sc = ds::ShardedTensor::scatter(c, dl::Shape({R, C}), devices);
    ds::ShardedTensor srow = ds::ShardedTensor::replicate(row, dl::Shape({1, C}), devices);
    ds::ShardedTensor scol = ds::ShardedTensor::scatter(col, dl::Shape({R, 1}), devices);
    ds::ShardedTensor sg = ds::ShardedTensor::replicate(g, dl::Shape({C}), devices);
    ds::ShardedTensor sbe = ds::ShardedTensor::replicate(be, dl::Shape({C}), devices);

    report("scatter / gather round trip", same_bits(sa.gather(), a));
    report("add", same_bits(ds::add(sa, sb).gather(), (wa + wb).to_host<float>()));
    report("div", same_bits(ds::div(sa, sb).gather(), (wa / wb).to_host<float>()));
    report("broadcast add against a replicated row", same_bits(ds::add(sa, srow).gather(), (wa + wrow).to_host<float>()));
    report("broadcast mul against a sharded column", same_bits(ds::mul(sa, scol).gather(), (wa * wcol).to_host<float>()));
    report("mul_add_relu", same_bits(ds::mul_add_relu(sa, sb, sc).gather(), dl::ops::mul_add_relu(wa, wb, wc).to_host<float>()));
    report("gelu", same_bits(ds::gelu(sa).gather(), dl::ops::gelu(wa).to_host<float>()));
    report("softmax", same_bits(ds::softmax(sa).gather(), dl::ops::softmax(wa).to_host<float>()));
    report("layernorm", same_bits(ds::layernorm(sa).gather(), dl::ops::layernorm(wa).to_host<float>()));
    report("layernorm + gamma, beta",
           same_bits(ds::layernorm(sa, sg, sbe).gather(), dl::ops::layernorm(wa, wg, wbe).to_host<float>()));
    report("sum along axis 1", same_bits(ds::sum_rows(sa).gather(), dl::ops::sum(wa, 1).to_host<float>()));
    report("max along axis 1", same_bits(ds::max_rows(sa).gather(), dl::ops::max(wa, 1).to_host<float>()));
    report("argmax along axis 1", ds::argmax_rows(sa).gather_int64() == dl::ops::argmax(wa, 1).to_host<int64_t>());

    double exact = 0.0, norm2 = 0.0;
    for (float v : a) { exact += v; norm2 += static_cast<double>(v) * v; }
    const double s = ds::sum(sa);
    report("full sum over the shards", std::fabs(s - exact) <= 1e-5 * std::max(std::fabs(exact), std::sqrt(norm2)));
    report("full sum is repeatable", ds::sum(sa) == s);

    const auto m = ds::mean_rows_of_whole(sa).to_host<float>();
    const auto mw = dl::ops::mean(wa, 0).to_host<float>();
    bool mean_ok = m.size() == mw.size();
    for (std::size_t i = 0; mean_ok && i < m.size(); ++i) mean_ok = std::fabs(m[i] - mw[i]) <= 1e-6f;
    report("mean along axis 0 of the whole tensor", mean_ok);

    ds::synchronize(sa);
    std::cout << "sharded_test : " << (g_failed == 0 ? "passed" : "not passed") << "\n";
    return g_failed == 0 ? 0 : 1;
}
