// Row-sharded tensors over the GPUs of one box (single process).
#include <dl/dist/Sharded.hpp>

#include <dl/core/CudaUtils.hpp>
#include <dl/ops/Ops.hpp>

#include <fdl_kernels.h>

#include <cuda_runtime.h>

#include <functional>
#include <stdexcept>
#include <utility>

namespace dl::dist {

namespace {

int64_t row_elems(const Shape& shape) {
    int64_t n = 1;
    for (int i = 1; i < shape.rank(); ++i) n *= shape[i];
    return n;
}

Shape with_rows(const Shape& shape, int64_t rows) {
    std::vector<int64_t> d = shape.dims;
    d[0] = rows;
    return Shape(d);
}

void require_compatible(const ShardedTensor& a, const ShardedTensor& b, const char* op) {
    if (a.num_shards() != b.num_shards()) {
        throw std::runtime_error(std::string(op) + ": operands are sharded over a different number of devices");
    }
    for (int i = 0; i < a.num_shards(); ++i) {
        if (a.shard(i).device().index != b.shard(i).device().index) {
            throw std::runtime_error(std::string(op) + ": shard " + std::to_string(i) + " lives on different devices");
        }
    }
}

using Binary = Tensor (*)(const Tensor&, const Tensor&);

ShardedTensor zip(const ShardedTensor& a, const ShardedTensor& b, Binary fn, const char* op) {
    require_compatible(a, b, op);
    std::vector<Tensor> out;
    for (int i = 0; i < a.num_shards(); ++i) out.push_back(fn(a.shard(i), b.shard(i)));
    // A replicated operand broadcasts; the result takes the sharded operand's global shape.
    const ShardedTensor& lead = a.replicated() ? b : a;
    return ShardedTensor::from_shards(std::move(out), lead.shape(), a.replicated() && b.replicated());
}

ShardedTensor map(const ShardedTensor& x, const std::function<Tensor(const Tensor&)>& fn, const Shape& shape) {
    std::vector<Tensor> out;
    for (int i = 0; i < x.num_shards(); ++i) out.push_back(fn(x.shard(i)));
    return ShardedTensor::from_shards(std::move(out), shape, x.replicated());
}

}  // namespace

ShardedTensor ShardedTensor::scatter(const std::vector<float>& data, const Shape& shape,
                                     const std::vector<int>& devices) {
    if (devices.empty()) throw std::runtime_error("scatter: no devices");
    if (shape.rank() < 1 || shape.numel() != static_cast<int64_t>(data.size())) {
        throw std::runtime_error("scatter: data size does not match shape");
    }
    const int64_t rows = shape[0], n = static_cast<int64_t>(devices.size()), per_row = row_elems(shape);
    if (rows < n) throw std::runtime_error("scatter: fewer rows than devices");
    ShardedTensor t;
    t.shape_ = shape;
    int64_t start = 0;
    for (int64_t i = 0; i < n; ++i) {
        const int64_t count = rows / n + (i < rows % n ? 1 : 0);
        Tensor s(with_rows(shape, count), DType::Float32, Device(DeviceType::CUDA, devices[static_cast<std::size_t>(i)]));
        s.copy_from_host(data.data() + start * per_row, static_cast<std::size_t>(count * per_row) * sizeof(float));
        t.shards_.push_back(std::move(s));
        t.offsets_.push_back(start);
        start += count;
    }
    return t;
}

ShardedTensor ShardedTensor::replicate(const std::vector<float>& data, const Shape& shape,
                                       const std::vector<int>& devices) {
    if (devices.empty()) throw std::runtime_error("replicate: no devices");
    ShardedTensor t;
    t.shape_ = shape;
    t.replicated_ = true;
    for (int dev : devices) {
        t.shards_.push_back(Tensor::from_host<float>(data, shape, Device(DeviceType::CUDA, dev)));
        t.offsets_.push_back(0);
    }
    return t;
}

ShardedTensor ShardedTensor::from_shards(std::vector<Tensor> shards, const Shape& global_shape, bool replicated) {
    ShardedTensor t;
    t.shape_ = global_shape;
    t.replicated_ = replicated;
    int64_t start = 0;
    for (Tensor& s : shards) {
        t.offsets_.push_back(replicated ? 0 : start);
        start += s.shape().rank() > 0 ? s.shape()[0] : 0;
        t.shards_.push_back(std::move(s));
    }
    return t;
}

std::vector<float> ShardedTensor::gather() const {
    if (replicated_) return shards_.at(0).to_host<float>();
    std::vector<float> out;
    out.reserve(static_cast<std::size_t>(shape_.numel()));
    for (const Tensor& s : shards_) {
        const std::vector<float> part = s.to_host<float>();
        out.insert(out.end(), part.begin(), part.end());
    }
    return out;
}

std::vector<int64_t> ShardedTensor::gather_int64() const {
    std::vector<int64_t> out;
    for (const Tensor& s : shards_) {
        const std::vector<int64_t> part = s.to_host<int64_t>();
        out.insert(out.end(), part.begin(), part.end());
    }
    return out;
}

ShardedTensor add(const ShardedTensor& a, const ShardedTensor& b) { return zip(a, b, &ops::add, "add"); }
ShardedTensor sub(const ShardedTensor& a, const ShardedTensor& b) { return zip(a, b, &ops::sub, "sub"); }
ShardedTensor mul(const ShardedTensor& a, const ShardedTensor& b) { return zip(a, b, &ops::mul, "mul"); }
ShardedTensor div(const ShardedTensor& a, const ShardedTensor& b) { return zip(a, b, &ops::div, "div"); }

ShardedTensor mul_add_relu(const ShardedTensor& a, const ShardedTensor& b, const ShardedTensor& c) {
    require_compatible(a, b, "mul_add_relu");
    require_compatible(a, c, "mul_add_relu");
    std::vector<Tensor> out;
    for (int i = 0; i < a.num_shards(); ++i) out.push_back(ops::mul_add_relu(a.shard(i), b.shard(i), c.shard(i)));
    return ShardedTensor::from_shards(std::move(out), a.shape(), false);
}

ShardedTensor relu(const ShardedTensor& x) { return map(x, &ops::relu, x.shape()); }
ShardedTensor gelu(const ShardedTensor& x) { return map(x, &ops::gelu, x.shape()); }
ShardedTensor sigmoid(const ShardedTensor& x) { return map(x, &ops::sigmoid, x.shape()); }
ShardedTensor tanh(const ShardedTensor& x) { return map(x, &ops::tanh, x.shape()); }
ShardedTensor softmax(const ShardedTensor& x) { return map(x, &ops::softmax, x.shape()); }

ShardedTensor layernorm(const ShardedTensor& x, float eps) {
    return map(x, [eps](const Tensor& t) { return ops::layernorm(t, eps); }, x.shape());
}

ShardedTensor layernorm(const ShardedTensor& x, const ShardedTensor& gamma, const ShardedTensor& beta, float eps) {
    require_compatible(x, gamma, "layernorm");
    require_compatible(x, beta, "layernorm");
    if (!gamma.replicated() || !beta.replicated()) {
        throw std::runtime_error("layernorm: gamma and beta must be replicated on every device");
    }
    std::vector<Tensor> out;
    for (int i = 0; i < x.num_shards(); ++i) {
        out.push_back(ops::layernorm(x.shard(i), gamma.shard(i), beta.shard(i), eps));
    }
    return ShardedTensor::from_shards(std::move(out), x.shape(), false);
}

ShardedTensor sum_rows(const ShardedTensor& x) {
    return map(x, [](const Tensor& t) { return ops::sum(t, -1); }, Shape({x.shape()[0]}));
}
ShardedTensor max_rows(const ShardedTensor& x) {
    return map(x, [](const Tensor& t) { return ops::max(t, -1); }, Shape({x.shape()[0]}));
}
ShardedTensor argmax_rows(const ShardedTensor& x) {
    return map(x, [](const Tensor& t) { return ops::argmax(t, -1); }, Shape({x.shape()[0]}));
}

double sum(const ShardedTensor& x) {
    if (x.replicated()) throw std::runtime_error("sum: tensor is replicated, not sharded");
    // Enqueue every GPU's reduction first, read the partials back afterwards.
    std::vector<Tensor> partials;
    for (int i = 0; i < x.num_shards(); ++i) {
        const Tensor& s = x.shard(i);
        Tensor p(Shape({1}), DType::Int64, s.device());  // 8 bytes holding a double
        cuda::set_device(s.device().index);
        cuda::check_fdl(fdl_sum_f32(static_cast<const float*>(s.data()), s.numel(), nullptr,
                                    static_cast<double*>(p.data()), nullptr, 0, nullptr),
                        "sum kernel launch failed");
        partials.push_back(std::move(p));
    }
    double total = 0.0;
    for (const Tensor& p : partials) {
        double v = 0.0;
        p.copy_to_host(&v, sizeof v);
        total += v;  // shard order
    }
    return total;
}

Tensor mean_rows_of_whole(const ShardedTensor& x) {
    if (x.replicated() || x.shape().rank() != 2) {
        throw std::runtime_error("mean_rows_of_whole: needs a row-sharded rank-2 tensor");
    }
    const int64_t cols = x.shape()[1];
    const double total_rows = static_cast<double>(x.shape()[0]);
    std::vector<Tensor> parts;
    for (int i = 0; i < x.num_shards(); ++i) {
        const Tensor& s = x.shard(i);
        Tensor p(Shape({cols}), DType::Float32, s.device());
        cuda::set_device(s.device().index);
        cuda::check_fdl(fdl_reduce_cols_f32(static_cast<const float*>(s.data()), 1, s.shape()[0], cols,
                                            static_cast<float*>(p.data()), FDL_REDUCE_MEAN, total_rows, nullptr, 0,
                                            nullptr),
                        "mean kernel launch failed");
        parts.push_back(std::move(p));
    }
    Tensor acc = parts[0];
    for (std::size_t i = 1; i < parts.size(); ++i) {
        Tensor here(Shape({cols}), DType::Float32, acc.device());
        here.copy_from(parts[i]);  // peer copy when the shard lives on another GPU
        acc = ops::add(acc, here);
    }
    return acc;
}

void synchronize(const ShardedTensor& x) {
    for (int i = 0; i < x.num_shards(); ++i) {
        cuda::check(cudaSetDevice(x.shard(i).device().index), "cudaSetDevice failed");
        cuda::check(cudaDeviceSynchronize(), "cudaDeviceSynchronize failed");
    }
}

}  // namespace dl::dist
