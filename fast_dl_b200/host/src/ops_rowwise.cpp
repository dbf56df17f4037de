// Row softmax, row layernorm, matmul / linear / cross-entropy wrappers.
#include <dl/ops/Ops.hpp>

#include <dl/core/CudaUtils.hpp>
#include <dl/kernels/kernels.hpp>
#include <dl/ops/OpUtils.hpp>

#include <cstddef>
#include <stdexcept>

namespace dl::ops {

namespace {
const float* fptr(const Tensor& t) { return static_cast<const float*>(t.data()); }
float* fptr(Tensor& t) { return static_cast<float*>(t.data()); }
}  // namespace

Tensor softmax(const Tensor& x) {
    check_defined(x, "softmax");
    check_rank(x, 2, "softmax");
    check_float32(x, "softmax");
    check_cuda(x, "softmax");
    const std::size_t rows = static_cast<std::size_t>(x.shape()[0]);
    const std::size_t cols = static_cast<std::size_t>(x.shape()[1]);
    if (rows == 0 || cols == 0) throw std::runtime_error("softmax rows and cols must be non-zero");
    Tensor out(x.shape(), x.dtype(), x.device());
    cuda::set_device(x.device().index);
    kernels::softmax(fptr(x), fptr(out), rows, cols, kernels::SoftmaxAlgo::WarpShuffleRegCache);
    cuda::check(cudaGetLastError(), "softmax kernel launch failed");
    return out;
}

namespace {
Tensor layernorm_impl(const Tensor& x, const Tensor* gamma, const Tensor* beta, float eps) {
    check_defined(x, "layernorm");
    check_rank(x, 2, "layernorm");
    check_float32(x, "layernorm");
    check_cuda(x, "layernorm");
    const int rows = static_cast<int>(x.shape()[0]);
    const int cols = static_cast<int>(x.shape()[1]);
    if (rows <= 0 || cols <= 0) throw std::runtime_error("layernorm rows and cols must be positive");
    for (const Tensor* p : {gamma, beta}) {
        if (p == nullptr) continue;
        const char* name = p == gamma ? "gamma" : "beta";
        check_defined(*p, "layernorm", name);
        check_float32(*p, "layernorm", name);
        check_cuda(*p, "layernorm", name);
        check_same_device(x, *p, "layernorm", "input", name);
        if (p->numel() != cols) throw std::runtime_error(std::string("layernorm: ") + name + " tensor must have shape [cols]");
    }
    Tensor out(x.shape(), x.dtype(), x.device());
    cuda::set_device(x.device().index);
    kernels::layernorm_affine(fptr(x), gamma ? fptr(*gamma) : nullptr, beta ? fptr(*beta) : nullptr, fptr(out),
                              rows, cols, eps);
    cuda::check(cudaGetLastError(), "layernorm kernel launch failed");
    return out;
}
}  // namespace

Tensor layernorm(const Tensor& x, float eps) { return layernorm_impl(x, nullptr, nullptr, eps); }
Tensor layernorm(const Tensor& x, const Tensor& gamma, const Tensor& beta, float eps) {
    return layernorm_impl(x, &gamma, &beta, eps);
}

Tensor matmul(const Tensor& a, const Tensor& b) {
    check_defined(a, "matmul", "left");
    check_defined(b, "matmul", "right");
    check_rank(a, 2, "matmul", "left");
    check_rank(b, 2, "matmul", "right");
    check_float32(a, "matmul", "left");
    check_float32(b, "matmul", "right");
    check_cuda(a, "matmul", "left");
    check_cuda(b, "matmul", "right");
    check_same_device(a, b, "matmul");
    if (a.shape()[1] != b.shape()[0]) throw std::runtime_error("matmul input tensors have incompatible shapes");
    Tensor out(Shape({a.shape()[0], b.shape()[1]}), a.dtype(), a.device());
    cuda::set_device(a.device().index);
    kernels::gemm(fptr(a), fptr(b), fptr(out), static_cast<int>(a.shape()[0]), static_cast<int>(b.shape()[1]),
                  static_cast<int>(a.shape()[1]), kernels::GemmAlgo::Cublas);
    cuda::check(cudaGetLastError(), "matmul kernel launch failed");
    return out;
}

namespace {
Tensor linear_impl(const Tensor& x, const Tensor& w, const Tensor& bias, bool fuse_relu) {
    check_defined(x, "linear", "input");
    check_defined(w, "linear", "weight");
    check_defined(bias, "linear", "bias");
    check_rank(x, 2, "linear", "input");
    check_rank(w, 2, "linear", "weight");
    check_rank(bias, 1, "linear", "bias");
    check_float32(x, "linear", "input");
    check_same_dtype(x, w, "linear", "input", "weight");
    check_same_dtype(x, bias, "linear", "input", "bias");
    check_cuda(x, "linear", "input");
    check_cuda(w, "linear", "weight");
    check_cuda(bias, "linear", "bias");
    check_same_device(x, w, "linear", "input", "weight");
    check_same_device(x, bias, "linear", "input", "bias");
    if (x.shape()[1] != w.shape()[0]) throw std::runtime_error("linear input and weight tensors have incompatible shapes");
    if (w.shape()[1] != bias.shape()[0]) throw std::runtime_error("linear bias shape must be [out_features]");
    Tensor out = matmul(x, w);
    cuda::set_device(x.device().index);
    const int rows = static_cast<int>(out.shape()[0]), cols = static_cast<int>(out.shape()[1]);
    if (fuse_relu) kernels::add_row_bias_relu(fptr(out), fptr(bias), rows, cols);
    else kernels::add_row_bias(fptr(out), fptr(bias), rows, cols);
    cuda::check(cudaGetLastError(), "linear bias kernel launch failed");
    return out;
}
}  // namespace

Tensor linear(const Tensor& x, const Tensor& w, const Tensor& bias) { return linear_impl(x, w, bias, false); }
Tensor linear_relu(const Tensor& x, const Tensor& w, const Tensor& bias) { return linear_impl(x, w, bias, true); }

Tensor cross_entropy(const Tensor& logits, const Tensor& labels) {
    check_defined(logits, "cross_entropy", "logits");
    check_defined(labels, "cross_entropy", "labels");
    check_rank(logits, 2, "cross_entropy", "logits");
    check_rank(labels, 1, "cross_entropy", "labels");
    check_float32(logits, "cross_entropy", "logits");
    check_dtype(labels, DType::Int64, "cross_entropy", "labels");
    check_cuda(logits, "cross_entropy", "logits");
    check_cuda(labels, "cross_entropy", "labels");
    check_same_device(logits, labels, "cross_entropy", "logits", "labels");
    if (logits.shape()[0] != labels.shape()[0]) throw std::runtime_error("cross_entropy logits and labels batch size mismatch");
    if (logits.shape()[1] <= 0) throw std::runtime_error("cross_entropy class count must be positive");
    Tensor loss(Shape({1}), DType::Float32, logits.device());
    cuda::set_device(logits.device().index);
    kernels::cross_entropy(fptr(logits), static_cast<const int64_t*>(labels.data()), fptr(loss),
                           static_cast<int>(logits.shape()[0]), static_cast<int>(logits.shape()[1]));
    cuda::check(cudaGetLastError(), "cross_entropy kernel launch failed");
    return loss;
}

}  // namespace dl::ops
