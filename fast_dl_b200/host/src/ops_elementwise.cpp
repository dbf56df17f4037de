// Binary ops (same-shape and broadcasting), the fused chain, activations.
#include <dl/ops/Ops.hpp>

#include <dl/core/CudaUtils.hpp>
#include <dl/kernels/kernels.hpp>
#include <dl/ops/OpUtils.hpp>

#include <fdl_kernels.h>

#include <climits>
#include <stdexcept>
#include <string>
#include <vector>

namespace dl {

Tensor operator+(const Tensor& a, const Tensor& b) { return ops::add(a, b); }
Tensor operator-(const Tensor& a, const Tensor& b) { return ops::sub(a, b); }
Tensor operator*(const Tensor& a, const Tensor& b) { return ops::mul(a, b); }
Tensor operator/(const Tensor& a, const Tensor& b) { return ops::div(a, b); }

namespace ops {

namespace {

const float* fptr(const Tensor& t) { return static_cast<const float*>(t.data()); }
float* fptr(Tensor& t) { return static_cast<float*>(t.data()); }

Tensor binary(const Tensor& a, const Tensor& b, kernels::ElementwiseOp op, const char* name) {
    // The reference's check order; the one relaxation is the shape test.
    check_defined(a, name, "left");
    check_defined(b, name, "right");
    std::vector<int64_t> oshape, sa, sb;
    const bool same = a.shape() == b.shape();
    if (!same && !broadcast_shapes(a.shape(), b.shape(), &oshape, &sa, &sb)) {
        check_same_shape(a, b, name);  // throws the reference's message
    }
    check_same_dtype(a, b, name);
    check_float32(a, name, "left");
    check_cuda(a, name, "left");
    check_cuda(b, name, "right");
    check_same_device(a, b, name);

    const std::string launch_msg = std::string(name) + " kernel launch failed";
    if (same) {
        Tensor out(a.shape(), a.dtype(), a.device());
        cuda::set_device(a.device().index);
        if (a.numel() <= INT_MAX) {
            kernels::elementwise(fptr(a), fptr(b), fptr(out), static_cast<int>(a.numel()), op);
        } else {
            // Beyond the reference's `int n`: call the 64-bit C entry point directly.
            cuda::check_fdl(fdl_binary_f32(fptr(a), fptr(b), fptr(out), a.numel(), static_cast<int>(op), nullptr),
                            launch_msg.c_str());
        }
        cuda::check(cudaGetLastError(), launch_msg.c_str());
        return out;
    }
    Tensor out(Shape(oshape), a.dtype(), a.device());
    cuda::set_device(a.device().index);
    cuda::check_fdl(fdl_broadcast_binary_f32(fptr(a), fptr(b), fptr(out), static_cast<int>(oshape.size()),
                                             oshape.data(), sa.data(), sb.data(), static_cast<int>(op), nullptr),
                    launch_msg.c_str());
    cuda::check(cudaGetLastError(), launch_msg.c_str());
    return out;
}

Tensor unary(const Tensor& x, kernels::ActivationOp op, const char* name, float alpha = 0.01f) {
    check_defined(x, name);
    check_float32(x, name);
    check_cuda(x, name);
    Tensor out(x.shape(), x.dtype(), x.device());
    cuda::set_device(x.device().index);
    if (x.numel() <= INT_MAX) {
        kernels::activation(fptr(x), fptr(out), static_cast<int>(x.numel()), op, alpha);
    } else {
        cuda::check_fdl(fdl_unary_f32(fptr(x), fptr(out), x.numel(), static_cast<int>(op), alpha, nullptr),
                        "activation kernel launch failed");
    }
    cuda::check(cudaGetLastError(), "activation kernel launch failed");
    return out;
}

}  // namespace

Tensor add(const Tensor& a, const Tensor& b) { return binary(a, b, kernels::ElementwiseOp::Add, "add"); }
Tensor sub(const Tensor& a, const Tensor& b) { return binary(a, b, kernels::ElementwiseOp::Sub, "sub"); }
Tensor mul(const Tensor& a, const Tensor& b) { return binary(a, b, kernels::ElementwiseOp::Mul, "mul"); }
Tensor div(const Tensor& a, const Tensor& b) { return binary(a, b, kernels::ElementwiseOp::Div, "div"); }

Tensor mul_add_relu(const Tensor& a, const Tensor& b, const Tensor& c) {
    check_binary_float_cuda_op(a, b, "mul_add_relu");
    check_defined(c, "mul_add_relu", "addend");
    check_same_shape(a, c, "mul_add_relu", "left", "addend");
    check_float32(c, "mul_add_relu", "addend");
    check_cuda(c, "mul_add_relu", "addend");
    check_same_device(a, c, "mul_add_relu", "left", "addend");
    Tensor out(a.shape(), a.dtype(), a.device());
    cuda::set_device(a.device().index);
    kernels::mul_add_relu(fptr(a), fptr(b), fptr(c), fptr(out), a.numel());
    cuda::check(cudaGetLastError(), "mul_add_relu kernel launch failed");
    return out;
}

Tensor relu(const Tensor& x) { return unary(x, kernels::ActivationOp::ReLU, "relu"); }
Tensor leaky_relu(const Tensor& x, float alpha) {
    return unary(x, kernels::ActivationOp::LeakyReLU, "leaky_relu", alpha);
}
Tensor gelu(const Tensor& x) { return unary(x, kernels::ActivationOp::GELU, "gelu"); }
Tensor sigmoid(const Tensor& x) { return unary(x, kernels::ActivationOp::Sigmoid, "sigmoid"); }
Tensor tanh(const Tensor& x) { return unary(x, kernels::ActivationOp::Tanh, "tanh"); }

}  // namespace ops
}  // namespace dl
