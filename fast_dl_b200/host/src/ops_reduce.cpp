// Reductions: full sum and sum / mean / max / argmax along an axis.
//
// A tensor of shape [d0..dk] reduced along `axis` is viewed as [outer, reduce, inner]:
// inner == 1 is a row-wise reduction of an [outer, reduce] matrix (fdl_reduce_rows_f32);
// otherwise `outer` stacked [reduce, inner] matrices reduced over their rows
// (fdl_reduce_cols_f32).  Results drop the reduced axis (a rank-1 input gives shape {1}).
#include <dl/ops/Ops.hpp>

#include <dl/core/CudaUtils.hpp>
#include <dl/ops/OpUtils.hpp>

#include <fdl_kernels.h>

#include <stdexcept>
#include <string>
#include <vector>

namespace dl::ops {

namespace {

struct AxisView {
    int64_t outer = 1, reduce = 1, inner = 1;
    Shape out_shape;
};

AxisView view_along(const Tensor& x, int axis, const char* op) {
    const int rank = static_cast<int>(x.shape().rank());
    if (axis < 0) axis += rank;
    if (axis < 0 || axis >= rank) throw std::runtime_error(std::string(op) + ": axis is out of range");
    AxisView v;
    std::vector<int64_t> dims;
    for (int i = 0; i < rank; ++i) {
        const int64_t d = x.shape()[i];
        if (i < axis) v.outer *= d;
        else if (i == axis) v.reduce = d;
        else v.inner *= d;
        if (i != axis) dims.push_back(d);
    }
    if (dims.empty()) dims.push_back(1);
    v.out_shape = Shape(dims);
    return v;
}

Tensor reduce_axis(const Tensor& x, int axis, int code, const char* op) {
    check_defined(x, op);
    check_float32(x, op);
    check_cuda(x, op);
    const AxisView v = view_along(x, axis, op);
    Tensor out(v.out_shape, DType::Float32, x.device());
    cuda::set_device(x.device().index);
    const float* src = static_cast<const float*>(x.data());
    float* dst = static_cast<float*>(out.data());
    const std::string msg = std::string(op) + " kernel launch failed";
    if (v.inner == 1) {
        cuda::check_fdl(fdl_reduce_rows_f32(src, v.outer, v.reduce, dst, code, nullptr), msg.c_str());
    } else {
        cuda::check_fdl(fdl_reduce_cols_f32(src, v.outer, v.reduce, v.inner, dst, code,
                                            static_cast<double>(v.reduce), nullptr, 0, nullptr),
                        msg.c_str());
    }
    cuda::check(cudaGetLastError(), msg.c_str());
    return out;
}

}  // namespace

Tensor sum(const Tensor& x) {
    check_defined(x, "sum");
    check_float32(x, "sum");
    check_cuda(x, "sum");
    Tensor out(Shape({1}), DType::Float32, x.device());
    cuda::set_device(x.device().index);
    cuda::check_fdl(fdl_sum_f32(static_cast<const float*>(x.data()), x.numel(), static_cast<float*>(out.data()),
                                nullptr, nullptr, 0, nullptr),
                    "sum kernel launch failed");
    cuda::check(cudaGetLastError(), "sum kernel launch failed");
    return out;
}

Tensor sum(const Tensor& x, int axis) { return reduce_axis(x, axis, FDL_REDUCE_SUM, "sum"); }
Tensor mean(const Tensor& x, int axis) { return reduce_axis(x, axis, FDL_REDUCE_MEAN, "mean"); }
Tensor max(const Tensor& x, int axis) { return reduce_axis(x, axis, FDL_REDUCE_MAX, "max"); }

Tensor argmax(const Tensor& x, int axis) {
    check_defined(x, "argmax");
    check_float32(x, "argmax");
    check_cuda(x, "argmax");
    const AxisView v = view_along(x, axis, "argmax");
    if (v.inner != 1) throw std::runtime_error("argmax: only the last axis is supported");
    Tensor out(v.out_shape, DType::Int64, x.device());
    cuda::set_device(x.device().index);
    cuda::check_fdl(fdl_argmax_rows_f32(static_cast<const float*>(x.data()), v.outer, v.reduce,
                                        static_cast<int64_t*>(out.data()), nullptr),
                    "argmax kernel launch failed");
    cuda::check(cudaGetLastError(), "argmax kernel launch failed");
    return out;
}

}  // namespace dl::ops
