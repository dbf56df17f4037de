// Argument checks and broadcast-shape arithmetic.
#include <dl/ops/OpUtils.hpp>

#include <algorithm>
#include <stdexcept>
#include <string>

namespace dl::ops {

namespace {
[[noreturn]] void fail(const char* op, const std::string& what) {
    throw std::runtime_error(std::string(op) + ": " + what);
}
}  // namespace

void check_defined(const Tensor& t, const char* op, const char* name) {
    if (!t.defined()) fail(op, std::string(name) + " tensor is not defined");
}

void check_rank(const Tensor& t, int64_t rank, const char* op, const char* name) {
    if (t.shape().rank() != rank) fail(op, std::string(name) + " tensor has incorrect rank");
}

void check_cuda(const Tensor& t, const char* op, const char* name) {
    if (!t.device().is_cuda()) fail(op, std::string(name) + " tensor must be CUDA");
}

void check_dtype(const Tensor& t, DType dtype, const char* op, const char* name) {
    if (t.dtype() != dtype) fail(op, std::string(name) + " tensor must be " + dtype_name(dtype));
}

void check_float32(const Tensor& t, const char* op, const char* name) {
    check_dtype(t, DType::Float32, op, name);
}

void check_same_device(const Tensor& a, const Tensor& b, const char* op, const char* an, const char* bn) {
    if (a.device().type != b.device().type || a.device().index != b.device().index) {
        fail(op, std::string(an) + " and " + bn + " tensors must be on the same device");
    }
}

void check_same_dtype(const Tensor& a, const Tensor& b, const char* op, const char* an, const char* bn) {
    if (a.dtype() != b.dtype()) fail(op, std::string(an) + " and " + bn + " tensors must have the same dtype");
}

void check_same_shape(const Tensor& a, const Tensor& b, const char* op, const char* an, const char* bn) {
    if (a.shape() != b.shape()) fail(op, std::string(an) + " and " + bn + " tensors must have the same shape");
}

void check_binary_float_cuda_op(const Tensor& a, const Tensor& b, const char* op) {
    check_defined(a, op, "left");
    check_defined(b, op, "right");
    check_same_shape(a, b, op);
    check_same_dtype(a, b, op);
    check_float32(a, op, "left");
    check_cuda(a, op, "left");
    check_cuda(b, op, "right");
    check_same_device(a, b, op);
}

bool broadcast_shapes(const Shape& a, const Shape& b, std::vector<int64_t>* out,
                      std::vector<int64_t>* a_strides, std::vector<int64_t>* b_strides) {
    const std::size_t nd = std::max(a.dims.size(), b.dims.size());
    out->assign(nd, 1);
    a_strides->assign(nd, 0);
    b_strides->assign(nd, 0);
    int64_t acc_a = 1, acc_b = 1;
    for (std::size_t k = 0; k < nd; ++k) {
        const std::size_t i = nd - 1 - k;  // walk from the innermost dimension
        const int64_t da = k < a.dims.size() ? a.dims[a.dims.size() - 1 - k] : 1;
        const int64_t db = k < b.dims.size() ? b.dims[b.dims.size() - 1 - k] : 1;
        if (da != db && da != 1 && db != 1) return false;
        (*out)[i] = std::max(da, db);
        (*a_strides)[i] = da == 1 ? 0 : acc_a;
        (*b_strides)[i] = db == 1 ? 0 : acc_b;
        acc_a *= da;
        acc_b *= db;
    }
    return true;
}

}  // namespace dl::ops
