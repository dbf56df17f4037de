// Shape, DType, Device and the CUDA / kernel-library error helpers.
#include <dl/core/CudaUtils.hpp>
#include <dl/core/Types.hpp>

#include <fdl_kernels.h>

#include <stdexcept>
#include <string>
#include <utility>

namespace dl {

Shape::Shape(std::initializer_list<int64_t> extents) : dims(extents) {}
Shape::Shape(std::vector<int64_t> extents) : dims(std::move(extents)) {}

int64_t Shape::rank() const { return static_cast<int64_t>(dims.size()); }

int64_t Shape::numel() const {
    if (dims.empty()) return 0;  // no rank-0 scalars in this library
    int64_t n = 1;
    for (int64_t d : dims) n *= d;
    return n;
}

int64_t Shape::operator[](int index) const { return dims[static_cast<std::size_t>(index)]; }

std::string Shape::str() const {
    std::string s = "(";
    for (std::size_t i = 0; i < dims.size(); ++i) {
        if (i != 0) s += ", ";
        s += std::to_string(dims[i]);
    }
    return s + ")";
}

namespace {
struct DTypeInfo {
    DType dtype;
    std::size_t size;
    const char* name;
};
constexpr DTypeInfo kDTypes[] = {
    {DType::Float32, 4, "float32"}, {DType::Float16, 2, "float16"}, {DType::Int32, 4, "int32"},
    {DType::Int64, 8, "int64"},     {DType::Bool, 1, "bool"},
};
const DTypeInfo& info_of(DType dtype) {
    for (const DTypeInfo& i : kDTypes) {
        if (i.dtype == dtype) return i;
    }
    throw std::invalid_argument("unknown dtype");
}
}  // namespace

std::size_t dtype_size(DType dtype) { return info_of(dtype).size; }
std::string dtype_name(DType dtype) { return info_of(dtype).name; }

Device::Device(DeviceType t, int i) : type(t), index(i) {}
bool Device::is_cuda() const { return type == DeviceType::CUDA; }
bool Device::is_cpu() const { return type == DeviceType::CPU; }
std::string Device::str() const { return is_cuda() ? "cuda:" + std::to_string(index) : std::string("cpu"); }

namespace cuda {

void check(cudaError_t status, const char* action) {
    if (status == cudaSuccess) return;
    throw std::runtime_error(std::string(action) + ": " + cudaGetErrorString(status));
}

void check_fdl(int status, const char* action) {
    if (status == FDL_OK) return;
    throw std::runtime_error(std::string(action) + ": " + fdl_error_string(status));
}

void set_device(int device_index) {
    check(cudaSetDevice(device_index), "cudaSetDevice failed");
    check_fdl(fdl_set_device(device_index), "cudaSetDevice failed");
}

void synchronize() { check(cudaDeviceSynchronize(), "cudaDeviceSynchronize failed"); }

int device_count() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

}  // namespace cuda
}  // namespace dl
