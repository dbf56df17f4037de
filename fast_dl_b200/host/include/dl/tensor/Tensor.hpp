// dl::Tensor -- a cheap-to-copy handle on a contiguous device buffer.
//
// Public surface identical to fast_dl's include/dl/tensor/Tensor.hpp:35-94 (constructors,
// factories, copies, to_host/from_host, accessors; copying a Tensor aliases the same
// storage).  What differs is underneath: storage comes from a per-device caching allocator
// (dl/tensor/Allocator.hpp) instead of one cudaMalloc/cudaFree per tensor.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <vector>

#include <dl/core/Types.hpp>

namespace dl {

class TensorImpl;

/// Maps a host element type to the DType it is stored as.
template <typename T>
DType tensor_dtype();
template <>
inline DType tensor_dtype<float>() { return DType::Float32; }
template <>
inline DType tensor_dtype<int32_t>() { return DType::Int32; }
template <>
inline DType tensor_dtype<int64_t>() { return DType::Int64; }

class Tensor {
public:
    /// An undefined tensor: no storage, numel() == 0, defined() == false.
    Tensor() = default;
    /// Uninitialised storage of `shape` x `dtype` on `device` (CUDA only).
    Tensor(const Shape& shape, DType dtype = DType::Float32, Device device = Device());

    ~Tensor() = default;
    Tensor(const Tensor&) = default;
    Tensor& operator=(const Tensor&) = default;
    Tensor(Tensor&&) noexcept = default;
    Tensor& operator=(Tensor&&) noexcept = default;

    // ---- factories ----
    static Tensor empty(const Shape& shape, DType dtype = DType::Float32, Device device = Device());
    static Tensor zeros(const Shape& shape, DType dtype = DType::Float32, Device device = Device());
    static Tensor empty_like(const Tensor& other);
    static Tensor zeros_like(const Tensor& other);
    /// N(mean, stddev) / U(low, high]: a pure function of (seed, element index).
    static Tensor randn(Shape shape, DType dtype, Device device, float mean, float stddev,
                        uint64_t seed = 1234);
    static Tensor uniform(Shape shape, DType dtype, Device device, float low, float high,
                          uint64_t seed = 1234);
    /// U(-l, l) with l = sqrt(6 / (fan_in + fan_out)); fans are the last two extents.
    static Tensor xavier_uniform(Shape shape, DType dtype, Device device, uint64_t seed = 1234);
    /// U(-l, l) with l = sqrt(6 / fan_in).
    static Tensor kaiming_uniform(Shape shape, DType dtype, Device device, uint64_t seed = 1234);

    template <typename T>
    static Tensor from_host(const std::vector<T>& data, const Shape& shape, Device device = Device()) {
        if (shape.numel() != static_cast<int64_t>(data.size())) {
            throw std::runtime_error("from_host data size does not match shape");
        }
        Tensor t(shape, tensor_dtype<T>(), device);
        t.copy_from_host(data.data(), data.size() * sizeof(T));
        return t;
    }

    // ---- accessors ----
    void* data();
    const void* data() const;
    const Shape& shape() const;
    DType dtype() const;
    Device device() const;
    int64_t numel() const;
    std::size_t nbytes() const;
    /// True when the handle owns non-empty storage (zero-element tensors are undefined).
    bool defined() const;

    // ---- data movement (blocking, like the reference) ----
    void copy_from_host(const void* src, std::size_t bytes);
    void copy_to_host(void* dst, std::size_t bytes) const;
    void copy_from(const Tensor& src);
    void copy_to(Tensor& dst) const;
    void zero_();

    template <typename T>
    std::vector<T> to_host() const {
        if (dtype() != tensor_dtype<T>()) {
            throw std::runtime_error("to_host dtype does not match requested host type");
        }
        std::vector<T> out(static_cast<std::size_t>(numel()));
        copy_to_host(out.data(), out.size() * sizeof(T));
        return out;
    }

    /// Same storage, different shape (numel must match).  Extension: fast_dl has no views.
    Tensor reshaped(const Shape& shape) const;

private:
    std::shared_ptr<TensorImpl> impl_;
};

}  // namespace dl

using Tensor = dl::Tensor;
using dl::tensor_dtype;
