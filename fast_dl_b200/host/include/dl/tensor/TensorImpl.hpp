// Storage behind dl::Tensor: shape + dtype + device + a block from the caching allocator.
// Several TensorImpl may share one block (reshaped views); the block returns to the
// allocator's free list when the last owner goes away.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>

#include <dl/core/Types.hpp>

namespace dl {

struct DeviceBlock;  // dl/tensor/Allocator.hpp

class TensorImpl {
public:
    TensorImpl(const Shape& shape, DType dtype, Device device);
    TensorImpl(const Shape& shape, const TensorImpl& shares_storage_with);
    ~TensorImpl() = default;
    TensorImpl(const TensorImpl&) = delete;
    TensorImpl& operator=(const TensorImpl&) = delete;

    void* data();
    const void* data() const;
    const Shape& shape() const { return shape_; }
    DType dtype() const { return dtype_; }
    Device device() const { return device_; }
    int64_t numel() const { return shape_.numel(); }
    std::size_t nbytes() const;

    void copy_from_host(const void* src, std::size_t bytes);
    void copy_to_host(void* dst, std::size_t bytes) const;
    void copy_from(const TensorImpl& src);
    void zero_();

private:
    Shape shape_;
    DType dtype_ = DType::Float32;
    Device device_;
    std::shared_ptr<DeviceBlock> block_;
};

}  // namespace dl

using TensorImpl = dl::TensorImpl;
