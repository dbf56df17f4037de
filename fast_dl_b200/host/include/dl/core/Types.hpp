// Value types shared by every layer of the host library: Shape, DType, Device.
//
// Same names, members and behaviour as fast_dl's include/dl/core/{Shape,DType,Device}.hpp
// (semantics pinned by src/core/Shape.cpp:17-23: numel() of a rank-0 shape is 0, not 1;
// src/core/DType.cpp:7-37: sizes 4/2/4/8/1 and lower-case names; src/core/Device.cpp:11-20:
// "cuda:<index>" / "cpu").  Kept in one header; the per-type headers forward here.
#pragma once

#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <string>
#include <vector>

namespace dl {

/// Dimension list of a dense row-major tensor.
class Shape {
public:
    std::vector<int64_t> dims;

    Shape() = default;
    Shape(std::initializer_list<int64_t> extents);
    explicit Shape(std::vector<int64_t> extents);

    /// Number of dimensions.
    int64_t rank() const;
    /// Product of the extents; 0 for a shape without dimensions.
    int64_t numel() const;
    /// Extent of dimension `index` (unchecked).
    int64_t operator[](int index) const;
    /// "(d0, d1, ...)".
    std::string str() const;

    bool operator==(const Shape& other) const { return dims == other.dims; }
    bool operator!=(const Shape& other) const { return dims != other.dims; }
};

enum class DType { Float32, Float16, Int32, Int64, Bool };

/// Bytes per element.  Throws std::invalid_argument for an unknown value.
std::size_t dtype_size(DType dtype);
/// "float32", "float16", "int32", "int64", "bool".
std::string dtype_name(DType dtype);

enum class DeviceType { CPU, CUDA };

/// Where a tensor lives.  Default: CUDA device 0.
class Device {
public:
    DeviceType type;
    int index;

    Device(DeviceType type = DeviceType::CUDA, int index = 0);

    bool is_cuda() const;
    bool is_cpu() const;
    std::string str() const;
};

}  // namespace dl

// fast_dl also exposes these names at global scope.
using Shape = dl::Shape;
using DType = dl::DType;
using DeviceType = dl::DeviceType;
using Device = dl::Device;
using dl::dtype_name;
using dl::dtype_size;
