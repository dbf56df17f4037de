// Caching allocator, TensorImpl and Tensor.
#include <dl/tensor/Allocator.hpp>
#include <dl/tensor/Tensor.hpp>
#include <dl/tensor/TensorImpl.hpp>

#include <dl/core/CudaUtils.hpp>
#include <dl/kernels/kernels.hpp>

#include <cuda_runtime.h>

#include <cmath>
#include <map>
#include <mutex>
#include <stdexcept>
#include <vector>

namespace dl {

// ---- allocator ----------------------------------------------------------------------------------

namespace allocator {
namespace {

struct State {
    std::mutex mutex;
    bool caching = true;
    // device -> capacity -> free pointers of exactly that capacity
    std::map<int, std::multimap<std::size_t, void*>> free_lists;
    Stats stats;
};

State& state() {
    static State* s = new State();  // leaked on purpose: blocks may be released during exit
    return *s;
}

// 512-byte granules up to 1 MiB, 2 MiB granules above: few distinct sizes, little waste.
std::size_t round_up(std::size_t bytes) {
    const std::size_t g = bytes <= (std::size_t{1} << 20) ? 512 : (std::size_t{2} << 20);
    return (bytes + g - 1) / g * g;
}

void free_cached_locked(State& s, int device_filter) {
    for (auto& [device, list] : s.free_lists) {
        if (device_filter >= 0 && device != device_filter) continue;
        cudaSetDevice(device);
        for (auto& [bytes, ptr] : list) {
            cudaFree(ptr);
            s.stats.bytes_cached -= bytes;
        }
        list.clear();
    }
}

}  // namespace

std::shared_ptr<DeviceBlock> allocate(std::size_t bytes, int device) {
    State& s = state();
    const std::size_t cap = round_up(bytes);
    auto block = std::make_shared<DeviceBlock>();
    block->bytes = cap;
    block->device = device;
    std::lock_guard<std::mutex> lock(s.mutex);
    if (s.caching) {
        auto& list = s.free_lists[device];
        auto it = list.lower_bound(cap);
        // Accept a cached block up to 25% larger than asked for.
        if (it != list.end() && it->first <= cap + cap / 4) {
            block->ptr = it->second;
            block->bytes = it->first;
            s.stats.bytes_cached -= it->first;
            s.stats.bytes_in_use += it->first;
            ++s.stats.cache_hits;
            list.erase(it);
            return block;
        }
    }
    dl::cuda::check(cudaSetDevice(device), "cudaSetDevice failed");
    cudaError_t e = cudaMalloc(&block->ptr, cap);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        free_cached_locked(s, device);
        e = cudaMalloc(&block->ptr, cap);
    }
    dl::cuda::check(e, "cudaMalloc failed");
    ++s.stats.cuda_malloc_calls;
    s.stats.bytes_in_use += cap;
    return block;
}

void empty_cache() {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    free_cached_locked(s, -1);
}

Stats stats() {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    return s.stats;
}

void set_caching(bool enabled) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mutex);
    s.caching = enabled;
    if (!enabled) free_cached_locked(s, -1);
}

}  // namespace allocator

DeviceBlock::~DeviceBlock() {
    if (ptr == nullptr) return;
    auto& s = allocator::state();
    std::lock_guard<std::mutex> lock(s.mutex);
    s.stats.bytes_in_use -= bytes;
    if (s.caching) {
        s.free_lists[device].emplace(bytes, ptr);
        s.stats.bytes_cached += bytes;
    } else {
        cudaSetDevice(device);
        cudaFree(ptr);
    }
}

// ---- TensorImpl -----------------------------------------------------------------------------------

TensorImpl::TensorImpl(const Shape& shape, DType dtype, Device device)
    : shape_(shape), dtype_(dtype), device_(device) {
    if (nbytes() == 0) return;  // zero-element tensors own nothing and count as undefined
    if (!device_.is_cuda()) throw std::runtime_error("Tensor currently supports CUDA allocation only");
    block_ = allocator::allocate(nbytes(), device_.index);
}

TensorImpl::TensorImpl(const Shape& shape, const TensorImpl& other)
    : shape_(shape), dtype_(other.dtype_), device_(other.device_), block_(other.block_) {}

void* TensorImpl::data() { return block_ ? block_->ptr : nullptr; }
const void* TensorImpl::data() const { return block_ ? block_->ptr : nullptr; }
std::size_t TensorImpl::nbytes() const { return static_cast<std::size_t>(numel()) * dtype_size(dtype_); }

namespace {
// One blocking cudaMemcpy / cudaMemset on `device`, with the library's error convention.  The four
// data-moving members below differ only in their size rule, their direction and their messages.
struct DeviceOp {
    int device;
    explicit DeviceOp(const Device& d, const char* cuda_only_message) : device(d.index) {
        if (!d.is_cuda()) throw std::runtime_error(cuda_only_message);
        dl::cuda::check(cudaSetDevice(device), "cudaSetDevice failed");
    }
    void copy(void* dst, const void* src, std::size_t bytes, cudaMemcpyKind kind, const char* failure) const {
        dl::cuda::check(cudaMemcpy(dst, src, bytes, kind), failure);
    }
};

void require_fits(std::size_t bytes, std::size_t capacity, const char* message) {
    if (bytes > capacity) throw std::runtime_error(message);
}
}  // namespace

void TensorImpl::copy_from_host(const void* src, std::size_t bytes) {
    require_fits(bytes, nbytes(), "copy_from_host exceeds tensor size");
    if (bytes != 0) {
        DeviceOp(device_, "copy_from_host currently supports CUDA tensors only")
            .copy(data(), src, bytes, cudaMemcpyHostToDevice, "cudaMemcpy host to device failed");
    }
}

void TensorImpl::copy_to_host(void* dst, std::size_t bytes) const {
    require_fits(bytes, nbytes(), "copy_to_host exceeds tensor size");
    if (bytes != 0) {
        DeviceOp(device_, "copy_to_host currently supports CUDA tensors only")
            .copy(dst, data(), bytes, cudaMemcpyDeviceToHost, "cudaMemcpy device to host failed");
    }
}

void TensorImpl::copy_from(const TensorImpl& src) {
    const std::size_t bytes = nbytes();
    if (src.nbytes() != bytes) throw std::runtime_error("tensor copy size mismatch");
    if (bytes == 0) return;
    const char* cuda_only = "copy_from currently supports CUDA to CUDA only";
    if (!src.device().is_cuda()) throw std::runtime_error(cuda_only);
    // cudaMemcpyDefault also covers a source on another GPU (peer copy through the driver).
    DeviceOp(device_, cuda_only).copy(data(), src.data(), bytes, cudaMemcpyDefault, "cudaMemcpy device to device failed");
}

void TensorImpl::zero_() {
    const std::size_t bytes = nbytes();
    if (bytes == 0) return;
    const DeviceOp op(device_, "zero_ currently supports CUDA tensors only");
    dl::cuda::check(cudaMemset(data(), 0, bytes), "cudaMemset failed");
}

// ---- Tensor ---------------------------------------------------------------------------------------

namespace {
const Shape& no_shape() {
    static const Shape s;
    return s;
}

Tensor random_fill(Shape shape, DType dtype, Device device, bool normal, float p0, float p1,
                   uint64_t seed, const char* who) {
    if (dtype != DType::Float32) throw std::runtime_error(std::string(who) + " currently supports Float32 only");
    if (!device.is_cuda()) throw std::runtime_error(std::string(who) + " currently supports CUDA only");
    Tensor out(shape, dtype, device);
    dl::cuda::set_device(device.index);
    if (normal) dl::kernels::normal_float32(static_cast<float*>(out.data()), out.numel(), p0, p1, seed);
    else dl::kernels::uniform_float32(static_cast<float*>(out.data()), out.numel(), p0, p1, seed);
    return out;
}
}  // namespace

Tensor::Tensor(const Shape& shape, DType dtype, Device device)
    : impl_(std::make_shared<TensorImpl>(shape, dtype, device)) {}

Tensor Tensor::empty(const Shape& shape, DType dtype, Device device) { return Tensor(shape, dtype, device); }

Tensor Tensor::zeros(const Shape& shape, DType dtype, Device device) {
    Tensor t(shape, dtype, device);
    t.zero_();
    return t;
}

Tensor Tensor::empty_like(const Tensor& other) {
    if (!other.defined()) throw std::runtime_error("empty_like requires a defined tensor");
    return Tensor(other.shape(), other.dtype(), other.device());
}

Tensor Tensor::zeros_like(const Tensor& other) {
    Tensor t = empty_like(other);
    t.zero_();
    return t;
}

Tensor Tensor::randn(Shape shape, DType dtype, Device device, float mean, float stddev, uint64_t seed) {
    return random_fill(shape, dtype, device, true, mean, stddev, seed, "Tensor::randn");
}

Tensor Tensor::uniform(Shape shape, DType dtype, Device device, float low, float high, uint64_t seed) {
    return random_fill(shape, dtype, device, false, low, high, seed, "Tensor::uniform");
}

namespace {
// The two fan sizes of a weight of rank >= 2: its last two extents.
struct Fans {
    float in, out;
    Fans(const Shape& shape, const char* who) {
        if (shape.rank() < 2) throw std::runtime_error(std::string(who) + " requires rank >= 2");
        const int r = static_cast<int>(shape.rank());
        in = static_cast<float>(shape[r - 2]);
        out = static_cast<float>(shape[r - 1]);
    }
};
}  // namespace

// uniform(-limit, limit) with limit = sqrt(6 / (fan_in + fan_out)) (Xavier) or sqrt(6 / fan_in) (Kaiming).
Tensor Tensor::xavier_uniform(Shape shape, DType dtype, Device device, uint64_t seed) {
    const Fans fans(shape, "Tensor::xavier_uniform");
    const float limit = std::sqrt(6.0f / (fans.in + fans.out));
    return uniform(shape, dtype, device, -limit, limit, seed);
}

Tensor Tensor::kaiming_uniform(Shape shape, DType dtype, Device device, uint64_t seed) {
    const Fans fans(shape, "Tensor::kaiming_uniform");
    const float limit = std::sqrt(6.0f / fans.in);
    return uniform(shape, dtype, device, -limit, limit, seed);
}

void* Tensor::data() { return impl_ ? impl_->data() : nullptr; }
const void* Tensor::data() const { return impl_ ? impl_->data() : nullptr; }
const Shape& Tensor::shape() const { return impl_ ? impl_->shape() : no_shape(); }
DType Tensor::dtype() const { return impl_ ? impl_->dtype() : DType::Float32; }
Device Tensor::device() const { return impl_ ? impl_->device() : Device(); }
int64_t Tensor::numel() const { return impl_ ? impl_->numel() : 0; }
std::size_t Tensor::nbytes() const { return impl_ ? impl_->nbytes() : 0; }
bool Tensor::defined() const { return impl_ != nullptr && impl_->data() != nullptr; }

void Tensor::copy_from_host(const void* src, std::size_t bytes) {
    if (!impl_) throw std::runtime_error("copy_from_host requires a defined tensor");
    impl_->copy_from_host(src, bytes);
}
void Tensor::copy_to_host(void* dst, std::size_t bytes) const {
    if (!impl_) throw std::runtime_error("copy_to_host requires a defined tensor");
    impl_->copy_to_host(dst, bytes);
}
void Tensor::copy_from(const Tensor& src) {
    if (!impl_ || !src.impl_) throw std::runtime_error("copy_from requires defined tensors");
    impl_->copy_from(*src.impl_);
}
void Tensor::copy_to(Tensor& dst) const { dst.copy_from(*this); }
void Tensor::zero_() {
    if (!impl_) throw std::runtime_error("zero_ requires a defined tensor");
    impl_->zero_();
}

Tensor Tensor::reshaped(const Shape& shape) const {
    if (!impl_) throw std::runtime_error("reshaped requires a defined tensor");
    if (shape.numel() != numel()) throw std::runtime_error("reshaped: element count differs");
    Tensor t;
    t.impl_ = std::make_shared<TensorImpl>(shape, *impl_);
    return t;
}

}  // namespace dl
