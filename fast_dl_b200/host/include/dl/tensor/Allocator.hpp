// Per-device caching allocator for tensor storage.
//
// fast_dl calls cudaMalloc in every TensorImpl constructor and cudaFree in every
// destructor (src/tensor/TensorImpl.cpp:69-89); both synchronise the device, and for the
// small and medium tensors of this path they cost more than the kernels.  Here freed
// blocks go to a size-bucketed free list and are handed out again.  Reuse is safe without
// events because all work of this library is enqueued on one stream per device (the
// legacy default stream): a block freed by the host after op A was enqueued can only be
// written by an op enqueued later on the same stream, i.e. after A has finished.
#pragma once

#include <cstddef>
#include <memory>

namespace dl {

struct DeviceBlock {
    void* ptr = nullptr;
    std::size_t bytes = 0;   // rounded-up capacity
    int device = 0;
    ~DeviceBlock();          // returns the block to the cache
};

namespace allocator {

/// A block of at least `bytes` on `device` (cache hit or cudaMalloc; on out-of-memory the
/// cache is emptied once and the allocation retried).  Throws std::runtime_error.
std::shared_ptr<DeviceBlock> allocate(std::size_t bytes, int device);

/// cudaFree everything that is cached (not blocks in use).
void empty_cache();

struct Stats {
    std::size_t cuda_malloc_calls = 0;
    std::size_t cache_hits = 0;
    std::size_t bytes_in_use = 0;
    std::size_t bytes_cached = 0;
};
Stats stats();

/// false: every allocation is a cudaMalloc and every release a cudaFree (the reference's
/// behaviour; for measuring what the cache buys).  Default true.
void set_caching(bool enabled);

}  // namespace allocator
}  // namespace dl
