// Host-buffer entry points: the same kernels, driven from HOST memory.
//
// This is what a caller that keeps its tensors in host memory pays end to end (the
// reference's Tensor::from_host -> op -> to_host round trip, src/tensor/TensorImpl.cpp:91-125).
// The input is cut into chunks that travel through a ring of device staging slots, each
// slot on its own stream: the host-to-device copy of chunk i+1, the kernel of chunk i and
// the device-to-host copy of chunk i-1 overlap, so a full-duplex PCIe link stays busy in
// both directions.  Staging buffers and streams are created once per device and kept
// (4 slots x 128 MiB).
// Host buffers should be pinned; pageable memory works but serialises the copies.
#include <mutex>

#include "fdl_common.cuh"

namespace fdl {

namespace {

constexpr int kSlots = 4;
constexpr int64_t kChunkElems = int64_t{8} << 20;  // 32 MiB of floats per operand per slot
constexpr int kMaxDevices = 64;

struct Pipeline {
    bool ready = false;
    cudaStream_t stream[kSlots] = {};
    float* a[kSlots] = {};
    float* b[kSlots] = {};
    float* out[kSlots] = {};
    float* out2[kSlots] = {};    // second result buffer (sweep)
    void* scratch[kSlots] = {};  // per-slot reduction scratch (sweep)
    double* partial = nullptr;   // one double per chunk of a sum
    int64_t partial_capacity = 0;
    float* row = nullptr;        // broadcast row vector
    int64_t row_capacity = 0;
};

std::mutex g_mutex;
Pipeline g_pipe[kMaxDevices];

int get_pipeline(Pipeline** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return FDL_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lock(g_mutex);
    Pipeline& p = g_pipe[dev];
    if (!p.ready) {
        for (int s = 0; s < kSlots; ++s) {
            e = cudaStreamCreateWithFlags(&p.stream[s], cudaStreamNonBlocking);
            if (e != cudaSuccess) return static_cast<int>(e);
            float* base = nullptr;
            const size_t scratch_bytes = fdl_sum_scratch_bytes(kChunkElems);
            e = cudaMalloc(&base, 4 * kChunkElems * sizeof(float) + scratch_bytes);
            if (e != cudaSuccess) return static_cast<int>(e);
            p.a[s] = base;
            p.b[s] = base + kChunkElems;
            p.out[s] = base + 2 * kChunkElems;
            p.out2[s] = base + 3 * kChunkElems;
            p.scratch[s] = base + 4 * kChunkElems;
            e = cudaMemset(p.scratch[s], 0, scratch_bytes);
            if (e != cudaSuccess) return static_cast<int>(e);
        }
        p.ready = true;
    }
    *out = &p;
    return FDL_OK;
}

int sync_all(Pipeline* p) {
    for (int s = 0; s < kSlots; ++s) {
        cudaError_t e = cudaStreamSynchronize(p->stream[s]);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    return FDL_OK;
}

#define FDL_TRY(expr)                                   \
    do {                                                \
        const int fdl_try_status = static_cast<int>(expr); \
        if (fdl_try_status != 0) return fdl_try_status; \
    } while (0)

}  // namespace

}  // namespace fdl

using namespace fdl;

extern "C" {

int fdl_host_binary_f32(const float* h_a, const float* h_b, float* h_out, int64_t n, int op) {
    if (n < 0 || (n > 0 && (h_a == nullptr || h_b == nullptr || h_out == nullptr))) {
        return FDL_ERR_INVALID_ARGUMENT;
    }
    Pipeline* p = nullptr;
    FDL_TRY(get_pipeline(&p));
    int slot = 0;
    for (int64_t off = 0; off < n; off += kChunkElems, slot = (slot + 1) % kSlots) {
        const int64_t m = n - off < kChunkElems ? n - off : kChunkElems;
        cudaStream_t s = p->stream[slot];
        FDL_TRY(cudaMemcpyAsync(p->a[slot], h_a + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_TRY(cudaMemcpyAsync(p->b[slot], h_b + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_TRY(fdl_binary_f32(p->a[slot], p->b[slot], p->out[slot], m, op, s));
        FDL_TRY(cudaMemcpyAsync(h_out + off, p->out[slot], m * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    return sync_all(p);
}

int fdl_host_unary_f32(const float* h_x, float* h_out, int64_t n, int op, float alpha) {
    if (n < 0 || (n > 0 && (h_x == nullptr || h_out == nullptr))) return FDL_ERR_INVALID_ARGUMENT;
    Pipeline* p = nullptr;
    FDL_TRY(get_pipeline(&p));
    int slot = 0;
    for (int64_t off = 0; off < n; off += kChunkElems, slot = (slot + 1) % kSlots) {
        const int64_t m = n - off < kChunkElems ? n - off : kChunkElems;
        cudaStream_t s = p->stream[slot];
        FDL_TRY(cudaMemcpyAsync(p->a[slot], h_x + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_TRY(fdl_unary_f32(p->a[slot], p->out[slot], m, op, alpha, s));
        FDL_TRY(cudaMemcpyAsync(h_out + off, p->out[slot], m * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    return sync_all(p);
}

int fdl_host_mul_add_relu_f32(const float* h_a, const float* h_b, const float* h_c, float* h_out,
                              int64_t n) {
    if (n < 0 || (n > 0 && (h_a == nullptr || h_b == nullptr || h_c == nullptr || h_out == nullptr))) {
        return FDL_ERR_INVALID_ARGUMENT;
    }
    Pipeline* p = nullptr;
    FDL_TRY(get_pipeline(&p));
    int slot = 0;
    for (int64_t off = 0; off < n; off += kChunkElems, slot = (slot + 1) % kSlots) {
        const int64_t m = n - off < kChunkElems ? n - off : kChunkElems;
        cudaStream_t s = p->stream[slot];
        // The third operand lands in the output buffer and is overwritten in place.
        FDL_TRY(cudaMemcpyAsync(p->a[slot], h_a + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_TRY(cudaMemcpyAsync(p->b[slot], h_b + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_TRY(cudaMemcpyAsync(p->out[slot], h_c + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_TRY(fdl_mul_add_relu_f32(p->a[slot], p->b[slot], p->out[slot], p->out[slot], m, s));
        FDL_TRY(cudaMemcpyAsync(h_out + off, p->out[slot], m * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    return sync_all(p);
}

int fdl_host_row_broadcast_f32(const float* h_a, const float* h_row, float* h_out, int64_t rows,
                               int64_t cols, int op) {
    if (rows < 0 || cols < 0) return FDL_ERR_INVALID_ARGUMENT;
    if (rows == 0 || cols == 0) return FDL_OK;
    if (h_a == nullptr || h_row == nullptr || h_out == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    if (cols > kChunkElems) return FDL_ERR_UNSUPPORTED;
    Pipeline* p = nullptr;
    FDL_TRY(get_pipeline(&p));
    if (p->row_capacity < cols) {
        FDL_TRY(sync_all(p));
        if (p->row != nullptr) cudaFree(p->row);
        p->row = nullptr;
        FDL_TRY(cudaMalloc(&p->row, cols * sizeof(float)));
        p->row_capacity = cols;
    }
    // The row vector is uploaded once and every slot's stream waits for it.
    cudaEvent_t row_ready;
    FDL_TRY(cudaEventCreateWithFlags(&row_ready, cudaEventDisableTiming));
    FDL_TRY(cudaMemcpyAsync(p->row, h_row, cols * sizeof(float), cudaMemcpyHostToDevice, p->stream[0]));
    FDL_TRY(cudaEventRecord(row_ready, p->stream[0]));
    for (int s = 1; s < kSlots; ++s) FDL_TRY(cudaStreamWaitEvent(p->stream[s], row_ready, 0));

    const int64_t rows_per_chunk = kChunkElems / cols;
    const int64_t shape[2] = {0, cols};
    const int64_t a_strides[2] = {cols, 1};
    const int64_t b_strides[2] = {0, 1};
    int slot = 0;
    int status = FDL_OK;
    for (int64_t r = 0; r < rows && status == FDL_OK; r += rows_per_chunk, slot = (slot + 1) % kSlots) {
        const int64_t nr = rows - r < rows_per_chunk ? rows - r : rows_per_chunk;
        const int64_t m = nr * cols;
        cudaStream_t s = p->stream[slot];
        int64_t shp[2] = {nr, shape[1]};
        status = static_cast<int>(cudaMemcpyAsync(p->a[slot], h_a + r * cols, m * sizeof(float),
                                                  cudaMemcpyHostToDevice, s));
        if (status == FDL_OK) {
            status = fdl_broadcast_binary_f32(p->a[slot], p->row, p->out[slot], 2, shp, a_strides,
                                              b_strides, op, s);
        }
        if (status == FDL_OK) {
            status = static_cast<int>(cudaMemcpyAsync(h_out + r * cols, p->out[slot], m * sizeof(float),
                                                      cudaMemcpyDeviceToHost, s));
        }
    }
    const int sync_status = sync_all(p);
    cudaEventDestroy(row_ready);
    return status != FDL_OK ? status : sync_status;
}

int fdl_host_sweep_f32(const float* h_x, const float* h_y, const float* h_row, float* h_z,
                       float* h_w, int64_t rows, int64_t cols, double* h_sum) {
    if (rows < 0 || cols < 0 || h_sum == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    *h_sum = 0.0;
    if (rows == 0 || cols == 0) return FDL_OK;
    if (h_x == nullptr || h_y == nullptr || h_row == nullptr || h_z == nullptr || h_w == nullptr) {
        return FDL_ERR_INVALID_ARGUMENT;
    }
    if (cols > kChunkElems) return FDL_ERR_UNSUPPORTED;
    Pipeline* p = nullptr;
    FDL_TRY(get_pipeline(&p));
    const int64_t rows_per_chunk = kChunkElems / cols;
    const int64_t nchunks = ceil_div(rows, rows_per_chunk);
    if (p->row_capacity < cols) {
        FDL_TRY(sync_all(p));
        if (p->row != nullptr) cudaFree(p->row);
        p->row = nullptr;
        FDL_TRY(cudaMalloc(&p->row, cols * sizeof(float)));
        p->row_capacity = cols;
    }
    if (p->partial_capacity < nchunks) {
        FDL_TRY(sync_all(p));
        if (p->partial != nullptr) cudaFree(p->partial);
        p->partial = nullptr;
        FDL_TRY(cudaMalloc(&p->partial, nchunks * sizeof(double)));
        p->partial_capacity = nchunks;
    }
    cudaEvent_t row_ready;
    FDL_TRY(cudaEventCreateWithFlags(&row_ready, cudaEventDisableTiming));
    int status = static_cast<int>(
        cudaMemcpyAsync(p->row, h_row, cols * sizeof(float), cudaMemcpyHostToDevice, p->stream[0]));
    if (status == FDL_OK) status = static_cast<int>(cudaEventRecord(row_ready, p->stream[0]));
    for (int s = 1; s < kSlots && status == FDL_OK; ++s) {
        status = static_cast<int>(cudaStreamWaitEvent(p->stream[s], row_ready, 0));
    }
    const size_t scratch_bytes = fdl_sum_scratch_bytes(kChunkElems);
    const int64_t a_strides[2] = {cols, 1};
    const int64_t b_strides[2] = {0, 1};
    int slot = 0;
    int64_t chunk = 0;
    for (int64_t r = 0; r < rows && status == FDL_OK; r += rows_per_chunk, ++chunk, slot = (slot + 1) % kSlots) {
        const int64_t nr = rows - r < rows_per_chunk ? rows - r : rows_per_chunk;
        const int64_t m = nr * cols;
        const int64_t shape[2] = {nr, cols};
        cudaStream_t s = p->stream[slot];
        const size_t bytes = m * sizeof(float);
        // Each chunk of x and y crosses the link once and feeds all three operations.
        status = static_cast<int>(cudaMemcpyAsync(p->a[slot], h_x + r * cols, bytes, cudaMemcpyHostToDevice, s));
        if (status == FDL_OK) status = static_cast<int>(cudaMemcpyAsync(p->b[slot], h_y + r * cols, bytes, cudaMemcpyHostToDevice, s));
        if (status == FDL_OK) status = fdl_binary_f32(p->a[slot], p->b[slot], p->out[slot], m, FDL_ADD, s);
        if (status == FDL_OK) status = static_cast<int>(cudaMemcpyAsync(h_z + r * cols, p->out[slot], bytes, cudaMemcpyDeviceToHost, s));
        if (status == FDL_OK) status = fdl_broadcast_binary_f32(p->a[slot], p->row, p->out2[slot], 2, shape, a_strides, b_strides, FDL_ADD, s);
        if (status == FDL_OK) status = static_cast<int>(cudaMemcpyAsync(h_w + r * cols, p->out2[slot], bytes, cudaMemcpyDeviceToHost, s));
        if (status == FDL_OK) status = fdl_sum_f32(p->a[slot], m, nullptr, p->partial + chunk, p->scratch[slot], scratch_bytes, s);
    }
    const int sync_status = sync_all(p);
    cudaEventDestroy(row_ready);
    if (status != FDL_OK) return status;
    if (sync_status != FDL_OK) return sync_status;
    double stack_buf[64];
    double* host_partials = nchunks <= 64 ? stack_buf : new double[nchunks];
    const cudaError_t e = cudaMemcpy(host_partials, p->partial, nchunks * sizeof(double), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) {
        double total = 0.0;
        for (int64_t k = 0; k < nchunks; ++k) total += host_partials[k];  // chunk order: deterministic
        *h_sum = total;
    }
    if (host_partials != stack_buf) delete[] host_partials;
    return static_cast<int>(e);
}

int fdl_host_sum_f32(const float* h_x, int64_t n, double* h_out) {
    if (n < 0 || h_out == nullptr || (n > 0 && h_x == nullptr)) return FDL_ERR_INVALID_ARGUMENT;
    Pipeline* p = nullptr;
    FDL_TRY(get_pipeline(&p));
    const int64_t nchunks = ceil_div(n, kChunkElems);
    if (nchunks == 0) {
        *h_out = 0.0;
        return FDL_OK;
    }
    if (p->partial_capacity < nchunks) {
        FDL_TRY(sync_all(p));
        if (p->partial != nullptr) cudaFree(p->partial);
        p->partial = nullptr;
        FDL_TRY(cudaMalloc(&p->partial, nchunks * sizeof(double)));
        p->partial_capacity = nchunks;
    }
    // Each slot reduces into its own scratch, so reductions of different chunks may overlap.
    const size_t scratch_bytes = fdl_sum_scratch_bytes(kChunkElems);
    int slot = 0;
    int64_t chunk = 0;
    for (int64_t off = 0; off < n; off += kChunkElems, ++chunk, slot = (slot + 1) % kSlots) {
        const int64_t m = n - off < kChunkElems ? n - off : kChunkElems;
        cudaStream_t s = p->stream[slot];
        FDL_TRY(cudaMemcpyAsync(p->a[slot], h_x + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_TRY(fdl_sum_f32(p->a[slot], m, nullptr, p->partial + chunk, p->scratch[slot], scratch_bytes, s));
    }
    FDL_TRY(sync_all(p));
    // Chunk partials are folded on the host in chunk order: deterministic.
    double stack_buf[64];
    double* host_partials = nchunks <= 64 ? stack_buf : new double[nchunks];
    cudaError_t e = cudaMemcpy(host_partials, p->partial, nchunks * sizeof(double), cudaMemcpyDeviceToHost);
    double total = 0.0;
    if (e == cudaSuccess) {
        for (int64_t k = 0; k < nchunks; ++k) total += host_partials[k];
        *h_out = total;
    }
    if (host_partials != stack_buf) delete[] host_partials;
    return static_cast<int>(e);
}

}  // extern "C"
