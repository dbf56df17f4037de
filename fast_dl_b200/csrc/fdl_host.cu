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
// The calls on one device share that ring: each call holds the device's lock from start to
// finish, so concurrent callers on the same device are serialised (different devices are
// independent).  Whatever goes wrong inside a call, it returns only after every copy it has
// enqueued has finished, so the caller may free its buffers as soon as it has the status.
#include <mutex>

#include "fdl_common.cuh"

namespace fdl {

namespace {

constexpr int kSlots = 4;
constexpr int64_t kChunkElems = int64_t{8} << 20;  // 32 MiB of floats per operand per slot
constexpr int kMaxDevices = 64;

struct Pipeline {
    std::mutex call_mutex;  // held for the whole of every fdl_host_* call on this device
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
        for (int s = 0; s < kSlots && e == cudaSuccess; ++s) {
            e = cudaStreamCreateWithFlags(&p.stream[s], cudaStreamNonBlocking);
            if (e != cudaSuccess) break;
            float* base = nullptr;
            const size_t scratch_bytes = fdl_sum_scratch_bytes(kChunkElems);
            e = cudaMalloc(&base, 4 * kChunkElems * sizeof(float) + scratch_bytes);
            if (e != cudaSuccess) break;
            p.a[s] = base;
            p.b[s] = base + kChunkElems;
            p.out[s] = base + 2 * kChunkElems;
            p.out2[s] = base + 3 * kChunkElems;
            p.scratch[s] = base + 4 * kChunkElems;
            e = cudaMemset(p.scratch[s], 0, scratch_bytes);
        }
        if (e != cudaSuccess) {
            // Give back what was created, so that a later call starts from nothing.
            for (int s = 0; s < kSlots; ++s) {
                if (p.a[s] != nullptr) cudaFree(p.a[s]);
                if (p.stream[s] != nullptr) cudaStreamDestroy(p.stream[s]);
                p.a[s] = p.b[s] = p.out[s] = p.out2[s] = nullptr;
                p.scratch[s] = nullptr;
                p.stream[s] = nullptr;
            }
            return static_cast<int>(e);
        }
        p.ready = true;
    }
    *out = &p;
    return FDL_OK;
}

// Waits for every slot even when one of them reports an error; returns the first error.
int sync_all(Pipeline* p) {
    int first = FDL_OK;
    for (int s = 0; s < kSlots; ++s) {
        const cudaError_t e = cudaStreamSynchronize(p->stream[s]);
        if (e != cudaSuccess && first == FDL_OK) first = static_cast<int>(e);
    }
    return first;
}

// Grows a device buffer of the pipeline (after draining the streams that may still use it).
template <class T>
int ensure_capacity(Pipeline* p, T** buffer, int64_t* capacity, int64_t want) {
    if (*capacity >= want) return FDL_OK;
    const int st = sync_all(p);
    if (st != FDL_OK) return st;
    if (*buffer != nullptr) cudaFree(*buffer);
    *buffer = nullptr;
    *capacity = 0;
    const cudaError_t e = cudaMalloc(buffer, want * sizeof(T));
    if (e != cudaSuccess) return static_cast<int>(e);
    *capacity = want;
    return FDL_OK;
}

// `status` keeps the first failure; later steps are skipped once it is set.
#define FDL_STEP(expr)                                       \
    do {                                                     \
        if (status == FDL_OK) status = static_cast<int>(expr); \
    } while (0)

// The end of every call: drain all slots whatever happened, report the first failure.
int finish(Pipeline* p, int status) {
    const int sync_status = sync_all(p);
    return status != FDL_OK ? status : sync_status;
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
    std::lock_guard<std::mutex> call(p->call_mutex);
    int slot = 0;
    int status = FDL_OK;
    for (int64_t off = 0; off < n && status == FDL_OK; off += kChunkElems, slot = (slot + 1) % kSlots) {
        const int64_t m = n - off < kChunkElems ? n - off : kChunkElems;
        cudaStream_t s = p->stream[slot];
        FDL_STEP(cudaMemcpyAsync(p->a[slot], h_a + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_STEP(cudaMemcpyAsync(p->b[slot], h_b + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_STEP(fdl_binary_f32(p->a[slot], p->b[slot], p->out[slot], m, op, s));
        FDL_STEP(cudaMemcpyAsync(h_out + off, p->out[slot], m * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    return finish(p, status);
}

int fdl_host_unary_f32(const float* h_x, float* h_out, int64_t n, int op, float alpha) {
    if (n < 0 || (n > 0 && (h_x == nullptr || h_out == nullptr))) return FDL_ERR_INVALID_ARGUMENT;
    Pipeline* p = nullptr;
    FDL_TRY(get_pipeline(&p));
    std::lock_guard<std::mutex> call(p->call_mutex);
    int slot = 0;
    int status = FDL_OK;
    for (int64_t off = 0; off < n && status == FDL_OK; off += kChunkElems, slot = (slot + 1) % kSlots) {
        const int64_t m = n - off < kChunkElems ? n - off : kChunkElems;
        cudaStream_t s = p->stream[slot];
        FDL_STEP(cudaMemcpyAsync(p->a[slot], h_x + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_STEP(fdl_unary_f32(p->a[slot], p->out[slot], m, op, alpha, s));
        FDL_STEP(cudaMemcpyAsync(h_out + off, p->out[slot], m * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    return finish(p, status);
}

int fdl_host_mul_add_relu_f32(const float* h_a, const float* h_b, const float* h_c, float* h_out,
                              int64_t n) {
    if (n < 0 || (n > 0 && (h_a == nullptr || h_b == nullptr || h_c == nullptr || h_out == nullptr))) {
        return FDL_ERR_INVALID_ARGUMENT;
    }
    Pipeline* p = nullptr;
    FDL_TRY(get_pipeline(&p));
    std::lock_guard<std::mutex> call(p->call_mutex);
    int slot = 0;
    int status = FDL_OK;
    for (int64_t off = 0; off < n && status == FDL_OK; off += kChunkElems, slot = (slot + 1) % kSlots) {
        const int64_t m = n - off < kChunkElems ? n - off : kChunkElems;
        cudaStream_t s = p->stream[slot];
        // The third operand lands in the output buffer and is overwritten in place.
        FDL_STEP(cudaMemcpyAsync(p->a[slot], h_a + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_STEP(cudaMemcpyAsync(p->b[slot], h_b + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_STEP(cudaMemcpyAsync(p->out[slot], h_c + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_STEP(fdl_mul_add_relu_f32(p->a[slot], p->b[slot], p->out[slot], p->out[slot], m, s));
        FDL_STEP(cudaMemcpyAsync(h_out + off, p->out[slot], m * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    return finish(p, status);
}

// Uploads the row vector on slot 0's stream and makes the other slots wait for it.
static int upload_row(Pipeline* p, const float* h_row, int64_t cols) {
    int status = ensure_capacity(p, &p->row, &p->row_capacity, cols);
    cudaEvent_t row_ready = nullptr;
    FDL_STEP(cudaEventCreateWithFlags(&row_ready, cudaEventDisableTiming));
    FDL_STEP(cudaMemcpyAsync(p->row, h_row, cols * sizeof(float), cudaMemcpyHostToDevice, p->stream[0]));
    FDL_STEP(cudaEventRecord(row_ready, p->stream[0]));
    for (int s = 1; s < kSlots; ++s) FDL_STEP(cudaStreamWaitEvent(p->stream[s], row_ready, 0));
    // Destroying an event that streams still wait on is allowed: its resources are released
    // once the waits have been satisfied.
    if (row_ready != nullptr) cudaEventDestroy(row_ready);
    return status;
}

int fdl_host_row_broadcast_f32(const float* h_a, const float* h_row, float* h_out, int64_t rows,
                               int64_t cols, int op) {
    if (rows < 0 || cols < 0) return FDL_ERR_INVALID_ARGUMENT;
    if (rows == 0 || cols == 0) return FDL_OK;
    if (h_a == nullptr || h_row == nullptr || h_out == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    if (cols > kChunkElems) return FDL_ERR_UNSUPPORTED;
    Pipeline* p = nullptr;
    FDL_TRY(get_pipeline(&p));
    std::lock_guard<std::mutex> call(p->call_mutex);
    int status = upload_row(p, h_row, cols);
    const int64_t rows_per_chunk = kChunkElems / cols;
    const int64_t a_strides[2] = {cols, 1};
    const int64_t b_strides[2] = {0, 1};
    int slot = 0;
    for (int64_t r = 0; r < rows && status == FDL_OK; r += rows_per_chunk, slot = (slot + 1) % kSlots) {
        const int64_t nr = rows - r < rows_per_chunk ? rows - r : rows_per_chunk;
        const int64_t m = nr * cols;
        cudaStream_t s = p->stream[slot];
        const int64_t shape[2] = {nr, cols};
        FDL_STEP(cudaMemcpyAsync(p->a[slot], h_a + r * cols, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_STEP(fdl_broadcast_binary_f32(p->a[slot], p->row, p->out[slot], 2, shape, a_strides, b_strides, op, s));
        FDL_STEP(cudaMemcpyAsync(h_out + r * cols, p->out[slot], m * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    return finish(p, status);
}

// Folds the chunk partials on the host in chunk order (deterministic).
static int fold_partials(Pipeline* p, int64_t nchunks, double* h_out) {
    double stack_buf[64];
    double* host_partials = nchunks <= 64 ? stack_buf : new double[nchunks];
    const cudaError_t e = cudaMemcpy(host_partials, p->partial, nchunks * sizeof(double), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) {
        double total = 0.0;
        for (int64_t k = 0; k < nchunks; ++k) total += host_partials[k];
        *h_out = total;
    }
    if (host_partials != stack_buf) delete[] host_partials;
    return static_cast<int>(e);
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
    std::lock_guard<std::mutex> call(p->call_mutex);
    const int64_t rows_per_chunk = kChunkElems / cols;
    const int64_t nchunks = ceil_div(rows, rows_per_chunk);
    int status = ensure_capacity(p, &p->partial, &p->partial_capacity, nchunks);
    FDL_STEP(upload_row(p, h_row, cols));
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
        FDL_STEP(cudaMemcpyAsync(p->a[slot], h_x + r * cols, bytes, cudaMemcpyHostToDevice, s));
        FDL_STEP(cudaMemcpyAsync(p->b[slot], h_y + r * cols, bytes, cudaMemcpyHostToDevice, s));
        FDL_STEP(fdl_binary_f32(p->a[slot], p->b[slot], p->out[slot], m, FDL_ADD, s));
        FDL_STEP(cudaMemcpyAsync(h_z + r * cols, p->out[slot], bytes, cudaMemcpyDeviceToHost, s));
        FDL_STEP(fdl_broadcast_binary_f32(p->a[slot], p->row, p->out2[slot], 2, shape, a_strides, b_strides, FDL_ADD, s));
        FDL_STEP(cudaMemcpyAsync(h_w + r * cols, p->out2[slot], bytes, cudaMemcpyDeviceToHost, s));
        FDL_STEP(fdl_sum_f32(p->a[slot], m, nullptr, p->partial + chunk, p->scratch[slot], scratch_bytes, s));
    }
    status = finish(p, status);
    if (status != FDL_OK) return status;
    return fold_partials(p, nchunks, h_sum);
}

int fdl_host_sum_f32(const float* h_x, int64_t n, double* h_out) {
    if (n < 0 || h_out == nullptr || (n > 0 && h_x == nullptr)) return FDL_ERR_INVALID_ARGUMENT;
    const int64_t nchunks = ceil_div(n, kChunkElems);
    if (nchunks == 0) {
        *h_out = 0.0;
        return FDL_OK;
    }
    Pipeline* p = nullptr;
    FDL_TRY(get_pipeline(&p));
    std::lock_guard<std::mutex> call(p->call_mutex);
    int status = ensure_capacity(p, &p->partial, &p->partial_capacity, nchunks);
    // Each slot reduces into its own scratch, so reductions of different chunks may overlap.
    const size_t scratch_bytes = fdl_sum_scratch_bytes(kChunkElems);
    int slot = 0;
    int64_t chunk = 0;
    for (int64_t off = 0; off < n && status == FDL_OK; off += kChunkElems, ++chunk, slot = (slot + 1) % kSlots) {
        const int64_t m = n - off < kChunkElems ? n - off : kChunkElems;
        cudaStream_t s = p->stream[slot];
        FDL_STEP(cudaMemcpyAsync(p->a[slot], h_x + off, m * sizeof(float), cudaMemcpyHostToDevice, s));
        FDL_STEP(fdl_sum_f32(p->a[slot], m, nullptr, p->partial + chunk, p->scratch[slot], scratch_bytes, s));
    }
    status = finish(p, status);
    if (status != FDL_OK) return status;
    return fold_partials(p, nchunks, h_out);
}

}  // extern "C"
