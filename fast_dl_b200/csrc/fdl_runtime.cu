// Runtime plumbing of the C ABI: device selection, error text, cached device
// properties and the library-owned per-device workspace.
#include <cstring>
#include <mutex>
#include <string>

#include "fdl_common.cuh"

namespace fdl {

namespace {

constexpr int kMaxDevices = 64;

std::mutex g_mutex;
DeviceInfo g_info[kMaxDevices];
bool g_info_valid[kMaxDevices] = {};

struct Workspace {
    void* ptr = nullptr;
    size_t bytes = 0;
};
Workspace g_workspace[kMaxDevices];

}  // namespace

namespace {
unsigned int* g_error_flag_host = nullptr;  // mapped pinned memory, one word per process
}

int error_flag_device_ptr(unsigned int** dev) {
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (g_error_flag_host == nullptr) {
            void* h = nullptr;
            cudaError_t e = cudaHostAlloc(&h, 256, cudaHostAllocMapped | cudaHostAllocPortable);
            if (e != cudaSuccess) return static_cast<int>(e);
            memset(h, 0, 256);
            g_error_flag_host = static_cast<unsigned int*>(h);
        }
    }
    void* d = nullptr;
    cudaError_t e = cudaHostGetDevicePointer(&d, g_error_flag_host, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    *dev = static_cast<unsigned int*>(d);
    return FDL_OK;
}

const unsigned long long* trace_words_host() {
    return g_error_flag_host == nullptr
               ? nullptr
               : reinterpret_cast<const unsigned long long*>(reinterpret_cast<const char*>(g_error_flag_host) + 64);
}

unsigned int read_and_clear_device_error_flag() {
    if (g_error_flag_host == nullptr) return 0;
    const unsigned int v = *reinterpret_cast<volatile unsigned int*>(g_error_flag_host);
    *reinterpret_cast<volatile unsigned int*>(g_error_flag_host) = 0;
    return v;
}

Tuning& tuning() {
    static Tuning t;
    return t;
}

const DeviceInfo* current_device_info(int* status) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        *status = static_cast<int>(e);
        return nullptr;
    }
    if (dev < 0 || dev >= kMaxDevices) {
        *status = FDL_ERR_NO_DEVICE;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_info_valid[dev]) {
        DeviceInfo info;
        info.device = dev;
        e = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) {
            e = cudaDeviceGetAttribute(&info.max_smem_optin,
                                       cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        }
        if (e != cudaSuccess) {
            *status = static_cast<int>(e);
            return nullptr;
        }
        g_info[dev] = info;
        g_info_valid[dev] = true;
    }
    *status = FDL_OK;
    return &g_info[dev];
}

int get_workspace(size_t bytes, void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return FDL_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lock(g_mutex);
    Workspace& ws = g_workspace[dev];
    if (ws.bytes < bytes) {
        // Growing is rare (sizes depend on the SM count, not on the tensor), and the old
        // block may still be in use by an enqueued kernel: wait for the device first.
        if (ws.ptr != nullptr) {
            e = cudaDeviceSynchronize();
            if (e != cudaSuccess) return static_cast<int>(e);
            cudaFree(ws.ptr);
            ws.ptr = nullptr;
            ws.bytes = 0;
        }
        size_t want = bytes < (size_t{1} << 20) ? (size_t{1} << 20) : bytes;
        e = cudaMalloc(&ws.ptr, want);
        if (e != cudaSuccess) return static_cast<int>(e);
        e = cudaMemset(ws.ptr, 0, want);
        if (e != cudaSuccess) return static_cast<int>(e);
        ws.bytes = want;
    }
    *out = ws.ptr;
    return FDL_OK;
}

// Zeroes the counter block of every device's workspace (the caller has synchronised).
void reset_workspace_counters() {
    int current = 0;
    if (cudaGetDevice(&current) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    for (int dev = 0; dev < kMaxDevices; ++dev) {
        Workspace& ws = g_workspace[dev];
        if (ws.ptr == nullptr || ws.bytes < static_cast<size_t>(kWorkspaceCounterBytes)) continue;
        if (cudaSetDevice(dev) != cudaSuccess || cudaMemset(ws.ptr, 0, kWorkspaceCounterBytes) != cudaSuccess) {
            cudaGetLastError();
        }
    }
    cudaSetDevice(current);
}

}  // namespace fdl

extern "C" {

int fdl_version(void) { return 1001; }

const char* fdl_error_string(int status) {
    switch (status) {
        case FDL_OK:
            return "success";
        case FDL_ERR_INVALID_ARGUMENT:
            return "fdl: invalid argument";
        case FDL_ERR_UNSUPPORTED:
            return "fdl: unsupported shape or configuration";
        case FDL_ERR_WORKSPACE:
            return "fdl: scratch buffer too small or misaligned";
        case FDL_ERR_DEVICE_WAIT:
            return "fdl: a bounded device-side wait ran out";
        case FDL_ERR_NO_DEVICE:
            return "fdl: no usable CUDA device";
        case FDL_ERR_TOO_LARGE_FOR_STATIC_SCRATCH:
            return "fdl: element count exceeds the 2^30 maximum of the static-scratch entry point";
        default:
            break;
    }
    if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
    return "fdl: unknown status";
}

int fdl_take_device_error(void) {
    if (fdl::read_and_clear_device_error_flag() == 0) return FDL_OK;
    // A kernel that gave up a wait may have left arrival counters half-way; the kernels that
    // share them expect zeros.
    fdl::reset_workspace_counters();
    return FDL_ERR_DEVICE_WAIT;
}

int fdl_set_tuning(const char* key, int value) {
    if (key == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    const std::string k(key);
    if (k == "sum_cluster" && (value == 1 || value == 2 || value == 4 || value == 8)) {
        fdl::tuning().sum_cluster = value;
        return FDL_OK;
    }
    if (k == "rows_span_argmax_from" && value >= 1) {
        fdl::tuning().rows_span_argmax_from = value;
        return FDL_OK;
    }
    if (k == "rows_split_from" && value >= 0) {
        fdl::tuning().rows_split_from = value;
        return FDL_OK;
    }
    if (k == "rows_split_lag" && value >= 0 && value <= 4096) {
        fdl::tuning().rows_split_lag = value;
        return FDL_OK;
    }
    if (k == "rows_split_hints" && (value == 0 || value == 1)) {
        fdl::tuning().rows_split_hints = value;
        return FDL_OK;
    }
    if (k == "rows_split_fused" && (value == 0 || value == 1)) {
        fdl::tuning().rows_split_fused = value;
        return FDL_OK;
    }
    if (k == "sum_tiles" && value >= 0 && value <= 64) {
        fdl::tuning().sum_tiles = value;
        return FDL_OK;
    }
    if (k == "cols_tx" && (value == 16 || value == 32 || value == 64 || value == 128 || value == 256)) {
        fdl::tuning().cols_tx = value;
        return FDL_OK;
    }
    if (k == "cols_cluster" && (value == 0 || value == 1 || value == 2 || value == 4 || value == 8 || value == 16)) {
        fdl::tuning().cols_cluster = value;
        return FDL_OK;
    }
    if (k == "rows_cluster_threads" && (value == 256 || value == 512)) {
        fdl::tuning().rows_cluster_threads = value;
        return FDL_OK;
    }
    if (k == "rows_warp16" && value >= -1 && value <= 1) {
        fdl::tuning().rows_warp16 = value;
        return FDL_OK;
    }
    if (k == "cols_chunks" && value >= 0 && value <= 65535) {
        fdl::tuning().cols_chunks = value;
        return FDL_OK;
    }
    if (k == "cols_regroup" && (value == 0 || value == 1)) {
        fdl::tuning().cols_regroup = value;
        return FDL_OK;
    }
    if (k == "cols_single" && (value == 0 || value == 1)) {
        fdl::tuning().cols_single = value;
        return FDL_OK;
    }
    if (k == "cols_ctas_per_sm" && value >= 1 && value <= 256) {
        fdl::tuning().cols_ctas_per_sm = value;
        return FDL_OK;
    }
    if (k == "rows_staged" && value >= -1 && value <= 1) {
        fdl::tuning().rows_staged = value;
        return FDL_OK;
    }
    if (k == "rows_smem_cluster" && (value == 0 || value == 2 || value == 4 || value == 8 || value == 16)) {
        fdl::tuning().rows_smem_cluster = value;
        return FDL_OK;
    }
    if (k == "rows_span_reduce_cols" && value >= 0 && value <= 2048) {
        fdl::tuning().rows_span_reduce_cols = value;
        return FDL_OK;
    }
    if (k == "rows_span_cols" && value >= 0 && value <= 256) {
        fdl::tuning().rows_span_cols = value;
        return FDL_OK;
    }
    if (k == "rows_smem_from" && value >= 0) {
        fdl::tuning().rows_smem_from = value;
        return FDL_OK;
    }
    if (k == "rows_smem" && (value == 0 || value == 1)) {
        fdl::tuning().rows_smem = value;
        return FDL_OK;
    }
    if (k == "pdl" && (value == 0 || value == 1)) {
        fdl::tuning().pdl = value;
        return FDL_OK;
    }
    if (k == "exchange_wait_ms" && value >= 1 && value <= 60000) {
        fdl::tuning().exchange_wait_ms = value;
        return FDL_OK;
    }
    if (k == "sum_trace" && (value == 0 || value == 1)) {
        fdl::tuning().sum_trace = value;
        return FDL_OK;
    }
    if (k == "bcast2d_rows" && (value == 0 || value == 1 || value == 2 || value == 4)) {
        fdl::tuning().bcast2d_rows = value;
        return FDL_OK;
    }
    if (k == "bcast2d" && (value == 0 || value == 1)) {
        fdl::tuning().bcast2d = value;
        return FDL_OK;
    }
    return FDL_ERR_INVALID_ARGUMENT;
}

int fdl_debug_sum_trace(unsigned long long* out8) {
    if (out8 == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    const unsigned long long* w = fdl::trace_words_host();
    for (int i = 0; i < fdl::kTraceWords; ++i) {
        out8[i] = w == nullptr ? 0ull : reinterpret_cast<const volatile unsigned long long*>(w)[i];
    }
    return FDL_OK;
}

int fdl_device_count(void) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return FDL_ERR_NO_DEVICE;
    }
    return n;
}

int fdl_set_device(int device) { return static_cast<int>(cudaSetDevice(device)); }

int fdl_stream_synchronize(void* stream) {
    return static_cast<int>(cudaStreamSynchronize(fdl::as_stream(stream)));
}

}  // extern "C"
