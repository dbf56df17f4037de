// Shared device/host helpers of the sm_100a kernel library.
//
// Everything on this path is HBM-bandwidth bound, so the helpers here are about moving
// bytes: 128-bit streaming loads/stores, warp/block reductions, launch sizing in whole
// multiples of the SM count, and bounded mbarrier waits for the bulk-async pipelines.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/fdl_kernels.h"

namespace fdl {

constexpr int kWarp = 32;
constexpr unsigned kFullMask = 0xffffffffu;

// ---- host side -----------------------------------------------------------------------

constexpr int kMaxDevicesTracked = 64;  // per-device bookkeeping arrays (device index modulo this)

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    int max_smem_optin = 0;
};

// Properties of the current device (cached per device index).  Returns nullptr and
// sets *status when the runtime cannot be queried.
const DeviceInfo* current_device_info(int* status);

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// Status of the launch that was just enqueued on this thread.
inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Launch-shape knobs that the bench can vary to show why the defaults were chosen
// (set through fdl_set_tuning).  Defaults are the measured best on B200.
struct Tuning {
    int sum_cluster = 4;   // CTAs per cluster in the full sum (1 = no cluster stage)
    int rows_span_argmax_from = 65;  // argmax along axis 1 of odd rows takes the span form from this many floats on
    int rows_split_from = 0;   // > 0: rows of at least this many floats take the split form whatever the other forms offer
    int rows_split_fused = 1;  // rows beyond a cluster's reach: 1 = one kernel, statistics and apply tasks pipelined through L2; 0 = two kernels
    int rows_split_lag = 0;    // rows between a row's statistics and its apply tasks in that kernel (0 = 36 MiB of rows)
    int rows_split_hints = 1;  // L2 eviction-priority hints on that kernel's loads
    int sum_tiles = 0;     // 32 KiB tiles a CTA of the full sum walks (0 = by size)
    int cols_tx = 64;            // column reduction: threads across columns per CTA (16..256)
    int cols_cluster = 0;        // column reduction: CTAs per cluster along the rows (1, 2, 4, 8, 16; 0 = 8 on the
                                 // 128-bit path, 2 on the 32-bit path)
    int cols_ctas_per_sm = 4;   // column reduction: CTAs aimed at per SM
    int cols_chunks = 0;         // column reduction: row chunks per column block (0 = derived)
    int cols_regroup = 1;        // column reduction: odd column counts walked as [rows / 4, 4 * cols] with 128-bit loads
    int cols_single = 1;         // column reduction: prefer one cluster of 8 per column block where it fits
    int rows_cluster_threads = 256;  // cluster form of rows up to 65536 floats: threads per CTA (256 or 512)
    int rows_warp16 = -1;        // row softmax/layernorm: rows of 1028..2048 floats by one warp, 16 packs a
                                 // lane (1), by a 256-thread CTA (0), or whichever measured faster (-1)
    int rows_staged = -1;  // row softmax/layernorm: 0 = direct loads, 1 = one bulk-async copy per CTA,
                           // -1 = staged for rows of up to 128 floats, direct beyond
    int rows_span_reduce_cols = 2048;  // row reductions: rows of up to this many floats at an odd length or
                                       // phase are staged as runs of rows through shared memory (0 = never)
    int rows_span_cols = 256;  // row softmax/layernorm: rows of up to this many floats at an odd length or phase
                               // are staged as runs of rows through shared memory (0 = never; at most 256)
    int rows_smem = 1;     // row softmax/layernorm: long rows in a cluster's shared memory, read once (0 = the
                           // register-cluster and two-kernel forms)
    int rows_smem_from = 0;     // aligned rows longer than this many floats take that form (0 = 65536)
    int rows_smem_cluster = 0;  // CTAs per row in that form: 2, 4, 8, 16 (0 = by row length)
    int pdl = 1;           // streaming kernels are launched with programmatic stream serialization: the
                           // next kernel's launch and ramp-up overlap this one's tail (0 = plain launches)
    int exchange_wait_ms = 2000;  // how long a cross-GPU exchange waits for its peers before giving up
    int sum_trace = 0;     // 1: the full sum's finishing CTA leaves %globaltimer stamps (fdl_debug_sum_trace)
    int bcast2d = 1;       // two-dimensional broadcasts take the division-free kernel (0 = the general one)
    int bcast2d_rows = 0;  // rows per thread in that kernel: 1, 2 or 4 (0 = by size)
};
Tuning& tuning();

// Per-device workspace the library owns (allocated on first use, grown on demand,
// never freed before process exit).  Used when a caller passes scratch == NULL.
int get_workspace(size_t bytes, void** out);
void reset_workspace_counters();  // zeroes the counter block of every device's workspace
// Every user of the workspace keeps its arrival counters in the first 64 KiB (zero between
// launches) and its partial results behind them.
constexpr int kWorkspaceCounterBytes = 65536;

// One word of host-mapped pinned memory per process in which kernels raise bits when a
// bounded device-side wait runs out (bit 0: bulk-copy wait, bit 1: cross-GPU exchange wait).
// The same 256-byte block carries, from byte 64 on, eight 64-bit time stamps that the full
// sum's finishing CTA writes when tuning().sum_trace is set.
int error_flag_device_ptr(unsigned int** dev);
unsigned int read_and_clear_device_error_flag();
constexpr int kTraceWords = 8;
const unsigned long long* trace_words_host();

// Launch with optional thread-block clusters along x (or y) and optional programmatic
// stream serialization.  With `pdl`, the kernel may be scheduled while the previous kernel
// of the stream is still draining; it must execute pdl_wait() before its first global
// access, which every kernel launched through here does.
template <class... KArgs, class... Args>
int launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
              dim3 cluster, bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    unsigned int n = 0;
    if (cluster.x * cluster.y * cluster.z > 1) {
        attrs[n].id = cudaLaunchAttributeClusterDimension;
        attrs[n].val.clusterDim.x = cluster.x;
        attrs[n].val.clusterDim.y = cluster.y;
        attrs[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    if (pdl) {
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return static_cast<int>(e);
    return static_cast<int>(cudaGetLastError());
}

// Persistent-grid size: enough blocks to fill every SM `blocks_per_sm` times, but never
// more than the work needs.
inline int persistent_grid(const DeviceInfo* info, int blocks_per_sm, int64_t work_blocks) {
    int64_t cap = static_cast<int64_t>(info->sm_count) * blocks_per_sm;
    int64_t g = work_blocks < cap ? work_blocks : cap;
    return g < 1 ? 1 : static_cast<int>(g);
}

// ---- device side -----------------------------------------------------------------------

#ifdef __CUDACC__

// Programmatic dependent launch.  pdl_wait(): returns once the previous kernel of the stream
// has completed and its writes are visible (a no-op for a kernel launched the plain way).
// pdl_trigger(): this CTA no longer delays the launch of the next kernel; that kernel's
// own pdl_wait() still waits for the whole of this grid.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Streaming (evict-first) 128-bit accesses: every byte on this path is touched once.
__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ float ld_stream(const float* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(float* p, float v) { __stcs(p, v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = kWarp / 2; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
    return v;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = kWarp / 2; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = kWarp / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
    return v;
}

// ---- mbarrier + 1-D bulk-async copy (TMA engine, non-multicast form only) ----------------

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals)
                 : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders generic-proxy smem accesses before later async-proxy (bulk copy) accesses.
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

__device__ __forceinline__ unsigned long long timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: gives up after kMbarSpinLimit polls so a lost copy can never hang the
// GPU.  Returns false on timeout; the caller records an error flag and leaves.
constexpr uint32_t kMbarSpinLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kMbarSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// global -> shared::cta bulk copy of `bytes` (multiple of 16; both addresses 16-B
// aligned), completion counted on `bar`.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_addr(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}

#endif  // __CUDACC__

}  // namespace fdl
