// Row softmax and row layernorm (fp32), one HBM read and one HBM write per element.
//
// Rows are staged into shared memory by the bulk-async copy engine (1-D cp.async.bulk
// completing on an mbarrier; the non-multicast form, so the same code runs on any number
// of GPUs).  Each "team" -- one warp for rows up to 2048 floats, one whole CTA for rows up
// to 16384 floats -- owns a private ring of stages and its own barriers, so in the warp
// configuration no block-wide barrier is ever executed: a lane-0 thread re-arms a stage as
// soon as the team has pulled its rows into registers, and the copy engine keeps
// streaming while the team does its exp / normalise arithmetic and 128-bit stores.
// A stage holds several consecutive rows when rows are short, so one bulk copy is always
// a few KiB.  Rows that are unaligned, not a multiple of 4 floats, or longer than 16384
// floats take a plain three-pass kernel (second and third pass hit L2).
//
// Every mbarrier wait is bounded; when one runs out the team raises a flag in
// host-visible memory, drains its other stages with bounded waits and leaves.
#include <climits>
#include <cmath>
#include <type_traits>

#include "fdl_common.cuh"

namespace fdl {

namespace {

constexpr int kRwThreads = 256;
constexpr int kRwWarps = kRwThreads / kWarp;
constexpr int kRwStages = 3;

struct SoftmaxOp {};
struct LayerNormOp {};

struct RowParams {
    const float* x;
    float* y;
    const float* gamma;  // layernorm only, may be null
    const float* beta;   // layernorm only, may be null
    float* mean_out;     // layernorm only, may be null
    float* rstd_out;     // layernorm only, may be null
    int64_t rows;
    int cols;
    int rows_per_stage;
    float eps;
    unsigned int* error_flag;  // host-mapped
};

// ---- team-wide reductions ---------------------------------------------------------------

template <int TPR>
__device__ __forceinline__ float team_max(float v, float* red) {
    v = warp_max(v);
    if (TPR == kWarp) return v;
    const int lane = threadIdx.x & (kWarp - 1);
    const int warp = threadIdx.x / kWarp;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int k = 1; k < kRwWarps; ++k) r = fmaxf(r, red[k]);
    __syncthreads();
    return r;
}

template <int TPR>
__device__ __forceinline__ float team_sum(float v, float* red) {
    v = warp_sum(v);
    if (TPR == kWarp) return v;
    const int lane = threadIdx.x & (kWarp - 1);
    const int warp = threadIdx.x / kWarp;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int k = 1; k < kRwWarps; ++k) r += red[k];
    __syncthreads();
    return r;
}

template <int TPR>
__device__ __forceinline__ void team_sync() {
    if (TPR == kWarp) __syncwarp();
    else __syncthreads();
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- per-row arithmetic on a register-resident row -----------------------------------------

template <int TPR, int NV>
__device__ __forceinline__ void row_math(SoftmaxOp, float4 (&v)[NV], int t, int nvec,
                                         const RowParams& p, int64_t row, float* red) {
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < nvec) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    }
    m = team_max<TPR>(m, red);
    // exp(x - m) as 2^((x - m) * log2(e)): the subtraction is the reference's own (exact
    // for the terms that matter, by Sterbenz), then one multiply and one ex2.approx
    // (relative error ~2^-22) instead of the ~9-instruction expf.
    constexpr float kLog2e = 1.4426950408889634f;
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < nvec) {
            v[i].x = fast_exp2((v[i].x - m) * kLog2e);
            v[i].y = fast_exp2((v[i].y - m) * kLog2e);
            v[i].z = fast_exp2((v[i].z - m) * kLog2e);
            v[i].w = fast_exp2((v[i].w - m) * kLog2e);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    }
    s = team_sum<TPR>(s, red);
    const float norm = 1.0f / s;
    float4* yr = reinterpret_cast<float4*>(p.y + row * p.cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < nvec) {
            st_stream(yr + t + i * TPR,
                      make_float4(v[i].x * norm, v[i].y * norm, v[i].z * norm, v[i].w * norm));
        }
    }
}

template <int TPR, int NV>
__device__ __forceinline__ void row_math(LayerNormOp, float4 (&v)[NV], int t, int nvec,
                                         const RowParams& p, int64_t row, float* red) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < nvec) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float inv_n = 1.0f / static_cast<float>(p.cols);
    const float mean = team_sum<TPR>(s, red) * inv_n;
    // Second moment about the mean from the registers: no E[x^2] - E[x]^2 cancellation.
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < nvec) {
            const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean,
                        dw = v[i].w - mean;
            q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
    }
    const float var = team_sum<TPR>(q, red) * inv_n;
    const float rstd = 1.0f / sqrtf(var + p.eps);
    if (t == 0) {
        if (p.mean_out != nullptr) p.mean_out[row] = mean;
        if (p.rstd_out != nullptr) p.rstd_out[row] = rstd;
    }
    float4* yr = reinterpret_cast<float4*>(p.y + row * p.cols);
    const float4* g4 = reinterpret_cast<const float4*>(p.gamma);
    const float4* b4 = reinterpret_cast<const float4*>(p.beta);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = t + i * TPR;
        if (c < nvec) {
            float4 o = make_float4((v[i].x - mean) * rstd, (v[i].y - mean) * rstd,
                                   (v[i].z - mean) * rstd, (v[i].w - mean) * rstd);
            if (g4 != nullptr) {
                const float4 g = __ldg(g4 + c);
                o.x *= g.x; o.y *= g.y; o.z *= g.z; o.w *= g.w;
            }
            if (b4 != nullptr) {
                const float4 b = __ldg(b4 + c);
                o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
            }
            st_stream(yr + c, o);
        }
    }
}

// ---- the staged kernel ---------------------------------------------------------------------
//
// Shared memory: [team][stage] row buffers (stage_bytes each, 128-byte aligned), then
// [team][stage] mbarriers.  Tile number `tile` covers rows
// [tile*rows_per_stage, (tile+1)*rows_per_stage) and is one contiguous span of the input.

template <class Op, int TPR, int NV>
__global__ void __launch_bounds__(kRwThreads)
rows_staged_kernel(const RowParams p, int stage_bytes) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ float red[kRwWarps];
    constexpr int kTeams = kRwThreads / TPR;
    const int team = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    unsigned char* my_stages = smem + static_cast<size_t>(team) * kRwStages * stage_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kTeams) * kRwStages * stage_bytes) +
                     team * kRwStages;

    if (t == 0) {
#pragma unroll
        for (int s = 0; s < kRwStages; ++s) mbar_init(bars + s, 1);
        fence_mbar_init();
    }
    __syncthreads();

    const int64_t ntiles = (p.rows + p.rows_per_stage - 1) / p.rows_per_stage;
    const int64_t team_id = static_cast<int64_t>(blockIdx.x) * kTeams + team;
    const int64_t team_stride = static_cast<int64_t>(gridDim.x) * kTeams;
    const int nvec = p.cols / 4;
    const size_t row_bytes = static_cast<size_t>(p.cols) * sizeof(float);

    auto issue = [&](int64_t tile, int stage) {
        const int64_t r0 = tile * p.rows_per_stage;
        int64_t nr = p.rows - r0;
        if (nr > p.rows_per_stage) nr = p.rows_per_stage;
        const uint32_t bytes = static_cast<uint32_t>(nr * row_bytes);
        mbar_expect_tx(bars + stage, bytes);
        bulk_g2s(my_stages + static_cast<size_t>(stage) * stage_bytes, p.x + r0 * p.cols, bytes,
                 bars + stage);
    };

    // Prologue: fill the ring.
    if (t == 0) {
#pragma unroll
        for (int s = 0; s < kRwStages; ++s) {
            const int64_t tile = team_id + s * team_stride;
            if (tile < ntiles) issue(tile, s);
        }
    }

    int stage = 0;
    uint32_t parity = 0;
    bool ok = true;
    int64_t tile = team_id;
    for (; tile < ntiles; tile += team_stride) {
        // The verdict is made uniform across the team so that nobody is left alone at a
        // later team barrier.
        bool landed = mbar_wait_bounded(bars + stage, parity);
        if (TPR == kWarp) landed = __all_sync(kFullMask, landed);
        else landed = __syncthreads_and(landed);
        if (!landed) {
            ok = false;
            break;
        }
        const int64_t r0 = tile * p.rows_per_stage;
        int nr = p.rows - r0 < p.rows_per_stage ? static_cast<int>(p.rows - r0) : p.rows_per_stage;
        const float4* src = reinterpret_cast<const float4*>(my_stages + static_cast<size_t>(stage) * stage_bytes);
        for (int r = 0; r < nr; ++r) {
            float4 v[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (t + i * TPR < nvec) v[i] = src[r * nvec + t + i * TPR];
            }
            if (r == nr - 1) {
                // The stage is now entirely in registers: hand it back to the copy engine.
                team_sync<TPR>();
                const int64_t next = tile + kRwStages * team_stride;
                if (t == 0 && next < ntiles) issue(next, stage);
            }
            row_math<TPR, NV>(Op{}, v, t, nvec, p, r0 + r, red);
        }
        if (++stage == kRwStages) {
            stage = 0;
            parity ^= 1u;
        }
    }

    if (!ok) {
        if (t == 0) atomicOr(p.error_flag, 1u);
        // Give copies that may still be in flight a bounded chance to land before the
        // shared memory is released.
        for (int k = 0; k < kRwStages; ++k) {
            if (tile + k * team_stride < ntiles) mbar_wait_bounded(bars + stage, parity);
            if (++stage == kRwStages) {
                stage = 0;
                parity ^= 1u;
            }
        }
    }
}

// ---- one-shot staged kernel: one bulk copy per CTA, no ring -----------------------------------
//
// A CTA owns one contiguous span of the input: kRwWarps * rows_per_stage rows when a warp
// works on a row (TPR = 32), one row when the whole CTA does (TPR = 256).  Thread 0 issues
// ONE bulk copy for the span, everybody waits on the same mbarrier and then works from
// shared memory.  There is no pipeline inside the CTA: overlap comes from the several
// CTAs resident per SM, and load balance from the block scheduler.

// Registers per thread are capped so that several CTAs stay resident per SM: the bytes
// in flight per SM are (resident CTAs) x (CTA span), and the row arithmetic is light.
constexpr int min_ctas_for(int nv) { return nv <= 4 ? 6 : (nv <= 8 ? 4 : 2); }

template <class Op, int TPR, int NV>
__global__ void __launch_bounds__(kRwThreads, min_ctas_for(NV))
rows_oneshot_kernel(const RowParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t bar;
    __shared__ float red[kRwWarps];
    constexpr int kTeams = kRwThreads / TPR;
    const int team = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int rows_per_cta = kTeams * p.rows_per_stage;
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
    int64_t nr = p.rows - r0;
    if (nr > rows_per_cta) nr = rows_per_cta;
    const int nvec = p.cols / 4;
    const size_t row_bytes = static_cast<size_t>(p.cols) * sizeof(float);

    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
        const uint32_t bytes = static_cast<uint32_t>(nr * row_bytes);
        mbar_expect_tx(&bar, bytes);
        bulk_g2s(smem, p.x + r0 * p.cols, bytes, &bar);
    }
    __syncthreads();  // the barrier is initialised before anyone polls it
    bool landed = mbar_wait_bounded(&bar, 0);
    landed = __syncthreads_and(landed);
    if (!landed) {
        if (threadIdx.x == 0) atomicOr(p.error_flag, 1u);
        return;
    }
    const float4* src = reinterpret_cast<const float4*>(smem);
    for (int r = team; r < nr; r += kTeams) {
        float4 v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (t + i * TPR < nvec) v[i] = src[r * nvec + t + i * TPR];
        }
        row_math<TPR, NV>(Op{}, v, t, nvec, p, r0 + r, red);
    }
}

// ---- direct kernel: registers straight from global memory --------------------------------------
//
// A team (warp or CTA) per row, all of a row's 128-bit loads issued at once.

template <class Op, int TPR, int NV>
__global__ void __launch_bounds__(kRwThreads, min_ctas_for(NV))
rows_direct_kernel(const RowParams p) {
    __shared__ float red[kRwWarps];
    constexpr int kTeams = kRwThreads / TPR;
    const int team = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kTeams + team;
    if (row >= p.rows) return;  // whole teams leave together; a CTA-wide team is the whole CTA
    const int nvec = p.cols / 4;
    const float4* src = reinterpret_cast<const float4*>(p.x + row * p.cols);
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < nvec) v[i] = ld_stream(src + t + i * TPR);
    }
    row_math<TPR, NV>(Op{}, v, t, nvec, p, row, red);
}

// ---- plain fallback: one CTA per row, three passes ---------------------------------------

template <class Op>
__global__ void __launch_bounds__(kRwThreads) rows_plain_kernel(const RowParams p) {
    __shared__ float red[kRwWarps];
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const float* xr = p.x + row * p.cols;
        float* yr = p.y + row * p.cols;
        if (kSoftmax) {
            float m = -INFINITY;
            for (int c = threadIdx.x; c < p.cols; c += kRwThreads) m = fmaxf(m, xr[c]);
            m = team_max<kRwThreads>(m, red);
            float s = 0.0f;
            for (int c = threadIdx.x; c < p.cols; c += kRwThreads) s += fast_exp2((xr[c] - m) * 1.4426950408889634f);
            s = team_sum<kRwThreads>(s, red);
            const float norm = 1.0f / s;
            for (int c = threadIdx.x; c < p.cols; c += kRwThreads) yr[c] = fast_exp2((xr[c] - m) * 1.4426950408889634f) * norm;
        } else {
            float s = 0.0f;
            for (int c = threadIdx.x; c < p.cols; c += kRwThreads) s += xr[c];
            const float inv_n = 1.0f / static_cast<float>(p.cols);
            const float mean = team_sum<kRwThreads>(s, red) * inv_n;
            float q = 0.0f;
            for (int c = threadIdx.x; c < p.cols; c += kRwThreads) {
                const float d = xr[c] - mean;
                q += d * d;
            }
            const float var = team_sum<kRwThreads>(q, red) * inv_n;
            const float rstd = 1.0f / sqrtf(var + p.eps);
            if (threadIdx.x == 0) {
                if (p.mean_out != nullptr) p.mean_out[row] = mean;
                if (p.rstd_out != nullptr) p.rstd_out[row] = rstd;
            }
            for (int c = threadIdx.x; c < p.cols; c += kRwThreads) {
                float o = (xr[c] - mean) * rstd;
                if (p.gamma != nullptr) o *= p.gamma[c];
                if (p.beta != nullptr) o += p.beta[c];
                yr[c] = o;
            }
        }
    }
}

// ---- host side -------------------------------------------------------------------------------

unsigned int* g_error_flag_host = nullptr;  // mapped pinned memory, one word per process

int error_flag_device_ptr(unsigned int** dev) {
    if (g_error_flag_host == nullptr) {
        void* h = nullptr;
        cudaError_t e = cudaHostAlloc(&h, 256, cudaHostAllocMapped | cudaHostAllocPortable);
        if (e != cudaSuccess) return static_cast<int>(e);
        g_error_flag_host = static_cast<unsigned int*>(h);
        *g_error_flag_host = 0;
    }
    void* d = nullptr;
    cudaError_t e = cudaHostGetDevicePointer(&d, g_error_flag_host, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    *dev = static_cast<unsigned int*>(d);
    return FDL_OK;
}

template <class Op, int TPR, int NV>
int launch_staged_cfg(const RowParams& p, const DeviceInfo* info, cudaStream_t stream) {
    constexpr int kTeams = kRwThreads / TPR;
    RowParams q = p;
    const size_t row_bytes = static_cast<size_t>(p.cols) * sizeof(float);
    // Short rows share a stage so that one bulk copy moves about 4 KiB.
    int rps = 1;
    if (TPR == kWarp && row_bytes < 4096) rps = static_cast<int>(4096 / row_bytes);
    if (rps > 64) rps = 64;
    q.rows_per_stage = rps;
    size_t stage_bytes = rps * row_bytes;
    stage_bytes = (stage_bytes + 127) / 128 * 128;
    const size_t smem = kTeams * kRwStages * (stage_bytes + sizeof(uint64_t));
    if (smem + 1024 > static_cast<size_t>(info->max_smem_optin)) return FDL_ERR_UNSUPPORTED;

    auto kernel = rows_staged_kernel<Op, TPR, NV>;
    static size_t configured_smem = 0;
    if (smem > configured_smem) {
        // Exactly what is needed: the opt-in ceiling covers static + dynamic together.
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) return static_cast<int>(e);
        configured_smem = smem;
    }
    int blocks_per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, kernel,
                                                                  kRwThreads, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (blocks_per_sm < 1) return FDL_ERR_UNSUPPORTED;
    const int64_t ntiles = ceil_div(p.rows, rps);
    const int grid = persistent_grid(info, blocks_per_sm, ceil_div(ntiles, kTeams));
    kernel<<<grid, kRwThreads, smem, stream>>>(q, static_cast<int>(stage_bytes));
    return launch_status();
}

template <class Op, int TPR, int NV>
int launch_oneshot_cfg(const RowParams& p, const DeviceInfo* info, cudaStream_t stream) {
    constexpr int kTeams = kRwThreads / TPR;
    RowParams q = p;
    const size_t row_bytes = static_cast<size_t>(p.cols) * sizeof(float);
    int rps = 1;
    if (TPR == kWarp && row_bytes < 4096) rps = static_cast<int>(4096 / row_bytes);
    if (rps > 64) rps = 64;
    q.rows_per_stage = rps;
    const size_t smem = static_cast<size_t>(kTeams) * rps * row_bytes;
    if (smem + 1024 > static_cast<size_t>(info->max_smem_optin)) return FDL_ERR_UNSUPPORTED;
    auto kernel = rows_oneshot_kernel<Op, TPR, NV>;
    static size_t configured_smem = 48 * 1024 - 256;
    if (smem > configured_smem) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) return static_cast<int>(e);
        configured_smem = smem;
    }
    int64_t grid = ceil_div(p.rows, static_cast<int64_t>(kTeams) * rps);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    kernel<<<static_cast<unsigned int>(grid), kRwThreads, smem, stream>>>(q);
    return launch_status();
}

template <class Op, int TPR, int NV>
int launch_direct_cfg(const RowParams& p, cudaStream_t stream) {
    constexpr int kTeams = kRwThreads / TPR;
    int64_t grid = ceil_div(p.rows, kTeams);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    rows_direct_kernel<Op, TPR, NV><<<static_cast<unsigned int>(grid), kRwThreads, 0, stream>>>(p);
    return launch_status();
}

// Picks the team size and registers-per-thread bucket for a row length.
#define FDL_ROW_DISPATCH(LAUNCH, ...)                                                   \
    do {                                                                                \
        const int nvec_ = p.cols / 4;                                                   \
        if (nvec_ <= 32 * 1) return LAUNCH<Op, kWarp, 1>(__VA_ARGS__);                  \
        if (nvec_ <= 32 * 2) return LAUNCH<Op, kWarp, 2>(__VA_ARGS__);                  \
        if (nvec_ <= 32 * 4) return LAUNCH<Op, kWarp, 4>(__VA_ARGS__);                  \
        if (nvec_ <= 32 * 8) return LAUNCH<Op, kWarp, 8>(__VA_ARGS__);                  \
        if (nvec_ <= 32 * 16) return LAUNCH<Op, kWarp, 16>(__VA_ARGS__);                \
        if (nvec_ <= kRwThreads * 4) return LAUNCH<Op, kRwThreads, 4>(__VA_ARGS__);     \
        if (nvec_ <= kRwThreads * 8) return LAUNCH<Op, kRwThreads, 8>(__VA_ARGS__);     \
        return LAUNCH<Op, kRwThreads, 16>(__VA_ARGS__);                                 \
    } while (0)

template <class Op>
int launch_rows_op(RowParams p, cudaStream_t stream) {
    if (p.rows < 0 || p.cols < 0) return FDL_ERR_INVALID_ARGUMENT;
    if (p.rows == 0 || p.cols == 0) return FDL_OK;
    if (p.x == nullptr || p.y == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    int status = FDL_OK;
    const DeviceInfo* info = current_device_info(&status);
    if (info == nullptr) return status;
    status = error_flag_device_ptr(&p.error_flag);
    if (status != FDL_OK) return status;

    const bool staged = p.cols % 4 == 0 && p.cols <= 16384 && aligned16(p.x) && aligned16(p.y) &&
                        (p.gamma == nullptr || aligned16(p.gamma)) &&
                        (p.beta == nullptr || aligned16(p.beta));
    if (staged) {
        switch (tuning().rows_staged) {
            case 1:
                FDL_ROW_DISPATCH(launch_staged_cfg, p, info, stream);
            case 2:
                FDL_ROW_DISPATCH(launch_oneshot_cfg, p, info, stream);
            default:
                FDL_ROW_DISPATCH(launch_direct_cfg, p, stream);
        }
    }
    const int grid = persistent_grid(info, 8, p.rows);
    rows_plain_kernel<Op><<<grid, kRwThreads, 0, stream>>>(p);
    return launch_status();
}

}  // namespace

unsigned int read_and_clear_device_error_flag() {
    if (g_error_flag_host == nullptr) return 0;
    const unsigned int v = *reinterpret_cast<volatile unsigned int*>(g_error_flag_host);
    *reinterpret_cast<volatile unsigned int*>(g_error_flag_host) = 0;
    return v;
}

}  // namespace fdl

using namespace fdl;

extern "C" {

int fdl_softmax_rows_f32(const float* x, float* y, int64_t rows, int64_t cols, void* stream) {
    if (cols >= INT_MAX) return FDL_ERR_UNSUPPORTED;
    RowParams p{};
    p.x = x;
    p.y = y;
    p.rows = rows;
    p.cols = static_cast<int>(cols);
    return launch_rows_op<SoftmaxOp>(p, as_stream(stream));
}

int fdl_layernorm_rows_f32(const float* x, const float* gamma, const float* beta, float* y,
                           float* mean_out, float* rstd_out, int64_t rows, int64_t cols,
                           float eps, void* stream) {
    if (cols >= INT_MAX) return FDL_ERR_UNSUPPORTED;
    RowParams p{};
    p.x = x;
    p.y = y;
    p.gamma = gamma;
    p.beta = beta;
    p.mean_out = mean_out;
    p.rstd_out = rstd_out;
    p.rows = rows;
    p.cols = static_cast<int>(cols);
    p.eps = eps;
    return launch_rows_op<LayerNormOp>(p, as_stream(stream));
}

int fdl_take_device_error(void) {
    return read_and_clear_device_error_flag() != 0 ? FDL_ERR_DEVICE_WAIT : FDL_OK;
}

}  // extern "C"
