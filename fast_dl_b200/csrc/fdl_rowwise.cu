// Row softmax and row layernorm (fp32), one HBM read and one HBM write per element.
//
// A "team" of TPR threads owns a row and keeps it in registers (NV 128-bit packs per
// thread): 8 or 16 lanes for very short rows, a warp up to 1024 floats (up to 2048 where that
// measured faster), a whole CTA of 256 threads up to 8192 floats and of 512 threads up to
// 16384 floats.  Every CTA handles one
// fixed group of rows and the hardware block scheduler spreads the CTAs over the SMs.
//
// Two ways of bringing a row in are built, selected by fdl_set_tuning("rows_staged", v):
//   v = -1 (default) staged for rows of up to 128 floats, direct for longer ones;
//   v = 0            direct: each thread issues all its 128-bit global loads at once;
//   v = 1            staged: thread 0 issues ONE bulk-async copy (cp.async.bulk on an
//                    mbarrier, non-multicast) for the CTA's whole span of rows into shared
//                    memory, and the teams read their rows from there.
// On B200 the direct form measures 104-107% of the copy-bandwidth yardstick across row
// lengths 256..16384, the staged form 92-101%, and a persistent per-team ring of bulk
// copies (removed) 81-90%: with this little arithmetic per byte, enough resident warps
// already keep the memory system full, and the staged form pays an extra trip through
// shared memory plus a CTA-wide wait.  Rows of up to 128 floats are the exception: there a
// thread of the direct form has one load in flight and measures 76-90%, the staged form
// 97-98%, so the default picks by row length.  Both forms stay selectable so the
// comparison can be repeated on the same build.
//
// Rows of 16384 < cols <= 131072 floats are shared by a thread-block cluster of 4 or 8
// CTAs: each keeps a slice in registers and the slice statistics cross the cluster once
// through distributed shared memory, so such a row is still read once and written once.
// Longer rows are cut into 32 KiB segments: one kernel leaves per-segment statistics and
// combines them per row, a second applies them (two reads, one write).
// Rows whose length is not a multiple of 4 floats, or whose base is not 16-byte aligned (x and y
// at the same phase), are read once too:
//   up to 256 floats    the span form: a CTA takes a run of consecutive rows -- one contiguous run of
//                       memory whatever the row length --, one bulk-async copy brings in the aligned
//                       packs that cover it, teams walk their rows float by float in shared memory;
//   up to 16384 floats  the masked form: 128-bit accesses laid over the flat buffer, the row in
//                       registers, edge packs lane by lane (buckets of nine packs a thread just above
//                       the powers of two, where a row at an odd phase covers one pack more);
//   up to 131072 floats the shared-memory cluster form: a cluster of 2, 4 or 8 CTAs keeps the row in
//                       shared memory (slices of up to 64 KiB, bulk-async copies), one exchange of
//                       slice statistics through distributed shared memory.
// What is left (longer such rows: the two-kernel form; x and y at different phases: a plain
// three-pass kernel whose second and third pass hit L2 while a row fits there).
//
// Every mbarrier wait is bounded; if one runs out the CTA raises a flag in host-visible
// memory (fdl_take_device_error) and stores nothing (in a cluster it still walks through the
// cluster barriers, where its peers wait).
#include <climits>
#include <cmath>
#include <type_traits>

#include <cooperative_groups.h>

#include "fdl_common.cuh"

namespace fdl {

namespace cg = cooperative_groups;

namespace {

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
    int rows_per_team;  // staged form: consecutive rows each team takes from the CTA span
    float eps;
    unsigned int* error_flag;  // host-mapped
};

constexpr int kMaxWarps = 16;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- team-wide reductions: TPR <= 32 stays inside a warp, larger teams are the whole CTA ------

template <int TPR, int TH>
__device__ __forceinline__ float team_max(float v, float* red) {
    constexpr int kLanes = TPR < kWarp ? TPR : kWarp;
#pragma unroll
    for (int o = kLanes / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
    if (TPR <= kWarp) return v;
    const int lane = threadIdx.x & (kWarp - 1);
    const int warp = threadIdx.x / kWarp;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int k = 1; k < TH / kWarp; ++k) r = fmaxf(r, red[k]);
    __syncthreads();
    return r;
}

template <int TPR, int TH>
__device__ __forceinline__ float team_sum(float v, float* red) {
    constexpr int kLanes = TPR < kWarp ? TPR : kWarp;
#pragma unroll
    for (int o = kLanes / 2; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
    if (TPR <= kWarp) return v;
    const int lane = threadIdx.x & (kWarp - 1);
    const int warp = threadIdx.x / kWarp;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int k = 1; k < TH / kWarp; ++k) r += red[k];
    __syncthreads();
    return r;
}

// Where a row's statistics are folded: inside a team of one CTA.
template <int TPR, int TH>
struct TeamScope {
    float* red;
    __device__ __forceinline__ float max(float v) { return team_max<TPR, TH>(v, red); }
    __device__ __forceinline__ float sum(float v) { return team_sum<TPR, TH>(v, red); }
};

// ---- per-row arithmetic on a register-resident row -----------------------------------------
//
// `active` is false for the lanes of a team that has no row (past the end); they run the
// same shuffles on neutral values and store nothing.

template <int TPR, int TH, int NV, class Scope>
__device__ __forceinline__ void row_math(SoftmaxOp, float4 (&v)[NV], int t, int nvec,
                                         const RowParams& p, int64_t row, bool active, Scope& scope,
                                         int voff = 0) {
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < nvec) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    }
    m = scope.max(m);
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
    s = scope.sum(s);
    if (!active) return;
    const float norm = 1.0f / s;
    float4* yr = reinterpret_cast<float4*>(p.y + row * p.cols) + voff;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < nvec) {
            st_stream(yr + t + i * TPR,
                      make_float4(v[i].x * norm, v[i].y * norm, v[i].z * norm, v[i].w * norm));
        }
    }
}

template <int TPR, int TH, int NV, class Scope>
__device__ __forceinline__ void row_math(LayerNormOp, float4 (&v)[NV], int t, int nvec,
                                         const RowParams& p, int64_t row, bool active, Scope& scope,
                                         int voff = 0) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < nvec) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float inv_n = 1.0f / static_cast<float>(p.cols);
    const float mean = scope.sum(s) * inv_n;
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
    const float var = scope.sum(q) * inv_n;
    if (!active) return;
    const float rstd = 1.0f / sqrtf(var + p.eps);
    if (t == 0 && voff == 0) {
        if (p.mean_out != nullptr) p.mean_out[row] = mean;
        if (p.rstd_out != nullptr) p.rstd_out[row] = rstd;
    }
    float4* yr = reinterpret_cast<float4*>(p.y + row * p.cols) + voff;
    const float4* g4 = p.gamma == nullptr ? nullptr : reinterpret_cast<const float4*>(p.gamma) + voff;
    const float4* b4 = p.beta == nullptr ? nullptr : reinterpret_cast<const float4*>(p.beta) + voff;
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

// Registers per thread are capped so that several CTAs stay resident per SM: the bytes in
// flight per SM are (resident CTAs) x (bytes a CTA requests), and the arithmetic is light.
constexpr int min_ctas_for(int th, int nv) {
    return th > 256 ? (nv <= 4 ? 3 : 2) : (nv <= 4 ? 6 : (nv <= 9 ? 4 : 2));
}

// ---- direct form ----------------------------------------------------------------------------------

template <class Op, int TPR, int TH, int NV>
__global__ void __launch_bounds__(TH, min_ctas_for(TH, NV))
rows_direct_kernel(const RowParams p) {
    __shared__ float red[kMaxWarps];
    constexpr int kTeams = TH / TPR;
    const int team = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kTeams + team;
    const bool active = row < p.rows;
    if (TPR >= kWarp && !active) return;  // whole warps / the whole CTA leave together
    const int nvec = p.cols / 4;
    const float4* src = reinterpret_cast<const float4*>(p.x + (active ? row : 0) * p.cols);
    float4 v[NV];
    pdl_wait();  // the input may be the previous kernel's output
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < nvec) {
            v[i] = active ? ld_stream(src + t + i * TPR) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    pdl_trigger();  // the row is on its way: the next kernel of the stream may be scheduled
    TeamScope<TPR, TH> scope{red};
    row_math<TPR, TH, NV>(Op{}, v, t, nvec, p, row, active, scope);
}

// ---- masked form: rows whose length is not a multiple of 4 floats (or whose base is not 16-byte
// aligned) ----------------------------------------------------------------------------------------
//
// Such rows start at any of the four phases of a 16-byte line, so the 128-bit loads are laid over
// the FLAT buffer instead: a row is covered by the aligned packs [first_pack, first_pack + npk) of
// the buffer, of which the first and the last may belong to the row only in part.  Interior
// packs are loaded and stored as 128 bits exactly like in the direct form; the (at most two)
// edge packs of a row are loaded and stored one valid float at a time -- they share their
// 16 bytes with a neighbouring row that another team writes -- and their foreign lanes hold
// values that cannot change the statistics (-inf for softmax; 0, then the row mean, for
// layernorm).  x and y must sit at the same phase (their addresses agree modulo 16).

struct RowEdges {
    int head;  // floats of the first pack that precede the row (0..3)
    int npk;   // aligned packs that cover the row
    int cols;
    // bit k set: lane k of pack `pi` belongs to the row
    __device__ __forceinline__ int valid(int pi) const {
        int first = head - pi * 4;
        int last = head + cols - pi * 4;
        first = first < 0 ? 0 : first;
        last = last > 4 ? 4 : last;
        return ((1 << last) - 1) & ~((1 << first) - 1);
    }
};

__device__ __forceinline__ float& lane_of(float4& q, int k) {
    return k == 0 ? q.x : (k == 1 ? q.y : (k == 2 ? q.z : q.w));
}

template <class Op, int TPR, int TH, int NV>
__global__ void __launch_bounds__(TH, min_ctas_for(TH, NV))
rows_masked_kernel(const RowParams p, int phase) {
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    constexpr float kLog2e = 1.4426950408889634f;
    __shared__ float red[kMaxWarps];
    constexpr int kTeams = TH / TPR;
    const int team = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kTeams + team;
    const bool active = row < p.rows;
    if (TPR >= kWarp && !active) return;
    // position of the row in units of floats from the 16-byte line that holds x[0]
    const int64_t e0 = phase + (active ? row : 0) * p.cols;
    RowEdges edge;
    edge.head = static_cast<int>(e0 & 3);
    edge.cols = p.cols;
    edge.npk = (edge.head + p.cols + 3) >> 2;
    const float* xline = p.x - phase;  // 16-byte aligned
    float* yline = p.y - phase;
    const float4* src = reinterpret_cast<const float4*>(xline) + (e0 >> 2);
    float4* dst = reinterpret_cast<float4*>(yline) + (e0 >> 2);
    const float neutral = kSoftmax ? -INFINITY : 0.0f;

    float4 v[NV];
    int okv[NV];  // which lanes of pack i belong to the row
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int pi = t + i * TPR;
        okv[i] = (active && pi < edge.npk) ? edge.valid(pi) : 0;
        if (pi < edge.npk) {
            const int ok = okv[i];
            if (ok == 15) {
                v[i] = ld_stream(src + pi);
            } else {
                v[i] = make_float4(neutral, neutral, neutral, neutral);
                const float* q = reinterpret_cast<const float*>(src + pi);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (ok & (1 << k)) lane_of(v[i], k) = ld_stream(q + k);
                }
            }
        }
    }
    // first statistic: row maximum / row mean
    float a = neutral;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (t + i * TPR < edge.npk) {
            if (kSoftmax) a = fmaxf(a, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
            else a += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    }
    const float inv_n = 1.0f / static_cast<float>(p.cols);
    if (kSoftmax) a = team_max<TPR, TH>(a, red);
    else a = team_sum<TPR, TH>(a, red) * inv_n;
    // second statistic: sum of exp(x - max) / sum of squared deviations
    float b = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int pi = t + i * TPR;
        if (pi < edge.npk) {
            if (kSoftmax) {
                v[i].x = fast_exp2((v[i].x - a) * kLog2e);
                v[i].y = fast_exp2((v[i].y - a) * kLog2e);
                v[i].z = fast_exp2((v[i].z - a) * kLog2e);
                v[i].w = fast_exp2((v[i].w - a) * kLog2e);
                b += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            } else {
                const int ok = okv[i];
                if (ok != 15) {  // foreign lanes sit on the mean: no deviation
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (!(ok & (1 << k))) lane_of(v[i], k) = a;
                    }
                }
                const float dx = v[i].x - a, dy = v[i].y - a, dz = v[i].z - a, dw = v[i].w - a;
                b += (dx * dx + dy * dy) + (dz * dz + dw * dw);
            }
        }
    }
    b = team_sum<TPR, TH>(b, red);
    if (!active) return;
    const float scale = kSoftmax ? 1.0f / b : 1.0f / sqrtf(b * inv_n + p.eps);
    if (!kSoftmax && t == 0) {
        if (p.mean_out != nullptr) p.mean_out[row] = a;
        if (p.rstd_out != nullptr) p.rstd_out[row] = scale;
    }
    const bool affine = !kSoftmax && (p.gamma != nullptr || p.beta != nullptr);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int pi = t + i * TPR;
        if (pi < edge.npk) {
            float4 o;
            if (kSoftmax) {
                o = make_float4(v[i].x * scale, v[i].y * scale, v[i].z * scale, v[i].w * scale);
            } else {
                o = make_float4((v[i].x - a) * scale, (v[i].y - a) * scale, (v[i].z - a) * scale,
                                (v[i].w - a) * scale);
                if (affine) {
                    const int c0 = pi * 4 - edge.head;  // column of lane 0 (negative on a head pack)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (okv[i] & (1 << k)) {
                            if (p.gamma != nullptr) lane_of(o, k) *= __ldg(p.gamma + c0 + k);
                            if (p.beta != nullptr) lane_of(o, k) += __ldg(p.beta + c0 + k);
                        }
                    }
                }
            }
            const int ok = okv[i];
            if (ok == 15) {
                st_stream(dst + pi, o);
            } else {
                float* q = reinterpret_cast<float*>(dst + pi);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (ok & (1 << k)) st_stream(q + k, lane_of(o, k));
                }
            }
        }
    }
}

// Short rows at any phase (up to 32 packs): a lane holds at most one pack of a row, so a team
// of TPR lanes keeps U rows in flight at once (teams take interleaved rows, so that a warp's
// loads stay contiguous).  Otherwise as rows_masked_kernel.
template <class Op, int TPR, int U>
__global__ void __launch_bounds__(256)
rows_masked_short_kernel(const RowParams p, int phase) {
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr int kTeams = 256 / TPR;
    const int team = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int64_t row0 = static_cast<int64_t>(blockIdx.x) * (kTeams * U) + team;
    const float neutral = kSoftmax ? -INFINITY : 0.0f;
    const float inv_n = 1.0f / static_cast<float>(p.cols);
    float4 v[U];
    int okv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t row = row0 + static_cast<int64_t>(u) * kTeams;
        const int64_t e0 = phase + (row < p.rows ? row : 0) * p.cols;
        RowEdges edge;
        edge.head = static_cast<int>(e0 & 3);
        edge.cols = p.cols;
        edge.npk = (edge.head + p.cols + 3) >> 2;
        okv[u] = (row < p.rows && t < edge.npk) ? edge.valid(t) : 0;
        const float4* src = reinterpret_cast<const float4*>(p.x - phase) + (e0 >> 2) + t;
        v[u] = make_float4(neutral, neutral, neutral, neutral);
        if (okv[u] == 15) {
            v[u] = ld_stream(src);
        } else {
            const float* q = reinterpret_cast<const float*>(src);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (okv[u] & (1 << k)) lane_of(v[u], k) = ld_stream(q + k);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t row = row0 + static_cast<int64_t>(u) * kTeams;
        float a = kSoftmax ? fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w))
                           : (v[u].x + v[u].y) + (v[u].z + v[u].w);
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(kFullMask, a, o);
            a = kSoftmax ? fmaxf(a, other) : a + other;
        }
        if (!kSoftmax) a *= inv_n;
        float b;
        if (kSoftmax) {
            v[u].x = fast_exp2((v[u].x - a) * kLog2e);
            v[u].y = fast_exp2((v[u].y - a) * kLog2e);
            v[u].z = fast_exp2((v[u].z - a) * kLog2e);
            v[u].w = fast_exp2((v[u].w - a) * kLog2e);
            b = (v[u].x + v[u].y) + (v[u].z + v[u].w);
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (!(okv[u] & (1 << k))) lane_of(v[u], k) = a;  // foreign lanes sit on the mean
            }
            const float dx = v[u].x - a, dy = v[u].y - a, dz = v[u].z - a, dw = v[u].w - a;
            b = (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) b += __shfl_xor_sync(kFullMask, b, o);
        if (row >= p.rows) continue;
        const float scale = kSoftmax ? 1.0f / b : 1.0f / sqrtf(b * inv_n + p.eps);
        if (!kSoftmax && t == 0) {
            if (p.mean_out != nullptr) p.mean_out[row] = a;
            if (p.rstd_out != nullptr) p.rstd_out[row] = scale;
        }
        if (okv[u] == 0) continue;
        const int64_t e0 = phase + row * p.cols;
        const int head = static_cast<int>(e0 & 3);
        float4 o4;
        if (kSoftmax) {
            o4 = make_float4(v[u].x * scale, v[u].y * scale, v[u].z * scale, v[u].w * scale);
        } else {
            o4 = make_float4((v[u].x - a) * scale, (v[u].y - a) * scale, (v[u].z - a) * scale,
                             (v[u].w - a) * scale);
            if (p.gamma != nullptr || p.beta != nullptr) {
                const int c0 = t * 4 - head;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (okv[u] & (1 << k)) {
                        if (p.gamma != nullptr) lane_of(o4, k) *= __ldg(p.gamma + c0 + k);
                        if (p.beta != nullptr) lane_of(o4, k) += __ldg(p.beta + c0 + k);
                    }
                }
            }
        }
        float4* dst = reinterpret_cast<float4*>(p.y - phase) + (e0 >> 2) + t;
        if (okv[u] == 15) {
            st_stream(dst, o4);
        } else {
            float* q = reinterpret_cast<float*>(dst);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (okv[u] & (1 << k)) st_stream(q + k, lane_of(o4, k));
            }
        }
    }
}

template <class Op, int TPR>
int launch_masked_short_cfg(const RowParams& p, cudaStream_t stream) {
    constexpr int U = 4;
    const int64_t grid = ceil_div(p.rows, static_cast<int64_t>(256 / TPR) * U);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    const int phase = static_cast<int>((reinterpret_cast<uintptr_t>(p.x) & 15u) / 4u);
    rows_masked_short_kernel<Op, TPR, U><<<static_cast<unsigned int>(grid), 256, 0, stream>>>(p, phase);
    return launch_status();
}

// ---- span form: short rows at any phase, staged through shared memory -----------------------------
//
// Rows of up to a few hundred floats whose length is not a multiple of 4 (or whose base is off
// the 16-byte grid).  In the masked form above a lane of such a row has a single 128-bit load
// in flight and the edge packs go float by float ([1048576,63]: 41-52% of the copy bandwidth).
// But consecutive rows are one contiguous run of memory whatever the row length: a CTA takes
// a run of rows, thread 0 asks the copy engine for the aligned packs that cover the run (one
// bulk-async copy, ~40 KiB in flight per CTA without a register held), teams of lanes then
// walk their rows float by float in shared memory -- consecutive lanes, consecutive floats --
// and write the results back in place, and the whole CTA stores the run as 128-bit packs.  Only
// the first and the last pack of the run can be shared with a neighbouring CTA's rows; those
// two are stored one valid float at a time.  x and y must sit at the same phase.  The kernel
// is bound by instruction issue (79% issue-active for layernorm on [1048576,63]), so EXTRAS
// compiles the layernorm's optional gamma / beta / mean / rstd away when none is passed, and
// the launcher gives a CTA a whole number of team trips.
template <class Op, int TPR, int NVS, bool EXTRAS>
__global__ void __launch_bounds__(256)
rows_span_kernel(const RowParams p, int phase, int rows_per_cta) {
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr int kTeams = 256 / TPR;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* buf = reinterpret_cast<float*>(smem_raw);
    __shared__ uint64_t bar;
    const int team = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
    int64_t nr64 = p.rows - r0;
    const int nr = static_cast<int>(nr64 < rows_per_cta ? nr64 : rows_per_cta);
    const int64_t e_lo = phase + r0 * p.cols;                     // first float of the run, from the line of x[0]
    const int64_t e_hi = e_lo + static_cast<int64_t>(nr) * p.cols;
    const int64_t pk_lo = e_lo >> 2;
    const int npk = static_cast<int>(((e_hi + 3) >> 2) - pk_lo);
    const int base = static_cast<int>(e_lo - 4 * pk_lo);          // where the run starts inside the first pack

    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_wait();  // the input may be the previous kernel's output
    if (threadIdx.x == 0) {
        mbar_expect_tx(&bar, static_cast<uint32_t>(npk) * 16u);
        bulk_g2s(buf, reinterpret_cast<const float4*>(p.x - phase) + pk_lo, static_cast<uint32_t>(npk) * 16u, &bar);
    }
    bool landed = mbar_wait_bounded(&bar, 0);
    landed = __syncthreads_and(landed);
    pdl_trigger();
    if (!landed) {
        if (threadIdx.x == 0) atomicOr(p.error_flag, 1u);
        return;
    }
    const float neutral = kSoftmax ? -INFINITY : 0.0f;
    const float inv_n = 1.0f / static_cast<float>(p.cols);
    // Team k takes rows k, k + kTeams, ...; every team runs the same number of trips, so that
    // the sub-warp teams of a warp shuffle together.
    const int trips = (nr + kTeams - 1) / kTeams;
    for (int trip = 0; trip < trips; ++trip) {
        const int i = trip * kTeams + team;
        const bool active = i < nr;
        float* rowp = buf + base + (active ? i : 0) * p.cols;
        float v[NVS];
#pragma unroll
        for (int k = 0; k < NVS; ++k) {
            const int c = t + k * TPR;
            v[k] = active && c < p.cols ? rowp[c] : neutral;
        }
        float a = v[0];
#pragma unroll
        for (int k = 1; k < NVS; ++k) a = kSoftmax ? fmaxf(a, v[k]) : a + v[k];
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(kFullMask, a, o);
            a = kSoftmax ? fmaxf(a, other) : a + other;
        }
        if (!kSoftmax) a *= inv_n;
        float b = 0.0f;
#pragma unroll
        for (int k = 0; k < NVS; ++k) {
            const int c = t + k * TPR;
            if (kSoftmax) {
                v[k] = fast_exp2((v[k] - a) * kLog2e);  // exp2(-inf) = 0 for the lanes beyond the row
                b += v[k];
            } else {
                const float d = active && c < p.cols ? v[k] - a : 0.0f;
                b += d * d;
            }
        }
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) b += __shfl_xor_sync(kFullMask, b, o);
        if (!active) continue;
        // Rows this short pay for every instruction per row: the reciprocal square root is the
        // hardware's approximate one (2 ulp), where the longer-row forms divide by sqrtf.
        const float scale = kSoftmax ? 1.0f / b : rsqrtf(b * inv_n + p.eps);
        if (!kSoftmax && EXTRAS && t == 0) {
            if (p.mean_out != nullptr) p.mean_out[r0 + i] = a;
            if (p.rstd_out != nullptr) p.rstd_out[r0 + i] = scale;
        }
#pragma unroll
        for (int k = 0; k < NVS; ++k) {
            const int c = t + k * TPR;
            if (c < p.cols) {
                float o = kSoftmax ? v[k] * scale : (v[k] - a) * scale;
                if (!kSoftmax && EXTRAS) {
                    if (p.gamma != nullptr) o *= __ldg(p.gamma + c);
                    if (p.beta != nullptr) o += __ldg(p.beta + c);
                }
                rowp[c] = o;
            }
        }
    }
    __syncthreads();
    // The run goes out as aligned packs; only its first and last pack can hold foreign floats.
    float4* dst = reinterpret_cast<float4*>(p.y - phase) + pk_lo;
    const float4* out4 = reinterpret_cast<const float4*>(buf);
    const int tail = static_cast<int>(e_hi & 3);
    for (int i = threadIdx.x; i < npk; i += 256) {
        const bool first = i == 0 && base != 0;
        const bool last = i == npk - 1 && tail != 0;
        if (!first && !last) {
            st_stream(dst + i, out4[i]);
        } else {
            float* q = reinterpret_cast<float*>(dst + i);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int64_t e = 4 * (pk_lo + i) + k;
                if (e >= e_lo && e < e_hi) q[k] = buf[4 * i + k];
            }
        }
    }
}

constexpr int kSpanBytes = 40 * 1024;  // of shared memory per CTA: five CTAs per SM

template <class Op, int TPR, int NVS>
int launch_span_cfg(const RowParams& p, cudaStream_t stream) {
    const int phase = static_cast<int>((reinterpret_cast<uintptr_t>(p.x) & 15u) / 4u);
    int64_t rows_per_cta = (kSpanBytes - 32) / (static_cast<int64_t>(p.cols) * 4);
    if (rows_per_cta < 1) return FDL_ERR_UNSUPPORTED;
    // A whole number of trips of the 256 / TPR teams: 162 rows of 63 floats would leave the
    // eleventh trip with 2 of 16 teams at work.
    constexpr int kTeams = 256 / TPR;
    if (rows_per_cta > kTeams) rows_per_cta -= rows_per_cta % kTeams;
    if (rows_per_cta > p.rows) rows_per_cta = p.rows;
    const int64_t grid = ceil_div(p.rows, rows_per_cta);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    const size_t smem = static_cast<size_t>((rows_per_cta * p.cols + 6) / 4 + 1) * 16;
    const bool extras = !std::is_same<Op, SoftmaxOp>::value &&
                        (p.gamma != nullptr || p.beta != nullptr || p.mean_out != nullptr || p.rstd_out != nullptr);
    const dim3 g(static_cast<unsigned int>(grid));
    if (extras)
        return launch_ex(rows_span_kernel<Op, TPR, NVS, true>, g, dim3(256), smem, stream, dim3(1, 1, 1),
                         tuning().pdl != 0, p, phase, static_cast<int>(rows_per_cta));
    return launch_ex(rows_span_kernel<Op, TPR, NVS, false>, g, dim3(256), smem, stream, dim3(1, 1, 1),
                     tuning().pdl != 0, p, phase, static_cast<int>(rows_per_cta));
}

// Team size and values per lane for a row of `cols` floats (at most 256).
template <class Op>
int launch_span(const RowParams& p, cudaStream_t stream) {
    const int c = p.cols;
    if (c <= 8) return launch_span_cfg<Op, 8, 1>(p, stream);
    if (c <= 16) return launch_span_cfg<Op, 8, 2>(p, stream);
    if (c <= 32) return launch_span_cfg<Op, 8, 4>(p, stream);
    if (c <= 64) return launch_span_cfg<Op, 16, 4>(p, stream);
    if (c <= 128) return launch_span_cfg<Op, 32, 4>(p, stream);
    if (c <= 256) return launch_span_cfg<Op, 32, 8>(p, stream);
    return FDL_ERR_UNSUPPORTED;
}

template <class Op, int TPR, int TH, int NV>
int launch_masked_cfg(const RowParams& p, const DeviceInfo*, cudaStream_t stream) {
    constexpr int kTeams = TH / TPR;
    const int64_t grid = ceil_div(p.rows, kTeams);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    const int phase = static_cast<int>((reinterpret_cast<uintptr_t>(p.x) & 15u) / 4u);
    rows_masked_kernel<Op, TPR, TH, NV><<<static_cast<unsigned int>(grid), TH, 0, stream>>>(p, phase);
    return launch_status();
}

// ---- staged form: one bulk copy per CTA ---------------------------------------------------------

// ---- cluster form: rows of 16384 < cols <= 8 x 16384 floats -----------------------------------------
//
// A thread-block cluster of CL CTAs (256 threads up to 65536 floats, 512 beyond; 8 packs a
// thread) owns one row: CTA `rank`
// keeps slice `rank` of it in registers and reduces it on its own; thread 0 stores the
// result into slot `rank` of EVERY CTA's shared memory (distributed shared memory) and after
// ONE cluster barrier each CTA combines the CL slots in rank order.  Softmax exchanges
// (slice maximum m_k, s_k = sum exp(x - m_k)): M = max m_k, S = sum s_k exp(m_k - M), and
// the slice's exponentials are multiplied by exp(m_rank - M) / S.  Layernorm exchanges
// (slice mean, sum of squared deviations from it), combined with the pairwise update of
// Chan et al.  The row is read once and written once.  (The wait half of the opening
// barrier sits right behind the loads: placed after the first CTA-wide reduction instead,
// the softmax kernel measured 134 us against 105 us on [2048,32768].)

constexpr int kClusterThreads = 512;
constexpr int kClusterNV = 8;

template <class Op, int CL, int TH>
__global__ void __launch_bounds__(TH, 2048 / TH / 2)
rows_cluster_kernel(const RowParams p, int slice_vecs) {
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    constexpr float kLog2e = 1.4426950408889634f;
    __shared__ float red[kMaxWarps];
    __shared__ float slots[2][8];
    cg::cluster_group cluster = cg::this_cluster();
    // Every CTA of the cluster must be running before anyone stores into its shared memory:
    // arrive now, wait once the loads have been issued.
    cluster.barrier_arrive();
    const int64_t row = blockIdx.x / CL;
    const int rank = static_cast<int>(cluster.block_rank());
    const int nvec = p.cols / 4;
    const int voff = rank * slice_vecs;
    int local = nvec - voff;
    if (local > slice_vecs) local = slice_vecs;
    if (local < 0) local = 0;
    const int t = threadIdx.x;
    const float4* src = reinterpret_cast<const float4*>(p.x + row * p.cols) + voff;
    float4 v[kClusterNV];
#pragma unroll
    for (int i = 0; i < kClusterNV; ++i) {
        if (t + i * TH < local) v[i] = ld_stream(src + t + i * TH);
    }
    cluster.barrier_wait();
    // ---- this CTA's slice on its own ----
    float a = kSoftmax ? -INFINITY : 0.0f;
#pragma unroll
    for (int i = 0; i < kClusterNV; ++i) {
        if (t + i * TH < local) {
            if (kSoftmax) a = fmaxf(a, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
            else a += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    }
    if (kSoftmax) a = team_max<TH, TH>(a, red);
    else a = local > 0 ? team_sum<TH, TH>(a, red) / static_cast<float>(local * 4) : team_sum<TH, TH>(a, red);
    float b = 0.0f;
#pragma unroll
    for (int i = 0; i < kClusterNV; ++i) {
        if (t + i * TH < local) {
            if (kSoftmax) {
                v[i].x = fast_exp2((v[i].x - a) * kLog2e);
                v[i].y = fast_exp2((v[i].y - a) * kLog2e);
                v[i].z = fast_exp2((v[i].z - a) * kLog2e);
                v[i].w = fast_exp2((v[i].w - a) * kLog2e);
                b += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            } else {
                const float dx = v[i].x - a, dy = v[i].y - a, dz = v[i].z - a, dw = v[i].w - a;
                b += (dx * dx + dy * dy) + (dz * dz + dw * dw);
            }
        }
    }
    b = team_sum<TH, TH>(b, red);
    // ---- exchange through distributed shared memory ----
    if (t == 0) {
#pragma unroll
        for (int k = 0; k < CL; ++k) {
            float* peer = cluster.map_shared_rank(&slots[0][0], k);
            peer[rank] = a;
            peer[8 + rank] = b;
        }
    }
    cluster.sync();
    float4* yr = reinterpret_cast<float4*>(p.y + row * p.cols) + voff;
    if (kSoftmax) {
        float m = slots[0][0];
#pragma unroll
        for (int k = 1; k < CL; ++k) m = fmaxf(m, slots[0][k]);
        float ssum = 0.0f;
#pragma unroll
        for (int k = 0; k < CL; ++k) ssum += slots[1][k] * fast_exp2((slots[0][k] - m) * kLog2e);
        const float f = fast_exp2((a - m) * kLog2e) / ssum;
#pragma unroll
        for (int i = 0; i < kClusterNV; ++i) {
            if (t + i * TH < local) {
                st_stream(yr + t + i * TH, make_float4(v[i].x * f, v[i].y * f, v[i].z * f, v[i].w * f));
            }
        }
    } else {
        const float inv_n = 1.0f / static_cast<float>(p.cols);
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < CL; ++k) {
            int nk = nvec - k * slice_vecs;
            nk = nk > slice_vecs ? slice_vecs : (nk < 0 ? 0 : nk);
            sum += static_cast<float>(nk * 4) * slots[0][k];
        }
        const float mean = sum * inv_n;
        float m2 = 0.0f;
#pragma unroll
        for (int k = 0; k < CL; ++k) {
            int nk = nvec - k * slice_vecs;
            nk = nk > slice_vecs ? slice_vecs : (nk < 0 ? 0 : nk);
            const float d = slots[0][k] - mean;
            m2 += slots[1][k] + static_cast<float>(nk * 4) * d * d;
        }
        const float rstd = 1.0f / sqrtf(m2 * inv_n + p.eps);
        if (t == 0 && rank == 0) {
            if (p.mean_out != nullptr) p.mean_out[row] = mean;
            if (p.rstd_out != nullptr) p.rstd_out[row] = rstd;
        }
        const float4* g4 = p.gamma == nullptr ? nullptr : reinterpret_cast<const float4*>(p.gamma) + voff;
        const float4* b4 = p.beta == nullptr ? nullptr : reinterpret_cast<const float4*>(p.beta) + voff;
#pragma unroll
        for (int i = 0; i < kClusterNV; ++i) {
            const int c = t + i * TH;
            if (c < local) {
                float4 o = make_float4((v[i].x - mean) * rstd, (v[i].y - mean) * rstd,
                                       (v[i].z - mean) * rstd, (v[i].w - mean) * rstd);
                if (g4 != nullptr) {
                    const float4 g = __ldg(g4 + c);
                    o.x *= g.x; o.y *= g.y; o.z *= g.z; o.w *= g.w;
                }
                if (b4 != nullptr) {
                    const float4 bb = __ldg(b4 + c);
                    o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
                }
                st_stream(yr + c, o);
            }
        }
    }
}

template <class Op, int CL, int TH>
int launch_cluster_cfg(const RowParams& p, cudaStream_t stream) {
    const int nvec = p.cols / 4;
    const int slice_vecs = static_cast<int>(ceil_div(static_cast<int64_t>(nvec), CL));
    if (p.rows * CL > 2147483647) return FDL_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned int>(p.rows * CL));
    cfg.blockDim = dim3(TH);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = CL;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, rows_cluster_kernel<Op, CL, TH>, p, slice_vecs);
    if (e != cudaSuccess) return static_cast<int>(e);
    return launch_status();
}

// ---- shared-memory cluster form: long rows at any phase, read once ------------------------------
//
// Beyond what a cluster's registers hold (and from 16384 floats on when the row length is not a
// multiple of 4), a cluster of CL CTAs keeps the row in SHARED memory: the row's aligned packs
// are cut into CL slices, thread 0 of each CTA asks the copy engine for its slice (bulk-async
// copies on an mbarrier: the whole slice is in flight without occupying a register), the CTA
// takes the slice's statistics from shared memory, ONE exchange of (maximum, sum of exp) or
// (mean, squared deviations) pairs crosses the cluster through distributed shared memory as
// in the register form, and the slice is normalised out of shared memory.  One read and one
// write per element, where the two-kernel form reads twice.  Slices of up to 64 KiB leave room
// for three or more CTAs per SM, so one CTA's arithmetic overlaps its neighbours' copies.  A
// row may start at any phase of a 16-byte line: the first and last pack of a row are then
// shared with the neighbouring rows; they are copied whole, read with the foreign lanes masked,
// and written back one valid float at a time.  x and y must sit at the same phase.
// A copy that does not complete in the bounded wait raises the device-error flag; the CTA then
// still walks through the cluster barriers (its peers wait there) and stores nothing.

template <class Op, int CL, int TH>
__global__ void __launch_bounds__(TH)
rows_smem_kernel(const RowParams p, int phase, int slice_pk) {
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    constexpr float kLog2e = 1.4426950408889634f;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float4* slice = reinterpret_cast<float4*>(smem_raw);
    __shared__ uint64_t bar;
    __shared__ float red[kMaxWarps];
    __shared__ float slots[2][16];
    cg::cluster_group cluster = cg::this_cluster();
    cluster.barrier_arrive();  // waited for once the copy has been requested
    const int64_t row = blockIdx.x / CL;
    const int rank = static_cast<int>(cluster.block_rank());
    const int t = threadIdx.x;
    const int64_t e0 = phase + row * p.cols;  // the row's first float, counted from the 16-byte line of x[0]
    RowEdges edge;
    edge.head = static_cast<int>(e0 & 3);
    edge.cols = p.cols;
    edge.npk = (edge.head + p.cols + 3) >> 2;
    const int pk0 = rank * slice_pk;
    int local = edge.npk - pk0;
    local = local > slice_pk ? slice_pk : (local < 0 ? 0 : local);
    const float4* src = reinterpret_cast<const float4*>(p.x - phase) + (e0 >> 2) + pk0;
    float4* dst = reinterpret_cast<float4*>(p.y - phase) + (e0 >> 2) + pk0;
    // floats of the row in slice k (the same arithmetic on every CTA)
    auto count_of = [&](int k) {
        int lo = 4 * k * slice_pk, hi = lo + 4 * slice_pk;
        lo = lo < edge.head ? edge.head : lo;
        hi = hi > edge.head + p.cols ? edge.head + p.cols : hi;
        return hi > lo ? hi - lo : 0;
    };

    if (t == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_wait();  // the input may be the previous kernel's output
    if (t == 0 && local > 0) {
        mbar_expect_tx(&bar, static_cast<uint32_t>(local) * 16u);
        constexpr int kChunk = 4096;  // packs per copy (64 KiB)
        for (int off = 0; off < local; off += kChunk) {
            const int n = local - off < kChunk ? local - off : kChunk;
            bulk_g2s(slice + off, src + off, static_cast<uint32_t>(n) * 16u, &bar);
        }
    }
    cluster.barrier_wait();
    bool landed = local == 0 || mbar_wait_bounded(&bar, 0);
    landed = __syncthreads_and(landed);
    pdl_trigger();
    if (!landed && t == 0) atomicOr(p.error_flag, 1u);

    // the packs of the row that this row owns only in part: at most the first and the last
    const bool ragged = edge.head != 0 || ((edge.head + p.cols) & 3) != 0;
    auto mask_of = [&](int i) { return ragged ? edge.valid(pk0 + i) : 15; };

    // ---- this CTA's slice on its own ----
    float a = kSoftmax ? -INFINITY : 0.0f;
    if (landed) {
        for (int i = t; i < local; i += TH) {
            float4 v = slice[i];
            const int ok = mask_of(i);
            if (ok != 15) {
                const float neutral = kSoftmax ? -INFINITY : 0.0f;
                if (!(ok & 1)) v.x = neutral;
                if (!(ok & 2)) v.y = neutral;
                if (!(ok & 4)) v.z = neutral;
                if (!(ok & 8)) v.w = neutral;
            }
            if (kSoftmax) a = fmaxf(a, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
            else a += (v.x + v.y) + (v.z + v.w);
        }
    }
    const int mine = count_of(rank);
    if (kSoftmax) a = team_max<TH, TH>(a, red);
    else a = mine > 0 ? team_sum<TH, TH>(a, red) / static_cast<float>(mine) : team_sum<TH, TH>(a, red);
    float b = 0.0f;
    if (landed) {
        for (int i = t; i < local; i += TH) {
            float4 v = slice[i];
            const int ok = mask_of(i);
            if (kSoftmax) {
                v.x = (ok & 1) ? fast_exp2((v.x - a) * kLog2e) : 0.0f;
                v.y = (ok & 2) ? fast_exp2((v.y - a) * kLog2e) : 0.0f;
                v.z = (ok & 4) ? fast_exp2((v.z - a) * kLog2e) : 0.0f;
                v.w = (ok & 8) ? fast_exp2((v.w - a) * kLog2e) : 0.0f;
                slice[i] = v;  // the exponentials replace the inputs
                b += (v.x + v.y) + (v.z + v.w);
            } else {
                const float dx = (ok & 1) ? v.x - a : 0.0f, dy = (ok & 2) ? v.y - a : 0.0f;
                const float dz = (ok & 4) ? v.z - a : 0.0f, dw = (ok & 8) ? v.w - a : 0.0f;
                b += (dx * dx + dy * dy) + (dz * dz + dw * dw);
            }
        }
    }
    b = team_sum<TH, TH>(b, red);
    // ---- exchange through distributed shared memory ----
    if (t == 0) {
#pragma unroll
        for (int k = 0; k < CL; ++k) {
            float* peer = cluster.map_shared_rank(&slots[0][0], k);
            peer[rank] = a;
            peer[16 + rank] = b;
        }
    }
    cluster.sync();
    if (!landed) return;
    // Writes a pack: whole when the row owns all of it, else its valid floats one by one.
    auto store_pack = [&](int i, float4 o) {
        const int ok = mask_of(i);
        if (ok == 15) {
            st_stream(dst + i, o);
        } else {
            float* q = reinterpret_cast<float*>(dst + i);
            if (ok & 1) q[0] = o.x;
            if (ok & 2) q[1] = o.y;
            if (ok & 4) q[2] = o.z;
            if (ok & 8) q[3] = o.w;
        }
    };
    if (kSoftmax) {
        float m = slots[0][0];
#pragma unroll
        for (int k = 1; k < CL; ++k) m = fmaxf(m, slots[0][k]);
        float ssum = 0.0f;
#pragma unroll
        for (int k = 0; k < CL; ++k) {
            // a slice without a float of the row reports (-inf, 0)
            ssum += slots[0][k] == -INFINITY ? 0.0f : slots[1][k] * fast_exp2((slots[0][k] - m) * kLog2e);
        }
        const float f = fast_exp2((a - m) * kLog2e) / ssum;
        for (int i = t; i < local; i += TH) {
            const float4 v = slice[i];
            store_pack(i, make_float4(v.x * f, v.y * f, v.z * f, v.w * f));
        }
    } else {
        const float inv_n = 1.0f / static_cast<float>(p.cols);
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < CL; ++k) sum += static_cast<float>(count_of(k)) * slots[0][k];
        const float mean = sum * inv_n;
        float m2 = 0.0f;
#pragma unroll
        for (int k = 0; k < CL; ++k) {
            const float d = slots[0][k] - mean;
            m2 += slots[1][k] + static_cast<float>(count_of(k)) * d * d;
        }
        const float rstd = 1.0f / sqrtf(m2 * inv_n + p.eps);
        if (t == 0 && rank == 0) {
            if (p.mean_out != nullptr) p.mean_out[row] = mean;
            if (p.rstd_out != nullptr) p.rstd_out[row] = rstd;
        }
        const bool affine = p.gamma != nullptr || p.beta != nullptr;
        for (int i = t; i < local; i += TH) {
            const float4 v = slice[i];
            float4 o = make_float4((v.x - mean) * rstd, (v.y - mean) * rstd, (v.z - mean) * rstd, (v.w - mean) * rstd);
            if (affine) {
                const int ok = mask_of(i);
                const int c0 = 4 * (pk0 + i) - edge.head;  // column of the pack's first lane
                float* lanes[4] = {&o.x, &o.y, &o.z, &o.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (ok & (1 << k)) {
                        if (p.gamma != nullptr) *lanes[k] *= __ldg(p.gamma + c0 + k);
                        if (p.beta != nullptr) *lanes[k] += __ldg(p.beta + c0 + k);
                    }
                }
            }
            store_pack(i, o);
        }
    }
}

// Packs per slice that one CTA may hold (dynamic shared memory, a little kept for the static part).
inline int smem_slice_limit_packs(const DeviceInfo* info) { return (info->max_smem_optin - 2048) / 16; }

template <class Op, int CL, int TH>
int launch_rows_smem_cfg(const RowParams& p, const DeviceInfo* info, int phase, int slice_pk, cudaStream_t stream) {
    auto kernel = rows_smem_kernel<Op, CL, TH>;
    const size_t smem = static_cast<size_t>(slice_pk) * 16;
    static size_t configured_smem[kMaxDevicesTracked] = {};
    static bool nonportable[kMaxDevicesTracked] = {};
    size_t& configured = configured_smem[info->device % kMaxDevicesTracked];
    if (smem > 48 * 1024 - 1024 && smem > configured) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = smem;
    }
    if (CL > 8 && !nonportable[info->device % kMaxDevicesTracked]) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return static_cast<int>(e);
        nonportable[info->device % kMaxDevicesTracked] = true;
    }
    return launch_ex(kernel, dim3(static_cast<unsigned int>(p.rows * CL)), dim3(TH), smem, stream, dim3(CL, 1, 1),
                     tuning().pdl != 0, p, phase, slice_pk);
}

// Picks the cluster size (tuning key rows_smem_cluster forces one): the smallest of 2, 4, 8 CTAs
// per row whose slices stay within `kSmemSliceTarget` packs, so that several CTAs fit an SM and one
// CTA's arithmetic overlaps its neighbours' copies; FDL_ERR_UNSUPPORTED when even 16 CTAs (beyond
// the portable cluster size) would need larger slices than one CTA's shared memory.
constexpr int kSmemSliceTarget = 4096;  // 64 KiB

template <class Op, int CL>
int launch_rows_smem_cl(const RowParams& p, const DeviceInfo* info, int phase, int64_t npk_worst, cudaStream_t stream) {
    const int64_t slice = ceil_div(npk_worst, CL);
    if (slice > smem_slice_limit_packs(info)) return FDL_ERR_UNSUPPORTED;
    if (slice <= kSmemSliceTarget) return launch_rows_smem_cfg<Op, CL, 256>(p, info, phase, static_cast<int>(slice), stream);
    return launch_rows_smem_cfg<Op, CL, 512>(p, info, phase, static_cast<int>(slice), stream);
}

template <class Op>
int launch_rows_smem(const RowParams& p, const DeviceInfo* info, cudaStream_t stream) {
    const int phase = static_cast<int>((reinterpret_cast<uintptr_t>(p.x) & 15u) / 4u);
    const int64_t npk_worst = (static_cast<int64_t>(p.cols) + 6) / 4;  // a row at the worst phase
    if (p.rows * 16 > 2147483647) return FDL_ERR_UNSUPPORTED;
    int cl = tuning().rows_smem_cluster;
    if (cl == 0) {
        cl = 2;
        while (cl < 8 && ceil_div(npk_worst, cl) > kSmemSliceTarget) cl <<= 1;
        if (ceil_div(npk_worst, cl) > kSmemSliceTarget) return FDL_ERR_UNSUPPORTED;  // longer rows: the two-kernel form
    }
    switch (cl) {
        case 2: return launch_rows_smem_cl<Op, 2>(p, info, phase, npk_worst, stream);
        case 4: return launch_rows_smem_cl<Op, 4>(p, info, phase, npk_worst, stream);
        case 8: return launch_rows_smem_cl<Op, 8>(p, info, phase, npk_worst, stream);
        default: return launch_rows_smem_cl<Op, 16>(p, info, phase, npk_worst, stream);
    }
}

// ---- staged form -------------------------------------------------------------------------------

template <class Op, int TPR, int TH, int NV>
__global__ void __launch_bounds__(TH, min_ctas_for(TH, NV))
rows_staged_kernel(const RowParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t bar;
    __shared__ float red[kMaxWarps];
    constexpr int kTeams = TH / TPR;
    const int team = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int rows_per_cta = kTeams * p.rows_per_team;
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
    // Team k takes rows k, k + kTeams, ... of the span; the trip count is the same for all
    // teams of a warp, so sub-warp teams shuffle together.
    for (int i0 = 0; i0 < p.rows_per_team; ++i0) {
        const int r = i0 * kTeams + team;
        const bool active = r < nr;
        if (TPR >= kWarp && !active) break;
        float4 v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (t + i * TPR < nvec) {
                v[i] = active ? src[r * nvec + t + i * TPR] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        TeamScope<TPR, TH> scope{red};
        row_math<TPR, TH, NV>(Op{}, v, t, nvec, p, r0 + r, active, scope);
    }
}

// ---- split form: rows longer than a cluster can hold -------------------------------------------
//
// Every row is cut into 32 KiB segments, one CTA each: the CTA keeps its segment in registers,
// leaves the segment's statistics in the workspace -- softmax: (max, sum of exp(x - max));
// layernorm: (mean, sum of squared deviations from it) -- and the last CTA of a row to arrive
// (ticket counter) combines the segments' statistics into the row's: softmax rescales each sum to
// the row maximum, layernorm uses the pairwise update of Chan et al., both in a fixed order.
//
// Two-kernel form: the first kernel ends with the statistics, a second one reads the rows again
// and applies them -- two reads and one write per element from DRAM (by the time the second
// kernel starts, the first has pushed the head of the tensor out of L2), against the three
// passes of the plain kernel.
//
// One-kernel form (the default): both passes are tasks of ONE launch, and a segment is applied
// `lag` rows after its statistics were taken, while it is still in L2 (the statistics pass loads
// with an L2 evict-last hint, the apply pass with evict-first, stores are streaming).  Every CTA
// first takes a ticket from a counter; tickets enumerate the nseg statistics tasks of row k
// followed by the nseg apply tasks of row k - lag, row after row.  An apply task waits for the
// row's statistics -- for tasks with SMALLER tickets, which CTAs that are already running hold (a
// CTA takes its ticket when it starts) and which wait for nothing themselves, so the wait ends
// whatever order the hardware starts CTAs in; it is bounded all the same.  A row's counter goes
// 0 .. nseg (arrivals), nseg + 1 (statistics ready), .. 2 nseg + 1 (apply tasks done), and the
// last task puts it back to 0.  The ticket counter is the last slot of the workspace's counter
// block (rows use the others); its last taker zeroes it.  `lag` covers the 5-9 us from a
// statistics task's start to the row's statistics (measured: a distance of 32-40 MB of rows is
// needed before apply tasks stop stalling; less, and they hold CTA slots while they wait).
//
// The kernel reads every element once from DRAM (profiled on [128,524288]: 273 MB read for a
// 268 MB tensor) but is bound by latency, not by DRAM (48-58% busy): a task is a chain of round
// trips to L2 -- ticket, loads, publish or wait -- during which its CTA slot holds no load in flight.
//
// (Measured and dropped: persistent CTAs with a ring of 32 KiB shared-memory stages filled by
// bulk-async copies a few tickets ahead, so that loads stay in flight while the threads reduce,
// publish and wait: 2 CTAs x 3 stages per SM 41%, 3 CTAs x 2 stages 54% -- the per-task chain of
// round trips is serial inside a CTA and fewer CTAs per SM run fewer chains at once.)
//
// (Measured and dropped: the CTAs of a row holding their segments in registers while they wait
// for the row's statistics, a cluster in software of up to 296 CTAs, one read and one write per
// element.  The chain load - reduce - publish - combine - flag - apply is ~10 us long and the
// register file holds 19 MB: 46-54% of the copy bandwidth on [128,524288] and [256,262144],
// against 56-67% for the two kernels.)

constexpr int kSplitThreads = 256;
constexpr int kSplitNV = 8;
constexpr int kSplitSegVecs = kSplitThreads * kSplitNV;  // 2048 packs = 32 KiB
constexpr int64_t kSplitMaxRows = kWorkspaceCounterBytes / 4;
constexpr unsigned long long kSplitWaitNs = 2000000000ull;  // bounded wait of the one-kernel form

// The kernels address a row through the aligned packs of the flat buffer (RowEdges, as in the
// masked form), so rows of any length and phase qualify; MASKED = false compiles the edge
// handling away for rows that are whole packs.

struct SplitSeg {
    RowEdges edge;
    int64_t first_pack;  // of the row, in the flat buffer
    int voff;            // first pack of the segment, counted from the row's first
    int local;           // packs of the row inside the segment
};

template <bool MASKED>
__device__ __forceinline__ SplitSeg split_segment(const RowParams& p, int phase, int64_t row, int seg) {
    SplitSeg sg;
    const int64_t e0 = phase + row * p.cols;
    sg.edge.head = MASKED ? static_cast<int>(e0 & 3) : 0;
    sg.edge.cols = p.cols;
    sg.edge.npk = (sg.edge.head + p.cols + 3) >> 2;
    sg.first_pack = e0 >> 2;
    sg.voff = seg * kSplitSegVecs;
    sg.local = sg.edge.npk - sg.voff;
    if (sg.local > kSplitSegVecs) sg.local = kSplitSegVecs;
    return sg;
}

__device__ __forceinline__ int split_count(const RowEdges& e, int seg) {
    // floats of the row inside segment `seg`
    const int lo = max(e.head, seg * kSplitSegVecs * 4);
    const int hi = min(e.head + e.cols, (seg + 1) * kSplitSegVecs * 4);
    return hi > lo ? hi - lo : 0;
}

// Loads with an L2 eviction-priority hint (policy from createpolicy).
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ float4 ld_hint(const float4* ptr, uint64_t policy) {
    float4 v;
    asm volatile("ld.global.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(ptr), "l"(policy));
    return v;
}
__device__ __forceinline__ float ld_hint(const float* ptr, uint64_t policy) {
    float v;
    asm volatile("ld.global.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(ptr), "l"(policy));
    return v;
}

// The segment into registers; lanes of an edge pack that belong to a neighbouring row get `neutral`.
// HINT 0: streaming loads; 1: the lines are to stay in L2 (evict last); 2: they are not (evict first).
template <bool MASKED, int HINT>
__device__ __forceinline__ void split_load(const RowParams& p, int phase, const SplitSeg& sg, float neutral,
                                           float4 (&v)[kSplitNV], int (&okv)[kSplitNV]) {
    const int t = threadIdx.x;
    uint64_t policy = 0;
    if (HINT == 1) policy = l2_policy_evict_last();
    if (HINT == 2) policy = l2_policy_evict_first();
    const float4* src = reinterpret_cast<const float4*>(p.x - phase) + sg.first_pack + sg.voff;
#pragma unroll
    for (int i = 0; i < kSplitNV; ++i) {
        const int li = t + i * kSplitThreads;
        okv[i] = li < sg.local ? (MASKED ? sg.edge.valid(sg.voff + li) : 15) : 0;
        if (li < sg.local) {
            if (okv[i] == 15) {
                v[i] = HINT == 0 ? ld_stream(src + li) : ld_hint(src + li, policy);
            } else {
                v[i] = make_float4(neutral, neutral, neutral, neutral);
                const float* q = reinterpret_cast<const float*>(src + li);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (okv[i] & (1 << k)) lane_of(v[i], k) = HINT == 0 ? ld_stream(q + k) : ld_hint(q + k, policy);
                }
            }
        }
    }
}

// The segment's statistics, in every thread.  Layernorm: foreign lanes of edge packs are moved
// onto the segment mean on the way (they are never stored).
template <class Op, bool MASKED>
__device__ __forceinline__ float2 split_segment_stats(const SplitSeg& sg, int seg, float4 (&v)[kSplitNV],
                                                      const int (&okv)[kSplitNV], float* red) {
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    constexpr float kLog2e = 1.4426950408889634f;
    const int t = threadIdx.x;
    float a = kSoftmax ? -INFINITY : 0.0f;
#pragma unroll
    for (int i = 0; i < kSplitNV; ++i) {
        if (t + i * kSplitThreads < sg.local) {
            if (kSoftmax) a = fmaxf(a, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
            else a += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    }
    const int count = split_count(sg.edge, seg);
    if (kSoftmax) a = team_max<kSplitThreads, kSplitThreads>(a, red);
    else a = team_sum<kSplitThreads, kSplitThreads>(a, red) / static_cast<float>(count > 0 ? count : 1);
    float b = 0.0f;
#pragma unroll
    for (int i = 0; i < kSplitNV; ++i) {
        if (t + i * kSplitThreads < sg.local) {
            if (kSoftmax) {
                b += (fast_exp2((v[i].x - a) * kLog2e) + fast_exp2((v[i].y - a) * kLog2e)) +
                     (fast_exp2((v[i].z - a) * kLog2e) + fast_exp2((v[i].w - a) * kLog2e));
            } else {
                if (MASKED && okv[i] != 15) {  // foreign lanes sit on the mean
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (!(okv[i] & (1 << k))) lane_of(v[i], k) = a;
                    }
                }
                const float dx = v[i].x - a, dy = v[i].y - a, dz = v[i].z - a, dw = v[i].w - a;
                b += (dx * dx + dy * dy) + (dz * dz + dw * dw);
            }
        }
    }
    b = team_sum<kSplitThreads, kSplitThreads>(b, red);
    if (kSoftmax && count == 0) b = 0.0f;  // an empty segment: exp(-inf - -inf) is not a number
    return make_float2(a, b);
}

// Leaves the segment's statistics in the workspace; the last CTA of the row to arrive combines
// them into row_stats[row].  SIGNAL: the row's counter is then set to nseg + 1 for the waiting
// CTAs instead of back to 0.
template <class Op, bool SIGNAL>
__device__ __forceinline__ void split_publish(const RowParams& p, const SplitSeg& sg, int64_t row, int seg, int nseg,
                                              float2 ab, float2* seg_stats, float2* row_stats, unsigned int* counters,
                                              float* red, bool* is_last) {
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    constexpr float kLog2e = 1.4426950408889634f;
    const int t = threadIdx.x;
    if (t == 0) {
        seg_stats[row * nseg + seg] = ab;
        __threadfence();
        const unsigned int ticket = atomicAdd(counters + row, 1u);
        *is_last = ticket == static_cast<unsigned int>(nseg - 1);
        if (*is_last && !SIGNAL) counters[row] = 0;
    }
    __syncthreads();
    if (!*is_last) return;
    __threadfence();
    // Thread k takes segments k, k + 256, ... in order.
    const float2* mine = seg_stats + row * nseg;
    float2 result;
    if (kSoftmax) {
        float m = -INFINITY;
        for (int k = t; k < nseg; k += kSplitThreads) m = fmaxf(m, __ldcg(&mine[k].x));
        m = team_max<kSplitThreads, kSplitThreads>(m, red);
        float s = 0.0f;
        for (int k = t; k < nseg; k += kSplitThreads) {
            const float sk = __ldcg(&mine[k].y);
            if (sk != 0.0f) s += sk * fast_exp2((__ldcg(&mine[k].x) - m) * kLog2e);
        }
        s = team_sum<kSplitThreads, kSplitThreads>(s, red);
        result = make_float2(m, 1.0f / s);
    } else {
        // mean = sum n_k mean_k / N;  M2 = sum (M2_k + n_k (mean_k - mean)^2)
        const float inv_n = 1.0f / static_cast<float>(p.cols);
        float s = 0.0f;
        for (int k = t; k < nseg; k += kSplitThreads) {
            s += static_cast<float>(split_count(sg.edge, k)) * __ldcg(&mine[k].x);
        }
        const float mean = team_sum<kSplitThreads, kSplitThreads>(s, red) * inv_n;
        float q = 0.0f;
        for (int k = t; k < nseg; k += kSplitThreads) {
            const float d = __ldcg(&mine[k].x) - mean;
            q += __ldcg(&mine[k].y) + static_cast<float>(split_count(sg.edge, k)) * d * d;
        }
        const float var = team_sum<kSplitThreads, kSplitThreads>(q, red) * inv_n;
        result = make_float2(mean, 1.0f / sqrtf(var + p.eps));
    }
    if (t == 0) {
        row_stats[row] = result;
        if (!kSoftmax) {
            if (p.mean_out != nullptr) p.mean_out[row] = result.x;
            if (p.rstd_out != nullptr) p.rstd_out[row] = result.y;
        }
        if (SIGNAL) {
            __threadfence();
            *reinterpret_cast<volatile unsigned int*>(counters + row) = static_cast<unsigned int>(nseg) + 1u;
        }
    }
}

// y = the row's statistics applied to the segment in registers.
template <class Op, bool MASKED>
__device__ __forceinline__ void split_apply_store(const RowParams& p, int phase, const SplitSeg& sg, float2 st,
                                                  const float4 (&v)[kSplitNV], const int (&okv)[kSplitNV]) {
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    constexpr float kLog2e = 1.4426950408889634f;
    const int t = threadIdx.x;
    float4* dst = reinterpret_cast<float4*>(p.y - phase) + sg.first_pack + sg.voff;
    const bool affine = !kSoftmax && (p.gamma != nullptr || p.beta != nullptr);
    // gamma / beta line up with the packs (and can be read 128 bits at a time)
    const bool affine_packs = (!MASKED || sg.edge.head == 0) &&
                              ((reinterpret_cast<uintptr_t>(p.gamma) | reinterpret_cast<uintptr_t>(p.beta)) & 15u) == 0;
#pragma unroll
    for (int i = 0; i < kSplitNV; ++i) {
        const int li = t + i * kSplitThreads;
        if (li < sg.local) {
            float4 o;
            if (kSoftmax) {
                o = make_float4(fast_exp2((v[i].x - st.x) * kLog2e) * st.y, fast_exp2((v[i].y - st.x) * kLog2e) * st.y,
                                fast_exp2((v[i].z - st.x) * kLog2e) * st.y, fast_exp2((v[i].w - st.x) * kLog2e) * st.y);
            } else {
                o = make_float4((v[i].x - st.x) * st.y, (v[i].y - st.x) * st.y, (v[i].z - st.x) * st.y,
                                (v[i].w - st.x) * st.y);
                if (affine) {
                    const int c0 = (sg.voff + li) * 4 - sg.edge.head;
                    if (affine_packs && okv[i] == 15) {
                        if (p.gamma != nullptr) {
                            const float4 g = __ldg(reinterpret_cast<const float4*>(p.gamma + c0));
                            o.x *= g.x; o.y *= g.y; o.z *= g.z; o.w *= g.w;
                        }
                        if (p.beta != nullptr) {
                            const float4 bb = __ldg(reinterpret_cast<const float4*>(p.beta + c0));
                            o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (okv[i] & (1 << k)) {
                                if (p.gamma != nullptr) lane_of(o, k) *= __ldg(p.gamma + c0 + k);
                                if (p.beta != nullptr) lane_of(o, k) += __ldg(p.beta + c0 + k);
                            }
                        }
                    }
                }
            }
            if (okv[i] == 15) {
                st_stream(dst + li, o);
            } else {
                float* q = reinterpret_cast<float*>(dst + li);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (okv[i] & (1 << k)) st_stream(q + k, lane_of(o, k));
                }
            }
        }
    }
}

template <class Op, bool MASKED>
__global__ void __launch_bounds__(kSplitThreads, MASKED ? 4 : 5)
rows_split_stats_kernel(const RowParams p, int phase, float2* seg_stats, float2* row_stats,
                        unsigned int* counters) {
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    __shared__ float red[kMaxWarps];
    __shared__ bool is_last;
    const int64_t row = blockIdx.y;
    const int seg = blockIdx.x;
    const SplitSeg sg = split_segment<MASKED>(p, phase, row, seg);
    float4 v[kSplitNV];
    int okv[kSplitNV];
    split_load<MASKED, 0>(p, phase, sg, kSoftmax ? -INFINITY : 0.0f, v, okv);
    const float2 ab = split_segment_stats<Op, MASKED>(sg, seg, v, okv, red);
    split_publish<Op, false>(p, sg, row, seg, gridDim.x, ab, seg_stats, row_stats, counters, red, &is_last);
}

template <class Op, bool MASKED>
__global__ void __launch_bounds__(kSplitThreads, MASKED ? 4 : 5)
rows_split_apply_kernel(const RowParams p, int phase, const float2* row_stats) {
    const int64_t row = blockIdx.y;
    const SplitSeg sg = split_segment<MASKED>(p, phase, row, blockIdx.x);
    float4 v[kSplitNV];
    int okv[kSplitNV];
    split_load<MASKED, 0>(p, phase, sg, 0.0f, v, okv);
    split_apply_store<Op, MASKED>(p, phase, sg, row_stats[row], v, okv);
}

// The one-kernel form.  Tickets enumerate: the statistics tasks of rows 0 .. lag-1; then, for
// row k = lag .. rows-1, the statistics tasks of row k followed by the apply tasks of row
// k - lag; then the apply tasks of the last lag rows.  HINTS = false uses plain streaming loads
// in both passes (tuning key rows_split_hints = 0, for comparison).
struct SplitPlan {
    int64_t rows;
    int nseg;
    int lag;
    unsigned int head;    // tickets before the first apply task: lag * nseg
    unsigned int middle;  // tickets of the rounds that hold both kinds: (rows - lag) * 2 * nseg
};

struct SplitTask {
    int64_t row;
    int seg;
    bool apply;
};

// The plan of `rows` rows of `nseg` segments with the apply pass `lag` rows behind (1 <= lag <= rows).
inline SplitPlan make_split_plan(int64_t rows, int64_t nseg, int64_t lag) {
    SplitPlan plan;
    plan.rows = rows;
    plan.nseg = static_cast<int>(nseg);
    plan.lag = static_cast<int>(lag);
    plan.head = static_cast<unsigned int>(lag * nseg);
    plan.middle = static_cast<unsigned int>((rows - lag) * 2 * nseg);
    return plan;
}

// Ticket -> task; tickets run from 0 to 2 * rows * nseg - 1.  Host and device share this function
// (fdl_debug_split_ticket lets a test on the host walk the whole enumeration).
__host__ __device__ inline SplitTask split_decode(const SplitPlan& plan, unsigned int ticket) {
    SplitTask task;
    const unsigned int n = static_cast<unsigned int>(plan.nseg);
    if (ticket < plan.head) {
        task.row = ticket / n;
        task.seg = static_cast<int>(ticket % n);
        task.apply = false;
    } else if (ticket < plan.head + plan.middle) {
        const unsigned int u = ticket - plan.head;
        const unsigned int k = u / (2u * n), j = u % (2u * n);
        task.apply = j >= n;
        task.row = task.apply ? k : static_cast<int64_t>(k) + plan.lag;
        task.seg = static_cast<int>(task.apply ? j - n : j);
    } else {
        const unsigned int u = ticket - plan.head - plan.middle;
        task.row = plan.rows - plan.lag + u / n;
        task.seg = static_cast<int>(u % n);
        task.apply = true;
    }
    return task;
}

template <class Op, bool MASKED, bool HINTS>
__global__ void __launch_bounds__(kSplitThreads, (MASKED || !std::is_same<Op, SoftmaxOp>::value) ? 4 : 5)
rows_split_pipelined_kernel(const RowParams p, int phase, const SplitPlan plan, float2* seg_stats, float2* row_stats,
                            unsigned int* counters) {
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    __shared__ float red[kMaxWarps];
    __shared__ bool is_last;
    __shared__ unsigned int ticket_shared;
    const int t = threadIdx.x;
    pdl_wait();  // the input may be the previous kernel's output
    unsigned int* queue = counters + (kSplitMaxRows - 1);
    if (t == 0) {
        ticket_shared = atomicAdd(queue, 1u);
        if (ticket_shared == gridDim.x - 1) *queue = 0;
    }
    __syncthreads();
    const SplitTask task = split_decode(plan, ticket_shared);
    const unsigned int n = static_cast<unsigned int>(plan.nseg);
    const int64_t row = task.row;
    const int seg = task.seg;
    const bool apply = task.apply;
    const SplitSeg sg = split_segment<MASKED>(p, phase, row, seg);
    float4 v[kSplitNV];
    int okv[kSplitNV];
    if (!apply) {
        split_load<MASKED, HINTS ? 1 : 0>(p, phase, sg, kSoftmax ? -INFINITY : 0.0f, v, okv);
        const float2 ab = split_segment_stats<Op, MASKED>(sg, seg, v, okv, red);
        split_publish<Op, true>(p, sg, row, seg, plan.nseg, ab, seg_stats, row_stats, counters, red, &is_last);
        return;
    }
    split_load<MASKED, HINTS ? 2 : 0>(p, phase, sg, 0.0f, v, okv);  // in flight while thread 0 waits
    bool ready = true;
    if (t == 0) {
        const volatile unsigned int* flag = counters + row;
        const unsigned long long t0 = timer_ns();
        unsigned int polls = 0;
        while (*flag <= n) {
            if ((++polls & 63u) == 0 && timer_ns() - t0 > kSplitWaitNs) {
                ready = false;
                break;
            }
        }
        __threadfence();
    }
    ready = __syncthreads_and(ready);
    if (ready) split_apply_store<Op, MASKED>(p, phase, sg, __ldcg(row_stats + row), v, okv);
    if (t == 0) {
        if (!ready) atomicOr(p.error_flag, 4u);
        const unsigned int before = atomicAdd(counters + row, 1u);
        if (before == 2u * n) counters[row] = 0;  // the row's last task
    }
}

constexpr int64_t kSplitLagBytes = 36ll << 20;

template <class Op, bool MASKED>
int launch_rows_split_pipelined(const RowParams& p, int phase, int64_t nseg, float2* seg_stats, float2* row_stats,
                                unsigned int* counters, cudaStream_t stream) {
    int64_t lag = tuning().rows_split_lag > 0 ? tuning().rows_split_lag
                                              : ceil_div(kSplitLagBytes, static_cast<int64_t>(p.cols) * 4);
    if (lag > p.rows) lag = p.rows;
    const int64_t tasks = 2 * p.rows * nseg;
    if (tasks > 2147483647 || p.rows >= kSplitMaxRows) return FDL_ERR_UNSUPPORTED;
    const SplitPlan plan = make_split_plan(p.rows, nseg, lag);
    const dim3 grid(static_cast<unsigned int>(tasks));
    if (tuning().rows_split_hints != 0)
        return launch_ex(rows_split_pipelined_kernel<Op, MASKED, true>, grid, dim3(kSplitThreads), 0, stream, dim3(1, 1, 1),
                         tuning().pdl != 0, p, phase, plan, seg_stats, row_stats, counters);
    return launch_ex(rows_split_pipelined_kernel<Op, MASKED, false>, grid, dim3(kSplitThreads), 0, stream, dim3(1, 1, 1),
                     tuning().pdl != 0, p, phase, plan, seg_stats, row_stats, counters);
}

template <class Op, bool MASKED>
int launch_rows_split(const RowParams& p, cudaStream_t stream) {
    const int phase = MASKED ? static_cast<int>((reinterpret_cast<uintptr_t>(p.x) & 15u) / 4u) : 0;
    const int64_t npk = MASKED ? (static_cast<int64_t>(p.cols) + 6) / 4 : p.cols / 4;
    const int64_t nseg = ceil_div(npk, static_cast<int64_t>(kSplitSegVecs));
    const size_t seg_bytes = static_cast<size_t>(p.rows) * nseg * sizeof(float2);
    const size_t row_bytes = ((static_cast<size_t>(p.rows) * sizeof(float2) + 255) / 256) * 256;
    void* scratch = nullptr;
    const int status = get_workspace(kWorkspaceCounterBytes + row_bytes + seg_bytes, &scratch);
    if (status != FDL_OK) return status;
    unsigned int* counters = static_cast<unsigned int*>(scratch);
    float2* row_stats = reinterpret_cast<float2*>(static_cast<char*>(scratch) + kWorkspaceCounterBytes);
    float2* seg_stats = reinterpret_cast<float2*>(static_cast<char*>(scratch) + kWorkspaceCounterBytes + row_bytes);
    if (tuning().rows_split_fused != 0) {
        const int st = launch_rows_split_pipelined<Op, MASKED>(p, phase, nseg, seg_stats, row_stats, counters, stream);
        if (st != FDL_ERR_UNSUPPORTED) return st;
    }
    if (p.rows > 65535) return FDL_ERR_UNSUPPORTED;
    const dim3 grid(static_cast<unsigned int>(nseg), static_cast<unsigned int>(p.rows));
    rows_split_stats_kernel<Op, MASKED><<<grid, kSplitThreads, 0, stream>>>(p, phase, seg_stats, row_stats, counters);
    int st = launch_status();
    if (st != FDL_OK) return st;
    rows_split_apply_kernel<Op, MASKED><<<grid, kSplitThreads, 0, stream>>>(p, phase, row_stats);
    return launch_status();
}

// ---- plain fallback: one CTA per row, three passes ---------------------------------------

constexpr int kPlainThreads = 256;

template <class Op>
__global__ void __launch_bounds__(kPlainThreads) rows_plain_kernel(const RowParams p) {
    __shared__ float red[kMaxWarps];
    constexpr bool kSoftmax = std::is_same<Op, SoftmaxOp>::value;
    constexpr int T = kPlainThreads;
    constexpr float kLog2e = 1.4426950408889634f;
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const float* xr = p.x + row * p.cols;
        float* yr = p.y + row * p.cols;
        if (kSoftmax) {
            float m = -INFINITY;
            for (int c = threadIdx.x; c < p.cols; c += T) m = fmaxf(m, xr[c]);
            m = team_max<T, T>(m, red);
            float s = 0.0f;
            for (int c = threadIdx.x; c < p.cols; c += T) s += fast_exp2((xr[c] - m) * kLog2e);
            s = team_sum<T, T>(s, red);
            const float norm = 1.0f / s;
            for (int c = threadIdx.x; c < p.cols; c += T) {
                yr[c] = fast_exp2((xr[c] - m) * kLog2e) * norm;
            }
        } else {
            float s = 0.0f;
            for (int c = threadIdx.x; c < p.cols; c += T) s += xr[c];
            const float inv_n = 1.0f / static_cast<float>(p.cols);
            const float mean = team_sum<T, T>(s, red) * inv_n;
            float q = 0.0f;
            for (int c = threadIdx.x; c < p.cols; c += T) {
                const float d = xr[c] - mean;
                q += d * d;
            }
            const float var = team_sum<T, T>(q, red) * inv_n;
            const float rstd = 1.0f / sqrtf(var + p.eps);
            if (threadIdx.x == 0) {
                if (p.mean_out != nullptr) p.mean_out[row] = mean;
                if (p.rstd_out != nullptr) p.rstd_out[row] = rstd;
            }
            for (int c = threadIdx.x; c < p.cols; c += T) {
                float o = (xr[c] - mean) * rstd;
                if (p.gamma != nullptr) o *= p.gamma[c];
                if (p.beta != nullptr) o += p.beta[c];
                yr[c] = o;
            }
        }
    }
}

// ---- host side -------------------------------------------------------------------------------

template <class Op, int TPR, int TH, int NV>
int launch_direct_cfg(const RowParams& p, const DeviceInfo*, cudaStream_t stream) {
    constexpr int kTeams = TH / TPR;
    const int64_t grid = ceil_div(p.rows, kTeams);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    return launch_ex(rows_direct_kernel<Op, TPR, TH, NV>, dim3(static_cast<unsigned int>(grid)), dim3(TH), 0, stream,
                     dim3(1, 1, 1), tuning().pdl != 0, p);
}

template <class Op, int TPR, int TH, int NV>
int launch_staged_cfg(const RowParams& p, const DeviceInfo* info, cudaStream_t stream) {
    constexpr int kTeams = TH / TPR;
    RowParams q = p;
    const size_t row_bytes = static_cast<size_t>(p.cols) * sizeof(float);
    // Short rows: each team takes several consecutive rows so that a CTA's one bulk copy
    // moves about 32 KiB.
    int rpt = 1;
    if (kTeams * row_bytes < 32768) rpt = static_cast<int>(32768 / (kTeams * row_bytes));
    if (rpt > 64) rpt = 64;
    q.rows_per_team = rpt;
    const size_t smem = static_cast<size_t>(kTeams) * rpt * row_bytes;
    if (smem + 1024 > static_cast<size_t>(info->max_smem_optin)) return FDL_ERR_UNSUPPORTED;
    auto kernel = rows_staged_kernel<Op, TPR, TH, NV>;
    // The attribute belongs to the device, so what has been configured is kept per device.
    static size_t configured_smem[kMaxDevicesTracked] = {};
    size_t& configured = configured_smem[info->device % kMaxDevicesTracked];
    if (smem > 48 * 1024 - 256 && smem > configured) {
        // Exactly what is needed: the opt-in ceiling covers static + dynamic together.
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = smem;
    }
    const int64_t grid = ceil_div(p.rows, static_cast<int64_t>(kTeams) * rpt);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    kernel<<<static_cast<unsigned int>(grid), TH, smem, stream>>>(q);
    return launch_status();
}

// Rows of 257..512 packs: a 256-thread CTA per row leaves every thread one or two packs and
// two CTA-wide barriers per statistic, which is slow at the low end of the range ([65536,1028]:
// 69-76% of the copy bandwidth); a warp per row with up to 16 packs a lane measures 87-89%
// there.  Layernorm is ahead with the warp form over the whole range (104% at 1536 and 2048
// floats), softmax -- a warp then evaluates up to 2048 exponentials -- only up to 320 packs.
template <class Op>
bool warp_takes_16_packs(int nvec) {
    const int mode = tuning().rows_warp16;  // -1: by measurement (default), 0: never, 1: always
    if (mode >= 0) return mode == 1;
    return std::is_same<Op, LayerNormOp>::value || nvec <= 320;
}

// Picks the team size and the registers-per-thread bucket for a row length.  The buckets of nine
// packs a thread sit just above the powers of two: a row of 1023 or 8191 floats at an odd phase
// covers 257 or 2049 packs, one more than the eight-pack bucket holds, and would otherwise
// land in a bucket of twice the registers (76-82% and 73-76% of the copy bandwidth).
#define FDL_ROW_DISPATCH(LAUNCH) FDL_ROW_DISPATCH_N(LAUNCH, p.cols / 4)
#define FDL_ROW_DISPATCH_N(LAUNCH, NVEC)                                                 \
    do {                                                                                 \
        const int nvec_ = (NVEC);                                                        \
        if (nvec_ <= 8) return LAUNCH<Op, 8, 256, 1>(p, info, stream);                   \
        if (nvec_ <= 16) return LAUNCH<Op, 16, 256, 1>(p, info, stream);                 \
        if (nvec_ <= 32) return LAUNCH<Op, 32, 256, 1>(p, info, stream);                 \
        if (nvec_ <= 64) return LAUNCH<Op, 32, 256, 2>(p, info, stream);                 \
        if (nvec_ <= 128) return LAUNCH<Op, 32, 256, 4>(p, info, stream);                \
        if (nvec_ <= 256) return LAUNCH<Op, 32, 256, 8>(p, info, stream);                \
        if (nvec_ <= 288) return LAUNCH<Op, 32, 256, 9>(p, info, stream);                \
        if (nvec_ <= 512 && warp_takes_16_packs<Op>(nvec_)) return LAUNCH<Op, 32, 256, 16>(p, info, stream); \
        if (nvec_ <= 512) return LAUNCH<Op, 256, 256, 2>(p, info, stream);               \
        if (nvec_ <= 1024) return LAUNCH<Op, 256, 256, 4>(p, info, stream);              \
        if (nvec_ <= 2048) return LAUNCH<Op, 256, 256, 8>(p, info, stream);              \
        if (nvec_ <= 2304) return LAUNCH<Op, 256, 256, 9>(p, info, stream);              \
        return LAUNCH<Op, 512, 512, 8>(p, info, stream);                                 \
    } while (0)

constexpr int64_t kStagedAutoMaxCols = 128;

template <class Op>
int dispatch_rows_staged(const RowParams& p, const DeviceInfo* info, cudaStream_t stream) {
    FDL_ROW_DISPATCH(launch_staged_cfg);
}

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

    const bool packs = p.cols % 4 == 0 && aligned16(p.x) && aligned16(p.y) &&
                       (p.gamma == nullptr || aligned16(p.gamma)) &&
                       (p.beta == nullptr || aligned16(p.beta));
    constexpr int kCtaMaxCols = kClusterThreads * kClusterNV * 4;  // 16384 floats in one CTA's registers
    const bool same_phase = ((reinterpret_cast<uintptr_t>(p.x) ^ reinterpret_cast<uintptr_t>(p.y)) & 15u) == 0;
    // Rows beyond 65536 floats (beyond 16384 when they do not consist of whole aligned packs):
    // the row in a cluster's shared memory, read once.
    if (tuning().rows_split_from > 0 && p.cols >= tuning().rows_split_from && same_phase && p.rows < kSplitMaxRows) {
        return packs ? launch_rows_split<Op, false>(p, stream) : launch_rows_split<Op, true>(p, stream);
    }
    const int smem_from = tuning().rows_smem_from > 0 ? tuning().rows_smem_from : 4 * kCtaMaxCols;
    if (tuning().rows_smem != 0 && same_phase && (packs ? p.cols > smem_from : p.cols + 6 > kCtaMaxCols)) {
        const int st = launch_rows_smem<Op>(p, info, stream);
        if (st != FDL_ERR_UNSUPPORTED) return st;
    }
    if (packs && p.cols > kCtaMaxCols && p.cols <= 8 * kCtaMaxCols) {
        if (tuning().rows_cluster_threads == 256 && p.cols <= 4 * kCtaMaxCols) {
            // 256-thread CTAs hold 8192 floats each: twice the CTAs per row, four resident per SM
            // (measured 86-91% against 79-86% with 512-thread CTAs; 128-thread CTAs add nothing)
            if (p.cols <= 2 * kCtaMaxCols) return launch_cluster_cfg<Op, 4, 256>(p, stream);
            return launch_cluster_cfg<Op, 8, 256>(p, stream);
        }
        if (p.cols <= 2 * kCtaMaxCols) return launch_cluster_cfg<Op, 2, 512>(p, stream);
        if (p.cols <= 4 * kCtaMaxCols) return launch_cluster_cfg<Op, 4, 512>(p, stream);
        return launch_cluster_cfg<Op, 8, 512>(p, stream);
    }
    if (packs && p.cols > 8 * kCtaMaxCols && p.rows <= kSplitMaxRows && p.rows <= 65535) {
        return launch_rows_split<Op, false>(p, stream);
    }
    // Rows at any phase of a 16-byte line (length not a multiple of 4, or a base that is not
    // 16-byte aligned): the masked form, as long as x and y share the phase and a row's packs
    // fit one CTA's registers.
    const int64_t packs_worst = (static_cast<int64_t>(p.cols) + 6) / 4;
    if (!packs && ((reinterpret_cast<uintptr_t>(p.x) ^ reinterpret_cast<uintptr_t>(p.y)) & 15u) == 0 &&
        packs_worst <= kCtaMaxCols / 4) {
        if (p.cols <= tuning().rows_span_cols) {
            const int st = launch_span<Op>(p, stream);
            if (st != FDL_ERR_UNSUPPORTED) return st;
        }
        if (packs_worst <= 8) return launch_masked_short_cfg<Op, 8>(p, stream);
        if (packs_worst <= 16) return launch_masked_short_cfg<Op, 16>(p, stream);
        if (packs_worst <= 32) return launch_masked_short_cfg<Op, 32>(p, stream);
        FDL_ROW_DISPATCH_N(launch_masked_cfg, static_cast<int>(packs_worst));
    }
    if (!packs && ((reinterpret_cast<uintptr_t>(p.x) ^ reinterpret_cast<uintptr_t>(p.y)) & 15u) == 0 &&
        p.rows <= kSplitMaxRows && p.rows <= 65535) {
        return launch_rows_split<Op, true>(p, stream);  // longer rows at any phase: the two-kernel form
    }
    const bool in_registers = packs && p.cols <= kCtaMaxCols;
    if (in_registers) {
        // -1 (default): staged for rows of up to 128 floats, where a thread of the direct
        // form has a single load in flight (measured 97-98% of the copy bandwidth staged
        // against 76-90% direct; from 256 floats on the direct form leads, 104-107%).
        const int mode = tuning().rows_staged;
        if (mode == 1 || (mode < 0 && p.cols <= kStagedAutoMaxCols)) {
            const int staged = dispatch_rows_staged<Op>(p, info, stream);
            if (staged != FDL_ERR_UNSUPPORTED || mode == 1) return staged;
        }
        FDL_ROW_DISPATCH(launch_direct_cfg);
    }
    int64_t grid = p.rows;
    if (grid > 2147483647) grid = 2147483647;
    rows_plain_kernel<Op><<<static_cast<unsigned int>(grid), kPlainThreads, 0, stream>>>(p);
    return launch_status();
}

}  // namespace

}  // namespace fdl

using namespace fdl;

extern "C" {

int fdl_softmax_rows_f32(const float* x, float* y, int64_t rows, int64_t cols, void* stream) {
    if (cols >= INT_MAX - 16384) return FDL_ERR_UNSUPPORTED;  // pack and segment arithmetic on a row stays inside int
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
    if (cols >= INT_MAX - 16384) return FDL_ERR_UNSUPPORTED;  // pack and segment arithmetic on a row stays inside int
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

int fdl_debug_split_ticket(int64_t rows, int64_t segments, int64_t lag, unsigned int ticket, int64_t* row, int* segment,
                           int* is_apply) {
    if (rows < 1 || segments < 1 || lag < 1 || lag > rows || row == nullptr || segment == nullptr || is_apply == nullptr)
        return FDL_ERR_INVALID_ARGUMENT;
    if (2 * rows * segments > 2147483647 || rows >= kSplitMaxRows) return FDL_ERR_UNSUPPORTED;
    if (ticket >= 2 * rows * segments) return FDL_ERR_INVALID_ARGUMENT;
    const SplitTask task = split_decode(make_split_plan(rows, segments, lag), ticket);
    *row = task.row;
    *segment = task.seg;
    *is_apply = task.apply ? 1 : 0;
    return FDL_OK;
}

}  // extern "C"
