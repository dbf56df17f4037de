// Elementwise, fused-chain and broadcast-binary kernels (fp32, HBM-bound).
//
// One streaming template serves every same-shape op.  Each CTA owns ONE tile (256 threads x
// kEwUnroll 128-bit packs per operand) and the hardware block scheduler hands tiles to SMs
// as they free up.  Measured on B200 this beats a persistent grid-stride grid sized to the
// SM count by ~10% (7.0 vs 6.4 TB/s on a 2^28-element add): the two dies do not reach HBM
// equally fast, and a static split finishes with its slowest SM.  Loads and stores carry
// the evict-first hint because every byte is touched once.
//
// The broadcast kernel uses the same tile walk over the OUTPUT and turns each linear
// index into operand offsets with multiply-high "fast division" constants that the host
// derives from the collapsed shape, so the device never executes an integer divide
// (the reference's row-bias kernel pays one `%` per element, src/kernels/cuda/bias.cu:10).
// When the extents are not multiples of 4 but one operand has the output's own layout, a
// second broadcast kernel walks that operand and the output as aligned packs of their flat
// buffers and indexes only the other operand per element.
#include "fdl_common.cuh"

namespace fdl {

namespace {

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;
constexpr int kMaxOuterDims = 7;

// ---- packs: W consecutive floats moved with one instruction ------------------------------

template <int W>
struct Pack {
    float v[W];
};

template <int W>
__device__ __forceinline__ Pack<W> load_pack(const float* base, int64_t pack_index);

template <>
__device__ __forceinline__ Pack<4> load_pack<4>(const float* base, int64_t i) {
    const float4 t = ld_stream(reinterpret_cast<const float4*>(base) + i);
    return Pack<4>{{t.x, t.y, t.z, t.w}};
}

template <>
__device__ __forceinline__ Pack<1> load_pack<1>(const float* base, int64_t i) {
    return Pack<1>{{ld_stream(base + i)}};
}

template <int W>
__device__ __forceinline__ void store_pack(float* base, int64_t pack_index, const Pack<W>& p);

template <>
__device__ __forceinline__ void store_pack<4>(float* base, int64_t i, const Pack<4>& p) {
    st_stream(reinterpret_cast<float4*>(base) + i, make_float4(p.v[0], p.v[1], p.v[2], p.v[3]));
}

template <>
__device__ __forceinline__ void store_pack<1>(float* base, int64_t i, const Pack<1>& p) {
    st_stream(base + i, p.v[0]);
}

template <int W>
__device__ __forceinline__ Pack<W> splat(float s) {
    Pack<W> p;
#pragma unroll
    for (int k = 0; k < W; ++k) p.v[k] = s;
    return p;
}

// ---- scalar functors.  Explicit _rn intrinsics keep nvcc from contracting a*b+c. ---------

struct AddFn {
    __device__ __forceinline__ float operator()(float a, float b, float) const {
        return __fadd_rn(a, b);
    }
};
struct SubFn {
    __device__ __forceinline__ float operator()(float a, float b, float) const {
        return __fsub_rn(a, b);
    }
};
struct MulFn {
    __device__ __forceinline__ float operator()(float a, float b, float) const {
        return __fmul_rn(a, b);
    }
};
struct DivFn {
    __device__ __forceinline__ float operator()(float a, float b, float) const {
        return __fdiv_rn(a, b);
    }
};
struct AddReluFn {
    __device__ __forceinline__ float operator()(float a, float b, float) const {
        return fmaxf(0.0f, __fadd_rn(a, b));
    }
};
struct MulAddReluFn {
    __device__ __forceinline__ float operator()(float a, float b, float c) const {
        return fmaxf(0.0f, __fadd_rn(__fmul_rn(a, b), c));
    }
};
struct ReluFn {
    __device__ __forceinline__ float operator()(float x, float, float) const {
        return fmaxf(0.0f, x);
    }
};
struct LeakyReluFn {
    float alpha;
    __device__ __forceinline__ float operator()(float x, float, float) const {
        return x > 0.0f ? x : __fmul_rn(alpha, x);
    }
};
// Same expression shape as the reference kernel (src/kernels/cuda/activation.cu:45-51),
// compiled with the same default contraction, so the bits match its GPU output.
struct GeluFn {
    __device__ __forceinline__ float operator()(float x, float, float) const {
        return 0.5f * x * (1.0f + tanhf(0.79788456f * (x + 0.044715f * x * x * x)));
    }
};
struct SigmoidFn {
    __device__ __forceinline__ float operator()(float x, float, float) const {
        return 1.0f / (1.0f + expf(-x));
    }
};
struct TanhFn {
    __device__ __forceinline__ float operator()(float x, float, float) const { return tanhf(x); }
};

template <int W, class F>
__device__ __forceinline__ Pack<W> apply(const F& f, const Pack<W>& a, const Pack<W>& b,
                                         const Pack<W>& c) {
    Pack<W> r;
#pragma unroll
    for (int k = 0; k < W; ++k) r.v[k] = f(a.v[k], b.v[k], c.v[k]);
    return r;
}

// ---- same-shape streaming map --------------------------------------------------------------

template <int W, int NIN, int kEwUnroll, class F>
__global__ void __launch_bounds__(kEwThreads)
map_kernel(F f, const float* in0, const float* in1, const float* in2, float* out, int64_t npack,
           int64_t n) {
    constexpr int64_t kTile = static_cast<int64_t>(kEwThreads) * kEwUnroll;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile + threadIdx.x;
    pdl_wait();  // the operands may be the previous kernel's output
    if (base + (kEwUnroll - 1) * kEwThreads < npack) {
        // Full tile (all CTAs but possibly the last): every load is issued before any use.
        Pack<W> x0[kEwUnroll], x1[kEwUnroll], x2[kEwUnroll];
#pragma unroll
        for (int u = 0; u < kEwUnroll; ++u) {
            const int64_t i = base + u * kEwThreads;
            x0[u] = load_pack<W>(in0, i);
            if (NIN > 1) x1[u] = load_pack<W>(in1, i);
            if (NIN > 2) x2[u] = load_pack<W>(in2, i);
        }
        pdl_trigger();  // loads are in flight: the next kernel of the stream may be scheduled
#pragma unroll
        for (int u = 0; u < kEwUnroll; ++u) {
            const int64_t i = base + u * kEwThreads;
            if (NIN < 2) x1[u] = x0[u];
            if (NIN < 3) x2[u] = x0[u];
            store_pack<W>(out, i, apply<W>(f, x0[u], x1[u], x2[u]));
        }
    } else {
#pragma unroll
        for (int u = 0; u < kEwUnroll; ++u) {
            const int64_t i = base + u * kEwThreads;
            if (i < npack) {
                Pack<W> a = load_pack<W>(in0, i);
                Pack<W> b = NIN > 1 ? load_pack<W>(in1, i) : a;
                Pack<W> c = NIN > 2 ? load_pack<W>(in2, i) : a;
                store_pack<W>(out, i, apply<W>(f, a, b, c));
            }
        }
    }
    // The last CTA also owns the n % W scalar tail.
    if (W > 1 && blockIdx.x == gridDim.x - 1) {
        for (int64_t i = npack * W + threadIdx.x; i < n; i += kEwThreads) {
            const float a = in0[i];
            const float b = NIN > 1 ? in1[i] : a;
            const float c = NIN > 2 ? in2[i] : a;
            out[i] = f(a, b, c);
        }
    }
}

constexpr int64_t kMaxGrid = 2147483647;  // gridDim.x limit

template <int W, int NIN, int U, class F>
int launch_map_wu(const F& f, const float* in0, const float* in1, const float* in2, float* out,
                  int64_t n, cudaStream_t stream) {
    constexpr int64_t kTile = static_cast<int64_t>(kEwThreads) * U;
    // One launch covers up to 2^31-1 tiles; longer tensors are cut into slabs.
    const int64_t slab_elems = (kMaxGrid - 1) * kTile * W;
    for (int64_t off = 0; off < n; off += slab_elems) {
        const int64_t m = n - off < slab_elems ? n - off : slab_elems;
        const int64_t npack = m / W;
        int64_t tiles = ceil_div(npack, kTile);
        if (tiles < 1) tiles = 1;
        const int st = launch_ex(map_kernel<W, NIN, U, F>, dim3(static_cast<unsigned int>(tiles)), dim3(kEwThreads),
                                 0, stream, dim3(1, 1, 1), tuning().pdl != 0, f, in0 + off,
                                 NIN > 1 ? in1 + off : nullptr, NIN > 2 ? in2 + off : nullptr, out + off, npack, m);
        if (st != FDL_OK) return st;
    }
    return FDL_OK;
}

template <int W, int NIN, class F>
int launch_map_w(const F& f, const float* in0, const float* in1, const float* in2, float* out,
                 int64_t n, cudaStream_t stream) {
    // Small tensors get one pack per thread so that there are enough CTAs for every SM.
    constexpr int64_t kSmall = int64_t{1} << 22;
    return n < kSmall ? launch_map_wu<W, NIN, 1, F>(f, in0, in1, in2, out, n, stream)
                      : launch_map_wu<W, NIN, kEwUnroll, F>(f, in0, in1, in2, out, n, stream);
}

template <int NIN, class F>
int launch_map(const F& f, const float* in0, const float* in1, const float* in2, float* out,
               int64_t n, cudaStream_t stream) {
    if (n == 0) return FDL_OK;
    const bool vec = aligned16(in0) && aligned16(out) && (NIN < 2 || aligned16(in1)) &&
                     (NIN < 3 || aligned16(in2));
    return vec ? launch_map_w<4, NIN, F>(f, in0, in1, in2, out, n, stream)
               : launch_map_w<1, NIN, F>(f, in0, in1, in2, out, n, stream);
}

// ---- broadcast binary ------------------------------------------------------------------------

// q = n / d for 0 <= n < 2^31 without a divide: q = (mulhi(n, magic) + n) >> shift.
struct FastDiv {
    uint32_t d;
    uint32_t magic;
    uint32_t shift;
};

FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    f.d = d;
    uint32_t shift = 0;
    while ((uint64_t{1} << shift) < d) ++shift;
    f.shift = shift;
    f.magic = static_cast<uint32_t>((((uint64_t{1} << shift) - d) << 32) / d + 1);
    return f;
}

__device__ __forceinline__ uint32_t fast_divide(uint32_t n, const FastDiv& f) {
    return (__umulhi(n, f.magic) + n) >> f.shift;
}

// Host-precomputed description of one broadcast launch.  The innermost collapsed
// dimension is walked in packs of W floats; the remaining ("outer") dimensions are
// peeled innermost-first with fast division.  Strides are in elements; 0 = broadcast.
struct BroadcastPlan {
    FastDiv inner_div;  // by the number of packs in the innermost dimension
    int nouter;
    FastDiv outer_div[kMaxOuterDims];
    int64_t a_outer[kMaxOuterDims];
    int64_t b_outer[kMaxOuterDims];
    int64_t a_inner;  // element stride of a along the innermost dimension
    int64_t b_inner;
    uint32_t total_packs;
};

template <int W>
__device__ __forceinline__ Pack<W> load_operand(const float* base, int64_t offset,
                                                int64_t inner_stride) {
    if (W == 1) return Pack<W>{{ld_stream(base + offset)}};
    // W == 4: the host guarantees inner_stride is 1 (vector load) or 0 (splat).
    if (inner_stride != 0) return load_pack<W>(base + offset, 0);
    // A value shared by the whole pack is re-read by many threads: default caching.
    return splat<W>(base[offset]);
}

template <int W>
__device__ __forceinline__ void decompose(const BroadcastPlan& plan, uint32_t item,
                                          int64_t* a_off, int64_t* b_off) {
    uint32_t outer = fast_divide(item, plan.inner_div);
    const uint32_t ip = item - outer * plan.inner_div.d;
    int64_t ao = static_cast<int64_t>(ip) * W * plan.a_inner;
    int64_t bo = static_cast<int64_t>(ip) * W * plan.b_inner;
#pragma unroll
    for (int k = 0; k < kMaxOuterDims; ++k) {
        if (k < plan.nouter) {
            uint32_t idx = outer;
            if (k + 1 < plan.nouter) {
                const uint32_t q = fast_divide(outer, plan.outer_div[k]);
                idx = outer - q * plan.outer_div[k].d;
                outer = q;
            }
            ao += static_cast<int64_t>(idx) * plan.a_outer[k];
            bo += static_cast<int64_t>(idx) * plan.b_outer[k];
        }
    }
    *a_off = ao;
    *b_off = bo;
}

template <int W, class F>
__global__ void __launch_bounds__(kEwThreads)
broadcast_kernel(F f, const __grid_constant__ BroadcastPlan plan, const float* a, const float* b,
                 float* out) {
    constexpr uint32_t kTile = kEwThreads * kEwUnroll;
    const uint32_t total = plan.total_packs;
    const uint32_t base = blockIdx.x * kTile + threadIdx.x;
    Pack<W> xa[kEwUnroll], xb[kEwUnroll];
    pdl_wait();
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
        const uint32_t item = base + u * kEwThreads;
        if (item < total) {
            int64_t ao, bo;
            decompose<W>(plan, item, &ao, &bo);
            xa[u] = load_operand<W>(a, ao, plan.a_inner);
            xb[u] = load_operand<W>(b, bo, plan.b_inner);
        }
    }
    pdl_trigger();
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
        const uint32_t item = base + u * kEwThreads;
        if (item < total) store_pack<W>(out, item, apply<W>(f, xa[u], xb[u], xa[u]));
    }
}

// ---- two collapsed dimensions: no index arithmetic at all -----------------------------------------
//
// [R, C] against [1, C], [R, 1] or another [R, C] with its own row stride -- the bias row, the
// per-row scale, the view of a wider matrix.  Threads are laid out TX across the packs of a
// row and 256 / TX down the rows; a thread walks ROWS rows at one pack position, so a row
// vector's pack is loaded once per thread and a column vector's value once per row, both
// through the read-only path (they are re-read by every CTA), while the dense operand and
// the output stream past with evict-first accesses.  Consecutive CTAs take consecutive column
// tiles of the same rows.  Operand kinds: 0 = one 128-bit load per row (inner stride 1, any
// row stride that keeps 16-byte alignment), 1 = a row vector (inner stride 1, row stride 0),
// 2 = one value per row (inner stride 0).
template <class F, int KA, int KB, int ROWS>
__global__ void __launch_bounds__(kEwThreads)
broadcast2d_kernel(F f, const float* a, const float* b, float* out, int64_t rows, int64_t cpacks,
                   int64_t a_rs, int64_t b_rs, int tx_shift, uint32_t col_tiles) {
    const int tx = 1 << tx_shift;
    const int ty = kEwThreads >> tx_shift;
    const int cx = threadIdx.x & (tx - 1);
    const int ry = threadIdx.x >> tx_shift;
    const uint32_t row_group = blockIdx.x / col_tiles;
    const uint32_t col_tile = blockIdx.x - row_group * col_tiles;
    const int64_t cp = static_cast<int64_t>(col_tile) * tx + cx;
    const int64_t r0 = static_cast<int64_t>(row_group) * (ty * ROWS) + ry;
    pdl_wait();
    if (cp >= cpacks) return;
    Pack<4> xa[ROWS], xb[ROWS];
    if (KA == 1) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(a) + cp);
        xa[0] = Pack<4>{{t.x, t.y, t.z, t.w}};
    }
    if (KB == 1) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(b) + cp);
        xb[0] = Pack<4>{{t.x, t.y, t.z, t.w}};
    }
#pragma unroll
    for (int u = 0; u < ROWS; ++u) {
        const int64_t r = r0 + u * ty;
        if (r < rows) {
            if (KA == 0) xa[u] = load_pack<4>(a + r * a_rs, cp);
            if (KA == 1) xa[u] = xa[0];
            if (KA == 2) xa[u] = splat<4>(__ldg(a + r * a_rs));
            if (KB == 0) xb[u] = load_pack<4>(b + r * b_rs, cp);
            if (KB == 1) xb[u] = xb[0];
            if (KB == 2) xb[u] = splat<4>(__ldg(b + r * b_rs));
        }
    }
    pdl_trigger();
#pragma unroll
    for (int u = 0; u < ROWS; ++u) {
        const int64_t r = r0 + u * ty;
        if (r < rows) store_pack<4>(out + r * cpacks * 4, cp, apply<4>(f, xa[u], xb[u], xa[u]));
    }
}

inline int operand_kind(int64_t row_stride, int64_t inner_stride) {
    return inner_stride == 0 ? 2 : (row_stride == 0 ? 1 : 0);
}

template <class F, int ROWS>
int launch_broadcast2d_rows(const F& f, const float* a, const float* b, float* out, int64_t rows, int64_t cols,
                            int64_t a_rs, int64_t a_cs, int64_t b_rs, int64_t b_cs, cudaStream_t stream) {
    const int64_t cpacks = cols / 4;
    int tx_shift = 0;
    while ((1 << tx_shift) < kEwThreads && (int64_t{1} << tx_shift) < cpacks) ++tx_shift;
    const int tx = 1 << tx_shift, ty = kEwThreads >> tx_shift;
    const int64_t col_tiles = ceil_div(cpacks, tx);
    const int64_t row_groups = ceil_div(rows, static_cast<int64_t>(ty) * ROWS);
    if (col_tiles * row_groups > kMaxGrid) return FDL_ERR_UNSUPPORTED;
    const dim3 grid(static_cast<unsigned int>(col_tiles * row_groups)), block(kEwThreads), one(1, 1, 1);
    const bool pdl = tuning().pdl != 0;
    const uint32_t ct = static_cast<uint32_t>(col_tiles);
#define FDL_B2D(KA, KB) \
    return launch_ex(broadcast2d_kernel<F, KA, KB, ROWS>, grid, block, 0, stream, one, pdl, f, a, b, out, rows, cpacks, \
                     a_rs, b_rs, tx_shift, ct)
    switch (operand_kind(a_rs, a_cs) * 3 + operand_kind(b_rs, b_cs)) {
        case 0: FDL_B2D(0, 0);
        case 1: FDL_B2D(0, 1);
        case 2: FDL_B2D(0, 2);
        case 3: FDL_B2D(1, 0);
        case 4: FDL_B2D(1, 1);
        case 5: FDL_B2D(1, 2);
        case 6: FDL_B2D(2, 0);
        case 7: FDL_B2D(2, 1);
        default: FDL_B2D(2, 2);
    }
#undef FDL_B2D
}

template <class F>
int launch_broadcast2d(const F& f, const float* a, const float* b, float* out, int64_t rows, int64_t cols,
                       int64_t a_rs, int64_t a_cs, int64_t b_rs, int64_t b_cs, cudaStream_t stream) {
    // Rows per thread: four 128-bit loads in flight per dense operand once the tensor is large
    // enough to fill every SM several times over, fewer below so that the last wave stays short.
    int rows_per_thread = tuning().bcast2d_rows;
    if (rows_per_thread == 0) rows_per_thread = rows * cols < (int64_t{1} << 22) ? 1 : 4;
    switch (rows_per_thread) {
        case 1: return launch_broadcast2d_rows<F, 1>(f, a, b, out, rows, cols, a_rs, a_cs, b_rs, b_cs, stream);
        case 2: return launch_broadcast2d_rows<F, 2>(f, a, b, out, rows, cols, a_rs, a_cs, b_rs, b_cs, stream);
        default: return launch_broadcast2d_rows<F, 4>(f, a, b, out, rows, cols, a_rs, a_cs, b_rs, b_cs, stream);
    }
}

// ---- dense operand at a row length that is not a multiple of 4 ------------------------------------
//
// When one operand has the output's own (contiguous) layout, it and the output can be walked
// as aligned 128-bit packs of the FLAT buffer whatever the extents are; only the other,
// broadcast operand needs an index per element.  The plan is in elements (W = 1).  A pack
// that stays inside one innermost run takes one decomposition (the common case: 4 / extent
// of the packs cross a run boundary); one that crosses takes four.  The broadcast operand's
// floats come through the default cache path: they are re-read by many packs.
template <class F, bool DENSE_IS_A>
__global__ void __launch_bounds__(kEwThreads)
broadcast_flat_kernel(F f, const __grid_constant__ BroadcastPlan plan, const float* dense,
                      const float* other, float* out, uint32_t n) {
    constexpr uint32_t kTile = kEwThreads * kEwUnroll;
    const uint32_t full = n >> 2;
    const uint32_t base = blockIdx.x * kTile + threadIdx.x;
    const int64_t other_inner = DENSE_IS_A ? plan.b_inner : plan.a_inner;
    Pack<4> xd[kEwUnroll], xo[kEwUnroll];
    pdl_wait();
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
        const uint32_t item = base + u * kEwThreads;
        if (item < full) {
            xd[u] = load_pack<4>(dense, item);
            const uint32_t e = item * 4;
            int64_t ao, bo;
            decompose<1>(plan, e, &ao, &bo);
            const int64_t o0 = DENSE_IS_A ? bo : ao;
            const uint32_t run = fast_divide(e, plan.inner_div);
            const uint32_t in_run = e - run * plan.inner_div.d;
            if (in_run + 3 < plan.inner_div.d) {
                if (other_inner == 0) {
                    const float v = other[o0];
                    xo[u] = Pack<4>{{v, v, v, v}};
                } else {
                    xo[u] = Pack<4>{{other[o0], other[o0 + other_inner], other[o0 + 2 * other_inner],
                                    other[o0 + 3 * other_inner]}};
                }
            } else if (plan.inner_div.d >= 4) {
                // One run boundary inside the pack: a second decomposition for the first
                // element behind it, the rest by the inner stride again.
                const uint32_t before = plan.inner_div.d - in_run;  // 1..3 elements of this run
                decompose<1>(plan, e + before, &ao, &bo);
                const int64_t o1 = DENSE_IS_A ? bo : ao;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int64_t off = static_cast<uint32_t>(k) < before
                                            ? o0 + k * other_inner
                                            : o1 + (k - static_cast<int>(before)) * other_inner;
                    xo[u].v[k] = other[off];
                }
            } else {
                xo[u].v[0] = other[o0];
#pragma unroll
                for (int k = 1; k < 4; ++k) {
                    decompose<1>(plan, e + k, &ao, &bo);
                    xo[u].v[k] = other[DENSE_IS_A ? bo : ao];
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
        const uint32_t item = base + u * kEwThreads;
        if (item < full) {
            store_pack<4>(out, item, DENSE_IS_A ? apply<4>(f, xd[u], xo[u], xd[u]) : apply<4>(f, xo[u], xd[u], xd[u]));
        }
    }
    // the last n % 4 elements, one thread
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
        for (uint32_t e = full * 4; e < n; ++e) {
            int64_t ao, bo;
            decompose<1>(plan, e, &ao, &bo);
            const Pack<1> d{{dense[e]}};
            const Pack<1> o{{other[DENSE_IS_A ? bo : ao]}};
            out[e] = (DENSE_IS_A ? apply<1>(f, d, o, d) : apply<1>(f, o, d, d)).v[0];
        }
    }
}

template <class F>
int launch_broadcast_flat(const F& f, const BroadcastPlan& plan, bool dense_is_a, const float* dense,
                          const float* other, float* out, uint32_t n, cudaStream_t stream) {
    int64_t tiles = ceil_div(static_cast<int64_t>(n >> 2), static_cast<int64_t>(kEwThreads) * kEwUnroll);
    if (tiles < 1) tiles = 1;
    const dim3 grid(static_cast<unsigned int>(tiles)), block(kEwThreads), one(1, 1, 1);
    const bool pdl = tuning().pdl != 0;
    return dense_is_a ? launch_ex(broadcast_flat_kernel<F, true>, grid, block, 0, stream, one, pdl, f, plan, dense, other, out, n)
                      : launch_ex(broadcast_flat_kernel<F, false>, grid, block, 0, stream, one, pdl, f, plan, dense, other, out, n);
}

template <int W, class F>
int launch_broadcast_w(const F& f, const BroadcastPlan& plan, const float* a, const float* b,
                       float* out, cudaStream_t stream) {
    const int64_t tiles = ceil_div(plan.total_packs, kEwThreads * kEwUnroll);
    return launch_ex(broadcast_kernel<W, F>, dim3(static_cast<unsigned int>(tiles)), dim3(kEwThreads), 0, stream,
                     dim3(1, 1, 1), tuning().pdl != 0, f, plan, a, b, out);
}

struct Dim {
    int64_t size;
    int64_t a;
    int64_t b;
};

// Drops size-1 dimensions and merges neighbours that both operands walk contiguously
// (or both broadcast), so [R, C] + [R, C] becomes 1-D and [N, R, C] + [1, 1, C] becomes 2-D.
int collapse_dims(int ndim, const int64_t* shape, const int64_t* a_strides,
                  const int64_t* b_strides, Dim* dims) {
    int nd = 0;
    for (int i = 0; i < ndim; ++i) {
        if (shape[i] == 1) continue;
        Dim d{shape[i], a_strides[i], b_strides[i]};
        if (nd > 0) {
            Dim& prev = dims[nd - 1];
            if (prev.a == d.a * d.size && prev.b == d.b * d.size) {
                prev.size *= d.size;
                prev.a = d.a;
                prev.b = d.b;
                continue;
            }
        }
        dims[nd++] = d;
    }
    if (nd == 0) {
        dims[0] = Dim{1, 0, 0};
        nd = 1;
    }
    return nd;
}

template <class F>
int run_broadcast(const F& f, const float* a, const float* b, float* out, int ndim,
                  const int64_t* shape, const int64_t* a_strides, const int64_t* b_strides,
                  cudaStream_t stream) {
    if (a == nullptr || b == nullptr || out == nullptr || shape == nullptr ||
        a_strides == nullptr || b_strides == nullptr || ndim < 1 || ndim > 8) {
        return FDL_ERR_INVALID_ARGUMENT;
    }
    int64_t total = 1;
    for (int i = 0; i < ndim; ++i) {
        if (shape[i] < 0 || a_strides[i] < 0 || b_strides[i] < 0) return FDL_ERR_INVALID_ARGUMENT;
        total *= shape[i];
    }
    if (total == 0) return FDL_OK;

    Dim dims[8];
    const int nd = collapse_dims(ndim, shape, a_strides, b_strides, dims);
    const Dim inner = dims[nd - 1];

    // Fully contiguous operands: the plain streaming kernel does it with no index math.
    if (nd == 1 && inner.a == 1 && inner.b == 1) {
        return launch_map<2, F>(f, a, b, nullptr, out, total, stream);
    }

    // 128-bit path: innermost extent a multiple of 4, unit or zero inner strides, and
    // every vector-loaded operand keeps 16-byte alignment across the outer dimensions.
    bool vec = (inner.size % 4 == 0) && (inner.a == 0 || inner.a == 1) &&
               (inner.b == 0 || inner.b == 1) && aligned16(out) &&
               (inner.a == 0 || aligned16(a)) && (inner.b == 0 || aligned16(b));
    for (int i = 0; i + 1 < nd && vec; ++i) {
        if (inner.a == 1 && dims[i].a % 4 != 0) vec = false;
        if (inner.b == 1 && dims[i].b % 4 != 0) vec = false;
    }
    if (vec && nd == 2 && tuning().bcast2d != 0 && dims[0].size < (int64_t{1} << 31)) {
        const int st = launch_broadcast2d<F>(f, a, b, out, dims[0].size, inner.size, dims[0].a, inner.a, dims[0].b,
                                             inner.b, stream);
        if (st != FDL_ERR_UNSUPPORTED) return st;
    }
    const int w = vec ? 4 : 1;
    const int64_t inner_packs = inner.size / w;
    if (inner_packs >= (int64_t{1} << 31)) return FDL_ERR_UNSUPPORTED;

    // Outer dimensions, innermost first.
    BroadcastPlan plan{};
    plan.inner_div = make_fastdiv(static_cast<uint32_t>(inner_packs));
    plan.a_inner = inner.a;
    plan.b_inner = inner.b;
    plan.nouter = nd - 1;
    int64_t outer_rows_below_top = 1;  // product of outer dims except the outermost
    for (int k = 0; k < nd - 1; ++k) {
        const Dim& d = dims[nd - 2 - k];
        if (d.size >= (int64_t{1} << 31)) return FDL_ERR_UNSUPPORTED;
        plan.outer_div[k] = make_fastdiv(static_cast<uint32_t>(d.size));
        plan.a_outer[k] = d.a;
        plan.b_outer[k] = d.b;
        if (k + 1 < nd - 1) outer_rows_below_top *= d.size;
    }

    // The device index is 31-bit: walk the outermost dimension in slabs that fit.
    constexpr int64_t kMaxPacks = (int64_t{1} << 31) - 4096;  // base + tile stays inside 32 bits
    const int64_t packs_per_top = inner_packs * outer_rows_below_top;
    if (packs_per_top > kMaxPacks) return FDL_ERR_UNSUPPORTED;
    const int64_t top_size = nd >= 2 ? dims[0].size : 1;
    const int64_t top_a = nd >= 2 ? dims[0].a : 0;
    const int64_t top_b = nd >= 2 ? dims[0].b : 0;
    const int64_t slab = kMaxPacks / packs_per_top;
    // Not 128-bit-able dimension by dimension, but one operand has the output's own layout:
    // 128-bit packs over the flat buffers, the other operand indexed per element.
    if (!vec && top_size <= slab && total < (int64_t{1} << 31) && aligned16(out)) {
        bool a_dense = aligned16(a), b_dense = aligned16(b);
        int64_t expect = 1;
        for (int i = nd - 1; i >= 0; --i) {
            if (dims[i].a != expect) a_dense = false;
            if (dims[i].b != expect) b_dense = false;
            expect *= dims[i].size;
        }
        if (a_dense || b_dense) {
            plan.total_packs = static_cast<uint32_t>(total);
            return launch_broadcast_flat<F>(f, plan, a_dense, a_dense ? a : b, a_dense ? b : a, out,
                                            static_cast<uint32_t>(total), stream);
        }
    }
    for (int64_t start = 0; start < top_size; start += slab) {
        const int64_t count = top_size - start < slab ? top_size - start : slab;
        plan.total_packs = static_cast<uint32_t>(count * packs_per_top);
        const float* a_s = a + start * top_a;
        const float* b_s = b + start * top_b;
        float* out_s = out + start * packs_per_top * w;
        const int st = vec ? launch_broadcast_w<4, F>(f, plan, a_s, b_s, out_s, stream)
                           : launch_broadcast_w<1, F>(f, plan, a_s, b_s, out_s, stream);
        if (st != FDL_OK) return st;
    }
    return FDL_OK;
}

}  // namespace

}  // namespace fdl

using namespace fdl;

extern "C" {

int fdl_binary_f32(const float* a, const float* b, float* out, int64_t n, int op, void* stream) {
    if (n < 0 || (n > 0 && (a == nullptr || b == nullptr || out == nullptr))) {
        return FDL_ERR_INVALID_ARGUMENT;
    }
    cudaStream_t s = as_stream(stream);
    switch (op) {
        case FDL_ADD:
            return launch_map<2>(AddFn{}, a, b, nullptr, out, n, s);
        case FDL_SUB:
            return launch_map<2>(SubFn{}, a, b, nullptr, out, n, s);
        case FDL_MUL:
            return launch_map<2>(MulFn{}, a, b, nullptr, out, n, s);
        case FDL_DIV:
            return launch_map<2>(DivFn{}, a, b, nullptr, out, n, s);
        default:
            return FDL_ERR_INVALID_ARGUMENT;
    }
}

int fdl_unary_f32(const float* x, float* out, int64_t n, int op, float alpha, void* stream) {
    if (n < 0 || (n > 0 && (x == nullptr || out == nullptr))) return FDL_ERR_INVALID_ARGUMENT;
    cudaStream_t s = as_stream(stream);
    switch (op) {
        case FDL_RELU:
            return launch_map<1>(ReluFn{}, x, nullptr, nullptr, out, n, s);
        case FDL_LEAKY_RELU:
            return launch_map<1>(LeakyReluFn{alpha}, x, nullptr, nullptr, out, n, s);
        case FDL_GELU:
            return launch_map<1>(GeluFn{}, x, nullptr, nullptr, out, n, s);
        case FDL_SIGMOID:
            return launch_map<1>(SigmoidFn{}, x, nullptr, nullptr, out, n, s);
        case FDL_TANH:
            return launch_map<1>(TanhFn{}, x, nullptr, nullptr, out, n, s);
        default:
            return FDL_ERR_INVALID_ARGUMENT;
    }
}

int fdl_mul_add_relu_f32(const float* a, const float* b, const float* c, float* out, int64_t n,
                         void* stream) {
    if (n < 0 || (n > 0 && (a == nullptr || b == nullptr || c == nullptr || out == nullptr))) {
        return FDL_ERR_INVALID_ARGUMENT;
    }
    return launch_map<3>(MulAddReluFn{}, a, b, c, out, n, as_stream(stream));
}

int fdl_broadcast_binary_f32(const float* a, const float* b, float* out, int ndim,
                             const int64_t* shape, const int64_t* a_strides,
                             const int64_t* b_strides, int op, void* stream) {
    cudaStream_t s = as_stream(stream);
    switch (op) {
        case FDL_ADD:
            return run_broadcast(AddFn{}, a, b, out, ndim, shape, a_strides, b_strides, s);
        case FDL_SUB:
            return run_broadcast(SubFn{}, a, b, out, ndim, shape, a_strides, b_strides, s);
        case FDL_MUL:
            return run_broadcast(MulFn{}, a, b, out, ndim, shape, a_strides, b_strides, s);
        case FDL_DIV:
            return run_broadcast(DivFn{}, a, b, out, ndim, shape, a_strides, b_strides, s);
        default:
            return FDL_ERR_INVALID_ARGUMENT;
    }
}

int fdl_add_row_bias_f32(float* out, const float* bias, int64_t rows, int64_t cols,
                         void* stream) {
    if (rows < 0 || cols < 0) return FDL_ERR_INVALID_ARGUMENT;
    const int64_t shape[2] = {rows, cols};
    const int64_t a_strides[2] = {cols, 1};
    const int64_t b_strides[2] = {0, 1};
    return run_broadcast(AddFn{}, out, bias, out, 2, shape, a_strides, b_strides,
                         as_stream(stream));
}

int fdl_add_row_bias_relu_f32(float* out, const float* bias, int64_t rows, int64_t cols,
                              void* stream) {
    if (rows < 0 || cols < 0) return FDL_ERR_INVALID_ARGUMENT;
    const int64_t shape[2] = {rows, cols};
    const int64_t a_strides[2] = {cols, 1};
    const int64_t b_strides[2] = {0, 1};
    return run_broadcast(AddReluFn{}, out, bias, out, 2, shape, a_strides, b_strides,
                         as_stream(stream));
}

}  // extern "C"
