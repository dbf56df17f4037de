// Kernels on the edge of the bandwidth path that the host library needs in order to stand
// in for the reference's kernel library as a whole: cross-entropy (a consumer of the row
// max / sum-exp statistics), square transpose and counter-based random fill.  (GEMM stays a
// cuBLAS call inside the host library; it is not part of this path.)
#include <climits>

#include "fdl_common.cuh"

namespace fdl {

namespace {

__device__ __forceinline__ bool aligned16_dev(const void* p) {
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// ---- cross-entropy ------------------------------------------------------------------------------
//
// The reference walks each row with ONE thread, twice, and adds loss_i / batch into a single
// float with atomicAdd (src/kernels/cuda/cross_entropy.cu:9-35): uncoalesced, two reads and
// order-dependent.  Here a team of TPR lanes owns a row and reads it ONCE with 128-bit loads:
// every lane keeps a running (max, sum of exp) pair that is rescaled when the maximum moves
// (the row statistics of softmax, computed online), the lanes' pairs meet through shuffles,
// and lane 0 forms log(sum) + max - x[label].  Rows whose label is out of range contribute 0,
// as in the reference (:17-19).
//
// With about twenty instructions per 128-bit pack -- four of them on the special-function
// unit -- the kernel is as much bound by instruction issue as by memory, so the form with the
// fewest instructions wins: one row per team, the row's packs loaded eight at a time by
// unrolled code with one address computation, the maximum as a tree, four independent sums.
// Forms that keep more loads in flight at the price of bookkeeping measured slower on
// [65536, 1024]: two eight-pack buffers used in turn over four rows per team 50 us, a ring
// of eight slots refilled one by one 56 us (80 instructions per pack, issue slots 77% busy).
//
// The batch mean is deterministic without float atomics and without a ticket: lane 0 adds its
// rows' losses in row order, thread 0 adds the CTA's teams in team order into one double per
// CTA, and a one-CTA kernel (launched so that its start overlaps this kernel's tail) folds the
// CTAs' doubles in index order.

constexpr int kCeThreads = 256;
constexpr int kCeInFlight = 8;  // items (128-bit packs, or floats) per lane and chunk
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// exp(a - b) for a <= b; 1 when both are -inf (a lane that has seen nothing yet).
__device__ __forceinline__ float exp_diff(float a, float b) {
    return a == b ? 1.0f : exp2_approx((a - b) * kLog2e);
}

template <int TPR, bool VEC>
__global__ void __launch_bounds__(kCeThreads, 5)
cross_entropy_rows_kernel(const float* logits, const int64_t* labels, double* cta_loss, int batch, int classes) {
    constexpr int kTeams = kCeThreads / TPR;
    constexpr int kW = VEC ? 4 : 1;
    __shared__ float team_loss[kTeams];
    const int lane = threadIdx.x % TPR;
    const int team = threadIdx.x / TPR;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kTeams + team;
    const bool active = row < batch;
    const int items = VEC ? classes / 4 : classes;
    const float* x = logits + (active ? row : 0) * classes;
    pdl_wait();
    // Lane 0 asks for the label and its logit before the row streams in.
    float picked = 0.0f;
    bool valid = false;
    if (lane == 0 && active) {
        const int64_t label = labels[row];
        valid = label >= 0 && label < classes;
        if (valid) picked = x[label];
    }
    float m = -INFINITY, s = 0.0f;
    for (int i0 = lane; i0 < items; i0 += TPR * kCeInFlight) {
        float v[kCeInFlight][kW];
#pragma unroll
        for (int u = 0; u < kCeInFlight; ++u) {
            const int i = i0 + u * TPR;
            if (VEC) {
                const float4 t = active && i < items ? ld_stream(reinterpret_cast<const float4*>(x) + i)
                                                     : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
                v[u][0] = t.x; v[u][1 % kW] = t.y; v[u][2 % kW] = t.z; v[u][3 % kW] = t.w;
            } else {
                v[u][0] = active && i < items ? ld_stream(x + i) : -INFINITY;
            }
        }
        // maximum of the chunk as a tree, then one rescale of the running sum
        float mx[kCeInFlight];
#pragma unroll
        for (int u = 0; u < kCeInFlight; ++u) {
            mx[u] = v[u][0];
#pragma unroll
            for (int k = 1; k < kW; ++k) mx[u] = fmaxf(mx[u], v[u][k]);
        }
#pragma unroll
        for (int o = kCeInFlight / 2; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < o; ++u) mx[u] = fmaxf(mx[u], mx[u + o]);
        }
        const float m_new = fmaxf(m, mx[0]);
        // (x - max) first: the difference of equal values is exactly 0 whatever their size,
        // which x * log2e - max * log2e does not guarantee for huge logits.
        float add[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int u = 0; u < kCeInFlight; ++u) {
#pragma unroll
            for (int k = 0; k < kW; ++k) add[(u * kW + k) & 3] += exp2_approx((v[u][k] - m_new) * kLog2e);
        }
        s = s * exp_diff(m, m_new) + ((add[0] + add[1]) + (add[2] + add[3]));
        m = m_new;
    }
    pdl_trigger();
    // team maximum, every lane rescales its sum once, team sum
    float big = m;
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) big = fmaxf(big, __shfl_xor_sync(kFullMask, big, o));
    float part = s * exp_diff(m, big);
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) part += __shfl_xor_sync(kFullMask, part, o);
    if (lane == 0) team_loss[team] = valid ? logf(part) + big - picked : 0.0f;
    __syncthreads();
    // The CTA's rows in team order into one double; no fence, no ticket: the CTA is done.
    if (threadIdx.x == 0) {
        double t = 0.0;
#pragma unroll 8
        for (int k = 0; k < kTeams; ++k) t += static_cast<double>(team_loss[k]);
        cta_loss[blockIdx.x] = t;
    }
}

// One CTA folds the per-CTA losses in index order and writes the batch mean.
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_finish_kernel(const double* cta_loss, int n, float* loss, double inv_batch) {
    __shared__ double red[kCeThreads];
    pdl_wait();
    double t = 0.0;
    for (int k = threadIdx.x; k < n; k += kCeThreads) t += cta_loss[k];
    red[threadIdx.x] = t;
    __syncthreads();
    for (int o = kCeThreads / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) *loss = static_cast<float>(red[0] * inv_batch);
}

template <int TPR>
int launch_cross_entropy(bool vec, unsigned int grid, cudaStream_t stream, const float* logits, const int64_t* labels,
                         double* cta_loss, int batch, int classes) {
    const bool pdl = tuning().pdl != 0;
    const dim3 g(grid), b(kCeThreads), one(1, 1, 1);
    return vec ? launch_ex(cross_entropy_rows_kernel<TPR, true>, g, b, 0, stream, one, pdl, logits, labels, cta_loss,
                           batch, classes)
               : launch_ex(cross_entropy_rows_kernel<TPR, false>, g, b, 0, stream, one, pdl, logits, labels, cta_loss,
                           batch, classes);
}

// ---- square transpose -------------------------------------------------------------------------------
//
// 64 x 64 tiles moved with 128-bit accesses in both directions.  A thread loads a 4 x 4
// block (one float4 from each of four consecutive rows), transposes it in registers, and
// parks the four resulting float4 in shared memory at the block's transposed position; after
// the barrier every thread reads float4s in the order in which 16 consecutive lanes write
// one 256-byte run of an output row.  The shared tile is [64][16] float4 without padding:
// the float4 column is XOR-ed with (row / 4), which makes both the parking stores (lanes
// differ in row / 4) and the reads (lanes differ in column) hit eight different 16-byte bank
// groups per quarter warp.  (The reference's best form is a 32 x 33 padded tile with 4-byte
// accesses, src/kernels/cuda/transpose.cu:54-69.)  Needs n % 4 == 0 and 16-byte aligned
// pointers; other sizes take the scalar 32 x 33 kernel below.

constexpr int kTr4Tile = 64;
constexpr int kTr4Threads = 256;

__global__ void __launch_bounds__(kTr4Threads)
transpose_vec4_kernel(const float* in, float* out, int64_t n) {
    __shared__ float4 tile[kTr4Tile][kTr4Tile / 4];
    const int64_t npack = n / 4;
    const int64_t bx = static_cast<int64_t>(blockIdx.x) * kTr4Tile;  // first input column of the tile
    const int64_t by = static_cast<int64_t>(blockIdx.y) * kTr4Tile;  // first input row
    const int c = threadIdx.x & 15;   // float4 column of the 4 x 4 block
    const int i = threadIdx.x >> 4;   // block row
    pdl_wait();
    float4 v[4];
    const int64_t cp = bx / 4 + c;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int64_t r = by + 4 * i + k;
        v[k] = (r < n && cp < npack) ? ld_stream(reinterpret_cast<const float4*>(in + r * n) + cp)
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_trigger();
    // Rows of the transposed block: output row 4c + j holds input rows 4i .. 4i+3 at column 4c + j.
    tile[4 * c + 0][i ^ c] = make_float4(v[0].x, v[1].x, v[2].x, v[3].x);
    tile[4 * c + 1][i ^ c] = make_float4(v[0].y, v[1].y, v[2].y, v[3].y);
    tile[4 * c + 2][i ^ c] = make_float4(v[0].z, v[1].z, v[2].z, v[3].z);
    tile[4 * c + 3][i ^ c] = make_float4(v[0].w, v[1].w, v[2].w, v[3].w);
    __syncthreads();
    const int p = threadIdx.x & 15;  // float4 column of the output row
    const int64_t op = by / 4 + p;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int jr = (threadIdx.x >> 4) + 16 * k;  // output row within the tile
        const int64_t r = bx + jr;
        if (r < n && op < npack) st_stream(reinterpret_cast<float4*>(out + r * n) + op, tile[jr][p ^ (jr >> 2)]);
    }
}

constexpr int kTrTile = 32;

__global__ void __launch_bounds__(kTrTile * 8)
transpose_kernel(const float* in, float* out, int64_t n) {
    __shared__ float tile[kTrTile][kTrTile + 1];  // +1: no bank conflicts on the transposed read
    const int64_t bx = static_cast<int64_t>(blockIdx.x) * kTrTile;
    const int64_t by = static_cast<int64_t>(blockIdx.y) * kTrTile;
    for (int j = threadIdx.y; j < kTrTile; j += 8) {
        const int64_t r = by + j, c = bx + threadIdx.x;
        if (r < n && c < n) tile[j][threadIdx.x] = in[r * n + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < kTrTile; j += 8) {
        const int64_t r = bx + j, c = by + threadIdx.x;
        if (r < n && c < n) out[r * n + c] = tile[threadIdx.x][j];
    }
}

// ---- random fill: Philox4x32-10, counter = element index / 4, key = seed --------------------------
//
// The reference seeds a fresh XORWOW state per element (src/kernels/cuda/random.cu:7-28), whose
// sequence skip dominates the kernel.  Its tests pin only "same seed, same values" and the
// value range, so the generator is free: Philox is counter-based, needs no state and yields
// four 32-bit words per call.

struct PhiloxKeys {
    uint32_t k0[10];  // seed's low word + r * 0x9E3779B9: the key schedule, computed once on the host
    uint32_t k1[10];  // seed's high word + r * 0xBB67AE85
};

PhiloxKeys philox_keys(uint64_t seed) {
    PhiloxKeys k;
    uint32_t a = static_cast<uint32_t>(seed), b = static_cast<uint32_t>(seed >> 32);
    for (int r = 0; r < 10; ++r) {
        k.k0[r] = a;
        k.k1[r] = b;
        a += 0x9E3779B9u;
        b += 0xBB67AE85u;
    }
    return k;
}

// Ten rounds; each round is two 32 x 32 -> 64-bit products and two three-way XORs.
__device__ __forceinline__ void philox4x32_10(uint64_t counter, const PhiloxKeys& keys, uint32_t (&out)[4]) {
    uint32_t c0 = static_cast<uint32_t>(counter), c1 = static_cast<uint32_t>(counter >> 32), c2 = 0u, c3 = 0u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
        const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
        const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ keys.k0[r];
        const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ keys.k1[r];
        c1 = static_cast<uint32_t>(p1);
        c3 = static_cast<uint32_t>(p0);
        c0 = n0;
        c2 = n2;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// (0, 1]: never 0, so the logarithm below is safe; same open/closed ends as curand_uniform.
// Twenty-three bits of the word become the mantissa of a float in [1, 2), which is subtracted
// from 2: one logic operation and an add, where an integer-to-float conversion would go
// through the quarter-rate conversion unit (it made the uniform fill conversion-bound).
__device__ __forceinline__ float unit_open_closed(uint32_t w) {
    return 2.0f - __uint_as_float((w & 0x007fffffu) | 0x3f800000u);
}

// Two quads of floats per thread: 128-bit stores, and two independent Philox chains to
// interleave.  NORMAL: Box-Muller on pairs with the hardware's approximate log2, square root
// and sine / cosine (absolute error about 2^-21 each -- far below what a fill needs -- where the
// exact routines cost several times the generator itself).
template <bool NORMAL>
__global__ void __launch_bounds__(256)
random_fill_kernel(float* data, int64_t n, float p0, float p1, const __grid_constant__ PhiloxKeys keys) {
    // The thread's two quads lie 256 quads apart, so that the 32 lanes of a warp store one
    // contiguous 512-byte run per instruction.
    const int64_t first = static_cast<int64_t>(blockIdx.x) * 512 + threadIdx.x;
    float v[2][4];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        uint32_t w[4];
        philox4x32_10(static_cast<uint64_t>(first + q * 256), keys, w);
        if (NORMAL) {
            // p0 = mean, p1 = stddev.
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const float u1 = unit_open_closed(w[2 * k]), u2 = unit_open_closed(w[2 * k + 1]);
                float r;  // sqrt(-2 ln u1)
                asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(-1.3862943611198906f * __log2f(u1)));
                float sn, cs;
                __sincosf(6.283185307179586f * u2, &sn, &cs);
                v[q][2 * k] = fmaf(p1, r * cs, p0);
                v[q][2 * k + 1] = fmaf(p1, r * sn, p0);
            }
        } else {
            // p0 = low, p1 = high.
#pragma unroll
            for (int k = 0; k < 4; ++k) v[q][k] = fmaf(unit_open_closed(w[k]), p1 - p0, p0);
        }
    }
    // The values depend on nothing in memory: only the stores have to wait for the previous
    // kernel of the stream (which may still be reading this buffer).
    pdl_wait();
    pdl_trigger();
    const bool vec = aligned16_dev(data);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const int64_t quad = first + q * 256;
        const int64_t base = quad * 4;
        if (base + 3 < n && vec) {
            st_stream(reinterpret_cast<float4*>(data) + quad, make_float4(v[q][0], v[q][1], v[q][2], v[q][3]));
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (base + k < n) data[base + k] = v[q][k];
            }
        }
    }
}

}  // namespace

}  // namespace fdl

using namespace fdl;

extern "C" {

int fdl_cross_entropy_f32(const float* logits, const int64_t* labels, float* loss, int64_t batch,
                          int64_t classes, void* stream) {
    if (batch < 0 || classes <= 0 || loss == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    if (batch > INT_MAX || classes > INT_MAX) return FDL_ERR_UNSUPPORTED;
    cudaStream_t s = as_stream(stream);
    if (batch == 0) return static_cast<int>(cudaMemsetAsync(loss, 0, sizeof(float), s));
    if (logits == nullptr || labels == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    const bool vec = classes % 4 == 0 && aligned16(logits);
    // A team of lanes per row: about eight items (packs on the 128-bit path) per lane and chunk.
    const int64_t items = vec ? classes / 4 : classes;
    int tpr = 1;
    while (tpr < kWarp && static_cast<int64_t>(tpr) * kCeInFlight < items) tpr <<= 1;
    const int64_t grid = ceil_div(batch, kCeThreads / tpr);
    void* ws = nullptr;
    int status = get_workspace(static_cast<size_t>(kWorkspaceCounterBytes) + static_cast<size_t>(grid) * sizeof(double), &ws);
    if (status != FDL_OK) return status;
    double* cta_loss = reinterpret_cast<double*>(static_cast<char*>(ws) + kWorkspaceCounterBytes);
    const unsigned int g = static_cast<unsigned int>(grid);
    const int b = static_cast<int>(batch), c = static_cast<int>(classes);
    switch (tpr) {
        case 1: status = launch_cross_entropy<1>(vec, g, s, logits, labels, cta_loss, b, c); break;
        case 2: status = launch_cross_entropy<2>(vec, g, s, logits, labels, cta_loss, b, c); break;
        case 4: status = launch_cross_entropy<4>(vec, g, s, logits, labels, cta_loss, b, c); break;
        case 8: status = launch_cross_entropy<8>(vec, g, s, logits, labels, cta_loss, b, c); break;
        case 16: status = launch_cross_entropy<16>(vec, g, s, logits, labels, cta_loss, b, c); break;
        default: status = launch_cross_entropy<32>(vec, g, s, logits, labels, cta_loss, b, c); break;
    }
    if (status != FDL_OK) return status;
    return launch_ex(cross_entropy_finish_kernel, dim3(1), dim3(kCeThreads), 0, s, dim3(1, 1, 1), tuning().pdl != 0,
                     static_cast<const double*>(cta_loss), static_cast<int>(grid), loss, 1.0 / static_cast<double>(batch));
}

int fdl_transpose_f32(const float* in, float* out, int64_t n, void* stream) {
    if (n < 0) return FDL_ERR_INVALID_ARGUMENT;
    if (n == 0) return FDL_OK;
    if (in == nullptr || out == nullptr || in == out) return FDL_ERR_INVALID_ARGUMENT;
    if (n % 4 == 0 && aligned16(in) && aligned16(out)) {
        const int64_t tiles = ceil_div(n, kTr4Tile);
        if (tiles > 65535) return FDL_ERR_UNSUPPORTED;
        const dim3 grid(static_cast<unsigned int>(tiles), static_cast<unsigned int>(tiles));
        return launch_ex(transpose_vec4_kernel, grid, dim3(kTr4Threads), 0, as_stream(stream), dim3(1, 1, 1),
                         tuning().pdl != 0, in, out, n);
    }
    const int64_t tiles = ceil_div(n, kTrTile);
    if (tiles > 65535) return FDL_ERR_UNSUPPORTED;
    const dim3 grid(static_cast<unsigned int>(tiles), static_cast<unsigned int>(tiles));
    transpose_kernel<<<grid, dim3(kTrTile, 8), 0, as_stream(stream)>>>(in, out, n);
    return launch_status();
}

static int random_fill(bool normal, float* data, int64_t n, float p0, float p1, uint64_t seed, void* stream) {
    if (n < 0 || (n > 0 && data == nullptr)) return FDL_ERR_INVALID_ARGUMENT;
    if (n == 0) return FDL_OK;
    const int64_t grid = ceil_div(ceil_div(n, 8), 256);  // eight floats per thread
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    const dim3 g(static_cast<unsigned int>(grid)), b(256), one(1, 1, 1);
    const PhiloxKeys keys = philox_keys(seed);
    const bool pdl = tuning().pdl != 0;
    return normal ? launch_ex(random_fill_kernel<true>, g, b, 0, as_stream(stream), one, pdl, data, n, p0, p1, keys)
                  : launch_ex(random_fill_kernel<false>, g, b, 0, as_stream(stream), one, pdl, data, n, p0, p1, keys);
}

int fdl_uniform_f32(float* data, int64_t n, float low, float high, uint64_t seed, void* stream) {
    return random_fill(false, data, n, low, high, seed, stream);
}

int fdl_normal_f32(float* data, int64_t n, float mean, float stddev, uint64_t seed, void* stream) {
    return random_fill(true, data, n, mean, stddev, seed, stream);
}

}  // extern "C"
