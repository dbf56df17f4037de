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
// The reference walks each row with ONE thread and adds loss_i / batch into a single float
// with atomicAdd (src/kernels/cuda/cross_entropy.cu:9-35): uncoalesced and order-dependent.
// Here a warp owns a row (coalesced 128-bit loads when possible), writes loss_i / batch to a
// scratch vector, and the deterministic full sum folds that vector.  Rows whose label is
// out of range contribute 0, as in the reference (:17-19).

constexpr int kCeThreads = 256;

__global__ void __launch_bounds__(kCeThreads)
cross_entropy_rows_kernel(const float* logits, const int64_t* labels, float* row_loss, int batch,
                          int classes, float inv_batch) {
    const int lane = threadIdx.x & (kWarp - 1);
    const int row = blockIdx.x * (kCeThreads / kWarp) + threadIdx.x / kWarp;
    if (row >= batch) return;
    const int64_t label = labels[row];
    if (label < 0 || label >= classes) {
        if (lane == 0) row_loss[row] = 0.0f;
        return;
    }
    const float* x = logits + static_cast<int64_t>(row) * classes;
    float m = -INFINITY;
    for (int c = lane; c < classes; c += kWarp) m = fmaxf(m, x[c]);
    m = warp_max(m);
    float s = 0.0f;
    for (int c = lane; c < classes; c += kWarp) s += expf(x[c] - m);
    s = warp_sum(s);
    if (lane == 0) row_loss[row] = (logf(s) + m - x[label]) * inv_batch;
}

// ---- square transpose -------------------------------------------------------------------------------

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

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
}

__device__ __forceinline__ void philox4x32_10(uint64_t counter, uint64_t seed, uint32_t (&out)[4]) {
    uint32_t c[4] = {static_cast<uint32_t>(counter), static_cast<uint32_t>(counter >> 32), 0u, 0u};
    uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = c[i];
}

// (0, 1]: never 0, so log() below is safe; same open/closed ends as curand_uniform.
__device__ __forceinline__ float unit_open_closed(uint32_t w) {
    return (static_cast<float>(w >> 8) + 1.0f) * (1.0f / 16777216.0f);
}

template <bool NORMAL>
__global__ void __launch_bounds__(256)
random_fill_kernel(float* data, int64_t n, float p0, float p1, uint64_t seed) {
    const int64_t quad = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    const int64_t base = quad * 4;
    if (base >= n) return;
    uint32_t w[4];
    philox4x32_10(static_cast<uint64_t>(quad), seed, w);
    float v[4];
    if (NORMAL) {
        // Box-Muller on two pairs; p0 = mean, p1 = stddev.
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float u1 = unit_open_closed(w[2 * k]), u2 = unit_open_closed(w[2 * k + 1]);
            const float r = sqrtf(-2.0f * logf(u1));
            float sn, cs;
            sincospif(2.0f * u2, &sn, &cs);
            v[2 * k] = p0 + p1 * (r * cs);
            v[2 * k + 1] = p0 + p1 * (r * sn);
        }
    } else {
        // p0 = low, p1 = high.
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = p0 + unit_open_closed(w[k]) * (p1 - p0);
    }
    if (base + 3 < n && aligned16_dev(data)) {
        reinterpret_cast<float4*>(data)[quad] = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (base + k < n) data[base + k] = v[k];
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
    const size_t sum_bytes = fdl_sum_scratch_bytes(batch);
    void* ws = nullptr;
    int status = get_workspace(sum_bytes + static_cast<size_t>(batch) * sizeof(float) + 256, &ws);
    if (status != FDL_OK) return status;
    float* row_loss = reinterpret_cast<float*>(static_cast<char*>(ws) + sum_bytes);
    const int rows_per_cta = kCeThreads / kWarp;
    const unsigned int grid = static_cast<unsigned int>(ceil_div(batch, rows_per_cta));
    cross_entropy_rows_kernel<<<grid, kCeThreads, 0, s>>>(
        logits, labels, row_loss, static_cast<int>(batch), static_cast<int>(classes),
        1.0f / static_cast<float>(batch));
    status = launch_status();
    if (status != FDL_OK) return status;
    return fdl_sum_f32(row_loss, batch, loss, nullptr, ws, sum_bytes, stream);
}

int fdl_transpose_f32(const float* in, float* out, int64_t n, void* stream) {
    if (n < 0) return FDL_ERR_INVALID_ARGUMENT;
    if (n == 0) return FDL_OK;
    if (in == nullptr || out == nullptr || in == out) return FDL_ERR_INVALID_ARGUMENT;
    const int64_t tiles = ceil_div(n, kTrTile);
    if (tiles > 65535) return FDL_ERR_UNSUPPORTED;
    const dim3 grid(static_cast<unsigned int>(tiles), static_cast<unsigned int>(tiles));
    transpose_kernel<<<grid, dim3(kTrTile, 8), 0, as_stream(stream)>>>(in, out, n);
    return launch_status();
}

int fdl_uniform_f32(float* data, int64_t n, float low, float high, uint64_t seed, void* stream) {
    if (n < 0 || (n > 0 && data == nullptr)) return FDL_ERR_INVALID_ARGUMENT;
    if (n == 0) return FDL_OK;
    const int64_t grid = ceil_div(ceil_div(n, 4), 256);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    random_fill_kernel<false><<<static_cast<unsigned int>(grid), 256, 0, as_stream(stream)>>>(
        data, n, low, high, seed);
    return launch_status();
}

int fdl_normal_f32(float* data, int64_t n, float mean, float stddev, uint64_t seed, void* stream) {
    if (n < 0 || (n > 0 && data == nullptr)) return FDL_ERR_INVALID_ARGUMENT;
    if (n == 0) return FDL_OK;
    const int64_t grid = ceil_div(ceil_div(n, 4), 256);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    random_fill_kernel<true><<<static_cast<unsigned int>(grid), 256, 0, as_stream(stream)>>>(
        data, n, mean, stddev, seed);
    return launch_status();
}

}  // extern "C"
