// Reductions (fp32 in; fp32 / int64 out): the reference-order 1024-block tree, the
// deterministic full sum, row-wise sum/mean/max/argmax and column-wise sum/mean/max.
//
// All of them read each input byte once with 128-bit loads and keep several independent
// accumulators per thread; the combine tree is registers -> warp shuffles -> shared
// memory -> distributed shared memory of a thread-block cluster -> (for grid-wide
// results) per-cluster partials in scratch that the last cluster to finish folds in a
// fixed order.  No floating-point atomics anywhere, so results are run-to-run identical.
//
// Which kernel a row reduction takes depends on the shape: rows of up to 256 floats go to
// teams of lanes with several rows in flight, longer ones to a warp or a CTA per row, a few
// very long rows are cut into segments (one CTA each, folded per row through scratch), and
// rows at an arbitrary phase of a 16-byte line (odd lengths, unaligned bases) are staged as
// runs of consecutive rows through shared memory by one bulk-async copy per CTA (up to 2048
// floats a row) or walked as aligned packs of the flat buffer with their two edge packs read
// float by float (beyond).
// Column reductions have a tree-free form for up to 8 rows and own four columns per thread
// (adjacent with 128-bit loads, a tile-width apart with 32-bit loads); where the shape allows,
// one cluster of eight CTAs covers all the rows of a column block and nothing goes through
// scratch.  The streaming kernels are launched with programmatic stream serialization and wait
// for the previous kernel of the stream before their first global access.
#include <cooperative_groups.h>

#include <cfloat>
#include <mutex>
#include <climits>
#include <cmath>
#include <cstring>

#include "fdl_common.cuh"

namespace cg = cooperative_groups;

namespace fdl {

namespace {

// ======================================================================================
// 1024-element block sums in the reference's pairing order
// ======================================================================================
//
// The reference reduces each 1024-float block in shared memory, pairing d[i] += d[i+s]
// with s = 512..1 ("address", src/kernels/cuda/reduction.cu:34-50) or d[i] += d[i+s] for
// i % 2s == 0 with s = 1..512 ("interleave", :8-24).  Both are binary trees over the ten
// bits of the element index: "address" folds bit 9 first and bit 0 last, "interleave"
// the other way round.  Here one WARP owns a block.  Lane l loads float4 number
// l + 32*r (r = 0..7), so an element's index bits are  [r:3][lane:5][component:2]:
// folding r happens in registers, folding the lane bits is five shuffles, folding the
// component bits is two adds.  Doing those three groups in the right order reproduces
// either tree bit for bit (float addition is commutative, so which side of a pair a
// value sits on does not matter).

constexpr int kBlk = 1024;
constexpr int kBlkThreads = 256;
constexpr int kBlkWarps = kBlkThreads / kWarp;

template <int TREE>
__device__ __forceinline__ float fold_block_vec(const float4 (&q)[8]) {
    if (TREE == FDL_TREE_ADDRESS) {
        float c[4];
        {
            // bits 9, 8, 7 (register index r)
            float4 a0, a1, a2, a3;
            a0.x = q[0].x + q[4].x; a0.y = q[0].y + q[4].y; a0.z = q[0].z + q[4].z; a0.w = q[0].w + q[4].w;
            a1.x = q[1].x + q[5].x; a1.y = q[1].y + q[5].y; a1.z = q[1].z + q[5].z; a1.w = q[1].w + q[5].w;
            a2.x = q[2].x + q[6].x; a2.y = q[2].y + q[6].y; a2.z = q[2].z + q[6].z; a2.w = q[2].w + q[6].w;
            a3.x = q[3].x + q[7].x; a3.y = q[3].y + q[7].y; a3.z = q[3].z + q[7].z; a3.w = q[3].w + q[7].w;
            a0.x += a2.x; a0.y += a2.y; a0.z += a2.z; a0.w += a2.w;
            a1.x += a3.x; a1.y += a3.y; a1.z += a3.z; a1.w += a3.w;
            c[0] = a0.x + a1.x; c[1] = a0.y + a1.y; c[2] = a0.z + a1.z; c[3] = a0.w + a1.w;
        }
        // bits 6..2 (lane bits 4..0)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int k = 0; k < 4; ++k) c[k] += __shfl_xor_sync(kFullMask, c[k], o);
        }
        // bits 1, 0 (component)
        c[0] += c[2];
        c[1] += c[3];
        return c[0] + c[1];
    } else {
        float w[8];
        // bits 0, 1 (component)
#pragma unroll
        for (int r = 0; r < 8; ++r) w[r] = (q[r].x + q[r].y) + (q[r].z + q[r].w);
        // bits 2..6 (lane bits 0..4)
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
            for (int r = 0; r < 8; ++r) w[r] += __shfl_xor_sync(kFullMask, w[r], o);
        }
        // bits 7, 8, 9 (register index)
        w[0] += w[1]; w[2] += w[3]; w[4] += w[5]; w[6] += w[7];
        w[0] += w[2]; w[4] += w[6];
        return w[0] + w[4];
    }
}

// Scalar-load variant for inputs that are not 16-byte aligned: lane l holds elements
// l + 32*r (r = 0..31), i.e. index bits [r:5][lane:5].
template <int TREE>
__device__ __forceinline__ float fold_block_scalar(float (&e)[32]) {
    if (TREE == FDL_TREE_ADDRESS) {
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
#pragma unroll
            for (int r = 0; r < s; ++r) e[r] += e[r + s];
        }
        float v = e[0];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
        return v;
    } else {
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
            for (int r = 0; r < 32; ++r) e[r] += __shfl_xor_sync(kFullMask, e[r], o);
        }
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
#pragma unroll
            for (int r = 0; r < 32; r += 2 * s) e[r] += e[r + s];
        }
        return e[0];
    }
}

template <int TREE, bool VEC>
__global__ void __launch_bounds__(kBlkThreads)
block_reduce_1024_kernel(const float* x, float* out, int64_t nblocks) {
    const int lane = threadIdx.x & (kWarp - 1);
    const int warp = threadIdx.x / kWarp;
    // One 1024-block per warp, eight per CTA; the grid covers every block once (the loop
    // only matters beyond 2^31 CTAs).
    for (int64_t blk = static_cast<int64_t>(blockIdx.x) * kBlkWarps + warp; blk < nblocks;
         blk += static_cast<int64_t>(gridDim.x) * kBlkWarps) {
        const float* src = x + blk * kBlk;
        float r;
        if (VEC) {
            float4 q[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i] = ld_stream(reinterpret_cast<const float4*>(src) + lane + 32 * i);
            r = fold_block_vec<TREE>(q);
        } else {
            float e[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) e[i] = ld_stream(src + lane + 32 * i);
            r = fold_block_scalar<TREE>(e);
        }
        if (lane == 0) out[blk] = r;
    }
}

// ======================================================================================
// Shared pieces of the grid-wide reductions
// ======================================================================================

constexpr int kSumThreads = 256;
constexpr int kSumUnroll = 8;                                  // 128-bit loads per thread per tile
constexpr int kSumTile = kSumThreads * kSumUnroll;             // float4 per tile (32 KiB)
constexpr int kSumMaxCluster = 8;
constexpr int kSumMaxPartials = 8192;                          // doubles in scratch
// Scratch layout shared by the full sum and the column reductions: a fixed 64 KiB region of
// arrival counters that every kernel leaves zeroed, then the partials.  The region has the
// same size for every problem so that one scratch buffer can serve calls of any shape.
constexpr int kCounterBytes = kWorkspaceCounterBytes;
constexpr int kStaticCounterBytes = 256;  // the static-scratch entry point has its own array

// Block-wide sum in double; result valid in thread 0.  `red` holds one slot per warp.
template <int THREADS>
__device__ __forceinline__ double block_sum_double(double v, double* red) {
    const int lane = threadIdx.x & (kWarp - 1);
    const int warp = threadIdx.x / kWarp;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double total = 0.0;
    if (warp == 0) {
        double t = lane < THREADS / kWarp ? red[lane] : 0.0;
        total = warp_sum(t);
    }
    __syncthreads();
    return total;
}

// ======================================================================================
// Full sum
// ======================================================================================
//
// Every CTA sums one 32 KiB tile (more only when the input exceeds 2 TiB) and the block
// scheduler balances tiles over the SMs.  CL CTAs form a cluster: each drops its partial
// into the leader's shared memory (DSMEM), the leader adds them in rank order and writes
// one double per cluster to scratch.  The last cluster to arrive (ticket counter) folds
// the per-cluster partials in index order, so the result does not depend on scheduling.
//
// Scratch layout: [0, 64 KiB): arrival counters (this kernel uses the first; zero between
// launches); then one double per cluster.

// Cross-GPU epilogue of the full sum.  Every rank owns a small exchange buffer that its
// peers can write (uint64 words[2][kMaxRanks][2]; mapped into each process with CUDA IPC).
// The one CTA that finishes a rank's sum sends the rank's partial (a double) to EVERY
// rank's buffer over NVLink as two self-validating 8-byte words, {high half, epoch} and
// {low half, epoch}, into entry [epoch&1][rank]: an 8-byte store is indivisible, so a reader
// that sees the epoch in both words has the whole value, and no fence or separate flag
// write sits between data and notification.  The CTA then waits -- for a bounded time --
// until all entries of its own buffer show the epoch, and adds the values in rank order.
// All ranks add the same numbers in the same order, so all get the same bits, without a
// separate collective kernel.  Two parities make it safe to start epoch e+1 while a slow
// peer still reads e.
constexpr int kMaxRanks = 16;

struct SumExchange {
    int world = 0;  // 0: single GPU, no exchange
    int rank = 0;
    int send_only = 0;  // 1: split-phase start -- send the partial, leave waiting to the finish kernel
    unsigned int epoch = 0;
    unsigned long long wait_ns = 2000000000ull;  // how long to wait for the peers before giving up
    unsigned long long* words[kMaxRanks] = {};  // each rank's buffer
    unsigned int* error_flag = nullptr;
    unsigned long long* trace = nullptr;  // not NULL: eight time stamps of the finishing CTA go here
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Cross-GPU epilogue of the column reductions: the same protocol, one 8-byte word
// {float bits, epoch} per column.  A rank's buffer holds words[2][world][kExchangeMaxCols].
constexpr int kExchangeMaxCols = 65536;

struct ColsExchange {
    int world = 0;  // 0: single GPU, no exchange
    int rank = 0;
    unsigned int epoch = 0;
    unsigned long long wait_ns = 2000000000ull;
    unsigned long long* words[kMaxRanks] = {};  // each rank's vector region
    unsigned int* error_flag = nullptr;
};

// Sends this rank's finished value of column `col` to every rank and folds the values of
// all ranks in rank order (each rank computes the same result).  Bounded wait.
template <class R>
__device__ __forceinline__ float exchange_column(const ColsExchange& xc, int64_t col, float value) {
    const unsigned long long tag = xc.epoch;
    const int64_t par = static_cast<int64_t>(xc.epoch & 1u) * xc.world * kExchangeMaxCols;
    const unsigned long long word = (static_cast<unsigned long long>(__float_as_uint(value)) << 32) | tag;
    for (int p = 0; p < xc.world; ++p) {
        volatile unsigned long long* dst = xc.words[p] + par + static_cast<int64_t>(xc.rank) * kExchangeMaxCols + col;
        *dst = word;
    }
    float acc = R::identity();
    const unsigned long long t0 = global_timer_ns();
    for (int q = 0; q < xc.world; ++q) {
        volatile unsigned long long* src = xc.words[xc.rank] + par + static_cast<int64_t>(q) * kExchangeMaxCols + col;
        unsigned long long w = *src;
        unsigned int polls = 0;
        while ((w & 0xffffffffull) != tag) {
            if ((++polls & 63u) == 0 && global_timer_ns() - t0 > xc.wait_ns) {
                atomicOr(xc.error_flag, 2u);
                return nanf("");
            }
            w = *src;
        }
        acc = R::combine(acc, __uint_as_float(static_cast<unsigned int>(w >> 32)));
    }
    return acc;
}


// Sends this rank's partial to rank `peer`: two indivisible 8-byte stores, each carrying
// the epoch, into entry [epoch&1][rank] of the peer's buffer.
__device__ __forceinline__ void exchange_send_partial(const SumExchange& xc, int peer, double value) {
    const int par = static_cast<int>(xc.epoch & 1u) * kMaxRanks * 2;
    const unsigned long long tag = xc.epoch;
    const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(value));
    volatile unsigned long long* dst = xc.words[peer] + par + 2 * xc.rank;
    dst[0] = ((bits >> 32) << 32) | tag;
    dst[1] = ((bits & 0xffffffffull) << 32) | tag;
}

// Waits (bounded) until every rank's partial of this epoch has arrived in this rank's own
// buffer and adds them in rank order; result valid in thread 0.  Called by all threads of a
// CTA of at least kMaxRanks threads.  A wait that runs out gives NaN and raises the flag.
__device__ __forceinline__ double exchange_fold_partials(const SumExchange& xc) {
    __shared__ double gathered[kMaxRanks];
    const int par = static_cast<int>(xc.epoch & 1u) * kMaxRanks * 2;
    const unsigned long long tag = xc.epoch;
    bool ok = true;
    if (threadIdx.x < xc.world) {
        volatile unsigned long long* src = xc.words[xc.rank] + par + 2 * threadIdx.x;
        const unsigned long long t0 = global_timer_ns();
        unsigned long long w0 = src[0], w1 = src[1];
        unsigned int polls = 0;
        while ((w0 & 0xffffffffull) != tag || (w1 & 0xffffffffull) != tag) {
            if ((++polls & 63u) == 0 && global_timer_ns() - t0 > xc.wait_ns) {
                ok = false;
                break;
            }
            w0 = src[0];
            w1 = src[1];
        }
        gathered[threadIdx.x] = __longlong_as_double(static_cast<long long>(((w0 >> 32) << 32) | (w1 >> 32)));
    }
    ok = __syncthreads_and(ok);
    double total = 0.0;
    if (threadIdx.x == 0) {
        if (ok) {
            for (int q = 0; q < xc.world; ++q) total += gathered[q];  // rank order
        } else {
            total = nan("");
            atomicOr(xc.error_flag, 2u);
        }
    }
    return total;
}

// Second half of the split-phase exchange: one warp folds the partials that the ranks'
// sum kernels sent (send_only) and writes the results.
__global__ void __launch_bounds__(kWarp) sum_exchange_finish_kernel(float* out_f32, double* out_f64,
                                                                  const SumExchange xc) {
    const double total = exchange_fold_partials(xc);
    if (threadIdx.x == 0) {
        if (out_f32 != nullptr) *out_f32 = static_cast<float>(total);
        if (out_f64 != nullptr) *out_f64 = total;
    }
}

template <int CL, bool VEC>
__global__ void __launch_bounds__(kSumThreads)
sum_kernel(const float* x, int64_t n, int64_t nvec, float* out_f32, double* out_f64,
           unsigned int* counter, double* partials, const SumExchange xc) {
    __shared__ double red[kSumThreads / kWarp];
    __shared__ double cluster_slots[kSumMaxCluster];
    __shared__ bool is_last;

    cg::cluster_group cluster = cg::this_cluster();
    // Arrive now, wait just before the first remote shared-memory access: by then every
    // CTA of the cluster is known to be running, which DSMEM stores require.
    if (CL > 1) cluster.barrier_arrive();
    if (xc.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) xc.trace[0] = global_timer_ns();
    pdl_wait();  // the input may be the previous kernel's output; the scratch was its scratch

    float acc = 0.0f;
    if (VEC) {
        const float4* xv = reinterpret_cast<const float4*>(x);
        for (int64_t tile = blockIdx.x; tile * kSumTile < nvec; tile += gridDim.x) {
            const int64_t base = tile * kSumTile + threadIdx.x;
            float4 v[kSumUnroll];
            if (base + (kSumUnroll - 1) * kSumThreads < nvec) {
#pragma unroll
                for (int u = 0; u < kSumUnroll; ++u) v[u] = ld_stream(xv + base + u * kSumThreads);
            } else {
#pragma unroll
                for (int u = 0; u < kSumUnroll; ++u) {
                    v[u] = base + u * kSumThreads < nvec ? ld_stream(xv + base + u * kSumThreads)
                                                         : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            float s[kSumUnroll];
#pragma unroll
            for (int u = 0; u < kSumUnroll; ++u) s[u] = (v[u].x + v[u].y) + (v[u].z + v[u].w);
            acc += ((s[0] + s[1]) + (s[2] + s[3])) + ((s[4] + s[5]) + (s[6] + s[7]));
        }
        // The n % 4 trailing floats.
        if (blockIdx.x == 0) {
            for (int64_t j = nvec * 4 + threadIdx.x; j < n; j += kSumThreads) acc += x[j];
        }
    } else {
        // Input not 16-byte aligned: same tiling with 32-bit loads.
        constexpr int64_t kScalarTile = static_cast<int64_t>(kSumTile) * 4;
        for (int64_t tile = blockIdx.x; tile * kScalarTile < n; tile += gridDim.x) {
            const int64_t base = tile * kScalarTile + threadIdx.x;
            float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
            for (int u = 0; u < kSumUnroll * 4; ++u) {
                const int64_t j = base + static_cast<int64_t>(u) * kSumThreads;
                if (j < n) s4[u & 3] += ld_stream(x + j);
            }
            acc += (s4[0] + s4[1]) + (s4[2] + s4[3]);
        }
    }

    pdl_trigger();  // every load of this CTA has been issued
    const double block_total = block_sum_double<kSumThreads>(static_cast<double>(acc), red);

    unsigned int nclusters = gridDim.x;
    unsigned int cluster_id = blockIdx.x;
    if (CL > 1) {
        // Cluster stage: every CTA drops its partial into the leader's shared memory.
        const unsigned int rank = cluster.block_rank();
        cluster.barrier_wait();
        if (threadIdx.x == 0) {
            double* leader_slots = cluster.map_shared_rank(cluster_slots, 0);
            leader_slots[rank] = block_total;
        }
        cluster.sync();
        if (rank != 0) return;
        nclusters = gridDim.x / CL;
        cluster_id = blockIdx.x / CL;
    }

    if (threadIdx.x == 0) {
        double t = block_total;
        if (CL > 1) {
            t = 0.0;
#pragma unroll
            for (int k = 0; k < CL; ++k) t += cluster_slots[k];
        }
        partials[cluster_id] = t;
        __threadfence();
        const unsigned int ticket = atomicAdd(counter, 1u);
        is_last = (ticket == nclusters - 1);
    }
    __syncthreads();
    if (!is_last) return;

    // The last cluster leader folds all partials in index order.
    const bool tracing = xc.trace != nullptr && threadIdx.x == 0;
    long long c_ticket = 0;
    if (tracing) {
        xc.trace[1] = global_timer_ns();
        c_ticket = clock64();
    }
    __threadfence();
    double t = 0.0;
    for (unsigned int k = threadIdx.x; k < nclusters; k += kSumThreads) t += __ldcg(partials + k);
    double total = block_sum_double<kSumThreads>(t, red);
    if (tracing) xc.trace[2] = global_timer_ns();
    if (xc.world > 0) {
        __shared__ double my_total;
        if (threadIdx.x == 0) my_total = total;
        __syncthreads();
        if (threadIdx.x < xc.world) exchange_send_partial(xc, threadIdx.x, my_total);
        if (tracing) xc.trace[3] = global_timer_ns();
        if (xc.send_only) {
            if (threadIdx.x == 0) *counter = 0;
            return;
        }
        total = exchange_fold_partials(xc);
        if (tracing) xc.trace[4] = global_timer_ns();
    }
    if (threadIdx.x == 0) {
        if (out_f32 != nullptr) *out_f32 = static_cast<float>(total);
        if (out_f64 != nullptr) *out_f64 = total;
        *counter = 0;  // ready for the next launch
    }
    if (tracing) {
        xc.trace[5] = global_timer_ns();
        xc.trace[6] = static_cast<unsigned long long>(clock64() - c_ticket);  // SM cycles, ticket to end
        xc.trace[7] = xc.epoch;
    }
}

template <int CL, bool VEC>
int launch_sum(const float* x, int64_t n, float* out_f32, double* out_f64, unsigned int* counter,
               double* partials, cudaStream_t stream, SumExchange xc = SumExchange(), bool pdl = true) {
    const int64_t nvec = VEC ? n / 4 : 0;
    int64_t tiles = VEC ? ceil_div(nvec, kSumTile) : ceil_div(n, static_cast<int64_t>(kSumTile) * 4);
    if (tiles < 1) tiles = 1;
    // Tiles a CTA walks (grid-stride).  From 8192 tiles (256 MiB) on, two per CTA halve the number
    // of cluster exchanges and tickets: measured 45.8 -> 45.1 us at 256 MiB, 153.6 -> 151.5 us at
    // 1 GiB; four or more lose again below 1 GiB.
    const int per_cta = tuning().sum_tiles > 0 ? tuning().sum_tiles : (tiles >= 8192 ? 2 : 1);
    int64_t grid = ceil_div(ceil_div(tiles, per_cta), CL) * CL;
    const int64_t cap = static_cast<int64_t>(kSumMaxPartials) * CL;
    if (grid > cap) grid = cap;
    if (tuning().sum_trace != 0) {
        unsigned int* flag = nullptr;
        const int st = error_flag_device_ptr(&flag);
        if (st != FDL_OK) return st;
        xc.trace = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(flag) + 64);
    }
    return launch_ex(sum_kernel<CL, VEC>, dim3(static_cast<unsigned int>(grid)), dim3(kSumThreads), 0, stream,
                     dim3(CL, 1, 1), pdl && tuning().pdl != 0, x, n, nvec, out_f32, out_f64, counter, partials, xc);
}

// ======================================================================================
// Row-wise reductions (axis 1 of a row-major matrix)
// ======================================================================================

struct SumRed {
    static constexpr bool kIsArgmax = false;
    using State = float;
    using Out = float;
    __device__ static State identity() { return 0.0f; }
    __device__ static State lift(float v, int) { return v; }
    __device__ static State combine(State a, State b) { return a + b; }
    // a chain that visits its columns in increasing order takes the next one
    __device__ static State combine_next(State a, float v, int) { return a + v; }
    __device__ static State shuffle_xor(State a, int o) { return __shfl_xor_sync(kFullMask, a, o); }
    template <int TPR>
    __device__ static State team_reduce(State s) {  // over aligned groups of TPR lanes, every lane of the warp calling
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(kFullMask, s, o);
        return s;
    }
    __device__ static State load_cg(const State* p) { return __ldcg(p); }  // L2, never a stale L1 line
    __device__ static State shift(State a, int) { return a; }
    __device__ static Out finish(State a, int64_t, float) { return a; }
};
struct MeanRed : SumRed {
    __device__ static Out finish(State a, int64_t, float divisor) { return a / divisor; }
};
struct MaxRed {
    static constexpr bool kIsArgmax = false;
    using State = float;
    using Out = float;
    __device__ static State identity() { return -INFINITY; }
    __device__ static State lift(float v, int) { return v; }
    __device__ static State combine(State a, State b) { return fmaxf(a, b); }
    __device__ static State combine_next(State a, float v, int) { return fmaxf(a, v); }
    __device__ static State shuffle_xor(State a, int o) { return __shfl_xor_sync(kFullMask, a, o); }
    template <int TPR>
    __device__ static State team_reduce(State s) {
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) s = fmaxf(s, __shfl_xor_sync(kFullMask, s, o));
        return s;
    }
    __device__ static State load_cg(const State* p) { return __ldcg(p); }
    __device__ static State shift(State a, int) { return a; }
    __device__ static Out finish(State a, int64_t, float) { return a; }
};
struct ArgState {
    float v;
    int i;
};
struct ArgmaxRed {
    static constexpr bool kIsArgmax = true;
    using State = ArgState;
    using Out = int64_t;
    __device__ static State identity() { return ArgState{-INFINITY, INT_MAX}; }
    __device__ static State lift(float v, int col) {
        return ArgState{v != v ? -INFINITY : v, col};  // NaN ranks as -inf
    }
    __device__ static State combine(State a, State b) {
        const bool take_b = (b.v > a.v) || (b.v == a.v && b.i < a.i);
        return take_b ? b : a;
    }
    // The next (higher) column of a chain wins only if it is strictly greater, so no index is
    // compared; fmaxf drops a NaN for -inf.
    __device__ static State combine_next(State a, float v, int col) {
        v = fmaxf(v, -INFINITY);
        const bool take = v > a.v;
        return ArgState{take ? v : a.v, take ? col : a.i};
    }
    __device__ static State shuffle_xor(State a, int o) {
        return ArgState{__shfl_xor_sync(kFullMask, a.v, o), __shfl_xor_sync(kFullMask, a.i, o)};
    }
    // The team's maximum and the lowest column that holds it, by two warp-wide integer reductions
    // (redux.sync) instead of a shuffle tree on (value, column) pairs.  The float is mapped onto
    // an integer of the same order; -0 and +0 share a key, as they compare equal.  s.v is never NaN.
    template <int TPR>
    __device__ static State team_reduce(State s) {
        const unsigned int lane = threadIdx.x & (kWarp - 1);
        const unsigned int mask = TPR == kWarp ? kFullMask : ((1u << TPR) - 1u) << (lane & ~static_cast<unsigned int>(TPR - 1));
        int key = __float_as_int(s.v);
        key ^= (key >> 31) & 0x7fffffff;
        if (s.v == 0.0f) key = 0;
        const int best = __reduce_max_sync(mask, key);
        const int col = __reduce_min_sync(mask, key == best ? s.i : INT_MAX);
        int bits = best ^ ((best >> 31) & 0x7fffffff);
        return ArgState{__int_as_float(bits), col};
    }
    __device__ static State load_cg(const State* p) { return ArgState{__ldcg(&p->v), __ldcg(&p->i)}; }
    // columns counted from the start of the row's first pack -> columns of the row
    __device__ static State shift(State a, int head) { return ArgState{a.v, a.i == INT_MAX ? a.i : a.i - head}; }
    __device__ static Out finish(State a, int64_t, float) {
        return a.i == INT_MAX ? 0 : static_cast<int64_t>(a.i);
    }
};

constexpr int kRowThreads = 256;
constexpr int kRowUnroll = 4;  // independent accumulator chains per thread

// What one thread makes of the items first, first + STRIDE, ... < npack of a row (items are
// 128-bit packs when W = 4, floats when W = 1): kRowUnroll independent chains, combined.
template <class R, int W, int STRIDE>
__device__ __forceinline__ typename R::State thread_reduce_span(const float* xr, int first, int npack) {
    using State = typename R::State;
    State acc[kRowUnroll];
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) acc[u] = R::identity();
    int p = first;
    if (R::kIsArgmax && W == 4) {
        // Argmax works on whole packs: three fmaxf (which skip NaNs) and one compare per
        // 128-bit load.  Only when a pack beats the running maximum -- rare once a few
        // packs have been seen -- is the winning lane inside it worked out.
        const float4* xv = reinterpret_cast<const float4*>(xr);
        float best[kRowUnroll];
        int best_col[kRowUnroll];
#pragma unroll
        for (int u = 0; u < kRowUnroll; ++u) {
            best[u] = -INFINITY;
            best_col[u] = INT_MAX;
        }
        for (; p + (kRowUnroll - 1) * STRIDE < npack; p += kRowUnroll * STRIDE) {
            float4 v[kRowUnroll];
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) v[u] = ld_stream(xv + p + u * STRIDE);
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) {
                const float m4 = fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w));
                if (m4 > best[u]) {
                    best[u] = m4;
                    best_col[u] = (p + u * STRIDE) * 4 +
                                  (v[u].x == m4 ? 0 : (v[u].y == m4 ? 1 : (v[u].z == m4 ? 2 : 3)));
                }
            }
        }
        for (; p < npack; p += STRIDE) {
            const float4 v = ld_stream(xv + p);
            const float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
            if (m4 > best[0]) {
                best[0] = m4;
                best_col[0] = p * 4 + (v.x == m4 ? 0 : (v.y == m4 ? 1 : (v.z == m4 ? 2 : 3)));
            }
        }
        // Chains hold disjoint, interleaved column sets: ties go to the lower column.
#pragma unroll
        for (int u = 0; u < kRowUnroll; ++u) acc[u] = R::lift(best[u], best_col[u]);
    } else if (W == 4) {
        const float4* xv = reinterpret_cast<const float4*>(xr);
        for (; p + (kRowUnroll - 1) * STRIDE < npack; p += kRowUnroll * STRIDE) {
            float4 v[kRowUnroll];
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) v[u] = ld_stream(xv + p + u * STRIDE);
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) {
                const int c = (p + u * STRIDE) * 4;
                acc[u] = R::combine(acc[u], R::lift(v[u].x, c));
                acc[u] = R::combine(acc[u], R::lift(v[u].y, c + 1));
                acc[u] = R::combine(acc[u], R::lift(v[u].z, c + 2));
                acc[u] = R::combine(acc[u], R::lift(v[u].w, c + 3));
            }
        }
        for (; p < npack; p += STRIDE) {
            const float4 v = ld_stream(xv + p);
            const int c = p * 4;
            acc[0] = R::combine(acc[0], R::lift(v.x, c));
            acc[0] = R::combine(acc[0], R::lift(v.y, c + 1));
            acc[0] = R::combine(acc[0], R::lift(v.z, c + 2));
            acc[0] = R::combine(acc[0], R::lift(v.w, c + 3));
        }
    } else {
        for (; p + (kRowUnroll - 1) * STRIDE < npack; p += kRowUnroll * STRIDE) {
            float v[kRowUnroll];
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) v[u] = ld_stream(xr + p + u * STRIDE);
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) {
                acc[u] = R::combine(acc[u], R::lift(v[u], p + u * STRIDE));
            }
        }
        for (; p < npack; p += STRIDE) acc[0] = R::combine(acc[0], R::lift(ld_stream(xr + p), p));
    }
    return R::combine(R::combine(acc[0], acc[1]), R::combine(acc[2], acc[3]));
}

// The same for a row at ANY phase of a 16-byte line (length not a multiple of 4 floats, or a
// base that is not 16-byte aligned): the row is covered by aligned packs of the flat buffer,
// the full ones go through thread_reduce_span as 128-bit loads, and the (at most two) packs
// that belong to the row only in part are read float by float by lanes 0 and 1.  Columns are
// counted from the start of the first pack (R::shift takes `head` off again at the end).
// [pk_begin, pk_end) limits the work to a segment of the row, in packs.
template <class R, int STRIDE>
__device__ __forceinline__ typename R::State thread_reduce_flat(const float* x, int phase, int64_t row,
                                                                 int cols, int t, int pk_begin, int pk_end,
                                                                 int* head_out) {
    using State = typename R::State;
    const int64_t e0 = phase + row * cols;
    const int head = static_cast<int>(e0 & 3);
    const int npk = (head + cols + 3) >> 2;
    const int tail = (head + cols) & 3;  // floats of the row in a partial last pack (0: it is full)
    const float* line = (x - phase) + (e0 - head);
    const int full_lo = head ? 1 : 0;
    const int full_hi = tail ? npk - 1 : npk;
    const int lo = full_lo > pk_begin ? full_lo : pk_begin;
    const int hi = full_hi < pk_end ? full_hi : pk_end;
    // The edge floats (at most three, in lane 0 for the head and lane 1 for the tail) are
    // requested before the packs, so that they arrive along with them.
    float edge[3];
    int edge_col = 0, edge_n = 0;
    if (t == 0 && head && pk_begin == 0) {
        edge_col = head;
        edge_n = (head + cols < 4 ? head + cols : 4) - head;
    } else if (t == 1 && tail && !(npk == 1 && head) && npk - 1 >= pk_begin && npk - 1 < pk_end) {
        edge_col = (npk - 1) * 4;
        edge_n = tail;
    }
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        if (k < edge_n) edge[k] = ld_stream(line + edge_col + k);
    }
    State s = thread_reduce_span<R, 4, STRIDE>(line, lo + t, hi);
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        if (k < edge_n) s = R::combine(s, R::lift(edge[k], edge_col + k));
    }
    *head_out = head;
    return s;
}

// TPR threads cooperate on a row (32: one warp per row, 8 rows per CTA; 256: one CTA per
// row).  W = 4 needs cols % 4 == 0 and a 16-byte aligned base; W = 1 takes rows at any phase
// (thread_reduce_flat), `phase` being the position of x[0] in its 16-byte line, in floats.
template <class R, int TPR, int W>
__global__ void __launch_bounds__(kRowThreads)
reduce_rows_kernel(const float* x, int64_t rows, int cols, typename R::Out* out, float divisor, int phase) {
    using State = typename R::State;
    constexpr int kRowsPerCta = kRowThreads / TPR;
    __shared__ State red[kRowThreads / kWarp];
    const int lane = threadIdx.x & (kWarp - 1);
    const int warp = threadIdx.x / kWarp;
    const int t = threadIdx.x % TPR;        // position inside the row team
    const int team = threadIdx.x / TPR;
    const int npack = cols / W;
    pdl_wait();  // the input may be the previous kernel's output

    for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + team; row < rows;
         row += static_cast<int64_t>(gridDim.x) * kRowsPerCta) {
        int head = 0;
        State s = W == 4 ? thread_reduce_span<R, 4, TPR>(x + row * cols, t, npack)
                         : thread_reduce_flat<R, TPR>(x, phase, row, cols, t, 0, INT_MAX, &head);
        pdl_trigger();
#pragma unroll
        for (int o = kWarp / 2; o > 0; o >>= 1) s = R::combine(s, R::shuffle_xor(s, o));
        if (TPR == kWarp) {
            if (lane == 0) out[row] = R::finish(R::shift(s, head), cols, divisor);
        } else {
            // One CTA per row: every thread of the CTA runs the same trip count.
            if (lane == 0) red[warp] = s;
            __syncthreads();
            if (warp == 0) {
                State z = lane < kRowThreads / kWarp ? red[lane] : R::identity();
#pragma unroll
                for (int o = kWarp / 2; o > 0; o >>= 1) z = R::combine(z, R::shuffle_xor(z, o));
                if (lane == 0) out[row] = R::finish(R::shift(z, head), cols, divisor);
            }
            __syncthreads();
        }
    }
}

// Short rows (up to 64 items: packs when W = 4, floats when W = 1).  A team of TPR lanes
// (a power of two) owns a row, every lane holds L items of it, and each team keeps U rows in
// flight, so a thread has L * U loads outstanding however short the row is.  Teams take
// consecutive rows, so a warp's loads are contiguous when TPR equals the row's item count.
template <class R, int TPR, int L, int U, int W>
__global__ void __launch_bounds__(kRowThreads)
reduce_rows_narrow_kernel(const float* x, int64_t rows, int cols, typename R::Out* out, float divisor) {
    using State = typename R::State;
    constexpr int kTeams = kRowThreads / TPR;
    const int t = threadIdx.x % TPR;
    const int team = threadIdx.x / TPR;
    const int nitem = cols / W;
    const int64_t row0 = static_cast<int64_t>(blockIdx.x) * (kTeams * U) + team;

    float v[U][L][W];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t row = row0 + static_cast<int64_t>(u) * kTeams;
        const float* xr = x + row * cols;
#pragma unroll
        for (int l = 0; l < L; ++l) {
            const int item = t + l * TPR;
            if (row < rows && item < nitem) {
                if (W == 4) {
                    const float4 q = ld_stream(reinterpret_cast<const float4*>(xr) + item);
                    v[u][l][0] = q.x; v[u][l][1 % W] = q.y; v[u][l][2 % W] = q.z; v[u][l][3 % W] = q.w;
                } else {
                    v[u][l][0] = ld_stream(xr + item);
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t row = row0 + static_cast<int64_t>(u) * kTeams;
        State s = R::identity();
#pragma unroll
        for (int l = 0; l < L; ++l) {
            const int item = t + l * TPR;
            if (row < rows && item < nitem) {
#pragma unroll
                for (int k = 0; k < W; ++k) s = R::combine(s, R::lift(v[u][l][k], item * W + k));
            }
        }
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) s = R::combine(s, R::shuffle_xor(s, o));
        if (t == 0 && row < rows) out[row] = R::finish(s, cols, divisor);
    }
}

// Argmax of short rows.  The generic state (value, column) costs two shuffles and a
// three-way select per step; here only the row maximum travels through the shuffles and one
// ballot per item slot finds the lowest lane that holds it.  Items are visited slot-major
// (slot 0 of every lane precedes slot 1 of any lane, as the columns do), so ties go to the
// lowest column; NaN ranks as -inf, and a row whose maximum is -inf answers column 0.
template <int TPR, int L, int U, int W>
__global__ void __launch_bounds__(kRowThreads)
argmax_rows_narrow_kernel(const float* x, int64_t rows, int cols, int64_t* out, float) {
    constexpr int kTeams = kRowThreads / TPR;
    const int t = threadIdx.x % TPR;
    const int team = threadIdx.x / TPR;
    const int lane = threadIdx.x & (kWarp - 1);
    const int team_shift = lane - t;  // first lane of this team inside its warp
    const unsigned int team_mask = TPR == kWarp ? kFullMask : ((1u << TPR) - 1u);
    const int nitem = cols / W;
    const int64_t row0 = static_cast<int64_t>(blockIdx.x) * (kTeams * U) + team;

    float v[U][L][W];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t row = row0 + static_cast<int64_t>(u) * kTeams;
        const float* xr = x + row * cols;
#pragma unroll
        for (int l = 0; l < L; ++l) {
            const int item = t + l * TPR;
            if (row < rows && item < nitem) {
                if (W == 4) {
                    const float4 q = ld_stream(reinterpret_cast<const float4*>(xr) + item);
                    v[u][l][0] = q.x; v[u][l][1 % W] = q.y; v[u][l][2 % W] = q.z; v[u][l][3 % W] = q.w;
                } else {
                    v[u][l][0] = ld_stream(xr + item);
                }
            } else {
#pragma unroll
                for (int k = 0; k < W; ++k) v[u][l][k] = -INFINITY;
            }
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t row = row0 + static_cast<int64_t>(u) * kTeams;
        float m[L];
        float best = -INFINITY;
#pragma unroll
        for (int l = 0; l < L; ++l) {
            float q = v[u][l][0];
            if (W == 4) q = fmaxf(fmaxf(q, v[u][l][1 % W]), fmaxf(v[u][l][2 % W], v[u][l][3 % W]));
            m[l] = fmaxf(q, -INFINITY);  // fmaxf skips NaNs; an all-NaN item becomes -inf
            best = fmaxf(best, m[l]);
        }
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(kFullMask, best, o));
        bool found = false;
#pragma unroll
        for (int l = 0; l < L; ++l) {
            const unsigned int votes = (__ballot_sync(kFullMask, m[l] == best) >> team_shift) & team_mask;
            if (!found && votes != 0u) {
                found = true;
                if (t == __ffs(static_cast<int>(votes)) - 1 && row < rows) {
                    int col = (t + l * TPR) * W;
                    if (W == 4) {
                        col += v[u][l][0] == best ? 0 : (v[u][l][1 % W] == best ? 1 : (v[u][l][2 % W] == best ? 2 : 3));
                    }
                    out[row] = best == -INFINITY ? 0 : static_cast<int64_t>(col);
                }
            }
        }
    }
}

template <class R, int TPR, int L, int U, int W>
struct NarrowKernel {
    static constexpr auto fn = reduce_rows_narrow_kernel<R, TPR, L, U, W>;
};
template <int TPR, int L, int U, int W>
struct NarrowKernel<ArgmaxRed, TPR, L, U, W> {
    static constexpr auto fn = argmax_rows_narrow_kernel<TPR, L, U, W>;
};

template <class R, int TPR, int L, int U, int W>
int launch_rows_narrow_cfg(const float* x, int64_t rows, int64_t cols, typename R::Out* out,
                           cudaStream_t stream) {
    constexpr int kRowsPerCta = kRowThreads / TPR * U;
    const int64_t grid = ceil_div(rows, kRowsPerCta);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    NarrowKernel<R, TPR, L, U, W>::fn<<<static_cast<unsigned int>(grid), kRowThreads, 0, stream>>>(
        x, rows, static_cast<int>(cols), out, static_cast<float>(cols));
    return launch_status();
}

constexpr int kNarrowMaxItems = 64;

template <class R, int W>
int launch_rows_narrow(const float* x, int64_t rows, int64_t cols, typename R::Out* out,
                       cudaStream_t stream) {
    const int64_t nitem = cols / W;
    if (nitem <= 1) return launch_rows_narrow_cfg<R, 1, 1, 8, W>(x, rows, cols, out, stream);
    if (nitem <= 2) return launch_rows_narrow_cfg<R, 2, 1, 8, W>(x, rows, cols, out, stream);
    if (nitem <= 4) return launch_rows_narrow_cfg<R, 4, 1, 8, W>(x, rows, cols, out, stream);
    if (nitem <= 8) return launch_rows_narrow_cfg<R, 8, 1, 8, W>(x, rows, cols, out, stream);
    if (nitem <= 16) return launch_rows_narrow_cfg<R, 16, 1, 8, W>(x, rows, cols, out, stream);
    if (nitem <= 32) return launch_rows_narrow_cfg<R, 32, 1, 8, W>(x, rows, cols, out, stream);
    return launch_rows_narrow_cfg<R, 32, 2, 4, W>(x, rows, cols, out, stream);
}

// A few very long rows: one CTA per row would leave most SMs idle, so every row is cut into
// segments of about 64 KiB, one CTA each (grid = segments x rows).  A CTA leaves its
// segment's state in scratch; the last CTA of a row to arrive (ticket counter) folds the
// row's segment states -- thread k takes segments k, k + 256, ... in order, then the usual
// tree -- so the result does not depend on which CTA came last.  Sums, maxima and argmax
// (ties: lowest column) all go through the same State type.
template <class R, int W>
__global__ void __launch_bounds__(kRowThreads)
reduce_rows_split_kernel(const float* x, int cols, int seg_items, typename R::State* partials,
                         unsigned int* counters, typename R::Out* out, float divisor, int phase) {
    using State = typename R::State;
    __shared__ State red[kRowThreads / kWarp];
    __shared__ bool is_last;
    const int lane = threadIdx.x & (kWarp - 1);
    const int warp = threadIdx.x / kWarp;
    const int64_t row = blockIdx.y;
    const int nseg = gridDim.x;
    const int seg = blockIdx.x;
    const int nitem = cols / W;
    const int begin = seg * seg_items;
    int end = begin + seg_items;
    if (end > nitem) end = nitem;

    int head = 0;
    State s = W == 4 ? thread_reduce_span<R, 4, kRowThreads>(x + row * cols, begin + static_cast<int>(threadIdx.x), end)
                     : thread_reduce_flat<R, kRowThreads>(x, phase, row, cols, static_cast<int>(threadIdx.x), begin,
                                                          begin + seg_items, &head);
    auto cta_fold = [&](State z) {
#pragma unroll
        for (int o = kWarp / 2; o > 0; o >>= 1) z = R::combine(z, R::shuffle_xor(z, o));
        if (lane == 0) red[warp] = z;
        __syncthreads();
        z = lane < kRowThreads / kWarp ? red[lane] : R::identity();
#pragma unroll
        for (int o = kWarp / 2; o > 0; o >>= 1) z = R::combine(z, R::shuffle_xor(z, o));
        __syncthreads();
        return z;  // every thread of warp 0 holds the CTA's state
    };
    s = cta_fold(s);
    if (threadIdx.x == 0) {
        partials[row * nseg + seg] = s;
        __threadfence();
        const unsigned int ticket = atomicAdd(counters + row, 1u);
        is_last = ticket == static_cast<unsigned int>(nseg - 1);
        if (is_last) counters[row] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    State z = R::identity();
    const State* mine = partials + row * nseg;
    for (int k = threadIdx.x; k < nseg; k += kRowThreads) z = R::combine(z, R::load_cg(mine + k));
    z = cta_fold(z);
    if (threadIdx.x == 0) out[row] = R::finish(R::shift(z, head), cols, divisor);
}

constexpr int64_t kSplitMaxRows = 1184;               // below 8 CTAs per SM of a B200
constexpr int64_t kSplitMinRowBytes = 256 * 1024;     // and rows long enough to cut
constexpr int64_t kSplitSegmentBytes = 64 * 1024;
constexpr int kSplitMaxSegments = 1024;

template <class R, int W>
int launch_rows_split(const float* x, int64_t rows, int64_t cols, typename R::Out* out,
                      cudaStream_t stream) {
    using State = typename R::State;
    // W = 4: packs of an aligned row.  W = 1: a row at any phase, also cut in (flat, aligned) packs;
    // one more than cols / 4 may be needed to cover it.
    const int64_t nitem = W == 4 ? cols / 4 : (cols + 6) / 4;
    int64_t nseg = ceil_div(cols * 4, kSplitSegmentBytes);
    if (nseg > kSplitMaxSegments) nseg = kSplitMaxSegments;
    // whole 128-byte lines per segment, so that segments of a row do not share a line
    const int64_t line_items = 8;
    const int64_t seg_items = ceil_div(ceil_div(nitem, nseg), line_items) * line_items;
    nseg = ceil_div(nitem, seg_items);
    void* scratch = nullptr;
    const size_t need = kCounterBytes + static_cast<size_t>(rows) * nseg * sizeof(State);
    const int status = get_workspace(need, &scratch);
    if (status != FDL_OK) return status;
    unsigned int* counters = static_cast<unsigned int*>(scratch);
    State* partials = reinterpret_cast<State*>(static_cast<char*>(scratch) + kCounterBytes);
    const dim3 grid(static_cast<unsigned int>(nseg), static_cast<unsigned int>(rows));
    reduce_rows_split_kernel<R, W><<<grid, kRowThreads, 0, stream>>>(
        x, static_cast<int>(cols), static_cast<int>(seg_items), partials, counters, out,
        static_cast<float>(cols), static_cast<int>((reinterpret_cast<uintptr_t>(x) & 15u) / 4u));
    return launch_status();
}

template <class R, int TPR, int W>
int launch_rows_cfg(const float* x, int64_t rows, int64_t cols, typename R::Out* out,
                    cudaStream_t stream) {
    constexpr int kRowsPerCta = kRowThreads / TPR;
    // One CTA per group of rows; the block scheduler balances them over the SMs.
    int64_t grid = ceil_div(rows, kRowsPerCta);
    if (grid > 2147483647) grid = 2147483647;
    const int phase = static_cast<int>((reinterpret_cast<uintptr_t>(x) & 15u) / 4u);
    return launch_ex(reduce_rows_kernel<R, TPR, W>, dim3(static_cast<unsigned int>(grid)), dim3(kRowThreads), 0, stream,
                     dim3(1, 1, 1), tuning().pdl != 0, x, rows, static_cast<int>(cols), out, static_cast<float>(cols), phase);
}

// ---- span form: rows at any phase of a 16-byte line, staged through shared memory -------------------
//
// Row lengths that are not a multiple of 4 floats (or a base off the 16-byte grid), up to 2048
// floats.  Consecutive rows are one contiguous run of memory whatever their length: a CTA takes
// a run of rows, thread 0 asks the copy engine for the aligned packs that cover it (one bulk-async
// copy, ~40 KiB in flight per CTA without a register held), and teams of lanes reduce their rows
// out of shared memory float by float -- consecutive lanes, consecutive floats, four independent
// chains a lane.  (The flat-pack forms above give such rows 40-65% of the copy bandwidth: one row
// per warp at a time, two dependent edge loads.)
constexpr int kRowSpanBytes = 40 * 1024;
constexpr int kRowSpanMaxCols = 2048;

template <class R, int TPR>
__global__ void __launch_bounds__(kRowThreads)
reduce_rows_span_kernel(const float* x, int64_t rows, int cols, typename R::Out* out, float divisor, int phase,
                        int rows_per_cta, unsigned int* error_flag) {
    using State = typename R::State;
    constexpr int kTeams = kRowThreads / TPR;
    extern __shared__ __align__(128) unsigned char span_raw[];
    const float* buf = reinterpret_cast<const float*>(span_raw);
    __shared__ uint64_t bar;
    const int team = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
    const int64_t left = rows - r0;
    const int nr = static_cast<int>(left < rows_per_cta ? left : rows_per_cta);
    const int64_t e_lo = phase + r0 * cols;  // first float of the run, counted from the 16-byte line of x[0]
    const int64_t e_hi = e_lo + static_cast<int64_t>(nr) * cols;
    const int64_t pk_lo = e_lo >> 2;
    const int npk = static_cast<int>(((e_hi + 3) >> 2) - pk_lo);
    const int base = static_cast<int>(e_lo - 4 * pk_lo);
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_wait();  // the input may be the previous kernel's output
    if (threadIdx.x == 0) {
        mbar_expect_tx(&bar, static_cast<uint32_t>(npk) * 16u);
        bulk_g2s(span_raw, reinterpret_cast<const float4*>(x - phase) + pk_lo, static_cast<uint32_t>(npk) * 16u, &bar);
    }
    bool landed = mbar_wait_bounded(&bar, 0);
    landed = __syncthreads_and(landed);
    pdl_trigger();
    if (!landed) {
        if (threadIdx.x == 0) atomicOr(error_flag, 1u);
        return;
    }
    // Team k takes rows k, k + kTeams, ...; the same number of trips for every team, so that the
    // sub-warp teams of a warp shuffle together.
    const int trips = (nr + kTeams - 1) / kTeams;
    for (int trip = 0; trip < trips; ++trip) {
        const int i = trip * kTeams + team;
        const bool active = i < nr;
        const float* rowp = buf + base + (active ? i : 0) * cols;
        State acc[kRowUnroll];
#pragma unroll
        for (int u = 0; u < kRowUnroll; ++u) acc[u] = R::identity();
        if (active) {
            // whole trips of the team without a bounds check (the same number for every lane),
            // then one checked trip
            int c = t;
            for (int covered = TPR * kRowUnroll; covered <= cols; covered += TPR * kRowUnroll, c += TPR * kRowUnroll) {
#pragma unroll
                for (int u = 0; u < kRowUnroll; ++u) acc[u] = R::combine_next(acc[u], rowp[c + u * TPR], c + u * TPR);
            }
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) {
                const int cc = c + u * TPR;
                if (cc < cols) acc[u] = R::combine_next(acc[u], rowp[cc], cc);
            }
        }
        State s = R::combine(R::combine(acc[0], acc[1]), R::combine(acc[2], acc[3]));
        s = R::template team_reduce<TPR>(s);
        if (active && t == 0) out[r0 + i] = R::finish(s, cols, divisor);
    }
}

template <class R, int TPR>
int launch_rows_span_cfg(const float* x, int64_t rows, int64_t cols, typename R::Out* out, cudaStream_t stream) {
    static_assert(kRowUnroll == 4, "four chains are combined pairwise above");
    unsigned int* flag = nullptr;
    const int st = error_flag_device_ptr(&flag);
    if (st != FDL_OK) return st;
    int64_t rows_per_cta = (kRowSpanBytes - 32) / (cols * 4);
    if (rows_per_cta < 1) return FDL_ERR_UNSUPPORTED;
    // A whole number of trips of the teams: 10 rows of 1001 floats over 8 teams would run a
    // second trip with 2 teams at work.
    constexpr int kTeams = kRowThreads / TPR;
    if (rows_per_cta > kTeams) rows_per_cta -= rows_per_cta % kTeams;
    if (rows_per_cta > rows) rows_per_cta = rows;
    const int64_t grid = ceil_div(rows, rows_per_cta);
    if (grid > 2147483647) return FDL_ERR_UNSUPPORTED;
    const size_t smem = static_cast<size_t>((rows_per_cta * cols + 6) / 4 + 1) * 16;
    const int phase = static_cast<int>((reinterpret_cast<uintptr_t>(x) & 15u) / 4u);
    return launch_ex(reduce_rows_span_kernel<R, TPR>, dim3(static_cast<unsigned int>(grid)), dim3(kRowThreads), smem,
                     stream, dim3(1, 1, 1), tuning().pdl != 0, x, rows, static_cast<int>(cols), out,
                     static_cast<float>(cols), phase, static_cast<int>(rows_per_cta), flag);
}

template <class R>
int launch_rows_span(const float* x, int64_t rows, int64_t cols, typename R::Out* out, cudaStream_t stream) {
    if (cols <= 32) return launch_rows_span_cfg<R, 8>(x, rows, cols, out, stream);
    if (cols <= 128) return launch_rows_span_cfg<R, 16>(x, rows, cols, out, stream);
    return launch_rows_span_cfg<R, 32>(x, rows, cols, out, stream);
}

template <class R>
int launch_rows(const float* x, int64_t rows, int64_t cols, typename R::Out* out,
                cudaStream_t stream) {
    if (rows < 0 || cols < 0) return FDL_ERR_INVALID_ARGUMENT;
    if (rows == 0) return FDL_OK;
    if (x == nullptr || out == nullptr || cols == 0) return FDL_ERR_INVALID_ARGUMENT;
    if (cols >= INT_MAX - 16) return FDL_ERR_UNSUPPORTED;  // pack arithmetic on a row stays inside int
    const bool vec = aligned16(x) && cols % 4 == 0;
    // (argmax on rows of up to 64 floats stays with the team kernels: its (value, index) pairs
    // cost two shuffles a step and the span form measured 50% against 60% on [1048576,63])
    if (!vec && cols <= tuning().rows_span_reduce_cols && cols <= kRowSpanMaxCols &&
        !(R::kIsArgmax && cols < tuning().rows_span_argmax_from)) {
        const int st = launch_rows_span<R>(x, rows, cols, out, stream);
        if (st != FDL_ERR_UNSUPPORTED) return st;
    }
    if ((vec ? cols / 4 : cols) <= kNarrowMaxItems) {
        return vec ? launch_rows_narrow<R, 4>(x, rows, cols, out, stream)
                   : launch_rows_narrow<R, 1>(x, rows, cols, out, stream);
    }
    if (rows < kSplitMaxRows && cols * 4 >= kSplitMinRowBytes) {
        return vec ? launch_rows_split<R, 4>(x, rows, cols, out, stream)
                   : launch_rows_split<R, 1>(x, rows, cols, out, stream);
    }
    const bool wide = cols >= 2048;  // a whole CTA per row once a warp would loop too long
    if (vec) {
        return wide ? launch_rows_cfg<R, kRowThreads, 4>(x, rows, cols, out, stream)
                    : launch_rows_cfg<R, kWarp, 4>(x, rows, cols, out, stream);
    }
    return wide ? launch_rows_cfg<R, kRowThreads, 1>(x, rows, cols, out, stream)
                : launch_rows_cfg<R, kWarp, 1>(x, rows, cols, out, stream);
}

// ======================================================================================
// Column-wise reductions (axis 0 of `batch` stacked row-major [rows, cols] matrices)
// ======================================================================================
//
// Threads own columns (4 adjacent ones each on the vector path) and march down the rows,
// so every warp-level load is one contiguous 512-byte run.  A CTA is TX threads wide and
// TY = 256/TX rows deep; gridDim.y slices the rows into chunks.  The TY partial rows are
// folded in shared memory; chunk partials go to scratch and the last chunk to arrive for
// a column block folds them in chunk order.
//
// Scratch layout: [0, 64 KiB) one arrival counter per column block (zero between launches),
// then float partials[groups][batch][cols].

constexpr int kColThreads = 256;

struct ColSum {
    __device__ static float identity() { return 0.0f; }
    __device__ static float combine(float a, float b) { return a + b; }
};
struct ColMax {
    __device__ static float identity() { return -INFINITY; }
    __device__ static float combine(float a, float b) { return fmaxf(a, b); }
};

template <class R, int W, int CL>
__global__ void __launch_bounds__(kColThreads)
reduce_cols_kernel(const float* x, int64_t rows, int64_t cols, float* out, float* partials,
                   unsigned int* counters, int tx, int rows_per_chunk, float scale,
                   const ColsExchange xc) {
    // Every thread owns C = 4 columns of the CTA's tile of tx * 4: with W = 4 four adjacent
    // ones (one 128-bit load per row), with W = 1 -- column counts that are not a multiple of
    // 4, unaligned bases -- the columns cx, cx + tx, cx + 2 tx, cx + 3 tx (four coalesced 32-bit
    // loads per row), so that either way a thread has 8 x 16 bytes outstanding.
    constexpr int C = 4;
    extern __shared__ float tile[];  // [TY][TX*C]
    __shared__ bool is_last;
    const int ty_count = kColThreads / tx;
    const int cx = threadIdx.x % tx;
    const int ry = threadIdx.x / tx;
    const int tile_w = tx * C;
    const int64_t col0 = static_cast<int64_t>(blockIdx.x) * tile_w;
    const int64_t col = col0 + (W == 4 ? cx * 4 : cx);  // first of the thread's columns
    const int cstep = W == 4 ? 1 : tx;                      // distance between them
    const int chunk = blockIdx.y;
    const int nchunks = gridDim.y;
    const int64_t b = blockIdx.z;
    const float* xb = x + b * rows * cols;

    constexpr int kInFlight = 8;  // rows in flight per thread: 32 KiB requested per CTA at a time
    constexpr int kAcc = 2;
    float acc[kAcc][C];
#pragma unroll
    for (int u = 0; u < kAcc; ++u) {
#pragma unroll
        for (int k = 0; k < C; ++k) acc[u][k] = R::identity();
    }

    const int64_t r_begin = static_cast<int64_t>(chunk) * rows_per_chunk;
    int64_t r_end = r_begin + rows_per_chunk;
    if (r_end > rows) r_end = rows;
    pdl_wait();  // the input may be the previous kernel's output; the scratch was its scratch
    // (A form that refills each of the eight slots as soon as it has been added, to keep
    // requests outstanding during the adds, measured slower: 60 against 54 us on [2097152, 32].)
    if (col < cols) {
        const float* xc = xb + col;
        bool have[C];  // W = 1: which of the four columns exist (the last tile may be ragged)
#pragma unroll
        for (int k = 0; k < C; ++k) have[k] = W == 4 || col + k * cstep < cols;
        int64_t r = r_begin + ry;
        for (; r + (kInFlight - 1) * ty_count < r_end; r += kInFlight * ty_count) {
            float v[kInFlight][C];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const float* src = xc + (r + u * ty_count) * cols;
                if (W == 4) {
                    const float4 t = ld_stream(reinterpret_cast<const float4*>(src));
                    v[u][0] = t.x; v[u][1] = t.y; v[u][2] = t.z; v[u][3] = t.w;
                } else {
#pragma unroll
                    for (int k = 0; k < C; ++k) v[u][k] = have[k] ? ld_stream(src + k * cstep) : R::identity();
                }
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
#pragma unroll
                for (int k = 0; k < C; ++k) acc[u % kAcc][k] = R::combine(acc[u % kAcc][k], v[u][k]);
            }
        }
        for (; r < r_end; r += ty_count) {
            const float* src = xc + r * cols;
            if (W == 4) {
                const float4 t = ld_stream(reinterpret_cast<const float4*>(src));
                acc[0][0] = R::combine(acc[0][0], t.x); acc[0][1] = R::combine(acc[0][1], t.y);
                acc[0][2] = R::combine(acc[0][2], t.z); acc[0][3] = R::combine(acc[0][3], t.w);
            } else {
#pragma unroll
                for (int k = 0; k < C; ++k) {
                    if (have[k]) acc[0][k] = R::combine(acc[0][k], ld_stream(src + k * cstep));
                }
            }
        }
    }
    pdl_trigger();
#pragma unroll
    for (int k = 0; k < C; ++k) {
        tile[ry * tile_w + (W == 4 ? cx * 4 + k : k * tx + cx)] = R::combine(acc[0][k], acc[1][k]);
    }
    __syncthreads();

    // Fold the TY rows of the tile (fixed order): thread c owns column c and leaves the
    // CTA's value for it in tile[c].
    for (int c = threadIdx.x; c < tile_w; c += kColThreads) {
        float s = tile[c];
        for (int y = 1; y < ty_count; ++y) s = R::combine(s, tile[y * tile_w + c]);
        tile[c] = s;
    }

    // Cluster stage: the CL CTAs of a cluster hold consecutive row chunks of the same
    // columns; the leader reads the others' values through distributed shared memory and
    // folds them in rank order.
    int groups = nchunks;
    int group = chunk;
    if (CL > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();  // every CTA's tile[0..tile_w) is final (and every CTA is running)
        const unsigned int rank = cluster.block_rank();
        if (rank == 0) {
            for (int c = threadIdx.x; c < tile_w; c += kColThreads) {
                float s = tile[c];
#pragma unroll
                for (int k = 1; k < CL; ++k) s = R::combine(s, cluster.map_shared_rank(tile, k)[c]);
                tile[c] = s;
            }
        }
        cluster.sync();  // peers stay resident until the leader has read them
        if (rank != 0) return;
        groups = nchunks / CL;
        group = chunk / CL;
    }

    float* dst = groups == 1 ? out + b * cols
                             : partials + (static_cast<int64_t>(group) * gridDim.z + b) * cols;
    for (int c = threadIdx.x; c < tile_w; c += kColThreads) {
        if (col0 + c >= cols) continue;
        if (groups != 1) {
            dst[col0 + c] = tile[c];
        } else if (xc.world == 0) {
            dst[col0 + c] = tile[c] * scale;
        } else {
            dst[col0 + c] = exchange_column<R>(xc, col0 + c, tile[c] * scale);
        }
    }
    if (groups == 1) return;

    // The CTA barrier orders every thread's partial stores before thread 0's fence, and
    // fences are cumulative, so one device-scope fence publishes the whole CTA's partials
    // (a fence in every thread costs a memory-barrier stall per CTA wave).
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        unsigned int* ctr = counters + b * gridDim.x + blockIdx.x;
        const unsigned int ticket = atomicAdd(ctr, 1u);
        is_last = ticket == static_cast<unsigned int>(groups - 1);
        if (is_last) *ctr = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // The last group to arrive folds all group partials of its columns.  Thread row ry takes
    // groups ry, ry + TY, ... of its own pack of columns (four loads in flight), the TY
    // results meet in shared memory and are folded in thread-row order: a fixed order, so
    // the result does not depend on which group came last, and no thread walks more than
    // groups / TY partials however many row chunks the matrix was cut into.
    {
        float s[C];
#pragma unroll
        for (int k = 0; k < C; ++k) s[k] = R::identity();
        if (col < cols) {
            const float* src = partials + b * cols + col;
            const int64_t stride = static_cast<int64_t>(gridDim.z) * cols;
            bool have[C];
#pragma unroll
            for (int k = 0; k < C; ++k) have[k] = W == 4 || col + k * cstep < cols;
            int g = ry;
            for (; g + 3 * ty_count < groups; g += 4 * ty_count) {
                float v[4][C];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float* q = src + (g + j * ty_count) * stride;
                    if (W == 4) {
                        const float4 t = __ldcg(reinterpret_cast<const float4*>(q));
                        v[j][0] = t.x; v[j][1] = t.y; v[j][2] = t.z; v[j][3] = t.w;
                    } else {
#pragma unroll
                        for (int k = 0; k < C; ++k) v[j][k] = have[k] ? __ldcg(q + k * cstep) : R::identity();
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
#pragma unroll
                    for (int k = 0; k < C; ++k) s[k] = R::combine(s[k], v[j][k]);
                }
            }
            for (; g < groups; g += ty_count) {
                const float* q = src + g * stride;
                if (W == 4) {
                    const float4 t = __ldcg(reinterpret_cast<const float4*>(q));
                    s[0] = R::combine(s[0], t.x); s[1] = R::combine(s[1], t.y);
                    s[2] = R::combine(s[2], t.z); s[3] = R::combine(s[3], t.w);
                } else {
#pragma unroll
                    for (int k = 0; k < C; ++k) {
                        if (have[k]) s[k] = R::combine(s[k], __ldcg(q + k * cstep));
                    }
                }
            }
        }
#pragma unroll
        for (int k = 0; k < C; ++k) tile[ry * tile_w + (W == 4 ? cx * 4 + k : k * tx + cx)] = s[k];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < tile_w; c += kColThreads) {
        if (col0 + c >= cols) continue;
        float s = tile[c];
        for (int y = 1; y < ty_count; ++y) s = R::combine(s, tile[y * tile_w + c]);
        s *= scale;
        if (xc.world > 0) s = exchange_column<R>(xc, col0 + c, s);
        out[b * cols + col0 + c] = s;
    }
}

// A handful of rows (an average of a few tensors): no tree at all.  Like an elementwise
// op, every thread owns U packs of columns, has all ROWS x U loads in flight and writes the
// result; one tile per CTA.  ROWS is a template parameter so that the row loop unrolls.
constexpr int kFewRows = 8;

template <class R, int W, int ROWS, int U>
__global__ void __launch_bounds__(kColThreads)
reduce_cols_few_kernel(const float* x, int64_t cols, float* out, float scale) {
    const int64_t npack = cols / W;
    const float* xb = x + static_cast<int64_t>(blockIdx.z) * ROWS * cols;
    float* ob = out + static_cast<int64_t>(blockIdx.z) * cols;
    const int64_t tile = static_cast<int64_t>(blockIdx.y) * gridDim.x + blockIdx.x;
    const int64_t base = tile * (kColThreads * U) + threadIdx.x;
    float v[U][ROWS][W];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t pk = base + u * kColThreads;
        if (pk < npack) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const float* src = xb + r * cols + pk * W;
                if (W == 4) {
                    const float4 t = ld_stream(reinterpret_cast<const float4*>(src));
                    v[u][r][0] = t.x; v[u][r][1 % W] = t.y; v[u][r][2 % W] = t.z; v[u][r][3 % W] = t.w;
                } else {
                    v[u][r][0] = ld_stream(src);
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t pk = base + u * kColThreads;
        if (pk >= npack) continue;
        float acc[W];
#pragma unroll
        for (int k = 0; k < W; ++k) acc[k] = R::identity();  // so that a NaN-only column gives what the tree gives
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
#pragma unroll
            for (int k = 0; k < W; ++k) acc[k] = R::combine(acc[k], v[u][r][k]);
        }
        float* dst = ob + pk * W;
        if (W == 4) {
            st_stream(reinterpret_cast<float4*>(dst),
                      make_float4(acc[0] * scale, acc[1 % W] * scale, acc[2 % W] * scale, acc[3 % W] * scale));
        } else {
            dst[0] = acc[0] * scale;
        }
    }
}

template <class R, int W, int ROWS>
int launch_cols_few_rows(const float* x, int64_t batch, int64_t cols, float* out, float scale,
                         cudaStream_t stream) {
    constexpr int U = ROWS <= 2 ? 4 : (ROWS <= 4 ? 2 : 1);
    const int64_t tiles = ceil_div(cols / W, static_cast<int64_t>(kColThreads) * U);
    // tiles fold into a 2-D grid so that any column count fits
    const int64_t gx = tiles < 65535 ? tiles : 65535;
    const int64_t gy = ceil_div(tiles, gx);
    if (gy > 65535) return FDL_ERR_UNSUPPORTED;
    const dim3 grid(static_cast<unsigned int>(gx), static_cast<unsigned int>(gy), static_cast<unsigned int>(batch));
    reduce_cols_few_kernel<R, W, ROWS, U><<<grid, kColThreads, 0, stream>>>(x, cols, out, scale);
    return launch_status();
}

template <class R, int W>
int launch_cols_few(const float* x, int64_t batch, int64_t rows, int64_t cols, float* out, float scale,
                    cudaStream_t stream) {
    switch (rows) {
        case 1: return launch_cols_few_rows<R, W, 1>(x, batch, cols, out, scale, stream);
        case 2: return launch_cols_few_rows<R, W, 2>(x, batch, cols, out, scale, stream);
        case 3: return launch_cols_few_rows<R, W, 3>(x, batch, cols, out, scale, stream);
        case 4: return launch_cols_few_rows<R, W, 4>(x, batch, cols, out, scale, stream);
        case 5: return launch_cols_few_rows<R, W, 5>(x, batch, cols, out, scale, stream);
        case 6: return launch_cols_few_rows<R, W, 6>(x, batch, cols, out, scale, stream);
        case 7: return launch_cols_few_rows<R, W, 7>(x, batch, cols, out, scale, stream);
        default: return launch_cols_few_rows<R, W, 8>(x, batch, cols, out, scale, stream);
    }
}

struct ColsGeometry {
    int tx;              // threads across columns (power of two, <= 256)
    int w;               // floats per thread (4 or 1)
    int col_blocks;      // gridDim.x
    int chunks;          // gridDim.y (a multiple of `cluster`)
    int cluster;         // CTAs per cluster along the chunk dimension (1 or kColCluster)
    int rows_per_chunk;
    size_t counter_bytes;
    size_t scratch_bytes;
};

int cols_geometry(int sm_count, int64_t batch, int64_t rows, int64_t cols, bool vec,
                  ColsGeometry* g) {
    g->w = vec ? 4 : 1;  // load width; a thread owns four columns either way
    const int64_t packs = ceil_div(cols, 4);
    // Preferred shape: ONE cluster of eight CTAs covers all the rows of a column block, so the
    // fold through distributed shared memory is the last stage -- no partials in global memory,
    // no ticket, no second pass (on [8192, 8192] that tail is worth 4 of 49 us).  It is taken when
    // a tile width of 32 to 256 threads gives between 2.5 and 5.5 CTAs per SM (all resident at
    // once, a CTA lives as long as the kernel) and every thread row still gets 16 rows.
    if (tuning().cols_single != 0 && tuning().cols_chunks == 0 && batch == 1) {
        constexpr int kSingle = 8;
        for (int tx = 32; tx <= kColThreads; tx <<= 1) {
            const int64_t blocks = ceil_div(packs, tx);
            const int64_t ctas = blocks * kSingle;
            const int ty = kColThreads / tx;
            if (ctas * 2 < static_cast<int64_t>(sm_count) * 5 || ctas * 2 > static_cast<int64_t>(sm_count) * 11) continue;
            if (rows < static_cast<int64_t>(kSingle) * ty * 16 || ceil_div(rows, kSingle) > 2147483647) continue;
            g->tx = tx;
            g->col_blocks = static_cast<int>(blocks);
            g->rows_per_chunk = static_cast<int>(ceil_div(rows, kSingle));
            g->chunks = kSingle;
            g->cluster = kSingle;
            g->counter_bytes = kCounterBytes;
            g->scratch_bytes = 0;
            return FDL_OK;
        }
    }
    int tx = 1;
    int tx_max = tuning().cols_tx;  // threads across columns (x4 floats = row bytes per CTA)
    // With few rows, thread rows beyond rows / 8 would sit idle: widen the tile instead (a
    // matrix of three rows is walked like an elementwise op, one thread per pack of columns).
    while (tx_max < kColThreads && static_cast<int64_t>(kColThreads / tx_max) * 8 > rows) tx_max <<= 1;
    while (tx < tx_max && tx < packs) tx <<= 1;
    g->tx = tx;
    g->col_blocks = static_cast<int>(ceil_div(packs, tx));
    const int ty = kColThreads / tx;
    // Many more CTAs than SMs (the block scheduler balances them), but at least 16 rows
    // per thread in a chunk so that partials stay a small fraction of the traffic.
    const int64_t target = static_cast<int64_t>(sm_count) * tuning().cols_ctas_per_sm;
    int64_t chunks = ceil_div(target, static_cast<int64_t>(g->col_blocks) * batch);
    const int64_t max_chunks = ceil_div(rows, static_cast<int64_t>(ty) * 32);
    if (tuning().cols_chunks > 0) chunks = tuning().cols_chunks;
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks < 1) chunks = 1;
    if (chunks > 65535) chunks = 65535;
    int64_t per_chunk = ceil_div(rows, chunks);
    // Whole batches of eight rows per thread row: the rows left over after the last full batch
    // are loaded one per trip, a memory latency each, at the end of EVERY chunk.  Rounding the
    // chunk up to a multiple of the batch leaves such a tail in the last chunk only.
    const int64_t batch_rows = static_cast<int64_t>(ty) * 8;
    if (per_chunk >= 4 * batch_rows) per_chunk = ceil_div(per_chunk, batch_rows) * batch_rows;
    g->rows_per_chunk = static_cast<int>(per_chunk);
    g->chunks = static_cast<int>(ceil_div(rows, g->rows_per_chunk));
    g->cluster = 1;
    // Chunk CTAs per cluster: eight on the 128-bit path (half as many partials and tickets as four:
    // [2097152,32] 49.2 -> 47.1 us), two on the 32-bit path of odd column counts ([65536,1001]
    // 58 -> 53 us), unless the tuning key says otherwise.
    const int want_cluster = tuning().cols_cluster > 0 ? tuning().cols_cluster : (vec ? 8 : 2);
    if (want_cluster > 1 && g->chunks >= want_cluster) {
        // Round up to whole clusters; trailing chunks may be empty (they contribute the
        // identity).
        g->cluster = want_cluster;
        g->chunks = static_cast<int>(ceil_div(g->chunks, want_cluster)) * want_cluster;
    }
    int groups = g->chunks / g->cluster;
    const size_t ncounters = static_cast<size_t>(g->col_blocks) * batch;
    if (groups > 1 && ncounters * sizeof(unsigned int) > static_cast<size_t>(kCounterBytes)) {
        // More column blocks than arrival counters: such a matrix is wide enough to fill the
        // GPU with one CTA per column block, each walking all the rows, and needs neither
        // partials nor counters.
        g->rows_per_chunk = static_cast<int>(rows < 2147483647 ? rows : 2147483647);
        if (g->rows_per_chunk != rows) return FDL_ERR_UNSUPPORTED;
        g->chunks = 1;
        g->cluster = 1;
        groups = 1;
    }
    g->counter_bytes = kCounterBytes;
    g->scratch_bytes =
        groups == 1
            ? 0
            : g->counter_bytes +
                  ((static_cast<size_t>(groups) * batch * cols * sizeof(float) + 255) / 256) * 256;
    return FDL_OK;
}

// Column counts that are not a multiple of 4.  A matrix [R, C] with C odd is, taken g = 4 rows at
// a time (g = 2 for C % 4 == 2), a matrix [R / g, g * C] whose row length IS a multiple of 4 floats:
// the same bytes, walked with 128-bit loads by the kernel above, four adjacent "columns" a thread.
// Its g * C column results fold into the C wanted ones (column c gathers c, c + C, ...) in a small
// second kernel, which also takes in the R % g rows left over and applies the mean's scale.  With
// 32-bit loads -- four columns a tile-width apart per thread -- the same shapes reach 67-77% of the
// copy bandwidth.
inline int regroup_factor(int64_t cols) { return cols % 2 != 0 ? 4 : (cols % 4 != 0 ? 2 : 1); }

template <class R>
__global__ void __launch_bounds__(256)
cols_regroup_finish_kernel(const float* grouped, int g, int64_t cols, const float* leftover, int leftover_rows,
                           float* out, float scale) {
    pdl_wait();  // `grouped` is the previous kernel's output
    const int64_t c = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (c >= cols) return;
    float acc = grouped[c];
    for (int i = 1; i < g; ++i) acc = R::combine(acc, grouped[c + i * cols]);
    for (int r = 0; r < leftover_rows; ++r) acc = R::combine(acc, leftover[r * cols + c]);
    out[c] = acc * scale;
}

// Whether the regrouped form applies, and the scratch it needs: the grouped matrix's own scratch,
// then its g * C results.
bool cols_regroup_applies(int64_t batch, int64_t rows, int64_t cols) {
    if (tuning().cols_regroup == 0 || batch != 1 || cols % 4 == 0) return false;
    const int g = regroup_factor(cols);
    return rows / g > kFewRows && g * cols <= 2147483647;
}

// The SM count enters the geometry, so the scratch query needs a device too; without
// one (a build-only machine) it assumes the 148 SMs of a B200.
int sm_count_or_default() {
    int status = FDL_OK;
    const DeviceInfo* info = current_device_info(&status);
    if (info == nullptr) {
        cudaGetLastError();
        return 148;
    }
    return info->sm_count;
}

}  // namespace

}  // namespace fdl

using namespace fdl;

extern "C" {

int fdl_block_reduce_1024_f32(const float* x, float* out, int64_t n, int tree, void* stream) {
    if (n < 0) return FDL_ERR_INVALID_ARGUMENT;
    const int64_t nblocks = n / kBlk;
    if (nblocks == 0) return FDL_OK;
    if (x == nullptr || out == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    if (tree != FDL_TREE_INTERLEAVE && tree != FDL_TREE_ADDRESS) return FDL_ERR_INVALID_ARGUMENT;
    int status = FDL_OK;
    const DeviceInfo* info = current_device_info(&status);
    if (info == nullptr) return status;
    (void)info;
    int64_t want_grid = ceil_div(nblocks, kBlkWarps);
    const int grid = want_grid > 2147483647 ? 2147483647 : static_cast<int>(want_grid);
    cudaStream_t s = as_stream(stream);
    const bool vec = aligned16(x);
    if (tree == FDL_TREE_ADDRESS) {
        if (vec) block_reduce_1024_kernel<FDL_TREE_ADDRESS, true><<<grid, kBlkThreads, 0, s>>>(x, out, nblocks);
        else block_reduce_1024_kernel<FDL_TREE_ADDRESS, false><<<grid, kBlkThreads, 0, s>>>(x, out, nblocks);
    } else {
        if (vec) block_reduce_1024_kernel<FDL_TREE_INTERLEAVE, true><<<grid, kBlkThreads, 0, s>>>(x, out, nblocks);
        else block_reduce_1024_kernel<FDL_TREE_INTERLEAVE, false><<<grid, kBlkThreads, 0, s>>>(x, out, nblocks);
    }
    return launch_status();
}

size_t fdl_sum_scratch_bytes(int64_t n) {
    (void)n;
    return kCounterBytes + kSumMaxPartials * sizeof(double);
}

int fdl_sum_f32(const float* x, int64_t n, float* out_f32, double* out_f64, void* scratch,
                size_t scratch_bytes, void* stream) {
    if (n < 0 || (out_f32 == nullptr && out_f64 == nullptr)) return FDL_ERR_INVALID_ARGUMENT;
    if (n > 0 && x == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    int status = FDL_OK;
    const size_t need = fdl_sum_scratch_bytes(n);
    if (scratch == nullptr) {
        status = get_workspace(need, &scratch);
        if (status != FDL_OK) return status;
    } else if (scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) {
        return FDL_ERR_WORKSPACE;
    }
    unsigned int* counter = static_cast<unsigned int*>(scratch);
    double* partials = reinterpret_cast<double*>(static_cast<char*>(scratch) + kCounterBytes);
    cudaStream_t s = as_stream(stream);
    if (!aligned16(x)) return launch_sum<1, false>(x, n, out_f32, out_f64, counter, partials, s);
    switch (tuning().sum_cluster) {
        case 1:
            return launch_sum<1, true>(x, n, out_f32, out_f64, counter, partials, s);
        case 2:
            return launch_sum<2, true>(x, n, out_f32, out_f64, counter, partials, s);
        case 4:
            return launch_sum<4, true>(x, n, out_f32, out_f64, counter, partials, s);
        default:
            return launch_sum<8, true>(x, n, out_f32, out_f64, counter, partials, s);
    }
}

// ---- full sum for callers that must not allocate ------------------------------------------------
//
// The scratch of the full sum (arrival counter + per-cluster partials) lives in a fixed
// array in device memory that is part of the library image: every GPU that loads the
// library carries these 65,792 bytes until the process exits.  In host code the array's name
// is only a handle for the runtime, not a device address; the address each device uses is
// asked for once, with that device current, through cudaGetSymbolAddress.

// Same layout and size as the scratch the regular entry point asks for: the kernel never
// writes more than kSumMaxPartials partials whatever n is (CTAs loop over tiles beyond
// that).  The element count is nevertheless capped at a stated maximum.
constexpr int64_t kStaticSumMaxElems = int64_t{1} << 30;
static __device__ __align__(256) unsigned char g_static_sum_scratch[kStaticCounterBytes + kSumMaxPartials * sizeof(double)];

static std::mutex g_static_mutex;
static void* g_static_sum_ptr[64] = {};

int fdl_sum_f32_static(const float* x, int64_t n, float* out_f32, double* out_f64, void* stream) {
    if (n < 0 || (out_f32 == nullptr && out_f64 == nullptr)) return FDL_ERR_INVALID_ARGUMENT;
    if (n > 0 && x == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    if (n > kStaticSumMaxElems) return FDL_ERR_TOO_LARGE_FOR_STATIC_SCRATCH;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= 64) return FDL_ERR_NO_DEVICE;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (g_static_sum_ptr[dev] == nullptr) {
            // Set-up, once per device, with that device current.
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_static_sum_scratch);
            if (e != cudaSuccess) return static_cast<int>(e);
            g_static_sum_ptr[dev] = ptr;
        }
        scratch = g_static_sum_ptr[dev];
    }
    cudaStream_t s = as_stream(stream);
    // The array keeps whatever the previous call left: the arrival counter must start at 0.
    e = cudaMemsetAsync(scratch, 0, kStaticCounterBytes, s);
    if (e != cudaSuccess) return static_cast<int>(e);
    unsigned int* counter = static_cast<unsigned int*>(scratch);
    double* partials = reinterpret_cast<double*>(static_cast<char*>(scratch) + kStaticCounterBytes);
    // Fixed launch shape (clusters of 4): at most kSumMaxPartials partials are written.
    // Plain launches: the memset above, not a kernel, is what precedes them on the stream.
    if (!aligned16(x)) return launch_sum<1, false>(x, n, out_f32, out_f64, counter, partials, s, SumExchange(), false);
    return launch_sum<4, true>(x, n, out_f32, out_f64, counter, partials, s, SumExchange(), false);
}

int fdl_reduce_rows_f32(const float* x, int64_t rows, int64_t cols, float* out, int op,
                        void* stream) {
    cudaStream_t s = as_stream(stream);
    switch (op) {
        case FDL_REDUCE_SUM:
            return launch_rows<SumRed>(x, rows, cols, out, s);
        case FDL_REDUCE_MEAN:
            return launch_rows<MeanRed>(x, rows, cols, out, s);
        case FDL_REDUCE_MAX:
            return launch_rows<MaxRed>(x, rows, cols, out, s);
        default:
            return FDL_ERR_INVALID_ARGUMENT;
    }
}

int fdl_argmax_rows_f32(const float* x, int64_t rows, int64_t cols, int64_t* out, void* stream) {
    return launch_rows<ArgmaxRed>(x, rows, cols, out, as_stream(stream));
}

// Scratch of the regrouped form: the grouped matrix's own scratch (always counters first, so that
// the layout does not depend on which geometry it takes), then its g * cols results.
static size_t regroup_inner_bytes(int64_t rows, int64_t cols) {
    const int g = regroup_factor(cols);
    const int sms = sm_count_or_default();
    ColsGeometry gi;
    cols_geometry(sms, 1, rows / g, g * cols, true, &gi);
    const size_t inner = gi.scratch_bytes > static_cast<size_t>(kCounterBytes) ? gi.scratch_bytes : kCounterBytes;
    return (inner + 255) / 256 * 256;
}
static size_t regroup_scratch_bytes(int64_t rows, int64_t cols) {
    const int g = regroup_factor(cols);
    return regroup_inner_bytes(rows, cols) + (static_cast<size_t>(g) * cols * sizeof(float) + 255) / 256 * 256;
}

size_t fdl_reduce_cols_scratch_bytes(int64_t batch, int64_t rows, int64_t cols) {
    if (batch <= 0 || rows <= 0 || cols <= 0) return 0;
    // Whether the 128-bit path is taken depends on pointer alignment too: report the
    // larger of the two geometries.
    const int sms = sm_count_or_default();
    ColsGeometry gv, gs;
    cols_geometry(sms, batch, rows, cols, cols % 4 == 0, &gv);
    cols_geometry(sms, batch, rows, cols, false, &gs);
    size_t need = gv.scratch_bytes > gs.scratch_bytes ? gv.scratch_bytes : gs.scratch_bytes;
    if (cols_regroup_applies(batch, rows, cols)) {
        const size_t grouped = regroup_scratch_bytes(rows, cols);
        if (grouped > need) need = grouped;
    }
    return need;
}

static int reduce_cols_impl(const float* x, int64_t batch, int64_t rows, int64_t cols, float* out,
                            int op, double mean_divisor, void* scratch, size_t scratch_bytes,
                            void* stream, const ColsExchange& xc) {
    if (batch < 0 || rows < 0 || cols < 0) return FDL_ERR_INVALID_ARGUMENT;
    if (batch == 0 || cols == 0) return FDL_OK;
    if (x == nullptr || out == nullptr || rows == 0) return FDL_ERR_INVALID_ARGUMENT;
    if (op != FDL_REDUCE_SUM && op != FDL_REDUCE_MEAN && op != FDL_REDUCE_MAX) {
        return FDL_ERR_INVALID_ARGUMENT;
    }
    if (op == FDL_REDUCE_MEAN && !(mean_divisor > 0.0)) return FDL_ERR_INVALID_ARGUMENT;
    if (batch > 65535) return FDL_ERR_UNSUPPORTED;
    int status = FDL_OK;
    const DeviceInfo* info = current_device_info(&status);
    if (info == nullptr) return status;

    const bool vec = aligned16(x) && cols % 4 == 0;
    if (rows <= kFewRows && xc.world == 0) {
        const bool vec_few = vec && aligned16(out);  // this kernel also stores 128 bits at a time
        const float few_scale = op == FDL_REDUCE_MEAN ? static_cast<float>(1.0 / mean_divisor) : 1.0f;
        cudaStream_t st = as_stream(stream);
        if (op == FDL_REDUCE_MAX) {
            return vec_few ? launch_cols_few<ColMax, 4>(x, batch, rows, cols, out, few_scale, st)
                       : launch_cols_few<ColMax, 1>(x, batch, rows, cols, out, few_scale, st);
        }
        return vec_few ? launch_cols_few<ColSum, 4>(x, batch, rows, cols, out, few_scale, st)
                   : launch_cols_few<ColSum, 1>(x, batch, rows, cols, out, few_scale, st);
    }
    if (!vec && aligned16(x) && xc.world == 0 && cols_regroup_applies(batch, rows, cols)) {
        const int gf = regroup_factor(cols);
        const int64_t grouped_rows = rows / gf, grouped_cols = gf * cols;
        const size_t need = regroup_scratch_bytes(rows, cols);
        if (scratch == nullptr) {
            status = get_workspace(need, &scratch);
            if (status != FDL_OK) return status;
        } else if (scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) {
            return FDL_ERR_WORKSPACE;
        }
        const size_t inner = regroup_inner_bytes(rows, cols);
        float* grouped = reinterpret_cast<float*>(static_cast<char*>(scratch) + inner);
        status = reduce_cols_impl(x, 1, grouped_rows, grouped_cols, grouped, op == FDL_REDUCE_MAX ? FDL_REDUCE_MAX : FDL_REDUCE_SUM,
                                  1.0, scratch, inner, stream, xc);
        if (status != FDL_OK) return status;
        const float fscale = op == FDL_REDUCE_MEAN ? static_cast<float>(1.0 / mean_divisor) : 1.0f;
        const int leftover = static_cast<int>(rows - grouped_rows * gf);
        const float* rest = x + grouped_rows * gf * cols;
        const dim3 fgrid(static_cast<unsigned int>(ceil_div(cols, 256))), fblock(256), one(1, 1, 1);
        const bool pdl = tuning().pdl != 0;
        return op == FDL_REDUCE_MAX
                   ? launch_ex(cols_regroup_finish_kernel<ColMax>, fgrid, fblock, 0, as_stream(stream), one, pdl,
                               static_cast<const float*>(grouped), gf, cols, rest, leftover, out, fscale)
                   : launch_ex(cols_regroup_finish_kernel<ColSum>, fgrid, fblock, 0, as_stream(stream), one, pdl,
                               static_cast<const float*>(grouped), gf, cols, rest, leftover, out, fscale);
    }
    ColsGeometry g;
    status = cols_geometry(info->sm_count, batch, rows, cols, vec, &g);
    if (status != FDL_OK) return status;
    float* partials = nullptr;
    unsigned int* counters = nullptr;
    if (g.chunks / g.cluster > 1) {
        if (scratch == nullptr) {
            status = get_workspace(g.scratch_bytes, &scratch);
            if (status != FDL_OK) return status;
        } else if (scratch_bytes < g.scratch_bytes ||
                   (reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) {
            return FDL_ERR_WORKSPACE;
        }
        counters = static_cast<unsigned int*>(scratch);
        partials = reinterpret_cast<float*>(static_cast<char*>(scratch) + g.counter_bytes);
    }
    const float scale = op == FDL_REDUCE_MEAN ? static_cast<float>(1.0 / mean_divisor) : 1.0f;
    const dim3 grid(g.col_blocks, g.chunks, static_cast<unsigned int>(batch)), block(kColThreads), cluster(1, g.cluster, 1);
    const size_t smem = static_cast<size_t>(kColThreads) * 4 * sizeof(float);
    const bool pdl = tuning().pdl != 0;
    cudaStream_t st = as_stream(stream);
    const bool is_max = op == FDL_REDUCE_MAX;
    int launched = FDL_OK;
#define FDL_LAUNCH_COLS(R, W, CL)                                                                           \
    launched = launch_ex(reduce_cols_kernel<R, W, CL>, grid, block, smem, st, cluster, pdl, x, rows, cols, out, \
                         partials, counters, g.tx, g.rows_per_chunk, scale, xc)
#define FDL_LAUNCH_COLS_CL(CL)                                                                  \
    do {                                                                                        \
        if (is_max) { if (vec) FDL_LAUNCH_COLS(ColMax, 4, CL); else FDL_LAUNCH_COLS(ColMax, 1, CL); } \
        else { if (vec) FDL_LAUNCH_COLS(ColSum, 4, CL); else FDL_LAUNCH_COLS(ColSum, 1, CL); }  \
    } while (0)
    switch (g.cluster) {
        case 16: {  // beyond the portable cluster size: every instantiation has to opt in
            cudaFuncSetAttribute(reduce_cols_kernel<ColMax, 4, 16>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            cudaFuncSetAttribute(reduce_cols_kernel<ColMax, 1, 16>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            cudaFuncSetAttribute(reduce_cols_kernel<ColSum, 4, 16>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            cudaFuncSetAttribute(reduce_cols_kernel<ColSum, 1, 16>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            FDL_LAUNCH_COLS_CL(16);
            break;
        }
        case 8: FDL_LAUNCH_COLS_CL(8); break;
        case 4: FDL_LAUNCH_COLS_CL(4); break;
        case 2: FDL_LAUNCH_COLS_CL(2); break;
        default: FDL_LAUNCH_COLS_CL(1); break;
    }
#undef FDL_LAUNCH_COLS_CL
#undef FDL_LAUNCH_COLS
    return launched;
}

int fdl_reduce_cols_f32(const float* x, int64_t batch, int64_t rows, int64_t cols, float* out,
                        int op, double mean_divisor, void* scratch, size_t scratch_bytes,
                        void* stream) {
    return reduce_cols_impl(x, batch, rows, cols, out, op, mean_divisor, scratch, scratch_bytes, stream,
                            ColsExchange());
}

}  // extern "C"

// ======================================================================================
// Full sum across the GPUs of one box: the exchange context and the fused entry point
// ======================================================================================

namespace fdl {
namespace {

constexpr size_t kExchangeSumBytes = 4096;  // the full sum's words, then the column-vector region

size_t exchange_bytes(int world) {
    return kExchangeSumBytes + 2 * static_cast<size_t>(world) * kExchangeMaxCols * sizeof(unsigned long long);
}

struct ExchangeContext {
    int world = 0;
    int rank = 0;
    int device = 0;
    unsigned int epoch = 0;      // full-sum exchanges so far
    unsigned int epoch_cols = 0; // column-vector exchanges so far
    bool sum_pending = false;    // a split-phase full sum has started and not finished
    void* local = nullptr;
    void* peer[kMaxRanks] = {};
    bool connected = false;
    bool by_pointer = false;  // peers were given as device pointers (same process): nothing to close
};

}  // namespace
}  // namespace fdl

extern "C" {

int fdl_exchange_create(int world, int rank, void** ctx_out) {
    if (ctx_out == nullptr || world < 1 || world > kMaxRanks || rank < 0 || rank >= world) {
        return FDL_ERR_INVALID_ARGUMENT;
    }
    auto* ctx = new ExchangeContext();
    ctx->world = world;
    ctx->rank = rank;
    cudaError_t e = cudaGetDevice(&ctx->device);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->local, exchange_bytes(world));
    if (e == cudaSuccess) e = cudaMemset(ctx->local, 0, exchange_bytes(world));
    if (e != cudaSuccess) {
        delete ctx;
        return static_cast<int>(e);
    }
    ctx->peer[rank] = ctx->local;
    ctx->connected = world == 1;
    *ctx_out = ctx;
    return FDL_OK;
}

int fdl_exchange_local_handle(void* ctx_in, unsigned char* handle64) {
    auto* ctx = static_cast<ExchangeContext*>(ctx_in);
    if (ctx == nullptr || handle64 == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, ctx->local);
    if (e != cudaSuccess) return static_cast<int>(e);
    memcpy(handle64, &h, 64);
    return FDL_OK;
}

int fdl_exchange_connect(void* ctx_in, const unsigned char* handles) {
    auto* ctx = static_cast<ExchangeContext*>(ctx_in);
    if (ctx == nullptr || handles == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    for (int p = 0; p < ctx->world; ++p) {
        if (p == ctx->rank || ctx->peer[p] != nullptr) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + 64 * p, 64);
        const cudaError_t e = cudaIpcOpenMemHandle(&ctx->peer[p], h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    ctx->connected = true;
    return FDL_OK;
}

int fdl_exchange_buffer(void* ctx_in, void** buffer_out) {
    auto* ctx = static_cast<ExchangeContext*>(ctx_in);
    if (ctx == nullptr || buffer_out == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    *buffer_out = ctx->local;
    return FDL_OK;
}

int fdl_exchange_connect_pointers(void* ctx_in, void* const* buffers) {
    auto* ctx = static_cast<ExchangeContext*>(ctx_in);
    if (ctx == nullptr || buffers == nullptr || ctx->connected) return FDL_ERR_INVALID_ARGUMENT;
    for (int p = 0; p < ctx->world; ++p) {
        if (buffers[p] == nullptr || (p == ctx->rank && buffers[p] != ctx->local)) return FDL_ERR_INVALID_ARGUMENT;
    }
    for (int p = 0; p < ctx->world; ++p) ctx->peer[p] = buffers[p];
    ctx->by_pointer = true;
    ctx->connected = true;
    return FDL_OK;
}

int fdl_exchange_destroy(void* ctx_in) {
    auto* ctx = static_cast<ExchangeContext*>(ctx_in);
    if (ctx == nullptr) return FDL_OK;
    cudaDeviceSynchronize();
    for (int p = 0; p < ctx->world && !ctx->by_pointer; ++p) {
        if (p != ctx->rank && ctx->peer[p] != nullptr) cudaIpcCloseMemHandle(ctx->peer[p]);
    }
    cudaFree(ctx->local);
    delete ctx;
    return FDL_OK;
}

static int sum_exchange_fill(ExchangeContext* ctx, SumExchange* xc) {
    xc->world = ctx->world;
    xc->rank = ctx->rank;
    xc->epoch = ctx->epoch;
    xc->wait_ns = static_cast<unsigned long long>(tuning().exchange_wait_ms) * 1000000ull;
    for (int p = 0; p < ctx->world; ++p) xc->words[p] = static_cast<unsigned long long*>(ctx->peer[p]);
    return error_flag_device_ptr(&xc->error_flag);
}

static int sum_allreduce_launch(const float* x, int64_t n, float* out_f32, double* out_f64,
                                ExchangeContext* ctx, void* scratch, size_t scratch_bytes, void* stream,
                                bool send_only) {
    if (ctx == nullptr || !ctx->connected || ctx->sum_pending) return FDL_ERR_INVALID_ARGUMENT;
    if (n < 0 || (!send_only && out_f32 == nullptr && out_f64 == nullptr)) return FDL_ERR_INVALID_ARGUMENT;
    if (n > 0 && x == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    int status = FDL_OK;
    const size_t need = fdl_sum_scratch_bytes(n);
    if (scratch == nullptr) {
        status = get_workspace(need, &scratch);
        if (status != FDL_OK) return status;
    } else if (scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) {
        return FDL_ERR_WORKSPACE;
    }
    ctx->epoch += 1;
    if (ctx->epoch == 0) ctx->epoch = 1;  // 0 is the buffers' initial state
    SumExchange xc;
    status = sum_exchange_fill(ctx, &xc);
    if (status != FDL_OK) return status;
    xc.send_only = send_only ? 1 : 0;
    unsigned int* counter = static_cast<unsigned int*>(scratch);
    double* partials = reinterpret_cast<double*>(static_cast<char*>(scratch) + kCounterBytes);
    cudaStream_t s = as_stream(stream);
    status = aligned16(x) ? launch_sum<4, true>(x, n, out_f32, out_f64, counter, partials, s, xc)
                          : launch_sum<1, false>(x, n, out_f32, out_f64, counter, partials, s, xc);
    if (status == FDL_OK && send_only) ctx->sum_pending = true;
    return status;
}

int fdl_sum_allreduce_f32(const float* x, int64_t n, float* out_f32, double* out_f64, void* ctx_in,
                          void* scratch, size_t scratch_bytes, void* stream) {
    return sum_allreduce_launch(x, n, out_f32, out_f64, static_cast<ExchangeContext*>(ctx_in), scratch,
                                scratch_bytes, stream, false);
}

int fdl_sum_allreduce_start_f32(const float* x, int64_t n, void* ctx_in, void* scratch, size_t scratch_bytes,
                                void* stream) {
    return sum_allreduce_launch(x, n, nullptr, nullptr, static_cast<ExchangeContext*>(ctx_in), scratch,
                                scratch_bytes, stream, true);
}

int fdl_sum_allreduce_finish_f32(float* out_f32, double* out_f64, void* ctx_in, void* stream) {
    auto* ctx = static_cast<ExchangeContext*>(ctx_in);
    if (ctx == nullptr || !ctx->connected || !ctx->sum_pending) return FDL_ERR_INVALID_ARGUMENT;
    if (out_f32 == nullptr && out_f64 == nullptr) return FDL_ERR_INVALID_ARGUMENT;
    SumExchange xc;
    const int status = sum_exchange_fill(ctx, &xc);
    if (status != FDL_OK) return status;
    sum_exchange_finish_kernel<<<1, kWarp, 0, as_stream(stream)>>>(out_f32, out_f64, xc);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    ctx->sum_pending = false;
    return FDL_OK;
}

int fdl_reduce_cols_allreduce_f32(const float* x, int64_t rows, int64_t cols, float* out, int op,
                                  double mean_divisor, void* ctx_in, void* scratch, size_t scratch_bytes,
                                  void* stream) {
    auto* ctx = static_cast<ExchangeContext*>(ctx_in);
    if (ctx == nullptr || !ctx->connected) return FDL_ERR_INVALID_ARGUMENT;
    if (cols > kExchangeMaxCols) return FDL_ERR_UNSUPPORTED;
    if (rows <= 0 || cols <= 0) return FDL_ERR_INVALID_ARGUMENT;  // collective: every rank must launch
    ColsExchange xc;
    xc.world = ctx->world;
    xc.rank = ctx->rank;
    ctx->epoch_cols += 1;
    if (ctx->epoch_cols == 0) ctx->epoch_cols = 1;
    xc.epoch = ctx->epoch_cols;
    xc.wait_ns = static_cast<unsigned long long>(tuning().exchange_wait_ms) * 1000000ull;
    for (int p = 0; p < ctx->world; ++p) {
        xc.words[p] = reinterpret_cast<unsigned long long*>(static_cast<char*>(ctx->peer[p]) + kExchangeSumBytes);
    }
    const int status = error_flag_device_ptr(&xc.error_flag);
    if (status != FDL_OK) return status;
    return reduce_cols_impl(x, 1, rows, cols, out, op, mean_divisor, scratch, scratch_bytes, stream, xc);
}

}  // extern "C"
