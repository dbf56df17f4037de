/*
 * fdl_kernels.h -- C ABI of the sm_100a kernel library (libfdl_kernels.so).
 *
 * This is the drop-in boundary for fast_dl's bandwidth-bound tensor path.  Every
 * entry point replaces (or extends in the same style) one host-callable function of
 * the reference's kernel library; the reference location is cited above each
 * declaration as <file>:<lines>, relative to the fast_dl source tree.
 *
 * Conventions shared by all entry points
 *   - Plain pointers and sizes only; nothing here depends on PyTorch or C++.
 *   - All data pointers are DEVICE pointers of the current device unless a name
 *     starts with `h_` (host pointers, only in the fdl_host_* family).
 *   - `stream` is a cudaStream_t passed as void*; NULL selects the legacy default
 *     stream, which is what the reference launches on.
 *   - The caller selects the device beforehand (fdl_set_device or cudaSetDevice in
 *     the same CUDA runtime), exactly as the reference's ops do before calling
 *     dl::kernels::*.
 *   - Return value: 0 (FDL_OK) on success; a positive value is a cudaError_t from
 *     the launch; a negative value is one of the FDL_ERR_* codes below.  Nothing
 *     throws and nothing falls back to a CPU path.
 *   - Launches are asynchronous with respect to the host, like the reference's.
 *   - Stream capture: the device-pointer entry points enqueue kernels on `stream` and
 *     nothing else, so a chain of them can be captured into a CUDA graph and replayed.
 *     An op's first use on a device may allocate the library's workspace, so run the
 *     chain once eagerly (or pass your own scratch) before the capture begins.  The
 *     cross-GPU entry points (fdl_*_allreduce_*) pass a per-call epoch as a kernel
 *     argument and must not be captured; the fdl_host_* family synchronises internally
 *     and cannot be.
 *   - Element counts are int64_t.  The reference takes `int`/`size_t`; the C++
 *     shims in dl::kernels keep those narrower types and widen here.
 */
#ifndef FDL_KERNELS_H_
#define FDL_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The library is built with hidden visibility; only the entry points declared here are exported. */
#if defined(FDL_BUILDING_LIBRARY) && defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define FDL_OK 0
#define FDL_ERR_INVALID_ARGUMENT (-1) /* null pointer, negative size, bad enum          */
#define FDL_ERR_UNSUPPORTED (-2)      /* shape outside what the entry point implements   */
#define FDL_ERR_WORKSPACE (-3)        /* caller-provided scratch too small or misaligned */
#define FDL_ERR_DEVICE_WAIT (-4)      /* a bounded device-side wait ran out              */
#define FDL_ERR_NO_DEVICE (-5)        /* no usable CUDA device / driver                  */
#define FDL_ERR_TOO_LARGE_FOR_STATIC_SCRATCH (-6) /* n above fdl_sum_f32_static's maximum */

/* Binary operator selector; numeric values equal dl::kernels::ElementwiseOp
 * (include/dl/kernels/elementwise.hpp:7-12). */
enum fdl_binary_op { FDL_ADD = 0, FDL_SUB = 1, FDL_MUL = 2, FDL_DIV = 3 };

/* Unary operator selector; numeric values equal dl::kernels::ActivationOp
 * (include/dl/kernels/activation.hpp:7-13). */
enum fdl_unary_op {
    FDL_RELU = 0,
    FDL_LEAKY_RELU = 1,
    FDL_GELU = 2,
    FDL_SIGMOID = 3,
    FDL_TANH = 4
};

/* Reduction selector for the axis reductions (no counterpart enum in the reference,
 * which has no axis reductions). */
enum fdl_reduce_op { FDL_REDUCE_SUM = 0, FDL_REDUCE_MEAN = 1, FDL_REDUCE_MAX = 2 };

/* Tree order selector; numeric values equal dl::kernels::ReductionAlgo
 * (include/dl/kernels/reduction.hpp:7-10). */
enum fdl_block_tree { FDL_TREE_INTERLEAVE = 0, FDL_TREE_ADDRESS = 1 };

/* ---- runtime -------------------------------------------------------------------- */

/* Library ABI version: major*1000 + minor. */
int fdl_version(void);

/* Human-readable text for any value returned by this library (FDL_ERR_* or a
 * cudaError_t).  Never NULL.  Plays the role of the message half of
 * dl::cuda::check (src/core/CudaUtils.cpp:8-13). */
const char* fdl_error_string(int status);

/* Number of visible CUDA devices, or a negative FDL_ERR_* code. */
int fdl_device_count(void);

/* Make `device` current for the calling thread in the library's CUDA runtime.
 * Replaces the cudaSetDevice call the reference's ops make before each kernel
 * (e.g. src/ops/Elementwise.cpp:41). */
int fdl_set_device(int device);

/* Block the host until `stream` has drained. */
int fdl_stream_synchronize(void* stream);

/* Kernels that wait on the copy engine bound every wait; one that gives up raises a
 * flag in host-visible memory instead of spinning.  This returns FDL_ERR_DEVICE_WAIT if
 * the flag was raised since the last call (and clears it), else FDL_OK.  Meaningful
 * after the stream has been synchronised; when it reports a wait that ran out it also
 * zeroes the arrival counters in the library's own workspace, which a kernel that gave up
 * may have left half-way, so the calls that follow start clean. */
int fdl_take_device_error(void);

/* Measurement aid: selects a launch shape so that a bench can show, on the same build,
 * why the default was chosen.  Keys: "sum_cluster" (1, 2, 4 or 8 CTAs per cluster in the
 * full sum; default 4), "rows_split_fused" (softmax/layernorm rows longer than a
 * cluster holds: 1 = one kernel whose statistics and apply tasks are pipelined through L2,
 * 0 = two kernels, the rows read twice from DRAM; default 1), "rows_split_lag" (rows between a
 * row's statistics and its apply tasks in that kernel, 1..4096; 0 = 36 MiB of rows; default 0),
 * "rows_split_hints" (1 = L2 eviction-priority hints on that kernel's loads, 0 = plain streaming
 * loads; default 1), "rows_split_from" (> 0: rows of at least this many floats take the split
 * form instead of the cluster forms; default 0),
 * "sum_tiles" (32 KiB tiles a CTA of the full sum walks, 1..64; 0 = two
 * from 256 MiB on, one below; default 0; applies to every full-sum entry point), "rows_staged" (0 = softmax/layernorm rows loaded straight into
 * registers, 1 = staged through shared memory by one bulk-async copy per CTA, -1 = staged
 * for rows of up to 128 floats and direct beyond; default -1), "rows_warp16" (rows of
 * 1028..2048 floats: 1 = one warp per row with 16 packs a lane, 0 = a 256-thread CTA per row,
 * -1 = whichever measured faster for the op and length; default -1), "rows_cluster_threads"
 * (256 or 512 threads per CTA in the cluster form of rows of 16388..65536 floats; default 256),
 * "rows_span_reduce_cols" (the same for the row reductions sum / mean / max / argmax along axis 1;
 * 0..2048, default 2048), "rows_span_argmax_from" (argmax along axis 1 takes that form from rows
 * of this many floats on; default 65),
 * "rows_span_cols" (rows of up to this many floats whose length is not a multiple of 4, or whose
 * base is off the 16-byte grid, are staged as runs of rows through shared memory; 0..256, default 256),
 * "rows_smem" (1 = rows beyond 65536 floats, or beyond 16384 at odd lengths, are kept in a
 * cluster's shared memory and read once; 0 = the register-cluster and two-kernel forms; default 1),
 * "rows_smem_cluster" (CTAs per row in that form: 2, 4, 8, 16, or 0 = by row length; default 0),
 * "rows_smem_from" (aligned rows longer than this many floats take that form; 0 = 65536, default),
 * and for the column reductions "cols_tx" (threads across columns per CTA: 16..256; default
 * 64), "cols_cluster" (1, 2, 4, 8, 16, or 0 = 8 with 128-bit loads and 2 with 32-bit loads; default
 * 0), "cols_ctas_per_sm" (default 4) and
 * "cols_chunks" (row chunks per column block; 0 = derived from cols_ctas_per_sm, default),
 * "cols_single" (1 = where the shape allows, one cluster of 8 CTAs covers all rows of a column
 * block and nothing goes through scratch; 0 = always the chunked form; default 1), "cols_regroup"
 * (1 = a matrix whose column count is not a multiple of 4 is reduced as [rows / 4, 4 * cols] with
 * 128-bit loads and its results folded by a second, small kernel; 0 = 32-bit loads; default 1);
 * "pdl" (1 = the streaming kernels are launched with programmatic stream serialization, so
 * that the next kernel's launch overlaps the tail of the one before; 0 = plain launches;
 * default 1), "bcast2d" (1 = two-dimensional broadcasts take the division-free kernel;
 * default 1) and "bcast2d_rows" (rows per thread there: 1, 2, 4, or 0 = by size).
 * Two keys are not launch shapes: "exchange_wait_ms" (1..60000, default 2000) is how long a
 * cross-GPU exchange waits for its peers before it gives up, and "sum_trace" (0 / 1) makes the
 * full sum's finishing CTA record time stamps for fdl_debug_sum_trace.
 * Not part of the reference's interface. */
int fdl_set_tuning(const char* key, int value);

/* Measurement aid: with the tuning key "sum_trace" set, the CTA that finishes a full sum
 * (fdl_sum_f32, fdl_sum_allreduce_f32) leaves eight 64-bit words in host-visible memory; this
 * copies the words of the most recent such kernel.  Words 0-5 are %globaltimer values in
 * nanoseconds: [0] first CTA started, [1] last cluster arrived (ticket taken), [2] partials
 * folded, [3] partial sent to the peers, [4] all peers' partials seen, [5] result written
 * ([3], [4] only with an exchange); [6] SM cycles from [1] to [5]; [7] the exchange epoch.
 * Read after the stream has been synchronised.  Not part of the reference's interface. */
int fdl_debug_sum_trace(unsigned long long* out8);

/* ---- elementwise ------------------------------------------------------------------ */

/* out[i] = a[i] (op) b[i], i in [0,n).  IEEE round-to-nearest for all four operators;
 * `out` may alias `a` or `b` exactly.  Replaces dl::kernels::elementwise
 * (include/dl/kernels/elementwise.hpp:16, src/kernels/cuda/elementwise.cu:5-31,51-54)
 * and, with op = FDL_ADD, dl::kernels::vector_add
 * (include/dl/kernels/vector_add.hpp:13-14, src/kernels/cuda/vector_add.cu:7-21,35-42). */
int fdl_binary_f32(const float* a, const float* b, float* out, int64_t n, int op,
                   void* stream);

/* out[i] = f(x[i]).  `alpha` is read only by FDL_LEAKY_RELU.  Formulas are the
 * reference's: relu fmaxf(0,x); leaky x>0?x:alpha*x; gelu tanh approximation with
 * 0.79788456 and 0.044715; sigmoid 1/(1+expf(-x)); tanh tanhf(x).  Replaces
 * dl::kernels::activation (include/dl/kernels/activation.hpp:17,
 * src/kernels/cuda/activation.cu:6-94). */
int fdl_unary_f32(const float* x, float* out, int64_t n, int op, float alpha,
                  void* stream);

/* out[i] = max(0, fl(fl(a[i]*b[i]) + c[i])): the chain relu(a*b + c) in one pass with
 * the two roundings the reference's three separate kernels produce (no FMA).
 * Fuses ops::mul -> ops::add -> ops::relu (src/ops/Elementwise.cpp:36-50,
 * src/ops/Activation.cpp:13-28). */
int fdl_mul_add_relu_f32(const float* a, const float* b, const float* c, float* out,
                         int64_t n, void* stream);

/* In place: out[r*cols + c] += bias[c].  Replaces dl::kernels::add_row_bias
 * (include/dl/kernels/bias.hpp:5, src/kernels/cuda/bias.cu:5-28). */
int fdl_add_row_bias_f32(float* out, const float* bias, int64_t rows, int64_t cols,
                         void* stream);

/* In place: out[r*cols + c] = max(0, out[r*cols + c] + bias[c]): the bias epilogue of
 * ops::linear followed by nn::ReLU in one pass (src/ops/Linear.cpp:38-45,
 * src/nn/ReLU.cpp:7-9). */
int fdl_add_row_bias_relu_f32(float* out, const float* bias, int64_t rows, int64_t cols,
                              void* stream);

/* Broadcasting binary op.  `ndim` (1..8) dimensions, `shape` is the OUTPUT shape,
 * `a_strides`/`b_strides` are element strides of each operand per output dimension
 * with 0 in broadcast dimensions (NumPy rules; the host precomputes them).  The
 * output is contiguous row-major.  The library collapses dimensions and derives
 * division-free index arithmetic on the host before launching.
 * The reference has no general broadcast (its binary ops demand equal shapes,
 * src/ops/OpUtils.cpp:74-101); its one broadcast is the row-bias kernel
 * (src/kernels/cuda/bias.cu:5-12), of which this is the out-of-place generalisation. */
int fdl_broadcast_binary_f32(const float* a, const float* b, float* out, int ndim,
                             const int64_t* shape, const int64_t* a_strides,
                             const int64_t* b_strides, int op, void* stream);

/* ---- reductions ------------------------------------------------------------------- */

/* out[k] = sum of x[1024k .. 1024k+1023] for k in [0, n/1024) with the exact pairing
 * order of the reference's shared-memory trees, so results are bit-identical to them:
 * FDL_TREE_ADDRESS pairs (i, i+s) for s = 512..1, FDL_TREE_INTERLEAVE for s = 1..512.
 * A tail of n % 1024 elements is ignored, as in the reference.  Replaces
 * dl::kernels::reduction (include/dl/kernels/reduction.hpp:14-15,
 * src/kernels/cuda/reduction.cu:8-57,75-85). */
int fdl_block_reduce_1024_f32(const float* x, float* out, int64_t n, int tree,
                              void* stream);

/* Scratch bytes fdl_sum_f32 / fdl_reduce_cols_f32 need for the given problem: a fixed
 * 64 KiB region of arrival counters followed by the partial results.  Always a multiple of
 * 256; the scratch pointer must be 256-byte aligned. */
size_t fdl_sum_scratch_bytes(int64_t n);
size_t fdl_reduce_cols_scratch_bytes(int64_t batch, int64_t rows, int64_t cols);

/* out_f32[0] = sum of x[0..n).  If out_f64 is not NULL it also receives the sum
 * before the final rounding to float (what a multi-GPU caller all-reduces).
 * Deterministic: same input, same launch -> same bits.  `scratch` may be NULL, in
 * which case the library uses a per-device workspace it allocates on first use and
 * keeps; otherwise it must hold fdl_sum_scratch_bytes(n), be 256-byte aligned, and have had
 * its first 65,536 bytes zeroed once (the kernels leave them zero; the same buffer may then
 * serve fdl_sum_f32 and fdl_reduce_cols_f32 calls of any shape).  Calls that may overlap on
 * the GPU (different streams) must not share scratch: pass each its own.  No counterpart in the
 * reference, whose reduction stops at one partial per 1024 elements
 * (src/kernels/cuda/reduction.cu:34-57). */
int fdl_sum_f32(const float* x, int64_t n, float* out_f32, double* out_f64,
                void* scratch, size_t scratch_bytes, void* stream);

/* Full sum for callers that cannot allocate device memory: a host framework whose own
 * allocator must account for every device byte, a service whose device-memory budget is
 * fixed at start-up, or latency-critical code that must not enter the driver's allocator
 * (cudaMalloc and cudaFree synchronise the device).  Same result as fdl_sum_f32 at its default
 * launch shape (clusters of 4; the tuning key "sum_cluster" does not apply here), but the scratch is a fixed 65,792-byte
 * array in the library's device image instead of caller- or library-allocated memory, and
 * the call performs no cudaMalloc/cudaFree or any other allocating routine.
 *   - n may be at most 2^30 (1,073,741,824) elements; larger n returns
 *     FDL_ERR_TOO_LARGE_FOR_STATIC_SCRATCH without launching anything.
 *   - The first call on each device looks the array's device address up (one
 *     cudaGetSymbolAddress with that device current); make that first call before any
 *     stream capture begins.  The address is kept for the life of the device's primary
 *     context: after a cudaDeviceReset the library must be reloaded.
 *   - All calls on a device share the one array: the arrival counter in it is cleared on
 *     the stream at the start of every call, and two calls whose kernels may overlap on
 *     the GPU (different streams without an ordering between them) race on it.  Serialise
 *     them, or use fdl_sum_f32 with separate scratch buffers.
 * This entry point has no counterpart in the reference. */
int fdl_sum_f32_static(const float* x, int64_t n, float* out_f32, double* out_f64,
                       void* stream);

/* ---- full sum across the GPUs of one box (one process per GPU) ------------------------------
 *
 * fdl_sum_allreduce_f32 is fdl_sum_f32 plus the exchange of the per-GPU partials, in ONE
 * kernel: the CTA that finishes a rank's sum stores the partial into a small buffer of every
 * peer over NVLink (plain 8-byte peer stores that carry an epoch tag, no multicast), waits --
 * at most two seconds (tuning key "exchange_wait_ms") -- for the peers' tagged values in its own buffer and adds them in rank order,
 * so every rank ends with the same bits and no separate collective kernel is launched.
 * A wait that runs out writes NaN to the outputs and raises the flag read by
 * fdl_take_device_error; it never hangs.
 *
 * Set-up, once per process: fdl_exchange_create (allocates this rank's buffer, 4 KiB + 1 MiB per rank, on the
 * current device) -> fdl_exchange_local_handle (64-byte CUDA IPC handle) -> all-gather the
 * handles with any host mechanism -> fdl_exchange_connect(world * 64 bytes, rank order).
 * Calls are collective: every rank must call fdl_sum_allreduce_f32 the same number of
 * times in the same order.  At most 16 ranks.  No counterpart in the reference (which has
 * no multi-GPU code at all). */
int fdl_exchange_create(int world, int rank, void** ctx_out);
int fdl_exchange_local_handle(void* ctx, unsigned char* handle64);
int fdl_exchange_connect(void* ctx, const unsigned char* handles);
/* For ranks that live in ONE process (one host thread driving several GPUs with peer access
 * enabled, or several contexts on one GPU): fdl_exchange_buffer returns the device pointer of
 * a context's own buffer, and fdl_exchange_connect_pointers takes all ranks' buffers, in rank
 * order, in place of the IPC handles.  No counterpart in the reference. */
int fdl_exchange_buffer(void* ctx, void** buffer_out);
int fdl_exchange_connect_pointers(void* ctx, void* const* buffers);
int fdl_exchange_destroy(void* ctx);
int fdl_sum_allreduce_f32(const float* x, int64_t n, float* out_f32, double* out_f64, void* ctx,
                          void* scratch, size_t scratch_bytes, void* stream);

/* The same exchange in two halves, so that other work can run while the partials cross
 * NVLink and while slower ranks catch up.  fdl_sum_allreduce_start_f32 launches the sum
 * kernel, whose last CTA sends this rank's partial to every rank and returns without
 * waiting; fdl_sum_allreduce_finish_f32 launches a one-warp kernel that waits (at most two
 * seconds, then NaN + the device-error flag) for all ranks' partials of that exchange and
 * adds them in rank order - the same bits as fdl_sum_allreduce_f32 on every rank.  Kernels
 * enqueued on `stream` between the two calls overlap the exchange.  Per context, start and
 * finish must alternate (a second start, or fdl_sum_allreduce_f32, before the finish returns
 * FDL_ERR_INVALID_ARGUMENT, as does a finish with nothing started); both halves of one
 * exchange go to the same stream, or to streams the caller has ordered.  Collective, same
 * ordering rule as above.  No counterpart in the reference. */
int fdl_sum_allreduce_start_f32(const float* x, int64_t n, void* ctx, void* scratch,
                                size_t scratch_bytes, void* stream);
int fdl_sum_allreduce_finish_f32(float* out_f32, double* out_f64, void* ctx, void* stream);

/* fdl_reduce_cols_f32 (one matrix) plus the exchange of the per-GPU [cols] results, in one
 * kernel and with the same protocol: the CTA that finishes a block of columns sends each
 * column's value to every rank as an 8-byte {float, epoch} peer store and folds all ranks'
 * values in rank order.  x is this rank's [rows, cols] row block; for FDL_REDUCE_MEAN pass
 * the GLOBAL row count as mean_divisor.  Every rank ends with the same out[cols].
 * cols <= 65536.  Collective, same ordering rule as above. */
int fdl_reduce_cols_allreduce_f32(const float* x, int64_t rows, int64_t cols, float* out, int op,
                                  double mean_divisor, void* ctx, void* scratch,
                                  size_t scratch_bytes, void* stream);

/* Row-wise reduction of a row-major [rows, cols] matrix along axis 1:
 * out[r] = op over c of x[r, c]; FDL_REDUCE_MAX ignores NaNs like fmaxf.  No counterpart
 * in the reference (row max / row sum exist only inside its softmax,
 * src/kernels/cuda/softmax.cu:157-221). */
int fdl_reduce_rows_f32(const float* x, int64_t rows, int64_t cols, float* out, int op,
                        void* stream);

/* out[r] = lowest column index of the row maximum (NaN compares as -inf).  int64
 * output.  No counterpart in the reference.
 * Both row reductions pick a kernel by shape: teams of lanes with several rows in flight for
 * rows of up to 256 floats, a warp or a CTA per row beyond, and -- for fewer than 1184 rows of
 * at least 256 KiB -- one CTA per 64 KiB segment with the segments' results folded per row
 * through the library's per-device workspace (allocated on first use; such calls must not
 * overlap on the GPU with other calls that use the workspace). */
int fdl_argmax_rows_f32(const float* x, int64_t rows, int64_t cols, int64_t* out,
                        void* stream);

/* Column-wise reduction along axis 0 of `batch` stacked row-major [rows, cols]
 * matrices: out[b, c] = scale-free op over r of x[b, r, c].  FDL_REDUCE_MEAN divides
 * by `mean_divisor` (pass rows, or the global row count when rows are one shard of a
 * larger tensor and the caller all-reduces sums itself).  Scratch as in fdl_sum_f32.
 * No counterpart in the reference. */
int fdl_reduce_cols_f32(const float* x, int64_t batch, int64_t rows, int64_t cols,
                        float* out, int op, double mean_divisor, void* scratch,
                        size_t scratch_bytes, void* stream);

/* ---- row-wise normalisations ---------------------------------------------------------- */

/* y[r, c] = exp(x[r, c] - max_r) * (1 / sum_c exp(x[r, c] - max_r)).  Replaces
 * dl::kernels::softmax for every SoftmaxAlgo value (include/dl/kernels/softmax.hpp:15-16,
 * src/kernels/cuda/softmax.cu:28-254,272-285).
 * Both row-wise normalisations read a row once and write it once up to 131072 floats per row
 * (registers of one CTA up to 16384 floats; beyond, the registers -- or, for row lengths that
 * are not a multiple of 4 floats or bases off the 16-byte grid, the shared memory -- of a
 * thread-block cluster of 2, 4 or 8 CTAs); longer rows take two kernels (per-segment statistics
 * combined per row through the library's workspace, then applied: two reads, one write). */
int fdl_softmax_rows_f32(const float* x, float* y, int64_t rows, int64_t cols,
                         void* stream);

/* y[r, c] = (x[r, c] - mean_r) * rstd_r * gamma[c] + beta[c] with
 * rstd_r = 1/sqrt(var_r + eps), biased variance.  gamma and beta may each be NULL
 * (treated as 1 and 0), which gives the reference's affine-free form.  If `mean_out` /
 * `rstd_out` are not NULL they receive the per-row statistics.  Replaces
 * dl::kernels::layernorm (include/dl/kernels/layernorm.hpp:5-6,
 * src/kernels/cuda/layernorm.cu:9-78). */
int fdl_layernorm_rows_f32(const float* x, const float* gamma, const float* beta,
                           float* y, float* mean_out, float* rstd_out, int64_t rows,
                           int64_t cols, float eps, void* stream);

/* Test aid, host only (no launch): the task that ticket `ticket` names in the one-launch form
 * of softmax / layernorm on rows longer than a cluster holds -- `rows` rows of `segments` 32 KiB
 * segments, the apply pass `lag` rows (1..rows) behind the statistics pass; tickets run from 0
 * to 2 * rows * segments - 1.  The kernel decodes its tickets with the same function.  What the
 * enumeration has to guarantee: every (row, segment, pass) exactly once, and every apply task
 * of a row after all of that row's statistics tasks, so that a task only waits for tasks that
 * CTAs which started earlier hold. */
int fdl_debug_split_ticket(int64_t rows, int64_t segments, int64_t lag, unsigned int ticket, int64_t* row,
                           int* segment, int* is_apply);

/* ---- neighbours of the path (needed to stand in for the whole kernel library) ------------ */

/* loss[0] = mean over rows of (log sum_c exp(logits[r,c]) - logits[r,label[r]]); rows whose
 * label is outside [0, classes) contribute 0.  Deterministic (no float atomics).  Replaces
 * dl::kernels::cross_entropy (include/dl/kernels/cross_entropy.hpp:7-8,
 * src/kernels/cuda/cross_entropy.cu:9-43). */
int fdl_cross_entropy_f32(const float* logits, const int64_t* labels, float* loss,
                          int64_t batch, int64_t classes, void* stream);

/* out = transpose of the square row-major matrix in[n, n] (out must not alias in).
 * Replaces dl::kernels::transpose (include/dl/kernels/transpose.hpp:15-16,
 * src/kernels/cuda/transpose.cu:7-111), all three algorithm values. */
int fdl_transpose_f32(const float* in, float* out, int64_t n, void* stream);

/* data[i] uniform in (low, high] / normal(mean, stddev), a pure function of (seed, i)
 * (Philox4x32-10; the reference's per-element XORWOW sequence is not reproduced -- its
 * tests require only same-seed repeatability and the range).  Replace
 * dl::kernels::uniform_float32 / normal_float32 (include/dl/kernels/random.hpp:7-8,
 * src/kernels/cuda/random.cu:7-56). */
int fdl_uniform_f32(float* data, int64_t n, float low, float high, uint64_t seed, void* stream);
int fdl_normal_f32(float* data, int64_t n, float mean, float stddev, uint64_t seed, void* stream);

/* ---- host-buffer entry points ---------------------------------------------------------- */

/* The same operations with HOST pointers (`h_*`): the library moves the data through a
 * ring of device staging buffers on its own streams, overlapping upload, kernel and
 * download, and returns when the result is in host memory.  They stand in for the
 * reference's Tensor::from_host -> dl::ops::<op> -> Tensor::to_host round trip
 * (include/dl/tensor/Tensor.hpp:97-121, src/tensor/TensorImpl.cpp:91-125) for callers
 * whose tensors live on the host.  Buffers should be page-locked (pageable memory works
 * but serialises the copies).  Staging memory (4 slots x 128 MiB per device) is allocated
 * on first use and kept.  The calls on one device share that ring: each holds the device's
 * lock from start to finish, so concurrent callers on the same device run one after another
 * (different devices are independent).  Whatever a call returns, every copy it enqueued has
 * finished by then: the host buffers may be released at once. */
int fdl_host_binary_f32(const float* h_a, const float* h_b, float* h_out, int64_t n, int op);
int fdl_host_unary_f32(const float* h_x, float* h_out, int64_t n, int op, float alpha);
int fdl_host_mul_add_relu_f32(const float* h_a, const float* h_b, const float* h_c,
                              float* h_out, int64_t n);
/* h_out[r, c] = h_a[r, c] (op) h_row[c] */
int fdl_host_row_broadcast_f32(const float* h_a, const float* h_row, float* h_out,
                               int64_t rows, int64_t cols, int op);
/* *h_out = sum of h_x[0..n) (double; chunk partials folded on the host in order). */
int fdl_host_sum_f32(const float* h_x, int64_t n, double* h_out);
/* Three results from one pass over host data x, y of shape [rows, cols] and row[cols]:
 * z = x + y, w = x + row (row broadcast over the rows), *h_sum = sum(x).  Each chunk of x
 * and y is uploaded once and feeds all three kernels, so the link carries 2 tensors up and
 * 2 down instead of 4 up and 2 down for three separate calls. */
int fdl_host_sweep_f32(const float* h_x, const float* h_y, const float* h_row, float* h_z,
                       float* h_w, int64_t rows, int64_t cols, double* h_sum);

#if defined(FDL_BUILDING_LIBRARY) && defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* FDL_KERNELS_H_ */
