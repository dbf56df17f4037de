/*
 * fdl_oracle.c -- CPU restatement of fast_dl's tensor hot path.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the tests, the smoke check and the bench's
 * cpu_baseline / reference legs may call into this file, and only as the checker or as
 * the timed CPU baseline.  The product path (fast_dl_b200/csrc) never links it and has
 * no CPU fallback.
 *
 * Plain scalar C, one function per operation, each citing the fast_dl source it restates
 * (paths relative to the fast_dl tree).  Build with
 *     gcc -O2 -ffp-contract=off -fno-fast-math
 * -ffp-contract=off matters: fast_dl's elementwise chain rounds a*b and (a*b)+c
 * separately, and gcc would otherwise be free to fuse them on FMA hardware.
 *
 * Pinning status
 *   PINNED by the reference's own vectors (tests/golden/reference_vectors.npz, taken
 *   from tests/tensor/elementwise_tensor_test.cpp:30-63, tests/nn/relu_module_test.cpp:22-29,
 *   tests/tensor/activation_tensor_test.cpp:71-74, tests/tensor/softmax_tensor_test.cpp:43-46,
 *   tests/tensor/layernorm_tensor_test.cpp:50-53) and by oracle/_ref (the reference's CPU
 *   check functions and CUDA kernels compiled in place): binary ops, activations, the
 *   1024-block trees, softmax, layernorm without affine, row bias.
 *   PARITY UNPINNED (the reference has no implementation, the definitions come from the
 *   task statement): general broadcast, axis sum/mean/max/argmax, full sum, affine
 *   layernorm, the fused chain as a single call.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* ---- binary, same shape: src/kernels/cuda/elementwise.cu:5-24; CPU twin
 * tests/benchmarks/vector_add/vector_add_benchmark.cu:13-18 (add) ---- */
void orc_binary_f32(const float* a, const float* b, float* out, int64_t n, int op) {
    int64_t i;
    switch (op) {
        case 0: for (i = 0; i < n; ++i) out[i] = a[i] + b[i]; break;
        case 1: for (i = 0; i < n; ++i) out[i] = a[i] - b[i]; break;
        case 2: for (i = 0; i < n; ++i) out[i] = a[i] * b[i]; break;
        case 3: for (i = 0; i < n; ++i) out[i] = a[i] / b[i]; break;
        default: break;
    }
}

/* ---- activations: src/kernels/cuda/activation.cu:6-64; CPU twins
 * tests/tensor/activation_tensor_test.cpp:26-65.  op codes follow ActivationOp
 * (include/dl/kernels/activation.hpp:7-13). ---- */
void orc_unary_f32(const float* x, float* out, int64_t n, int op, float alpha) {
    int64_t i;
    switch (op) {
        case 0: /* std::max(0.0f, x): NaN -> 0, -0 -> +0 */
            for (i = 0; i < n; ++i) out[i] = x[i] > 0.0f ? x[i] : 0.0f;
            break;
        case 1:
            for (i = 0; i < n; ++i) out[i] = x[i] > 0.0f ? x[i] : alpha * x[i];
            break;
        case 2:
            for (i = 0; i < n; ++i) {
                const float v = x[i];
                out[i] = 0.5f * v * (1.0f + tanhf(0.79788456f * (v + 0.044715f * v * v * v)));
            }
            break;
        case 3:
            for (i = 0; i < n; ++i) out[i] = 1.0f / (1.0f + expf(-x[i]));
            break;
        case 4:
            for (i = 0; i < n; ++i) out[i] = tanhf(x[i]);
            break;
        default:
            break;
    }
}

/* ---- fused chain relu(a*b + c) as fast_dl computes it with three kernels
 * (src/ops/Elementwise.cpp:36-50 twice, src/ops/Activation.cpp:13-28): two roundings. ---- */
void orc_mul_add_relu_f32(const float* a, const float* b, const float* c, float* out, int64_t n) {
    int64_t i;
    for (i = 0; i < n; ++i) {
        volatile float p = a[i] * b[i]; /* forces the intermediate rounding */
        const float s = p + c[i];
        out[i] = s > 0.0f ? s : 0.0f;
    }
}

/* ---- row bias, in place: src/kernels/cuda/bias.cu:5-12 ---- */
void orc_add_row_bias_f32(float* out, const float* bias, int64_t rows, int64_t cols, int relu) {
    int64_t r, c;
    for (r = 0; r < rows; ++r) {
        for (c = 0; c < cols; ++c) {
            float v = out[r * cols + c] + bias[c];
            if (relu) v = v > 0.0f ? v : 0.0f;
            out[r * cols + c] = v;
        }
    }
}

/* out[r, c] = x[r, c] + row[c], out of place: the row-bias arithmetic of
 * src/kernels/cuda/bias.cu:5-12 written to a separate result. */
void orc_add_row_f32(const float* x, const float* row, float* out, int64_t rows, int64_t cols) {
    int64_t r, c;
    for (r = 0; r < rows; ++r)
        for (c = 0; c < cols; ++c) out[r * cols + c] = x[r * cols + c] + row[c];
}

/* ---- general broadcast binary (not in fast_dl; NumPy semantics): the elementwise IEEE
 * op on the broadcast-expanded operands.  Strides in elements, 0 = broadcast. ---- */
void orc_broadcast_binary_f32(const float* a, const float* b, float* out, int ndim,
                              const int64_t* shape, const int64_t* a_strides,
                              const int64_t* b_strides, int op) {
    int64_t idx[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int64_t total = 1, i;
    int d;
    for (d = 0; d < ndim; ++d) total *= shape[d];
    for (i = 0; i < total; ++i) {
        int64_t ao = 0, bo = 0;
        float x, y, r;
        for (d = 0; d < ndim; ++d) {
            ao += idx[d] * a_strides[d];
            bo += idx[d] * b_strides[d];
        }
        x = a[ao];
        y = b[bo];
        switch (op) {
            case 0: r = x + y; break;
            case 1: r = x - y; break;
            case 2: r = x * y; break;
            default: r = x / y; break;
        }
        out[i] = r;
        for (d = ndim - 1; d >= 0; --d) {
            if (++idx[d] < shape[d]) break;
            idx[d] = 0;
        }
    }
}

/* ---- 1024-element block sums in fast_dl's two tree orders:
 * src/kernels/cuda/reduction.cu:8-24 (interleave), :34-50 (address); CPU twins
 * tests/benchmarks/reduction/reduction_benchmark.cu:14-56.  tree: 0 interleave, 1 address. */
void orc_block_reduce_1024_f32(const float* x, float* out, int64_t n, int tree) {
    const int64_t blocks = n / 1024;
    int64_t blk;
    for (blk = 0; blk < blocks; ++blk) {
        float d[1024];
        int s, t;
        memcpy(d, x + blk * 1024, sizeof d);
        if (tree == 1) {
            for (s = 512; s > 0; s >>= 1)
                for (t = 0; t < s; ++t) d[t] += d[t + s];
        } else {
            for (s = 1; s < 1024; s *= 2)
                for (t = 0; t < 1024; t += 2 * s) d[t] += d[t + s];
        }
        out[blk] = d[0];
    }
}

/* ---- full sum (not in fast_dl): accumulated in double, rounded once. ---- */
double orc_sum_f64(const float* x, int64_t n) {
    double s = 0.0;
    int64_t i;
    for (i = 0; i < n; ++i) s += (double)x[i];
    return s;
}

/* Euclidean norm of the addends: the natural scale of a sum's rounding error. */
double orc_norm2_f64(const float* x, int64_t n) {
    double s = 0.0;
    int64_t i;
    for (i = 0; i < n; ++i) s += (double)x[i] * (double)x[i];
    return sqrt(s);
}

/* ---- axis-1 reductions of a row-major [rows, cols] matrix (not in fast_dl).
 * op: 0 sum, 1 mean, 2 max.  Sums in double.  max ignores NaN like fmaxf, the function
 * fast_dl uses for row maxima (src/kernels/cuda/softmax.cu:13-18). ---- */
void orc_reduce_rows_f32(const float* x, int64_t rows, int64_t cols, float* out, int op) {
    int64_t r, c;
    for (r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        if (op == 2) {
            float m = -INFINITY;
            for (c = 0; c < cols; ++c) m = fmaxf(m, xr[c]);
            out[r] = m;
        } else {
            double s = 0.0;
            for (c = 0; c < cols; ++c) s += (double)xr[c];
            out[r] = (float)(op == 1 ? s / (double)cols : s);
        }
    }
}

/* argmax along axis 1: lowest index of the maximum; NaN ranks as -inf. */
void orc_argmax_rows_f32(const float* x, int64_t rows, int64_t cols, int64_t* out) {
    int64_t r, c;
    for (r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float best = -INFINITY;
        int64_t arg = 0;
        int have = 0;
        for (c = 0; c < cols; ++c) {
            const float v = xr[c] != xr[c] ? -INFINITY : xr[c];
            if (!have || v > best) {
                best = v;
                arg = c;
                have = 1;
            }
        }
        out[r] = arg;
    }
}

/* ---- axis-0 reductions of `batch` stacked [rows, cols] matrices (not in fast_dl). ---- */
void orc_reduce_cols_f32(const float* x, int64_t batch, int64_t rows, int64_t cols, float* out,
                         int op, double mean_divisor) {
    int64_t b, r, c;
    for (b = 0; b < batch; ++b) {
        const float* xb = x + b * rows * cols;
        for (c = 0; c < cols; ++c) {
            if (op == 2) {
                float m = -INFINITY;
                for (r = 0; r < rows; ++r) m = fmaxf(m, xb[r * cols + c]);
                out[b * cols + c] = m;
            } else {
                double s = 0.0;
                for (r = 0; r < rows; ++r) s += (double)xb[r * cols + c];
                out[b * cols + c] = (float)(op == 1 ? s / mean_divisor : s);
            }
        }
    }
}

/* ---- row softmax: max-shift, expf, divide by the fp32 running sum -- the arithmetic of
 * tests/tensor/softmax_tensor_test.cpp:10-35 and
 * tests/benchmarks/softmax/softmax_benchmark.cu:14-36, themselves twins of
 * src/kernels/cuda/softmax.cu:28-53. ---- */
void orc_softmax_rows_f32(const float* x, float* y, int64_t rows, int64_t cols) {
    int64_t r, c;
    for (r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float* yr = y + r * cols;
        float m = xr[0];
        float sum = 0.0f;
        for (c = 1; c < cols; ++c) m = xr[c] > m ? xr[c] : m;
        for (c = 0; c < cols; ++c) {
            const float e = expf(xr[c] - m);
            yr[c] = e;
            sum += e;
        }
        for (c = 0; c < cols; ++c) yr[c] /= sum;
    }
}

/* ---- row layernorm, fast_dl's formula: mean = S1/C, var = max(S2/C - mean^2, 0),
 * y = (x - mean) / sqrt(var + eps): tests/tensor/layernorm_tensor_test.cpp:9-37, twin of
 * src/kernels/cuda/layernorm.cu:22-50.  gamma/beta (nullable) are the affine extension:
 * y*gamma + beta applied to that result. ---- */
void orc_layernorm_rows_f32(const float* x, const float* gamma, const float* beta, float* y,
                            int64_t rows, int64_t cols, float eps) {
    int64_t r, c;
    for (r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float* yr = y + r * cols;
        float sum = 0.0f, sq = 0.0f, mean, mean_sq, var, inv_std;
        for (c = 0; c < cols; ++c) {
            const float v = xr[c];
            sum += v;
            sq += v * v;
        }
        mean = sum / (float)cols;
        mean_sq = sq / (float)cols;
        var = mean_sq - mean * mean;
        var = var > 0.0f ? var : 0.0f;
        inv_std = 1.0f / sqrtf(var + eps);
        for (c = 0; c < cols; ++c) {
            float o = (xr[c] - mean) * inv_std;
            if (gamma) o = o * gamma[c];
            if (beta) o = o + beta[c];
            yr[c] = o;
        }
    }
}

/* Same quantity with every accumulation in double: the accuracy yardstick used to show
 * that a difference from orc_layernorm_rows_f32 is rounding, not a wrong formula. */
void orc_layernorm_rows_f64(const float* x, const float* gamma, const float* beta, double* y,
                            int64_t rows, int64_t cols, double eps) {
    int64_t r, c;
    for (r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        double* yr = y + r * cols;
        double sum = 0.0, sq = 0.0, mean, var, inv_std;
        for (c = 0; c < cols; ++c) sum += (double)xr[c];
        mean = sum / (double)cols;
        for (c = 0; c < cols; ++c) sq += ((double)xr[c] - mean) * ((double)xr[c] - mean);
        var = sq / (double)cols;
        inv_std = 1.0 / sqrt(var + eps);
        for (c = 0; c < cols; ++c) {
            double o = ((double)xr[c] - mean) * inv_std;
            if (gamma) o *= (double)gamma[c];
            if (beta) o += (double)beta[c];
            yr[c] = o;
        }
    }
}

void orc_softmax_rows_f64(const float* x, double* y, int64_t rows, int64_t cols) {
    int64_t r, c;
    for (r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        double* yr = y + r * cols;
        double m = (double)xr[0], sum = 0.0;
        for (c = 1; c < cols; ++c) m = (double)xr[c] > m ? (double)xr[c] : m;
        for (c = 0; c < cols; ++c) {
            yr[c] = exp((double)xr[c] - m);
            sum += yr[c];
        }
        for (c = 0; c < cols; ++c) yr[c] /= sum;
    }
}

/* ---- cross-entropy: per row log(sum exp(x - max)) + max - x[label], mean over the batch
 * (each term divided by batch before the add); rows with an out-of-range label contribute 0:
 * src/kernels/cuda/cross_entropy.cu:9-35.  Accumulated in double here. ---- */
double orc_cross_entropy_f64(const float* logits, const int64_t* labels, int64_t batch, int64_t classes) {
    double total = 0.0;
    int64_t r, c;
    for (r = 0; r < batch; ++r) {
        const float* x = logits + r * classes;
        float m;
        double s = 0.0;
        if (labels[r] < 0 || labels[r] >= classes) continue;
        m = x[0];
        for (c = 1; c < classes; ++c) m = x[c] > m ? x[c] : m;
        for (c = 0; c < classes; ++c) s += exp((double)x[c] - (double)m);
        total += (log(s) + (double)m - (double)x[labels[r]]) / (double)batch;
    }
    return total;
}

/* ---- square transpose: src/kernels/cuda/transpose.cu:7-15 ---- */
void orc_transpose_f32(const float* in, float* out, int64_t n) {
    int64_t r, c;
    for (r = 0; r < n; ++r)
        for (c = 0; c < n; ++c) out[c * n + r] = in[r * n + c];
}
