"""Per-op CPU baseline for the five workload configurations, on this machine's host cores.

    python tests/cpu_opbench.py [--configs c1,c2,c3,c4,c5] [--json out.json]

Each op runs the reference's own CPU function where it has one (its test and benchmark check
functions, compiled in place into oracle/_ref/libref.so) and the oracle port otherwise, once on
one thread exactly as written and once with the rows split over all host threads (the count is
printed).  GB/s uses the same algorithmic bytes as the GPU table.  Configuration 5 runs on a
bounded sample (4096 of its 16384 rows).  Test infrastructure: nothing here is on the product path.
"""
import argparse
import ctypes as C
import json
import os
import sys
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from oracle import oracle as orc  # noqa: E402
from oracle import ref  # noqa: E402

THREADS = os.cpu_count() or 1
POOL = ThreadPoolExecutor(THREADS)
FP = C.POINTER(C.c_float)
IP = C.POINTER(C.c_int64)
I64 = C.c_int64


def fptr(a, offset=0):
    return C.cast(a.ctypes.data + 4 * offset, FP)


def blocks(rows, parts):
    per = -(-rows // parts)
    return [(lo, min(rows, lo + per)) for lo in range(0, rows, per)]


def best_of(fn, reps=3):
    fn()
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return min(times)


RESULTS = []


def report(config, op, nbytes, source, run):
    """run(parts) executes the op with the rows split into `parts` blocks on the pool."""
    t1 = best_of(lambda: run(1))
    tn = best_of(lambda: run(THREADS))
    row = {"config": config, "op": op, "bytes": nbytes, "source": source, "threads": THREADS,
           "ms_1_thread": t1 * 1e3, "GBps_1_thread": nbytes / t1 / 1e9,
           "ms_all_threads": tn * 1e3, "GBps_all_threads": nbytes / tn / 1e9}
    RESULTS.append(row)
    print(f"{config:3s} {op:36s} 1 thread {row['GBps_1_thread']:7.2f} GB/s ({t1 * 1e3:9.1f} ms)   "
          f"{THREADS} threads {row['GBps_all_threads']:7.2f} GB/s ({tn * 1e3:8.1f} ms)   [{source}]", flush=True)


def over_rows(fn, rows):
    """fn(lo, hi) on row blocks, in parallel."""
    def run(parts):
        list(POOL.map(lambda p: fn(*p), blocks(rows, parts)))
    return run


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="c1,c2,c3,c4,c5")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    cfgs = args.configs.split(",")
    lib = orc.lib()
    have_ref = ref.available()
    rng = np.random.default_rng(42)
    print(f"host threads: {THREADS}; reference CPU functions {'available' if have_ref else 'NOT built: oracle port only'}")

    if "c1" in cfgs:
        n = 1 << 20
        a, b, c = (rng.uniform(-1, 1, n).astype(np.float32) for _ in range(3))
        out = np.empty_like(a)
        report("c1", "relu(a*b+c)", 16 * n, "oracle port",
               over_rows(lambda lo, hi: lib.orc_mul_add_relu_f32(fptr(a, lo), fptr(b, lo), fptr(c, lo), fptr(out, lo),
                                                                 I64(hi - lo)), n))

    if "c2" in cfgs:
        R = Cc = 4096
        A = rng.normal(0, 1, (R, Cc)).astype(np.float32)
        bias = rng.normal(0, 1, Cc).astype(np.float32)
        scale = rng.uniform(0.5, 2, R).astype(np.float32)
        out = np.empty_like(A)
        nb = 8 * R * Cc + 4 * Cc
        report("c2", "A + b[1,4096]", nb, "oracle port",
               over_rows(lambda lo, hi: lib.orc_add_row_f32(fptr(A, lo * Cc), fptr(bias), fptr(out, lo * Cc),
                                                            I64(hi - lo), I64(Cc)), R))
        arr2 = I64 * 2

        def col_scale(lo, hi):
            lib.orc_broadcast_binary_f32(fptr(A, lo * Cc), fptr(scale, lo), fptr(out, lo * Cc), 2,
                                         arr2(hi - lo, Cc), arr2(Cc, 1), arr2(1, 0), 2)
        report("c2", "A * s[4096,1]", nb, "oracle port (strided walk)", over_rows(col_scale, R))

    if "c3" in cfgs:
        R = Cc = 8192
        X = rng.normal(0, 1, (R, Cc)).astype(np.float32)
        o32 = np.empty(R, dtype=np.float32)
        o64 = np.empty(R, dtype=np.int64)
        for name, op in (("sum axis 1", 0), ("max axis 1", 2)):
            report("c3", name, 4 * R * Cc + 4 * R, "oracle port",
                   over_rows(lambda lo, hi, op=op: lib.orc_reduce_rows_f32(fptr(X, lo * Cc), I64(hi - lo), I64(Cc),
                                                                           fptr(o32, lo), op), R))
        report("c3", "argmax axis 1 (int64)", 4 * R * Cc + 8 * R, "oracle port",
               over_rows(lambda lo, hi: lib.orc_argmax_rows_f32(fptr(X, lo * Cc), I64(hi - lo), I64(Cc),
                                                                C.cast(o64.ctypes.data + 8 * lo, IP)), R))
        partial = np.empty((THREADS, Cc), dtype=np.float32)

        def col_mean(parts):
            bl = blocks(R, parts)
            list(POOL.map(lambda ip: lib.orc_reduce_cols_f32(fptr(X, ip[1][0] * Cc), I64(1), I64(ip[1][1] - ip[1][0]),
                                                             I64(Cc), fptr(partial, ip[0] * Cc), 0, C.c_double(1.0)),
                          enumerate(bl)))
            return partial[:len(bl)].sum(axis=0, dtype=np.float64) / R
        report("c3", "mean axis 0", 4 * R * Cc + 4 * Cc, "oracle port (block sums, then added)", col_mean)
        lib.orc_sum_f64.restype = C.c_double

        def full_sum(parts):
            return sum(POOL.map(lambda p: lib.orc_sum_f64(fptr(X, p[0] * Cc), I64((p[1] - p[0]) * Cc)), blocks(R, parts)))
        report("c3", "full sum", 4 * R * Cc + 4, "oracle port (double accumulation)", full_sum)
        if have_ref:
            flat = X.reshape(-1)
            report("c3", "1024-block partial sums (address)", 4 * R * Cc + 4 * R * Cc // 1024,
                   "reference reduction_benchmark.cu CPU tree", lambda parts: ref.cpu_block_reduce(flat, 1, threads=parts))

    if "c4" in cfgs:
        R, Cc = 65536, 1024
        L = rng.normal(0, 3, (R, Cc)).astype(np.float32)
        g = rng.uniform(0.9, 1.1, Cc).astype(np.float32)
        be = rng.uniform(-0.1, 0.1, Cc).astype(np.float32)
        out = np.empty_like(L)
        if have_ref:
            report("c4", "row softmax", 8 * R * Cc, "reference softmax_cpu",
                   lambda parts: ref.cpu_softmax(L, threads=parts, out=out))
            report("c4", "layernorm", 8 * R * Cc, "reference layernorm_cpu",
                   lambda parts: ref.cpu_layernorm(L, threads=parts, out=out))
        report("c4", "layernorm + gamma, beta", 8 * R * Cc + 8 * Cc, "oracle port",
               over_rows(lambda lo, hi: lib.orc_layernorm_rows_f32(fptr(L, lo * Cc), fptr(g), fptr(be), fptr(out, lo * Cc),
                                                                   I64(hi - lo), I64(Cc), C.c_float(1e-5)), R))
        flat, oflat = L.reshape(-1), out.reshape(-1)
        for name, op in (("activation gelu", 2), ("activation relu", 0)):
            if have_ref:
                report("c4", name, 8 * R * Cc, "reference activation_tensor_test.cpp *_cpu",
                       lambda parts, op=op: ref.cpu_activation(flat, op, 0.01, threads=parts, out=oflat))
                continue
            report("c4", name, 8 * R * Cc, "oracle port of the reference's *_cpu",
                   over_rows(lambda lo, hi, op=op: lib.orc_unary_f32(fptr(flat, lo), fptr(oflat, lo), I64(hi - lo), op,
                                                                     C.c_float(0.01)), R * Cc))

    if "c5" in cfgs:
        R, Cc = 4096, 16384      # bounded sample: a quarter of the rows
        x = rng.uniform(-1, 1, R * Cc).astype(np.float32)
        y = rng.uniform(-1, 1, R * Cc).astype(np.float32)
        rowv = rng.uniform(-1, 1, Cc).astype(np.float32)
        out = np.empty_like(x)
        n = R * Cc
        if have_ref:
            report("c5", "binary add (4096 of 16384 rows)", 12 * n, "reference vector_add_cpu",
                   lambda parts: ref.cpu_vector_add(x, y, threads=parts, out=out))
        else:
            report("c5", "binary add (4096 of 16384 rows)", 12 * n, "oracle port",
                   over_rows(lambda lo, hi: lib.orc_binary_f32(fptr(x, lo), fptr(y, lo), fptr(out, lo), I64(hi - lo), 0), n))
        report("c5", "broadcast add + row (4096 rows)", 8 * n + 4 * Cc, "oracle port",
               over_rows(lambda lo, hi: lib.orc_add_row_f32(fptr(x, lo * Cc), fptr(rowv), fptr(out, lo * Cc),
                                                            I64(hi - lo), I64(Cc)), R))
        lib.orc_sum_f64.restype = C.c_double
        report("c5", "full sum (4096 rows)", 4 * n + 4, "oracle port (double accumulation)",
               lambda parts: sum(POOL.map(lambda p: lib.orc_sum_f64(fptr(x, p[0]), I64(p[1] - p[0])), blocks(n, parts))))

    if args.json:
        Path(args.json).write_text(json.dumps({"threads": THREADS, "results": RESULTS}, indent=1))


if __name__ == "__main__":
    main()
