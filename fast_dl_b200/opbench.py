"""Per-operation bandwidth table for the five workload configurations.

    python -m fast_dl_b200.opbench [--configs c1,c2,c3,c4,c5] [--iters 20] [--json out.json]

For every op of every configuration it reports the median launch time (CUDA events around
each launch; between launches the L2 is flushed by READING a 512 MiB buffer, which leaves
clean lines behind -- flushing by writing would leave ~100 MB of dirty lines whose
write-back is then billed to the kernel under test), the algorithmic
GB/s (compulsory bytes only) and that as a fraction of the measured HBM copy bandwidth.
A caller may hand main() an object with the reference's own kernel launchers; they are then
timed on the same buffers as the speed bar (tests/opbench_reference.py does that with the
reference's kernels recompiled for sm_100a).  This module itself knows only the product.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def peak_gbs() -> float:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"])
    return 6650.0


def main(ref=None) -> None:
    import torch
    from fast_dl_b200 import capi

    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="c1,c2,c3,c4,c5")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    ap.add_argument("--tune", action="append", default=[], help="key=value passed to fdl_set_tuning")
    args = ap.parse_args()

    torch.cuda.set_device(0)
    capi.lib()
    capi.use_device(0)
    for kv in args.tune:
        k, v = kv.split("=")
        capi.set_tuning(k, int(v))
    dev = torch.device("cuda", 0)
    peak = peak_gbs()
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    gen = torch.Generator(device=dev).manual_seed(42)

    def uniform(shape, lo=-1.0, hi=1.0):
        return torch.empty(shape, dtype=torch.float32, device=dev).uniform_(lo, hi, generator=gen)

    def normal(shape, std=1.0):
        return torch.empty(shape, dtype=torch.float32, device=dev).normal_(0.0, std, generator=gen)

    results = []

    def timeit(fn, sync_ref=False):
        times = []
        for i in range(args.iters + 3):
            capi.full_sum(flush)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            if i >= 3:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times), min(times)

    def record(config, op, nbytes, fn, ref_fn=None):
        med, best = timeit(fn)
        row = {"config": config, "op": op, "bytes": nbytes, "ms": med, "ms_min": best,
               "GBps": nbytes / med / 1e6, "frac_of_measured_peak": nbytes / med / 1e6 / peak}
        if ref_fn is not None:
            rmed, _ = timeit(ref_fn)
            row["reference_kernel_ms"] = rmed
            row["reference_kernel_GBps"] = nbytes / rmed / 1e6
            row["speedup_vs_reference_kernel"] = rmed / med
        results.append(row)
        extra = f"  ref {row['reference_kernel_GBps']:8.1f} GB/s  x{row['speedup_vs_reference_kernel']:.2f}" if ref_fn else ""
        print(f"{config:3s} {op:34s} {med * 1e3:9.1f} us {row['GBps']:8.1f} GB/s  {100 * row['frac_of_measured_peak']:5.1f}%{extra}",
              flush=True)

    def graphed(fn):
        """fn captured into a CUDA graph (after an eager pass: first uses allocate); returns the replay."""
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        keep.append(graph)
        return graph.replay

    keep = []
    cfgs = args.configs.split(",")

    if "c1" in cfgs:
        n = 1 << 20
        a, b, c = uniform(n), uniform(n), uniform(n)
        out, t1, t2 = torch.empty_like(a), torch.empty_like(a), torch.empty_like(a)
        record("c1", "fused relu(a*b+c)", 16 * n, lambda: capi.mul_add_relu(a, b, c, out=out))

        def unfused():
            capi.binary(a, b, capi.MUL, out=t1)
            capi.binary(t1, c, capi.ADD, out=t2)
            capi.unary(t2, capi.RELU, out=out)

        def ref_unfused():
            ref.gpu_elementwise(a.data_ptr(), b.data_ptr(), t1.data_ptr(), n, 2)
            ref.gpu_elementwise(t1.data_ptr(), c.data_ptr(), t2.data_ptr(), n, 0)
            ref.gpu_activation(t2.data_ptr(), out.data_ptr(), n, 0)

        record("c1", "unfused mul, add, relu (3 launches)", 32 * n, unfused, ref_unfused if ref else None)
        record("c1", "the same 3 launches replayed from a CUDA graph", 32 * n, graphed(unfused))

    if "c2" in cfgs:
        R = C = 4096
        A, bias, scale = normal((R, C)), normal((1, C)), uniform((R, 1), 0.5, 2.0)
        out = torch.empty_like(A)
        nb = 8 * R * C + 4 * C
        record("c2", "A + b[1,4096]", nb, lambda: capi.broadcast_binary(A, bias, capi.ADD, out=out))
        record("c2", "A * s[4096,1]", nb, lambda: capi.broadcast_binary(A, scale, capi.MUL, out=out))
        record("c2", "row bias in place", nb, lambda: capi.add_row_bias_(A, bias.view(-1)),
               (lambda: ref.gpu_add_row_bias(A.data_ptr(), bias.data_ptr(), R, C)) if ref else None)

    if "c3" in cfgs:
        R = C = 8192
        X = normal((R, C))
        record("c3", "sum axis 1", 4 * R * C + 4 * R, lambda: capi.reduce_rows(X, capi.REDUCE_SUM))
        record("c3", "max axis 1", 4 * R * C + 4 * R, lambda: capi.reduce_rows(X, capi.REDUCE_MAX))
        record("c3", "argmax axis 1 (int64)", 4 * R * C + 8 * R, lambda: capi.argmax_rows(X))
        record("c3", "mean axis 0", 4 * R * C + 4 * C, lambda: capi.reduce_cols(X, capi.REDUCE_MEAN))
        record("c3", "full sum", 4 * R * C + 4, lambda: capi.full_sum(X))
        part = torch.empty(R * C // 1024, dtype=torch.float32, device=dev)
        record("c3", "1024-block partial sums (address)", 4 * R * C + 4 * R * C // 1024,
               lambda: capi.block_reduce_1024(X.view(-1), capi.TREE_ADDRESS),
               (lambda: ref.gpu_reduction(X.data_ptr(), part.data_ptr(), R * C, 1)) if ref else None)

    if "c4" in cfgs:
        R, C = 65536, 1024
        L = normal((R, C), 3.0)
        g, be = uniform(C, 0.9, 1.1), uniform(C, -0.1, 0.1)
        out = torch.empty_like(L)
        record("c4", "row softmax", 8 * R * C, lambda: capi.softmax_rows(L, out=out),
               (lambda: ref.gpu_softmax(L.data_ptr(), out.data_ptr(), R, C, 2)) if ref else None)
        record("c4", "layernorm", 8 * R * C, lambda: capi.layernorm_rows(L, out=out),
               (lambda: ref.gpu_layernorm(L.data_ptr(), out.data_ptr(), R, C, 1e-5)) if ref else None)
        record("c4", "layernorm + gamma, beta", 8 * R * C + 8 * C, lambda: capi.layernorm_rows(L, g, be, out=out))
        for op, name in ((capi.GELU, "gelu"), (capi.SIGMOID, "sigmoid"), (capi.TANH, "tanh"), (capi.RELU, "relu")):
            record("c4", f"activation {name}", 8 * R * C, lambda op=op: capi.unary(L, op, out=out),
                   (lambda op=op: ref.gpu_activation(L.data_ptr(), out.data_ptr(), R * C, op)) if ref else None)

    if "next" in cfgs:  # the path's neighbours: cross-entropy, square transpose, random fill
        R, C = 65536, 1024
        L = normal((R, C), 3.0)
        labels = torch.randint(0, C, (R,), device=dev, generator=gen)
        loss = torch.empty(1, dtype=torch.float32, device=dev)
        record("nxt", "cross-entropy [65536,1024]", 4 * R * C + 8 * R + 4, lambda: capi.cross_entropy(L, labels),
               (lambda: ref.gpu_cross_entropy(L.data_ptr(), labels.data_ptr(), loss.data_ptr(), R, C)) if ref else None)
        del L
        for n in (4096, 8192, 16384):
            X = normal((n, n))
            out = torch.empty_like(X)
            record("nxt", f"transpose [{n},{n}]", 8 * n * n,
                   lambda: capi.check(capi.lib().fdl_transpose_f32(X.data_ptr(), out.data_ptr(), n, capi._stream()), "transpose"),
                   (lambda: ref.gpu_transpose(X.data_ptr(), out.data_ptr(), n, 2)) if ref else None)
            del X, out
        n = 1 << 28
        buf = torch.empty(n, dtype=torch.float32, device=dev)
        record("nxt", "uniform fill, 2^28 floats", 4 * n,
               lambda: capi.check(capi.lib().fdl_uniform_f32(buf.data_ptr(), n, -1.0, 1.0, 1234, capi._stream()), "uniform"),
               (lambda: ref.gpu_uniform(buf.data_ptr(), n, -1.0, 1.0, 1234)) if ref else None)
        record("nxt", "normal fill, 2^28 floats", 4 * n,
               lambda: capi.check(capi.lib().fdl_normal_f32(buf.data_ptr(), n, 0.0, 1.0, 1234, capi._stream()), "normal"),
               (lambda: ref.gpu_normal(buf.data_ptr(), n, 0.0, 1.0, 1234)) if ref else None)
        del buf

    if "rows" in cfgs:  # extra row-wise shapes: short and long rows
        for R, C in ((1 << 21, 32), (1 << 20, 64), (1 << 19, 128), (1 << 18, 256), (1 << 15, 2048), (1 << 14, 4096), (8192, 8192), (4096, 16384),
                     (2048, 32768), (1024, 65536), (512, 131072), (256, 262144), (128, 524288)):
            L = normal((R, C), 3.0)
            out = torch.empty_like(L)
            record("row", f"softmax [{R},{C}]", 8 * R * C, lambda: capi.softmax_rows(L, out=out))
            record("row", f"layernorm [{R},{C}]", 8 * R * C, lambda: capi.layernorm_rows(L, out=out))
            del L, out

    if "shapes" in cfgs:  # 256 MiB inputs in shapes far from the configurations': where are the weak spots?
        n = 1 << 26
        for R, C in ((1 << 21, 32), (1 << 19, 128), (1 << 17, 512), (1 << 13, 8192), (64, 1 << 20), (3, n // 12 * 4)):
            X = normal((R, C))
            record("shp", f"sum axis 1 [{R},{C}]", 4 * R * C + 4 * R, lambda: capi.reduce_rows(X, capi.REDUCE_SUM))
            record("shp", f"argmax axis 1 [{R},{C}]", 4 * R * C + 8 * R, lambda: capi.argmax_rows(X))
            record("shp", f"mean axis 0 [{R},{C}]", 4 * R * C + 4 * C, lambda: capi.reduce_cols(X, capi.REDUCE_MEAN))
            del X
        X = normal((64, 1024, 1024))
        record("shp", "mean axis 1 of [64,1024,1024] (batched)", 4 * n + 4 * 65536,
               lambda: capi.reduce_cols(X, capi.REDUCE_MEAN))
        out = torch.empty_like(X)
        for name, other in (("[64,1024,1024] + [1024] (innermost)", uniform((1024,))),
                            ("[64,1024,1024] + [1024,1] (middle)", uniform((1024, 1))),
                            ("[64,1024,1024] + [64,1,1] (outermost)", uniform((64, 1, 1))),
                            ("[64,1024,1024] + [64,1,1024]", uniform((64, 1, 1024))),
                            ("[64,1024,1024] + [1,1024,1]", uniform((1, 1024, 1)))):
            record("shp", name, 8 * n + 4 * other.numel(),
                   lambda other=other: capi.broadcast_binary(X, other, capi.ADD, out=out))
        X4 = X.view(64, 64, 128, 128)
        out4 = out.view(64, 64, 128, 128)
        ch = uniform((1, 64, 1, 1))
        record("shp", "[64,64,128,128] * [1,64,1,1] (per channel)", 8 * n + 256,
               lambda: capi.broadcast_binary(X4, ch, capi.MUL, out=out4))
        flat, oflat = X.view(-1), out.view(-1)
        record("shp", "add, operands offset by 4 bytes (scalar path)", 12 * (n - 1),
               lambda: capi.binary(flat[1:], out.view(-1)[1:], capi.ADD, out=oflat[1:]))
        for k in (1 << 10, 1 << 14, 1 << 18, 1 << 22):
            record("shp", f"full sum of {k} elements", 4 * k + 4, lambda k=k: capi.full_sum(flat[:k]))
        del X, out

    if "odd" in cfgs:  # row lengths that are not a multiple of 4 floats: every row at another phase of a 16-byte line
        for R, C in ((65536, 1001), (65536, 1023), (8192, 50257), (4096, 8191), (1 << 20, 63), (262144, 255), (2048, 100003)):
            L = normal((R, C), 3.0)
            out = torch.empty_like(L)
            record("odd", f"softmax [{R},{C}]", 8 * R * C, lambda: capi.softmax_rows(L, out=out))
            record("odd", f"layernorm [{R},{C}]", 8 * R * C, lambda: capi.layernorm_rows(L, out=out))
            record("odd", f"sum axis 1 [{R},{C}]", 4 * R * C + 4 * R, lambda: capi.reduce_rows(L, capi.REDUCE_SUM))
            record("odd", f"argmax axis 1 [{R},{C}]", 4 * R * C + 8 * R, lambda: capi.argmax_rows(L))
            record("odd", f"mean axis 0 [{R},{C}]", 4 * R * C + 4 * C, lambda: capi.reduce_cols(L, capi.REDUCE_MEAN))
            del L, out

    if "c5" in cfgs:
        n, C = 1 << 28, 16384
        x, y = uniform(n), uniform(n)
        row = uniform((1, C))
        out = torch.empty_like(x)
        record("c5", "binary add", 12 * n, lambda: capi.binary(x, y, capi.ADD, out=out),
               (lambda: ref.gpu_vector_add(x.data_ptr(), y.data_ptr(), out.data_ptr(), n)) if ref else None)
        record("c5", "broadcast add [16384,16384]+[1,16384]", 8 * n + 4 * C,
               lambda: capi.broadcast_binary(x.view(n // C, C), row, capi.ADD, out=out.view(n // C, C)))
        record("c5", "full sum", 4 * n + 4, lambda: capi.full_sum(x))

    torch.cuda.synchronize()
    capi.take_device_error()
    if args.json:
        Path(args.json).write_text(json.dumps({"peak_gbs": peak, "results": results}, indent=1))


def main_sharded() -> None:
    """Per-op table with every tensor row-sharded over the ranks of a torch.distributed job.

        python -m torch.distributed.run --nproc-per-node N -m fast_dl_b200.opbench --sharded [--json out.json]

    Configurations C2-C5, total sizes fixed (strong scaling).  Every rank times its shard
    (CUDA events per launch, read-flushed L2, median of --iters launches); the slowest rank
    defines the time.  Aggregate GB/s = whole-tensor algorithmic bytes / that time; the
    per-GPU fraction divides by N x the measured copy bandwidth.  Ops with an exchange (full
    sum, mean along axis 0) exchange their per-GPU results inside the kernel over NVLink.
    """
    import os

    import torch
    import torch.distributed as dist
    from fast_dl_b200 import capi
    from fast_dl_b200.sharding import shard_rows

    ap = argparse.ArgumentParser()
    ap.add_argument("--sharded", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    capi.lib()
    capi.use_device(local)
    dev = torch.device("cuda", local)
    exchange = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

        def gather(handle):
            handles = [None] * world
            dist.all_gather_object(handles, handle)
            return handles
        exchange = capi.Exchange(world, rank, gather)
        dist.barrier()
    peak = peak_gbs()
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    gen = torch.Generator(device=dev).manual_seed(42 + rank)
    results = []

    def rnd(shape, kind="u", a=-1.0, b=1.0):
        t = torch.empty(shape, dtype=torch.float32, device=dev)
        return t.uniform_(a, b, generator=gen) if kind == "u" else t.normal_(a, b, generator=gen)

    def record(config, op, total_bytes, fn):
        times = []
        for i in range(args.iters + 3):
            if world > 1:
                dist.barrier()  # ranks start each launch together, as a sharded op would
            # The flush (~80 us) also lets the host enqueue the timed launch before the GPU
            # gets to it, so no host launch latency is measured.
            capi.full_sum(flush)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            if i >= 3:
                times.append(e0.elapsed_time(e1))
        t = torch.tensor([statistics.median(times)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
        gbs = total_bytes / ms / 1e6
        results.append({"config": config, "op": op, "n_gpus": world, "bytes": total_bytes, "ms": ms, "GBps": gbs,
                        "frac_per_gpu": gbs / (world * peak)})
        if rank == 0:
            print(f"{config:3s} {op:40s} {ms * 1e3:9.1f} us {gbs:9.1f} GB/s  {100 * gbs / (world * peak):5.1f}% per GPU",
                  flush=True)

    s32 = torch.zeros(1, dtype=torch.float32, device=dev)
    s64 = torch.zeros(1, dtype=torch.float64, device=dev)

    def total_sum(x):
        if exchange is not None:
            exchange.sum(x.reshape(-1), s32, s64)
        else:
            capi.full_sum(x.reshape(-1))

    # C2
    R = C = 4096
    r = shard_rows(R, world, rank).count
    A, bias, scale = rnd((r, C), "n", 0.0, 1.0), rnd((1, C), "n", 0.0, 1.0), rnd((r, 1), "u", 0.5, 2.0)
    out = torch.empty_like(A)
    record("c2", "A + b[1,4096]", 8 * R * C + 4 * C * world, lambda: capi.broadcast_binary(A, bias, capi.ADD, out=out))
    record("c2", "A * s[4096,1]", 8 * R * C + 4 * R, lambda: capi.broadcast_binary(A, scale, capi.MUL, out=out))
    del A, out
    # C3
    R = C = 8192
    r = shard_rows(R, world, rank).count
    X = rnd((r, C), "n", 0.0, 1.0)
    record("c3", "sum axis 1", 4 * R * C + 4 * R, lambda: capi.reduce_rows(X, capi.REDUCE_SUM))
    record("c3", "max axis 1", 4 * R * C + 4 * R, lambda: capi.reduce_rows(X, capi.REDUCE_MAX))
    record("c3", "argmax axis 1 (int64)", 4 * R * C + 8 * R, lambda: capi.argmax_rows(X))

    mean_out = torch.empty(C, dtype=torch.float32, device=dev)

    def mean0():
        if exchange is not None:
            exchange.reduce_cols(X, capi.REDUCE_MEAN, R, mean_out)
        else:
            capi.reduce_cols(X, capi.REDUCE_MEAN, mean_divisor=R)
    record("c3", "mean axis 0 (+ exchange)", 4 * R * C + 4 * C * world, mean0)
    record("c3", "full sum (+ exchange)", 4 * R * C + 4, lambda: total_sum(X))
    del X
    # C4
    R, C = 65536, 1024
    r = shard_rows(R, world, rank).count
    L = rnd((r, C), "n", 0.0, 3.0)
    g, be = rnd(C, "u", 0.9, 1.1), rnd(C, "u", -0.1, 0.1)
    out = torch.empty_like(L)
    record("c4", "row softmax", 8 * R * C, lambda: capi.softmax_rows(L, out=out))
    record("c4", "layernorm + gamma, beta", 8 * R * C + 8 * C * world, lambda: capi.layernorm_rows(L, g, be, out=out))
    record("c4", "activation gelu", 8 * R * C, lambda: capi.unary(L, capi.GELU, out=out))
    del L, out
    # C5
    R, C = 16384, 16384
    r = shard_rows(R, world, rank).count
    x, y, row = rnd(r * C), rnd(r * C), rnd((1, C))
    out = torch.empty_like(x)
    n = R * C
    record("c5", "binary add", 12 * n, lambda: capi.binary(x, y, capi.ADD, out=out))
    record("c5", "broadcast add [16384,16384]+[1,16384]", 8 * n + 4 * C * world,
           lambda: capi.broadcast_binary(x.view(r, C), row, capi.ADD, out=out.view(r, C)))
    record("c5", "full sum (+ exchange)", 4 * n + 4, lambda: total_sum(x))

    torch.cuda.synchronize()
    capi.take_device_error()
    if rank == 0 and args.json:
        Path(args.json).write_text(json.dumps({"peak_gbs": peak, "n_gpus": world, "results": results}, indent=1))
    if world > 1:
        dist.barrier()
        exchange.close()
        dist.destroy_process_group()


def main_sum_trace() -> None:
    """Where the time of the fused full sum + exchange goes, per rank.

        python -m torch.distributed.run --nproc-per-node N -m fast_dl_b200.opbench --sum-trace [--json out.json]

    Every rank runs the large-sweep step (add, broadcast add, full sum with the exchange in the
    kernel) on its shard of 2^28 / N elements, `--steps` steps back to back, `--reps` times.  With
    the tuning key "sum_trace" set, the CTA that finishes the last sum of a repetition leaves
    %globaltimer stamps; the table gives, per rank, the mean time from the kernel's start to the
    last cluster's ticket (the streaming part), from there to the folded partial, to the peer
    stores, to the moment all peers' partials have been seen (NVLink latency + the skew between
    ranks that the exchange absorbs) and to the written result.
    """
    import os

    import torch
    import torch.distributed as dist
    from fast_dl_b200 import capi
    from fast_dl_b200.sharding import shard_rows

    ap = argparse.ArgumentParser()
    ap.add_argument("--sum-trace", action="store_true")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--json", default=None)
    ap.add_argument("--tune", action="append", default=[])
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    capi.lib()
    capi.use_device(local)
    for kv in args.tune:
        k, v = kv.split("=")
        capi.set_tuning(k, int(v))
    dev = torch.device("cuda", local)
    exchange = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

        def gather(handle):
            handles = [None] * world
            dist.all_gather_object(handles, handle)
            return handles
        exchange = capi.Exchange(world, rank, gather)
        dist.barrier()
    R = C = 16384
    r = shard_rows(R, world, rank).count
    gen = torch.Generator(device=dev).manual_seed(42 + rank)
    a, b, d, f = (torch.empty(r * C, dtype=torch.float32, device=dev).uniform_(-1, 1, generator=gen) for _ in range(4))
    c, e = torch.empty_like(a), torch.empty_like(a)
    row = torch.empty((1, C), dtype=torch.float32, device=dev).uniform_(-1, 1, generator=gen)
    s32 = torch.zeros(1, dtype=torch.float32, device=dev)
    s64 = torch.zeros(1, dtype=torch.float64, device=dev)

    def step():
        capi.binary(a, b, capi.ADD, out=c)
        capi.broadcast_binary(d.view(r, C), row, capi.ADD, out=e.view(r, C))
        if exchange is not None:
            exchange.sum(f, s32, s64)
        else:
            capi.full_sum(f)

    for _ in range(5):
        step()
    torch.cuda.synchronize()
    capi.set_tuning("sum_trace", 1)
    names = ["stream_us", "fold_us", "send_us", "wait_peers_us", "write_us", "tail_cycles"]
    rows = []
    for _ in range(args.reps):
        if world > 1:
            dist.barrier()
        for _ in range(args.steps):
            step()
        torch.cuda.synchronize()
        w = capi.sum_trace()
        t_fold_end = w[2]
        sent = w[3] if exchange is not None else t_fold_end
        seen = w[4] if exchange is not None else sent
        rows.append([(w[1] - w[0]) / 1e3, (w[2] - w[1]) / 1e3, (sent - t_fold_end) / 1e3, (seen - sent) / 1e3,
                     (w[5] - seen) / 1e3, float(w[6])])
    capi.set_tuning("sum_trace", 0)
    mean = [statistics.mean(col) for col in zip(*rows)]
    med = [statistics.median(col) for col in zip(*rows)]
    mine = {"rank": rank, "mean": dict(zip(names, mean)), "median": dict(zip(names, med))}
    everyone = [mine]
    if world > 1:
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
    if rank == 0:
        print(f"full sum + exchange on {world} GPU(s), shard {r * C} elements; median over {args.reps} repetitions")
        print("rank  " + "  ".join(f"{n:>14s}" for n in names))
        for rec in everyone:
            print(f"{rec['rank']:4d}  " + "  ".join(f"{rec['median'][n]:14.2f}" for n in names))
        if args.json:
            Path(args.json).write_text(json.dumps({"n_gpus": world, "ranks": everyone}, indent=1))
    torch.cuda.synchronize()
    capi.take_device_error()
    if world > 1:
        dist.barrier()
        exchange.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    if "--sum-trace" in sys.argv:
        main_sum_trace()
    elif "--sharded" in sys.argv:
        main_sharded()
    else:
        main()
