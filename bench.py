#!/usr/bin/env python
"""Bench of the fast_dl tensor hot path on B200: effective GB/s and fraction of the HBM roofline.

Workload: the large-tensor sweep over 268,435,456 fp32 elements,
uniform [-1, 1], viewed as [16384, 16384].  One "step" is
    z = x + y                 binary add                       12 B/element
    w = x + row[1, 16384]     broadcast add against a row       8 B/element (+ the row)
    s = sum(x)                full sum (+ all-reduce of the per-GPU partials when N > 1)   4 B/element
The tensors are partitioned along the leading dimension over the N ranks (one process per
GPU, row vector replicated), so total work is fixed as N grows ("strong" scaling).  In the
device-resident leg every operand is a DISTINCT tensor, so each step streams 6 x (1 GiB / N)
per GPU -- far more than the L2; in the end-to-end leg x and y are host tensors.

    python bench.py [--gpus N] [--steps K] [--warmup W]          # this repository's CUDA path
    python bench.py --impl reference [...]                       # the reference's CPU code on the host cores

Prints ONE JSON line (rank 0).  `value`: whole-job algorithmic GB/s, inputs resident in HBM,
K steps launched back to back.  `per_op` / `roofline`: a second pass with an event between
the launches (the dominant kernel is the binary add).  `sustained`: the same step repeated for
at least a second with the clocks sampled.  `check`: the results of one more step verified on
every rank -- z and w bit for bit against torch, the sums against an fp64 sum (an NCCL
all-reduce of the ranks' fp64 sums at N > 1), all ranks' result bits against each other; a
mismatch makes the run exit non-zero.  `config4_per_op`: row softmax / layernorm on
[65536,1024] sharded by rows over the N ranks.  `e2e`: the same metric through the host-buffer
C-ABI entry point (pinned host tensors in, results in host memory, copies inside the timed
region), beside the three separate host calls.  `cpu_baseline`: the reference's CPU code on
this box's host cores.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_ELEMS = 268_435_456
COLS = 16_384
ROWS = N_ELEMS // COLS
METRIC = "effective_GBps_large_tensor_sweep"
WORKLOAD = "large_tensor_sweep_268435456_f32: z=x+y, w=x+row[1,16384], s=sum(x)"


def workload_config(n_gpus: int, rows: int) -> dict:
    """What is computed and how it is partitioned: the same dictionary in both arms."""
    cfg = {"workload": WORKLOAD,
           "partition": f"leading dimension ({rows} rows of 16384 floats) in contiguous blocks over {n_gpus} GPU(s)",
           "l2": "inputs larger than L2"}
    if rows != ROWS:
        cfg["workload"] += f" (REDUCED to {rows} rows for a profiler capture; not a bench value)"
    return cfg


def algorithmic_bytes(rows: int, cols: int) -> dict:
    n = rows * cols
    return {"add": 12 * n, "broadcast_add": 8 * n + 4 * cols, "sum": 4 * n + 4}


def measured_peak_gbs() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._nv = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# ---------------------------------------------------------------------------------------------
# CPU side: the reference's own CPU code (oracle/_ref) where it has some, the oracle port else.
# Only this leg (cpu_baseline / --impl reference) touches oracle/.
# ---------------------------------------------------------------------------------------------

def _fptr(arr, offset_elems=0):
    return C.cast(arr.ctypes.data + 4 * offset_elems, C.POINTER(C.c_float))


class CpuPath:
    """One step of the sweep on the host cores over `rows` rows of the [ROWS, COLS] view."""

    def __init__(self, threads: int | None = None):
        from oracle import oracle as orc
        from oracle import ref
        self.lib, self.ref = orc.lib(), ref
        self.have_ref = ref.available()
        self.threads = threads or os.cpu_count() or 1
        self.pool = ThreadPoolExecutor(self.threads)

    @property
    def kind(self) -> str:
        return "reference" if self.have_ref else "port"

    def describe(self) -> str:
        add = ("the reference's vector_add_cpu (tests/benchmarks/vector_add/vector_add_benchmark.cu:13-18)"
               if self.have_ref else "oracle port of the reference's vector_add_cpu")
        return (f"add: {add}; broadcast add and full sum: oracle port (the reference has no such op); "
                f"rows split over {self.threads} threads")

    def _split(self, rows: int):
        per = -(-rows // self.threads)
        return [(lo, min(rows, lo + per)) for lo in range(0, rows, per)]

    def step(self, x, y, z, w, row, rows: int) -> float:
        """x, y, z, w: numpy float32 of at least rows*COLS elements; returns sum(x)."""
        lib, parts = self.lib, self._split(rows)
        n = rows * COLS
        if self.have_ref:
            self.ref.cpu_vector_add(x[:n], y[:n], threads=self.threads, out=z)
        else:
            list(self.pool.map(lambda p: lib.orc_binary_f32(
                _fptr(x, p[0] * COLS), _fptr(y, p[0] * COLS), _fptr(z, p[0] * COLS),
                C.c_int64((p[1] - p[0]) * COLS), 0), parts))
        list(self.pool.map(lambda p: lib.orc_add_row_f32(
            _fptr(x, p[0] * COLS), _fptr(row), _fptr(w, p[0] * COLS), C.c_int64(p[1] - p[0]), C.c_int64(COLS)), parts))
        sums = list(self.pool.map(lambda p: lib.orc_sum_f64(
            _fptr(x, p[0] * COLS), C.c_int64((p[1] - p[0]) * COLS)), parts))
        return float(sum(sums))


def time_cpu(cpu: CpuPath, host, rows: int, steps: int, warmup: int) -> float:
    """Seconds per step of the CPU path over `rows` rows."""
    for _ in range(warmup):
        cpu.step(*host, rows)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu.step(*host, rows)
    return (time.perf_counter() - t0) / steps


def host_inputs(rows: int, seed: int, pinned: bool):
    """Seeded uniform[-1,1] host tensors x, y (inputs), z, w (results), row, for `rows` rows."""
    import torch
    g = torch.Generator().manual_seed(seed)
    n = rows * COLS

    def mk(count, fill=True):
        t = torch.empty(count, dtype=torch.float32, pin_memory=pinned)
        if fill:
            t.uniform_(-1.0, 1.0, generator=g)
        else:
            t.zero_()  # touch the pages
        return t

    return mk(n), mk(n), mk(n, False), mk(n, False), mk(COLS)


# ---------------------------------------------------------------------------------------------
# reference arm: the reference's CPU implementation of the path on the host cores
# ---------------------------------------------------------------------------------------------

def run_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cpu = CpuPath()
    # Bounded sample: as many leading rows as keep the whole run within ~2 minutes.
    probe_rows = ROWS // 64
    host = tuple(t.numpy() for t in host_inputs(probe_rows, 42, pinned=False))
    t_probe = time_cpu(cpu, host, probe_rows, steps=2, warmup=1)
    budget = 120.0 / max(1, args.steps + args.warmup)
    rows = int(min(ROWS, max(probe_rows, probe_rows * budget / max(t_probe, 1e-9))))
    rows = max(64, rows // 64 * 64)
    if rows != probe_rows:
        host = tuple(t.numpy() for t in host_inputs(rows, 42, pinned=False))
    sec = time_cpu(cpu, host, rows, args.steps, args.warmup)
    gbs = sum(algorithmic_bytes(rows, COLS).values()) / sec / 1e9
    sample = f"{rows} of {ROWS} rows of the [16384,16384] view per step ({rows * COLS} elements); " + cpu.describe()
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus, ROWS),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cpu.threads, "kind": cpu.kind, "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# this repository's CUDA path
# ---------------------------------------------------------------------------------------------

def traffic_per_launch(algorithmic: int):
    """DRAM bytes per launch of the add kernel from the committed ncu capture, scaled by size."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if not p.exists():
        return None
    try:
        rec = json.loads(p.read_text())["map_kernel_add"]
        return rec["dram_bytes"] / rec["algorithmic_bytes"] * algorithmic
    except Exception:
        return None


def run_ours(args) -> None:
    import statistics

    import torch
    import torch.distributed as dist
    from fast_dl_b200 import capi
    from fast_dl_b200.sharding import shard_rows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1:
        raise SystemExit("launch with `python -m torch.distributed.run --nproc-per-node N bench.py --gpus N`")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    capi.lib()
    capi.use_device(local)
    for kv in args.tune:
        key, val = kv.split("=")
        capi.set_tuning(key, int(val))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    shard = shard_rows(args.rows, world, rank)
    rows, n = shard.count, shard.count * COLS
    dev = torch.device("cuda", local)
    gen = torch.Generator(device=dev).manual_seed(42 + rank)

    def uni(count):
        return torch.empty(count, dtype=torch.float32, device=dev).uniform_(-1.0, 1.0, generator=gen)

    # Six distinct tensors per step so that nothing is L2-resident from the previous op.
    a, b, d, f = uni(n), uni(n), uni(n), uni(n)
    c, e = torch.empty_like(a), torch.empty_like(a)
    row = uni(COLS)
    if world > 1:
        dist.broadcast(row, 0)
    sum32 = torch.zeros(1, dtype=torch.float32, device=dev)
    sum64 = torch.zeros(1, dtype=torch.float64, device=dev)
    exchange = None
    if world > 1 and args.allreduce in ("fused", "split"):
        def gather(handle: bytes):
            handles = [None] * world
            dist.all_gather_object(handles, handle)
            return handles
        exchange = capi.Exchange(world, rank, gather)
        dist.barrier()
    stream = torch.cuda.current_stream().cuda_stream
    lib = capi.lib()

    split = exchange is not None and args.allreduce == "split"

    # The timed loop calls the C ABI with arguments converted once: at 8 GPUs a step is ~150 us
    # and per-call Python work (tensor checks, shape arithmetic) would otherwise rival it.
    import ctypes as C
    ADD = capi.ADD
    pa, pb, pc, pd, pe, pf, prow = (t.data_ptr() for t in (a, b, c, d, e, f, row))
    p32, p64 = sum32.data_ptr(), sum64.data_ptr()
    i64x2 = C.c_int64 * 2
    bshape, bstr_a, bstr_row = i64x2(rows, COLS), i64x2(COLS, 1), i64x2(0, 1)
    xctx = exchange.ctx if exchange is not None else None

    def must(status, where):
        if status != 0:
            capi.check(status, where)

    def op_add():
        must(lib.fdl_binary_f32(pa, pb, pc, n, ADD, stream), "fdl_binary_f32")

    def op_broadcast():
        must(lib.fdl_broadcast_binary_f32(pd, prow, pe, 2, bshape, bstr_a, bstr_row, ADD, stream),
             "fdl_broadcast_binary_f32")

    def op_sum():
        if exchange is not None:
            # sum + exchange of the per-GPU partials over NVLink in ONE kernel
            must(lib.fdl_sum_allreduce_f32(pf, n, p32, p64, xctx, None, 0, stream), "fdl_sum_allreduce_f32")
        else:
            must(lib.fdl_sum_f32(pf, n, p32, p64, None, 0, stream), "fdl_sum_f32")

    def op_sum_start():
        must(lib.fdl_sum_allreduce_start_f32(pf, n, xctx, None, 0, stream), "fdl_sum_allreduce_start_f32")

    def op_sum_finish():
        must(lib.fdl_sum_allreduce_finish_f32(p32, p64, xctx, stream), "fdl_sum_allreduce_finish_f32")

    if split:
        # The three ops of a step are independent, so the sum goes first: its kernel sends the
        # rank's partial to all ranks and returns; the add and the broadcast add run while the
        # partials cross NVLink and slower ranks catch up; a one-warp kernel folds them last.
        plan = [("sum", op_sum_start), ("add", op_add), ("broadcast_add", op_broadcast), ("sum", op_sum_finish)]
    else:
        plan = [("add", op_add), ("broadcast_add", op_broadcast), ("sum", op_sum)]
    launches_per_step = len(plan)
    fns = [fn for _, fn in plan]
    nccl_sum = world > 1 and exchange is None

    def step():
        for fn in fns:
            fn()
        if nccl_sum:
            dist.all_reduce(sum64)  # per-GPU partials -> global sum: same stream, no host round trip

    def step_with_events(events):
        for i, fn in enumerate(fns):
            events[i].record()
            fn()
        events[len(fns)].record()
        if nccl_sum:
            dist.all_reduce(sum64)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()

    # ---- timed region: exactly K steps, launches back to back (no events between the ops) ----------
    K = args.steps
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local, period_s=0.002)
    sampler.start()
    barrier()
    start.record()
    # Host time to enqueue a step, over the first steps only: later the driver's launch queue
    # is full and the host waits for the GPU, which says nothing about the host.
    k_host = min(K, 100)
    t_host = time.perf_counter()
    for k in range(K):
        if k == k_host:
            enqueue_us = (time.perf_counter() - t_host) * 1e6 / k_host
        step()
    stop.record()
    if K == k_host:
        enqueue_us = (time.perf_counter() - t_host) * 1e6 / k_host
    barrier()
    clocks = sampler.stop()
    ms_total = start.elapsed_time(stop)

    # ---- second pass, outside the headline: the same steps with an event between the ops -----------
    K2 = max(3, min(K, 50))
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(plan) + 1)] for _ in range(K2)]
    barrier()
    for k in range(K2):
        step_with_events(ev[k])
    barrier()
    per_op = [sum(ev[k][i].elapsed_time(ev[k][i + 1]) for k in range(K2) for i, (name, _) in enumerate(plan)
                  if name == which) / K2 for which in ("add", "broadcast_add", "sum")]

    # ---- third pass: the same step for at least a second, with the clocks sampled under load ----
    K3 = int(min(20000, max(K, args.sustain_s * 1e3 / max(ms_total / K, 1e-3))))
    if world > 1:
        k3 = torch.tensor([K3], dtype=torch.int64, device=dev)
        dist.all_reduce(k3, op=dist.ReduceOp.MAX)
        K3 = int(k3.item())
    s_start, s_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler3 = ClockSampler(local, period_s=0.01)
    sampler3.start()
    barrier()
    s_start.record()
    for _ in range(K3):
        step()
    s_stop.record()
    barrier()
    clocks3 = sampler3.stop()
    ms_sustained = s_start.elapsed_time(s_stop)

    # ---- results of the last step, checked outside every timed region --------------------------------
    step()
    torch.cuda.synchronize()
    check = {}
    check["add"] = int((c.view(torch.int32) != (a + b).view(torch.int32)).sum().item())
    check["broadcast"] = int((e.view(torch.int32) != (d.view(rows, COLS) + row).view(-1).view(torch.int32)).sum().item())
    ref64 = f.double().sum().reshape(1)
    sq = (f.double() * f.double()).sum().reshape(1)
    if world > 1:
        dist.all_reduce(ref64)
        dist.all_reduce(sq)
    norm = float(sq.sqrt().item())
    got64, got32 = float(sum64.item()), float(sum32.item())
    check["sum_rel"] = abs(got64 - float(ref64.item())) / max(abs(float(ref64.item())), norm)
    # With --allreduce nccl only the fp64 partial is all-reduced; the fp32 output stays per rank.
    check["sum_f32_rel"] = 0.0 if nccl_sum else abs(got32 - float(ref64.item())) / max(abs(float(ref64.item())), norm)
    agree = True
    if world > 1:
        mine = torch.cat([sum64.view(torch.int64), (sum64 if nccl_sum else sum32.double()).view(torch.int64)])
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        agree = all(bool(torch.equal(t, everyone[0])) for t in everyone)
    check["ranks_agree"] = agree
    bad = torch.tensor([check["add"], check["broadcast"], int(check["sum_rel"] > 1e-5), int(check["sum_f32_rel"] > 1e-5),
                        int(not agree)], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(bad)  # a mismatch on any rank fails the run
    check["add"], check["broadcast"] = int(bad[0].item()), int(bad[1].item())
    check["what"] = ("differing elements of z = x + y and w = x + row against torch on the device (all ranks); the fp64 "
                     "and fp32 full sums against an fp64 sum of the same data (NCCL all-reduce of the ranks' fp64 sums "
                     "at N > 1), relative to max(|sum|, ||x||_2), allowed 1e-5; the result bits of all ranks compared")
    check_failed = bool(bad.sum().item() != 0)
    del ref64, sq

    # ---- configuration 4 (row softmax / layernorm on [65536,1024]) sharded by rows over the ranks ----
    del c, e, d, f, a, b
    torch.cuda.empty_cache()
    config4 = None
    if not args.no_c4:
        config4 = config4_per_op(capi, dist, dev, world, rank)

    # ---- end to end: host tensors in, host results out, through the C ABI ------------------------
    need_host = not args.no_e2e or (rank == 0 and world == 1 and not args.no_cpu)
    host = None
    e2e_steps, e2e_sec, e2e3_sec, link_sec = 0, float("nan"), 0.0, 0.0
    if need_host:
        host = host_inputs(rows, 1000 + rank, pinned=True)
    if not args.no_e2e:
        hx, hy, hz, hw, hrow = host
        hx2, hy2, hz2, hw2 = (t.view(rows, COLS) for t in (hx, hy, hz, hw))
        tsum = torch.zeros(1, dtype=torch.float64, device=dev)

        def finish_sum(s):
            if world > 1:
                tsum.fill_(s)
                dist.all_reduce(tsum)
                s = float(tsum.item())
            return s

        def e2e_step():
            return finish_sum(capi.host_sweep(hx2, hy2, hrow, hz2, hw2))

        def e2e_three_calls():
            # The same three results from three separate calls: x crosses the link three times.
            capi.host_binary(hx, hy, hz, ADD)
            capi.host_row_broadcast(hx2, hrow, hw2, ADD)
            return finish_sum(capi.host_sum(hx))

        def time_host(fn, steps):
            fn()
            barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                fn()
            barrier()
            return (time.perf_counter() - t0) / steps

        e2e_steps = max(2, min(5, K))
        e2e_sec = time_host(e2e_step, e2e_steps)
        e2e3_sec = time_host(e2e_three_calls, 2)

        # What the host link itself gives on this box, for the e2e figure to be read against:
        # x up and z down as two plain pinned copies running at the same time (all ranks at once).
        up_dst = torch.empty_like(hx, device=dev)
        down_src = torch.empty_like(hx, device=dev).fill_(1.0)
        s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()

        def duplex_copy():
            with torch.cuda.stream(s_up):
                up_dst.copy_(hx, non_blocking=True)
            with torch.cuda.stream(s_down):
                hz.copy_(down_src, non_blocking=True)

        duplex_copy()
        barrier()
        t0 = time.perf_counter()
        for _ in range(3):
            duplex_copy()
        barrier()
        link_sec = (time.perf_counter() - t0) / 3
        del up_dst, down_src

    # ---- reduce over ranks: the slowest rank defines the time --------------------------------------
    stats = torch.tensor([ms_total, e2e_sec if e2e_steps else 0.0, *per_op, enqueue_us, link_sec, ms_sustained,
                          e2e3_sec], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms_total, e2e_sec, t_add, t_bc, t_sum, enqueue_us, link_sec, ms_sustained, e2e3_sec = stats.tolist()

    total_bytes = sum(algorithmic_bytes(args.rows, COLS).values()) + (world - 1) * (4 * COLS + 4)
    value = total_bytes * K / (ms_total * 1e-3) / 1e9
    peak, peak_kind = measured_peak_gbs()
    big = algorithmic_bytes(shard_rows(args.rows, world, 0).count, COLS)  # rank 0 holds a largest shard
    achieved = big["add"] / (t_add * 1e-3) / 1e9

    def op_line(name, t):
        gbs = big[name] / t / 1e6
        return {"ms": t, "GBps": gbs, "frac": gbs / peak}

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": K, "warmup": warmup,
        "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(world, args.rows),
        "clocks": clocks,
        "check": check,
        "e2e": {"value": (total_bytes / e2e_sec / 1e9) if e2e_steps else None, "unit": "GB/s",
                "h2d_bytes_per_step": (2 * args.rows * COLS + world * COLS) * 4,
                "d2h_bytes_per_step": 2 * args.rows * COLS * 4 + 8 * world, "steps": e2e_steps,
                "api": "fdl_host_sweep_f32 (pinned host tensors in, host results out)",
                "three_separate_calls": (None if not e2e3_sec else {
                    "value": total_bytes / e2e3_sec / 1e9, "unit": "GB/s",
                    "api": "fdl_host_binary_f32 + fdl_host_row_broadcast_f32 + fdl_host_sum_f32",
                    "h2d_bytes_per_step": (4 * args.rows * COLS + world * COLS) * 4,
                    "d2h_bytes_per_step": 2 * args.rows * COLS * 4 + 8 * world}),
                # e2e moves 2 tensors up and 2 down per step; the link line is one up + one down at once
                "link": (None if not link_sec else {
                    "duplex_GBps_per_direction": args.rows * COLS * 4 / link_sec / 1e9,
                    "floor_ms_per_step": 2 * link_sec * 1e3,
                    "frac_of_link_floor": 2 * link_sec / e2e_sec,
                    "what": "plain pinned copies of one tensor up and one down at the same time, all ranks"})},
        "gpu_launches": launches_per_step * K * world,
        "host_enqueue_us_per_step": enqueue_us,
        "roofline": {"bound": "hbm", "kernel": "map_kernel<4,2,4,AddFn> (binary add)", "achieved": achieved,
                     "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind,
                     "traffic": traffic_per_launch(big["add"]),
                     "timed": f"events around each launch in a second pass of {K2} steps (not in the headline region)"},
        "per_op": {"add": op_line("add", t_add), "broadcast_add": op_line("broadcast_add", t_bc),
                   "sum": op_line("sum", t_sum)},
        "sustained": {"value": total_bytes * K3 / (ms_sustained * 1e-3) / 1e9, "unit": "GB/s", "steps": K3,
                      "seconds": ms_sustained * 1e-3, "ms_per_step": ms_sustained / K3, "clocks": clocks3},
        "implementation": {
            "tensors": "six distinct device tensors stream per step",
            "full_sum_exchange": ("none (1 GPU)" if world == 1 else
                                  "split: the sum kernel sends the partial over NVLink (peer stores), the "
                                  "other two ops overlap the exchange, a one-warp kernel folds" if split else
                                  "fused into the sum kernel (peer stores over NVLink)" if exchange is not None
                                  else "NCCL all-reduce of one double"),
            "tuning": args.tune},
    }
    if config4 is not None:
        line["config4_per_op"] = config4

    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            cpu = CpuPath()
            sample_rows = min(ROWS // 4, rows)
            sec = time_cpu(cpu, tuple(t.numpy() for t in host), sample_rows, steps=3, warmup=1)
            nb = sum(algorithmic_bytes(sample_rows, COLS).values())
            line["cpu_baseline"] = {
                "value": nb / sec / 1e9, "unit": "GB/s", "cores": cpu.threads, "kind": cpu.kind,
                "sample": f"3 steps over {sample_rows} of {ROWS} rows ({sample_rows * COLS} elements); " + cpu.describe()}
        except Exception as exc:  # the baseline is a report, never a reason to lose the GPU line
            line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port",
                                    "sample": f"failed: {exc!r}"}

    torch.cuda.synchronize()
    capi.take_device_error()  # raises if a bounded device-side wait ran out
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        if exchange is not None:
            exchange.close()
        dist.destroy_process_group()
    if check_failed:
        raise SystemExit(f"result check failed: {check}")


def config4_per_op(capi, dist, dev, world: int, rank: int, iters: int = 10) -> dict:
    """Row softmax and layernorm on logits[65536,1024], sharded by rows over the ranks: each rank
    times its shard (CUDA events around one launch, L2 flushed by reading 512 MiB before it,
    median of `iters`), the slowest rank defines the time, GB/s is whole-tensor bytes over it."""
    import statistics

    import torch
    from fast_dl_b200.sharding import shard_rows

    R, Ccols = 65536, 1024
    r = shard_rows(R, world, rank).count
    gen = torch.Generator(device=dev).manual_seed(4242 + rank)
    logits = torch.empty((r, Ccols), dtype=torch.float32, device=dev).normal_(0.0, 3.0, generator=gen)
    gamma = torch.empty(Ccols, dtype=torch.float32, device=dev).uniform_(0.9, 1.1, generator=gen)
    beta = torch.empty(Ccols, dtype=torch.float32, device=dev).uniform_(-0.1, 0.1, generator=gen)
    out = torch.empty_like(logits)
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    peak, _ = measured_peak_gbs()
    ops = {
        "softmax": (8 * R * Ccols, lambda: capi.softmax_rows(logits, out=out)),
        "layernorm": (8 * R * Ccols, lambda: capi.layernorm_rows(logits, out=out)),
        "layernorm_gamma_beta": (8 * R * Ccols + 8 * Ccols * world, lambda: capi.layernorm_rows(logits, gamma, beta, out=out)),
    }
    res = {"shape": [R, Ccols], "rows_per_gpu": r, "method": "per-launch CUDA events, read-flushed L2, median, max over ranks"}
    for name, (nbytes, fn) in ops.items():
        times = []
        for i in range(iters + 3):
            if world > 1:
                dist.barrier()
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
        ms = float(t.item())
        res[name] = {"ms": ms, "GBps": nbytes / ms / 1e6, "frac_per_gpu": nbytes / ms / 1e6 / (world * peak)}
    # correctness of the shard-local results: rows sum to one; layernorm rows have mean 0, variance 1
    capi.softmax_rows(logits, out=out)
    res["softmax_row_sum_err"] = float((out.double().sum(dim=1) - 1.0).abs().max().item())
    capi.layernorm_rows(logits, out=out)
    res["layernorm_row_mean_abs"] = float(out.double().mean(dim=1).abs().max().item())
    del logits, out, flush
    torch.cuda.empty_cache()
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--allreduce", choices=["fused", "split", "nccl"], default="fused",
                    help="N > 1: exchange the full-sum partials inside the sum kernel over NVLink peer stores "
                         "in one call (fused), in two halves with the other ops of the step between them "
                         "(split), or with a separate NCCL all-reduce (nccl)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-c4", action="store_true", help="skip the per-op figures of configuration 4")
    ap.add_argument("--sustain-s", type=float, default=1.0,
                    help="length in seconds of the extra pass that repeats the step with the clocks sampled")
    ap.add_argument("--tune", action="append", default=[], help="key=value passed to fdl_set_tuning")
    ap.add_argument("--rows", type=int, default=ROWS,
                    help="rows of the [rows, 16384] view; smaller than 16384 only for profiler captures")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
