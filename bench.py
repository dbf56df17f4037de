#!/usr/bin/env python
"""Bench of the fast_dl tensor hot path on B200: effective GB/s and fraction of the HBM roofline.

Workload: the large-tensor sweep (268,435,456 fp32 elements, uniform [-1, 1]) -- one "step" is
    1. c = a + b                                   (12 B/element)
    2. e = view(d, [16384, 16384]) + row[1, 16384] ( 8 B/element + the row)
    3. s = sum(f)  (+ all-reduce of the per-GPU partials when N > 1)   (4 B/element)
The tensors are partitioned along the leading dimension over the N ranks (one process per
GPU; row vector replicated), so total work is fixed as N grows ("strong" scaling).  The six
tensors are distinct, so every step streams 6 x (1 GiB / N) per GPU: far more than the L2.

    python bench.py [--gpus N] [--steps K] [--warmup W]          # this repository's CUDA path
    python bench.py --impl reference [...]                       # the reference's CPU code on the host cores

Prints ONE JSON line (rank 0).  `value` is whole-job algorithmic GB/s with inputs resident in
HBM; `e2e` is the same metric through the host-buffer C-ABI entry points, host<->device copies
inside the timed region; `roofline` describes the dominant kernel (the binary add);
`cpu_baseline` is the reference's CPU code timed on this box's host cores.
"""
from __future__ import annotations

import argparse
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

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None

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
# ---------------------------------------------------------------------------------------------

class CpuPath:
    """One step of the sweep on the host cores, over `rows` rows of the [ROWS, COLS] view."""

    def __init__(self, threads: int | None = None):
        from oracle import oracle as orc
        from oracle import ref
        self.orc, self.ref = orc, ref
        self.have_ref = ref.available()
        self.threads = threads or os.cpu_count() or 1
        self.pool = ThreadPoolExecutor(self.threads)
        orc.lib()

    @property
    def kind(self) -> str:
        return "reference" if self.have_ref else "port"

    def describe(self) -> str:
        add = ("vector_add_cpu of the reference (tests/benchmarks/vector_add/vector_add_benchmark.cu:13-18)"
               if self.have_ref else "oracle port of the reference's vector_add_cpu")
        return (f"add: {add}; broadcast add and full sum: oracle port (the reference has no such op); "
                f"rows split over {self.threads} threads")

    def _split(self, rows: int):
        per = -(-rows // self.threads)
        return [(lo, min(rows, lo + per)) for lo in range(0, rows, per)]

    def step(self, a, b, c, row, rows: int) -> float:
        """a, b, c: numpy float32 [rows*COLS]; returns the sum (float)."""
        import numpy as np
        orc, ref = self.orc, self.ref
        parts = self._split(rows)
        if self.have_ref:
            ref.cpu_vector_add(a[:rows * COLS], b[:rows * COLS], threads=self.threads, out=c)
        else:
            list(self.pool.map(lambda p: orc.lib().orc_binary_f32(
                _fptr(a, p[0] * COLS), _fptr(b, p[0] * COLS), _fptr(c, p[0] * COLS),
                _i64((p[1] - p[0]) * COLS), 0), parts))
        # row-broadcast add: the reference's row-bias arithmetic (src/kernels/cuda/bias.cu:5-12), in place on c
        list(self.pool.map(lambda p: orc.lib().orc_add_row_bias_f32(
            _fptr(c, p[0] * COLS), _fptr(row, 0), _i64(p[1] - p[0]), _i64(COLS), 0), parts))
        sums = list(self.pool.map(lambda p: orc.lib().orc_sum_f64(
            _fptr(b, p[0] * COLS), _i64((p[1] - p[0]) * COLS)), parts))
        return float(np.sum(np.asarray(sums, dtype=np.float64)))


def _fptr(arr, offset_elems):
    import ctypes as C
    return C.cast(arr.ctypes.data + 4 * offset_elems, C.POINTER(C.c_float))


def _i64(v):
    import ctypes as C
    return C.c_int64(v)


def time_cpu(cpu: CpuPath, host, rows: int, steps: int, warmup: int) -> float:
    """Seconds per step of the CPU path over `rows` rows."""
    a, b, c, row = host
    for _ in range(warmup):
        cpu.step(a, b, c, row, rows)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu.step(a, b, c, row, rows)
    return (time.perf_counter() - t0) / steps


def host_inputs(rows: int, seed: int, pinned: bool):
    """Seeded uniform[-1,1] host tensors for `rows` rows (torch CPU tensors + numpy views)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    n = rows * COLS

    def mk(count):
        t = torch.empty(count, dtype=torch.float32, pin_memory=pinned)
        t.uniform_(-1.0, 1.0, generator=g)
        return t

    return mk(n), mk(n), torch.empty(n, dtype=torch.float32, pin_memory=pinned), mk(COLS)


# ---------------------------------------------------------------------------------------------
# reference arm
# ---------------------------------------------------------------------------------------------

def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = CpuPath()
    # Bounded sample: as many leading rows as keep the whole run within ~2 minutes.
    probe_rows = ROWS // 64
    host = host_inputs(probe_rows, 42, pinned=False)
    np_host = tuple(t.numpy() for t in host)
    t_probe = time_cpu(cpu, np_host, probe_rows, steps=2, warmup=1)
    budget = 120.0 / max(1, args.steps + args.warmup)
    rows = int(min(ROWS, max(probe_rows, probe_rows * budget / max(t_probe, 1e-9))))
    rows = max(64, rows // 64 * 64)
    if rows != probe_rows:
        host = host_inputs(rows, 42, pinned=False)
        np_host = tuple(t.numpy() for t in host)
    sec = time_cpu(cpu, np_host, rows, args.steps, args.warmup)
    nbytes = sum(algorithmic_bytes(rows, COLS).values())
    gbs = nbytes / sec / 1e9
    sample = f"{rows} of {ROWS} rows of the [16384,16384] view per step ({rows * COLS} elements); " + cpu.describe()
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "large_tensor_sweep_268435456_f32: add, row-broadcast add, full sum",
                   "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cpu.threads, "kind": cpu.kind, "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# this repository's CUDA path
# ---------------------------------------------------------------------------------------------

def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from fast_dl_b200 import capi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    capi.lib()
    capi.use_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    total_rows = args.rows
    rows = total_rows // world + (1 if rank < total_rows % world else 0)
    n = rows * COLS
    dev = torch.device("cuda", local)
    gen = torch.Generator(device=dev).manual_seed(42 + rank)

    def uni(count):
        return torch.empty(count, dtype=torch.float32, device=dev).uniform_(-1.0, 1.0, generator=gen)

    a, b, d, f = uni(n), uni(n), uni(n), uni(n)
    c, e = torch.empty_like(a), torch.empty_like(a)
    row = uni(COLS)
    if world > 1:
        dist.broadcast(row, 0)
    sum32 = torch.zeros(1, dtype=torch.float32, device=dev)
    sum64 = torch.zeros(1, dtype=torch.float64, device=dev)
    d2 = d.view(rows, COLS)
    e2 = e.view(rows, COLS)

    def step(events=None):
        if events is not None:
            events[0].record()
        capi.binary(a, b, capi.ADD, out=c)
        if events is not None:
            events[1].record()
        capi.broadcast_binary(d2, row.view(1, COLS), capi.ADD, out=e2)
        if events is not None:
            events[2].record()
        capi.check(capi.lib().fdl_sum_f32(f.data_ptr(), n, sum32.data_ptr(), sum64.data_ptr(), None, 0,
                                          torch.cuda.current_stream().cuda_stream), "fdl_sum_f32")
        if events is not None:
            events[3].record()
        if world > 1:
            dist.all_reduce(sum64)  # per-GPU partials -> global sum, on the same stream

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- timed region: exactly K steps ---------------------------------------------------------
    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(K)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    sampler.start()
    barrier()
    start.record()
    for k in range(K):
        step(ev[k])
    stop.record()
    barrier()
    clocks = sampler.stop()
    ms_total = start.elapsed_time(stop)
    per_op = [sum(ev[k][i].elapsed_time(ev[k][i + 1]) for k in range(K)) / K for i in range(3)]

    # ---- end to end through the host-buffer entry points ------------------------------------------
    need_host = not args.no_e2e or (rank == 0 and world == 1 and not args.no_cpu)
    ha = hb = hc = hrow = ha2 = hc2 = None
    if need_host:
        ha, hb, hc, hrow = host_inputs(rows, 1000 + rank, pinned=True)
        ha2, hc2 = ha.view(rows, COLS), hc.view(rows, COLS)

    def e2e_step():
        capi.host_binary(ha, hb, hc, capi.ADD)
        capi.host_row_broadcast(ha2, hrow, hc2, capi.ADD)
        s = capi.host_sum(hb)
        if world > 1:
            t = torch.tensor([s], dtype=torch.float64, device=dev)
            dist.all_reduce(t)
            s = float(t.item())
        return s

    e2e_steps = 0 if args.no_e2e else max(2, min(5, K))
    e2e_sec = float("nan")
    if e2e_steps:
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_sec = (time.perf_counter() - t0) / e2e_steps

    # ---- reduce over ranks ------------------------------------------------------------------------------
    stats = torch.tensor([ms_total, e2e_sec, *per_op], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms_total, e2e_sec, t_add, t_bc, t_sum = stats.tolist()

    total_bytes = sum(algorithmic_bytes(total_rows, COLS).values()) + (world - 1) * (4 * COLS + 4)
    value = total_bytes * K / (ms_total * 1e-3) / 1e9
    e2e_value = total_bytes / e2e_sec / 1e9
    peak, peak_kind = measured_peak_gbs()
    shard = algorithmic_bytes(rows, COLS)
    achieved = shard["add"] / (t_add * 1e-3) / 1e9

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "large_tensor_sweep_268435456_f32: add, row-broadcast add, full sum",
                   "partition": f"leading dimension over {world} GPU(s), {rows} of {total_rows} rows on rank 0",
                   "l2": "inputs larger than L2 (six distinct tensors stream per step)"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "GB/s",
                "h2d_bytes_per_step": (4 * n + COLS) * 4 * world, "d2h_bytes_per_step": (2 * n * 4 + 8) * world,
                "steps": e2e_steps},
        "gpu_launches": 3 * K * world,
        "roofline": {"bound": "hbm", "kernel": "map_kernel<4,2,AddFn> (binary add)", "achieved": achieved,
                     "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind,
                     "traffic": traffic_per_launch(shard["add"])},
        "per_op": {
            "add": {"ms": t_add, "GBps": shard["add"] / t_add / 1e6, "frac": shard["add"] / t_add / 1e6 / peak},
            "broadcast_add": {"ms": t_bc, "GBps": shard["broadcast_add"] / t_bc / 1e6,
                              "frac": shard["broadcast_add"] / t_bc / 1e6 / peak},
            "sum": {"ms": t_sum, "GBps": shard["sum"] / t_sum / 1e6, "frac": shard["sum"] / t_sum / 1e6 / peak},
        },
    }

    if args.rows != ROWS:
        line["config"]["workload"] += f" (REDUCED to {args.rows} rows for profiling; not a bench value)"
    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            cpu = CpuPath()
            sample_rows = min(ROWS // 4, rows)
            np_host = (ha.numpy(), hb.numpy(), hc.numpy(), hrow.numpy())
            sec = time_cpu(cpu, np_host, sample_rows, steps=3, warmup=1)
            nb = sum(algorithmic_bytes(sample_rows, COLS).values())
            line["cpu_baseline"] = {
                "value": nb / sec / 1e9, "unit": "GB/s", "cores": cpu.threads, "kind": cpu.kind,
                "sample": f"3 steps over {sample_rows} of {ROWS} rows ({sample_rows * COLS} elements); " + cpu.describe()}
        except Exception as exc:  # the baseline is a report, never a reason to lose the GPU line
            line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port",
                                    "sample": f"failed: {exc!r}"}

    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--rows", type=int, default=ROWS,
                    help="rows of the [rows, 16384] view; smaller than 16384 only for profiler captures")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
