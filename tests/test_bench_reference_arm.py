"""The bench's reference arm on the host cores (no GPU): one bounded step through the command
line, its JSON line checked against the keys both arms have to agree on."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_the_contract_line():
    sys.path.insert(0, str(ROOT))
    import bench

    run = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [l for l in run.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, run.stdout[-2000:]
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    assert line["metric"] == "effective_GBps_large_tensor_sweep" and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["config"] == bench.workload_config(1, bench.ROWS)          # the same dictionary as the GPU arm's
    assert line["value"] > 0 and line["ms_per_step"] > 0
    base = line["cpu_baseline"]
    assert base["kind"] in ("reference", "port") and base["cores"] >= 1 and base["value"] == line["value"]
    assert base["sample"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == line["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_reference_arm_under_the_launcher_prints_one_line_from_rank_0():
    """Launched like the GPU arm for N = 2: rank 0 measures and prints, the other rank leaves with 0."""
    sys.path.insert(0, str(ROOT))
    import bench

    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29617", str(ROOT / "bench.py"),
                          "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [l for l in run.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, run.stdout[-2000:]
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2
    assert line["config"] == bench.workload_config(2, bench.ROWS)


def test_algorithmic_bytes_of_the_step():
    sys.path.insert(0, str(ROOT))
    import bench

    b = bench.algorithmic_bytes(bench.ROWS, bench.COLS)
    assert b == {"add": 3_221_225_472, "broadcast_add": 2_147_549_184, "sum": 1_073_741_828}
    for n in (1, 2, 4, 8):
        cfg = bench.workload_config(n, bench.ROWS)
        assert set(cfg) == {"workload", "partition", "l2"} and f"over {n} GPU(s)" in cfg["partition"]
