"""Builds oracle/_build/libfdl_oracle.so from oracle/fdl_oracle.c (test infrastructure).

    python -m oracle.build_oracle

Flags are part of the oracle's definition: -O2 -ffp-contract=off -fno-fast-math, baseline
x86-64 (no -march=native), so a*b+c is never fused and results do not depend on the host.
"""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "fdl_oracle.c"
OUT = HERE / "_build" / "libfdl_oracle.so"
CFLAGS = ["-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-std=c99", "-Wall", "-Wextra"]


def build(force: bool = False) -> Path:
    OUT.parent.mkdir(parents=True, exist_ok=True)
    if force or not OUT.exists() or OUT.stat().st_mtime < SRC.stat().st_mtime:
        cmd = ["gcc", *CFLAGS, str(SRC), "-o", str(OUT), "-lm"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("oracle build failed:\n" + proc.stdout + proc.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
