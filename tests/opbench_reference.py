"""Per-op table with the reference's own CUDA kernels timed beside this library's.

    python tests/opbench_reference.py [--configs c1,...] [--json out.json]

The reference's kernels (recompiled for sm_100a into oracle/_ref/libref.so by
oracle/build_ref.py) are test infrastructure, so this entry point lives with the tests; the
table machinery is fast_dl_b200/opbench.py, which knows nothing about them.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from fast_dl_b200 import opbench  # noqa: E402
from oracle import ref  # noqa: E402

if __name__ == "__main__":
    opbench.main(ref=ref if ref.available() else None)
