"""The C-ABI library loads on a machine without a GPU and exports what the header declares."""
import ctypes
import re

import pytest
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "fdl_kernels.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fdl_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "fdl_binary_f32" in names and "fdl_softmax_rows_f32" in names and len(names) >= 20


def test_library_exports_every_declared_symbol(fdl):
    handle = ctypes.CDLL(str(fdl.library_path()))
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} is declared in include/fdl_kernels.h but not exported"


def test_binding_covers_every_declared_symbol(fdl):
    assert sorted(fdl.PROTOTYPES) == declared_symbols()


def test_no_gpu_calls_needed_for_metadata(fdl):
    lib = fdl.lib()
    assert lib.fdl_version() >= 1000
    assert lib.fdl_error_string(0) == b"success"
    assert b"invalid" in lib.fdl_error_string(-1)
    assert lib.fdl_sum_scratch_bytes(1 << 28) % 256 == 0
    assert lib.fdl_reduce_cols_scratch_bytes(1, 8192, 8192) % 256 == 0
    # an odd column count is reduced four rows at a time: room for the 4 * cols grouped results
    odd = lib.fdl_reduce_cols_scratch_bytes(1, 65537, 1001)
    assert odd % 256 == 0 and odd >= 65536 + 4 * 1001 * 4
    assert lib.fdl_reduce_cols_scratch_bytes(0, 10, 10) == 0


def test_product_does_not_import_the_oracle():
    """No file of the package may reach into oracle/ (no CPU fallback in the product)."""
    for path in (ROOT / "fast_dl_b200").rglob("*"):
        if path.suffix in {".py", ".cu", ".cuh", ".cpp", ".hpp", ".h"} and "build" not in path.parts[-3:-1]:
            text = path.read_text()
            if path.name == "build.py":
                continue  # compiles the checker, does not use it
            assert "oracle" not in text, f"{path} mentions the oracle"


def test_every_documented_tuning_key_is_accepted(fdl):
    """The keys named in the header's description of fdl_set_tuning, each with its documented
    default; an unknown key and an out-of-range value are refused.  No GPU involved."""
    import re
    header = (ROOT / "include" / "fdl_kernels.h").read_text()
    doc = header[header.index("Measurement aid: selects a launch shape"):header.index("int fdl_set_tuning")]
    keys = re.findall(r'"([a-z0-9_]+)"', doc)
    defaults = {"sum_cluster": 4, "sum_tiles": 0, "rows_split_fused": 1, "rows_split_lag": 0, "rows_split_hints": 1, "rows_split_from": 0, "rows_staged": -1, "rows_warp16": -1, "rows_cluster_threads": 256, "rows_span_cols": 256, "rows_span_reduce_cols": 2048, "rows_span_argmax_from": 65, "rows_smem": 1, "rows_smem_cluster": 0, "rows_smem_from": 0,
                "cols_tx": 64, "cols_cluster": 0, "cols_ctas_per_sm": 4, "cols_chunks": 0, "cols_single": 1, "cols_regroup": 1,
                "pdl": 1, "bcast2d": 1, "bcast2d_rows": 0, "exchange_wait_ms": 2000, "sum_trace": 0}
    assert sorted(keys) == sorted(defaults), keys
    lib = fdl.lib()
    for key, value in defaults.items():
        assert lib.fdl_set_tuning(key.encode(), value) == 0, key
    assert lib.fdl_set_tuning(b"no_such_key", 1) != 0
    assert lib.fdl_set_tuning(b"sum_cluster", 3) != 0
    assert lib.fdl_set_tuning(b"rows_cluster_threads", 128) != 0
    assert lib.fdl_set_tuning(b"exchange_wait_ms", 0) != 0


def test_library_exports_nothing_but_the_c_abi(fdl):
    """The dynamic symbol table of the library holds the fdl_* entry points and no C++ symbol
    of its internals (it is built with hidden visibility)."""
    import shutil
    import subprocess
    if shutil.which("nm") is None:
        pytest.skip("no nm")
    out = subprocess.run(["nm", "-D", "--defined-only", str(fdl.library_path())], check=True, capture_output=True,
                         text=True).stdout
    names = [line.split()[-1] for line in out.splitlines() if line.strip()]
    foreign = [n for n in names if not n.startswith("fdl_")]
    assert not foreign, f"exported besides the C ABI: {foreign[:10]}"
    assert sorted(n for n in names if n.startswith("fdl_")) == declared_symbols()


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 on its own, and a C caller must
    link against the library with nothing but the header (no C++ runtime symbols in the interface)."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    header = ROOT / "include" / "fdl_kernels.h"
    subprocess.run(["gcc", "-std=c99", "-pedantic", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", str(header)],
                   check=True)
    src = tmp_path / "caller.c"
    src.write_text('#include "fdl_kernels.h"\n#include <stdio.h>\n'
                   'int main(void) { printf("%d %s\\n", fdl_version(), fdl_error_string(FDL_ERR_WORKSPACE)); return 0; }\n')
    from fast_dl_b200 import build
    lib = build.build_kernels()
    exe = tmp_path / "caller"
    subprocess.run(["gcc", "-std=c99", "-I", str(ROOT / "include"), str(src), "-o", str(exe),
                    "-L", str(lib.parent), "-lfdl_kernels", f"-Wl,-rpath,{lib.parent}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split(maxsplit=1)
    assert int(out[0]) >= 1000 and "scratch" in out[1].lower()
