"""In-tree build of the native libraries (no JIT cache, no install step).

    python -m fast_dl_b200.build            # kernels + host library + oracle (+ reference if present)
    python -m fast_dl_b200.build kernels    # just libfdl_kernels.so

Everything is compiled for sm_100a only.  Outputs:

    fast_dl_b200/lib/libfdl_kernels.so   CUDA kernels behind the C ABI of include/fdl_kernels.h
    fast_dl_b200/lib/libdl_core.so       C++ host library with the fast_dl `dl::` API on top of it
    oracle/_build/libfdl_oracle.so       CPU restatement used by the tests (test infrastructure)
    oracle/_ref/...                      the reference's own code compiled in place (see oracle/build_ref.py)

A target is rebuilt when any of its sources or headers is newer than the output.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "fast_dl_b200"
CSRC = PKG / "csrc"
LIB = PKG / "lib"
HOST = PKG / "host"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# Hidden visibility: the header marks the extern "C" entry points default-visible when
# FDL_BUILDING_LIBRARY is defined, so the library exports the C ABI and nothing else.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "-DFDL_BUILDING_LIBRARY"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the kernel library cannot be built")
    return exe


def _newer(output: Path, inputs: list[Path]) -> bool:
    if not output.exists():
        return True
    t = output.stat().st_mtime
    return any(p.stat().st_mtime > t for p in inputs)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))


def kernels_lib_path() -> Path:
    return LIB / "libfdl_kernels.so"


def core_lib_path() -> Path:
    return LIB / "libdl_core.so"


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """nvcc every csrc/*.cu for sm_100a and link libfdl_kernels.so (static cudart)."""
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + [ROOT / "include" / "fdl_kernels.h"]
    out = kernels_lib_path()
    LIB.mkdir(parents=True, exist_ok=True)
    objdir = PKG / "build" / "kernels"
    objdir.mkdir(parents=True, exist_ok=True)
    objects = []
    for src in sources:
        obj = objdir / (src.stem + ".o")
        objects.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            _run(cmd)
    if force or _newer(out, objects):
        _run([_nvcc(), *ARCH_FLAGS, "-shared", "-o", str(out), *map(str, objects)])
    return out


def build_core(force: bool = False) -> Path | None:
    """g++ the C++ host library (the fast_dl `dl::` API) against libfdl_kernels.so."""
    if not HOST.exists():
        return None
    sources = sorted((HOST / "src").rglob("*.cpp"))
    headers = sorted((HOST / "include").rglob("*.hpp")) + [ROOT / "include" / "fdl_kernels.h"]
    out = core_lib_path()
    objdir = PKG / "build" / "core"
    objdir.mkdir(parents=True, exist_ok=True)
    cuda_home = Path(_nvcc()).resolve().parent.parent
    objects = []
    for src in sources:
        obj = objdir / ("_".join(src.relative_to(HOST / "src").with_suffix("").parts) + ".o")
        objects.append(obj)
        if force or _newer(obj, [src] + headers):
            _run(["g++", "-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra",
                  "-I", str(HOST / "include"), "-I", str(ROOT / "include"),
                  "-I", str(cuda_home / "include"), "-c", str(src), "-o", str(obj)])
    if force or _newer(out, objects + [kernels_lib_path()]):
        _run(["g++", "-shared", "-o", str(out), *map(str, objects),
              "-L", str(LIB), "-lfdl_kernels", "-Wl,-rpath,$ORIGIN",
              "-L", str(cuda_home / "lib64"), "-lcudart_static", "-lcublas", "-ldl", "-lrt", "-lpthread"])
    # The host library's own test programs (run on a GPU box by the test suite).
    for src in sorted((HOST / "tests").glob("*.cpp")):
        exe = LIB / src.stem
        if force or _newer(exe, [src, out] + headers):
            _run(["g++", "-O1", "-std=c++17", "-I", str(HOST / "include"), "-I", str(cuda_home / "include"),
                  str(src), "-o", str(exe), "-L", str(LIB), "-ldl_core", "-lfdl_kernels", "-Wl,-rpath,$ORIGIN"])
    return out


def build_oracle(force: bool = False) -> Path:
    sys.path.insert(0, str(ROOT))
    from oracle import build_oracle as bo  # test infrastructure, built here but never used by the product
    return bo.build(force=force)


def build_reference(force: bool = False):
    sys.path.insert(0, str(ROOT))
    from oracle import build_ref
    return build_ref.build(force=force)


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_core(force)
    build_oracle(force)
    build_reference(force)


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    force = "--force" in sys.argv
    if what == "kernels":
        print(build_kernels(force, verbose="-v" in sys.argv))
    elif what == "core":
        print(build_core(force))
    elif what == "oracle":
        print(build_oracle(force))
    elif what == "reference":
        print(build_reference(force))
    else:
        build_all(force)
        print("built")
