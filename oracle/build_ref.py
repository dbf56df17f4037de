"""Compiles the reference's own code for the hot path, in place, into oracle/_ref/.

    python -m oracle.build_ref

Nothing from the reference is copied into this repository: the reference's sources are
compiled where they lie (environment variable REFERENCE_ROOT; by default the directory
`reference` beside this repository) and only build outputs
land in oracle/_ref/, which is git-ignored but travels with the working tree to a GPU
box.  The reference's CMake build is NOT run; these are direct gcc/nvcc invocations on the
few files the path needs.  When the reference tree is absent this is a no-op and the
previously built files (if any) are used as they are.

Outputs
  oracle/_ref/libref.so       - the reference's CUDA kernels for the path (elementwise,
                                activation, vector_add, bias, reduction, softmax, layernorm) and
                                its neighbours (cross_entropy, transpose, random),
                                recompiled for sm_100a, plus the CPU check functions that live
                                in its tests/benchmarks, all behind the C shims of
                                oracle/ref_shims/*.cpp.  CPU flags: g++ -O2 -ffp-contract=off
                                (the reference sets no build type; contraction is turned off so
                                that its a*b+c style expressions round like its GPU chain of
                                separate kernels).
  oracle/_ref/tests/<name>    - the reference's own test programs (tests/tensor, tests/nn)
                                compiled UNMODIFIED against this repository's dl:: headers and
                                linked with libdl_core.so / libfdl_kernels.so.
  oracle/_ref/libdl_core_reference.so
                              - the reference's link line (CMakeLists.txt:24-56, 75) with the
                                kernel library swapped: its UNMODIFIED src/core, src/tensor,
                                src/ops and src/nn sources compiled against its own include/,
                                plus this repository's forwarding source
                                (fast_dl_b200/host/src/kernels_shim.cpp and gemm.cpp, compiled
                                against the reference's include/dl/kernels/*.hpp) in place of
                                dl_cuda_kernels, linked with libfdl_kernels.so.
  oracle/_ref/tests_refcore/<name>
                              - the same 17 test programs compiled against the reference's
                                headers and linked with that library: the replacement kernel
                                library behind the reference's own host code.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
REF = Path(os.environ.get("REFERENCE_ROOT", str(ROOT.parent / "reference")))
OUT = HERE / "_ref"
SHIMS = HERE / "ref_shims"

REF_KERNELS = ["elementwise", "activation", "vector_add", "bias", "reduction", "softmax", "layernorm",
               "cross_entropy", "transpose", "random"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CPU_FLAGS = ["-O2", "-ffp-contract=off", "-std=c++17", "-fPIC"]


def _run(cmd):
    proc = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), proc.stdout, proc.stderr))


def reference_available() -> bool:
    return (REF / "src" / "kernels" / "cuda" / "softmax.cu").exists()


def lib_path() -> Path:
    return OUT / "libref.so"


def build_lib(force: bool = False) -> Path | None:
    if not reference_available():
        return lib_path() if lib_path().exists() else None
    out = lib_path()
    if out.exists() and not force:
        newest = max(p.stat().st_mtime for p in SHIMS.glob("*.cpp"))
        if out.stat().st_mtime > newest:
            return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cuda_inc = Path(nvcc).resolve().parent.parent / "include"
    objdir = OUT / "obj"
    objdir.mkdir(parents=True, exist_ok=True)
    objects = []
    # The reference's kernels: nvcc defaults (as its CMake sets none), retargeted to sm_100a.
    for name in REF_KERNELS:
        obj = objdir / f"ref_{name}.o"
        _run([nvcc, *ARCH, "-std=c++17", "-Xcompiler", "-fPIC", "-I", REF / "include",
              "-c", REF / "src" / "kernels" / "cuda" / f"{name}.cu", "-o", obj])
        objects.append(obj)
    # Host-only shims that include the reference's test/benchmark files in place.
    for shim in sorted(SHIMS.glob("*.cpp")):
        obj = objdir / f"shim_{shim.stem}.o"
        _run(["g++", *CPU_FLAGS, "-x", "c++", "-I", REF, "-I", REF / "include", "-I", cuda_inc,
              "-c", shim, "-o", obj])
        objects.append(obj)
    _run([nvcc, *ARCH, "-shared", "-o", out, *objects, "-lpthread"])
    return out


REF_TESTS = [
    "tensor/test_tensor", "tensor/tensor_copy_test", "tensor/tensor_uniform_test",
    "tensor/tensor_randn_test", "tensor/elementwise_tensor_test", "tensor/activation_tensor_test",
    "tensor/softmax_tensor_test", "tensor/layernorm_tensor_test", "tensor/matmul_tensor_test",
    "tensor/linear_tensor_test", "tensor/cross_entropy_tensor_test",
    "nn/relu_module_test", "nn/linear_module_test", "nn/sequential_module_test",
    "nn/custom_module_test", "nn/linear_init_test", "nn/linear_kaiming_init_test",
]


def build_tests(force: bool = False) -> list[Path]:
    """The reference's 17 test programs against this repository's headers and libraries."""
    host_inc = ROOT / "fast_dl_b200" / "host" / "include"
    libdir = ROOT / "fast_dl_b200" / "lib"
    core = libdir / "libdl_core.so"
    outdir = OUT / "tests"
    if not reference_available() or not core.exists():
        return sorted(outdir.glob("*")) if outdir.exists() else []
    outdir.mkdir(parents=True, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cuda_home = Path(nvcc).resolve().parent.parent
    built = []
    for rel in REF_TESTS:
        src = REF / "tests" / (rel + ".cpp")
        exe = outdir / Path(rel).name
        if force or not exe.exists() or exe.stat().st_mtime < core.stat().st_mtime:
            _run(["g++", "-O1", "-std=c++17", "-I", host_inc, "-I", cuda_home / "include", src, "-o", exe,
                  "-L", libdir, "-ldl_core", "-lfdl_kernels",
                  "-Wl,-rpath,$ORIGIN/../../../fast_dl_b200/lib"])
        built.append(exe)
    return built


REF_CORE_DIRS = ["core", "tensor", "ops", "nn"]


def refcore_lib_path() -> Path:
    return OUT / "libdl_core_reference.so"


def build_refcore(force: bool = False) -> list[Path]:
    """The reference's own dl_core on top of libfdl_kernels.so, and its 17 tests against it."""
    libdir = ROOT / "fast_dl_b200" / "lib"
    kernels = libdir / "libfdl_kernels.so"
    outdir = OUT / "tests_refcore"
    if not reference_available() or not kernels.exists():
        return sorted(outdir.glob("*")) if outdir.exists() else []
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cuda_home = Path(nvcc).resolve().parent.parent
    objdir = OUT / "obj_refcore"
    objdir.mkdir(parents=True, exist_ok=True)
    outdir.mkdir(parents=True, exist_ok=True)
    host_src = ROOT / "fast_dl_b200" / "host" / "src"
    # The include directories of the reference's dl_core target (CMakeLists.txt:59-67).
    ref_inc = [REF / "include", REF / "include" / "dl"] + [REF / "include" / "dl" / d for d in
                                                        ("core", "kernels", "ops", "tensor")]
    inc = [a for d in ref_inc for a in ("-I", d)] + ["-I", cuda_home / "include"]
    sources = [p for d in REF_CORE_DIRS for p in sorted((REF / "src" / d).glob("*.cpp"))]
    forwards = [host_src / "kernels_shim.cpp", host_src / "gemm.cpp"]
    lib = refcore_lib_path()
    stamp = max(p.stat().st_mtime for p in forwards + [kernels])
    if force or not lib.exists() or lib.stat().st_mtime < stamp:
        objects = []
        for src in sources:
            obj = objdir / f"ref_{src.parent.name}_{src.stem}.o"
            _run(["g++", "-O2", "-std=c++17", "-fPIC", *inc, "-c", src, "-o", obj])
            objects.append(obj)
        for src in forwards:  # against the REFERENCE's kernel headers, plus the C ABI header
            obj = objdir / f"fwd_{src.stem}.o"
            _run(["g++", "-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra", *inc, "-I", ROOT / "include",
                  "-c", src, "-o", obj])
            objects.append(obj)
        _run(["g++", "-shared", "-o", lib, *objects, "-L", libdir, "-lfdl_kernels",
              "-Wl,-rpath,$ORIGIN/../../fast_dl_b200/lib", "-L", cuda_home / "lib64", "-lcudart", "-lcublas"])
    built = []
    for rel in REF_TESTS:
        src = REF / "tests" / (rel + ".cpp")
        exe = outdir / Path(rel).name
        if force or not exe.exists() or exe.stat().st_mtime < lib.stat().st_mtime:
            _run(["g++", "-O1", "-std=c++17", *inc, src, "-o", exe, "-L", OUT, "-ldl_core_reference",
                  "-L", libdir, "-lfdl_kernels", "-L", cuda_home / "lib64", "-lcudart",
                  "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath,$ORIGIN/../../../fast_dl_b200/lib"])
        built.append(exe)
    return built


def build(force: bool = False):
    return build_lib(force), build_tests(force), build_refcore(force)


if __name__ == "__main__":
    lib, tests, refcore_tests = build(force=True)
    print(lib)
    print(len(tests), "reference test programs against this repository's host library")
    print(len(refcore_tests), "reference test programs against the reference's own host library + libfdl_kernels.so")
