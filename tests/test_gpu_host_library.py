"""The C++ host library on a GPU: the reference's own 17 test programs, compiled unmodified,
in two builds (oracle/build_ref.py), and the host library's own test programs for the API
additions (fast_dl_b200/host/tests).

Build 1: against this repository's `dl::` headers and libdl_core.so.
Build 2: against the REFERENCE's own headers and its own, unmodified src/core, src/tensor,
src/ops and src/nn (oracle/_ref/libdl_core_reference.so), with this repository's forwarding
source + libfdl_kernels.so where the reference links dl_cuda_kernels (CMakeLists.txt:75):
the replacement kernel library behind the existing host code."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF_TESTS = ROOT / "oracle" / "_ref" / "tests"
REFCORE_TESTS = ROOT / "oracle" / "_ref" / "tests_refcore"
pytestmark = pytest.mark.gpu

REFERENCE_PROGRAMS = [
    "test_tensor", "tensor_copy_test", "tensor_uniform_test", "tensor_randn_test", "elementwise_tensor_test",
    "activation_tensor_test", "softmax_tensor_test", "layernorm_tensor_test", "matmul_tensor_test",
    "linear_tensor_test", "cross_entropy_tensor_test", "relu_module_test", "linear_module_test",
    "sequential_module_test", "custom_module_test", "linear_init_test", "linear_kaiming_init_test",
]


def run(exe):
    return subprocess.run([str(exe)], capture_output=True, text=True, timeout=120, cwd=str(ROOT))


@pytest.mark.parametrize("name", REFERENCE_PROGRAMS)
def test_reference_program_passes_against_this_library(cuda, name):
    exe = REF_TESTS / name
    if not exe.exists():
        pytest.skip("oracle/_ref/tests was not built (needs the reference tree at build time)")
    proc = run(exe)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "not passed" not in proc.stdout and "passed" in proc.stdout, proc.stdout


@pytest.mark.parametrize("name", REFERENCE_PROGRAMS)
def test_reference_program_passes_on_the_reference_host_code_over_this_kernel_library(cuda, name):
    exe = REFCORE_TESTS / name
    if not exe.exists():
        pytest.skip("oracle/_ref/tests_refcore was not built (needs the reference tree at build time)")
    proc = run(exe)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "not passed" not in proc.stdout and "passed" in proc.stdout, proc.stdout


@pytest.mark.parametrize("program", ["host_ops_test", "sharded_test"])
def test_host_library_additions(cuda, program):
    exe = ROOT / "fast_dl_b200" / "lib" / program
    assert exe.exists(), "run python -m fast_dl_b200.build core"
    proc = run(exe)
    assert proc.returncode == 0 and "not passed" not in proc.stdout, proc.stdout + proc.stderr
