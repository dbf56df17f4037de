"""The five workload configurations at their FULL sizes, every element compared.

The reference's own large-size check is a bit-exact comparison of a 2^24-element vector_add
against a CPU loop (tests/benchmarks/vector_add/vector_add_benchmark.cu:51-56) and a
4096 x 1024 softmax against its CPU twin (tests/benchmarks/softmax/softmax_benchmark.cu:85-95).
These tests do the same at the sizes this library is measured on: 3 x 2^20 elements for the
fused chain, [4096,4096] broadcasts, [8192,8192] reductions, all 65,536 rows of the
[65536,1024] softmax / layernorm and all 2^28 elements of the large sweep (add, broadcast add
against a [1,16384] row, full sum).  The figures are produced by tests/parity_report.py (the
same functions print the table under profiles/); here every figure outside its allowance is
a test failure.

Against: the CPU oracle (scalar C, fp64 for sums/softmax/layernorm), the reference's CPU
check functions, and the reference's own CUDA kernels on the same device buffers when
oracle/_ref/libref.so was built.
"""
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("config", ["c1", "c2", "c3", "c4", "c5"])
def test_configuration_at_full_size(fdl, cuda, config):
    from oracle import ref
    from tests import parity_report as pr

    free, _ = cuda.cuda.mem_get_info()
    if config == "c5" and free < 6 * (1 << 30):
        pytest.skip("configuration 5 needs 6 GiB of free device memory")
    have_ref = ref.available()
    if have_ref:
        ref.gpu_set_device(0)
    del pr.ROWS[:], pr.FAILED[:]
    pr.CONFIGS[config](have_ref)
    cuda.cuda.synchronize()
    fdl.take_device_error()
    cuda.cuda.empty_cache()
    checked = [r for r in pr.ROWS if r[5] != pr.INFO]
    assert len(checked) >= 5, "the configuration produced too few checked figures"
    assert not pr.FAILED, f"outside allowance: {pr.FAILED}"
