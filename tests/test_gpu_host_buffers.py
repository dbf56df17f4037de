"""GPU parity of the host-buffer entry points (pinned host tensors in, host results out)."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import assert_bit_exact, assert_sum_close

pytestmark = pytest.mark.gpu


def pinned(cuda, a):
    t = cuda.from_numpy(np.ascontiguousarray(a)).pin_memory()
    return t


@pytest.mark.parametrize("n", [1, 1000, (8 << 20) + 5, (20 << 20) + 1])
def test_host_binary_unary_chain(fdl, cuda, n):
    rng = np.random.default_rng(42)
    a, b, c = (rng.uniform(-1, 1, n).astype(np.float32) for _ in range(3))
    ha, hb, hc = pinned(cuda, a), pinned(cuda, b), pinned(cuda, c)
    out = cuda.empty(n, dtype=cuda.float32).pin_memory()
    fdl.host_binary(ha, hb, out, fdl.MUL)
    assert_bit_exact(out.numpy(), orc.binary(a, b, fdl.MUL), "host mul")
    fdl.host_unary(ha, out, fdl.RELU)
    assert_bit_exact(out.numpy(), orc.unary(a, fdl.RELU), "host relu")
    fdl.host_mul_add_relu(ha, hb, hc, out)
    assert_bit_exact(out.numpy(), orc.mul_add_relu(a, b, c), "host chain")
    s = fdl.host_sum(ha)
    assert_sum_close(s, orc.full_sum(a), max(orc.norm2(a), 1e-30), "host sum")


@pytest.mark.parametrize("rows,cols", [(1, 4), (100, 36), (3000, 4096), (700, 16384), (9001, 4096), (7, 1 << 20)])
def test_host_sweep_and_row_broadcast(fdl, cuda, rows, cols):
    rng = np.random.default_rng(43)
    x = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    y = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    row = rng.uniform(-1, 1, cols).astype(np.float32)
    hx, hy, hrow = pinned(cuda, x), pinned(cuda, y), pinned(cuda, row)
    hz = cuda.empty((rows, cols), dtype=cuda.float32).pin_memory()
    hw = cuda.empty((rows, cols), dtype=cuda.float32).pin_memory()
    for _ in range(2):  # staging buffers and scratch are reused across calls
        s = fdl.host_sweep(hx, hy, hrow, hz, hw)
        assert_bit_exact(hz.numpy(), x + y, "z = x + y")
        assert_bit_exact(hw.numpy(), x + row[None, :], "w = x + row")
        assert_sum_close(s, orc.full_sum(x), orc.norm2(x), "s = sum(x)")
    fdl.host_row_broadcast(hx, hrow, hw, fdl.MUL)
    assert_bit_exact(hw.numpy(), x * row[None, :], "host row broadcast mul")
