"""Seeded random sequences of ops and shapes through the C ABI, each checked against the
oracle.  The kernels keep state between calls (workspace, arrival counters, per-kernel
attributes), so the ORDER of calls is part of what is tested."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import assert_bit_exact, assert_close_scaled, assert_sum_close, to_np

pytestmark = pytest.mark.gpu


def dev(cuda, a):
    return cuda.from_numpy(np.ascontiguousarray(a)).cuda()


def random_matrix_shape(rng):
    kind = rng.integers(0, 6)
    if kind == 4:   # a few very long rows: the segmented reductions, the cluster and two-kernel row forms
        return int(rng.integers(1, 7)), int(rng.choice([20000, 40004, 100000, 131072, 200001, 262148, 400000]))
    if kind == 5:   # a handful of rows, or very short ones
        return (int(rng.integers(1, 9)), int(rng.integers(1, 300000))) if rng.integers(0, 2) else \
               (int(rng.integers(1, 200000)), int(rng.choice([1, 2, 4, 8, 12, 16, 32, 33, 64, 100, 128, 256])))
    if kind == 0:
        return int(rng.integers(1, 64)), int(rng.integers(1, 70000))
    if kind == 1:
        return int(rng.integers(1, 5000)), int(rng.integers(1, 600))
    if kind == 2:
        return int(rng.integers(1, 300)) , int(rng.choice([4, 64, 128, 256, 1024, 2048, 4096, 8192, 16384, 16388]))
    return int(rng.integers(1, 40)), int(rng.integers(1, 40))


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_random_op_sequence(fdl, cuda, seed):
    rng = np.random.default_rng(seed)
    for step in range(40):
        op = int(rng.integers(0, 8))
        rows, cols = random_matrix_shape(rng)
        if rows * cols > 3_000_000:
            rows = max(1, 3_000_000 // cols)
        x = rng.normal(0, 2, (rows, cols)).astype(np.float32)
        # a third of the steps run on a view that starts 1..3 floats off the 16-byte grid
        off = int(rng.integers(1, 4)) if rng.integers(0, 3) == 0 else 0
        if off:
            buf = cuda.zeros(rows * cols + 4, dtype=cuda.float32, device="cuda")
            buf[off:off + rows * cols] = dev(cuda, x).reshape(-1)
            xd = buf[off:off + rows * cols].view(rows, cols)
        else:
            xd = dev(cuda, x)

        def like_x():   # an output at the same phase as the input view
            o = cuda.full((rows * cols + 4,), np.float32(-7.0), dtype=cuda.float32, device="cuda")
            return o, o[off:off + rows * cols].view(rows, cols)

        what = f"seed {seed} step {step} op {op} shape {rows}x{cols} off {off}"
        x64 = x.astype(np.float64)
        if op == 0:
            y = rng.uniform(0.5, 2, (rows, cols)).astype(np.float32)
            k = int(rng.integers(0, 4))
            assert_bit_exact(to_np(fdl.binary(xd, dev(cuda, y), k)), orc.binary(x, y, k).reshape(rows, cols), what)
        elif op == 1:
            other = [(1, cols), (rows, 1), (cols,), (1, 1)][int(rng.integers(0, 4))]
            y = rng.uniform(0.5, 2, other).astype(np.float32)
            k = int(rng.integers(0, 4))
            assert_bit_exact(to_np(fdl.broadcast_binary(xd, dev(cuda, y), k)), orc.broadcast_binary(x, y, k), what)
        elif op == 2:
            norm = np.sqrt((x64 ** 2).sum(axis=1))
            assert_sum_close(to_np(fdl.reduce_rows(xd, fdl.REDUCE_SUM)), x64.sum(axis=1), norm, what)
            assert_bit_exact(to_np(fdl.reduce_rows(xd, fdl.REDUCE_MAX)), x.max(axis=1), what)
            np.testing.assert_array_equal(to_np(fdl.argmax_rows(xd)), x.argmax(axis=1), what)
        elif op == 3:
            norm = np.sqrt((x64 ** 2).sum(axis=0))
            assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), x64.sum(axis=0), norm, what)
            assert_bit_exact(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MAX)), x.max(axis=0), what)
        elif op == 4:
            assert_sum_close(to_np(fdl.full_sum(xd.reshape(-1)))[0], x64.sum(), np.sqrt((x64 ** 2).sum()), what)
        elif op == 5:
            whole, view = like_x()
            fdl.softmax_rows(xd, out=view)
            assert_close_scaled(to_np(view), orc.softmax_rows_f64(x), what)
            edge = to_np(whole)
            assert (edge[:off] == -7.0).all() and (edge[off + rows * cols:] == -7.0).all(), what
        elif op == 6:
            g = rng.uniform(0.9, 1.1, cols).astype(np.float32)
            b = rng.uniform(-0.1, 0.1, cols).astype(np.float32)
            whole, view = like_x()
            fdl.layernorm_rows(xd, dev(cuda, g), dev(cuda, b), out=view)
            assert_close_scaled(to_np(view), orc.layernorm_rows_f64(x, g, b), what)
            edge = to_np(whole)
            assert (edge[:off] == -7.0).all() and (edge[off + rows * cols:] == -7.0).all(), what
        else:
            k = int(rng.integers(0, 5))
            got, want = to_np(fdl.unary(xd, k, 0.02)), orc.unary(x, k, 0.02).reshape(rows, cols)
            if k < 2:
                assert_bit_exact(got, want, what)
            else:
                assert np.abs(got - want).max() < 1e-5, what
    cuda.cuda.synchronize()
    fdl.take_device_error()
