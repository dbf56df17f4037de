"""Programmatic launches keep stream order for data.

The streaming kernels are launched so that the next kernel of a stream may be scheduled while
the previous one drains; each waits for its predecessor before its first global access.  A
kernel that did not would read half-written inputs exactly in chains like the ones below,
where every op consumes what the op before it has just produced (or overwrites what it has
just read).  The chains run many times with programmatic launches and must give, bit for bit,
what plain launches give (tuning key "pdl" = 0).
"""
import numpy as np
import pytest

from tests.helpers import assert_bit_exact, to_np

pytestmark = pytest.mark.gpu


def _chain(fdl, cuda, a, b, c, row, labels):
    n = a.numel()
    cols = row.numel()
    y = fdl.binary(a, b, fdl.ADD)                       # y = a + b
    z = fdl.binary(y, c, fdl.MUL)                       # reads y at once
    fdl.unary(z, fdl.RELU, out=z)                       # in place
    w = fdl.broadcast_binary(z.view(-1, cols), row.view(1, cols), fdl.ADD)
    fdl.add_row_bias_(w, row)                           # in place on the result
    s = fdl.full_sum(w.view(-1))                        # reads w
    sm = fdl.softmax_rows(w)
    ln = fdl.layernorm_rows(sm)                         # reads the softmax's output
    rs = fdl.reduce_rows(ln, fdl.REDUCE_SUM)
    cm = fdl.reduce_cols(ln, fdl.REDUCE_MEAN)
    am = fdl.argmax_rows(sm)
    ce = fdl.cross_entropy(w, labels)
    m = min(w.shape[0], cols) // 4 * 4
    t = fdl.transpose(w[:m, :m].contiguous())
    fdl.binary(a, b, fdl.SUB, out=y)                    # overwrites what z was computed from
    fdl.mul_add_relu(y, z, c, out=y)
    u = fdl.random_fill(n, False, -1.0, 1.0, 7)
    fdl.binary(u, y, fdl.ADD, out=u)                    # the fill's buffer is consumed right away
    return [to_np(v) for v in (y, z, w, s, sm, ln, rs, cm, ce, t, u)] + [to_np(am).astype(np.float32)]


@pytest.mark.parametrize("rows,cols", [(4096, 1024), (1537, 2048)])
def test_chains_give_the_same_bits_with_and_without_programmatic_launches(fdl, cuda, rows, cols):
    rng = np.random.default_rng(9)
    n = rows * cols
    a, b, c = (cuda.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)).cuda() for _ in range(3))
    row = cuda.from_numpy(rng.uniform(-1, 1, cols).astype(np.float32)).cuda()
    labels = cuda.from_numpy(rng.integers(0, cols, rows).astype(np.int64)).cuda()
    fdl.set_tuning("pdl", 0)
    try:
        want = _chain(fdl, cuda, a, b, c, row, labels)
    finally:
        fdl.set_tuning("pdl", 1)
    for _ in range(10):
        got = _chain(fdl, cuda, a, b, c, row, labels)
        for k, (g, w) in enumerate(zip(got, want)):
            assert_bit_exact(g, w, f"result {k} of the chain")
    fdl.take_device_error()
