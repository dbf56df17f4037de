"""GPU parity of the path's neighbours: cross-entropy, transpose, random fill."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import assert_bit_exact, to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,classes", [(1, 1), (3, 5), (64, 1000), (4096, 37), (257, 4096), (1000, 10), (33, 1 << 17),
                                           (513, 1028), (7, 30001), (65536, 1024)])
def test_cross_entropy(fdl, cuda, batch, classes):
    rng = np.random.default_rng(42)
    logits = rng.normal(0, 3, (batch, classes)).astype(np.float32)
    labels = rng.integers(0, classes, batch).astype(np.int64)
    if batch > 2:
        labels[1] = -1          # invalid labels are skipped, as in the reference kernel
        labels[2] = classes
    got = to_np(fdl.cross_entropy(cuda.from_numpy(logits).cuda(), cuda.from_numpy(labels).cuda()))[0]
    want = orc.cross_entropy(logits, labels)
    assert abs(got - want) <= 1e-5 * max(1.0, abs(want))   # the reference test allows 1e-4
    again = to_np(fdl.cross_entropy(cuda.from_numpy(logits).cuda(), cuda.from_numpy(labels).cuda()))[0]
    assert got == again  # deterministic: no float atomics


def test_cross_entropy_edge_values(fdl, cuda):
    """Very negative and very positive logits, a row with a single finite entry, logits off the
    16-byte grid (the 32-bit path), all labels invalid."""
    rng = np.random.default_rng(5)
    logits = rng.normal(0, 30, (64, 128)).astype(np.float32)
    logits[3, :] = -1e30
    logits[3, 17] = 2.5
    logits[4, :] = 80.0
    labels = rng.integers(0, 128, 64).astype(np.int64)
    labels[3] = 17
    want = orc.cross_entropy(logits, labels)
    d = cuda.from_numpy(logits).cuda()
    got = to_np(fdl.cross_entropy(d, cuda.from_numpy(labels).cuda()))[0]
    assert abs(got - want) <= 1e-5 * max(1.0, abs(want))
    padded = cuda.zeros(64 * 128 + 1, dtype=cuda.float32, device="cuda")
    padded[1:] = d.reshape(-1)
    shifted = padded[1:].view(64, 128)
    loss = cuda.empty(1, dtype=cuda.float32, device="cuda")
    fdl.check(fdl.lib().fdl_cross_entropy_f32(shifted.data_ptr(), cuda.from_numpy(labels).cuda().data_ptr(), loss.data_ptr(),
                                              64, 128, None), "fdl_cross_entropy_f32")
    assert abs(to_np(loss)[0] - want) <= 1e-5 * max(1.0, abs(want))
    none = cuda.full((64,), -1, dtype=cuda.int64, device="cuda")
    assert to_np(fdl.cross_entropy(d, none))[0] == 0.0


@pytest.mark.parametrize("n", [1, 4, 31, 32, 33, 60, 64, 68, 100, 1000, 1001, 1024, 4096, 4100, 8192])
def test_transpose_bit_exact(fdl, cuda, n):
    rng = np.random.default_rng(42)
    x = rng.normal(size=(n, n)).astype(np.float32)
    got = to_np(fdl.transpose(cuda.from_numpy(x).cuda()))
    assert_bit_exact(got, orc.transpose(x), f"transpose {n}")
    assert_bit_exact(got, x.T, "vs numpy")


def test_transpose_unaligned_pointers(fdl, cuda):
    """Input or output off the 16-byte grid: the 32-bit tile kernel."""
    n = 260
    rng = np.random.default_rng(3)
    x = rng.normal(size=(n, n)).astype(np.float32)
    buf = cuda.zeros(n * n + 1, dtype=cuda.float32, device="cuda")
    buf[1:] = cuda.from_numpy(x).cuda().reshape(-1)
    out = cuda.empty(n * n + 1, dtype=cuda.float32, device="cuda")
    fdl.check(fdl.lib().fdl_transpose_f32(buf[1:].data_ptr(), out[1:].data_ptr(), n, None), "fdl_transpose_f32")
    assert_bit_exact(to_np(out[1:]).reshape(n, n), x.T, "unaligned transpose")


def test_random_fill_properties(fdl, cuda):
    n = (1 << 20) + 3
    u1 = to_np(fdl.random_fill(n, False, -2.0, 3.0, 1234))
    u2 = to_np(fdl.random_fill(n, False, -2.0, 3.0, 1234))
    u3 = to_np(fdl.random_fill(n, False, -2.0, 3.0, 1235))
    assert np.array_equal(u1, u2) and not np.array_equal(u1, u3)     # what the reference's tests pin
    assert u1.min() > -2.0 and u1.max() <= 3.0
    assert abs(u1.mean() - 0.5) < 0.01 and abs(u1.std() - 5 / np.sqrt(12)) < 0.01
    # a prefix of a longer fill equals the shorter fill: values depend on (seed, index) only
    assert np.array_equal(to_np(fdl.random_fill(1000, False, -2.0, 3.0, 1234)), u1[:1000])
    g = to_np(fdl.random_fill(n, True, 1.0, 2.0, 99))
    assert np.isfinite(g).all() and abs(g.mean() - 1.0) < 0.01 and abs(g.std() - 2.0) < 0.01
    assert np.array_equal(g, to_np(fdl.random_fill(n, True, 1.0, 2.0, 99)))
