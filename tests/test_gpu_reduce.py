"""GPU parity: reductions through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle import ref
from tests.helpers import assert_bit_exact, assert_sum_close, to_np

pytestmark = pytest.mark.gpu


def dev(cuda, a):
    return cuda.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("tree", [0, 1])
@pytest.mark.parametrize("nblocks", [1, 7, 8, 9, 1000, 16384])
def test_block_reduce_matches_reference_tree_bit_for_bit(fdl, cuda, tree, nblocks):
    rng = np.random.default_rng(42)
    x = rng.uniform(-1, 1, nblocks * 1024 + 17).astype(np.float32)  # the 17-element tail is ignored
    got = to_np(fdl.block_reduce_1024(dev(cuda, x), tree))
    assert_bit_exact(got, orc.block_reduce_1024(x, tree), f"tree {tree}")
    # unaligned input takes the scalar-load path; same bits
    xd = dev(cuda, np.concatenate([[0.0], x]).astype(np.float32))[1:]
    assert_bit_exact(to_np(fdl.block_reduce_1024(xd, tree)), orc.block_reduce_1024(x, tree), "unaligned")


def test_block_reduce_golden_and_reference_kernels(fdl, cuda, golden):
    x = golden["seeded_reduce_input"]
    assert_bit_exact(to_np(fdl.block_reduce_1024(dev(cuda, x), 0)), golden["seeded_reduce_interleave"], "golden i")
    assert_bit_exact(to_np(fdl.block_reduce_1024(dev(cuda, x), 1)), golden["seeded_reduce_address"], "golden a")
    if ref.available():
        rng = np.random.default_rng(1)
        big = dev(cuda, rng.uniform(-1, 1, 1 << 22).astype(np.float32))
        for tree in (0, 1):
            want = cuda.empty(big.numel() // 1024, dtype=cuda.float32, device="cuda")
            cuda.cuda.synchronize()
            ref.gpu_reduction(big.data_ptr(), want.data_ptr(), big.numel(), tree)
            ref.gpu_sync()
            assert_bit_exact(to_np(fdl.block_reduce_1024(big, tree)), to_np(want), f"reference kernel tree {tree}")


@pytest.mark.parametrize("n", [0, 1, 3, 1023, 1025, 65536, 65537, (1 << 22) + 3, 1 << 26])
def test_full_sum(fdl, cuda, n):
    rng = np.random.default_rng(42)
    x = rng.uniform(-1, 1, n).astype(np.float32)
    out32, out64 = fdl.full_sum(dev(cuda, x), want_f64=True)
    want = orc.full_sum(x)
    norm = max(orc.norm2(x), 1e-30)
    assert_sum_close(to_np(out32)[0], want, norm, f"sum n={n}")
    assert_sum_close(to_np(out64)[0], want, norm, f"sum64 n={n}")
    assert np.float32(to_np(out64)[0]) == to_np(out32)[0]


def test_full_sum_is_deterministic_and_scratch_is_reusable(fdl, cuda):
    rng = np.random.default_rng(2)
    x = dev(cuda, rng.normal(size=(1 << 24) + 11).astype(np.float32))
    first = to_np(fdl.full_sum(x))
    for _ in range(5):
        assert_bit_exact(to_np(fdl.full_sum(x)), first, "repeat")
    nbytes = fdl.lib().fdl_sum_scratch_bytes(x.numel())
    scratch = cuda.zeros(nbytes, dtype=cuda.uint8, device="cuda")
    for _ in range(3):
        assert_bit_exact(to_np(fdl.full_sum(x, scratch=scratch)), first, "caller scratch")
    with pytest.raises(fdl.FdlError):
        fdl.full_sum(x, scratch=scratch[:64])
    unaligned = dev(cuda, np.concatenate([[0.0], to_np(x)]).astype(np.float32))[1:]
    assert_sum_close(to_np(fdl.full_sum(unaligned))[0], orc.full_sum(to_np(x)), orc.norm2(to_np(x)), "unaligned")


SHAPES = [(1, 1), (1, 7), (5, 3), (17, 128), (33, 1000), (64, 2048), (9, 2052), (300, 4096), (3, 100003),
          (2048, 33), (1024, 1024)]
# short rows (teams of 1..32 lanes, several rows in flight) and a few very long rows (cut into segments)
ROW_SHAPES = SHAPES + [(100000, 4), (70001, 8), (50000, 12), (33333, 32), (20000, 36), (9999, 64), (5000, 128),
                       (4097, 200), (3000, 256), (3001, 260), (1000, 2), (777, 37), (500, 64), (501, 65),
                       (3, 1 << 20), (5, (1 << 20) + 4), (2, (1 << 21) + 3), (64, 1 << 17), (1, 70000), (1183, 65536)]


@pytest.mark.parametrize("rows,cols", ROW_SHAPES)
def test_row_reductions(fdl, cuda, rows, cols):
    rng = np.random.default_rng(42)
    x = rng.normal(size=(rows, cols)).astype(np.float32)
    xd = dev(cuda, x)
    norm = np.sqrt((x.astype(np.float64) ** 2).sum(axis=1))
    assert_sum_close(to_np(fdl.reduce_rows(xd, fdl.REDUCE_SUM)), orc.reduce_rows(x, 0), norm, "row sum")
    assert_sum_close(to_np(fdl.reduce_rows(xd, fdl.REDUCE_MEAN)), orc.reduce_rows(x, 1), norm / cols, "row mean")
    assert_bit_exact(to_np(fdl.reduce_rows(xd, fdl.REDUCE_MAX)), orc.reduce_rows(x, 2), "row max")
    np.testing.assert_array_equal(to_np(fdl.argmax_rows(xd)), orc.argmax_rows(x))
    if cols > 1:   # unaligned base: the 32-bit paths of the same kernels
        flat = dev(cuda, np.concatenate([np.zeros(1, np.float32), x.reshape(-1)]))
        xu = flat[1:].view(rows, cols)
        assert_sum_close(to_np(fdl.reduce_rows(xu, fdl.REDUCE_SUM)), orc.reduce_rows(x, 0), norm, "row sum, unaligned")
        np.testing.assert_array_equal(to_np(fdl.argmax_rows(xu)), orc.argmax_rows(x))
    ties = rng.integers(0, 3, size=(rows, cols)).astype(np.float32)
    np.testing.assert_array_equal(to_np(fdl.argmax_rows(dev(cuda, ties))), orc.argmax_rows(ties))
    fdl.full_sum(xd.reshape(-1))   # shares the workspace counters with the segmented row kernel
    assert_bit_exact(to_np(fdl.reduce_rows(xd, fdl.REDUCE_MAX)), orc.reduce_rows(x, 2), "row max again")


def test_argmax_ties_nan_inf(fdl, cuda):
    rng = np.random.default_rng(8)
    x = rng.integers(0, 4, size=(512, 4096)).astype(np.float32)  # many ties
    x[3, :] = -np.inf
    x[4, :] = np.nan
    x[5, 100] = np.inf
    x[5, 50] = np.nan
    x[6, ::2] = np.nan
    got = to_np(fdl.argmax_rows(dev(cuda, x)))
    np.testing.assert_array_equal(got, orc.argmax_rows(x))
    assert got.dtype == np.int64 and got[3] == 0 and got[4] == 0 and got[5] == 100
    for shape in ((3000, 8), (2000, 32), (1000, 128), (4, 1 << 18)):      # the short-row and segmented kernels
        y = rng.integers(0, 4, size=shape).astype(np.float32)
        y[1, :] = np.nan
        y[2, :] = -np.inf
        y[3, ::3] = np.nan
        y[0, shape[1] - 1] = np.inf
        got = to_np(fdl.argmax_rows(dev(cuda, y)))
        np.testing.assert_array_equal(got, orc.argmax_rows(y))
        assert got[1] == 0 and got[2] == 0 and got[0] == shape[1] - 1
        assert_bit_exact(to_np(fdl.reduce_rows(dev(cuda, y), fdl.REDUCE_MAX)), orc.reduce_rows(y, 2), f"max {shape}")
    for shape in ((3000, 7), (2000, 63), (1000, 129), (700, 255), (300, 1001), (40, 2047), (9, 8191)):  # odd lengths
        y = rng.integers(0, 4, size=shape).astype(np.float32)
        y[1, :] = np.nan
        y[2, :] = -np.inf
        y[3, ::3] = np.nan
        y[0, shape[1] - 1] = np.inf
        y[4, :] = -3.0
        y[4, 2], y[4, shape[1] - 2] = -0.0, 0.0     # equal as floats: the lower column wins
        y[5, :] = -np.inf
        y[5, shape[1] - 1] = -1e30
        y[6, :] = np.nan
        y[6, 5] = -np.inf                           # NaN ranks as -inf: column 0
        for tune in (65, 1):                        # short rows: the team kernels, then the span form
            fdl.set_tuning("rows_span_argmax_from", tune)
            try:
                got = to_np(fdl.argmax_rows(dev(cuda, y)))
            finally:
                fdl.set_tuning("rows_span_argmax_from", 65)
            np.testing.assert_array_equal(got, orc.argmax_rows(y))
            assert got[1] == 0 and got[2] == 0 and got[0] == shape[1] - 1 and got[4] == 2
            assert got[5] == shape[1] - 1 and got[6] == 0
        y[4, 2] = 0.0   # (the sign of a zero maximum is whatever fmaxf makes of the order of evaluation)
        assert_bit_exact(to_np(fdl.reduce_rows(dev(cuda, y), fdl.REDUCE_MAX)), orc.reduce_rows(y, 2), f"max {shape}")
    small = rng.integers(0, 3, size=(1000, 37)).astype(np.float32)
    np.testing.assert_array_equal(to_np(fdl.argmax_rows(dev(cuda, small))), orc.argmax_rows(small))
    assert_bit_exact(to_np(fdl.reduce_rows(dev(cuda, x), fdl.REDUCE_MAX)), orc.reduce_rows(x, 2), "max with nan")


@pytest.mark.parametrize("rows,cols", SHAPES + [(8192, 256), (100000, 4), (3, 5000000), (2, 4500001), (200000, 32),
                                                (1, 1000), (8, 4096), (7, 130001), (9, 4096), (400000, 8), (150000, 36)])
def test_column_reductions(fdl, cuda, rows, cols):
    rng = np.random.default_rng(42)
    x = rng.normal(size=(rows, cols)).astype(np.float32)
    xd = dev(cuda, x)
    norm = np.sqrt((x.astype(np.float64) ** 2).sum(axis=0))
    assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), orc.reduce_cols(x, 0), norm, "col sum")
    assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MEAN)), orc.reduce_cols(x, 1), norm / rows, "col mean")
    assert_bit_exact(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MAX)), orc.reduce_cols(x, 2), "col max")
    again = to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM))
    assert_bit_exact(again, to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), "deterministic")


def test_column_reductions_of_changing_shapes_share_the_workspace(fdl, cuda):
    """Back-to-back calls whose scratch layouts differ (more column blocks, fewer groups, and the
    full sum in between) must not see each other's leftovers in the arrival counters."""
    rng = np.random.default_rng(5)
    for rows, cols in [(5000, 32768), (1000, 65536), (300, 256), (1000, 65536), (100, 65536), (2000, 16384)]:
        x = rng.normal(size=(rows, cols)).astype(np.float32)
        xd = dev(cuda, x)
        norm = np.sqrt((x.astype(np.float64) ** 2).sum(axis=0)) / rows
        for _ in range(2):
            assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MEAN)), orc.reduce_cols(x, 1), norm, f"{rows}x{cols}")
            fdl.full_sum(xd)
        assert_bit_exact(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MAX)), orc.reduce_cols(x, 2), "col max")


def test_column_reduction_batched_and_caller_scratch(fdl, cuda):
    rng = np.random.default_rng(3)
    x = rng.normal(size=(5, 700, 96)).astype(np.float32)
    xd = dev(cuda, x)
    got = to_np(fdl.reduce_cols(xd, fdl.REDUCE_MEAN))
    norm = np.sqrt((x.astype(np.float64) ** 2).sum(axis=1)) / 700
    assert_sum_close(got, orc.reduce_cols(x, 1), norm, "batched mean")
    nbytes = fdl.lib().fdl_reduce_cols_scratch_bytes(5, 700, 96)
    scratch = cuda.zeros(max(nbytes, 256), dtype=cuda.uint8, device="cuda")
    for _ in range(2):
        assert_bit_exact(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MEAN, scratch=scratch)), got, "caller scratch")


def test_column_reduction_batched_few_rows_and_many_chunks(fdl, cuda):
    """Batched matrices of a handful of rows (the no-tree kernel) and a tall narrow one whose
    row chunks are folded by all thread rows of the last CTA."""
    rng = np.random.default_rng(4)
    for shape in ((6, 5, 1000), (3, 8, 4100), (4, 2, 37), (2, 300000, 16), (3, 100000, 40)):
        x = rng.normal(size=shape).astype(np.float32)
        xd = dev(cuda, x)
        norm = np.sqrt((x.astype(np.float64) ** 2).sum(axis=1))
        assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), orc.reduce_cols(x, 0), norm, f"sum {shape}")
        assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MEAN)), orc.reduce_cols(x, 1), norm / shape[1], f"mean {shape}")
        assert_bit_exact(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MAX)), orc.reduce_cols(x, 2), f"max {shape}")
        assert_bit_exact(to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), "same bits")


@pytest.mark.parametrize("rows,cols", [(16384, 4), (20000, 8), (1 << 17, 16), (300001, 32), (65536 + 7, 64), (40000, 128),
                                       (1 << 21, 32),
                                       # column counts that are not a multiple of 4: taken 4 (or 2) rows at a time
                                       # with 128-bit loads, rows left over, results folded by a second kernel
                                       (300001, 33), (65537, 1001), (70002, 6), (1001, 255), (40, 50257), (9, 7), (13, 2)])
def test_column_reduction_of_tall_narrow_matrices(fdl, cuda, rows, cols):
    """Rows of 4 ... 128 floats: a single column block, hundreds of row chunks, the last CTA
    folding them; and odd column counts; with the library's and with the caller's scratch, twice
    in a row (the arrival counters must come back to zero), and the full sum on the same
    workspace afterwards."""
    rng = np.random.default_rng(rows + cols)
    x = rng.normal(size=(rows, cols)).astype(np.float32)
    x[rows // 2, cols - 1] = 1e6   # a lone large value must land in its own column
    xd = dev(cuda, x)
    x64 = x.astype(np.float64)
    norm = np.sqrt((x64 ** 2).sum(axis=0))
    nbytes = fdl.lib().fdl_reduce_cols_scratch_bytes(1, rows, cols)
    scratch = cuda.zeros(max(nbytes, 256), dtype=cuda.uint8, device="cuda")
    for use in (None, scratch, None):
        assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM, scratch=use)), x64.sum(axis=0), norm, "col sum")
        assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MEAN, scratch=use)), x64.mean(axis=0), norm / rows, "col mean")
        assert_bit_exact(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MAX, scratch=use)), x.max(axis=0), "col max")
    assert_bit_exact(to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), "deterministic")
    assert_sum_close(to_np(fdl.full_sum(xd))[0], x64.sum(), np.sqrt((x64 ** 2).sum()), "full sum afterwards")
    if cols % 4:
        fdl.set_tuning("cols_regroup", 0)
        try:
            assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), x64.sum(axis=0), norm, "col sum, 32-bit loads")
            assert_bit_exact(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MAX)), x.max(axis=0), "col max, 32-bit loads")
        finally:
            fdl.set_tuning("cols_regroup", 1)


@pytest.mark.parametrize("rows,cols", [(8192, 8192), (4096, 8192), (5000, 12288), (2048, 16384), (3000, 32768), (1100, 65536)])
def test_column_reduction_one_cluster_per_column_block(fdl, cuda, rows, cols):
    """Shapes that take the form in which one cluster of eight CTAs covers all rows of a column
    block (no scratch): against numpy in fp64 and against the chunked form (cols_single = 0)."""
    rng = np.random.default_rng(cols)
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    xd = dev(cuda, x)
    x64 = x.astype(np.float64)
    norm = np.sqrt((x64 ** 2).sum(axis=0))
    single = to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM))
    assert_sum_close(single, x64.sum(axis=0), norm, "col sum")
    assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MEAN)), x64.mean(axis=0), norm / rows, "col mean")
    assert_bit_exact(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MAX)), x.max(axis=0), "col max")
    assert_bit_exact(single, to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), "deterministic")
    fdl.set_tuning("cols_single", 0)
    try:
        chunked = to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM))
    finally:
        fdl.set_tuning("cols_single", 1)
    assert_sum_close(single, chunked, norm, "single cluster vs chunked")


def test_config3_shapes(fdl, cuda):
    """X[8192,8192] ~ N(0,1): sum/max axis 1, mean axis 0, argmax axis 1, full sum."""
    rng = np.random.default_rng(42)
    x = rng.standard_normal((8192, 8192), dtype=np.float32)
    xd = dev(cuda, x)
    x64 = x.astype(np.float64)
    n1 = np.sqrt((x64 ** 2).sum(axis=1))
    n0 = np.sqrt((x64 ** 2).sum(axis=0))
    assert_sum_close(to_np(fdl.reduce_rows(xd, fdl.REDUCE_SUM)), x64.sum(axis=1), n1, "sum axis 1")
    assert_bit_exact(to_np(fdl.reduce_rows(xd, fdl.REDUCE_MAX)), x.max(axis=1), "max axis 1")
    assert_sum_close(to_np(fdl.reduce_cols(xd, fdl.REDUCE_MEAN)), x64.mean(axis=0), n0 / 8192, "mean axis 0")
    np.testing.assert_array_equal(to_np(fdl.argmax_rows(xd)), x.argmax(axis=1))
    assert_sum_close(to_np(fdl.full_sum(xd))[0], x64.sum(), np.sqrt((x64 ** 2).sum()), "full sum")
