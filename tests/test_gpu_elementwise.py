"""GPU parity: elementwise, fused chain, activations, broadcast -- through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle import ref
from tests.helpers import assert_bit_exact, to_np

pytestmark = pytest.mark.gpu

SIZES = [1, 3, 4, 255, 257, 1023, 1025, 4096, 4099, 1 << 20, (1 << 20) + 7]
ACT = ["relu", "leaky_relu", "gelu", "sigmoid", "tanh"]


def dev(cuda, a):
    return cuda.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("op", range(4))
def test_reference_literals(fdl, cuda, golden, op):
    name = ["add", "sub", "mul", "div"][op]
    got = fdl.binary(dev(cuda, golden["elementwise_a"]), dev(cuda, golden["elementwise_b"]), op)
    assert_bit_exact(to_np(got), golden["elementwise_expected_" + name], name)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("op", range(4))
def test_binary_bit_exact(fdl, cuda, n, op):
    rng = np.random.default_rng(42 + op)
    a = rng.uniform(-1, 1, n).astype(np.float32)
    b = rng.uniform(-1, 1, n).astype(np.float32)
    if n > 8:
        a[:8] = [0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, 3e38, -3e38]
        b[:8] = [0.0, 0.0, np.inf, 1.0, 1.0, 1e-45, 3e38, 3e38]
    got = fdl.binary(dev(cuda, a), dev(cuda, b), op)
    assert_bit_exact(to_np(got), orc.binary(a, b, op), f"op{op} n={n}")


def test_binary_unaligned_views_and_aliasing(fdl, cuda):
    rng = np.random.default_rng(1)
    n = 10007
    a = dev(cuda, rng.uniform(-1, 1, n + 3).astype(np.float32))
    b = dev(cuda, rng.uniform(-1, 1, n + 3).astype(np.float32))
    for off in (1, 2, 3):
        av, bv = a[off:off + n], b[off:off + n]
        out = cuda.empty(n + 3, dtype=cuda.float32, device="cuda")[off:off + n]
        fdl.binary(av, bv, fdl.MUL, out=out)
        assert_bit_exact(to_np(out), orc.binary(to_np(av), to_np(bv), fdl.MUL), f"offset {off}")
    want = orc.binary(to_np(a), to_np(b), fdl.ADD)
    fdl.binary(a, b, fdl.ADD, out=a)  # in place
    assert_bit_exact(to_np(a), want, "in place")


def test_empty_and_bad_arguments(fdl, cuda):
    e = cuda.empty(0, dtype=cuda.float32, device="cuda")
    assert fdl.binary(e, e, fdl.ADD).numel() == 0
    x = cuda.ones(8, dtype=cuda.float32, device="cuda")
    with pytest.raises(fdl.FdlError):
        fdl.binary(x, x, 17)
    with pytest.raises(fdl.FdlError):
        fdl.unary(x, 9)
    assert fdl.lib().fdl_binary_f32(None, None, None, 4, 0, None) == -1


@pytest.mark.parametrize("n", [1, 5, 1023, 4096, (1 << 20) + 3])
def test_fused_chain_two_roundings(fdl, cuda, n):
    rng = np.random.default_rng(42)
    a, b, c = (rng.uniform(-1, 1, n).astype(np.float32) for _ in range(3))
    got = to_np(fdl.mul_add_relu(dev(cuda, a), dev(cuda, b), dev(cuda, c)))
    assert_bit_exact(got, orc.mul_add_relu(a, b, c), f"chain n={n}")
    # and it equals the three separate kernels the reference would launch
    t = fdl.binary(dev(cuda, a), dev(cuda, b), fdl.MUL)
    t = fdl.binary(t, dev(cuda, c), fdl.ADD)
    assert_bit_exact(got, to_np(fdl.unary(t, fdl.RELU)), "vs unfused")


@pytest.mark.parametrize("op", [0, 1])
@pytest.mark.parametrize("n", [1, 6, 1025, (1 << 18) + 1])
def test_exact_activations(fdl, cuda, n, op):
    rng = np.random.default_rng(11)
    x = rng.normal(0, 3, n).astype(np.float32)
    if n > 6:
        x[:6] = [0.0, -0.0, np.nan, np.inf, -np.inf, -1e-45]
    got = to_np(fdl.unary(dev(cuda, x), op, 0.01))
    assert_bit_exact(got, orc.unary(x, op, 0.01), ACT[op])


# Distance allowed against the CPU twins.  The kernels call the same CUDA math functions as
# the reference's kernels (and match those bit for bit, next test); CUDA documents expf and
# tanhf to 2 ulp of the true value and glibc's are good to 1 ulp, so two correct results can
# sit 3 ulp apart.  gelu and sigmoid stay within 2 ulp of the CPU twin on these inputs.
CPU_TWIN_ULP = {2: 2, 3: 2, 4: 3}


@pytest.mark.parametrize("op", [2, 3, 4])
def test_transcendental_activations_vs_cpu(fdl, cuda, golden, op):
    """Against the CPU functions of the reference's activation test (golden vectors)."""
    for key in ("activation_input", "seeded_activation_input"):
        x = golden[key]
        want = golden[("activation_expected_" if key == "activation_input" else "seeded_activation_") + ACT[op]]
        got = to_np(fdl.unary(dev(cuda, x), op, 0.01))
        assert np.abs(got[np.isfinite(want)] - want[np.isfinite(want)]).max() < 1e-5  # the reference test's check
        ulp = orc.ulp_distance(got, want)
        ok = ulp <= CPU_TWIN_ULP[op]
        if op == 2:
            # 1 + tanh(u) cancels for u << 0; there the reference formula itself only promises
            # absolute accuracy of a few ulp of 0.5*|x|, so the ulp test is applied to that scale.
            with np.errstate(invalid="ignore"):
                slack = 2 * np.spacing(np.abs(0.5 * x).astype(np.float32)).astype(np.float64)
                ok |= np.abs(got.astype(np.float64) - want.astype(np.float64)) <= slack
        ok |= np.isnan(got) & np.isnan(want)
        assert ok.all(), f"{ACT[op]}: max ulp {ulp[~ok].max()} at x={x[~ok][:4]}"


@pytest.mark.parametrize("op", range(5))
def test_activations_bit_exact_vs_reference_gpu_kernels(fdl, cuda, op):
    """Same bits as the reference's own CUDA kernels (compiled in place for sm_100a)."""
    if not ref.available():
        pytest.skip("oracle/_ref/libref.so was not built")
    rng = np.random.default_rng(21)
    n = (1 << 20) + 5
    x = dev(cuda, rng.normal(0, 3, n).astype(np.float32))
    want = cuda.empty_like(x)
    cuda.cuda.synchronize()
    ref.gpu_activation(x.data_ptr(), want.data_ptr(), n, op, 0.01)
    ref.gpu_sync()
    assert_bit_exact(to_np(fdl.unary(x, op, 0.01)), to_np(want), ACT[op])


@pytest.mark.parametrize("op", range(4))
def test_binary_bit_exact_vs_reference_gpu_kernels(fdl, cuda, op):
    if not ref.available():
        pytest.skip("oracle/_ref/libref.so was not built")
    rng = np.random.default_rng(22)
    n = (1 << 20) + 1
    a = dev(cuda, rng.uniform(-1, 1, n).astype(np.float32))
    b = dev(cuda, rng.uniform(-1, 1, n).astype(np.float32))
    want = cuda.empty_like(a)
    cuda.cuda.synchronize()
    ref.gpu_elementwise(a.data_ptr(), b.data_ptr(), want.data_ptr(), n, op)
    ref.gpu_sync()
    assert_bit_exact(to_np(fdl.binary(a, b, op)), to_np(want), f"op {op}")


BCAST = [((4096, 4096), (1, 4096)), ((4096, 4096), (4096, 1)), ((33, 70), (1, 70)), ((33, 70), (33, 1)),
         ((7, 5, 12), (5, 1)), ((3, 1, 8), (1, 6, 1)), ((6, 4), (4,)), ((2, 3, 4, 5, 6), (1, 3, 1, 5, 1)),
         ((1,), (5, 3)), ((5, 3), (1,)), ((64, 1), (1, 64)), ((9, 8), (9, 8)),
         # extents that are not multiples of 4: 128-bit packs over the flat buffers of the dense operand and
         # the output, the broadcast operand per element (packs that cross a row, tails of 1-3 elements)
         ((1001, 1001), (1, 1001)), ((1001, 1001), (1001, 1)), ((1001,), (777, 1001)), ((333, 1), (333, 1023)),
         ((5, 63, 7, 9), (1, 63, 1, 1)), ((37, 3), (3,)), ((37, 3), (37, 1)), ((2, 2, 2, 3), (2, 1, 2, 1)),
         ((1023, 5), (1,)), ((7,), (1,)), ((3, 1), (3, 2)), ((64, 1023, 31), (1023, 1)), ((50001,), (1,))]


@pytest.mark.parametrize("sa,sb", BCAST)
def test_broadcast_bit_exact(fdl, cuda, sa, sb):
    rng = np.random.default_rng(43)
    a = rng.normal(size=sa).astype(np.float32)
    b = rng.uniform(0.5, 2.0, size=sb).astype(np.float32)
    ops = range(4) if np.prod(sa) < 100000 else (0, 2)
    for op in ops:
        got = to_np(fdl.broadcast_binary(dev(cuda, a), dev(cuda, b), op))
        assert_bit_exact(got, orc.broadcast_binary(a, b, op), f"{sa} {sb} op{op}")


@pytest.mark.parametrize("rows,cols", [(1, 4), (5, 8), (1000, 64), (777, 1028), (4096, 4096), (3, 40000), (70000, 16)])
@pytest.mark.parametrize("rows_per_thread", [0, 1, 2, 4])
def test_two_dimensional_broadcast_forms(fdl, cuda, rows, cols, rows_per_thread):
    """Every pairing of operand kinds of the two-dimensional kernel -- dense rows, a [1, C] row vector, an
    [R, 1] column vector -- for every rows-per-thread variant, plus a dense operand that is a column
    window of a wider matrix (row stride larger than the row) and the in-place use."""
    import ctypes as C
    rng = np.random.default_rng(46)
    dense = rng.normal(size=(rows, cols)).astype(np.float32)
    rowv = rng.uniform(0.5, 2.0, size=(1, cols)).astype(np.float32)
    colv = rng.uniform(0.5, 2.0, size=(rows, 1)).astype(np.float32)
    fdl.set_tuning("bcast2d_rows", rows_per_thread)
    try:
        for a, b in ((dense, rowv), (rowv, dense), (dense, colv), (colv, dense), (colv, rowv), (rowv, colv)):
            for op in (fdl.ADD, fdl.DIV):
                got = to_np(fdl.broadcast_binary(dev(cuda, a), dev(cuda, b), op))
                assert_bit_exact(got, orc.broadcast_binary(a, b, op), f"{a.shape} {b.shape} op{op}")
        # a window [rows, cols] of a matrix with cols + 8 columns: strides (cols + 8, 1)
        wide = rng.normal(size=(rows, cols + 8)).astype(np.float32)
        wd, rd = dev(cuda, wide), dev(cuda, rowv)
        out = cuda.empty((rows, cols), dtype=cuda.float32, device="cuda")
        arr = C.c_int64 * 2
        fdl.check(fdl.lib().fdl_broadcast_binary_f32(wd.data_ptr() + 16, rd.data_ptr(), out.data_ptr(), 2, arr(rows, cols),
                                                     arr(cols + 8, 1), arr(0, 1), fdl.MUL, None), "window")
        assert_bit_exact(to_np(out), wide[:, 4:4 + cols] * rowv, "window of a wider matrix")
        # in place: the output is the dense operand
        dd = dev(cuda, dense)
        fdl.broadcast_binary(dd, dev(cuda, colv), fdl.MUL, out=dd)
        assert_bit_exact(to_np(dd), dense * colv, "in place")
    finally:
        fdl.set_tuning("bcast2d_rows", 0)


def test_two_dimensional_kernel_equals_general_kernel(fdl, cuda):
    rng = np.random.default_rng(47)
    a = dev(cuda, rng.normal(size=(513, 2052)).astype(np.float32))
    for other in (rng.normal(size=(1, 2052)), rng.normal(size=(513, 1))):
        b = dev(cuda, other.astype(np.float32))
        fast = to_np(fdl.broadcast_binary(a, b, fdl.SUB))
        fdl.set_tuning("bcast2d", 0)
        try:
            general = to_np(fdl.broadcast_binary(a, b, fdl.SUB))
        finally:
            fdl.set_tuning("bcast2d", 1)
        assert_bit_exact(fast, general, "2-D kernel vs general kernel")


def test_config2_bias_then_scale(fdl, cuda):
    """A[4096,4096] + b[1,4096], then * s[4096,1] (stride-0 indexing on either axis)."""
    rng = np.random.default_rng(44)
    A = rng.normal(size=(4096, 4096)).astype(np.float32)
    b = rng.normal(size=(1, 4096)).astype(np.float32)
    s = rng.uniform(0.5, 2.0, size=(4096, 1)).astype(np.float32)
    t = fdl.broadcast_binary(dev(cuda, A), dev(cuda, b), fdl.ADD)
    got = to_np(fdl.broadcast_binary(t, dev(cuda, s), fdl.MUL))
    assert_bit_exact(got, ((A + b).astype(np.float32) * s).astype(np.float32), "config 2")


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 5), (128, 1000), (1000, 4096), (999, 1001), (4096, 63)])
def test_row_bias_in_place(fdl, cuda, rows, cols):
    rng = np.random.default_rng(45)
    x = rng.normal(size=(rows, cols)).astype(np.float32)
    bias = rng.normal(size=cols).astype(np.float32)
    got = to_np(fdl.add_row_bias_(dev(cuda, x), dev(cuda, bias)))
    assert_bit_exact(got, orc.add_row_bias(x, bias), "row bias")
    got = to_np(fdl.add_row_bias_(dev(cuda, x), dev(cuda, bias), relu=True))
    assert_bit_exact(got, orc.add_row_bias(x, bias, relu=True), "row bias + relu")
    if ref.available():
        d = dev(cuda, x)
        cuda.cuda.synchronize()
        ref.gpu_add_row_bias(d.data_ptr(), dev(cuda, bias).data_ptr(), rows, cols)
        ref.gpu_sync()
        assert_bit_exact(to_np(d), orc.add_row_bias(x, bias), "reference kernel vs oracle")
