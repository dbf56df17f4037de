"""GPU parity: row softmax and row layernorm through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle import ref
from tests.helpers import assert_close_scaled, to_np

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1), (2, 4), (3, 5), (7, 128), (100, 132), (33, 1000), (64, 1024), (4096, 1024), (65, 2048),
          (37, 2052), (19, 4096), (11, 8192), (5, 16384), (3, 16388), (2, 40000), (1001, 36), (50000, 8),
          # rows shared by a cluster of 2, 4, 8 CTAs; beyond 131072 floats and odd lengths: the plain kernel
          (5, 32768), (9, 32772), (3, 65536), (4, 100000), (2, 131072), (2, 131076), (3, 50001),
          # lengths that are not a multiple of 4 floats: 128-bit accesses over the flat buffer, masked edges
          (7, 127), (1000, 63), (50000, 7), (513, 255), (65, 1001), (33, 1023), (19, 4095), (11, 8191), (5, 16381),
          (4, 16383), (1000, 2), (999, 3), (300, 129), (17, 2049),
          # longer still: the row in a cluster's shared memory (8 or 16 CTAs), then segments + per-row combination
          (3, 262144), (5, 200004), (2, 1 << 20), (1, 3000000), (2, 131077), (40, 50257), (3, 300000), (3, 300001),
          (2, 500004), (2, 524288), (3, 800003), (2, 900000)]


def dev(cuda, a):
    return cuda.from_numpy(np.ascontiguousarray(a)).cuda()


def test_reference_literals(fdl, cuda, golden):
    got = to_np(fdl.softmax_rows(dev(cuda, golden["softmax_input"])))
    assert np.abs(got - golden["softmax_expected"]).max() <= 1e-4  # the reference test's tolerance
    assert np.abs(got.sum(axis=1) - 1).max() <= 1e-4               # and its row-sum property
    assert_close_scaled(got, golden["softmax_expected"], "softmax literal")
    got = to_np(fdl.layernorm_rows(dev(cuda, golden["layernorm_input"]), eps=1e-5))
    assert np.abs(got - golden["layernorm_expected"]).max() <= 1e-4
    assert_close_scaled(got, golden["layernorm_expected"], "layernorm literal")
    for key in ("softmax", "layernorm"):
        x = golden[f"seeded_{key}_input"]
        want = golden["seeded_softmax_bench"] if key == "softmax" else golden["seeded_layernorm_expected"]
        fn = fdl.softmax_rows if key == "softmax" else fdl.layernorm_rows
        assert_close_scaled(to_np(fn(dev(cuda, x))), want, f"seeded {key}")


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_softmax(fdl, cuda, rows, cols):
    rng = np.random.default_rng(42)
    x = rng.normal(0, 3, (rows, cols)).astype(np.float32)
    got = to_np(fdl.softmax_rows(dev(cuda, x)))
    truth = orc.softmax_rows_f64(x)
    assert_close_scaled(got, truth, f"softmax vs f64 {rows}x{cols}")
    assert_close_scaled(got, orc.softmax_rows(x), f"softmax {rows}x{cols}", truth=truth if cols > 4096 else None)
    assert np.abs(got.astype(np.float64).sum(axis=1) - 1).max() <= 1e-5
    fdl.take_device_error()


def test_softmax_reference_benchmark_case(fdl, cuda):
    """4096 x 1024 uniform[-10, 10], the reference benchmark's case and tolerance."""
    rng = np.random.default_rng(42)
    x = rng.uniform(-10, 10, (4096, 1024)).astype(np.float32)
    xd = dev(cuda, x)
    got = to_np(fdl.softmax_rows(xd))
    assert_close_scaled(got, orc.softmax_rows(x), "bench case")
    if ref.available():
        for algo in (0, 1, 2):
            want = cuda.empty_like(xd)
            cuda.cuda.synchronize()
            ref.gpu_softmax(xd.data_ptr(), want.data_ptr(), 4096, 1024, algo)
            ref.gpu_sync()
            assert_close_scaled(got, to_np(want), f"reference kernel algo {algo}")


def test_softmax_extremes(fdl, cuda):
    x = np.zeros((4, 1024), dtype=np.float32)
    x[0, :] = 1e30
    x[1, 0] = 88.0
    x[2, :] = -1e30
    x[3, 5] = -np.inf
    got = to_np(fdl.softmax_rows(dev(cuda, x)))
    assert_close_scaled(got, orc.softmax_rows(x), "extremes")


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("affine", [False, True])
def test_layernorm(fdl, cuda, rows, cols, affine):
    rng = np.random.default_rng(42)
    x = rng.normal(0, 3, (rows, cols)).astype(np.float32)
    g = rng.uniform(0.9, 1.1, cols).astype(np.float32) if affine else None
    b = rng.uniform(-0.1, 0.1, cols).astype(np.float32) if affine else None
    gd = dev(cuda, g) if affine else None
    bd = dev(cuda, b) if affine else None
    got, mean, rstd = fdl.layernorm_rows(dev(cuda, x), gd, bd, eps=1e-5, want_stats=True)
    got = to_np(got)
    truth = orc.layernorm_rows_f64(x, g, b, 1e-5)
    assert_close_scaled(got, truth, f"layernorm vs f64 {rows}x{cols}")
    if cols > 1:
        # the twin's one-pass variance cancels on rows of two or three nearly equal values
        assert_close_scaled(got, orc.layernorm_rows(x, g, b, 1e-5), f"layernorm {rows}x{cols}",
                            truth=truth if cols > 4096 or cols < 4 else None)
    x64 = x.astype(np.float64)
    assert_close_scaled(to_np(mean), x64.mean(axis=1), "mean")
    np.testing.assert_allclose(to_np(rstd), 1 / np.sqrt(x64.var(axis=1) + 1e-5), rtol=1e-5)
    fdl.take_device_error()


def test_layernorm_vs_reference_kernel(fdl, cuda):
    if not ref.available():
        pytest.skip("oracle/_ref/libref.so was not built")
    rng = np.random.default_rng(42)
    x = dev(cuda, rng.normal(0, 3, (4096, 1024)).astype(np.float32))
    want = cuda.empty_like(x)
    cuda.cuda.synchronize()
    ref.gpu_layernorm(x.data_ptr(), want.data_ptr(), 4096, 1024, 1e-5)
    ref.gpu_sync()
    assert_close_scaled(to_np(fdl.layernorm_rows(x)), to_np(want), "reference kernel")


def test_config4_shape(fdl, cuda):
    """logits[65536,1024] ~ N(0,3); gamma ~ U[0.9,1.1], beta ~ U[-0.1,0.1], eps 1e-5.
    Full size: checked through size-independent properties plus a sampled oracle comparison."""
    rng = np.random.default_rng(42)
    x = (rng.standard_normal((65536, 1024), dtype=np.float32) * np.float32(3))
    g = rng.uniform(0.9, 1.1, 1024).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, 1024).astype(np.float32)
    xd = dev(cuda, x)
    sm = to_np(fdl.softmax_rows(xd))
    assert np.abs(sm.astype(np.float64).sum(axis=1) - 1).max() <= 1e-5
    assert (sm >= 0).all() and np.array_equal(sm.argmax(axis=1), x.argmax(axis=1))
    pick = rng.choice(65536, 512, replace=False)
    assert_close_scaled(sm[pick], orc.softmax_rows(x[pick]), "softmax sample")
    ln = to_np(fdl.layernorm_rows(xd, dev(cuda, g), dev(cuda, b), eps=1e-5))
    assert_close_scaled(ln[pick], orc.layernorm_rows(x[pick], g, b, 1e-5), "layernorm sample")
    plain = to_np(fdl.layernorm_rows(xd)).astype(np.float64)
    assert np.abs(plain.mean(axis=1)).max() <= 1e-5 and np.abs(plain.var(axis=1) - 1).max() <= 1e-4
    fdl.take_device_error()


@pytest.mark.parametrize("rows,cols", [(1, 4), (1001, 36), (50000, 8), (70000, 32), (4097, 64), (7, 128), (3000, 128),
                                       (513, 256), (64, 1024), (65, 2048), (11, 8192), (5, 16384)])
def test_direct_and_staged_forms_agree(fdl, cuda, rows, cols):
    """The two ways of bringing rows in (direct loads / one bulk-async copy per CTA), each forced
    through the tuning knob: both within tolerance of the oracle (they are two kernels, and the
    compiler need not contract their arithmetic alike, so they are not compared bit for bit).
    The default picks between them by row length."""
    rng = np.random.default_rng(7)
    x = rng.normal(0, 3, (rows, cols)).astype(np.float32)
    g = rng.uniform(0.9, 1.1, cols).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, cols).astype(np.float32)
    xd, gd, bd = dev(cuda, x), dev(cuda, g), dev(cuda, b)
    out = {}
    try:
        for mode in (0, 1, -1):
            fdl.set_tuning("rows_staged", mode)
            out[mode] = (to_np(fdl.softmax_rows(xd)), to_np(fdl.layernorm_rows(xd, gd, bd)))
            cuda.cuda.synchronize()
            fdl.take_device_error()
    finally:
        fdl.set_tuning("rows_staged", -1)
    truth_sm, truth_ln = orc.softmax_rows_f64(x), orc.layernorm_rows_f64(x, g, b, 1e-5)
    for mode in (0, 1, -1):
        assert_close_scaled(out[mode][0], truth_sm, f"softmax form {mode} {rows}x{cols}")
        assert_close_scaled(out[mode][1], truth_ln, f"layernorm form {mode} {rows}x{cols}")
    # The default is one of the two, picked by row length alone (so a shape always gets the same bits).
    picked = 1 if cols <= 128 else 0
    for k in (0, 1):
        assert np.array_equal(out[-1][k].view(np.uint32), out[picked][k].view(np.uint32))


@pytest.mark.parametrize("rows,cols", [(6, 16390), (3, 50257), (5, 65540), (4, 131072), (3, 262144), (2, 400002), (2, 524288)])
def test_shared_memory_cluster_form_agrees_with_the_other_forms(fdl, cuda, rows, cols):
    """Long rows kept in a cluster's shared memory (the default) against the register-cluster and
    two-kernel forms (tuning key rows_smem = 0) and against the fp64 oracle, with statistics."""
    rng = np.random.default_rng(cols)
    x = rng.normal(0, 3, (rows, cols)).astype(np.float32)
    g = rng.uniform(0.9, 1.1, cols).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, cols).astype(np.float32)
    xd, gd, bd = dev(cuda, x), dev(cuda, g), dev(cuda, b)
    out = {}
    for mode in (1, 0):
        fdl.set_tuning("rows_smem", mode)
        try:
            sm = to_np(fdl.softmax_rows(xd))
            ln, mean, rstd = (to_np(t) for t in fdl.layernorm_rows(xd, gd, bd, want_stats=True))
        finally:
            fdl.set_tuning("rows_smem", 1)
        out[mode] = (sm, ln, mean, rstd)
    fdl.take_device_error()
    assert_close_scaled(out[1][0], orc.softmax_rows_f64(x), "softmax vs fp64")
    assert_close_scaled(out[1][1], orc.layernorm_rows_f64(x, g, b, 1e-5), "layernorm vs fp64")
    assert np.abs(out[1][0].sum(axis=1) - 1).max() <= 1e-5
    x64 = x.astype(np.float64)
    assert np.abs(out[1][2] - x64.mean(axis=1)).max() <= 1e-5
    assert np.abs(out[1][3] / (1 / np.sqrt(x64.var(axis=1) + 1e-5)) - 1).max() <= 1e-5
    assert_close_scaled(out[1][0], out[0][0], "softmax: shared-memory form vs the other forms")
    assert_close_scaled(out[1][1], out[0][1], "layernorm: shared-memory form vs the other forms")


@pytest.mark.parametrize("rows,cols", [(1, 131076), (2, 524288), (3, 300001), (41, 140000), (67, 131077), (300, 132000),
                                       (5, 2100004)])
@pytest.mark.parametrize("lag,hints", [(0, 1), (1, 1), (3, 0)])
def test_one_kernel_form_of_rows_longer_than_a_cluster_equals_the_two_kernel_form(fdl, cuda, rows, cols, lag, hints):
    """Rows beyond 131072 floats.  The default takes the statistics of a row and applies them in
    ONE launch, the apply tasks a few rows behind so that they read from L2.  It gives the bits of
    the two-kernel form (tuning key rows_split_fused = 0) at any lag, with and without the L2
    hints, leaves no device error, and leaves the shared counters at zero: a second call, and
    the other ops that use the counters, still answer right."""
    rng = np.random.default_rng(rows * 1000003 + cols)
    x = rng.normal(0, 3, (rows, cols)).astype(np.float32)
    g = rng.uniform(0.9, 1.1, cols).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, cols).astype(np.float32)
    xd, gd, bd = dev(cuda, x), dev(cuda, g), dev(cuda, b)
    out = {}
    for fused in (1, 0, 1):
        fdl.set_tuning("rows_split_fused", fused)
        fdl.set_tuning("rows_split_lag", lag)
        fdl.set_tuning("rows_split_hints", hints)
        try:
            sm = to_np(fdl.softmax_rows(xd))
            ln, mean, rstd = (to_np(t) for t in fdl.layernorm_rows(xd, gd, bd, want_stats=True))
        finally:
            fdl.set_tuning("rows_split_fused", 1)
            fdl.set_tuning("rows_split_lag", 0)
            fdl.set_tuning("rows_split_hints", 1)
        if fused in out:
            for first, again in zip(out[fused], (sm, ln, mean, rstd)):
                assert np.array_equal(first, again)
        out[fused] = (sm, ln, mean, rstd)
    fdl.take_device_error()  # raises if a bounded wait ran out
    for one, two in zip(out[1], out[0]):
        assert np.array_equal(one, two)
    assert_close_scaled(out[1][0], orc.softmax_rows_f64(x), "softmax vs fp64")
    assert_close_scaled(out[1][1], orc.layernorm_rows_f64(x, g, b, 1e-5), "layernorm vs fp64")
    # the column reduction and the full sum share the counter block
    col = to_np(fdl.reduce_cols(xd, fdl.REDUCE_SUM))
    assert np.abs(col - x.astype(np.float64).sum(axis=0)).max() <= 1e-4 * max(1.0, np.abs(x).sum(axis=0).max())
    total = float(to_np(fdl.full_sum(xd)).reshape(-1)[0])
    assert abs(total - x.astype(np.float64).sum()) <= 1e-5 * np.abs(x).sum()


@pytest.mark.parametrize("rows,cols", [(64, 1024), (100, 1001), (1000, 63), (7, 4096), (9, 8190), (5, 16380),
                                       (3, 40001), (2, 20000), (2, 140002), (3, 65537), (2, 460001)])
@pytest.mark.parametrize("x_off,y_off", [(1, 1), (3, 3), (2, 2), (1, 2), (0, 1)])
def test_rows_at_any_phase_of_a_16_byte_line(fdl, cuda, rows, cols, x_off, y_off):
    """Views whose base is not 16-byte aligned: same phase for x and y (the masked form) and
    different phases (the plain kernel); the floats around the views must stay untouched."""
    rng = np.random.default_rng(11)
    x = rng.normal(0, 3, (rows, cols)).astype(np.float32)
    g = rng.uniform(0.9, 1.1, cols).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, cols).astype(np.float32)
    n = rows * cols
    xbuf = cuda.full((n + 8,), 7.0, dtype=cuda.float32, device="cuda")
    xbuf[x_off:x_off + n] = dev(cuda, x).reshape(-1)
    xv = xbuf[x_off:x_off + n].view(rows, cols)
    gbuf = dev(cuda, np.concatenate([np.zeros(1, np.float32), g]))[1:]     # gamma off the 16-byte grid too
    bd = dev(cuda, b)
    for name in ("softmax", "layernorm"):
        ybuf = cuda.full((n + 8,), -5.0, dtype=cuda.float32, device="cuda")
        yv = ybuf[y_off:y_off + n].view(rows, cols)
        if name == "softmax":
            fdl.softmax_rows(xv, out=yv)
            truth = orc.softmax_rows_f64(x)
        else:
            fdl.layernorm_rows(xv, gbuf, bd, out=yv)
            truth = orc.layernorm_rows_f64(x, g, b, 1e-5)
        cuda.cuda.synchronize()
        assert_close_scaled(to_np(yv), truth, f"{name} {rows}x{cols} phases {x_off},{y_off}")
        guard = to_np(ybuf)
        assert (guard[:y_off] == -5.0).all() and (guard[y_off + n:] == -5.0).all(), "wrote outside the view"
    fdl.take_device_error()
