"""fdl_sum_f32_static: the full sum for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is not allowed -- their own framework's
allocator has to account for every device byte, the service's memory budget was fixed at
start-up, or the code path must never enter the driver's allocator because cudaMalloc and
cudaFree synchronise the device.  For them the library offers one variant of the full sum whose scratch is a fixed array inside
the library's device image.  This file checks, through the C ABI, that it gives the same
answer as the regular entry point on two calls in a row (the array keeps the previous
call's contents, so the second call is the interesting one), that it also agrees when the
two are interleaved, and that sizes above its stated maximum are refused before anything
is launched.

The file name sorts last so that a run which stops at the first failure has already
exercised every other test.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import assert_sum_close, to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 1000, (1 << 20) + 3, 1 << 24])
def test_static_scratch_sum_matches_regular_entry_point_twice(fdl, cuda, n):
    rng = np.random.default_rng(42)
    x = rng.uniform(-1, 1, n).astype(np.float32)
    xd = cuda.from_numpy(x).cuda()
    want32, want64 = fdl.full_sum(xd, want_f64=True)
    want32, want64 = to_np(want32)[0], to_np(want64)[0]
    norm = max(orc.norm2(x), 1e-30)
    for call in range(2):
        got32, got64 = fdl.full_sum_static(xd, want_f64=True)
        assert_sum_close(to_np(got32)[0], want32, norm, f"static sum call {call} n={n}")
        assert_sum_close(to_np(got64)[0], want64, norm, f"static sum (f64) call {call} n={n}")
        assert_sum_close(to_np(got32)[0], orc.full_sum(x), norm, f"static sum vs oracle call {call}")


def test_static_and_regular_calls_interleave(fdl, cuda):
    rng = np.random.default_rng(7)
    a = cuda.from_numpy(rng.normal(size=(1 << 22) + 5).astype(np.float32)).cuda()
    b = cuda.from_numpy(rng.normal(size=12345).astype(np.float32)).cuda()
    ra, rb = to_np(fdl.full_sum(a))[0], to_np(fdl.full_sum(b))[0]
    na, nb = orc.norm2(to_np(a)), orc.norm2(to_np(b))
    for _ in range(3):  # same stream, so the calls are ordered and may share the array
        assert_sum_close(to_np(fdl.full_sum_static(a))[0], ra, na, "a")
        assert_sum_close(to_np(fdl.full_sum_static(b))[0], rb, nb, "b")
        assert_sum_close(to_np(fdl.full_sum(a))[0], ra, na, "regular a")
    unaligned = cuda.from_numpy(np.concatenate([[0.0], to_np(b)]).astype(np.float32)).cuda()[1:]
    assert_sum_close(to_np(fdl.full_sum_static(unaligned))[0], rb, nb, "unaligned input")


def test_no_device_memory_is_taken(fdl, cuda):
    """The point of the entry point: the device's free memory is the same before the first
    call, after it and after later calls (the regular entry point, in contrast, may allocate
    the library's workspace on its first use)."""
    x = cuda.ones(1 << 22, dtype=cuda.float32, device="cuda")
    out = cuda.zeros(1, dtype=cuda.float32, device="cuda")
    cuda.cuda.synchronize()
    free_before, _ = cuda.cuda.mem_get_info()
    for _ in range(3):
        fdl.check(fdl.lib().fdl_sum_f32_static(x.data_ptr(), x.numel(), out.data_ptr(), None, None), "static sum")
        cuda.cuda.synchronize()
        free_now, _ = cuda.cuda.mem_get_info()
        assert free_now == free_before
    assert out.item() == float(1 << 22)


def test_static_entry_in_a_cuda_graph_after_one_eager_call(fdl, cuda):
    """After one eager call (which looks up the array's address for the device) the call is a
    memset node and a kernel node: captured once, replayed on changed data, it follows the data."""
    x = cuda.full((1 << 22,), 0.5, dtype=cuda.float32, device="cuda")
    out = cuda.zeros(1, dtype=cuda.float32, device="cuda")
    out64 = cuda.zeros(1, dtype=cuda.float64, device="cuda")
    fdl.check(fdl.lib().fdl_sum_f32_static(x.data_ptr(), x.numel(), out.data_ptr(), out64.data_ptr(), None), "eager")
    cuda.cuda.synchronize()
    assert out.item() == 0.5 * (1 << 22)
    side = cuda.cuda.Stream()
    side.wait_stream(cuda.cuda.current_stream())
    graph = cuda.cuda.CUDAGraph()
    with cuda.cuda.stream(side):
        with cuda.cuda.graph(graph, stream=side):
            fdl.check(fdl.lib().fdl_sum_f32_static(x.data_ptr(), x.numel(), out.data_ptr(), out64.data_ptr(),
                                                   side.cuda_stream), "captured")
    cuda.cuda.current_stream().wait_stream(side)
    for value in (0.25, 2.0, -1.0):
        x.fill_(value)
        out.zero_()
        graph.replay()
        cuda.cuda.synchronize()
        assert out.item() == value * (1 << 22) and out64.item() == value * (1 << 22)
    fdl.take_device_error()


def test_the_maximum_size_itself_is_accepted(fdl, cuda):
    n = 1 << 30
    free, _ = cuda.cuda.mem_get_info()
    if free < n * 4 + (1 << 30):
        pytest.skip("not enough free device memory for 2^30 floats")
    x = cuda.full((n,), 0.25, dtype=cuda.float32, device="cuda")
    for _ in range(2):
        s32, s64 = fdl.full_sum_static(x, want_f64=True)
        assert s64.item() == 0.25 * n and s32.item() == 0.25 * n   # exact in both widths
    x[n - 1] = 1.25
    assert fdl.full_sum_static(x, want_f64=True)[1].item() == 0.25 * n + 1.0


def test_sizes_above_the_maximum_are_refused(fdl, cuda):
    x = cuda.zeros(16, dtype=cuda.float32, device="cuda")
    out = cuda.zeros(1, dtype=cuda.float32, device="cuda")
    status = fdl.lib().fdl_sum_f32_static(x.data_ptr(), (1 << 30) + 1, out.data_ptr(), None, None)
    assert status == -6
    assert b"2^30" in fdl.lib().fdl_error_string(status)
    assert fdl.lib().fdl_sum_f32_static(x.data_ptr(), -1, out.data_ptr(), None, None) == -1
    assert fdl.lib().fdl_sum_f32_static(x.data_ptr(), 16, None, None, None) == -1
