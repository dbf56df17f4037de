"""Sizes beyond the reference's `int n` interface (2^31 elements and a little more), checked
on the device through size-independent properties: 64-bit indexing must not wrap."""
import pytest

pytestmark = pytest.mark.gpu


def test_more_than_int_max_elements(fdl, cuda):
    n = (1 << 31) + 5
    free, _ = cuda.cuda.mem_get_info()
    if free < 5 * n * 4:
        pytest.skip("not enough free device memory")
    a = cuda.empty(n, dtype=cuda.float32, device="cuda")
    a.copy_(cuda.arange(0, 1 << 20, dtype=cuda.float32, device="cuda").repeat((n >> 20) + 1)[:n])
    b = cuda.full((n,), 0.5, dtype=cuda.float32, device="cuda")
    out = fdl.binary(a, b, fdl.ADD)
    # spot checks across the whole range, including both sides of 2^31 and the ragged tail
    for i in (0, 1, (1 << 30) + 7, (1 << 31) - 1, 1 << 31, n - 2, n - 1):
        assert out[i].item() == a[i].item() + 0.5, i
    assert cuda.equal(out[-4096:], a[-4096:] + 0.5) and cuda.equal(out[:4096], a[:4096] + 0.5)
    mid = (1 << 31) - 2048
    assert cuda.equal(out[mid:mid + 4096], a[mid:mid + 4096] + 0.5)
    del out
    r = fdl.unary(b, fdl.RELU)
    assert r[n - 1].item() == 0.5 and r[1 << 31].item() == 0.5
    del r
    s32, s64 = fdl.full_sum(b, want_f64=True)
    assert s64.item() == 0.5 * n      # exact in double
    ones = b.fill_(1.0)
    assert fdl.full_sum(ones, want_f64=True)[1].item() == float(n)
