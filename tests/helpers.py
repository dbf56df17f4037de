"""Shared helpers of the GPU parity tests: seeded inputs and the error metrics.

Tolerances (from the task statement):
  exact ops (add, sub, mul, div, max, relu, leaky_relu, argmax, broadcast, block trees) -> 0 differing bits
  transcendental activations                                                      -> <= 2 ulp
  sums / means                                                                    -> 1e-5 relative, with
      the Euclidean norm of the addends as the floor of the denominator (a sum of n
      random terms has rounding error proportional to that norm, not to the sum, which
      may be arbitrarily close to zero)
  softmax / layernorm                                                             -> 1e-5 * max(1, |ref|), the form of
      the reference's own softmax benchmark check (tests/benchmarks/softmax/softmax_benchmark.cu:38-48)
"""
import numpy as np

REL_TOL = 1e-5


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bit_exact(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    diff = bits(got) != bits(want)
    # NaN payloads are not part of the contract: NaN matches NaN.
    diff &= ~(np.isnan(got) & np.isnan(want))
    n = int(diff.sum())
    if n:
        i = int(np.flatnonzero(diff.ravel())[0])
        raise AssertionError(f"{what}: {n} elements differ; first at {i}: got {got.ravel()[i]!r} want {want.ravel()[i]!r}")


def assert_close_scaled(got, want, what="", truth=None):
    """|got - want| <= 1e-5 * max(1, |want|).  When `truth` (a float64 evaluation of the same
    formula) is given, the CPU twin's own distance from it is granted on top: the reference's
    CPU functions accumulate long rows sequentially in fp32 and drift from the exact value by
    more than the tolerance once rows reach several thousand elements."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    allowed = REL_TOL * np.maximum(1.0, np.abs(want))
    if truth is not None:
        allowed = allowed + np.abs(want - np.asarray(truth, dtype=np.float64))
    excess = np.abs(got - want) - allowed
    worst = float(excess.max()) if excess.size else 0.0
    assert worst <= 0.0, f"{what}: error exceeds the allowance by {worst:.3e}"
    err = np.abs(got - want) / np.maximum(1.0, np.abs(want))
    return float(err.max()) if err.size else 0.0


def assert_sum_close(got, want, norm2, what=""):
    got, want, norm2 = (np.asarray(v, dtype=np.float64) for v in (got, want, norm2))
    err = np.abs(got - want) / np.maximum(np.abs(want), norm2)
    worst = float(err.max()) if err.size else 0.0
    assert worst <= REL_TOL, f"{what}: max relative error {worst:.3e} > {REL_TOL}"
    return worst


def to_np(t):
    return t.detach().cpu().numpy()
