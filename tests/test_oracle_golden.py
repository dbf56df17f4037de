"""The CPU oracle against the reference's own vectors (no GPU needed).

tests/golden/reference_vectors.npz holds (1) the literal arrays of the reference's tests
for this path and (2) outputs of the reference's CPU check functions on seeded inputs;
tests/golden/make_golden.py regenerates it from the reference tree.  The oracle must
reproduce every one of them: bit for bit where the arithmetic is the same libm / IEEE
sequence, within the reference test's own tolerance where the literal was hand-written.
"""
import numpy as np
import pytest

from oracle import oracle as orc

ACT = ["relu", "leaky_relu", "gelu", "sigmoid", "tanh"]


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_elementwise_literals(golden):
    a, b = golden["elementwise_a"], golden["elementwise_b"]
    for op, name in enumerate(["add", "sub", "mul", "div"]):
        np.testing.assert_array_equal(bits(orc.binary(a, b, op)), bits(golden["elementwise_expected_" + name]))


def test_relu_module_literals(golden):
    got = orc.unary(golden["relu_module_input"], 0)
    np.testing.assert_array_equal(bits(got), bits(golden["relu_module_expected"]))


@pytest.mark.parametrize("op", range(5))
def test_activation_test_vector(golden, op):
    got = orc.unary(golden["activation_input"], op, 0.01)
    np.testing.assert_array_equal(bits(got), bits(golden["activation_expected_" + ACT[op]]))


@pytest.mark.parametrize("op", range(5))
def test_activation_seeded(golden, op):
    x = golden["seeded_activation_input"]
    got, want = orc.unary(x, op, 0.01), golden["seeded_activation_" + ACT[op]]
    np.testing.assert_array_equal(bits(got), bits(want))


def test_softmax_test_vector(golden):
    got = orc.softmax_rows(golden["softmax_input"])
    np.testing.assert_array_equal(bits(got), bits(golden["softmax_expected"]))
    np.testing.assert_allclose(got.sum(axis=1), 1.0, atol=1e-4)  # the reference test's own property


def test_softmax_seeded_both_reference_variants(golden):
    x = golden["seeded_softmax_input"]
    got = orc.softmax_rows(x)
    # tests/tensor/softmax_tensor_test.cpp starts the max at x[0], the benchmark twin at -FLT_MAX:
    # identical for finite inputs, and both are reproduced bit for bit.
    np.testing.assert_array_equal(bits(got), bits(golden["seeded_softmax_test"]))
    np.testing.assert_array_equal(bits(got), bits(golden["seeded_softmax_bench"]))


def test_layernorm_test_vector(golden):
    got = orc.layernorm_rows(golden["layernorm_input"], eps=1e-5)
    np.testing.assert_array_equal(bits(got), bits(golden["layernorm_expected"]))


def test_layernorm_seeded(golden):
    got = orc.layernorm_rows(golden["seeded_layernorm_input"], eps=1e-5)
    np.testing.assert_array_equal(bits(got), bits(golden["seeded_layernorm_expected"]))


def test_vector_add_seeded(golden):
    got = orc.binary(golden["seeded_add_a"], golden["seeded_add_b"], 0)
    np.testing.assert_array_equal(bits(got), bits(golden["seeded_add_expected"]))


def test_block_reduce_both_trees(golden):
    x = golden["seeded_reduce_input"]
    np.testing.assert_array_equal(bits(orc.block_reduce_1024(x, 0)), bits(golden["seeded_reduce_interleave"]))
    np.testing.assert_array_equal(bits(orc.block_reduce_1024(x, 1)), bits(golden["seeded_reduce_address"]))
    # the two trees really are different orders
    assert np.any(bits(golden["seeded_reduce_interleave"]) != bits(golden["seeded_reduce_address"]))


# ---- definitions that the reference does not pin: check them against numpy ----------------


def test_chain_has_two_roundings():
    rng = np.random.default_rng(7)
    a, b, c = (rng.uniform(-1, 1, 100000).astype(np.float32) for _ in range(3))
    want = np.maximum(np.float32(0), (a * b).astype(np.float32) + c)
    np.testing.assert_array_equal(bits(orc.mul_add_relu(a, b, c)), bits(want))
    fused = np.maximum(0.0, a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)
    assert np.any(bits(fused) != bits(want)), "inputs should distinguish FMA from mul-then-add"


@pytest.mark.parametrize("sa,sb", [((5, 7), (1, 7)), ((5, 7), (5, 1)), ((3, 1, 4), (1, 6, 1)), ((4,), (3, 4)),
                                   ((2, 3, 4), (2, 3, 4)), ((1,), (3, 2))])
def test_broadcast_matches_numpy(sa, sb):
    rng = np.random.default_rng(3)
    a = rng.normal(size=sa).astype(np.float32)
    b = rng.uniform(0.5, 2.0, size=sb).astype(np.float32)
    for op, fn in enumerate([np.add, np.subtract, np.multiply, np.divide]):
        np.testing.assert_array_equal(bits(orc.broadcast_binary(a, b, op)), bits(fn(a, b)))


def test_axis_reductions_match_numpy():
    rng = np.random.default_rng(5)
    x = rng.normal(size=(37, 129)).astype(np.float32)
    np.testing.assert_array_equal(orc.reduce_rows(x, 2), x.max(axis=1))
    np.testing.assert_allclose(orc.reduce_rows(x, 0), x.astype(np.float64).sum(axis=1), rtol=1e-6)
    np.testing.assert_allclose(orc.reduce_rows(x, 1), x.astype(np.float64).mean(axis=1), rtol=1e-6, atol=1e-9)
    np.testing.assert_allclose(orc.reduce_cols(x, 1), x.astype(np.float64).mean(axis=0), rtol=1e-6, atol=1e-9)
    np.testing.assert_array_equal(orc.reduce_cols(x, 2), x.max(axis=0))
    np.testing.assert_array_equal(orc.argmax_rows(x), x.argmax(axis=1))
    assert abs(orc.full_sum(x) - x.astype(np.float64).sum()) < 1e-9


def test_argmax_ties_and_nan():
    x = np.array([[1, 3, 3, 2], [np.nan, -np.inf, -np.inf, np.nan], [np.nan, 5, np.nan, 5],
                  [-np.inf, -np.inf, -np.inf, -np.inf]], dtype=np.float32)
    np.testing.assert_array_equal(orc.argmax_rows(x), [1, 0, 1, 0])


def test_layernorm_affine_is_composition():
    rng = np.random.default_rng(9)
    x = rng.normal(0, 3, (5, 64)).astype(np.float32)
    g = rng.uniform(0.9, 1.1, 64).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, 64).astype(np.float32)
    plain = orc.layernorm_rows(x)
    np.testing.assert_array_equal(bits(orc.layernorm_rows(x, g, b)), bits((plain * g).astype(np.float32) + b))
    np.testing.assert_allclose(orc.layernorm_rows(x, g, b), orc.layernorm_rows_f64(x, g, b), atol=2e-6, rtol=1e-5)
