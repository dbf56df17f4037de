"""Generates tests/golden/reference_vectors.npz from the reference itself.

Run where the reference tree is available (environment variable REFERENCE_ROOT; by default the
directory `reference` beside this repository):

    python tests/golden/make_golden.py

Two kinds of vectors are recorded:
  1. the literal input/expected arrays of the reference's own tests for this path, read
     out of the test sources at generation time (tests/tensor/elementwise_tensor_test.cpp,
     tests/nn/relu_module_test.cpp, tests/tensor/activation_tensor_test.cpp,
     tests/tensor/softmax_tensor_test.cpp, tests/tensor/layernorm_tensor_test.cpp);
  2. outputs of the reference's CPU check functions (compiled in place into
     oracle/_ref/libref.so) on seeded inputs with the shapes and distributions of the
     reference's benchmark runs.
The resulting file is small and is what travels; the reference tree does not.
"""
from __future__ import annotations

import os
import re
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
REF = Path(os.environ.get("REFERENCE_ROOT", str(ROOT.parent / "reference")))

from oracle import build_ref, ref  # noqa: E402


def literal(path: Path, name: str) -> np.ndarray:
    """The float initialiser list of `std::vector<float> <name> = {...};` in a test source."""
    text = path.read_text()
    m = re.search(r"std::vector<float>\s+" + re.escape(name) + r"\s*=\s*\{([^}]*)\}", text)
    if m is None:
        raise KeyError(f"{name} not found in {path}")
    vals = [float(tok.rstrip("f")) for tok in re.findall(r"-?\d+\.?\d*f?", m.group(1))]
    return np.asarray(vals, dtype=np.float32)


def main() -> None:
    build_ref.build_lib()
    g = {}
    t = REF / "tests" / "tensor"
    ew = t / "elementwise_tensor_test.cpp"
    for name in ("a", "b", "expected_add", "expected_sub", "expected_mul", "expected_div"):
        g["elementwise_" + name] = literal(ew, name)
    relu = REF / "tests" / "nn" / "relu_module_test.cpp"
    g["relu_module_input"] = literal(relu, "input")
    g["relu_module_expected"] = literal(relu, "expected")

    act_in = literal(t / "activation_tensor_test.cpp", "input")
    g["activation_input"] = act_in
    for op, name in enumerate(("relu", "leaky_relu", "gelu", "sigmoid", "tanh")):
        g["activation_expected_" + name] = ref.cpu_activation(act_in, op, 0.01)

    sm_in = literal(t / "softmax_tensor_test.cpp", "input").reshape(2, 4)
    g["softmax_input"] = sm_in
    g["softmax_expected"] = ref.cpu_softmax_test(sm_in)
    ln_in = literal(t / "layernorm_tensor_test.cpp", "input").reshape(2, 4)
    g["layernorm_input"] = ln_in
    g["layernorm_expected"] = ref.cpu_layernorm(ln_in, 1e-5)

    # Seeded cases with the distributions of the reference's benchmark runs.
    rng = np.random.default_rng(42)
    x = rng.uniform(-1.0, 1.0, 4 * 1024).astype(np.float32)
    y = rng.uniform(-1.0, 1.0, 4 * 1024).astype(np.float32)
    g["seeded_add_a"], g["seeded_add_b"] = x, y
    g["seeded_add_expected"] = ref.cpu_vector_add(x, y)
    g["seeded_reduce_input"] = x
    g["seeded_reduce_interleave"] = ref.cpu_block_reduce(x, 0)
    g["seeded_reduce_address"] = ref.cpu_block_reduce(x, 1)
    act = np.concatenate([rng.normal(0.0, 3.0, 2000), [0.0, -0.0, 1e-30, -1e-30, 20.0, -20.0, 88.0, -88.0,
                                                        100.0, -100.0, np.inf, -np.inf]]).astype(np.float32)
    g["seeded_activation_input"] = act
    for op, name in enumerate(("relu", "leaky_relu", "gelu", "sigmoid", "tanh")):
        g["seeded_activation_" + name] = ref.cpu_activation(act, op, 0.01)
    sm = rng.uniform(-10.0, 10.0, (6, 1024)).astype(np.float32)
    g["seeded_softmax_input"] = sm
    g["seeded_softmax_bench"] = ref.cpu_softmax(sm)
    g["seeded_softmax_test"] = ref.cpu_softmax_test(sm)
    ln = rng.normal(0.0, 3.0, (6, 1024)).astype(np.float32)
    g["seeded_layernorm_input"] = ln
    g["seeded_layernorm_expected"] = ref.cpu_layernorm(ln, 1e-5)

    out = Path(__file__).with_name("reference_vectors.npz")
    np.savez_compressed(out, **g)
    print(out, out.stat().st_size, "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
