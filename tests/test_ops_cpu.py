"""The golden vectors of the generic tensor operations (made by the reference library, see
tests/golden/make_golden.py) against their plain definition in numpy, and - when the reference
library is built here - against the reference run live."""
import os

import numpy as np
import pytest

import cases
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ops_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "ops_golden.npz"))


def definitions(inp):
    f = np.float32
    return {
        "transpose_t4": inp["t4"].transpose(0, 1, 3, 2), "transpose_t4_ragged": inp["t4_ragged"].transpose(0, 1, 3, 2),
        "transpose_t2": inp["t2"].T, "add": inp["a"] + inp["b"], "add_bias": inp["a"] + inp["bias"],
        "mul": inp["a"] * inp["b"], "mul_scalar": inp["a"] * f(inp["scalar"]), "add_": inp["a"] + inp["b"],
        "sub_": inp["a"] - inp["b"],
        "matmul3": inp["m3a"].astype(np.float64) @ inp["m3b"].astype(np.float64),
        "matmul4": inp["m4a"].astype(np.float64) @ inp["m4b"].astype(np.float64),
    }


def test_golden_ops_are_what_the_definitions_say(ops_golden):
    want = definitions(cases.ops_inputs())
    assert set(ops_golden.files) == set(want)
    for key, w in want.items():
        g = ops_golden[key]
        assert g.shape == w.shape, key
        if key.startswith("matmul"):
            assert np.abs(g - w).max() <= 1e-5 * np.abs(w).max(), key      # FP32 sums in the reference's order
        else:
            assert np.array_equal(g, w), key                                # one rounding per element: exact


def test_reference_4d_transpose_case_is_in_the_golden_vectors(ops_golden):
    """The reference's own test fills [2,2,3,4] with 1..48 and swaps the last two dimensions."""
    t = ops_golden["transpose_t4"]
    assert t.shape == (2, 2, 4, 3)
    assert t[0, 0, 0, 1] == 5.0 and t[1, 1, 3, 2] == 48.0


@pytest.mark.skipif(not oracle.have_ref(), reason="reference library not built (no reference tree on this machine)")
def test_golden_ops_equal_the_reference_run_live(ops_golden):
    live = oracle.ref_ops(cases.ops_inputs())
    for key in ops_golden.files:
        assert np.array_equal(live[key], ops_golden[key]), key
