"""CPU tests of the checker for the layers around attention: pinned parts against the
reference's golden vectors, unpinned parts (the reference has only stubs) against central
differences of their own forward."""
import numpy as np
import pytest

import cases
from oracle import oracle


def test_layernorm_forward_reproduces_reference_golden(golden):
    ln = cases.layernorm_inputs()
    assert np.array_equal(oracle.port_layernorm(ln["x"], ln["w"], ln["b"], ln["eps"]), golden["layernorm/y"])
    assert np.array_equal(oracle.port_layernorm(ln["x"], None, None, ln["eps"]), golden["layernorm/y_plain"])


def test_dense_forward_and_accumulating_backward_reproduce_reference_golden(golden):
    de = cases.dense_inputs()
    assert np.array_equal(oracle.port_dense(de["x"], de["w"], de["b"]), golden["dense/y"])
    dx, dw, db = oracle.port_dense_backward(de["x"], de["w"], de["dy"])
    dx, dw, db = oracle.port_dense_backward(de["x"], de["w"], de["dy"], dw, db)      # second call accumulates
    assert np.array_equal(dx, golden["dense/dx"])
    assert np.array_equal(dw, golden["dense/dw"]) and np.array_equal(db, golden["dense/db"])


@pytest.mark.skipif(not oracle.have_ref(), reason="reference library not built on this machine")
def test_layernorm_and_dense_equal_reference_library_live():
    ln = cases.layernorm_inputs((2, 5), 32)
    assert np.array_equal(oracle.port_layernorm(ln["x"], ln["w"], ln["b"], 1e-6), oracle.ref_layernorm(ln["x"], ln["w"], ln["b"], 1e-6))
    de = cases.dense_inputs(7, 16, 8)
    ref = oracle.ref_dense_step(de["x"], de["w"], None, de["dy"])
    dx, dw, _ = oracle.port_dense_backward(de["x"], de["w"], de["dy"], bias=False)
    assert np.array_equal(oracle.port_dense(de["x"], de["w"], None), ref["y"])
    assert np.array_equal(dx, ref["dx"]) and np.array_equal(dw, ref["dw"])


def _fd(f, x, dy, eps=1e-3):
    """d/dx of sum(f(x) * dy) by central differences in float64-evaluated float32 forward."""
    g = np.zeros(x.size, np.float64)
    flat = x.ravel()
    for i in range(x.size):
        old = flat[i]
        flat[i] = old + eps
        up = float((f(x).astype(np.float64) * dy).sum())
        flat[i] = old - eps
        dn = float((f(x).astype(np.float64) * dy).sum())
        flat[i] = old
        g[i] = (up - dn) / (2 * eps)
    return g.reshape(x.shape)


def test_layernorm_backward_matches_finite_differences():
    """Parity unpinned (reference stub): the analytic backward against differences of the
    pinned forward."""
    ln = cases.layernorm_inputs((2, 3), 12)
    x, w, b, dy = ln["x"].copy(), ln["w"], ln["b"], ln["dy"].astype(np.float64)
    dx, dg, db = oracle.port_layernorm_backward(ln["dy"], x, w, ln["eps"])
    fd_x = _fd(lambda a: oracle.port_layernorm(a, w, b, ln["eps"]), x, dy)
    assert np.abs(dx - fd_x).max() <= 2e-3 * np.abs(fd_x).max()
    wv = w.copy()
    fd_w = _fd(lambda a: oracle.port_layernorm(x, a, b, ln["eps"]), wv, dy)
    assert np.abs(dg - fd_w).max() <= 2e-3 * np.abs(fd_w).max()
    assert np.allclose(db, ln["dy"].reshape(-1, 12).sum(0), rtol=1e-5, atol=1e-6)


def test_gelu_matches_definition_and_finite_differences():
    x = np.linspace(-6, 6, 241).astype(np.float32)
    y = oracle.port_gelu(x)
    from math import erf, sqrt
    want = np.array([0.5 * v * (1 + erf(v / sqrt(2))) for v in x.astype(np.float64)])
    assert np.abs(y - want).max() <= 1e-6
    dy = np.ones_like(x)
    g = oracle.port_gelu_backward(dy, x)
    h = 1e-4
    fd = np.array([(0.5 * (v + h) * (1 + erf((v + h) / sqrt(2))) - 0.5 * (v - h) * (1 + erf((v - h) / sqrt(2)))) / (2 * h)
                   for v in x.astype(np.float64)])
    assert np.abs(g - fd).max() <= 1e-5
