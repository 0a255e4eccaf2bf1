"""Autodiff graphs on the CPU side: golden vectors made by the reference's autodiff
(boat_var_attention, boat_var_add, boat_var_matmul, boat_var_dense, boat_var_mul, boat_var_sub,
boat_variable_backward) against the restatement of the pieces, and against the reference
library run live."""
import os

import numpy as np
import pytest

import cases
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def graph_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "graph_golden.npz"))


def test_residual_attention_graph_is_attention_plus_identity(graph_golden):
    case = cases.GRAPH_CASE
    inp = case.inputs()
    p = oracle.port_step(inp["q"], inp["q"], inp["q"], inp["w"], inp["b"], inp["dout"], case.nh, case.causal)
    assert np.array_equal(graph_golden["residual/out"], p["out"] + inp["q"])
    # x.grad = gout (through the add) + dq + dk + dv (through the attention op), summed in that order
    want = ((inp["dout"] + p["dq"]) + p["dk"]) + p["dv"]
    assert np.abs(graph_golden["residual/dx"] - want).max() <= 1e-6 * np.abs(want).max()
    for i, name in enumerate("qkvo"):
        assert np.array_equal(graph_golden["residual/dw" + name], p["dw"][i])
        assert np.array_equal(graph_golden["residual/db" + name], p["db"][i])


def test_mlp_graph_matches_float64_formulas(graph_golden):
    g = {k: v.astype(np.float64) for k, v in cases.graph_mlp_inputs().items()}
    h = g["a"] @ g["wm"]
    d = h @ g["wd"] + g["bd"]
    gd = g["gout"] * g["m"]
    want = {"out": d * g["m"] - g["c"], "dc": -g["gout"], "dm": g["gout"] * d, "dwd": h.T @ gd, "dbd": gd.sum(0),
            "dwm": g["a"].T @ (gd @ g["wd"].T), "da": (gd @ g["wd"].T) @ g["wm"].T}
    for key, ref in want.items():
        assert np.abs(graph_golden["mlp/" + key] - ref).max() <= 1e-5 * np.abs(ref).max(), key


@pytest.mark.skipif(not oracle.have_ref(), reason="reference library not built here")
def test_golden_graphs_equal_the_reference_library_live(graph_golden):
    case = cases.GRAPH_CASE
    inp = case.inputs()
    res = oracle.ref_graph_residual_attention(inp["q"], inp["w"], inp["b"], case.nh, case.causal, inp["dout"])
    assert np.array_equal(res["out"], graph_golden["residual/out"]) and np.array_equal(res["dx"], graph_golden["residual/dx"])
    g = cases.graph_mlp_inputs()
    res = oracle.ref_graph_mlp(g["a"], g["wm"], g["wd"], g["bd"], g["c"], g["m"], g["gout"])
    for key, val in res.items():
        assert np.array_equal(val, graph_golden["mlp/" + key]), key
