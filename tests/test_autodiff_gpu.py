"""Autodiff ops next to attention on the GPU through the C ABI (boat_var_add / sub / mul /
matmul / dense / attention + boat_variable_backward), with host and with CUDA tensors, against
golden vectors produced by the reference's own autodiff."""
import os

import numpy as np
import pytest

import cases
from boat_b200 import capi
from boat_b200.host import Attention, Dense, Tensor, Variable

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = 1e-5
DEVICES = pytest.mark.parametrize("device", [capi.DEVICE_CPU, capi.DEVICE_CUDA], ids=["host_tensors", "cuda_tensors"])


@pytest.fixture(scope="module")
def graph_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "graph_golden.npz"))


def rel(a, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.abs(np.asarray(a, np.float64) - ref).max() / np.abs(ref).max())


@DEVICES
def test_residual_attention_graph(gpu_lib, graph_golden, device):
    case = cases.GRAPH_CASE
    inp = case.inputs()
    layer = Attention(case.H, case.nh, causal=case.causal)
    layer.set_params(**{n: a for n, a in zip(Attention.PARAMS, list(inp["w"]) + list(inp["b"]))})
    if device == capi.DEVICE_CUDA:
        layer.to_device(device)
    layer.set_precision(capi.MMA_FP32)
    x = Variable(Tensor.from_numpy(inp["q"], device))
    r = x.attention(layer) + x
    assert r.data.device == device and r.data.shape == inp["q"].shape
    assert rel(r.data.numpy(), graph_golden["residual/out"]) <= TOL
    r.backward(Tensor.from_numpy(inp["dout"], device))
    assert x.grad.device == device
    assert rel(x.grad.numpy(), graph_golden["residual/dx"]) <= TOL
    scale = max(np.abs(graph_golden["residual/db" + p]).max() for p in "qkvo")
    for p in "qkvo":
        assert rel(layer.param("grad_weight_" + p).numpy(), graph_golden["residual/dw" + p]) <= TOL
        got, want = layer.param("grad_bias_" + p).numpy(), graph_golden["residual/db" + p]
        assert np.abs(got - want).max() <= TOL * scale          # the key bias gradient is zero in exact arithmetic


@DEVICES
def test_matmul_dense_mul_sub_graph(gpu_lib, graph_golden, device):
    g = cases.graph_mlp_inputs()
    dense = Dense(g["wd"].shape[0], g["wd"].shape[1], g["wd"], g["bd"], device=device)
    leaf = {k: Variable(Tensor.from_numpy(g[k], device)) for k in ("a", "wm", "m", "c")}
    z = (leaf["a"] @ leaf["wm"]).dense(dense) * leaf["m"] - leaf["c"]
    assert z.data.device == device
    assert rel(z.data.numpy(), graph_golden["mlp/out"]) <= TOL
    z.backward(Tensor.from_numpy(g["gout"], device))
    for name, key in (("a", "da"), ("wm", "dwm"), ("m", "dm"), ("c", "dc")):
        assert leaf[name].grad.device == device
        assert rel(leaf[name].grad.numpy(), graph_golden["mlp/" + key]) <= TOL, key
    dw, db = dense.grads()
    assert rel(dw, graph_golden["mlp/dwd"]) <= TOL and rel(db, graph_golden["mlp/dbd"]) <= TOL


def test_gradients_accumulate_and_untracked_inputs_get_none(gpu_lib):
    a = Variable(Tensor.from_numpy(np.full((4, 4), 2.0, np.float32), capi.DEVICE_CUDA))
    b = Variable(Tensor.from_numpy(np.full((4, 4), 3.0, np.float32), capi.DEVICE_CUDA), requires_grad=False)
    y = a * b + a                                     # dy/da = b + 1
    y.backward()                                      # gradient of ones
    assert np.array_equal(a.grad.numpy(), np.full((4, 4), 4.0, np.float32))
    # A second backward without zeroing: the intermediate a*b keeps its gradient (1 -> 2) and
    # hands all of it on again, so a.grad = 4 + 1 + 2*3 = 11 - the reference's library gives
    # exactly this (its intermediates are never cleared either).
    y.backward()
    assert np.array_equal(a.grad.numpy(), np.full((4, 4), 11.0, np.float32))
    assert b.grad is None
    c = Variable(Tensor.from_numpy(np.ones((4, 4), np.float32), capi.DEVICE_CUDA), requires_grad=False)
    d = Variable(Tensor.from_numpy(np.ones((4, 4), np.float32), capi.DEVICE_CUDA), requires_grad=False)
    z = c - d
    z.backward()                                      # nothing requires a gradient: a no-op
    assert c.grad is None and d.grad is None
