"""Adam on the GPU through the C ABI (boat/optimizers.h and boat_cuda_adam_step): the bits must
equal the reference's, i.e. the committed golden vectors and the CPU restatement, for host and
CUDA parameter tensors, ragged sizes and long lists; plus the optimizer driving the attention
layer, and the reference's own unit-test program linked against this library."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import cases
from boat_b200 import capi, rng
from boat_b200.host import Adam, Attention, Tensor
from oracle import oracle

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def adam_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "adam_golden.npz"))


def run_steps(params, grads, hyper, device):
    opt = Adam(hyper["lr"], hyper["beta1"], hyper["beta2"], hyper["eps"])
    ps = [Tensor.from_numpy(p, device) for p in params]
    gs = [Tensor.from_numpy(np.zeros_like(p), device) for p in params]
    for p, g in zip(ps, gs):
        opt.add(p, g)
    after = []
    for step in grads:
        for g, a in zip(gs, step):
            g.set(a)
        opt.step()
        after.append([p.numpy() for p in ps])
    opt.free()
    return after


@pytest.mark.parametrize("device", [capi.DEVICE_CPU, capi.DEVICE_CUDA], ids=["host_tensors", "cuda_tensors"])
def test_every_step_is_bit_identical_to_the_reference_golden(gpu_lib, adam_golden, device):
    params, grads = cases.adam_inputs()
    after = run_steps(params, grads, cases.ADAM_HYPER, device)
    for s, ps in enumerate(after, start=1):
        for i, p in enumerate(ps):
            assert np.array_equal(p.reshape(-1), adam_golden["step%d/p%d" % (s, i)].reshape(-1)), (s, i)


def test_long_list_and_odd_sizes_equal_the_restatement(gpu_lib):
    # 61 tensors: more than one launch table; sizes around the chunk and vector boundaries
    sizes = [1, 2, 3, 4, 5, 4095, 4096, 4097, 8191, 8192, 12289] + [37 * (i + 1) for i in range(50)]
    params, grads = cases.adam_inputs(shapes=tuple((n,) for n in sizes), steps=3, stream=300)
    hyper = dict(lr=0.003, beta1=0.85, beta2=0.995, eps=1e-7)
    got = run_steps(params, grads, hyper, capi.DEVICE_CUDA)[-1]
    want = oracle.port_adam(params, grads, **hyper)
    for a, b in zip(got, want):
        assert np.array_equal(a, b)


def test_unaligned_views_take_the_scalar_path(gpu_lib):
    """boat_cuda_adam_step on pointers that are only 4-byte aligned."""
    from boat_b200.host import DeviceBuffer
    n = 10000
    p0, g0 = rng.normal(7, 1, (n + 1,)), rng.normal(7, 2, (n + 1,), 0.3)
    bufs = [DeviceBuffer.from_numpy(a) for a in (p0, g0, np.zeros(n + 1, np.float32), np.zeros(n + 1, np.float32))]
    ptrs = [(C.c_void_p * 1)(b.p.value + 4) for b in bufs]
    lens = (C.c_int64 * 1)(n)
    h = cases.ADAM_HYPER
    corr1 = np.float32(1.0) - np.float32(h["beta1"])
    corr2 = np.float32(1.0) - np.float32(h["beta2"])
    rc = gpu_lib.boat_cuda_adam_step(1, ptrs[0], ptrs[1], ptrs[2], ptrs[3], lens, h["lr"], h["beta1"], h["beta2"],
                                     h["eps"], float(corr1), float(corr2))
    assert rc == 0, gpu_lib.boat_cuda_last_error()
    got = bufs[0].numpy((n + 1,))
    want = oracle.port_adam([p0[1:]], [[g0[1:]]], **h)[0]
    assert got[0] == p0[0]                       # the element before the view is untouched
    assert np.array_equal(got[1:], want)


def test_zero_grad_and_learning_rate(gpu_lib):
    p = Tensor.from_numpy(np.ones(100, np.float32), capi.DEVICE_CUDA)
    g = Tensor.from_numpy(np.full(100, 0.5, np.float32), capi.DEVICE_CUDA)
    hg = Tensor.from_numpy(np.full(10, 0.5, np.float32))
    hp = Tensor.from_numpy(np.ones(10, np.float32))
    opt = Adam(0.01)
    opt.add(p, g)
    opt.add(hp, hg)
    opt.zero_grad()
    assert not g.numpy().any() and not hg.numpy().any()
    opt.step()                                   # zero gradient: m = v = 0, update 0 / (0 + eps) = 0
    assert np.array_equal(p.numpy(), np.ones(100, np.float32))
    opt.lr = 0.25
    assert opt.lr == 0.25
    opt.free()


def test_rejects_non_fp32_and_mismatched_pairs(gpu_lib, capfd):
    opt = Adam(0.01)
    a = Tensor.from_numpy(np.ones(8, np.float32), capi.DEVICE_CUDA)
    b = Tensor.from_numpy(np.ones(9, np.float32), capi.DEVICE_CUDA)
    h = Tensor.from_numpy(np.ones(8, np.float32), capi.DEVICE_CUDA, bf16=True)
    before = a.numpy()
    opt.add(a, b)
    opt.add(h, h)
    opt.step()
    assert np.array_equal(a.numpy(), before)     # nothing was registered
    assert "FP32" in capfd.readouterr().err
    opt.free()


def test_adam_drives_the_attention_layer_like_the_restatement(gpu_lib):
    """forward + backward on the GPU (FP32 path), then Adam over the layer's eight parameters,
    twice; against the CPU restatement of both (attention within its FP32 tolerance, so the
    comparison after Adam is a tolerance too, scaled by the learning rate)."""
    case = cases.Case("adam_layer", B=2, S=24, H=32, nh=4, causal=True)
    inp = case.inputs()
    layer = Attention(case.H, case.nh, causal=True)
    layer.set_params(**{n: a for n, a in zip(Attention.PARAMS, list(inp["w"]) + list(inp["b"]))})
    layer.to_device(capi.DEVICE_CUDA)
    layer.set_precision(capi.MMA_FP32)
    opt = Adam(**{"lr": 0.01, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8})
    opt.add_attention(layer)
    grad_ptr = layer.param("grad_weight_q").data_ptr
    w, b = [a.copy() for a in inp["w"]], [a.copy() for a in inp["b"]]
    dev = lambda a: Tensor.from_numpy(a, capi.DEVICE_CUDA)
    history = []
    for _ in range(2):
        layer.forward(dev(inp["q"]), dev(inp["k"]), dev(inp["v"]))
        layer.backward(dev(inp["dout"]))
        assert layer.param("grad_weight_q").data_ptr == grad_ptr      # stable gradient tensors
        opt.step()
        res = oracle.port_step(inp["q"], inp["k"], inp["v"], w, b, inp["dout"], case.nh, True)
        history.append([res["dw"][i] for i in range(4)] + [res["db"][i] for i in range(4)])
        # run the restatement's Adam from the start each time (it keeps no state between calls)
        new = oracle.port_adam(list(inp["w"]) + list(inp["b"]), history, lr=0.01, beta1=0.9, beta2=0.999, eps=1e-8)
        w, b = new[:4], new[4:]
    for name, want, start in zip(Attention.PARAMS, w + b, list(inp["w"]) + list(inp["b"])):
        got = layer.param(name).numpy()
        moved = np.abs(want - start).max()
        assert moved > 0
        # each Adam step moves an entry by at most ~lr; a tiny gradient difference can flip
        # the direction only where the gradient is ~0 (the key bias), hence the lr-sized bound
        assert np.abs(got.reshape(-1) - want.reshape(-1)).max() <= (2.1 * 0.01 if name == "bias_k" else 2e-4), name
    opt.free()
    layer.free()


def test_reference_adam_test_program(gpu_lib, tmp_path):
    path = os.path.join(ROOT, "oracle", "_ref", "dropin_test_optimizer_adam")
    if not os.path.exists(path):
        pytest.skip("not built (needs the reference source tree at build time)")
    proc = subprocess.run([path], cwd=str(tmp_path), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                          timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:]
    assert "All Adam optimizer tests passed" in proc.stdout
