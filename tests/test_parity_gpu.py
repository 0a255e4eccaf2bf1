"""GPU parity: the CUDA path, called through the C ABI, against the reference's golden
vectors and against the CPU restatement on seeded inputs.

Tolerances (max|ours - ref| / max|ref| per tensor):
  exact FP32 path   1e-5   (summation order differs from the reference, nothing else)
  TF32 tensor cores 5e-3
  BF16 tensor cores 2e-2
"""
import numpy as np
import pytest

import cases
from boat_b200 import capi, rng
from gpu_driver import gpu_step
from oracle import oracle

pytestmark = pytest.mark.gpu

TOL_FP32, TOL_TF32, TOL_BF16 = 1e-5, 5e-3, 2e-2


def assert_close(res, ref, tol, what):
    flat, fref = cases.flatten_result(res), cases.flatten_result(ref)
    for key, r in fref.items():
        assert flat[key].shape == r.shape, (what, key)
        assert np.isfinite(flat[key]).all(), (what, key, "non-finite values")
    worst = cases.errors(flat, fref)
    bad = {k: v for k, v in worst.items() if v > tol}
    assert not bad, "%s: relative error above %g: %s (all: %s)" % (what, tol, bad, worst)


@pytest.mark.parametrize("device", [capi.DEVICE_CPU, capi.DEVICE_CUDA], ids=["host_tensors", "cuda_tensors"])
@pytest.mark.parametrize("case", cases.GOLDEN_CASES, ids=lambda c: c.name)
def test_fp32_path_matches_reference_golden(gpu_lib, golden, case, device):
    inp = case.inputs()
    res = gpu_step(inp, case.nh, case.causal, device=device, precision=capi.MMA_FP32)
    ref = {k.split("/", 1)[1]: golden[k] for k in golden.files if k.startswith(case.name + "/") and "digest" not in k}
    worst = cases.errors(cases.flatten_result(res), ref)
    bad = {k: v for k, v in worst.items() if v > TOL_FP32}
    assert not bad, "%s: %s" % (case.name, bad)


@pytest.mark.parametrize("shape", [(1, 1, 8, 1), (2, 3, 24, 3), (1, 65, 32, 2), (2, 130, 64, 4), (1, 200, 256, 2),
                                   (1, 257, 128, 1)])
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
def test_fp32_path_matches_restatement_on_ragged_shapes(gpu_lib, shape, causal):
    B, S, H, nh = shape
    case = cases.Case("ragged", B, S, H, nh, causal=causal, self_attn=False, bias_std=0.1)
    inp = case.inputs()
    ref = oracle.port_step(inp["q"], inp["k"], inp["v"], inp["w"], inp["b"], inp["dout"], nh, causal)
    res = gpu_step(inp, nh, causal, device=capi.DEVICE_CUDA, precision=capi.MMA_FP32)
    assert_close(res, ref, TOL_FP32, str(shape))


def test_self_attention_sums_into_one_gradient_through_autodiff(gpu_lib):
    """boat_var_attention + boat_variable_backward: one variable passed as query, key and
    value ends with dq + dk + dv in its .grad."""
    import ctypes as C
    from boat_b200.host import Attention, Tensor
    case = cases.Case("autodiff", 2, 16, 32, 4, causal=True, bias_std=0.1)
    inp = case.inputs()
    ref = oracle.port_step(inp["q"], inp["q"], inp["q"], inp["w"], inp["b"], inp["dout"], 4, True)
    lib = gpu_lib
    layer = Attention(32, 4, causal=True)
    for i, p in enumerate("qkvo"):
        layer.param("weight_" + p).set(inp["w"][i])
        layer.param("bias_" + p).set(inp["b"][i])
    layer.set_precision(capi.MMA_FP32)
    x = Tensor.from_numpy(inp["q"])
    var = C.c_void_p(lib.boat_variable_create(x.h, True))
    out = C.c_void_p(lib.boat_var_attention(var, var, var, layer.h, None))
    assert out.value
    g = Tensor.from_numpy(inp["dout"])
    lib.boat_variable_backward(out, g.h)
    grad = Tensor(lib.boat_variable_grad(var), own=False).numpy()
    want = ref["dq"] + ref["dk"] + ref["dv"]
    assert cases.rel_err(grad, want) <= TOL_FP32
    assert cases.rel_err(Tensor(lib.boat_variable_data(out), own=False).numpy(), ref["out"]) <= TOL_FP32
    lib.boat_variable_free(out)
    lib.boat_variable_free(var)
    layer.free()


def test_sgd_update_is_bit_exact(gpu_lib):
    case = cases.GOLDEN_CASES[1]
    inp = case.inputs()
    for device in (capi.DEVICE_CPU, capi.DEVICE_CUDA):
        res = gpu_step(inp, case.nh, case.causal, device=device, precision=capi.MMA_FP32, lr=0.01)
        for i in range(4):
            assert np.array_equal(res["w_after"][i], oracle.port_sgd(inp["w"][i], res["dw"][i], 0.01))
            assert np.array_equal(res["b_after"][i], oracle.port_sgd(inp["b"][i], res["db"][i], 0.01))


def test_reference_training_loop_losses(gpu_lib):
    """The reference's training test (5 steps, lr 0.01) through our library prints the same
    losses as the reference does: 0.324671 ... 0.324215."""
    import ctypes
    from boat_b200.host import Attention, Tensor
    libc = ctypes.CDLL(None)
    libc.rand.restype = ctypes.c_int
    f32 = np.float32
    draw = lambda: f32(f32(libc.rand()) / f32(2147483647))
    libc.srand(1)
    layer = Attention(32, 4, head_size=8)           # draws its weights from rand(), like the reference
    libc.srand(42)
    n = 2 * 4 * 32
    q, k, v = np.empty(n, f32), np.empty(n, f32), np.empty(n, f32)
    for i in range(n):
        q[i] = draw() * f32(2) - f32(1)
        k[i] = draw() * f32(2) - f32(1)
        v[i] = draw() * f32(2) - f32(1)
    target = np.array([draw() * f32(2) - f32(1) for _ in range(n)], dtype=f32)
    tq, tk, tv = (Tensor.from_numpy(a.reshape(2, 4, 32)) for a in (q, k, v))
    losses = []
    for _ in range(5):
        out = layer.forward(tq, tk, tv)
        diff = out.numpy().ravel() - target
        losses.append(float(np.mean(diff.astype(np.float64) ** 2)))
        g = Tensor.from_numpy((f32(2) * diff / f32(n)).reshape(2, 4, 32))
        layer.backward(g)
        layer.update(0.01)
    assert np.allclose(losses, [0.324671, 0.324557, 0.324443, 0.324329, 0.324215], atol=2e-6), losses
    dwq = layer.param("grad_weight_q").numpy().ravel()
    assert abs(float(np.abs(dwq[:10]).sum()) - 0.002070) < 2e-6
    layer.free()


def test_error_behaviour_matches_reference(gpu_lib):
    import ctypes as C
    from boat_b200.host import Attention, Tensor
    lib = gpu_lib
    cfg = capi.AttentionConfig(30, 4, 0, 0.0, False, True, False, 10000.0)
    assert not lib.boat_attention_create(C.byref(cfg))            # 30 % 4 != 0
    assert not lib.boat_attention_create(None)
    layer = Attention(32, 4)
    x = Tensor.from_numpy(np.zeros((2, 4, 32), np.float32))
    assert not lib.boat_attention_forward(layer.h, None, x.h, x.h, None)
    assert not lib.boat_attention_forward(None, x.h, x.h, x.h, None)
    g = Tensor.from_numpy(np.ones((2, 4, 32), np.float32))
    gq = C.c_void_p()
    assert lib.boat_attention_backward(layer.h, g.h, C.byref(gq), None, None) is False   # no forward yet
    assert lib.boat_attention_get_grad_weight_q(layer.h) is None                       # NULL before backward
    bad = Tensor.from_numpy(np.zeros((2, 4, 16), np.float32))
    assert not lib.boat_attention_forward(layer.h, bad.h, bad.h, bad.h, None)           # wrong hidden size
    out = layer.forward(x)
    assert lib.boat_attention_backward(layer.h, g.h, None, None, None) is True          # NULL out-params tolerated
    assert lib.boat_attention_get_grad_weight_q(layer.h) is not None
    layer.free()


def test_scaled_dot_product_attention_entry_point(gpu_lib):
    import ctypes as C
    from boat_b200.host import Tensor
    lib = gpu_lib
    case = cases.Case("sdpa", 2, 19, 24, 3, self_attn=False)
    inp = case.inputs()
    shp = (2, 3, 19, 8)
    q, k, v = (inp[n].reshape(shp) for n in "qkv")
    for causal in (False, True):
        ref = oracle.port_core(q.reshape(6, 19, 8), k.reshape(6, 19, 8), v.reshape(6, 19, 8), None, causal, 0.3)
        tq, tk, tv = (Tensor.from_numpy(a) for a in (q, k, v))
        out = Tensor(lib.boat_scaled_dot_product_attention(tq.h, tk.h, tv.h, 0.3, None, causal, 0.0))
        assert out.shape == shp
        assert cases.rel_err(out.numpy().reshape(6, 19, 8), ref["o"]) <= TOL_FP32
    t3 = Tensor.from_numpy(inp["v"])                                       # 3-D: copy of value
    out = Tensor(lib.boat_scaled_dot_product_attention(t3.h, t3.h, t3.h, 1.0, None, False, 0.0))
    assert np.array_equal(out.numpy(), inp["v"])


# ---- tensor-core paths of the whole layer -----------------------------------------------------------

TC_CASES = [
    # name, B, S, H, nh, causal
    ("hs64_full", 2, 256, 256, 4, False),
    ("hs64_causal", 2, 384, 256, 4, True),
    ("hs128_causal", 1, 256, 256, 2, True),
    ("hs64_long", 1, 1024, 128, 2, True),
]


@pytest.mark.parametrize("name,B,S,H,nh,causal", TC_CASES, ids=[c[0] for c in TC_CASES])
@pytest.mark.parametrize("device", [capi.DEVICE_CPU, capi.DEVICE_CUDA], ids=["host_tensors", "cuda_tensors"])
def test_bf16_tensor_core_path_matches_restatement(gpu_lib, name, B, S, H, nh, causal, device):
    case = cases.Case(name, B, S, H, nh, causal=causal, bias_std=0.1)
    inp = case.inputs(bf16=True)           # both sides start from the BF16-rounded values
    ref = oracle.port_step(inp["q"], inp["k"], inp["v"], inp["w"], inp["b"], inp["dout"], nh, causal)
    res = gpu_step(inp, nh, causal, device=device, precision=capi.MMA_BF16, bf16=True)
    assert_close(res, ref, TOL_BF16, name)


@pytest.mark.parametrize("name,B,S,H,nh,causal", [c for c in TC_CASES if c[3] // c[4] == 64], ids=lambda v: str(v))
def test_tf32_tensor_core_path_matches_restatement(gpu_lib, name, B, S, H, nh, causal):
    case = cases.Case(name, B, S, H, nh, causal=causal, bias_std=0.1)
    inp = case.inputs()
    ref = oracle.port_step(inp["q"], inp["k"], inp["v"], inp["w"], inp["b"], inp["dout"], nh, causal)
    res = gpu_step(inp, nh, causal, device=capi.DEVICE_CUDA, precision=capi.MMA_TF32)
    assert_close(res, ref, TOL_TF32, name)


def test_fp32_inputs_with_bf16_arithmetic(gpu_lib):
    """FP32 tensors in, BF16 tensor cores inside, FP32 tensors out."""
    case = cases.Case("mixed", 1, 256, 128, 2, causal=True)
    inp = case.inputs(bf16=True)
    ref = oracle.port_step(inp["q"], inp["k"], inp["v"], inp["w"], inp["b"], inp["dout"], 2, True)
    res = gpu_step(inp, 2, True, device=capi.DEVICE_CUDA, precision=capi.MMA_BF16, bf16=False)
    assert_close(res, ref, TOL_BF16, "mixed")


def test_automatic_precision_keeps_fp32_tensors_exact_at_tensor_core_shapes(gpu_lib):
    """Without an explicit choice FP32 tensors are computed in exact FP32 even where the shape
    would suit the tensor cores (S a multiple of 128, head size 64): a reference program's
    numbers do not change with the sequence length.  BF16 tensors select BF16 arithmetic."""
    case = cases.Case("auto", 1, 256, 128, 2)
    inp = case.inputs()
    ref = oracle.port_step(inp["q"], inp["k"], inp["v"], inp["w"], inp["b"], inp["dout"], 2, False)
    res = gpu_step(inp, 2, False, device=capi.DEVICE_CUDA, precision=-1)
    assert_close(res, ref, TOL_FP32, "auto, fp32 tensors")
    inp = case.inputs(bf16=True)
    ref = oracle.port_step(inp["q"], inp["k"], inp["v"], inp["w"], inp["b"], inp["dout"], 2, False)
    res = gpu_step(inp, 2, False, device=capi.DEVICE_CUDA, precision=-1, bf16=True)
    assert_close(res, ref, TOL_BF16, "auto, bf16 tensors")


# ---- host tensors travel in overlapped chunks of batch entries: same numbers as in one piece --------------

@pytest.mark.parametrize("B,S,H,nh,precision,bf16,self_attn", [
    (10, 128, 128, 2, capi.MMA_BF16, True, True),      # 10 entries in 8 chunks: uneven chunk sizes
    (3, 256, 256, 2, capi.MMA_BF16, True, False),      # fewer entries than chunks; distinct q, k, v (three uploads)
    (9, 128, 128, 2, capi.MMA_TF32, False, True),      # FP32 host tensors, TF32 rounding per chunk
    (5, 40, 48, 3, capi.MMA_FP32, False, False),       # exact path, ragged shape
], ids=["bf16_10x128", "bf16_3x256_qkv", "tf32_9x128", "fp32_5x40_qkv"])
def test_chunked_host_path_equals_the_device_path(gpu_lib, B, S, H, nh, precision, bf16, self_attn):
    case = cases.Case("chunks", B, S, H, nh, causal=True, self_attn=self_attn, bias_std=0.1)
    inp = case.inputs(bf16=bf16)
    host = gpu_step(inp, nh, True, device=capi.DEVICE_CPU, precision=precision, bf16=bf16)
    dev = gpu_step(inp, nh, True, device=capi.DEVICE_CUDA, precision=precision, bf16=bf16)
    fh, fd = cases.flatten_result(host), cases.flatten_result(dev)
    for key in fd:
        if key.startswith(("dw", "db")):
            # sums over all rows: computed once over all rows in both paths, but their kernels
            # combine partial sums with atomics, whose order varies from launch to launch
            assert np.abs(fh[key] - fd[key]).max() <= 1e-5 * np.abs(fd[key]).max(), key
        else:
            # per-row arithmetic is the same in both paths
            assert np.array_equal(fh[key], fd[key]), key


@pytest.mark.parametrize("precision,bf16,tol", [(capi.MMA_BF16, True, TOL_BF16), (capi.MMA_TF32, False, TOL_TF32)],
                         ids=["bf16", "tf32"])
def test_cuda_layer_sees_every_weight_change(gpu_lib, precision, bf16, tol):
    """A CUDA layer keeps tensor-core copies of its FP32 weights from a forward to the backward of
    the same step.  Each way the weights can change - an SGD update, writing a weight tensor fetched
    through an accessor (also between forward and backward), moving the layer - must show in the
    next result as it does in the restatement run with the changed weights."""
    from boat_b200.host import Attention, Tensor
    B, S, H, nh = 1, 256, 128, 2
    case = cases.Case("shadow", B, S, H, nh, causal=True, bias_std=0.1)
    inp = case.inputs(bf16=bf16)
    names = ["weight_q", "weight_k", "weight_v", "weight_o"]
    layer = Attention(H, nh, causal=True, use_bias=True)
    for i, n in enumerate(names):
        layer.param(n).set(inp["w"][i])
    for i, p in enumerate("qkvo"):
        layer.param("bias_" + p).set(inp["b"][i])
    layer.to_device(capi.DEVICE_CUDA)
    layer.set_precision(precision)
    x = Tensor.from_numpy(inp["q"], capi.DEVICE_CUDA, bf16=bf16)
    g = Tensor.from_numpy(inp["dout"], capi.DEVICE_CUDA, bf16=bf16)

    def ours():
        out = layer.forward(x, x, x)
        gq, gk, gv = layer.backward(g)
        res = {"out": out.numpy(), "dq": gq.numpy(), "dk": gk.numpy(), "dv": gv.numpy(),
               "dw": [layer.param("grad_" + n).numpy() for n in names],
               "db": [layer.param("grad_bias_" + p).numpy() for p in "qkvo"]}
        return res

    def theirs(w, b):
        # the layer rounds its FP32 weights to the arithmetic's format at every forward
        wr = [rng.bf16_round(x) for x in w] if bf16 else w
        return oracle.port_step(inp["q"], inp["q"], inp["q"], wr, b, inp["dout"], nh, True)

    w = [a.copy() for a in inp["w"]]
    b = [a.copy() for a in inp["b"]]
    first = ours()
    assert_close(first, theirs(w, b), tol, "first step")
    # an SGD update that moves the weights by up to a third of their size
    lr = np.float32(0.33 * max(np.abs(x).max() for x in w) / max(np.abs(g).max() for g in first["dw"]))
    layer.update(float(lr))
    w = [wi - lr * gi for wi, gi in zip(w, first["dw"])]
    b = [bi - lr * gi for bi, gi in zip(b, first["db"])]
    second = ours()
    assert_close(second, theirs(w, b), tol, "after update")
    assert cases.rel_err(second["out"], first["out"]) > 2 * tol      # the change is visible at all
    # a weight written between forward and backward: the backward must use the new values
    out = layer.forward(x, x, x)
    w[3] = np.ascontiguousarray(w[3][::-1] * np.float32(0.5)).astype(np.float32)
    layer.param("weight_o").set(w[3])
    gq, gk, gv = layer.backward(g)
    ref = theirs(w, b)
    assert cases.rel_err(gq.numpy(), ref["dq"]) <= tol
    assert cases.rel_err(layer.param("grad_weight_q").numpy(), ref["dw"][0]) <= tol
    # moving the layer to the host and back keeps working
    layer.to_device(capi.DEVICE_CPU)
    layer.to_device(capi.DEVICE_CUDA)
    third = ours()
    assert_close(third, theirs(w, b), tol, "after moving the layer")
    layer.free()
