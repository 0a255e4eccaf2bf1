"""safetensors loader on the GPU: parameters land transposed ([out,in] -> Boat's [in,out]) in host
and in CUDA layers, for F32 / BF16 / F16 checkpoints, and the loaded layer computes what the CPU
restatement computes with the same weights."""
import numpy as np
import pytest

import cases
import safetensors_util as st
from boat_b200 import capi, rng
from boat_b200.host import Attention, Tensor
from oracle import oracle

pytestmark = pytest.mark.gpu


def stored(a, dtype):
    """The value a tensor has after being written in `dtype`."""
    if dtype == "BF16":
        return rng.bf16_round(a)
    if dtype == "F16":
        return a.astype(np.float16).astype(np.float32)
    return a


@pytest.mark.parametrize("dtype", ["F32", "BF16", "F16"])
@pytest.mark.parametrize("device", [capi.DEVICE_CPU, capi.DEVICE_CUDA], ids=["host_layer", "cuda_layer"])
def test_parameters_are_loaded_transposed_and_exact(gpu_lib, dtype, device, tmp_path):
    H = 48
    tensors, want = st.bert_style(H, dtype=dtype)
    layer = Attention(H, 4)
    if device == capi.DEVICE_CUDA:
        layer.to_device(device)
    path = tmp_path / "model.safetensors"
    path.write_bytes(st.image(tensors, dtype=dtype, metadata={"format": "pt"}))
    assert layer.load_safetensors(path, prefix="encoder.layer.0.") == 0
    for name, ref in want.items():
        got = layer.param(name)
        assert got.device == device
        assert np.array_equal(got.numpy(), stored(ref, dtype)), name
    layer.free()


def test_prefix_selects_one_of_several_layers_and_missing_biases_keep_their_values(gpu_lib):
    H = 32
    tensors, _ = st.bert_style(H, seed=3, prefix="encoder.layer.0.")
    second, want = st.bert_style(H, seed=4, prefix="encoder.layer.1.", with_bias=False, extra=False)
    tensors.update(second)
    layer = Attention(H, 4)
    layer.param("bias_q").set(np.full(H, 0.25, np.float32))
    assert layer.load_safetensors(st.image(tensors), prefix="encoder.layer.1.") == 0
    for name, ref in want.items():
        assert np.array_equal(layer.param(name).numpy(), ref), name
    assert np.array_equal(layer.param("bias_q").numpy(), np.full(H, 0.25, np.float32))
    layer.free()


def test_loaded_layer_computes_what_the_restatement_computes(gpu_lib):
    case = cases.Case("st", B=2, S=16, H=32, nh=4, causal=True)
    tensors, want = st.bert_style(case.H, seed=5)
    layer = Attention(case.H, case.nh, causal=True)
    layer.to_device(capi.DEVICE_CUDA)
    layer.set_precision(capi.MMA_FP32)
    assert layer.load_safetensors(st.image(tensors)) == 0
    x = rng.normal(5, 50, (case.B, case.S, case.H))
    out = layer.forward(Tensor.from_numpy(x, capi.DEVICE_CUDA)).numpy()
    w = [np.ascontiguousarray(want["weight_" + p]) for p in "qkvo"]
    b = [want["bias_" + p] for p in "qkvo"]
    ref = oracle.port_step(x, x, x, w, b, None, case.nh, True)["out"]
    assert np.abs(out - ref).max() <= 1e-5 * np.abs(ref).max()
    layer.free()
