"""boat_attention_forward_units: one fixed [B,S,H] problem split over contiguous ranges of
(batch, head) units, each range given only its own token rows - the split the strong-scaling
benchmark runs over GPUs.  Here the ranges run one after the other on one GPU; their outputs and
input gradients must be the owned rows of the full step, and their parameter gradients must add
up to the full step's (the sum the multi-GPU path does with one all-reduce)."""
import numpy as np
import pytest

import cases
from boat_b200 import capi, shard
from boat_b200.host import Attention, Tensor
from oracle import oracle

pytestmark = pytest.mark.gpu

NAMES = ["weight_q", "weight_k", "weight_v", "weight_o"]


def make_layer(inp, H, nh, causal, device, precision):
    layer = Attention(H, nh, causal=causal, use_bias=True)
    for i, n in enumerate(NAMES):
        layer.param(n).set(inp["w"][i])
    for i, p in enumerate("qkvo"):
        layer.param("bias_" + p).set(inp["b"][i])
    if device == capi.DEVICE_CUDA:
        layer.to_device(device)
    layer.set_precision(precision)
    return layer


CASES = [
    # name, B, S, H, nh, causal, ranges, precision, bf16, tolerance
    ("fp32_half_sequences", 3, 24, 32, 4, True, 2, capi.MMA_FP32, False, 1e-5),
    ("fp32_uneven_five_ranges", 2, 40, 48, 4, False, 5, capi.MMA_FP32, False, 1e-5),
    ("bf16_tensor_cores_hs64", 2, 512, 256, 4, True, 4, capi.MMA_BF16, True, 2e-2),
    ("bf16_tensor_cores_hs128", 1, 1024, 512, 4, True, 2, capi.MMA_BF16, True, 2e-2),
]


@pytest.mark.parametrize("device", [capi.DEVICE_CUDA, capi.DEVICE_CPU], ids=["cuda_tensors", "host_tensors"])
@pytest.mark.parametrize("name,B,S,H,nh,causal,world,precision,bf16,tol", CASES, ids=[c[0] for c in CASES])
def test_unit_ranges_reproduce_the_full_step(gpu_lib, name, B, S, H, nh, causal, world, precision, bf16, tol, device):
    case = cases.Case(name, B, S, H, nh, causal=causal, bias_std=0.1)
    inp = case.inputs(bf16=bf16)
    ref = oracle.port_step(inp["q"], inp["q"], inp["q"], inp["w"], inp["b"], inp["dout"], nh, causal)
    x2, g2 = inp["q"].reshape(-1, H), inp["dout"].reshape(-1, H)
    bucket = None
    got = {k: np.zeros((B * S, H), np.float32) for k in ("out", "dq", "dk", "dv")}
    layer = make_layer(inp, H, nh, causal, device, precision)
    for rank in range(world):
        u = shard.head_unit_range(B, nh, world, rank)
        r0, r1 = shard.unit_rows(u, S, nh)
        x = Tensor.from_numpy(x2[r0:r1], device, bf16=bf16)
        out = layer.forward_units(x, S)
        assert out.shape == (r1 - r0, H) and out.device == device
        gq, gk, gv = layer.backward(Tensor.from_numpy(g2[r0:r1], device, bf16=bf16))
        got["out"][r0:r1], got["dq"][r0:r1] = out.numpy(), gq.numpy()
        got["dk"][r0:r1], got["dv"][r0:r1] = gk.numpy(), gv.numpy()
        part = np.concatenate([layer.param("grad_" + n).numpy().ravel() for n in NAMES] +
                              [layer.param("grad_bias_" + p).numpy().ravel() for p in "qkvo"]).astype(np.float64)
        bucket = part if bucket is None else bucket + part
    layer.free()
    for key in ("out", "dq", "dk", "dv"):
        assert cases.rel_err(got[key], ref[key].reshape(-1, H)) <= tol, (name, key)
    want_w = np.concatenate([w.ravel() for w in ref["dw"]])
    want_b = np.concatenate([b.ravel() for b in ref["db"]])
    n_w = want_w.size
    for i in range(4):
        seg = slice(i * H * H, (i + 1) * H * H)
        assert cases.rel_err(bucket[seg], want_w[seg]) <= tol, (name, "dw%d" % i)
    assert np.abs(bucket[n_w:] - want_b).max() <= tol * np.abs(want_b).max(), (name, "db")


def test_unit_range_entry_refuses_what_it_cannot_split(gpu_lib):
    lib = gpu_lib
    layer = Attention(32, 4)
    x = Tensor.from_numpy(np.zeros((12, 32), np.float32))
    assert not lib.boat_attention_forward_units(layer.h, x.h, x.h, x.h, 26)       # 26 is not a multiple of 4 heads
    assert not lib.boat_attention_forward_units(layer.h, x.h, x.h, x.h, 40)       # 12 rows are not whole units of 10 rows
    x3 = Tensor.from_numpy(np.zeros((1, 12, 32), np.float32))
    assert not lib.boat_attention_forward_units(layer.h, x3.h, x3.h, x3.h, 24)    # wants [rows, H]
    assert not lib.boat_attention_forward_units(None, x.h, x.h, x.h, 24)
    out = layer.forward_units(x, 24)                                              # 12 rows = 2 of the 4 units of S=24
    assert out.shape == (12, 32)
    layer.free()
