"""The generic tensor operations of the attention path through Boat's C API (boat_transpose,
boat_add, boat_mul, boat_mul_scalar, boat_add_, boat_sub_, boat_matmul) on host and CUDA tensors,
against golden vectors made by the reference library."""
import ctypes as C
import os

import numpy as np
import pytest

import cases
from boat_b200 import capi
from boat_b200.host import Tensor

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEVICES = [capi.DEVICE_CPU, capi.DEVICE_CUDA]
IDS = ["host_tensors", "cuda_tensors"]


@pytest.fixture(scope="module")
def ops_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "ops_golden.npz"))


def call(lib, name, *args):
    h = getattr(lib, name)(*args)
    assert h, "%s returned NULL: %s" % (name, lib.boat_cuda_last_error())
    return Tensor(h)


@pytest.mark.parametrize("device", DEVICES, ids=IDS)
def test_transpose_matches_reference(gpu_lib, ops_golden, device):
    lib, inp = gpu_lib, cases.ops_inputs()
    for key, dims in (("t4", (2, 3)), ("t4_ragged", (2, 3)), ("t4_ragged", (3, 2)), ("t2", (0, 1))):
        t = Tensor.from_numpy(inp[key], device)
        out = call(lib, "boat_transpose", t.h, dims[0], dims[1])
        assert out.device == device
        want = ops_golden["transpose_" + key]
        assert out.shape == want.shape, key
        assert np.array_equal(out.numpy(), want), key
    # anything but the last two dimensions is refused, like out-of-range dimensions
    t = Tensor.from_numpy(inp["t4"], device)
    assert not lib.boat_transpose(t.h, 0, 3)
    assert not lib.boat_transpose(t.h, 2, 4)
    assert not lib.boat_transpose(None, 0, 1)


@pytest.mark.parametrize("device", DEVICES, ids=IDS)
def test_elementwise_ops_match_reference_bit_for_bit(gpu_lib, ops_golden, device):
    lib, inp = gpu_lib, cases.ops_inputs()
    a, b, bias = (Tensor.from_numpy(inp[k], device) for k in ("a", "b", "bias"))
    for name, args, key in (("boat_add", (a.h, b.h), "add"), ("boat_add", (a.h, bias.h), "add_bias"),
                            ("boat_add", (bias.h, a.h), "add_bias"), ("boat_mul", (a.h, b.h), "mul"),
                            ("boat_mul_scalar", (a.h, C.c_double(inp["scalar"])), "mul_scalar")):
        out = call(lib, name, *args)
        assert out.device == device and out.shape == inp["a"].shape, key
        assert np.array_equal(out.numpy(), ops_golden[key]), key
    assert np.array_equal(a.numpy(), inp["a"])                      # operands untouched
    for name, key in (("boat_add_", "add_"), ("boat_sub_", "sub_")):
        acc = Tensor.from_numpy(inp["a"], device)
        getattr(lib, name)(acc.h, b.h)
        assert np.array_equal(acc.numpy(), ops_golden[key]), key
    # size mismatch: in-place ops do nothing (src/ops/arithmetic.c:371-375), boat_add gives NULL
    acc = Tensor.from_numpy(inp["a"], device)
    lib.boat_add_(acc.h, bias.h)
    assert np.array_equal(acc.numpy(), inp["a"])
    odd = Tensor.from_numpy(np.ones((5,), np.float32), device)
    assert not lib.boat_add(a.h, odd.h)


def test_elementwise_ops_mix_host_and_cuda_operands(gpu_lib, ops_golden):
    lib, inp = gpu_lib, cases.ops_inputs()
    a = Tensor.from_numpy(inp["a"], capi.DEVICE_CUDA)
    b = Tensor.from_numpy(inp["b"], capi.DEVICE_CPU)
    out = call(lib, "boat_add", a.h, b.h)
    assert out.device == capi.DEVICE_CUDA                           # the result lives where the first operand lives
    assert np.array_equal(out.numpy(), ops_golden["add"])
    lib.boat_sub_(b.h, a.h)                                         # host accumulator, CUDA operand
    assert np.array_equal(b.numpy(), inp["b"] - inp["a"])


@pytest.mark.parametrize("device", DEVICES, ids=IDS)
def test_batched_matmul_matches_reference(gpu_lib, ops_golden, device):
    lib, inp = gpu_lib, cases.ops_inputs()
    for ka, kb, key in (("m3a", "m3b", "matmul3"), ("m4a", "m4b", "matmul4")):
        a, b = Tensor.from_numpy(inp[ka], device), Tensor.from_numpy(inp[kb], device)
        out = call(lib, "boat_matmul", a.h, b.h)
        want = ops_golden[key]
        assert out.shape == want.shape and out.device == device
        assert cases.rel_err(out.numpy(), want) <= 1e-5, key
    # batch dimensions must match exactly (src/ops/linear.c:32-36)
    a, b = Tensor.from_numpy(inp["m3a"], device), Tensor.from_numpy(inp["m4b"], device)
    assert not lib.boat_matmul(a.h, b.h)
