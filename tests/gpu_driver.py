"""Runs an attention step through the C-ABI library (boat_b200) for the GPU tests."""
import numpy as np

from boat_b200 import capi
from boat_b200.host import Attention, Tensor


def gpu_step(inp, nh, causal, device=capi.DEVICE_CPU, precision=-1, bf16=False, backward=True, lr=None):
    """inp: dict from cases.Case.inputs().  device: where inputs and the layer live.
    Returns the same dict layout as oracle.port_step (+ "w_after"/"b_after" when lr is given)."""
    q = inp["q"]
    B, S, H = q.shape
    layer = Attention(H, nh, causal=causal, use_bias=inp["b"] is not None)
    try:
        names = ["weight_q", "weight_k", "weight_v", "weight_o"]
        for i, n in enumerate(names):
            layer.param(n).set(inp["w"][i])
        if inp["b"] is not None:
            for i, n in enumerate(["bias_q", "bias_k", "bias_v", "bias_o"]):
                layer.param(n).set(inp["b"][i])
        if device == capi.DEVICE_CUDA:
            layer.to_device(capi.DEVICE_CUDA)
        layer.set_precision(precision)
        tq = Tensor.from_numpy(q, device, bf16=bf16)
        tk = tq if inp["k"] is q else Tensor.from_numpy(inp["k"], device, bf16=bf16)
        tv = tq if inp["v"] is q else Tensor.from_numpy(inp["v"], device, bf16=bf16)
        out = layer.forward(tq, tk, tv)
        res = {"out": out.numpy()}
        assert out.shape == (B, S, H) and out.device == device
        if backward:
            tg = Tensor.from_numpy(inp["dout"], device, bf16=bf16)
            gq, gk, gv = layer.backward(tg)
            res.update(dq=gq.numpy(), dk=gk.numpy(), dv=gv.numpy())
            res["dw"] = [layer.param("grad_" + n).numpy() for n in names]
            res["db"] = ([layer.param("grad_bias_" + p).numpy() for p in "qkvo"]
                         if inp["b"] is not None else None)
            if lr is not None:
                layer.update(lr)
                res["w_after"] = [layer.param(n).numpy() for n in names]
                if inp["b"] is not None:
                    res["b_after"] = [layer.param("bias_" + p).numpy() for p in "qkvo"]
        return res
    finally:
        layer.free()
