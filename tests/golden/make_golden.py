"""Regenerate tests/golden/attention_golden.npz, adam_golden.npz, graph_golden.npz and
ops_golden.npz from the reference itself.

Run in a checkout that has the reference tree (oracle/Makefile builds
oracle/_ref/libboat_ref.so from it):

    python tests/golden/make_golden.py

Also stored: the reference's boat_layernorm_forward and its dense layer (forward, two
accumulating backward calls) on the seeded inputs of tests/cases.py.

adam_golden.npz holds the parameters after every step of the reference's Adam optimizer
(boat_adam_optimizer_create / boat_optimizer_step) on cases.adam_inputs().

graph_golden.npz holds outputs and gradients of two graphs run through the reference's
autodiff (boat_var_attention + boat_var_add; boat_var_matmul, boat_var_dense, boat_var_mul,
boat_var_sub) with boat_variable_backward.

ops_golden.npz holds the reference's boat_transpose, boat_add (equal shapes and bias broadcast),
boat_mul, boat_mul_scalar, boat_add_, boat_sub_ and batched boat_matmul on cases.ops_inputs().

For every case in tests/cases.py::GOLDEN_CASES the reference's own boat_attention_forward
and boat_attention_backward are executed on the seeded inputs and every output and gradient
is stored (FP32, bit patterns as the reference produced them), together with a checksum of
the inputs so that drift of the input generator is noticed.
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import oracle          # noqa: E402
import cases                       # noqa: E402


def input_digest(inp):
    h = hashlib.sha256()
    for key in ("q", "k", "v", "dout"):
        h.update(np.ascontiguousarray(inp[key]).tobytes())
    for w in inp["w"]:
        h.update(np.ascontiguousarray(w).tobytes())
    for b in inp["b"] or []:
        h.update(np.ascontiguousarray(b).tobytes())
    return h.hexdigest()


def main():
    oracle.build()
    out = {}
    for case in cases.GOLDEN_CASES:
        inp = case.inputs()
        res = oracle.ref_step(inp["q"], inp["k"], inp["v"], inp["w"], inp["b"], inp["dout"], case.nh, case.causal)
        for key, val in cases.flatten_result(res).items():
            out["%s/%s" % (case.name, key)] = val
        out["%s/digest" % case.name] = np.frombuffer(input_digest(inp).encode(), dtype=np.uint8)
        print(case.name, "ok")
    # layers around attention that the reference implements: LayerNorm forward, dense forward/backward
    ln = cases.layernorm_inputs()
    out["layernorm/y"] = oracle.ref_layernorm(ln["x"], ln["w"], ln["b"], ln["eps"])
    out["layernorm/y_plain"] = oracle.ref_layernorm(ln["x"], None, None, ln["eps"])
    de = cases.dense_inputs()
    res = oracle.ref_dense_step(de["x"], de["w"], de["b"], de["dy"], repeats=2)
    for key in ("y", "dx", "dw", "db"):
        out["dense/" + key] = res[key]
    print("layernorm, dense ok")
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attention_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")
    params, grads = cases.adam_inputs()
    adam = {}
    for steps in range(1, len(grads) + 1):
        for i, p in enumerate(oracle.ref_adam(params, grads[:steps], **cases.ADAM_HYPER)):
            adam["step%d/p%d" % (steps, i)] = p
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "adam_golden.npz")
    np.savez_compressed(path, **adam)
    print("wrote", path, os.path.getsize(path), "bytes")


def graphs():
    out = {}
    case = cases.GRAPH_CASE
    inp = case.inputs()
    res = oracle.ref_graph_residual_attention(inp["q"], inp["w"], inp["b"], case.nh, case.causal, inp["dout"])
    for key in ("out", "dx"):
        out["residual/" + key] = res[key]
    for i, p in enumerate("qkvo"):
        out["residual/dw" + p] = res["dw"][i]
        out["residual/db" + p] = res["db"][i]
    g = cases.graph_mlp_inputs()
    res = oracle.ref_graph_mlp(g["a"], g["wm"], g["wd"], g["bd"], g["c"], g["m"], g["gout"])
    for key, val in res.items():
        out["mlp/" + key] = val
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "graph_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def ops():
    out = oracle.ref_ops(cases.ops_inputs())
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ops_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
    graphs()
    ops()
