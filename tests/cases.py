"""Seeded attention-step problems shared by the golden-vector generator and the tests.

Inputs follow the configurations of the benchmark specification: X ~ N(0, std_x),
W ~ N(0, std_w), upstream gradient ~ N(0, 1); seed 42 and fixed tensor ids
(boat_b200.rng).  `self_attn` means query = key = value (one tensor), as in the workload.
"""
import numpy as np

from boat_b200 import rng

SEED = 42


class Case:
    def __init__(self, name, B, S, H, nh, causal=False, bias=True, self_attn=True, std_x=1.0, std_w=None,
                 bias_std=0.0):
        self.name, self.B, self.S, self.H, self.nh = name, B, S, H, nh
        self.causal, self.bias, self.self_attn = causal, bias, self_attn
        self.std_x = std_x
        self.std_w = std_w if std_w is not None else 1.0 / np.sqrt(H)
        self.bias_std = bias_std

    def inputs(self, bf16=False):
        """dict: q,k,v,dout [B,S,H]; w (4 x [H,H]); b (4 x [H]) or None.  With bf16 every
        value is rounded to BF16 first (still FP32 arrays), so that a BF16 device path and
        the FP32 CPU checker start from identical numbers."""
        shape = (self.B, self.S, self.H)
        f = rng.bf16_round if bf16 else (lambda a: a)
        q = f(rng.normal(SEED, rng.X, shape, self.std_x))
        if self.self_attn:
            k = v = q
        else:
            k = f(rng.normal(SEED, rng.KEY, shape, self.std_x))
            v = f(rng.normal(SEED, rng.VALUE, shape, self.std_x))
        w = [f(rng.normal(SEED, rng.WQ + i, (self.H, self.H), self.std_w)) for i in range(4)]
        b = None
        if self.bias:
            b = [rng.normal(SEED, rng.BQ + i, (self.H,), self.bias_std) if self.bias_std > 0
                 else np.zeros(self.H, np.float32) for i in range(4)]
        dout = f(rng.normal(SEED, rng.DOUT, shape, 1.0))
        return dict(q=q, k=k, v=v, w=w, b=b, dout=dout)


# Small problems whose reference outputs are committed under tests/golden/.
GOLDEN_CASES = [
    # the reference's CPU-runnable configuration: B=2, S=64, d=64, 4 heads, N(0,0.02), zero bias
    Case("c1", 2, 64, 64, 4, std_x=0.02, std_w=0.02),
    Case("c1_causal_bias", 2, 64, 64, 4, causal=True, std_x=0.02, std_w=0.02, bias_std=0.1),
    # shape of the reference's own attention tests (B=2, S=4, H=32, 4 heads), distinct q/k/v
    Case("reftest_shape", 2, 4, 32, 4, self_attn=False, bias_std=0.1),
    # ragged: S not a multiple of anything useful, 3 heads of 16, causal, no bias
    Case("ragged_causal_nobias", 1, 37, 48, 3, causal=True, bias=False, self_attn=False),
    # one token: softmax over a single score
    Case("single_token", 3, 1, 16, 2, bias_std=0.1),
    # 128-row tile boundary with head size 64 (shapes the tensor-core kernels take)
    Case("tile_128x64", 1, 128, 128, 2, causal=True, bias_std=0.1),
]

RESULT_KEYS = ("out", "dq", "dk", "dv", "dw0", "dw1", "dw2", "dw3", "db0", "db1", "db2", "db3")


def flatten_result(res):
    """dict from oracle.port_step/ref_step or the GPU path -> flat dict of arrays."""
    flat = {k: res[k] for k in ("out", "dq", "dk", "dv")}
    for i in range(4):
        flat["dw%d" % i] = res["dw"][i]
        if res.get("db") is not None:
            flat["db%d" % i] = res["db"][i]
    return flat


def rel_err(a, ref):
    """max|a - ref| / max|ref|, the error measure of the benchmark specification."""
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = np.abs(ref).max()
    return float(np.abs(a - ref).max() / denom) if denom > 0 else float(np.abs(a).max())


def errors(res, ref):
    """Per-tensor max|res - ref| / max|ref| for two flat result dicts.

    The key-bias gradient is identically zero in exact arithmetic (adding a constant to
    every key shifts all scores of a query alike, which the softmax ignores), so the
    reference value of db1 is round-off noise; the four bias gradients are therefore
    measured against their common largest magnitude."""
    db_scale = max([float(np.abs(ref[k]).max()) for k in ref if k.startswith("db")] or [0.0])
    out = {}
    for key, r in ref.items():
        a = np.asarray(res[key], dtype=np.float64)
        r64 = np.asarray(r, dtype=np.float64)
        denom = db_scale if key.startswith("db") else float(np.abs(r64).max())
        diff = float(np.abs(a - r64).max())
        out[key] = diff / denom if denom > 0 else diff
    return out


# ---- layers around attention: seeded inputs for the golden vectors and tests --------------------------

def layernorm_inputs(rows_shape=(3, 7), H=48):
    x = rng.normal(SEED, 20, rows_shape + (H,)) * np.float32(1.7) + np.float32(0.3)
    w = rng.normal(SEED, 21, (H,), 0.5) + np.float32(1.0)
    b = rng.normal(SEED, 22, (H,), 0.2)
    dy = rng.normal(SEED, 23, rows_shape + (H,))
    return dict(x=x, w=w, b=b, dy=dy, eps=1e-5)


def dense_inputs(N=19, I=24, O=40):
    return dict(x=rng.normal(SEED, 30, (N, I)), w=rng.normal(SEED, 31, (I, O), 0.2), b=rng.normal(SEED, 32, (O,), 0.1),
                dy=rng.normal(SEED, 33, (N, O)))


# ---- Adam: seeded parameters and a sequence of gradients ------------------------------------------------

ADAM_HYPER = dict(lr=0.01, beta1=0.9, beta2=0.999, eps=1e-8)


def adam_inputs(shapes=((33, 17), (4096 + 5,), (7,), (64, 64)), steps=6, stream=40):
    """Parameter tensors of ragged sizes (vector and scalar code paths) and `steps` gradients each; a few
    gradient entries are exactly zero or tiny so that the epsilon term matters."""
    params = [rng.normal(SEED, stream + i, s) for i, s in enumerate(shapes)]
    grads = []
    for t in range(steps):
        gs = []
        for i, s in enumerate(shapes):
            g = rng.normal(SEED, stream + 100 * (t + 1) + i, s, 0.3)
            flat = g.reshape(-1)
            flat[::11] = 0.0
            flat[5::13] *= np.float32(1e-6)
            gs.append(g)
        grads.append(gs)
    return params, grads


# ---- autodiff graphs: seeded inputs for the golden vectors and tests ---------------------------------------

GRAPH_CASE = Case("graph_residual", B=2, S=24, H=32, nh=4, causal=True, bias_std=0.1)


def graph_mlp_inputs(N=19, I=24, M=40, O=16):
    """z = sub(mul(dense(matmul(a, wm)), m), c): a [N,I], wm [I,M], dense M -> O, m and c [N,O]."""
    return dict(a=rng.normal(SEED, 60, (N, I)), wm=rng.normal(SEED, 61, (I, M), 0.2), wd=rng.normal(SEED, 62, (M, O), 0.2),
                bd=rng.normal(SEED, 63, (O,), 0.1), c=rng.normal(SEED, 64, (N, O)), m=rng.normal(SEED, 65, (N, O)),
                gout=rng.normal(SEED, 66, (N, O)))


# ---- generic tensor operations the path exports: seeded inputs for the golden vectors and tests -----------

def ops_inputs():
    """Operands for boat_transpose (the reference's own 4-D case, tests/unit/test_transpose.c:55-103, and
    a ragged one), boat_add with a trailing-dimension broadcast (src/ops/arithmetic.c:199-203), boat_mul,
    boat_mul_scalar, boat_add_ / boat_sub_ and batched boat_matmul."""
    return dict(
        t4=(np.arange(2 * 2 * 3 * 4, dtype=np.float32) + np.float32(1.0)).reshape(2, 2, 3, 4),
        t4_ragged=rng.normal(SEED, 80, (3, 2, 37, 19)),
        t2=rng.normal(SEED, 81, (45, 70)),
        a=rng.normal(SEED, 82, (3, 17, 24)),
        b=rng.normal(SEED, 83, (3, 17, 24)),
        bias=rng.normal(SEED, 84, (24,)),
        scalar=-0.37,
        m3a=rng.normal(SEED, 85, (3, 9, 14)), m3b=rng.normal(SEED, 86, (3, 14, 11)),
        m4a=rng.normal(SEED, 87, (2, 3, 8, 5)), m4b=rng.normal(SEED, 88, (2, 3, 5, 6)))
