"""The attention backward entry point that brings its own scratch memory.

boat_cuda_attn_bwd_static exists for callers that may not allocate device memory at the
place they call from - a serving loop that bans cudaMalloc because it can stall the whole
device, a program whose HBM budget is fixed at start-up, a plugin inside a framework that
owns all device memory.  It must give the same gradients as boat_cuda_attn_bwd (which takes
scratch from the caller), call after call: the built-in block is shared by all calls and
still holds the previous call's data, so the second call here uses different inputs and a
different shape than the first.

Collected last on purpose (file name), so that a run that stops at the first failure has
already executed every other test.  Works alone in a fresh process and after the others.
"""
import ctypes as C

import numpy as np
import pytest

from boat_b200 import capi, rng
from boat_b200.host import DeviceBuffer, check

pytestmark = pytest.mark.gpu

TOL = {capi.MMA_FP32: 1e-5, capi.MMA_BF16: 2e-2}


def backward_both_ways(lib, mma, units, S, hs, causal, seed, numpy_rng=False):
    bf = mma == capi.MMA_BF16
    io = capi.CUDA_BF16 if bf else capi.CUDA_F32
    f = rng.bf16_round if bf else (lambda a: a)
    shape = (units, S, hs)
    if numpy_rng:        # tens of millions of elements: numpy's generator is much faster than the counter-based one
        g = np.random.default_rng(seed)
        q, k, v, go = (g.standard_normal(shape, dtype=np.float32) for _ in range(4))
    else:
        q, k, v, go = (f(rng.normal(seed, i, shape)) for i in range(4))
    scale = 1.0 / np.sqrt(hs)
    dq_, dk_, dv_, dgo = (DeviceBuffer.from_numpy(a, bf16=bf) for a in (q, k, v, go))
    es = 2 if bf else 4
    n = units * S * hs
    o, lse = DeviceBuffer(n * es), DeviceBuffer(units * S * 4)
    check(lib.boat_cuda_attn_fwd(mma, units, S, hs, int(causal), C.c_float(scale), dq_.p, dk_.p, dv_.p, io, o.p, lse.p))
    # existing entry point: scratch from the caller
    need = lib.boat_cuda_attn_bwd_scratch_bytes(mma, units, S, hs)
    assert need <= lib.boat_cuda_attn_bwd_static_capacity()
    scratch = DeviceBuffer(max(need, 256))
    a = [DeviceBuffer(n * es) for _ in range(3)]
    check(lib.boat_cuda_attn_bwd(mma, units, S, hs, int(causal), C.c_float(scale), dq_.p, dk_.p, dv_.p, o.p, dgo.p,
                                 lse.p, io, a[0].p, a[1].p, a[2].p, scratch.p, scratch.nbytes), "attn_bwd")
    # new entry point: no scratch argument, nothing allocated inside
    b = [DeviceBuffer(n * es) for _ in range(3)]
    in_use = lib.boat_cuda_bytes_in_use()
    check(lib.boat_cuda_attn_bwd_static(mma, units, S, hs, int(causal), C.c_float(scale), dq_.p, dk_.p, dv_.p, o.p,
                                        dgo.p, lse.p, io, b[0].p, b[1].p, b[2].p), "attn_bwd_static")
    assert lib.boat_cuda_bytes_in_use() == in_use
    check(lib.boat_cuda_sync(), "sync")
    return [x.numpy(shape, bf16=bf) for x in a], [x.numpy(shape, bf16=bf) for x in b]


def assert_same(ref, got, tol, what):
    for name, r, g in zip(("dq", "dk", "dv"), ref, got):
        assert np.isfinite(g).all(), (what, name)
        err = float(np.abs(g.astype(np.float64) - r).max() / np.abs(r).max())
        assert err <= tol, (what, name, err)


def test_static_scratch_backward_matches_on_two_calls_in_a_row(gpu_lib):
    lib = gpu_lib
    # tensor-core path: delta + FP32 dQ sum live in the built-in block (4.2 MiB, then 8.4 MiB)
    ref, got = backward_both_ways(lib, capi.MMA_BF16, 4, 512, 128, True, seed=21)
    assert_same(ref, got, TOL[capi.MMA_BF16], "first call")
    ref, got = backward_both_ways(lib, capi.MMA_BF16, 16, 512, 64, False, seed=22)
    assert_same(ref, got, TOL[capi.MMA_BF16], "second call")
    # exact path (only delta is scratch) right after, on a ragged shape
    ref, got = backward_both_ways(lib, capi.MMA_FP32, 3, 77, 16, True, seed=23)
    assert_same(ref, got, TOL[capi.MMA_FP32], "third call, fp32")


def test_static_scratch_refuses_problems_beyond_its_capacity(gpu_lib):
    lib = gpu_lib
    units, S, hs = 64, 4096, 128                         # needs 128 MiB of dQ sum
    assert lib.boat_cuda_attn_bwd_scratch_bytes(capi.MMA_BF16, units, S, hs) > lib.boat_cuda_attn_bwd_static_capacity()
    dummy = DeviceBuffer(256)
    rc = lib.boat_cuda_attn_bwd_static(capi.MMA_BF16, units, S, hs, 1, C.c_float(0.1), dummy.p, dummy.p, dummy.p, dummy.p,
                                       dummy.p, dummy.p, capi.CUDA_BF16, dummy.p, dummy.p, dummy.p)
    assert rc != 0
    msg = lib.boat_cuda_last_error().decode()
    assert "scratch" in msg and str(lib.boat_cuda_attn_bwd_static_capacity()) in msg


def test_static_scratch_accepts_a_problem_of_exactly_its_capacity(gpu_lib):
    """The exact path needs 4 bytes of scratch per (unit, row): 32768 units of 128 rows fill the
    16 MiB block to the last byte and are served; one unit more is refused."""
    lib = gpu_lib
    cap = lib.boat_cuda_attn_bwd_static_capacity()
    units, S, hs = cap // (128 * 4), 128, 8
    assert lib.boat_cuda_attn_bwd_scratch_bytes(capi.MMA_FP32, units, S, hs) == cap
    ref, got = backward_both_ways(lib, capi.MMA_FP32, units, S, hs, True, seed=24, numpy_rng=True)
    assert_same(ref, got, TOL[capi.MMA_FP32], "problem of exactly the capacity")
    dummy = DeviceBuffer(256)
    rc = lib.boat_cuda_attn_bwd_static(capi.MMA_FP32, units + 1, S, hs, 1, C.c_float(0.1), dummy.p, dummy.p, dummy.p,
                                       dummy.p, dummy.p, dummy.p, capi.CUDA_F32, dummy.p, dummy.p, dummy.p)
    assert rc != 0 and "scratch" in lib.boat_cuda_last_error().decode()
