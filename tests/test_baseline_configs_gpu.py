"""GPU parity on the benchmarked configurations themselves.

The benchmark times sequence lengths, head sizes and unit counts far beyond the small parity
cases: 64-tile walks, more (batch, head) units than the backward schedules together (several
CTA groups, the last one short), both walk-pairing schedules, FP32 dQ sums of hundreds of MB.
These tests run exactly those shapes - as slices that the CPU restatement of the reference
finishes in seconds - and compare with it per tensor:

  kernel ABI   boat_cuda_attn_fwd / _bwd on [units, S, hs] slices of configs 3, 4, 5 and of the
               target point (B=8, S=4096, head size 128), with more units than one CTA group
               holds, under BOAT_BWD_PAIR=0 and 1
  layer        boat_attention_forward / _backward for config 2 at full size (TF32) and for one
               batch entry of configs 3, 5 and (half the sequence) 4: out, dq, dk, dv, all dW, db

Tolerance: max|ours - ref| / max|ref| <= 2e-2 (BF16) / 5e-3 (TF32) per tensor; BF16 cases feed
BF16-rounded values to both sides.
"""
import ctypes as C
import os

import numpy as np
import pytest

import cases
from boat_b200 import capi, rng
from boat_b200.host import DeviceBuffer, check
from gpu_driver import gpu_step
from oracle import oracle

pytestmark = pytest.mark.gpu

TOL_TF32, TOL_BF16 = 5e-3, 2e-2

# name: units, S, hs, causal - each with more units than the backward's CTA group for that shape
# (64 MB / (S*hs*16 B): 4, 8, 32 and 64 units), so a second, shorter group exists
CORE_SLICES = {
    "c4_S8192_hs128": (6, 8192, 128, True),
    "target_S4096_hs128": (10, 4096, 128, True),
    "c3_S2048_hs64": (40, 2048, 64, True),
    "c5_S1024_hs64": (72, 1024, 64, False),
}

_core_cache = {}


def core_problem(name):
    """Seeded BF16-rounded q, k, v, dO of a slice and the restatement's o, dq, dk, dv (computed
    once per process: both schedules are compared with the same reference)."""
    if name not in _core_cache:
        units, S, hs, causal = CORE_SLICES[name]
        shape = (units, S, hs)
        q, k, v, go = (rng.bf16_round(rng.normal(1234, i, shape)) for i in range(4))
        ref = oracle.port_core(q, k, v, go, causal, 1.0 / np.sqrt(hs))
        _core_cache[name] = (q, k, v, go, ref)
    return _core_cache[name]


def run_core_bf16(lib, q, k, v, go, causal):
    units, S, hs = q.shape
    scale = 1.0 / np.sqrt(hs)
    n = q.size
    dq_, dk_, dv_, dgo = (DeviceBuffer.from_numpy(a, bf16=True) for a in (q, k, v, go))
    do_, dlse = DeviceBuffer(n * 2), DeviceBuffer(units * S * 4)
    check(lib.boat_cuda_attn_fwd(capi.MMA_BF16, units, S, hs, int(causal), C.c_float(scale), dq_.p, dk_.p, dv_.p,
                                 capi.CUDA_BF16, do_.p, dlse.p), "attn_fwd")
    gq, gk, gv = DeviceBuffer(n * 2), DeviceBuffer(n * 2), DeviceBuffer(n * 2)
    scratch = DeviceBuffer(max(lib.boat_cuda_attn_bwd_scratch_bytes(capi.MMA_BF16, units, S, hs), 256))
    check(lib.boat_cuda_attn_bwd(capi.MMA_BF16, units, S, hs, int(causal), C.c_float(scale), dq_.p, dk_.p, dv_.p, do_.p,
                                 dgo.p, dlse.p, capi.CUDA_BF16, gq.p, gk.p, gv.p, scratch.p, scratch.nbytes), "attn_bwd")
    check(lib.boat_cuda_sync(), "sync")
    shape = (units, S, hs)
    return {"o": do_.numpy(shape, bf16=True), "dq": gq.numpy(shape, bf16=True), "dk": gk.numpy(shape, bf16=True),
            "dv": gv.numpy(shape, bf16=True)}


@pytest.mark.parametrize("pair", ["0", "1"], ids=["one_walk_per_cta", "two_walks_per_cta"])
@pytest.mark.parametrize("name", list(CORE_SLICES))
def test_attention_core_slice_of_benchmarked_config(gpu_lib, name, pair):
    q, k, v, go, ref = core_problem(name)
    causal = CORE_SLICES[name][3]
    old = os.environ.get("BOAT_BWD_PAIR")
    os.environ["BOAT_BWD_PAIR"] = pair
    try:
        got = run_core_bf16(gpu_lib, q, k, v, go, causal)
    finally:
        if old is None:
            del os.environ["BOAT_BWD_PAIR"]
        else:
            os.environ["BOAT_BWD_PAIR"] = old
    for key in ("o", "dq", "dk", "dv"):
        assert np.isfinite(got[key]).all(), (name, key)
        # every unit is held to the tolerance on its own scale: a wrong unit must not hide
        # behind a larger one
        for u in range(q.shape[0]):
            err = cases.rel_err(got[key][u], ref[key][u])
            assert err <= TOL_BF16, (name, key, "unit %d" % u, err)


@pytest.mark.parametrize("group", ["1", "4", "5"])
def test_forward_unit_groups(gpu_lib, monkeypatch, group):
    """The forward schedules the CTAs of a few units at a time (their K and V share L2) and puts a
    short group first when the units do not divide; BOAT_FWD_GROUP forces small groups on the
    6-unit slice of config 4: six groups of one, a short group of 2 before one of 4, 1 before 5."""
    monkeypatch.setenv("BOAT_FWD_GROUP", group)
    name = "c4_S8192_hs128"
    q, k, v, go, ref = core_problem(name)
    got = run_core_bf16(gpu_lib, q, k, v, go, True)
    for u in range(q.shape[0]):
        assert cases.rel_err(got["o"][u], ref["o"][u]) <= TOL_BF16, (group, u)
        assert cases.rel_err(got["dq"][u], ref["dq"][u]) <= TOL_BF16, (group, u)      # through the saved lse


def test_schedule_default_matches_forced_choice(gpu_lib):
    """Without BOAT_BWD_PAIR the launcher picks a schedule by problem size; whatever it picks
    must give the numbers of that schedule when forced."""
    name = "c3_S2048_hs64"
    q, k, v, go, ref = core_problem(name)
    old = os.environ.pop("BOAT_BWD_PAIR", None)
    try:
        got = run_core_bf16(gpu_lib, q, k, v, go, True)
    finally:
        if old is not None:
            os.environ["BOAT_BWD_PAIR"] = old
    for key in ("o", "dq", "dk", "dv"):
        assert cases.rel_err(got[key], ref[key]) <= TOL_BF16, key


def assert_step_close(res, ref, tol, what):
    flat, fref = cases.flatten_result(res), cases.flatten_result(ref)
    for key, r in fref.items():
        assert flat[key].shape == r.shape, (what, key)
        assert np.isfinite(flat[key]).all(), (what, key, "non-finite values")
    worst = cases.errors(flat, fref)
    bad = {k: v for k, v in worst.items() if v > tol}
    assert not bad, "%s: relative error above %g: %s (all: %s)" % (what, tol, bad, worst)


def test_config2_full_size_tf32(gpu_lib):
    """B=8, S=512, d_model=512, 8 heads of 64, non-causal, FP32 storage with TF32 arithmetic."""
    case = cases.Case("c2", 8, 512, 512, 8, causal=False, bias_std=0.1)
    inp = case.inputs()
    ref = oracle.port_step(inp["q"], inp["k"], inp["v"], inp["w"], inp["b"], inp["dout"], 8, False)
    for device in (capi.DEVICE_CUDA, capi.DEVICE_CPU):
        res = gpu_step(inp, 8, False, device=device, precision=capi.MMA_TF32)
        assert_step_close(res, ref, TOL_TF32, "c2 on device %d" % device)


LAYER_SLICES = [
    # name, B, S, d_model, heads, causal
    ("c3_one_batch_entry", 1, 2048, 1024, 16, True),
    ("c5_one_batch_entry", 1, 1024, 1024, 16, False),
    ("c4_one_batch_entry_half_sequence", 1, 4096, 2048, 16, True),
]


@pytest.mark.parametrize("name,B,S,H,nh,causal", LAYER_SLICES, ids=[c[0] for c in LAYER_SLICES])
def test_layer_step_on_one_batch_entry_of_benchmarked_config(gpu_lib, name, B, S, H, nh, causal):
    case = cases.Case(name, B, S, H, nh, causal=causal, bias_std=0.1)
    inp = case.inputs(bf16=True)
    ref = oracle.port_step(inp["q"], inp["k"], inp["v"], inp["w"], inp["b"], inp["dout"], nh, causal)
    res = gpu_step(inp, nh, causal, device=capi.DEVICE_CUDA, precision=capi.MMA_BF16, bf16=True)
    assert_step_close(res, ref, TOL_BF16, name)
