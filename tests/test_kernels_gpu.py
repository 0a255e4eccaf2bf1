"""GPU tests of the kernel ABI (include/boat_cuda.h) one entry point at a time, against
numpy in float64 on the same (storage-rounded) inputs."""
import ctypes as C

import numpy as np
import pytest

from boat_b200 import capi, rng
from boat_b200.host import DeviceBuffer, check

pytestmark = pytest.mark.gpu

TOL = {capi.MMA_FP32: 1e-5, capi.MMA_TF32: 5e-3, capi.MMA_BF16: 2e-2}


def rel(a, ref):
    return float(np.abs(a.astype(np.float64) - ref).max() / np.abs(ref).max())


def run_gemm(lib, mma, ta, tb, M, N, K, out_bf16=False, bias=True, seed=1):
    bf = mma == capi.MMA_BF16
    a_shape = (K, M) if ta else (M, K)
    b_shape = (N, K) if tb else (K, N)
    A = rng.normal(seed, 0, a_shape)
    B = rng.normal(seed, 1, b_shape, std=1.0 / np.sqrt(K))
    bvec = rng.normal(seed, 2, (N,)) if bias else None
    if bf:
        A, B = rng.bf16_round(A), rng.bf16_round(B)
    dA, dB = DeviceBuffer.from_numpy(A, bf16=bf), DeviceBuffer.from_numpy(B, bf16=bf)
    dbias = DeviceBuffer.from_numpy(bvec) if bias else None
    dC = DeviceBuffer(M * N * (2 if out_bf16 else 4))
    check(lib.boat_cuda_gemm(mma, ta, tb, M, N, K, dA.p, a_shape[1], dB.p, b_shape[1],
                             capi.CUDA_BF16 if bf else capi.CUDA_F32, dC.p, N,
                             capi.CUDA_BF16 if out_bf16 else capi.CUDA_F32, dbias.p if bias else None), "gemm")
    check(lib.boat_cuda_sync(), "sync")
    got = dC.numpy((M, N), bf16=out_bf16)
    opA = A.T if ta else A
    opB = B.T if tb else B
    ref = opA.astype(np.float64) @ opB.astype(np.float64)
    if bias:
        ref = ref + bvec.astype(np.float64)
    return got, ref


LAYOUTS = [(0, 0), (0, 1), (1, 0)]


@pytest.mark.parametrize("mma", [capi.MMA_FP32, capi.MMA_BF16, capi.MMA_TF32], ids=["fp32", "bf16", "tf32"])
@pytest.mark.parametrize("layout", LAYOUTS, ids=["nn", "nt", "tn"])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 512), (384, 256, 192), (1024, 1024, 1024),
                                   (200, 328, 136), (4096, 512, 512)])
def test_gemm_matches_float64(gpu_lib, mma, layout, shape):
    M, N, K = shape
    got, ref = run_gemm(gpu_lib, mma, layout[0], layout[1], M, N, K)
    assert np.isfinite(got).all()
    assert rel(got, ref) <= TOL[mma]


@pytest.mark.parametrize("layout", LAYOUTS, ids=["nn", "nt", "tn"])
def test_gemm_bf16_output_and_no_bias(gpu_lib, layout):
    got, ref = run_gemm(gpu_lib, capi.MMA_BF16, layout[0], layout[1], 512, 256, 256, out_bf16=True, bias=False)
    assert rel(got, ref) <= TOL[capi.MMA_BF16]


def test_gemm_can_round_its_output_to_tf32_for_the_next_contraction(gpu_lib):
    """Output type BOAT_CUDA_F32_TF32: the same numbers as an FP32 output followed by boat_cuda_round_tf32,
    on the tensor-core kernel and on the CUDA-core kernel."""
    lib = gpu_lib
    for (M, N, K) in ((256, 256, 128), (37, 24, 19)):
        A, B = rng.normal(5, 0, (M, K)), rng.normal(5, 1, (K, N), std=1.0 / np.sqrt(K))
        dA, dB = DeviceBuffer.from_numpy(A), DeviceBuffer.from_numpy(B)
        plain, rounded = DeviceBuffer(M * N * 4), DeviceBuffer(M * N * 4)
        for out, typ in ((plain, capi.CUDA_F32), (rounded, capi.CUDA_F32_TF32)):
            check(lib.boat_cuda_gemm(capi.MMA_TF32, 0, 0, M, N, K, dA.p, K, dB.p, N, capi.CUDA_F32, out.p, N, typ, None))
        check(lib.boat_cuda_round_tf32(plain.p, plain.p, M * N))
        got, want = rounded.numpy((M, N)), plain.numpy((M, N))
        assert not (got.view(np.uint32) & np.uint32(0x1FFF)).any()
        assert np.array_equal(got, want), (M, N, K)


def test_weight_gradient_shape_uses_split_k(gpu_lib):
    """dW = X^T dY: 512 x 512 outputs, K = 16384 rows - few tiles, long K."""
    for mma in (capi.MMA_BF16, capi.MMA_TF32):
        got, ref = run_gemm(gpu_lib, mma, 1, 0, 512, 512, 16384, bias=False)
        assert rel(got, ref) <= TOL[mma]


@pytest.mark.parametrize("mma", [capi.MMA_FP32, capi.MMA_BF16, capi.MMA_TF32], ids=["fp32", "bf16", "tf32"])
def test_gemm_tiny_and_ragged_shapes(gpu_lib, mma):
    for (M, N, K) in [(1, 1, 1), (3, 5, 7), (8, 32, 32), (127, 65, 33)]:
        got, ref = run_gemm(gpu_lib, mma, 0, 0, M, N, K)
        assert rel(got, ref) <= TOL[mma], (M, N, K)


def test_elementwise_tail(gpu_lib):
    lib = gpu_lib
    for n in (1, 7, 1024, 100003):
        x, y = rng.normal(3, 0, (n,)), rng.normal(3, 1, (n,))
        dx, dy = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(y)
        check(lib.boat_cuda_axpy(dy.p, dx.p, C.c_float(-0.01), n))
        assert np.array_equal(dy.numpy((n,)), y + (np.float32(-0.01) * x))
        check(lib.boat_cuda_scale(dy.p, dx.p, C.c_float(0.5), n))
        assert np.array_equal(dy.numpy((n,)), x * np.float32(0.5))
        check(lib.boat_cuda_mul(dy.p, dx.p, dx.p, n))
        assert np.array_equal(dy.numpy((n,)), x * x)
        db = DeviceBuffer(n * 2)
        check(lib.boat_cuda_cast(db.p, capi.CUDA_BF16, dx.p, capi.CUDA_F32, n))
        assert np.array_equal(db.numpy((n,), bf16=True), rng.bf16_round(x))
        check(lib.boat_cuda_cast(dy.p, capi.CUDA_F32, db.p, capi.CUDA_BF16, n))
        assert np.array_equal(dy.numpy((n,)), rng.bf16_round(x))
    for rows, cols in ((1, 1), (5, 3), (1000, 64), (4096, 520), (33, 1000)):
        x = rng.normal(4, 0, (rows, cols))
        for bf in (False, True):
            xs = rng.bf16_round(x) if bf else x
            dx = DeviceBuffer.from_numpy(xs, bf16=bf)
            out = DeviceBuffer(cols * 4)
            check(lib.boat_cuda_colsum(dx.p, capi.CUDA_BF16 if bf else capi.CUDA_F32, rows, cols, out.p))
            ref = xs.astype(np.float64).sum(0)
            assert np.abs(out.numpy((cols,)) - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())
        b = rng.normal(4, 1, (cols,))
        dx, db_, dy = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(b), DeviceBuffer(rows * cols * 4)
        check(lib.boat_cuda_add_bias(dy.p, dx.p, db_.p, rows, cols))
        assert np.array_equal(dy.numpy((rows, cols)), x + b)
    x = rng.normal(5, 0, (3, 45, 70))
    dx, dy = DeviceBuffer.from_numpy(x), DeviceBuffer(x.size * 4)
    check(lib.boat_cuda_transpose(dy.p, dx.p, 3, 45, 70))
    assert np.array_equal(dy.numpy((3, 70, 45)), x.transpose(0, 2, 1))


# ---- attention core through boat_cuda_attn_fwd / boat_cuda_attn_bwd ----------------------------

def np_core(q, k, v, go, causal, scale):
    """float64 attention core on [units,S,hs]: O, lse and (with go) dQ,dK,dV."""
    q, k, v = (a.astype(np.float64) for a in (q, k, v))
    s = np.einsum("uid,ujd->uij", q, k) * scale
    if causal:
        S = q.shape[1]
        s = np.where(np.triu(np.ones((S, S), bool), 1)[None], -np.inf, s)
    m = s.max(-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(-1, keepdims=True)
    p = e / l
    res = {"o": p @ v, "lse": (m + np.log(l))[..., 0]}
    if go is not None:
        go = go.astype(np.float64)
        dv = np.einsum("uij,uid->ujd", p, go)
        dp = np.einsum("uid,ujd->uij", go, v)
        ds = p * (dp - (dp * p).sum(-1, keepdims=True)) * scale
        res.update(dq=ds @ k, dk=np.einsum("uij,uid->ujd", ds, q), dv=dv)
    return res


def run_core(lib, mma, units, S, hs, causal, backward=True, seed=7):
    bf = mma == capi.MMA_BF16
    io = capi.CUDA_BF16 if bf else capi.CUDA_F32
    f = rng.bf16_round if bf else (lambda a: a)
    shape = (units, S, hs)
    q, k, v, go = (f(rng.normal(seed, i, shape)) for i in range(4))
    scale = 1.0 / np.sqrt(hs)
    dq_, dk_, dv_, dgo = (DeviceBuffer.from_numpy(a, bf16=bf) for a in (q, k, v, go))
    es = 2 if bf else 4
    n = units * S * hs
    do_, dlse = DeviceBuffer(n * es), DeviceBuffer(units * S * 4)
    check(lib.boat_cuda_attn_fwd(mma, units, S, hs, int(causal), C.c_float(scale), dq_.p, dk_.p, dv_.p, io, do_.p, dlse.p),
          "attn_fwd")
    check(lib.boat_cuda_sync(), "sync")
    got = {"o": do_.numpy(shape, bf16=bf), "lse": dlse.numpy((units, S))}
    if backward:
        gq, gk, gv = DeviceBuffer(n * es), DeviceBuffer(n * es), DeviceBuffer(n * es)
        nbytes = lib.boat_cuda_attn_bwd_scratch_bytes(mma, units, S, hs)
        scratch = DeviceBuffer(max(nbytes, 256))
        check(lib.boat_cuda_attn_bwd(mma, units, S, hs, int(causal), C.c_float(scale), dq_.p, dk_.p, dv_.p, do_.p, dgo.p,
                                     dlse.p, io, gq.p, gk.p, gv.p, scratch.p, scratch.nbytes), "attn_bwd")
        check(lib.boat_cuda_sync(), "sync")
        got.update(dq=gq.numpy(shape, bf16=bf), dk=gk.numpy(shape, bf16=bf), dv=gv.numpy(shape, bf16=bf))
    ref = np_core(q, k, v, go if backward else None, causal, scale)
    return got, ref


@pytest.mark.parametrize("mma,hs", [(capi.MMA_FP32, 16), (capi.MMA_FP32, 64), (capi.MMA_BF16, 64), (capi.MMA_BF16, 128),
                                    (capi.MMA_TF32, 64)], ids=["fp32_hs16", "fp32_hs64", "bf16_hs64", "bf16_hs128", "tf32_hs64"])
@pytest.mark.parametrize("S", [128, 384, 1024])
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
def test_attention_core_matches_float64(gpu_lib, mma, hs, S, causal):
    got, ref = run_core(gpu_lib, mma, 3, S, hs, causal)
    tol = TOL[mma]
    for key in ("o", "dq", "dk", "dv"):
        assert np.isfinite(got[key]).all(), key
        assert rel(got[key], ref[key]) <= tol, (key, rel(got[key], ref[key]))
    assert np.abs(got["lse"] - ref["lse"]).max() <= (1e-4 if mma == capi.MMA_FP32 else 2e-2)


def test_attention_core_large_scores_do_not_overflow(gpu_lib):
    """Rows whose running max keeps growing exercise the rescale of the accumulator."""
    lib = gpu_lib
    units, S, hs = 2, 512, 64
    q = rng.bf16_round(rng.normal(11, 0, (units, S, hs)) * 6.0)
    k = rng.bf16_round(rng.normal(11, 1, (units, S, hs)) * np.linspace(0.2, 6.0, S)[None, :, None])
    v = rng.bf16_round(rng.normal(11, 2, (units, S, hs)))
    scale = 1.0 / np.sqrt(hs)
    bufs = [DeviceBuffer.from_numpy(a, bf16=True) for a in (q, k, v)]
    do_, dlse = DeviceBuffer(q.size * 2), DeviceBuffer(units * S * 4)
    check(lib.boat_cuda_attn_fwd(capi.MMA_BF16, units, S, hs, 0, C.c_float(scale), bufs[0].p, bufs[1].p, bufs[2].p,
                                 capi.CUDA_BF16, do_.p, dlse.p))
    check(lib.boat_cuda_sync())
    ref = np_core(q, k, v, None, False, scale)
    o = do_.numpy((units, S, hs), bf16=True)
    assert np.isfinite(o).all()
    assert rel(o, ref["o"]) <= TOL[capi.MMA_BF16]


def test_round_tf32_is_round_to_nearest_on_10_mantissa_bits(gpu_lib):
    lib = gpu_lib
    for n in (5, 4096, 100001):
        x = rng.normal(9, 0, (n,)) * np.float32(3.7)
        dx, dy = DeviceBuffer.from_numpy(x), DeviceBuffer(n * 4)
        check(lib.boat_cuda_round_tf32(dy.p, dx.p, n))
        y = dy.numpy((n,))
        assert not (y.view(np.uint32) & np.uint32(0x1FFF)).any()          # low 13 mantissa bits are clear
        assert np.abs(y - x).max() <= np.abs(x).max() * 2.0 ** -11 * 1.0001   # within half a TF32 ulp
        check(lib.boat_cuda_round_tf32(dx.p, dx.p, n))                     # in place
        assert np.array_equal(dx.numpy((n,)), y)


def test_pinned_host_pool_reuses_blocks(gpu_lib):
    lib = gpu_lib
    big = 97 << 20                                       # larger than anything the other tests leave in the pool
    a = lib.boat_cuda_host_alloc(big)
    assert a
    assert lib.boat_cuda_host_free(a) == 0
    b = lib.boat_cuda_host_alloc(big - 4096)             # close enough in size: the same block comes back
    assert b == a
    c = lib.boat_cuda_host_alloc(big)
    assert c and c != b
    assert lib.boat_cuda_host_free(b) == 0 and lib.boat_cuda_host_free(c) == 0
    assert lib.boat_cuda_host_free(C.c_void_p(12345)) != 0


def test_profile_report_lists_kernel_families(gpu_lib):
    lib = gpu_lib
    check(lib.boat_cuda_profile_enable(1))
    run_gemm(lib, capi.MMA_BF16, 0, 0, 256, 256, 256)
    buf = C.create_string_buffer(4096)
    check(lib.boat_cuda_profile_report(buf, 4096))
    check(lib.boat_cuda_profile_enable(0))
    names = {line.split()[0]: float(line.split()[2]) for line in buf.value.decode().splitlines()}
    assert "gemm_tc_nn" in names and names["gemm_tc_nn"] > 0


def test_backward_schedules_one_and_two_walks_per_cta():
    """The tensor-core backward picks one or two key-tile walks per CTA from the problem size;
    BOAT_BWD_PAIR forces either.  The attention-core and layer parity tests must pass under both
    (sequence lengths of 1, 2, 3 and 8 tiles cover the unpaired middle tile and the causal pairing)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for forced in ("0", "1"):
        env = dict(os.environ, BOAT_BWD_PAIR=forced)
        proc = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "tests/test_kernels_gpu.py", "tests/test_parity_gpu.py",
                               "-k", "attention_core or bf16_tensor_core or chunked"],
                              cwd=root, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
        assert proc.returncode == 0, "BOAT_BWD_PAIR=%s:\n%s" % (forced, proc.stdout[-3000:])


# ---- several problems in one launch -------------------------------------------------------------

def _ptr_table(bufs):
    """ctypes array of device pointers (None entries become NULL)."""
    arr = (C.c_void_p * len(bufs))()
    for i, b in enumerate(bufs):
        arr[i] = None if b is None else b.p
    return arr


@pytest.mark.parametrize("mma", [capi.MMA_BF16, capi.MMA_TF32, capi.MMA_FP32], ids=["bf16", "tf32", "fp32"])
@pytest.mark.parametrize("layout", LAYOUTS, ids=["nn", "nt", "tn"])
@pytest.mark.parametrize("shape,groups,shared_a", [((512, 512, 256), 3, True), ((1024, 256, 512), 3, False),
                                                   ((256, 768, 8192), 3, True), ((384, 256, 192), 2, False),
                                                   ((128, 1024, 128), 4, False), ((64, 40, 24), 3, False)],
                         ids=["shared_x", "distinct", "long_k_split", "two", "four", "cuda_core_shape"])
def test_grouped_gemm_equals_single_calls(gpu_lib, mma, layout, shape, groups, shared_a):
    """boat_cuda_gemm_grouped against `groups` boat_cuda_gemm calls on the same operands: the same
    bits when no K split is involved (one accumulation order), within the arithmetic's tolerance
    when pieces of K are added by atomics."""
    lib = gpu_lib
    M, N, K = shape
    ta, tb = layout
    bf = mma == capi.MMA_BF16
    typ = capi.CUDA_BF16 if bf else capi.CUDA_F32
    a_shape = (K, M) if ta else (M, K)
    b_shape = (N, K) if tb else (K, N)
    hA = [rng.normal(11, 0 if shared_a else g, a_shape) for g in range(groups)]
    hB = [rng.normal(12, g, b_shape, std=1.0 / np.sqrt(K)) for g in range(groups)]
    hbias = [rng.normal(13, g, (N,)) if g != 1 else None for g in range(groups)]        # one group without a bias
    if bf:
        hA, hB = [rng.bf16_round(x) for x in hA], [rng.bf16_round(x) for x in hB]
    dA0 = DeviceBuffer.from_numpy(hA[0], bf16=bf)
    dA = [dA0 if shared_a else DeviceBuffer.from_numpy(hA[g], bf16=bf) for g in range(groups)]
    dB = [DeviceBuffer.from_numpy(hB[g], bf16=bf) for g in range(groups)]
    dbias = [None if b is None else DeviceBuffer.from_numpy(b) for b in hbias]
    for out_type in sorted({typ, capi.CUDA_F32}):
        split_possible = out_type == capi.CUDA_F32      # FP32 outputs of few tiles with a long K are summed by atomics
        osz = 2 if out_type == capi.CUDA_BF16 else 4
        single = [DeviceBuffer(M * N * osz) for _ in range(groups)]
        grouped = [DeviceBuffer(M * N * osz) for _ in range(groups)]
        for g in range(groups):
            check(lib.boat_cuda_gemm(mma, ta, tb, M, N, K, dA[g].p, a_shape[1], dB[g].p, b_shape[1], typ, single[g].p, N,
                                     out_type, None if dbias[g] is None else dbias[g].p), "gemm")
        check(lib.boat_cuda_gemm_grouped(mma, ta, tb, groups, M, N, K, _ptr_table(dA), a_shape[1], _ptr_table(dB),
                                         b_shape[1], typ, _ptr_table(grouped), N, out_type, _ptr_table(dbias)), "grouped")
        check(lib.boat_cuda_sync(), "sync")
        for g in range(groups):
            one = single[g].numpy((M, N), bf16=out_type == capi.CUDA_BF16)
            many = grouped[g].numpy((M, N), bf16=out_type == capi.CUDA_BF16)
            opA = hA[g].T if ta else hA[g]
            opB = hB[g].T if tb else hB[g]
            ref = opA.astype(np.float64) @ opB.astype(np.float64) + (0 if hbias[g] is None else hbias[g].astype(np.float64))
            assert rel(many, ref) <= TOL[mma], (g, out_type)
            if not (split_possible and K >= 2048):
                assert np.array_equal(one, many), (g, out_type)


def test_grouped_gemm_argument_errors(gpu_lib):
    lib = gpu_lib
    buf = DeviceBuffer(128 * 128 * 4)
    tab = _ptr_table([buf, buf])
    assert lib.boat_cuda_gemm_grouped(capi.MMA_TF32, 0, 0, 0, 128, 128, 128, tab, 128, tab, 128, capi.CUDA_F32, tab, 128,
                                      capi.CUDA_F32, None) != 0
    assert lib.boat_cuda_gemm_grouped(capi.MMA_TF32, 0, 0, 5, 128, 128, 128, tab, 128, tab, 128, capi.CUDA_F32, tab, 128,
                                      capi.CUDA_F32, None) != 0
    assert lib.boat_cuda_gemm_grouped(capi.MMA_TF32, 0, 0, 2, 128, 128, 128, None, 128, tab, 128, capi.CUDA_F32, tab, 128,
                                      capi.CUDA_F32, None) != 0
    hole = _ptr_table([buf, None])
    assert lib.boat_cuda_gemm_grouped(capi.MMA_TF32, 0, 0, 2, 128, 128, 128, hole, 128, tab, 128, capi.CUDA_F32, tab, 128,
                                      capi.CUDA_F32, None) != 0


@pytest.mark.parametrize("bf", [True, False], ids=["bf16", "f32"])
@pytest.mark.parametrize("rows,cols,count", [(4096, 1024, 3), (333, 72, 2), (8, 2048, 4), (1000, 13, 3)])
def test_colsum_multi(gpu_lib, bf, rows, cols, count):
    """Column sums of several matrices in one launch, with the outputs next to one another (as in
    the layer's gradient bucket) and apart."""
    lib = gpu_lib
    hx = [rng.normal(21, i, (rows, cols)) for i in range(count)]
    if bf:
        hx = [rng.bf16_round(x) for x in hx]
    dx = [DeviceBuffer.from_numpy(x, bf16=bf) for x in hx]
    packed = DeviceBuffer(count * cols * 4)
    apart = [DeviceBuffer(cols * 4) for _ in range(count)]
    out_packed = (C.c_void_p * count)(*[packed.p.value + i * cols * 4 for i in range(count)])
    typ = capi.CUDA_BF16 if bf else capi.CUDA_F32
    check(lib.boat_cuda_colsum_multi(_ptr_table(dx), typ, rows, cols, out_packed, count), "colsum_multi")
    check(lib.boat_cuda_colsum_multi(_ptr_table(dx), typ, rows, cols, _ptr_table(apart), count), "colsum_multi")
    check(lib.boat_cuda_sync(), "sync")
    got = packed.numpy((count, cols))
    for i in range(count):
        ref = hx[i].astype(np.float64).sum(axis=0)
        scale = np.abs(hx[i]).astype(np.float64).sum(axis=0).max()
        assert np.abs(got[i] - ref).max() <= 1e-6 * scale
        assert np.abs(apart[i].numpy((cols,)) - ref).max() <= 1e-6 * scale


@pytest.mark.parametrize("sizes", [(1 << 20, 1 << 20, 1 << 20, 1 << 20), (4096, 8, 100000, 24), (7, 1001, 64)])
def test_convert_multi_equals_single_conversions(gpu_lib, sizes):
    """Several FP32 tensors to BF16 / to TF32-valued FP32 in one launch: the bits of boat_cuda_cast /
    boat_cuda_round_tf32 on each."""
    lib = gpu_lib
    hx = [rng.normal(31, i, (n,)) for i, n in enumerate(sizes)]
    dx = [DeviceBuffer.from_numpy(x) for x in hx]
    counts = (C.c_int64 * len(sizes))(*sizes)
    for dst_type, esz in ((capi.CUDA_BF16, 2), (capi.CUDA_F32_TF32, 4)):
        many = [DeviceBuffer(n * esz) for n in sizes]
        one = [DeviceBuffer(n * esz) for n in sizes]
        check(lib.boat_cuda_convert_multi(_ptr_table(many), dst_type, _ptr_table(dx), counts, len(sizes)), "convert_multi")
        for i, n in enumerate(sizes):
            if dst_type == capi.CUDA_BF16:
                check(lib.boat_cuda_cast(one[i].p, capi.CUDA_BF16, dx[i].p, capi.CUDA_F32, n), "cast")
            else:
                check(lib.boat_cuda_round_tf32(one[i].p, dx[i].p, n), "round_tf32")
        check(lib.boat_cuda_sync(), "sync")
        for i, n in enumerate(sizes):
            bf = dst_type == capi.CUDA_BF16
            assert np.array_equal(many[i].numpy((n,), bf16=bf), one[i].numpy((n,), bf16=bf)), (dst_type, i)
    assert lib.boat_cuda_convert_multi(_ptr_table(dx), capi.CUDA_F32, _ptr_table(dx), counts, len(sizes)) != 0


@pytest.mark.parametrize("mma", [capi.MMA_BF16, capi.MMA_TF32], ids=["bf16", "tf32"])
@pytest.mark.parametrize("layout", LAYOUTS, ids=["nn", "nt", "tn"])
def test_gemm_one_cta_per_tile_gives_the_same_bits(gpu_lib, mma, layout):
    """boat_cuda_gemm_set_yielding(1): one CTA per output tile instead of one persistent CTA per SM
    (the attention backward uses it beside a running gradient sum) - the same tiles, the same
    accumulation order, the same bits; more tiles than SMs so that the two launches really differ."""
    lib = gpu_lib
    M, N, K = 4096, 2048, 512          # 256 tiles of 128 x 256
    try:
        got_persistent, ref = run_gemm(lib, mma, layout[0], layout[1], M, N, K, out_bf16=mma == capi.MMA_BF16)
        check(lib.boat_cuda_gemm_set_yielding(1), "set_yielding")
        got_yielding, _ = run_gemm(lib, mma, layout[0], layout[1], M, N, K, out_bf16=mma == capi.MMA_BF16)
    finally:
        check(lib.boat_cuda_gemm_set_yielding(0), "set_yielding")
    assert rel(got_persistent, ref) <= TOL[mma]
    assert np.array_equal(got_persistent, got_yielding)
