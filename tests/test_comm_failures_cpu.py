"""Failure handling of the gradient exchange (boat_cuda_comm_* in comm.cu), exercised on the
CPU against a stand-in NCCL library (tests/fake_nccl.c) that plays the failing peer: a rank
that never joins, an error while joining, a peer that dies before a collective is accepted, an
NCCL error from a collective, and a peer that brings a bucket of another size.  Every case must
end in an error status within the deadline, with the communicator aborted and the library back
to a world of one - never in a stuck host thread.  Each scenario runs in a process of its own,
because the loaded NCCL library and the communicator are process-wide."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def fake_lib(tmp_path_factory, lib):
    out = tmp_path_factory.mktemp("fake_nccl") / "libfake_nccl.so"
    subprocess.run(["gcc", "-O1", "-shared", "-fPIC", "-fvisibility=hidden", "-o", str(out),
                    os.path.join(ROOT, "tests", "fake_nccl.c")], check=True)
    return str(out)


def run_scenario(fake_lib, mode, body, extra_env=None, timeout=60):
    script = textwrap.dedent("""
        import ctypes as C, sys, time
        sys.path.insert(0, %r)
        from boat_b200 import capi
        lib = capi.load()
        fake = C.CDLL(%r, mode=C.RTLD_GLOBAL)
        ident = (C.c_ubyte * 128)()
        assert lib.boat_cuda_comm_unique_id(ident) == 0, lib.boat_cuda_last_error()
        def err():
            return lib.boat_cuda_last_error().decode()
    """ % (ROOT, fake_lib)) + textwrap.dedent(body)
    env = dict(os.environ, BOAT_NCCL_LIB=fake_lib, FAKE_NCCL_MODE=mode, BOAT_COMM_INIT_TIMEOUT_S="0.5",
               BOAT_COMM_TIMEOUT_S="0.5")
    env.update(extra_env or {})
    proc = subprocess.run([sys.executable, "-c", script], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                          text=True, timeout=timeout)
    assert proc.returncode == 0, proc.stdout[-3000:]
    return proc.stdout


def test_a_rank_that_never_joins_ends_in_an_error_and_an_abort(fake_lib):
    run_scenario(fake_lib, "never_joins", """
        t0 = time.perf_counter()
        rc = lib.boat_cuda_comm_init(0, 2, ident)
        waited = time.perf_counter() - t0
        assert rc == 23, (rc, err())
        assert "never joined" in err() and "aborted" in err()
        assert 0.4 < waited < 5.0, waited
        assert fake.fake_nccl_abort_count() == 1
        assert lib.boat_cuda_comm_world() == 1
        buf = (C.c_float * 4)(1, 2, 3, 4)
        assert lib.boat_cuda_allreduce_sum_f32(buf, 4) == 0        # a world of one: nothing to do
        assert list(buf) == [1, 2, 3, 4]
        assert lib.boat_cuda_comm_destroy() == 0
    """)


def test_an_error_while_joining_is_reported_with_nccls_text(fake_lib):
    run_scenario(fake_lib, "init_error", """
        rc = lib.boat_cuda_comm_init(0, 2, ident)
        assert rc == 2002, (rc, err())                               # 2000 + ncclSystemError
        assert "unhandled system error" in err()
        assert fake.fake_nccl_abort_count() == 1 and lib.boat_cuda_comm_world() == 1
    """)


def test_healthy_exchange_then_a_peer_with_another_bucket_size(fake_lib):
    run_scenario(fake_lib, "ok", """
        import os
        assert lib.boat_cuda_comm_init(0, 2, ident) == 0, err()
        assert lib.boat_cuda_comm_world() == 2
        assert lib.boat_cuda_comm_init(0, 2, ident) != 0               # a second communicator is refused
        buf = (C.c_float * 6)(*range(6))
        assert lib.boat_cuda_allreduce_sum_f32(buf, 6) == 0, err()
        assert list(buf) == [0, 2, 4, 6, 8, 10]                        # the stand-in peer brought the same values
        # overlapped form: two pieces in one group, then the join
        a, b = (C.c_float * 3)(1, 1, 1), (C.c_float * 2)(5, 5)
        ptrs = (C.c_void_p * 2)(C.addressof(a), C.addressof(b))
        counts = (C.c_int64 * 2)(3, 2)
        assert lib.boat_cuda_allreduce_begin(ptrs, counts, 2) == 0, err()
        assert lib.boat_cuda_allreduce_pending() == 1
        assert lib.boat_cuda_allreduce_join() == 0 and lib.boat_cuda_allreduce_pending() == 0
        assert list(a) == [2, 2, 2] and list(b) == [10, 10]
        # several starts before one join, as an encoder block's backward issues them (one per layer)
        c, d, e = (C.c_float * 4)(1, 2, 3, 4), (C.c_float * 1)(7), (C.c_float * 2)(0.5, -0.5)
        for arr in (c, d, e):
            one = (C.c_void_p * 1)(C.addressof(arr))
            assert lib.boat_cuda_allreduce_begin(one, (C.c_int64 * 1)(len(arr)), 1) == 0, err()
            assert lib.boat_cuda_allreduce_pending() == 1
        assert lib.boat_cuda_allreduce_join() == 0 and lib.boat_cuda_allreduce_pending() == 0
        assert list(c) == [2, 4, 6, 8] and list(d) == [14] and list(e) == [1.0, -1.0]
        assert lib.boat_cuda_allreduce_join() == 0                      # nothing under way: a no-op
        # from now on the peer claims 7 elements where this rank brings 8
        os.environ["FAKE_NCCL_PEER_COUNT"] = "7"
        big = (C.c_float * 8)(*([1.0] * 8))
        before = fake.fake_nccl_float_reduce_count()
        rc = lib.boat_cuda_allreduce_sum_f32(big, 8)
        assert rc == 25, (rc, err())
        assert "8 elements" in err() and "one size" in err()
        assert fake.fake_nccl_float_reduce_count() == before            # the mismatched sum was never issued
        assert list(big) == [1.0] * 8
        assert lib.boat_cuda_comm_world() == 2                          # the communicator itself is still fine
        assert lib.boat_cuda_allreduce_sum_f32(buf, 6) == 0             # a length agreed on earlier still works
        assert lib.boat_cuda_comm_destroy() == 0
        assert fake.fake_nccl_destroy_count() == 1 and lib.boat_cuda_comm_world() == 1
    """)


def test_a_peer_that_dies_before_the_collective_is_accepted(fake_lib):
    run_scenario(fake_lib, "peer_dies", """
        assert lib.boat_cuda_comm_init(0, 2, ident) == 0, err()
        buf = (C.c_float * 4)(1, 2, 3, 4)
        t0 = time.perf_counter()
        rc = lib.boat_cuda_allreduce_sum_f32(buf, 4)
        waited = time.perf_counter() - t0
        assert rc == 23 and "aborted" in err(), (rc, err())
        assert 0.4 < waited < 5.0, waited
        assert fake.fake_nccl_abort_count() == 1 and lib.boat_cuda_comm_world() == 1
        assert lib.boat_cuda_allreduce_sum_f32(buf, 4) == 0            # world of one again: a no-op, not a hang
    """)


def test_an_nccl_error_from_a_collective_aborts_the_communicator(fake_lib):
    run_scenario(fake_lib, "call_error", """
        assert lib.boat_cuda_comm_init(0, 2, ident) == 0, err()
        buf = (C.c_float * 4)(1, 2, 3, 4)
        rc = lib.boat_cuda_allreduce_sum_f32(buf, 4)
        assert rc == 2003 and "internal error" in err(), (rc, err())     # 2000 + ncclInternalError
        assert fake.fake_nccl_abort_count() == 1 and lib.boat_cuda_comm_world() == 1
        a = (C.c_float * 3)(1, 1, 1)
        ptrs, counts = (C.c_void_p * 1)(C.addressof(a)), (C.c_int64 * 1)(3)
        assert lib.boat_cuda_allreduce_begin(ptrs, counts, 1) == 0     # no communicator, one rank: nothing to do
        assert lib.boat_cuda_allreduce_pending() == 0
    """)
