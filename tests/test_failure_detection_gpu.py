"""The bounded waits of the tensor-core kernels, made to run out in a harmless way.

Nothing here hangs or faults a GPU: the self-test kernel waits a few milliseconds on a barrier
that only it could complete, gives up, records its role code and returns like any kernel.
The test checks what the host sees afterwards and that the library keeps working.
"""
import pytest

from boat_b200 import capi
from boat_b200.host import check
from test_kernels_gpu import run_gemm, rel, TOL

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_once_and_the_library_recovers(gpu_lib):
    lib = gpu_lib
    check(lib.boat_cuda_sync(), "sync before")
    check(lib.boat_cuda_selftest_wait_timeout(3_000_000), "selftest launch")          # 3 ms
    rc = lib.boat_cuda_sync()
    assert rc == 30, (rc, lib.boat_cuda_last_error())
    assert b"role code 9" in lib.boat_cuda_last_error()
    # the word was cleared by the report: the next synchronisation is clean
    assert lib.boat_cuda_sync() == 0
    # and real tensor-core kernels run normally afterwards
    got, ref = run_gemm(lib, capi.MMA_BF16, 0, 0, 512, 512, 512)
    assert rel(got, ref) <= TOL[capi.MMA_BF16]
    assert lib.boat_cuda_sync() == 0


def test_kernels_queued_behind_a_give_up_abort_their_waits_until_the_host_looks(gpu_lib):
    """The status word stays set until the host reads it; a kernel that starts a long wait while
    it is set gives up too (its results are invalid anyway).  After the report, all is normal."""
    lib = gpu_lib
    check(lib.boat_cuda_selftest_wait_timeout(1_000_000), "selftest launch")
    check(lib.boat_cuda_selftest_wait_timeout(500_000_000), "second selftest launch")   # would wait 0.5 s
    import time
    t0 = time.perf_counter()
    rc = lib.boat_cuda_sync()
    waited = time.perf_counter() - t0
    assert rc == 30
    assert waited < 0.4, "the second wait should have seen the first one's code and stopped early (%.3f s)" % waited
    assert lib.boat_cuda_sync() == 0


def test_selftest_rejects_limits_it_will_not_wait_for(gpu_lib):
    assert gpu_lib.boat_cuda_selftest_wait_timeout(0) != 0
    assert gpu_lib.boat_cuda_selftest_wait_timeout(2_000_000_000) != 0
    assert gpu_lib.boat_cuda_sync() == 0
