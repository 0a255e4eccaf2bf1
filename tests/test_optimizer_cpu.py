"""Adam on the CPU side: the restatement in oracle/optimizer_oracle.c against the reference's
golden vectors and against the reference library itself, plus the parts of the optimizer API
that need no GPU (argument checks, learning-rate access)."""
import os

import numpy as np
import pytest

import cases
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def adam_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "adam_golden.npz"))


def test_restatement_reproduces_reference_golden_after_every_step(adam_golden):
    params, grads = cases.adam_inputs()
    for steps in range(1, len(grads) + 1):
        got = oracle.port_adam(params, grads[:steps], **cases.ADAM_HYPER)
        for i, p in enumerate(got):
            assert np.array_equal(p.reshape(-1), adam_golden["step%d/p%d" % (steps, i)].reshape(-1)), (steps, i)


@pytest.mark.skipif(not oracle.have_ref(), reason="reference library not built here")
def test_restatement_equals_reference_library_over_many_steps():
    # 40 steps: the bias corrections 1 - beta^t move through several binades of beta2^t
    params, grads = cases.adam_inputs(shapes=((257,), (16, 9)), steps=40, stream=70)
    hyper = dict(lr=0.05, beta1=0.8, beta2=0.99, eps=1e-6)
    want = oracle.ref_adam(params, grads, **hyper)
    got = oracle.port_adam(params, grads, **hyper)
    for a, b in zip(got, want):
        assert np.array_equal(a.reshape(-1), b.reshape(-1))


def test_zero_gradient_leaves_parameters_unchanged():
    p = [np.arange(5, dtype=np.float32)]
    got = oracle.port_adam(p, [[np.zeros(5, np.float32)]], **cases.ADAM_HYPER)
    assert np.array_equal(got[0], p[0])


def test_create_rejects_what_the_reference_rejects(lib):
    # adam.c:37-49 and the reference's tests/unit/test_optimizer_adam.c, test 1
    assert lib.boat_adam_optimizer_create(0.0, 0.9, 0.999, 1e-8) is None
    assert lib.boat_adam_optimizer_create(-1.0, 0.9, 0.999, 1e-8) is None
    assert lib.boat_adam_optimizer_create(0.001, 1.1, 0.999, 1e-8) is None
    assert lib.boat_adam_optimizer_create(0.001, 0.0, 0.999, 1e-8) is None
    assert lib.boat_adam_optimizer_create(0.001, 0.9, 1.5, 1e-8) is None
    assert lib.boat_adam_optimizer_create(0.001, 0.9, 1.0, 1e-8) is None
    # SGD's create function is a stub in the reference (optimizer_common.c:77-82)
    assert lib.boat_sgd_optimizer_create(0.1, 0.9) is None


def test_learning_rate_access_and_null_handling(lib):
    opt = lib.boat_adam_optimizer_create(0.001, 0.9, 0.999, 1e-8)
    assert opt
    assert lib.boat_optimizer_get_learning_rate(opt) == pytest.approx(0.001)
    lib.boat_optimizer_set_learning_rate(opt, 0.5)
    assert lib.boat_optimizer_get_learning_rate(opt) == 0.5
    lib.boat_optimizer_step(opt)          # nothing registered: only the timestep moves
    lib.boat_optimizer_zero_grad(opt)
    lib.boat_optimizer_add_parameter(opt, None, None)
    lib.boat_optimizer_free(opt)
    # NULL optimizer: every entry point is a no-op, as in optimizer_common.c
    assert lib.boat_optimizer_get_learning_rate(None) == 0.0
    lib.boat_optimizer_step(None)
    lib.boat_optimizer_zero_grad(None)
    lib.boat_optimizer_set_learning_rate(None, 1.0)
    lib.boat_optimizer_free(None)
