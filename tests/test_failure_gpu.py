"""The ZN_ERR_TIMEOUT path on a GPU, in forms that fault, trap or hang nothing: a bounded wait that is
allowed to run out (a barrier nothing arrives at, a limit of a few thousand cycles, the kernel returns
normally) and a status word written from the host.  After either, the error is reported once, the word is
cleared and the context computes as before."""
import numpy as np
import pytest

import zigneuron_b200 as zn
from util import assert_close, round_bf16

pytestmark = pytest.mark.gpu
ZN_ERR_TIMEOUT = 9


def gemm_still_works(be):
    rng = np.random.default_rng(5)
    m, n, k = 300, 260, 200
    a, b = round_bf16(rng.standard_normal((m, k))), round_bf16(rng.standard_normal((k, n)))
    c = np.zeros((m, n), np.float32)
    be.matMul(a, b, c, m, n, k)
    assert_close(c, a.astype(np.float64) @ b.astype(np.float64), 1e-5, "GEMM after a reported timeout")


def test_bounded_wait_runs_out_and_is_reported_once():
    be = zn.Backend(0, zn.Precision.BF16_TC)
    gemm_still_works(be)
    be.debug_bounded_wait_probe(20000)            # ~10 microseconds of waiting, then the kernel gives up
    with pytest.raises(zn.ZnError) as ei:
        be.endCommandBatch()
    assert ei.value.status == ZN_ERR_TIMEOUT and "code 99" in str(ei.value)
    be.endCommandBatch()                          # the word was cleared by the report
    gemm_still_works(be)
    be.deinit()


def test_first_code_wins_and_later_calls_are_clean():
    be = zn.Backend(0, zn.Precision.BF16_TC)
    be.debug_bounded_wait_probe(5000)
    be.debug_bounded_wait_probe(5000)             # the second kernel finds the word taken and leaves it
    with pytest.raises(zn.ZnError) as ei:
        be.endCommandBatch()
    assert ei.value.status == ZN_ERR_TIMEOUT
    be.endCommandBatch()
    with pytest.raises(zn.ZnError):
        be.debug_bounded_wait_probe(-1)
    be.deinit()


def test_status_word_written_from_the_host_surfaces_in_the_next_call():
    be = zn.Backend(0, zn.Precision.FP32_SIMT)
    net = zn.Network(be, zn.Precision.FP32_SIMT)
    net.addDense(8, 4, "linear")
    x = np.ones((2, 8), np.float32)
    t = np.zeros((2, 4), np.float32)
    net.trainStep(x, t, 0.01, zn.Loss.mse)
    be.debug_set_device_status(13)                # what a GEMM's mbarrier wait writes when it gives up
    with pytest.raises(zn.ZnError) as ei:
        net.trainStep(x, t, 0.01, zn.Loss.mse)
    assert ei.value.status == ZN_ERR_TIMEOUT and "code 13" in str(ei.value)
    loss = net.trainStep(x, t, 0.01, zn.Loss.mse)  # cleared; the network keeps training
    assert np.isfinite(loss)
    net.deinit()
    be.deinit()
