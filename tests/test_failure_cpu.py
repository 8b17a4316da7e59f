"""Failure detection, the part that needs no GPU: the polling loop every data-parallel host wait runs
(zn_wait_poll) driven by fakes of its three questions -- is the work done, has the communicator
reported an error, has the deadline passed.  The failures are made on the host: a completion that
never comes, an error code from a fake of the communicator query."""
import ctypes as C
import time

from zigneuron_b200 import _lib

READY, COMM_ERROR, DEADLINE, QUERY_FAILED = 0, 1, 2, 3
READY_FN = C.CFUNCTYPE(C.c_int, C.c_void_p)
ERROR_FN = C.CFUNCTYPE(C.c_int, C.c_void_p)


def poll(ready, comm_error, deadline_ms):
    calls = {"ready": 0, "error": 0}

    def r(_):
        calls["ready"] += 1
        return ready(calls["ready"])

    def e(_):
        calls["error"] += 1
        return comm_error(calls["error"])

    rf, ef = READY_FN(r), ERROR_FN(e)
    code = C.c_int32(-1)
    res = _lib.lib.zn_wait_poll(C.cast(rf, C.c_void_p), C.cast(ef, C.c_void_p) if comm_error else None, None,
                                deadline_ms, C.byref(code))
    return res, code.value, calls


def test_completion_is_reported_without_asking_anything_else_first():
    res, code, calls = poll(lambda n: 1, lambda n: 7, 1000)
    assert res == READY and code == 0 and calls["ready"] == 1 and calls["error"] == 0


def test_completion_after_a_while():
    t0 = time.perf_counter()
    res, code, calls = poll(lambda n: 1 if time.perf_counter() - t0 > 0.02 else 0, lambda n: 0, 5000)
    assert res == READY and code == 0
    assert calls["error"] >= 5          # the communicator was asked about once a millisecond meanwhile


def test_communicator_error_ends_the_wait_with_its_code():
    # the work never completes (a peer rank is gone); the third health check reports error 6
    res, code, calls = poll(lambda n: 0, lambda n: 6 if n >= 3 else 0, 60000)
    assert res == COMM_ERROR and code == 6 and calls["error"] == 3


def test_deadline_ends_a_wait_that_nothing_else_would():
    t0 = time.perf_counter()
    res, code, _ = poll(lambda n: 0, lambda n: 0, 50)
    dt = time.perf_counter() - t0
    assert res == DEADLINE and code == 0 and 0.05 <= dt < 1.0


def test_deadline_without_a_communicator_query():
    res, _, calls = poll(lambda n: 0, None, 20)
    assert res == DEADLINE and calls["error"] == 0


def test_failed_completion_query_is_its_own_outcome():
    res, _, _ = poll(lambda n: -1 if n >= 4 else 0, lambda n: 0, 1000)
    assert res == QUERY_FAILED
    assert _lib.lib.zn_wait_poll(None, None, None, 10, None) == QUERY_FAILED


def test_dp_timeout_needs_a_context():
    assert _lib.lib.zn_dp_set_timeout_ms(None, 1000) == 3           # ZN_ERR_NOT_INITIALIZED
    assert _lib.lib.zn_debug_set_device_status(None, 1) == 3
    assert _lib.lib.zn_debug_bounded_wait_probe(None, 1000) == 3
