"""Host-side failure handling (no GPU): tgaf_watchdog_wait is the loop tgaf_synchronize runs while a
context holds a communicator - poll the stream, poll the collective library's asynchronous error state,
abort the communicator on an error or at the wall-clock limit.  Here its three hooks are a fake of the
collective library's table: a rank that never joins is a stream that never finishes."""
import ctypes as C
import time

import pytest

OK, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT = 0, 2, 4, 6


@pytest.fixture(scope="module")
def lib():
    from talu_b200 import build, _capi
    build.build()
    return _capi.load()


class FakeComm:
    """work_done turns 1 after `finish_after` polls (never when None); the async error appears after
    `error_after` polls."""

    def __init__(self, finish_after=None, error_after=None, fail_stream=False):
        self.finish_after, self.error_after, self.fail_stream = finish_after, error_after, fail_stream
        self.polls = self.error_polls = self.aborts = 0

    def fns(self):
        from talu_b200 import _capi

        def work_done(_):
            self.polls += 1
            if self.fail_stream:
                return -1
            return 1 if self.finish_after is not None and self.polls > self.finish_after else 0

        def async_error(_):
            self.error_polls += 1
            return 5 if self.error_after is not None and self.error_polls > self.error_after else 0

        def abort(_):
            self.aborts += 1

        self._keep = (_capi.WORK_DONE_FN(work_done), _capi.ASYNC_ERROR_FN(async_error), _capi.ABORT_FN(abort))
        return _capi.WatchFns(*self._keep)


def wait(lib, fake, timeout_ms):
    fns = fake.fns()
    return lib.tgaf_watchdog_wait(C.byref(fns), None, timeout_ms)


def test_finishes(lib):
    f = FakeComm(finish_after=100)
    assert wait(lib, f, 5000) == OK
    assert f.aborts == 0 and f.polls == 101


def test_missing_rank_times_out_and_aborts(lib):
    f = FakeComm(finish_after=None)
    t0 = time.perf_counter()
    assert wait(lib, f, 150) == ERR_TIMEOUT
    dt = time.perf_counter() - t0
    assert 0.14 <= dt < 2.0, dt
    assert f.aborts == 1


def test_async_error_aborts(lib):
    f = FakeComm(finish_after=None, error_after=20)
    assert wait(lib, f, 5000) == ERR_NCCL
    assert f.aborts == 1 and f.error_polls == 21


def test_stream_failure_is_a_cuda_status(lib):
    f = FakeComm(fail_stream=True)
    assert wait(lib, f, 5000) == ERR_CUDA
    assert f.aborts == 0


def test_optional_hooks_and_bad_arguments(lib):
    from talu_b200 import _capi
    assert lib.tgaf_watchdog_wait(None, None, 10) == 1
    n = [0]

    def done(_):
        n[0] += 1
        return 1 if n[0] > 3 else 0

    fns = _capi.WatchFns(_capi.WORK_DONE_FN(done), _capi.ASYNC_ERROR_FN(0), _capi.ABORT_FN(0))
    assert lib.tgaf_watchdog_wait(C.byref(fns), None, 0) == OK       # no limit, no error hook
    never = _capi.WatchFns(_capi.WORK_DONE_FN(lambda _: 0), _capi.ASYNC_ERROR_FN(0), _capi.ABORT_FN(0))
    assert lib.tgaf_watchdog_wait(C.byref(never), None, 20) == ERR_TIMEOUT   # no abort hook: just the status
