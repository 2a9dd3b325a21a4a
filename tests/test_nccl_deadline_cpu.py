"""Failure handling of the NCCL exchange path, on the CPU, against a stand-in for NCCL.

qm_nccl_wait is the host loop that keeps a hung or broken collective from blocking a rank for ever: it polls the
stream and the communicator's asynchronous error and aborts the communicator when an error shows up or a deadline
passes.  Here the NCCL functions and the stream query are replaced through qm_nccl_set_api by Python callbacks, so
every branch runs without a GPU and without NCCL: a collective that completes, one that reports an asynchronous
error, one that never completes (a rank that left), a stream that fails, and a failing status query.
"""
import ctypes
import time
from ctypes import CFUNCTYPE, POINTER, c_int, c_size_t, c_void_p

import pytest

NCCL_SUCCESS, NCCL_SYSTEM_ERROR, NCCL_IN_PROGRESS = 0, 2, 7

ALL_GATHER = CFUNCTYPE(c_int, c_void_p, c_void_p, c_size_t, c_int, c_void_p, c_void_p)
GET_ASYNC = CFUNCTYPE(c_int, c_void_p, POINTER(c_int))
ABORT = CFUNCTYPE(c_int, c_void_p)
COUNT = CFUNCTYPE(c_int, c_void_p, POINTER(c_int))
ERROR_STRING = CFUNCTYPE(c_void_p, c_int)     # a char*; the text lives in a buffer the fake owns
STREAM_QUERY = CFUNCTYPE(c_int, c_void_p)


class Api(ctypes.Structure):
    _fields_ = [("all_gather", ALL_GATHER), ("comm_get_async_error", GET_ASYNC), ("comm_abort", ABORT),
                ("comm_count", COUNT), ("get_error_string", ERROR_STRING), ("stream_query", STREAM_QUERY)]


class FakeNccl:
    """Scripted behaviour: the stream finishes after `busy_polls` queries (never if None); the communicator reports
    `async_error` from poll `error_after` on; `query_result` is what ncclCommGetAsyncError itself returns."""

    def __init__(self, busy_polls=None, async_error=NCCL_SUCCESS, error_after=0, query_result=NCCL_SUCCESS,
                 stream_fails_after=None):
        self.busy_polls, self.async_error, self.error_after = busy_polls, async_error, error_after
        self.query_result, self.stream_fails_after = query_result, stream_fails_after
        self.polls = self.aborts = 0

        def all_gather(send, recv, count, dtype, comm, stream):
            return NCCL_SUCCESS

        def get_async(comm, out):
            out[0] = self.async_error if self.polls > self.error_after else NCCL_IN_PROGRESS
            return self.query_result

        def abort(comm):
            self.aborts += 1
            return NCCL_SUCCESS

        def count(comm, out):
            out[0] = 2
            return NCCL_SUCCESS

        self.text = ctypes.create_string_buffer(b"scripted failure")

        def error_string(code):
            return ctypes.addressof(self.text)

        def stream_query(stream):
            self.polls += 1
            if self.stream_fails_after is not None and self.polls > self.stream_fails_after:
                return -1
            if self.busy_polls is not None and self.polls > self.busy_polls:
                return 0
            return 1

        # the callback objects must outlive the table
        self.keep = [ALL_GATHER(all_gather), GET_ASYNC(get_async), ABORT(abort), COUNT(count), ERROR_STRING(error_string),
                     STREAM_QUERY(stream_query)]
        self.table = Api(*self.keep)


@pytest.fixture
def lib(qm):
    library = qm.load_library()
    yield library
    library.qm_nccl_set_api(None)


def install(lib, fake):
    assert lib.qm_nccl_set_api(ctypes.byref(fake.table)) == 0


COMM = c_void_p(0x1234)     # never dereferenced: every NCCL function is the stand-in's


def test_collective_that_completes_returns_ok_without_abort(lib, qm):
    fake = FakeNccl(busy_polls=5)
    install(lib, fake)
    assert lib.qm_nccl_wait(COMM, None, 2000) == qm.QM_OK
    assert fake.aborts == 0 and fake.polls == 6


def test_asynchronous_error_aborts_the_communicator(lib, qm):
    fake = FakeNccl(busy_polls=None, async_error=NCCL_SYSTEM_ERROR, error_after=3)
    install(lib, fake)
    assert lib.qm_nccl_wait(COMM, None, 5000) == qm.QM_ENCCL
    assert fake.aborts == 1
    assert b"scripted failure" in lib.qm_last_error_string()


def test_rank_that_never_arrives_hits_the_deadline(lib, qm):
    fake = FakeNccl(busy_polls=None)          # the stream never finishes, NCCL keeps saying "in progress"
    install(lib, fake)
    t0 = time.time()
    assert lib.qm_nccl_wait(COMM, None, 300) == qm.QM_ETIMEOUT
    assert 0.25 <= time.time() - t0 < 5.0
    assert fake.aborts == 1
    assert b"deadline" in lib.qm_last_error_string()


def test_stream_error_aborts_too(lib, qm):
    fake = FakeNccl(busy_polls=None, stream_fails_after=2)
    install(lib, fake)
    assert lib.qm_nccl_wait(COMM, None, 5000) == qm.QM_ECUDA
    assert fake.aborts == 1


def test_failing_status_query_counts_as_failure(lib, qm):
    fake = FakeNccl(busy_polls=None, query_result=NCCL_SYSTEM_ERROR)
    install(lib, fake)
    assert lib.qm_nccl_wait(COMM, None, 5000) == qm.QM_ENCCL
    assert fake.aborts == 1


def test_arguments_are_checked(lib, qm):
    fake = FakeNccl(busy_polls=0)
    install(lib, fake)
    assert lib.qm_nccl_wait(None, None, 10) == qm.QM_EINVAL
    assert lib.qm_nccl_wait(COMM, None, -1) == qm.QM_EINVAL
    incomplete = Api()
    assert lib.qm_nccl_set_api(ctypes.byref(incomplete)) == qm.QM_EINVAL
    # the sharded entry point refuses a world that disagrees with the communicator before it launches anything
    assert lib.qm_decode_attention_sharded(None, 0, None, None, None, 1, 1, 16, None, c_void_p(8), c_void_p(8), 4, None, 0,
                                           COMM, None) == qm.QM_EINVAL
    assert b"rank count" in lib.qm_last_error_string()
