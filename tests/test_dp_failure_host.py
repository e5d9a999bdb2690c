"""CPU: failure handling of the data-parallel layer, with the failures made on the host.

No GPU is faulted, trapped or hung by any of this: NCCL is replaced by an in-process stand-in that moves no data
(ts_dp_install_fake_nccl), so that a rank that never joins the rendezvous, a collective that returns an error and a
peer that dies (an asynchronous error on the communicator) can each be produced at will, and a rank 0 that never
publishes the communicator id is simply a file that never appears."""
import ctypes as C
import time

import pytest


@pytest.fixture
def fake_nccl(ts):
    lib = ts._ffi.lib()
    yield lib
    lib.ts_dp_finalize()
    lib.ts_dp_install_fake_nccl(-1)


def test_rendezvous_that_never_completes_times_out(ts, fake_nccl):
    lib = fake_nccl
    lib.ts_dp_install_fake_nccl(1)                  # the stand-in's ncclCommInitRank never returns: a peer never joined
    uid = ts.distributed.get_unique_id()
    t0 = time.monotonic()
    with pytest.raises(ts.TrainStationError, match="did not complete within 0.3 s"):
        ts.distributed.init(uid, 0, 2, timeout=0.3)
    assert 0.25 < time.monotonic() - t0 < 5.0
    assert ts.distributed.world_size() == 1         # nothing half-initialised is left behind
    # the same thread can join a healthy communicator afterwards
    lib.ts_dp_install_fake_nccl(0)
    ts.distributed.init(uid, 1, 2, timeout=5.0)
    assert (ts.distributed.rank(), ts.distributed.world_size()) == (1, 2)
    assert ts.distributed.healthy()


def test_asynchronous_error_aborts_the_communicator(ts, fake_nccl):
    lib = fake_nccl
    lib.ts_dp_install_fake_nccl(0)
    ts.distributed.init(ts.distributed.get_unique_id(), 0, 2, timeout=5.0)
    assert ts.distributed.healthy()
    aborts = lib.ts_dp_fake_nccl_aborts()
    lib.ts_dp_install_fake_nccl(3)                  # the peer dies: ncclCommGetAsyncError now reports a remote error
    assert not ts.distributed.healthy()
    assert "asynchronous error" in ts._ffi.last_error() and "aborted" in ts._ffi.last_error()
    assert lib.ts_dp_fake_nccl_aborts() == aborts + 1   # aborted exactly once, so that nothing can block on it any more
    assert not ts.distributed.healthy()                 # and it stays refused, without a second abort
    assert lib.ts_dp_fake_nccl_aborts() == aborts + 1
    assert "was aborted" in ts._ffi.last_error()
    # finalize resets the state; a new communicator can be created
    lib.ts_dp_finalize()
    lib.ts_dp_install_fake_nccl(0)
    ts.distributed.init(ts.distributed.get_unique_id(), 0, 2, timeout=5.0)
    assert ts.distributed.healthy()


def test_bad_rendezvous_arguments_are_refused(ts, fake_nccl):
    fake_nccl.ts_dp_install_fake_nccl(0)
    uid = ts.distributed.get_unique_id()
    for rank, world in ((2, 2), (-1, 2), (0, 0)):
        with pytest.raises(ts.TrainStationError, match="bad arguments"):
            ts.distributed.init(uid, rank, world, timeout=1.0)
    ts.distributed.init(uid, 0, 2, timeout=1.0)
    with pytest.raises(ts.TrainStationError, match="already initialised"):
        ts.distributed.init(uid, 0, 2, timeout=1.0)


def test_rank_zero_that_never_publishes_the_id(ts, tmp_path):
    t0 = time.monotonic()
    with pytest.raises(TimeoutError, match="did not publish"):
        ts.distributed.exchange_id_through_file(str(tmp_path / "nccl_id"), rank=1, timeout=0.2)
    assert time.monotonic() - t0 < 2.0
    # and the ordinary case: a published id is read back whole
    p = tmp_path / "id2"
    p.write_bytes(bytes(range(128)))
    assert ts.distributed.exchange_id_through_file(str(p), rank=3, timeout=1.0) == bytes(range(128))
