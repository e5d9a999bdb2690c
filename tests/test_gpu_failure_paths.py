"""GPU: the error-reporting paths, exercised without faulting, trapping or hanging anything.

* The device error word: a host-side write of a code into it (a plain copy) must make the next ts_sync_stream fail
  with that code in the message, exactly once.
* A bounded wait that runs out: the one-CTA tensor-core GEMM is launched with a main-loop wait budget of zero cycles, so
  the first wait that is not already satisfied gives up.  The kernel must record an error code, drain its own copies
  (that bound stays at its full two seconds), free its tensor memory and RETURN; the host reads the code at its next
  synchronisation, and an ordinary GEMM on the same context afterwards is exact.
"""
import numpy as np
import pytest

from devbuf import DevBuf

pytestmark = pytest.mark.gpu


def test_error_word_written_from_the_host_is_reported_once(gpu):
    lib = gpu._ffi.lib()
    assert lib.ts_sync_stream(None) is True
    word = lib.ts_device_error_word()
    assert word
    code = np.array([104], np.int32)
    gpu._ffi.check(lib.cuda_memcpy(word, code.ctypes.data, 1, 0), "write the error word")   # one 4-byte element, host to device
    assert lib.ts_sync_stream(None) is False
    msg = gpu._ffi.last_error()
    assert "104" in msg and "bounded wait" in msg
    assert lib.ts_sync_stream(None) is True          # reported once, then cleared
    with pytest.raises(gpu.TrainStationError):       # the same through the public API
        gpu._ffi.check(lib.cuda_memcpy(word, code.ctypes.data, 1, 0))
        gpu.synchronize()
    gpu.synchronize()


def _gemm(gpu, a, b):
    m, k = a.shape
    n = b.shape[1]
    da, db, dc = DevBuf(gpu, a), DevBuf(gpu, b), DevBuf(gpu, n=m * n)
    ok = gpu._ffi.lib().launch_gemm_kernel(da.ptr, db.ptr, dc.ptr, m, n, k, 0, 0, None, 0, None, 1, None)
    return ok, dc


def test_a_gemm_wait_that_runs_out_returns_an_error_and_the_context_stays_usable(gpu):
    lib = gpu._ffi.lib()
    rng = np.random.default_rng(3)
    a = rng.integers(-4, 5, (128, 256)).astype(np.float32)      # one 128 x 128 tile: one CTA of the one-CTA kernel
    b = rng.integers(-4, 5, (256, 128)).astype(np.float32)
    exact = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    gpu.synchronize()
    lib.ts_debug_set_gemm_wait_budget(0)
    try:
        ok, _ = _gemm(gpu, a, b)
        assert ok, "the launch itself succeeds; the failure is reported by the device"
        assert lib.ts_sync_stream(None) is False
        msg = gpu._ffi.last_error()
        assert any(str(code) in msg for code in (101, 102, 103, 104)), msg
    finally:
        lib.ts_debug_set_gemm_wait_budget(-1)
    assert lib.ts_sync_stream(None) is True
    ok, dc = _gemm(gpu, a, b)
    assert ok and lib.ts_sync_stream(None) is True
    assert np.array_equal(dc.get().reshape(128, 128), exact)
