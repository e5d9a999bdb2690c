"""GPU: the column sum that allocates nothing (launch_colsum_kernel_static_scratch).

It exists for hosts that cannot get device memory when they need a bias gradient: a plugin
inside another framework's fixed memory budget, a process whose device memory is already
fully handed out, a latency-bound loop that must stay out of the driver's allocator.  Such
a caller has no scratch buffer to give launch_colsum_kernel, so this variant keeps its
partial sums in an array built into the library.

The test calls it through the C ABI twice in a row on different data and requires the same
bits as launch_colsum_kernel (both run the same two kernels, only the scratch differs), checks
that the library's allocator did not reach the driver, that the largest plan this device can
produce fits the built-in scratch, and that bad pointers are refused.  The file name sorts last so that a run stopping
at the first failure has already been through every other test.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_bit_equal
from devbuf import DevBuf

pytestmark = pytest.mark.gpu


def test_static_scratch_colsum_matches_regular_entry_point_twice(gpu):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    rng = np.random.default_rng(2024)
    cases = [(4096, 1024), (3001, 516)]          # two calls in a row, different shapes: the second reuses the array
    bufs = []
    for rows, cols in cases:
        g = rng.standard_normal((rows, cols), dtype=np.float32)
        bufs.append((rows, cols, g, DevBuf(gpu, g), DevBuf(gpu, n=cols), DevBuf(gpu, n=cols),
                     DevBuf(gpu, n=int(lib.ts_colsum_scratch_elems(rows, cols)))))
    gpu.synchronize()

    def free_bytes():
        f = C.c_ulonglong()
        chk(lib.ts_device_memory_info(C.byref(f), None), "memory info")
        return int(f.value)

    # The first call on a device resolves the built-in array's address; that look-up is part of set-up, so the
    # claim "takes no device memory" is checked around the calls that follow it: free memory as the driver reports
    # it must not move, with the library's per-kernel event profiling switched on as well (creating an event would
    # allocate, so this entry point must not bracket its launches).
    # (Each shape is also run once beforehand: the CUDA runtime loads a kernel's code onto the device at its first
    # launch, which is the runtime's allocation, not this entry point's.)
    for rows, cols, g, dg, out_static, out_ref, scratch in bufs:
        chk(lib.launch_colsum_kernel_static_scratch(dg.ptr, out_static.ptr, rows, cols, None), "static scratch, first call")
    gpu.synchronize()
    before, free_before = gpu.allocator_stats(), free_bytes()
    lib.ts_profile_reset()
    lib.ts_profile_enable(1)
    try:
        for rows, cols, g, dg, out_static, out_ref, scratch in bufs:
            chk(lib.launch_colsum_kernel_static_scratch(dg.ptr, out_static.ptr, rows, cols, None), "static scratch")
        gpu.synchronize()
        free_after = free_bytes()
    finally:
        lib.ts_profile_enable(0)
        lib.ts_profile_reset()
    after = gpu.allocator_stats()
    assert free_after == free_before, f"device memory moved by {free_before - free_after} bytes across calls that must not allocate"
    assert after["driver_allocations"] == before["driver_allocations"]
    assert after["bytes_reserved"] == before["bytes_reserved"] and after["bytes_in_use"] == before["bytes_in_use"]
    for rows, cols, g, dg, out_static, out_ref, scratch in bufs:
        chk(lib.launch_colsum_kernel(dg.ptr, out_ref.ptr, rows, cols, scratch.ptr, None), "regular")
        assert_bit_equal(out_static.get(), out_ref.get(), f"{rows}x{cols}")
        exact = g.astype(np.float64).sum(axis=0)
        mag = np.abs(g).astype(np.float64).sum(axis=0)
        assert np.all(np.abs(out_static.get() - exact) <= 1e-6 * mag)


def test_static_scratch_colsum_small_and_degenerate_shapes(gpu):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    g = np.arange(12, dtype=np.float32).reshape(3, 4)
    dg, out = DevBuf(gpu, g), DevBuf(gpu, n=4)
    chk(lib.launch_colsum_kernel_static_scratch(dg.ptr, out.ptr, 3, 4, None))     # one split: the scratch is not even touched
    assert out.get().tolist() == [12.0, 15.0, 18.0, 21.0]
    chk(lib.launch_colsum_kernel_static_scratch(dg.ptr, out.ptr, 0, 4, None))     # no rows: zeros, as sum_dims over an empty axis
    assert out.get().tolist() == [0.0] * 4
    assert lib.launch_colsum_kernel_static_scratch(dg.ptr, out.ptr, 3, 0, None) is True


def test_static_scratch_colsum_largest_plan_and_bad_pointers(gpu):
    lib = gpu._ffi.lib()
    d = DevBuf(gpu, n=16)
    # The partial sums take (row splits) x (columns) elements and the kernel plans at most 4 CTAs per SM, so the
    # need grows with the SM count: on a 148-SM B200 it peaks at 592 x 128 = 75776 elements, inside the 131072 the
    # built-in array holds; a device with more than 256 SMs could exceed it and is then refused with a message.
    # What can be checked here: the largest plan of this device is served, and bad pointers are refused.
    rows, cols = 4096, 128 * 296                      # 296 column tiles -> 2 row splits -> 75776 partial sums
    g = np.ones((rows, cols), np.float32)
    dg, out = DevBuf(gpu, g), DevBuf(gpu, n=cols)
    gpu._ffi.check(lib.launch_colsum_kernel_static_scratch(dg.ptr, out.ptr, rows, cols, None))
    assert np.all(out.get() == rows)
    assert lib.launch_colsum_kernel_static_scratch(None, d.ptr, 8, 8, None) is False
    assert "null" in gpu._ffi.last_error()
