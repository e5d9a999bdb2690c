"""GPU: the column sum that allocates nothing (launch_colsum_kernel_static_scratch).

It exists for hosts that cannot get device memory when they need a bias gradient: a plugin
inside another framework's fixed memory budget, a process whose device memory is already
fully handed out, a latency-bound loop that must stay out of the driver's allocator.  Such
a caller has no scratch buffer to give launch_colsum_kernel, so this variant keeps its
partial sums in an array built into the library.

The test calls it through the C ABI twice in a row on different data and requires the same
bits as launch_colsum_kernel (both run the same two kernels, only the scratch differs), checks
that the library's allocator did not reach the driver, and that a problem larger than the
built-in scratch is refused with a message.  The file name sorts last so that a run stopping
at the first failure has already been through every other test.
"""
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
    before = gpu.allocator_stats()
    for rows, cols, g, dg, out_static, out_ref, scratch in bufs:
        chk(lib.launch_colsum_kernel_static_scratch(dg.ptr, out_static.ptr, rows, cols, None), "static scratch")
    after = gpu.allocator_stats()
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


def test_static_scratch_colsum_refuses_what_does_not_fit(gpu):
    lib = gpu._ffi.lib()
    d = DevBuf(gpu, n=16)
    # 75648 columns are 591 column tiles; filling 4 CTAs per SM on 148 SMs then takes 2 row splits, i.e.
    # 2 x 75648 = 151296 partial sums, more than the 131072 the built-in array holds.  The call is refused
    # before any launch, so the (far too small) buffers are never dereferenced.
    assert lib.launch_colsum_kernel_static_scratch(d.ptr, d.ptr, 4096, 75648, None) is False
    msg = gpu._ffi.last_error()
    assert "scratch" in msg and "131072" in msg and "151296" in msg
    assert lib.launch_colsum_kernel_static_scratch(None, d.ptr, 8, 8, None) is False
