"""GPU: the kernels of the path at the full sizes of the benchmark configurations, checked through properties that do
not need the oracle to run at that size.

* The three GEMM layouts of a C5 layer (batch 65536, 4096 -> 8192) in TF32 mode on operands drawn from {-1, 0, 1}:
  such operands are exact in TF32 and every partial sum is an integer below 2^24, so each of the 5 x 10^8 results
  must be exactly the integer product.  Checked by two checksums of checksums that every element enters (row sums
  and column sums against matrix-vector products computed on the host in float64) and by whole rows recomputed on
  the host.
* The fused Adam over the six parameter tensors of C5 (134 238 208 elements): the update is element-wise, so slices
  of every tensor must equal the oracle run on just those slices, bit for bit.
* add / mul at 2^28 elements (C2) on integer-valued data against numpy, element for element.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_bit_equal
from devbuf import DevBuf

pytestmark = pytest.mark.gpu

BATCH, D_IN, D_OUT = 65536, 4096, 8192


def ternary(rng, shape):
    return rng.integers(-1, 2, shape, dtype=np.int8).astype(np.float32)


def gemm(gpu, da, db, m, n, k, ta, tb, precision=1):
    dc = DevBuf(gpu, n=m * n)
    gpu._ffi.check(gpu._ffi.lib().launch_gemm_kernel(da.ptr, db.ptr, dc.ptr, m, n, k, ta, tb, None, 0, None, precision, None), "gemm")
    gpu.synchronize()
    out = dc.get().reshape(m, n)
    dc.free()
    return out


def check_product(got, a, b, rows):
    """got == a @ b for integer-valued a [m, k], b [k, n]: both checksums and `rows` recomputed exactly."""
    k = a.shape[1]
    a_colsum = a.sum(axis=0, dtype=np.float64)                        # [k]
    b_rowsum = b.sum(axis=1, dtype=np.float64)                        # [k]
    # column sums of the product = (column sums of a) . b; row sums = a . (row sums of b); float64 in blocks of k
    # (every intermediate is an integer far below 2^53)
    want_cols = np.zeros(b.shape[1], np.float64)
    for lo in range(0, k, 4096):
        want_cols += a_colsum[lo:lo + 4096] @ b[lo:lo + 4096].astype(np.float64)
    want_rows = np.zeros(a.shape[0], np.float64)
    for lo in range(0, a.shape[0], 1024):
        want_rows[lo:lo + 1024] = a[lo:lo + 1024].astype(np.float64) @ b_rowsum
    np.testing.assert_array_equal(got.sum(axis=0, dtype=np.float64), want_cols)
    np.testing.assert_array_equal(got.sum(axis=1, dtype=np.float64), want_rows)
    # whole rows: float32 arithmetic on the host is exact here whatever its order (integers below 2^24)
    np.testing.assert_array_equal(got[rows], a[rows] @ b)


def test_c5_layer_gemms_exact_on_ternary_operands(gpu):
    rng = np.random.default_rng(5)
    x, w, g = ternary(rng, (BATCH, D_IN)), ternary(rng, (D_IN, D_OUT)), ternary(rng, (BATCH, D_OUT))
    dx, dw, dg = DevBuf(gpu, x), DevBuf(gpu, w), DevBuf(gpu, g)
    rows = rng.integers(0, BATCH, 48)
    # forward: y = x . w
    y = gemm(gpu, dx, dw, BATCH, D_OUT, D_IN, 0, 0)
    check_product(y, x, w, rows)
    # the FP32 kernel (the bit-parity mode) and the 3xTF32 mode must give the same integers
    for precision in (0, 2):
        assert np.array_equal(gemm(gpu, dx, dw, BATCH, D_OUT, D_IN, 0, 0, precision), y), precision
    del y
    # input gradient: dx = g . w^T (w stored [D_IN, D_OUT] is the transposed right operand)
    gx = gemm(gpu, dg, dw, BATCH, D_IN, D_OUT, 0, 1)
    check_product(gx, g, np.ascontiguousarray(w.T), rows)
    del gx
    # weight gradient: dw = x^T . g, a sum over all 65536 batch rows per element
    gw = gemm(gpu, dx, dg, D_IN, D_OUT, BATCH, 1, 0)
    xt = np.ascontiguousarray(x.T)
    check_product(gw, xt, g, rng.integers(0, D_IN, 8))
    for b in (dx, dw, dg):
        b.free()


def test_c5_forward_rows_match_the_oracle(gpu, ora):
    """The C5 network (4096-8192-8192-4096) at batch 65536 through the engine.  A row of the output depends on that row
    of the input only, so rows sampled from the full-batch result must equal the oracle run on just those rows: bit
    for bit in FP32 mode (same summation order per element whatever the batch), within the TF32 bound otherwise."""
    T = gpu.Tensor
    rng = np.random.default_rng(55)
    dims = [D_IN, D_OUT, D_OUT, D_IN]
    ws = [((rng.random((dims[i], dims[i + 1]), dtype=np.float32) - np.float32(0.5)) * np.float32(2.0 * np.sqrt(6.0 / dims[i])))
          for i in range(3)]
    bs = [((rng.random(dims[i + 1], dtype=np.float32) - np.float32(0.5)) * np.float32(0.1)) for i in range(3)]
    x = rng.random((BATCH, D_IN), dtype=np.float32) - np.float32(0.5)
    rows = np.sort(rng.choice(BATCH, 24, replace=False))
    ref = ora.mlp_step(ora.MlpState(ws, bs), np.ascontiguousarray(x[rows]), loss_kind=ora.LOSS_SUM, do_adam=False, want_y=True)["y"]
    W = [T.from_slice(w, list(w.shape)) for w in ws]
    B = [T.from_slice(b, list(b.shape)) for b in bs]
    X = T.from_slice(x, [BATCH, D_IN])
    for mode in (gpu.FP32, gpu.TF32):
        gpu.set_matmul_precision(mode)
        with gpu.NoGradTrack():
            h = X
            for i in range(3):
                h = h.matmul(W[i]).add_tensor(B[i])
                if i < 2:
                    h = h.relu()
            y = h.data()[rows]
        if mode == gpu.FP32:
            assert_bit_equal(y, ref, "sampled rows of the full-batch forward, FP32 mode")
        else:
            scale = float(np.abs(ref).max())
            assert float(np.abs(y - ref).max()) <= 2e-3 * scale, float(np.abs(y - ref).max()) / scale
        del h


def test_c5_adam_matches_the_oracle_on_slices_of_every_tensor(gpu, ora):
    sizes = [D_IN * D_OUT, D_OUT, D_OUT * D_OUT, D_OUT, D_OUT * D_IN, D_IN]
    assert sum(sizes) == 134238208
    lib = gpu._ffi.lib()
    rng = np.random.default_rng(8)
    host = {k: [(rng.random(n, dtype=np.float32) - np.float32(0.5)) * np.float32(s) for n in sizes]
            for k, s in (("p", 2.0), ("g", 0.2), ("m", 0.02))}
    host["v"] = [rng.random(n, dtype=np.float32) * np.float32(1e-3) for n in sizes]
    dev = {k: [DevBuf(gpu, a) for a in host[k]] for k in ("p", "g", "m", "v")}
    lr, b1, b2, eps, step = 1e-3, 0.9, 0.999, 1e-8, 7
    f1 = np.float32(1.0) / np.float32(1.0 - float(np.float32(b1)) ** float(np.float32(step)))
    f2 = np.float32(1.0) / np.float32(1.0 - float(np.float32(b2)) ** float(np.float32(step)))
    tab = lambda bufs: (C.c_void_p * len(bufs))(*[b.ptr for b in bufs])
    szs = (C.c_ulonglong * len(sizes))(*sizes)
    gpu._ffi.check(lib.launch_adam_multi_tensor_kernel(tab(dev["p"]), tab(dev["g"]), tab(dev["m"]), tab(dev["v"]), szs, len(sizes), lr, b1,
                                                       b2, eps, 0.0, float(f1), float(f2), 1.0, None), "adam")
    gpu.synchronize()
    for i, n in enumerate(sizes):
        got = {k: dev[k][i].get() for k in ("p", "m", "v")}
        width = min(n, 1 << 18)
        for lo in sorted({0, (n // 2) // 8 * 8, n - width}):          # slices start on multiples of 8 (the SIMD body)
            sl = slice(lo, lo + width)
            p, m, v = (host[k][i][sl].copy() for k in ("p", "m", "v"))
            ora.adam_update(p, host["g"][i][sl], m, v, step, lr, b1, b2, eps, 0.0)
            assert_bit_equal(got["p"][sl], p, f"p tensor {i} at {lo}")
            assert_bit_equal(got["m"][sl], m, f"m tensor {i} at {lo}")
            assert_bit_equal(got["v"][sl], v, f"v tensor {i} at {lo}")
        # nothing outside the update formula's reach: the gradient buffer is untouched
        assert_bit_equal(dev["g"][i].get()[:1024], host["g"][i][:1024], f"g tensor {i}")
    for bufs in dev.values():
        for b in bufs:
            b.free()


def test_c2_elementwise_at_two_to_the_28(gpu):
    n = 1 << 28
    lib = gpu._ffi.lib()
    rng = np.random.default_rng(28)
    a = rng.integers(-1000, 1001, n, dtype=np.int16).astype(np.float32)
    b = rng.integers(-1000, 1001, n, dtype=np.int16).astype(np.float32)
    da, db, do = DevBuf(gpu, a), DevBuf(gpu, b), DevBuf(gpu, n=n)
    gpu._ffi.check(lib.launch_add_kernel(da.ptr, db.ptr, do.ptr, n, None), "add")
    assert np.array_equal(do.get(), a + b)
    gpu._ffi.check(lib.launch_mul_kernel(da.ptr, db.ptr, do.ptr, n, None), "mul")
    assert np.array_equal(do.get(), a * b)
    gpu._ffi.check(lib.launch_sub_kernel(da.ptr, db.ptr, do.ptr, n, None), "sub")
    assert np.array_equal(do.get(), a - b)
    for buf in (da, db, do):
        buf.free()
