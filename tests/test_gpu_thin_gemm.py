"""GPU: the FFMA kernels for products with one dimension of at most 16 (a 10-class output layer, the gradient of its
weights, the gradient of its input), which the TF32 and 3xTF32 modes use in place of 32-wide tiles.

Small integers make every product and sum exact, so a wrong index shows as a wrong integer whatever the summation
order; real data is compared with an f64 product at FP32 accuracy (the kernels multiply the operands as given).  The
FP32 mode never takes these kernels: its results must stay bit-equal to the tiled kernel's chain order."""
import numpy as np
import pytest

from devbuf import DevBuf

pytestmark = pytest.mark.gpu


def _run(gpu, a_st, b_st, m, n, k, ta, tb, bias=None, relu=0, mask=None, precision=1, colsum=False):
    lib = gpu._ffi.lib()
    da, db, dc = DevBuf(gpu, a_st), DevBuf(gpu, b_st), DevBuf(gpu, -np.ones(m * n, np.float32))
    dbias = DevBuf(gpu, bias) if bias is not None else None
    dmask = DevBuf(gpu, mask) if mask is not None else None
    ds = DevBuf(gpu, -np.ones(n, np.float32)) if colsum else None
    if colsum:
        gpu._ffi.check(lib.launch_gemm_colsum_kernel(da.ptr, db.ptr, dc.ptr, m, n, k, ta, tb, dbias.ptr if dbias else None, relu,
                                                     dmask.ptr if dmask else None, precision, ds.ptr, None), "gemm + column sums")
    else:
        gpu._ffi.check(lib.launch_gemm_kernel(da.ptr, db.ptr, dc.ptr, m, n, k, ta, tb, dbias.ptr if dbias else None, relu,
                                              dmask.ptr if dmask else None, precision, None), "gemm")
    gpu.synchronize()
    out = dc.get().reshape(m, n)
    return (out, ds.get()) if colsum else out


def _ints(rng, shape, lim=4):
    return rng.integers(-lim, lim + 1, shape).astype(np.float32)


def _exact(a, b):
    return (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)


# forward layout: [m x k] . [k x n], n <= 16
@pytest.mark.parametrize("m,n,k", [(4096, 10, 1024), (256, 1, 128), (259, 3, 130), (1000, 4, 513), (300, 12, 1500), (2049, 16, 1027),
                                   (257, 7, 512), (65536 + 5, 10, 256), (16384 + 3, 12, 2500), (20000, 16, 700)])
def test_narrow_result_forward_layout(gpu, m, n, k):
    rng = np.random.default_rng(m + n + k)
    a, b = _ints(rng, (m, k)), _ints(rng, (k, n))
    exact = _exact(a, b)
    for precision in (1, 2):
        assert np.array_equal(_run(gpu, a, b, m, n, k, 0, 0, precision=precision), exact), precision
    bias = _ints(rng, n, 50)
    mask = rng.standard_normal((m, n), dtype=np.float32)
    got = _run(gpu, a, b, m, n, k, 0, 0, bias=bias, relu=1)
    assert np.array_equal(got, np.maximum(exact + bias, 0))
    got, sums = _run(gpu, a, b, m, n, k, 0, 0, bias=bias, mask=mask, colsum=True)
    want = np.where(mask > 0, exact + bias, 0).astype(np.float32)
    assert np.array_equal(got, want)
    assert np.array_equal(sums, want.sum(axis=0, dtype=np.float64).astype(np.float32))


# weight-gradient layout: [k x m]^T . [k x n], n <= 16, k the long reduction
@pytest.mark.parametrize("m,n,k", [(1024, 10, 4096), (64, 1, 256), (1000, 5, 4099), (70, 16, 300), (513, 12, 777), (256, 8, 65536),
                                   (1000, 10, 16400), (132, 16, 20000), (1001, 3, 16384)])
def test_narrow_result_weight_gradient_layout(gpu, m, n, k):
    rng = np.random.default_rng(m * 3 + n + k)
    a, b = _ints(rng, (m, k), 3), _ints(rng, (k, n), 3)
    exact = _exact(a, b)
    a_st = np.ascontiguousarray(a.T)
    for precision in (1, 2):
        assert np.array_equal(_run(gpu, a_st, b, m, n, k, 1, 0, precision=precision), exact), precision
    got, sums = _run(gpu, a_st, b, m, n, k, 1, 0, colsum=True)
    assert np.array_equal(got, exact)
    assert np.array_equal(sums, exact.sum(axis=0, dtype=np.float64).astype(np.float32))


# input-gradient layout: [m x k] . [n x k]^T, k <= 16
@pytest.mark.parametrize("m,n,k", [(4096, 1024, 10), (256, 128, 1), (300, 130, 7), (4097, 1030, 16), (259, 2052, 12), (1000, 1024, 4),
                                   (65536 + 3, 256, 10)])
def test_short_reduction_input_gradient_layout(gpu, m, n, k):
    rng = np.random.default_rng(m + n * 5 + k)
    a, b = _ints(rng, (m, k)), _ints(rng, (k, n))
    exact = _exact(a, b)
    b_st = np.ascontiguousarray(b.T)
    for precision in (1, 2):
        assert np.array_equal(_run(gpu, a, b_st, m, n, k, 0, 1, precision=precision), exact), precision
    bias = _ints(rng, n, 50)
    mask = rng.standard_normal((m, n), dtype=np.float32)
    assert np.array_equal(_run(gpu, a, b_st, m, n, k, 0, 1, bias=bias, relu=1), np.maximum(exact + bias, 0))
    for with_mask in (False, True):
        got, sums = _run(gpu, a, b_st, m, n, k, 0, 1, mask=mask if with_mask else None, colsum=True)
        want = np.where(mask > 0, exact, 0).astype(np.float32) if with_mask else exact
        assert np.array_equal(got, want), with_mask
        assert np.array_equal(sums, want.sum(axis=0, dtype=np.float64).astype(np.float32)), with_mask


def test_thin_products_on_real_data_are_fp32_accurate_and_repeat(gpu):
    rng = np.random.default_rng(11)
    cases = [((4096, 10, 1024), 0, 0), ((1024, 10, 4096), 1, 0), ((4096, 1024, 10), 0, 1)]
    for (m, n, k), ta, tb in cases:
        a, b = rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((k, n), dtype=np.float32)
        a_st = np.ascontiguousarray(a.T) if ta else a
        b_st = np.ascontiguousarray(b.T) if tb else b
        exact = a.astype(np.float64) @ b.astype(np.float64)
        mag = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
        first = _run(gpu, a_st, b_st, m, n, k, ta, tb)
        assert np.all(np.abs(first - exact) <= 2e-6 * mag), (m, n, k)
        assert np.array_equal(first, _run(gpu, a_st, b_st, m, n, k, ta, tb)), "a second run must repeat bit for bit"
        # FP32 mode: the tiled kernel's chain order, untouched by the thin kernels (the engine tests pin it to the oracle)
        chain = _run(gpu, a_st, b_st, m, n, k, ta, tb, precision=0)
        assert np.all(np.abs(chain - exact) <= 4e-6 * mag)


def test_thin_product_that_feeds_a_gemm_is_stored_rounded(gpu):
    """TF32 mode through the engine: the input gradient of a 10-wide layer goes into the next layer's tensor-core GEMMs,
    so it is stored already rounded to TF32 (no rounding pass of its own) and the gradients still meet the tolerance."""
    ts = gpu
    ts.set_matmul_precision(ts.TF32)
    try:
        rng = np.random.default_rng(5)
        batch, d0, d1, d2 = 512, 256, 384, 10
        x = rng.standard_normal((batch, d0), dtype=np.float32)
        w1 = (rng.standard_normal((d0, d1)) / np.sqrt(d0)).astype(np.float32)
        w2 = (rng.standard_normal((d1, d2)) / np.sqrt(d1)).astype(np.float32)
        T = ts.Tensor
        W1, W2 = T.from_slice(w1, w1.shape).with_requires_grad(), T.from_slice(w2, w2.shape).with_requires_grad()
        h = T.from_slice(x, x.shape).matmul(W1).relu()
        y = h.matmul(W2)
        y.mul_tensor(y).sum().backward(None)
        g1, g2 = W1.grad_by_value().data(), W2.grad_by_value().data()
        hd = h.data().astype(np.float64)
        yd = hd @ w2.astype(np.float64)
        dy = 2 * yd
        want_g2 = hd.T @ dy
        dh = (dy @ w2.astype(np.float64).T) * (hd > 0)
        want_g1 = x.astype(np.float64).T @ dh
        for got, want in ((g2, want_g2), (g1, want_g1)):
            assert np.linalg.norm(got - want) <= 2e-3 * np.linalg.norm(want)
    finally:
        ts.set_matmul_precision(ts.FP32)
        ts.clear_gradients()
