"""GPU: the tcgen05 (tensor-core) GEMM in TF32 mode against an f64 product, for every operand
layout, edge tiles, and the fused epilogues; then whole training steps in TF32 mode within
the tolerance the task states (rel 2e-3)."""
import numpy as np
import pytest

from conftest import assert_bit_equal
from devbuf import DevBuf

pytestmark = pytest.mark.gpu

TF32_RTOL = 2e-3   # relative to the magnitude sum_k |a||b| of each output element


def _run(gpu, a_st, b_st, m, n, k, ta, tb, bias=None, relu=0, mask=None, precision=1):
    da, db, dc = DevBuf(gpu, a_st), DevBuf(gpu, b_st), DevBuf(gpu, n=m * n)
    dbias = DevBuf(gpu, bias) if bias is not None else None
    dmask = DevBuf(gpu, mask) if mask is not None else None
    gpu._ffi.check(gpu._ffi.lib().launch_gemm_kernel(da.ptr, db.ptr, dc.ptr, m, n, k, ta, tb, dbias.ptr if dbias else None, relu,
                                                     dmask.ptr if dmask else None, precision, None))
    gpu.synchronize()   # also surfaces a bounded wait that gave up inside the kernel
    return dc.get().reshape(m, n)


def _check(got, a, b, extra=None):
    exact = a.astype(np.float64) @ b.astype(np.float64)
    mag = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    if extra is not None:
        exact = extra(exact)
    err = np.abs(got - exact)
    assert np.all(err <= TF32_RTOL * mag + 1e-30), f"max err/mag {np.max(err / (mag + 1e-30)):.3e}"


SHAPES = [(128, 256, 32), (128, 128, 64), (256, 512, 128), (32, 128, 784), (100, 260, 36), (129, 132, 8), (4, 4, 4),
          (512, 1024, 1024), (1000, 264, 520), (2048, 10 * 4, 96), (148 * 128 + 5, 256, 64)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_tf32_gemm_all_layouts(gpu, m, n, k, ta, tb):
    if (ta and m % 4) or (not ta and k % 4) or (tb and k % 4) or n % 4:
        pytest.skip("row pitch not a multiple of 16 bytes: handled by the FP32 kernel")
    rng = np.random.default_rng(m * 31 + n * 7 + k + ta * 2 + tb)
    a, b = rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((k, n), dtype=np.float32)
    a_st = np.ascontiguousarray(a.T) if ta else a
    b_st = np.ascontiguousarray(b.T) if tb else b
    _check(_run(gpu, a_st, b_st, m, n, k, ta, tb), a, b)


def test_tf32_gemm_exact_on_small_integers(gpu):
    """Integers up to 2^10 are exact in TF32 and their sums exact in FP32: any layout or descriptor slip shows as a wrong integer."""
    rng = np.random.default_rng(0)
    m, n, k = 384, 512, 160
    a = rng.integers(-8, 9, (m, k)).astype(np.float32)
    b = rng.integers(-8, 9, (k, n)).astype(np.float32)
    exact = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    for ta, tb in ((0, 0), (0, 1), (1, 0), (1, 1)):
        got = _run(gpu, np.ascontiguousarray(a.T) if ta else a, np.ascontiguousarray(b.T) if tb else b, m, n, k, ta, tb)
        assert np.array_equal(got, exact), (ta, tb, int((got != exact).sum()))


@pytest.fixture(params=["tiles from a counter", "fixed stride"])
def tile_schedule(request, gpu):
    """The two-CTA kernel hands tiles out from a counter by default; the fixed stride per CTA pair stays as a switch."""
    gpu._ffi.lib().ts_debug_set_gemm_dynamic(1 if request.param == "tiles from a counter" else 0)
    yield request.param
    gpu._ffi.lib().ts_debug_set_gemm_dynamic(-1)


@pytest.mark.parametrize("m,n,k", [(4096, 4096, 96), (2308, 8196, 132)])
def test_two_cta_kernel_exact_on_small_integers(gpu, ora, m, n, k, tile_schedule):
    """Problems with at least 74 tiles of 256 x 256 run on CTA pairs (cta_group::2): every layout, edge tiles, epilogues."""
    rng = np.random.default_rng(m + k)
    a = rng.integers(-4, 5, (m, k)).astype(np.float32)
    b = rng.integers(-4, 5, (k, n)).astype(np.float32)
    exact = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    for ta, tb in ((0, 0), (0, 1), (1, 0), (1, 1)):
        got = _run(gpu, np.ascontiguousarray(a.T) if ta else a, np.ascontiguousarray(b.T) if tb else b, m, n, k, ta, tb)
        assert np.array_equal(got, exact), (ta, tb, int((got != exact).sum()))
    bias = rng.integers(-50, 50, n).astype(np.float32)
    mask = rng.standard_normal((m, n), dtype=np.float32)
    assert_bit_equal(_run(gpu, a, b, m, n, k, 0, 0, bias=bias, relu=1), ora.relu(ora.add_row(exact, bias)), "bias+relu")
    assert_bit_equal(_run(gpu, a, b, m, n, k, 0, 0, mask=mask), ora.relu_bwd(mask, exact), "mask")
    got3 = _run(gpu, a, b, m, n, k, 0, 0, precision=2)
    assert np.array_equal(got3, exact), "3xTF32 on integers"


@pytest.mark.parametrize("m,n,k", [(1024, 1024, 4096), (784, 1024, 4096), (200, 136, 2080), (128, 128, 16384), (256, 384, 2048)])
@pytest.mark.parametrize("ta,tb", [(1, 0), (0, 0), (0, 1)])
def test_split_k_products_are_exact_on_small_integers(gpu, m, n, k, ta, tb):
    """Few output tiles and a long K: the tensor-core kernel splits K over otherwise idle SMs and a second kernel adds
    the partial products.  On small integers every partial sum is exact, so any slip in the split ranges (a k-block
    counted twice or dropped, a ragged last split, a wrong slab) shows as a wrong integer.  3xTF32 takes the same route."""
    rng = np.random.default_rng(m + n + k + ta * 2 + tb)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    exact = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)      # integers far below 2^53: exact
    a_st = np.ascontiguousarray(a.T) if ta else a
    b_st = np.ascontiguousarray(b.T) if tb else b
    for precision in (1, 2):
        got = _run(gpu, a_st, b_st, m, n, k, ta, tb, precision=precision)
        assert np.array_equal(got, exact), (precision, int((got != exact).sum()))


def test_split_k_products_on_real_data(gpu):
    rng = np.random.default_rng(77)
    m, n, k = 1024, 1024, 4096
    a, b = rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((k, n), dtype=np.float32)
    _check(_run(gpu, np.ascontiguousarray(a.T), b, m, n, k, 1, 0), a, b)
    # the [1024 x 10] weight gradient of a 10-class output layer over a batch of 4096: not a tensor-core shape (row
    # pitch of 40 bytes); in the TF32 modes the FP32 kernel splits K as a batched launch.  FP32-level accuracy.
    m, n, k = 1024, 10, 4096
    a, b = rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((k, n), dtype=np.float32)
    a_st = np.ascontiguousarray(a.T)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    mag = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    for precision in (1, 2):
        got = _run(gpu, a_st, b, m, n, k, 1, 0, precision=precision)
        assert np.all(np.abs(got - exact) <= 2e-6 * mag), precision
    # FP32 mode keeps the single chain over K, bit for bit the reference's order: split results may differ from it in the last bits
    chain = _run(gpu, a_st, b, m, n, k, 1, 0, precision=0)
    assert np.all(np.abs(chain - exact) <= 4e-6 * mag)


@pytest.mark.parametrize("m,n,k", [(300, 384, 200), (128, 128, 64), (4096, 4096, 96), (2308, 8196, 132), (1000, 264, 520), (33, 36, 40)])
def test_column_sums_from_the_gemm_epilogue_are_exact_on_small_integers(gpu, m, n, k):
    """The bias gradient from the epilogue of the GEMM that produces the pre-activation gradient: per-warp partial sums
    (32 rows each) by a transposing butterfly, then a second kernel.  One-CTA and two-CTA kernels, edge tiles, with the
    ReLU mask applied first, in TF32 and 3xTF32 mode; the FP32 mode falls back to the ordinary column sum."""
    rng = np.random.default_rng(m + n + k)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    mask = rng.standard_normal((m, n), dtype=np.float32)
    exact = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)      # integers far below 2^53: exact
    lib = gpu._ffi.lib()
    da, db, dm = DevBuf(gpu, a), DevBuf(gpu, b), DevBuf(gpu, mask)
    for precision in (1, 2, 0):
        for with_mask in (False, True):
            dc, ds = DevBuf(gpu, n=m * n), DevBuf(gpu, -np.ones(n, np.float32))
            gpu._ffi.check(lib.launch_gemm_colsum_kernel(da.ptr, db.ptr, dc.ptr, m, n, k, 0, 0, None, 0, dm.ptr if with_mask else None,
                                                         precision, ds.ptr, None), "gemm + column sums")
            gpu.synchronize()
            want = np.where(mask > 0, exact, 0.0).astype(np.float32) if with_mask else exact
            assert np.array_equal(dc.get().reshape(m, n), want), (precision, with_mask)
            assert np.array_equal(ds.get(), want.sum(axis=0, dtype=np.float64).astype(np.float32)), (precision, with_mask)


def test_tf32_gemm_epilogues(gpu, ora):
    rng = np.random.default_rng(5)
    m, n, k = 300, 384, 200
    a = rng.integers(-4, 5, (m, k)).astype(np.float32)
    b = rng.integers(-4, 5, (k, n)).astype(np.float32)
    bias = rng.integers(-50, 50, n).astype(np.float32)
    mask = rng.standard_normal((m, n), dtype=np.float32)
    exact = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    assert_bit_equal(_run(gpu, a, b, m, n, k, 0, 0, bias=bias, relu=1), ora.relu(ora.add_row(exact, bias)), "bias+relu")
    assert_bit_equal(_run(gpu, a, b, m, n, k, 0, 0, mask=mask), ora.relu_bwd(mask, exact), "mask")
    assert_bit_equal(_run(gpu, a, b, m, n, k, 0, 0, bias=bias), ora.add_row(exact, bias), "bias")


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (1000, 264, 520), (512, 1024, 2048)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_tf32x3_gemm_is_fp32_accurate(gpu, m, n, k, ta, tb):
    """3xTF32 (operands split into TF32-exact high and low parts, three tensor-core sweeps): error at the FP32 level."""
    rng = np.random.default_rng(m + n + k + ta * 2 + tb)
    a, b = rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((k, n), dtype=np.float32)
    a_st = np.ascontiguousarray(a.T) if ta else a
    b_st = np.ascontiguousarray(b.T) if tb else b
    got = _run(gpu, a_st, b_st, m, n, k, ta, tb, precision=2)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    mag = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    err = np.abs(got - exact) / mag
    assert err.max() <= 2e-6, f"max err/mag {err.max():.3e}"      # a sequential f32 chain over k is allowed k * 6e-8
    fp32 = _run(gpu, a_st, b_st, m, n, k, ta, tb, precision=0)
    # the FP32 kernel's own sequential chain carries up to ~sqrt(k) * 6e-8 * mag of rounding error
    assert np.all(np.abs(got - fp32) <= 4e-6 * mag)


def test_training_step_tf32x3_meets_fp32_tolerance(gpu, ora):
    from test_gpu_engine import _mlp_device
    rng = np.random.default_rng(12)
    dims, batch = [256, 512, 512, 128], 384
    ws = [rng.uniform(-np.sqrt(6 / dims[i]), np.sqrt(6 / dims[i]), (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(dims[i + 1], np.float32) for i in range(3)]
    x, t = rng.standard_normal((batch, dims[0]), dtype=np.float32), rng.standard_normal((batch, dims[-1]), dtype=np.float32)
    st = ora.MlpState(ws, bs)
    ref = ora.mlp_step(st, x, t, loss_kind=ora.LOSS_MSE)
    gpu.set_matmul_precision(gpu.TF32X3)
    got = _mlp_device(gpu, ws, bs, x, t, "mse", False)
    assert abs(got["loss"] - float(ref["loss"])) <= 1e-5 * abs(float(ref["loss"]))
    for i in range(3):
        np.testing.assert_allclose(got["gw"][i], st.gw[i], rtol=1e-5, atol=1e-6)     # the task's FP32-mode tolerance
        # First Adam step: p -= lr * g / (|g| + eps).  Where |g| is near eps = 1e-8 a last-bit difference in g changes
        # the step by a sizeable fraction of lr, so parameters are compared where the gradient is well above eps
        # and bounded by 2 * lr everywhere.
        solid = np.abs(st.gw[i]) > 1e-6
        np.testing.assert_allclose(got["w"][i][solid], st.w[i][solid], rtol=1e-5, atol=2e-6)
        assert np.abs(got["w"][i] - st.w[i]).max() <= 2e-3


def test_tf32_long_k_accumulation(gpu):
    rng = np.random.default_rng(6)
    m, n, k = 256, 256, 16384
    a, b = rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((k, n), dtype=np.float32)
    _check(_run(gpu, np.ascontiguousarray(a.T), b, m, n, k, 1, 0), a, b)   # the dW layout with a long reduction


def test_training_step_tf32_within_tolerance(gpu, ora, capsys):
    """A 3-layer MLP step in TF32 mode vs the oracle: loss, gradients and post-Adam parameters within rel 2e-3."""
    from test_gpu_engine import _mlp_device
    rng = np.random.default_rng(4)
    dims, batch = [256, 512, 512, 128], 384
    ws = [rng.uniform(-np.sqrt(6 / dims[i]), np.sqrt(6 / dims[i]), (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(dims[i + 1], np.float32) for i in range(3)]
    x, t = rng.standard_normal((batch, dims[0]), dtype=np.float32), rng.standard_normal((batch, dims[-1]), dtype=np.float32)
    st = ora.MlpState(ws, bs)
    ref = ora.mlp_step(st, x, t, loss_kind=ora.LOSS_MSE)
    gpu.set_matmul_precision(gpu.TF32)
    got = _mlp_device(gpu, ws, bs, x, t, "mse", False)
    assert abs(got["loss"] - float(ref["loss"])) <= 2e-3 * abs(float(ref["loss"]))
    for i in range(3):
        assert np.abs(got["w"][i] - st.w[i]).max() <= 2.1e-3   # one Adam step moves a weight by at most lr = 1e-3 each way

    # A pre-activation within TF32 error of zero gets the other ReLU mask than on the FP32 path, and a
    # flipped mask element changes that element's gradient outright, whatever the GEMM's accuracy.  So
    # (1) masks must agree with the exact ones wherever |z| is outside the TF32 error band, the number of
    #     flips inside it is bounded and reported, and
    # (2) gradients are compared with an f64 evaluation that uses the masks the device forward produced:
    #     what is left is GEMM arithmetic, held to rel 2e-3 of each gradient tensor (Frobenius norm).
    T = gpu.Tensor
    W = [T.from_slice(w, w.shape).with_requires_grad() for w in ws]
    B = [T.from_slice(b, b.shape).with_requires_grad() for b in bs]
    h, hidden = T.from_slice(x, x.shape), []
    for i in range(3):
        h = h.matmul(W[i]).add_tensor(B[i])
        if i < 2:
            h = h.relu()
            hidden.append(h)
    loss = h.sub_tensor(T.from_slice(t, t.shape)).pow_scalar(2.0).mean()
    loss.backward(None)
    masks = [hd.data() > 0 for hd in hidden]
    chk = ora.reduced_precision_step_check(ws, bs, x, t, masks, [w.grad_by_value().data() for w in W],
                                           [b.grad_by_value().data() for b in B])
    with capsys.disabled():
        print(f"\n  TF32 step: ReLU mask flips {chk['flips']} of {chk['elements']} (inside the 2e-3 band: {chk['in_band']})")
    assert chk["outside_mismatch"] == [0, 0], chk
    for flips, n in zip(chk["flips"], chk["elements"]):
        assert flips <= 1e-3 * n, chk          # a flip needs |z| below the GEMM's actual error, far inside the band
    assert max(chk["rel_gw"]) <= 2e-3 and max(chk["rel_gb"]) <= 2e-3, chk


def test_relu_mask_is_exact_for_the_device_forward(gpu):
    """The mask used in backward is exactly (z_device > 0) for the z this forward produced, in TF32 mode too."""
    rng = np.random.default_rng(8)
    gpu.set_matmul_precision(gpu.TF32)
    x = rng.standard_normal((256, 128), dtype=np.float32)
    w = rng.standard_normal((128, 256), dtype=np.float32)
    X = gpu.Tensor.from_slice(x, x.shape).with_requires_grad()
    W = gpu.Tensor.from_slice(w, w.shape)
    y = X.matmul(W).relu()
    y.sum().backward(None)
    gx = X.grad_by_value().data()
    mask = (y.data() > 0).astype(np.float32)
    gpu.set_matmul_precision(gpu.FP32)
    want = gpu.Tensor.from_slice(mask, mask.shape).matmul(gpu.Tensor.from_slice(np.ascontiguousarray(w.T), [256, 128])).data()
    np.testing.assert_allclose(gx, want, rtol=2e-3, atol=2e-3 * np.abs(want).max())
