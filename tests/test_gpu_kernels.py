"""GPU: every raw kernel launcher against the CPU oracle, through the C ABI.
Single-operation kernels must match bit for bit; tree reductions are compared with the
f64 value within a stated tolerance and with the oracle's sequential f32 sum."""
import numpy as np
import pytest

from conftest import assert_bit_equal
from devbuf import DevBuf

pytestmark = pytest.mark.gpu

SIZES = [0, 1, 3, 4, 7, 8, 9, 31, 33, 255, 1024, 4099, (1 << 20) + 3]


def _ab(n, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal(n, dtype=np.float32)
    b = (rng.random(n, dtype=np.float32) * 1.5 + 0.5).astype(np.float32)   # divisor in [0.5, 2)
    return a, b


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_binary_forward_bit_exact(gpu, ora, op, n):
    a, b = _ab(n, n + 1)
    da, db, do = DevBuf(gpu, a), DevBuf(gpu, b), DevBuf(gpu, n=n)
    fn = getattr(gpu._ffi.lib(), f"launch_{op}_kernel")
    gpu._ffi.check(fn(da.ptr, db.ptr, do.ptr, n, None), op)
    assert_bit_equal(do.get(), getattr(ora, op)(a, b), f"{op} n={n}")


@pytest.mark.parametrize("offset", [1, 2, 3])
def test_binary_unaligned_pointers(gpu, ora, offset):
    n = 1000
    a, b = _ab(n, 99)
    da, db, do = DevBuf(gpu, a, offset=offset), DevBuf(gpu, b), DevBuf(gpu, n=n, offset=offset)
    gpu._ffi.check(gpu._ffi.lib().launch_div_kernel(da.ptr, db.ptr, do.ptr, n, None))
    assert_bit_equal(do.get(), ora.div(a, b))


def test_null_pointers_are_refused(gpu):
    lib = gpu._ffi.lib()
    d = DevBuf(gpu, n=8)
    assert lib.launch_add_kernel(None, d.ptr, d.ptr, 8, None) is False      # cuda_wrapper.cpp:64
    assert lib.launch_matmul_kernel(d.ptr, None, d.ptr, 2, 2, 2, None) is False
    assert "null" in gpu._ffi.last_error()
    assert lib.cuda_memcpy(d.ptr, None, 8, 0) is False
    assert lib.cuda_memcpy(d.ptr, d.ptr, 8, 7) is False


def test_explicit_stream(gpu, ora):
    lib = gpu._ffi.lib()
    s = lib.create_cuda_stream()
    assert s
    a, b = _ab(5000, 5)
    da, db, do = DevBuf(gpu, a), DevBuf(gpu, b), DevBuf(gpu, n=5000)
    gpu._ffi.check(lib.launch_mul_kernel(da.ptr, db.ptr, do.ptr, 5000, s))
    gpu._ffi.check(lib.ts_sync_stream(s))
    assert_bit_equal(do.get(), ora.mul(a, b))
    lib.destroy_cuda_stream(s)


@pytest.mark.parametrize("n", [0, 5, 8, 1025, (1 << 18) + 1])
def test_unary_and_backward_kernels_bit_exact(gpu, ora, n):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n, dtype=np.float32)
    if n >= 5:
        x[:5] = [np.nan, -0.0, 0.0, -np.inf, np.inf]
    go = rng.standard_normal(n, dtype=np.float32)
    a, b = _ab(n, n + 7)
    dx, dgo, da, db = DevBuf(gpu, x), DevBuf(gpu, go), DevBuf(gpu, a), DevBuf(gpu, b)
    o1, o2 = DevBuf(gpu, n=n), DevBuf(gpu, n=n)
    chk(lib.launch_relu_kernel(dx.ptr, o1.ptr, n, None))
    y = o1.get()
    assert_bit_equal(y, ora.relu(x), "relu")
    assert not np.isnan(y).any() and not np.signbit(y).any()   # NaN -> 0, -0 -> +0
    chk(lib.launch_relu_backward_kernel(dx.ptr, dgo.ptr, o1.ptr, n, None))
    assert_bit_equal(o1.get(), ora.relu_bwd(x, go), "relu_bwd")
    dy = DevBuf(gpu, y)   # the ReLU output is an equivalent mask
    chk(lib.launch_relu_backward_kernel(dy.ptr, dgo.ptr, o1.ptr, n, None))
    assert_bit_equal(o1.get(), ora.relu_bwd(x, go), "relu_bwd via output")
    chk(lib.launch_square_kernel(da.ptr, o1.ptr, n, None))
    assert_bit_equal(o1.get(), ora.square(a), "square")
    chk(lib.launch_square_backward_kernel(da.ptr, dgo.ptr, o1.ptr, n, None))
    assert_bit_equal(o1.get(), ora.square_bwd(a, go), "square_bwd")
    chk(lib.launch_mul_backward_kernel(da.ptr, db.ptr, dgo.ptr, o1.ptr, o2.ptr, n, None))
    ga, gb = ora.mul_bwd(a, b, go)
    assert_bit_equal(o1.get(), ga, "mul_bwd a"); assert_bit_equal(o2.get(), gb, "mul_bwd b")
    chk(lib.launch_div_backward_kernel(da.ptr, db.ptr, dgo.ptr, o1.ptr, o2.ptr, n, None))
    ga, gb = ora.div_bwd(a, b, go)
    assert_bit_equal(o1.get(), ga, "div_bwd a"); assert_bit_equal(o2.get(), gb, "div_bwd b")
    chk(lib.launch_scale_kernel(da.ptr, -1.0, o1.ptr, n, None))
    assert_bit_equal(o1.get(), ora.neg(a), "neg")
    chk(lib.launch_fill_kernel(o1.ptr, 2.5, n, None))
    assert np.all(o1.get() == 2.5)
    if n:
        sc = DevBuf(gpu, np.array([3.0], np.float32))
        chk(lib.launch_fill_from_scalar_kernel(o1.ptr, sc.ptr, 1.0 / np.float32(n), n, None))
        assert np.all(o1.get() == np.float32(np.float32(1.0) / np.float32(n)) * np.float32(3.0))


@pytest.mark.parametrize("rows,cols,relu", [(1, 1, 0), (5, 3, 1), (32, 128, 1), (33, 10, 0), (257, 1024, 1), (64, 4100, 0)])
def test_bias_act(gpu, ora, rows, cols, relu):
    rng = np.random.default_rng(rows * cols)
    z, b = rng.standard_normal((rows, cols), dtype=np.float32), rng.standard_normal(cols, dtype=np.float32)
    dz, db, do = DevBuf(gpu, z), DevBuf(gpu, b), DevBuf(gpu, n=rows * cols)
    gpu._ffi.check(gpu._ffi.lib().launch_bias_act_kernel(dz.ptr, db.ptr, do.ptr, rows, cols, relu, None))
    want = ora.add_row(z, b)
    if relu:
        want = ora.relu(want)
    assert_bit_equal(do.get().reshape(rows, cols), want)


@pytest.mark.parametrize("n", [0, 1, 3, 1000, 4097, (1 << 20) + 5, 1 << 24])
@pytest.mark.parametrize("mean", [0, 1])
def test_sum_mean(gpu, ora, n, mean):
    lib = gpu._ffi.lib()
    rng = np.random.default_rng(n + mean)
    x = rng.standard_normal(n, dtype=np.float32)
    dx, do, sc = DevBuf(gpu, x), DevBuf(gpu, n=1), DevBuf(gpu, n=int(lib.ts_reduce_scratch_elems()))
    gpu._ffi.check(lib.launch_sum_kernel(dx.ptr, do.ptr, n, mean, sc.ptr, None))
    got = float(do.get()[0])
    exact = float(x.astype(np.float64).sum()) / (n if (mean and n) else 1)
    seq = float(ora.mean(x) if mean else ora.total(x))
    scale = float(np.abs(x.astype(np.float64)).sum()) / (n if (mean and n) else 1)
    # a pairwise tree in f32: error bounded by a few ulp of the sum of magnitudes
    assert abs(got - exact) <= 1e-6 * scale + 1e-30
    # and it is at least as close to the exact value as the reference's sequential sum (plus slack)
    assert abs(got - exact) <= abs(seq - exact) + 1e-6 * scale
    gpu._ffi.check(lib.launch_sum_kernel(dx.ptr, do.ptr, n, mean, sc.ptr, None))
    assert float(do.get()[0]) == got   # deterministic


@pytest.mark.parametrize("rows,cols", [(1, 1), (7, 3), (32, 128), (100, 10), (4096, 1024), (1000, 36), (5000, 132)])
def test_colsum_and_fused_relu_backward(gpu, ora, rows, cols):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    rng = np.random.default_rng(rows + cols)
    g = rng.standard_normal((rows, cols), dtype=np.float32)
    ref = rng.standard_normal((rows, cols), dtype=np.float32)
    dg, dref = DevBuf(gpu, g), DevBuf(gpu, ref)
    out, gi = DevBuf(gpu, n=cols), DevBuf(gpu, n=rows * cols)
    sc = DevBuf(gpu, n=int(lib.ts_colsum_scratch_elems(rows, cols)))
    chk(lib.launch_colsum_kernel(dg.ptr, out.ptr, rows, cols, sc.ptr, None))
    exact = g.astype(np.float64).sum(axis=0)
    mag = np.abs(g).astype(np.float64).sum(axis=0)
    assert np.all(np.abs(out.get() - exact) <= 1e-6 * mag + 1e-30)
    np.testing.assert_allclose(out.get(), ora.colsum(g), rtol=1e-4, atol=1e-5 * np.sqrt(rows))
    chk(lib.launch_relu_backward_colsum_kernel(dref.ptr, dg.ptr, gi.ptr, out.ptr, rows, cols, sc.ptr, None))
    want_gi = ora.relu_bwd(ref, g)
    assert_bit_equal(gi.get().reshape(rows, cols), want_gi, "fused relu backward")
    exact = want_gi.astype(np.float64).sum(axis=0)
    assert np.all(np.abs(out.get() - exact) <= 1e-6 * mag + 1e-30)


SGEMM_SHAPES = [(1, 1, 1), (2, 2, 2), (32, 128, 784), (17, 23, 19), (64, 48, 40), (130, 10, 257), (5, 300, 129),
                (256, 256, 256), (128, 136, 8), (3, 7, 1000), (200, 100, 0),
                # at least 74 tiles of 128 x 128: the large-tile kernel (the shapes above run on 32 x 32 tiles)
                (1200, 1156, 70), (1281, 1034, 33),
                # fewer than 74 tiles of 128 x 128 but at least 74 of 64 x 64: the middle kernel (tail columns in two)
                (520, 1100, 70), (1024, 1024, 100), (600, 603, 129)]


@pytest.mark.parametrize("m,n,k", SGEMM_SHAPES)
def test_fp32_gemm_matches_reference_order_bit_exact(gpu, ora, m, n, k):
    """FP32 mode reproduces the reference's per-element FMA chain (and the mul+add of the n%8 tail columns)."""
    rng = np.random.default_rng(m * 7919 + n * 31 + k)
    a, b = rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((k, n), dtype=np.float32)
    da, db, dc = DevBuf(gpu, a), DevBuf(gpu, b), DevBuf(gpu, n=m * n)
    gpu._ffi.check(gpu._ffi.lib().launch_gemm_kernel(da.ptr, db.ptr, dc.ptr, m, n, k, 0, 0, None, 0, None, 0, None))
    assert_bit_equal(dc.get().reshape(m, n), ora.matmul(a, b), f"sgemm {m}x{n}x{k}")


@pytest.mark.parametrize("m,n,k", [(33, 65, 70), (128, 10, 300), (64, 256, 129), (1300, 1102, 40), (520, 1100, 45), (577, 650, 33)])
def test_fp32_gemm_transposed_operands_and_epilogue(gpu, ora, m, n, k):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    rng = np.random.default_rng(m + n + k)
    a, b = rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((k, n), dtype=np.float32)
    bias, mask = rng.standard_normal(n, dtype=np.float32), rng.standard_normal((m, n), dtype=np.float32)
    at, bt = np.ascontiguousarray(a.T), np.ascontiguousarray(b.T)
    da, db, dat, dbt, dc = DevBuf(gpu, a), DevBuf(gpu, b), DevBuf(gpu, at), DevBuf(gpu, bt), DevBuf(gpu, n=m * n)
    want = ora.matmul(a, b)
    for ta, tb, pa, pb in ((0, 1, da, dbt), (1, 0, dat, db), (1, 1, dat, dbt)):
        chk(lib.launch_gemm_kernel(pa.ptr, pb.ptr, dc.ptr, m, n, k, ta, tb, None, 0, None, 0, None))
        assert_bit_equal(dc.get().reshape(m, n), want, f"trans {ta}{tb}")
    dbias, dmask = DevBuf(gpu, bias), DevBuf(gpu, mask)
    chk(lib.launch_gemm_kernel(da.ptr, db.ptr, dc.ptr, m, n, k, 0, 0, dbias.ptr, 1, None, 0, None))
    assert_bit_equal(dc.get().reshape(m, n), ora.relu(ora.add_row(want, bias)), "bias+relu epilogue")
    chk(lib.launch_gemm_kernel(da.ptr, db.ptr, dc.ptr, m, n, k, 0, 0, None, 0, dmask.ptr, 0, None))
    assert_bit_equal(dc.get().reshape(m, n), ora.relu_bwd(mask, want), "mask epilogue")


def test_launch_matmul_kernel_stub_signature(gpu, ora):
    """The reference's own launch_matmul_kernel (cuda_wrapper.cpp:81-94) and its 2x2 known answer."""
    a, b = np.array([1, 2, 3, 4], np.float32), np.array([5, 6, 7, 8], np.float32)
    da, db, dc = DevBuf(gpu, a), DevBuf(gpu, b), DevBuf(gpu, n=4)
    gpu._ffi.check(gpu._ffi.lib().launch_matmul_kernel(da.ptr, db.ptr, dc.ptr, 2, 2, 2, None))
    assert dc.get().tolist() == [19, 22, 43, 50]


@pytest.mark.parametrize("sizes", [[1], [7], [8, 11, 16384, 16385, 3], [100480, 128], [1 << 20, 1000, 10]])
@pytest.mark.parametrize("wd", [0.0, 0.01])
def test_adam_multi_tensor_bit_exact(gpu, ora, sizes, wd):
    import ctypes as C
    lib = gpu._ffi.lib()
    rng = np.random.default_rng(sum(sizes))
    P = [rng.standard_normal(n, dtype=np.float32) for n in sizes]
    M = [np.zeros(n, np.float32) for n in sizes]
    V = [np.zeros(n, np.float32) for n in sizes]
    dP, dM, dV = [DevBuf(gpu, p) for p in P], [DevBuf(gpu, m) for m in M], [DevBuf(gpu, v) for v in V]
    lr, b1, b2, eps = 1e-3, 0.9, 0.999, 1e-8
    vp = C.c_void_p
    for step in range(1, 4):
        G = [rng.standard_normal(n, dtype=np.float32) * (10.0 ** rng.integers(-3, 2)) for n in sizes]
        dG = [DevBuf(gpu, g) for g in G]
        bc1 = np.float32(1.0 - float(np.float32(b1)) ** float(np.float32(step)))
        bc2 = np.float32(1.0 - float(np.float32(b2)) ** float(np.float32(step)))
        f1, f2 = np.float32(1.0) / bc1, np.float32(1.0) / bc2
        tab = lambda bufs: (vp * len(bufs))(*[b.ptr for b in bufs])
        szs = (C.c_ulonglong * len(sizes))(*sizes)
        gpu._ffi.check(lib.launch_adam_multi_tensor_kernel(tab(dP), tab(dG), tab(dM), tab(dV), szs, len(sizes), lr, b1, b2,
                                                           eps, wd, float(f1), float(f2), 1.0, None))
        for i in range(len(sizes)):
            ora.adam_update(P[i], G[i], M[i], V[i], step, lr, b1, b2, eps, wd)
            assert_bit_equal(dP[i].get(), P[i], f"p step {step} tensor {i}")
            assert_bit_equal(dM[i].get(), M[i], f"m step {step} tensor {i}")
            assert_bit_equal(dV[i].get(), V[i], f"v step {step} tensor {i}")


def test_allocator_reuse_and_limit(gpu):
    lib = gpu._ffi.lib()
    gpu.synchronize()
    lib.ts_allocator_release_cached()
    s0 = gpu.allocator_stats()
    p = lib.cuda_malloc(1 << 20)
    assert p
    lib.cuda_free(p)
    q = lib.cuda_malloc(1 << 20)
    assert q == p, "a freed block of the same size is reused"
    lib.cuda_free(q)
    s1 = gpu.allocator_stats()
    assert s1["driver_allocations"] == s0["driver_allocations"] + 1 and s1["cache_hits"] >= s0["cache_hits"] + 1
    # injected cap: the request fails with NULL and a message, nothing aborts
    lib.ts_allocator_set_limit(s1["bytes_reserved"] + (1 << 20))
    big = lib.cuda_malloc(1 << 28)
    assert big is None and "limit" in gpu._ffi.last_error()
    lib.ts_allocator_set_limit(0)
    lib.cuda_free(None)
