"""GPU: reductions over axes (raw launchers and engine ops) against the oracle and f64.

Bars.  max / min and every backward formula given the same saved values: bit for bit.  Sums: within the f64 value by
1e-6 of the sum of magnitudes (the device adds in a tree where the range is split or a warp shares an output, and in
the reference's sequential order where one thread owns an output and the range is not split: those are exact
against the oracle)."""
import ctypes as C
import itertools

import numpy as np
import pytest

from conftest import assert_bit_equal
from devbuf import DevBuf

pytestmark = pytest.mark.gpu
OPS = {"sum": 0, "max": 1, "min": 2, "sumsq": 3, "sqdev": 4, "counteq": 5}


def raw_reduce(gpu, op, x, dims, aux=None):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    dx = DevBuf(gpu, x)
    kept = [s for i, s in enumerate(x.shape) if i not in dims]
    n_out = int(np.prod(kept, dtype=np.int64)) if kept else 1
    do = DevBuf(gpu, n=n_out)
    da = DevBuf(gpu, aux) if aux is not None else None
    sc = DevBuf(gpu, n=int(lib.ts_reduce_dims_scratch_elems()))
    d = (C.c_ulonglong * x.ndim)(*x.shape)
    ax = (C.c_ulonglong * max(len(dims), 1))(*dims)
    chk(lib.launch_reduce_dims_kernel(OPS[op], dx.ptr, da.ptr if da else None, do.ptr, d, x.ndim, ax, len(dims), sc.ptr, None), op)
    return do.get().reshape(kept or [1])


def f64(op, x, dims, aux=None):
    x = x.astype(np.float64)
    ax = tuple(dims)
    if op == "sum": return x.sum(axis=ax)
    if op == "max": return x.max(axis=ax)
    if op == "min": return x.min(axis=ax)
    if op == "sumsq": return (x * x).sum(axis=ax)
    a = np.expand_dims(aux.astype(np.float64), ax)
    if op == "sqdev": return ((x.astype(np.float32) - a.astype(np.float32)).astype(np.float64) ** 2).sum(axis=ax)
    return (x == a).sum(axis=ax).astype(np.float64)


@pytest.mark.parametrize("shape", [(7,), (5, 9), (33, 65), (3, 40, 50), (2, 3, 4, 5), (6, 1, 7), (1, 1, 5), (300, 1000), (4099, 3)])
def test_raw_forward_every_axis_subset(gpu, shape):
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape).astype(np.float32)
    subsets = [d for k in range(1, len(shape) + 1) for d in itertools.combinations(range(len(shape)), k)]
    for dims in subsets:
        dims = list(dims)
        for op in ("sum", "max", "min", "sumsq"):
            got = raw_reduce(gpu, op, x, dims)
            want = f64(op, x, dims)
            if op in ("max", "min"):
                assert_bit_equal(got.reshape(-1), want.astype(np.float32).reshape(-1), f"{op} {shape} {dims}")
            else:
                mag = f64("sum", np.abs(x) if op == "sum" else x * x, dims) if op == "sum" else want
                assert np.all(np.abs(got.reshape(-1) - want.reshape(-1)) <= 1e-6 * np.maximum(np.abs(mag).reshape(-1), 1e-30) + 1e-30), (op, shape, dims)
        mean = (f64("sum", x, dims) / np.prod([shape[i] for i in dims])).astype(np.float32)
        got = raw_reduce(gpu, "sqdev", x, dims, aux=mean)
        want = f64("sqdev", x, dims, aux=mean)
        assert np.all(np.abs(got.reshape(-1) - want.reshape(-1)) <= 2e-6 * np.abs(want).reshape(-1) + 1e-30), (shape, dims)
        mx = f64("max", x, dims).astype(np.float32)
        cnt = raw_reduce(gpu, "counteq", x, dims, aux=mx)
        assert_bit_equal(cnt.reshape(-1), f64("counteq", x, dims, aux=mx).astype(np.float32).reshape(-1), f"counteq {shape} {dims}")


def test_sequential_order_when_one_thread_owns_an_output(gpu, ora):
    """Leading axes reduced, no split (many outputs): the device adds in the reference's order, so sums are exact."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal((40, 600000)).astype(np.float32)           # 600000 outputs fill the GPU without a split
    got = raw_reduce(gpu, "sum", x, [0])
    assert_bit_equal(got, ora.reduce_dims("sum", x, [0], False), "column sums in row order")


def test_large_split_reductions(gpu):
    """268 MB, few outputs: the reduced range is split over the whole GPU and combined by a second launch."""
    rng = np.random.default_rng(2)
    x = rng.standard_normal((1 << 26) + 3, dtype=np.float32)
    for op in ("sum", "max", "min", "sumsq"):
        got = raw_reduce(gpu, op, x, [0])
        want = f64(op, x, [0])
        if op in ("max", "min"):
            assert float(got[0]) == float(want)
        else:
            scale = float(np.abs(x).astype(np.float64).sum()) if op == "sum" else float(want)
            assert abs(float(got[0]) - float(want)) <= 1e-6 * scale
    m = x[: (1 << 26)].reshape(8192, 8192)
    for dims in ([0], [1]):
        got = raw_reduce(gpu, "sum", m, dims)
        want = f64("sum", m, dims)
        assert np.all(np.abs(got - want) <= 1e-6 * np.abs(m).astype(np.float64).sum(axis=dims[0]))
        assert_bit_equal(raw_reduce(gpu, "max", m, dims), m.max(axis=dims[0]))


def test_nan_and_empty(gpu):
    x = np.array([[np.nan, 1.0, 3.0], [np.nan, np.nan, np.nan]], np.float32)
    assert raw_reduce(gpu, "max", x, [1]).tolist() == [3.0, -np.inf]
    assert raw_reduce(gpu, "min", x, [1]).tolist() == [1.0, np.inf]
    e = np.zeros((0, 3), np.float32)
    assert raw_reduce(gpu, "sum", e, [0]).tolist() == [0, 0, 0]
    assert raw_reduce(gpu, "max", e, [0]).tolist() == [-np.inf] * 3
    lib = gpu._ffi.lib()
    d = DevBuf(gpu, n=8)
    assert lib.launch_reduce_dims_kernel(0, d.ptr, None, d.ptr, (C.c_ulonglong * 2)(2, 4), 2, (C.c_ulonglong * 1)(2), 1, d.ptr, None) is False
    assert "out of bounds" in gpu._ffi.last_error()


KINDS = ["sum", "mean", "max", "min", "norm", "var", "std"]


@pytest.mark.parametrize("kind", KINDS)
def test_engine_dims_ops_against_oracle(gpu, ora, kind):
    rng = np.random.default_rng(len(kind))
    T = gpu.Tensor
    for shape in [(4, 5), (3, 4, 5), (2, 3, 4, 5)]:
        xh = rng.standard_normal(shape).astype(np.float32)
        for dims in ([0], [len(shape) - 1], [0, len(shape) - 1], list(range(len(shape)))):
            for keepdim in (False, True):
                x = T.from_slice(xh, list(shape)).with_requires_grad()
                y = getattr(x, kind + "_dims")(dims, keepdim)
                want, mu = ora.reduce_dims(kind, xh, dims, keepdim, want_mean=True)
                assert y.shape().dims == list(want.shape)
                if kind in ("max", "min"):
                    assert_bit_equal(y.data(), want)
                else:
                    np.testing.assert_allclose(y.data(), want, rtol=2e-6, atol=1e-6)
                up = rng.standard_normal(want.shape).astype(np.float32)
                y.backward(T.from_slice(up, list(want.shape)))
                g = x.grad_by_value()
                assert g.shape().dims == list(shape)
                # backward from the DEVICE's forward values, so that the comparison is of the formula alone
                gi = ora.reduce_dims_backward(kind, xh, y.data(), _device_mean(kind, xh, dims, keepdim, ora), up, dims)
                if kind in ("var", "std", "norm"):
                    np.testing.assert_allclose(g.data(), gi, rtol=3e-6, atol=1e-6)
                else:
                    assert_bit_equal(g.data(), gi, f"{kind} {shape} {dims}")
                gpu.clear_gradients()


def _device_mean(kind, xh, dims, keepdim, ora):
    if kind not in ("var", "std"):
        return None
    return ora.reduce_dims("sum", xh, dims, keepdim) / np.float32(np.prod([xh.shape[d] for d in set(dims)]))


@pytest.mark.parametrize("kind", ["max", "min", "norm", "var", "std"])
def test_engine_whole_tensor_forms(gpu, ora, kind):
    rng = np.random.default_rng(3)
    xh = rng.standard_normal((37, 11)).astype(np.float32)
    x = gpu.Tensor.from_slice(xh, [37, 11]).with_requires_grad()
    y = getattr(x, kind)()
    want, mu = ora.reduce_all(kind, xh, want_mean=True)
    assert y.shape().dims == [1]
    np.testing.assert_allclose(y.data(), want, rtol=2e-6)
    y.backward()
    gi = ora.reduce_dims_backward(kind, xh, y.data(), mu, np.ones(1, np.float32), None)
    np.testing.assert_allclose(x.grad_by_value().data(), gi, rtol=3e-6, atol=1e-7)


def test_engine_ties_and_errors(gpu):
    T = gpu.Tensor
    x = T.from_slice([1, 5, 5, 2, 3, 3, 3, 3], [2, 4]).with_requires_grad()
    x.max_dims([1], False).backward(T.from_slice([1.0, 2.0], [2]))
    assert x.grad_by_value().data().tolist() == [[0, 0.5, 0.5, 0], [0.5, 0.5, 0.5, 0.5]]      # grad_fn/reductions/max.rs
    E = gpu.TrainStationError
    with pytest.raises(E, match="requires at least one dimension"):
        T.ones([2, 3]).sum_dims([], False)
    with pytest.raises(E, match="out of bounds for rank 2"):
        T.ones([2, 3]).mean_dims([2], False)
    assert T.ones([2, 3]).sum_dims([0, 0, 1], False).data().tolist() == [6.0]               # duplicates are dropped (sum.rs:238-240)
    assert T.new([0]).var().data().tolist() == [0.0]
    # layer-norm style chain through the engine: (x - mean) / std over the last axis
    xh = np.random.default_rng(0).standard_normal((6, 8)).astype(np.float32)
    x = T.from_slice(xh, [6, 8]).with_requires_grad()
    mu = x.mean_dims([1], True)
    sd = x.std_dims([1], True)
    assert mu.shape().dims == [6, 1] and sd.shape().dims == [6, 1]
    np.testing.assert_allclose(mu.data()[:, 0], xh.mean(axis=1), rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(sd.data()[:, 0], xh.std(axis=1), rtol=2e-6)
