"""GPU: transpose() / t() / permute() return VIEWS that share the tensor's storage, as in the reference
(tensor/transform/transpose.rs:181-184, core/allocation.rs:220-237): a write to the tensor is seen through the view and a
write through the view lands in the tensor; contiguous() makes the copy; reshape of a view copies first; a transposed 2-D
view as a matmul operand costs no kernel at all (the GEMM flips its transposition flag)."""
import numpy as np
import pytest

from conftest import assert_bit_equal

pytestmark = pytest.mark.gpu


def test_view_and_tensor_alias_each_other(gpu):
    T = gpu.Tensor
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    x = T.from_slice(a, [3, 4])
    v = x.t()
    assert v.shape().dims == [4, 3] and not v.is_contiguous() and x.is_contiguous()
    assert_bit_equal(v.data(), a.T, "the view reads the tensor's elements in transposed order")
    x.fill(2.0)                                   # a write to the tensor is seen through the view
    assert np.all(v.data() == 2.0)
    b = np.arange(12, dtype=np.float32).reshape(4, 3) * 10
    v.copy_from_host(b)                           # a write through the view lands in the tensor, transposed back
    assert_bit_equal(x.data(), b.T, "write through the view")
    assert_bit_equal(v.data(), b, "and the view shows what was written")
    v.fill(-1.0)
    assert np.all(x.data() == -1.0)
    c = v.contiguous()                            # the copy: no longer aliased
    assert c.is_contiguous()
    x.fill(5.0)
    assert np.all(c.data() == -1.0) and np.all(v.data() == 5.0)


def test_permute_views_compose_and_reshape_copies(gpu):
    T = gpu.Tensor
    rng = np.random.default_rng(0)
    a = rng.standard_normal((3, 4, 5), dtype=np.float32)
    x = T.from_slice(a, [3, 4, 5])
    p = x.permute([2, 0, 1])
    assert_bit_equal(p.data(), a.transpose(2, 0, 1), "permute")
    q = p.permute([1, 2, 0])                      # back to the original order: an ordinary alias again
    assert q.is_contiguous()
    assert_bit_equal(q.data(), a, "composed permutations")
    assert_bit_equal(p.transpose(0, 2).data(), a.transpose(2, 0, 1).transpose(2, 1, 0), "a view of a view")
    r = p.reshape([5, 12])                        # reshape of a view copies first (reshape.rs), so it does not alias
    want = np.ascontiguousarray(a.transpose(2, 0, 1)).reshape(5, 12)
    assert_bit_equal(r.data(), want, "reshape of a view")
    x.fill(0.0)
    assert_bit_equal(r.data(), want, "the reshaped copy is its own tensor")
    assert np.all(p.data() == 0.0)
    # every other op sees the view's logical order
    y = T.from_slice(a.transpose(2, 0, 1).copy(), [5, 3, 4])
    x.copy_from_host(a)
    assert_bit_equal(p.add_tensor(y).data(), 2 * a.transpose(2, 0, 1), "elementwise on a view")
    assert_bit_equal(p.sum_dims([0], False).data(), y.sum_dims([0], False).data(), "reduction over a view")


def test_transposed_view_as_matmul_operand_costs_no_kernel(gpu, ora):
    T = gpu.Tensor
    lib = gpu._ffi.lib()
    rng = np.random.default_rng(1)
    a = rng.standard_normal((96, 64), dtype=np.float32)      # stored [k, m]; used as a.t(): [m, k]
    w = rng.standard_normal((96, 80), dtype=np.float32)
    for mode in (gpu.FP32, gpu.TF32):
        gpu.set_matmul_precision(mode)
        X, W = T.from_slice(a, [96, 64]), T.from_slice(w, [96, 80])
        gpu.synchronize()
        n0 = int(lib.ts_launch_count())
        y = X.t().matmul(W)
        out = y.data()
        launches = int(lib.ts_launch_count()) - n0
        # FP32 mode: the one GEMM.  TF32 mode: the GEMM plus the rounded copies of its two operands.  No transposing copy in either.
        assert launches == (1 if mode == gpu.FP32 else 3), launches
        if mode == gpu.FP32:
            assert_bit_equal(out, ora.matmul(np.ascontiguousarray(a.T), w), "x.t().matmul(w), FP32 mode")
        else:
            exact = a.T.astype(np.float64) @ w.astype(np.float64)
            mag = np.abs(a.T).astype(np.float64) @ np.abs(w).astype(np.float64)
            assert np.all(np.abs(out - exact) <= 2e-3 * mag)
        # the other side: x.matmul(w.t())
        b = rng.standard_normal((80, 64), dtype=np.float32)
        z = T.from_slice(a.T.copy(), [64, 96]).matmul(T.from_slice(np.ascontiguousarray(w.T), [80, 96]).t())
        if mode == gpu.FP32:
            assert_bit_equal(z.data(), ora.matmul(np.ascontiguousarray(a.T), w), "x.matmul(w.t()), FP32 mode")
        del b


def test_gradients_flow_through_views(gpu):
    T = gpu.Tensor
    rng = np.random.default_rng(2)
    a = rng.standard_normal((24, 16), dtype=np.float32)
    w = rng.standard_normal((24, 8), dtype=np.float32)
    X, W = T.from_slice(a, [24, 16]).with_requires_grad(), T.from_slice(w, [24, 8]).with_requires_grad()
    y = X.t().matmul(W)                           # [16, 8]
    y.sum().backward(None)
    ones = np.ones((16, 8))
    np.testing.assert_allclose(X.grad_by_value().data(), (ones @ w.T.astype(np.float64)).T, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(W.grad_by_value().data(), a.astype(np.float64) @ ones, rtol=1e-5, atol=1e-5)
    gpu.clear_gradients()
    # a view used by an elementwise op and a reduction
    P = T.from_slice(a, [24, 16]).with_requires_grad()
    P.permute([1, 0]).mul_tensor(T.from_slice(a.T.copy(), [16, 24])).sum().backward(None)
    np.testing.assert_allclose(P.grad_by_value().data(), a, rtol=1e-6, atol=1e-7)


def test_a_view_cannot_be_an_optimizer_parameter(gpu):
    x = gpu.Tensor.ones([4, 6]).with_requires_grad()
    v = x.t()
    opt = gpu.Adam.new()
    opt.add_parameter(v)
    v.sum().backward(None)
    with pytest.raises(gpu.TrainStationError, match="view"):
        opt.step([v])
