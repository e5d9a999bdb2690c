"""GPU: cat / stack / split / split_with_sizes (tensor/transform/{cat,stack,split}.rs) and their GradFns
(grad_fn/transforms/{cat,split}.rs).  Data movement only: every comparison with numpy is bit for bit."""
import numpy as np
import pytest

from conftest import assert_bit_equal

pytestmark = pytest.mark.gpu


def test_cat_every_axis(gpu):
    T = gpu.Tensor
    rng = np.random.default_rng(0)
    for shape, lens, dim in [((3, 4), [4, 1, 7], 1), ((3, 4), [2, 5], 0), ((2, 3, 4), [1, 2, 3], 1), ((2, 3, 4), [4, 4], 2), ((5,), [5, 0, 2], 0),
                             ((300, 70), [70, 130], 1)]:
        parts = []
        for n in lens:
            s = list(shape)
            s[dim] = n
            parts.append(rng.standard_normal(s).astype(np.float32))
        y = T.cat([T.from_slice(p, list(p.shape)) for p in parts], dim)
        want = np.concatenate(parts, axis=dim)
        assert y.shape().dims == list(want.shape)
        assert_bit_equal(y.data(), want, f"{shape} dim {dim}")


def test_cat_and_stack_gradients(gpu):
    T = gpu.Tensor
    rng = np.random.default_rng(1)
    a, b, c = (rng.standard_normal(s).astype(np.float32) for s in [(2, 3), (2, 5), (2, 1)])
    ta, tb, tc = T.from_slice(a, [2, 3]).with_requires_grad(), T.from_slice(b, [2, 5]), T.from_slice(c, [2, 1]).with_requires_grad()
    w = rng.standard_normal((2, 9)).astype(np.float32)
    T.cat([ta, tb, tc], 1).mul_tensor(T.from_slice(w, [2, 9])).sum().backward()
    assert_bit_equal(ta.grad_by_value().data(), w[:, :3])
    assert_bit_equal(tc.grad_by_value().data(), w[:, 8:])
    assert tb.grad_by_value() is None
    gpu.clear_gradients()
    xs = [rng.standard_normal((2, 3)).astype(np.float32) for _ in range(4)]
    ts_ = [T.from_slice(x, [2, 3]).with_requires_grad() for x in xs]
    for dim in (0, 1, 2):
        s = T.stack(ts_, dim)
        want = np.stack(xs, axis=dim)
        assert s.shape().dims == list(want.shape)
        assert_bit_equal(s.data(), want, f"stack {dim}")
        up = rng.standard_normal(want.shape).astype(np.float32)
        s.mul_tensor(T.from_slice(up, list(want.shape))).sum().backward()
        for k, t in enumerate(ts_):
            assert_bit_equal(t.grad_by_value().data(), np.take(up, k, axis=dim), f"stack grad {dim} {k}")
        gpu.clear_gradients()


def test_split_forward_and_gradient(gpu):
    T = gpu.Tensor
    xh = np.arange(12, dtype=np.float32).reshape(2, 6)                # split.rs tests: test_split_equal_forward
    x = T.from_slice(xh, [2, 6]).with_requires_grad()
    parts = x.split(2, 1)
    assert [p.shape().dims for p in parts] == [[2, 2]] * 3
    for k, p in enumerate(parts):
        assert_bit_equal(p.data(), xh[:, 2 * k:2 * k + 2])
    uneven = x.split(4, 1)
    assert [p.shape().dims for p in uneven] == [[2, 4], [2, 2]]
    rows = x.split_with_sizes([1, 0, 1], 0)
    assert [p.shape().dims for p in rows] == [[1, 6], [0, 6], [1, 6]]
    # every piece contributes to the input's gradient in its own slab; pieces used twice accumulate
    loss = parts[0].sum().add_tensor(parts[2].mul_tensor(parts[2]).sum()).add_tensor(parts[0].sum())
    loss.backward()
    want = np.zeros_like(xh)
    want[:, 0:2] = 2.0
    want[:, 4:6] = 2.0 * xh[:, 4:6]
    assert_bit_equal(x.grad_by_value().data(), want)


def test_errors(gpu):
    T = gpu.Tensor
    E = gpu.TrainStationError
    a, b = T.ones([2, 3]), T.ones([3, 3])
    with pytest.raises(E, match="at least one tensor"):
        T.cat([], 0)
    with pytest.raises(E, match="out of bounds for rank 2"):
        T.cat([a, a], 2)
    with pytest.raises(E, match="All dims except concat dim must match"):
        T.cat([a, b], 1)
    with pytest.raises(E, match="same rank"):
        T.cat([a, T.ones([2, 3, 1])], 0)
    with pytest.raises(E, match="identical shapes"):
        T.stack([a, b], 0)
    with pytest.raises(E, match="stack dim 3 out of bounds"):
        T.stack([a, a], 3)
    with pytest.raises(E, match="split_size must be > 0"):
        a.split(0, 0)
    with pytest.raises(E, match="must equal size 3 of dim 1"):
        a.split_with_sizes([1, 1], 1)
    with pytest.raises(E, match="split dim 2 out of bounds"):
        a.split(1, 2)
    assert T.new([0, 3]).split(2, 0) == []
