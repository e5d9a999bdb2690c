"""CPU: the oracle's reductions over axes against f64 evaluations and against each other.  The literal values of the
reference's unit tests for these ops run through test_oracle_golden.py (reference_known_answers.json)."""
import itertools

import numpy as np
import pytest

SHAPES = [(7,), (4, 5), (3, 4, 5), (2, 3, 4, 5), (1, 6, 1), (5, 1, 3)]
KINDS = ["sum", "mean", "max", "min", "norm", "var", "std"]


def f64_reduce(kind, x, dims, keepdim):
    x = x.astype(np.float64)
    ax = tuple(sorted(set(dims)))
    f = {"sum": np.sum, "mean": np.mean, "max": np.max, "min": np.min, "var": np.var, "std": np.std,
         "norm": lambda a, axis, keepdims: np.sqrt(np.sum(a * a, axis=axis, keepdims=keepdims))}[kind]
    r = f(x, axis=ax, keepdims=keepdim)
    return np.asarray(r).reshape(r.shape if np.ndim(r) else (1,))


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("kind", KINDS)
def test_forward_every_axis_subset(ora, kind, shape):
    rng = np.random.default_rng(len(shape) + len(kind))
    x = rng.standard_normal(shape).astype(np.float32)
    for k in range(1, len(shape) + 1):
        for dims in itertools.combinations(range(len(shape)), k):
            for keepdim in (False, True):
                got = ora.reduce_dims(kind, x, list(dims), keepdim)
                want = f64_reduce(kind, x, dims, keepdim)
                assert list(got.shape) == (list(want.shape) or [1]), (kind, shape, dims, keepdim)
                np.testing.assert_allclose(got.reshape(-1), want.reshape(-1), rtol=2e-6, atol=2e-6)


@pytest.mark.parametrize("kind", ["max", "min", "norm", "var", "std"])
def test_whole_tensor_forms_agree_with_all_axes(ora, kind):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((6, 7, 3)).astype(np.float32)
    a = ora.reduce_all(kind, x)
    b = ora.reduce_dims(kind, x, [0, 1, 2], False)
    assert a.shape == (1,) and b.shape == (1,)
    np.testing.assert_allclose(a, b, rtol=1e-6)
    assert ora.reduce_all("var", np.zeros(0, np.float32))[0] == 0.0        # var.rs:103-105
    assert ora.reduce_all("max", np.zeros(0, np.float32))[0] == -np.inf    # max.rs:33-35


def numeric_grad(kind, x, dims, keepdim, up):
    """Central differences in f64 of sum(up * reduce(x))."""
    x64 = x.astype(np.float64)
    g = np.zeros_like(x64)
    eps = 1e-6
    it = np.nditer(x64, flags=["multi_index"])
    for _ in it:
        i = it.multi_index
        xp, xm = x64.copy(), x64.copy()
        xp[i] += eps; xm[i] -= eps
        fp = f64_reduce(kind, xp, dims, keepdim).reshape(-1)
        fm = f64_reduce(kind, xm, dims, keepdim).reshape(-1)
        g[i] = np.sum(up.reshape(-1) * (fp - fm)) / (2 * eps)
    return g


@pytest.mark.parametrize("kind", ["sum", "mean", "norm", "var", "std", "max", "min"])
def test_backward_matches_numeric_gradient(ora, kind):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((3, 4, 2)).astype(np.float32)       # distinct values: no ties for max / min
    for dims in ([1], [0, 2], [0, 1, 2]):
        y, mu = ora.reduce_dims(kind, x, dims, False, want_mean=True)
        up = rng.standard_normal(y.shape).astype(np.float32)
        gi = ora.reduce_dims_backward(kind, x, y, mu, up, dims)
        np.testing.assert_allclose(gi, numeric_grad(kind, x, dims, False, up.astype(np.float64)), rtol=2e-4, atol=2e-5)


def test_ties_share_the_gradient_equally(ora):
    """grad_fn/reductions/max.rs:40-75: every element equal to the maximum gets upstream / count."""
    x = np.array([[1, 5, 5, 2], [3, 3, 3, 3]], np.float32)
    y = ora.reduce_dims("max", x, [1], False)
    gi = ora.reduce_dims_backward("max", x, y, None, np.array([1.0, 2.0], np.float32), [1])
    assert gi.tolist() == [[0, 0.5, 0.5, 0], [0.5, 0.5, 0.5, 0.5]]
    ya = ora.reduce_all("min", x)
    ga = ora.reduce_dims_backward("min", x, ya, None, np.array([3.0], np.float32), None)
    assert ga.tolist() == [[3.0, 0, 0, 0], [0, 0, 0, 0]]
    # a scalar upstream is used for every output (max.rs: `if grad_output.size() == 1`)
    gs = ora.reduce_dims_backward("max", x, y, None, np.array([4.0], np.float32), [1])
    assert gs.tolist() == [[0, 2, 2, 0], [1, 1, 1, 1]]


def test_zero_norm_and_zero_std_have_zero_gradient(ora):
    x = np.array([[0, 0, 0], [2, 2, 2]], np.float32)
    n, _ = ora.reduce_dims("norm", x, [1], False, want_mean=True)
    g = ora.reduce_dims_backward("norm", x, n, None, np.ones(2, np.float32), [1])
    assert g[0].tolist() == [0, 0, 0] and np.all(g[1] > 0)
    s, mu = ora.reduce_dims("std", x, [1], False, want_mean=True)
    g = ora.reduce_dims_backward("std", x, s, mu, np.ones(2, np.float32), [1])
    assert np.all(g == 0)


def test_nan_is_ignored_by_max_and_min(ora):
    x = np.array([[np.nan, 1.0, 3.0], [np.nan, np.nan, np.nan]], np.float32)
    assert ora.reduce_dims("max", x, [1], False).tolist() == [3.0, -np.inf]     # `if val > cur` never takes a NaN
    assert ora.reduce_dims("min", x, [1], False).tolist() == [1.0, np.inf]


def test_errors(ora):
    x = np.zeros((2, 3), np.float32)
    with pytest.raises(ValueError):
        ora.reduce_dims("sum", x, [], False)        # sum.rs:226
    with pytest.raises(IndexError):
        ora.reduce_dims("sum", x, [2], False)       # sum.rs:228-235
