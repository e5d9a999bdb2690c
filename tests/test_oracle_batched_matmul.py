"""CPU: the oracle's batched matmul (tensor/ops/matmul/mod.rs:634-835) and its gradients
(gradtrack/grad_fn/ops/matmul.rs, the batched branches) against float64 numpy, whose matmul broadcasts batch axes by
the same right-aligned rule."""
import numpy as np
import pytest

# (left, right): the batched shapes libtorch-validation/src/validation/tensor/ops/matmul.rs runs, plus broadcasts
# over more than one axis and 2-D operands on either side
CASES = [((2, 3, 3), (2, 3, 4)), ((3, 2, 4), (3, 4, 2)), ((1, 3, 4), (2, 4, 5)), ((3, 2, 3), (1, 3, 4)),
         ((2, 3, 4), (4, 5)), ((3, 4), (2, 4, 5)), ((1, 3, 4), (4, 5)), ((3, 4), (1, 4, 5)),
         ((2, 1, 3, 4), (5, 4, 2)), ((2, 3, 2, 4), (1, 3, 4, 2)), ((4, 1, 2, 3), (1, 5, 3, 2))]


def want_shape(a, b):
    full = list(np.broadcast_shapes(a[:-2], b[:-2])) + [a[-2], b[-1]]
    if (len(a) == 2 or len(b) == 2) and len(full) > 2 and full[0] == 1:     # mod.rs:752-756
        full = full[1:]
    return full


@pytest.mark.parametrize("sa,sb", CASES)
def test_forward_against_f64(ora, sa, sb):
    rng = np.random.default_rng(sum(sa) * 31 + sum(sb))
    a, b = rng.standard_normal(sa).astype(np.float32), rng.standard_normal(sb).astype(np.float32)
    got = ora.batched_matmul(a, b)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    assert list(got.shape) == want_shape(sa, sb)
    np.testing.assert_allclose(got.reshape(-1), want.reshape(-1), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("sa,sb", CASES)
def test_gradients_against_f64(ora, sa, sb):
    rng = np.random.default_rng(sum(sa) * 17 + sum(sb))
    a, b = rng.standard_normal(sa).astype(np.float32), rng.standard_normal(sb).astype(np.float32)
    y = ora.batched_matmul(a, b)
    go = rng.standard_normal(y.shape).astype(np.float32)
    ga, gb = ora.batched_matmul_backward(a, b, go)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    full = np.matmul(a64, b64)
    g64 = go.astype(np.float64).reshape(full.shape)
    wa = np.matmul(g64, np.swapaxes(b64, -1, -2))
    wb = np.matmul(np.swapaxes(a64, -1, -2), g64)

    def fold(g, shape):        # sum a broadcast gradient back to the operand's shape
        while g.ndim > len(shape):
            g = g.sum(axis=0)
        for i, s in enumerate(shape):
            if s == 1 and g.shape[i] > 1:
                g = g.sum(axis=i, keepdims=True)
        return g

    assert ga.shape == a.shape and gb.shape == b.shape
    np.testing.assert_allclose(ga, fold(wa, sa), rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(gb, fold(wb, sb), rtol=2e-5, atol=2e-5)


def test_reference_unit_test_values(ora):
    """mod.rs test_simple_batched_gradient: [2,2,2] @ [2,2,2] with a gradient of ones; the expected left gradient rows
    are the row sums of the right operand, which the test writes out for both batch entries."""
    left = np.arange(1, 9, dtype=np.float32).reshape(2, 2, 2)
    right = (np.arange(1, 9, dtype=np.float32) * 0.5).reshape(2, 2, 2)
    y = ora.batched_matmul(left, right)
    np.testing.assert_array_equal(y, np.array([[[3.5, 5.0], [7.5, 11.0]], [[33.5, 39.0], [45.5, 53.0]]], np.float32))
    ga, gb = ora.batched_matmul_backward(left, right, np.ones((2, 2, 2), np.float32))
    np.testing.assert_array_equal(ga, np.array([[[1.5, 3.5], [1.5, 3.5]], [[5.5, 7.5], [5.5, 7.5]]], np.float32))
    np.testing.assert_array_equal(gb, np.array([[[4.0, 4.0], [6.0, 6.0]], [[12.0, 12.0], [14.0, 14.0]]], np.float32))


def test_errors(ora):
    with pytest.raises(ValueError, match="Inner dimensions must match for batched matmul: 4 vs 3"):
        ora.batched_matmul(np.zeros((2, 3, 4), np.float32), np.zeros((2, 3, 4), np.float32))
    with pytest.raises(ValueError, match="Cannot broadcast dimensions 2 and 3"):
        ora.batched_matmul(np.zeros((2, 3, 4), np.float32), np.zeros((3, 4, 2), np.float32))
    with pytest.raises(ValueError, match="at least 2D"):
        ora.batched_matmul(np.zeros((2, 3, 4), np.float32), np.zeros((4,), np.float32))
