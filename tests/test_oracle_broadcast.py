"""CPU: the oracle's broadcasting add/sub/mul/div (tensor/ops/{add,sub,mul,div}.rs through broadcasting.rs) and the
reduction of their gradients to the operands' shapes (gradtrack/grad_fn/utils.rs:23-60) against numpy, whose
broadcasting rule is the one the reference implements."""
import numpy as np
import pytest

OPS = ["add", "sub", "mul", "div"]
# pairs of shapes: trailing match, column times row, interior 1s, rank differences, one-element operands, and sizes
# whose innermost axis takes the vector path of the device kernel
SHAPES = [((2, 3), (1, 3)), ((3, 1), (1, 4)), ((2, 3, 4), (3, 1)), ((4,), (3, 1)), ((2, 1, 4), (3, 1)), ((1,), (2, 3)),
          ((2, 3), (1,)), ((1, 1, 1), (5, 6)), ((8, 1, 6, 1), (7, 1, 5)), ((64, 128), (128,)), ((64, 1), (1, 128)),
          ((5, 7), (7,)), ((6, 8), (6, 1)), ((3, 1, 8), (1, 5, 1)), ((2, 2, 1, 1, 3, 1, 4), (2, 1, 3, 1, 5, 1))]
NP = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide}


def operands(sa, sb, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal(sa).astype(np.float32)
    b = (rng.standard_normal(sb) + np.where(rng.random(sb) < 0.5, 3.0, -3.0)).astype(np.float32)    # away from zero for div
    return a, b


@pytest.mark.parametrize("sa,sb", SHAPES)
@pytest.mark.parametrize("op", OPS)
def test_forward_is_numpy_bit_for_bit(ora, op, sa, sb):
    a, b = operands(sa, sb, len(sa) * 7 + len(sb))
    got = ora.binary_broadcast(op, a, b)
    want = NP[op](a, b)
    assert got.shape == want.shape
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def fold(g, shape):
    while g.ndim > len(shape):
        g = g.sum(axis=0)
    for i, s in enumerate(shape):
        if s == 1 and g.shape[i] > 1:
            g = g.sum(axis=i, keepdims=True)
    return g


@pytest.mark.parametrize("sa,sb", SHAPES)
@pytest.mark.parametrize("op", OPS)
def test_gradients_against_f64(ora, op, sa, sb):
    a, b = operands(sa, sb, len(sa) * 11 + len(sb))
    out_shape = np.broadcast_shapes(sa, sb)
    go = np.random.default_rng(5).standard_normal(out_shape).astype(np.float32)
    ga, gb = ora.binary_broadcast_backward(op, a, b, go)
    a64, b64, g64 = a.astype(np.float64), b.astype(np.float64), go.astype(np.float64)
    full = {"add": (g64 + 0 * b64, g64 + 0 * a64), "sub": (g64 + 0 * b64, -g64 + 0 * a64), "mul": (g64 * b64, g64 * a64),
            "div": (g64 / b64, -(g64 * a64) / (b64 * b64))}[op]
    assert ga.shape == a.shape and gb.shape == b.shape
    np.testing.assert_allclose(ga, fold(np.broadcast_to(full[0], out_shape), sa), rtol=3e-5, atol=3e-5)
    np.testing.assert_allclose(gb, fold(np.broadcast_to(full[1], out_shape), sb), rtol=3e-5, atol=3e-5)


def test_reference_unit_tests_of_the_gradient_reduction(ora):
    """grad_fn/utils.rs tests: ones of [2, 3] reduced to [2, 1] give 3s, reduced to [3] give 2s."""
    ones = np.ones((2, 3), np.float32)
    ga, gb = ora.binary_broadcast_backward("add", np.zeros((2, 1), np.float32), np.zeros((3,), np.float32), ones)
    np.testing.assert_array_equal(ga, np.full((2, 1), 3.0, np.float32))
    np.testing.assert_array_equal(gb, np.full((3,), 2.0, np.float32))


def test_incompatible_shapes_message(ora):
    with pytest.raises(ValueError, match=r"Cannot broadcast tensor shapes \[2, 3\] and \[4, 2\]: Cannot broadcast shapes \[2, 3\] "
                                         r"and \[4, 2\]: incompatible dimensions at axis 1"):
        ora.binary_broadcast("add", np.zeros((2, 3), np.float32), np.zeros((4, 2), np.float32))
    with pytest.raises(ValueError, match="incompatible dimensions at axis 0"):
        ora.binary_broadcast("mul", np.zeros((2, 3), np.float32), np.zeros((4, 3), np.float32))
