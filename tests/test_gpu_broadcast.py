"""GPU: add/sub/mul/div_tensor with NumPy-style broadcasting (tensor/ops/{add,sub,mul,div}.rs through
broadcasting.rs:100-135) and the reduction of their gradients to the operands' shapes (grad_fn/utils.rs:23-60).
The forward is one rounded IEEE operation per element, so it equals the oracle bit for bit; the gradients add up
many terms in another order than the oracle's axis-by-axis sums and are compared within a few ulps of the sum."""
import numpy as np
import pytest

from conftest import assert_bit_equal
from test_oracle_broadcast import OPS, SHAPES, operands

pytestmark = pytest.mark.gpu


def dev_op(t, op, other):
    return getattr(t, f"{op}_tensor")(other)


@pytest.mark.parametrize("sa,sb", SHAPES)
@pytest.mark.parametrize("op", OPS)
def test_forward_and_gradients_against_the_oracle(gpu, ora, op, sa, sb):
    T = gpu.Tensor
    a, b = operands(sa, sb, len(sa) * 5 + len(sb))
    ta, tb = T.from_slice(a, list(sa)).with_requires_grad(), T.from_slice(b, list(sb)).with_requires_grad()
    y = dev_op(ta, op, tb)
    want = ora.binary_broadcast(op, a, b)
    assert y.shape().dims == list(want.shape)
    assert_bit_equal(y.data(), want, f"{op} {sa} {sb}")
    go = np.random.default_rng(9).standard_normal(want.shape).astype(np.float32)
    y.backward(T.from_slice(go, list(want.shape)))
    wa, wb = ora.binary_broadcast_backward(op, a, b, go)
    for got, w, shape in ((ta.grad_by_value(), wa, sa), (tb.grad_by_value(), wb, sb)):
        assert got.shape().dims == list(shape)
        terms = want.size // w.size
        if terms == 1:
            assert_bit_equal(got.data(), w, f"grad {op} {sa} {sb}")
        else:
            np.testing.assert_allclose(got.data(), w, rtol=1e-5, atol=2e-6 * terms)


@pytest.mark.parametrize("op", OPS)
def test_large_row_column_and_outer_shapes(gpu, op):
    """Sizes that fill the grid several times over, through the vector path (innermost extent a multiple of 4, one
    operand stretched along it or along the outer axis) and the scalar path (odd innermost extent)."""
    T = gpu.Tensor
    for sa, sb in [((1500, 1024), (1, 1024)), ((1500, 1024), (1500, 1)), ((1500, 1), (1, 1024)), ((3, 700, 333), (700, 1)),
                   ((1023, 1), (1, 1025))]:
        a, b = operands(sa, sb, sa[0])
        y = dev_op(T.from_slice(a, list(sa)), op, T.from_slice(b, list(sb))).data()
        want = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide}[op](a, b)
        assert_bit_equal(y, want, f"{op} {sa} {sb}")


def test_result_shape_keeps_the_leading_ones_of_a_one_element_operand(gpu):
    T = gpu.Tensor
    y = T.ones([1, 1, 1]).add_tensor(T.ones([5, 6]))
    assert y.shape().dims == [1, 5, 6]
    assert T.ones([5, 6]).add_tensor(T.ones([1])).shape().dims == [5, 6]


def test_reference_unit_tests_of_the_gradient_reduction(gpu):
    """grad_fn/utils.rs tests: ones of [2, 3] reduced to [2, 1] give 3s, reduced to [3] give 2s."""
    T = gpu.Tensor
    a, b = T.zeros([2, 1]).with_requires_grad(), T.zeros([3]).with_requires_grad()
    a.add_tensor(b).backward(T.ones([2, 3]))
    assert_bit_equal(a.grad_by_value().data(), np.full((2, 1), 3.0, np.float32))
    assert_bit_equal(b.grad_by_value().data(), np.full((3,), 2.0, np.float32))


def test_broadcast_inside_a_graph(gpu, ora):
    """A normalisation written with broadcasting: (x - mean over rows) / (std over rows), then a weighted sum."""
    T = gpu.Tensor
    rng = np.random.default_rng(12)
    xh, wh = rng.standard_normal((6, 40)).astype(np.float32), rng.standard_normal((6, 40)).astype(np.float32)
    x = T.from_slice(xh, [6, 40]).with_requires_grad()
    mu = x.mean_dims([1], True)
    sd = x.std_dims([1], True)
    z = x.sub_tensor(mu).div_tensor(sd)
    z.mul_tensor(T.from_slice(wh, [6, 40])).sum().backward()
    x64, w64 = xh.astype(np.float64), wh.astype(np.float64)
    n = 40
    m = x64.mean(1, keepdims=True)
    s = x64.std(1, keepdims=True, ddof=1) if _unbiased(gpu) else x64.std(1, keepdims=True)
    z64 = (x64 - m) / s
    np.testing.assert_allclose(z.data(), z64, rtol=2e-5, atol=2e-6)
    ddof = 1 if _unbiased(gpu) else 0
    gz = w64
    gs = -(gz * (x64 - m)).sum(1, keepdims=True) / (s * s)
    gx = gz / s + gs * (x64 - m) / ((n - ddof) * s) - (gz / s).sum(1, keepdims=True) / n
    np.testing.assert_allclose(x.grad_by_value().data(), gx, rtol=2e-4, atol=2e-5)


def _unbiased(gpu):
    T = gpu.Tensor
    v = T.from_slice(np.array([1.0, 3.0], np.float32), [1, 2]).std_dims([1], True).data()[0, 0]
    return abs(v - np.sqrt(2.0)) < 1e-6


def test_incompatible_shapes_message(gpu):
    T = gpu.Tensor
    with pytest.raises(gpu.TrainStationError, match=r"Cannot broadcast tensor shapes \[2, 3\] and \[4, 2\]: Cannot broadcast shapes "
                                                    r"\[2, 3\] and \[4, 2\]: incompatible dimensions at axis 1"):
        T.ones([2, 3]).add_tensor(T.ones([4, 2]))
    for op in OPS:
        with pytest.raises(gpu.TrainStationError, match="incompatible dimensions at axis 0"):
            dev_op(T.ones([2, 3]), op, T.ones([4, 3]))
