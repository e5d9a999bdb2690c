"""GPU: batched matmul (tensor/ops/matmul/mod.rs:634-835) and its gradients (gradtrack/grad_fn/ops/matmul.rs, the
batched branches) against the oracle.  Each batch entry is the 2-D product on offsets into the operands, so in FP32
mode the batched result must equal, bit for bit, the 2-D device products of the same slices."""
import numpy as np
import pytest

from conftest import assert_bit_equal
from test_oracle_batched_matmul import CASES, want_shape

pytestmark = pytest.mark.gpu


def _close(got, want, k):
    """FP32 accumulation in a different order than the oracle's blocked kernel: a few ulps of sqrt(k)-sized sums."""
    tol = 4e-6 * max(1.0, float(np.sqrt(k))) * max(1.0, float(np.abs(want).max()))
    np.testing.assert_allclose(got, want, rtol=0, atol=tol)


@pytest.mark.parametrize("sa,sb", CASES)
def test_forward_and_gradients_against_the_oracle(gpu, ora, sa, sb):
    T = gpu.Tensor
    rng = np.random.default_rng(sum(sa) * 13 + sum(sb))
    a, b = rng.standard_normal(sa).astype(np.float32), rng.standard_normal(sb).astype(np.float32)
    ta, tb = T.from_slice(a, list(sa)).with_requires_grad(), T.from_slice(b, list(sb)).with_requires_grad()
    y = ta.matmul(tb)
    want = ora.batched_matmul(a, b)
    assert y.shape().dims == want_shape(sa, sb) == list(want.shape)
    _close(y.data(), want, sa[-1])
    go = rng.standard_normal(want.shape).astype(np.float32)
    y.backward(T.from_slice(go, list(want.shape)))
    wa, wb = ora.batched_matmul_backward(a, b, go)
    batch = int(np.prod(np.broadcast_shapes(sa[:-2], sb[:-2]), dtype=np.int64))
    _close(ta.grad_by_value().data(), wa, sb[-1] * batch)
    _close(tb.grad_by_value().data(), wb, sa[-2] * batch)


def test_entries_equal_the_two_dimensional_product_bitwise(gpu):
    T = gpu.Tensor
    rng = np.random.default_rng(3)
    a, b = rng.standard_normal((3, 1, 70, 130)).astype(np.float32), rng.standard_normal((2, 130, 45)).astype(np.float32)
    y = T.from_slice(a, list(a.shape)).matmul(T.from_slice(b, list(b.shape))).data()
    assert y.shape == (3, 2, 70, 45)
    for i in range(3):
        for j in range(2):
            one = T.from_slice(a[i, 0], [70, 130]).matmul(T.from_slice(b[j], [130, 45])).data()
            assert_bit_equal(y[i, j], one, f"entry {i},{j}")


def test_reference_unit_test_values(gpu):
    """mod.rs test_simple_batched_gradient."""
    T = gpu.Tensor
    left = T.from_slice(np.arange(1, 9, dtype=np.float32), [2, 2, 2]).with_requires_grad()
    right = T.from_slice(np.arange(1, 9, dtype=np.float32) * 0.5, [2, 2, 2]).with_requires_grad()
    y = left.matmul(right)
    assert_bit_equal(y.data(), np.array([[[3.5, 5.0], [7.5, 11.0]], [[33.5, 39.0], [45.5, 53.0]]], np.float32))
    y.backward(T.ones([2, 2, 2]))
    assert_bit_equal(left.grad_by_value().data(), np.array([[[1.5, 3.5], [1.5, 3.5]], [[5.5, 7.5], [5.5, 7.5]]], np.float32))
    assert_bit_equal(right.grad_by_value().data(), np.array([[[4.0, 4.0], [6.0, 6.0]], [[12.0, 12.0], [14.0, 14.0]]], np.float32))


def test_tf32_mode_small_entries_take_the_fp32_launch(gpu, ora):
    """TF32 mode, entries of at most 512^3 multiply-adds at a fixed stride: one FP32 launch over the batch instead
    of a tensor-core launch per entry, so the result is the FP32 mode's, bit for bit."""
    T = gpu.Tensor
    rng = np.random.default_rng(6)
    a, b = rng.standard_normal((8, 96, 160)).astype(np.float32), rng.standard_normal((8, 160, 72)).astype(np.float32)
    gpu.set_matmul_precision(gpu.FP32)
    want = T.from_slice(a, list(a.shape)).matmul(T.from_slice(b, list(b.shape))).data()
    gpu.set_matmul_precision(gpu.TF32)
    got = T.from_slice(a, list(a.shape)).matmul(T.from_slice(b, list(b.shape))).data()
    assert_bit_equal(got, want, "TF32 mode, small entries")
    assert_bit_equal(got[3], ora.matmul(a[3], b[3]), "an entry against the oracle")


def test_tf32_mode_entries(gpu):
    """TF32 mode, entries too large for the shared FP32 launch: each is the tensor-core product of operands rounded to
    TF32; checked against float64 of the rounded operands (the bound the 2-D TF32 tests use: FP32 accumulation only)."""
    T = gpu.Tensor
    rng = np.random.default_rng(4)
    a = (rng.standard_normal((4, 256, 8192)) / 8).astype(np.float32)      # 256 x 128 x 8192 = 2^28 multiply-adds per entry
    b = (rng.standard_normal((8192, 128)) / 8).astype(np.float32)

    def rna(x):     # round to nearest, ties away, to 10 mantissa bits: cvt.rna.tf32.f32
        u = x.view(np.uint32).astype(np.uint64) + 0x1000
        return (u & 0xFFFFE000).astype(np.uint32).view(np.float32)

    gpu.set_matmul_precision(gpu.TF32)
    ta, tb = T.from_slice(a, list(a.shape)).with_requires_grad(), T.from_slice(b, list(b.shape)).with_requires_grad()
    y = ta.matmul(tb)
    want = np.matmul(rna(a).astype(np.float64), rna(b).astype(np.float64))
    np.testing.assert_allclose(y.data(), want, rtol=0, atol=2e-4)
    y.sum().backward()
    ones = np.ones((4, 256, 128))
    np.testing.assert_allclose(ta.grad_by_value().data(), np.matmul(ones, rna(b).astype(np.float64).T), rtol=0, atol=2e-4)
    np.testing.assert_allclose(tb.grad_by_value().data(), np.matmul(np.swapaxes(rna(a).astype(np.float64), -1, -2), ones).sum(0),
                               rtol=0, atol=1e-3)


def test_errors(gpu):
    T = gpu.Tensor
    E = gpu.TrainStationError
    with pytest.raises(E, match="Inner dimensions must match for batched matmul: 4 vs 3"):
        T.ones([2, 3, 4]).matmul(T.ones([2, 3, 4]))
    with pytest.raises(E, match="Cannot broadcast dimensions 2 and 3"):
        T.ones([2, 3, 4]).matmul(T.ones([3, 4, 2]))
    with pytest.raises(E, match="Batched matmul requires at least 2D tensors"):
        T.ones([2, 3, 4]).matmul(T.ones([4]))
