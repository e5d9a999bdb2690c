"""GPU: permute / transpose / reshape family.  Pure data movement, so every comparison is bit for bit against the
numpy restatement in the oracle; gradients go through the inverse permutation (grad_fn/transforms/*.rs)."""
import ctypes as C
import itertools

import numpy as np
import pytest

from conftest import assert_bit_equal
from devbuf import DevBuf

pytestmark = pytest.mark.gpu


def _permute_raw(gpu, x, perm):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    dx, dy = DevBuf(gpu, x), DevBuf(gpu, n=x.size)
    dims = (C.c_ulonglong * x.ndim)(*x.shape)
    p = (C.c_int * x.ndim)(*perm)
    chk(lib.launch_permute_kernel(dx.ptr, dy.ptr, dims, p, x.ndim, None), "permute")
    return dy.get().reshape([x.shape[i] for i in perm])


@pytest.mark.parametrize("shape", [(2, 3), (33, 65), (1, 7), (7, 1), (128, 256), (31, 32, 33), (2, 3, 4, 5), (1, 5, 1, 6), (3, 1, 4),
                                   (2, 2, 2, 2, 2, 3)])
def test_every_permutation_of_small_ranks(gpu, ora, shape):
    rng = np.random.default_rng(len(shape) * 100 + shape[0])
    x = rng.standard_normal(shape).astype(np.float32)
    perms = list(itertools.permutations(range(len(shape))))
    if len(perms) > 24:
        perms = [perms[i] for i in rng.choice(len(perms), 24, replace=False)]
    for perm in perms:
        assert_bit_equal(_permute_raw(gpu, x, perm), ora.permute(x, perm), f"{shape} {perm}")


def test_transpose_edges_and_errors(gpu, ora):
    lib = gpu._ffi.lib()
    x = np.arange(37 * 70, dtype=np.float32).reshape(37, 70)       # ragged tiles
    assert_bit_equal(_permute_raw(gpu, x, (1, 0)), x.T.copy())
    b = np.arange(3 * 37 * 70, dtype=np.float32).reshape(3, 37, 70)  # batched
    assert_bit_equal(_permute_raw(gpu, b, (0, 2, 1)), np.ascontiguousarray(b.transpose(0, 2, 1)))
    e = np.zeros((0, 4), np.float32)
    assert _permute_raw(gpu, e, (1, 0)).shape == (4, 0)
    d = DevBuf(gpu, n=8)
    dims = (C.c_ulonglong * 2)(2, 4)
    assert lib.launch_permute_kernel(d.ptr, d.ptr, dims, (C.c_int * 2)(0, 0), 2, None) is False
    assert "not a permutation" in gpu._ffi.last_error()
    assert lib.launch_permute_kernel(d.ptr, d.ptr, dims, (C.c_int * 2)(0, 2), 2, None) is False
    assert lib.launch_permute_kernel(None, d.ptr, dims, (C.c_int * 2)(1, 0), 2, None) is False


def test_engine_shape_ops_match_reference_behaviour(gpu):
    T = gpu.Tensor
    x = T.from_slice(np.arange(24, dtype=np.float32), [2, 3, 4])
    assert x.transpose(0, 2).shape().dims == [4, 3, 2]                      # transpose.rs:489-495
    assert x.reshape([6, -1]).shape().dims == [6, 4]                        # reshape.rs:314-320
    assert x.flatten().shape().dims == [24]
    assert T.from_slice([1.0, 2.0, 3.0], [1, 3, 1]).squeeze().shape().dims == [3]      # squeeze.rs tests
    assert T.from_slice([1.0, 2.0, 3.0], [1, 3, 1]).squeeze(0).shape().dims == [3, 1]
    assert T.from_slice([5.0], [1, 1, 1]).squeeze().shape().dims == [1]
    assert T.from_slice([1.0, 2.0, 3.0], [3]).unsqueeze(1).shape().dims == [3, 1]      # unsqueeze.rs tests
    assert T.from_slice([1.0, 2.0, 3.0, 4.0], [2, 2]).unsqueeze(2).shape().dims == [2, 2, 1]
    E = gpu.TrainStationError
    with pytest.raises(E, match="Only one dimension can be -1"):            # reshape.rs:334-338
        x.reshape([-1, -1])
    with pytest.raises(E, match="Cannot reshape"):                          # reshape.rs:341-345
        x.reshape([5, 5])
    with pytest.raises(E, match="must be positive"):                        # reshape.rs:348-351
        x.reshape([-2, 12])
    with pytest.raises(E, match="out of bounds"):                           # transpose.rs:523-527
        x.transpose(0, 3)
    with pytest.raises(E, match="at least 2 dimensions"):                   # transpose.rs:530-533
        T.ones([3]).t()
    with pytest.raises(E, match="out of bounds"):
        T.ones([3]).unsqueeze(4)
    with pytest.raises(E, match="Cannot squeeze"):
        x.squeeze(1)
    with pytest.raises(E, match="duplicate dimension"):
        x.permute([0, 0, 1])
    with pytest.raises(E, match="length equal to rank"):
        x.permute([0, 1])
    # reshape shares the storage, as the reference's view does: a write through the source shows in the view
    a = T.from_slice([1.0, 2.0, 3.0, 4.0], [2, 2])
    v = a.reshape([4])
    a.fill(7.0)
    assert v.data().tolist() == [7.0] * 4
    # gradient requirement follows the source (reshape.rs:323-331, transpose.rs:513-520); transpose(d, d) detaches
    g = T.ones([2, 2]).with_requires_grad()
    assert g.reshape([4]).requires_grad() and g.transpose(0, 1).requires_grad() and g.contiguous().requires_grad()
    assert not g.transpose(1, 1).requires_grad()


def test_gradients_through_permute_reshape_and_matmul(gpu, ora):
    """loss = sum((x^T . w).reshape(...) * c): the gradient of x comes back through the inverse permutation."""
    rng = np.random.default_rng(3)
    xh = rng.standard_normal((6, 5)).astype(np.float32)
    wh = rng.standard_normal((6, 4)).astype(np.float32)
    ch = rng.standard_normal((4, 5)).astype(np.float32)
    T = gpu.Tensor
    x, w = T.from_slice(xh, [6, 5]).with_requires_grad(), T.from_slice(wh, [6, 4]).with_requires_grad()
    y = x.t().matmul(w)                       # [5, 4]
    z = y.permute([1, 0]).reshape([2, 10]).reshape([4, 5]).mul_tensor(T.from_slice(ch, [4, 5])).sum()
    z.backward()
    from oracle_graph import OracleGraph
    G = OracleGraph(ora)
    ox, ow, oc = G.leaf(xh, xh.shape, True), G.leaf(wh, wh.shape, True), G.leaf(ch, ch.shape)
    oy = G.op("matmul", G.op("t", ox), ow)
    oz = G.op("sum", G.op("mul_tensor", G.op("reshape", G.op("reshape", G.op("permute", oy, [1, 0]), [2, 10]), [4, 5]), oc))
    G.backward(oz)
    np.testing.assert_allclose(z.value(), float(oz.data.reshape(-1)[0]), rtol=1e-6)
    assert_bit_equal(x.grad_by_value().data(), G.grad(ox), "dx")     # FP32 GEMMs in the reference's order: exact
    assert_bit_equal(w.grad_by_value().data(), G.grad(ow), "dw")


def test_large_transpose_round_trip(gpu):
    """268 MB: transpose twice is the identity; a corner block against numpy."""
    rows, cols = 8192 + 3, 8192 + 5
    rng = np.random.default_rng(11)
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    dx, dy, dz = DevBuf(gpu, x), DevBuf(gpu, n=x.size), DevBuf(gpu, n=x.size)
    p = (C.c_int * 2)(1, 0)
    chk(lib.launch_permute_kernel(dx.ptr, dy.ptr, (C.c_ulonglong * 2)(rows, cols), p, 2, None))
    chk(lib.launch_permute_kernel(dy.ptr, dz.ptr, (C.c_ulonglong * 2)(cols, rows), p, 2, None))
    y = dy.get().reshape(cols, rows)
    assert_bit_equal(y[-40:, -40:], np.ascontiguousarray(x[-40:, -40:].T))
    assert_bit_equal(dz.get().reshape(rows, cols), x)
