"""GPU: the AMSGrad branch of the fused Adam kernel and Tensor::randn, against the oracle (bit for bit) and the
reference's LibTorch procedure for AMSGrad (tests/golden/torch_amsgrad.npz)."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import assert_bit_equal
from devbuf import DevBuf

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _tables(bufs):
    return (C.c_void_p * len(bufs))(*[b.ptr for b in bufs])


@pytest.mark.parametrize("sizes", [[1], [7], [8, 9], [1000, 33, 4099], [(1 << 20) + 5, 16384, 16385, 3]])
@pytest.mark.parametrize("wd", [0.0, 0.01])
def test_amsgrad_kernel_bit_exact(gpu, ora, sizes, wd):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    rng = np.random.default_rng(len(sizes) + int(wd * 100))
    P = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    M = [np.zeros(n, np.float32) for n in sizes]
    V = [np.zeros(n, np.float32) for n in sizes]
    X = [np.zeros(n, np.float32) for n in sizes]
    dP, dM, dV, dX = ([DevBuf(gpu, a) for a in arrs] for arrs in (P, M, V, X))
    sz = (C.c_ulonglong * len(sizes))(*sizes)
    lr, b1, b2, eps = 1e-3, 0.9, 0.999, 1e-8
    for step in range(1, 6):
        scale = 3.0 if step < 3 else 0.2          # the early maximum has to be held later
        G = [(rng.standard_normal(n) * scale).astype(np.float32) for n in sizes]
        dG = [DevBuf(gpu, g) for g in G]
        bc1 = np.float32(1.0 - float(np.float32(b1)) ** float(np.float32(step)))
        bc2 = np.float32(1.0 - float(np.float32(b2)) ** float(np.float32(step)))
        f1, f2 = np.float32(1.0) / bc1, np.float32(1.0) / bc2
        chk(lib.launch_adam_amsgrad_multi_tensor_kernel(_tables(dP), _tables(dG), _tables(dM), _tables(dV), _tables(dX), sz, len(sizes),
                                                        lr, b1, b2, eps, wd, float(f1), float(f2), 1.0, None), "amsgrad")
        for i in range(len(sizes)):
            ora.adam_update_amsgrad(P[i], G[i], M[i], V[i], X[i], step, lr, b1, b2, eps, wd)
    for i in range(len(sizes)):
        assert_bit_equal(dP[i].get(), P[i], f"p[{i}]")
        assert_bit_equal(dM[i].get(), M[i], f"m[{i}]")
        assert_bit_equal(dV[i].get(), V[i], f"v[{i}]")
        assert_bit_equal(dX[i].get(), X[i], f"v_hat_max[{i}]")
    assert any(np.any(X[i] > V[i] * 2) for i in range(len(sizes))), "the running maximum was never the larger value"


def test_amsgrad_kernel_unaligned_and_null(gpu, ora):
    lib = gpu._ffi.lib()
    n = 1001
    rng = np.random.default_rng(4)
    p, g = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    m, v, x = (np.zeros(n, np.float32) for _ in range(3))
    dp, dg, dm, dv, dx = DevBuf(gpu, p, offset=1), DevBuf(gpu, g), DevBuf(gpu, m), DevBuf(gpu, v), DevBuf(gpu, x, offset=3)
    sz = (C.c_ulonglong * 1)(n)
    f1, f2 = float(np.float32(1) / np.float32(1 - float(np.float32(0.9)))), float(np.float32(1) / np.float32(1 - float(np.float32(0.999))))
    assert lib.launch_adam_amsgrad_multi_tensor_kernel(_tables([dp]), _tables([dg]), _tables([dm]), _tables([dv]), _tables([dx]), sz, 1,
                                                       1e-3, 0.9, 0.999, 1e-8, 0.0, f1, f2, 1.0, None) is True
    ora.adam_update_amsgrad(p, g, m, v, x, 1)
    assert_bit_equal(dp.get(), p)
    assert_bit_equal(dx.get(), x)
    assert lib.launch_adam_amsgrad_multi_tensor_kernel(_tables([dp]), _tables([dg]), _tables([dm]), _tables([dv]), None, sz, 1,
                                                       1e-3, 0.9, 0.999, 1e-8, 0.0, f1, f2, 1.0, None) is False


def _close_ref(got, want, rtol, atol):
    d = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    return bool(np.all((d <= rtol * np.abs(want)) | (d <= atol)))


def test_engine_amsgrad_matches_libtorch_procedure(gpu):
    """adam.rs:65-160 with amsgrad (:1355-1364, :1718-1776): loss = sum(2p + 1), written sum(p + p) as its gradient is the same 2."""
    z = np.load(os.path.join(GOLDEN, "torch_amsgrad.npz"))
    for i in range(int(z["count"])):
        steps, lr, b1, b2, eps, wd = z[f"case{i}_cfg"]
        init = z[f"case{i}_init"]
        p = gpu.Tensor.from_slice(init, init.shape).with_requires_grad()
        opt = gpu.Adam.with_config(gpu.AdamConfig(lr, b1, b2, eps, wd, True))
        opt.add_parameter(p)
        for _ in range(int(steps)):
            p.add_tensor(p).sum().backward(None)
            opt.step([p])
            opt.zero_grad([p])
        assert _close_ref(p.data(), z[f"case{i}_final"], 1e-4, 1e-4), i
        assert len(opt.state(p)) == 3


def test_engine_amsgrad_bit_exact_against_oracle(gpu, ora):
    rng = np.random.default_rng(8)
    shapes = [(37, 5), (64,), (3, 3, 3)]
    P = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    M, V, X = ([np.zeros(s, np.float32) for s in shapes] for _ in range(3))
    T = gpu.Tensor
    dev = [T.from_slice(a, list(a.shape)).with_requires_grad() for a in P]
    opt = gpu.Adam.with_config(gpu.AdamConfig(amsgrad=True, weight_decay=0.001))
    opt.add_parameters(dev)
    plain = gpu.Adam.new()
    for step in range(1, 8):
        C_ = [(rng.standard_normal(s) * (2.0 if step < 3 else 0.1)).astype(np.float32) for s in shapes]
        loss = None
        for d, c in zip(dev, C_):     # d/dp sum(p * c) = c exactly
            term = d.mul_tensor(T.from_slice(c, list(c.shape))).sum()
            loss = term if loss is None else loss.add_tensor(term)
        loss.backward()
        opt.step(dev)
        opt.zero_grad(dev)
        for i in range(len(shapes)):
            ora.adam_update_amsgrad(P[i].reshape(-1), C_[i].reshape(-1), M[i].reshape(-1), V[i].reshape(-1), X[i].reshape(-1), step,
                                    weight_decay=0.001)
    for i, d in enumerate(dev):
        m, v, x = opt.state(d)
        assert_bit_equal(d.data(), P[i], f"p{i}")
        assert_bit_equal(m.data(), M[i]); assert_bit_equal(v.data(), V[i]); assert_bit_equal(x.data(), X[i])
    # a plain optimizer has no third state
    q = T.ones([4]).with_requires_grad()
    plain.add_parameter(q)
    assert len(plain.state(q)) == 2


# ----------------------------------------------------------------------------- randn
def test_randn_reproduces_the_references_stream(gpu, ora):
    T = gpu.Tensor
    for shape, seed in (([100, 100], 42), ([100], 12345), ([2, 3], 7), ([1], 1), ([3, 1, 5], (1 << 64) - 1)):
        t = T.randn(shape, seed)
        assert t.shape().dims == shape
        assert_bit_equal(t.data(), ora.randn(shape, seed), f"seed {seed}")
    a, b = T.randn([100], 12345).data(), T.randn([100], 12345).data()     # random.rs:638-649
    assert_bit_equal(a, b)
    assert not np.array_equal(T.randn([100], 1).data(), T.randn([100], 2).data())   # :652-670
    big = T.randn([100, 100], 42).data()                                   # :699-732
    assert abs(float(big.mean())) < 0.1 and big.min() > -4.0 and big.max() < 4.0
    u1, u2 = T.randn([10], None).data(), T.randn([10], None).data()       # :673-689
    assert np.any(u1 != 0) and not np.array_equal(u1, u2)
    assert T.randn([0], 3).size() == 0                                     # :692-696


def test_randn_feeds_the_readme_step(gpu):
    """README quick start with randn inputs: the tensors take part in a step like any other."""
    T = gpu.Tensor
    x = T.randn([32, 784], 1)
    w = T.randn([784, 128], 2).with_requires_grad()
    b = T.zeros([128]).with_requires_grad()
    opt = gpu.Adam.new()
    opt.add_parameters([w, b])
    before = w.data().copy()
    loss = x.matmul(w).add_tensor(b).relu().sum()
    loss.backward()
    opt.step([w, b])
    assert np.isfinite(loss.value()) and not np.array_equal(before, w.data())
