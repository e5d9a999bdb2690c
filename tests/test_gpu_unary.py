"""GPU: the unary / scalar elementwise ops and softmax, raw launchers and engine ops, against the CPU oracle
and the reference's LibTorch procedures (tests/golden/torch_unary.npz).

Bars.  One-rounded-operation kernels (sqrt, leaky_relu, the scalar ops, pow with exponent 2 or 0.5 and every
backward formula given the same saved tensor) must match the oracle bit for bit.  exp, log, tanh, sigmoid and
general pow call CUDA's full-precision expf / logf / tanhf / powf where the reference calls the host libm:
those are compared in units in the last place, with the bound written beside each (CUDA documents 2, 1, 2 and
4 ulp for them, glibc stays within 1)."""
import os

import numpy as np
import pytest

from conftest import assert_bit_equal
from devbuf import DevBuf

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "torch_unary.npz"))
SIZES = [0, 1, 3, 4, 5, 31, 33, 1024, 4099, (1 << 20) + 3]
EXACT = {"sqrt", "leaky_relu", "add_scalar", "sub_scalar", "mul_scalar", "div_scalar"}
ULPS = {"exp": 3, "log": 2, "tanh": 3, "sigmoid": 4, "pow_scalar": 9}
PARAM = {"leaky_relu": 0.01, "add_scalar": 1.25, "sub_scalar": -0.3, "mul_scalar": -2.5, "div_scalar": 3.0, "pow_scalar": 3.0}


def assert_ulps(got, want, ulps, what=""):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, what
    both_nan = np.isnan(got) & np.isnan(want)
    same_inf = np.isinf(want) & (got == want)
    fin = ~(both_nan | same_inf)
    if not fin.any():
        return
    d = np.abs(got[fin].astype(np.float64) - want[fin].astype(np.float64))
    spacing = np.maximum(np.spacing(np.abs(want[fin])).astype(np.float64), 1.5e-45)
    worst = float(np.max(d / spacing))
    assert worst <= ulps, f"{what}: {worst:.2f} ulp from the oracle (allowed {ulps})"


def inputs_for(name, n, seed):
    rng = np.random.default_rng(seed)
    if name in ("log", "sqrt"):
        return (rng.random(n, dtype=np.float32) * 20 + 1e-3).astype(np.float32)
    if name == "pow_scalar":
        return (rng.random(n, dtype=np.float32) * 4 + 0.05).astype(np.float32)
    if name == "exp":
        return (rng.standard_normal(n, dtype=np.float32) * 6).astype(np.float32)
    return (rng.standard_normal(n, dtype=np.float32) * 3).astype(np.float32)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("name", sorted(EXACT | set(ULPS)))
def test_raw_forward_and_backward(gpu, ora, name, n):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    code, p = ora.UNARY[name], PARAM.get(name, 0.0)
    x = inputs_for(name, n, n + 7)
    dx, dy = DevBuf(gpu, x), DevBuf(gpu, n=n)
    chk(lib.launch_unary_kernel(code, dx.ptr, dy.ptr, n, p, None), name)
    want = ora.unary(name, x, p)
    if name in EXACT:
        assert_bit_equal(dy.get(), want, f"{name} n={n}")
    else:
        assert_ulps(dy.get(), want, ULPS[name], f"{name} n={n}")
    # backward with the saved tensor the reference keeps, taken from the oracle so that both sides see the same bits
    saved = {"out": want, "in": x, None: None}[ora.UNARY_SAVES[name]]
    go = np.random.default_rng(n + 11).standard_normal(n, dtype=np.float32)
    ds = DevBuf(gpu, saved) if saved is not None else None
    dg, di = DevBuf(gpu, go), DevBuf(gpu, n=n)
    chk(lib.launch_unary_backward_kernel(code, ds.ptr if ds else None, dg.ptr, di.ptr, n, p, None), name + " backward")
    want_g = ora.unary_backward(name, saved, go, p)
    if name == "pow_scalar":
        assert_ulps(di.get(), want_g, ULPS[name], f"{name} backward n={n}")
    else:
        assert_bit_equal(di.get(), want_g, f"{name} backward n={n}")


@pytest.mark.parametrize("e", [2.0, 0.5, 0.0, 1.0, -1.0])
def test_pow_scalar_special_exponents(gpu, ora, e):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    x = inputs_for("pow_scalar", 1003, 3)
    dx, dy, dg, di = DevBuf(gpu, x), DevBuf(gpu, n=x.size), DevBuf(gpu, np.ones_like(x)), DevBuf(gpu, n=x.size)
    chk(lib.launch_unary_kernel(ora.UNARY["pow_scalar"], dx.ptr, dy.ptr, x.size, e, None))
    chk(lib.launch_unary_backward_kernel(ora.UNARY["pow_scalar"], dx.ptr, dg.ptr, di.ptr, x.size, e, None))
    want, want_g = ora.unary("pow_scalar", x, e), ora.unary_backward("pow_scalar", x, np.ones_like(x), e)
    if e in (2.0, 0.5):     # x*x and sqrt: pow.rs:139-156
        assert_bit_equal(dy.get(), want)
    else:
        assert_ulps(dy.get(), want, ULPS["pow_scalar"])
    if e == 0.0:            # grad_fn/ops/pow.rs:17-19
        assert_bit_equal(di.get(), np.zeros_like(x))
    else:
        assert_ulps(di.get(), want_g, ULPS["pow_scalar"])


def test_special_values(gpu, ora):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    x = np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 1e-42, -1e-42, 88.8, -104.0, 3.4e38, -3.4e38, 1.0], np.float32)
    for name in ("exp", "tanh", "sigmoid", "leaky_relu", "sqrt", "mul_scalar", "add_scalar"):
        dx, dy = DevBuf(gpu, x), DevBuf(gpu, n=x.size)
        p = PARAM.get(name, 0.0)
        chk(lib.launch_unary_kernel(ora.UNARY[name], dx.ptr, dy.ptr, x.size, p, None), name)
        got, want = dy.get(), ora.unary(name, x, p)
        assert np.array_equal(np.isnan(got), np.isnan(want)), name
        if name in EXACT:
            assert_bit_equal(got, want, name)
        else:
            assert_ulps(got, want, ULPS[name], name)


@pytest.mark.parametrize("offset", [1, 2, 3])
def test_unaligned_pointers(gpu, ora, offset):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    x = inputs_for("sqrt", 1001, 1)
    dx, dy = DevBuf(gpu, x, offset=offset), DevBuf(gpu, n=x.size, offset=offset)
    chk(lib.launch_unary_kernel(ora.UNARY["sqrt"], dx.ptr, dy.ptr, x.size, 0.0, None))
    assert_bit_equal(dy.get(), ora.unary("sqrt", x))


def test_log_domain_error_is_reported(gpu, ora):
    """log.rs:68-107 panics on x <= 0.  Raw launcher: reported by the next ts_sync_stream, once.  Engine: at the call."""
    lib = gpu._ffi.lib()
    x = np.array([1.0, 2.0, 0.0, 4.0], np.float32)
    dx, dy = DevBuf(gpu, x), DevBuf(gpu, n=4)
    assert lib.launch_unary_kernel(ora.UNARY["log"], dx.ptr, dy.ptr, 4, 0.0, None) is True
    assert lib.ts_sync_stream(None) is False
    assert "log domain error" in gpu._ffi.last_error()
    assert lib.ts_sync_stream(None) is True          # the word is cleared once read
    got = dy.get()
    assert got[2] == -np.inf and got[0] == 0.0        # the IEEE results are still stored
    T = gpu.Tensor
    with pytest.raises(gpu.TrainStationError, match="log domain error"):
        T.from_slice([1.0, -1.0], [2]).log()
    with pytest.raises(gpu.TrainStationError, match="log domain error"):
        T.from_slice([float("nan")], [1]).log()
    assert T.from_slice([1.0, 2.0], [2]).log().data()[0] == 0.0     # and the context is still usable
    lib.ts_set_domain_checks(0)
    try:
        y = T.from_slice([1.0, -1.0], [2]).log()      # deferred: no failure at the call
        with pytest.raises(gpu.TrainStationError, match="log domain error"):
            gpu.synchronize()
        assert np.isnan(y.data()[1])
    finally:
        lib.ts_set_domain_checks(1)
    assert T.new([0]).log().size() == 0


def test_division_by_zero_scalar_is_refused(gpu):
    with pytest.raises(gpu.TrainStationError, match="Division by zero"):     # div.rs:705-709 should_panic
        gpu.Tensor.ones([2, 3]).div_scalar(0.0)
    d = DevBuf(gpu, n=8)
    assert gpu._ffi.lib().launch_unary_kernel(9, d.ptr, d.ptr, 8, 0.0, None) is False
    assert gpu._ffi.lib().launch_unary_kernel(77, d.ptr, d.ptr, 8, 0.0, None) is False
    assert "unknown op" in gpu._ffi.last_error()


# ----------------------------------------------------------------------------- softmax
SOFTMAX_SHAPES = [((4, 10), 1), ((1, 1), 1), ((7,), 0), ((3, 50, 4), 1), ((5, 7, 33), 0), ((2, 3, 4), 2), ((64, 32), 1),
                  ((300, 1000), 1), ((9, 33), 1), ((2, 70000), 1), ((40, 2000), 1), ((3, 8192), 1), ((3, 8193), 1), ((1000, 32), 1),
                  ((515, 10), 1), ((3, 300, 40), 1), ((2, 256, 100), 1), ((2, 257, 33), 1)]


@pytest.mark.parametrize("shape,dim", SOFTMAX_SHAPES)
def test_softmax_raw_forward_and_backward(gpu, ora, shape, dim):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    rng = np.random.default_rng(sum(shape) + dim)
    x = (rng.standard_normal(shape, dtype=np.float32) * 4).astype(np.float32)
    outer = int(np.prod(shape[:dim], dtype=np.int64)); reduce = shape[dim]; inner = int(np.prod(shape[dim + 1:], dtype=np.int64))
    dx, dy = DevBuf(gpu, x), DevBuf(gpu, n=x.size)
    chk(lib.launch_softmax_kernel(dx.ptr, dy.ptr, outer, reduce, inner, None))
    y, want = dy.get().reshape(shape), ora.softmax(x, dim)
    # against the exact value: exp within 3 ulp, a tree sum, one division and one multiply
    # (x - max is one f32 subtraction in the reference too: its rounding, up to |x - max| * 6e-8, is part of the definition)
    e64 = np.exp((x - x.max(axis=dim, keepdims=True)).astype(np.float64))
    np.testing.assert_allclose(y, e64 / e64.sum(axis=dim, keepdims=True), rtol=1e-6, atol=1e-37)
    # against the oracle, whose sequential f32 sum of `reduce` terms is itself off by up to reduce/2 ulp
    np.testing.assert_allclose(y, want, rtol=1e-6 + reduce * 6e-8, atol=1e-37)
    np.testing.assert_allclose(y.sum(axis=dim, dtype=np.float64), 1.0, atol=2e-6)
    go = rng.standard_normal(shape, dtype=np.float32)
    dw, dg, di = DevBuf(gpu, want), DevBuf(gpu, go), DevBuf(gpu, n=x.size)
    chk(lib.launch_softmax_backward_kernel(dw.ptr, dg.ptr, di.ptr, outer, reduce, inner, None))
    got_g, want_g = di.get().reshape(shape), ora.softmax_backward(want, go, dim)
    if inner == 1 and reduce <= 32:
        # short rows: one thread per row, the reference's order, no transcendental in the backward
        assert_bit_equal(got_g, want_g, "short-row backward follows the reference's order")
    else:
        ref64 = want.astype(np.float64) * (go - (go.astype(np.float64) * want).sum(axis=dim, keepdims=True))
        assert np.max(np.abs(got_g - ref64)) <= 4e-7 * max(1.0, float(np.max(np.abs(go))))
        assert np.max(np.abs(got_g - want_g)) <= (4e-7 + reduce * 6e-8) * max(1.0, float(np.max(np.abs(go))))


def test_softmax_errors(gpu):
    T = gpu.Tensor
    with pytest.raises(gpu.TrainStationError, match="out of bounds"):        # softmax.rs:112-117
        T.ones([2, 3]).softmax(2)
    with pytest.raises(gpu.TrainStationError, match="empty dimension"):      # softmax.rs:121
        T.new([2, 0]).softmax(1)
    assert T.new([0, 3]).softmax(1).size() == 0


# ----------------------------------------------------------------------------- engine ops against the LibTorch procedures
def _split(case):
    if case.startswith("pow_scalar_"):
        return "pow_scalar", float(case.split("_")[-1])
    name = case.rstrip("0123456789")
    return name, (0.1 if name == "leaky_relu" else None)


@pytest.mark.parametrize("case", [str(c) for c in GOLDEN["cases"]])
def test_engine_matches_libtorch_procedure(gpu, case):
    name, p = _split(case)
    rtol = 1e-6 if name in ("exp", "log", "sqrt") else 1e-5          # the reference's validator settings
    T = gpu.Tensor
    call = (lambda t: getattr(t, name)()) if p is None else (lambda t: getattr(t, name)(p))
    x = GOLDEN[case + "_x"]
    y = call(T.from_slice(x, list(x.shape)))
    assert y.shape().dims == list(x.shape)
    np.testing.assert_allclose(y.data(), GOLDEN[case + "_y"], rtol=rtol, atol=1e-8)
    gx = GOLDEN[case + "_gx"]
    t = T.from_slice(gx, list(gx.shape)).with_requires_grad()
    call(t).backward(None)
    g = t.grad_by_value()
    assert g is not None and g.shape().dims == list(gx.shape)
    np.testing.assert_allclose(g.data(), GOLDEN[case + "_grad"], rtol=rtol, atol=1.2e-7 if name == "tanh" else 1e-8)


def test_engine_exp_chain_and_softmax_procedures(gpu):
    T = gpu.Tensor
    for i in range(int(GOLDEN["exp_chain_count"])):
        xh = GOLDEN[f"exp_chain{i}_x"]
        x = T.from_slice(xh, list(xh.shape)).with_requires_grad()
        ex = x.exp()
        ex.mul_tensor(x).add_tensor(ex).backward(None)       # libtorch-validation .../ops/exp.rs:91-105
        np.testing.assert_allclose(x.grad_by_value().data(), GOLDEN[f"exp_chain{i}_grad"], rtol=2e-6, atol=1e-8)
        gpu.clear_gradients()
    for i in range(int(GOLDEN["softmax_count"])):
        dim = int(GOLDEN[f"softmax{i}_dim"])
        xh = GOLDEN[f"softmax{i}_x"]
        np.testing.assert_allclose(T.from_slice(xh, list(xh.shape)).softmax(dim).data(), GOLDEN[f"softmax{i}_y"], rtol=1e-5, atol=1e-8)
        gh = GOLDEN[f"softmax{i}_gx"]
        x = T.from_slice(gh, list(gh.shape)).with_requires_grad()
        x.softmax(dim).sum().backward(None)                  # .../ops/softmax.rs:27-45
        assert np.max(np.abs(x.grad_by_value().data())) < 2.5e-7
        gpu.clear_gradients()
        x = T.from_slice(gh, list(gh.shape)).with_requires_grad()
        up = GOLDEN[f"softmax{i}_up"]
        x.softmax(dim).mul_tensor(T.from_slice(up, list(up.shape))).sum().backward(None)
        np.testing.assert_allclose(x.grad_by_value().data(), GOLDEN[f"softmax{i}_grad_up"], rtol=1e-5, atol=2e-7)
        gpu.clear_gradients()


def test_operator_forms(gpu):
    """tensor/core/operators.rs:418-705: Tensor (op) f32, f32 (op) Tensor, negation."""
    T = gpu.Tensor
    a = T.from_slice([1.0, 2.0, 3.0, 4.0], [2, 2])
    assert (a + 5.0).data().reshape(-1).tolist() == [6, 7, 8, 9]
    assert (5.0 + a).data().reshape(-1).tolist() == [6, 7, 8, 9]
    assert (a - 2.0).data().reshape(-1).tolist() == [-1, 0, 1, 2]
    assert (10.0 - a).data().reshape(-1).tolist() == [9, 8, 7, 6]
    assert (a * 3.0).data().reshape(-1).tolist() == [3, 6, 9, 12]
    assert (3.0 * a).data().reshape(-1).tolist() == [3, 6, 9, 12]
    assert (a / 2.0).data().reshape(-1).tolist() == [0.5, 1, 1.5, 2]
    np.testing.assert_allclose((12.0 / a).data().reshape(-1), [12, 6, 4, 3], rtol=1e-6)
    assert (-a).data().reshape(-1).tolist() == [-1, -2, -3, -4]
    assert (a + a).data().reshape(-1).tolist() == [2, 4, 6, 8]
    # gradients: x*3 + 1 -> 3; 2/x -> -2/x^2; the f32 - &Tensor form detaches (it works on a clone in the reference)
    x = T.from_slice([1.0, 2.0, 4.0], [3]).with_requires_grad()
    (x * 3.0 + 1.0).sum().backward()
    assert x.grad_by_value().data().tolist() == [3, 3, 3]
    gpu.clear_gradients()
    x = T.from_slice([1.0, 2.0, 4.0], [3]).with_requires_grad()
    (2.0 / x).sum().backward()
    np.testing.assert_allclose(x.grad_by_value().data(), [-2.0, -0.5, -0.125], rtol=1e-6)
    gpu.clear_gradients()
    x = T.from_slice([1.0, 2.0, 4.0], [3]).with_requires_grad()
    r = 1.0 - x
    assert not r.requires_grad() and r.data().tolist() == [0, -1, -3]
    (-x).sum().backward()
    assert x.grad_by_value().data().tolist() == [-1, -1, -1]


def test_example_network_with_tanh_sigmoid_softmax(gpu, ora):
    """A small classifier in the style of the reference's examples, every op on the device, against the oracle tape."""
    from oracle_graph import OracleGraph
    rng = np.random.default_rng(21)
    B, I, H, O = 64, 20, 48, 10
    xh = rng.standard_normal((B, I), dtype=np.float32)
    w1h = (rng.standard_normal((I, H), dtype=np.float32) * 0.3).astype(np.float32)
    w2h = (rng.standard_normal((H, O), dtype=np.float32) * 0.3).astype(np.float32)
    b1h, b2h = np.zeros(H, np.float32) + 0.1, np.zeros(O, np.float32)
    th = np.eye(O, dtype=np.float32)[rng.integers(0, O, B)]
    T = gpu.Tensor
    w1, b1, w2, b2 = (T.from_slice(a, list(a.shape)).with_requires_grad() for a in (w1h, b1h, w2h, b2h))
    x, t = T.from_slice(xh, [B, I]), T.from_slice(th, [B, O])
    h = x.matmul(w1).add_tensor(b1).tanh().mul_scalar(1.5).sigmoid()
    p = h.matmul(w2).add_tensor(b2).softmax(1)
    loss = p.add_scalar(1e-6).log().mul_tensor(t).sum().mul_scalar(-1.0 / B)
    loss.backward()
    G = OracleGraph(ora)
    ow1, ob1, ow2, ob2 = (G.leaf(a, a.shape, True) for a in (w1h, b1h, w2h, b2h))
    ox, ot = G.leaf(xh, xh.shape), G.leaf(th, th.shape)
    oh = G.op("sigmoid", G.op("mul_scalar", G.op("tanh", G.op("add_tensor", G.op("matmul", ox, ow1), ob1)), 1.5))
    op_ = G.op("softmax", G.op("add_tensor", G.op("matmul", oh, ow2), ob2), 1)
    ol = G.op("mul_scalar", G.op("sum", G.op("mul_tensor", G.op("log", G.op("add_scalar", op_, 1e-6)), ot)), -1.0 / B)
    G.backward(ol)
    np.testing.assert_allclose(loss.value(), float(ol.data.reshape(-1)[0]), rtol=2e-6)
    np.testing.assert_allclose(p.data(), op_.data, rtol=3e-6, atol=1e-9)
    for dev, orc, nm in ((w1, ow1, "w1"), (b1, ob1, "b1"), (w2, ow2, "w2"), (b2, ob2, "b2")):
        g, want = dev.grad_by_value().data(), G.grad(orc)
        scale = float(np.max(np.abs(want)))
        assert np.max(np.abs(g - want)) <= 2e-5 * scale, nm      # north-star FP32 bar: rel 1e-5 / abs 1e-6 per element, here on the tensor's scale


# ----------------------------------------------------------------------------- full-size properties (inputs larger than L2)
def test_large_inputs_properties(gpu, ora):
    lib, chk = gpu._ffi.lib(), gpu._ffi.check
    n = (1 << 26) + 5                                    # 268 MB per array
    rng = np.random.default_rng(2)
    x = (rng.random(n, dtype=np.float32) * 9 + 0.5).astype(np.float32)
    dx, dy, dz = DevBuf(gpu, x), DevBuf(gpu, n=n), DevBuf(gpu, n=n)
    # exp(log(x)) = x to a few ulp of x * |log x| conditioning; sqrt(x)^2 = x to 1 ulp-ish
    chk(lib.launch_unary_kernel(ora.UNARY["log"], dx.ptr, dy.ptr, n, 0.0, None))
    chk(lib.launch_unary_kernel(ora.UNARY["exp"], dy.ptr, dz.ptr, n, 0.0, None))
    np.testing.assert_allclose(dz.get(), x, rtol=1e-6)
    chk(lib.launch_unary_kernel(ora.UNARY["sqrt"], dx.ptr, dy.ptr, n, 0.0, None))
    sl = slice(n - 100003, n)
    assert_bit_equal(dy.get()[sl], ora.unary("sqrt", x[sl]))                     # a slice against the oracle, tail included
    chk(lib.launch_unary_kernel(ora.UNARY["pow_scalar"], dy.ptr, dz.ptr, n, 2.0, None))
    np.testing.assert_allclose(dz.get(), x, rtol=2.5e-7)
    # tanh is odd, sigmoid(x) + sigmoid(-x) = 1
    chk(lib.launch_unary_kernel(ora.UNARY["mul_scalar"], dx.ptr, dy.ptr, n, -1.0, None))
    chk(lib.launch_unary_kernel(ora.UNARY["sigmoid"], dx.ptr, dz.ptr, n, 0.0, None))
    s_pos = dz.get()
    chk(lib.launch_unary_kernel(ora.UNARY["sigmoid"], dy.ptr, dz.ptr, n, 0.0, None))
    np.testing.assert_allclose(s_pos.astype(np.float64) + dz.get(), 1.0, atol=2e-7)
    assert lib.ts_sync_stream(None) is True
    # softmax over [65536, 1000] (262 MB): rows sum to one, a slice against the oracle
    rows, cols = 65536, 1000
    xs = x[: rows * cols].reshape(rows, cols)
    chk(lib.launch_softmax_kernel(dx.ptr, dy.ptr, rows, cols, 1, None))
    y = dy.get()[: rows * cols].reshape(rows, cols)
    np.testing.assert_allclose(y.sum(axis=1, dtype=np.float64), 1.0, atol=2e-6)
    np.testing.assert_allclose(y[-50:], ora.softmax(xs[-50:], 1), rtol=1e-6 + cols * 6e-8)   # the oracle's sum is sequential
