"""CPU: the oracle restatement against (1) the reference's literal known answers and
(2) the reference's LibTorch differential procedures replayed with PyTorch."""
import json
import os

import numpy as np
import pytest

from oracle_graph import run_case_oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
KNOWN = json.load(open(os.path.join(GOLDEN, "reference_known_answers.json")))
KNOWN["cases"] = KNOWN["cases"] + json.load(open(os.path.join(GOLDEN, "reference_known_answers_broadcast.json")))["cases"]


@pytest.mark.parametrize("case", KNOWN["cases"], ids=[c["name"] for c in KNOWN["cases"]])
def test_reference_known_answers(ora, case):
    values, grads = run_case_oracle(ora, case)
    tol = case["tol"]
    for name, exp in case.get("expect", {}).items():
        got = values[name]
        assert list(got.shape) == exp["dims"], (name, got.shape)
        np.testing.assert_allclose(got.reshape(-1), np.array(exp["data"], np.float32), rtol=0, atol=tol)
    for name, exp in case.get("expect_grad", {}).items():
        if exp is None:
            assert grads[name] is None
            continue
        got = grads[name]
        assert got is not None, name
        assert list(got.shape) == exp["dims"]
        np.testing.assert_allclose(got.reshape(-1), np.array(exp["data"], np.float32), rtol=0, atol=tol)


@pytest.mark.parametrize("case", KNOWN["kernel_formula_cases"]["cases"], ids=lambda c: f"{c['m']}x{c['n']}x{c['k']}")
def test_kernel_formula_cases_are_exact(ora, case):
    m, n, k = case["m"], case["n"], case["k"]
    gen = lambda cnt, mod: np.array([(i % mod + 1) if mod else (i + 1) for i in range(cnt)], np.float32)
    a, b = gen(m * k, case["a_mod"]).reshape(m, k), gen(k * n, case["b_mod"]).reshape(k, n)
    exact = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    assert np.array_equal(ora.matmul(a, b), exact)
    assert np.array_equal(ora.matmul(a, b, naive=True), exact)


# Integer data for every block-size class of MatmulConfig::for_dimensions and for shapes whose
# blocks are narrower than the matrix (the case the reference mishandles): exact in f32.
@pytest.mark.parametrize("m,n,k", [(17, 23, 19), (32, 24, 16), (64, 48, 40), (33, 65, 70), (128, 128, 128),
                                   (130, 10, 257), (5, 300, 129), (256, 256, 256), (32, 128, 784)])
def test_blocked_driver_exact_on_integers(ora, m, n, k):
    rng = np.random.default_rng(m * 1000003 + n * 1009 + k)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    exact = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    assert np.array_equal(ora.matmul(a, b), exact)


def test_matmul_summation_order(ora):
    """Body columns are an FMA chain over ascending p; the n % 8 tail columns multiply, round, then add."""
    rng = np.random.default_rng(7)
    m, n, k = 3, 10, 300
    a, b = rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((k, n), dtype=np.float32)
    got = ora.matmul(a, b)
    for i in range(m):
        for j in range(n):
            acc = np.float32(0)
            for p in range(k):
                if j < 8:  # fused: exact product added, one rounding
                    acc = np.float32(np.float64(a[i, p]) * np.float64(b[p, j]) + np.float64(acc))
                else:
                    acc = np.float32(acc + np.float32(a[i, p] * b[p, j]))
            assert got[i, j] == acc, (i, j)


def _allclose_ref(got, want, rtol, atol):
    """The reference validator's rule (libtorch-validation/src/validation/core.rs:138-141):
    an element passes if diff <= rtol*|torch| OR diff <= atol."""
    d = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    return bool(np.all((d <= rtol * np.abs(want)) | (d <= atol)))


def test_torch_differential_matmul(ora):
    z = np.load(os.path.join(GOLDEN, "torch_differential.npz"))
    for i in range(int(z["matmul_count"])):
        l, r = z[f"matmul{i}_left"], z[f"matmul{i}_right"]
        out = ora.matmul(l, r)
        assert _allclose_ref(out, z[f"matmul{i}_out"], 1e-5, 1e-8), i
        go = np.ones_like(out)
        assert _allclose_ref(ora.matmul(go, np.ascontiguousarray(r.T)), z[f"matmul{i}_grad_left"], 1e-5, 1e-8), i
        assert _allclose_ref(ora.matmul(np.ascontiguousarray(l.T), go), z[f"matmul{i}_grad_right"], 1e-5, 1e-8), i


def test_torch_differential_linear_and_relu(ora):
    z = np.load(os.path.join(GOLDEN, "torch_differential.npz"))
    for i in range(int(z["linear_count"])):
        x, w, b = z[f"linear{i}_x"], z[f"linear{i}_w"], z[f"linear{i}_b"]
        st = ora.MlpState([w], [b])
        r = ora.mlp_step(st, x, loss_kind=ora.LOSS_SUM, do_adam=False, want_gx=True, want_y=True)
        assert _allclose_ref(r["y"], z[f"linear{i}_out"], 1e-5, 1e-8)
        assert _allclose_ref(st.gw[0], z[f"linear{i}_grad_w"], 1e-5, 1e-8)
        assert _allclose_ref(st.gb[0], z[f"linear{i}_grad_b"], 1e-5, 1e-8)
        assert np.all(st.gb[0] == x.shape[0])  # bias gradient = batch size, broadcasting_gradients.rs:272-350
        assert _allclose_ref(r["gx"], z[f"linear{i}_grad_x"], 1e-5, 1e-8)
    x = z["relu_x"]
    assert np.array_equal(ora.relu(x), z["relu_out"])
    assert np.array_equal(ora.relu_bwd(x, np.ones_like(x)), z["relu_grad"])


def test_torch_differential_adam(ora):
    z = np.load(os.path.join(GOLDEN, "torch_differential.npz"))
    for i in range(int(z["adam_count"])):
        steps, lr, b1, b2, eps, wd = z[f"adam{i}_cfg"]
        p = z[f"adam{i}_init"].copy()
        m, v = np.zeros_like(p), np.zeros_like(p)
        g = np.full_like(p, 2.0)  # d/dp sum(2p+1)
        for t in range(1, int(steps) + 1):
            ora.adam_update(p.reshape(-1), g.reshape(-1), m.reshape(-1), v.reshape(-1), t, lr, b1, b2, eps, wd)
        assert _allclose_ref(p, z[f"adam{i}_final"], 1e-4, 1e-4), i  # the reference's Adam tolerance, adam.rs:47-51


def test_adam_matches_f64_textbook(ora):
    rng = np.random.default_rng(3)
    n = 1003
    p = rng.standard_normal(n, dtype=np.float32)
    p64, m64, v64 = p.astype(np.float64), np.zeros(n), np.zeros(n)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    for t in range(1, 6):
        g = rng.standard_normal(n, dtype=np.float32)
        ora.adam_update(p, g, m, v, t)
        p64, m64, v64 = ora.adam_update_f64(p64, g, m64, v64, t)
    np.testing.assert_allclose(p, p64, rtol=1e-5, atol=1e-6)


def test_adam_tail_association(ora):
    """Elements past size/8*8 use ((1-beta2)*g)*g, the others (1-beta2)*(g*g) (adam/mod.rs:761-772)."""
    g = np.array([1.1, -2.3, 0.7, 3.9, -0.01, 5.5, 1e-3, 7.7, 0.3, -0.9, 2.2], np.float32)
    p, m, v = np.zeros(11, np.float32), np.zeros(11, np.float32), np.zeros(11, np.float32)
    ora.adam_update(p, g, m, v, 1)
    c2 = np.float32(1.0) - np.float32(0.999)
    body = (c2 * (g * g)).astype(np.float32)
    tail = ((c2 * g).astype(np.float32) * g).astype(np.float32)
    assert np.array_equal(v[:8], body[:8]) and np.array_equal(v[8:], tail[8:])


def test_reductions_follow_reference_order(ora):
    rng = np.random.default_rng(5)
    x = rng.standard_normal(1003, dtype=np.float32)
    acc = np.float32(0)
    for i in range(0, 1000, 4):
        acc = np.float32(acc + np.float32(np.float32(np.float32(x[i] + x[i + 1]) + x[i + 2]) + x[i + 3]))
    for i in range(1000, 1003):
        acc = np.float32(acc + x[i])
    assert ora.total(x) == acc
    assert ora.mean(x) == np.float32(acc / np.float32(1003))
    assert ora.total(np.zeros(0, np.float32)) == 0 and ora.mean(np.zeros(0, np.float32)) == 0
    g = rng.standard_normal((37, 5), dtype=np.float32)
    col = np.zeros(5, np.float32)
    for i in range(37):
        col = (col + g[i]).astype(np.float32)
    assert np.array_equal(ora.colsum(g), col)


def test_relu_special_values(ora):
    x = np.array([np.nan, -0.0, 0.0, -np.inf, np.inf, 1e-45, -1e-45, 3.0, np.nan, -2.0, 5.0], np.float32)
    y = ora.relu(x)  # 8-wide body then scalar tail: both map NaN -> 0 and -0 -> +0
    assert not np.isnan(y).any()
    assert not np.signbit(y).any()
    assert y[4] == np.inf and y[5] == np.float32(1e-45) and y[7] == 3.0 and y[10] == 5.0


def test_mlp_step_matches_f64_twin(ora):
    rng = np.random.default_rng(11)
    dims, batch = [20, 33, 17, 6], 29
    ws = [(rng.standard_normal((dims[i], dims[i + 1])) / np.sqrt(dims[i])).astype(np.float32) for i in range(3)]
    bs = [rng.standard_normal(dims[i + 1]).astype(np.float32) * 0.1 for i in range(3)]
    x = rng.standard_normal((batch, dims[0]), dtype=np.float32)
    t = rng.standard_normal((batch, dims[-1]), dtype=np.float32)
    for kind, relu_last in ((ora.LOSS_MSE, False), (ora.LOSS_SUM, True), (ora.LOSS_MEAN, True)):
        st = ora.MlpState(ws, bs)
        r = ora.mlp_step(st, x, t, loss_kind=kind, relu_last=relu_last, do_adam=False, want_gx=True)
        f = ora.mlp_step_f64(ws, bs, x, t, loss_kind=kind, relu_last=relu_last)
        np.testing.assert_allclose(r["loss"], f["loss"], rtol=1e-5)
        for l in range(3):
            np.testing.assert_allclose(st.gw[l], f["gw"][l], rtol=1e-4, atol=1e-6)
            np.testing.assert_allclose(st.gb[l], f["gb"][l], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(r["gx"], f["gx"], rtol=1e-4, atol=1e-6)
        # the variant that also performs the reference's operand deep copies computes the same bits
        st2 = ora.MlpState(ws, bs)
        r2 = ora.mlp_step(st2, x, t, loss_kind=kind, relu_last=relu_last, do_adam=False, as_written=True)
        assert r2["loss"] == r["loss"] and all(np.array_equal(a, b) for a, b in zip(st.gw, st2.gw))
