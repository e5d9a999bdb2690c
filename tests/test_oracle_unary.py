"""CPU: the oracle's unary / scalar ops and softmax against the reference's LibTorch differential
procedures replayed with PyTorch (tests/golden/torch_unary.npz, made by make_torch_unary.py) and the
reference's panics.  The literal known answers of the reference's unit tests for these ops run through
test_oracle_golden.py with the other cases of reference_known_answers.json."""
import os

import numpy as np
import pytest

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "torch_unary.npz"))
CASES = [str(c) for c in GOLDEN["cases"]]


def split_case(case):
    if case.startswith("pow_scalar_"):
        return "pow_scalar", float(case.split("_")[-1])
    name = case.rstrip("0123456789")
    return name, (0.1 if name == "leaky_relu" else 0.0)


def tolerances(name):
    # the reference's validator: (1e-6, 1e-8) for exp, log and sqrt, its default (1e-5, 1e-8) for the others
    return (1e-6, 1e-8) if name in ("exp", "log", "sqrt") else (1e-5, 1e-8)


@pytest.mark.parametrize("case", CASES)
def test_forward_and_gradient_match_libtorch_procedure(ora, case):
    name, p = split_case(case)
    rtol, atol = tolerances(name)
    x, want = GOLDEN[case + "_x"], GOLDEN[case + "_y"]
    got = ora.unary(name, x, p)
    assert got.shape == want.shape
    np.testing.assert_allclose(got, want, rtol=rtol, atol=atol)
    gx, want_g = GOLDEN[case + "_gx"], GOLDEN[case + "_grad"]
    y = ora.unary(name, gx, p)
    saved = {"out": y, "in": gx, None: None}[ora.UNARY_SAVES[name]]
    got_g = ora.unary_backward(name, saved, np.ones_like(gx), p)
    # tanh'(x) = 1 - t*t cancels near |t| -> 1: the absolute floor is one rounding of t*t
    np.testing.assert_allclose(got_g, want_g, rtol=rtol, atol=max(atol, 1.2e-7 if name == "tanh" else 0))


def test_exp_chain_gradient(ora):
    """z = exp(x)*x + exp(x), upstream ones: dz/dx = exp(x)*x + exp(x) + exp(x) (libtorch-validation .../ops/exp.rs:91-150)."""
    for i in range(int(GOLDEN["exp_chain_count"])):
        x = GOLDEN[f"exp_chain{i}_x"]
        ex = ora.unary("exp", x)
        ones = np.ones_like(x)
        # backward in the reference's order: add -> (g, g); mul -> (g*x, g*ex); exp receives g*x then + g
        g_ex = ora.add(ora.mul(ones, x), ones)
        g_x = ora.add(ora.mul(ones, ex), ora.unary_backward("exp", ex, g_ex))
        np.testing.assert_allclose(g_x, GOLDEN[f"exp_chain{i}_grad"], rtol=2e-6, atol=1e-8)


@pytest.mark.parametrize("i", range(int(GOLDEN["softmax_count"])))
def test_softmax_matches_libtorch_procedure(ora, i):
    dim = int(GOLDEN[f"softmax{i}_dim"])
    y = ora.softmax(GOLDEN[f"softmax{i}_x"], dim)
    np.testing.assert_allclose(y, GOLDEN[f"softmax{i}_y"], rtol=1e-5, atol=1e-8)
    yg = ora.softmax(GOLDEN[f"softmax{i}_gx"], dim)
    # d sum(softmax) / dx is zero up to rounding: y * (1 - dot) with dot = 1 +- a couple of ulp
    g = ora.softmax_backward(yg, np.ones_like(yg), dim)
    assert np.max(np.abs(g)) < 2.5e-7
    g_up = ora.softmax_backward(yg, GOLDEN[f"softmax{i}_up"], dim)
    np.testing.assert_allclose(g_up, GOLDEN[f"softmax{i}_grad_up"], rtol=1e-5, atol=2e-7)


def test_softmax_is_sequential_in_the_reduced_axis(ora):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 50, 4)).astype(np.float32)
    y = ora.softmax(x, 1)
    for o in range(3):
        for i in range(4):
            col = x[o, :, i]
            e = np.exp((col - col.max()).astype(np.float32)).astype(np.float32)
            s = np.float32(0)
            for v in e:
                s = np.float32(s + v)
            # exp is libm's here and numpy's there: compare to a few ulp, the order of the sum is the point
            np.testing.assert_allclose(y[o, :, i], e * (np.float32(1) / s), rtol=3e-7)


def test_panics_of_the_reference_are_reported(ora):
    with pytest.raises(ora.DomainError):
        ora.unary("log", np.array([1.0, 0.0], np.float32))          # log.rs:177-182 should_panic
    with pytest.raises(ora.DomainError):
        ora.unary("log", np.array([np.nan], np.float32))            # `x > 0.0` is false for NaN
    with pytest.raises(ora.DomainError):
        ora.unary("div_scalar", np.ones(6, np.float32), 0.0)        # div.rs:705-709 should_panic
    assert ora.unary("log", np.array([], np.float32)).size == 0


def test_pow_scalar_special_exponents(ora):
    x = np.array([0.0, 0.25, 2.0, 9.0, 1e-20], np.float32)
    assert np.array_equal(ora.unary("pow_scalar", x, 2.0), x * x)                 # pow.rs:139-147
    assert np.array_equal(ora.unary("pow_scalar", x, 0.5), np.sqrt(x))            # pow.rs:148-156
    g = ora.unary_backward("pow_scalar", x, np.ones_like(x), 0.0)                 # grad_fn/ops/pow.rs:17-19
    assert np.array_equal(g, np.zeros_like(x))
    g2 = ora.unary_backward("pow_scalar", x, np.full_like(x, 3.0), 2.0)           # go * (2 * x^1)
    assert np.array_equal(g2, np.float32(3.0) * (np.float32(2.0) * x))


def test_backward_association_is_the_references(ora):
    """sigmoid: (go*s)*(1-s), not go*(s*(1-s)); sqrt: go*((1/y)*0.5), not go/(2y)."""
    rng = np.random.default_rng(9)
    s = rng.uniform(0.01, 0.99, 4096).astype(np.float32)
    go = rng.standard_normal(4096).astype(np.float32)
    want = (go * s) * (np.float32(1) - s)
    assert np.array_equal(ora.unary_backward("sigmoid", s, go), want)
    y = rng.uniform(0.1, 4.0, 4096).astype(np.float32)
    want = go * ((np.float32(1) / y) * np.float32(0.5))
    assert np.array_equal(ora.unary_backward("sqrt", y, go), want)
    t = rng.uniform(-0.99, 0.99, 4096).astype(np.float32)
    assert np.array_equal(ora.unary_backward("tanh", t, go), go * (np.float32(1) - t * t))
