"""CPU: the AMSGrad branch of Adam and the seeded normal initialiser.

* oracle AMSGrad against the reference's LibTorch procedure replayed with PyTorch (tests/golden/torch_amsgrad.npz)
  and against an f64 evaluation of the reference's definition on varying gradients;
* oracle randn: the integer generator against arbitrary-precision integers, the float stage against f64 math, and
  the properties the reference's own tests assert (tensor/init/random.rs:623-760);
* the library's host generator (ts_randn_host, no device involved) against the oracle, bit for bit."""
import ctypes as C
import math
import os

import numpy as np
import pytest

from conftest import assert_bit_equal

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
M64 = (1 << 64) - 1


def py_xorshift(seed, n):
    s, out = seed & M64, []
    for _ in range(n):
        s ^= (s << 13) & M64
        s ^= s >> 7
        s ^= (s << 17) & M64
        out.append(s)
    return out


def test_xorshift_matches_big_integer_arithmetic(ora):
    for seed in (1, 42, 12345, 0xDEADBEEFCAFEBABE, M64):
        assert ora.xorshift_u64(seed, 64).tolist() == py_xorshift(seed, 64)
    assert ora.xorshift_u64(0, 8).tolist() == [0] * 8       # a zero state never leaves zero (random.rs:524-529)
    # first step from state 1, by hand: 1 ^ 1<<13 = 0x2001; ^ >>7 = 0x2001 ^ 0x40 = 0x2041; ^ <<17 = 0x2041 ^ 0x40820000
    assert int(ora.xorshift_u64(1, 1)[0]) == 0x40822041


def test_randn_float_stage(ora):
    for seed in (1, 42, 12345):
        n = 257
        got = ora.randn([n], seed)
        draws = py_xorshift(seed, 2 * n)
        for i in range(n):
            b1 = (draws[2 * i] & 0x7FFFFF) | (126 << 23)
            b2 = (draws[2 * i + 1] & 0x7FFFFF) | (126 << 23)
            u1 = float(np.array([b1], np.uint32).view(np.float32)[0])
            u2 = float(np.array([b2], np.uint32).view(np.float32)[0])
            assert 0.5 <= u1 < 1.0 and 0.5 <= u2 < 1.0        # exponent field 126, not the [0, 1) the comment claims
            # each f32 step rounded from its f64 value: agrees with libm's logf / cosf except where they miss
            # correct rounding by an ulp, hence the 2-ulp allowance on the product
            r = np.float32(math.sqrt(float(np.float32(np.float32(-2.0) * np.float32(math.log(u1))))))
            ang = np.float32(np.float32(2.0) * np.float32(math.pi)) * np.float32(u2)
            z = np.float32(r * np.float32(math.cos(float(ang))))
            assert abs(float(got[i]) - float(z)) <= 2 * float(np.spacing(np.abs(z))) + 1e-12, (seed, i)


def test_randn_properties_the_reference_asserts(ora):
    a, b = ora.randn([100], 12345), ora.randn([100], 12345)
    assert_bit_equal(a, b)                                         # random.rs:638-649
    assert not np.array_equal(ora.randn([100], 1), ora.randn([100], 2))   # :652-670
    t = ora.randn([100, 100], 42)                                  # :699-732
    assert abs(float(t.mean())) < 0.1 and t.min() > -4.0 and t.max() < 4.0
    assert np.any(t != 0)
    assert ora.randn([0], 7).size == 0                             # :692-696
    # a prefix of a longer draw is the shorter draw: one serial stream
    assert_bit_equal(ora.randn([10], 9), ora.randn([1000], 9)[:10])
    # u1 in [0.5, 1) bounds the radius by sqrt(2 ln 2)
    assert float(np.abs(ora.randn([100000], 3)).max()) <= math.sqrt(2 * math.log(2)) + 1e-6


def test_library_host_generator_matches_oracle(ts, ora):
    lib = ts._ffi.lib()
    for seed, n in ((42, 10000), (12345, 100), (1, 7), (0, 5), (M64, 33)):
        out = np.empty(n, np.float32)
        assert lib.ts_randn_host(out.ctypes.data_as(C.c_void_p), n, seed) is True
        assert_bit_equal(out, ora.randn([n], seed), f"seed {seed}")
    assert lib.ts_randn_host(None, 4, 1) is False


# ----------------------------------------------------------------------------- AMSGrad
def _close_ref(got, want, rtol, atol):
    d = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    return bool(np.all((d <= rtol * np.abs(want)) | (d <= atol)))


def test_amsgrad_matches_libtorch_procedure(ora):
    z = np.load(os.path.join(GOLDEN, "torch_amsgrad.npz"))
    for i in range(int(z["count"])):
        steps, lr, b1, b2, eps, wd = z[f"case{i}_cfg"]
        p = z[f"case{i}_init"].copy()
        m, v, vm = np.zeros_like(p), np.zeros_like(p), np.zeros_like(p)
        g = np.full_like(p, 2.0)
        for t in range(1, int(steps) + 1):
            ora.adam_update_amsgrad(p.reshape(-1), g.reshape(-1), m.reshape(-1), v.reshape(-1), vm.reshape(-1), t, lr, b1, b2, eps, wd)
        assert _close_ref(p, z[f"case{i}_final"], 1e-4, 1e-4), i      # the reference's Adam tolerance, adam.rs:47-51


def amsgrad_f64(p, g, m, v, vm, t, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8):
    """optimizers/adam/mod.rs:485-556 with amsgrad, in float64, betas as the f32 values the reference holds."""
    b1, b2 = float(np.float32(b1)), float(np.float32(b2))
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    mh, vh = m / (1 - b1 ** t), v / (1 - b2 ** t)
    vm = np.maximum(vm, vh)
    return p - lr * mh / (np.sqrt(vm) + eps), m, v, vm


def test_amsgrad_on_varying_gradients_follows_the_references_definition(ora):
    rng = np.random.default_rng(17)
    n = 1003
    p = rng.standard_normal(n).astype(np.float32)
    m, v, vm = (np.zeros(n, np.float32) for _ in range(3))
    p64, m64, v64, vm64 = p.astype(np.float64), np.zeros(n), np.zeros(n), np.zeros(n)
    held = False
    for t in range(1, 31):
        g = (rng.standard_normal(n) * (3.0 if t < 5 else 0.3)).astype(np.float32)   # large early gradients: the maximum must hold
        ora.adam_update_amsgrad(p, g, m, v, vm, t)
        p64, m64, v64, vm64 = amsgrad_f64(p64, g.astype(np.float64), m64, v64, vm64, t)
        held = held or bool(np.any(vm64 > v64 / (1 - float(np.float32(0.999)) ** t) * 1.5))
    assert held, "the test data never exercised the running maximum"
    np.testing.assert_allclose(p, p64, rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(vm, vm64, rtol=1e-5, atol=1e-12)
    # and the maximum is of the bias-corrected moment, not PyTorch's maximum of the raw one
    assert np.all(vm >= v)


def test_amsgrad_zero_start_equals_copy_of_first_v_hat(ora):
    """The reference creates v_hat_max as a clone of the first v_hat (adam/mod.rs:535-537); starting from zero is the same."""
    g = np.array([0.0, -0.0, 1e-30, 3.0, -2.5, np.nan, 1e19, -1e-20, 0.5], np.float32)
    p, m, v, vm = (np.zeros(9, np.float32) for _ in range(4))
    ora.adam_update_amsgrad(p, g, m, v, vm, 1)
    f2 = np.float32(1.0) / np.float32(1.0 - float(np.float32(0.999)))
    assert_bit_equal(vm, v * f2)
    p2, m2, v2 = (np.zeros(9, np.float32) for _ in range(3))
    ora.adam_update(p2, g, m2, v2, 1)
    assert_bit_equal(p, p2)        # on the first step AMSGrad and plain Adam coincide
