"""GPU: the Tensor / gradtrack / Adam engine through the Python mirror of the reference API,
checked against the reference's known answers, the LibTorch-differential fixtures and the
CPU oracle on the BASELINE configurations (reduced where the oracle would take minutes)."""
import json
import os

import numpy as np
import pytest

from conftest import assert_bit_equal
from oracle_graph import run_case_device

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
KNOWN = json.load(open(os.path.join(GOLDEN, "reference_known_answers.json")))
KNOWN["cases"] = KNOWN["cases"] + json.load(open(os.path.join(GOLDEN, "reference_known_answers_broadcast.json")))["cases"]


@pytest.mark.parametrize("fusion", [True, False])
@pytest.mark.parametrize("case", KNOWN["cases"], ids=[c["name"] for c in KNOWN["cases"]])
def test_reference_known_answers_on_device(gpu, case, fusion):
    gpu.set_fusion(fusion)
    values, grads = run_case_device(gpu, case)
    tol = case["tol"]
    for name, exp in case.get("expect", {}).items():
        got, dims = values[name]
        assert dims == exp["dims"], (name, dims)
        np.testing.assert_allclose(got.reshape(-1), np.array(exp["data"], np.float32), rtol=0, atol=tol)
    for name, exp in case.get("expect_grad", {}).items():
        if exp is None:
            assert grads[name] is None
            continue
        assert grads[name] is not None, name
        got, dims = grads[name]
        assert dims == exp["dims"], (name, dims)
        np.testing.assert_allclose(got.reshape(-1), np.array(exp["data"], np.float32), rtol=0, atol=tol)


def _close_ref(got, want, rtol, atol):
    d = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    return bool(np.all((d <= rtol * np.abs(want)) | (d <= atol)))


def test_torch_differential_on_device(gpu):
    z = np.load(os.path.join(GOLDEN, "torch_differential.npz"))
    T = gpu.Tensor
    for i in range(int(z["matmul_count"])):
        l, r = z[f"matmul{i}_left"], z[f"matmul{i}_right"]
        a, b = T.from_slice(l, l.shape).with_requires_grad(), T.from_slice(r, r.shape).with_requires_grad()
        y = a.matmul(b)
        y.backward(T.ones(y.shape().dims))
        assert _close_ref(y.data(), z[f"matmul{i}_out"], 1e-5, 1e-8)
        assert _close_ref(a.grad_by_value().data(), z[f"matmul{i}_grad_left"], 1e-5, 1e-8)
        assert _close_ref(b.grad_by_value().data(), z[f"matmul{i}_grad_right"], 1e-5, 1e-8)
        gpu.clear_gradients()
    for i in range(int(z["linear_count"])):
        x, w, b = (T.from_slice(z[f"linear{i}_{k}"], z[f"linear{i}_{k}"].shape).with_requires_grad() for k in "xwb")
        y = x.matmul(w).add_tensor(b)
        y.sum().backward(None)
        assert _close_ref(y.data(), z[f"linear{i}_out"], 1e-5, 1e-8)
        for k, t in zip("xwb", (x, w, b)):
            assert _close_ref(t.grad_by_value().data(), z[f"linear{i}_grad_{k}"], 1e-5, 1e-8), (i, k)
        gpu.clear_gradients()
    x = T.from_slice(z["relu_x"], z["relu_x"].shape).with_requires_grad()
    y = x.relu()
    y.sum().backward(None)
    assert np.array_equal(y.data(), z["relu_out"]) and np.array_equal(x.grad_by_value().data(), z["relu_grad"])


def test_torch_differential_adam_on_device(gpu):
    """adam.rs:65-160: loss = sum(2p + 1) written with the ops of this path: sum(p + p) has the same gradient 2."""
    z = np.load(os.path.join(GOLDEN, "torch_differential.npz"))
    for i in range(int(z["adam_count"])):
        steps, lr, b1, b2, eps, wd = z[f"adam{i}_cfg"]
        init = z[f"adam{i}_init"]
        p = gpu.Tensor.from_slice(init, init.shape).with_requires_grad()
        opt = gpu.Adam.with_config(gpu.AdamConfig(lr, b1, b2, eps, wd))
        opt.add_parameter(p)
        for _ in range(int(steps)):
            p.add_tensor(p).sum().backward(None)
            opt.step([p])
            opt.zero_grad([p])
        assert _close_ref(p.data(), z[f"adam{i}_final"], 1e-4, 1e-4), i


def _mlp_device(ts, ws, bs, x, tgt, loss_kind, relu_last, steps=1, lr=1e-3):
    T = ts.Tensor
    W = [T.from_slice(w, w.shape).with_requires_grad() for w in ws]
    B = [T.from_slice(b, b.shape).with_requires_grad() for b in bs]
    params = [p for pair in zip(W, B) for p in pair]
    opt = ts.Adam.with_learning_rate(lr)
    opt.add_parameters(params)
    X = T.from_slice(x, x.shape)
    Tg = T.from_slice(tgt, tgt.shape) if tgt is not None else None
    out = {}
    for s in range(steps):
        h = X
        for i in range(len(W)):
            h = h.matmul(W[i]).add_tensor(B[i])
            if i + 1 < len(W) or relu_last:
                h = h.relu()
        if loss_kind == "sum":
            loss = h.sum()
        elif loss_kind == "mean":
            loss = h.mean()
        else:
            loss = h.sub_tensor(Tg).pow_scalar(2.0).mean()
        loss.backward(None)
        out = {"loss": loss.value(), "y": h.data(), "gw": [w.grad_by_value().data() for w in W],
               "gb": [b.grad_by_value().data() for b in B]}
        opt.step(params)
        opt.zero_grad(params)
    out["w"] = [w.data() for w in W]
    out["b"] = [b.data() for b in B]
    out["m"] = [opt.state(w)[0].data() for w in W]
    out["v"] = [opt.state(w)[1].data() for w in W]
    return out


def _config1(rng):
    x = rng.standard_normal((32, 784), dtype=np.float32)
    w = rng.standard_normal((784, 128), dtype=np.float32)
    return [w], [np.zeros(128, np.float32)], x


@pytest.mark.parametrize("fusion", [True, False])
def test_config1_readme_step_fp32(gpu, ora, fusion):
    """BASELINE config 1: y = relu(x.w + b); loss = sum(y); backward; one Adam step; seed 0.
    FP32 mode reproduces the reference's GEMM summation order, so everything except the two
    tree reductions (loss, bias gradient) is bit-identical to the CPU path."""
    gpu.set_fusion(fusion)
    ws, bs, x = _config1(np.random.default_rng(0))
    st = ora.MlpState(ws, bs)
    ref = ora.mlp_step(st, x, loss_kind=ora.LOSS_SUM, relu_last=True, want_y=True)
    got = _mlp_device(gpu, ws, bs, x, None, "sum", True)
    assert_bit_equal(got["y"], ref["y"], "forward")                 # includes the ReLU mask, bit-exact
    assert_bit_equal(got["gw"][0], st.gw[0], "weight gradient")
    np.testing.assert_allclose(got["gb"][0], st.gb[0], rtol=1e-5, atol=1e-6)   # tree vs sequential column sum
    assert abs(got["loss"] - float(ref["loss"])) <= 1e-5 * abs(float(ref["loss"]))
    assert_bit_equal(got["w"][0], st.w[0], "weights after Adam")
    assert_bit_equal(got["m"][0], st.mw[0], "Adam m")
    assert_bit_equal(got["v"][0], st.vw[0], "Adam v")
    np.testing.assert_allclose(got["b"][0], st.b[0], rtol=1e-5, atol=1e-6)


def test_fusion_does_not_change_results(gpu):
    rng = np.random.default_rng(42)
    dims, batch = [64, 96, 80, 12], 48
    ws = [(rng.standard_normal((dims[i], dims[i + 1])) / np.sqrt(dims[i])).astype(np.float32) for i in range(3)]
    bs = [rng.standard_normal(dims[i + 1]).astype(np.float32) * 0.1 for i in range(3)]
    x, t = rng.standard_normal((batch, dims[0]), dtype=np.float32), rng.standard_normal((batch, dims[-1]), dtype=np.float32)
    gpu.set_fusion(True)
    a = _mlp_device(gpu, ws, bs, x, t, "mse", False, steps=3)
    gpu.set_fusion(False)
    b = _mlp_device(gpu, ws, bs, x, t, "mse", False, steps=3)
    assert a["loss"] == b["loss"]
    for k in ("gw", "w", "m", "v", "b"):
        for u, v in zip(a[k], b[k]):
            assert_bit_equal(u, v, k)
    # the fused ReLU-backward + column-sum kernel may partition rows differently from the plain column sum
    for u, v in zip(a["gb"], b["gb"]):
        np.testing.assert_allclose(u, v, rtol=1e-5, atol=1e-7)


def test_config4_shape_mlp_steps_fp32(gpu, ora):
    """BASELINE config 4 (784-1024-1024-10, Kaiming-uniform, one-hot targets, MSE) at batch 256 for 5 steps."""
    rng = np.random.default_rng(3)
    dims, batch, steps = [784, 1024, 1024, 10], 256, 5
    ws = [rng.uniform(-np.sqrt(6 / dims[i]), np.sqrt(6 / dims[i]), (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(dims[i + 1], np.float32) for i in range(3)]
    x = rng.standard_normal((batch, dims[0]), dtype=np.float32)
    t = np.eye(10, dtype=np.float32)[rng.integers(0, 10, batch)]
    st = ora.MlpState(ws, bs)
    for _ in range(steps):
        ref = ora.mlp_step(st, x, t, loss_kind=ora.LOSS_MSE)
    got = _mlp_device(gpu, ws, bs, x, t, "mse", False, steps=steps)
    assert abs(got["loss"] - float(ref["loss"])) <= 1e-5 * abs(float(ref["loss"])) + 1e-6
    for i in range(3):
        np.testing.assert_allclose(got["gw"][i], st.gw[i], rtol=1e-5, atol=1e-6)   # north-star FP32 tolerance
        np.testing.assert_allclose(got["gb"][i], st.gb[i], rtol=1e-5, atol=1e-6)
        # Adam normalises the step, so a last-bit gradient difference can move a parameter by up to ~lr*1e-3
        np.testing.assert_allclose(got["w"][i], st.w[i], rtol=1e-5, atol=2e-6)
        np.testing.assert_allclose(got["b"][i], st.b[i], rtol=1e-5, atol=2e-6)


def test_config3_shape_dense_layer_mean_loss(gpu, ora):
    """BASELINE config 3 at 512^3: Y = relu(X.W + b), loss = mean(Y), gradients w.r.t. X, W and b."""
    rng = np.random.default_rng(2)
    n = 512
    x = rng.standard_normal((n, n), dtype=np.float32)
    w = (rng.standard_normal((n, n)) * np.sqrt(1.0 / n)).astype(np.float32)
    b = np.zeros(n, np.float32)
    st = ora.MlpState([w], [b])
    ref = ora.mlp_step(st, x, loss_kind=ora.LOSS_MEAN, relu_last=True, want_gx=True, do_adam=False)
    T = gpu.Tensor
    X, W, B = (T.from_slice(a, a.shape).with_requires_grad() for a in (x, w, b))
    loss = X.matmul(W).add_tensor(B).relu().mean()
    loss.backward(None)
    assert abs(loss.value() - float(ref["loss"])) <= 1e-5 * abs(float(ref["loss"]))
    assert_bit_equal(X.grad_by_value().data(), ref["gx"], "dX")
    assert_bit_equal(W.grad_by_value().data(), st.gw[0], "dW")
    np.testing.assert_allclose(B.grad_by_value().data(), st.gb[0], rtol=1e-5, atol=1e-9)


def test_elementwise_sweep_config2_gradients(gpu, ora):
    """BASELINE config 2 at 2^20: out = op(a, b), loss = sum(out), backward to both; gradients are exact single ops."""
    n = 1 << 20
    rng = np.random.default_rng(1)
    a = rng.standard_normal(n, dtype=np.float32)
    b = (rng.random(n, dtype=np.float32) * 1.5 + 0.5).astype(np.float32)
    ones = np.ones(n, np.float32)
    want = {"add": (ones, ones), "sub": (ones, ora.neg(ones)), "mul": ora.mul_bwd(a, b, ones), "div": ora.div_bwd(a, b, ones)}
    for op in ("add", "sub", "mul", "div"):
        A = gpu.Tensor.from_slice(a, [n]).with_requires_grad()
        Bt = gpu.Tensor.from_slice(b, [n]).with_requires_grad()
        out = getattr(A, f"{op}_tensor")(Bt)
        assert_bit_equal(out.data(), getattr(ora, op)(a, b), op)
        out.sum().backward(None)
        assert_bit_equal(A.grad_by_value().data(), want[op][0], f"{op} grad a")
        assert_bit_equal(Bt.grad_by_value().data(), want[op][1], f"{op} grad b")
        gpu.clear_gradients()


def test_gradient_accumulates_over_two_uses(gpu):
    x = gpu.Tensor.from_slice([1.0, 2.0, 3.0], [3]).with_requires_grad()
    y = x.mul_tensor(x).add_tensor(x)      # x^2 + x  ->  2x + 1
    y.sum().backward(None)
    assert x.grad_by_value().data().tolist() == [3.0, 5.0, 7.0]


def test_second_operand_only_requires_grad(gpu):
    """The reference mis-assigns the gradient when only the second operand requires grad
    (add.rs:135-142 vs engine.rs:1000-1001); this path gives each operand its own."""
    a = gpu.Tensor.from_slice([1.0, 2.0], [2])
    b = gpu.Tensor.from_slice([4.0, 8.0], [2]).with_requires_grad()
    a.div_tensor(b).sum().backward(None)
    assert a.grad_by_value() is None
    np.testing.assert_allclose(b.grad_by_value().data(), [-1.0 / 16.0, -2.0 / 64.0])


def test_no_grad_track(gpu):
    x = gpu.Tensor.ones([2, 2]).with_requires_grad()
    n0 = gpu.tape_len()
    with gpu.NoGradTrack():
        assert not gpu.is_grad_enabled()
        y = x.mul_tensor(x)
        assert not y.requires_grad() and gpu.tape_len() == n0
    assert gpu.is_grad_enabled()
    assert x.mul_tensor(x).requires_grad() and gpu.tape_len() == n0 + 1


def test_error_behaviour(gpu):
    T = gpu.Tensor
    with pytest.raises(gpu.TrainStationError):
        T.from_slice([1.0, 2.0, 3.0], [2, 2])
    with pytest.raises(gpu.TrainStationError):
        T.ones([2, 3]).matmul(T.ones([4, 2]))
    with pytest.raises(gpu.TrainStationError):
        T.ones([2, 3]).add_tensor(T.ones([2]))
    with pytest.raises(gpu.TrainStationError):
        T.ones([3]).value()
    # Adam: unlinked parameter is an error; a linked parameter without gradient is skipped with a message
    p = T.ones([4]).with_requires_grad()
    opt = gpu.Adam.new()
    with pytest.raises(gpu.TrainStationError):
        opt.step([p])
    opt.add_parameter(p)
    opt.step([p])
    assert "no gradient" in opt.last_message and p.data().tolist() == [1.0] * 4
    with pytest.raises(gpu.TrainStationError):
        opt.add_parameter(T.ones([2]))        # must require grad, adam/mod.rs:287-300


def test_in_place_write_between_forward_and_backward_is_detected(gpu):
    w = gpu.Tensor.ones([4, 4]).with_requires_grad()
    x = gpu.Tensor.ones([2, 4]).with_requires_grad()
    loss = x.matmul(w).sum()
    w.fill(2.0)
    with pytest.raises(gpu.TrainStationError, match="modified in place"):
        loss.backward(None)


def test_async_upload_overlaps_and_is_ordered(gpu, ora):
    n = 1 << 20
    pin = gpu.PinnedBuffer(n)
    rng = np.random.default_rng(9)
    a = rng.standard_normal(n, dtype=np.float32)
    pin.array[:] = a
    t = gpu.Tensor.from_pinned_async(pin, [n])
    assert_bit_equal(t.add_tensor(t).data(), ora.add(a, a))


def test_host_running_ahead_of_the_gpu_changes_nothing(gpu):
    """Every call only enqueues work, so the host may be many steps ahead of the GPU.  Whatever a queued launch
    needs (the Adam pointer table in particular) must be captured when it is enqueued: a run that synchronises
    after every step and a run that never does must end with identical bits, also when gradient buffers change
    address from step to step."""
    rng = np.random.default_rng(21)
    x = rng.standard_normal((8192, 2048), dtype=np.float32)
    w0 = (rng.standard_normal((2048, 2048)) / np.sqrt(2048)).astype(np.float32)

    def run(sync_each_step):
        gpu.clear_gradients()
        X = gpu.Tensor.from_slice(x, x.shape)
        W = gpu.Tensor.from_slice(w0, w0.shape).with_requires_grad()
        opt = gpu.Adam.with_learning_rate(1e-3)
        opt.add_parameter(W)
        held = None
        for s in range(10):
            if s % 2:
                held = gpu.Tensor.new(w0.shape)     # occupies the block the last gradient used: the next one lands elsewhere
            X.matmul(W).relu().sum().backward(None)
            opt.step([W])
            opt.zero_grad([W])
            if s % 2 == 0:
                held = None
            if sync_each_step:
                gpu.synchronize()
        return W.data()

    assert_bit_equal(run(False), run(True), "weights after 10 steps")


def test_storage_is_recycled_across_steps(gpu):
    rng = np.random.default_rng(0)
    ws, bs, x = _config1(rng)
    _mlp_device(gpu, ws, bs, x, None, "sum", True, steps=2)
    s0 = gpu.allocator_stats()
    _mlp_device(gpu, ws, bs, x, None, "sum", True, steps=4)
    s1 = gpu.allocator_stats()
    assert s1["driver_allocations"] == s0["driver_allocations"], "steady-state steps must not reach cudaMalloc"


def test_backward_seed_of_a_scalar_is_shared_and_cannot_be_overwritten(gpu):
    """backward(None) on a one-element root seeds with a 1.0 that lives once per device (no launch to write it).  The
    handle a caller gets for that gradient reads 1.0; writing into it (fill, upload, the raw pointer) lands in a private
    copy, so the next backward still starts from 1.0."""
    T = gpu.Tensor
    x = T.from_slice(np.arange(6, dtype=np.float32), [2, 3]).with_requires_grad()
    loss = x.mul_tensor(x).sum()
    loss.backward(None)
    g_root = loss.grad_by_value()
    assert g_root is not None and g_root.data().tolist() == [1.0]
    np.testing.assert_array_equal(x.grad_by_value().data(), 2 * np.arange(6, dtype=np.float32).reshape(2, 3))
    g_root.fill(5.0)
    assert g_root.data().tolist() == [5.0]
    g_root.copy_from_host(np.array([7.0], np.float32))
    assert g_root.data().tolist() == [7.0]
    assert g_root.data_ptr() != 0
    gpu.clear_gradients()
    y = T.from_slice(np.arange(6, dtype=np.float32), [2, 3]).with_requires_grad()
    loss2 = y.mul_tensor(y).sum()
    loss2.backward(None)
    assert loss2.grad_by_value().data().tolist() == [1.0]
    np.testing.assert_array_equal(y.grad_by_value().data(), 2 * np.arange(6, dtype=np.float32).reshape(2, 3))
