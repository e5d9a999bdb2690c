"""The C++ host mirror (include/train_station_b200.hpp) through its test program tests/cpp/mirror_step.cpp.

CPU: the header compiles warning-free against the C ABI and the program refuses to run without a device.
GPU: the program trains the same networks as the Python-side engine tests and its results are compared with the
oracle under the same bounds (FP32 mode: forward, weight gradients and Adam state bit for bit)."""
import os
import subprocess
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as entry  # noqa: E402

from conftest import assert_bit_equal  # noqa: E402


def run_program(tmp_path, ws, bs, x, target, loss, relu_last, steps, timed=0):
    dims = [ws[0].shape[0]] + [w.shape[1] for w in ws]
    batch = x.shape[0]
    tgt = target if target is not None else np.zeros((batch, dims[-1]), np.float32)
    inp, out = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        f.write(np.array([len(ws), batch] + dims, np.int32).tobytes())
        f.write(np.ascontiguousarray(x, np.float32).tobytes())
        f.write(np.ascontiguousarray(tgt, np.float32).tobytes())
        for w, b in zip(ws, bs):
            f.write(np.ascontiguousarray(w, np.float32).tobytes())
            f.write(np.ascontiguousarray(b, np.float32).tobytes())
    exe = entry.build_cpp_tests()
    r = subprocess.run([exe, str(inp), str(out), str(steps), loss, "1" if relu_last else "0", str(timed)], stdout=subprocess.PIPE,
                       stderr=subprocess.PIPE, text=True, timeout=600)
    if r.returncode != 0:
        return r, None
    flat = np.fromfile(out, np.float32)
    pos = 0

    def take(shape):
        nonlocal pos
        n = int(np.prod(shape))
        a = flat[pos:pos + n].reshape(shape)
        pos += n
        return a

    got = {"loss": float(take((1,))[0]), "y": take((batch, dims[-1])), "gw": [], "gb": [], "w": [], "b": [], "m": [], "v": []}
    for w, b in zip(ws, bs):
        got["gw"].append(take(w.shape))
        got["gb"].append(take(b.shape))
    for w, b in zip(ws, bs):
        got["w"].append(take(w.shape))
        got["b"].append(take(b.shape))
        got["m"].append(take(w.shape))
        got["v"].append(take(w.shape))
    assert pos == flat.size
    return r, got


def test_program_builds_and_refuses_to_run_without_a_device(tmp_path):
    exe = entry.build_cpp_tests(force=True)
    assert os.access(exe, os.X_OK)
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present: the refusal is what the CPU run checks")
    rng = np.random.default_rng(0)
    r, got = run_program(tmp_path, [rng.standard_normal((4, 3), dtype=np.float32)], [np.zeros(3, np.float32)],
                         rng.standard_normal((2, 4), dtype=np.float32), None, "sum", True, 1)
    assert got is None and r.returncode == 1
    assert "no CUDA device" in r.stderr


@pytest.mark.gpu
def test_readme_step_fp32_matches_the_oracle(gpu, ora, tmp_path):
    """BASELINE config 1 through the C++ mirror: y = relu(x.w + b); loss = sum(y); backward; one Adam step."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((32, 784), dtype=np.float32)
    ws, bs = [rng.standard_normal((784, 128), dtype=np.float32)], [np.zeros(128, np.float32)]
    st = ora.MlpState(ws, bs)
    ref = ora.mlp_step(st, x, loss_kind=ora.LOSS_SUM, relu_last=True, want_y=True)
    r, got = run_program(tmp_path, ws, bs, x, None, "sum", True, 1, timed=2000)
    assert r.returncode == 0, r.stderr
    assert_bit_equal(got["y"], ref["y"], "forward")
    assert_bit_equal(got["gw"][0], st.gw[0], "weight gradient")
    np.testing.assert_allclose(got["gb"][0], st.gb[0], rtol=1e-5, atol=1e-6)
    assert abs(got["loss"] - float(ref["loss"])) <= 1e-5 * abs(float(ref["loss"]))
    assert_bit_equal(got["w"][0], st.w[0], "weights after Adam")
    assert_bit_equal(got["m"][0], st.mw[0], "Adam m")
    assert_bit_equal(got["v"][0], st.vw[0], "Adam v")
    rate = float(r.stdout.split("steps_per_s")[1].split()[0])
    print(f"C++ host, README step: {rate:.0f} steps/s")
    assert rate > 0


@pytest.mark.gpu
def test_three_layer_mse_steps_match_the_oracle(gpu, ora, tmp_path):
    rng = np.random.default_rng(3)
    dims, batch, steps = [96, 128, 64, 12], 64, 4
    ws = [(rng.standard_normal((dims[i], dims[i + 1])) / np.sqrt(dims[i])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(dims[i + 1], np.float32) for i in range(3)]
    x, t = rng.standard_normal((batch, dims[0]), dtype=np.float32), rng.standard_normal((batch, dims[-1]), dtype=np.float32)
    st = ora.MlpState(ws, bs)
    for _ in range(steps):
        ref = ora.mlp_step(st, x, t, loss_kind=ora.LOSS_MSE)
    r, got = run_program(tmp_path, ws, bs, x, t, "mse", False, steps)
    assert r.returncode == 0, r.stderr
    assert abs(got["loss"] - float(ref["loss"])) <= 1e-5 * abs(float(ref["loss"])) + 1e-6
    for i in range(3):
        np.testing.assert_allclose(got["gw"][i], st.gw[i], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(got["gb"][i], st.gb[i], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(got["w"][i], st.w[i], rtol=1e-5, atol=2e-6)
        np.testing.assert_allclose(got["b"][i], st.b[i], rtol=1e-5, atol=2e-6)
