"""GPU: checkpoints in the reference's formats through the public API — a tensor survives a save / load bit for bit,
and a training run that is saved, loaded into fresh tensors and relinked continues exactly like the uninterrupted one."""
import os

import numpy as np
import pytest

from conftest import assert_bit_equal

pytestmark = pytest.mark.gpu


def test_tensor_round_trip_all_forms(gpu, tmp_path):
    T = gpu.Tensor
    rng = np.random.default_rng(0)
    xh = rng.standard_normal((5, 7)).astype(np.float32)
    x = T.from_slice(xh, [5, 7]).with_requires_grad()
    for form in ("json", "binary"):
        blob = x.to_json() if form == "json" else x.to_binary()
        y = T.from_json(blob) if form == "json" else T.from_binary(blob)
        assert y.shape().dims == [5, 7] and y.requires_grad()
        assert_bit_equal(y.data(), xh, form)
        path = os.path.join(tmp_path, "t." + ("json" if form == "json" else "bin"))
        x.save(path, form)
        z = T.load(path, form)
        assert_bit_equal(z.data(), xh, form + " file")
    assert not T.from_binary(T.from_slice(xh, [5, 7]).to_binary()).requires_grad()
    with pytest.raises(gpu.TrainStationError):
        x.save(os.path.join(tmp_path, "t.txt"), "yaml")
    with pytest.raises(gpu.serialization.SerializationError, match="Invalid magic"):
        T.from_binary(b"\x00" * 64)
    # a loaded tensor takes part in a step like any other
    w = T.from_json(x.to_json())
    w.mul_tensor(w).sum().backward()
    assert_bit_equal(w.grad_by_value().data(), xh + xh)


def _train(gpu, params, opt, steps, seed):
    rng = np.random.default_rng(seed)
    T = gpu.Tensor
    for _ in range(steps):
        loss = None
        for p in params:
            c = T.from_slice(rng.standard_normal(p.shape().dims).astype(np.float32), p.shape().dims)
            term = p.mul_tensor(c).sum()
            loss = term if loss is None else loss.add_tensor(term)
        loss.backward()
        opt.step(params)
        opt.zero_grad(params)


@pytest.mark.parametrize("form", ["json", "binary"])
@pytest.mark.parametrize("amsgrad", [False, True])
def test_resume_is_identical_to_an_uninterrupted_run(gpu, form, amsgrad):
    T = gpu.Tensor
    rng = np.random.default_rng(4)
    init = [rng.standard_normal(s).astype(np.float32) for s in [(6, 4), (4,), (3, 3, 2)]]
    cfg = gpu.AdamConfig(learning_rate=1e-2, weight_decay=0.01, amsgrad=amsgrad)

    # uninterrupted: 3 + 2 steps (the two legs draw their data from seeds 10 and 11)
    ref = [T.from_slice(a, list(a.shape)).with_requires_grad() for a in init]
    ref_opt = gpu.Adam.with_config(cfg)
    ref_opt.add_parameters(ref)
    _train(gpu, ref, ref_opt, 3, 10)
    _train(gpu, ref, ref_opt, 2, 11)

    # interrupted after 3 steps: parameters and optimizer go through the checkpoint formats
    a = [T.from_slice(x, list(x.shape)).with_requires_grad() for x in init]
    opt = gpu.Adam.with_config(cfg)
    opt.add_parameters(a)
    _train(gpu, a, opt, 3, 10)
    saved_params = [p.to_json() if form == "json" else p.to_binary() for p in a]
    saved_opt = opt.to_json() if form == "json" else opt.to_binary()
    del a, opt
    gpu.clear_gradients()

    b = [(T.from_json(s) if form == "json" else T.from_binary(s)) for s in saved_params]
    assert all(p.requires_grad() for p in b)
    opt2 = gpu.Adam.from_json(saved_opt) if form == "json" else gpu.Adam.from_binary(saved_opt)
    assert opt2.step_count() == 3 and opt2.saved_parameter_count() == 3 and opt2.config.amsgrad == amsgrad
    assert np.float32(opt2.learning_rate()) == np.float32(1e-2)
    opt2.relink_parameters(b)
    assert opt2.saved_parameter_count() == 0
    _train(gpu, b, opt2, 2, 11)
    assert opt2.step_count() == 5
    for p, q in zip(b, ref):
        assert_bit_equal(p.data(), q.data(), "parameters after resume")
        for s, t in zip(opt2.state(p), ref_opt.state(q)):
            assert_bit_equal(s.data(), t.data(), "optimizer state after resume")
    # the resumed optimizer serialises again with its NEW tensor ids, in order
    again = gpu.serialization.adam_from_fields(gpu.serialization.json_to_fields(opt2.to_json()))
    assert again[3] == [p.id() for p in b] and again[2] == 5


def test_relink_errors(gpu):
    """optimizers/adam/mod.rs:396-436."""
    T = gpu.Tensor
    p = [T.ones([2, 2]).with_requires_grad(), T.ones([3]).with_requires_grad()]
    opt = gpu.Adam.new()
    opt.add_parameters(p)
    _train(gpu, p, opt, 1, 0)
    blob = opt.to_binary()
    E = gpu.TrainStationError
    with pytest.raises(E, match="Parameter count mismatch: expected 2 parameters, got 1"):
        gpu.Adam.from_binary(blob).relink_parameters([T.ones([2, 2]).with_requires_grad()])
    with pytest.raises(E, match="Parameter at index 1 must require gradients"):
        gpu.Adam.from_binary(blob).relink_parameters([T.ones([2, 2]).with_requires_grad(), T.ones([3])])
    with pytest.raises(E, match="Shape mismatch for parameter at position 0"):
        gpu.Adam.from_binary(blob).relink_parameters([T.ones([4]).with_requires_grad(), T.ones([3]).with_requires_grad()])
    with pytest.raises(E, match="not loaded from a checkpoint"):
        opt.relink_parameters(p)
    # before relinking, a step on unlinked tensors is refused like any unlinked parameter
    loaded = gpu.Adam.from_binary(blob)
    q = T.ones([2, 2]).with_requires_grad()
    q.sum().backward()
    with pytest.raises(E, match="not linked"):
        loaded.step([q])
