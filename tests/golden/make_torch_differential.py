"""Generates tests/golden/torch_differential.npz.

The reference validates itself differentially against LibTorch
(libtorch-validation/src/validation/**): the same formula-generated data goes through both
libraries and results must agree to (rtol, atol) = (1e-6..1e-5, 1e-8) for ops and
(1e-4, 1e-4) for Adam.  LibTorch is PyTorch's C++ core, so replaying those procedures with
PyTorch on the CPU reproduces the reference's own oracle.  Run from the repository root:

    python tests/golden/make_torch_differential.py

Procedures replayed (paths inside ewhinery8/train-station):
  matmul forward + gradients, data left[i] = 0.1 i + 1, right[i] = 0.2 i + 0.5, grad = ones
      libtorch-validation/src/validation/tensor/ops/matmul.rs:186-260, 325-343, shapes :395-408
  linear layer x = 0.1 i, w = 0.05 i, b = 0.02 i, loss = sum(x.w + b)
      libtorch-validation/src/validation/tensor/broadcasting_gradients.rs:272-350
  relu on 0.2 i - 1, gradient of its sum
      libtorch-validation/src/validation/tensor/ops/relu.rs:6-25
  Adam: p[i] = 0.01 i - 0.5, loss = sum(2 p + 1), N steps
      libtorch-validation/src/validation/optimizers/adam.rs:65-160
"""
import os

import numpy as np
import torch

torch.set_num_threads(1)
torch.backends.cuda.matmul.allow_tf32 = False
out = {}


def seq(n, a, b):
    return (np.arange(n, dtype=np.float32) * np.float32(a) + np.float32(b)).astype(np.float32)


# --- matmul
MATMUL_SHAPES = [((2, 3), (3, 2)), ((3, 4), (4, 5)), ((1, 3), (3, 1)), ((5, 1), (1, 5)), ((32, 32), (32, 32)),
                 ((64, 48), (48, 56))]
for i, (ls, rs) in enumerate(MATMUL_SHAPES):
    l = torch.tensor(seq(ls[0] * ls[1], 0.1, 1.0).reshape(ls), requires_grad=True)
    r = torch.tensor(seq(rs[0] * rs[1], 0.2, 0.5).reshape(rs), requires_grad=True)
    y = l @ r
    y.backward(torch.ones_like(y))
    out[f"matmul{i}_left"] = l.detach().numpy()
    out[f"matmul{i}_right"] = r.detach().numpy()
    out[f"matmul{i}_out"] = y.detach().numpy()
    out[f"matmul{i}_grad_left"] = l.grad.numpy()
    out[f"matmul{i}_grad_right"] = r.grad.numpy()
out["matmul_count"] = np.array(len(MATMUL_SHAPES))

# --- linear layer with bias broadcast
for i, (batch, fin, fout) in enumerate([(2, 3, 4), (4, 8, 3), (16, 32, 10)]):
    x = torch.tensor(seq(batch * fin, 0.1, 0.0).reshape(batch, fin), requires_grad=True)
    w = torch.tensor(seq(fin * fout, 0.05, 0.0).reshape(fin, fout), requires_grad=True)
    b = torch.tensor(seq(fout, 0.02, 0.0), requires_grad=True)
    y = x @ w + b
    y.sum().backward()
    for k, v in dict(x=x, w=w, b=b).items():
        out[f"linear{i}_{k}"] = v.detach().numpy()
        out[f"linear{i}_grad_{k}"] = v.grad.numpy()
    out[f"linear{i}_out"] = y.detach().numpy()
out["linear_count"] = np.array(3)

# --- relu
x = torch.tensor(seq(24, 0.2, -1.0).reshape(4, 6), requires_grad=True)
y = torch.relu(x)
y.sum().backward()
out["relu_x"], out["relu_out"], out["relu_grad"] = x.detach().numpy(), y.detach().numpy(), x.grad.numpy()

# --- Adam
ADAM_CASES = [dict(shape=(4,), steps=1, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.0),
              dict(shape=(3, 5), steps=5, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.0),
              dict(shape=(10, 10), steps=20, lr=1e-2, b1=0.8, b2=0.99, eps=1e-6, wd=0.0),
              dict(shape=(7,), steps=10, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01)]
for i, c in enumerate(ADAM_CASES):
    n = int(np.prod(c["shape"]))
    p = torch.tensor(seq(n, 0.01, -0.5).reshape(c["shape"]), requires_grad=True)
    out[f"adam{i}_init"] = p.detach().numpy().copy()
    opt = torch.optim.Adam([p], lr=c["lr"], betas=(c["b1"], c["b2"]), eps=c["eps"], weight_decay=c["wd"])
    for _ in range(c["steps"]):
        loss = (p * 2.0 + 1.0).sum()
        loss.backward()
        opt.step()
        opt.zero_grad()
    out[f"adam{i}_final"] = p.detach().numpy()
    out[f"adam{i}_cfg"] = np.array([c["steps"], c["lr"], c["b1"], c["b2"], c["eps"], c["wd"]], dtype=np.float64)
out["adam_count"] = np.array(len(ADAM_CASES))

path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "torch_differential.npz")
np.savez_compressed(path, **out)
print(path, os.path.getsize(path), "bytes, torch", torch.__version__)
