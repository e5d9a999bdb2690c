"""Generates tests/golden/torch_unary.npz.

The reference validates its unary / scalar ops and softmax differentially against LibTorch
(libtorch-validation/src/validation/tensor/ops/*.rs) at (rtol, atol) = (1e-6, 1e-8) for exp,
log and sqrt and the default (1e-5, 1e-8) for the others.  LibTorch is PyTorch's C++ core,
so replaying those procedures with PyTorch on the CPU reproduces the reference's own oracle.
Run from the repository root:

    python tests/golden/make_torch_unary.py

Procedures replayed (paths inside ewhinery8/train-station, data[i] = a*i + b):
  exp      fwd 0.1 i - 2.5; grad 0.05 i - 1.0 (ones upstream); chain z = exp(x)*x + exp(x), 0.01 i - 0.5
           ops/exp.rs:13-150, shapes :161-169
  log      fwd 0.1 i + 0.5; grad 0.05 i + 0.2                                   ops/log.rs:11-86
  sqrt     fwd 0.1 i + 0.01; grad 0.03 i + 0.2; chain 0.01 i + 0.5             ops/sqrt.rs:10-130
  tanh, sigmoid, leaky_relu(0.1)   fwd and grad on 0.2 i - 1.0, shapes [3], [2,3], [2,3,4]
           ops/tanh.rs:6-90, ops/sigmoid.rs:6-90, ops/leaky_relu.rs:6-100
  softmax  fwd 0.1 i - 0.5; grad of sum(softmax(x)) on (i mod 7) - 3; ([2,3], dim 1), ([2,3,4], dim 2)
           ops/softmax.rs:6-90
  pow_scalar e in {0.5, 1, 2, 3}: fwd 0.1 i + 0.1; grad 0.05 i + 0.2 on [2,3]  ops/pow.rs:6-66, :167-178
"""
import os

import numpy as np
import torch

torch.set_num_threads(1)
out = {}


def seq(shape, a, b):
    n = int(np.prod(shape))
    return (np.arange(n, dtype=np.float32) * np.float32(a) + np.float32(b)).astype(np.float32).reshape(shape)


def fwd_and_grad(tag, fn, shape, fwd_ab, grad_ab):
    x = torch.tensor(seq(shape, *fwd_ab))
    out[f"{tag}_x"] = x.numpy()
    out[f"{tag}_y"] = fn(x).numpy()
    g = torch.tensor(seq(shape, *grad_ab), requires_grad=True)
    y = fn(g)
    y.backward(torch.ones_like(y))
    out[f"{tag}_gx"] = g.detach().numpy()
    out[f"{tag}_grad"] = g.grad.numpy()


SHAPES_A = [(1,), (3,), (2, 2), (1, 4), (2, 3), (1, 1, 3), (100, 100)]
SHAPES_B = [(3,), (2, 3), (2, 3, 4)]
cases = []
for i, s in enumerate(SHAPES_A):
    fwd_and_grad(f"exp{i}", torch.exp, s, (0.1, -2.5), (0.05, -1.0)); cases.append(f"exp{i}")
    sl = s if s != (100, 100) else (50, 50)
    fwd_and_grad(f"log{i}", torch.log, sl, (0.1, 0.5), (0.05, 0.2)); cases.append(f"log{i}")
    fwd_and_grad(f"sqrt{i}", torch.sqrt, s, (0.1, 0.01), (0.03, 0.2)); cases.append(f"sqrt{i}")
for i, s in enumerate(SHAPES_B):
    fwd_and_grad(f"tanh{i}", torch.tanh, s, (0.2, -1.0), (0.2, -1.0)); cases.append(f"tanh{i}")
    fwd_and_grad(f"sigmoid{i}", torch.sigmoid, s, (0.2, -1.0), (0.2, -1.0)); cases.append(f"sigmoid{i}")
    fwd_and_grad(f"leaky_relu{i}", lambda t: torch.nn.functional.leaky_relu(t, 0.1), s, (0.2, -1.0), (0.2, -1.0))
    cases.append(f"leaky_relu{i}")
for e in (0.5, 1.0, 2.0, 3.0):
    tag = f"pow_scalar_{e}"
    fwd_and_grad(tag, lambda t, e=e: torch.pow(t, e), (2, 3), (0.1, 0.1), (0.05, 0.2)); cases.append(tag)
out["cases"] = np.array(cases)

# chains
for i, s in enumerate([(3,), (2, 3), (10, 10)]):
    x = torch.tensor(seq(s, 0.01, -0.5), requires_grad=True)
    ex = torch.exp(x)
    z = ex * x + ex
    z.backward(torch.ones_like(z))
    out[f"exp_chain{i}_x"], out[f"exp_chain{i}_grad"] = x.detach().numpy(), x.grad.numpy()
out["exp_chain_count"] = np.array(3)

# softmax
for i, (s, dim) in enumerate([((2, 3), 1), ((2, 3, 4), 2), ((2, 3, 4), 1), ((4, 5), 0)]):
    x = torch.tensor(seq(s, 0.1, -0.5))
    out[f"softmax{i}_x"], out[f"softmax{i}_y"], out[f"softmax{i}_dim"] = x.numpy(), torch.softmax(x, dim).numpy(), np.array(dim)
    n = int(np.prod(s))
    g = torch.tensor(((np.arange(n) % 7).astype(np.float32) - 3.0).reshape(s), requires_grad=True)
    torch.softmax(g, dim).sum().backward()
    out[f"softmax{i}_gx"], out[f"softmax{i}_grad"] = g.detach().numpy(), g.grad.numpy()
    # a non-trivial upstream as well (the sum's gradient of ones makes the exact answer zero)
    g2 = torch.tensor(((np.arange(n) % 7).astype(np.float32) - 3.0).reshape(s), requires_grad=True)
    up = torch.tensor(seq(s, 0.3, -1.0))
    (torch.softmax(g2, dim) * up).sum().backward()
    out[f"softmax{i}_up"], out[f"softmax{i}_grad_up"] = up.numpy(), g2.grad.numpy()
out["softmax_count"] = np.array(4)

path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "torch_unary.npz")
np.savez_compressed(path, **out)
print(path, os.path.getsize(path), "bytes, torch", torch.__version__)
