"""Generates tests/golden/torch_amsgrad.npz.

The reference validates AMSGrad differentially against LibTorch with its usual Adam procedure
(libtorch-validation/src/validation/optimizers/adam.rs:65-160: p[i] = 0.01 i - 0.5, loss = sum(2 p + 1), N steps,
tolerance 1e-4 / 1e-4) in test_adam_with_amsgrad (:1355-1364, shape [3,4], 1 step... default config),
test_adam_amsgrad_state_persistence (:1718-1738, 20 steps, shapes [3,3], [5], [2,2,2]) and
test_adam_amsgrad_vs_regular (:1741-1776, 10 steps, [3,3]).  Replayed here with PyTorch on the CPU:

    python tests/golden/make_torch_amsgrad.py

Note on definitions: the reference keeps the running maximum of the BIAS-CORRECTED second moment
(optimizers/adam/mod.rs:534-541) while PyTorch keeps the maximum of the raw one and corrects afterwards.  With
this procedure's constant gradient both give the same update, which is why the reference's comparison passes;
parity for varying gradients is checked against an f64 evaluation of the reference's definition instead
(tests/test_oracle_variants.py).
"""
import os

import numpy as np
import torch

torch.set_num_threads(1)
out = {}
CASES = [dict(shape=(3, 4), steps=1), dict(shape=(3, 3), steps=20), dict(shape=(5,), steps=20), dict(shape=(2, 2, 2), steps=20),
         dict(shape=(3, 3), steps=10), dict(shape=(7, 5), steps=50, lr=1e-2)]
# (no weight-decay case: it makes the gradient vary from step to step, where the two definitions part by 3e-4)
for i, c in enumerate(CASES):
    n = int(np.prod(c["shape"]))
    lr, wd = c.get("lr", 1e-3), c.get("wd", 0.0)
    p = torch.tensor((np.arange(n, dtype=np.float32) * np.float32(0.01) + np.float32(-0.5)).reshape(c["shape"]), requires_grad=True)
    out[f"case{i}_init"] = p.detach().numpy().copy()
    opt = torch.optim.Adam([p], lr=lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=wd, amsgrad=True)
    for _ in range(c["steps"]):
        (p * 2.0 + 1.0).sum().backward()
        opt.step()
        opt.zero_grad()
    out[f"case{i}_final"] = p.detach().numpy()
    out[f"case{i}_cfg"] = np.array([c["steps"], lr, 0.9, 0.999, 1e-8, wd], dtype=np.float64)
out["count"] = np.array(len(CASES))
path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "torch_amsgrad.npz")
np.savez_compressed(path, **out)
print(path, os.path.getsize(path), "bytes, torch", torch.__version__)
