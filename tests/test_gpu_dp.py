"""GPU (2 or more devices): the data-parallel step through the library's own NCCL communicator.

Two child processes, one GPU each, exchange the NCCL id through a file, register the parameters, run
three training steps on their row shards and must end with bit-identical parameters that match a
single-GPU run on the whole batch.  Skipped when fewer than two GPUs are visible.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import os, sys, time
import numpy as np
sys.path.insert(0, {root!r})
import __graft_entry__ as entry
rank, world, out = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
ts = entry.load_package()
ts.set_default_device(rank)
idfile = os.path.join(out, "nccl_id")
if world > 1:
    if rank == 0:
        with open(idfile + ".tmp", "wb") as f:
            f.write(ts.distributed.get_unique_id())
        os.replace(idfile + ".tmp", idfile)
    t0 = time.time()
    while not os.path.exists(idfile):
        assert time.time() - t0 < 60, "rank 0 never published the NCCL id"
        time.sleep(0.05)
    ts.distributed.init(open(idfile, "rb").read(), rank, world)
rng = np.random.default_rng(4)
dims, batch = [256, 512, 384, 128], 512
ws = [rng.uniform(-np.sqrt(6 / dims[i]), np.sqrt(6 / dims[i]), (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
bs = [np.zeros(dims[i + 1], np.float32) for i in range(3)]
x = rng.standard_normal((batch, dims[0]), dtype=np.float32)
t = rng.standard_normal((batch, dims[-1]), dtype=np.float32)
a, b = ts.distributed.shard_rows(batch, rank, world)
T = ts.Tensor
W = [T.from_slice(w, w.shape).with_requires_grad() for w in ws]
B = [T.from_slice(v, v.shape).with_requires_grad() for v in bs]
params = [p for pair in zip(W, B) for p in pair]
opt = ts.Adam.with_learning_rate(1e-3)
opt.add_parameters(params)
if world > 1:
    ts.distributed.register_parameters(params)
    opt.grad_scale = 1.0 / world
X, Tg = T.from_slice(x[a:b], [b - a, dims[0]]), T.from_slice(t[a:b], [b - a, dims[-1]])
losses = []
for step in range(3):
    h = X
    for i in range(3):
        h = h.matmul(W[i]).add_tensor(B[i])
        if i < 2:
            h = h.relu()
    loss = h.sub_tensor(Tg).pow_scalar(2.0).mean()
    loss.backward(None)
    opt.step(params)
    opt.zero_grad(params)
    losses.append(loss.value())
ts.synchronize()
np.savez(os.path.join(out, f"rank{{rank}}_of{{world}}.npz"), *[p.data() for p in params], losses=np.array(losses))
if world > 1:
    ts.distributed.finalize()
"""


def _run(world, out):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.pop("LOCAL_RANK", None)
    procs = [subprocess.Popen([sys.executable, "-c", CHILD.format(root=ROOT), str(r), str(world), str(out)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    for p in procs:
        try:
            log, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        assert p.returncode == 0, log[-3000:]


def test_two_gpu_step_matches_one_gpu(gpu, tmp_path):
    if gpu.cuda_device_count() < 2:
        pytest.skip("needs two GPUs")
    d2, d1 = tmp_path / "w2", tmp_path / "w1"
    d2.mkdir(); d1.mkdir()
    _run(2, d2)
    _run(1, d1)
    r0, r1, s = np.load(d2 / "rank0_of2.npz"), np.load(d2 / "rank1_of2.npz"), np.load(d1 / "rank0_of1.npz")
    keys = [k for k in r0.files if k.startswith("arr_")]
    for k in keys:
        assert np.array_equal(r0[k], r1[k]), f"replicas diverged in {k}"
        np.testing.assert_allclose(r0[k], s[k], rtol=1e-5, atol=3e-6)
    np.testing.assert_allclose((r0["losses"] + r1["losses"]) / 2, s["losses"], rtol=1e-5)
