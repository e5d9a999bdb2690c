"""GPU (2 or more devices): the data-parallel step through the library's own NCCL communicator.

Child processes, one GPU each, exchange the NCCL id through a file, register the parameters and train on their
row shards.  Large gradients are reduce-scattered, Adam runs on each rank's slice and the parameters are
all-gathered; small ones are all-reduced and updated everywhere.  Every scenario must end with bit-identical
replicas that match a single GPU doing the same arithmetic:

  mlp      three steps of a 3-layer MLP (two sharded weight tensors, one replicated, three biases): parameters,
           losses, the last step's gradients and the Adam moments (gathered from their owners)
  accum    two backward() calls per step before zero_grad: sum(G1) + sum(G2), not world * sum(G1) + sum(G2)
  bias1d   a registered bias added to an activation of its own shape (1-D x . W + b): the gradient object is
           shared with the matmul's upstream gradient and must not be summed in place under it
  uneven   batch % world != 0 with each rank's backward seeded by its shard weight
  mlp_tf32 the first scenario with TF32 GEMMs, where the update also maintains the rounded copies the GEMMs read

The single-GPU side runs the ranks' micro-batches one after the other with grad_scale = 1 / 2, which is the same
arithmetic without any communication.  Skipped when fewer than two GPUs are visible.
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
rank, world, out, scenario = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
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
T = ts.Tensor
if scenario.endswith("_tf32"):       # TF32 GEMMs: the update also writes and gathers the TF32-rounded copies of the weights
    ts.set_matmul_precision(ts.TF32)
    scenario = scenario[:-5]
rng = np.random.default_rng(4)
VIRTUAL = 2                      # the single-GPU run plays both ranks, one after the other
ranks_here = [rank] if world > 1 else list(range(VIRTUAL))

if scenario == "bias1d":
    k, n = 96, 65536 * 2         # W and b (same shape as x . W) are both large enough to be sharded
    w0 = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    b0 = (rng.standard_normal(n) * 0.1).astype(np.float32)
    xs = rng.standard_normal((VIRTUAL, k), dtype=np.float32)
    W, B = T.from_slice(w0, w0.shape).with_requires_grad(), T.from_slice(b0, b0.shape).with_requires_grad()
    params = [W, B]
    def losses_for(r):
        y = T.from_slice(xs[r], [k]).matmul(W).add_tensor(B)      # [n] + [n]: Add hands one gradient object to both operands
        return [(y.mul_tensor(y).sum(), None)]
else:
    dims = [256, 512, 384, 128]
    batch = 511 if scenario == "uneven" else 512
    ws = [rng.uniform(-np.sqrt(6 / dims[i]), np.sqrt(6 / dims[i]), (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(dims[i + 1], np.float32) for i in range(3)]
    x = rng.standard_normal((batch, dims[0]), dtype=np.float32)
    t = rng.standard_normal((batch, dims[-1]), dtype=np.float32)
    Ws = [T.from_slice(w, w.shape).with_requires_grad() for w in ws]
    Bs = [T.from_slice(v, v.shape).with_requires_grad() for v in bs]
    params = [p for pair in zip(Ws, Bs) for p in pair]
    def mse(lo, hi):
        h = T.from_slice(x[lo:hi], [hi - lo, dims[0]])
        for i in range(3):
            h = h.matmul(Ws[i]).add_tensor(Bs[i])
            if i < 2:
                h = h.relu()
        return h.sub_tensor(T.from_slice(t[lo:hi], [hi - lo, dims[-1]])).pow_scalar(2.0).mean()
    def losses_for(r):
        a, b = ts.distributed.shard_rows(batch, r, VIRTUAL)
        if scenario == "accum":                                  # two micro-batches, two backward() calls
            mid = (a + b) // 2
            return [(mse(a, mid), None), (mse(mid, b), None)]
        if scenario == "uneven":
            wgt = ts.distributed.shard_weight(batch, r, VIRTUAL)
            return [(mse(a, b), T.from_slice(np.array([wgt], np.float32), [1]))]
        return [(mse(a, b), None)]

opt = ts.Adam.with_learning_rate(1e-3)
opt.add_parameters(params)
if world > 1:
    ts.distributed.register_parameters(params)
opt.grad_scale = 1.0 / VIRTUAL
losses = []
for step in range(3):
    per_rank = []
    for r in ranks_here:
        vals = []
        for loss, seed in losses_for(r):
            loss.backward(seed)
            vals.append(loss)
        per_rank.append(vals)
    grads = [p.grad_by_value().data() for p in params] if step == 2 else None      # a collective read on the last step
    opt.step(params)
    opt.zero_grad(params)
    losses.append([[v.value() for v in vals] for vals in per_rank])
ts.synchronize()
state = {{}}
for i, p in enumerate(params):
    m, v = opt.state(p)[:2]
    state[f"m{{i}}"], state[f"v{{i}}"] = m.data(), v.data()
for i, g in enumerate(grads):
    state[f"g{{i}}"] = g
np.savez(os.path.join(out, f"rank{{rank}}_of{{world}}.npz"), *[p.data() for p in params], losses=np.array(losses), **state)
if world > 1:
    ts.distributed.finalize()
"""


def _run(world, out, scenario, extra_env=None):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **(extra_env or {}))
    env.pop("LOCAL_RANK", None)
    procs = [subprocess.Popen([sys.executable, "-c", CHILD.format(root=ROOT), str(r), str(world), str(out), scenario], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    for p in procs:
        try:
            log, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        assert p.returncode == 0, log[-3000:]


def _compare(d2, d1, rtol, atol):
    r0, r1, s = np.load(d2 / "rank0_of2.npz"), np.load(d2 / "rank1_of2.npz"), np.load(d1 / "rank0_of1.npz")
    keys = [k for k in r0.files if k != "losses"]
    assert any(k.startswith("m") for k in keys) and any(k.startswith("g") for k in keys)
    for k in keys:
        assert np.array_equal(r0[k], r1[k]), f"replicas diverged in {k}"
        np.testing.assert_allclose(r0[k], s[k], rtol=rtol, atol=atol, err_msg=k)
    # rank r's losses are the single GPU's losses for virtual rank r
    both = np.concatenate([r0["losses"], r1["losses"]], axis=1)
    np.testing.assert_allclose(both, s["losses"], rtol=1e-5)


@pytest.mark.parametrize("scenario", ["mlp", "mlp_tf32", "accum", "bias1d", "uneven"])
def test_two_gpu_training_matches_one_gpu(gpu, tmp_path, scenario):
    if gpu.cuda_device_count() < 2:
        pytest.skip("needs two GPUs")
    d2, d1 = tmp_path / "w2", tmp_path / "w1"
    d2.mkdir(); d1.mkdir()
    _run(2, d2, scenario)
    _run(1, d1, scenario)
    # Adam normalises the step: last-bit differences in a summed gradient can move a parameter by a small fraction of lr
    _compare(d2, d1, rtol=1e-5, atol=3e-6)


def test_sharded_and_replicated_updates_agree_bit_for_bit(gpu, tmp_path):
    """The reduce-scatter / sliced Adam / all-gather path against plain all-reduce + replicated Adam (TS_DP_SHARD=0)
    on the same two GPUs: NCCL's ring reduce-scatter and all-reduce may add the two ranks' terms in either order, and
    a two-term float sum does not depend on it, so the results must be identical."""
    if gpu.cuda_device_count() < 2:
        pytest.skip("needs two GPUs")
    da, db = tmp_path / "sharded", tmp_path / "replicated"
    da.mkdir(); db.mkdir()
    _run(2, da, "mlp")
    _run(2, db, "mlp", {"TS_DP_SHARD": "0"})
    a, b = np.load(da / "rank0_of2.npz"), np.load(db / "rank0_of2.npz")
    for k in a.files:
        assert np.array_equal(a[k], b[k]), k
    # TF32 mode: every rank rounding its own copies after the gather (default) against gathering the copies the
    # slices' owners wrote (TS_DP_GATHER_TF32=1): the same values by either route
    dc, dd = tmp_path / "round_locally", tmp_path / "gather_rounded"
    dc.mkdir(); dd.mkdir()
    _run(2, dc, "mlp_tf32")
    _run(2, dd, "mlp_tf32", {"TS_DP_GATHER_TF32": "1"})
    a, b = np.load(dc / "rank0_of2.npz"), np.load(dd / "rank0_of2.npz")
    for k in a.files:
        assert np.array_equal(a[k], b[k]), k
