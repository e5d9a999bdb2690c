"""CPU: host-side logic of the data-parallel path, with two gloo ranks standing in for two GPUs.

What is checked is the arithmetic contract the device path implements (distributed.py, ts_dp_* in
engine.cu): contiguous row shards, per-rank mean loss, SUM all-reduce of the parameter gradients,
Adam reading gradients scaled by 1/world, identical parameters on every rank afterwards and equal
(to rounding) to the single-process step on the whole batch.  The per-rank math here is done by the
CPU oracle; the GPU tests cover the kernels themselves.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_rows_partitions_the_batch(ts):
    sr = ts.distributed.shard_rows
    for n, w in [(65536, 1), (65536, 8), (10, 4), (7, 8), (0, 2)]:
        blocks = [sr(n, r, w) for r in range(w)]
        assert blocks[0][0] == 0 and blocks[-1][1] == n
        assert all(blocks[i][1] == blocks[i + 1][0] for i in range(w - 1))
        sizes = [b - a for a, b in blocks]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    assert sr(65536, 3, 8) == (24576, 32768)


def test_unique_id_buffer_size(ts):
    assert ts.distributed.UNIQUE_ID_BYTES == 128


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    ora = entry.load_oracle()
    ts = entry.load_package()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    # the rendezvous pattern bench.py uses for the NCCL id: rank 0 makes 128 bytes, everyone receives them
    ids = [bytes(range(128)) if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    assert ids[0] == bytes(range(128))

    rng = np.random.default_rng(4)          # same seed on every rank: identical parameters and global batch
    dims, batch = [24, 40, 40, 12], 64
    ws = [rng.uniform(-np.sqrt(6 / dims[i]), np.sqrt(6 / dims[i]), (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(dims[i + 1], np.float32) for i in range(3)]
    x = rng.standard_normal((batch, dims[0]), dtype=np.float32)
    t = rng.standard_normal((batch, dims[-1]), dtype=np.float32)
    a, b = ts.distributed.shard_rows(batch, rank, world)
    st = ora.MlpState(ws, bs)
    losses = []
    for step in range(1, 4):
        r = ora.mlp_step(st, x[a:b], t[a:b], loss_kind=ora.LOSS_MSE, do_adam=False)   # local mean loss, local gradients
        losses.append(float(r["loss"]))
        for g in st.gw + st.gb:
            tg = torch.from_numpy(g)
            dist.all_reduce(tg, op=dist.ReduceOp.SUM)                                   # in place, like ncclAllReduce
        scale = np.float32(1.0 / world)
        for l in range(3):                                                              # Adam with grad_scale = 1/world
            ora.adam_update(st.w[l].reshape(-1), (st.gw[l] * scale).reshape(-1), st.mw[l].reshape(-1), st.vw[l].reshape(-1), step)
            ora.adam_update(st.b[l], st.gb[l] * scale, st.mb[l], st.vb[l], step)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), *st.w, *st.b, losses=np.array(losses))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_data_parallel_step_matches_single_process(ora, tmp_path):
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    keys = [k for k in r0.files if k.startswith("arr_")]
    for k in keys:                                    # replicas stay bit-identical
        assert np.array_equal(r0[k], r1[k]), k
    # single process on the whole batch
    rng = np.random.default_rng(4)
    dims, batch = [24, 40, 40, 12], 64
    ws = [rng.uniform(-np.sqrt(6 / dims[i]), np.sqrt(6 / dims[i]), (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(dims[i + 1], np.float32) for i in range(3)]
    x = rng.standard_normal((batch, dims[0]), dtype=np.float32)
    t = rng.standard_normal((batch, dims[-1]), dtype=np.float32)
    st = ora.MlpState(ws, bs)
    full_losses = [float(ora.mlp_step(st, x, t, loss_kind=ora.LOSS_MSE)["loss"]) for _ in range(3)]
    single = st.w + st.b
    for i, k in enumerate(keys):
        # Adam normalises by sqrt(v): last-bit differences in the summed gradient move a parameter by ~1e-3 * lr
        np.testing.assert_allclose(r0[k], single[i], rtol=1e-5, atol=3e-6)
    # the global mean loss is the mean of the per-rank mean losses (equal shard sizes)
    np.testing.assert_allclose((r0["losses"] + r1["losses"]) / 2, full_losses, rtol=1e-5)


def test_shard_weight_makes_unequal_shards_add_up_to_the_global_mean(ts, ora):
    """batch % world != 0: each rank's loss is the mean over its own rows, so a plain sum / world over-weights the
    rows of the shorter shards.  Seeding each rank's backward with shard_weight() repairs that."""
    rng = np.random.default_rng(11)
    dims, batch, world = [12, 20, 6], 50, 4
    ws = [rng.standard_normal((dims[i], dims[i + 1])) for i in range(2)]
    bs = [rng.standard_normal(dims[i + 1]) for i in range(2)]
    x, t = rng.standard_normal((batch, dims[0])), rng.standard_normal((batch, dims[-1]))
    full = ora.mlp_step_f64(ws, bs, x, t)
    shards = [ts.distributed.shard_rows(batch, r, world) for r in range(world)]
    assert [b - a for a, b in shards] == [13, 13, 12, 12] and shards[0][0] == 0 and shards[-1][1] == batch
    weights = [ts.distributed.shard_weight(batch, r, world) for r in range(world)]
    assert abs(sum(weights) - world) < 1e-12
    plain = [np.zeros_like(w) for w in ws]
    weighted = [np.zeros_like(w) for w in ws]
    for (a, b), wgt in zip(shards, weights):
        g = ora.mlp_step_f64(ws, bs, x[a:b], t[a:b])["gw"]
        for l in range(2):
            plain[l] += g[l] / world
            weighted[l] += wgt * g[l] / world
    for l in range(2):
        np.testing.assert_allclose(weighted[l], full["gw"][l], rtol=1e-12, atol=1e-14)
        assert np.abs(plain[l] - full["gw"][l]).max() > 1e-4 * np.abs(full["gw"][l]).max()   # the unweighted sum is measurably off
    assert ts.distributed.shard_weight(64, 1, 4) == 1.0


def test_data_parallel_shard_plan_for_every_world_size(ts):
    """Which slice of a parameter a rank owns (host arithmetic, `ts_debug_dp_shard_plan`): the C5 tensors at 1, 2, 4 and
    8 ranks, the slices tile the tensor, every slice starts on a multiple of 8 elements, small or indivisible tensors
    stay whole."""
    import ctypes as C
    lib = ts._ffi.lib()

    def plan(n, world, rank):
        lo, cnt = C.c_ulonglong(0), C.c_ulonglong(0)
        sliced = lib.ts_debug_dp_shard_plan(n, world, rank, C.byref(lo), C.byref(cnt))
        return bool(sliced), lo.value, cnt.value

    weights = [4096 * 8192, 8192 * 8192, 8192 * 4096]
    biases = [8192, 8192, 4096]
    for world in (2, 4, 8):
        for n in weights:
            covered = 0
            for rank in range(world):
                sliced, lo, cnt = plan(n, world, rank)
                assert sliced and lo == covered and lo % 8 == 0 and cnt == n // world
                covered += cnt
            assert covered == n
        for n in biases:
            assert plan(n, world, world - 1) == (False, 0, n), "a few thousand elements: all-reduced, updated on every rank"
    assert plan(weights[0], 1, 0) == (False, 0, weights[0])
    assert plan((1 << 20) + 8, 8, 3) == (False, 0, (1 << 20) + 8), "not a multiple of 8 * world: kept whole"
    assert plan(3 * (1 << 16), 3, 2) == (True, 2 * (1 << 16), 1 << 16)
