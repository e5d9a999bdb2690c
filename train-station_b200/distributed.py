"""Data parallelism over the batch: every rank holds all parameters and runs forward and
backward on its contiguous block of batch rows.  During backward each parameter gradient is
summed across ranks on a communication stream as soon as it is final: large tensors by a
reduce-scatter, after which Adam updates only this rank's slice (its moments are sharded) and
the updated parameters are all-gathered while the next forward starts; small tensors by an
all-reduce followed by the same update on every rank.  Adam divides by the world size.  The reference has no multi-device code; this module is the
host side of section 5 of the C ABI.

Rendezvous (who is rank 0, how the NCCL id reaches the others) is the caller's business:
``init_from_torch_distributed`` uses an existing torch.distributed process group of any
backend for that and nothing else."""
from __future__ import annotations

import ctypes as C
from typing import Sequence, Tuple

from . import _ffi
from ._ffi import check, vp
from .tensor import Tensor

UNIQUE_ID_BYTES = 128


def get_unique_id() -> bytes:
    buf = C.create_string_buffer(UNIQUE_ID_BYTES)
    check(_ffi.lib().ts_dp_get_unique_id(buf), "ts_dp_get_unique_id")
    return buf.raw


def init(unique_id: bytes, rank: int, world_size: int, timeout: float | None = None) -> None:
    """Joins the communicator.  Blocks until every rank has called it, but at most `timeout` seconds (default: the
    TS_DP_INIT_TIMEOUT environment variable, else 300): a rank that never joins raises instead of hanging the others."""
    assert len(unique_id) == UNIQUE_ID_BYTES
    buf = C.create_string_buffer(unique_id, UNIQUE_ID_BYTES)
    if timeout is None:
        check(_ffi.lib().ts_dp_init(buf, int(rank), int(world_size)), "ts_dp_init")
    else:
        check(_ffi.lib().ts_dp_init_with_timeout(buf, int(rank), int(world_size), float(timeout)), "ts_dp_init")


def healthy() -> bool:
    """False once NCCL has reported an asynchronous error (a peer that died, a transport fault); the communicator has
    then been aborted and every later collective call fails with a message instead of blocking."""
    return bool(_ffi.lib().ts_dp_healthy())


def exchange_id_through_file(path: str, rank: int, timeout: float = 60.0) -> bytes:
    """The simplest rendezvous: rank 0 creates the NCCL id and publishes it at `path` (written under another name and
    renamed, so a reader never sees half a file); the other ranks wait for the file, at most `timeout` seconds."""
    import os
    import time
    if rank == 0:
        uid = get_unique_id()
        with open(path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(path + ".tmp", path)
        return uid
    t0 = time.monotonic()
    while not os.path.exists(path):
        if time.monotonic() - t0 > timeout:
            raise TimeoutError(f"rank 0 did not publish the NCCL id at {path} within {timeout:g} s")
        time.sleep(0.02)
    with open(path, "rb") as f:
        return f.read()


def init_from_torch_distributed() -> Tuple[int, int]:
    """Bootstraps the library's NCCL communicator through torch.distributed (id broadcast)."""
    import torch
    import torch.distributed as dist
    rank, world = dist.get_rank(), dist.get_world_size()
    ids = [get_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    init(ids[0], rank, world)
    return rank, world


def finalize() -> None:
    _ffi.lib().ts_dp_finalize()


def world_size() -> int:
    return int(_ffi.lib().ts_dp_world_size())


def rank() -> int:
    return int(_ffi.lib().ts_dp_rank())


def register_parameters(params: Sequence[Tensor]) -> None:
    arr = (vp * max(len(params), 1))(*[p._h for p in params])
    check(_ffi.lib().ts_dp_register_parameters(arr, len(params)), "ts_dp_register_parameters")


def shard_rows(n_rows: int, rank_: int, world: int) -> Tuple[int, int]:
    """Contiguous block [start, stop) of batch rows for a rank; the first n_rows % world
    ranks get one extra row (see shard_weight for what unequal shards need)."""
    base, extra = divmod(int(n_rows), int(world))
    start = rank_ * base + min(rank_, extra)
    return start, start + base + (1 if rank_ < extra else 0)


def shard_weight(n_rows: int, rank_: int, world: int) -> float:
    """Weight of a rank's mean loss in the mean over the whole batch, times `world`: rows_local * world / n_rows.

    Each rank's loss is the mean over its own rows and Adam multiplies the summed gradients by 1 / world, which is the
    gradient of the global mean only when every shard has the same number of rows.  With n_rows % world != 0 seed each
    rank's backward with this weight (``loss.backward(Tensor.from_slice([w], [1]))``): the sum over ranks of
    w_r * grad_r, divided by world, is then the gradient of the mean over all rows.  It is 1.0 for equal shards."""
    a, b = shard_rows(n_rows, rank_, world)
    return (b - a) * float(world) / float(n_rows)


def describe() -> str:
    """One line on how gradients are combined, for benchmark records."""
    return ("NCCL on a communication stream, overlapped with backward: large gradients reduce-scattered, Adam on each rank's "
            "slice, parameters all-gathered under the next forward; small gradients all-reduced; Adam scales by 1/world")
