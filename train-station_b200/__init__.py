"""train-station's training-step hot path on NVIDIA B200 (sm_100a).

The names exported here are the ones the reference re-exports at its crate root
(src/lib.rs:276-291) plus ``optimizers`` (src/optimizers/mod.rs).  Everything runs through
libtrain_station_b200.so (include/train_station_b200.h); there is no CPU fallback.

The directory name contains a hyphen, so the package is loaded under the module name
``train_station_b200`` (see ``__graft_entry__.load_package``).
"""
from . import _ffi
from ._ffi import TrainStationError
from .tensor import PinnedBuffer, Shape, Tensor
from .gradtrack import (NoGradTrack, clear_gradients, is_grad_enabled, set_grad_enabled, tape_len,
                        with_no_grad)
from .device import (FP32, TF32, TF32X3, allocator_stats, cuda_device_count, cuda_is_available,
                     current_device, matmul_precision, release_cached_memory, set_default_device,
                     set_fusion, set_matmul_precision, synchronize)
from . import optim as optimizers
from .optim import Adam, AdamConfig, Optimizer
from . import distributed
from . import serialization

__all__ = [
    "Tensor", "Shape", "PinnedBuffer", "TrainStationError", "NoGradTrack", "with_no_grad",
    "is_grad_enabled", "set_grad_enabled", "clear_gradients", "tape_len", "cuda_is_available",
    "cuda_device_count", "set_default_device", "current_device", "set_matmul_precision",
    "matmul_precision", "set_fusion", "synchronize", "allocator_stats", "release_cached_memory",
    "FP32", "TF32", "TF32X3", "optimizers", "Adam", "AdamConfig", "Optimizer", "distributed",
]
