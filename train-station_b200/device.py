"""Device selection, precision mode and allocator statistics (src/device.rs:344-380,
567-580, 728-797; src/cuda/context.rs).  One host thread (or process) drives one GPU."""
from __future__ import annotations

import ctypes as C

from . import _ffi
from ._ffi import check

FP32, TF32, TF32X3 = 0, 1, 2


def cuda_device_count() -> int:
    return int(_ffi.lib().get_cuda_device_count())


def cuda_is_available() -> bool:
    return cuda_device_count() > 0


def set_default_device(index: int) -> None:
    check(_ffi.lib().set_cuda_device(int(index)), "set_cuda_device")
    check(_ffi.lib().cuda_ffi_initialize(), "cuda_ffi_initialize")


def current_device() -> int:
    return int(_ffi.lib().get_current_cuda_device())


def set_matmul_precision(mode: int) -> None:
    check(_ffi.lib().ts_set_matmul_precision(int(mode)), "ts_set_matmul_precision")


def matmul_precision() -> int:
    return int(_ffi.lib().ts_get_matmul_precision())


def set_fusion(enabled: bool) -> None:
    _ffi.lib().ts_set_fusion(1 if enabled else 0)


def synchronize() -> None:
    """Waits for the compute stream and raises if a kernel reported a device-side error."""
    check(_ffi.lib().ts_sync_stream(None), "synchronize")


def allocator_stats() -> dict:
    st = _ffi.AllocatorStats()
    check(_ffi.lib().ts_allocator_get_stats(C.byref(st)), "ts_allocator_get_stats")
    return {k: int(getattr(st, k)) for k, _ in st._fields_}


def release_cached_memory() -> None:
    _ffi.lib().ts_allocator_release_cached()
