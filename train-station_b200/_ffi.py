"""ctypes binding of libtrain_station_b200.so (declared in include/train_station_b200.h).

This is the Python counterpart of the reference's ``extern "C"`` block
(src/cuda/mod.rs:139-208): nothing but pointers and sizes crosses the boundary.
There is no CPU fallback: if the library is missing the import fails.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtrain_station_b200.so")

f32p = C.POINTER(C.c_float)
u64 = C.c_ulonglong
u64p = C.POINTER(u64)
vp = C.c_void_p


class AllocatorStats(C.Structure):
    _fields_ = [("bytes_in_use", u64), ("bytes_reserved", u64), ("peak_bytes_in_use", u64),
                ("driver_allocations", u64), ("cache_hits", u64)]


# name -> (restype, argtypes); kept as a table so tests can check every exported symbol.
SIGNATURES = {
    # 1. the reference's fifteen symbols
    "cuda_ffi_initialize": (C.c_bool, []),
    "cuda_ffi_cleanup": (None, []),
    "get_cuda_device_count": (C.c_int, []),
    "set_cuda_device": (C.c_bool, [C.c_int]),
    "get_current_cuda_device": (C.c_int, []),
    "cuda_malloc": (vp, [u64]),
    "cuda_free": (None, [vp]),
    "cuda_memcpy": (C.c_bool, [vp, vp, u64, C.c_int]),
    "create_cuda_stream": (vp, []),
    "destroy_cuda_stream": (None, [vp]),
    "launch_add_kernel": (C.c_bool, [vp, vp, vp, u64, vp]),
    "launch_sub_kernel": (C.c_bool, [vp, vp, vp, u64, vp]),
    "launch_mul_kernel": (C.c_bool, [vp, vp, vp, u64, vp]),
    "launch_matmul_kernel": (C.c_bool, [vp, vp, vp, u64, u64, u64, vp]),
    # 2. status, streams, allocator
    "ts_last_error": (C.c_char_p, []),
    "ts_sync_stream": (C.c_bool, [vp]),
    "ts_compute_stream": (vp, []),
    "ts_device_error_word": (vp, []),
    "ts_debug_set_gemm_wait_budget": (None, [C.c_longlong]),
    "ts_debug_set_gemm_dynamic": (None, [C.c_int]),
    "ts_host_alloc_pinned": (vp, [u64]),
    "ts_host_free_pinned": (None, [vp]),
    "ts_memcpy_async": (C.c_bool, [vp, vp, u64, C.c_int, vp]),
    "ts_allocator_get_stats": (C.c_bool, [C.POINTER(AllocatorStats)]),
    "ts_allocator_release_cached": (None, []),
    "ts_allocator_set_limit": (None, [u64]),
    "ts_device_memory_info": (C.c_bool, [u64p, u64p]),
    "ts_event_create": (vp, []),
    "ts_event_destroy": (None, [vp]),
    "ts_event_record": (C.c_bool, [vp, vp]),
    "ts_event_elapsed_ms": (C.c_float, [vp, vp]),
    "ts_launch_count": (u64, []),
    "ts_profile_enable": (None, [C.c_int]),
    "ts_profile_collect": (C.c_bool, []),
    "ts_profile_reset": (None, []),
    "ts_profile_get": (C.c_bool, [C.c_int, u64p, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "ts_set_matmul_precision": (C.c_bool, [C.c_int]),
    "ts_get_matmul_precision": (C.c_int, []),
    "ts_set_fusion": (None, [C.c_int]),
    "ts_get_fusion": (C.c_int, []),
    # 3. raw kernel launchers
    "launch_div_kernel": (C.c_bool, [vp, vp, vp, u64, vp]),
    "launch_bias_act_kernel": (C.c_bool, [vp, vp, vp, u64, u64, C.c_int, vp]),
    "launch_relu_kernel": (C.c_bool, [vp, vp, u64, vp]),
    "launch_relu_backward_kernel": (C.c_bool, [vp, vp, vp, u64, vp]),
    "launch_square_kernel": (C.c_bool, [vp, vp, u64, vp]),
    "launch_square_backward_kernel": (C.c_bool, [vp, vp, vp, u64, vp]),
    "launch_mul_backward_kernel": (C.c_bool, [vp, vp, vp, vp, vp, u64, vp]),
    "launch_div_backward_kernel": (C.c_bool, [vp, vp, vp, vp, vp, u64, vp]),
    "launch_binary_broadcast_kernel": (C.c_bool, [C.c_int, vp, u64p, C.c_int, vp, u64p, C.c_int, vp, vp]),
    "launch_binary_broadcast_backward_kernel": (C.c_bool, [C.c_int, vp, u64p, C.c_int, vp, u64p, C.c_int, vp, vp, vp, vp]),
    "launch_scale_kernel": (C.c_bool, [vp, C.c_float, vp, u64, vp]),
    "launch_fill_kernel": (C.c_bool, [vp, C.c_float, u64, vp]),
    "ts_debug_dp_shard_plan": (C.c_int, [u64, C.c_int, C.c_int, C.POINTER(u64), C.POINTER(u64)]),
    "ts_debug_gemm_route": (C.c_int, [u64, u64, u64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(u64)]),
    "launch_fill_from_scalar_kernel": (C.c_bool, [vp, vp, C.c_float, u64, vp]),
    "launch_unary_kernel": (C.c_bool, [C.c_int, vp, vp, u64, C.c_float, vp]),
    "launch_unary_backward_kernel": (C.c_bool, [C.c_int, vp, vp, vp, u64, C.c_float, vp]),
    "launch_permute_kernel": (C.c_bool, [vp, vp, u64p, C.POINTER(C.c_int), C.c_int, vp]),
    "ts_reduce_dims_scratch_elems": (u64, []),
    "launch_reduce_dims_kernel": (C.c_bool, [C.c_int, vp, vp, vp, u64p, C.c_int, u64p, C.c_int, vp, vp]),
    "launch_reduce_dims_backward_kernel": (C.c_bool, [C.c_int, vp, vp, vp, vp, vp, u64p, C.c_int, u64p, C.c_int, C.c_int,
                                                      C.c_float, vp]),
    "launch_softmax_kernel": (C.c_bool, [vp, vp, u64, u64, u64, vp]),
    "launch_softmax_backward_kernel": (C.c_bool, [vp, vp, vp, u64, u64, u64, vp]),
    "ts_reduce_scratch_elems": (u64, []),
    "launch_sum_kernel": (C.c_bool, [vp, vp, u64, C.c_int, vp, vp]),
    "ts_colsum_scratch_elems": (u64, [u64, u64]),
    "launch_colsum_kernel": (C.c_bool, [vp, vp, u64, u64, vp, vp]),
    "launch_colsum_kernel_static_scratch": (C.c_bool, [vp, vp, u64, u64, vp]),
    "launch_relu_backward_colsum_kernel": (C.c_bool, [vp, vp, vp, vp, u64, u64, vp, vp]),
    "launch_gemm_kernel": (C.c_bool, [vp, vp, vp, u64, u64, u64, C.c_int, C.c_int, vp, C.c_int, vp, C.c_int, vp]),
    "launch_gemm_colsum_kernel": (C.c_bool, [vp, vp, vp, u64, u64, u64, C.c_int, C.c_int, vp, C.c_int, vp, C.c_int, vp, vp]),
    "launch_adam_multi_tensor_kernel": (C.c_bool, [C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), u64p,
                                                   C.c_int, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float,
                                                   C.c_float, C.c_float, C.c_float, vp]),
    "launch_adam_amsgrad_multi_tensor_kernel": (C.c_bool, [C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp),
                                                           u64p, C.c_int, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float,
                                                           C.c_float, C.c_float, C.c_float, vp]),
    # 4. tensor / gradtrack / Adam engine
    "ts_tensor_new": (vp, [u64p, C.c_int]),
    "ts_tensor_zeros": (vp, [u64p, C.c_int]),
    "ts_tensor_ones": (vp, [u64p, C.c_int]),
    "ts_tensor_from_slice": (vp, [vp, u64p, C.c_int]),
    "ts_tensor_from_pinned_async": (vp, [vp, u64p, C.c_int]),
    "ts_tensor_randn": (vp, [u64p, C.c_int, u64, C.c_int]),
    "ts_randn_host": (C.c_bool, [vp, u64, u64]),
    "ts_tensor_free": (None, [vp]),
    "ts_tensor_id": (u64, [vp]),
    "ts_tensor_rank": (C.c_int, [vp]),
    "ts_tensor_size": (u64, [vp]),
    "ts_tensor_dims": (C.c_bool, [vp, u64p]),
    "ts_tensor_requires_grad": (C.c_bool, [vp]),
    "ts_tensor_is_contiguous": (C.c_bool, [vp]),
    "ts_tensor_set_requires_grad": (C.c_bool, [vp, C.c_bool]),
    "ts_tensor_data_ptr": (vp, [vp]),
    "ts_tensor_to_host": (C.c_bool, [vp, vp]),
    "ts_tensor_copy_from_host": (C.c_bool, [vp, vp]),
    "ts_tensor_fill": (C.c_bool, [vp, C.c_float]),
    "ts_tensor_matmul": (vp, [vp, vp]),
    "ts_tensor_add_tensor": (vp, [vp, vp]),
    "ts_tensor_sub_tensor": (vp, [vp, vp]),
    "ts_tensor_mul_tensor": (vp, [vp, vp]),
    "ts_tensor_div_tensor": (vp, [vp, vp]),
    "ts_tensor_relu": (vp, [vp]),
    "ts_tensor_pow_scalar": (vp, [vp, C.c_float]),
    "ts_tensor_exp": (vp, [vp]),
    "ts_tensor_log": (vp, [vp]),
    "ts_tensor_sqrt": (vp, [vp]),
    "ts_tensor_tanh": (vp, [vp]),
    "ts_tensor_sigmoid": (vp, [vp]),
    "ts_tensor_leaky_relu": (vp, [vp, C.c_float]),
    "ts_tensor_softmax": (vp, [vp, u64]),
    "ts_tensor_add_scalar": (vp, [vp, C.c_float]),
    "ts_tensor_sub_scalar": (vp, [vp, C.c_float]),
    "ts_tensor_mul_scalar": (vp, [vp, C.c_float]),
    "ts_tensor_div_scalar": (vp, [vp, C.c_float]),
    "ts_tensor_reduce_dims": (vp, [vp, C.c_int, u64p, C.c_int, C.c_int]),
    "ts_tensor_reduce_all": (vp, [vp, C.c_int]),
    "ts_tensor_reshape": (vp, [vp, C.POINTER(C.c_longlong), C.c_int]),
    "ts_tensor_permute": (vp, [vp, u64p, C.c_int]),
    "ts_tensor_transpose": (vp, [vp, u64, u64]),
    "ts_tensor_contiguous": (vp, [vp]),
    "ts_tensor_clone": (vp, [vp]),
    "ts_tensor_cat": (vp, [C.POINTER(vp), C.c_int, u64]),
    "ts_tensor_split_piece": (vp, [vp, u64, u64, u64]),
    "ts_set_domain_checks": (None, [C.c_int]),
    "ts_get_domain_checks": (C.c_int, []),
    "ts_tensor_sum": (vp, [vp]),
    "ts_tensor_mean": (vp, [vp]),
    "ts_tensor_backward": (C.c_bool, [vp, vp]),
    "ts_tensor_grad_by_value": (vp, [vp]),
    "ts_clear_gradients": (None, []),
    "ts_no_grad_push": (None, []),
    "ts_no_grad_pop": (None, []),
    "ts_is_grad_enabled": (C.c_bool, []),
    "ts_tape_len": (u64, []),
    "ts_adam_new": (vp, [C.c_float, C.c_float, C.c_float, C.c_float, C.c_float]),
    "ts_adam_new_amsgrad": (vp, [C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int]),
    "ts_adam_state_v_hat_max": (vp, [vp, vp]),
    "ts_adam_set_step_count": (None, [vp, u64]),
    "ts_adam_param_step": (u64, [vp, vp]),
    "ts_adam_set_param_step": (C.c_bool, [vp, vp, u64]),
    "ts_adam_free": (None, [vp]),
    "ts_adam_add_parameter": (C.c_bool, [vp, vp]),
    "ts_adam_step": (C.c_bool, [vp, C.POINTER(vp), C.c_int, C.c_float]),
    "ts_adam_zero_grad": (None, [vp, C.POINTER(vp), C.c_int]),
    "ts_adam_learning_rate": (C.c_float, [vp]),
    "ts_adam_set_learning_rate": (None, [vp, C.c_float]),
    "ts_adam_step_count": (u64, [vp]),
    "ts_adam_state_m": (vp, [vp, vp]),
    "ts_adam_state_v": (vp, [vp, vp]),
    # 5. data parallelism
    "ts_dp_get_unique_id": (C.c_bool, [C.c_char_p]),
    "ts_dp_init": (C.c_bool, [C.c_char_p, C.c_int, C.c_int]),
    "ts_dp_init_with_timeout": (C.c_bool, [C.c_char_p, C.c_int, C.c_int, C.c_double]),
    "ts_dp_healthy": (C.c_bool, []),
    "ts_dp_install_fake_nccl": (None, [C.c_int]),
    "ts_dp_fake_nccl_aborts": (C.c_int, []),
    "ts_dp_finalize": (None, []),
    "ts_dp_world_size": (C.c_int, []),
    "ts_dp_rank": (C.c_int, []),
    "ts_dp_register_parameters": (C.c_bool, [C.POINTER(vp), C.c_int]),
    "ts_dp_all_reduce": (C.c_bool, [vp, u64]),
}

_lib = None


def lib() -> C.CDLL:
    """Loads the shared library once and attaches the signatures. Raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing. Build it with `python train-station_b200/build.py` "
                "(needs nvcc); this package has no CPU or PyTorch fallback.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class TrainStationError(RuntimeError):
    pass


def last_error() -> str:
    return lib().ts_last_error().decode("utf-8", "replace")


def check(ok, what: str = ""):
    """Raises with the library's error text when a bool/pointer result signals failure."""
    if not ok:
        raise TrainStationError(f"{what}: {last_error()}" if what else last_error())
    return ok
