// Generated from train_station_b200.h by make_rust_bindings.py: do not edit by hand.
// The C ABI of libtrain_station_b200.so as a Rust `extern "C"` block.  Sizes are element counts, not bytes;
// a null `stream` is the library's compute stream; `bool` results are success flags and ts_last_error() holds
// the message of the last failure on the calling thread; handles are owned by the caller and released with
// ts_tensor_free / ts_adam_free.
#![allow(non_camel_case_types, dead_code)]
use std::os::raw::{c_char, c_void};

#[repr(C)]
pub struct TsTensor { _private: [u8; 0] }

#[repr(C)]
pub struct TsAdam { _private: [u8; 0] }

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct TsAllocatorStats {
    pub bytes_in_use: u64,
    pub bytes_reserved: u64,
    pub peak_bytes_in_use: u64,
    pub driver_allocations: u64,
    pub cache_hits: u64,
}

pub const TS_PROFILE_CLASSES: i32 = 5;
pub const TS_DEVICE_ERROR_LOG_DOMAIN: i32 = 100;
pub const TS_DP_UNIQUE_ID_BYTES: usize = 128;
pub const TS_UNARY_EXP: i32 = 0;
pub const TS_UNARY_LOG: i32 = 1;
pub const TS_UNARY_SQRT: i32 = 2;
pub const TS_UNARY_TANH: i32 = 3;
pub const TS_UNARY_SIGMOID: i32 = 4;
pub const TS_UNARY_LEAKY_RELU: i32 = 5;
pub const TS_UNARY_ADD_SCALAR: i32 = 6;
pub const TS_UNARY_SUB_SCALAR: i32 = 7;
pub const TS_UNARY_MUL_SCALAR: i32 = 8;
pub const TS_UNARY_DIV_SCALAR: i32 = 9;
pub const TS_UNARY_POW_SCALAR: i32 = 10;
pub const TS_REDUCE_SUM: i32 = 0;
pub const TS_REDUCE_MEAN: i32 = 1;
pub const TS_REDUCE_MAX: i32 = 2;
pub const TS_REDUCE_MIN: i32 = 3;
pub const TS_REDUCE_NORM: i32 = 4;
pub const TS_REDUCE_VAR: i32 = 5;
pub const TS_REDUCE_STD: i32 = 6;

#[link(name = "train_station_b200")]
extern "C" {
    pub fn cuda_ffi_initialize() -> bool;
    pub fn cuda_ffi_cleanup();
    pub fn get_cuda_device_count() -> i32;
    pub fn set_cuda_device(device_id: i32) -> bool;
    pub fn get_current_cuda_device() -> i32;
    pub fn cuda_malloc(size: u64) -> *mut f32;
    pub fn cuda_free(ptr: *mut f32);
    pub fn cuda_memcpy(dst: *mut f32, src: *const f32, size: u64, kind: i32) -> bool;
    pub fn create_cuda_stream() -> *mut c_void;
    pub fn destroy_cuda_stream(stream: *mut c_void);
    pub fn launch_add_kernel(a: *const f32, b: *const f32, result: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_sub_kernel(a: *const f32, b: *const f32, result: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_mul_kernel(a: *const f32, b: *const f32, result: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_matmul_kernel(a: *const f32, b: *const f32, result: *mut f32, m: u64, n: u64, k: u64, stream: *mut c_void) -> bool;
    pub fn ts_last_error() -> *const c_char;
    pub fn ts_sync_stream(stream: *mut c_void) -> bool;
    pub fn ts_device_error_word() -> *mut i32;
    pub fn ts_debug_set_gemm_wait_budget(cycles: i64);
    pub fn ts_debug_gemm_route(m: u64, n: u64, k: u64, trans_a: i32, trans_b: i32, precision: i32, epilogue: i32, sm_count: i32, splits: *mut u64) -> i32;
    pub fn ts_debug_set_gemm_dynamic(enabled: i32);
    pub fn ts_compute_stream() -> *mut c_void;
    pub fn ts_host_alloc_pinned(size: u64) -> *mut f32;
    pub fn ts_host_free_pinned(ptr: *mut f32);
    pub fn ts_memcpy_async(dst: *mut f32, src: *const f32, size: u64, kind: i32, stream: *mut c_void) -> bool;
    pub fn ts_allocator_get_stats(out: *mut TsAllocatorStats) -> bool;
    pub fn ts_allocator_release_cached();
    pub fn ts_allocator_set_limit(bytes: u64);
    pub fn ts_device_memory_info(free_bytes: *mut u64, total_bytes: *mut u64) -> bool;
    pub fn ts_event_create() -> *mut c_void;
    pub fn ts_event_destroy(event: *mut c_void);
    pub fn ts_event_record(event: *mut c_void, stream: *mut c_void) -> bool;
    pub fn ts_event_elapsed_ms(start: *mut c_void, end: *mut c_void) -> f32;
    pub fn ts_launch_count() -> u64;
    pub fn ts_profile_enable(enabled: i32);
    pub fn ts_profile_collect() -> bool;
    pub fn ts_profile_reset();
    pub fn ts_profile_get(kernel_class: i32, launches: *mut u64, total_ms: *mut f64, work: *mut f64) -> bool;
    pub fn ts_set_matmul_precision(mode: i32) -> bool;
    pub fn ts_get_matmul_precision() -> i32;
    pub fn ts_set_fusion(enabled: i32);
    pub fn ts_get_fusion() -> i32;
    pub fn launch_div_kernel(a: *const f32, b: *const f32, result: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_bias_act_kernel(z: *const f32, bias: *const f32, out: *mut f32, rows: u64, cols: u64, relu: i32, stream: *mut c_void) -> bool;
    pub fn launch_relu_kernel(x: *const f32, out: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_relu_backward_kernel(ref_: *const f32, grad_out: *const f32, grad_in: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_square_kernel(x: *const f32, out: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_square_backward_kernel(x: *const f32, grad_out: *const f32, grad_in: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_mul_backward_kernel(a: *const f32, b: *const f32, grad_out: *const f32, grad_a: *mut f32, grad_b: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_binary_broadcast_kernel(op: i32, a: *const f32, dims_a: *const u64, rank_a: i32, b: *const f32, dims_b: *const u64, rank_b: i32, out: *mut f32, stream: *mut c_void) -> bool;
    pub fn launch_binary_broadcast_backward_kernel(op: i32, a: *const f32, dims_a: *const u64, rank_a: i32, b: *const f32, dims_b: *const u64, rank_b: i32, grad_out: *const f32, grad_a: *mut f32, grad_b: *mut f32, stream: *mut c_void) -> bool;
    pub fn launch_div_backward_kernel(a: *const f32, b: *const f32, grad_out: *const f32, grad_a: *mut f32, grad_b: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_scale_kernel(x: *const f32, alpha: f32, out: *mut f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_fill_kernel(out: *mut f32, value: f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_fill_from_scalar_kernel(out: *mut f32, scalar: *const f32, scale: f32, size: u64, stream: *mut c_void) -> bool;
    pub fn launch_unary_kernel(op: i32, x: *const f32, out: *mut f32, size: u64, param: f32, stream: *mut c_void) -> bool;
    pub fn launch_unary_backward_kernel(op: i32, saved: *const f32, grad_out: *const f32, grad_in: *mut f32, size: u64, param: f32, stream: *mut c_void) -> bool;
    pub fn launch_softmax_kernel(x: *const f32, out: *mut f32, outer: u64, reduce: u64, inner: u64, stream: *mut c_void) -> bool;
    pub fn launch_softmax_backward_kernel(y: *const f32, grad_out: *const f32, grad_in: *mut f32, outer: u64, reduce: u64, inner: u64, stream: *mut c_void) -> bool;
    pub fn launch_permute_kernel(in_: *const f32, out: *mut f32, dims: *const u64, perm: *const i32, rank: i32, stream: *mut c_void) -> bool;
    pub fn ts_reduce_dims_scratch_elems() -> u64;
    pub fn launch_reduce_dims_kernel(op: i32, x: *const f32, aux: *const f32, out: *mut f32, dims: *const u64, rank: i32, axes: *const u64, n_axes: i32, scratch: *mut f32, stream: *mut c_void) -> bool;
    pub fn launch_reduce_dims_backward_kernel(mode: i32, x: *const f32, a1: *const f32, a2: *const f32, grad_out: *const f32, grad_in: *mut f32, dims: *const u64, rank: i32, axes: *const u64, n_axes: i32, grad_out_is_scalar: i32, scale: f32, stream: *mut c_void) -> bool;
    pub fn ts_reduce_scratch_elems() -> u64;
    pub fn launch_sum_kernel(x: *const f32, out: *mut f32, size: u64, mean: i32, scratch: *mut f32, stream: *mut c_void) -> bool;
    pub fn ts_colsum_scratch_elems(rows: u64, cols: u64) -> u64;
    pub fn launch_colsum_kernel(g: *const f32, out: *mut f32, rows: u64, cols: u64, scratch: *mut f32, stream: *mut c_void) -> bool;
    pub fn launch_colsum_kernel_static_scratch(g: *const f32, out: *mut f32, rows: u64, cols: u64, stream: *mut c_void) -> bool;
    pub fn launch_relu_backward_colsum_kernel(ref_: *const f32, grad_out: *const f32, grad_in: *mut f32, bias_grad: *mut f32, rows: u64, cols: u64, scratch: *mut f32, stream: *mut c_void) -> bool;
    pub fn launch_gemm_kernel(a: *const f32, b: *const f32, c: *mut f32, m: u64, n: u64, k: u64, trans_a: i32, trans_b: i32, bias: *const f32, relu: i32, mask: *const f32, precision: i32, stream: *mut c_void) -> bool;
    pub fn launch_gemm_colsum_kernel(a: *const f32, b: *const f32, c: *mut f32, m: u64, n: u64, k: u64, trans_a: i32, trans_b: i32, bias: *const f32, relu: i32, mask: *const f32, precision: i32, colsum_out: *mut f32, stream: *mut c_void) -> bool;
    pub fn launch_adam_multi_tensor_kernel(params: *const *mut f32, grads: *const *const f32, m: *const *mut f32, v: *const *mut f32, sizes: *const u64, n_tensors: i32, lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32, f1: f32, f2: f32, grad_scale: f32, stream: *mut c_void) -> bool;
    pub fn launch_adam_amsgrad_multi_tensor_kernel(params: *const *mut f32, grads: *const *const f32, m: *const *mut f32, v: *const *mut f32, v_hat_max: *const *mut f32, sizes: *const u64, n_tensors: i32, lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32, f1: f32, f2: f32, grad_scale: f32, stream: *mut c_void) -> bool;
    pub fn ts_tensor_new(dims: *const u64, rank: i32) -> *mut TsTensor;
    pub fn ts_tensor_zeros(dims: *const u64, rank: i32) -> *mut TsTensor;
    pub fn ts_tensor_ones(dims: *const u64, rank: i32) -> *mut TsTensor;
    pub fn ts_tensor_from_slice(host: *const f32, dims: *const u64, rank: i32) -> *mut TsTensor;
    pub fn ts_tensor_from_pinned_async(host: *const f32, dims: *const u64, rank: i32) -> *mut TsTensor;
    pub fn ts_tensor_randn(dims: *const u64, rank: i32, seed: u64, has_seed: i32) -> *mut TsTensor;
    pub fn ts_randn_host(out: *mut f32, size: u64, seed: u64) -> bool;
    pub fn ts_tensor_free(t: *mut TsTensor);
    pub fn ts_tensor_id(t: *const TsTensor) -> u64;
    pub fn ts_tensor_rank(t: *const TsTensor) -> i32;
    pub fn ts_tensor_size(t: *const TsTensor) -> u64;
    pub fn ts_tensor_dims(t: *const TsTensor, dims_out: *mut u64) -> bool;
    pub fn ts_tensor_is_contiguous(t: *const TsTensor) -> bool;
    pub fn ts_tensor_requires_grad(t: *const TsTensor) -> bool;
    pub fn ts_tensor_set_requires_grad(t: *mut TsTensor, requires_grad: bool) -> bool;
    pub fn ts_tensor_data_ptr(t: *mut TsTensor) -> *mut f32;
    pub fn ts_tensor_to_host(t: *mut TsTensor, host_out: *mut f32) -> bool;
    pub fn ts_tensor_copy_from_host(t: *mut TsTensor, host: *const f32) -> bool;
    pub fn ts_tensor_fill(t: *mut TsTensor, value: f32) -> bool;
    pub fn ts_tensor_matmul(a: *mut TsTensor, b: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_add_tensor(a: *mut TsTensor, b: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_sub_tensor(a: *mut TsTensor, b: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_mul_tensor(a: *mut TsTensor, b: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_div_tensor(a: *mut TsTensor, b: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_relu(x: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_pow_scalar(x: *mut TsTensor, exponent: f32) -> *mut TsTensor;
    pub fn ts_tensor_exp(x: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_log(x: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_sqrt(x: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_tanh(x: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_sigmoid(x: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_leaky_relu(x: *mut TsTensor, negative_slope: f32) -> *mut TsTensor;
    pub fn ts_tensor_softmax(x: *mut TsTensor, dim: u64) -> *mut TsTensor;
    pub fn ts_tensor_add_scalar(x: *mut TsTensor, scalar: f32) -> *mut TsTensor;
    pub fn ts_tensor_sub_scalar(x: *mut TsTensor, scalar: f32) -> *mut TsTensor;
    pub fn ts_tensor_mul_scalar(x: *mut TsTensor, scalar: f32) -> *mut TsTensor;
    pub fn ts_tensor_div_scalar(x: *mut TsTensor, scalar: f32) -> *mut TsTensor;
    pub fn ts_tensor_reshape(x: *mut TsTensor, new_shape: *const i64, rank: i32) -> *mut TsTensor;
    pub fn ts_tensor_permute(x: *mut TsTensor, order: *const u64, n: i32) -> *mut TsTensor;
    pub fn ts_tensor_transpose(x: *mut TsTensor, dim0: u64, dim1: u64) -> *mut TsTensor;
    pub fn ts_tensor_contiguous(x: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_clone(x: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_cat(tensors: *const *mut TsTensor, n: i32, dim: u64) -> *mut TsTensor;
    pub fn ts_tensor_split_piece(x: *mut TsTensor, dim: u64, start: u64, length: u64) -> *mut TsTensor;
    pub fn ts_tensor_reduce_dims(x: *mut TsTensor, kind: i32, dims: *const u64, n_dims: i32, keepdim: i32) -> *mut TsTensor;
    pub fn ts_tensor_reduce_all(x: *mut TsTensor, kind: i32) -> *mut TsTensor;
    pub fn ts_set_domain_checks(at_the_call: i32);
    pub fn ts_get_domain_checks() -> i32;
    pub fn ts_tensor_sum(x: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_mean(x: *mut TsTensor) -> *mut TsTensor;
    pub fn ts_tensor_backward(t: *mut TsTensor, grad_output: *mut TsTensor) -> bool;
    pub fn ts_tensor_grad_by_value(t: *const TsTensor) -> *mut TsTensor;
    pub fn ts_clear_gradients();
    pub fn ts_no_grad_push();
    pub fn ts_no_grad_pop();
    pub fn ts_is_grad_enabled() -> bool;
    pub fn ts_tape_len() -> u64;
    pub fn ts_adam_new(lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32) -> *mut TsAdam;
    pub fn ts_adam_new_amsgrad(lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32, amsgrad: i32) -> *mut TsAdam;
    pub fn ts_adam_free(opt: *mut TsAdam);
    pub fn ts_adam_add_parameter(opt: *mut TsAdam, p: *const TsTensor) -> bool;
    pub fn ts_adam_step(opt: *mut TsAdam, params: *const *mut TsTensor, n: i32, grad_scale: f32) -> bool;
    pub fn ts_adam_zero_grad(opt: *mut TsAdam, params: *const *mut TsTensor, n: i32);
    pub fn ts_adam_learning_rate(opt: *const TsAdam) -> f32;
    pub fn ts_adam_set_learning_rate(opt: *mut TsAdam, lr: f32);
    pub fn ts_adam_step_count(opt: *const TsAdam) -> u64;
    pub fn ts_adam_state_m(opt: *const TsAdam, p: *const TsTensor) -> *mut TsTensor;
    pub fn ts_adam_state_v(opt: *const TsAdam, p: *const TsTensor) -> *mut TsTensor;
    pub fn ts_adam_state_v_hat_max(opt: *const TsAdam, p: *const TsTensor) -> *mut TsTensor;
    pub fn ts_adam_set_step_count(opt: *mut TsAdam, n: u64);
    pub fn ts_adam_param_step(opt: *const TsAdam, p: *const TsTensor) -> u64;
    pub fn ts_adam_set_param_step(opt: *mut TsAdam, p: *const TsTensor, n: u64) -> bool;
    pub fn ts_dp_get_unique_id(id_out: *mut u8) -> bool;
    pub fn ts_dp_init(id: *const u8, rank: i32, world_size: i32) -> bool;
    pub fn ts_dp_init_with_timeout(id: *const u8, rank: i32, world_size: i32, timeout_seconds: f64) -> bool;
    pub fn ts_debug_dp_shard_plan(n: u64, world: i32, rank: i32, lo: *mut u64, count: *mut u64) -> i32;
    pub fn ts_dp_healthy() -> bool;
    pub fn ts_dp_install_fake_nccl(mode: i32);
    pub fn ts_dp_fake_nccl_aborts() -> i32;
    pub fn ts_dp_finalize();
    pub fn ts_dp_world_size() -> i32;
    pub fn ts_dp_rank() -> i32;
    pub fn ts_dp_register_parameters(params: *const *mut TsTensor, n: i32) -> bool;
    pub fn ts_dp_all_reduce(data: *mut f32, size: u64) -> bool;
}
