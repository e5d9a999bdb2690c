/*
 * train_station_b200.h -- C ABI of libtrain_station_b200.so
 *
 * The device side of train-station's training-step hot path (MLP forward, gradtrack
 * backward(), Adam::step) for NVIDIA B200 (sm_100a).  Plain pointers and sizes only.
 * Reference citations are paths inside the train-station repository.
 *
 * Conventions, all inherited from the reference's FFI (src/cuda/cuda_wrapper.h:10-31,
 * src/cuda/cuda_wrapper.cpp:37-94, src/cuda/mod.rs:139-208):
 *   - sizes are counts of f32 elements, never bytes;
 *   - tensors are row-major contiguous f32; matmul is A[m,k] . B[k,n] -> C[m,n];
 *   - bool results: true = success; pointer results: NULL = failure; nothing throws,
 *     nothing aborts; ts_last_error() holds the reason (per host thread);
 *   - `stream == NULL` means the library's per-device compute stream;
 *   - the caller owns every buffer it allocates;
 *   - the current device, the autograd tape and the grad mode are per host thread,
 *     as in the reference (src/device.rs:567, src/gradtrack/engine.rs:697-699), so
 *     one host thread (or process) drives one GPU.
 * There is no CPU fallback: without a usable CUDA device every call fails.
 */
#ifndef TRAIN_STATION_B200_H
#define TRAIN_STATION_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ===================================================================================
 * 1. The reference's fifteen symbols, same names, same meaning
 *    (src/cuda/cuda_wrapper.h:10-31; Rust imports at src/cuda/mod.rs:139-208).
 * =================================================================================== */

/* cuda_wrapper.h:10-11.  Initialises the runtime for this thread's current device. */
bool cuda_ffi_initialize(void);
void cuda_ffi_cleanup(void);

/* cuda_wrapper.h:14-16.  The stub returns 0 devices; this returns the real count. */
int get_cuda_device_count(void);
bool set_cuda_device(int device_id);
int get_current_cuda_device(void);

/* cuda_wrapper.h:19-21.  size in f32 elements; kind 0 = host->device, 1 = device->host
 * (src/cuda/memory.rs:73,95); kind 2 = device->device is an extension.  Memory comes
 * from the caching allocator of the current device.  cuda_memcpy returns after the
 * copy has completed. */
float* cuda_malloc(unsigned long long size);
void cuda_free(float* ptr);
bool cuda_memcpy(float* dst, const float* src, unsigned long long size, int kind);

/* cuda_wrapper.h:24-25 */
void* create_cuda_stream(void);
void destroy_cuda_stream(void* stream);

/* cuda_wrapper.h:28-31.  Device pointers.  launch_matmul_kernel uses the process-wide
 * GEMM precision mode (ts_set_matmul_precision). */
bool launch_add_kernel(const float* a, const float* b, float* result, unsigned long long size, void* stream);
bool launch_sub_kernel(const float* a, const float* b, float* result, unsigned long long size, void* stream);
bool launch_mul_kernel(const float* a, const float* b, float* result, unsigned long long size, void* stream);
bool launch_matmul_kernel(const float* a, const float* b, float* result, unsigned long long m,
                          unsigned long long n, unsigned long long k, void* stream);

/* ===================================================================================
 * 2. Status, streams, allocator
 * =================================================================================== */

/* Pattern of libtorch_get_last_error (libtorch-validation/src/ffi/libtorch_wrapper.h:113-115).
 * Valid until the next failing call on the same thread.  Never NULL. */
const char* ts_last_error(void);
/* Blocks until `stream` (NULL: the compute stream) is idle, then reports any deferred
 * device-side error (for example a bounded wait inside a kernel that gave up). */
bool ts_sync_stream(void* stream);
/* The device word (one int, device memory) in which a kernel records that one of its bounded waits gave up; zero when
 * all is well.  ts_sync_stream copies it back, reports a non-zero value as an error and clears it.  Exposed so that a
 * host can poll or clear it with its own copies, and so that a test can exercise the reporting with a plain write. */
int* ts_device_error_word(void);
/* Cycle budget of the main-loop waits of the next one-CTA tensor-core GEMM launches (negative: back to the default of
 * about two seconds).  For tests of the abort path only: with a budget of 0 the first wait that is not already
 * satisfied gives up, the kernel records an error code (101..104), drains its own copies with the full bound, frees
 * its tensor memory and returns; nothing faults and the context stays usable.  The two-CTA kernel ignores it. */
void ts_debug_set_gemm_wait_budget(long long cycles);
/* Which kernel launch_gemm_kernel would send a product to on a device with sm_count SMs: host arithmetic only, usable
 * without a GPU.  epilogue: bit 0 bias, 1 ReLU, 2 mask, 3 store rounded to TF32, 4 column sums.  Returns
 * 0 FP32 tiled kernel, 1 the same over a split K, 2 / 3 / 4 thin-product kernels (narrow result forward layout, narrow
 * result weight-gradient layout, short reduction), 5 / 6 one-CTA tensor-core kernel on 128 x 128 / 128 x 256 tiles,
 * 7 CTA pairs on 256 x 256 tiles, 8 / 9 one-CTA kernel over a split K on narrow / wide tiles; *splits receives the
 * number of K splits (1 when there is none). */
int ts_debug_gemm_route(unsigned long long m, unsigned long long n, unsigned long long k, int trans_a, int trans_b,
                        int precision, int epilogue, int sm_count, unsigned long long* splits);
/* The two-CTA tensor-core GEMM hands its tiles out from a counter (1, the default) or by a fixed stride per CTA pair (0);
 * negative: back to the default / the TS_GEMM_DYNAMIC environment variable.  For A/B measurements and for tests that
 * run both schedules. */
void ts_debug_set_gemm_dynamic(int enabled);
/* The per-device compute stream as a cudaStream_t, for callers that time with events. */
void* ts_compute_stream(void);
/* Page-locked host memory for uploads that overlap compute (size in f32 elements). */
float* ts_host_alloc_pinned(unsigned long long size);
void ts_host_free_pinned(float* ptr);
/* Asynchronous variant of cuda_memcpy on `stream`; host memory should be pinned. */
bool ts_memcpy_async(float* dst, const float* src, unsigned long long size, int kind, void* stream);

/* Device caching allocator; replaces one std::alloc per tensor
 * (src/tensor/core/allocation.rs:105-118, src/tensor/core/utils.rs:145-171). */
typedef struct ts_allocator_stats {
    unsigned long long bytes_in_use;     /* handed out and not yet freed */
    unsigned long long bytes_reserved;   /* obtained from the driver, in use or cached */
    unsigned long long peak_bytes_in_use;
    unsigned long long driver_allocations; /* calls that reached the driver */
    unsigned long long cache_hits;
} ts_allocator_stats;
bool ts_allocator_get_stats(ts_allocator_stats* out);
void ts_allocator_release_cached(void);              /* return cached blocks to the driver */
void ts_allocator_set_limit(unsigned long long bytes); /* 0 = no limit; for out-of-memory tests */
/* Free and total device memory as the driver reports them (cudaMemGetInfo), in bytes; either pointer may be NULL.
 * A read-only query: lets a caller check from outside the allocator's own counters that a call took nothing. */
bool ts_device_memory_info(unsigned long long* free_bytes, unsigned long long* total_bytes);

/* CUDA events on a stream of this library, for callers that time kernels without any other CUDA binding.
 * ts_event_elapsed_ms waits for `end` and returns the milliseconds between the two records (negative on error). */
void* ts_event_create(void);
void ts_event_destroy(void* event);
bool ts_event_record(void* event, void* stream);
float ts_event_elapsed_ms(void* start, void* end);
/* Kernels launched by this library on this thread's device since the library was loaded. */
unsigned long long ts_launch_count(void);
/* Built-in per-kernel-class timing.  While enabled, every launch is bracketed by two events on its own
 * stream; ts_profile_collect waits for the compute stream and adds the measured durations to the totals.
 * Classes: 0 tensor-core GEMM, 1 FP32 GEMM, 2 elementwise, 3 reductions, 4 Adam.
 * `work` is the algorithmic work of the class in flop (GEMM) or bytes (the others). */
#define TS_PROFILE_CLASSES 5
void ts_profile_enable(int enabled);
bool ts_profile_collect(void);
void ts_profile_reset(void);
bool ts_profile_get(int kernel_class, unsigned long long* launches, double* total_ms, double* work);

/* GEMM precision: 0 = FP32 (FFMA, the reference's summation order),
 * 1 = TF32 tensor cores (tcgen05), 2 = 3xTF32 split on tensor cores (FP32-accurate).
 * Process-wide; the environment variable TS_MATMUL_PRECISION (fp32|tf32|tf32x3) sets the default. */
bool ts_set_matmul_precision(int mode);
int ts_get_matmul_precision(void);
/* Lazy epilogue fusion in the tensor engine (bias add / ReLU / ReLU-mask folded into the
 * producing GEMM).  1 = on (default), 0 = every op launches its own kernel. */
void ts_set_fusion(int enabled);
int ts_get_fusion(void);

/* ===================================================================================
 * 3. Raw kernel launchers beyond the stub set (device pointers, element counts)
 * =================================================================================== */

/* div.rs:347-420: IEEE division, no trap on zero. */
bool launch_div_kernel(const float* a, const float* b, float* result, unsigned long long size, void* stream);
/* Row-broadcast add with optional ReLU: out[i,j] = act(z[i,j] + bias[j])
 * (add.rs:107-146 + broadcasting.rs:299-333 + relu.rs:77-90 in one pass). */
bool launch_bias_act_kernel(const float* z, const float* bias, float* out, unsigned long long rows,
                            unsigned long long cols, int relu, void* stream);
/* relu.rs:175-215: max(x,0) with NaN -> 0 and -0 -> +0. */
bool launch_relu_kernel(const float* x, float* out, unsigned long long size, void* stream);
/* grad_fn/ops/relu.rs:4-16: gi = ref > 0 ? go : 0.  `ref` may be the ReLU input or its
 * output (relu(x) > 0 <=> x > 0). */
bool launch_relu_backward_kernel(const float* ref, const float* grad_out, float* grad_in,
                                 unsigned long long size, void* stream);
/* pow.rs:195-240 with exponent 2 (x*x) and grad_fn/ops/pow.rs:5-27 (go * (2*x)). */
bool launch_square_kernel(const float* x, float* out, unsigned long long size, void* stream);
bool launch_square_backward_kernel(const float* x, const float* grad_out, float* grad_in,
                                   unsigned long long size, void* stream);
/* grad_fn/ops/mul.rs:4-49: ga = go*b, gb = go*a.  Either output may be NULL. */
bool launch_mul_backward_kernel(const float* a, const float* b, const float* grad_out, float* grad_a,
                                float* grad_b, unsigned long long size, void* stream);
/* add / sub / mul / div (op 0..3) of two contiguous operands of different shapes under NumPy-style broadcasting
 * (tensor/ops/broadcasting.rs:100-135; what add_tensor does at add.rs:113-125 by first materialising both stretched
 * operands, broadcasting.rs:299-333).  out is contiguous over the broadcast shape; ranks 1..8; false with
 * "incompatible dimensions at axis N" when the shapes do not broadcast. */
bool launch_binary_broadcast_kernel(int op, const float* a, const unsigned long long* dims_a, int rank_a, const float* b,
                                    const unsigned long long* dims_b, int rank_b, float* out, void* stream);
/* The full-size gradients of a broadcast mul (op 2: go*b, go*a) or div (op 3: go/b, -((go*a)/(b*b))) over the
 * broadcast shape (grad_fn/ops/mul.rs, div.rs with original_shapes); grad_out is contiguous over that shape; the
 * caller sums each back to its operand's shape (grad_fn/utils.rs:23-60).  Either output may be NULL. */
bool launch_binary_broadcast_backward_kernel(int op, const float* a, const unsigned long long* dims_a, int rank_a, const float* b,
                                             const unsigned long long* dims_b, int rank_b, const float* grad_out, float* grad_a,
                                             float* grad_b, void* stream);
/* grad_fn/ops/div.rs:4-49: ga = go/b, gb = -((go*a)/(b*b)).  Either output may be NULL. */
bool launch_div_backward_kernel(const float* a, const float* b, const float* grad_out, float* grad_a,
                                float* grad_b, unsigned long long size, void* stream);
/* out = alpha * x  (negation for grad_fn/ops/sub.rs:26-31 is alpha = -1) */
bool launch_scale_kernel(const float* x, float alpha, float* out, unsigned long long size, void* stream);
/* init/basic.rs:304-360 (fill) */
bool launch_fill_kernel(float* out, float value, unsigned long long size, void* stream);
/* out[i] = scale * (*scalar): backward of sum()/mean() without a host round trip
 * (grad_fn/reductions/sum.rs:4-16, mean.rs:4-30: scale = 1 or 1/numel as f32). */
bool launch_fill_from_scalar_kernel(float* out, const float* scalar, float scale,
                                    unsigned long long size, void* stream);
/* Unary and scalar elementwise ops next to the MLP path, forward and backward, one launcher each.
 *   forward:  out = f(x [, param])
 *   backward: grad_in = grad_out * f'(saved [, param]); `saved` is what the reference's GradFn keeps:
 *             the op's OUTPUT for exp, sqrt, tanh, sigmoid; its INPUT for log, leaky_relu, pow_scalar;
 *             ignored (may be NULL) for the four scalar ops.
 * Reference: tensor/ops/{exp.rs:148-163, log.rs:68-107, sqrt.rs:136-280, tanh.rs:174-190, sigmoid.rs:90-110,
 * leaky_relu.rs:124-330 (param = negative slope), add.rs:450 ff., sub.rs:504 ff., mul.rs:495 ff., div.rs:511-575
 * (param = the scalar), pow.rs:125-160 (param = exponent; 2 -> x*x, 0.5 -> sqrt, else powf)} and
 * gradtrack/grad_fn/ops/{exp,log,sqrt,tanh,sigmoid,leaky_relu,pow,add,sub,mul,div}.rs.
 * Where the reference panics: a zero divisor scalar makes the call return false before any launch;
 * log of x <= 0 (or NaN) still stores the IEEE result and raises the device error word
 * TS_DEVICE_ERROR_LOG_DOMAIN, which the next ts_sync_stream reports as a failure. */
enum ts_unary_op {
    TS_UNARY_EXP = 0, TS_UNARY_LOG = 1, TS_UNARY_SQRT = 2, TS_UNARY_TANH = 3, TS_UNARY_SIGMOID = 4,
    TS_UNARY_LEAKY_RELU = 5, TS_UNARY_ADD_SCALAR = 6, TS_UNARY_SUB_SCALAR = 7, TS_UNARY_MUL_SCALAR = 8,
    TS_UNARY_DIV_SCALAR = 9, TS_UNARY_POW_SCALAR = 10
};
#define TS_DEVICE_ERROR_LOG_DOMAIN 100
bool launch_unary_kernel(int op, const float* x, float* out, unsigned long long size, float param, void* stream);
bool launch_unary_backward_kernel(int op, const float* saved, const float* grad_out, float* grad_in,
                                  unsigned long long size, float param, void* stream);
/* softmax over the middle axis of a contiguous [outer, reduce, inner] tensor (tensor/ops/softmax.rs:110-158:
 * subtract the maximum, exponentiate, multiply by the reciprocal of the sum) and its backward
 * (grad_fn/ops/softmax.rs:4-35: grad_in = y * (grad_out - sum_j grad_out*y)). */
bool launch_softmax_kernel(const float* x, float* out, unsigned long long outer, unsigned long long reduce,
                           unsigned long long inner, void* stream);
bool launch_softmax_backward_kernel(const float* y, const float* grad_out, float* grad_in, unsigned long long outer,
                                    unsigned long long reduce, unsigned long long inner, void* stream);
/* out = in with its axes permuted (output axis i is input axis perm[i]; `dims` are the input's, rank 1..8): the
 * contiguous result of transform/permute.rs:147-190 or transpose.rs:156-200 followed by contiguous.rs:123-160.
 * A batched swap of the last two merged axes runs as a tiled transpose, anything else as a gather. */
bool launch_permute_kernel(const float* in, float* out, const unsigned long long* dims, const int* perm, int rank,
                           void* stream);
/* Reduction of a contiguous tensor over a set of its axes (`axes`: n_axes axis numbers; `dims`: the input's
 * extents, rank 1..8).  out has one element per combination of the kept axes, in their order.
 *   op 0 sum, 1 max, 2 min, 3 sum of squares, 4 sum of squared deviations from aux[output],
 *      5 number of elements equal to aux[output]   (aux is only read by ops 4 and 5)
 * These are the accumulation loops of tensor/reductions/{sum.rs:250-290, max.rs:90-130, min.rs, norm.rs, var.rs,
 * std.rs}; the scaling, square root and two-pass structure on top of them are done by the caller (the engine).
 * `scratch`: ts_reduce_dims_scratch_elems() f32 elements.  Max and min ignore NaN as the reference's comparisons do. */
unsigned long long ts_reduce_dims_scratch_elems(void);
bool launch_reduce_dims_kernel(int op, const float* x, const float* aux, float* out, const unsigned long long* dims,
                               int rank, const unsigned long long* axes, int n_axes, float* scratch, void* stream);
/* The matching backward passes (gradtrack/grad_fn/reductions/*.rs): grad_in has the input's shape, grad_out the
 * output's (or is a single value when grad_out_is_scalar).
 *   mode 0 sum: grad_out[o]                      1 mean: grad_out[o] * scale, scale = 1/count
 *   mode 2 max/min: x == a1[o] ? grad_out[o] / a2[o] : 0   (a1 the extremum, a2 the number of ties)
 *   mode 3 norm: a1[o] > 0 ? x * (grad_out[o] / a1[o]) : 0
 *   mode 4 var: (x - a1[o]) * (grad_out[o] * scale), a1 the mean, scale = 2/count
 *   mode 5 std: a2[o] > 0 ? (x - a1[o]) * (grad_out[o] * scale / a2[o]) : 0, a1 the mean, a2 the std, scale = 1/count */
bool launch_reduce_dims_backward_kernel(int mode, const float* x, const float* a1, const float* a2, const float* grad_out,
                                        float* grad_in, const unsigned long long* dims, int rank,
                                        const unsigned long long* axes, int n_axes, int grad_out_is_scalar, float scale,
                                        void* stream);
/* reductions/sum.rs:80-143 and mean.rs:48-110: out[0] = sum(x) or sum(x)/(f32)size.
 * Deterministic two-level tree (the reference adds sequentially).  `scratch` needs
 * ts_reduce_scratch_elems() f32 elements of device memory. */
unsigned long long ts_reduce_scratch_elems(void);
bool launch_sum_kernel(const float* x, float* out, unsigned long long size, int mean, float* scratch,
                       void* stream);
/* sum_dims(&[0]) of a [rows, cols] matrix (reductions/sum.rs:225-306): out[j] = sum_i g[i,j].
 * `scratch` needs ts_colsum_scratch_elems(rows, cols) elements. */
unsigned long long ts_colsum_scratch_elems(unsigned long long rows, unsigned long long cols);
bool launch_colsum_kernel(const float* g, float* out, unsigned long long rows, unsigned long long cols,
                          float* scratch, void* stream);
/* launch_colsum_kernel for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  A host that lives inside someone else's fixed memory budget, that has already given all
 * device memory away, or that must not enter the driver's allocator on its hot loop (the allocator can
 * synchronise the whole device) has no scratch buffer to hand to launch_colsum_kernel; this variant
 * keeps the partial sums in a 512 KiB array built into the library (held on every GPU that loads the
 * library, until the process exits) and itself calls no allocation routine of any kind (with
 * ts_profile_enable(1) its launches are counted but not bracketed by events, since creating an event
 * allocates).
 *   - Limit: the row splits times `cols` must fit 131,072 elements (65536 x 8192 needs 73,728; the
 *     kernel plans at most four CTAs per SM, so a 148-SM B200 never needs more than 75,776 and the
 *     limit only bites on devices with more SMs); a problem that does not fit is refused with a
 *     message in ts_last_error().
 *   - The library must already be initialised on the current device (cuda_ffi_initialize() allocates
 *     and therefore is not done here); otherwise the call fails with a message.
 *   - The first call on each device looks up the device address of the built-in array; make that
 *     first call before starting any stream capture.
 *   - All calls on a device share the one array, which keeps whatever the last call left in it.  Each
 *     call overwrites every element it later reads, so nothing needs clearing, but two calls that
 *     overlap on the GPU (different streams, no ordering between them) race on it. */
bool launch_colsum_kernel_static_scratch(const float* g, float* out, unsigned long long rows,
                                         unsigned long long cols, void* stream);
/* Fused ReLU backward + bias gradient: grad_in = ref > 0 ? go : 0 and
 * bias_grad[j] = sum_i grad_in[i,j] in one pass over the data. */
bool launch_relu_backward_colsum_kernel(const float* ref, const float* grad_out, float* grad_in,
                                        float* bias_grad, unsigned long long rows,
                                        unsigned long long cols, float* scratch, void* stream);

/* General GEMM: C[m,n] = op(A) . op(B) with op = transpose when trans* != 0.
 * A is stored [m,k] (or [k,m] when trans_a), B is stored [k,n] (or [n,k] when trans_b),
 * all row-major contiguous.  Covers matmul forward (matmul/mod.rs:572-611) and the two
 * backward GEMMs dA = dC . B^T, dB = A^T . dC (grad_fn/ops/matmul.rs:68-80) without the
 * materialised transposes the reference makes.
 * Epilogue (applied in this order, each optional):
 *   bias   != NULL : C[i,j] += bias[j]
 *   relu   != 0    : C = max(C, 0)
 *   mask   != NULL : C[i,j] = mask[i,j] > 0 ? C[i,j] : 0      (mask is [m,n])
 * precision: 0/1/2 as for ts_set_matmul_precision, -1 = the process-wide mode.  Shapes the
 * tensor-core path cannot take (row strides that are not multiples of 4 elements, or very
 * small problems) run on the FP32 kernel in every mode.  In modes 1 and 2 a product with one
 * dimension of at most 16 and long other dimensions (n <= 16 without transposition or with
 * trans_a only; k <= 16 with trans_b only: a 10-class layer, its weight gradient, its input
 * gradient) runs on FFMA kernels laid out along the long dimensions: FP32 products of the
 * operands as given, a fixed but not the reference's summation order. */
bool launch_gemm_kernel(const float* a, const float* b, float* c, unsigned long long m,
                        unsigned long long n, unsigned long long k, int trans_a, int trans_b,
                        const float* bias, int relu, const float* mask, int precision, void* stream);
/* launch_gemm_kernel that also writes colsum_out[j] = sum_i C[i,j] of the stored result (after bias / ReLU / mask): the
 * bias gradient (reductions/sum.rs:225-306 on the pre-activation gradient, grad_fn/ops/add.rs:14-20) without reading
 * the result back.  The tensor-core kernels produce per-32-row partial sums in their epilogue and a second small
 * kernel adds them in row order (deterministic); the FP32 kernel is followed by the ordinary column sum. */
bool launch_gemm_colsum_kernel(const float* a, const float* b, float* c, unsigned long long m, unsigned long long n,
                               unsigned long long k, int trans_a, int trans_b, const float* bias, int relu,
                               const float* mask, int precision, float* colsum_out, void* stream);

/* Fused multi-tensor Adam (optimizers/adam/mod.rs:485-556, 635-1030): one launch updates
 * every tensor.  f1 = 1/bias_correction1, f2 = 1/bias_correction2 as computed on the host
 * (adam/mod.rs:526-531, 793); grad_scale multiplies every gradient first (1.0, or 1/world
 * after a gradient all-reduce).  The four pointer tables are host arrays of device pointers. */
bool launch_adam_multi_tensor_kernel(float* const* params, const float* const* grads, float* const* m,
                                     float* const* v, const unsigned long long* sizes, int n_tensors,
                                     float lr, float beta1, float beta2, float eps, float weight_decay,
                                     float f1, float f2, float grad_scale, void* stream);
/* The AMSGrad branch (adam/mod.rs:534-541, 846-900): v_hat_max[i] = max(v_hat_max[i], v[i]*f2), i.e. the running
 * maximum of the BIAS-CORRECTED second moment, and the update divides by sqrt(v_hat_max) + eps.  The reference
 * creates v_hat_max as a copy of the first v_hat; a zero-filled buffer gives the same values since v_hat >= 0.
 * 36 bytes per parameter. */
bool launch_adam_amsgrad_multi_tensor_kernel(float* const* params, const float* const* grads, float* const* m,
                                             float* const* v, float* const* v_hat_max,
                                             const unsigned long long* sizes, int n_tensors, float lr, float beta1,
                                             float beta2, float eps, float weight_decay, float f1, float f2,
                                             float grad_scale, void* stream);

/* ===================================================================================
 * 4. Tensor, gradtrack and Adam engine: what the reference's Rust API maps onto
 * =================================================================================== */

typedef struct ts_tensor ts_tensor;   /* src/tensor/core/mod.rs:231-299 */
typedef struct ts_adam ts_adam;       /* src/optimizers/adam/mod.rs:201-206 */

/* Constructors (core/utils.rs:121-171, init/basic.rs:137-180,304-360, init/data.rs:227-247).
 * Every returned handle must be released with ts_tensor_free. */
ts_tensor* ts_tensor_new(const unsigned long long* dims, int rank);            /* uninitialised */
ts_tensor* ts_tensor_zeros(const unsigned long long* dims, int rank);
ts_tensor* ts_tensor_ones(const unsigned long long* dims, int rank);
ts_tensor* ts_tensor_from_slice(const float* host, const unsigned long long* dims, int rank);
/* Upload queued on the copy stream; `host` must be pinned and stay valid until the tensor is
 * first used (the compute stream then waits for the copy). */
ts_tensor* ts_tensor_from_pinned_async(const float* host, const unsigned long long* dims, int rank);
/* Tensor::randn(dims, seed) (tensor/init/random.rs:231-236): the reference's own generator, value for value —
 * xorshift64 (13, 7, 17) from state = seed, draws in [0.5, 1), Box-Muller with the host libm (random.rs:473-616) —
 * produced on the host and uploaded.  has_seed == 0 is randn(dims, None): a clock-derived seed, not reproducible. */
ts_tensor* ts_tensor_randn(const unsigned long long* dims, int rank, unsigned long long seed, int has_seed);
/* The same generator into a host buffer; needs no device. */
bool ts_randn_host(float* out, unsigned long long size, unsigned long long seed);
void ts_tensor_free(ts_tensor* t);

unsigned long long ts_tensor_id(const ts_tensor* t);
int ts_tensor_rank(const ts_tensor* t);
unsigned long long ts_tensor_size(const ts_tensor* t);
bool ts_tensor_dims(const ts_tensor* t, unsigned long long* dims_out);
/* False for a transposed / permuted view (ts_tensor_transpose, ts_tensor_permute), which shares its source's storage:
 * tensor/transform/transpose.rs:181-184.  ts_tensor_contiguous makes the copy. */
bool ts_tensor_is_contiguous(const ts_tensor* t);
bool ts_tensor_requires_grad(const ts_tensor* t);
bool ts_tensor_set_requires_grad(ts_tensor* t, bool requires_grad); /* with_requires_grad */
/* Device pointer of the tensor's data (forces any deferred kernel to run). */
float* ts_tensor_data_ptr(ts_tensor* t);
/* Tensor::data() / value(): copies to host after the producing kernels finish. */
bool ts_tensor_to_host(ts_tensor* t, float* host_out);
/* Overwrites the data from host memory (data_mut()); bumps the storage version. */
bool ts_tensor_copy_from_host(ts_tensor* t, const float* host);
bool ts_tensor_fill(ts_tensor* t, float value);

/* Ops.  Each returns a new tensor and records a GradFn when grad mode is on and an input
 * requires grad (template: tensor/ops/relu.rs:77-90). */
/* matmul/mod.rs:263-310: 1-D and 2-D operands in every pairing; with an operand of rank > 2 the batched product of
 * mod.rs:634-760 (both operands at least 2-D, batch axes broadcast from the right, a leading batch axis of extent 1
 * squeezed away when one operand is 2-D; errors "Batched matmul requires at least 2D tensors", "Inner dimensions
 * must match for batched matmul: K vs K'", "Cannot broadcast dimensions A and B"). */
ts_tensor* ts_tensor_matmul(ts_tensor* a, ts_tensor* b);
ts_tensor* ts_tensor_add_tensor(ts_tensor* a, ts_tensor* b);   /* add.rs:107-146 (+ broadcast) */
ts_tensor* ts_tensor_sub_tensor(ts_tensor* a, ts_tensor* b);   /* sub.rs:121-160 */
ts_tensor* ts_tensor_mul_tensor(ts_tensor* a, ts_tensor* b);   /* mul.rs:94-135 */
ts_tensor* ts_tensor_div_tensor(ts_tensor* a, ts_tensor* b);   /* div.rs:109-150 */
ts_tensor* ts_tensor_relu(ts_tensor* x);                       /* relu.rs:77-90 */
ts_tensor* ts_tensor_pow_scalar(ts_tensor* x, float exponent); /* pow.rs:79-160 */
/* The unary and scalar ops of the reference's example networks; each records the GradFn the reference records
 * (what it saves is listed at launch_unary_backward_kernel). */
ts_tensor* ts_tensor_exp(ts_tensor* x);                         /* exp.rs:96-110 */
ts_tensor* ts_tensor_log(ts_tensor* x);                         /* log.rs:68-140; x <= 0 fails, see ts_set_domain_checks */
ts_tensor* ts_tensor_sqrt(ts_tensor* x);                        /* sqrt.rs:99-214 */
ts_tensor* ts_tensor_tanh(ts_tensor* x);                        /* tanh.rs:140-190 */
ts_tensor* ts_tensor_sigmoid(ts_tensor* x);                     /* sigmoid.rs:90-125 */
ts_tensor* ts_tensor_leaky_relu(ts_tensor* x, float negative_slope); /* leaky_relu.rs:80-330 */
ts_tensor* ts_tensor_softmax(ts_tensor* x, unsigned long long dim);  /* softmax.rs:110-175 */
ts_tensor* ts_tensor_add_scalar(ts_tensor* x, float scalar);    /* add.rs:236-250 */
ts_tensor* ts_tensor_sub_scalar(ts_tensor* x, float scalar);    /* sub.rs:264-278 */
ts_tensor* ts_tensor_mul_scalar(ts_tensor* x, float scalar);    /* mul.rs:239-255 */
ts_tensor* ts_tensor_div_scalar(ts_tensor* x, float scalar);    /* div.rs:247-265; a zero scalar fails */
/* Shape and layout.  reshape shares the storage (transform/reshape.rs:139-215; one -1 is inferred); flatten, squeeze
 * and unsqueeze are reshapes in the reference too (flatten.rs:124, squeeze.rs:184, unsqueeze.rs:218).  permute and
 * transpose (permute.rs:147-190, transpose.rs:156-200; t() swaps the last two axes, :283-291) return the permuted
 * contiguous copy, since tensors here carry no strides; transpose(d, d) is a detached copy as in the reference.
 * contiguous (contiguous.rs:123-137) is a copy connected to its source in the graph. */
ts_tensor* ts_tensor_reshape(ts_tensor* x, const long long* new_shape, int rank);
ts_tensor* ts_tensor_permute(ts_tensor* x, const unsigned long long* order, int n);
ts_tensor* ts_tensor_transpose(ts_tensor* x, unsigned long long dim0, unsigned long long dim1);
ts_tensor* ts_tensor_contiguous(ts_tensor* x);
ts_tensor* ts_tensor_clone(ts_tensor* x);   /* Clone (tensor/core/mod.rs:344-378): same values, no gradient history */
/* Tensor::cat (tensor/transform/cat.rs:110-230) and one piece of split / split_with_sizes (split.rs:159-330:
 * elements [start, start + length) of axis dim); strided device-to-device copies, GradFn::Cat / GradFn::Split. */
ts_tensor* ts_tensor_cat(ts_tensor* const* tensors, int n, unsigned long long dim);
ts_tensor* ts_tensor_split_piece(ts_tensor* x, unsigned long long dim, unsigned long long start, unsigned long long length);
/* Reductions over axes (tensor/reductions/*.rs): sum_dims, mean_dims, max_dims, min_dims, norm_dims, var_dims,
 * std_dims with `keepdim`, and the whole-tensor max / min / norm / var / std (result [1]).  Variance and standard
 * deviation are the population ones (divide by the count), as in the reference. */
enum ts_reduce_kind {
    TS_REDUCE_SUM = 0, TS_REDUCE_MEAN = 1, TS_REDUCE_MAX = 2, TS_REDUCE_MIN = 3, TS_REDUCE_NORM = 4,
    TS_REDUCE_VAR = 5, TS_REDUCE_STD = 6
};
ts_tensor* ts_tensor_reduce_dims(ts_tensor* x, int kind, const unsigned long long* dims, int n_dims, int keepdim);
ts_tensor* ts_tensor_reduce_all(ts_tensor* x, int kind);
/* The reference panics inside log() when an element is <= 0.  1 (default): ts_tensor_log waits for its kernel and
 * fails at the call, like the panic.  0: no wait; the failure is reported by the next ts_sync_stream. */
void ts_set_domain_checks(int at_the_call);
int ts_get_domain_checks(void);
ts_tensor* ts_tensor_sum(ts_tensor* x);                        /* reductions/sum.rs:80-143 */
ts_tensor* ts_tensor_mean(ts_tensor* x);                       /* reductions/mean.rs:48-110 */

/* gradtrack (gradtrack/engine.rs:962-1047, core/utils.rs:492-534,634-636). */
bool ts_tensor_backward(ts_tensor* t, ts_tensor* grad_output /* NULL = ones */);
ts_tensor* ts_tensor_grad_by_value(const ts_tensor* t);        /* NULL if no gradient */
void ts_clear_gradients(void);                                 /* engine.rs:812-816 */
void ts_no_grad_push(void);                                    /* NoGradTrack::new */
void ts_no_grad_pop(void);                                     /* drop(NoGradTrack) */
bool ts_is_grad_enabled(void);
unsigned long long ts_tape_len(void);                          /* recorded operations */

/* Adam (optimizers/adam/mod.rs:91-117 config defaults 1e-3, 0.9, 0.999, 1e-8, 0, false). */
ts_adam* ts_adam_new(float lr, float beta1, float beta2, float eps, float weight_decay);
/* The same with AdamConfig::amsgrad (adam/mod.rs:103): each parameter also gets a v_hat_max state. */
ts_adam* ts_adam_new_amsgrad(float lr, float beta1, float beta2, float eps, float weight_decay, int amsgrad);
void ts_adam_free(ts_adam* opt);
bool ts_adam_add_parameter(ts_adam* opt, const ts_tensor* p);  /* adam/mod.rs:287-320 */
/* Optimizer::step (adam/mod.rs:1036-1044): parameters without a gradient are skipped with
 * a message in ts_last_error(), as the reference prints and skips.  grad_scale as above. */
bool ts_adam_step(ts_adam* opt, ts_tensor* const* params, int n, float grad_scale);
/* Optimizer::zero_grad (adam/mod.rs:1061-1068): clears the whole tape of this thread. */
void ts_adam_zero_grad(ts_adam* opt, ts_tensor* const* params, int n);
float ts_adam_learning_rate(const ts_adam* opt);
void ts_adam_set_learning_rate(ts_adam* opt, float lr);
unsigned long long ts_adam_step_count(const ts_adam* opt);
/* Device copies of the moment estimates, for parity checks (NULL if p is not linked). */
ts_tensor* ts_adam_state_m(const ts_adam* opt, const ts_tensor* p);
ts_tensor* ts_adam_state_v(const ts_adam* opt, const ts_tensor* p);
ts_tensor* ts_adam_state_v_hat_max(const ts_adam* opt, const ts_tensor* p);   /* NULL unless amsgrad */
/* Counters for checkpoints (optimizers/adam/serialization.rs:692-752; the moments are written through the views above). */
void ts_adam_set_step_count(ts_adam* opt, unsigned long long n);
unsigned long long ts_adam_param_step(const ts_adam* opt, const ts_tensor* p);
bool ts_adam_set_param_step(ts_adam* opt, const ts_tensor* p, unsigned long long n);

/* ===================================================================================
 * 5. Data parallelism: batch rows sharded over GPUs, one NCCL all-reduce of the parameter
 *    gradients before Adam.  No counterpart in the reference (it is single-device).
 * =================================================================================== */
#define TS_DP_UNIQUE_ID_BYTES 128
/* Rank 0 creates the id; the caller broadcasts the bytes to the other ranks by any means. */
bool ts_dp_get_unique_id(unsigned char id_out[TS_DP_UNIQUE_ID_BYTES]);
bool ts_dp_init(const unsigned char id[TS_DP_UNIQUE_ID_BYTES], int rank, int world_size);
/* ts_dp_init waits at most TS_DP_INIT_TIMEOUT seconds (environment, default 300; 0 = for ever) for the other ranks:
 * a rank that never joins costs a bounded wait and an error, not a hang. */
bool ts_dp_init_with_timeout(const unsigned char id[TS_DP_UNIQUE_ID_BYTES], int rank, int world_size, double timeout_seconds);
/* How the data-parallel path would split a registered parameter of n elements over `world` ranks: returns 1 and the
 * rank's slice [*lo, *lo + *count) when its gradient is reduce-scattered and updated slice by slice (large tensors
 * whose size is a multiple of 8 * world, so that every slice starts on Adam's 8-element boundary), 0 with [0, n) when it
 * is all-reduced and updated whole.  Host arithmetic only: usable without a GPU and without a communicator. */
int ts_debug_dp_shard_plan(unsigned long long n, int world, int rank, unsigned long long* lo, unsigned long long* count);
/* False once the communicator has reported an asynchronous error (a peer that died, a transport fault).  The
 * communicator is then aborted, so that no later call can block on it, and every later collective call fails with a
 * message.  Checked by the library at every collective it enqueues; a host may also poll it between steps. */
bool ts_dp_healthy(void);
/* Test hooks for the two above, usable without a GPU: mode 0..3 replaces NCCL by an in-process stand-in that moves no
 * data (0: every call succeeds, 1: the rendezvous never completes, 2: collectives return an error, 3: an asynchronous
 * remote error is reported); a negative mode removes it.  ts_dp_fake_nccl_aborts counts the stand-in's aborts. */
void ts_dp_install_fake_nccl(int mode);
int ts_dp_fake_nccl_aborts(void);
void ts_dp_finalize(void);
int ts_dp_world_size(void);   /* 1 when not initialised */
int ts_dp_rank(void);
/* Registers the tensors whose gradients are to be summed across ranks.  During
 * ts_tensor_backward each one's all-reduce is enqueued on a communication stream as soon
 * as its gradient is final, overlapping the rest of backward; ts_adam_step waits for it. */
bool ts_dp_register_parameters(ts_tensor* const* params, int n);
/* Sums `size` elements in place across ranks on the communication stream and makes the
 * compute stream wait for the result. */
bool ts_dp_all_reduce(float* data, unsigned long long size);

#ifdef __cplusplus
}
#endif
#endif /* TRAIN_STATION_B200_H */
