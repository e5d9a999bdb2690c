// Elementwise forward and backward kernels: HBM-bound, 128-bit vectorised, grid sized in
// multiples of the SM count.  Every arithmetic step is a single IEEE-rounded operation
// written with explicit intrinsics so that nvcc cannot contract a*b+c into an FMA: the
// reference (Rust, no fast-math) rounds each operation separately.
#include "../../include/train_station_b200.h"
#include "common.h"

namespace ts {
namespace k {

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;        // float4 loads in flight per thread per input
constexpr int kCtasPerSm = 8;

inline int grid_for(size_t n_vec, int sm_count) {
    size_t per_cta = (size_t)kThreads * kUnroll;
    size_t want = (n_vec + per_cta - 1) / per_cta;
    size_t cap = (size_t)sm_count * kCtasPerSm;
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// F::apply(in[NIN], out[NOUT]) on scalars; the same functor serves the vector body and the tail.
template <int NIN, int NOUT>
struct Ptrs {
    const float* in[NIN ? NIN : 1];
    float* out[NOUT];   // an output may be null (skipped)
};

template <int NIN, int NOUT, class F>
__global__ void __launch_bounds__(kThreads) ew_vec_kernel(Ptrs<NIN, NOUT> p, size_t n_vec, size_t n, F f) {
    grid_dependency_sync();
    const size_t stride = (size_t)gridDim.x * kThreads * kUnroll;
    for (size_t base = (size_t)blockIdx.x * kThreads * kUnroll + threadIdx.x; base < n_vec; base += stride) {
        float4 vin[kUnroll][NIN ? NIN : 1];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            size_t i = base + (size_t)u * kThreads;
            if (i < n_vec) {
#pragma unroll
                for (int a = 0; a < NIN; ++a) vin[u][a] = __ldcs(reinterpret_cast<const float4*>(p.in[a]) + i);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            size_t i = base + (size_t)u * kThreads;
            if (i < n_vec) {
                float xi[4][NIN ? NIN : 1], xo[4][NOUT];
#pragma unroll
                for (int a = 0; a < NIN; ++a) {
                    xi[0][a] = vin[u][a].x; xi[1][a] = vin[u][a].y; xi[2][a] = vin[u][a].z; xi[3][a] = vin[u][a].w;
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) f.apply(xi[e], xo[e]);
#pragma unroll
                for (int o = 0; o < NOUT; ++o) {
                    if (p.out[o]) {
                        float4 v = make_float4(xo[0][o], xo[1][o], xo[2][o], xo[3][o]);
                        __stcs(reinterpret_cast<float4*>(p.out[o]) + i, v);
                    }
                }
            }
        }
    }
    // scalar tail (n mod 4 elements), done by the first CTA
    if (blockIdx.x == 0) {
        size_t i = n_vec * 4 + threadIdx.x;
        if (i < n) {
            float xi[NIN ? NIN : 1], xo[NOUT];
#pragma unroll
            for (int a = 0; a < NIN; ++a) xi[a] = p.in[a][i];
            f.apply(xi, xo);
#pragma unroll
            for (int o = 0; o < NOUT; ++o)
                if (p.out[o]) p.out[o][i] = xo[o];
        }
    }
}

// Fallback for pointers that are not 16-byte aligned (sub-buffers handed in through the raw ABI).
template <int NIN, int NOUT, class F>
__global__ void __launch_bounds__(kThreads) ew_scalar_kernel(Ptrs<NIN, NOUT> p, size_t n, F f) {
    grid_dependency_sync();
    const size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        float xi[NIN == 0 ? 1 : NIN], xo[NOUT];
#pragma unroll
        for (int a = 0; a < NIN; ++a) xi[a] = p.in[a][i];
        f.apply(xi, xo);
#pragma unroll
        for (int o = 0; o < NOUT; ++o)
            if (p.out[o]) p.out[o][i] = xo[o];
    }
}

template <int NIN, int NOUT, class F>
bool launch_ew(Ptrs<NIN, NOUT> p, size_t n, F f, cudaStream_t s) {
    if (n == 0) return true;
    DeviceCtx* c = ctx();
    if (!c) return false;
    for (int a = 0; a < NIN; ++a)
        if (!p.in[a]) { set_error("elementwise kernel: null input pointer"); return false; }
    bool any_out = false, al = true;
    for (int a = 0; a < NIN; ++a) al = al && aligned16(p.in[a]);
    for (int o = 0; o < NOUT; ++o) { any_out = any_out || p.out[o]; al = al && aligned16(p.out[o]); }
    if (!any_out) { set_error("elementwise kernel: null output pointer"); return false; }
    int n_arrays = NIN;
    for (int o = 0; o < NOUT; ++o) n_arrays += p.out[o] ? 1 : 0;
    ProfScope prof(kProfElementwise, s, 4.0 * (double)n * n_arrays);
    if (al) {
        size_t n_vec = n / 4;
        launch_dep(ew_vec_kernel<NIN, NOUT, F>, dim3(grid_for(n_vec, c->sm_count)), dim3(kThreads), 0, s, p, n_vec, n, f);
    } else {
        launch_dep(ew_scalar_kernel<NIN, NOUT, F>, dim3(grid_for((n + 3) / 4, c->sm_count)), dim3(kThreads), 0, s, p, n, f);
    }
    return cuda_ok(cudaGetLastError(), "elementwise launch");
}

// ---- functors: one rounded IEEE operation per arithmetic step -------------------------
struct AddF { __device__ void apply(const float* x, float* o) const { o[0] = __fadd_rn(x[0], x[1]); } };
struct SubF { __device__ void apply(const float* x, float* o) const { o[0] = __fsub_rn(x[0], x[1]); } };
struct MulF { __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(x[0], x[1]); } };
struct DivF { __device__ void apply(const float* x, float* o) const { o[0] = __fdiv_rn(x[0], x[1]); } };
// max(x,0) as the AVX2 maxps does it: NaN -> 0, -0 -> +0 (relu.rs:175-215).
struct ReluF { __device__ void apply(const float* x, float* o) const { o[0] = x[0] > 0.0f ? x[0] : 0.0f; } };
struct ReluBwdF { __device__ void apply(const float* x, float* o) const { o[0] = x[0] > 0.0f ? x[1] : 0.0f; } };
struct SquareF { __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(x[0], x[0]); } };
// go * (2 * x): grad_fn/ops/pow.rs:5-27 with exponent 2
struct SquareBwdF { __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(x[1], __fmul_rn(2.0f, x[0])); } };
// inputs a, b, go -> go*b, go*a
struct MulBwdF { __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(x[2], x[1]); o[1] = __fmul_rn(x[2], x[0]); } };
// inputs a, b, go -> go/b, -((go*a)/(b*b))
struct DivBwdF {
    __device__ void apply(const float* x, float* o) const {
        o[0] = __fdiv_rn(x[2], x[1]);
        o[1] = -__fdiv_rn(__fmul_rn(x[2], x[0]), __fmul_rn(x[1], x[1]));
    }
};
struct ScaleF { float alpha; __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(alpha, x[0]); } };
struct FillF { float v; __device__ void apply(const float*, float* o) const { o[0] = v; } };
struct FillFromScalarF {
    const float* scalar; float scale;
    __device__ void apply(const float*, float* o) const { o[0] = __fmul_rn(scale, __ldg(scalar)); }
};
struct AddScalarBcastF {
    const float* scalar;
    __device__ void apply(const float* x, float* o) const { o[0] = __fadd_rn(x[0], __ldg(scalar)); }
};
// round to the nearest TF32 value, ties away from zero; the low 13 mantissa bits of the result are zero
struct RoundTf32F {
    __device__ void apply(const float* x, float* o) const {
        uint32_t r;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x[0]));
        o[0] = __uint_as_float(r);
    }
};
// x = hi + lo with both parts exact in TF32 (the subtraction is exact in FP32: hi shares x's leading bits)
struct SplitTf32F {
    __device__ void apply(const float* x, float* o) const {
        uint32_t h, l;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x[0]));
        const float hi = __uint_as_float(h);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(__fsub_rn(x[0], hi)));
        o[0] = hi;
        o[1] = __uint_as_float(l);
    }
};
// inputs y, t: ((inv_n * upstream) * (2 * (y - t))): ReduceMean -> PowScalar(2) -> Sub chain
// (grad_fn/reductions/mean.rs:10-19, grad_fn/ops/pow.rs:5-27, grad_fn/ops/sub.rs:26-31).
// round_tf32: the gradient goes straight into tensor-core GEMMs in TF32 mode, so it is stored rounded to the nearest
// TF32 value (what those GEMMs would otherwise get from a separate rounding pass).
struct MseGradF {
    const float* upstream; float inv_n; bool round_tf32;
    __device__ void apply(const float* x, float* o) const {
        float sc = __fmul_rn(inv_n, __ldg(upstream));
        float g = __fmul_rn(sc, __fmul_rn(2.0f, __fsub_rn(x[0], x[1])));
        if (round_tf32) {
            uint32_t r;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(g));
            g = __uint_as_float(r);
        }
        o[0] = g;
    }
};

// (a - b)^2 with the difference and the square rounded separately, as sub_tensor followed by pow_scalar(2.0)
struct SqDiffF { __device__ void apply(const float* x, float* o) const { float d = __fsub_rn(x[0], x[1]); o[0] = __fmul_rn(d, d); } };
// (scale * upstream) * (2 * x): ReduceMean / ReduceSum backward followed by PowScalar(2) backward in one pass
struct SquareBwdScalarF {
    const float* upstream; float scale;
    __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(__fmul_rn(scale, __ldg(upstream)), __fmul_rn(2.0f, x[0])); }
};
// ---- unary and scalar ops beside the MLP path (tensor/ops/{exp,log,sqrt,tanh,sigmoid,leaky_relu,pow}.rs and
// the *_scalar variants of add/sub/mul/div).  The transcendental functions are CUDA's full-precision expf, logf,
// tanhf and powf (1-4 ulp from the host libm the reference calls); every other step is one rounded operation.
struct ExpF { __device__ void apply(const float* x, float* o) const { o[0] = expf(x[0]); } };
// log.rs:68-107 panics on x <= 0 (NaN included): the kernel still stores the IEEE result and raises the device word.
struct LogF {
    int* flag;
    __device__ void apply(const float* x, float* o) const {
        if (!(x[0] > 0.0f)) atomicCAS(flag, 0, TS_DEVICE_ERROR_LOG_DOMAIN);
        o[0] = logf(x[0]);
    }
};
struct SqrtF { __device__ void apply(const float* x, float* o) const { o[0] = __fsqrt_rn(x[0]); } };
struct TanhF { __device__ void apply(const float* x, float* o) const { o[0] = tanhf(x[0]); } };
// sigmoid.rs:90-110, the two-branch stable form: x >= 0 -> 1/(1+exp(-x)), else exp(x)/(1+exp(x)).  Both branches
// exponentiate -|x|, so one expf and one division serve both without divergence (a NaN takes the second branch
// in the reference and stays a NaN here).
struct SigmoidF {
    __device__ void apply(const float* x, float* o) const {
        const float z = expf(-fabsf(x[0]));
        const float num = x[0] >= 0.0f ? 1.0f : z;
        o[0] = __fdiv_rn(num, __fadd_rn(1.0f, z));
    }
};
struct LeakyReluF { float slope; __device__ void apply(const float* x, float* o) const { o[0] = x[0] > 0.0f ? x[0] : __fmul_rn(slope, x[0]); } };
struct AddScalarF { float v; __device__ void apply(const float* x, float* o) const { o[0] = __fadd_rn(x[0], v); } };
struct SubScalarF { float v; __device__ void apply(const float* x, float* o) const { o[0] = __fsub_rn(x[0], v); } };
struct DivScalarF { float v; __device__ void apply(const float* x, float* o) const { o[0] = __fdiv_rn(x[0], v); } };
struct PowF { float e; __device__ void apply(const float* x, float* o) const { o[0] = powf(x[0], e); } };
// backward functors: inputs (saved, go)
struct ExpBwdF { __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(x[1], x[0]); } };
struct LogBwdF { __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(x[1], __fdiv_rn(1.0f, x[0])); } };
struct SqrtBwdF { __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(x[1], __fmul_rn(__fdiv_rn(1.0f, x[0]), 0.5f)); } };
struct TanhBwdF { __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(x[1], __fsub_rn(1.0f, __fmul_rn(x[0], x[0]))); } };
struct SigmoidBwdF { __device__ void apply(const float* x, float* o) const { o[0] = __fmul_rn(__fmul_rn(x[1], x[0]), __fsub_rn(1.0f, x[0])); } };
struct LeakyReluBwdF { float slope; __device__ void apply(const float* x, float* o) const { o[0] = x[0] > 0.0f ? x[1] : __fmul_rn(slope, x[1]); } };
// go * (e * x^(e-1)), zero when e == 0 (grad_fn/ops/pow.rs:5-27)
struct PowBwdF {
    float e;
    __device__ void apply(const float* x, float* o) const {
        float local = e == 0.0f ? 0.0f : __fmul_rn(e, powf(x[0], __fsub_rn(e, 1.0f)));
        o[0] = __fmul_rn(x[1], local);
    }
};

// out[i,j] = act(z[i,j] + bias[j]); cols % 4 == 0 and aligned pointers take the vector path.
template <bool RELU>
__global__ void __launch_bounds__(kThreads) bias_act_vec_kernel(const float4* __restrict__ z, const float4* __restrict__ bias,
                                                                float4* __restrict__ out, size_t n_vec, unsigned cols_vec) {
    grid_dependency_sync();
    const size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n_vec; i += stride) {
        float4 v = __ldcs(z + i);
        float4 b = __ldg(bias + (unsigned)(i % cols_vec));
        v.x = __fadd_rn(v.x, b.x); v.y = __fadd_rn(v.y, b.y); v.z = __fadd_rn(v.z, b.z); v.w = __fadd_rn(v.w, b.w);
        if (RELU) {
            v.x = v.x > 0.0f ? v.x : 0.0f; v.y = v.y > 0.0f ? v.y : 0.0f;
            v.z = v.z > 0.0f ? v.z : 0.0f; v.w = v.w > 0.0f ? v.w : 0.0f;
        }
        __stcs(out + i, v);
    }
}
template <bool RELU>
__global__ void __launch_bounds__(kThreads) bias_act_scalar_kernel(const float* __restrict__ z, const float* __restrict__ bias,
                                                                   float* __restrict__ out, size_t n, size_t cols) {
    grid_dependency_sync();
    const size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        float v = __fadd_rn(z[i], __ldg(bias + (i % cols)));
        if (RELU) v = v > 0.0f ? v : 0.0f;
        out[i] = v;
    }
}

// ---- NumPy-style broadcasting (tensor/ops/broadcasting.rs:100-135) without the reference's materialised operands:
// outputs are contiguous over the broadcast shape, each input is read through element strides that are 0 along the
// axes it is stretched over.  Axes are merged on the host, innermost first, so that typical cases (row, column,
// outer product) reach the kernel with rank 1-3.
constexpr int kBcastRank = 6;
template <int NIN>
struct BcastGeom {
    int rank;
    unsigned dims[kBcastRank];                               // innermost first
    unsigned long long stride[NIN][kBcastRank];
    bool reused[NIN];                                        // stretched along at least one axis
};

// One group of VEC consecutive outputs along the innermost axis per thread and iteration.  VEC == 4 needs the
// innermost extent to be a multiple of 4, innermost strides of 0 or 1 and 16-byte aligned rows (host-checked).
// IDX is unsigned when the group count fits 32 bits (cheap divisions), size_t otherwise.  kUnroll groups per thread
// are loaded before any is computed, as in ew_vec_kernel, so that several 128-bit loads are in flight per thread.
template <int NIN, int NOUT, class F, int VEC, typename IDX>
__global__ void __launch_bounds__(kThreads) bcast_kernel(Ptrs<NIN, NOUT> p, BcastGeom<NIN> g, size_t n_groups, F f) {
    grid_dependency_sync();
    const size_t step = (size_t)gridDim.x * kThreads * kUnroll;
    const unsigned d0 = g.dims[0] / VEC;
    for (size_t base = (size_t)blockIdx.x * kThreads * kUnroll + threadIdx.x; base < n_groups; base += step) {
        float xi[kUnroll][VEC][NIN];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t gi = base + (size_t)u * kThreads;
            if (gi >= n_groups) break;
            IDX rem = (IDX)gi / d0;
            const size_t c0 = (size_t)((IDX)gi - rem * d0) * VEC;
            size_t off[NIN];
#pragma unroll
            for (int a = 0; a < NIN; ++a) off[a] = c0 * g.stride[a][0];
            for (int d = 1; d < g.rank; ++d) {
                const IDX q = rem / g.dims[d];
                const size_t cd = rem - q * g.dims[d];
                rem = q;
#pragma unroll
                for (int a = 0; a < NIN; ++a) off[a] += cd * g.stride[a][d];
            }
#pragma unroll
            for (int a = 0; a < NIN; ++a) {
                if (VEC == 4 && g.stride[a][0] == 1) {
                    // an operand that is stretched along some axis is read many times: keep it cached
                    const float4* q4 = reinterpret_cast<const float4*>(p.in[a] + off[a]);
                    const float4 v = g.reused[a] ? __ldg(q4) : __ldcs(q4);
                    xi[u][0][a] = v.x; xi[u][1 % VEC][a] = v.y; xi[u][2 % VEC][a] = v.z; xi[u][3 % VEC][a] = v.w;
                } else {
                    const float v = __ldg(p.in[a] + off[a]);     // stretched along the innermost axis (or VEC == 1)
#pragma unroll
                    for (int e = 0; e < VEC; ++e) xi[u][e][a] = v;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t gi = base + (size_t)u * kThreads;
            if (gi >= n_groups) break;
            float xo[VEC][NOUT];
#pragma unroll
            for (int e = 0; e < VEC; ++e) f.apply(xi[u][e], xo[e]);
#pragma unroll
            for (int o = 0; o < NOUT; ++o) {
                if (!p.out[o]) continue;
                if (VEC == 4) {
                    __stcs(reinterpret_cast<float4*>(p.out[o]) + gi, make_float4(xo[0][o], xo[1 % VEC][o], xo[2 % VEC][o], xo[3 % VEC][o]));
                } else {
                    p.out[o][gi] = xo[0][o];
                }
            }
        }
    }
}

// The same for rank 1 or 2 after merging (a row, a column, an outer product: the usual cases).  The (row, group within
// the row) position of each of a thread's kUnroll groups is carried along and advanced by a constant per iteration, so
// the loop has no division: with two 32-bit divisions per 16 bytes stored the general kernel is bound by instruction
// issue, not by memory (a column plus a row broadcast to a matrix, which only writes: 3.7 TB/s against the 6.2 TB/s a
// plain fill reaches).
template <int NIN, int NOUT, class F, int VEC>
__global__ void __launch_bounds__(kThreads) bcast2_kernel(Ptrs<NIN, NOUT> p, BcastGeom<NIN> g, size_t n_groups, F f) {
    grid_dependency_sync();
    const unsigned d0 = g.dims[0] / VEC;                                   // groups per row
    const unsigned step = gridDim.x * kThreads * kUnroll;
    const unsigned step_r = step / d0, step_c = step - step_r * d0;
    size_t gi[kUnroll];
    unsigned row[kUnroll], col[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        gi[u] = (size_t)blockIdx.x * kThreads * kUnroll + threadIdx.x + (size_t)u * kThreads;
        row[u] = (unsigned)(gi[u] / d0);
        col[u] = (unsigned)(gi[u] - (size_t)row[u] * d0);
    }
    while (gi[0] < n_groups) {
        float xi[kUnroll][VEC][NIN];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (gi[u] >= n_groups) break;
#pragma unroll
            for (int a = 0; a < NIN; ++a) {
                const size_t off = (size_t)col[u] * VEC * g.stride[a][0] + (size_t)row[u] * g.stride[a][1];
                if (VEC == 4 && g.stride[a][0] == 1) {
                    const float4* q4 = reinterpret_cast<const float4*>(p.in[a] + off);
                    const float4 v = g.reused[a] ? __ldg(q4) : __ldcs(q4);
                    xi[u][0][a] = v.x; xi[u][1 % VEC][a] = v.y; xi[u][2 % VEC][a] = v.z; xi[u][3 % VEC][a] = v.w;
                } else {
                    const float v = __ldg(p.in[a] + off);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) xi[u][e][a] = v;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (gi[u] >= n_groups) break;
            float xo[VEC][NOUT];
#pragma unroll
            for (int e = 0; e < VEC; ++e) f.apply(xi[u][e], xo[e]);
#pragma unroll
            for (int o = 0; o < NOUT; ++o) {
                if (!p.out[o]) continue;
                if (VEC == 4) {
                    __stcs(reinterpret_cast<float4*>(p.out[o]) + gi[u], make_float4(xo[0][o], xo[1 % VEC][o], xo[2 % VEC][o], xo[3 % VEC][o]));
                } else {
                    p.out[o][gi[u]] = xo[0][o];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            gi[u] += step;
            row[u] += step_r;
            col[u] += step_c;
            if (col[u] >= d0) { col[u] -= d0; ++row[u]; }
        }
    }
}

// dims (outermost first) and per-input strides over them; `contiguous_inputs` trailing inputs (the upstream
// gradient of a backward pass) are read with the output's own contiguous strides.
template <int NIN, int NOUT, class F>
bool launch_bcast(Ptrs<NIN, NOUT> p, const size_t* dims, int rank, const size_t* const* strides, int strided_inputs, F f, cudaStream_t s) {
    DeviceCtx* c = ctx();
    if (!c) return false;
    size_t n = 1;
    for (int d = 0; d < rank; ++d) n *= dims[d];
    if (n == 0) return true;
    for (int a = 0; a < NIN; ++a)
        if (!p.in[a]) { set_error("broadcast kernel: null input pointer"); return false; }
    // innermost first, extents of 1 dropped, neighbours merged while every input walks them as one axis
    BcastGeom<NIN> g;
    g.rank = 0;
    size_t contiguous = 1;
    for (int d = rank - 1; d >= 0; --d) {
        const size_t ext = dims[d];
        size_t st[NIN];
        for (int a = 0; a < NIN; ++a) st[a] = a < strided_inputs ? (ext == 1 ? 0 : strides[a][d]) : contiguous;
        contiguous *= ext;
        if (ext == 1) continue;
        bool merge = g.rank > 0;
        for (int a = 0; a < NIN && merge; ++a) merge = st[a] == g.stride[a][g.rank - 1] * g.dims[g.rank - 1];
        if (merge && (size_t)g.dims[g.rank - 1] * ext <= 0xFFFFFFFFull) {
            g.dims[g.rank - 1] *= (unsigned)ext;
            continue;
        }
        if (g.rank == kBcastRank || ext > 0xFFFFFFFFull) { set_error("broadcast: more than %d separate axes after merging", kBcastRank); return false; }
        g.dims[g.rank] = (unsigned)ext;
        for (int a = 0; a < NIN; ++a) g.stride[a][g.rank] = st[a];
        ++g.rank;
    }
    if (g.rank == 0) {                                       // a single element
        g.rank = 1;
        g.dims[0] = 1;
        for (int a = 0; a < NIN; ++a) g.stride[a][0] = 0;
    }
    bool vec = g.dims[0] % 4 == 0;
    for (int a = 0; a < NIN && vec; ++a) {
        vec = g.stride[a][0] <= 1 && (g.stride[a][0] == 0 || aligned16(p.in[a]));
        for (int d = 1; d < g.rank && vec; ++d) vec = g.stride[a][0] == 0 || g.stride[a][d] % 4 == 0;
    }
    for (int o = 0; o < NOUT; ++o) vec = vec && aligned16(p.out[o]);
    int n_out = 0;
    for (int o = 0; o < NOUT; ++o) n_out += p.out[o] ? 1 : 0;
    if (!n_out) { set_error("broadcast kernel: null output pointer"); return false; }
    ProfScope prof(kProfElementwise, s, 4.0 * (double)n * (n_out + NIN - strided_inputs));
    for (int a = 0; a < NIN; ++a) {
        g.reused[a] = false;
        for (int d = 0; d < g.rank; ++d) g.reused[a] = g.reused[a] || (g.stride[a][d] == 0 && g.dims[d] > 1);
    }
    const size_t n_groups = vec ? n / 4 : n;
    const int grid = grid_for(n_groups, c->sm_count);
    const bool small = n_groups <= 0xFFFFFFFFull;
    if (g.rank <= 2 && small) {
        if (g.rank == 1) {   // one row: the second axis does not exist
            g.dims[1] = 1;
            for (int a = 0; a < NIN; ++a) g.stride[a][1] = 0;
        }
        if (vec) launch_dep(bcast2_kernel<NIN, NOUT, F, 4>, dim3(grid), dim3(kThreads), 0, s, p, g, n_groups, f);
        else launch_dep(bcast2_kernel<NIN, NOUT, F, 1>, dim3(grid), dim3(kThreads), 0, s, p, g, n_groups, f);
    } else if (vec && small) launch_dep(bcast_kernel<NIN, NOUT, F, 4, unsigned>, dim3(grid), dim3(kThreads), 0, s, p, g, n_groups, f);
    else if (vec) launch_dep(bcast_kernel<NIN, NOUT, F, 4, size_t>, dim3(grid), dim3(kThreads), 0, s, p, g, n_groups, f);
    else if (small) launch_dep(bcast_kernel<NIN, NOUT, F, 1, unsigned>, dim3(grid), dim3(kThreads), 0, s, p, g, n_groups, f);
    else launch_dep(bcast_kernel<NIN, NOUT, F, 1, size_t>, dim3(grid), dim3(kThreads), 0, s, p, g, n_groups, f);
    return cuda_ok(cudaGetLastError(), "broadcast launch");
}

}  // namespace

bool binary_bcast(int op, const float* a, const float* b, float* o, const size_t* dims, int rank, const size_t* stride_a,
                  const size_t* stride_b, cudaStream_t s) {
    Ptrs<2, 1> p{{a, b}, {o}};
    const size_t* st[2] = {stride_a, stride_b};
    switch (op) {
        case 0: return launch_bcast(p, dims, rank, st, 2, AddF{}, s);
        case 1: return launch_bcast(p, dims, rank, st, 2, SubF{}, s);
        case 2: return launch_bcast(p, dims, rank, st, 2, MulF{}, s);
        case 3: return launch_bcast(p, dims, rank, st, 2, DivF{}, s);
    }
    set_error("binary_bcast: unknown op %d", op);
    return false;
}

// Full-size gradients of a broadcast mul (op 2) or div (op 3): ga = go*b or go/b, gb = go*a or -((go*a)/(b*b)),
// each over the broadcast shape (grad_fn/ops/mul.rs, div.rs); the caller sums them back to the operands' shapes.
bool binary_bcast_bwd(int op, const float* a, const float* b, const float* go, float* ga, float* gb, const size_t* dims, int rank,
                      const size_t* stride_a, const size_t* stride_b, cudaStream_t s) {
    Ptrs<3, 2> p{{a, b, go}, {ga, gb}};
    const size_t* st[2] = {stride_a, stride_b};
    if (op == 2) return launch_bcast(p, dims, rank, st, 2, MulBwdF{}, s);
    if (op == 3) return launch_bcast(p, dims, rank, st, 2, DivBwdF{}, s);
    set_error("binary_bcast_bwd: unknown op %d", op);
    return false;
}

bool binary(int op, const float* a, const float* b, float* o, size_t n, cudaStream_t s) {
    Ptrs<2, 1> p{{a, b}, {o}};
    switch (op) {
        case 0: return launch_ew(p, n, AddF{}, s);
        case 1: return launch_ew(p, n, SubF{}, s);
        case 2: return launch_ew(p, n, MulF{}, s);
        case 3: return launch_ew(p, n, DivF{}, s);
    }
    set_error("binary: unknown op %d", op);
    return false;
}
bool relu(const float* x, float* o, size_t n, cudaStream_t s) { return launch_ew(Ptrs<1, 1>{{x}, {o}}, n, ReluF{}, s); }
bool relu_bwd(const float* ref, const float* go, float* gi, size_t n, cudaStream_t s) {
    return launch_ew(Ptrs<2, 1>{{ref, go}, {gi}}, n, ReluBwdF{}, s);
}
bool square(const float* x, float* o, size_t n, cudaStream_t s) { return launch_ew(Ptrs<1, 1>{{x}, {o}}, n, SquareF{}, s); }
bool square_bwd(const float* x, const float* go, float* gi, size_t n, cudaStream_t s) {
    return launch_ew(Ptrs<2, 1>{{x, go}, {gi}}, n, SquareBwdF{}, s);
}
bool mul_bwd(const float* a, const float* b, const float* go, float* ga, float* gb, size_t n, cudaStream_t s) {
    return launch_ew(Ptrs<3, 2>{{a, b, go}, {ga, gb}}, n, MulBwdF{}, s);
}
bool div_bwd(const float* a, const float* b, const float* go, float* ga, float* gb, size_t n, cudaStream_t s) {
    return launch_ew(Ptrs<3, 2>{{a, b, go}, {ga, gb}}, n, DivBwdF{}, s);
}
bool scale(const float* x, float alpha, float* o, size_t n, cudaStream_t s) {
    return launch_ew(Ptrs<1, 1>{{x}, {o}}, n, ScaleF{alpha}, s);
}
bool fill(float* o, float v, size_t n, cudaStream_t s) { return launch_ew(Ptrs<0, 1>{{nullptr}, {o}}, n, FillF{v}, s); }

namespace {
template <bool VEC>
__global__ void __launch_bounds__(kThreads) sum_slabs_kernel(const float* __restrict__ part, float* __restrict__ out, size_t n, int slabs) {
    grid_dependency_sync();
    const size_t step = (size_t)gridDim.x * kThreads;
    if (VEC) {
        const size_t nv = n / 4;
        for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < nv; i += step) {
            float4 acc = __ldcs(reinterpret_cast<const float4*>(part) + i);
            for (int s = 1; s < slabs; ++s) {
                const float4 v = __ldcs(reinterpret_cast<const float4*>(part + (size_t)s * n) + i);
                acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
            }
            reinterpret_cast<float4*>(out)[i] = acc;
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += step) {
            float acc = part[i];
            for (int s = 1; s < slabs; ++s) acc = __fadd_rn(acc, part[(size_t)s * n + i]);
            out[i] = acc;
        }
    }
}
}  // namespace

bool sum_slabs(const float* part, float* out, size_t n, size_t slabs, cudaStream_t s) {
    if (n == 0) return true;
    if (!part || !out || slabs == 0) { set_error("sum_slabs: bad arguments"); return false; }
    DeviceCtx* c = ctx();
    if (!c) return false;
    ProfScope prof(kProfElementwise, s, 4.0 * (double)n * (double)(slabs + 1));
    const bool vec = n % 4 == 0 && aligned16(part) && aligned16(out);
    const size_t work = vec ? n / 4 : n;
    size_t grid = (work + kThreads - 1) / kThreads;
    const size_t cap = (size_t)c->sm_count * 8;
    if (grid > cap) grid = cap;
    if (vec) launch_dep(sum_slabs_kernel<true>, dim3((unsigned)grid), dim3(kThreads), 0, s, part, out, n, (int)slabs);
    else launch_dep(sum_slabs_kernel<false>, dim3((unsigned)grid), dim3(kThreads), 0, s, part, out, n, (int)slabs);
    return cuda_ok(cudaGetLastError(), "sum_slabs launch");
}
bool fill_from_scalar(float* o, const float* scalar, float sc, size_t n, cudaStream_t s) {
    if (!scalar) { set_error("fill_from_scalar: null scalar"); return false; }
    return launch_ew(Ptrs<0, 1>{{nullptr}, {o}}, n, FillFromScalarF{scalar, sc}, s);
}
bool add_scalar_bcast(const float* a, const float* scalar_dev, float* o, size_t n, cudaStream_t s) {
    if (!scalar_dev) { set_error("add_scalar_bcast: null scalar"); return false; }
    return launch_ew(Ptrs<1, 1>{{a}, {o}}, n, AddScalarBcastF{scalar_dev}, s);
}
bool split_tf32(const float* x, float* hi, float* lo, size_t n, cudaStream_t s) {
    if (!hi || !lo) { set_error("split_tf32: null output"); return false; }
    return launch_ew(Ptrs<1, 2>{{x}, {hi, lo}}, n, SplitTf32F{}, s);
}
bool round_to_tf32(const float* x, float* o, size_t n, cudaStream_t s) { return launch_ew(Ptrs<1, 1>{{x}, {o}}, n, RoundTf32F{}, s); }
bool sqdiff(const float* a, const float* b, float* o, size_t n, cudaStream_t s) { return launch_ew(Ptrs<2, 1>{{a, b}, {o}}, n, SqDiffF{}, s); }
bool square_bwd_scalar(const float* x, const float* upstream, float scale, float* gi, size_t n, cudaStream_t s) {
    if (!upstream) { set_error("square_bwd_scalar: null upstream"); return false; }
    return launch_ew(Ptrs<1, 1>{{x}, {gi}}, n, SquareBwdScalarF{upstream, scale}, s);
}
bool mse_grad(const float* y, const float* t, const float* upstream, float inv_n, float* gy, size_t n, bool round_tf32, cudaStream_t s) {
    if (!upstream) { set_error("mse_grad: null upstream"); return false; }
    return launch_ew(Ptrs<2, 1>{{y, t}, {gy}}, n, MseGradF{upstream, inv_n, round_tf32}, s);
}

bool unary(int op, const float* x, float* o, size_t n, float p, cudaStream_t s) {
    Ptrs<1, 1> ptrs{{x}, {o}};
    switch (op) {
        case TS_UNARY_EXP: return launch_ew(ptrs, n, ExpF{}, s);
        case TS_UNARY_LOG: {
            DeviceCtx* c = ctx();
            return c && launch_ew(ptrs, n, LogF{c->error_flag}, s);
        }
        case TS_UNARY_SQRT: return launch_ew(ptrs, n, SqrtF{}, s);
        case TS_UNARY_TANH: return launch_ew(ptrs, n, TanhF{}, s);
        case TS_UNARY_SIGMOID: return launch_ew(ptrs, n, SigmoidF{}, s);
        case TS_UNARY_LEAKY_RELU: return launch_ew(ptrs, n, LeakyReluF{p}, s);
        case TS_UNARY_ADD_SCALAR: return launch_ew(ptrs, n, AddScalarF{p}, s);
        case TS_UNARY_SUB_SCALAR: return launch_ew(ptrs, n, SubScalarF{p}, s);
        case TS_UNARY_MUL_SCALAR: return launch_ew(ptrs, n, ScaleF{p}, s);
        case TS_UNARY_DIV_SCALAR:
            // div.rs:511-514 panics before touching the data
            if (p == 0.0f) { set_error("Division by zero: cannot divide tensor by zero scalar"); return false; }
            return launch_ew(ptrs, n, DivScalarF{p}, s);
        case TS_UNARY_POW_SCALAR:
            // pow.rs:125-160: exponent 2 is x*x, 0.5 is sqrt, anything else powf
            if (p == 2.0f) return launch_ew(ptrs, n, SquareF{}, s);
            if (p == 0.5f) return launch_ew(ptrs, n, SqrtF{}, s);
            return launch_ew(ptrs, n, PowF{p}, s);
    }
    set_error("unary: unknown op %d", op);
    return false;
}

bool unary_bwd(int op, const float* saved, const float* go, float* gi, size_t n, float p, cudaStream_t s) {
    const bool needs_saved = op == TS_UNARY_EXP || op == TS_UNARY_LOG || op == TS_UNARY_SQRT || op == TS_UNARY_TANH ||
                             op == TS_UNARY_SIGMOID || op == TS_UNARY_LEAKY_RELU || op == TS_UNARY_POW_SCALAR;
    if (needs_saved && !saved && n) { set_error("unary backward: op %d needs the saved tensor", op); return false; }
    Ptrs<2, 1> two{{saved, go}, {gi}};
    Ptrs<1, 1> one{{go}, {gi}};
    switch (op) {
        case TS_UNARY_EXP: return launch_ew(two, n, ExpBwdF{}, s);
        case TS_UNARY_LOG: return launch_ew(two, n, LogBwdF{}, s);
        case TS_UNARY_SQRT: return launch_ew(two, n, SqrtBwdF{}, s);
        case TS_UNARY_TANH: return launch_ew(two, n, TanhBwdF{}, s);
        case TS_UNARY_SIGMOID: return launch_ew(two, n, SigmoidBwdF{}, s);
        case TS_UNARY_LEAKY_RELU: return launch_ew(two, n, LeakyReluBwdF{p}, s);
        case TS_UNARY_POW_SCALAR: return launch_ew(two, n, PowBwdF{p}, s);
        case TS_UNARY_ADD_SCALAR:
        case TS_UNARY_SUB_SCALAR: return launch_ew(one, n, ScaleF{1.0f}, s);   // the gradient itself (a copy)
        case TS_UNARY_MUL_SCALAR: return launch_ew(one, n, ScaleF{p}, s);
        case TS_UNARY_DIV_SCALAR:
            if (p == 0.0f) { set_error("Division by zero: cannot divide tensor by zero scalar"); return false; }
            return launch_ew(one, n, DivScalarF{p}, s);
    }
    set_error("unary backward: unknown op %d", op);
    return false;
}

bool bias_act(const float* z, const float* bias, float* o, size_t rows, size_t cols, bool relu_on, cudaStream_t s) {
    size_t n = rows * cols;
    if (n == 0) return true;
    if (!z || !bias || !o) { set_error("bias_act: null pointer"); return false; }
    DeviceCtx* c = ctx();
    if (!c) return false;
    ProfScope prof(kProfElementwise, s, 8.0 * (double)n);
    if (cols % 4 == 0 && aligned16(z) && aligned16(bias) && aligned16(o) && cols / 4 < (1ull << 32)) {
        size_t n_vec = n / 4;
        size_t want = (n_vec + kThreads - 1) / kThreads, cap = (size_t)c->sm_count * kCtasPerSm * 2;
        int grid = (int)(want < cap ? want : cap);
        if (relu_on) launch_dep(bias_act_vec_kernel<true>, dim3(grid), dim3(kThreads), 0, s, (const float4*)z, (const float4*)bias, (float4*)o, n_vec, (unsigned)(cols / 4));
        else launch_dep(bias_act_vec_kernel<false>, dim3(grid), dim3(kThreads), 0, s, (const float4*)z, (const float4*)bias, (float4*)o, n_vec, (unsigned)(cols / 4));
    } else {
        size_t want = (n + kThreads - 1) / kThreads, cap = (size_t)c->sm_count * kCtasPerSm * 2;
        int grid = (int)(want < cap ? want : cap);
        if (relu_on) launch_dep(bias_act_scalar_kernel<true>, dim3(grid), dim3(kThreads), 0, s, z, bias, o, n, cols);
        else launch_dep(bias_act_scalar_kernel<false>, dim3(grid), dim3(kThreads), 0, s, z, bias, o, n, cols);
    }
    return cuda_ok(cudaGetLastError(), "bias_act launch");
}

}  // namespace k
}  // namespace ts

// ====================================================================== C ABI
using namespace ts;

#define TS_STREAM_OR_FAIL(var)                 \
    cudaStream_t var = ts::pick_stream(stream); \
    if (!var) return false;

TS_API bool launch_add_kernel(const float* a, const float* b, float* r, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    if (!a || !b || !r) { if (n == 0) return true; set_error("launch_add_kernel: null pointer"); return false; }
    return k::binary(0, a, b, r, n, s);
}
TS_API bool launch_sub_kernel(const float* a, const float* b, float* r, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    if (!a || !b || !r) { if (n == 0) return true; set_error("launch_sub_kernel: null pointer"); return false; }
    return k::binary(1, a, b, r, n, s);
}
TS_API bool launch_mul_kernel(const float* a, const float* b, float* r, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    if (!a || !b || !r) { if (n == 0) return true; set_error("launch_mul_kernel: null pointer"); return false; }
    return k::binary(2, a, b, r, n, s);
}
TS_API bool launch_div_kernel(const float* a, const float* b, float* r, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    if (!a || !b || !r) { if (n == 0) return true; set_error("launch_div_kernel: null pointer"); return false; }
    return k::binary(3, a, b, r, n, s);
}
TS_API bool launch_bias_act_kernel(const float* z, const float* bias, float* out, unsigned long long rows,
                                   unsigned long long cols, int relu, void* stream) {
    TS_STREAM_OR_FAIL(s);
    return k::bias_act(z, bias, out, rows, cols, relu != 0, s);
}
TS_API bool launch_relu_kernel(const float* x, float* out, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    return k::relu(x, out, n, s);
}
TS_API bool launch_relu_backward_kernel(const float* ref, const float* go, float* gi, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    return k::relu_bwd(ref, go, gi, n, s);
}
TS_API bool launch_square_kernel(const float* x, float* out, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    return k::square(x, out, n, s);
}
TS_API bool launch_square_backward_kernel(const float* x, const float* go, float* gi, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    return k::square_bwd(x, go, gi, n, s);
}
TS_API bool launch_mul_backward_kernel(const float* a, const float* b, const float* go, float* ga, float* gb,
                                       unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    return k::mul_bwd(a, b, go, ga, gb, n, s);
}
namespace {
// shapes of the two operands -> the broadcast shape and each operand's strides over it; false on a mismatch
bool broadcast_plan(const unsigned long long* dims_a, int rank_a, const unsigned long long* dims_b, int rank_b, size_t* out, size_t* sa,
                    size_t* sb, int* rank) {
    if (rank_a < 1 || rank_b < 1 || rank_a > 8 || rank_b > 8 || !dims_a || !dims_b) { ts::set_error("broadcast: rank must be 1..8"); return false; }
    const int n = rank_a > rank_b ? rank_a : rank_b;
    size_t run_a = 1, run_b = 1;
    for (int i = 0; i < n; ++i) {
        const size_t da = i < rank_a ? dims_a[rank_a - 1 - i] : 1, db = i < rank_b ? dims_b[rank_b - 1 - i] : 1;
        if (da != db && da != 1 && db != 1) { ts::set_error("broadcast: incompatible dimensions at axis %d", n - 1 - i); return false; }
        out[n - 1 - i] = da == 1 ? db : da;
        sa[n - 1 - i] = da == 1 ? 0 : run_a;
        sb[n - 1 - i] = db == 1 ? 0 : run_b;
        run_a *= da;
        run_b *= db;
    }
    *rank = n;
    return true;
}
}  // namespace
TS_API bool launch_binary_broadcast_kernel(int op, const float* a, const unsigned long long* dims_a, int rank_a, const float* b,
                                           const unsigned long long* dims_b, int rank_b, float* out, void* stream) {
    TS_STREAM_OR_FAIL(s);
    size_t od[8], sa[8], sb[8];
    int rank;
    if (!broadcast_plan(dims_a, rank_a, dims_b, rank_b, od, sa, sb, &rank)) return false;
    return k::binary_bcast(op, a, b, out, od, rank, sa, sb, s);
}
TS_API bool launch_binary_broadcast_backward_kernel(int op, const float* a, const unsigned long long* dims_a, int rank_a, const float* b,
                                                    const unsigned long long* dims_b, int rank_b, const float* go, float* ga, float* gb,
                                                    void* stream) {
    TS_STREAM_OR_FAIL(s);
    size_t od[8], sa[8], sb[8];
    int rank;
    if (!broadcast_plan(dims_a, rank_a, dims_b, rank_b, od, sa, sb, &rank)) return false;
    return k::binary_bcast_bwd(op, a, b, go, ga, gb, od, rank, sa, sb, s);
}
TS_API bool launch_div_backward_kernel(const float* a, const float* b, const float* go, float* ga, float* gb,
                                       unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    return k::div_bwd(a, b, go, ga, gb, n, s);
}
TS_API bool launch_scale_kernel(const float* x, float alpha, float* out, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    return k::scale(x, alpha, out, n, s);
}
TS_API bool launch_fill_kernel(float* out, float value, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    return k::fill(out, value, n, s);
}
TS_API bool launch_fill_from_scalar_kernel(float* out, const float* scalar, float scale, unsigned long long n, void* stream) {
    TS_STREAM_OR_FAIL(s);
    return k::fill_from_scalar(out, scalar, scale, n, s);
}
TS_API bool launch_unary_kernel(int op, const float* x, float* out, unsigned long long n, float param, void* stream) {
    TS_STREAM_OR_FAIL(s);
    if (!x || !out) { if (n == 0) return true; set_error("launch_unary_kernel: null pointer"); return false; }
    return k::unary(op, x, out, n, param, s);
}
TS_API bool launch_unary_backward_kernel(int op, const float* saved, const float* go, float* gi, unsigned long long n, float param,
                                         void* stream) {
    TS_STREAM_OR_FAIL(s);
    if (!go || !gi) { if (n == 0) return true; set_error("launch_unary_backward_kernel: null pointer"); return false; }
    return k::unary_bwd(op, saved, go, gi, n, param, s);
}
