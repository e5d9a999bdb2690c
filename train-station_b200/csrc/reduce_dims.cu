// Reductions over a subset of the axes of a contiguous tensor, and their backward passes.
// HBM-bound: the forward reads the input once per sweep (one sweep for sum / max / min / sum of squares, two for the
// variance: mean, then squared deviations); the backward reads the input (and a few per-output values) and writes
// the gradient.
//
// Reference: tensor/reductions/{sum.rs:225-306, mean.rs:186-215, max.rs:65-145, min.rs, norm.rs:202-300,
// var.rs:294-420, std.rs:316-440} and gradtrack/grad_fn/reductions/*.rs.  The reference walks the input in linear
// order and adds each element into its output slot, i.e. each output is a sequential f32 sum over its reduced
// coordinates in increasing order.  Here:
//  * when the last input axis is kept, one thread owns an output element and walks its reduced coordinates in the
//    same increasing order (neighbouring threads read neighbouring addresses), so sums come out in the reference's
//    order unless the reduced range is split;
//  * when the last input axis is reduced, a warp owns an output element, lanes stride over the reduced range and
//    combine with a shuffle tree;
//  * when there are too few outputs to fill the GPU, the reduced range is split, partial results go to a scratch
//    buffer and a second launch combines them in split order (deterministic).
#include <cfloat>

#include "../../include/train_station_b200.h"
#include "common.h"

namespace ts {
namespace k {

namespace {

constexpr int kThreads = 256;

// forward modes: what is accumulated per element, and how partials combine
enum { kSum = 0, kMax = 1, kMin = 2, kSumSq = 3, kSqDev = 4, kCountEq = 5 };

struct Plan {
    int nk, nr;                                   // kept and reduced axes after merging (each <= 8)
    unsigned long long kdim[8], kstr[8];          // kept axes: extent, input stride
    unsigned long long rdim[8], rstr[8];          // reduced axes: extent, input stride
    unsigned long long n_out, n_red;
};

__device__ __forceinline__ size_t radix_offset(size_t idx, const unsigned long long* dims, const unsigned long long* strides, int n) {
    size_t off = 0;
#pragma unroll
    for (int d = 7; d >= 0; --d) {
        if (d < n) {
            const size_t q = idx / dims[d];
            off += (idx - q * dims[d]) * strides[d];
            idx = q;
        }
    }
    return off;
}

template <int OP>
__device__ __forceinline__ float identity() { return OP == kMax ? -INFINITY : OP == kMin ? INFINITY : 0.0f; }
template <int OP>
__device__ __forceinline__ float term(float v, float aux) {
    if (OP == kSumSq) return __fmul_rn(v, v);
    if (OP == kSqDev) { const float d = __fsub_rn(v, aux); return __fmul_rn(d, d); }
    if (OP == kCountEq) return v == aux ? 1.0f : 0.0f;
    return v;
}
// a NaN never wins a comparison, as in the reference's `if val > cur` / `if val < cur`
template <int OP>
__device__ __forceinline__ float combine(float acc, float t) {
    if (OP == kMax) return t > acc ? t : acc;
    if (OP == kMin) return t < acc ? t : acc;
    return __fadd_rn(acc, t);
}

// One thread per (output, split): the last input axis is kept, so neighbouring outputs are neighbouring addresses.
template <int OP>
__global__ void __launch_bounds__(kThreads) reduce_kept_inner_kernel(const float* __restrict__ x, const float* __restrict__ aux,
                                                                     float* __restrict__ out, Plan p, size_t chunk) {
    grid_dependency_sync();
    const size_t o = (size_t)blockIdx.x * kThreads + threadIdx.x;
    if (o >= p.n_out) return;
    const size_t base = radix_offset(o, p.kdim, p.kstr, p.nk);
    const size_t r0 = (size_t)blockIdx.y * chunk;
    size_t r1 = r0 + chunk;
    if (r1 > p.n_red) r1 = p.n_red;
    const float a = (OP == kSqDev || OP == kCountEq) ? aux[o] : 0.0f;
    float acc = identity<OP>();
    if (p.nr == 1) {
        const size_t rs = p.rstr[0];
        for (size_t r = r0; r < r1; ++r) acc = combine<OP>(acc, term<OP>(x[base + r * rs], a));
    } else {
        for (size_t r = r0; r < r1; ++r) acc = combine<OP>(acc, term<OP>(x[base + radix_offset(r, p.rdim, p.rstr, p.nr)], a));
    }
    out[(size_t)blockIdx.y * p.n_out + o] = acc;
}

// The same with four adjacent outputs per thread (128-bit loads, eight rows in flight): the innermost kept extent is a
// multiple of 4 and everything is 16-byte aligned.  Each output still adds its terms in increasing reduced order.
template <int OP>
__global__ void __launch_bounds__(kThreads) reduce_kept_inner_vec4_kernel(const float* __restrict__ x, const float* __restrict__ aux,
                                                                          float* __restrict__ out, Plan p, size_t chunk) {
    grid_dependency_sync();
    const size_t o = ((size_t)blockIdx.x * kThreads + threadIdx.x) * 4;
    if (o >= p.n_out) return;
    const size_t base = radix_offset(o, p.kdim, p.kstr, p.nk);
    const size_t r0 = (size_t)blockIdx.y * chunk;
    size_t r1 = r0 + chunk;
    if (r1 > p.n_red) r1 = p.n_red;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (OP == kSqDev || OP == kCountEq) a = *reinterpret_cast<const float4*>(aux + o);
    float4 acc = make_float4(identity<OP>(), identity<OP>(), identity<OP>(), identity<OP>());
    auto fold = [&](const float4& v) {
        acc.x = combine<OP>(acc.x, term<OP>(v.x, a.x));
        acc.y = combine<OP>(acc.y, term<OP>(v.y, a.y));
        acc.z = combine<OP>(acc.z, term<OP>(v.z, a.z));
        acc.w = combine<OP>(acc.w, term<OP>(v.w, a.w));
    };
    if (p.nr == 1) {
        const size_t rs = p.rstr[0];
        size_t r = r0;
        for (; r + 8 <= r1; r += 8) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcs(reinterpret_cast<const float4*>(x + base + (r + u) * rs));
#pragma unroll
            for (int u = 0; u < 8; ++u) fold(v[u]);
        }
        for (; r < r1; ++r) fold(__ldcs(reinterpret_cast<const float4*>(x + base + r * rs)));
    } else {
        for (size_t r = r0; r < r1; ++r) fold(__ldcs(reinterpret_cast<const float4*>(x + base + radix_offset(r, p.rdim, p.rstr, p.nr))));
    }
    *reinterpret_cast<float4*>(out + (size_t)blockIdx.y * p.n_out + o) = acc;
}

// One warp per (output, split): the last input axis is reduced, lanes stride over the reduced range.
template <int OP>
__global__ void __launch_bounds__(kThreads) reduce_reduced_inner_kernel(const float* __restrict__ x, const float* __restrict__ aux,
                                                                        float* __restrict__ out, Plan p, size_t chunk, size_t splits) {
    grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const size_t units = p.n_out * splits;
    for (size_t u = (size_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); u < units; u += (size_t)gridDim.x * (kThreads / 32)) {
        const size_t s = u / p.n_out, o = u - s * p.n_out;
        const size_t base = radix_offset(o, p.kdim, p.kstr, p.nk);
        const size_t r0 = s * chunk;
        size_t r1 = r0 + chunk;
        if (r1 > p.n_red) r1 = p.n_red;
        const float a = (OP == kSqDev || OP == kCountEq) ? aux[o] : 0.0f;
        float acc = identity<OP>();
        if (p.nr == 1 && p.rstr[0] == 1) {
            // a contiguous run: scalar loads up to the first 16-byte boundary, then four independent 128-bit loads
            // and accumulators per lane (2 KB in flight per warp), then a scalar tail
            const float* row = x + base;
            const size_t mis = (reinterpret_cast<uintptr_t>(row + r0) & 15) >> 2;
            size_t head = mis ? 4 - mis : 0;
            if (head > r1 - r0) head = r1 - r0;
            if ((size_t)lane < head) acc = combine<OP>(acc, term<OP>(row[r0 + lane], a));
            const size_t rv = r0 + head, nvec = (r1 - rv) / 4;
            const float4* v = reinterpret_cast<const float4*>(row + rv);
            float a1 = identity<OP>(), a2 = identity<OP>(), a3 = identity<OP>();
            auto fold = [&](float acc_, const float4& q) {
                acc_ = combine<OP>(acc_, term<OP>(q.x, a));
                acc_ = combine<OP>(acc_, term<OP>(q.y, a));
                acc_ = combine<OP>(acc_, term<OP>(q.z, a));
                return combine<OP>(acc_, term<OP>(q.w, a));
            };
            size_t i = lane;
            for (; i + 96 < nvec; i += 128) {
                const float4 v0 = __ldcs(v + i), v1 = __ldcs(v + i + 32), v2 = __ldcs(v + i + 64), v3 = __ldcs(v + i + 96);
                acc = fold(acc, v0);
                a1 = fold(a1, v1);
                a2 = fold(a2, v2);
                a3 = fold(a3, v3);
            }
            for (; i < nvec; i += 32) acc = fold(acc, __ldcs(v + i));
            const size_t t = rv + nvec * 4 + lane;
            if (t < r1) a1 = combine<OP>(a1, term<OP>(row[t], a));
            acc = combine<OP>(combine<OP>(acc, a1), combine<OP>(a2, a3));
        } else {
            for (size_t r = r0 + lane; r < r1; r += 32) acc = combine<OP>(acc, term<OP>(x[base + radix_offset(r, p.rdim, p.rstr, p.nr)], a));
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) acc = combine<OP>(acc, __shfl_xor_sync(0xffffffffu, acc, d));
        if (lane == 0) out[s * p.n_out + o] = acc;
    }
}

template <int OP>
bool launch_forward(const float* x, const float* aux, float* out, const Plan& p, float* scratch, size_t scratch_elems, int sm, cudaStream_t s) {
    const bool reduced_inner = p.nr > 0 && p.rstr[p.nr - 1] == 1;
    // how many ways to split the reduced range so that the GPU is busy
    size_t splits = 1;
    bool vec4 = false;
    if (reduced_inner) {
        const size_t want_warps = (size_t)sm * 64;
        if (p.n_out < want_warps) splits = (want_warps + p.n_out - 1) / p.n_out;
        const size_t max_splits = (p.n_red + 2047) / 2048;     // at least 2048 elements per warp
        if (splits > max_splits) splits = max_splits;
    } else {
        auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
        vec4 = p.nk > 0 && p.kstr[p.nk - 1] == 1 && p.kdim[p.nk - 1] % 4 == 0 && al16(x) && al16(out) && al16(scratch) && (!aux || al16(aux));
        for (int d = 0; d + 1 < p.nk && vec4; ++d) vec4 = p.kstr[d] % 4 == 0;
        for (int d = 0; d < p.nr && vec4; ++d) vec4 = p.rstr[d] % 4 == 0;
        const size_t want_threads = (size_t)sm * (vec4 ? 1024 : 2048), owners = vec4 ? p.n_out / 4 : p.n_out;
        if (owners * 2 <= want_threads) splits = (want_threads + owners - 1) / owners;   // half a GPU of owners is enough
        const size_t max_splits = (p.n_red + 31) / 32;         // at least 32 elements per thread
        if (splits > max_splits) splits = max_splits;
    }
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
    if (splits > 1 && splits * p.n_out > scratch_elems) splits = scratch_elems / p.n_out;
    if (splits < 1) splits = 1;
    size_t chunk = (p.n_red + splits - 1) / splits;
    if (reduced_inner && splits > 1) chunk = (chunk + 127) / 128 * 128;    // every split starts on the row's alignment
    splits = (p.n_red + chunk - 1) / chunk;
    float* dst = splits > 1 ? scratch : out;
    if (reduced_inner) {
        const size_t units = p.n_out * splits, want = (units + 7) / 8, cap = (size_t)sm * 32;
        launch_dep(reduce_reduced_inner_kernel<OP>, dim3((unsigned)(want < cap ? want : cap)), dim3(kThreads), 0, s, x, aux, dst, p, chunk, splits);
    } else if (vec4) {
        dim3 grid((unsigned)((p.n_out / 4 + kThreads - 1) / kThreads), (unsigned)splits);
        launch_dep(reduce_kept_inner_vec4_kernel<OP>, dim3(grid), dim3(kThreads), 0, s, x, aux, dst, p, chunk);
    } else {
        dim3 grid((unsigned)((p.n_out + kThreads - 1) / kThreads), (unsigned)splits);
        launch_dep(reduce_kept_inner_kernel<OP>, dim3(grid), dim3(kThreads), 0, s, x, aux, dst, p, chunk);
    }
    if (!cuda_ok(cudaGetLastError(), "reduce_dims launch")) return false;
    if (splits > 1) {
        // partials are [splits][n_out]: combine over the split axis, one thread per output, in split order
        Plan q{};
        q.nk = 1; q.kdim[0] = p.n_out; q.kstr[0] = 1;
        q.nr = 1; q.rdim[0] = splits; q.rstr[0] = p.n_out;
        q.n_out = p.n_out; q.n_red = splits;
        constexpr int OP2 = (OP == kMax || OP == kMin) ? OP : kSum;
        if (OP2 == kSum && splits > 8 && p.n_out >= 1024) {
            // many partial rows of many outputs (column sums of a tall matrix): lanes along the outputs, warps along the
            // partial rows, so the rows are read as contiguous runs; rows added in a fixed order
            if (!colsum_finish(scratch, out, p.n_out, splits, s)) return false;
        } else if (splits > 32) {
            // many partials per output (few outputs): a warp per output instead of one thread walking them all
            const size_t want = (p.n_out + 7) / 8, cap = (size_t)sm * 32;
            launch_dep(reduce_reduced_inner_kernel<OP2>, dim3((unsigned)(want < cap ? want : cap)), dim3(kThreads), 0, s, scratch, nullptr, out, q, splits, 1);
        } else {
            dim3 grid((unsigned)((p.n_out + kThreads - 1) / kThreads), 1);
            launch_dep(reduce_kept_inner_kernel<OP2>, dim3(grid), dim3(kThreads), 0, s, scratch, nullptr, out, q, splits);
        }
        if (!cuda_ok(cudaGetLastError(), "reduce_dims combine launch")) return false;
    }
    return true;
}

// ---- backward: one thread per input element
enum { kBwdSum = 0, kBwdScaled = 1, kBwdExtremum = 2, kBwdNorm = 3, kBwdVar = 4, kBwdStd = 5 };

struct BwdPlan {
    int n;                                        // merged input axes
    unsigned long long dim[8], ostr[8];           // extent, stride in the OUTPUT (0 for a reduced axis)
};

template <int MODE>
__global__ void __launch_bounds__(kThreads) reduce_bwd_kernel(const float* __restrict__ x, const float* __restrict__ a1, const float* __restrict__ a2,
                                                              const float* __restrict__ go, float* __restrict__ gi, size_t n, BwdPlan p,
                                                              int go_is_scalar, float scale) {
    grid_dependency_sync();
    const size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        const size_t o = radix_offset(i, p.dim, p.ostr, p.n);
        const float up = go_is_scalar ? __ldg(go) : go[o];
        float g;
        if (MODE == kBwdSum) g = up;                                           // grad_fn/reductions/sum.rs:17-60
        else if (MODE == kBwdScaled) g = __fmul_rn(up, scale);                 // mean.rs:30-50: the sum's gradient times 1/count
        else if (MODE == kBwdExtremum) {                                       // max.rs / min.rs: shared equally among the ties
            const float cnt = a2[o];
            g = x[i] == a1[o] ? (cnt > 0.0f ? __fdiv_rn(up, cnt) : 0.0f) : 0.0f;
        } else if (MODE == kBwdNorm) {                                         // norm.rs: x * (up / norm), zero where the norm is zero
            const float nv = a1[o];
            g = nv > 0.0f ? __fmul_rn(x[i], __fdiv_rn(up, nv)) : 0.0f;
        } else if (MODE == kBwdVar) {                                          // var.rs: (x - mean) * (up * (2/n))
            g = __fmul_rn(__fsub_rn(x[i], a1[o]), __fmul_rn(up, scale));
        } else {                                                               // std.rs: (x - mean) * (up * (1/n) / std), zero where std is zero
            const float sd = a2[o];
            g = sd > 0.0f ? __fmul_rn(__fsub_rn(x[i], a1[o]), __fdiv_rn(__fmul_rn(up, scale), sd)) : 0.0f;
        }
        gi[i] = g;
    }
}

// Splits the input axes into kept and reduced ones and merges neighbours of the same kind.
bool make_plans(const size_t* dims, int rank, const unsigned char* reduced, Plan* fwd, BwdPlan* bwd) {
    if (rank < 1 || rank > 8) { set_error("reduce_dims: rank %d not supported (1..8)", rank); return false; }
    size_t in_stride[8], out_stride[8];
    size_t acc = 1;
    for (int i = rank - 1; i >= 0; --i) { in_stride[i] = acc; acc *= dims[i]; }
    acc = 1;
    for (int i = rank - 1; i >= 0; --i) { out_stride[i] = reduced[i] ? 0 : acc; if (!reduced[i]) acc *= dims[i]; }
    Plan f{};
    BwdPlan b{};
    f.n_out = 1; f.n_red = 1;
    int last_kind = -1;
    for (int i = 0; i < rank; ++i) {
        if (dims[i] == 1) continue;                      // contributes nothing to any offset
        const int kind = reduced[i] ? 1 : 0;
        if (kind == last_kind) {                         // same kind as the previous axis: adjacent in memory, merge
            if (kind) { f.rdim[f.nr - 1] *= dims[i]; f.rstr[f.nr - 1] = in_stride[i]; }
            else { f.kdim[f.nk - 1] *= dims[i]; f.kstr[f.nk - 1] = in_stride[i]; }
            b.dim[b.n - 1] *= dims[i];
            b.ostr[b.n - 1] = out_stride[i];
        } else {
            if (kind) { f.rdim[f.nr] = dims[i]; f.rstr[f.nr] = in_stride[i]; ++f.nr; }
            else { f.kdim[f.nk] = dims[i]; f.kstr[f.nk] = in_stride[i]; ++f.nk; }
            b.dim[b.n] = dims[i]; b.ostr[b.n] = out_stride[i]; ++b.n;
        }
        if (kind) f.n_red *= dims[i]; else f.n_out *= dims[i];
        last_kind = kind;
    }
    if (fwd) *fwd = f;
    if (bwd) *bwd = b;
    return true;
}

}  // namespace

size_t reduce_dims_scratch_elems() { return (size_t)1 << 22; }   // 16 MiB of partial results at most

// out[n_out] = reduction of x over the axes flagged in `reduced`.  op: 0 sum, 1 max, 2 min, 3 sum of squares,
// 4 sum of squared deviations from aux[output], 5 count of elements equal to aux[output].
bool reduce_dims(int op, const float* x, const float* aux, float* out, const size_t* dims, int rank, const unsigned char* reduced,
                 float* scratch, cudaStream_t s) {
    Plan p;
    if (!make_plans(dims, rank, reduced, &p, nullptr)) return false;
    size_t n_in = 1;
    for (int i = 0; i < rank; ++i) n_in *= dims[i];
    DeviceCtx* c = ctx();
    if (!c) return false;
    if (p.n_out == 0) return true;
    if (!out) { set_error("reduce_dims: null output"); return false; }
    if (n_in == 0 || p.n_red == 0) {   // nothing to accumulate: the identity of the operation
        return fill(out, op == kMax ? -INFINITY : op == kMin ? INFINITY : 0.0f, p.n_out, s);
    }
    if (!x || ((op == kSqDev || op == kCountEq) && !aux) || !scratch) { set_error("reduce_dims: null pointer"); return false; }
    ProfScope prof(kProfReduce, s, 4.0 * (double)n_in);
    const size_t se = reduce_dims_scratch_elems();
    switch (op) {
        case kSum: return launch_forward<kSum>(x, aux, out, p, scratch, se, c->sm_count, s);
        case kMax: return launch_forward<kMax>(x, aux, out, p, scratch, se, c->sm_count, s);
        case kMin: return launch_forward<kMin>(x, aux, out, p, scratch, se, c->sm_count, s);
        case kSumSq: return launch_forward<kSumSq>(x, aux, out, p, scratch, se, c->sm_count, s);
        case kSqDev: return launch_forward<kSqDev>(x, aux, out, p, scratch, se, c->sm_count, s);
        case kCountEq: return launch_forward<kCountEq>(x, aux, out, p, scratch, se, c->sm_count, s);
    }
    set_error("reduce_dims: unknown op %d", op);
    return false;
}

// gi[input] from go[output] (or the single value go[0] when go_is_scalar).  mode: 0 sum, 1 scaled sum (mean),
// 2 max/min (a1 = the extremum, a2 = how many elements equal it), 3 norm (a1 = norm), 4 var (a1 = mean, scale = 2/n),
// 5 std (a1 = mean, a2 = std, scale = 1/n).
bool reduce_dims_backward(int mode, const float* x, const float* a1, const float* a2, const float* go, float* gi, const size_t* dims,
                          int rank, const unsigned char* reduced, bool go_is_scalar, float scale, cudaStream_t s) {
    BwdPlan b;
    if (!make_plans(dims, rank, reduced, nullptr, &b)) return false;
    size_t n = 1;
    for (int i = 0; i < rank; ++i) n *= dims[i];
    if (n == 0) return true;
    if (!go || !gi || (mode >= kBwdExtremum && (!x || !a1)) || ((mode == kBwdExtremum || mode == kBwdStd) && !a2)) {
        set_error("reduce_dims_backward: null pointer");
        return false;
    }
    DeviceCtx* c = ctx();
    if (!c) return false;
    ProfScope prof(kProfElementwise, s, (mode >= kBwdExtremum ? 8.0 : 4.0) * (double)n);
    const size_t want = (n + kThreads - 1) / kThreads, cap = (size_t)c->sm_count * 16;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    const int gs = go_is_scalar ? 1 : 0;
    switch (mode) {
        case kBwdSum: launch_dep(reduce_bwd_kernel<kBwdSum>, dim3(grid), dim3(kThreads), 0, s, x, a1, a2, go, gi, n, b, gs, scale); break;
        case kBwdScaled: launch_dep(reduce_bwd_kernel<kBwdScaled>, dim3(grid), dim3(kThreads), 0, s, x, a1, a2, go, gi, n, b, gs, scale); break;
        case kBwdExtremum: launch_dep(reduce_bwd_kernel<kBwdExtremum>, dim3(grid), dim3(kThreads), 0, s, x, a1, a2, go, gi, n, b, gs, scale); break;
        case kBwdNorm: launch_dep(reduce_bwd_kernel<kBwdNorm>, dim3(grid), dim3(kThreads), 0, s, x, a1, a2, go, gi, n, b, gs, scale); break;
        case kBwdVar: launch_dep(reduce_bwd_kernel<kBwdVar>, dim3(grid), dim3(kThreads), 0, s, x, a1, a2, go, gi, n, b, gs, scale); break;
        case kBwdStd: launch_dep(reduce_bwd_kernel<kBwdStd>, dim3(grid), dim3(kThreads), 0, s, x, a1, a2, go, gi, n, b, gs, scale); break;
        default: set_error("reduce_dims_backward: unknown mode %d", mode); return false;
    }
    return cuda_ok(cudaGetLastError(), "reduce_dims backward launch");
}

}  // namespace k
}  // namespace ts

// ====================================================================== C ABI
using namespace ts;

static bool unpack(const unsigned long long* dims, int rank, const unsigned long long* axes, int n_axes, size_t* d, unsigned char* red,
                   const char* who) {
    if (rank < 1 || rank > 8 || !dims || (n_axes > 0 && !axes)) { set_error("%s: rank must be 1..8 and the tables non-null", who); return false; }
    for (int i = 0; i < rank; ++i) { d[i] = (size_t)dims[i]; red[i] = 0; }
    for (int i = 0; i < n_axes; ++i) {
        if (axes[i] >= (unsigned long long)rank) { set_error("%s: dim %llu out of bounds for rank %d", who, axes[i], rank); return false; }
        red[axes[i]] = 1;
    }
    return true;
}

TS_API unsigned long long ts_reduce_dims_scratch_elems(void) { return k::reduce_dims_scratch_elems(); }

TS_API bool launch_reduce_dims_kernel(int op, const float* x, const float* aux, float* out, const unsigned long long* dims, int rank,
                                      const unsigned long long* axes, int n_axes, float* scratch, void* stream) {
    cudaStream_t s = pick_stream(stream);
    if (!s) return false;
    size_t d[8];
    unsigned char red[8];
    if (!unpack(dims, rank, axes, n_axes, d, red, "launch_reduce_dims_kernel")) return false;
    return k::reduce_dims(op, x, aux, out, d, rank, red, scratch, s);
}

TS_API bool launch_reduce_dims_backward_kernel(int mode, const float* x, const float* a1, const float* a2, const float* grad_out, float* grad_in,
                                               const unsigned long long* dims, int rank, const unsigned long long* axes, int n_axes,
                                               int grad_out_is_scalar, float scale, void* stream) {
    cudaStream_t s = pick_stream(stream);
    if (!s) return false;
    size_t d[8];
    unsigned char red[8];
    if (!unpack(dims, rank, axes, n_axes, d, red, "launch_reduce_dims_backward_kernel")) return false;
    return k::reduce_dims_backward(mode, x, a1, a2, grad_out, grad_in, d, rank, red, grad_out_is_scalar != 0, scale, s);
}
