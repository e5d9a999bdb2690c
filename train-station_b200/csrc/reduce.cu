// Reductions: full-tensor sum / mean (and the fused MSE loss), column sums for bias
// gradients, and the fused ReLU-backward + column-sum.  All are HBM-bound single passes
// over the data followed by a tiny second stage; both stages add in a fixed order, so
// results are deterministic run to run.  The reference adds sequentially in f32
// (reductions/sum.rs:93-105, :255-290); a tree differs from that in the last bits and is
// closer to the exact sum.
#include "../../include/train_station_b200.h"
#include "common.h"

namespace ts {
namespace k {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide sum; the result is valid in thread 0.
__device__ __forceinline__ float block_sum(float v) {
    __shared__ float sm[kThreads / 32];
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
    if (threadIdx.x < 32) {
        r = threadIdx.x < kThreads / 32 ? sm[threadIdx.x] : 0.0f;
        r = warp_sum(r);
    }
    __syncthreads();
    return r;
}

// MODE 0: sum(x); MODE 1: sum((x-y)^2)
template <int MODE>
__global__ void __launch_bounds__(kThreads) sum_stage1(const float* __restrict__ x, const float* __restrict__ y,
                                                       float* __restrict__ partial, size_t n, int vec_ok, float* __restrict__ out,
                                                       float divisor) {
    grid_dependency_sync();
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const size_t tid = (size_t)blockIdx.x * kThreads + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * kThreads;
    if (vec_ok) {
        const size_t n_vec = n / 4;
        const float4* xv = reinterpret_cast<const float4*>(x);
        const float4* yv = reinterpret_cast<const float4*>(y);
        size_t i = tid;
        // four independent loads in flight per thread
        for (; i + 3 * nthreads < n_vec; i += 4 * nthreads) {
            float4 a[4], b[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) a[u] = __ldcs(xv + i + u * nthreads);
            if (MODE == 1) {
#pragma unroll
                for (int u = 0; u < 4; ++u) b[u] = __ldcs(yv + i + u * nthreads);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (MODE == 1) {
                    float d0 = __fsub_rn(a[u].x, b[u].x), d1 = __fsub_rn(a[u].y, b[u].y);
                    float d2 = __fsub_rn(a[u].z, b[u].z), d3 = __fsub_rn(a[u].w, b[u].w);
                    acc[0] += __fmul_rn(d0, d0); acc[1] += __fmul_rn(d1, d1);
                    acc[2] += __fmul_rn(d2, d2); acc[3] += __fmul_rn(d3, d3);
                } else {
                    acc[0] += a[u].x; acc[1] += a[u].y; acc[2] += a[u].z; acc[3] += a[u].w;
                }
            }
        }
        for (; i < n_vec; i += nthreads) {
            float4 a = __ldcs(xv + i);
            if (MODE == 1) {
                float4 b = __ldcs(yv + i);
                float d0 = __fsub_rn(a.x, b.x), d1 = __fsub_rn(a.y, b.y), d2 = __fsub_rn(a.z, b.z), d3 = __fsub_rn(a.w, b.w);
                acc[0] += __fmul_rn(d0, d0); acc[1] += __fmul_rn(d1, d1); acc[2] += __fmul_rn(d2, d2); acc[3] += __fmul_rn(d3, d3);
            } else {
                acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
            }
        }
        size_t t = n_vec * 4 + tid;   // n mod 4 leftovers
        if (t < n) {
            float a = x[t];
            if (MODE == 1) { float d = __fsub_rn(a, y[t]); a = __fmul_rn(d, d); }
            acc[0] += a;
        }
    } else {
        for (size_t i = tid; i < n; i += nthreads) {
            float a = x[i];
            if (MODE == 1) { float d = __fsub_rn(a, y[i]); a = __fmul_rn(d, d); }
            acc[0] += a;
        }
    }
    float v = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    v = block_sum(v);
    if (threadIdx.x != 0) return;
    // a single CTA already holds the whole sum: the second stage (which would add 0s to it) is skipped
    if (gridDim.x == 1) out[0] = divisor > 0.0f ? __fdiv_rn(v, divisor) : v;
    else partial[blockIdx.x] = v;
}

__global__ void __launch_bounds__(kThreads) sum_stage2(const float* __restrict__ partial, int n_partial, float* __restrict__ out,
                                                       float divisor) {
    grid_dependency_sync();
    float v = 0.0f;
    for (int i = threadIdx.x; i < n_partial; i += kThreads) v += partial[i];
    v = block_sum(v);
    if (threadIdx.x == 0) out[0] = divisor > 0.0f ? __fdiv_rn(v, divisor) : v;
}

template <int MODE>
bool sum_impl(const float* x, const float* y, float* out, size_t n, bool mean, float* scratch, cudaStream_t s) {
    if (!out) { set_error("sum: null output"); return false; }
    DeviceCtx* c = ctx();
    if (!c) return false;
    if (n == 0) return fill(out, 0.0f, 1, s);   // sum.rs:82-83 / mean.rs:50-52: empty -> 0
    if (!x || (MODE == 1 && !y) || !scratch) { set_error("sum: null pointer"); return false; }
    size_t per_cta = (size_t)kThreads * 16;
    size_t want = (n + per_cta - 1) / per_cta;
    size_t cap = (size_t)c->sm_count * 4;
    if (cap > kReduceScratchElems) cap = kReduceScratchElems;
    int grid = (int)(want < cap ? want : cap);
    int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && (MODE == 0 || (reinterpret_cast<uintptr_t>(y) & 15) == 0);
    const float divisor = mean ? (float)n : 0.0f;
    ProfScope prof(kProfReduce, s, 4.0 * (double)n * (MODE == 1 ? 2 : 1), grid == 1 ? 1 : 2);
    launch_dep(sum_stage1<MODE>, dim3(grid), dim3(kThreads), 0, s, x, y, scratch, n, vec_ok, out, divisor);
    if (grid > 1) launch_dep(sum_stage2, dim3(1), dim3(kThreads), 0, s, scratch, grid, out, divisor);
    return cuda_ok(cudaGetLastError(), "sum launch");
}

// ---------------------------------------------------------------- column sums
// CTA = 32 column lanes x 8 row lanes; a column lane owns 4 adjacent columns (one float4).
constexpr int kColLanes = 32, kRowLanes = 8, kTileCols = kColLanes * 4;

struct ColsumPlan { int col_tiles; int splits; size_t rows_per_split; bool vec; };

ColsumPlan plan_colsum(size_t rows, size_t cols, int sm_count, bool aligned) {
    ColsumPlan p;
    p.vec = aligned && (cols % 4 == 0);
    size_t tile = p.vec ? kTileCols : kColLanes;
    p.col_tiles = (int)((cols + tile - 1) / tile);
    // Four CTAs of this kernel are resident per SM (64 registers x 256 threads).  Rounding the split count down
    // keeps the grid within one wave; rounding up left a second, nearly empty wave (640 CTAs on 592 slots for
    // 8192 columns) and held the kernel at 64 % of DRAM bandwidth.
    size_t target = (size_t)sm_count * 4;
    size_t s = target / p.col_tiles;
    size_t max_s = (rows + 63) / 64;            // at least 64 rows per split
    if (s > max_s) s = max_s;
    if (s < 1) s = 1;
    if (s > 1024) s = 1024;
    p.rows_per_split = (rows + s - 1) / s;
    p.splits = (int)((rows + p.rows_per_split - 1) / p.rows_per_split);
    return p;
}

// What stage 1 sums.  Plain: the columns of g.  ReluBwd: gi = ref > 0 ? g : 0 is written and its columns summed.
// MseGrad: gi = (inv_n * *upstream) * (2 * (g - ref)), optionally rounded to TF32, is written and its columns summed:
// the gradient of mean((y - t)^2) with respect to y and, in the same pass, of the bias that was added to make y
// (the operations and their order are those of the stand-alone gradient kernel, so the bits are the same).
enum ColsumMode { kColsumPlain = 0, kColsumReluBwd = 1, kColsumMseGrad = 2 };
struct ColsumExtra { const float* upstream; float inv_n; int round_tf32; };

template <int MODE>
__device__ __forceinline__ float colsum_value(float g, float ref, float sc, int round_tf32) {
    if (MODE == kColsumReluBwd) return ref > 0.0f ? g : 0.0f;
    if (MODE == kColsumMseGrad) {
        float v = __fmul_rn(sc, __fmul_rn(2.0f, __fsub_rn(g, ref)));
        if (round_tf32) {
            uint32_t r;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
            v = __uint_as_float(r);
        }
        return v;
    }
    return g;
}

template <int MODE, bool VEC>
__global__ void __launch_bounds__(kThreads) colsum_stage1(const float* __restrict__ g, const float* __restrict__ ref,
                                                          float* __restrict__ gi, float* __restrict__ partial, size_t rows,
                                                          size_t cols, size_t rows_per_split, ColsumExtra ex) {
    grid_dependency_sync();
    constexpr bool FUSED = MODE != kColsumPlain;
    const int cl = threadIdx.x % kColLanes, rl = threadIdx.x / kColLanes;
    const size_t r0 = (size_t)blockIdx.y * rows_per_split;
    size_t r1 = r0 + rows_per_split;
    if (r1 > rows) r1 = rows;
    const float sc = MODE == kColsumMseGrad ? __fmul_rn(ex.inv_n, __ldg(ex.upstream)) : 0.0f;
    __shared__ float4 sm[kRowLanes][kColLanes];
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (VEC) {
        const size_t col = ((size_t)blockIdx.x * kColLanes + cl) * 4;
        if (col < cols) {
            size_t r = r0 + rl;
            if (!FUSED) {
                // four rows in flight per thread: the plain column sum has nothing else to hide latency with
                for (; r + 3 * kRowLanes < r1; r += 4 * kRowLanes) {
                    float4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) v[u] = __ldcs(reinterpret_cast<const float4*>(g) + ((r + u * kRowLanes) * cols + col) / 4);
#pragma unroll
                    for (int u = 0; u < 4; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
                }
            }
            for (; r < r1; r += kRowLanes) {
                size_t off = (r * cols + col) / 4;
                float4 v = __ldcs(reinterpret_cast<const float4*>(g) + off);
                if (FUSED) {
                    float4 x = __ldcs(reinterpret_cast<const float4*>(ref) + off);
                    v.x = colsum_value<MODE>(v.x, x.x, sc, ex.round_tf32); v.y = colsum_value<MODE>(v.y, x.y, sc, ex.round_tf32);
                    v.z = colsum_value<MODE>(v.z, x.z, sc, ex.round_tf32); v.w = colsum_value<MODE>(v.w, x.w, sc, ex.round_tf32);
                    __stcs(reinterpret_cast<float4*>(gi) + off, v);
                }
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        }
    } else {
        const size_t col = (size_t)blockIdx.x * kColLanes + cl;
        if (col < cols) {
            for (size_t r = r0 + rl; r < r1; r += kRowLanes) {
                size_t off = r * cols + col;
                float v = g[off];
                if (FUSED) { v = colsum_value<MODE>(v, ref[off], sc, ex.round_tf32); gi[off] = v; }
                acc.x += v;
            }
        }
    }
    sm[rl][cl] = acc;
    __syncthreads();
    if (rl == 0) {
        float4 t = sm[0][cl];
#pragma unroll
        for (int i = 1; i < kRowLanes; ++i) { float4 u = sm[i][cl]; t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w; }
        float* dst = partial + (size_t)blockIdx.y * cols;
        if (VEC) {
            const size_t col = ((size_t)blockIdx.x * kColLanes + cl) * 4;
            if (col < cols) { dst[col] = t.x; dst[col + 1] = t.y; dst[col + 2] = t.z; dst[col + 3] = t.w; }
        } else {
            const size_t col = (size_t)blockIdx.x * kColLanes + cl;
            if (col < cols) dst[col] = t.x;
        }
    }
}

__global__ void __launch_bounds__(kThreads) colsum_stage2(const float* __restrict__ partial, float* __restrict__ out, size_t cols,
                                                          int splits) {
    grid_dependency_sync();
    size_t col = (size_t)blockIdx.x * kThreads + threadIdx.x;
    if (col >= cols) return;
    float v = 0.0f;
    for (int s = 0; s < splits; ++s) v += partial[(size_t)s * cols + col];
    out[col] = v;
}

// Adds the rows of a [rows][cols] matrix of partial sums (thousands of rows when they come from a GEMM epilogue: one per
// 32 result rows).  One CTA per 32 columns, so that 8192 columns occupy the whole GPU instead of 32 CTAs: lane = column
// (a warp reads 128 contiguous bytes per row), the 8 warps take rows w, w + 8, ... with four loads in flight, and the 8
// warp totals are added in warp order.  The order of additions is fixed, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256) colsum_rows_kernel(const float* __restrict__ part, float* __restrict__ out, size_t cols, int rows) {
    grid_dependency_sync();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const size_t col = (size_t)blockIdx.x * 32 + lane;
    __shared__ float sm[8][32];
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    if (col < cols) {
        int r = w;
        for (; r + 24 < rows; r += 32) {
            const float v0 = __ldcs(part + (size_t)r * cols + col), v1 = __ldcs(part + (size_t)(r + 8) * cols + col);
            const float v2 = __ldcs(part + (size_t)(r + 16) * cols + col), v3 = __ldcs(part + (size_t)(r + 24) * cols + col);
            a0 += v0; a1 += v1; a2 += v2; a3 += v3;
        }
        for (; r < rows; r += 8) a0 += __ldcs(part + (size_t)r * cols + col);
    }
    sm[w][lane] = (a0 + a1) + (a2 + a3);
    __syncthreads();
    if (w == 0 && col < cols) {
        float t = sm[0][lane];
#pragma unroll
        for (int i = 1; i < 8; ++i) t += sm[i][lane];
        out[col] = t;
    }
}

template <int MODE>
bool colsum_impl(const float* g, const float* ref, float* gi, float* out, size_t rows, size_t cols, float* scratch, cudaStream_t s,
                 ColsumExtra ex = ColsumExtra{nullptr, 0.0f, 0}) {
    constexpr bool FUSED = MODE != kColsumPlain;
    if (cols == 0) return true;
    if (!out) { set_error("colsum: null output"); return false; }
    DeviceCtx* c = ctx();
    if (!c) return false;
    if (rows == 0) return fill(out, 0.0f, cols, s);
    if (!g || (FUSED && (!ref || !gi)) || (MODE == kColsumMseGrad && !ex.upstream)) { set_error("colsum: null pointer"); return false; }
    bool aligned = (reinterpret_cast<uintptr_t>(g) & 15) == 0 &&
                   (!FUSED || ((reinterpret_cast<uintptr_t>(ref) & 15) == 0 && (reinterpret_cast<uintptr_t>(gi) & 15) == 0));
    ColsumPlan p = plan_colsum(rows, cols, c->sm_count, aligned);
    if (p.splits > 1 && !scratch) { set_error("colsum: scratch buffer required"); return false; }
    float* partial = p.splits > 1 ? scratch : out;
    dim3 grid(p.col_tiles, p.splits);
    ProfScope prof(kProfReduce, s, 4.0 * (double)rows * (double)cols * (FUSED ? 3 : 1), p.splits > 1 ? 2 : 1);
    if (p.vec) launch_dep(colsum_stage1<MODE, true>, grid, dim3(kThreads), 0, s, g, ref, gi, partial, rows, cols, p.rows_per_split, ex);
    else launch_dep(colsum_stage1<MODE, false>, grid, dim3(kThreads), 0, s, g, ref, gi, partial, rows, cols, p.rows_per_split, ex);
    if (p.splits > 1) launch_dep(colsum_stage2, dim3((unsigned)((cols + kThreads - 1) / kThreads)), dim3(kThreads), 0, s, partial, out, cols, (int)p.splits);
    return cuda_ok(cudaGetLastError(), "colsum launch");
}

}  // namespace

bool sum(const float* x, float* out, size_t n, bool mean, float* scratch, cudaStream_t s) {
    return sum_impl<0>(x, nullptr, out, n, mean, scratch, s);
}
bool mse_loss(const float* y, const float* t, float* out, size_t n, float* scratch, cudaStream_t s) {
    return sum_impl<1>(y, t, out, n, true, scratch, s);
}

size_t colsum_scratch_elems(size_t rows, size_t cols) {
    // Upper bound over every plan: at most 1024 row splits, and never more than rows/64 + 1.
    size_t s = (rows + 63) / 64;
    if (s > 1024) s = 1024;
    if (s < 1) s = 1;
    return s * cols;
}
bool colsum(const float* g, float* out, size_t rows, size_t cols, float* scratch, cudaStream_t s) {
    return colsum_impl<kColsumPlain>(g, nullptr, nullptr, out, rows, cols, scratch, s);
}
bool colsum_finish(const float* partial, float* out, size_t cols, size_t partial_rows, cudaStream_t s) {
    if (cols == 0) return true;
    if (!partial || !out || partial_rows == 0 || partial_rows > 0x7fffffff) { set_error("colsum_finish: bad arguments"); return false; }
    ProfScope prof(kProfReduce, s, 4.0 * (double)cols * (double)(partial_rows + 1));
    launch_dep(colsum_rows_kernel, dim3((unsigned)((cols + 31) / 32)), dim3(256), 0, s, partial, out, cols, (int)partial_rows);
    return cuda_ok(cudaGetLastError(), "colsum_finish launch");
}
bool relu_bwd_colsum(const float* ref, const float* go, float* gi, float* bias_grad, size_t rows, size_t cols, float* scratch,
                     cudaStream_t s) {
    return colsum_impl<kColsumReluBwd>(go, ref, gi, bias_grad, rows, cols, scratch, s);
}
bool mse_grad_colsum(const float* y, const float* t, const float* upstream, float inv_n, float* gy, float* bias_grad, size_t rows,
                     size_t cols, bool round_tf32, float* scratch, cudaStream_t s) {
    return colsum_impl<kColsumMseGrad>(y, t, gy, bias_grad, rows, cols, scratch, s, ColsumExtra{upstream, inv_n, round_tf32 ? 1 : 0});
}

}  // namespace k
}  // namespace ts

// ====================================================================== C ABI
using namespace ts;

TS_API unsigned long long ts_reduce_scratch_elems(void) { return k::kReduceScratchElems; }
TS_API bool launch_sum_kernel(const float* x, float* out, unsigned long long n, int mean, float* scratch, void* stream) {
    cudaStream_t s = pick_stream(stream);
    if (!s) return false;
    return k::sum(x, out, n, mean != 0, scratch, s);
}
TS_API unsigned long long ts_colsum_scratch_elems(unsigned long long rows, unsigned long long cols) {
    return k::colsum_scratch_elems(rows, cols);
}
TS_API bool launch_colsum_kernel(const float* g, float* out, unsigned long long rows, unsigned long long cols, float* scratch,
                                 void* stream) {
    cudaStream_t s = pick_stream(stream);
    if (!s) return false;
    return k::colsum(g, out, rows, cols, scratch, s);
}
TS_API bool launch_relu_backward_colsum_kernel(const float* ref, const float* go, float* gi, float* bias_grad,
                                               unsigned long long rows, unsigned long long cols, float* scratch, void* stream) {
    cudaStream_t s = pick_stream(stream);
    if (!s) return false;
    return k::relu_bwd_colsum(ref, go, gi, bias_grad, rows, cols, scratch, s);
}

// ---------------------------------------------------------------------------------------------
// Column sum for callers that must not allocate.
//
// Some hosts of this library cannot obtain device memory at the moment they need a bias gradient:
// a plugin that runs inside another framework's memory budget and may not grow it, a service whose
// device memory was carved up at start-up and is now fully handed out, or a latency-bound loop in
// which a call into the driver's allocator (which may synchronise the device) is not acceptable.
// launch_colsum_kernel asks such callers for a scratch buffer they have no way to provide.
// The first call on a device performs the symbol look-up below: make it before any stream capture.
//
// This variant keeps the scratch (the per-row-split partial sums) in a fixed array that is part of
// the library image: every GPU that loads the library holds these 512 KiB until the process exits.
// The array's name below is, in host code, only a handle of the host-side shadow of the symbol, not
// a device address; the device address is obtained once per device with cudaGetSymbolAddress while
// that device is current, and that pointer is what the kernels receive.
constexpr size_t kStaticColsumScratchElems = size_t(1) << 17;   // 131072 floats = 512 KiB
static __device__ __align__(256) float g_colsum_static_scratch[kStaticColsumScratchElems];
static float* g_colsum_static_ptr[64] = {nullptr};   // per device, filled at the first call on that device
static std::mutex g_colsum_static_mu;

TS_API bool launch_colsum_kernel_static_scratch(const float* g, float* out, unsigned long long rows, unsigned long long cols,
                                                void* stream) {
    // The library must already be initialised on this device (cuda_ffi_initialize or any earlier call):
    // creating the per-device context allocates, and this entry point must not.
    DeviceCtx* c = ctx_if_initialized();
    if (!c) {
        set_error("launch_colsum_kernel_static_scratch: the library is not initialised on the current device; call "
                  "cuda_ffi_initialize() first (this entry point never allocates, so it cannot do that itself)");
        return false;
    }
    cudaStream_t s = stream ? (cudaStream_t)stream : c->compute;
    if (cols == 0) return true;
    if (!out || (rows && !g)) { set_error("launch_colsum_kernel_static_scratch: null pointer"); return false; }
    bool aligned = (reinterpret_cast<uintptr_t>(g) & 15) == 0;
    k::ColsumPlan p = k::plan_colsum((size_t)rows ? (size_t)rows : 1, (size_t)cols, c->sm_count, aligned);
    size_t need = p.splits > 1 ? (size_t)p.splits * (size_t)cols : 0;
    if (need > kStaticColsumScratchElems) {
        set_error("launch_colsum_kernel_static_scratch: a %llu x %llu column sum needs %zu scratch elements, the built-in scratch holds "
                  "%zu; use launch_colsum_kernel with a caller-provided buffer", rows, cols, need, kStaticColsumScratchElems);
        return false;
    }
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_colsum_static_mu);
        if (!g_colsum_static_ptr[c->device]) {
            // one-time set-up for this device (which ctx_if_initialized made current): resolve the symbol
            void* p_dev = nullptr;
            if (!cuda_ok(cudaGetSymbolAddress(&p_dev, g_colsum_static_scratch), "cudaGetSymbolAddress(static colsum scratch)")) return false;
            g_colsum_static_ptr[c->device] = (float*)p_dev;
        }
        scratch = g_colsum_static_ptr[c->device];
    }
    // Every partial the second stage reads is written by the first stage of the same call, so nothing in the
    // array has to start at zero and stale contents of an earlier call are never read.
    // With ts_profile_enable(1) a launch is normally bracketed by two events, and creating an event allocates:
    // here the launch is only counted.
    ProfSuspend no_events;
    return k::colsum(g, out, rows, cols, scratch, s);
}
