// softmax over the middle axis of a contiguous [outer, reduce, inner] tensor, forward and backward.
// HBM-bound: 8 bytes per element forward (read x, write y), 12 backward (read y and go, write gi).  Every
// mapping below reads its inputs from HBM once: a line's values stay in registers (or in shared memory for
// very short rows) between the max / sum / scale sweeps, and the loads of the NEXT line are issued before the
// current one is reduced, so that a CTA always has a line in flight.
//
// Reference: tensor/ops/softmax.rs:110-158 (max; e = exp(x - max), summed; y = e * (1/sum)) and
// gradtrack/grad_fn/ops/softmax.rs:4-35 (dot = sum_j go*y; gi = y * (go - dot)).  The reference adds the terms
// of a line sequentially; here a line's sum is a fixed tree over the threads that share it (deterministic,
// and closer to the exact sum than the sequential chain), except for rows of at most 32 elements, which one
// thread sums in the reference's order.
//
// Mappings:
//  * rows (inner == 1, reduce > 32): G threads share a row and keep 8 elements each; G = 32 ... 1024 by row
//    length (several rows per CTA while G < 256), so rows up to 8192 elements are register-resident.
//    Longer rows fall back to three sweeps over global memory (the second and third hit L2).
//  * short rows (inner == 1, reduce <= 32): a CTA stages 256 rows through shared memory with coalesced copies,
//    transposed and padded so that both the copy and the per-row sweep are free of bank conflicts.
//  * columns (inner > 1): when inner is a multiple of 4 (16-byte rows), a CTA streams whole [reduce][TI] tiles of
//    32, 64 or 128 neighbouring lines into shared memory with asynchronous 16-byte copies, double-buffered, and
//    its 512 threads split the reduced axis (the tile limit is 200 KB of shared memory: lines up to about 780
//    elements).  Otherwise a CTA owns 32 neighbouring lines, its W warps (8, 16 or 32 by line length) hold 8
//    elements per thread in registers and combine through shared memory; lines longer than 256 elements then take
//    the three-sweep fallback.
#include <cfloat>

#include "../../include/train_station_b200.h"
#include "common.h"

namespace ts {
namespace k {

namespace {

constexpr int kV = 8;             // elements of a line one thread keeps in registers
constexpr int kShortMax = 32;     // rows up to this length take the shared-memory path
constexpr int kShortThreads = 256;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}
// Combines one value per thread over the G consecutive threads that share a row.  Groups wider than a warp go
// through `red` (one float per warp of the CTA); every thread of the CTA must call it.
template <int G, bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, float* red) {
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    if (G == 32) return v;
    constexpr int WG = G / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int first = (warp / WG) * WG;
    float r = red[first];
#pragma unroll
    for (int w = 1; w < WG; ++w) r = IS_MAX ? fmaxf(r, red[first + w]) : __fadd_rn(r, red[first + w]);
    __syncthreads();
    return r;
}

template <int G>
struct RowsCfg {
    static constexpr int kCta = G > 256 ? G : 256;
    static constexpr int kRpc = kCta / G;   // rows per CTA
};

// ------------------------------------------------------------------ rows: inner == 1, reduce > 32
template <int G, bool CACHED>
__global__ void __launch_bounds__(RowsCfg<G>::kCta) softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ y, size_t rows,
                                                                        size_t reduce) {
    grid_dependency_sync();
    constexpr int RPC = RowsCfg<G>::kRpc;
    __shared__ float red[32];
    const int g = threadIdx.x / G, t = threadIdx.x % G;
    const size_t step = (size_t)gridDim.x * RPC;
    float nx[kV];
    auto load = [&](size_t r0) {
        const size_t row = r0 + g;
#pragma unroll
        for (int k = 0; k < kV; ++k) {
            const size_t j = (size_t)t + (size_t)k * G;
            nx[k] = (row < rows && j < reduce) ? __ldcs(x + row * reduce + j) : -INFINITY;
        }
    };
    size_t row0 = (size_t)blockIdx.x * RPC;
    if (CACHED && row0 < rows) load(row0);
    for (; row0 < rows; row0 += step) {
        const size_t row = row0 + g;
        const bool active = row < rows;
        const float* xr = x + row * reduce;
        float* yr = y + row * reduce;
        float v[kV];
        float mx = -INFINITY;
        if (CACHED) {
#pragma unroll
            for (int k = 0; k < kV; ++k) v[k] = nx[k];
            if (row0 + step < rows) load(row0 + step);
#pragma unroll
            for (int k = 0; k < kV; ++k) if (v[k] > mx) mx = v[k];   // a NaN never compares greater (softmax.rs:136-138)
        } else if (active) {
            for (size_t j = t; j < reduce; j += G) { float a = xr[j]; if (a > mx) mx = a; }
        }
        mx = group_reduce<G, true>(mx, red);
        float sum = 0.0f;
        if (CACHED) {
#pragma unroll
            for (int k = 0; k < kV; ++k) {
                const size_t j = (size_t)t + (size_t)k * G;
                v[k] = (active && j < reduce) ? expf(__fsub_rn(v[k], mx)) : 0.0f;
                sum = __fadd_rn(sum, v[k]);
            }
        } else if (active) {
            for (size_t j = t; j < reduce; j += G) sum = __fadd_rn(sum, expf(__fsub_rn(xr[j], mx)));
        }
        sum = group_reduce<G, false>(sum, red);
        const float inv = __fdiv_rn(1.0f, sum);
        if (CACHED) {
#pragma unroll
            for (int k = 0; k < kV; ++k) {
                const size_t j = (size_t)t + (size_t)k * G;
                if (active && j < reduce) __stcs(yr + j, __fmul_rn(v[k], inv));
            }
        } else if (active) {
            for (size_t j = t; j < reduce; j += G) yr[j] = __fmul_rn(expf(__fsub_rn(xr[j], mx)), inv);
        }
    }
}

template <int G, bool CACHED>
__global__ void __launch_bounds__(RowsCfg<G>::kCta) softmax_bwd_rows_kernel(const float* __restrict__ y, const float* __restrict__ go,
                                                                            float* __restrict__ gi, size_t rows, size_t reduce) {
    grid_dependency_sync();
    constexpr int RPC = RowsCfg<G>::kRpc;
    __shared__ float red[32];
    const int g = threadIdx.x / G, t = threadIdx.x % G;
    const size_t step = (size_t)gridDim.x * RPC;
    float ny[kV], ng[kV];
    auto load = [&](size_t r0) {
        const size_t row = r0 + g;
#pragma unroll
        for (int k = 0; k < kV; ++k) {
            const size_t j = (size_t)t + (size_t)k * G;
            const bool in = row < rows && j < reduce;
            ny[k] = in ? __ldcs(y + row * reduce + j) : 0.0f;
            ng[k] = in ? __ldcs(go + row * reduce + j) : 0.0f;
        }
    };
    size_t row0 = (size_t)blockIdx.x * RPC;
    if (CACHED && row0 < rows) load(row0);
    for (; row0 < rows; row0 += step) {
        const size_t row = row0 + g;
        const bool active = row < rows;
        const float* yr = y + row * reduce;
        const float* gr = go + row * reduce;
        float* out = gi + row * reduce;
        float vy[kV], vg[kV];
        float dot = 0.0f;
        if (CACHED) {
#pragma unroll
            for (int k = 0; k < kV; ++k) { vy[k] = ny[k]; vg[k] = ng[k]; }
            if (row0 + step < rows) load(row0 + step);
#pragma unroll
            for (int k = 0; k < kV; ++k) dot = __fadd_rn(dot, __fmul_rn(vg[k], vy[k]));
        } else if (active) {
            for (size_t j = t; j < reduce; j += G) dot = __fadd_rn(dot, __fmul_rn(gr[j], yr[j]));
        }
        dot = group_reduce<G, false>(dot, red);
        if (CACHED) {
#pragma unroll
            for (int k = 0; k < kV; ++k) {
                const size_t j = (size_t)t + (size_t)k * G;
                if (active && j < reduce) __stcs(out + j, __fmul_rn(vy[k], __fsub_rn(vg[k], dot)));
            }
        } else if (active) {
            for (size_t j = t; j < reduce; j += G) out[j] = __fmul_rn(yr[j], __fsub_rn(gr[j], dot));
        }
    }
}

// ------------------------------------------------------------------ short rows: inner == 1, reduce <= 32
// Element (r, j) of a TR-row tile sits at j * (TR + 1) + r: consecutive elements of the copy (same r, j + 1) and
// consecutive rows of the sweep (same j, r + 1) both fall into different banks.  A thread's elements of a tile
// are e = tid + u * 256; NU of them cover TR * 32 elements.
template <int TR, int NU>
struct ShortTile {
    __device__ static void fetch(float* regs, const float* src, int nelem) {
#pragma unroll
        for (int u = 0; u < NU; ++u) {
            const int e = threadIdx.x + u * kShortThreads;
            regs[u] = e < nelem ? __ldcs(src + e) : 0.0f;
        }
    }
    __device__ static void put(float* tile, const float* regs, int nelem, int reduce) {
        int r = threadIdx.x / reduce, j = threadIdx.x % reduce;
        const int dr = kShortThreads / reduce, dj = kShortThreads % reduce;
#pragma unroll
        for (int u = 0; u < NU; ++u) {
            const int e = threadIdx.x + u * kShortThreads;
            if (e < nelem) tile[j * (TR + 1) + r] = regs[u];
            j += dj; r += dr;
            if (j >= reduce) { j -= reduce; ++r; }
        }
    }
    __device__ static void store(const float* tile, float* dst, int nelem, int reduce) {
        int r = threadIdx.x / reduce, j = threadIdx.x % reduce;
        const int dr = kShortThreads / reduce, dj = kShortThreads % reduce;
#pragma unroll
        for (int u = 0; u < NU; ++u) {
            const int e = threadIdx.x + u * kShortThreads;
            if (e < nelem) __stcs(dst + e, tile[j * (TR + 1) + r]);
            j += dj; r += dr;
            if (j >= reduce) { j -= reduce; ++r; }
        }
    }
};

template <int RMAX>   // reduce <= RMAX: sizes the staging tile and the prefetch registers
__global__ void __launch_bounds__(kShortThreads) softmax_short_kernel(const float* __restrict__ x, float* __restrict__ y, size_t rows, int reduce) {
    grid_dependency_sync();
    constexpr int TR = 256, NU = TR * RMAX / kShortThreads;
    using Tile = ShortTile<TR, NU>;
    __shared__ float tile[RMAX * (TR + 1)];
    const size_t step = (size_t)gridDim.x * TR;
    auto count = [&](size_t r0) { return (int)(rows - r0 < (size_t)TR ? rows - r0 : TR) * reduce; };
    float nx[NU];
    size_t row0 = (size_t)blockIdx.x * TR;
    if (row0 < rows) Tile::fetch(nx, x + row0 * reduce, count(row0));
    for (; row0 < rows; row0 += step) {
        const int nelem = count(row0), nrows = nelem / reduce;
        Tile::put(tile, nx, nelem, reduce);
        __syncthreads();
        if (row0 + step < rows) Tile::fetch(nx, x + (row0 + step) * reduce, count(row0 + step));
        if ((int)threadIdx.x < nrows) {
            // the row lives in registers between its one read and one write of the tile
            float* col = tile + threadIdx.x;
            float v[RMAX];
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < RMAX; ++j) {
                v[j] = j < reduce ? col[j * (TR + 1)] : -INFINITY;
                if (v[j] > mx) mx = v[j];
            }
            float sum = 0.0f;   // sequential, the reference's order
#pragma unroll
            for (int j = 0; j < RMAX; ++j) {
                if (j < reduce) {
                    v[j] = expf(__fsub_rn(v[j], mx));
                    sum = __fadd_rn(sum, v[j]);
                }
            }
            const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
            for (int j = 0; j < RMAX; ++j)
                if (j < reduce) col[j * (TR + 1)] = __fmul_rn(v[j], inv);
        }
        __syncthreads();
        Tile::store(tile, y + row0 * reduce, nelem, reduce);
        __syncthreads();
    }
}

// Row lengths whose stride over the 32 shared-memory banks repeats at most every second lane (odd lengths and
// 2 x odd: 10 classes among them): a warp owns 32 consecutive rows, which are one contiguous run of 32 x reduce floats.
// It copies the run into its own staging area with coalesced 128-bit loads, every lane reads its row from there at the
// row's natural pitch (no transposition, at most 2-way bank conflicts), writes the result back in place, and the warp
// streams the run out again.  No block-wide barrier: the staging area is private to the warp.
template <int RMAX>
__global__ void __launch_bounds__(kShortThreads) softmax_short_warp_kernel(const float* __restrict__ x, float* __restrict__ y, size_t rows,
                                                                          int reduce) {
    grid_dependency_sync();
    __shared__ __align__(16) float stage[kShortThreads / 32][32 * RMAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* st = stage[warp];
    const size_t n_warps = (size_t)gridDim.x * (kShortThreads / 32);
    const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    for (size_t w = (size_t)blockIdx.x * (kShortThreads / 32) + warp; w * 32 < rows; w += n_warps) {
        const size_t r0 = w * 32;
        const int nrows = rows - r0 < 32 ? (int)(rows - r0) : 32, nelem = nrows * reduce;
        const float* src = x + r0 * reduce;      // r0 is a multiple of 32: the run starts 16-byte aligned when x does
        float* dst = y + r0 * reduce;
        const int nvec = al ? nelem / 4 : 0;
        for (int e = lane; e < nvec; e += 32) reinterpret_cast<float4*>(st)[e] = __ldcs(reinterpret_cast<const float4*>(src) + e);
        for (int e = nvec * 4 + lane; e < nelem; e += 32) st[e] = __ldcs(src + e);
        __syncwarp();
        if (lane < nrows) {
            float* row = st + lane * reduce;
            float v[RMAX];
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < RMAX; ++j) {
                v[j] = j < reduce ? row[j] : -INFINITY;
                if (v[j] > mx) mx = v[j];
            }
            float sum = 0.0f;   // sequential, the reference's order
#pragma unroll
            for (int j = 0; j < RMAX; ++j) {
                if (j < reduce) {
                    v[j] = expf(__fsub_rn(v[j], mx));
                    sum = __fadd_rn(sum, v[j]);
                }
            }
            const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
            for (int j = 0; j < RMAX; ++j)
                if (j < reduce) row[j] = __fmul_rn(v[j], inv);
        }
        __syncwarp();
        for (int e = lane; e < nvec; e += 32) __stcs(reinterpret_cast<float4*>(dst) + e, reinterpret_cast<const float4*>(st)[e]);
        for (int e = nvec * 4 + lane; e < nelem; e += 32) __stcs(dst + e, st[e]);
        __syncwarp();
    }
}

template <int RMAX>
__global__ void __launch_bounds__(kShortThreads) softmax_bwd_short_kernel(const float* __restrict__ y, const float* __restrict__ go,
                                                                          float* __restrict__ gi, size_t rows, int reduce) {
    grid_dependency_sync();
    constexpr int TR = 128, NU = TR * RMAX / kShortThreads;
    using Tile = ShortTile<TR, NU>;
    __shared__ float ty[RMAX * (TR + 1)];
    __shared__ float tg[RMAX * (TR + 1)];
    const size_t step = (size_t)gridDim.x * TR;
    auto count = [&](size_t r0) { return (int)(rows - r0 < (size_t)TR ? rows - r0 : TR) * reduce; };
    float ny[NU], ng[NU];
    size_t row0 = (size_t)blockIdx.x * TR;
    if (row0 < rows) { Tile::fetch(ny, y + row0 * reduce, count(row0)); Tile::fetch(ng, go + row0 * reduce, count(row0)); }
    for (; row0 < rows; row0 += step) {
        const int nelem = count(row0), nrows = nelem / reduce;
        Tile::put(ty, ny, nelem, reduce);
        Tile::put(tg, ng, nelem, reduce);
        __syncthreads();
        if (row0 + step < rows) {
            Tile::fetch(ny, y + (row0 + step) * reduce, count(row0 + step));
            Tile::fetch(ng, go + (row0 + step) * reduce, count(row0 + step));
        }
        if ((int)threadIdx.x < nrows) {
            const float* cy = ty + threadIdx.x;
            float* cg = tg + threadIdx.x;
            float dot = 0.0f;   // sequential, the reference's order
            for (int j = 0; j < reduce; ++j) dot = __fadd_rn(dot, __fmul_rn(cg[j * (TR + 1)], cy[j * (TR + 1)]));
            for (int j = 0; j < reduce; ++j) cg[j * (TR + 1)] = __fmul_rn(cy[j * (TR + 1)], __fsub_rn(cg[j * (TR + 1)], dot));
        }
        __syncthreads();
        Tile::store(tg, gi + row0 * reduce, nelem, reduce);
        __syncthreads();
    }
}

// ------------------------------------------------------------------ columns: inner > 1
// Thread (lane, warp) of a tile owns line i = tile_i * 32 + lane and the elements j = warp + W*k of it.
template <int W, bool IS_MAX>
__device__ __forceinline__ float cross_warp(float v, float (*red)[32]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    red[warp][lane] = v;
    __syncthreads();
    float r = red[0][lane];
#pragma unroll
    for (int w = 1; w < W; ++w) r = IS_MAX ? fmaxf(r, red[w][lane]) : __fadd_rn(r, red[w][lane]);
    __syncthreads();
    return r;
}

template <int W, bool CACHED>
__global__ void __launch_bounds__(32 * W) softmax_cols_kernel(const float* __restrict__ x, float* __restrict__ y, size_t outer, size_t reduce,
                                                              size_t inner) {
    grid_dependency_sync();
    __shared__ float red[W][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t itiles = (inner + 31) / 32, tiles = outer * itiles;
    float nx[kV];
    auto load = [&](size_t tile) {
        const size_t o = tile / itiles, i = (tile - o * itiles) * 32 + lane;
        const size_t base = o * reduce * inner + i;
#pragma unroll
        for (int k = 0; k < kV; ++k) {
            const size_t j = (size_t)warp + (size_t)k * W;
            nx[k] = (i < inner && j < reduce) ? __ldcs(x + base + j * inner) : -INFINITY;
        }
    };
    size_t tile = blockIdx.x;
    if (CACHED && tile < tiles) load(tile);
    for (; tile < tiles; tile += gridDim.x) {
        const size_t o = tile / itiles, i = (tile - o * itiles) * 32 + lane;
        const bool active = i < inner;
        const size_t base = o * reduce * inner + i;
        float v[kV];
        float mx = -INFINITY;
        if (CACHED) {
#pragma unroll
            for (int k = 0; k < kV; ++k) v[k] = nx[k];
            if (tile + gridDim.x < tiles) load(tile + gridDim.x);
#pragma unroll
            for (int k = 0; k < kV; ++k) if (v[k] > mx) mx = v[k];
        } else if (active) {
            for (size_t j = warp; j < reduce; j += W) { float a = x[base + j * inner]; if (a > mx) mx = a; }
        }
        mx = cross_warp<W, true>(mx, red);
        float sum = 0.0f;
        if (CACHED) {
#pragma unroll
            for (int k = 0; k < kV; ++k) {
                const size_t j = (size_t)warp + (size_t)k * W;
                v[k] = (active && j < reduce) ? expf(__fsub_rn(v[k], mx)) : 0.0f;
                sum = __fadd_rn(sum, v[k]);
            }
        } else if (active) {
            for (size_t j = warp; j < reduce; j += W) sum = __fadd_rn(sum, expf(__fsub_rn(x[base + j * inner], mx)));
        }
        sum = cross_warp<W, false>(sum, red);
        const float inv = __fdiv_rn(1.0f, sum);
        if (CACHED) {
#pragma unroll
            for (int k = 0; k < kV; ++k) {
                const size_t j = (size_t)warp + (size_t)k * W;
                if (active && j < reduce) __stcs(y + base + j * inner, __fmul_rn(v[k], inv));
            }
        } else if (active) {
            for (size_t j = warp; j < reduce; j += W) y[base + j * inner] = __fmul_rn(expf(__fsub_rn(x[base + j * inner], mx)), inv);
        }
    }
}

template <int W, bool CACHED>
__global__ void __launch_bounds__(32 * W) softmax_bwd_cols_kernel(const float* __restrict__ y, const float* __restrict__ go,
                                                                  float* __restrict__ gi, size_t outer, size_t reduce, size_t inner) {
    grid_dependency_sync();
    __shared__ float red[W][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t itiles = (inner + 31) / 32, tiles = outer * itiles;
    float ny[kV], ng[kV];
    auto load = [&](size_t tile) {
        const size_t o = tile / itiles, i = (tile - o * itiles) * 32 + lane;
        const size_t base = o * reduce * inner + i;
#pragma unroll
        for (int k = 0; k < kV; ++k) {
            const size_t j = (size_t)warp + (size_t)k * W;
            const bool in = i < inner && j < reduce;
            ny[k] = in ? __ldcs(y + base + j * inner) : 0.0f;
            ng[k] = in ? __ldcs(go + base + j * inner) : 0.0f;
        }
    };
    size_t tile = blockIdx.x;
    if (CACHED && tile < tiles) load(tile);
    for (; tile < tiles; tile += gridDim.x) {
        const size_t o = tile / itiles, i = (tile - o * itiles) * 32 + lane;
        const bool active = i < inner;
        const size_t base = o * reduce * inner + i;
        float vy[kV], vg[kV];
        float dot = 0.0f;
        if (CACHED) {
#pragma unroll
            for (int k = 0; k < kV; ++k) { vy[k] = ny[k]; vg[k] = ng[k]; }
            if (tile + gridDim.x < tiles) load(tile + gridDim.x);
#pragma unroll
            for (int k = 0; k < kV; ++k) dot = __fadd_rn(dot, __fmul_rn(vg[k], vy[k]));
        } else if (active) {
            for (size_t j = warp; j < reduce; j += W) dot = __fadd_rn(dot, __fmul_rn(go[base + j * inner], y[base + j * inner]));
        }
        dot = cross_warp<W, false>(dot, red);
        if (CACHED) {
#pragma unroll
            for (int k = 0; k < kV; ++k) {
                const size_t j = (size_t)warp + (size_t)k * W;
                if (active && j < reduce) __stcs(gi + base + j * inner, __fmul_rn(vy[k], __fsub_rn(vg[k], dot)));
            }
        } else if (active) {
            for (size_t j = warp; j < reduce; j += W)
                gi[base + j * inner] = __fmul_rn(y[base + j * inner], __fsub_rn(go[base + j * inner], dot));
        }
    }
}

// ------------------------------------------------------------------ columns, staged: inner > 1, inner % 4 == 0
// A CTA copies a whole [reduce][TI] tile of neighbouring lines into shared memory with 16-byte asynchronous
// copies (no registers held while the data is in flight), double-buffered: the next tile streams in while the
// current one is reduced.  Thread (col, jg) owns line `col` of the tile and the elements j = jg, jg + JG, ...
constexpr int kStagedThreads = 512;

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src, int src_bytes) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Streams tile `tile` of `src` into buf[reduce][TI]; columns past `inner` are zero-filled (src_bytes = 0 reads nothing).
template <int TI>
__device__ __forceinline__ void stage_tile(float* buf, const float* __restrict__ src, size_t tile, size_t itiles, size_t reduce, size_t inner) {
    const size_t o = tile / itiles, i0 = (tile - o * itiles) * TI;
    const int chunks_per_row = TI / 4, total = (int)reduce * chunks_per_row;
    for (int c = threadIdx.x; c < total; c += kStagedThreads) {
        const int j = c / chunks_per_row, q = c - j * chunks_per_row;
        const size_t i = i0 + (size_t)q * 4;
        const bool in = i < inner;                       // inner % 4 == 0: a chunk is entirely inside or outside
        const float* g = in ? src + (o * reduce + j) * inner + i : src;
        cp_async16(buf + j * TI + q * 4, g, in ? 16 : 0);
    }
}
template <int JG, int TI, bool IS_MAX>
__device__ __forceinline__ float cross_groups(float v, float* red) {
    const int col = threadIdx.x % TI, jg = threadIdx.x / TI;
    red[jg * TI + col] = v;
    __syncthreads();
    float r = red[col];
#pragma unroll
    for (int g = 1; g < JG; ++g) r = IS_MAX ? fmaxf(r, red[g * TI + col]) : __fadd_rn(r, red[g * TI + col]);
    __syncthreads();
    return r;
}

template <int TI>
__global__ void __launch_bounds__(kStagedThreads) softmax_cols_staged_kernel(const float* __restrict__ x, float* __restrict__ y, size_t outer,
                                                                             size_t reduce, size_t inner) {
    grid_dependency_sync();
    constexpr int JG = kStagedThreads / TI;
    extern __shared__ __align__(16) float smem[];
    const size_t tile_elems = reduce * TI;   // buffer b starts at smem + b * tile_elems
    float* red = smem + 2 * tile_elems;
    const int col = threadIdx.x % TI, jg = threadIdx.x / TI;
    const size_t itiles = (inner + TI - 1) / TI, tiles = outer * itiles;
    size_t tile = blockIdx.x;
    if (tile < tiles) stage_tile<TI>(smem, x, tile, itiles, reduce, inner);
    cp_async_commit();
    int cur = 0;
    for (; tile < tiles; tile += gridDim.x, cur ^= 1) {
        if (tile + gridDim.x < tiles) stage_tile<TI>(smem + (size_t)(cur ^ 1) * tile_elems, x, tile + gridDim.x, itiles, reduce, inner);
        cp_async_commit();
        cp_async_wait<1>();          // everything but the newest group has landed: the current tile
        __syncthreads();
        float* t = smem + (size_t)cur * tile_elems;
        const size_t o = tile / itiles, i = (tile - o * itiles) * TI + col;
        const bool active = i < inner;
        float mx = -INFINITY;
        for (size_t j = jg; j < reduce; j += JG) { const float a = t[j * TI + col]; if (a > mx) mx = a; }
        mx = cross_groups<JG, TI, true>(mx, red);
        float sum = 0.0f;
        for (size_t j = jg; j < reduce; j += JG) {
            const float e = expf(__fsub_rn(t[j * TI + col], mx));
            t[j * TI + col] = e;
            sum = __fadd_rn(sum, e);
        }
        sum = cross_groups<JG, TI, false>(sum, red);
        const float inv = __fdiv_rn(1.0f, sum);
        if (active) {
            float* dst = y + o * reduce * inner + i;
            for (size_t j = jg; j < reduce; j += JG) __stcs(dst + j * inner, __fmul_rn(t[j * TI + col], inv));
        }
        __syncthreads();             // the buffer is free for the copy issued in the next iteration
    }
    cp_async_wait<0>();
}

template <int TI>
__global__ void __launch_bounds__(kStagedThreads) softmax_bwd_cols_staged_kernel(const float* __restrict__ y, const float* __restrict__ go,
                                                                                 float* __restrict__ gi, size_t outer, size_t reduce, size_t inner) {
    grid_dependency_sync();
    constexpr int JG = kStagedThreads / TI;
    extern __shared__ __align__(16) float smem[];
    const size_t tile_elems = reduce * TI;
    float* red = smem + 4 * tile_elems;      // buffer b holds y at smem + 2b * tile_elems and go right after it
    const int col = threadIdx.x % TI, jg = threadIdx.x / TI;
    const size_t itiles = (inner + TI - 1) / TI, tiles = outer * itiles;
    size_t tile = blockIdx.x;
    if (tile < tiles) { stage_tile<TI>(smem, y, tile, itiles, reduce, inner); stage_tile<TI>(smem + tile_elems, go, tile, itiles, reduce, inner); }
    cp_async_commit();
    int cur = 0;
    for (; tile < tiles; tile += gridDim.x, cur ^= 1) {
        if (tile + gridDim.x < tiles) {
            float* nb = smem + (size_t)(cur ^ 1) * 2 * tile_elems;
            stage_tile<TI>(nb, y, tile + gridDim.x, itiles, reduce, inner);
            stage_tile<TI>(nb + tile_elems, go, tile + gridDim.x, itiles, reduce, inner);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const float* ty = smem + (size_t)cur * 2 * tile_elems;
        const float* tg = ty + tile_elems;
        const size_t o = tile / itiles, i = (tile - o * itiles) * TI + col;
        float dot = 0.0f;
        for (size_t j = jg; j < reduce; j += JG) dot = __fadd_rn(dot, __fmul_rn(tg[j * TI + col], ty[j * TI + col]));
        dot = cross_groups<JG, TI, false>(dot, red);
        if (i < inner) {
            float* dst = gi + o * reduce * inner + i;
            for (size_t j = jg; j < reduce; j += JG) __stcs(dst + j * inner, __fmul_rn(ty[j * TI + col], __fsub_rn(tg[j * TI + col], dot)));
        }
        __syncthreads();
    }
    cp_async_wait<0>();
}

constexpr size_t kStagedSmemLimit = 200 * 1024;   // of the 227 KB a CTA may have

template <int TI>
bool launch_cols_staged(bool bwd, const float* a, const float* b, float* o, size_t outer, size_t reduce, size_t inner, int sm, cudaStream_t s) {
    const size_t tiles_in_smem = bwd ? 4 : 2;
    const size_t bytes = (tiles_in_smem * reduce * TI + (size_t)kStagedThreads) * sizeof(float);
    if (bytes > kStagedSmemLimit) return false;
    const size_t tiles = outer * ((inner + TI - 1) / TI);
    int per_sm = (int)(kStagedSmemLimit / bytes);
    if (per_sm > 2048 / kStagedThreads) per_sm = 2048 / kStagedThreads;
    if (per_sm < 1) per_sm = 1;
    const size_t cap = (size_t)sm * per_sm;
    const unsigned grid = (unsigned)(tiles < cap ? tiles : cap);
    if (bwd) {
        if (!cuda_ok(cudaFuncSetAttribute(softmax_bwd_cols_staged_kernel<TI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), "softmax smem")) return false;
        launch_dep(softmax_bwd_cols_staged_kernel<TI>, dim3(grid), dim3(kStagedThreads), bytes, s, a, b, o, outer, reduce, inner);
    } else {
        if (!cuda_ok(cudaFuncSetAttribute(softmax_cols_staged_kernel<TI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), "softmax smem")) return false;
        launch_dep(softmax_cols_staged_kernel<TI>, dim3(grid), dim3(kStagedThreads), bytes, s, a, o, outer, reduce, inner);
    }
    return true;
}

// The widest tile whose buffers fit; false when the line is too long, too short to be worth it, or unaligned.
bool try_cols_staged(bool bwd, const float* a, const float* b, float* o, size_t outer, size_t reduce, size_t inner, int sm, cudaStream_t s) {
    if (inner % 4 != 0 || inner < 32 || reduce < 16) return false;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (bwd && (reinterpret_cast<uintptr_t>(b) & 15))) return false;
    const size_t per_col = (bwd ? 4 : 2) * reduce * sizeof(float);      // shared-memory bytes per tile column
    if (inner >= 128 && per_col * 128 + 2048 <= kStagedSmemLimit) return launch_cols_staged<128>(bwd, a, b, o, outer, reduce, inner, sm, s);
    if (inner >= 64 && per_col * 64 + 2048 <= kStagedSmemLimit) return launch_cols_staged<64>(bwd, a, b, o, outer, reduce, inner, sm, s);
    if (per_col * 32 + 2048 <= kStagedSmemLimit) return launch_cols_staged<32>(bwd, a, b, o, outer, reduce, inner, sm, s);
    return false;
}

// ------------------------------------------------------------------ dispatch
inline int grid_for(size_t units, int sm_count, int cta_threads) {
    int per_sm = 1536 / cta_threads;
    if (per_sm < 1) per_sm = 1;
    size_t cap = (size_t)sm_count * per_sm;
    if (units < 1) units = 1;
    return (int)(units < cap ? units : cap);
}

bool check(const void* a, const void* b, size_t reduce, const char* what) {
    if (!a || !b) { set_error("%s: null pointer", what); return false; }
    if (reduce == 0) { set_error("%s: cannot softmax over empty dimension", what); return false; }   // softmax.rs:121
    return true;
}

template <int G>
void launch_rows(bool bwd, const float* a, const float* b, float* o, size_t rows, size_t reduce, int sm, cudaStream_t s) {
    constexpr int CTA = RowsCfg<G>::kCta, RPC = RowsCfg<G>::kRpc;
    const int grid = grid_for((rows + RPC - 1) / RPC, sm, CTA);
    if (bwd) launch_dep(softmax_bwd_rows_kernel<G, true>, dim3(grid), dim3(CTA), 0, s, a, b, o, rows, reduce);
    else launch_dep(softmax_rows_kernel<G, true>, dim3(grid), dim3(CTA), 0, s, a, o, rows, reduce);
}
template <int W>
void launch_cols(bool bwd, const float* a, const float* b, float* o, size_t outer, size_t reduce, size_t inner, int sm, cudaStream_t s) {
    const int grid = grid_for(outer * ((inner + 31) / 32), sm, 32 * W);
    if (bwd) launch_dep(softmax_bwd_cols_kernel<W, true>, dim3(grid), dim3(32 * W), 0, s, a, b, o, outer, reduce, inner);
    else launch_dep(softmax_cols_kernel<W, true>, dim3(grid), dim3(32 * W), 0, s, a, o, outer, reduce, inner);
}

template <int RMAX>
void launch_short(bool bwd, const float* a, const float* b, float* o, size_t rows, int reduce, int sm, cudaStream_t s) {
    if (bwd) launch_dep(softmax_bwd_short_kernel<RMAX>, dim3(grid_for((rows + 127) / 128, sm, kShortThreads)), dim3(kShortThreads), 0, s, a, b, o, rows, reduce);
    else if (reduce % 4 != 0)   // the row pitch repeats over the banks at most every second lane
        launch_dep(softmax_short_warp_kernel<RMAX>, dim3(grid_for((rows + kShortThreads - 1) / kShortThreads, sm, kShortThreads)), dim3(kShortThreads), 0, s, a, o, rows, reduce);
    else launch_dep(softmax_short_kernel<RMAX>, dim3(grid_for((rows + 255) / 256, sm, kShortThreads)), dim3(kShortThreads), 0, s, a, o, rows, reduce);
}

// forward: a = x, b unused; backward: a = y, b = go
void dispatch(bool bwd, const float* a, const float* b, float* o, size_t outer, size_t reduce, size_t inner, int sm, cudaStream_t s) {
    if (inner == 1) {
        if (reduce <= 8) launch_short<8>(bwd, a, b, o, outer, (int)reduce, sm, s);
        else if (reduce <= 12) launch_short<12>(bwd, a, b, o, outer, (int)reduce, sm, s);   // 10 classes: 12 unrolled slots instead of 16
        else if (reduce <= 16) launch_short<16>(bwd, a, b, o, outer, (int)reduce, sm, s);
        else if (reduce <= kShortMax) launch_short<kShortMax>(bwd, a, b, o, outer, (int)reduce, sm, s);
        else if (reduce <= 32 * kV) launch_rows<32>(bwd, a, b, o, outer, reduce, sm, s);
        else if (reduce <= 64 * kV) launch_rows<64>(bwd, a, b, o, outer, reduce, sm, s);
        else if (reduce <= 128 * kV) launch_rows<128>(bwd, a, b, o, outer, reduce, sm, s);
        else if (reduce <= 256 * kV) launch_rows<256>(bwd, a, b, o, outer, reduce, sm, s);
        else if (reduce <= 512 * kV) launch_rows<512>(bwd, a, b, o, outer, reduce, sm, s);
        else if (reduce <= 1024 * kV) launch_rows<1024>(bwd, a, b, o, outer, reduce, sm, s);
        else if (bwd) launch_dep(softmax_bwd_rows_kernel<256, false>, dim3(grid_for(outer, sm, 256)), dim3(256), 0, s, a, b, o, outer, reduce);
        else launch_dep(softmax_rows_kernel<256, false>, dim3(grid_for(outer, sm, 256)), dim3(256), 0, s, a, o, outer, reduce);
    } else {
        if (try_cols_staged(bwd, a, b, o, outer, reduce, inner, sm, s)) return;
        if (reduce <= 8 * kV) launch_cols<8>(bwd, a, b, o, outer, reduce, inner, sm, s);
        else if (reduce <= 16 * kV) launch_cols<16>(bwd, a, b, o, outer, reduce, inner, sm, s);
        else if (reduce <= 32 * kV) launch_cols<32>(bwd, a, b, o, outer, reduce, inner, sm, s);
        else {
            const int grid = grid_for(outer * ((inner + 31) / 32), sm, 256);
            if (bwd) launch_dep(softmax_bwd_cols_kernel<8, false>, dim3(grid), dim3(256), 0, s, a, b, o, outer, reduce, inner);
            else launch_dep(softmax_cols_kernel<8, false>, dim3(grid), dim3(256), 0, s, a, o, outer, reduce, inner);
        }
    }
}

}  // namespace

bool softmax(const float* x, float* y, size_t outer, size_t reduce, size_t inner, cudaStream_t s) {
    if (outer * inner == 0 && reduce != 0) return true;
    if (!check(x, y, reduce, "softmax")) return false;
    DeviceCtx* c = ctx();
    if (!c) return false;
    ProfScope prof(kProfReduce, s, 8.0 * (double)outer * reduce * inner);
    dispatch(false, x, nullptr, y, outer, reduce, inner, c->sm_count, s);
    return cuda_ok(cudaGetLastError(), "softmax launch");
}

bool softmax_bwd(const float* y, const float* go, float* gi, size_t outer, size_t reduce, size_t inner, cudaStream_t s) {
    if (outer * inner == 0 && reduce != 0) return true;
    if (!check(y, go, reduce, "softmax backward") || !check(gi, gi, reduce, "softmax backward")) return false;
    DeviceCtx* c = ctx();
    if (!c) return false;
    ProfScope prof(kProfReduce, s, 12.0 * (double)outer * reduce * inner);
    dispatch(true, y, go, gi, outer, reduce, inner, c->sm_count, s);
    return cuda_ok(cudaGetLastError(), "softmax backward launch");
}

}  // namespace k
}  // namespace ts

// ====================================================================== C ABI
using namespace ts;

TS_API bool launch_softmax_kernel(const float* x, float* out, unsigned long long outer, unsigned long long reduce,
                                  unsigned long long inner, void* stream) {
    cudaStream_t s = pick_stream(stream);
    if (!s) return false;
    return k::softmax(x, out, outer, reduce, inner, s);
}
TS_API bool launch_softmax_backward_kernel(const float* y, const float* go, float* gi, unsigned long long outer,
                                           unsigned long long reduce, unsigned long long inner, void* stream) {
    cudaStream_t s = pick_stream(stream);
    if (!s) return false;
    return k::softmax_bwd(y, go, gi, outer, reduce, inner, s);
}
