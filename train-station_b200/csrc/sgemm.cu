// FP32 GEMM on the CUDA cores (FFMA), any shape, any transposition.
//
// This is the FP32 precision mode and the path for shapes the tensor-core kernel cannot
// take.  It reproduces the reference's summation order exactly: every output element is
// one chain over p = 0..k-1 of acc = fma(A[i,p], B[p,j], acc), which is what the AVX2
// micro-kernels compute (tensor/ops/matmul/kernels.rs:278-305, :378-385, :474-497; k-blocks
// are accumulated through C, which is exact).  The reference's n mod 8 trailing columns use
// a rounded multiply followed by an add instead of an FMA (kernels.rs:312-335); the
// HAS_TAIL variant does the same for those columns.  With identical inputs the result is
// therefore bit-identical to the reference's CPU path.
#include "../../include/train_station_b200.h"
#include "common.h"

namespace ts {
namespace k {

namespace {

constexpr int BM = 128, BN = 128, BK = 8, kThreads = 256;

template <bool TA, bool TB, bool HAS_TAIL>
__global__ void __launch_bounds__(kThreads) sgemm_kernel(GemmArgs g) {
    __shared__ __align__(16) float As[2][BK][BM];
    __shared__ __align__(16) float Bs[2][BK][BN];
    const int t = threadIdx.x;
    const size_t m0 = (size_t)blockIdx.y * BM, n0 = (size_t)blockIdx.x * BN;
    const size_t M = g.m, N = g.n, K = g.k;
    const int ty = t / 16, tx = t % 16;

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    // which of this thread's 8 columns are reference "tail" columns (mul+add instead of fma)
    bool tailc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        size_t col = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
        tailc[j] = HAS_TAIL && col >= N / 8 * 8;
    }

    float ra[4], rb[4];
    auto load_tiles = [&](size_t k0) {
        if (TA) {  // A stored [K][M]: M contiguous
            int kr = t / 32, mc = (t % 32) * 4;
            size_t p = k0 + kr;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                size_t i = m0 + mc + e;
                ra[e] = (p < K && i < M) ? g.a[p * M + i] : 0.0f;
            }
        } else {   // A stored [M][K]: K contiguous
            int mr = t / 2, kc = (t % 2) * 4;
            size_t i = m0 + mr;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                size_t p = k0 + kc + e;
                ra[e] = (p < K && i < M) ? g.a[i * K + p] : 0.0f;
            }
        }
        if (TB) {  // B stored [N][K]: K contiguous
            int nr = t / 2, kc = (t % 2) * 4;
            size_t j = n0 + nr;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                size_t p = k0 + kc + e;
                rb[e] = (p < K && j < N) ? g.b[j * K + p] : 0.0f;
            }
        } else {   // B stored [K][N]: N contiguous
            int kr = t / 32, nc = (t % 32) * 4;
            size_t p = k0 + kr;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                size_t j = n0 + nc + e;
                rb[e] = (p < K && j < N) ? g.b[p * N + j] : 0.0f;
            }
        }
    };
    auto store_tiles = [&](int buf) {
        if (TA) {
            int kr = t / 32, mc = (t % 32) * 4;
            *reinterpret_cast<float4*>(&As[buf][kr][mc]) = make_float4(ra[0], ra[1], ra[2], ra[3]);
        } else {
            int mr = t / 2, kc = (t % 2) * 4;
#pragma unroll
            for (int e = 0; e < 4; ++e) As[buf][kc + e][mr] = ra[e];
        }
        if (TB) {
            int nr = t / 2, kc = (t % 2) * 4;
#pragma unroll
            for (int e = 0; e < 4; ++e) Bs[buf][kc + e][nr] = rb[e];
        } else {
            int kr = t / 32, nc = (t % 32) * 4;
            *reinterpret_cast<float4*>(&Bs[buf][kr][nc]) = make_float4(rb[0], rb[1], rb[2], rb[3]);
        }
    };

    const size_t ktiles = (K + BK - 1) / BK;
    if (ktiles > 0) {
        load_tiles(0);
        store_tiles(0);
    }
    __syncthreads();
    for (size_t kt = 0; kt < ktiles; ++kt) {
        int buf = (int)(kt & 1);
        if (kt + 1 < ktiles) load_tiles((kt + 1) * BK);
#pragma unroll
        for (int p = 0; p < BK; ++p) {
            float4 a0 = *reinterpret_cast<const float4*>(&As[buf][p][ty * 4]);
            float4 a1 = *reinterpret_cast<const float4*>(&As[buf][p][64 + ty * 4]);
            float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][p][tx * 4]);
            float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][p][64 + tx * 4]);
            float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (HAS_TAIL && tailc[j]) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
                    else acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
                }
        }
        if (kt + 1 < ktiles) store_tiles(buf ^ 1);
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        size_t row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (row >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            size_t col = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (col >= N) continue;
            float v = acc[i][j];
            if (g.bias) v = __fadd_rn(v, __ldg(g.bias + col));
            if (g.relu) v = v > 0.0f ? v : 0.0f;
            if (g.mask) v = g.mask[row * N + col] > 0.0f ? v : 0.0f;
            g.c[row * N + col] = v;
        }
    }
}

template <bool TA, bool TB>
void launch(const GemmArgs& g, dim3 grid, cudaStream_t s) {
    if (g.n % 8 != 0) sgemm_kernel<TA, TB, true><<<grid, kThreads, 0, s>>>(g);
    else sgemm_kernel<TA, TB, false><<<grid, kThreads, 0, s>>>(g);
}

// The same arithmetic on 32 x 32 tiles (2 x 2 outputs per thread, 32 k per stage) for results that would fill only a
// few 128 x 128 tiles: a [1024 x 10] bias-layer weight gradient reduced over 4096 rows is 8 CTAs of the big kernel,
// each walking all of K alone, but 32 CTAs here.  Per output element the chain over p is unchanged.
constexpr int SM_T = 32;

template <bool TA, bool TB, bool HAS_TAIL>
__global__ void __launch_bounds__(kThreads) sgemm_small_kernel(GemmArgs g) {
    __shared__ float As[SM_T][SM_T + 1];   // [k][m]
    __shared__ float Bs[SM_T][SM_T + 1];   // [k][n]
    const int t = threadIdx.x, ty = t / 16, tx = t % 16;
    const size_t m0 = (size_t)blockIdx.y * SM_T, n0 = (size_t)blockIdx.x * SM_T;
    const size_t M = g.m, N = g.n, K = g.k;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    bool tailc[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) tailc[j] = HAS_TAIL && (n0 + tx * 2 + j) >= N / 8 * 8;

    for (size_t k0 = 0; k0 < K; k0 += SM_T) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int e = t + kThreads * q, lo = e % SM_T, hi = e / SM_T;
            {   // A: stored [K][M] (TA, contiguous along m) or [M][K] (contiguous along k)
                const int kk = TA ? hi : lo, mm = TA ? lo : hi;
                const size_t p = k0 + kk, i = m0 + mm;
                As[kk][mm] = (p < K && i < M) ? (TA ? g.a[p * M + i] : g.a[i * K + p]) : 0.0f;
            }
            {   // B: stored [N][K] (TB, contiguous along k) or [K][N] (contiguous along n)
                const int kk = TB ? lo : hi, nn = TB ? hi : lo;
                const size_t p = k0 + kk, j = n0 + nn;
                Bs[kk][nn] = (p < K && j < N) ? (TB ? g.b[j * K + p] : g.b[p * N + j]) : 0.0f;
            }
        }
        __syncthreads();
        const int pmax = (K - k0) < (size_t)SM_T ? (int)(K - k0) : SM_T;   // no padded terms enter the chain
        for (int p = 0; p < pmax; ++p) {
            const float a0 = As[p][ty * 2], a1 = As[p][ty * 2 + 1];
            const float b[2] = {Bs[p][tx * 2], Bs[p][tx * 2 + 1]};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (HAS_TAIL && tailc[j]) {
                    acc[0][j] = __fadd_rn(acc[0][j], __fmul_rn(a0, b[j]));
                    acc[1][j] = __fadd_rn(acc[1][j], __fmul_rn(a1, b[j]));
                } else {
                    acc[0][j] = fmaf(a0, b[j], acc[0][j]);
                    acc[1][j] = fmaf(a1, b[j], acc[1][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const size_t row = m0 + ty * 2 + i;
        if (row >= M) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const size_t col = n0 + tx * 2 + j;
            if (col >= N) continue;
            float v = acc[i][j];
            if (g.bias) v = __fadd_rn(v, __ldg(g.bias + col));
            if (g.relu) v = v > 0.0f ? v : 0.0f;
            if (g.mask) v = g.mask[row * N + col] > 0.0f ? v : 0.0f;
            g.c[row * N + col] = v;
        }
    }
}

template <bool TA, bool TB>
void launch_small(const GemmArgs& g, dim3 grid, cudaStream_t s) {
    if (g.n % 8 != 0) sgemm_small_kernel<TA, TB, true><<<grid, kThreads, 0, s>>>(g);
    else sgemm_small_kernel<TA, TB, false><<<grid, kThreads, 0, s>>>(g);
}

}  // namespace

bool sgemm(const GemmArgs& g, cudaStream_t s) {
    if (g.m == 0 || g.n == 0) return true;
    if (!g.a || !g.b || !g.c) {
        if (g.k == 0 && g.c) { /* fallthrough: zero-filled result */ }
        else { set_error("gemm: null pointer"); return false; }
    }
    size_t gx = (g.n + BN - 1) / BN, gy = (g.m + BM - 1) / BM;
    if (gy > 65535) { set_error("gemm: m = %zu too large for the FP32 kernel's grid", g.m); return false; }
    dim3 grid((unsigned)gx, (unsigned)gy);
    ProfScope prof(kProfGemmFp32, s, 2.0 * (double)g.m * (double)g.n * (double)g.k);
    DeviceCtx* c = ctx();
    const size_t sgy = (g.m + SM_T - 1) / SM_T;
    if (c && gx * gy < (size_t)c->sm_count / 2 && sgy <= 65535) {
        // too few 128 x 128 tiles to occupy the GPU: 32 x 32 tiles, sixteen times as many CTAs
        dim3 sgrid((unsigned)((g.n + SM_T - 1) / SM_T), (unsigned)sgy);
        if (g.trans_a) { if (g.trans_b) launch_small<true, true>(g, sgrid, s); else launch_small<true, false>(g, sgrid, s); }
        else { if (g.trans_b) launch_small<false, true>(g, sgrid, s); else launch_small<false, false>(g, sgrid, s); }
        return cuda_ok(cudaGetLastError(), "sgemm (small tiles) launch");
    }
    if (g.trans_a) { if (g.trans_b) launch<true, true>(g, grid, s); else launch<true, false>(g, grid, s); }
    else { if (g.trans_b) launch<false, true>(g, grid, s); else launch<false, false>(g, grid, s); }
    return cuda_ok(cudaGetLastError(), "sgemm launch");
}

}  // namespace k
}  // namespace ts
