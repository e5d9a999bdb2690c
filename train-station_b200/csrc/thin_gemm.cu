// FFMA kernels for products with one very short dimension (at most 16): the 10-class output layer of an MLP, the
// gradient of its weights and the gradient of its input.  For the modes that promise no summation order (TF32, 3xTF32)
// only: the FP32 mode keeps the reference's chain order on the tiled kernel (sgemm.cu).
//
// Tiles of 32 or more columns are mostly padding on such a product and a tile's CTA walks the whole of the long
// dimension alone; these three kernels are instead laid out along the long dimensions, read every operand once with
// coalesced loads and keep the short dimension in registers, so each is bound by the memory it has to touch:
//
//   thin_n_nn   C[m x n] = A[m x k] . B[k x n],   n <= 16   (forward: activations times a narrow weight matrix)
//   thin_n_tn   C[m x n] = A[k x m]^T . B[k x n], n <= 16   (weight gradient: activations^T times a narrow gradient)
//   thin_k_nt   C[m x n] = A[m x k] . B[n x k]^T, k <= 16   (input gradient: a narrow gradient times the weights^T)
//
// The operands are used as given (FP32 products of FP32 values, FP32 accumulation), which is at least as accurate as
// the tensor-core path these shapes cannot take; every sum is added in a fixed order, so results repeat bit for bit.
#include "common.h"

#include <cstdlib>

namespace ts {
namespace k {
namespace {

constexpr int kThin = 16;
constexpr int kThreads = 256;
// result rows per CTA of the short-reduction kernel: 16, or 64 when there are many rows (a thread fetches its 4 x k
// values of B once per CTA, which 16 rows of work do not amortise; on 4096 rows 64 would leave most SMs without a CTA)
inline int nt_rows(size_t m) { return m >= 32768 ? 64 : 16; }

__device__ __forceinline__ float rn_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// bias, ReLU, mask and rounding in the order every GEMM epilogue of this library applies them
__device__ __forceinline__ float finish(const GemmArgs& g, float v, size_t row, size_t col) {
    if (g.bias) v = __fadd_rn(v, __ldg(g.bias + col));
    if (g.relu) v = v > 0.0f ? v : 0.0f;
    if (g.mask) v = g.mask[row * g.n + col] > 0.0f ? v : 0.0f;
    if (g.round_tf32) v = rn_tf32(v);
    return v;
}

// ---- C[m x n] = A[m x k] . B[k x n], n <= NP.  A warp takes R rows, a CTA 8 R; the lanes split K (lane l takes
// k = l, l + 32, ...: a warp reads 128 contiguous bytes of each row per step, 8 R such loads in flight per lane) and B
// sits in shared memory in chunks of KC rows, each row padded to a pitch that lets eight consecutive rows be read as
// float4 without bank conflicts.  The 32 partial sums of every result are then added by a butterfly.  The kernel is bound
// by memory latency, so what matters is how many loads are in flight per SM, and that depends on the size: with few rows
// (a CTA per SM or fewer) four rows per warp and chunks of 512 rows fetched in one go are fastest (4096 rows: 9.9 us
// against 13.2); with many rows that version's 160 registers hold an SM to one CTA and a fifth of HBM's rate, where two
// rows per warp (about 75 registers, three or four CTAs per SM) and chunks of 1024 rows run 1.8 times as fast
// (65536 x 10 over K = 1024: 0.113 against 0.203 ms).
template <int NP, int R, int KC>
__global__ void __launch_bounds__(kThreads) thin_n_nn_kernel(GemmArgs g) {
    constexpr int S = NP == 4 ? 4 : (NP == 16 ? 20 : 12);
    constexpr int BATCH = KC * NP / kThreads <= 24 ? KC * NP / kThreads : 8;   // loads of a B chunk in flight per thread
    static_assert((size_t)KC * S * sizeof(float) <= 48 * 1024, "a chunk of B must fit static shared memory");
    __shared__ __align__(16) float bs[KC * S];
    grid_dependency_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t M = g.m, N = g.n, K = g.k;
    const size_t row0 = (size_t)blockIdx.x * (R * kThreads / 32) + (size_t)warp * R;
    const float* arow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const size_t rr = row0 + r < M ? row0 + r : M - 1;   // rows past the end re-read the last one and are not stored
        arow[r] = g.a + rr * K;
    }
    float acc[R][NP];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < NP; ++j) acc[r][j] = 0.0f;

    for (size_t kc = 0; kc < K; kc += KC) {
        const int kn = (int)(K - kc < (size_t)KC ? K - kc : (size_t)KC);
        __syncthreads();   // the previous chunk has been consumed
        for (int base = 0; base < kn * NP; base += BATCH * kThreads) {
            float stage[BATCH];
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                const int idx = base + threadIdx.x + u * kThreads, kk = idx / NP, j = idx % NP;
                stage[u] = (kk < kn && (size_t)j < N) ? __ldg(g.b + (kc + kk) * N + j) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                const int idx = base + threadIdx.x + u * kThreads, kk = idx / NP, j = idx % NP;
                if (kk < kn) bs[kk * S + j] = stage[u];
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = lane; kk < kn; kk += 32) {
            float av[R];
#pragma unroll
            for (int r = 0; r < R; ++r) av[r] = __ldg(arow[r] + kc + kk);
            const float4* bp = reinterpret_cast<const float4*>(bs + kk * S);
#pragma unroll
            for (int q = 0; q < NP / 4; ++q) {
                const float4 b = bp[q];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    acc[r][q * 4 + 0] = fmaf(av[r], b.x, acc[r][q * 4 + 0]);
                    acc[r][q * 4 + 1] = fmaf(av[r], b.y, acc[r][q * 4 + 1]);
                    acc[r][q * 4 + 2] = fmaf(av[r], b.z, acc[r][q * 4 + 2]);
                    acc[r][q * 4 + 3] = fmaf(av[r], b.w, acc[r][q * 4 + 3]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float mine = 0.0f;
#pragma unroll
        for (int j = 0; j < NP; ++j) {
            float v = acc[r][j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == j) mine = v;
        }
        const size_t row = row0 + r;
        if (row < M && (size_t)lane < N) g.c[row * N + lane] = finish(g, mine, row, lane);
    }
}

// ---- C[m x n] = sum over r of A[r][i] * B[r][j], A stored [k x m], B stored [k x n], n <= NP.  A CTA owns 32
// columns i of A (a lane each: a warp reads 128 contiguous bytes of a row) over one slab of the k rows; its eight warps
// take the slab's rows in turn (warp w: rows w, w + 8, ...) and their partial results are added through shared memory
// in warp order.  The grid's second axis cuts the k rows into slabs whose results land side by side in `out` (slab s at
// out + s * m * n) for a second launch to add in slab order.  B's rows are staged in shared memory, 512 at a time, and
// a warp reads one of them at a time (broadcast).
template <int NP>
__global__ void __launch_bounds__(kThreads) thin_n_tn_kernel(GemmArgs g, float* out, unsigned rows_per_slab) {
    constexpr int RC = 512;
    constexpr int PER = RC * NP / kThreads;
    __shared__ __align__(16) float bs[RC * NP];
    grid_dependency_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t M = g.m, N = g.n, K = g.k;
    const size_t i = (size_t)blockIdx.x * 32 + lane;
    const size_t ic = i < M ? i : M - 1;   // columns past the end re-read the last one and are not stored
    const size_t r0 = (size_t)blockIdx.y * rows_per_slab;
    const size_t r1 = r0 + rows_per_slab < K ? r0 + rows_per_slab : K;
    float acc[NP];
#pragma unroll
    for (int j = 0; j < NP; ++j) acc[j] = 0.0f;
    for (size_t rc = r0; rc < r1; rc += RC) {
        const int rn = (int)(r1 - rc < (size_t)RC ? r1 - rc : (size_t)RC);
        float stage[PER];
#pragma unroll
        for (int t = 0; t < PER; ++t) {
            const int idx = threadIdx.x + t * kThreads, rr = idx / NP, j = idx % NP;
            stage[t] = (rr < rn && (size_t)j < N) ? __ldg(g.b + (rc + rr) * N + j) : 0.0f;
        }
        __syncthreads();   // the previous chunk has been consumed
#pragma unroll
        for (int t = 0; t < PER; ++t) bs[threadIdx.x + t * kThreads] = stage[t];
        __syncthreads();
        const float* ap = g.a + rc * M + ic;
#pragma unroll 8
        for (int rr = warp; rr < rn; rr += 8) {
            const float a = __ldg(ap + (size_t)rr * M);
            const float4* bp = reinterpret_cast<const float4*>(bs + rr * NP);
#pragma unroll
            for (int q = 0; q < NP / 4; ++q) {
                const float4 b = bp[q];
                acc[q * 4 + 0] = fmaf(a, b.x, acc[q * 4 + 0]);
                acc[q * 4 + 1] = fmaf(a, b.y, acc[q * 4 + 1]);
                acc[q * 4 + 2] = fmaf(a, b.z, acc[q * 4 + 2]);
                acc[q * 4 + 3] = fmaf(a, b.w, acc[q * 4 + 3]);
            }
        }
    }
    __syncthreads();   // bs is reused for the warps' partial results: [warp][column][j]
    float* red = bs;
#pragma unroll
    for (int j = 0; j < NP; ++j) red[(warp * 32 + lane) * NP + j] = acc[j];
    __syncthreads();
    // 32 columns x n results, added over the 8 warps in warp order and written as one contiguous run of the slab
    float* o = out + (size_t)blockIdx.y * M * N + (size_t)blockIdx.x * 32 * N;
    const size_t valid = (M - (size_t)blockIdx.x * 32 < 32 ? M - (size_t)blockIdx.x * 32 : 32) * N;
    for (size_t e = threadIdx.x; e < valid; e += kThreads) {
        const size_t col = e / N, j = e % N;
        float v = red[col * NP + j];
#pragma unroll
        for (int w = 1; w < 8; ++w) v += red[(w * 32 + col) * NP + j];
        o[e] = v;
    }
}

// ---- The same product when A's row pitch allows 128-bit loads (m % 4 == 0, 16-byte aligned): a lane owns FOUR adjacent
// columns of A, a CTA of four warps 128 columns over a slab of the k rows, the warps taking the slab's rows in turn with
// four float4 loads in flight per lane.  Four times as many bytes in flight per load instruction as the kernel above and
// small CTAs (five per SM): the kernel is bound by memory latency, and the scalar version reached a quarter of HBM's
// rate.  K is cut into many short slabs (about four CTAs per SM), which a second launch adds in slab order.
template <int NP>
__global__ void __launch_bounds__(128) thin_n_tn4_kernel(GemmArgs g, float* out, unsigned rows_per_slab) {
    constexpr int RC = 512, W = 4;                 // rows of B staged at a time; warps
    constexpr int PER = RC * NP / 128;
    __shared__ __align__(16) float bs[RC * NP];    // B's rows, then the warps' partial results [warp][column][j] (W * 128 * NP floats)
    grid_dependency_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t M = g.m, N = g.n, K = g.k;
    const size_t col = (size_t)blockIdx.x * 128 + (size_t)lane * 4;
    const size_t colc = col + 4 <= M ? col : 0;    // lanes past the end re-read the first columns and are not stored
    const size_t r0 = (size_t)blockIdx.y * rows_per_slab;
    const size_t r1 = r0 + rows_per_slab < K ? r0 + rows_per_slab : K;
    float acc[4][NP];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int j = 0; j < NP; ++j) acc[c][j] = 0.0f;
    for (size_t rc = r0; rc < r1; rc += RC) {
        const int rn = (int)(r1 - rc < (size_t)RC ? r1 - rc : (size_t)RC);
        __syncthreads();   // the previous chunk has been consumed
        for (int base = 0; base < rn * NP; base += 8 * 128) {
            float stage[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + threadIdx.x + u * 128, rr = idx / NP, j = idx % NP;
                stage[u] = (rr < rn && (size_t)j < N) ? __ldg(g.b + (rc + rr) * N + j) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + threadIdx.x + u * 128;
                if (idx < rn * NP) bs[idx] = stage[u];
            }
        }
        __syncthreads();
        const float* ap = g.a + rc * M + colc;
#pragma unroll 4
        for (int rr = warp; rr < rn; rr += W) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(ap + (size_t)rr * M));
            const float4* bp = reinterpret_cast<const float4*>(bs + rr * NP);
#pragma unroll
            for (int q = 0; q < NP / 4; ++q) {
                const float4 b = bp[q];
                const float bq[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    acc[0][q * 4 + e] = fmaf(a.x, bq[e], acc[0][q * 4 + e]);
                    acc[1][q * 4 + e] = fmaf(a.y, bq[e], acc[1][q * 4 + e]);
                    acc[2][q * 4 + e] = fmaf(a.z, bq[e], acc[2][q * 4 + e]);
                    acc[3][q * 4 + e] = fmaf(a.w, bq[e], acc[3][q * 4 + e]);
                }
            }
        }
    }
    (void)PER;
    __syncthreads();   // bs is reused for the warps' partial results
    float* red = bs;
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int j = 0; j < NP; ++j) red[((size_t)warp * 128 + lane * 4 + c) * NP + j] = acc[c][j];
    __syncthreads();
    // 128 columns x n results, added over the warps in warp order and written as one contiguous run of the slab
    float* o = out + (size_t)blockIdx.y * M * N + (size_t)blockIdx.x * 128 * N;
    const size_t cols_here = M - (size_t)blockIdx.x * 128 < 128 ? M - (size_t)blockIdx.x * 128 : 128;
    const size_t valid = cols_here * N;
    for (size_t e = threadIdx.x; e < valid; e += 128) {
        const size_t c = e / N, j = e % N;
        float v = red[c * NP + j];
#pragma unroll
        for (int w = 1; w < W; ++w) v += red[((size_t)w * 128 + c) * NP + j];
        o[e] = v;
    }
}

// ---- C[m x n] = A[m x k] . B[n x k]^T, k <= KP.  A thread owns four consecutive result columns and keeps their four
// rows of B in registers; a CTA covers ROWS result rows (A's rows sit in shared memory and are read by all threads at
// once) by 1024 columns.  Every result is finished (bias, ReLU, mask, rounding) and stored as it is made, a row of
// 4 KiB per step of the CTA; the column sums of the stored values over the CTA's rows go to row blockIdx.x of
// g.colsum_partial when that is set.  VEC: n % 4 == 0 and C and the mask are 16-byte aligned (float4 stores and loads).
template <int KP, bool VEC, int ROWS>
__global__ void __launch_bounds__(kThreads) thin_k_nt_kernel(GemmArgs g) {
    constexpr int kNtRows = ROWS;
    __shared__ __align__(16) float as[kNtRows * KP];
    grid_dependency_sync();
    const size_t M = g.m, N = g.n, K = g.k;
    const size_t row0 = (size_t)blockIdx.x * kNtRows;
    const size_t j0 = ((size_t)blockIdx.y * kThreads + threadIdx.x) * 4;
    for (int idx = threadIdx.x; idx < kNtRows * KP; idx += kThreads) {
        const int rr = idx / KP, kk = idx % KP;
        as[idx] = (row0 + rr < M && (size_t)kk < K) ? __ldg(g.a + (row0 + rr) * K + kk) : 0.0f;
    }
    float bw[4][KP];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int kk = 0; kk < KP; ++kk) bw[q][kk] = (j0 + q < N && (size_t)kk < K) ? __ldg(g.b + (j0 + q) * K + kk) : 0.0f;
    __syncthreads();
    if (j0 >= N) return;
    float cs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float bias[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (g.bias) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (j0 + q < N) bias[q] = __ldg(g.bias + j0 + q);
    }
    const int rows = (int)(M - row0 < (size_t)kNtRows ? M - row0 : (size_t)kNtRows);
#pragma unroll 8
    for (int rr = 0; rr < rows; ++rr) {
        const size_t row = row0 + rr;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float4* ap = reinterpret_cast<const float4*>(as + rr * KP);
#pragma unroll
        for (int kq = 0; kq < KP / 4; ++kq) {
            const float4 a = ap[kq];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                v[q] = fmaf(a.x, bw[q][kq * 4 + 0], v[q]);
                v[q] = fmaf(a.y, bw[q][kq * 4 + 1], v[q]);
                v[q] = fmaf(a.z, bw[q][kq * 4 + 2], v[q]);
                v[q] = fmaf(a.w, bw[q][kq * 4 + 3], v[q]);
            }
        }
        if (g.bias) {
#pragma unroll
            for (int q = 0; q < 4; ++q) v[q] = __fadd_rn(v[q], bias[q]);
        }
        if (g.relu) {
#pragma unroll
            for (int q = 0; q < 4; ++q) v[q] = v[q] > 0.0f ? v[q] : 0.0f;
        }
        if (VEC) {
            if (g.mask) {
                const float4 mk = __ldcs(reinterpret_cast<const float4*>(g.mask + row * N + j0));
                v[0] = mk.x > 0.0f ? v[0] : 0.0f; v[1] = mk.y > 0.0f ? v[1] : 0.0f;
                v[2] = mk.z > 0.0f ? v[2] : 0.0f; v[3] = mk.w > 0.0f ? v[3] : 0.0f;
            }
            if (g.round_tf32) {
#pragma unroll
                for (int q = 0; q < 4; ++q) v[q] = rn_tf32(v[q]);
            }
            *reinterpret_cast<float4*>(g.c + row * N + j0) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (j0 + q < N) {
                    if (g.mask) v[q] = g.mask[row * N + j0 + q] > 0.0f ? v[q] : 0.0f;
                    if (g.round_tf32) v[q] = rn_tf32(v[q]);
                    g.c[row * N + j0 + q] = v[q];
                } else {
                    v[q] = 0.0f;
                }
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) cs[q] += v[q];
    }
    if (g.colsum_partial) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (j0 + q < N) g.colsum_partial[(size_t)blockIdx.x * N + j0 + q] = cs[q];
    }
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// 0: not a thin product; 1 thin_n_nn, 2 thin_n_tn, 3 thin_k_nt.  The long dimensions must be long enough for the layout
// to pay; everything else stays on the tiled kernels.
int thin_case(const GemmArgs& g) {
    static const bool on = [] { const char* e = getenv("TS_GEMM_THIN"); return !(e && e[0] == '0'); }();   // TS_GEMM_THIN=0: tiled kernels only
    if (!on) return 0;
    if (g.batch != 1 || g.a_lo || g.b_lo || !g.a || !g.b || !g.c) return 0;
    if (g.m == 0 || g.n == 0 || g.k == 0) return 0;
    if (g.m >= (1ull << 31) || g.n >= (1ull << 31) || g.k >= (1ull << 31)) return 0;
    if (!g.trans_a && !g.trans_b && g.n <= (size_t)kThin && g.m >= 256 && g.k >= 128) return 1;
    if (g.trans_a && !g.trans_b && g.n <= (size_t)kThin && g.k >= 256 && g.m >= 64 && !g.bias && !g.relu && !g.mask && !g.round_tf32) return 2;
    if (!g.trans_a && g.trans_b && g.k <= (size_t)kThin && g.m >= 256 && g.n >= 128 && (g.n + 1023) / 1024 <= 65535) return 3;
    return 0;
}

template <int NP>
bool launch_nn(const GemmArgs& g, cudaStream_t s) {
    if (g.m >= 16384) {   // many rows: small CTAs, several per SM
        constexpr int KC = NP == 4 ? 3072 : (NP == 16 ? 512 : 1024);
        launch_dep(thin_n_nn_kernel<NP, 2, KC>, dim3((unsigned)((g.m + 15) / 16)), dim3(kThreads), 0, s, g);
    } else {
        launch_dep(thin_n_nn_kernel<NP, 4, 512>, dim3((unsigned)((g.m + 31) / 32)), dim3(kThreads), 0, s, g);
    }
    return cuda_ok(cudaGetLastError(), "thin GEMM (NN) launch");
}
template <int NP>
bool launch_tn(const GemmArgs& g, float* out, unsigned col_blocks, unsigned slabs, unsigned rows_per_slab, cudaStream_t s) {
    launch_dep(thin_n_tn_kernel<NP>, dim3(col_blocks, slabs), dim3(kThreads), 0, s, g, out, rows_per_slab);
    return cuda_ok(cudaGetLastError(), "thin GEMM (TN) launch");
}
template <int NP>
bool launch_tn4(const GemmArgs& g, float* out, unsigned col_blocks, unsigned slabs, unsigned rows_per_slab, cudaStream_t s) {
    launch_dep(thin_n_tn4_kernel<NP>, dim3(col_blocks, slabs), dim3(128), 0, s, g, out, rows_per_slab);
    return cuda_ok(cudaGetLastError(), "thin GEMM (TN, 128-bit loads) launch");
}
template <int KP>
bool launch_nt(const GemmArgs& g, cudaStream_t s) {
    const int rows = nt_rows(g.m);
    const dim3 grid((unsigned)((g.m + rows - 1) / rows), (unsigned)((g.n + 1023) / 1024));
    const bool vec = g.n % 4 == 0 && al16(g.c) && (!g.mask || al16(g.mask));
    if (rows == 64) {
        if (vec) launch_dep(thin_k_nt_kernel<KP, true, 64>, grid, dim3(kThreads), 0, s, g);
        else launch_dep(thin_k_nt_kernel<KP, false, 64>, grid, dim3(kThreads), 0, s, g);
    } else {
        if (vec) launch_dep(thin_k_nt_kernel<KP, true, 16>, grid, dim3(kThreads), 0, s, g);
        else launch_dep(thin_k_nt_kernel<KP, false, 16>, grid, dim3(kThreads), 0, s, g);
    }
    return cuda_ok(cudaGetLastError(), "thin GEMM (NT) launch");
}

}  // namespace

int gemm_thin_kind(const GemmArgs& g) { return thin_case(g); }
bool gemm_thin_supported(const GemmArgs& g) { return thin_case(g) != 0; }
bool gemm_thin_rounds(const GemmArgs& g) { const int t = thin_case(g); return t == 1 || t == 3; }

bool gemm_thin(const GemmArgs& g, DeviceCtx* c, cudaStream_t s) {
    const int which = thin_case(g);
    if (!which || !c) { set_error("gemm: not a thin product"); return false; }
    if (g.colsum_out && !(which == 3 && g.colsum_partial)) {
        if (which == 3) {
            // column sums of the stored result: one partial row per CTA row of the kernel, added in row order
            const size_t prow = (g.m + nt_rows(g.m) - 1) / nt_rows(g.m);
            float* part = c->alloc.alloc(prow * g.n * sizeof(float));
            if (!part) return false;
            GemmArgs h = g;
            h.colsum_partial = part;
            bool ok = gemm_thin(h, c, s) && colsum_finish(part, g.colsum_out, g.n, prow, s);
            if (s != c->compute) cudaStreamSynchronize(s);   // the block is recycled in compute-stream order only
            c->alloc.free(part);
            return ok;
        }
        GemmArgs h = g;
        h.colsum_out = nullptr;
        if (!gemm_thin(h, c, s)) return false;
        float* scratch = c->alloc.alloc(colsum_scratch_elems(g.m, g.n) * sizeof(float));
        if (!scratch) return false;
        bool ok = colsum(g.c, g.colsum_out, g.m, g.n, scratch, s);
        if (s != c->compute) cudaStreamSynchronize(s);
        c->alloc.free(scratch);
        return ok;
    }
    const double flop = 2.0 * (double)g.m * (double)g.n * (double)g.k;
    if (which == 1) {
        ProfScope prof(kProfGemmFp32, s, flop);
        const size_t np = (g.n + 3) / 4 * 4;
        return np == 4 ? launch_nn<4>(g, s) : np == 8 ? launch_nn<8>(g, s) : np == 12 ? launch_nn<12>(g, s) : launch_nn<16>(g, s);
    }
    if (which == 3) {
        ProfScope prof(kProfGemmFp32, s, flop);
        const size_t kp = (g.k + 3) / 4 * 4;
        return kp == 4 ? launch_nt<4>(g, s) : kp == 8 ? launch_nt<8>(g, s) : kp == 12 ? launch_nt<12>(g, s) : launch_nt<16>(g, s);
    }
    // weight-gradient layout: K is cut into slabs whose partial results a second launch adds in slab order.  With 128-bit
    // loads (m % 4 == 0, aligned A): 128 columns and 128 threads per CTA, about four CTAs per SM, at least 32 rows a slab;
    // otherwise 32 columns and 256 threads per CTA, about two CTAs per SM, at least 64 rows a slab.
    // (a reduction of a few thousand rows is faster on the first kernel with its few slabs: 10.0 against 13.3 us for
    // 1024 x 10 over K = 4096; over K = 65536 the second one takes 0.089 against 0.156 ms)
    const bool wide = g.m % 4 == 0 && al16(g.a) && g.k >= 16384;
    const size_t col_blocks = wide ? (g.m + 127) / 128 : (g.m + 31) / 32;
    size_t slabs = (size_t)c->sm_count * (wide ? 4 : 2) / col_blocks;
    const size_t min_rows = wide ? 32 : 64;
    if (slabs > g.k / min_rows) slabs = g.k / min_rows;
    if (slabs > 65535) slabs = 65535;
    if (slabs < 1) slabs = 1;
    size_t rows_per_slab = (g.k + slabs - 1) / slabs;
    rows_per_slab = (rows_per_slab + 7) / 8 * 8;
    slabs = (g.k + rows_per_slab - 1) / rows_per_slab;   // no empty slab
    const size_t mn = g.m * g.n;
    const size_t np = (g.n + 3) / 4 * 4;
    float* part = nullptr;
    if (slabs > 1) {
        part = c->alloc.alloc(slabs * mn * sizeof(float));
        if (!part) return false;
    }
    float* out = part ? part : g.c;
    bool ok;
    {
        ProfScope prof(kProfGemmFp32, s, flop);
        const unsigned cb = (unsigned)col_blocks, sl = (unsigned)slabs, rps = (unsigned)rows_per_slab;
        if (wide)
            ok = np == 4 ? launch_tn4<4>(g, out, cb, sl, rps, s) : np == 8 ? launch_tn4<8>(g, out, cb, sl, rps, s)
                 : np == 12 ? launch_tn4<12>(g, out, cb, sl, rps, s) : launch_tn4<16>(g, out, cb, sl, rps, s);
        else
            ok = np == 4 ? launch_tn<4>(g, out, cb, sl, rps, s) : np == 8 ? launch_tn<8>(g, out, cb, sl, rps, s)
                 : np == 12 ? launch_tn<12>(g, out, cb, sl, rps, s) : launch_tn<16>(g, out, cb, sl, rps, s);
    }
    if (part) {
        // many slabs of a small result: lanes along the outputs, warps along the slabs (contiguous reads); few: one thread per output
        ok = ok && (slabs > 8 && mn >= 1024 ? colsum_finish(part, g.c, mn, slabs, s) : sum_slabs(part, g.c, mn, slabs, s));
        if (s != c->compute) cudaStreamSynchronize(s);
        c->alloc.free(part);
    }
    return ok;
}

}  // namespace k
}  // namespace ts
