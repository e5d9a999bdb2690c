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

constexpr int BM = 128, BN = 128, BK = 16, kThreads = 256;

// One operand tile (128 rows or columns x 16 k) from global memory into 8 registers per thread, and from there into
// shared memory as [k][128].  K_CONTIG: the operand is stored with k contiguous (A not transposed, B transposed):
// a thread takes 4 consecutive k of one row and scatters them; otherwise the 128-wide dimension is contiguous and a
// thread takes 4 consecutive elements of one k row.  The vector path needs an aligned base, a leading dimension that
// is a multiple of 4 and a tile that lies inside the matrix; edge tiles and odd pitches take scalar guarded loads.
template <bool K_CONTIG>
__device__ __forceinline__ void tile_load(float (&r)[8], const float* __restrict__ base, size_t ld, size_t x0, size_t X, size_t k0, size_t K,
                                          bool vec) {
    const int t = threadIdx.x;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (K_CONTIG) {
            const size_t x = x0 + t / 4 + 64 * h, p = k0 + (t % 4) * 4;
            if (vec && x < X && p + 4 <= K) {
                const float4 v = *reinterpret_cast<const float4*>(base + x * ld + p);
                r[4 * h] = v.x; r[4 * h + 1] = v.y; r[4 * h + 2] = v.z; r[4 * h + 3] = v.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) r[4 * h + e] = (x < X && p + e < K) ? base[x * ld + p + e] : 0.0f;
            }
        } else {
            const size_t p = k0 + t / 32 + 8 * h, x = x0 + (t % 32) * 4;
            if (vec && p < K && x + 4 <= X) {
                const float4 v = *reinterpret_cast<const float4*>(base + p * ld + x);
                r[4 * h] = v.x; r[4 * h + 1] = v.y; r[4 * h + 2] = v.z; r[4 * h + 3] = v.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) r[4 * h + e] = (p < K && x + e < X) ? base[p * ld + x + e] : 0.0f;
            }
        }
    }
}
// Column swizzle of the shared-memory tiles: in k-row p the 128 columns are stored at column ^ swz(p), which moves whole
// groups of 8 floats inside each 32-float window by (p / 4) mod 4.  A k-contiguous operand is written as scalars, four
// lanes of a warp holding the same column of four different groups of k-rows: without the swizzle those four hit one bank
// (rows are 128 floats apart), with it they land in four different groups of banks.  Reads are 128-bit at multiples of
// four columns, which the swizzle keeps whole.
__device__ __forceinline__ int swz(int p) { return ((p >> 2) & 3) << 3; }

template <bool K_CONTIG>
__device__ __forceinline__ void tile_store(float (*sm)[BM], const float (&r)[8]) {
    const int t = threadIdx.x;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (K_CONTIG) {
            const int kc = (t % 4) * 4, x = (t / 4 + 64 * h) ^ swz(kc);   // rows kc .. kc + 3 share one swizzle
#pragma unroll
            for (int e = 0; e < 4; ++e) sm[kc + e][x] = r[4 * h + e];
        } else {
            const int kr = t / 32 + 8 * h, x = ((t % 32) * 4) ^ swz(kr);
            *reinterpret_cast<float4*>(&sm[kr][x]) = make_float4(r[4 * h], r[4 * h + 1], r[4 * h + 2], r[4 * h + 3]);
        }
    }
}

template <bool TA, bool TB, bool HAS_TAIL>
__global__ void __launch_bounds__(kThreads, 2) sgemm_kernel(GemmArgs g) {
    grid_dependency_sync();
    g.a += (size_t)blockIdx.z * g.batch_stride_a;     // one product per grid z (a batch of 1 has strides 0)
    g.b += (size_t)blockIdx.z * g.batch_stride_b;
    g.c += (size_t)blockIdx.z * g.m * g.n;
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
    // A thread's columns are two aligned groups of four, and the boundary N/8*8 is a multiple of 8: a group is tail or not as a whole.
    const bool tail_lo = HAS_TAIL && n0 + tx * 4 >= N / 8 * 8;
    const bool tail_hi = HAS_TAIL && n0 + 64 + tx * 4 >= N / 8 * 8;

    // A is [M][K] (k contiguous) unless TA, then [K][M]; B is [K][N] unless TB, then [N][K] (k contiguous)
    const size_t lda = TA ? M : K, ldb = TB ? K : N;
    const bool vec_a = (reinterpret_cast<uintptr_t>(g.a) & 15) == 0 && lda % 4 == 0;
    const bool vec_b = (reinterpret_cast<uintptr_t>(g.b) & 15) == 0 && ldb % 4 == 0;
    float ra[8], rb[8];
    // Where this thread's two 128-bit loads of each operand start (at k = 0) and whether they lie inside the matrix: the
    // index arithmetic of tile_load is done once, and a k-tile that lies wholly inside K (all but possibly the last)
    // costs a pointer bump and a load per half instead of a dozen integer instructions that compete with the FFMAs for
    // issue slots.  Anything else (edge rows or columns, odd pitches, the partial last tile) takes tile_load's guarded path.
    const float* fa;   // this thread's first load of the NEXT k-tile of A (its second one lies 64 rows, or 8 k-rows, further on)
    const float* fb;
    bool fast;
    {
        const size_t xa = !TA ? m0 + t / 4 : m0 + (t % 32) * 4, xb = TB ? n0 + t / 4 : n0 + (t % 32) * 4;
        fa = !TA ? g.a + xa * lda + (t % 4) * 4 : g.a + (size_t)(t / 32) * lda + xa;
        fb = TB ? g.b + xb * ldb + (t % 4) * 4 : g.b + (size_t)(t / 32) * ldb + xb;
        fast = vec_a && vec_b && (!TA ? xa + 64 < M : xa + 4 <= M) && (TB ? xb + 64 < N : xb + 4 <= N);
    }
    auto load_tiles = [&](size_t k0) {
        const float* pa = fa;
        const float* pb = fb;
        fa += !TA ? (size_t)BK : (size_t)BK * lda;     // calls come in k order, one per tile
        fb += TB ? (size_t)BK : (size_t)BK * ldb;
        if (fast && k0 + BK <= K) {
            const float4 va0 = *reinterpret_cast<const float4*>(pa), va1 = *reinterpret_cast<const float4*>(pa + (!TA ? 64 : 8) * lda);
            const float4 vb0 = *reinterpret_cast<const float4*>(pb), vb1 = *reinterpret_cast<const float4*>(pb + (TB ? 64 : 8) * ldb);
            ra[0] = va0.x; ra[1] = va0.y; ra[2] = va0.z; ra[3] = va0.w; ra[4] = va1.x; ra[5] = va1.y; ra[6] = va1.z; ra[7] = va1.w;
            rb[0] = vb0.x; rb[1] = vb0.y; rb[2] = vb0.z; rb[3] = vb0.w; rb[4] = vb1.x; rb[5] = vb1.y; rb[6] = vb1.z; rb[7] = vb1.w;
            return;
        }
        tile_load<!TA>(ra, g.a, lda, m0, M, k0, K, vec_a);
        tile_load<TB>(rb, g.b, ldb, n0, N, k0, K, vec_b);
    };
    auto store_tiles = [&](int buf) {
        tile_store<!TA>(As[buf], ra);
        tile_store<TB>(Bs[buf], rb);
    };
    auto k_step = [&](int buf, int p) {
        const int ca = (ty * 4) ^ swz(p), cb = (tx * 4) ^ swz(p);
        float4 a0 = *reinterpret_cast<const float4*>(&As[buf][p][ca]);
        float4 a1 = *reinterpret_cast<const float4*>(&As[buf][p][64 + ca]);
        float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][p][cb]);
        float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][p][64 + cb]);
        float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        if (HAS_TAIL && (tail_lo || tail_hi)) {
            // only threads of the last column block get here: a rounded multiply, then an add (kernels.rs:312-335)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                if (half == 0 ? tail_lo : tail_hi) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            acc[i][half * 4 + j] = __fadd_rn(acc[i][half * 4 + j], __fmul_rn(av[i], bv[half * 4 + j]));
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[i][half * 4 + j] = fmaf(av[i], bv[half * 4 + j], acc[i][half * 4 + j]);
                }
            }
        } else {
            // boustrophedon over the 8 x 8 outputs: consecutive FFMAs share one operand (a row's a value along the row, the
            // b value at the turn), which is what the operand reuse of the register file rewards
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                // two rows per instruction: the packed FP32 fused multiply-add of sm_100 (each half is an ordinary
                // fmaf, so the bits are those of 64 single FFMAs) halves the instructions this issue-bound loop needs
                const float2 bd = make_float2(bv[j], bv[j]);
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    const int ip = (j & 1) ? 3 - ii : ii;
                    const float2 c = __ffma2_rn(make_float2(av[2 * ip], av[2 * ip + 1]), bd, make_float2(acc[2 * ip][j], acc[2 * ip + 1][j]));
                    acc[2 * ip][j] = c.x;
                    acc[2 * ip + 1][j] = c.y;
                }
            }
        }
    };

    const size_t ktiles = (K + BK - 1) / BK;
    if (ktiles > 0) {
        load_tiles(0);
        store_tiles(0);
    }
    __syncthreads();
    for (size_t kt = 0; kt < ktiles; ++kt) {
        const int buf = (int)(kt & 1);
        // the next tile's loads are issued a whole tile (16 k steps, about a thousand instructions) ahead of their use
        if (kt + 1 < ktiles) load_tiles((kt + 1) * BK);
        if ((kt + 1) * BK <= K) {
#pragma unroll
            for (int p = 0; p < BK; ++p) k_step(buf, p);
        } else {
            // last, partial tile: only the k that exist enter the chain (a padded fma(0, 0, acc) would turn -0 into +0)
            const int pmax = (int)(K - kt * BK);
            for (int p = 0; p < pmax; ++p) k_step(buf, p);
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
    if (g.n % 8 != 0) launch_dep(sgemm_kernel<TA, TB, true>, dim3(grid), dim3(kThreads), 0, s, g);
    else launch_dep(sgemm_kernel<TA, TB, false>, dim3(grid), dim3(kThreads), 0, s, g);
}

// The same arithmetic on 32 x 32 tiles (2 x 2 outputs per thread, 32 k per stage) for results that would fill only a
// few 128 x 128 tiles: a [1024 x 10] bias-layer weight gradient reduced over 4096 rows is 8 CTAs of the big kernel,
// each walking all of K alone, but 32 CTAs here.  Per output element the chain over p is unchanged.
// These shapes are latency-bound (a handful of CTAs, each walking all of K), so the k-stages arrive through a ring
// of asynchronous 4-byte copies (transposing as they land, zero-filled outside the matrices) three stages ahead of
// the one being multiplied: a stage costs its 32 multiply-add steps, not a round trip to memory.
constexpr int SM_T = 32;
constexpr int SM_STAGES = 4;

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(valid ? 4 : 0) : "memory");
}

template <bool TA, bool TB, bool HAS_TAIL>
__global__ void __launch_bounds__(kThreads) sgemm_small_kernel(GemmArgs g) {
    grid_dependency_sync();
    g.a += (size_t)blockIdx.z * g.batch_stride_a;     // one product per grid z (a batch of 1 has strides 0)
    g.b += (size_t)blockIdx.z * g.batch_stride_b;
    g.c += (size_t)blockIdx.z * g.m * g.n;
    __shared__ float As[SM_STAGES][SM_T][SM_T + 1];   // [stage][k][m]
    __shared__ float Bs[SM_STAGES][SM_T][SM_T + 1];   // [stage][k][n]
    const int t = threadIdx.x, ty = t / 16, tx = t % 16;
    const size_t m0 = (size_t)blockIdx.y * SM_T, n0 = (size_t)blockIdx.x * SM_T;
    const size_t M = g.m, N = g.n, K = g.k;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    bool tailc[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) tailc[j] = HAS_TAIL && (n0 + tx * 2 + j) >= N / 8 * 8;

    auto issue = [&](int slot, size_t k0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int e = t + kThreads * q, lo = e % SM_T, hi = e / SM_T;
            {   // A: stored [K][M] (TA, contiguous along m) or [M][K] (contiguous along k)
                const int kk = TA ? hi : lo, mm = TA ? lo : hi;
                const size_t p = k0 + kk, i = m0 + mm;
                const bool in = p < K && i < M;
                cp_async4(&As[slot][kk][mm], in ? (TA ? g.a + p * M + i : g.a + i * K + p) : g.a, in);
            }
            {   // B: stored [N][K] (TB, contiguous along k) or [K][N] (contiguous along n)
                const int kk = TB ? lo : hi, nn = TB ? hi : lo;
                const size_t p = k0 + kk, j = n0 + nn;
                const bool in = p < K && j < N;
                cp_async4(&Bs[slot][kk][nn], in ? (TB ? g.b + j * K + p : g.b + p * N + j) : g.b, in);
            }
        }
    };

    const size_t nk = (K + SM_T - 1) / SM_T;
#pragma unroll
    for (int st = 0; st < SM_STAGES - 1; ++st) {
        if ((size_t)st < nk) issue(st, (size_t)st * SM_T);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    for (size_t kt = 0; kt < nk; ++kt) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(SM_STAGES - 2) : "memory");   // this thread's part of stage kt landed
        __syncthreads();                            // everyone's part landed; everyone is done with stage kt - 1
        const size_t nxt = kt + SM_STAGES - 1;
        if (nxt < nk) issue((int)(nxt % SM_STAGES), nxt * SM_T);     // into the slot stage kt - 1 used
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        const int slot = (int)(kt % SM_STAGES);
        const size_t k0 = kt * SM_T;
        const int pmax = (K - k0) < (size_t)SM_T ? (int)(K - k0) : SM_T;   // no padded terms enter the chain
#pragma unroll 8
        for (int p = 0; p < pmax; ++p) {
            const float a0 = As[slot][p][ty * 2], a1 = As[slot][p][ty * 2 + 1];
            const float b[2] = {Bs[slot][p][tx * 2], Bs[slot][p][tx * 2 + 1]};
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
    if (g.n % 8 != 0) launch_dep(sgemm_small_kernel<TA, TB, true>, dim3(grid), dim3(kThreads), 0, s, g);
    else launch_dep(sgemm_small_kernel<TA, TB, false>, dim3(grid), dim3(kThreads), 0, s, g);
}

// The smallest tiling: 16 x 16 tiles, 64 threads, 2 x 2 outputs per thread, 64 k per stage, for results of fewer than
// 74 tiles of 32 x 32 with K <= 1024 (see the dispatch in sgemm()): a quarter of the outputs per CTA is a quarter of
// the work per step of the chain, and four times the CTAs spread over SMs that would have been idle.  Per output
// element the chain over p is unchanged.
constexpr int TN_T = 16, TN_K = 64, TN_THREADS = 64, TN_PITCH = TN_T + 2;    // rows stay 8-byte aligned

template <bool TA, bool TB, bool HAS_TAIL>
__global__ void __launch_bounds__(TN_THREADS) sgemm_tiny_kernel(GemmArgs g) {
    grid_dependency_sync();
    g.a += (size_t)blockIdx.z * g.batch_stride_a;     // one product per grid z (a batch of 1 has strides 0)
    g.b += (size_t)blockIdx.z * g.batch_stride_b;
    g.c += (size_t)blockIdx.z * g.m * g.n;
    __shared__ __align__(16) float As[SM_STAGES][TN_K][TN_PITCH];   // [stage][k][m]
    __shared__ __align__(16) float Bs[SM_STAGES][TN_K][TN_PITCH];   // [stage][k][n]
    const int t = threadIdx.x, ty = t / 8, tx = t % 8;              // rows ty*2 .. +1, columns tx*2 .. +1
    const size_t m0 = (size_t)blockIdx.y * TN_T, n0 = (size_t)blockIdx.x * TN_T;
    const size_t M = g.m, N = g.n, K = g.k;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    // a thread's two columns are one aligned pair, and the boundary N/8*8 is even: tail or not as a whole
    const bool tail = HAS_TAIL && n0 + tx * 2 >= N / 8 * 8;

    auto issue = [&](int slot, size_t k0) {
#pragma unroll
        for (int q = 0; q < TN_T * TN_K / TN_THREADS; ++q) {
            const int e = t + TN_THREADS * q;             // 0 .. 511: one element of the 16 x 32 operand tile
            {   // A: stored [K][M] (TA, contiguous along m) or [M][K] (contiguous along k)
                const int kk = TA ? e / TN_T : e % TN_K, mm = TA ? e % TN_T : e / TN_K;
                const size_t p = k0 + kk, i = m0 + mm;
                const bool in = p < K && i < M;
                cp_async4(&As[slot][kk][mm], in ? (TA ? g.a + p * M + i : g.a + i * K + p) : g.a, in);
            }
            {   // B: stored [N][K] (TB, contiguous along k) or [K][N] (contiguous along n)
                const int kk = TB ? e % TN_K : e / TN_T, nn = TB ? e / TN_K : e % TN_T;
                const size_t p = k0 + kk, j = n0 + nn;
                const bool in = p < K && j < N;
                cp_async4(&Bs[slot][kk][nn], in ? (TB ? g.b + j * K + p : g.b + p * N + j) : g.b, in);
            }
        }
    };

    const size_t nk = (K + TN_K - 1) / TN_K;
#pragma unroll
    for (int st = 0; st < SM_STAGES - 1; ++st) {
        if ((size_t)st < nk) issue(st, (size_t)st * TN_K);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    for (size_t kt = 0; kt < nk; ++kt) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(SM_STAGES - 2) : "memory");
        __syncthreads();
        const size_t nxt = kt + SM_STAGES - 1;
        if (nxt < nk) issue((int)(nxt % SM_STAGES), nxt * TN_K);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        const int slot = (int)(kt % SM_STAGES);
        const size_t k0 = kt * TN_K;
        const int pmax = (K - k0) < (size_t)TN_K ? (int)(K - k0) : TN_K;    // no padded terms enter the chain
#pragma unroll 8
        for (int p = 0; p < pmax; ++p) {
            const float2 a2 = *reinterpret_cast<const float2*>(&As[slot][p][ty * 2]);
            const float2 b2 = *reinterpret_cast<const float2*>(&Bs[slot][p][tx * 2]);
            if (HAS_TAIL && tail) {
                acc[0][0] = __fadd_rn(acc[0][0], __fmul_rn(a2.x, b2.x)); acc[0][1] = __fadd_rn(acc[0][1], __fmul_rn(a2.x, b2.y));
                acc[1][0] = __fadd_rn(acc[1][0], __fmul_rn(a2.y, b2.x)); acc[1][1] = __fadd_rn(acc[1][1], __fmul_rn(a2.y, b2.y));
            } else {
                acc[0][0] = fmaf(a2.x, b2.x, acc[0][0]); acc[0][1] = fmaf(a2.x, b2.y, acc[0][1]);
                acc[1][0] = fmaf(a2.y, b2.x, acc[1][0]); acc[1][1] = fmaf(a2.y, b2.y, acc[1][1]);
            }
        }
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
void launch_tiny(const GemmArgs& g, dim3 grid, cudaStream_t s) {
    if (g.n % 8 != 0) launch_dep(sgemm_tiny_kernel<TA, TB, true>, dim3(grid), dim3(TN_THREADS), 0, s, g);
    else launch_dep(sgemm_tiny_kernel<TA, TB, false>, dim3(grid), dim3(TN_THREADS), 0, s, g);
}

// Between the two: 64 x 64 tiles, 4 x 4 outputs per thread, 16 k per stage through the same ring of asynchronous
// copies.  For results of a few hundred such tiles (1024 x 1024, or a batch of 128 x 128 products) the 128 x 128 tiles
// would leave most SMs idle and the 32 x 32 tiles spend one shared-memory load per multiply-add; here it is one
// 128-bit load per eight.  Per output element the chain over p is again unchanged.
constexpr int MD_T = 64, MD_K = 16, MD_PITCH = MD_T + 4;     // rows stay 16-byte aligned

template <bool TA, bool TB, bool HAS_TAIL>
__global__ void __launch_bounds__(kThreads) sgemm_mid_kernel(GemmArgs g) {
    grid_dependency_sync();
    g.a += (size_t)blockIdx.z * g.batch_stride_a;     // one product per grid z (a batch of 1 has strides 0)
    g.b += (size_t)blockIdx.z * g.batch_stride_b;
    g.c += (size_t)blockIdx.z * g.m * g.n;
    __shared__ __align__(16) float As[SM_STAGES][MD_K][MD_PITCH];   // [stage][k][m]
    __shared__ __align__(16) float Bs[SM_STAGES][MD_K][MD_PITCH];   // [stage][k][n]
    const int t = threadIdx.x, ty = t / 16, tx = t % 16;
    const size_t m0 = (size_t)blockIdx.y * MD_T, n0 = (size_t)blockIdx.x * MD_T;
    const size_t M = g.m, N = g.n, K = g.k;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    // a thread's four columns are one aligned group, and the boundary N/8*8 is a multiple of 8: tail or not as a whole
    const bool tail = HAS_TAIL && n0 + tx * 4 >= N / 8 * 8;

    auto issue = [&](int slot, size_t k0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int e = t + kThreads * q;               // 0 .. 1023: one element of the 64 x 16 operand tile
            {   // A: stored [K][M] (TA, contiguous along m) or [M][K] (contiguous along k)
                const int kk = TA ? e / MD_T : e % MD_K, mm = TA ? e % MD_T : e / MD_K;
                const size_t p = k0 + kk, i = m0 + mm;
                const bool in = p < K && i < M;
                cp_async4(&As[slot][kk][mm], in ? (TA ? g.a + p * M + i : g.a + i * K + p) : g.a, in);
            }
            {   // B: stored [N][K] (TB, contiguous along k) or [K][N] (contiguous along n)
                const int kk = TB ? e % MD_K : e / MD_T, nn = TB ? e / MD_K : e % MD_T;
                const size_t p = k0 + kk, j = n0 + nn;
                const bool in = p < K && j < N;
                cp_async4(&Bs[slot][kk][nn], in ? (TB ? g.b + j * K + p : g.b + p * N + j) : g.b, in);
            }
        }
    };

    const size_t nk = (K + MD_K - 1) / MD_K;
#pragma unroll
    for (int st = 0; st < SM_STAGES - 1; ++st) {
        if ((size_t)st < nk) issue(st, (size_t)st * MD_K);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    for (size_t kt = 0; kt < nk; ++kt) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(SM_STAGES - 2) : "memory");
        __syncthreads();
        const size_t nxt = kt + SM_STAGES - 1;
        if (nxt < nk) issue((int)(nxt % SM_STAGES), nxt * MD_K);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        const int slot = (int)(kt % SM_STAGES);
        const size_t k0 = kt * MD_K;
        const int pmax = (K - k0) < (size_t)MD_K ? (int)(K - k0) : MD_K;    // no padded terms enter the chain
#pragma unroll 4
        for (int p = 0; p < pmax; ++p) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[slot][p][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4*>(&Bs[slot][p][tx * 4]);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
            if (HAS_TAIL && tail) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 bd = make_float2(bv[j], bv[j]);   // two rows per packed FP32x2 fused multiply-add, as in sgemm_kernel
#pragma unroll
                    for (int ii = 0; ii < 2; ++ii) {
                        const int ip = (j & 1) ? 1 - ii : ii;
                        const float2 c = __ffma2_rn(make_float2(av[2 * ip], av[2 * ip + 1]), bd, make_float2(acc[2 * ip][j], acc[2 * ip + 1][j]));
                        acc[2 * ip][j] = c.x;
                        acc[2 * ip + 1][j] = c.y;
                    }
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const size_t row = m0 + ty * 4 + i;
        if (row >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const size_t col = n0 + tx * 4 + j;
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
void launch_mid(const GemmArgs& g, dim3 grid, cudaStream_t s) {
    if (g.n % 8 != 0) launch_dep(sgemm_mid_kernel<TA, TB, true>, dim3(grid), dim3(kThreads), 0, s, g);
    else launch_dep(sgemm_mid_kernel<TA, TB, false>, dim3(grid), dim3(kThreads), 0, s, g);
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
    if (g.batch == 0) return true;
    if (g.batch > 65535 || (g.batch > 1 && (g.bias || g.mask))) { set_error("gemm: unsupported batch of %zu products", g.batch); return false; }
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)g.batch);
    ProfScope prof(kProfGemmFp32, s, 2.0 * (double)g.m * (double)g.n * (double)g.k * (double)g.batch);
    DeviceCtx* c = ctx();
    const size_t sgy = (g.m + SM_T - 1) / SM_T;
    const size_t mgx = (g.n + MD_T - 1) / MD_T, mgy = (g.m + MD_T - 1) / MD_T;
    // A result at most 32 columns wide (the 10-class output layer and its weight gradient) would be mostly padding in
    // 128- or 64-wide tiles, however many of them there are: it goes straight to the 32- and 16-wide tilings below.
    const bool narrow = g.n <= (size_t)SM_T;
    if (!narrow && c && gx * gy * g.batch < (size_t)c->sm_count / 2 && mgx * mgy * g.batch >= (size_t)c->sm_count / 2 && mgy <= 65535) {
        // too few 128 x 128 tiles to occupy the GPU, enough 64 x 64 ones
        dim3 mgrid((unsigned)mgx, (unsigned)mgy, (unsigned)g.batch);
        if (g.trans_a) { if (g.trans_b) launch_mid<true, true>(g, mgrid, s); else launch_mid<true, false>(g, mgrid, s); }
        else { if (g.trans_b) launch_mid<false, true>(g, mgrid, s); else launch_mid<false, false>(g, mgrid, s); }
        return cuda_ok(cudaGetLastError(), "sgemm (64 x 64 tiles) launch");
    }
    const size_t sgx = (g.n + SM_T - 1) / SM_T, tgy = (g.m + TN_T - 1) / TN_T;
    if (c && sgx * sgy * g.batch < (size_t)c->sm_count / 2 && tgy <= 65535 && g.k <= 1024) {
        // too few even of 32 x 32 tiles and a short chain: 16 x 16 ones.  Measured, not derived: the 32 x 784 . 784 x 128
        // product runs 15 % faster here, but a [1024 x 10] result over K = 4096 took 236 us against 143 us on 32 x 32
        // tiles, so long chains stay there.
        dim3 tgrid((unsigned)((g.n + TN_T - 1) / TN_T), (unsigned)tgy, (unsigned)g.batch);
        if (g.trans_a) { if (g.trans_b) launch_tiny<true, true>(g, tgrid, s); else launch_tiny<true, false>(g, tgrid, s); }
        else { if (g.trans_b) launch_tiny<false, true>(g, tgrid, s); else launch_tiny<false, false>(g, tgrid, s); }
        return cuda_ok(cudaGetLastError(), "sgemm (16 x 16 tiles) launch");
    }
    if (c && (narrow || gx * gy * g.batch < (size_t)c->sm_count / 2) && sgy <= 65535) {
        // too few even of those: 32 x 32 tiles, sixteen times as many CTAs as 128 x 128 ones
        dim3 sgrid((unsigned)((g.n + SM_T - 1) / SM_T), (unsigned)sgy, (unsigned)g.batch);
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
