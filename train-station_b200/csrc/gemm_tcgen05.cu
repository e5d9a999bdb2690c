// TF32 GEMM on the 5th-generation tensor cores of sm_100a: TMA -> shared-memory ring ->
// tcgen05.mma (kind::tf32, operands from shared memory, FP32 accumulators in tensor
// memory) -> tcgen05.ld epilogue (bias / ReLU / ReLU-mask) -> global stores.
//
// One persistent CTA per SM walks a grouped tile order.  Warp roles:
//   warp 0      : TMA producer (one lane)
//   warp 1      : tensor-memory allocation (whole warp) and MMA issue (one lane)
//   warps 2..5  : epilogue; warp w reads the TMEM lanes 32*(w%4) .. +31, one output row per thread
// The accumulator is double-buffered in tensor memory so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
// Operand layouts.  C[m,n] = sum_k A(m,k) B(k,n), all matrices row-major in global memory:
//   A stored [m][k]  -> "K-major":  TMA box 32(k) x 128 rows, 128-byte swizzle
//   A stored [k][m]  -> "MN-major": TMA boxes 32(m) x 32(k), four per tile, 128-byte swizzle of 32-byte chunks
//   B stored [n][k]  -> K-major;   B stored [k][n] -> MN-major (BN/32 boxes per tile)
// so forward (A K-major, B MN-major), dA = dC.B^T (both K-major) and dB = A^T.dC (both
// MN-major) all run without materialising a transpose.
//
// Every wait is bounded: when a barrier does not complete in about two seconds the waiting
// thread raises the CTA's abort flag, writes an error code to a global word that the host
// checks at its next synchronisation, drains its own copies (again bounded), and the CTA
// frees its tensor memory and returns.
//
// No TMA load in this file uses cluster multicast: each CTA fetches its own tiles.
#include <cuda.h>

#include <atomic>

#include "../../include/train_station_b200.h"
#include "common.h"

namespace ts {
namespace k {

namespace {

constexpr int BM = 128;          // rows of C per tile = TMEM lanes
constexpr int BK = 32;           // f32 elements of K per pipeline stage = one 128-byte swizzle row
constexpr int UMMA_K = 8;        // K of one tcgen05.mma.kind::tf32
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr long long kWaitCycles = 4000000000ll;   // about two seconds at 1.9 GHz
std::atomic<long long> g_wait_budget{kWaitCycles};  // host side: what the next one-CTA launch gets as its main-loop budget

enum ErrCode { kErrFullWait = 101, kErrEmptyWait = 102, kErrAccFullWait = 103, kErrAccEmptyWait = 104, kErrDrain = 105 };

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when it gave up or when another thread of the CTA already had.  `budget` is in clock
// cycles; the abort flag and the clock are looked at on the first failed poll and then every 256 polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, long long budget = kWaitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        if ((it & 255u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 >= budget) { *abort_flag = 1; return false; }
        }
        if (mbar_try_wait(bar, parity)) return true;
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] . B[smem]
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit accumulators: one row of 32 values per thread.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: layout type in bits 61..63, descriptor version 1 in bits 46..47.
// Addresses and offsets are stored without their 4 low bits.
// Layout types used here: 2 = 128-byte swizzle of 16-byte chunks (K-major operands);
// 1 = 128-byte swizzle of 32-byte chunks, the only swizzled layout the tensor core accepts for
// MN-major 32-bit operands (its atom is four k-rows of 128 bytes).
constexpr uint32_t kLayoutSw128 = 2, kLayoutSw128Base32 = 1;
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)layout_type << 61;
    return d;
}

// Instruction descriptor of kind::tf32 with FP32 accumulation:
// bits 4-5 D format (1 = F32), 7-9 A format (2 = TF32), 10-12 B format, 15 A major, 16 B major
// (0 = K, 1 = MN), 17-22 N >> 3, 24-28 M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(bool a_mn, bool b_mn, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}

// Column sums over the 32 rows a warp holds (one row per lane, 32 columns per lane in v): a transposing butterfly.
// Round `off` splits the columns a lane still holds in two halves, keeps the half its bit `off` selects and adds the
// partner's values for that half, so after five rounds lane j holds the sum of column j.  31 shuffles, fixed order.
__device__ __forceinline__ float warp_column_sums(float (&v)[32], int lane) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < off; ++i) {
            const float send = upper ? v[i] : v[i + off];
            const float keep = upper ? v[i + off] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    return v[0];
}

template <int BN>
struct Cfg {
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kABytes = BM * BK * 4;     // 16 KiB
    static constexpr int kBBytes = BN * BK * 4;     // 32 or 16 KiB
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;        // two accumulator buffers
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;   // + alignment slack
};

struct KernelArgs {
    float* c;
    const float* bias;
    const float* mask;
    int relu;
    int round_out;
    int a_grouped, b_grouped;   // MN-major operand described by a 3-D [group][k][32] tensor map
    int passes;                 // 1 = TF32, 3 = 3xTF32 (hi/lo split operands)
    uint32_t m, n, k;
    int* error_flag;
    // Split along K (one-CTA kernel only): work item = (tile, split); split s covers k-blocks
    // [s * kb_per_split, min((s + 1) * kb_per_split, num_kb)) and writes its partial product to c + s * m * n.
    uint32_t splits, kb_per_split;
    // Cycle budget of the main-loop waits of the one-CTA kernel (the drains before a CTA retires always keep the full
    // bound, so that no bulk copy is in flight when it does).  Normally kWaitCycles; a host test shortens it to see
    // the abort path run: error word set, tensor memory freed, kernel returns, context usable.
    long long wait_budget;
    // When set: column sums of the stored result (the bias gradient of the layer this result is the pre-activation
    // gradient of).  Row r of `colsum_partial` ([ceil(m / 32)][n], rounded up to whole tiles) receives the sums over rows
    // 32 r .. 32 r + 31; every element is written by exactly one warp, with no synchronisation between warps, and a
    // second kernel adds the rows in order.
    float* colsum_partial;
    // Two-CTA kernel: when set, tiles are handed out from this counter (zeroed before the launch) instead of by a fixed
    // stride: concurrently running pairs then stay on neighbouring tiles (shared panels stay in L2), and a pair that
    // starts late or runs slowly takes fewer tiles instead of stretching the whole launch.
    int* tile_counter;
    uint32_t stages;       // two-CTA kernel: depth of the shared-memory ring in use (stages of 32 KiB)
    uint32_t group;        // two-CTA kernel: row tiles that sweep the columns together (tile order)
    uint32_t l2_hints;     // two-CTA kernel: 0 none; 1 A evict_last + B evict_first; 2 both evict_first; 3 A evict_first + B evict_last
};

__device__ __forceinline__ float rn_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// one 32-column chunk of one output row: bias, ReLU, mask, rounding, store; the stored values are left in vals[]
// (zero for a row or a column outside the matrix) for the column sums
__device__ __forceinline__ void store_chunk(const KernelArgs& args, const uint32_t (&r)[32], float (&vals)[32], bool row_ok, float* crow,
                                            const float* mrow, uint32_t col0) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const uint32_t col = col0 + q * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row_ok && col < args.n) {   // n % 4 == 0: a float4 is either fully inside or fully outside
            v = make_float4(__uint_as_float(r[q * 4]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]),
                            __uint_as_float(r[q * 4 + 3]));
            if (args.bias) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(args.bias + col));
                v.x = __fadd_rn(v.x, b.x); v.y = __fadd_rn(v.y, b.y); v.z = __fadd_rn(v.z, b.z); v.w = __fadd_rn(v.w, b.w);
            }
            if (args.relu) {
                v.x = v.x > 0.f ? v.x : 0.f; v.y = v.y > 0.f ? v.y : 0.f; v.z = v.z > 0.f ? v.z : 0.f; v.w = v.w > 0.f ? v.w : 0.f;
            }
            if (mrow) {
                const float4 mk = __ldcs(reinterpret_cast<const float4*>(mrow + col));
                v.x = mk.x > 0.f ? v.x : 0.f; v.y = mk.y > 0.f ? v.y : 0.f; v.z = mk.z > 0.f ? v.z : 0.f; v.w = mk.w > 0.f ? v.w : 0.f;
            }
            if (args.round_out) { v.x = rn_tf32(v.x); v.y = rn_tf32(v.y); v.z = rn_tf32(v.z); v.w = rn_tf32(v.w); }
            *reinterpret_cast<float4*>(crow + col) = v;
        }
        vals[q * 4] = v.x; vals[q * 4 + 1] = v.y; vals[q * 4 + 2] = v.z; vals[q * 4 + 3] = v.w;
    }
}
template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_a_lo, const __grid_constant__ CUtensorMap tm_b_lo, KernelArgs args) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle atoms are 1024 bytes: align the ring to that.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + C::kStages * C::kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::kStages + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * C::kStages + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * C::kStages + 2 + a); };
    const uint32_t drain_bar = bar_base + 8u * (2 * C::kStages + 4);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + C::kStages * C::kStageBytes + 8 * (2 * C::kStages + 5));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t tiles_m = (args.m + BM - 1) / BM, tiles_n = (args.n + BN - 1) / BN;
    const uint32_t num_tiles = tiles_m * tiles_n;
    const uint32_t num_kb = (args.k + BK - 1) / BK;
    // Work items: every tile once per K split, split-major so that the items running together share their panels.
    const uint32_t num_items = num_tiles * args.splits;
    // 3xTF32: with a = a_hi + a_lo and b = b_hi + b_lo (each part exact in TF32), the accumulator receives
    // a_lo.b_hi, then a_hi.b_lo, then a_hi.b_hi: three sweeps over the item's k-blocks into the same tensor-memory tile.
    auto item_kb = [&](uint32_t item, uint32_t& kb_begin, uint32_t& kb_cnt) {
        kb_begin = (item / num_tiles) * args.kb_per_split;
        const uint32_t left = num_kb - kb_begin;
        kb_cnt = left < args.kb_per_split ? left : args.kb_per_split;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), kEpiThreads); }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    grid_dependency_sync();   // barriers and tensor memory are set up beside the tail of the kernel before; global memory from here on

    // grouped tile order: 16 row-tiles share their B panels in L2 while they sweep the columns
    constexpr uint32_t kGroup = 16;
    auto tile_coords = [&](uint32_t tile, uint32_t& tm, uint32_t& tn) {
        const uint32_t per_group = kGroup * tiles_n;
        const uint32_t g = tile / per_group, r = tile % per_group;
        const uint32_t first = g * kGroup;
        const uint32_t gsz = (tiles_m - first) < kGroup ? (tiles_m - first) : kGroup;
        tm = first + r % gsz;
        tn = r / gsz;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_b) : "memory");
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            int armed_parity[C::kStages];
#pragma unroll
            for (int s = 0; s < C::kStages; ++s) armed_parity[s] = -1;
            for (uint32_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                uint32_t tm, tn, kb_begin, kb_cnt;
                tile_coords(item % num_tiles, tm, tn);
                item_kb(item, kb_begin, kb_cnt);
                const uint32_t total_kb = kb_cnt * (uint32_t)args.passes;
                const int m0 = (int)(tm * BM), n0 = (int)(tn * BN);
                for (uint32_t vkb = 0; vkb < total_kb; ++vkb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, args.wait_budget)) { atomicCAS(args.error_flag, 0, kErrEmptyWait); ok = false; break; }
                    const uint32_t sa = smem_base + stage * C::kStageBytes, sb = sa + C::kABytes;
                    const uint32_t pass = vkb / kb_cnt;
                    const int k0 = (int)((kb_begin + vkb - pass * kb_cnt) * BK);
                    const CUtensorMap* pa = (args.passes == 3 && pass == 0) ? &tm_a_lo : &tm_a;
                    const CUtensorMap* pb = (args.passes == 3 && pass == 1) ? &tm_b_lo : &tm_b;
                    mbar_expect_tx(full_bar(stage), C::kStageBytes);
                    // An MN-major tile is BM/32 (BN/32) boxes of 32 columns x 32 k-rows.  When the row length is a
                    // multiple of 32 the matrix is also described as [column group][k][32] and one 3-D copy brings
                    // all boxes of the tile; otherwise one 2-D copy per box.
                    if (A_MN) {
                        if (args.a_grouped) {
                            tma_load_3d(sa, pa, full_bar(stage), 0, k0, m0 / 32);
                        } else {
#pragma unroll
                            for (int b = 0; b < BM / 32; ++b) tma_load_2d(sa + b * 4096, pa, full_bar(stage), m0 + 32 * b, k0);
                        }
                    } else {
                        tma_load_2d(sa, pa, full_bar(stage), k0, m0);
                    }
                    if (B_MN) {
                        if (args.b_grouped) {
                            tma_load_3d(sb, pb, full_bar(stage), 0, k0, n0 / 32);
                        } else {
#pragma unroll
                            for (int b = 0; b < BN / 32; ++b) tma_load_2d(sb + b * 4096, pb, full_bar(stage), n0 + 32 * b, k0);
                        }
                    } else {
                        tma_load_2d(sb, pb, full_bar(stage), k0, n0);
                    }
#pragma unroll
                    for (int s = 0; s < C::kStages; ++s)
                        if (s == (int)stage) armed_parity[s] = (int)phase;
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok || *abort_flag) {
                // bounded drain of this thread's own copies before the CTA retires
#pragma unroll
                for (int s = 0; s < C::kStages; ++s) {
                    if (armed_parity[s] >= 0) {
                        const long long t0 = clock64();
                        while (!mbar_try_wait(full_bar(s), (uint32_t)armed_parity[s])) {
                            if (clock64() - t0 > kWaitCycles) { atomicCAS(args.error_flag, 0, kErrDrain); break; }
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(A_MN, B_MN, BN);
            uint32_t stage = 0, phase = 0, it = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++it) {
                uint32_t kb_begin, kb_cnt;
                item_kb(item, kb_begin, kb_cnt);
                const uint32_t total_kb = kb_cnt * (uint32_t)args.passes;
                const uint32_t acc = it & 1u, acc_phase = (it >> 1) & 1u;
                if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag, args.wait_budget)) { atomicCAS(args.error_flag, 0, kErrAccEmptyWait); ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < total_kb; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, args.wait_budget)) { atomicCAS(args.error_flag, 0, kErrFullWait); ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * C::kStageBytes, sb = sa + C::kABytes;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        // K-major: 32 bytes further inside the 128-byte swizzled row, 8-row groups 1024 B apart.
                        // MN-major: eight k-rows (two 4-row swizzle atoms, 512 B apart) per MMA, so 1024 B per
                        // step; the 32-element column groups (one TMA box each) are 4096 B apart.
                        const uint64_t da = A_MN ? smem_desc(sa + kk * 1024, 4096, 512, kLayoutSw128Base32)
                                                 : smem_desc(sa + kk * 32, 16, 1024, kLayoutSw128);
                        const uint64_t db = B_MN ? smem_desc(sb + kk * 1024, 4096, 512, kLayoutSw128Base32)
                                                 : smem_desc(sb + kk * 32, 16, 1024, kLayoutSw128);
                        umma_tf32(d_tmem, da, db, idesc, (kb | (uint32_t)kk) != 0u ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));   // frees the stage once these MMAs have read it
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(acc_full_bar(acc));      // accumulator complete
            }
            if (!ok || *abort_flag) {
                umma_commit(drain_bar);
                const long long t0 = clock64();
                while (!mbar_try_wait(drain_bar, 0)) {
                    if (clock64() - t0 > kWaitCycles) { atomicCAS(args.error_flag, 0, kErrDrain); break; }
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue
        const uint32_t lane_group = (uint32_t)(warp & 3);
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++it) {
            uint32_t tm, tn;
            tile_coords(item % num_tiles, tm, tn);
            const uint32_t acc = it & 1u, acc_phase = (it >> 1) & 1u;
            if (!mbar_wait(acc_full_bar(acc), acc_phase, abort_flag, args.wait_budget)) { atomicCAS(args.error_flag, 0, kErrAccFullWait); ok = false; break; }
            tc_fence_after();
            const uint32_t row = tm * BM + lane_group * 32 + lane;
            const bool row_ok = row < args.m;
            float* crow = args.c + (size_t)(item / num_tiles) * args.m * args.n + (size_t)row * args.n;
            const float* mrow = args.mask ? args.mask + (size_t)row * args.n : nullptr;
#pragma unroll 1
            for (int ch = 0; ch < BN / 32; ++ch) {
                uint32_t r[32];
                float vals[32];
                tmem_ld32(tmem_base + ((lane_group * 32u) << 16) + acc * BN + ch * 32, r);
                tmem_ld_wait();
                store_chunk(args, r, vals, row_ok, crow, mrow, tn * BN + ch * 32);
                if (args.colsum_partial) {
                    // this warp's 32 rows of these 32 columns: one 128-byte store into the warp's row of the partial sums
                    const float t = warp_column_sums(vals, lane);
                    const uint32_t col = tn * BN + ch * 32 + lane;
                    if (col < args.n) args.colsum_partial[(size_t)(tm * (BM / 32) + lane_group) * args.n + col] = t;
                }
            }
            tc_fence_before();
            mbar_arrive(acc_empty_bar(acc));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// =====================================================================================================
// Two-CTA variant: a cluster of two CTAs on the two SMs of a TPC computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA loads its 128 rows of A and ITS HALF of the B tile (128 columns),
// so per SM the shared-memory traffic per flop drops by a third and a stage is 32 KiB instead of 48 KiB:
// six stages fit, which is what hides the TMA latency for 4-byte operands.
//   * the leader CTA (cluster rank 0) issues every MMA; the tensor cores of both SMs read A from their own
//     shared memory and B from both; each SM accumulates its 128 rows in its own tensor memory;
//   * both producers signal the LEADER's full barrier (TMA copies of the peer carry .cta_group::2 so that
//     their completion may land on the other CTA's mbarrier); the leader arms it with the bytes of both;
//   * the leader's commits arrive on the stage-empty and accumulator-full barriers of BOTH CTAs (one
//     commit per CTA, addressed through mapa);
//   * both epilogues arrive on the leader's accumulator-empty barrier (the peer's with a cluster-scope
//     remote arrive).
// No copy uses cluster multicast.  All waits are bounded exactly as in the one-CTA kernel; the two cluster
// barriers (after set-up, before exit) complete because every thread of both CTAs reaches them.
constexpr int kBN2 = 256, kStages2 = 6;   // the ring's depth; KernelArgs::stages <= 6 of them are used (5, 6 and 7 measured the same)
constexpr int kHalfBytes = BM * BK * 4;               // 16 KiB: 128 rows (or columns) x 32 k
constexpr int kStageBytes2 = 2 * kHalfBytes;          // A half-tile + B half-tile
constexpr int kSmemBytes2 = kStages2 * kStageBytes2 + 256 + 1024;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Wait whose acquire covers writes made by the other CTA of the pair (a tile index published into this CTA's shared memory).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        if ((it & 255u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 >= kWaitCycles) { *abort_flag = 1; return false; }
        }
        if (mbar_try_wait_cluster(bar, parity)) return true;
    }
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// TMA copies whose completion is signalled on an mbarrier that may live in the other CTA of the pair
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar_cluster, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma2_load_3d(uint32_t dst, const CUtensorMap* tm, uint32_t bar_cluster, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar_cluster), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy(int kind) {   // 1 evict_first, 2 evict_last
    uint64_t p;
    if (kind == 1) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    else asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma2_load_2d_hint(uint32_t dst, const CUtensorMap* tm, uint32_t bar_cluster, int x, int y, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(tm), "r"(bar_cluster), "r"(x), "r"(y), "l"(pol)
        : "memory");
}
__device__ __forceinline__ void tma2_load_3d_hint(uint32_t dst, const CUtensorMap* tm, uint32_t bar_cluster, int x, int y, int z, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(dst), "l"(tm), "r"(bar_cluster), "r"(x), "r"(y), "r"(z), "l"(pol)
        : "memory");
}
__device__ __forceinline__ void umma2_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma2_commit(uint32_t bar_cluster) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tmem2_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem2_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__host__ __device__ constexpr uint32_t make_idesc2(bool a_mn, bool b_mn) {   // M = 256 across the pair, N = 256
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(kBN2 >> 3) << 17) |
           ((uint32_t)(256 >> 4) << 24);
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_tf32_2cta_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_a_lo, const __grid_constant__ CUtensorMap tm_b_lo, KernelArgs args) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // same offset in both CTAs of the pair
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kStages2 * kStageBytes2;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages2 + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages2 + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages2 + 2 + a); };
    const uint32_t drain_bar = bar_base + 8u * (2 * kStages2 + 4);
    auto tile_full_bar = [&](int t) { return bar_base + 8u * (2 * kStages2 + 5 + t); };     // a tile index has been published (both CTAs)
    auto tile_empty_bar = [&](int t) { return bar_base + 8u * (2 * kStages2 + 7 + t); };    // ... and read by all ten readers (leader only)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + kStages2 * kStageBytes2 + 8 * (2 * kStages2 + 9));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* tile_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);               // [2]
    const bool dynamic = args.tile_counter != nullptr;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t rank = cluster_ctarank();                 // 0 = leader
    const uint32_t pair = blockIdx.x / 2, num_pairs = gridDim.x / 2;
    const uint32_t tiles_m = (args.m + 255) / 256, tiles_n = (args.n + kBN2 - 1) / kBN2;
    const uint32_t num_tiles = tiles_m * tiles_n;
    const uint32_t num_kb = (args.k + BK - 1) / BK;
    const uint32_t total_kb = num_kb * (uint32_t)args.passes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 2 * kEpiThreads); }
        mbar_init(drain_bar, 1);
        // readers of a published tile index: the leader's MMA thread and four epilogue warps, the peer's producer and four epilogue warps
        for (int t = 0; t < 2; ++t) { mbar_init(tile_full_bar(t), 1); mbar_init(tile_empty_bar(t), 10); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem2_alloc(smem_u32(tmem_slot), 512);     // both CTAs, same warp, same slot offset
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                        // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    grid_dependency_sync();   // set-up runs beside the tail of the kernel before; global memory is touched from here on

    const uint32_t kGroup = args.group;                        // row-tiles of 256 that share their B panels in L2 (8 by default)
    auto tile_coords = [&](uint32_t tile, uint32_t& tm, uint32_t& tn) {
        const uint32_t per_group = kGroup * tiles_n;
        const uint32_t g = tile / per_group, r = tile % per_group;
        const uint32_t first = g * kGroup;
        const uint32_t gsz = (tiles_m - first) < kGroup ? (tiles_m - first) : kGroup;
        tm = first + r % gsz;
        tn = r / gsz;
    };
    // Which tile iteration `it` of this pair works on; false when there is none left (or the CTA is aborting).
    // Static: a fixed stride.  Dynamic: the leader's producer thread draws an index from the global counter and publishes
    // it, through a two-slot ring guarded by the tile_full / tile_empty barriers, to the nine other readers of the pair.
    auto publish_tile = [&](uint32_t it, int& tile) -> bool {           // the leader's producer thread only
        const int sl = (int)(it & 1u);
        if (!mbar_wait(tile_empty_bar(sl), ((it >> 1) & 1u) ^ 1u, abort_flag)) { atomicCAS(args.error_flag, 0, kErrEmptyWait); return false; }
        const int t = atomicAdd(args.tile_counter, 1);
        tile = t < (int)num_tiles ? t : -1;
        tile_slot[sl] = tile;
        st_shared_cluster_u32(map_to_cta(smem_u32(const_cast<int*>(tile_slot + sl)), 1), (uint32_t)tile);
        mbar_arrive_cluster(map_to_cta(tile_full_bar(sl), 0));          // release: the two stores above are visible to whoever waits
        mbar_arrive_cluster(map_to_cta(tile_full_bar(sl), 1));
        return tile >= 0;
    };
    auto read_tile = [&](uint32_t it, int& tile) -> bool {              // one thread per reader
        const int sl = (int)(it & 1u);
        if (!mbar_wait_cluster(tile_full_bar(sl), (it >> 1) & 1u, abort_flag)) { atomicCAS(args.error_flag, 0, kErrFullWait); tile = -1; return false; }
        tile = tile_slot[sl];
        mbar_arrive_cluster(map_to_cta(tile_empty_bar(sl), 0));
        return tile >= 0;
    };
    auto static_tile = [&](uint32_t it, int& tile) -> bool {
        const uint32_t t = pair + it * num_pairs;
        tile = t < num_tiles ? (int)t : -1;
        return tile >= 0;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_b) : "memory");
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            const uint64_t pol_a = l2_policy(args.l2_hints == 1 ? 2 : 1), pol_b = l2_policy(args.l2_hints == 3 ? 2 : 1);
            int armed_parity[kStages2];
#pragma unroll
            for (int s = 0; s < kStages2; ++s) armed_parity[s] = -1;
            for (uint32_t it = 0; ok; ++it) {
                int tile;
                if (!(dynamic ? (rank == 0 ? publish_tile(it, tile) : read_tile(it, tile)) : static_tile(it, tile))) break;
                uint32_t tm, tn;
                tile_coords((uint32_t)tile, tm, tn);
                const int m0 = (int)(tm * 256 + rank * 128);          // this CTA's rows of A
                const int n0 = (int)(tn * kBN2 + rank * 128);         // this CTA's columns of B
                for (uint32_t vkb = 0; vkb < total_kb; ++vkb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { atomicCAS(args.error_flag, 0, kErrEmptyWait); ok = false; break; }
                    const uint32_t sa = smem_base + stage * kStageBytes2, sb = sa + kHalfBytes;
                    const uint32_t pass = vkb / num_kb;
                    const int k0 = (int)((vkb - pass * num_kb) * BK);
                    const CUtensorMap* pa = (args.passes == 3 && pass == 0) ? &tm_a_lo : &tm_a;
                    const CUtensorMap* pb = (args.passes == 3 && pass == 1) ? &tm_b_lo : &tm_b;
                    const uint32_t lead_full = map_to_cta(full_bar(stage), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * kStageBytes2);   // the bytes of both CTAs
                    if (args.l2_hints) {
                        if (A_MN) {
                            if (args.a_grouped) tma2_load_3d_hint(sa, pa, lead_full, 0, k0, m0 / 32, pol_a);
                            else {
#pragma unroll
                                for (int b = 0; b < 4; ++b) tma2_load_2d_hint(sa + b * 4096, pa, lead_full, m0 + 32 * b, k0, pol_a);
                            }
                        } else tma2_load_2d_hint(sa, pa, lead_full, k0, m0, pol_a);
                        if (B_MN) {
                            if (args.b_grouped) tma2_load_3d_hint(sb, pb, lead_full, 0, k0, n0 / 32, pol_b);
                            else {
#pragma unroll
                                for (int b = 0; b < 4; ++b) tma2_load_2d_hint(sb + b * 4096, pb, lead_full, n0 + 32 * b, k0, pol_b);
                            }
                        } else tma2_load_2d_hint(sb, pb, lead_full, k0, n0, pol_b);
                    } else {
                    if (A_MN) {
                        if (args.a_grouped) {
                            tma2_load_3d(sa, pa, lead_full, 0, k0, m0 / 32);
                        } else {
#pragma unroll
                            for (int b = 0; b < 4; ++b) tma2_load_2d(sa + b * 4096, pa, lead_full, m0 + 32 * b, k0);
                        }
                    } else {
                        tma2_load_2d(sa, pa, lead_full, k0, m0);
                    }
                    if (B_MN) {
                        if (args.b_grouped) {
                            tma2_load_3d(sb, pb, lead_full, 0, k0, n0 / 32);
                        } else {
#pragma unroll
                            for (int b = 0; b < 4; ++b) tma2_load_2d(sb + b * 4096, pb, lead_full, n0 + 32 * b, k0);
                        }
                    } else {
                        tma2_load_2d(sb, pb, lead_full, k0, n0);
                    }
                    }
#pragma unroll
                    for (int s = 0; s < kStages2; ++s)
                        if (s == (int)stage) armed_parity[s] = (int)phase;
                    if (++stage == args.stages) { stage = 0; phase ^= 1u; }
                }
            }
            if ((!ok || *abort_flag) && rank == 0) {
                // Bounded drain before the pair retires: the leader's full barriers count the bytes of both CTAs'
                // copies, so waiting on them here covers the peer's outstanding copies too.
#pragma unroll
                for (int s = 0; s < kStages2; ++s) {
                    if (armed_parity[s] >= 0) {
                        const long long t0 = clock64();
                        while (!mbar_try_wait(full_bar(s), (uint32_t)armed_parity[s])) {
                            if (clock64() - t0 > kWaitCycles) { atomicCAS(args.error_flag, 0, kErrDrain); break; }
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc2(A_MN, B_MN);
            uint32_t stage = 0, phase = 0, it = 0;
            bool ok = true;
            for (; ok; ++it) {
                int tile;
                if (!(dynamic ? read_tile(it, tile) : static_tile(it, tile))) break;
                const uint32_t acc = it & 1u, acc_phase = (it >> 1) & 1u;
                if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag)) { atomicCAS(args.error_flag, 0, kErrAccEmptyWait); ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBN2;
                for (uint32_t kb = 0; kb < total_kb; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) { atomicCAS(args.error_flag, 0, kErrFullWait); ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * kStageBytes2, sb = sa + kHalfBytes;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t da = A_MN ? smem_desc(sa + kk * 1024, 4096, 512, kLayoutSw128Base32)
                                                 : smem_desc(sa + kk * 32, 16, 1024, kLayoutSw128);
                        const uint64_t db = B_MN ? smem_desc(sb + kk * 1024, 4096, 512, kLayoutSw128Base32)
                                                 : smem_desc(sb + kk * 32, 16, 1024, kLayoutSw128);
                        umma2_tf32(d_tmem, da, db, idesc, (kb | (uint32_t)kk) != 0u ? 1u : 0u);
                    }
                    umma2_commit(map_to_cta(empty_bar(stage), 0));   // the stage is free in both CTAs once these MMAs have read it
                    umma2_commit(map_to_cta(empty_bar(stage), 1));
                    if (++stage == args.stages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma2_commit(map_to_cta(acc_full_bar(acc), 0));      // accumulators complete in both CTAs
                umma2_commit(map_to_cta(acc_full_bar(acc), 1));
            }
            if (!ok || *abort_flag) {
                umma2_commit(map_to_cta(drain_bar, 0));
                const long long t0 = clock64();
                while (!mbar_try_wait(drain_bar, 0)) {
                    if (clock64() - t0 > kWaitCycles) { atomicCAS(args.error_flag, 0, kErrDrain); break; }
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const uint32_t lane_group = (uint32_t)(warp & 3);
        uint32_t it = 0;
        bool ok = true;
        for (; ok; ++it) {
            int tile = -1;
            if (dynamic) {
                if (lane == 0) read_tile(it, tile);          // one reader per warp; the others get the index by shuffle
                tile = __shfl_sync(0xffffffffu, tile, 0);
            } else {
                static_tile(it, tile);
            }
            if (tile < 0) break;
            uint32_t tm, tn;
            tile_coords((uint32_t)tile, tm, tn);
            const uint32_t acc = it & 1u, acc_phase = (it >> 1) & 1u;
            if (!mbar_wait(acc_full_bar(acc), acc_phase, abort_flag)) { atomicCAS(args.error_flag, 0, kErrAccFullWait); ok = false; break; }
            tc_fence_after();
            const uint32_t row = tm * 256 + rank * 128 + lane_group * 32 + lane;
            const bool row_ok = row < args.m;
            float* crow = args.c + (size_t)row * args.n;
            const float* mrow = args.mask ? args.mask + (size_t)row * args.n : nullptr;
#pragma unroll 1
            for (int ch = 0; ch < kBN2 / 32; ++ch) {
                uint32_t r[32];
                float vals[32];
                tmem_ld32(tmem_base + ((lane_group * 32u) << 16) + acc * kBN2 + ch * 32, r);
                tmem_ld_wait();
                store_chunk(args, r, vals, row_ok, crow, mrow, tn * kBN2 + ch * 32);
                if (args.colsum_partial) {
                    const float t = warp_column_sums(vals, lane);
                    const uint32_t col = tn * kBN2 + ch * 32 + lane;
                    if (col < args.n) args.colsum_partial[(size_t)((tm * 2 + rank) * 4 + lane_group) * args.n + col] = t;
                }
            }
            tc_fence_before();
            mbar_arrive_cluster(map_to_cta(acc_empty_bar(acc), 0));   // the leader's MMA thread owns the accumulators' reuse
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other may still touch it
    if (warp == 1) {
        tc_fence_after();
        tmem2_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            cudaGetLastError();
    }
    return fn;
}

int env_int(const char* name, int dflt, int lo, int hi);
CUtensorMapL2promotion l2_promotion() {
    const int v = env_int("TS_GEMM_L2_PROMOTION", 256, 0, 256);
    return v == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE : v == 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
         : v == 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
}

// 2-D row-major f32 matrix [rows][cols]; box = box_cols (inner) x box_rows.
bool make_map(CUtensorMap* tm, const float* ptr, size_t rows, size_t cols, uint32_t box_cols, uint32_t box_rows, bool mn_major) {
    EncodeTiledFn enc = get_encode();
    if (!enc) { set_error("gemm: cuTensorMapEncodeTiled is not available from the driver"); return false; }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(float)};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                     l2_promotion(), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("gemm: cuTensorMapEncodeTiled failed with code %d (rows %zu cols %zu box %u x %u)", (int)r, rows, cols, box_cols, box_rows); return false; }
    return true;
}

// The same [rows][cols] matrix (cols a multiple of 32) seen as [cols/32 groups][rows][32]: dimension 0 is
// the 32 contiguous elements of a group, dimension 1 the row (pitch cols*4 bytes), dimension 2 the group
// (pitch 128 bytes).  A box of 32 x box_rows x box_groups lands in shared memory group by group, each
// group box_rows rows of 128 bytes: the layout of box_groups separate 2-D boxes, in one copy.
bool make_map_grouped(CUtensorMap* tm, const float* ptr, size_t rows, size_t cols, uint32_t box_rows, uint32_t box_groups) {
    EncodeTiledFn enc = get_encode();
    if (!enc) { set_error("gemm: cuTensorMapEncodeTiled is not available from the driver"); return false; }
    cuuint64_t dims[3] = {32, (cuuint64_t)rows, (cuuint64_t)(cols / 32)};
    cuuint64_t strides[2] = {(cuuint64_t)cols * sizeof(float), 128};
    cuuint32_t box[3] = {32, box_rows, box_groups};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, l2_promotion(), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("gemm: cuTensorMapEncodeTiled (grouped) failed with code %d (rows %zu cols %zu)", (int)r, rows, cols); return false; }
    return true;
}

template <int BN, bool A_MN, bool B_MN>
bool launch_tc(const GemmArgs& g, DeviceCtx* c, cudaStream_t s, uint32_t splits = 1, uint32_t kb_per_split = 0) {
    using Cf = Cfg<BN>;
    CUtensorMap tm_a, tm_b, tm_a_lo, tm_b_lo;
    // the grouped description is an optimisation: if the driver refuses it, the per-box maps still work
    bool a_grouped = A_MN && g.m % 32 == 0 && make_map_grouped(&tm_a, g.a, g.k, g.m, BK, BM / 32);
    bool b_grouped = B_MN && g.n % 32 == 0 && make_map_grouped(&tm_b, g.b, g.k, g.n, BK, BN / 32);
    // A: stored [k][m] when transposed (MN-major) else [m][k];  B: stored [k][n] when not transposed (MN-major) else [n][k]
    auto map_a = [&](CUtensorMap* tm, const float* p) {
        if (a_grouped) return make_map_grouped(tm, p, g.k, g.m, BK, BM / 32);
        return A_MN ? make_map(tm, p, g.k, g.m, 32, 32, true) : make_map(tm, p, g.m, g.k, BK, BM, false);
    };
    auto map_b = [&](CUtensorMap* tm, const float* p) {
        if (b_grouped) return make_map_grouped(tm, p, g.k, g.n, BK, BN / 32);
        return B_MN ? make_map(tm, p, g.k, g.n, 32, 32, true) : make_map(tm, p, g.n, g.k, BK, BN, false);
    };
    if (!a_grouped && !map_a(&tm_a, g.a)) return false;
    if (!b_grouped && !map_b(&tm_b, g.b)) return false;
    const bool split3 = g.a_lo && g.b_lo;
    if (split3) {
        if (!map_a(&tm_a_lo, g.a_lo) || !map_b(&tm_b_lo, g.b_lo)) return false;
    } else {
        tm_a_lo = tm_a;
        tm_b_lo = tm_b;
    }
    auto kern = gemm_tf32_kernel<BN, A_MN, B_MN>;
    static bool attr_set[64] = {false};   // the attribute is per device
    if (!attr_set[c->device]) {
        TS_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cf::kSmemBytes));
        attr_set[c->device] = true;
    }
    size_t tiles = ((g.m + BM - 1) / BM) * ((g.n + BN - 1) / BN) * splits;
    const size_t sms = (size_t)(c->sm_count - c->sm_reserved);
    int grid = (int)(tiles < sms ? tiles : sms);
    if (kb_per_split == 0) kb_per_split = (uint32_t)((g.k + BK - 1) / BK);
    KernelArgs ka{g.c, g.bias, g.mask, g.relu ? 1 : 0, g.round_tf32 ? 1 : 0, a_grouped ? 1 : 0, b_grouped ? 1 : 0, split3 ? 3 : 1,
                  (uint32_t)g.m, (uint32_t)g.n, (uint32_t)g.k, c->error_flag, splits, kb_per_split, g_wait_budget.load(), g.colsum_partial, nullptr, 0u, 0u, 0u};
    ProfScope prof(kProfGemmTc, s, 2.0 * (double)g.m * (double)g.n * (double)g.k);   // algorithmic flop, whatever the pass count
    launch_dep(kern, dim3(grid), dim3(kThreads), Cf::kSmemBytes, s, tm_a, tm_b, tm_a_lo, tm_b_lo, ka);
    return cuda_ok(cudaGetLastError(), "tcgen05 gemm launch");
}

// Tuning switches read once from the environment (defaults are the measured best).
int env_int(const char* name, int dflt, int lo, int hi) {
    static std::map<std::string, int> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    // what is cached is the variable's own value (or that it is unset or out of range): the default may differ from call
    // to call (it can depend on the device's SM count)
    constexpr int kUnset = -2147483647 - 1;
    auto it = cache.find(name);
    if (it == cache.end()) {
        int v = kUnset;
        if (const char* e = getenv(name)) v = atoi(e);
        if (v < lo || v > hi) v = kUnset;
        it = cache.emplace(name, v).first;
    }
    return it->second == kUnset ? dflt : it->second;
}

// TS_GEMM_DYNAMIC=0 (or ts_debug_set_gemm_dynamic(0)) goes back to the fixed stride, for A/B measurements and tests.
std::atomic<int> g_dynamic_tiles{-1};
bool dynamic_tiles(const DeviceCtx* c) {
    int v = g_dynamic_tiles.load();
    if (v < 0) { const char* e = getenv("TS_GEMM_DYNAMIC"); v = (e && e[0] == '0') ? 0 : 1; g_dynamic_tiles.store(v); }
    return c->tile_counter && v == 1;
}

// Two-CTA kernel: 256 x 256 tiles, each CTA of the pair loads 128 rows of A and 128 columns of B per stage.
template <bool A_MN, bool B_MN>
bool launch_tc2(const GemmArgs& g, DeviceCtx* c, cudaStream_t s) {
    CUtensorMap tm_a, tm_b, tm_a_lo, tm_b_lo;
    bool a_grouped = A_MN && g.m % 32 == 0 && make_map_grouped(&tm_a, g.a, g.k, g.m, BK, 4);
    bool b_grouped = B_MN && g.n % 32 == 0 && make_map_grouped(&tm_b, g.b, g.k, g.n, BK, 4);
    auto map_a = [&](CUtensorMap* tm, const float* p) {
        if (a_grouped) return make_map_grouped(tm, p, g.k, g.m, BK, 4);
        return A_MN ? make_map(tm, p, g.k, g.m, 32, 32, true) : make_map(tm, p, g.m, g.k, BK, 128, false);
    };
    auto map_b = [&](CUtensorMap* tm, const float* p) {
        if (b_grouped) return make_map_grouped(tm, p, g.k, g.n, BK, 4);
        return B_MN ? make_map(tm, p, g.k, g.n, 32, 32, true) : make_map(tm, p, g.n, g.k, BK, 128, false);
    };
    if (!a_grouped && !map_a(&tm_a, g.a)) return false;
    if (!b_grouped && !map_b(&tm_b, g.b)) return false;
    const bool split3 = g.a_lo && g.b_lo;
    if (split3) {
        if (!map_a(&tm_a_lo, g.a_lo) || !map_b(&tm_b_lo, g.b_lo)) return false;
    } else {
        tm_a_lo = tm_a;
        tm_b_lo = tm_b;
    }
    auto kern = gemm_tf32_2cta_kernel<A_MN, B_MN>;
    static bool attr_set[64] = {false};
    if (!attr_set[c->device]) {
        TS_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes2));
        attr_set[c->device] = true;
    }
    size_t tiles = ((g.m + 255) / 256) * ((g.n + kBN2 - 1) / kBN2);
    size_t pairs = (size_t)(c->sm_count - c->sm_reserved) / 2;
    int grid = 2 * (int)(tiles < pairs ? tiles : pairs);
    // Tiles from a counter instead of a fixed stride.  The CTA pairs then always work on the most recently drawn, i.e.
    // neighbouring, tiles, whose panels they share in L2; with a fixed stride pairs drift apart over the hundred tiles
    // each walks and the shared panels fall out of L2 (C5 step, same GPU: 79.6 -> 72.1 ms, at a higher clock under the
    // same power cap).  And a pair whose SMs a collective's CTAs hold for a while takes fewer tiles instead of
    // stretching the launch.  The one counter belongs to the compute stream's launches.
    int* counter = (dynamic_tiles(c) && s == c->compute) ? c->tile_counter : nullptr;
    if (counter) TS_CHECK(cudaMemsetAsync(counter, 0, sizeof(int), s));
    KernelArgs ka{g.c, g.bias, g.mask, g.relu ? 1 : 0, g.round_tf32 ? 1 : 0, a_grouped ? 1 : 0, b_grouped ? 1 : 0, split3 ? 3 : 1,
                  (uint32_t)g.m, (uint32_t)g.n, (uint32_t)g.k, c->error_flag, 1u, 0u, kWaitCycles, g.colsum_partial, counter,
                  (uint32_t)env_int("TS_GEMM_STAGES", 6, 2, kStages2), (uint32_t)env_int("TS_GEMM_GROUP", 8, 1, 64),
                  (uint32_t)env_int("TS_GEMM_L2_HINTS", 0, 0, 3)};
    ProfScope prof(kProfGemmTc, s, 2.0 * (double)g.m * (double)g.n * (double)g.k);
    launch_dep(kern, dim3(grid), dim3(kThreads), kSmemBytes2, s, tm_a, tm_b, tm_a_lo, tm_b_lo, ka);
    return cuda_ok(cudaGetLastError(), "tcgen05 2-CTA gemm launch");
}

bool launch_tc2_any(const GemmArgs& g, DeviceCtx* c, cudaStream_t s) {
    const bool a_mn = g.trans_a, b_mn = !g.trans_b;
    if (a_mn) return b_mn ? launch_tc2<true, true>(g, c, s) : launch_tc2<true, false>(g, c, s);
    return b_mn ? launch_tc2<false, true>(g, c, s) : launch_tc2<false, false>(g, c, s);
}

// TS_GEMM_SPLITK=0 turns the K split off (for A/B measurements).
bool split_k_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("TS_GEMM_SPLITK"); v = (e && e[0] == '0') ? 0 : 1; }
    return v == 1;
}

// TS_GEMM_2CTA=0 keeps every GEMM on the one-CTA kernel (for A/B measurements).
bool two_cta_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("TS_GEMM_2CTA"); v = (e && e[0] == '0') ? 0 : 1; }
    return v == 1;
}

template <int BN>
bool launch_tc_bn(const GemmArgs& g, DeviceCtx* c, cudaStream_t s, uint32_t splits = 1, uint32_t kb_per_split = 0) {
    const bool a_mn = g.trans_a, b_mn = !g.trans_b;
    if (a_mn) return b_mn ? launch_tc<BN, true, true>(g, c, s, splits, kb_per_split) : launch_tc<BN, true, false>(g, c, s, splits, kb_per_split);
    return b_mn ? launch_tc<BN, false, true>(g, c, s, splits, kb_per_split) : launch_tc<BN, false, false>(g, c, s, splits, kb_per_split);
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

bool gemm_tc_supported(const GemmArgs& g) {
    if (g.m == 0 || g.n == 0 || g.k == 0) return false;
    if (g.m >= (1ull << 31) || g.n >= (1ull << 31) || g.k >= (1ull << 31)) return false;
    // TMA needs 16-byte aligned bases and row pitches; the epilogue stores float4.
    const size_t a_cols = g.trans_a ? g.m : g.k, b_cols = g.trans_b ? g.k : g.n;
    if (a_cols % 4 || b_cols % 4 || g.n % 4) return false;
    if (!al16(g.a) || !al16(g.b) || !al16(g.c)) return false;
    if (g.bias && !al16(g.bias)) return false;
    if (g.mask && !al16(g.mask)) return false;
    return true;
}

// Which tensor-core kernel a supported product runs on: host arithmetic only, the one place these thresholds live
// (gemm_tc acts on it, ts_debug_gemm_route reports it).
TcRoute tc_route(const GemmArgs& g, int sm_count) {
    TcRoute r{kRouteTc128, 1, 0};
    const size_t sms = (size_t)(sm_count > 0 ? sm_count : 1);
    // Large problems: pairs of CTAs on 256 x 256 tiles, as long as every pair gets at least one tile.
    const size_t tiles_pair = ((g.m + 255) / 256) * ((g.n + 255) / 256);
    if (two_cta_enabled() && sms >= 2 && tiles_pair >= (size_t)env_int("TS_GEMM_2CTA_MIN_TILES", (int)(sms / 2), 1, 1 << 20)) {
        r.kind = kRouteTcPairs;
        return r;
    }
    const size_t tiles256 = ((g.m + BM - 1) / BM) * ((g.n + 255) / 256);
    const size_t tiles128 = ((g.m + BM - 1) / BM) * ((g.n + 127) / 128);
    const size_t num_kb = (g.k + BK - 1) / BK;
    // A result with few tiles and a long reduction (the weight gradient of a small layer over a large batch) leaves
    // most SMs idle while a few walk all of K.  Without an epilogue to apply, K is split.  FP32 mode never comes here
    // (its order is fixed).  At this size a CTA is bound by what it pulls out of L2, (rows + columns of its tile) x its
    // share of K, so of the two tile widths the one with the smaller such product is taken (1024 x 1024 over K = 4096:
    // four splits of 128 x 256 tiles move a quarter less than two splits of 128 x 128 tiles).
    if (!g.bias && !g.relu && !g.mask && !g.round_tf32 && !g.colsum_partial && !g.colsum_out && tiles128 * 2 <= sms && num_kb >= 64 &&
        split_k_enabled()) {
        auto plan = [&](size_t tiles, size_t width, size_t* splits, size_t* kbps) {
            size_t sp = sms / tiles;
            if (sp > num_kb / 32) sp = num_kb / 32;          // at least 1024 elements of K per split
            if (sp > 16) sp = 16;
            if (sp < 1) sp = 1;
            *kbps = (num_kb + sp - 1) / sp;
            *splits = (num_kb + *kbps - 1) / *kbps;          // no empty split
            return (BM + width) * *kbps;
        };
        size_t sp128 = 1, kb128 = 0, sp256 = 1, kb256 = 0;
        const size_t cost128 = plan(tiles128, 128, &sp128, &kb128);
        const size_t cost256 = g.n > 128 ? plan(tiles256, 256, &sp256, &kb256) : ~size_t(0);
        const bool wide = cost256 < cost128;
        const size_t splits = wide ? sp256 : sp128;
        if (splits >= 2) {
            r.kind = wide ? kRouteTcSplitK256 : kRouteTcSplitK128;
            r.splits = splits;
            r.kb_per_split = wide ? kb256 : kb128;
            return r;
        }
    }
    // 128 x 128 tiles while those fit in one wave (twice as many CTAs at work as 128 x 256 tiles would give); beyond
    // that one wave of 128 x 256 tiles beats two of the narrow ones, because each CTA then pulls a third less through L2
    // per flop (4096 x 1024 x 1024: 20.5 against 28.6 us).  TS_GEMM_BN256_MIN_TILES moves the switch-over.
    if (g.n > 128 && tiles256 >= (size_t)env_int("TS_GEMM_BN256_MIN_TILES", (int)(sms / 2 + 1), 1, 1 << 20)) r.kind = kRouteTc256;
    return r;
}

// FP32-kernel split of a long reduction in the modes without a fixed summation order (0: none)
static size_t fp32_splits(const GemmArgs& g, int precision, int sm_count) {
    if (!(precision >= 1 && g.trans_a && !g.trans_b && !g.bias && !g.relu && !g.mask && g.batch == 1 && g.k >= 2048 && split_k_enabled())) return 0;
    const size_t tiles32 = ((g.m + 31) / 32) * ((g.n + 31) / 32);
    size_t splits = 0;
    for (size_t cand = 32; cand >= 2; cand /= 2)
        if (g.k % cand == 0 && g.k / cand >= 128 && tiles32 * cand <= (size_t)sm_count * 8) { splits = cand; break; }
    return (splits >= 2 && tiles32 <= (size_t)sm_count) ? splits : 0;
}

GemmRoute gemm_route(const GemmArgs& g, int precision, int sm_count) {
    if (precision < 0) precision = matmul_precision();
    if (precision >= 1) {
        const int thin = gemm_thin_kind(g);
        if (thin) return GemmRoute{thin == 1 ? kRouteThinNN : thin == 2 ? kRouteThinTN : kRouteThinNT, 1, 0};
        if (gemm_tc_supported(g)) {
            const TcRoute t = tc_route(g, sm_count);
            return GemmRoute{t.kind, t.splits, t.kb_per_split};
        }
    }
    GemmArgs h = g;
    h.colsum_out = nullptr;   // the FP32 kernels make the column sums in a pass of their own
    const size_t sp = fp32_splits(h, precision, sm_count);
    return sp ? GemmRoute{kRouteFp32SplitK, sp, 0} : GemmRoute{kRouteFp32, 1, 0};
}

bool gemm_tc(const GemmArgs& g, bool split3, DeviceCtx* c, cudaStream_t s) {
    if (!gemm_tc_supported(g)) { set_error("gemm: shape or alignment not supported by the tensor-core kernel"); return false; }
    if (split3 && !(g.a_lo && g.b_lo)) {
        // The caller passed plain FP32 operands: split them into TF32-exact high and low parts in scratch memory.
        const size_t na = g.m * g.k, nb = g.k * g.n;
        float* buf = c->alloc.alloc(2 * (na + nb) * sizeof(float) + 4 * 256);
        if (!buf) return false;
        auto up = [](size_t x) { return (x + 63) & ~size_t(63); };   // keep every part 256-byte aligned
        float *a_hi = buf, *a_lo = a_hi + up(na), *b_hi = a_lo + up(na), *b_lo = b_hi + up(nb);
        GemmArgs h = g;
        h.a = a_hi; h.a_lo = a_lo; h.b = b_hi; h.b_lo = b_lo;
        bool ok = split_tf32(g.a, a_hi, a_lo, na, s) && split_tf32(g.b, b_hi, b_lo, nb, s) && gemm_tc(h, true, c, s);
        if (s != c->compute) cudaStreamSynchronize(s);   // the block is recycled in compute-stream order only
        c->alloc.free(buf);
        return ok;
    }
    if (!split3 && (g.a_lo || g.b_lo)) { set_error("gemm: low parts given without the 3xTF32 mode"); return false; }
    const TcRoute route = tc_route(g, c->sm_count);
    const bool pairs = route.kind == kRouteTcPairs;
    if (g.colsum_out && !g.colsum_partial) {
        // Column sums of the result from the epilogue: one partial row per 32 result rows of every tile the chosen
        // kernel walks (rows past m contribute zeros), in scratch, then one small launch that adds them in order.
        const size_t prow = pairs ? ((g.m + 255) / 256) * 8 : ((g.m + BM - 1) / BM) * 4;
        float* part = c->alloc.alloc(prow * g.n * sizeof(float));
        if (!part) return false;
        GemmArgs h = g;
        h.colsum_partial = part;
        bool ok = gemm_tc(h, split3, c, s) && colsum_finish(part, g.colsum_out, g.n, prow, s);
        if (s != c->compute) cudaStreamSynchronize(s);
        c->alloc.free(part);
        return ok;
    }
    if (pairs) return launch_tc2_any(g, c, s);
    if (route.kind == kRouteTcSplitK128 || route.kind == kRouteTcSplitK256) {
        // every (tile, split) pair is a work item of the same launch, the partial products land side by side in scratch
        // and a second kernel adds them in split order, so the result does not depend on scheduling
        const size_t mn = g.m * g.n;
        float* part = c->alloc.alloc(route.splits * mn * sizeof(float));
        if (!part) return false;
        GemmArgs h = g;
        h.c = part;
        bool ok = (route.kind == kRouteTcSplitK256 ? launch_tc_bn<256>(h, c, s, (uint32_t)route.splits, (uint32_t)route.kb_per_split)
                                                   : launch_tc_bn<128>(h, c, s, (uint32_t)route.splits, (uint32_t)route.kb_per_split)) &&
                  sum_slabs(part, g.c, mn, route.splits, s);
        if (s != c->compute) cudaStreamSynchronize(s);   // the block is recycled in compute-stream order only
        c->alloc.free(part);
        return ok;
    }
    return route.kind == kRouteTc256 ? launch_tc_bn<256>(g, c, s) : launch_tc_bn<128>(g, c, s);
}

bool gemm(const GemmArgs& g, int precision, DeviceCtx* c, cudaStream_t s) {
    if (precision < 0) precision = matmul_precision();
    if (precision >= 1 && c && gemm_thin_supported(g)) return gemm_thin(g, c, s);
    if (precision >= 1 && gemm_tc_supported(g)) return gemm_tc(g, precision == 2, c, s);
    if (g.colsum_out) {   // the FP32 kernels have no such epilogue: the product first, then the ordinary column sum
        GemmArgs h = g;
        h.colsum_out = nullptr;
        if (!gemm(h, precision, c, s)) return false;
        float* scratch = c->alloc.alloc(colsum_scratch_elems(g.m, g.n) * sizeof(float));
        if (!scratch) return false;
        bool ok = colsum(g.c, g.colsum_out, g.m, g.n, scratch, s);
        if (s != c->compute) cudaStreamSynchronize(s);
        c->alloc.free(scratch);
        return ok;
    }
    // A shape the tensor-core kernel cannot take, in a mode that promises no summation order: when the result is small
    // and K long (a [1024 x 10] weight gradient over K = 4096 with the thin kernels switched off: 32 CTAs each walking
    // the whole chain), K is split into equal parts that run as one batched launch of the FP32 kernel and are then added
    // in split order.  This works on offsets alone when both operands are stored K-outermost (op(A) = A^T, op(B) = B:
    // the weight-gradient layout).
    if (const size_t splits = c ? fp32_splits(g, precision, c->sm_count) : 0) {
        const size_t mn = g.m * g.n, ks = g.k / splits;
        float* part = c->alloc.alloc(splits * mn * sizeof(float));
        if (!part) return false;
        GemmArgs h = g;
        h.c = part; h.k = ks; h.batch = splits; h.batch_stride_a = ks * g.m; h.batch_stride_b = ks * g.n;
        bool ok = sgemm(h, s) && sum_slabs(part, g.c, mn, splits, s);
        if (s != c->compute) cudaStreamSynchronize(s);
        c->alloc.free(part);
        return ok;
    }
    return sgemm(g, s);
}

}  // namespace k
}  // namespace ts

// ====================================================================== C ABI
using namespace ts;

TS_API bool launch_gemm_kernel(const float* a, const float* b, float* cc, unsigned long long m, unsigned long long n,
                               unsigned long long kk, int trans_a, int trans_b, const float* bias, int relu, const float* mask,
                               int precision, void* stream) {
    cudaStream_t s = pick_stream(stream);
    DeviceCtx* c = ctx();
    if (!s || !c) return false;
    if (precision < -1 || precision > 2) { set_error("launch_gemm_kernel: precision %d out of range", precision); return false; }
    if (m && n && (!cc || (kk && (!a || !b)))) { set_error("launch_gemm_kernel: null pointer"); return false; }
    k::GemmArgs g{a, b, cc, (size_t)m, (size_t)n, (size_t)kk, trans_a != 0, trans_b != 0, bias, relu != 0, mask};
    return k::gemm(g, precision, c, s);
}

TS_API bool launch_gemm_colsum_kernel(const float* a, const float* b, float* cc, unsigned long long m, unsigned long long n,
                                      unsigned long long kk, int trans_a, int trans_b, const float* bias, int relu, const float* mask,
                                      int precision, float* colsum_out, void* stream) {
    cudaStream_t s = pick_stream(stream);
    DeviceCtx* c = ctx();
    if (!s || !c) return false;
    if (precision < -1 || precision > 2) { set_error("launch_gemm_colsum_kernel: precision %d out of range", precision); return false; }
    if (m && n && (!cc || !colsum_out || (kk && (!a || !b)))) { set_error("launch_gemm_colsum_kernel: null pointer"); return false; }
    k::GemmArgs g{a, b, cc, (size_t)m, (size_t)n, (size_t)kk, trans_a != 0, trans_b != 0, bias, relu != 0, mask};
    g.colsum_out = colsum_out;
    return k::gemm(g, precision, c, s);
}

TS_API int ts_debug_gemm_route(unsigned long long m, unsigned long long n, unsigned long long kk, int trans_a, int trans_b, int precision,
                               int epilogue, int sm_count, unsigned long long* splits) {
    // stand-in operand addresses: only their alignment is looked at
    float* const aligned = reinterpret_cast<float*>(uintptr_t(1) << 20);
    k::GemmArgs g{aligned, aligned, aligned, (size_t)m, (size_t)n, (size_t)kk, trans_a != 0, trans_b != 0,
                  (epilogue & 1) ? aligned : nullptr, (epilogue & 2) != 0, (epilogue & 4) ? aligned : nullptr};
    g.round_tf32 = (epilogue & 8) != 0;
    g.colsum_out = (epilogue & 16) ? aligned : nullptr;
    const k::GemmRoute r = k::gemm_route(g, precision, sm_count);
    if (splits) *splits = r.splits;
    return r.kind;
}

TS_API void ts_debug_set_gemm_dynamic(int enabled) { k::g_dynamic_tiles.store(enabled < 0 ? -1 : (enabled ? 1 : 0)); }

TS_API void ts_debug_set_gemm_wait_budget(long long cycles) {
    k::g_wait_budget.store(cycles < 0 ? k::kWaitCycles : cycles);
}

TS_API bool launch_matmul_kernel(const float* a, const float* b, float* result, unsigned long long m, unsigned long long n,
                                 unsigned long long kk, void* stream) {
    if (!a || !b || !result) { set_error("launch_matmul_kernel: null pointer"); return false; }   // cuda_wrapper.cpp:82
    return launch_gemm_kernel(a, b, result, m, n, kk, 0, 0, nullptr, 0, nullptr, -1, stream);
}
