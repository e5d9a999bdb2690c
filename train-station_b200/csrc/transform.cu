// Layout changes on contiguous tensors: permute (transpose is a permute of two axes).
// HBM-bound: 8 bytes per element (read once, write once).
//
// The reference's transpose / permute return strided views of the same allocation
// (tensor/transform/transpose.rs:156-200, permute.rs:147-190) and `contiguous()` materialises them
// (contiguous.rs:123-160); tensors here are always contiguous, so the permuted copy is produced at once.
// The values and the shape a caller reads are the same.
//
// Axes that stay adjacent and in order are merged first.  What is left is, in almost every use, a batched
// 2-D transpose [B, R, C] -> [B, C, R]: 64 x 64 tiles through padded shared memory (sixteen loads in flight per
// thread), 128-byte coalesced on both sides.  Anything else (rank up to 8) gathers: consecutive threads write consecutive output elements and read
// through the permuted strides.
#include "../../include/train_station_b200.h"
#include "common.h"

namespace ts {
namespace k {

namespace {

constexpr int kMaxRank = 8;
constexpr int kTile = 64;

__global__ void __launch_bounds__(256) transpose_tiles_kernel(const float* __restrict__ in, float* __restrict__ out, size_t rows, size_t cols,
                                                              size_t tiles_r, size_t tiles_c, size_t n_tiles) {
    grid_dependency_sync();
    __shared__ float tile[kTile][kTile + 1];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8 threads, sixteen elements each
    for (size_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const size_t b = t / (tiles_r * tiles_c), rem = t - b * tiles_r * tiles_c;
        const size_t tr = rem / tiles_c, tc = rem - tr * tiles_c;
        const float* src = in + b * rows * cols;
        float* dst = out + b * rows * cols;
        float v[kTile / 8][2];
#pragma unroll
        for (int k = 0; k < kTile / 8; ++k)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const size_t r = tr * kTile + ty + 8 * k, c = tc * kTile + tx + 32 * h;
                v[k][h] = (r < rows && c < cols) ? __ldcs(src + r * cols + c) : 0.0f;
            }
#pragma unroll
        for (int k = 0; k < kTile / 8; ++k) { tile[ty + 8 * k][tx] = v[k][0]; tile[ty + 8 * k][tx + 32] = v[k][1]; }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kTile / 8; ++k)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const size_t c = tc * kTile + ty + 8 * k, r = tr * kTile + tx + 32 * h;   // output is [cols][rows]
                if (r < rows && c < cols) __stcs(dst + c * rows + r, tile[tx + 32 * h][ty + 8 * k]);
            }
        __syncthreads();
    }
}

struct GatherPlan {
    int rank;
    unsigned long long out_dims[kMaxRank];
    unsigned long long in_strides[kMaxRank];   // stride in the input of the axis that output axis i walks
};

__global__ void __launch_bounds__(256) permute_gather_kernel(const float* __restrict__ in, float* __restrict__ out, size_t n, GatherPlan p) {
    grid_dependency_sync();
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        size_t rem = i, off = 0;
#pragma unroll
        for (int d = kMaxRank - 1; d >= 0; --d) {
            if (d < p.rank) {
                const size_t q = rem / p.out_dims[d];
                off += (rem - q * p.out_dims[d]) * p.in_strides[d];
                rem = q;
            }
        }
        out[i] = in[off];
    }
}

}  // namespace

// out = in permuted: output axis i is input axis perm[i].  dims are the INPUT dimensions.
bool permute(const float* in, float* out, const size_t* dims, const int* perm, int rank, cudaStream_t s) {
    if (rank < 1 || rank > kMaxRank) { set_error("permute: rank %d not supported (1..%d)", rank, kMaxRank); return false; }
    size_t n = 1;
    for (int i = 0; i < rank; ++i) n *= dims[i];
    if (n == 0) return true;
    if (!in || !out) { set_error("permute: null pointer"); return false; }
    DeviceCtx* c = ctx();
    if (!c) return false;
    // input strides, then merge output axes that are adjacent and in order in the input; axes of extent 1 vanish
    size_t in_stride[kMaxRank];
    size_t acc = 1;
    for (int i = rank - 1; i >= 0; --i) { in_stride[i] = acc; acc *= dims[i]; }
    size_t od[kMaxRank], os[kMaxRank];
    int r = 0;
    for (int i = 0; i < rank; ++i) {
        const int a = perm[i];
        if (dims[a] == 1) continue;
        if (r > 0 && os[r - 1] == dims[a] * in_stride[a]) {   // one step of the previous axis spans this whole axis: one longer axis
            od[r - 1] *= dims[a];
            os[r - 1] = in_stride[a];
            continue;
        }
        od[r] = dims[a]; os[r] = in_stride[a];
        ++r;
    }
    ProfScope prof(kProfElementwise, s, 8.0 * (double)n);
    if (r <= 1) {   // the data does not move
        return cuda_ok(cudaMemcpyAsync(out, in, n * sizeof(float), cudaMemcpyDeviceToDevice, s), "permute copy");
    }
    const bool swap_last_two = (r == 2 && os[0] == 1 && os[1] == od[0]) ||
                               (r == 3 && os[2] == od[1] && os[1] == 1 && os[0] == od[1] * od[2]);
    if (swap_last_two) {
        const size_t batch = r == 3 ? od[0] : 1;
        const size_t out_rows = od[r - 2], out_cols = od[r - 1];   // output [out_rows][out_cols] = input [out_cols][out_rows]
        const size_t rows = out_cols, cols = out_rows;             // input matrix is [rows][cols]
        const size_t tiles_r = (rows + kTile - 1) / kTile, tiles_c = (cols + kTile - 1) / kTile, n_tiles = batch * tiles_r * tiles_c;
        const size_t cap = (size_t)c->sm_count * 16;
        launch_dep(transpose_tiles_kernel, dim3((unsigned)(n_tiles < cap ? n_tiles : cap)), dim3(256), 0, s, in, out, rows, cols, tiles_r, tiles_c, n_tiles);
        return cuda_ok(cudaGetLastError(), "transpose launch");
    }
    GatherPlan p;
    p.rank = r;
    for (int i = 0; i < kMaxRank; ++i) { p.out_dims[i] = i < r ? od[i] : 1; p.in_strides[i] = i < r ? os[i] : 0; }
    const size_t want = (n + 255) / 256, cap = (size_t)c->sm_count * 16;
    launch_dep(permute_gather_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), 0, s, in, out, n, p);
    return cuda_ok(cudaGetLastError(), "permute launch");
}

}  // namespace k
}  // namespace ts

// ====================================================================== C ABI
using namespace ts;

TS_API bool launch_permute_kernel(const float* in, float* out, const unsigned long long* dims, const int* perm, int rank, void* stream) {
    cudaStream_t s = pick_stream(stream);
    if (!s) return false;
    if (rank < 1 || rank > 8 || !dims || !perm) { set_error("launch_permute_kernel: rank must be 1..8 and the tables non-null"); return false; }
    size_t d[8];
    bool seen[8] = {false, false, false, false, false, false, false, false};
    for (int i = 0; i < rank; ++i) {
        d[i] = (size_t)dims[i];
        if (perm[i] < 0 || perm[i] >= rank || seen[perm[i]]) { set_error("launch_permute_kernel: perm is not a permutation of 0..%d", rank - 1); return false; }
        seen[perm[i]] = true;
    }
    return k::permute(in, out, d, perm, rank, s);
}
