// Fused multi-tensor Adam: one launch updates every parameter tensor of the optimizer.
// HBM-bound: 28 bytes per parameter (read p, g, m, v; write p, m, v), 32 when the TF32-rounded copy of the
// parameter that the tensor-core GEMMs read is written in the same pass.
//
// Arithmetic follows optimizers/adam/mod.rs operation by operation, each step rounded
// separately (no FMA contraction), so that with identical gradients the updated
// parameters and moments are bit-identical to the reference's:
//   m = (beta1*m) + ((1-beta1)*g)                                        :685-687
//   v = (beta2*v) + ((1-beta2)*(g*g))        elements below size/8*8     :761-765
//   v = (beta2*v) + (((1-beta2)*g)*g)        the size%8 tail elements    :770-772
//   p = p - ((lr*(m*f1)) / (sqrt(v*f2) + eps))                           :791-840, :984-1006
// with g replaced by g + wd*p first when weight decay is on (:567-620).
#include <cstring>

#include "../../include/train_station_b200.h"
#include "common.h"

namespace ts {
namespace k {

namespace {

constexpr int kThreads = 256;
constexpr unsigned long long kChunk = 16384;   // elements per CTA: 256 threads x 4 floats x 16 trips

struct ChunkEntry {
    int tensor;
    int pad;
    unsigned long long offset;   // first element of the chunk inside the tensor
};

struct Scalars { float lr, beta1, beta2, eps, wd, f1, f2, grad_scale, c1, c2; };

// AMS: v_hat_max = max(v_hat_max, v_hat) on the bias-corrected second moment (`if a > b { a } else { b }`,
// adam/mod.rs:534-541, :846-900), and the update divides by sqrt(v_hat_max) + eps.
template <bool AMS>
__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, float& vmx, bool body, const Scalars& sc) {
    if (sc.grad_scale != 1.0f) g = __fmul_rn(g, sc.grad_scale);
    if (sc.wd > 0.0f) g = __fadd_rn(g, __fmul_rn(sc.wd, p));
    m = __fadd_rn(__fmul_rn(sc.beta1, m), __fmul_rn(sc.c1, g));
    float gg = body ? __fmul_rn(sc.c2, __fmul_rn(g, g)) : __fmul_rn(__fmul_rn(sc.c2, g), g);
    v = __fadd_rn(__fmul_rn(sc.beta2, v), gg);
    float mh = __fmul_rn(m, sc.f1), vh = __fmul_rn(v, sc.f2);
    if (AMS) { vmx = vmx > vh ? vmx : vh; vh = vmx; }
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(sc.lr, mh), __fadd_rn(__fsqrt_rn(vh), sc.eps)));
}

__device__ __forceinline__ float rn_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// The tensor table travels in the kernel's parameters: the pointers are captured when the launch is
// enqueued, so a host that runs steps ahead of the GPU cannot overwrite a table that a queued launch
// has yet to read (a table staged in reused pinned memory did exactly that).
constexpr int kMaxTensorsPerLaunch = 40;   // 40 records of 56 bytes: inside the 4 KiB of kernel parameters with room to spare
struct AdamTable { AdamTensor t[kMaxTensorsPerLaunch]; };

template <bool AMS>
__global__ void __launch_bounds__(kThreads) adam_kernel(const __grid_constant__ AdamTable tab, const ChunkEntry* __restrict__ chunks,
                                                        int chunk_base, int tensor_base, int split_log2, Scalars sc) {
    grid_dependency_sync();
    // 2^split_log2 CTAs share a chunk (each a 1024-element-aligned slice of it): small parameter sets, which would
    // otherwise run as a handful of CTAs making sixteen dependent trips each, spread over the SMs instead
    const ChunkEntry ce = chunks[chunk_base + (blockIdx.x >> split_log2)];
    const AdamTensor t = tab.t[ce.tensor - tensor_base];
    const unsigned long long body = t.n / 8 * 8;
    const unsigned long long slice = kChunk >> split_log2;
    const unsigned long long start = ce.offset + (blockIdx.x & ((1u << split_log2) - 1)) * slice;
    if (start >= t.n) return;
    unsigned long long end = start + slice;
    if (end > t.n) end = t.n;
    uintptr_t bits = reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.g) | reinterpret_cast<uintptr_t>(t.m) |
                     reinterpret_cast<uintptr_t>(t.v);
    if (AMS) bits |= reinterpret_cast<uintptr_t>(t.vmax);
    bits |= reinterpret_cast<uintptr_t>(t.tf32_out);
    const bool vec = (bits & 15) == 0;
    float unused = 0.0f;
    if (vec) {
        // start is a multiple of 1024, hence of 4
        const unsigned long long v0 = start / 4, v1 = end / 4;
        float4* pp = reinterpret_cast<float4*>(t.p);
        const float4* gp = reinterpret_cast<const float4*>(t.g);
        float4* mp = reinterpret_cast<float4*>(t.m);
        float4* vp = reinterpret_cast<float4*>(t.v);
        float4* xp = reinterpret_cast<float4*>(t.vmax);
        for (unsigned long long i = v0 + threadIdx.x; i < v1; i += 2 * kThreads) {
            // two float4 per array in flight
            unsigned long long j = i + kThreads;
            bool has2 = j < v1;
            float4 p0 = pp[i], g0 = __ldcs(gp + i), m0 = mp[i], w0 = vp[i];
            float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
            if (AMS) x0 = xp[i];
            float4 p1, g1, m1, w1;
            if (has2) { p1 = pp[j]; g1 = __ldcs(gp + j); m1 = mp[j]; w1 = vp[j]; if (AMS) x1 = xp[j]; }
            unsigned long long e = i * 4;
            adam_one<AMS>(p0.x, g0.x, m0.x, w0.x, x0.x, e < body, sc);
            adam_one<AMS>(p0.y, g0.y, m0.y, w0.y, x0.y, e + 1 < body, sc);
            adam_one<AMS>(p0.z, g0.z, m0.z, w0.z, x0.z, e + 2 < body, sc);
            adam_one<AMS>(p0.w, g0.w, m0.w, w0.w, x0.w, e + 3 < body, sc);
            pp[i] = p0; mp[i] = m0; vp[i] = w0;
            if (AMS) xp[i] = x0;
            if (t.tf32_out) reinterpret_cast<float4*>(t.tf32_out)[i] = make_float4(rn_tf32(p0.x), rn_tf32(p0.y), rn_tf32(p0.z), rn_tf32(p0.w));
            if (has2) {
                e = j * 4;
                adam_one<AMS>(p1.x, g1.x, m1.x, w1.x, x1.x, e < body, sc);
                adam_one<AMS>(p1.y, g1.y, m1.y, w1.y, x1.y, e + 1 < body, sc);
                adam_one<AMS>(p1.z, g1.z, m1.z, w1.z, x1.z, e + 2 < body, sc);
                adam_one<AMS>(p1.w, g1.w, m1.w, w1.w, x1.w, e + 3 < body, sc);
                pp[j] = p1; mp[j] = m1; vp[j] = w1;
                if (AMS) xp[j] = x1;
                if (t.tf32_out) reinterpret_cast<float4*>(t.tf32_out)[j] = make_float4(rn_tf32(p1.x), rn_tf32(p1.y), rn_tf32(p1.z), rn_tf32(p1.w));
            }
        }
        for (unsigned long long i = v1 * 4 + threadIdx.x; i < end; i += kThreads) {
            float p = t.p[i], m = t.m[i], v = t.v[i], x = AMS ? t.vmax[i] : unused;
            adam_one<AMS>(p, t.g[i], m, v, x, i < body, sc);
            t.p[i] = p; t.m[i] = m; t.v[i] = v;
            if (AMS) t.vmax[i] = x;
            if (t.tf32_out) t.tf32_out[i] = rn_tf32(p);
        }
    } else {
        for (unsigned long long i = start + threadIdx.x; i < end; i += kThreads) {
            float p = t.p[i], m = t.m[i], v = t.v[i], x = AMS ? t.vmax[i] : unused;
            adam_one<AMS>(p, t.g[i], m, v, x, i < body, sc);
            t.p[i] = p; t.m[i] = m; t.v[i] = v;
            if (AMS) t.vmax[i] = x;
            if (t.tf32_out) t.tf32_out[i] = rn_tf32(p);
        }
    }
}

}  // namespace

// The chunk map depends only on the tensor sizes, so callers build and upload it once per
// parameter set; the tensor table (pointers) is refreshed every step.
int adam_chunk_count(const unsigned long long* sizes, int n) {
    size_t c = 0;
    for (int i = 0; i < n; ++i) c += (size_t)((sizes[i] + kChunk - 1) / kChunk);
    return (int)c;
}
size_t adam_chunk_bytes(int n_chunks) { return (size_t)n_chunks * sizeof(ChunkEntry); }
void adam_build_chunks(const unsigned long long* sizes, int n, void* host_out) {
    ChunkEntry* ce = (ChunkEntry*)host_out;
    int c = 0;
    for (int i = 0; i < n; ++i)
        for (unsigned long long off = 0; off < sizes[i]; off += kChunk) ce[c++] = ChunkEntry{i, 0, off};
}

// tensors: HOST array of n records; chunks_dev: device chunk map built by adam_build_chunks for the same sizes.
// One launch per 48 tensors (a single launch for any MLP of the path).
bool adam_launch(const AdamTensor* tensors, int n, const void* chunks_dev, float lr, float beta1, float beta2, float eps, float wd,
                 float f1, float f2, float grad_scale, cudaStream_t s) {
    return adam_launch_range(tensors, 0, n, chunks_dev, lr, beta1, beta2, eps, wd, f1, f2, grad_scale, s);
}

// Updates tensors [first, last) of the table only; chunks_dev is still the map of the WHOLE table, so the range's
// chunks start after those of the tensors before it.
bool adam_launch_range(const AdamTensor* tensors, int first, int last, const void* chunks_dev, float lr, float beta1, float beta2,
                       float eps, float wd, float f1, float f2, float grad_scale, cudaStream_t s) {
    Scalars sc{lr, beta1, beta2, eps, wd, f1, f2, grad_scale, 1.0f - beta1, 1.0f - beta2};
    int chunk_base = 0;
    for (int i = 0; i < first; ++i) chunk_base += (int)((tensors[i].n + kChunk - 1) / kChunk);
    const int n = last;
    for (int t0 = first; t0 < n; t0 += kMaxTensorsPerLaunch) {
        const int cnt = n - t0 < kMaxTensorsPerLaunch ? n - t0 : kMaxTensorsPerLaunch;
        AdamTable tab;
        memset(&tab, 0, sizeof(tab));
        int n_chunks = 0;
        double elems = 0, tf32_elems = 0;
        for (int i = 0; i < cnt; ++i) {
            tab.t[i] = tensors[t0 + i];
            n_chunks += (int)((tensors[t0 + i].n + kChunk - 1) / kChunk);
            elems += (double)tensors[t0 + i].n;
            if (tensors[t0 + i].tf32_out) tf32_elems += (double)tensors[t0 + i].n;
        }
        if (n_chunks > 0) {
            // every tensor of one optimizer has a running maximum, or none has
            const bool ams = tab.t[0].vmax != nullptr;
            ProfScope prof(kProfAdam, s, (ams ? 36.0 : 28.0) * elems + 4.0 * tf32_elems);
            DeviceCtx* c = ctx();
            const int want = 2 * (c ? c->sm_count : 148);
            int split_log2 = 0;
            while (split_log2 < 4 && (n_chunks << split_log2) < want) ++split_log2;
            const int grid = n_chunks << split_log2;
            if (ams) launch_dep(adam_kernel<true>, dim3(grid), dim3(kThreads), 0, s, tab, (const ChunkEntry*)chunks_dev, chunk_base, t0, split_log2, sc);
            else launch_dep(adam_kernel<false>, dim3(grid), dim3(kThreads), 0, s, tab, (const ChunkEntry*)chunks_dev, chunk_base, t0, split_log2, sc);
            if (!cuda_ok(cudaGetLastError(), "adam launch")) return false;
        }
        chunk_base += n_chunks;
    }
    return true;
}

}  // namespace k
}  // namespace ts

// ====================================================================== C ABI
using namespace ts;

// vmax == nullptr: plain Adam; otherwise a table of running maxima (AMSGrad)
static bool adam_tables_launch(float* const* params, const float* const* grads, float* const* m, float* const* v, float* const* vmax,
                               const unsigned long long* sizes, int n_tensors, float lr, float beta1, float beta2, float eps,
                               float weight_decay, float f1, float f2, float grad_scale, void* stream) {
    cudaStream_t s = pick_stream(stream);
    DeviceCtx* c = ctx();
    if (!s || !c) return false;
    if (n_tensors <= 0) return true;
    if (!params || !grads || !m || !v || !sizes) { set_error("launch_adam_multi_tensor_kernel: null table"); return false; }
    std::vector<k::AdamTensor> t((size_t)n_tensors);
    for (int i = 0; i < n_tensors; ++i) {
        if (sizes[i] && (!params[i] || !grads[i] || !m[i] || !v[i] || (vmax && !vmax[i]))) {
            set_error("launch_adam_multi_tensor_kernel: null tensor pointer at index %d", i);
            return false;
        }
        t[i] = k::AdamTensor{params[i], grads[i], m[i], v[i], sizes[i], vmax ? vmax[i] : nullptr};
    }
    std::vector<unsigned long long> sz(sizes, sizes + n_tensors);
    int n_chunks = k::adam_chunk_count(sz.data(), n_tensors);
    if (n_chunks == 0) return true;
    size_t bytes = k::adam_chunk_bytes(n_chunks);
    std::vector<char> host(bytes);
    k::adam_build_chunks(sz.data(), n_tensors, host.data());
    float* dev = c->alloc.alloc(bytes);
    if (!dev) return false;
    // the pageable source is staged before cudaMemcpyAsync returns, so `host` may go out of scope
    bool ok = cuda_ok(cudaMemcpyAsync(dev, host.data(), bytes, cudaMemcpyHostToDevice, s), "adam chunk map upload");
    ok = ok && k::adam_launch(t.data(), n_tensors, dev, lr, beta1, beta2, eps, weight_decay, f1, f2, grad_scale, s);
    // Freed blocks are only reused by later work, which is ordered after this kernel when it runs on
    // the compute stream; a caller-supplied stream is drained first.
    if (s != c->compute) cudaStreamSynchronize(s);
    c->alloc.free(dev);
    return ok;
}

TS_API bool launch_adam_multi_tensor_kernel(float* const* params, const float* const* grads, float* const* m, float* const* v,
                                            const unsigned long long* sizes, int n_tensors, float lr, float beta1, float beta2,
                                            float eps, float weight_decay, float f1, float f2, float grad_scale, void* stream) {
    return adam_tables_launch(params, grads, m, v, nullptr, sizes, n_tensors, lr, beta1, beta2, eps, weight_decay, f1, f2, grad_scale, stream);
}

TS_API bool launch_adam_amsgrad_multi_tensor_kernel(float* const* params, const float* const* grads, float* const* m, float* const* v,
                                                    float* const* v_hat_max, const unsigned long long* sizes, int n_tensors, float lr,
                                                    float beta1, float beta2, float eps, float weight_decay, float f1, float f2,
                                                    float grad_scale, void* stream) {
    if (n_tensors > 0 && !v_hat_max) { set_error("launch_adam_amsgrad_multi_tensor_kernel: null table"); return false; }
    return adam_tables_launch(params, grads, m, v, v_hat_max, sizes, n_tensors, lr, beta1, beta2, eps, weight_decay, f1, f2, grad_scale, stream);
}
