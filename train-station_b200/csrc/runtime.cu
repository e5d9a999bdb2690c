// Device runtime: error state, per-device context, caching allocator, and the
// reference's fifteen FFI symbols (src/cuda/cuda_wrapper.h:10-31) implemented on a GPU.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/train_station_b200.h"
#include "common.h"

namespace ts {

// ------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
const char* last_error() { return g_err; }

bool cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return true;
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return false;
}

// ------------------------------------------------------------------ allocator
size_t Allocator::round_size(size_t bytes) {
    if (bytes == 0) bytes = 1;
    if (bytes <= (1u << 20)) return (bytes + 511) & ~size_t(511);          // 512 B granules up to 1 MiB
    return (bytes + ((2u << 20) - 1)) & ~size_t((2u << 20) - 1);            // 2 MiB granules above
}

float* Allocator::alloc(size_t bytes) {
    size_t sz = round_size(bytes);
    std::lock_guard<std::mutex> lk(mu_);
    auto it = cache_.lower_bound(sz);
    // Reuse a cached block when it wastes at most an eighth of itself (exact for the common
    // case of a training loop that asks for the same sizes every step).
    if (it != cache_.end() && it->first - sz <= it->first / 8) {
        void* p = it->second;
        size_t bsz = it->first;
        cache_.erase(it);
        live_[p] = bsz;
        in_use_ += bsz;
        if (in_use_ > peak_) peak_ = in_use_;
        ++hits_;
        return (float*)p;
    }
    if (limit_ && reserved_ + sz > limit_) {
        // Try to get under the limit by dropping cached blocks first.
        for (auto& kv : cache_) { cudaFree(kv.second); reserved_ -= kv.first; }
        cache_.clear();
        if (reserved_ + sz > limit_) {
            set_error("device allocator: limit of %zu bytes exceeded (reserved %zu, request %zu)", limit_,
                      reserved_, sz);
            return nullptr;
        }
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, sz);
    if (e != cudaSuccess) {
        cudaGetLastError();
        for (auto& kv : cache_) { cudaFree(kv.second); reserved_ -= kv.first; }
        cache_.clear();
        e = cudaMalloc(&p, sz);
        if (e != cudaSuccess) {
            cudaGetLastError();
            set_error("device allocator: cudaMalloc of %zu bytes failed (%s)", sz, cudaGetErrorString(e));
            return nullptr;
        }
    }
    ++driver_allocs_;
    reserved_ += sz;
    live_[p] = sz;
    in_use_ += sz;
    if (in_use_ > peak_) peak_ = in_use_;
    return (float*)p;
}

void Allocator::free(float* p) {
    if (!p) return;
    std::lock_guard<std::mutex> lk(mu_);
    auto it = live_.find(p);
    if (it == live_.end()) return;  // not ours: ignore, as freeing must never abort
    size_t sz = it->second;
    live_.erase(it);
    in_use_ -= sz;
    cache_.emplace(sz, (void*)p);
}

void Allocator::release_cached() {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& kv : cache_) { cudaFree(kv.second); reserved_ -= kv.first; }
    cache_.clear();
}

void Allocator::stats(unsigned long long* in_use, unsigned long long* reserved, unsigned long long* peak,
                      unsigned long long* driver_allocs, unsigned long long* hits) {
    std::lock_guard<std::mutex> lk(mu_);
    *in_use = in_use_; *reserved = reserved_; *peak = peak_; *driver_allocs = driver_allocs_; *hits = hits_;
}

Allocator::~Allocator() {}  // device memory is reclaimed by the driver at process exit

// ------------------------------------------------------------------ contexts
static std::mutex g_ctx_mu;
static DeviceCtx* g_ctxs[64] = {nullptr};
static thread_local int g_current = -1;   // -1: not chosen yet -> device 0 (or LOCAL_RANK)
static int g_precision = -1;
static int g_fusion = 1;

static int default_device() {
    // One process per GPU under torchrun: LOCAL_RANK selects the device unless the caller does.
    const char* lr = getenv("LOCAL_RANK");
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) { cudaGetLastError(); return 0; }
    if (lr) { int v = atoi(lr); if (v >= 0 && v < n) return v; }
    return 0;
}

int current_device() {
    if (g_current < 0) g_current = default_device();
    return g_current;
}

bool set_device(int dev) {
    int n = 0;
    if (!cuda_ok(cudaGetDeviceCount(&n), "cudaGetDeviceCount")) return false;
    if (dev < 0 || dev >= n || dev >= 64) { set_error("set_cuda_device: device %d out of range (count %d)", dev, n); return false; }
    if (!cuda_ok(cudaSetDevice(dev), "cudaSetDevice")) return false;
    g_current = dev;
    return true;
}

DeviceCtx* ctx() {
    int dev = current_device();
    if (dev < 0 || dev >= 64) { set_error("no current device"); return nullptr; }
    {
        std::lock_guard<std::mutex> lk(g_ctx_mu);
        if (g_ctxs[dev]) {
            cudaSetDevice(dev);
            return g_ctxs[dev];
        }
    }
    int n = 0;
    if (!cuda_ok(cudaGetDeviceCount(&n), "cudaGetDeviceCount")) return nullptr;
    if (n <= 0 || dev >= n) { set_error("no CUDA device available (count %d); this library has no CPU fallback", n); return nullptr; }
    if (!cuda_ok(cudaSetDevice(dev), "cudaSetDevice")) return nullptr;
    cudaDeviceProp prop;
    if (!cuda_ok(cudaGetDeviceProperties(&prop, dev), "cudaGetDeviceProperties")) return nullptr;
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library is built for sm_100a (B200) only", dev, prop.major, prop.minor);
        return nullptr;
    }
    DeviceCtx* c = new DeviceCtx();
    c->device = dev;
    c->sm_count = prop.multiProcessorCount;
    bool ok = cuda_ok(cudaStreamCreateWithFlags(&c->compute, cudaStreamNonBlocking), "cudaStreamCreate") &&
              cuda_ok(cudaStreamCreateWithFlags(&c->copy, cudaStreamNonBlocking), "cudaStreamCreate") &&
              cuda_ok(cudaStreamCreateWithFlags(&c->comm, cudaStreamNonBlocking), "cudaStreamCreate") &&
              cuda_ok(cudaMalloc(&c->reduce_scratch, k::kReduceScratchElems * sizeof(float)), "cudaMalloc scratch") &&
              cuda_ok(cudaMalloc(&c->error_flag, sizeof(int)), "cudaMalloc flag") &&
              cuda_ok(cudaMalloc(&c->tile_counter, sizeof(int)), "cudaMalloc counter") &&
              cuda_ok(cudaMemset(c->error_flag, 0, sizeof(int)), "cudaMemset flag") &&
              cuda_ok(cudaMallocHost(&c->error_flag_host, sizeof(int)), "cudaMallocHost flag");
    if (!ok) { delete c; return nullptr; }
    *c->error_flag_host = 0;
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    if (!g_ctxs[dev]) g_ctxs[dev] = c;
    return g_ctxs[dev];
}

DeviceCtx* ctx_if_initialized() {
    int dev = current_device();
    if (dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    if (g_ctxs[dev]) cudaSetDevice(dev);
    return g_ctxs[dev];
}

cudaStream_t pick_stream(void* user_stream) {
    if (user_stream) return (cudaStream_t)user_stream;
    DeviceCtx* c = ctx();
    return c ? c->compute : nullptr;
}

bool dependent_launch_enabled() {
    static const bool on = [] { const char* e = getenv("TS_PDL"); return !(e && e[0] == '0'); }();
    return on;
}

int matmul_precision() {
    if (g_precision < 0) {
        const char* e = getenv("TS_MATMUL_PRECISION");
        g_precision = 0;
        if (e) {
            if (!strcmp(e, "tf32")) g_precision = 1;
            else if (!strcmp(e, "tf32x3")) g_precision = 2;
        }
    }
    return g_precision;
}
bool fusion_enabled() { return g_fusion != 0; }

// ------------------------------------------------------------------ launch accounting
struct ProfRecord { cudaEvent_t a, b; ProfClass cls; double work; };
static thread_local unsigned long long g_launches = 0;
static thread_local bool g_prof_on = false;
static thread_local std::vector<ProfRecord> g_prof_pending;
static thread_local std::vector<cudaEvent_t> g_event_pool;
static thread_local unsigned long long g_prof_launches[kProfClasses] = {0};
static thread_local double g_prof_ms[kProfClasses] = {0}, g_prof_work[kProfClasses] = {0};

static cudaEvent_t take_event() {
    if (!g_event_pool.empty()) { cudaEvent_t e = g_event_pool.back(); g_event_pool.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return e;
}

ProfScope::ProfScope(ProfClass c, cudaStream_t s, double w, int launches) : cls(c), stream(s), work(w) {
    g_launches += (unsigned long long)launches;
    if (g_prof_on) {
        start = take_event();
        if (start) cudaEventRecord(start, stream);
    }
}
ProfScope::~ProfScope() {
    if (!start) return;
    cudaEvent_t end = take_event();
    if (!end) { g_event_pool.push_back(start); return; }
    cudaEventRecord(end, stream);
    g_prof_pending.push_back(ProfRecord{start, end, cls, work});
}

ProfSuspend::ProfSuspend() : was_on(g_prof_on) { g_prof_on = false; }
ProfSuspend::~ProfSuspend() { g_prof_on = was_on; }

}  // namespace ts

using namespace ts;

TS_API void* ts_event_create(void) {
    if (!ctx()) return nullptr;
    cudaEvent_t e = nullptr;
    if (!cuda_ok(cudaEventCreate(&e), "cudaEventCreate")) return nullptr;
    return (void*)e;
}
TS_API void ts_event_destroy(void* e) { if (e) cudaEventDestroy((cudaEvent_t)e); }
TS_API bool ts_event_record(void* e, void* stream) {
    cudaStream_t s = pick_stream(stream);
    if (!s || !e) { if (!e) set_error("ts_event_record: null event"); return false; }
    return cuda_ok(cudaEventRecord((cudaEvent_t)e, s), "cudaEventRecord");
}
TS_API float ts_event_elapsed_ms(void* a, void* b) {
    if (!a || !b) { set_error("ts_event_elapsed_ms: null event"); return -1.0f; }
    if (!cuda_ok(cudaEventSynchronize((cudaEvent_t)b), "cudaEventSynchronize")) return -1.0f;
    float ms = -1.0f;
    if (!cuda_ok(cudaEventElapsedTime(&ms, (cudaEvent_t)a, (cudaEvent_t)b), "cudaEventElapsedTime")) return -1.0f;
    return ms;
}
TS_API unsigned long long ts_launch_count(void) { return ts::g_launches; }
TS_API void ts_profile_enable(int on) { ts::g_prof_on = on != 0; }
TS_API void ts_profile_reset(void) {
    for (auto& r : ts::g_prof_pending) { ts::g_event_pool.push_back(r.a); ts::g_event_pool.push_back(r.b); }
    ts::g_prof_pending.clear();
    for (int i = 0; i < kProfClasses; ++i) { ts::g_prof_launches[i] = 0; ts::g_prof_ms[i] = 0; ts::g_prof_work[i] = 0; }
}
TS_API bool ts_profile_collect(void) {
    DeviceCtx* c = ctx();
    if (!c) return false;
    TS_CHECK(cudaStreamSynchronize(c->compute));
    bool ok = true;
    for (auto& r : ts::g_prof_pending) {
        float ms = 0.0f;
        if (cudaEventSynchronize(r.b) == cudaSuccess && cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
            ts::g_prof_launches[r.cls] += 1; ts::g_prof_ms[r.cls] += ms; ts::g_prof_work[r.cls] += r.work;
        } else { cudaGetLastError(); ok = false; }
        ts::g_event_pool.push_back(r.a); ts::g_event_pool.push_back(r.b);
    }
    ts::g_prof_pending.clear();
    if (!ok) set_error("ts_profile_collect: some events could not be read");
    return ok;
}
TS_API bool ts_profile_get(int cls, unsigned long long* launches, double* total_ms, double* work) {
    if (cls < 0 || cls >= kProfClasses) { set_error("ts_profile_get: class %d out of range", cls); return false; }
    if (launches) *launches = ts::g_prof_launches[cls];
    if (total_ms) *total_ms = ts::g_prof_ms[cls];
    if (work) *work = ts::g_prof_work[cls];
    return true;
}


// ====================================================================== C ABI
TS_API const char* ts_last_error(void) { return ts::last_error(); }

TS_API bool cuda_ffi_initialize(void) { return ctx() != nullptr; }

TS_API void cuda_ffi_cleanup(void) {
    DeviceCtx* c = ctx();
    if (!c) return;
    cudaStreamSynchronize(c->compute);
    cudaStreamSynchronize(c->copy);
    cudaStreamSynchronize(c->comm);
    c->alloc.release_cached();
}

TS_API int get_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}
TS_API bool set_cuda_device(int device_id) { return ts::set_device(device_id); }
TS_API int get_current_cuda_device(void) { return ts::current_device(); }

TS_API float* cuda_malloc(unsigned long long size) {
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    return c->alloc.alloc((size_t)size * sizeof(float));
}
TS_API void cuda_free(float* ptr) {
    DeviceCtx* c = ctx();
    if (c) c->alloc.free(ptr);
}

static bool do_memcpy(float* dst, const float* src, unsigned long long size, int kind, cudaStream_t s, bool sync) {
    if (size == 0) return true;
    if (!dst || !src) { set_error("cuda_memcpy: null pointer"); return false; }
    cudaMemcpyKind mk;
    switch (kind) {
        case 0: mk = cudaMemcpyHostToDevice; break;
        case 1: mk = cudaMemcpyDeviceToHost; break;
        case 2: mk = cudaMemcpyDeviceToDevice; break;
        default: set_error("cuda_memcpy: unknown kind %d (0 = host to device, 1 = device to host, 2 = device to device)", kind); return false;
    }
    TS_CHECK(cudaMemcpyAsync(dst, src, (size_t)size * sizeof(float), mk, s));
    if (sync) TS_CHECK(cudaStreamSynchronize(s));
    return true;
}

TS_API bool cuda_memcpy(float* dst, const float* src, unsigned long long size, int kind) {
    DeviceCtx* c = ctx();
    if (!c) return false;
    return do_memcpy(dst, src, size, kind, c->compute, true);
}
TS_API bool ts_memcpy_async(float* dst, const float* src, unsigned long long size, int kind, void* stream) {
    cudaStream_t s = pick_stream(stream);
    if (!s) return false;
    return do_memcpy(dst, src, size, kind, s, false);
}

TS_API void* create_cuda_stream(void) {
    if (!ctx()) return nullptr;
    cudaStream_t s = nullptr;
    if (!cuda_ok(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate")) return nullptr;
    return (void*)s;
}
TS_API void destroy_cuda_stream(void* stream) {
    if (stream) cudaStreamDestroy((cudaStream_t)stream);
}

TS_API void* ts_compute_stream(void) {
    DeviceCtx* c = ctx();
    return c ? (void*)c->compute : nullptr;
}

TS_API bool ts_sync_stream(void* stream) {
    DeviceCtx* c = ctx();
    if (!c) return false;
    cudaStream_t s = stream ? (cudaStream_t)stream : c->compute;
    TS_CHECK(cudaMemcpyAsync(c->error_flag_host, c->error_flag, sizeof(int), cudaMemcpyDeviceToHost, s));
    TS_CHECK(cudaStreamSynchronize(s));
    if (*c->error_flag_host != 0) {
        int code = *c->error_flag_host;
        *c->error_flag_host = 0;
        cudaMemsetAsync(c->error_flag, 0, sizeof(int), s);
        cudaStreamSynchronize(s);
        if (code == TS_DEVICE_ERROR_LOG_DOMAIN) set_error("log domain error: x <= 0");   // the reference's panic text, log.rs:80-83
        else set_error("a kernel reported device-side error code %d (a bounded wait gave up); results of the last launches are invalid", code);
        return false;
    }
    return true;
}

TS_API int* ts_device_error_word(void) {
    DeviceCtx* c = ctx();
    return c ? c->error_flag : nullptr;
}

TS_API float* ts_host_alloc_pinned(unsigned long long size) {
    if (!ctx()) return nullptr;
    void* p = nullptr;
    if (!cuda_ok(cudaMallocHost(&p, (size_t)(size ? size : 1) * sizeof(float)), "cudaMallocHost")) return nullptr;
    return (float*)p;
}
TS_API void ts_host_free_pinned(float* ptr) {
    if (ptr) cudaFreeHost(ptr);
}

TS_API bool ts_allocator_get_stats(ts_allocator_stats* out) {
    DeviceCtx* c = ctx();
    if (!c || !out) return false;
    c->alloc.stats(&out->bytes_in_use, &out->bytes_reserved, &out->peak_bytes_in_use, &out->driver_allocations,
                   &out->cache_hits);
    return true;
}
TS_API void ts_allocator_release_cached(void) {
    DeviceCtx* c = ctx();
    if (!c) return;
    cudaStreamSynchronize(c->compute);
    c->alloc.release_cached();
}
TS_API bool ts_device_memory_info(unsigned long long* free_bytes, unsigned long long* total_bytes) {
    if (!ctx()) return false;
    size_t f = 0, t = 0;
    TS_CHECK(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return true;
}
TS_API void ts_allocator_set_limit(unsigned long long bytes) {
    DeviceCtx* c = ctx();
    if (c) c->alloc.set_limit((size_t)bytes);
}

TS_API bool ts_set_matmul_precision(int mode) {
    if (mode < 0 || mode > 2) { set_error("matmul precision must be 0 (fp32), 1 (tf32) or 2 (tf32x3), got %d", mode); return false; }
    ts::matmul_precision();
    ts::g_precision = mode;
    return true;
}
TS_API int ts_get_matmul_precision(void) { return ts::matmul_precision(); }
TS_API void ts_set_fusion(int enabled) { ts::g_fusion = enabled ? 1 : 0; }
TS_API int ts_get_fusion(void) { return ts::g_fusion; }
