// Tensor, gradtrack and Adam engine behind the C ABI: the device counterpart of the
// reference's src/tensor/core (storage, constructors), src/tensor/ops + reductions (the ops
// of the MLP training step), src/gradtrack (tape, backward) and src/optimizers/adam.
//
// Design, B200-first rather than a translation:
//   * every op only enqueues kernels on the per-device compute stream and returns;
//   * saved tensors are held by reference (refcounted storage) with a version counter that
//     makes an in-place write between forward and backward an error instead of a silent
//     wrong gradient (the reference deep-copies, tensor/ops/matmul/mod.rs:296-297);
//   * a matmul is not launched until its result is needed, so that a following row-broadcast
//     add, ReLU, or (in backward) ReLU mask folds into the GEMM epilogue;
//   * backward walks the tape in descending tensor-id order, which is a topological order
//     because ids are handed out monotonically (tensor/core/mod.rs:131); the reference uses a
//     LIFO worklist (gradtrack/engine.rs:962-1047) that computes the same sums;
//   * binary ops give each operand its own gradient (the reference zips gradients to
//     input ids positionally and mis-assigns them when only the second operand requires
//     grad: tensor/ops/add.rs:135-142 vs gradtrack/engine.rs:1000-1001).
#include <dlfcn.h>
#include <nccl.h>   // types only: the functions are resolved at run time, see NcclApi

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <thread>
#include <cstring>
#include <ctime>
#include <memory>
#include <unordered_set>

#include "../../include/train_station_b200.h"
#include "common.h"

namespace ts {

// ------------------------------------------------------------------ storage and tensors
struct Storage {
    float* ptr = nullptr;
    size_t n = 0;
    DeviceCtx* c = nullptr;
    uint64_t version = 0;
    cudaEvent_t ready = nullptr;   // set while an upload on the copy stream is outstanding
    // TF32 mode: the tensor core drops the low 13 mantissa bits of an FP32 operand (truncation, a
    // bias toward zero).  Operands are therefore rounded to nearest first: either the producing
    // GEMM stored them already rounded (tf32_clean), or a rounded copy is kept beside the data.
    bool tf32_clean = false;
    float* tf32_copy = nullptr;
    uint64_t tf32_copy_version = 0;
    float* tf32_lo = nullptr;          // 3xTF32 mode: rn_tf32(data - tf32_copy)
    uint64_t tf32_lo_version = 0;
    bool constant = false;             // shared read-only contents (the 1.0 that seeds backward): written through a private copy only
    ~Storage() {
        // an upload nobody waited for must land before the block goes back to the allocator
        if (ready) { cudaEventSynchronize(ready); cudaEventDestroy(ready); }
        if (c && tf32_copy) c->alloc.free(tf32_copy);
        if (c && tf32_lo) c->alloc.free(tf32_lo);
        if (c && ptr) c->alloc.free(ptr);
    }
};
using StorageP = std::shared_ptr<Storage>;

struct TensorImpl;
using TensorP = std::shared_ptr<TensorImpl>;

// A GEMM that has been requested but not launched: op(a) . op(b) [+ bias] [relu] [mask].
struct PendingGemm {
    TensorP a, b;
    bool ta = false, tb = false;
    size_t m = 0, n = 0, k = 0;
    TensorP bias, mask;
    bool relu = false;
    TensorP colsum;   // when set ([n]): receives the column sums of the result (a bias gradient), from the GEMM's epilogue
};

// An elementwise result that has been requested but not launched, so that the MSE spelling
// pred.sub_tensor(target).pow_scalar(2.0).mean() and its backward run as one pass each (the difference and its
// square are only written to memory if something else reads them):
//   Diff        a - b
//   SqDiff      (a - b) * (a - b)
//   ScalarFill  scale * a[0] in every element (the gradient ReduceMean / ReduceSum hand to their input)
struct PendingEw {
    enum Kind { Diff, SqDiff, ScalarFill } kind;
    TensorP a, b;
    float scale = 1.0f;
};

static std::atomic<uint64_t> g_next_id{1};

struct TensorImpl {
    uint64_t id;
    std::vector<size_t> dims;
    size_t size = 1;
    StorageP st;                          // null while `pending` or `pending_ew` is set
    std::unique_ptr<PendingGemm> pending;
    std::unique_ptr<PendingEw> pending_ew;
    bool requires_grad = false;
    // A transposed / permuted VIEW, as transpose() / t() / permute() return in the reference (transform/transpose.rs:181-184,
    // core/allocation.rs:220-237): it shares `st` with the tensor it was taken from, and its axis i is axis view_perm[i] of
    // the contiguous tensor of shape base_dims that st holds.  A write to either is seen through the other.  Empty
    // view_perm: an ordinary contiguous tensor.  `contig` caches the elements in the view's own order for consumers that
    // need them so (everything but a 2-D GEMM operand, which just flips its transposition flag); it is remade when
    // the shared storage's version moves on.
    std::vector<int> view_perm;
    std::vector<size_t> base_dims;
    StorageP contig;
    uint64_t contig_version = 0;
    explicit TensorImpl(const std::vector<size_t>& d) : id(g_next_id.fetch_add(1)), dims(d) {
        for (size_t x : d) size *= x;
    }
};

}  // namespace ts

struct ts_tensor { ts::TensorP t; };

namespace ts {

static StorageP new_storage(DeviceCtx* c, size_t n) {
    float* p = c->alloc.alloc((n ? n : 1) * sizeof(float));
    if (!p) return nullptr;
    auto s = std::make_shared<Storage>();
    s->ptr = p; s->n = n; s->c = c;
    return s;
}

// The one-element storage holding 1.0 that seeds backward() of a scalar: made once per device and shared by every
// seed, so that a step does not spend a launch on writing a single float.  It is never written again: the entry points
// that write into a tensor's storage in place give a tensor that holds it a private copy first (make_writable).
static StorageP ones_scalar(DeviceCtx* c) {
    static std::mutex mu;
    static StorageP* cache = new StorageP[64];   // never destroyed: must outlive every tensor that shares it
    std::lock_guard<std::mutex> lk(mu);
    if (c->device < 0 || c->device >= 64) return nullptr;
    StorageP& s = cache[c->device];
    if (!s) {
        StorageP fresh = new_storage(c, 1);
        if (!fresh || !k::fill(fresh->ptr, 1.0f, 1, c->compute)) return nullptr;
        fresh->constant = true;
        s = fresh;
    }
    return s;
}

static TensorP new_tensor(DeviceCtx* c, const std::vector<size_t>& dims) {
    auto t = std::make_shared<TensorImpl>(dims);
    t->st = new_storage(c, t->size);
    if (!t->st) return nullptr;
    return t;
}

// for_gemm: the caller is a tensor-core GEMM (or knows the result feeds one), so in TF32 mode
// the deferred GEMM may store its result already rounded to TF32.
static bool materialize(const TensorP& t, bool for_gemm = false);

static bool is_view(const TensorP& t) { return !t->view_perm.empty(); }
static bool view_refresh(const TensorP& t);

// Device pointer for reading on the compute stream (launches a deferred GEMM, waits for an upload).  For a view:
// the pointer to its elements in its own order (a cached permuted copy of the shared storage).
static const float* rptr(const TensorP& t, bool for_gemm = false) {
    if (!materialize(t, for_gemm)) return nullptr;
    Storage* s = t->st.get();
    if (s->ready) {
        cudaStreamWaitEvent(s->c->compute, s->ready, 0);
        cudaEventDestroy(s->ready);
        s->ready = nullptr;
    }
    if (is_view(t)) return view_refresh(t) ? t->contig->ptr : nullptr;
    return s->ptr;
}
// The storage that holds t's elements in t's own (logical, row-major) order: its own for an ordinary tensor, the
// cached permuted copy for a view.  Call after rptr(t).
static Storage* logical_storage(const TensorP& t) { return is_view(t) ? t->contig.get() : t->st.get(); }

// The operand as the TF32 tensor core should see it: the data itself when it is already exactly
// representable in TF32, otherwise a rounded-to-nearest copy cached beside it (refreshed when the
// data's version changes; the forward and the two backward GEMMs of a layer share it).
static const float* tf32_operand(DeviceCtx* c, const TensorP& t) {
    Storage* s = logical_storage(t);
    if (s->tf32_clean) return s->ptr;
    if (s->tf32_copy && s->tf32_copy_version == s->version) return s->tf32_copy;
    if (!s->tf32_copy) {
        s->tf32_copy = c->alloc.alloc((s->n ? s->n : 1) * sizeof(float));
        if (!s->tf32_copy) return nullptr;
    }
    if (!k::round_to_tf32(s->ptr, s->tf32_copy, s->n, c->compute)) return nullptr;
    s->tf32_copy_version = s->version;
    return s->tf32_copy;
}

// 3xTF32 mode: the operand as a TF32-exact high part plus a TF32-exact low part, cached like the copy above.
static bool tf32_split_operand(DeviceCtx* c, const TensorP& t, const float** hi, const float** lo) {
    Storage* s = logical_storage(t);
    const bool fresh = s->tf32_copy && s->tf32_lo && s->tf32_copy_version == s->version && s->tf32_lo_version == s->version;
    if (!fresh) {
        const size_t bytes = (s->n ? s->n : 1) * sizeof(float);
        if (!s->tf32_copy && !(s->tf32_copy = c->alloc.alloc(bytes))) return false;
        if (!s->tf32_lo && !(s->tf32_lo = c->alloc.alloc(bytes))) return false;
        if (!k::split_tf32(s->ptr, s->tf32_copy, s->tf32_lo, s->n, c->compute)) return false;
        s->tf32_copy_version = s->tf32_lo_version = s->version;
    }
    *hi = s->tf32_copy;
    *lo = s->tf32_lo;
    return true;
}

// (Re)makes a view's permuted copy when the shared storage has changed since it was made.  A copy that somebody else
// holds by now (reshape of a view shares it) is left alone and a new one is made.
static bool view_refresh(const TensorP& t) {
    Storage* base = t->st.get();
    if (t->contig && t->contig_version == base->version) return true;
    if (!t->contig || t->contig.use_count() > 1) {
        t->contig = new_storage(base->c, t->size);
        if (!t->contig) return false;
    }
    if (t->size && !k::permute(base->ptr, t->contig->ptr, t->base_dims.data(), t->view_perm.data(), (int)t->view_perm.size(), base->c->compute))
        return false;
    t->contig->version++;
    t->contig->tf32_clean = false;
    t->contig_version = base->version;
    return true;
}
// The contiguous tensor a view was taken from, as an operand: same storage, the storage's own shape.
static TensorP view_base(const TensorP& t) {
    auto b = std::make_shared<TensorImpl>(t->base_dims);
    b->st = t->st;
    return b;
}
// op(t) for a 2-D GEMM: a transposed view of a contiguous matrix is that matrix with the transposition flag flipped,
// so x.t().matmul(w) and the w.t() of a backward cost no copy (the reference materialises them, matmul/mod.rs:586-595).
static TensorP gemm_operand(const TensorP& t, bool* trans) {
    if (t->view_perm.size() == 2 && t->view_perm[0] == 1 && t->view_perm[1] == 0 && t->st) {
        *trans = !*trans;
        return view_base(t);
    }
    return t;
}

static bool materialize(const TensorP& t, bool for_gemm) {
    if (t->pending_ew) {
        DeviceCtx* c = ctx();
        if (!c) return false;
        PendingEw& p = *t->pending_ew;
        const float* a = rptr(p.a);
        const float* b = p.b ? rptr(p.b) : nullptr;
        if (!a || (p.b && !b)) return false;
        StorageP st = new_storage(c, t->size);
        if (!st) return false;
        bool ok = false;
        switch (p.kind) {
            case PendingEw::Diff: ok = k::binary(1, a, b, st->ptr, t->size, c->compute); break;
            case PendingEw::SqDiff: ok = k::sqdiff(a, b, st->ptr, t->size, c->compute); break;
            case PendingEw::ScalarFill: ok = k::fill_from_scalar(st->ptr, a, p.scale, t->size, c->compute); break;
        }
        if (!ok) return false;
        t->st = st;
        t->pending_ew.reset();
        return true;
    }
    if (!t->pending) return t->st != nullptr;
    DeviceCtx* c = ctx();
    if (!c) return false;
    PendingGemm& p = *t->pending;
    const float* a = rptr(p.a, true);
    const float* b = rptr(p.b, true);
    const float* bias = p.bias ? rptr(p.bias) : nullptr;
    const float* mask = p.mask ? rptr(p.mask) : nullptr;
    if (!a || !b || (p.bias && !bias) || (p.mask && !mask)) return false;
    StorageP st = new_storage(c, t->size);
    if (!st) return false;
    k::GemmArgs g{a, b, st->ptr, p.m, p.n, p.k, p.ta, p.tb, bias, p.relu, mask};
    if (p.colsum) g.colsum_out = p.colsum->st->ptr;
    if (matmul_precision() == 1 && k::gemm_tc_supported(g)) {
        g.a = tf32_operand(c, p.a);
        g.b = tf32_operand(c, p.b);
        if (!g.a || !g.b) return false;
        g.round_tf32 = for_gemm;
        st->tf32_clean = for_gemm;
    } else if (matmul_precision() == 2 && k::gemm_tc_supported(g)) {
        if (!tf32_split_operand(c, p.a, &g.a, &g.a_lo) || !tf32_split_operand(c, p.b, &g.b, &g.b_lo)) return false;
    }
    if (matmul_precision() == 1 && for_gemm && !g.round_tf32 && k::gemm_thin_rounds(g)) {
        g.round_tf32 = true;     // a thin product that feeds a tensor-core GEMM: rounded as it is stored, no pass of its own
        st->tf32_clean = true;
    }
    if (!k::gemm(g, -1, c, c->compute)) return false;
    t->st = st;
    t->pending.reset();   // releases the operand references
    return true;
}

// ------------------------------------------------------------------ tape
enum class Op { Add, Sub, Mul, Div, Relu, MatMul, PowScalar, ReduceSum, ReduceMean, Unary, Softmax, Reshape, Permute, ReduceDims, Cat, Split };

struct Saved {
    TensorP t;
    uint64_t version = 0;
    void set(const TensorP& x) { t = x; version = x->st ? x->st->version : 0; }
    bool check(const char* what) const {
        uint64_t now = t->st ? t->st->version : 0;
        if (now != version) {
            set_error("backward: the tensor saved for %s (id %llu) was modified in place after the forward pass", what,
                      (unsigned long long)t->id);
            return false;
        }
        return true;
    }
};

struct Node {
    Op op;
    std::vector<uint64_t> inputs;       // ids, positional: [a, b] or [x]
    std::vector<bool> needs;            // which inputs want a gradient
    Saved s0, s1, s2;                   // saved tensors (meaning depends on op)
    std::vector<size_t> dims0, dims1;   // operand shapes
    float scalar = 0.0f;
    int code = 0;                       // Unary: the ts_unary_op; Softmax: the axis
    std::vector<int> perm;              // Permute: output axis i is input axis perm[i]; ReduceDims: 1 for each reduced axis
};

struct Graph {
    std::unordered_map<uint64_t, Node> ops;
    std::unordered_map<uint64_t, TensorP> grads;
    std::unordered_map<uint64_t, TensorP> bias_grad_ready;   // column sums produced early by a fused kernel, keyed by the Add output id
};

static thread_local Graph g_graph;
static thread_local int g_no_grad_depth = 0;
static thread_local std::vector<std::weak_ptr<TensorImpl>> g_pending_registry;

static bool grad_on() { return g_no_grad_depth == 0; }

static void register_pending(const TensorP& t) {
    if (g_pending_registry.size() > 4096) {
        auto& v = g_pending_registry;
        v.erase(std::remove_if(v.begin(), v.end(),
                               [](const std::weak_ptr<TensorImpl>& w) { auto s = w.lock(); return !s || (!s->pending && !s->pending_ew); }),
                v.end());
    }
    g_pending_registry.push_back(t);
}
// Does the value of t depend on one of the storages in `written`?
static bool reads_any(const TensorP& t, const std::unordered_set<const Storage*>& written) {
    if (!t) return false;
    if (t->pending) {
        const PendingGemm& p = *t->pending;
        return reads_any(p.a, written) || reads_any(p.b, written) || reads_any(p.bias, written) || reads_any(p.mask, written);
    }
    if (t->pending_ew) return reads_any(t->pending_ew->a, written) || reads_any(t->pending_ew->b, written);
    return t->st && written.count(t->st.get()) != 0;
}
// Before an in-place write to the storages in `written`: launch every deferred operation that reads one of them,
// so that it sees the old contents.  Deferred operations on other data stay deferred.
static bool flush_pending(const std::unordered_set<const Storage*>& written) {
    auto reg = std::move(g_pending_registry);
    g_pending_registry.clear();
    bool ok = true;
    for (auto& w : reg) {
        TensorP t = w.lock();
        if (!t || (!t->pending && !t->pending_ew)) continue;
        if (reads_any(t, written)) ok = materialize(t) && ok;
        else g_pending_registry.push_back(w);
    }
    return ok;
}

// ------------------------------------------------------------------ NCCL, bound at run time
// NCCL is opened with dlopen when data parallelism is first used, not linked: a process that also
// imports PyTorch must end up with ONE libnccl.so.2 (PyTorch bundles a newer one than the system's,
// and whichever is loaded first is the one both get).  Loading it lazily means a single-GPU process
// never loads NCCL at all, and a multi-GPU process that imported PyTorch first shares PyTorch's copy.
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
    bool fake = false;   // an in-process stand-in installed by ts_dp_install_fake_nccl (host-side failure tests)
};
static NcclApi g_nccl;
static std::mutex g_nccl_mu;
// ---- an in-process stand-in for NCCL, for host-side tests of the failure handling (no GPU, no second process).
// It moves no data.  mode 0: every call succeeds; 1: ncclCommInitRank never returns (a peer that never joins);
// 2: the collectives return an error; 3: ncclCommGetAsyncError reports a remote error (a peer that died).
static std::atomic<int> g_fake_mode{0}, g_fake_aborts{0};
static ncclResult_t fake_get_unique_id(ncclUniqueId* id) { memset(id, 0x5a, sizeof(*id)); return ncclSuccess; }
static ncclResult_t fake_comm_init_rank(ncclComm_t* comm, int, ncclUniqueId, int) {
    if (g_fake_mode.load() == 1) {
        std::mutex m;
        std::condition_variable never;
        std::unique_lock<std::mutex> lk(m);
        never.wait(lk, [] { return false; });
    }
    *comm = reinterpret_cast<ncclComm_t>(uintptr_t(0x1));
    return ncclSuccess;
}
static ncclResult_t fake_collective() { return g_fake_mode.load() == 2 ? ncclInternalError : ncclSuccess; }
static ncclResult_t fake_all_reduce(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) { return fake_collective(); }
static ncclResult_t fake_reduce_scatter(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) { return fake_collective(); }
static ncclResult_t fake_all_gather(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) { return fake_collective(); }
static ncclResult_t fake_async_error(ncclComm_t, ncclResult_t* out) { *out = g_fake_mode.load() == 3 ? ncclRemoteError : ncclSuccess; return ncclSuccess; }
static ncclResult_t fake_abort(ncclComm_t) { g_fake_aborts.fetch_add(1); return ncclSuccess; }
static ncclResult_t fake_destroy(ncclComm_t) { return ncclSuccess; }
static const char* fake_error_string(ncclResult_t r) {
    return r == ncclSuccess ? "no error" : r == ncclRemoteError ? "remote process exited or there was a network error" : "internal error";
}

static NcclApi* nccl_api() {
    NcclApi& api = g_nccl;
    std::lock_guard<std::mutex> lk(g_nccl_mu);
    if (api.ok) return &api;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!h) { set_error("data parallelism needs NCCL: dlopen(libnccl.so.2) failed: %s", dlerror()); return nullptr; }
    api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
    api.AllReduce = (decltype(api.AllReduce))dlsym(h, "ncclAllReduce");
    api.ReduceScatter = (decltype(api.ReduceScatter))dlsym(h, "ncclReduceScatter");
    api.AllGather = (decltype(api.AllGather))dlsym(h, "ncclAllGather");
    api.CommGetAsyncError = (decltype(api.CommGetAsyncError))dlsym(h, "ncclCommGetAsyncError");
    api.CommAbort = (decltype(api.CommAbort))dlsym(h, "ncclCommAbort");
    api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
    api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
    if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.ReduceScatter || !api.AllGather || !api.CommGetAsyncError ||
        !api.CommAbort || !api.CommDestroy || !api.GetErrorString) {
        set_error("data parallelism needs NCCL: a required symbol is missing from libnccl.so.2");
        return nullptr;
    }
    api.ok = true;
    return &api;
}

// ------------------------------------------------------------------ data-parallel state
// The cross-rank sum of one registered parameter's gradient since the last zero_grad.  Large tensors are
// reduce-scattered: this rank then holds the sum only for elements [lo, lo + cnt), runs Adam on that slice alone and
// the updated parameters are all-gathered, so that neither the optimizer's 28 bytes per parameter nor its arithmetic
// are replicated on every GPU.  Small or oddly sized tensors are all-reduced and updated on every rank.
struct DpGrad {
    TensorP buf;             // full-size buffer
    bool sliced = false;     // produced by a reduce-scatter: [lo, lo + cnt) holds the sum over ranks
    bool gathered = false;   // ... and the other ranks' slices have since been all-gathered into it (grad_by_value)
    size_t lo = 0, cnt = 0;
};
struct DpState {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    std::unordered_set<uint64_t> params;
    cudaEvent_t ev_compute = nullptr, ev_comm = nullptr, ev_grads = nullptr;
    bool comm_outstanding = false;    // work on the communication stream that the compute stream has not been ordered after
    bool grads_outstanding = false;   // ... some of which reads or writes gradient buffers (ev_grads marks its end)
    std::unordered_map<uint64_t, DpGrad> red;
    std::unordered_map<uint64_t, cudaEvent_t> done_event;   // per parameter: its gradient's sum has landed
    std::vector<TensorP> retired;     // buffers the communication stream may still read; released at the next join
    bool failed = false;              // the communicator reported an asynchronous error and was aborted
};
static thread_local DpState g_dp;

// Tensors below this size, or whose size is not a multiple of 8 * world, keep the all-reduce and the replicated update
// (a slice must start on a multiple of 8 elements so that Adam's 8-wide body / tail association, adam/mod.rs:761-772,
// is the one the whole tensor would get).
constexpr size_t kMinShardElems = size_t(1) << 16;
static bool dp_shard_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("TS_DP_SHARD"); v = (e && e[0] == '0') ? 0 : 1; }   // TS_DP_SHARD=0: all-reduce everything
    return v == 1;
}

// Sharded update in TF32 mode: only the parameters are all-gathered and every rank then rounds its own TF32 copy
// (default), or the slices' owners also write the rounded copies and those are all-gathered too (TS_DP_GATHER_TF32=1:
// no rounding pass, but half as much traffic again on NVLink beside the next forward's GEMMs).  Measured on 4 GPUs
// (C5): 18.8 ms per step against 20.3, because collectives that run beside the persistent GEMM kernels slow those down.
static bool dp_gather_tf32_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("TS_DP_GATHER_TF32"); v = (e && e[0] == '1') ? 1 : 0; }
    return v == 1;
}

// Which part of a gradient of n elements rank `rank` of `world` owns after the sum: the whole of it ([0, n), not sliced)
// when the tensor is small, when n is not a multiple of 8 * world, or when sharding is switched off; else the rank's
// contiguous n / world elements.  Host arithmetic only (ts_debug_dp_shard_plan reports it without a device).
static bool dp_shard_plan(size_t n, size_t world, size_t rank, size_t* lo, size_t* cnt) {
    const bool slice = world > 1 && dp_shard_enabled() && n >= kMinShardElems && n % (8 * world) == 0;
    *cnt = slice ? n / world : n;
    *lo = slice ? rank * *cnt : 0;
    return slice;
}

static bool dp_nccl_ok(NcclApi* nc, ncclResult_t r, const char* what) {
    if (r == ncclSuccess) return true;
    set_error("%s failed: %s", what, nc->GetErrorString(r));
    return false;
}
// Polls the communicator for an asynchronous error (a peer that died, a transport fault).  On error the
// communicator is aborted, so that no later call can block on it, and every later collective is refused.
static bool dp_healthy() {
    if (g_dp.failed) { set_error("data parallelism: the communicator was aborted after an asynchronous NCCL error"); return false; }
    if (!g_dp.comm) return true;
    NcclApi* nc = nccl_api();
    if (!nc) return false;
    ncclResult_t async = ncclSuccess;
    ncclResult_t r = nc->CommGetAsyncError(g_dp.comm, &async);
    if (r == ncclSuccess && (async == ncclSuccess || async == ncclInProgress)) return true;
    const ncclResult_t shown = r != ncclSuccess ? r : async;
    nc->CommAbort(g_dp.comm);
    g_dp.comm = nullptr;
    g_dp.failed = true;
    set_error("data parallelism: NCCL reported an asynchronous error (%s); the communicator was aborted", nc->GetErrorString(shown));
    return false;
}
static bool dp_events() {
    if (g_dp.ev_compute) return true;
    TS_CHECK(cudaEventCreateWithFlags(&g_dp.ev_compute, cudaEventDisableTiming));
    TS_CHECK(cudaEventCreateWithFlags(&g_dp.ev_comm, cudaEventDisableTiming));
    TS_CHECK(cudaEventCreateWithFlags(&g_dp.ev_grads, cudaEventDisableTiming));
    return true;
}
// The communication stream waits for everything enqueued on the compute stream so far.
static bool dp_comm_after_compute(DeviceCtx* c) {
    if (!dp_events()) return false;
    TS_CHECK(cudaEventRecord(g_dp.ev_compute, c->compute));
    TS_CHECK(cudaStreamWaitEvent(c->comm, g_dp.ev_compute, 0));
    return true;
}
// Marks the end of the gradient-touching work enqueued on the communication stream so far.
static bool dp_mark_grads(DeviceCtx* c) {
    TS_CHECK(cudaEventRecord(g_dp.ev_grads, c->comm));
    g_dp.comm_outstanding = g_dp.grads_outstanding = true;
    return true;
}

static bool dp_all_reduce_async(DeviceCtx* c, float* data, size_t n) {
    if (!g_dp.comm || g_dp.world <= 1) return true;
    if (!dp_healthy() || !dp_comm_after_compute(c)) return false;
    NcclApi* nc = nccl_api();
    if (!nc || !dp_nccl_ok(nc, nc->AllReduce(data, data, n, ncclFloat32, ncclSum, g_dp.comm, c->comm), "ncclAllReduce")) return false;
    return dp_mark_grads(c);
}
// The compute stream waits for everything enqueued on the communication stream so far.
static bool dp_join(DeviceCtx* c) {
    if (!g_dp.comm_outstanding) return true;
    TS_CHECK(cudaEventRecord(g_dp.ev_comm, c->comm));
    TS_CHECK(cudaStreamWaitEvent(c->compute, g_dp.ev_comm, 0));
    g_dp.comm_outstanding = g_dp.grads_outstanding = false;
    g_dp.retired.clear();
    return dp_healthy();
}
// The compute stream waits for the gradient-touching part only: what gradient buffers need before they are reused.
// All-gathers of updated parameters that follow it on the communication stream keep running.
static bool dp_join_grads(DeviceCtx* c) {
    if (!g_dp.grads_outstanding) return true;
    TS_CHECK(cudaStreamWaitEvent(c->compute, g_dp.ev_grads, 0));
    g_dp.grads_outstanding = false;
    g_dp.retired.clear();
    return true;
}

// Starts the cross-rank sum of a registered parameter's finished local gradient `lg` (which nothing else references)
// on the communication stream and files it under the parameter's id.  A parameter that already holds a sum from an
// earlier backward() since the last zero_grad gets the new sum added to it: sum(G1) + sum(G2), as the reference
// accumulates G1 + G2 (gradtrack/engine.rs:514-524).
static bool dp_reduce_leaf(DeviceCtx* c, uint64_t id, const TensorP& lg) {
    NcclApi* nc = nccl_api();
    if (!nc || !dp_healthy() || !dp_comm_after_compute(c)) return false;
    const size_t n = lg->size;
    const size_t world = (size_t)g_dp.world;
    auto have = g_dp.red.find(id);
    size_t lo = 0, cnt = n;
    bool slice = dp_shard_plan(n, world, (size_t)g_dp.rank, &lo, &cnt);
    if (slice && have != g_dp.red.end() && (!have->second.sliced || have->second.gathered)) {   // the earlier sum is held in full
        slice = false;
        lo = 0; cnt = n;
    }
    float* p = lg->st->ptr;
    if (slice) {
        if (!dp_nccl_ok(nc, nc->ReduceScatter(p, p + lo, cnt, ncclFloat32, ncclSum, g_dp.comm, c->comm), "ncclReduceScatter")) return false;
    } else {
        if (!dp_nccl_ok(nc, nc->AllReduce(p, p, n, ncclFloat32, ncclSum, g_dp.comm, c->comm), "ncclAllReduce")) return false;
    }
    if (have == g_dp.red.end()) {
        DpGrad g;
        g.buf = lg; g.sliced = slice; g.lo = lo; g.cnt = cnt;
        g_dp.red[id] = g;
    } else {
        float* acc = have->second.buf->st->ptr;
        if (!k::binary(0, acc + lo, p + lo, acc + lo, cnt, c->comm)) return false;
        g_dp.retired.push_back(lg);   // read by the add above: kept until the compute stream is ordered after it
    }
    cudaEvent_t& ev = g_dp.done_event[id];
    if (!ev) TS_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    TS_CHECK(cudaEventRecord(ev, c->comm));
    return dp_mark_grads(c);
}
// Makes a reduce-scattered gradient whole on every rank (for a caller that wants to read it).
static bool dp_gather_grad(DeviceCtx* c, DpGrad& g) {
    if (!g.sliced || g.gathered) return true;
    NcclApi* nc = nccl_api();
    if (!nc || !dp_healthy()) return false;
    float* p = g.buf->st->ptr;
    if (!dp_nccl_ok(nc, nc->AllGather(p + g.lo, p, g.cnt, ncclFloat32, g_dp.comm, c->comm), "ncclAllGather")) return false;
    g.gathered = true;
    return dp_mark_grads(c);
}

// ------------------------------------------------------------------ helpers
static bool same_dims(const std::vector<size_t>& a, const std::vector<size_t>& b) { return a == b; }

static std::vector<size_t> strip_leading_ones(const std::vector<size_t>& d) {
    size_t i = 0;
    while (i + 1 < d.size() && d[i] == 1) ++i;
    return std::vector<size_t>(d.begin() + i, d.end());
}
// `small` broadcasts over the leading dimensions of `big` (e.g. [M,N] + [N], [M,N] + [1,N]).
static bool is_suffix_broadcast(const std::vector<size_t>& big, const std::vector<size_t>& small, size_t* rows, size_t* cols) {
    size_t small_n = 1, big_n = 1;
    for (size_t x : small) small_n *= x;
    for (size_t x : big) big_n *= x;
    if (small_n == 1) { *rows = big_n; *cols = 1; return true; }   // a one-element tensor broadcasts over everything
    std::vector<size_t> s = strip_leading_ones(small);
    if (s.size() > big.size()) return false;
    size_t off = big.size() - s.size();
    size_t c = 1;
    for (size_t i = 0; i < s.size(); ++i) {
        if (s[i] != big[off + i]) return false;
        c *= s[i];
    }
    size_t r = 1;
    for (size_t i = 0; i < off; ++i) r *= big[i];
    *rows = r; *cols = c;
    return true;
}

// a shape as Rust's {:?} prints a Vec<usize>: "[2, 3]"
static std::string dims_debug(const std::vector<size_t>& d) {
    std::string s = "[";
    for (size_t i = 0; i < d.size(); ++i) s += (i ? ", " : "") + std::to_string(d[i]);
    return s + "]";
}
// tensor/ops/broadcasting.rs:100-135: axes pair up from the right; equal extents or a 1 on either side; the message
// is the one add/sub/mul/div_tensor panic with (add.rs:114-122 around the Display of BroadcastError).
static bool broadcast_shape(const std::vector<size_t>& a, const std::vector<size_t>& b, std::vector<size_t>* out) {
    const size_t ra = a.size(), rb = b.size(), n = ra > rb ? ra : rb;
    out->assign(n, 1);
    for (size_t i = 0; i < n; ++i) {
        const size_t da = i < ra ? a[ra - 1 - i] : 1, db = i < rb ? b[rb - 1 - i] : 1;
        if (da != db && da != 1 && db != 1) {
            const std::string sa = dims_debug(a), sb = dims_debug(b);
            set_error("Cannot broadcast tensor shapes %s and %s: Cannot broadcast shapes %s and %s: incompatible dimensions at axis %zu",
                      sa.c_str(), sb.c_str(), sa.c_str(), sb.c_str(), n - 1 - i);
            return false;
        }
        (*out)[n - 1 - i] = da == 1 ? db : da;
    }
    return true;
}
// element strides of a contiguous operand of shape `own` along the axes of the broadcast shape `out`: 0 where the
// operand is stretched (broadcasting.rs compute_broadcast_strides)
static std::vector<size_t> broadcast_strides(const std::vector<size_t>& own, const std::vector<size_t>& out) {
    std::vector<size_t> st(out.size(), 0);
    size_t run = 1;
    for (size_t i = 0; i < own.size(); ++i) {
        const size_t d = own[own.size() - 1 - i];
        if (d != 1) st[out.size() - 1 - i] = run;
        run *= d;
    }
    return st;
}

static TensorP grad_lookup(uint64_t id) {
    auto it = g_graph.grads.find(id);
    if (it != g_graph.grads.end()) return it->second;
    auto r = g_dp.red.find(id);   // a registered parameter's gradient lives with the data-parallel state once its sum has started
    return r == g_dp.red.end() ? nullptr : r->second.buf;
}

// gradtrack/engine.rs:514-524: existing + new into a fresh tensor.
static bool accumulate(DeviceCtx* c, uint64_t id, const TensorP& g) {
    auto it = g_graph.grads.find(id);
    if (it == g_graph.grads.end()) { g_graph.grads[id] = g; return true; }
    g_graph.bias_grad_ready.erase(id);   // a second contribution invalidates early column sums
    const float* a = rptr(it->second);
    const float* b = rptr(g);
    if (!a || !b) return false;
    if (it->second->size != g->size) { set_error("backward: gradient size mismatch for tensor %llu", (unsigned long long)id); return false; }
    TensorP out = new_tensor(c, it->second->dims);
    if (!out) return false;
    if (!k::binary(0, a, b, out->st->ptr, out->size, c->compute)) return false;
    it->second = out;
    return true;
}

static TensorP reshaped_alias(const TensorP& t, const std::vector<size_t>& dims) {
    if (t->dims == dims) return t;
    if (!materialize(t)) return nullptr;
    auto r = std::make_shared<TensorImpl>(dims);
    if (is_view(t)) {   // the elements in the view's order live in its permuted copy
        if (!rptr(t)) return nullptr;
        r->st = t->contig;
    } else {
        r->st = t->st;
    }
    return r;
}

// `rows` runs of `width` contiguous elements from src (row pitch src_pitch, starting at src_off) to dst (row pitch
// dst_pitch, starting at dst_off): the slab of an axis that cat / split address.  A strided device-to-device copy.
static bool copy_slab(float* dst, size_t dst_pitch, size_t dst_off, const float* src, size_t src_pitch, size_t src_off, size_t width,
                      size_t rows, cudaStream_t s) {
    if (width == 0 || rows == 0) return true;
    if (rows == 1 || (dst_pitch == width && src_pitch == width))
        return cuda_ok(cudaMemcpyAsync(dst + dst_off, src + src_off, rows * width * sizeof(float), cudaMemcpyDeviceToDevice, s), "slab copy");
    return cuda_ok(cudaMemcpy2DAsync(dst + dst_off, dst_pitch * sizeof(float), src + src_off, src_pitch * sizeof(float),
                                     width * sizeof(float), rows, cudaMemcpyDeviceToDevice, s), "slab copy");
}

// ---- batched matmul (tensor/ops/matmul/mod.rs:634-835): the last two axes multiply, the leading axes broadcast
// right-aligned; one GEMM launch per batch entry on offsets into the operands.
struct BatchGeom {
    std::vector<size_t> batch;      // broadcast batch dims of the result
    size_t count = 1;
};
// element offset of batch entry `idx` (over `batch`) in an operand whose own batch dims are `own` (right-aligned,
// extent 1 broadcasts) and whose matrices have `mat` elements (mod.rs:764-835)
static size_t batch_offset(size_t idx, const std::vector<size_t>& batch, const std::vector<size_t>& own, size_t mat) {
    size_t off = 0, stride = mat;
    const size_t nb = batch.size(), no = own.size();
    for (size_t i = 0; i < nb; ++i) {            // from the innermost batch axis outwards
        const size_t bd = batch[nb - 1 - i];
        const size_t coord = idx % bd;
        idx /= bd;
        if (i < no) {
            const size_t od = own[no - 1 - i];
            if (od != 1) off += coord * stride;
            stride *= od;
        }
    }
    return off;
}
static bool broadcast_batch(const std::vector<size_t>& a, const std::vector<size_t>& b, BatchGeom* g) {
    const size_t na = a.size(), nb = b.size(), n = na > nb ? na : nb;
    g->batch.assign(n, 1);
    g->count = 1;
    for (size_t i = 0; i < n; ++i) {
        const size_t da = i < na ? a[na - 1 - i] : 1, db = i < nb ? b[nb - 1 - i] : 1;
        if (da != 1 && db != 1 && da != db) { set_error("Cannot broadcast dimensions %zu and %zu", da, db); return false; }   // mod.rs:672
        g->batch[n - 1 - i] = da == 1 ? db : da;
        g->count *= g->batch[n - 1 - i];
    }
    return true;
}
// out[batch][m][n] = op(A)[batch] . op(B)[batch]; a_batch / b_batch are the operands' own batch dims.
static bool batched_gemm(DeviceCtx* c, const TensorP& ta, const std::vector<size_t>& a_batch, bool trans_a, const TensorP& tb,
                         const std::vector<size_t>& b_batch, bool trans_b, float* out, const BatchGeom& g, size_t m, size_t n, size_t kk) {
    const float* pa = rptr(ta, true);
    const float* pb = rptr(tb, true);
    if (!pa || !pb) return false;
    const int prec = matmul_precision();
    const size_t a_mat = m * kk, b_mat = kk * n;
    // The FP32 kernel takes the whole batch as one launch (grid z) when every entry's operands sit at a fixed stride
    // from the previous entry's (equal batch shapes, or an operand without batch axes: stride 0).
    // In TF32 mode the tensor-core kernel runs one launch (and three tensor maps) per entry, about 8 us of fixed cost
    // each: entries of up to 512^3 multiply-adds are faster, and more accurate, as one FP32 launch over the batch.
    k::GemmArgs probe{pa, pb, out, m, n, kk, trans_a, trans_b, nullptr, false, nullptr};
    const bool small_entries = (double)m * (double)n * (double)kk <= (double)(1u << 27);
    if (g.count > 1 && g.count <= 65535 && (prec == 0 || (prec == 1 && (small_entries || !k::gemm_tc_supported(probe))))) {
        const size_t sa = batch_offset(1, g.batch, a_batch, a_mat), sb = batch_offset(1, g.batch, b_batch, b_mat);
        bool affine = true;
        for (size_t i = 2; i < g.count && affine; ++i)
            affine = batch_offset(i, g.batch, a_batch, a_mat) == i * sa && batch_offset(i, g.batch, b_batch, b_mat) == i * sb;
        if (affine) {
            k::GemmArgs all{pa, pb, out, m, n, kk, trans_a, trans_b, nullptr, false, nullptr};
            all.batch = g.count;
            all.batch_stride_a = sa;
            all.batch_stride_b = sb;
            return k::sgemm(all, c->compute);
        }
    }
    const float *ra = pa, *rb = pb;
    if (prec == 1) {   // TF32: operands rounded to nearest first (cached copies beside the data)
        ra = tf32_operand(c, ta);
        rb = tf32_operand(c, tb);
        if (!ra || !rb) return false;
    }
    for (size_t i = 0; i < g.count; ++i) {
        const size_t ao = batch_offset(i, g.batch, a_batch, a_mat), bo = batch_offset(i, g.batch, b_batch, b_mat);
        k::GemmArgs ga{ra + ao, rb + bo, out + i * m * n, m, n, kk, trans_a, trans_b, nullptr, false, nullptr};
        bool ok;
        if (prec == 1 && !k::gemm_tc_supported(ga)) {
            k::GemmArgs raw{pa + ao, pb + bo, out + i * m * n, m, n, kk, trans_a, trans_b, nullptr, false, nullptr};
            ok = k::sgemm(raw, c->compute);      // shapes the tensor-core kernel cannot take run in FP32 on the unrounded data
        } else {
            ok = k::gemm(ga, prec, c, c->compute);
        }
        if (!ok) return false;
    }
    return true;
}
// grad_fn/ops/matmul.rs reduce_gradient_to_original_shape: leading extra axes are summed away, then axes that
// were 1 in the operand are summed with keepdim.
static TensorP reduce_to_shape(DeviceCtx* c, const TensorP& g, const std::vector<size_t>& want) {
    if (g->dims == want) return g;
    if (!rptr(g)) return nullptr;
    if (g->size == 0) {                          // nothing to sum: zeros of the wanted shape
        TensorP z = new_tensor(c, want);
        if (z && z->size && !k::fill(z->st->ptr, 0.0f, z->size, c->compute)) return nullptr;
        return z;
    }
    TensorP cur = g;
    auto sum_axes = [&](const std::vector<unsigned char>& red, const std::vector<size_t>& od) -> TensorP {
        TensorP o = new_tensor(c, od);
        float* scratch = o ? c->alloc.alloc(k::reduce_dims_scratch_elems() * sizeof(float)) : nullptr;
        if (!scratch) return nullptr;
        bool ok = k::reduce_dims(0, rptr(cur), nullptr, o->st->ptr, cur->dims.data(), (int)cur->dims.size(), red.data(), scratch, c->compute);
        c->alloc.free(scratch);
        return ok ? o : nullptr;
    };
    if (cur->dims.size() > want.size()) {
        const size_t extra = cur->dims.size() - want.size();
        std::vector<unsigned char> red(cur->dims.size(), 0);
        for (size_t i = 0; i < extra; ++i) red[i] = 1;
        cur = sum_axes(red, std::vector<size_t>(cur->dims.begin() + extra, cur->dims.end()));
        if (!cur) return nullptr;
    }
    std::vector<unsigned char> red(cur->dims.size(), 0);
    bool any = false;
    for (size_t i = 0; i < cur->dims.size() && i < want.size(); ++i)
        if (want[i] == 1 && cur->dims[i] > 1) { red[i] = 1; any = true; }
    if (any) {
        cur = sum_axes(red, want);
        if (!cur) return nullptr;
    }
    if (cur->dims != want) cur = reshaped_alias(cur, want);
    return cur;
}

// ------------------------------------------------------------------ backward of one node
static bool apply_node(DeviceCtx* c, uint64_t out_id, Node& nd, const TensorP& go, std::vector<TensorP>& gin) {
    cudaStream_t s = c->compute;
    gin.assign(nd.inputs.size(), nullptr);
    switch (nd.op) {
        case Op::Add: {
            // grad_fn/ops/add.rs:4-28 + grad_fn/utils.rs:23-60: the gradient itself, summed back over
            // broadcast dimensions for the smaller operand.
            for (int i = 0; i < 2; ++i) {
                if (!nd.needs[i]) continue;
                const std::vector<size_t>& od = i == 0 ? nd.dims0 : nd.dims1;
                const std::vector<size_t>& other = i == 0 ? nd.dims1 : nd.dims0;
                size_t osz = 1; for (size_t x : od) osz *= x;
                if (osz == go->size) { gin[i] = reshaped_alias(go, od); if (!gin[i]) return false; continue; }
                size_t rows, cols;
                if (!is_suffix_broadcast(other, od, &rows, &cols)) {
                    gin[i] = reduce_to_shape(c, go, od);       // broadcasting in general
                    if (!gin[i]) return false;
                    continue;
                }
                auto pre = g_graph.bias_grad_ready.find(out_id);
                if (pre != g_graph.bias_grad_ready.end() && pre->second->size == cols) {
                    gin[i] = reshaped_alias(pre->second, od);
                    g_graph.bias_grad_ready.erase(pre);
                    continue;
                }
                // When the other operand came out of a matmul, this gradient goes on into that matmul's
                // two backward GEMMs: let a deferred GEMM that produces it store TF32-rounded values.
                auto other_prod = g_graph.ops.find(nd.inputs[1 - i]);
                const bool feeds_gemm = other_prod != g_graph.ops.end() && other_prod->second.op == Op::MatMul;
                if (fusion_enabled() && matmul_precision() != 0 && go->pending && !go->pending->colsum && cols > 1 &&
                    go->pending->m == rows && go->pending->n == cols) {
                    // The gradient is itself a deferred GEMM (the input gradient of the next layer, ReLU mask folded in):
                    // its epilogue also produces the column sums, so the full-size gradient is not read back for them.
                    // (The TF32 modes only: the FP32 kernels have no such epilogue and their column sums stay a pass of their own.)
                    TensorP r = new_tensor(c, od);
                    if (!r) return false;
                    go->pending->colsum = r;
                    if (!rptr(go, feeds_gemm)) return false;
                    gin[i] = r;
                    continue;
                }
                const float* gp = rptr(go, feeds_gemm);
                if (!gp) return false;
                TensorP r = new_tensor(c, od);
                if (!r) return false;
                if (cols == 1) {
                    if (!k::sum(gp, r->st->ptr, go->size, false, c->reduce_scratch, s)) return false;
                } else {
                    size_t sc = k::colsum_scratch_elems(rows, cols);
                    float* scratch = c->alloc.alloc(sc * sizeof(float));
                    if (!scratch) return false;
                    bool ok = k::colsum(gp, r->st->ptr, rows, cols, scratch, s);
                    c->alloc.free(scratch);   // reused only by later work on the same stream
                    if (!ok) return false;
                }
                gin[i] = r;
            }
            return true;
        }
        case Op::Sub: {
            // grad_fn/ops/sub.rs:4-33: (go, -go), each summed back to its operand's shape after a broadcast
            // (negating before or after the sums gives the same bits)
            if (nd.needs[0]) {
                gin[0] = nd.dims0 == go->dims ? go : reduce_to_shape(c, go, nd.dims0);
                if (!gin[0]) return false;
            }
            if (nd.needs[1]) {
                TensorP g1 = nd.dims1 == go->dims ? go : reduce_to_shape(c, go, nd.dims1);
                const float* gp = g1 ? rptr(g1) : nullptr;
                TensorP r = gp ? new_tensor(c, g1->dims) : nullptr;
                if (!r || !k::scale(gp, -1.0f, r->st->ptr, r->size, s)) return false;
                gin[1] = r;
            }
            return true;
        }
        case Op::Mul:
        case Op::Div: {
            if (!nd.s0.check("mul/div") || !nd.s1.check("mul/div")) return false;
            const float *a = rptr(nd.s0.t), *b = rptr(nd.s1.t), *gp = rptr(go);
            if (!a || !b || !gp) return false;
            if (nd.dims0 != nd.dims1) {
                // grad_fn/ops/mul.rs, div.rs with original_shapes: the full-size gradients over the broadcast
                // shape, then each summed back to its operand's shape (grad_fn/utils.rs:23-60)
                std::vector<size_t> od;
                if (!broadcast_shape(nd.dims0, nd.dims1, &od)) return false;
                TensorP fa = nd.needs[0] ? new_tensor(c, od) : nullptr;
                TensorP fb = nd.needs[1] ? new_tensor(c, od) : nullptr;
                if ((nd.needs[0] && !fa) || (nd.needs[1] && !fb)) return false;
                const std::vector<size_t> sa = broadcast_strides(nd.dims0, od), sb = broadcast_strides(nd.dims1, od);
                if (!k::binary_bcast_bwd(nd.op == Op::Mul ? 2 : 3, a, b, gp, fa ? fa->st->ptr : nullptr, fb ? fb->st->ptr : nullptr, od.data(),
                                         (int)od.size(), sa.data(), sb.data(), s))
                    return false;
                if (fa && !(gin[0] = reduce_to_shape(c, fa, nd.dims0))) return false;
                if (fb && !(gin[1] = reduce_to_shape(c, fb, nd.dims1))) return false;
                return true;
            }
            TensorP ga = nd.needs[0] ? new_tensor(c, go->dims) : nullptr;
            TensorP gb = nd.needs[1] ? new_tensor(c, go->dims) : nullptr;
            if ((nd.needs[0] && !ga) || (nd.needs[1] && !gb)) return false;
            bool ok = nd.op == Op::Mul ? k::mul_bwd(a, b, gp, ga ? ga->st->ptr : nullptr, gb ? gb->st->ptr : nullptr, go->size, s)
                                       : k::div_bwd(a, b, gp, ga ? ga->st->ptr : nullptr, gb ? gb->st->ptr : nullptr, go->size, s);
            if (!ok) return false;
            gin[0] = ga; gin[1] = gb;
            return true;
        }
        case Op::Relu: {
            // grad_fn/ops/relu.rs:4-16 with the saved OUTPUT as the mask: relu(x) > 0 <=> x > 0.
            if (!nd.needs[0]) return true;
            if (!nd.s0.check("relu")) return false;
            if (fusion_enabled() && go->pending && !go->pending->bias && !go->pending->relu && !go->pending->mask && go.use_count() == 1) {
                go->pending->mask = nd.s0.t;   // fold the mask into the GEMM that produces this gradient
                gin[0] = go;
                return true;
            }
            const float *y = rptr(nd.s0.t), *gp = rptr(go);
            if (!y || !gp) return false;
            TensorP r = new_tensor(c, go->dims);
            if (!r) return false;
            // When the ReLU input came from a bias add, produce the bias gradient in the same pass.
            auto prod = g_graph.ops.find(nd.inputs[0]);
            if (fusion_enabled() && prod != g_graph.ops.end() && prod->second.op == Op::Add && g_graph.grads.find(nd.inputs[0]) == g_graph.grads.end()) {
                Node& add = prod->second;
                for (int i = 0; i < 2; ++i) {
                    const std::vector<size_t>& od = i == 0 ? add.dims0 : add.dims1;
                    const std::vector<size_t>& other = i == 0 ? add.dims1 : add.dims0;
                    size_t osz = 1; for (size_t x : od) osz *= x;
                    size_t rows, cols;
                    if (add.needs[i] && osz != go->size && is_suffix_broadcast(other, od, &rows, &cols) && cols > 1) {
                        TensorP db = new_tensor(c, {cols});
                        if (!db) return false;
                        size_t sc = k::colsum_scratch_elems(rows, cols);
                        float* scratch = c->alloc.alloc(sc * sizeof(float));
                        if (!scratch) return false;
                        bool ok = k::relu_bwd_colsum(y, gp, r->st->ptr, db->st->ptr, rows, cols, scratch, s);
                        c->alloc.free(scratch);
                        if (!ok) return false;
                        g_graph.bias_grad_ready[nd.inputs[0]] = db;
                        gin[0] = r;
                        return true;
                    }
                }
            }
            if (!k::relu_bwd(y, gp, r->st->ptr, r->size, s)) return false;
            gin[0] = r;
            return true;
        }
        case Op::MatMul: {
            // grad_fn/ops/matmul.rs:68-80: dA = go . B^T, dB = A^T . go; the transposes are operand
            // layouts of the GEMM, not copies.
            if (!nd.s0.check("matmul") || !nd.s1.check("matmul")) return false;
            if (nd.dims0.size() > 2 || nd.dims1.size() > 2) {
                // batched (matmul.rs, the general branch): dA = go . B^T and dB = A^T . go per batch entry, then summed
                // back over the axes the operand was broadcast along
                const std::vector<size_t>&da = nd.dims0, &db = nd.dims1;
                const size_t m = da[da.size() - 2], kk = da.back(), n = db.back();
                const std::vector<size_t> a_batch(da.begin(), da.end() - 2), b_batch(db.begin(), db.end() - 2);
                BatchGeom g;
                if (!broadcast_batch(a_batch, b_batch, &g)) return false;
                if (!materialize(go)) return false;
                const std::vector<size_t> no_batch;
                for (int side = 0; side < 2; ++side) {
                    if (!nd.needs[side]) continue;
                    std::vector<size_t> raw_dims = g.batch;
                    raw_dims.push_back(side == 0 ? m : kk);
                    raw_dims.push_back(side == 0 ? kk : n);
                    TensorP raw = new_tensor(c, raw_dims);
                    if (!raw) return false;
                    // the upstream gradient has one [m, n] matrix per batch entry whatever squeezing the forward did
                    bool ok = side == 0 ? batched_gemm(c, go, g.batch, false, nd.s1.t, b_batch, true, raw->st->ptr, g, m, kk, n)
                                        : batched_gemm(c, nd.s0.t, a_batch, true, go, g.batch, false, raw->st->ptr, g, kk, n, m);
                    if (!ok) return false;
                    gin[side] = reduce_to_shape(c, raw, side == 0 ? da : db);
                    if (!gin[side]) return false;
                }
                return true;
            }
            const size_t m = nd.dims0.size() == 2 ? nd.dims0[0] : 1, kk = nd.dims0.back();
            const size_t n = nd.dims1.size() == 2 ? nd.dims1[1] : 1;
            const bool mats = nd.dims0.size() == 2 && nd.dims1.size() == 2;   // saved transposed views stay flags here too
            if (nd.needs[0]) {
                auto t = std::make_shared<TensorImpl>(nd.dims0);
                bool tb = true;
                TensorP ob = mats ? gemm_operand(nd.s1.t, &tb) : nd.s1.t;
                t->pending.reset(new PendingGemm{go, ob, false, tb, m, kk, n, nullptr, nullptr, false});
                register_pending(t);
                gin[0] = t;
            }
            if (nd.needs[1]) {
                auto t = std::make_shared<TensorImpl>(nd.dims1);
                bool ta = true;
                TensorP oa = mats ? gemm_operand(nd.s0.t, &ta) : nd.s0.t;
                t->pending.reset(new PendingGemm{oa, go, ta, false, kk, n, m, nullptr, nullptr, false});
                register_pending(t);
                gin[1] = t;
            }
            return true;
        }
        case Op::PowScalar: {
            if (!nd.needs[0]) return true;
            if (!nd.s0.check("pow_scalar")) return false;
            if (fusion_enabled() && go->pending_ew && go->pending_ew->kind == PendingEw::ScalarFill) {
                // The upstream gradient is scale * u in every element (it comes from mean() or sum()) and has not been
                // written out: go * (2 * x) = (scale * u) * (2 * x) in one pass, and when x itself is a deferred
                // difference a - b, straight from a and b.  Same operations, same order, same bits as the unfused chain.
                const float* up = rptr(go->pending_ew->a);
                const float scale = go->pending_ew->scale;
                TensorP r = up ? new_tensor(c, go->dims) : nullptr;
                if (!r) return false;
                const TensorP& x = nd.s0.t;
                if (x->pending_ew && x->pending_ew->kind == PendingEw::Diff) {
                    const float *pa = rptr(x->pending_ew->a), *pb = rptr(x->pending_ew->b);
                    // In TF32 mode, when the minuend came out of a matmul (directly or through its bias add) and only it
                    // wants a gradient, this gradient's consumers are that matmul's two backward GEMMs and the bias
                    // column sum: store it already rounded to TF32, as a deferred GEMM that produces a gradient does.
                    bool round_out = false;
                    // When the minuend is (matmul result) + (row bias) and only it wants a gradient, the same pass also
                    // yields the bias gradient (the column sums of this gradient), handed to the Add node's backward.
                    uint64_t add_id = 0;
                    size_t bias_rows = 0, bias_cols = 0;
                    auto sub = g_graph.ops.find(nd.inputs[0]);
                    if (sub != g_graph.ops.end() && sub->second.op == Op::Sub && sub->second.needs[0] && !sub->second.needs[1]) {
                        auto prod = g_graph.ops.find(sub->second.inputs[0]);
                        if (prod != g_graph.ops.end() && prod->second.op == Op::Add) {
                            // a row-bias add only: the other operand is the matmul result, the bias gets a column sum
                            if (prod->second.dims0 != prod->second.dims1) {
                                const int big = prod->second.dims0.size() >= prod->second.dims1.size() ? 0 : 1;
                                auto mm = g_graph.ops.find(prod->second.inputs[big]);
                                if (matmul_precision() == 1) round_out = mm != g_graph.ops.end() && mm->second.op == Op::MatMul;
                                const std::vector<size_t>& od = big == 0 ? prod->second.dims1 : prod->second.dims0;
                                const std::vector<size_t>& other = big == 0 ? prod->second.dims0 : prod->second.dims1;
                                size_t osz = 1; for (size_t v : od) osz *= v;
                                size_t rows, cols;
                                if (prod->second.needs[1 - big] && osz != r->size && is_suffix_broadcast(other, od, &rows, &cols) && cols > 1 &&
                                    rows * cols == r->size && g_graph.grads.find(sub->second.inputs[0]) == g_graph.grads.end()) {
                                    add_id = sub->second.inputs[0]; bias_rows = rows; bias_cols = cols;
                                }
                            }
                        } else if (matmul_precision() == 1) {
                            round_out = prod != g_graph.ops.end() && prod->second.op == Op::MatMul;
                        }
                    }
                    if (!pa || !pb) return false;
                    if (add_id) {
                        TensorP db = new_tensor(c, {bias_cols});
                        if (!db) return false;
                        float* scratch = c->alloc.alloc(k::colsum_scratch_elems(bias_rows, bias_cols) * sizeof(float));
                        if (!scratch) return false;
                        const bool ok = k::mse_grad_colsum(pa, pb, up, scale, r->st->ptr, db->st->ptr, bias_rows, bias_cols, round_out, scratch, s);
                        c->alloc.free(scratch);   // reused only by later work on the same stream
                        if (!ok) return false;
                        g_graph.bias_grad_ready[add_id] = db;
                    } else if (!k::mse_grad(pa, pb, up, scale, r->st->ptr, r->size, round_out, s)) {
                        return false;
                    }
                    r->st->tf32_clean = round_out;
                } else {
                    const float* px = rptr(x);
                    if (!px || !k::square_bwd_scalar(px, up, scale, r->st->ptr, r->size, s)) return false;
                }
                gin[0] = r;
                return true;
            }
            const float *x = rptr(nd.s0.t), *gp = rptr(go);
            TensorP r = (x && gp) ? new_tensor(c, go->dims) : nullptr;
            if (!r || !k::square_bwd(x, gp, r->st->ptr, r->size, s)) return false;
            gin[0] = r;
            return true;
        }
        case Op::Unary: {
            // grad_fn/ops/{exp,log,sqrt,tanh,sigmoid,leaky_relu,pow}.rs and the scalar branches of add/sub/mul/div.rs
            if (!nd.needs[0]) return true;
            if (nd.code == TS_UNARY_ADD_SCALAR || nd.code == TS_UNARY_SUB_SCALAR) { gin[0] = go; return true; }
            const float* saved = nullptr;
            if (nd.s0.t) {
                if (!nd.s0.check("a unary op")) return false;
                saved = rptr(nd.s0.t);
                if (!saved) return false;
            }
            const float* gp = rptr(go);
            TensorP r = gp ? new_tensor(c, go->dims) : nullptr;
            if (!r || !k::unary_bwd(nd.code, saved, gp, r->st->ptr, r->size, nd.scalar, s)) return false;
            gin[0] = r;
            return true;
        }
        case Op::ReduceDims: {
            // grad_fn/reductions/{sum,mean,max,min,norm,var,std}.rs, the *_dims variants (the whole-tensor variants are
            // the same formulas with every axis reduced)
            if (!nd.needs[0]) return true;
            const int rank = (int)nd.dims0.size();
            std::vector<unsigned char> red((size_t)rank);
            size_t factor = 1;
            for (int i = 0; i < rank; ++i) { red[i] = (unsigned char)nd.perm[i]; if (red[i]) factor *= nd.dims0[i]; }
            const float* gp = rptr(go);
            TensorP r = gp ? new_tensor(c, nd.dims0) : nullptr;
            if (!r) return false;
            const bool scalar_go = go->size == 1;
            const float inv = factor > 0 ? 1.0f / (float)factor : 0.0f;
            const float *x = nullptr, *a1 = nullptr, *a2 = nullptr;
            TensorP counts;
            int mode = 0;
            float scale = 1.0f;
            switch (nd.code) {
                case TS_REDUCE_SUM: mode = 0; break;
                case TS_REDUCE_MEAN: mode = 1; scale = inv; break;
                case TS_REDUCE_MAX:
                case TS_REDUCE_MIN: {
                    if (!nd.s0.check("max/min") || !nd.s1.check("max/min")) return false;
                    x = rptr(nd.s0.t); a1 = rptr(nd.s1.t);
                    counts = (x && a1) ? new_tensor(c, nd.s1.t->dims) : nullptr;
                    float* scratch = counts ? c->alloc.alloc(k::reduce_dims_scratch_elems() * sizeof(float)) : nullptr;
                    if (!scratch) return false;
                    bool ok = k::reduce_dims(5, x, a1, counts->st->ptr, nd.dims0.data(), rank, red.data(), scratch, s);
                    c->alloc.free(scratch);
                    if (!ok) return false;
                    a2 = counts->st->ptr;
                    mode = 2;
                    break;
                }
                case TS_REDUCE_NORM:
                    if (!nd.s0.check("norm") || !nd.s1.check("norm")) return false;
                    x = rptr(nd.s0.t); a1 = rptr(nd.s1.t); mode = 3;
                    break;
                case TS_REDUCE_VAR:
                    if (!nd.s0.check("var")) return false;
                    x = rptr(nd.s0.t); a1 = rptr(nd.s2.t); mode = 4;
                    scale = factor > 0 ? 2.0f / (float)factor : 0.0f;
                    break;
                case TS_REDUCE_STD:
                    if (!nd.s0.check("std") || !nd.s1.check("std")) return false;
                    x = rptr(nd.s0.t); a1 = rptr(nd.s2.t); a2 = rptr(nd.s1.t); mode = 5; scale = inv;
                    break;
                default: set_error("backward: unknown reduction"); return false;
            }
            if (mode >= 2 && (!x || !a1)) return false;
            if (!k::reduce_dims_backward(mode, x, a1, a2, gp, r->st->ptr, nd.dims0.data(), rank, red.data(), scalar_go, scale, s)) return false;
            gin[0] = r;
            return true;
        }
        case Op::Cat: {
            // grad_fn/transforms/cat.rs: each input gets its slab of the gradient (nd.dims0 = output dims, nd.perm = lengths along the axis)
            const float* gp = rptr(go);
            if (!gp) return false;
            const int dim = nd.code;
            size_t outer = 1, inner = 1, prefix = 0;
            for (int d = 0; d < dim; ++d) outer *= nd.dims0[d];
            for (size_t d = dim + 1; d < nd.dims0.size(); ++d) inner *= nd.dims0[d];
            const size_t total = nd.dims0[dim];
            for (size_t i = 0; i < nd.inputs.size(); ++i) {
                const size_t len = (size_t)nd.perm[i];
                if (nd.needs[i]) {
                    std::vector<size_t> gd = nd.dims0;
                    gd[dim] = len;
                    TensorP r = new_tensor(c, gd);
                    if (!r || !copy_slab(r->st->ptr, len * inner, 0, gp, total * inner, prefix * inner, len * inner, outer, s)) return false;
                    gin[i] = r;
                }
                prefix += len;
            }
            return true;
        }
        case Op::Split: {
            // grad_fn/transforms/split.rs: zeros of the input's shape with the gradient added into its slab
            if (!nd.needs[0]) return true;
            const float* gp = rptr(go);
            TensorP r = gp ? new_tensor(c, nd.dims0) : nullptr;
            if (!r || !k::fill(r->st->ptr, 0.0f, r->size, s)) return false;
            const int dim = nd.code;
            const size_t start = (size_t)nd.perm[0], len = (size_t)nd.perm[1];
            size_t outer = 1, inner = 1;
            for (int d = 0; d < dim; ++d) outer *= nd.dims0[d];
            for (size_t d = dim + 1; d < nd.dims0.size(); ++d) inner *= nd.dims0[d];
            if (!copy_slab(r->st->ptr, nd.dims0[dim] * inner, start * inner, gp, len * inner, 0, len * inner, outer, s)) return false;
            gin[0] = r;
            return true;
        }
        case Op::Reshape: {
            // grad_fn/transforms/reshape.rs: the gradient with the input's shape (same data); Contiguous is the same
            if (!nd.needs[0]) return true;
            gin[0] = reshaped_alias(go, nd.dims0);
            return gin[0] != nullptr;
        }
        case Op::Permute: {
            // grad_fn/transforms/permute.rs, transpose.rs: the gradient through the inverse permutation
            if (!nd.needs[0]) return true;
            const int rank = (int)nd.perm.size();
            std::vector<int> inv(rank);
            std::vector<size_t> go_dims(rank);
            for (int i = 0; i < rank; ++i) { inv[nd.perm[i]] = i; go_dims[i] = nd.dims0[nd.perm[i]]; }
            const float* gp = rptr(go);
            TensorP r = gp ? new_tensor(c, nd.dims0) : nullptr;
            if (!r || !k::permute(gp, r->st->ptr, go_dims.data(), inv.data(), rank, s)) return false;
            gin[0] = r;
            return true;
        }
        case Op::Softmax: {
            // grad_fn/ops/softmax.rs:4-35
            if (!nd.needs[0]) return true;
            if (!nd.s0.check("softmax")) return false;
            const float *y = rptr(nd.s0.t), *gp = rptr(go);
            TensorP r = (y && gp) ? new_tensor(c, nd.dims0) : nullptr;
            if (!r) return false;
            size_t outer = 1, inner = 1;
            for (int d = 0; d < nd.code; ++d) outer *= nd.dims0[d];
            for (size_t d = nd.code + 1; d < nd.dims0.size(); ++d) inner *= nd.dims0[d];
            if (!k::softmax_bwd(y, gp, r->st->ptr, outer, nd.dims0[nd.code], inner, s)) return false;
            gin[0] = r;
            return true;
        }
        case Op::ReduceSum:
        case Op::ReduceMean: {
            // grad_fn/reductions/sum.rs:4-16, mean.rs:4-30: fill with upstream, or (1/numel as f32) * upstream.
            if (!nd.needs[0]) return true;
            size_t n_in = 1;
            for (size_t d : nd.dims0) n_in *= d;
            float scale = 1.0f;
            if (nd.op == Op::ReduceMean) scale = n_in > 0 ? 1.0f / (float)n_in : 0.0f;
            if (fusion_enabled() && n_in > 0) {
                // deferred: whoever consumes this gradient either folds the constant in or has it written out
                auto r = std::make_shared<TensorImpl>(nd.dims0);
                r->pending_ew.reset(new PendingEw{PendingEw::ScalarFill, go, nullptr, scale});
                register_pending(r);
                gin[0] = r;
                return true;
            }
            const float* gp = rptr(go);
            TensorP r = gp ? new_tensor(c, nd.dims0) : nullptr;
            if (!r) return false;
            if (!k::fill_from_scalar(r->st->ptr, gp, scale, r->size, s)) return false;
            gin[0] = r;
            return true;
        }
    }
    set_error("backward: unknown op");
    return false;
}

// A leaf's gradient is final: launch the GEMM that produces it and, under data parallelism,
// start its cross-rank sum on the communication stream while the rest of backward proceeds.
static bool finalize_leaf(DeviceCtx* c, uint64_t id, std::unordered_set<uint64_t>& reduced) {
    TensorP lg = g_graph.grads[id];
    if (!rptr(lg)) return false;
    if (!g_dp.comm || !g_dp.params.count(id) || reduced.count(id)) return true;
    // The sum runs in place on the communication stream, so the buffer must belong to this gradient alone.  It does
    // not when another gradient shares the storage, or the tensor object itself (Add hands the same object to both
    // operands of equal shape, Sub hands the upstream gradient on, a deferred GEMM keeps its operands): two
    // references are this function's and the gradient map's, any more is somebody else.
    if (lg.use_count() > 2 || lg->st.use_count() > 1) {
        TensorP priv = new_tensor(c, lg->dims);
        if (!priv || !cuda_ok(cudaMemcpyAsync(priv->st->ptr, lg->st->ptr, lg->size * sizeof(float), cudaMemcpyDeviceToDevice, c->compute), "gradient copy")) return false;
        lg = priv;
    }
    reduced.insert(id);
    g_graph.grads.erase(id);   // from here on the gradient is the data-parallel state's (grad_lookup finds it there)
    return dp_reduce_leaf(c, id, lg);
}

static bool backward(const TensorP& root, const TensorP& grad_output) {
    DeviceCtx* c = ctx();
    if (!c) return false;
    // seed: gradtrack/engine.rs:964-978
    TensorP seed = grad_output;
    if (!seed && root->size == 1) {
        seed = std::make_shared<TensorImpl>(root->dims);
        seed->st = ones_scalar(c);
        if (!seed->st) return false;
    } else if (!seed) {
        seed = new_tensor(c, root->dims);
        if (!seed || !k::fill(seed->st->ptr, 1.0f, seed->size, c->compute)) return false;
    } else if (seed->size != root->size) {
        set_error("backward: grad_output has %zu elements, tensor has %zu", seed->size, root->size);
        return false;
    }
    if (!accumulate(c, root->id, seed)) return false;

    // reachable operations, processed by descending id
    std::vector<uint64_t> order, stack{root->id};
    std::unordered_set<uint64_t> seen{root->id};
    std::unordered_map<uint64_t, int> leaf_uses;   // leaf id -> number of reachable nodes that feed it a gradient
    while (!stack.empty()) {
        uint64_t id = stack.back();
        stack.pop_back();
        auto it = g_graph.ops.find(id);
        if (it == g_graph.ops.end()) continue;
        order.push_back(id);
        Node& nd = it->second;
        for (size_t i = 0; i < nd.inputs.size(); ++i) {
            if (!nd.needs[i]) continue;
            uint64_t in = nd.inputs[i];
            if (g_graph.ops.find(in) == g_graph.ops.end()) leaf_uses[in]++;
            if (seen.insert(in).second) stack.push_back(in);
        }
    }
    std::sort(order.begin(), order.end(), std::greater<uint64_t>());

    std::vector<TensorP> gin;
    std::unordered_set<uint64_t> reduced;
    for (uint64_t id : order) {
        auto git = g_graph.grads.find(id);
        if (git == g_graph.grads.end()) continue;
        TensorP go = git->second;
        if (id != root->id) g_graph.grads.erase(git);   // take_gradient, engine.rs:990-995; the root keeps its own
        else go = git->second;
        Node& nd = g_graph.ops[id];
        if (!apply_node(c, id, nd, go, gin)) return false;
        go.reset();
        for (size_t i = 0; i < gin.size(); ++i) {
            if (!gin[i]) continue;
            uint64_t in = nd.inputs[i];
            if (!accumulate(c, in, gin[i])) return false;
            gin[i].reset();
            auto lu = leaf_uses.find(in);
            if (lu != leaf_uses.end() && --lu->second == 0) {
                // the leaf's gradient is final: run its GEMM now and, under data parallelism,
                // start its all-reduce while the rest of backward proceeds
                if (!finalize_leaf(c, in, reduced)) return false;
            }
        }
    }
    // registered parameters whose gradient did not go through the counting above
    if (g_dp.comm)
        for (uint64_t id : g_dp.params)
            if (!reduced.count(id) && g_graph.grads.count(id) && !finalize_leaf(c, id, reduced)) return false;
    g_graph.bias_grad_ready.clear();
    // The all-reduces may still be running on the communication stream.  Whoever reads a gradient next waits for
    // them: grad_by_value() for all, Adam::step per parameter, so that early layers' sums overlap late layers' updates.
    return true;
}

// ------------------------------------------------------------------ Adam
struct AdamState {
    StorageP m, v, vmax;   // vmax only under amsgrad
    uint64_t step = 0;
    size_t n = 0;
    // Data parallel, sharded update: since the last gather only elements [lo, lo + cnt) of m, v (vmax) are current on this rank
    bool sharded = false;
    size_t lo = 0, cnt = 0;
};
struct ChunkCache {          // the kernel's chunk map for one list of tensor sizes, kept on the device
    std::vector<unsigned long long> sizes;
    float* dev = nullptr;
    int n = 0;
};

}  // namespace ts

struct ts_adam {
    float lr, beta1, beta2, eps, wd;
    bool amsgrad = false;
    uint64_t step_count = 0;
    std::unordered_map<uint64_t, ts::AdamState> states;
    std::vector<uint64_t> order;                 // insertion order, adam/mod.rs:201-206
    ts::ChunkCache whole, sliced;                // launch tables of the replicated and of the sharded update
    ts::DeviceCtx* c = nullptr;
};

namespace ts {
static thread_local std::unordered_set<ts_adam*> g_adams;   // live optimizers of this thread (their state may be sharded)

// After sharded updates only this rank's slice of the moments is current: all-gather them in place.  A collective:
// every rank must get here (reading optimizer state, a replicated update of the tensor, or ts_dp_finalize).
static bool gather_adam_state(DeviceCtx* c, AdamState& st) {
    if (!st.sharded) return true;
    NcclApi* nc = nccl_api();
    if (!nc || !g_dp.comm) {
        set_error("Adam state of a parameter is sharded across ranks but the communicator is gone; gather it before ts_dp_finalize");
        return false;
    }
    if (!dp_healthy() || !dp_comm_after_compute(c)) return false;
    for (const StorageP& sp : {st.m, st.v, st.vmax}) {
        if (!sp) continue;
        if (!dp_nccl_ok(nc, nc->AllGather(sp->ptr + st.lo, sp->ptr, st.cnt, ncclFloat32, g_dp.comm, c->comm), "ncclAllGather")) return false;
    }
    g_dp.comm_outstanding = true;
    st.sharded = false;
    return dp_join(c);
}
}  // namespace ts

using namespace ts;

// ====================================================================== C ABI: tensors
static std::vector<size_t> to_dims(const unsigned long long* dims, int rank) {
    std::vector<size_t> d;
    for (int i = 0; i < rank; ++i) d.push_back((size_t)dims[i]);
    if (d.empty()) d.push_back(1);
    return d;
}
static ts_tensor* wrap(const TensorP& t) {
    if (!t) return nullptr;
    ts_tensor* h = new ts_tensor();
    h->t = t;
    return h;
}

TS_API ts_tensor* ts_tensor_new(const unsigned long long* dims, int rank) {
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    if (rank < 0 || (rank > 0 && !dims)) { set_error("ts_tensor_new: bad shape"); return nullptr; }
    return wrap(new_tensor(c, to_dims(dims, rank)));
}
static ts_tensor* filled(const unsigned long long* dims, int rank, float v) {
    ts_tensor* h = ts_tensor_new(dims, rank);
    if (!h) return nullptr;
    if (!k::fill(h->t->st->ptr, v, h->t->size, h->t->st->c->compute)) { delete h; return nullptr; }
    return h;
}
TS_API ts_tensor* ts_tensor_zeros(const unsigned long long* dims, int rank) { return filled(dims, rank, 0.0f); }
TS_API ts_tensor* ts_tensor_ones(const unsigned long long* dims, int rank) { return filled(dims, rank, 1.0f); }

TS_API ts_tensor* ts_tensor_from_slice(const float* host, const unsigned long long* dims, int rank) {
    ts_tensor* h = ts_tensor_new(dims, rank);
    if (!h) return nullptr;
    if (h->t->size && !host) { set_error("ts_tensor_from_slice: null data"); delete h; return nullptr; }
    DeviceCtx* c = h->t->st->c;
    if (h->t->size) {
        if (!cuda_ok(cudaMemcpyAsync(h->t->st->ptr, host, h->t->size * sizeof(float), cudaMemcpyHostToDevice, c->compute), "upload") ||
            !cuda_ok(cudaStreamSynchronize(c->compute), "upload sync")) { delete h; return nullptr; }
    }
    return h;
}

// Tensor::randn (tensor/init/random.rs:231-236, 270-300, 473-616): a host-side generator, because the reference's
// stream is one serial xorshift64 chain (shifts 13, 7, 17 from state = seed) and a seeded tensor must reproduce it
// value for value.  next_f32 puts the low 23 bits under exponent field 126, i.e. in [0.5, 1); a sample is
// sqrt(-2 ln u1) * cos(2 pi u2) from two consecutive draws, NaN or infinity replaced by 0.  logf / sqrtf / cosf are
// the host libm's, which is what Rust's f32::ln / sqrt / cos call.
static inline uint64_t xorshift64(uint64_t& s) {
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    return s;
}
static inline float half_open_unit(uint64_t& s) {
    const uint32_t bits = (uint32_t)(xorshift64(s) & 0x7FFFFFu) | (126u << 23);
    float f;
    std::memcpy(&f, &bits, sizeof f);
    return f;
}
static void fill_randn_host(float* out, size_t n, uint64_t seed) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; ++i) {
        float u1 = half_open_unit(s);
        const float u2 = half_open_unit(s);
        if (u1 <= 0.0f) u1 = 1e-7f;                    // random.rs:598-604, unreachable for values in [0.5, 1)
        else if (u1 >= 1.0f) u1 = 1.0f - 1e-7f;
        const float z = sqrtf(-2.0f * logf(u1)) * cosf((2.0f * 3.14159265358979323846f) * u2);
        out[i] = (std::isnan(z) || std::isinf(z)) ? 0.0f : z;
    }
}
// The generator alone, into host memory: needs no device (fill_randn on a host buffer, random.rs:270-300).
TS_API bool ts_randn_host(float* out, unsigned long long n, unsigned long long seed) {
    if (!out && n) { set_error("ts_randn_host: null buffer"); return false; }
    fill_randn_host(out, (size_t)n, (uint64_t)seed);
    return true;
}
// has_seed == 0 mirrors randn(dims, None): the reference hashes the wall clock (random.rs:492-497); here the seed
// mixes the clock with a per-process counter.  Such tensors are not reproducible in either library.
TS_API ts_tensor* ts_tensor_randn(const unsigned long long* dims, int rank, unsigned long long seed, int has_seed) {
    ts_tensor* h = ts_tensor_new(dims, rank);
    if (!h) return nullptr;
    const size_t n = h->t->size;
    if (n == 0) return h;
    if (!has_seed) {
        static std::atomic<uint64_t> counter{0x9E3779B97F4A7C15ull};
        timespec tp;
        clock_gettime(CLOCK_REALTIME, &tp);
        seed = ((uint64_t)tp.tv_sec * 1000000000ull + (uint64_t)tp.tv_nsec) ^ counter.fetch_add(0x9E3779B97F4A7C15ull);
        if (seed == 0) seed = 1;
    }
    std::vector<float> host(n);
    fill_randn_host(host.data(), n, (uint64_t)seed);
    DeviceCtx* c = h->t->st->c;
    if (!cuda_ok(cudaMemcpyAsync(h->t->st->ptr, host.data(), n * sizeof(float), cudaMemcpyHostToDevice, c->compute), "randn upload") ||
        !cuda_ok(cudaStreamSynchronize(c->compute), "randn upload sync")) { delete h; return nullptr; }
    return h;
}

TS_API ts_tensor* ts_tensor_from_pinned_async(const float* host, const unsigned long long* dims, int rank) {
    ts_tensor* h = ts_tensor_new(dims, rank);
    if (!h) return nullptr;
    if (h->t->size && !host) { set_error("ts_tensor_from_pinned_async: null data"); delete h; return nullptr; }
    DeviceCtx* c = h->t->st->c;
    Storage* st = h->t->st.get();
    // The block may have been used by kernels already queued on the compute stream: the copy waits for those.
    cudaEvent_t before = nullptr;
    bool ok = cuda_ok(cudaEventCreateWithFlags(&before, cudaEventDisableTiming), "event") &&
              cuda_ok(cudaEventRecord(before, c->compute), "event record") &&
              cuda_ok(cudaStreamWaitEvent(c->copy, before, 0), "stream wait") &&
              cuda_ok(cudaMemcpyAsync(st->ptr, host, h->t->size * sizeof(float), cudaMemcpyHostToDevice, c->copy), "async upload") &&
              cuda_ok(cudaEventCreateWithFlags(&st->ready, cudaEventDisableTiming), "event") &&
              cuda_ok(cudaEventRecord(st->ready, c->copy), "event record");
    if (before) cudaEventDestroy(before);
    if (!ok) { delete h; return nullptr; }
    return h;
}

TS_API void ts_tensor_free(ts_tensor* t) { delete t; }

TS_API unsigned long long ts_tensor_id(const ts_tensor* t) { return t ? t->t->id : 0; }
TS_API int ts_tensor_rank(const ts_tensor* t) { return t ? (int)t->t->dims.size() : 0; }
TS_API unsigned long long ts_tensor_size(const ts_tensor* t) { return t ? t->t->size : 0; }
TS_API bool ts_tensor_dims(const ts_tensor* t, unsigned long long* out) {
    if (!t || !out) { set_error("ts_tensor_dims: null argument"); return false; }
    for (size_t i = 0; i < t->t->dims.size(); ++i) out[i] = t->t->dims[i];
    return true;
}
TS_API bool ts_tensor_requires_grad(const ts_tensor* t) { return t && t->t->requires_grad; }
TS_API bool ts_tensor_is_contiguous(const ts_tensor* t) { return t && !is_view(t->t); }
TS_API bool ts_tensor_set_requires_grad(ts_tensor* t, bool rg) {
    if (!t) { set_error("ts_tensor_set_requires_grad: null tensor"); return false; }
    t->t->requires_grad = rg;
    return true;
}
// Before a write into t's storage in place: a tensor that shares read-only contents gets its own copy of them.
static bool make_writable(const TensorP& t) {
    if (!t->st || !t->st->constant) return true;
    StorageP priv = new_storage(t->st->c, t->st->n);
    if (!priv) return false;
    TS_CHECK(cudaMemcpyAsync(priv->ptr, t->st->ptr, (t->st->n ? t->st->n : 1) * sizeof(float), cudaMemcpyDeviceToDevice, t->st->c->compute));
    t->st = priv;
    return true;
}
TS_API float* ts_tensor_data_ptr(ts_tensor* t) {
    if (!t) { set_error("ts_tensor_data_ptr: null tensor"); return nullptr; }
    if (!make_writable(t->t)) return nullptr;   // the caller may write through the pointer
    return const_cast<float*>(rptr(t->t));
}
TS_API bool ts_tensor_to_host(ts_tensor* t, float* out) {
    if (!t || (!out && t->t->size)) { set_error("ts_tensor_to_host: null argument"); return false; }
    const float* p = rptr(t->t);
    if (!p) return false;
    DeviceCtx* c = t->t->st->c;
    if (t->t->size) TS_CHECK(cudaMemcpyAsync(out, p, t->t->size * sizeof(float), cudaMemcpyDeviceToHost, c->compute));
    return ts_sync_stream(nullptr);
}
TS_API bool ts_tensor_copy_from_host(ts_tensor* t, const float* host) {
    if (!t || (!host && t->t->size)) { set_error("ts_tensor_copy_from_host: null argument"); return false; }
    if (!make_writable(t->t)) return false;
    if (is_view(t->t)) {
        // a write through a view lands in the shared storage: upload in the view's order, then scatter through the inverse permutation
        const TensorP& v = t->t;
        if (!materialize(v) || !flush_pending({v->st.get()})) return false;
        Storage* st = v->st.get();
        if (st->ready) { cudaStreamWaitEvent(st->c->compute, st->ready, 0); cudaEventDestroy(st->ready); st->ready = nullptr; }
        const int rank = (int)v->view_perm.size();
        std::vector<int> inv((size_t)rank);
        for (int i = 0; i < rank; ++i) inv[v->view_perm[i]] = i;
        float* tmp = st->c->alloc.alloc((v->size ? v->size : 1) * sizeof(float));
        if (!tmp) return false;
        bool ok = cuda_ok(cudaMemcpyAsync(tmp, host, v->size * sizeof(float), cudaMemcpyHostToDevice, st->c->compute), "upload") &&
                  (v->size == 0 || k::permute(tmp, st->ptr, v->dims.data(), inv.data(), rank, st->c->compute)) &&
                  cuda_ok(cudaStreamSynchronize(st->c->compute), "upload sync");
        st->c->alloc.free(tmp);
        if (!ok) return false;
        st->version++;
        st->tf32_clean = false;
        return true;
    }
    if (!rptr(t->t) || !flush_pending({t->t->st.get()})) return false;
    Storage* st = t->t->st.get();
    TS_CHECK(cudaMemcpyAsync(st->ptr, host, t->t->size * sizeof(float), cudaMemcpyHostToDevice, st->c->compute));
    TS_CHECK(cudaStreamSynchronize(st->c->compute));
    st->version++;
    st->tf32_clean = false;
    return true;
}
TS_API bool ts_tensor_fill(ts_tensor* t, float v) {
    if (!t) { set_error("ts_tensor_fill: null tensor"); return false; }
    if (!make_writable(t->t)) return false;
    // (a view covers every element of the storage it shares exactly once, so filling it fills the storage)
    if (!rptr(is_view(t->t) ? view_base(t->t) : t->t) || !flush_pending({t->t->st.get()})) return false;
    Storage* st = t->t->st.get();
    if (!k::fill(st->ptr, v, t->t->size, st->c->compute)) return false;
    st->version++;
    st->tf32_clean = false;
    return true;
}

// ====================================================================== C ABI: ops
static void record(const TensorP& out, Node&& nd) {
    out->requires_grad = true;
    g_graph.ops[out->id] = std::move(nd);
}

static ts_tensor* binary_op(ts_tensor* ha, ts_tensor* hb, int op, const char* name) {
    if (!ha || !hb) { set_error("%s: null tensor", name); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP a = ha->t, b = hb->t;
    TensorP out;
    bool track = grad_on() && (a->requires_grad || b->requires_grad);
    if (same_dims(a->dims, b->dims) && op == 1 && fusion_enabled() && a->size > 0) {
        // the difference is deferred: squared and averaged (the MSE spelling) it never has to be written out
        out = std::make_shared<TensorImpl>(a->dims);
        out->pending_ew.reset(new PendingEw{PendingEw::Diff, a, b});
        register_pending(out);
    } else if (same_dims(a->dims, b->dims)) {
        const float *pa = rptr(a), *pb = rptr(b);
        out = (pa && pb) ? new_tensor(c, a->dims) : nullptr;
        if (!out || !k::binary(op, pa, pb, out->st->ptr, out->size, c->compute)) return nullptr;
    } else {
        // NumPy-style broadcasting (add.rs:107-146 -> broadcasting.rs:299-333), read through strides instead of
        // the reference's materialised operands
        std::vector<size_t> od;
        if (!broadcast_shape(a->dims, b->dims, &od)) return nullptr;
        TensorP big = a->size >= b->size ? a : b, small = a->size >= b->size ? b : a;
        size_t rows = 0, cols = 0;
        const bool bias_like = op == 0 && od == big->dims && is_suffix_broadcast(big->dims, small->dims, &rows, &cols);
        if (bias_like && fusion_enabled() && big->pending && !big->pending->bias && !big->pending->relu && !big->pending->mask &&
            cols == big->pending->n && cols > 1) {
            // deferred GEMM + row bias: fold the add into the GEMM epilogue
            out = std::make_shared<TensorImpl>(big->dims);
            out->pending.reset(new PendingGemm(*big->pending));
            out->pending->bias = small;
            register_pending(out);
        } else if (bias_like) {
            // the smaller operand matches the trailing dimensions of the larger one
            const float *pb = rptr(big), *ps = rptr(small);
            out = (pb && ps) ? new_tensor(c, big->dims) : nullptr;
            if (!out) return nullptr;
            bool ok = cols == 1 ? k::add_scalar_bcast(pb, ps, out->st->ptr, out->size, c->compute)
                                : k::bias_act(pb, ps, out->st->ptr, rows, cols, false, c->compute);
            if (!ok) return nullptr;
        } else {
            const float *pa = rptr(a), *pb = rptr(b);
            out = (pa && pb) ? new_tensor(c, od) : nullptr;
            if (!out) return nullptr;
            const std::vector<size_t> sa = broadcast_strides(a->dims, od), sb = broadcast_strides(b->dims, od);
            if (!k::binary_bcast(op, pa, pb, out->st->ptr, od.data(), (int)od.size(), sa.data(), sb.data(), c->compute)) return nullptr;
        }
    }
    if (track) {
        Node nd;
        nd.op = op == 0 ? Op::Add : op == 1 ? Op::Sub : op == 2 ? Op::Mul : Op::Div;
        nd.inputs = {a->id, b->id};
        nd.needs = {a->requires_grad, b->requires_grad};
        nd.dims0 = a->dims; nd.dims1 = b->dims;
        if (op >= 2) { nd.s0.set(a); nd.s1.set(b); }
        record(out, std::move(nd));
    }
    return wrap(out);
}
TS_API ts_tensor* ts_tensor_add_tensor(ts_tensor* a, ts_tensor* b) { return binary_op(a, b, 0, "add_tensor"); }
TS_API ts_tensor* ts_tensor_sub_tensor(ts_tensor* a, ts_tensor* b) { return binary_op(a, b, 1, "sub_tensor"); }
TS_API ts_tensor* ts_tensor_mul_tensor(ts_tensor* a, ts_tensor* b) { return binary_op(a, b, 2, "mul_tensor"); }
TS_API ts_tensor* ts_tensor_div_tensor(ts_tensor* a, ts_tensor* b) { return binary_op(a, b, 3, "div_tensor"); }

TS_API ts_tensor* ts_tensor_matmul(ts_tensor* ha, ts_tensor* hb) {
    if (!ha || !hb) { set_error("matmul: null tensor"); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP a = ha->t, b = hb->t;
    const size_t ra = a->dims.size(), rb = b->dims.size();
    if (ra < 1 || rb < 1) { set_error("matmul: operands need at least one dimension"); return nullptr; }
    if (ra > 2 || rb > 2) {
        // N-D . N-D (matmul/mod.rs:634-760): batch axes broadcast, one GEMM per batch entry, launched now
        if (ra < 2 || rb < 2) { set_error("Batched matmul requires at least 2D tensors"); return nullptr; }
        const size_t m = a->dims[ra - 2], ka = a->dims[ra - 1], kb = b->dims[rb - 2], n = b->dims[rb - 1];
        if (ka != kb) { set_error("Inner dimensions must match for batched matmul: %zu vs %zu", ka, kb); return nullptr; }
        const std::vector<size_t> a_batch(a->dims.begin(), a->dims.end() - 2), b_batch(b->dims.begin(), b->dims.end() - 2);
        BatchGeom g;
        if (!broadcast_batch(a_batch, b_batch, &g)) return nullptr;
        std::vector<size_t> od = g.batch;
        od.push_back(m);
        od.push_back(n);
        TensorP out = new_tensor(c, od);
        if (!out) return nullptr;
        if (out->size && !batched_gemm(c, a, a_batch, false, b, b_batch, false, out->st->ptr, g, m, n, ka)) return nullptr;
        // mod.rs:752-756: with a 2-D operand, a leading batch axis of extent 1 is squeezed away
        if ((ra == 2 || rb == 2) && od.size() > 2 && od[0] == 1) {
            out = reshaped_alias(out, std::vector<size_t>(od.begin() + 1, od.end()));
            if (!out) return nullptr;
        }
        if (grad_on() && (a->requires_grad || b->requires_grad)) {
            Node nd;
            nd.op = Op::MatMul;
            nd.inputs = {a->id, b->id};
            nd.needs = {a->requires_grad, b->requires_grad};
            nd.dims0 = a->dims; nd.dims1 = b->dims;
            nd.s0.set(a); nd.s1.set(b);
            record(out, std::move(nd));
        }
        return wrap(out);
    }
    // rank dispatch: matmul/mod.rs:263-310
    const size_t m = ra == 2 ? a->dims[0] : 1, ka = a->dims.back();
    const size_t kb = b->dims[0], n = rb == 2 ? b->dims[1] : 1;
    if (ka != kb) { set_error("matmul: inner dimensions differ (%zu vs %zu)", ka, kb); return nullptr; }
    std::vector<size_t> od;
    if (ra == 2) od.push_back(m);
    if (rb == 2) od.push_back(n);   // 1-D . 1-D gives a rank-0 tensor with one element (matmul/mod.rs:88-98)
    auto out = std::make_shared<TensorImpl>(od);
    bool ta = false, tb = false;
    TensorP oa = ra == 2 ? gemm_operand(a, &ta) : a, ob = rb == 2 ? gemm_operand(b, &tb) : b;   // transposed views: flags, not copies
    out->pending.reset(new PendingGemm{oa, ob, ta, tb, m, n, ka, nullptr, nullptr, false});
    if (fusion_enabled()) register_pending(out);
    else if (!materialize(out)) return nullptr;
    if (grad_on() && (a->requires_grad || b->requires_grad)) {
        Node nd;
        nd.op = Op::MatMul;
        nd.inputs = {a->id, b->id};
        nd.needs = {a->requires_grad, b->requires_grad};
        nd.dims0 = a->dims; nd.dims1 = b->dims;
        nd.s0.set(a); nd.s1.set(b);
        record(out, std::move(nd));
    }
    return wrap(out);
}

TS_API ts_tensor* ts_tensor_relu(ts_tensor* hx) {
    if (!hx) { set_error("relu: null tensor"); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP x = hx->t, out;
    if (fusion_enabled() && x->pending && !x->pending->relu && !x->pending->mask) {
        out = std::make_shared<TensorImpl>(x->dims);
        out->pending.reset(new PendingGemm(*x->pending));
        out->pending->relu = true;
        register_pending(out);
    } else {
        const float* px = rptr(x);
        out = px ? new_tensor(c, x->dims) : nullptr;
        if (!out || !k::relu(px, out->st->ptr, out->size, c->compute)) return nullptr;
    }
    if (grad_on() && x->requires_grad) {
        Node nd;
        nd.op = Op::Relu;
        nd.inputs = {x->id};
        nd.needs = {true};
        nd.dims0 = x->dims;
        nd.s0.set(out);   // the output doubles as the mask
        record(out, std::move(nd));
    }
    return wrap(out);
}

// ---- unary and scalar ops: one kernel forward, one backward, the tensor the reference's GradFn saves kept by reference
static std::atomic<int> g_domain_checks{1};
TS_API void ts_set_domain_checks(int at_the_call) { g_domain_checks.store(at_the_call ? 1 : 0); }
TS_API int ts_get_domain_checks(void) { return g_domain_checks.load(); }

static ts_tensor* unary_op(ts_tensor* hx, int code, float param, const char* name) {
    if (!hx) { set_error("%s: null tensor", name); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP x = hx->t;
    const float* px = rptr(x);
    TensorP out = px ? new_tensor(c, x->dims) : nullptr;
    if (!out || !k::unary(code, px, out->st->ptr, out->size, param, c->compute)) return nullptr;
    if (code == TS_UNARY_LOG && g_domain_checks.load() && out->size) {
        // log.rs:68-107 panics at the call; here the kernel raises a device word, read back now
        if (!ts_sync_stream(nullptr)) return nullptr;
    }
    if (grad_on() && x->requires_grad) {
        Node nd;
        nd.op = Op::Unary;
        nd.code = code;
        nd.scalar = param;
        nd.inputs = {x->id};
        nd.needs = {true};
        nd.dims0 = x->dims;
        switch (code) {
            case TS_UNARY_EXP: case TS_UNARY_SQRT: case TS_UNARY_TANH: case TS_UNARY_SIGMOID: nd.s0.set(out); break;
            case TS_UNARY_LOG: case TS_UNARY_LEAKY_RELU: case TS_UNARY_POW_SCALAR: nd.s0.set(x); break;
            default: break;
        }
        record(out, std::move(nd));
    }
    return wrap(out);
}
TS_API ts_tensor* ts_tensor_exp(ts_tensor* x) { return unary_op(x, TS_UNARY_EXP, 0.0f, "exp"); }
TS_API ts_tensor* ts_tensor_log(ts_tensor* x) { return unary_op(x, TS_UNARY_LOG, 0.0f, "log"); }
TS_API ts_tensor* ts_tensor_sqrt(ts_tensor* x) { return unary_op(x, TS_UNARY_SQRT, 0.0f, "sqrt"); }
TS_API ts_tensor* ts_tensor_tanh(ts_tensor* x) { return unary_op(x, TS_UNARY_TANH, 0.0f, "tanh"); }
TS_API ts_tensor* ts_tensor_sigmoid(ts_tensor* x) { return unary_op(x, TS_UNARY_SIGMOID, 0.0f, "sigmoid"); }
TS_API ts_tensor* ts_tensor_leaky_relu(ts_tensor* x, float negative_slope) { return unary_op(x, TS_UNARY_LEAKY_RELU, negative_slope, "leaky_relu"); }
TS_API ts_tensor* ts_tensor_add_scalar(ts_tensor* x, float v) { return unary_op(x, TS_UNARY_ADD_SCALAR, v, "add_scalar"); }
TS_API ts_tensor* ts_tensor_sub_scalar(ts_tensor* x, float v) { return unary_op(x, TS_UNARY_SUB_SCALAR, v, "sub_scalar"); }
TS_API ts_tensor* ts_tensor_mul_scalar(ts_tensor* x, float v) { return unary_op(x, TS_UNARY_MUL_SCALAR, v, "mul_scalar"); }
TS_API ts_tensor* ts_tensor_div_scalar(ts_tensor* x, float v) { return unary_op(x, TS_UNARY_DIV_SCALAR, v, "div_scalar"); }

TS_API ts_tensor* ts_tensor_softmax(ts_tensor* hx, unsigned long long dim) {
    if (!hx) { set_error("softmax: null tensor"); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP x = hx->t;
    if (dim >= x->dims.size()) {   // softmax.rs:112-117
        set_error("softmax dim %llu out of bounds for rank %zu", dim, x->dims.size());
        return nullptr;
    }
    size_t outer = 1, inner = 1;
    for (size_t d = 0; d < dim; ++d) outer *= x->dims[d];
    for (size_t d = dim + 1; d < x->dims.size(); ++d) inner *= x->dims[d];
    const float* px = rptr(x);
    TensorP out = px ? new_tensor(c, x->dims) : nullptr;
    if (!out || !k::softmax(px, out->st->ptr, outer, x->dims[dim], inner, c->compute)) return nullptr;
    if (grad_on() && x->requires_grad) {
        Node nd;
        nd.op = Op::Softmax;
        nd.code = (int)dim;
        nd.inputs = {x->id};
        nd.needs = {true};
        nd.dims0 = x->dims;
        nd.s0.set(out);
        record(out, std::move(nd));
    }
    return wrap(out);
}

// ---- shape and layout ops.  Tensors here are always contiguous: reshape shares the storage (as the reference's
// view does), permute / transpose produce the permuted copy at once (the reference returns a strided view and
// copies in contiguous()).
TS_API ts_tensor* ts_tensor_reshape(ts_tensor* hx, const long long* new_shape, int rank) {
    if (!hx || (rank > 0 && !new_shape)) { set_error("reshape: null argument"); return nullptr; }
    TensorP x = hx->t;
    // transform/reshape.rs:185-215: one -1 is inferred, everything else must be positive
    std::vector<size_t> dims((size_t)rank);
    int infer = -1;
    size_t known = 1;
    for (int i = 0; i < rank; ++i) {
        if (new_shape[i] == -1) {
            if (infer >= 0) { set_error("Only one dimension can be -1 for automatic inference"); return nullptr; }
            infer = i;
        } else if (new_shape[i] <= 0) {
            set_error("Dimension sizes must be positive, got %lld", new_shape[i]);
            return nullptr;
        } else {
            dims[i] = (size_t)new_shape[i];
            known *= dims[i];
        }
    }
    if (infer >= 0) {
        if (known == 0 || x->size % known != 0) {
            set_error("Cannot infer dimension size: total size %zu not divisible by known size %zu", x->size, known);
            return nullptr;
        }
        dims[infer] = x->size / known;
    }
    if (dims.empty()) dims.push_back(1);
    size_t n = 1;
    for (size_t d : dims) n *= d;
    if (n != x->size) { set_error("Cannot reshape tensor of size %zu to a shape of size %zu", x->size, n); return nullptr; }   // reshape.rs:142-150
    if (!materialize(x)) return nullptr;
    auto out = std::make_shared<TensorImpl>(dims);
    if (is_view(x)) {   // reshape.rs: a non-contiguous tensor is made contiguous first, so the result does not alias it
        if (!rptr(x)) return nullptr;
        out->st = x->contig;
    } else {
        out->st = x->st;
    }
    if (x->requires_grad) {
        Node nd;
        nd.op = Op::Reshape;
        nd.inputs = {x->id};
        nd.needs = {true};
        nd.dims0 = x->dims;
        record(out, std::move(nd));
    }
    return wrap(out);
}

// transpose / t / permute (transform/transpose.rs:156-207, permute.rs): a view that shares the storage.  Nothing is
// launched; whoever needs the elements in the new order gets a permuted copy then (see TensorImpl::contig), and a 2-D
// GEMM operand needs none at all.
static ts_tensor* permute_op(const TensorP& x, const std::vector<int>& perm) {
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    const int rank = (int)perm.size();
    std::vector<size_t> od((size_t)rank);
    for (int i = 0; i < rank; ++i) od[i] = x->dims[perm[i]];
    if (!materialize(x)) return nullptr;
    auto out = std::make_shared<TensorImpl>(od);
    out->st = x->st;
    // relative to the contiguous tensor the storage holds: a view of a view composes the permutations
    std::vector<int> composed((size_t)rank);
    for (int i = 0; i < rank; ++i) composed[i] = is_view(x) ? x->view_perm[perm[i]] : perm[i];
    bool identity = true;
    for (int i = 0; i < rank; ++i) identity = identity && composed[i] == i;
    if (!identity) {
        out->view_perm = composed;
        out->base_dims = is_view(x) ? x->base_dims : x->dims;
    }
    if (x->requires_grad) {
        Node nd;
        nd.op = Op::Permute;
        nd.inputs = {x->id};
        nd.needs = {true};
        nd.dims0 = x->dims;
        nd.perm = perm;
        record(out, std::move(nd));
    }
    return wrap(out);
}

TS_API ts_tensor* ts_tensor_permute(ts_tensor* hx, const unsigned long long* order, int n) {
    if (!hx || (n > 0 && !order)) { set_error("permute: null argument"); return nullptr; }
    TensorP x = hx->t;
    const int rank = (int)x->dims.size();
    if (n != rank) { set_error("permute order must have length equal to rank"); return nullptr; }   // permute.rs:149-153
    if (rank > 8) { set_error("permute: rank %d not supported (up to 8)", rank); return nullptr; }
    std::vector<int> perm((size_t)rank);
    std::vector<bool> seen((size_t)rank, false);
    for (int i = 0; i < rank; ++i) {
        if (order[i] >= (unsigned long long)rank) { set_error("permute index %llu out of bounds for rank %d", order[i], rank); return nullptr; }
        if (seen[order[i]]) { set_error("duplicate dimension %llu in permute", order[i]); return nullptr; }
        seen[order[i]] = true;
        perm[i] = (int)order[i];
    }
    return permute_op(x, perm);
}

TS_API ts_tensor* ts_tensor_transpose(ts_tensor* hx, unsigned long long dim0, unsigned long long dim1) {
    if (!hx) { set_error("transpose: null tensor"); return nullptr; }
    TensorP x = hx->t;
    const size_t rank = x->dims.size();
    if (dim0 >= rank) { set_error("dim0 %llu out of bounds for tensor with rank %zu", dim0, rank); return nullptr; }   // transpose.rs:157-168
    if (dim1 >= rank) { set_error("dim1 %llu out of bounds for tensor with rank %zu", dim1, rank); return nullptr; }
    if (rank > 8) { set_error("transpose: rank %zu not supported (up to 8)", rank); return nullptr; }
    if (dim0 == dim1) {
        // transpose.rs:169-171 returns self.clone(): a copy with no gradient history
        DeviceCtx* c = ctx();
        const float* px = c ? rptr(x) : nullptr;
        TensorP out = px ? new_tensor(c, x->dims) : nullptr;
        if (!out) return nullptr;
        if (x->size && !cuda_ok(cudaMemcpyAsync(out->st->ptr, px, x->size * sizeof(float), cudaMemcpyDeviceToDevice, c->compute), "clone")) return nullptr;
        return wrap(out);
    }
    std::vector<int> perm(rank);
    for (size_t i = 0; i < rank; ++i) perm[i] = (int)i;
    std::swap(perm[dim0], perm[dim1]);
    return permute_op(x, perm);
}

// Clone for Tensor (tensor/core/mod.rs:344-378): a fresh tensor with the same values and no gradient history.
TS_API ts_tensor* ts_tensor_clone(ts_tensor* hx) {
    if (!hx) { set_error("clone: null tensor"); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP x = hx->t;
    const float* px = rptr(x);
    TensorP out = px ? new_tensor(c, x->dims) : nullptr;
    if (!out) return nullptr;
    if (x->size && !cuda_ok(cudaMemcpyAsync(out->st->ptr, px, x->size * sizeof(float), cudaMemcpyDeviceToDevice, c->compute), "clone")) return nullptr;
    return wrap(out);
}

// contiguous.rs:123-137: for a contiguous tensor, a copy that stays connected to its source in the graph
TS_API ts_tensor* ts_tensor_contiguous(ts_tensor* hx) {
    if (!hx) { set_error("contiguous: null tensor"); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP x = hx->t;
    const float* px = rptr(x);
    TensorP out;
    if (px && is_view(x)) {
        // contiguous.rs:138-160: the one copy a view costs; the view gives its permuted copy away and makes another if asked again
        out = std::make_shared<TensorImpl>(x->dims);
        out->st = x->contig;
        x->contig.reset();
    } else {
        out = px ? new_tensor(c, x->dims) : nullptr;
        if (!out) return nullptr;
        if (x->size && !cuda_ok(cudaMemcpyAsync(out->st->ptr, px, x->size * sizeof(float), cudaMemcpyDeviceToDevice, c->compute), "contiguous")) return nullptr;
    }
    if (x->requires_grad) {
        Node nd;
        nd.op = Op::Reshape;   // the gradient passes through unchanged (GradFn::Contiguous)
        nd.inputs = {x->id};
        nd.needs = {true};
        nd.dims0 = x->dims;
        record(out, std::move(nd));
    }
    return wrap(out);
}

// ---- joining and splitting along an axis (tensor/transform/cat.rs:110-230, split.rs:159-330)
TS_API ts_tensor* ts_tensor_cat(ts_tensor* const* tensors, int n, unsigned long long dim) {
    if (n <= 0 || !tensors) { set_error("cat requires at least one tensor"); return nullptr; }   // cat.rs:111
    for (int i = 0; i < n; ++i)
        if (!tensors[i]) { set_error("cat: null tensor at index %d", i); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    const std::vector<size_t>& base = tensors[0]->t->dims;
    const size_t rank = base.size();
    if (dim >= rank) { set_error("concat dim %llu out of bounds for rank %zu", dim, rank); return nullptr; }
    std::vector<size_t> od = base;
    size_t total = 0;
    bool any_grad = false;
    for (int i = 0; i < n; ++i) {
        const std::vector<size_t>& d = tensors[i]->t->dims;
        if (d.size() != rank) { set_error("All tensors must have same rank"); return nullptr; }
        for (size_t a = 0; a < rank; ++a)
            if (a != dim && d[a] != base[a]) {
                set_error("All dims except concat dim must match (dim %zu: %zu vs %zu)", a, base[a], d[a]);
                return nullptr;
            }
        total += d[dim];
        any_grad = any_grad || tensors[i]->t->requires_grad;
    }
    od[dim] = total;
    TensorP out = new_tensor(c, od);
    if (!out) return nullptr;
    size_t outer = 1, inner = 1, prefix = 0;
    for (size_t a = 0; a < dim; ++a) outer *= od[a];
    for (size_t a = dim + 1; a < rank; ++a) inner *= od[a];
    for (int i = 0; i < n; ++i) {
        const size_t len = tensors[i]->t->dims[dim];
        if (len && outer && inner) {
            const float* px = rptr(tensors[i]->t);
            if (!px || !copy_slab(out->st->ptr, total * inner, prefix * inner, px, len * inner, 0, len * inner, outer, c->compute)) return nullptr;
        }
        prefix += len;
    }
    if (any_grad) {   // cat.rs registers GradFn::Cat whenever an input requires a gradient
        Node nd;
        nd.op = Op::Cat;
        nd.code = (int)dim;
        nd.dims0 = od;
        for (int i = 0; i < n; ++i) {
            nd.inputs.push_back(tensors[i]->t->id);
            nd.needs.push_back(tensors[i]->t->requires_grad);
            nd.perm.push_back((int)tensors[i]->t->dims[dim]);
        }
        record(out, std::move(nd));
    }
    return wrap(out);
}

// One piece of split_with_sizes: elements [start, start + length) of axis `dim`, as a contiguous copy.
TS_API ts_tensor* ts_tensor_split_piece(ts_tensor* hx, unsigned long long dim, unsigned long long start, unsigned long long length) {
    if (!hx) { set_error("split: null tensor"); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP x = hx->t;
    const size_t rank = x->dims.size();
    if (dim >= rank) { set_error("split dim %llu out of bounds for rank %zu", dim, rank); return nullptr; }   // split.rs:161-167
    if (start + length > x->dims[dim]) { set_error("split: piece [%llu, %llu) exceeds size %zu of dim %llu", start, start + length, x->dims[dim], dim); return nullptr; }
    std::vector<size_t> od = x->dims;
    od[dim] = (size_t)length;
    TensorP out = new_tensor(c, od);
    if (!out) return nullptr;
    size_t outer = 1, inner = 1;
    for (size_t a = 0; a < dim; ++a) outer *= od[a];
    for (size_t a = dim + 1; a < rank; ++a) inner *= od[a];
    if (out->size) {
        const float* px = rptr(x);
        if (!px || !copy_slab(out->st->ptr, length * inner, 0, px, x->dims[dim] * inner, start * inner, length * inner, outer, c->compute)) return nullptr;
    }
    if (x->requires_grad && length > 0) {   // split.rs:300-312; zero-length pieces are plain zeros tensors
        Node nd;
        nd.op = Op::Split;
        nd.code = (int)dim;
        nd.inputs = {x->id};
        nd.needs = {true};
        nd.dims0 = x->dims;
        nd.perm = {(int)start, (int)length};
        record(out, std::move(nd));
    }
    return wrap(out);
}

// ---- reductions over axes: sum_dims / mean_dims / max_dims / min_dims / norm_dims / var_dims / std_dims and the
// whole-tensor max / min / norm / var / std (every axis reduced, result [1])
static const char* reduce_name(int kind, bool all) {
    static const char* dims_names[] = {"sum_dims", "mean_dims", "max_dims", "min_dims", "norm_dims", "var_dims", "std_dims"};
    static const char* all_names[] = {"sum", "mean", "max", "min", "norm", "var", "std"};
    return (kind < 0 || kind > 6) ? "reduce" : (all ? all_names[kind] : dims_names[kind]);
}

static ts_tensor* reduce_dims_op(ts_tensor* hx, int kind, const unsigned long long* axes, int n_axes, bool keepdim, bool all) {
    const char* name = reduce_name(kind, all);
    if (!hx) { set_error("%s: null tensor", name); return nullptr; }
    if (kind < TS_REDUCE_SUM || kind > TS_REDUCE_STD) { set_error("reduce: unknown kind %d", kind); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP x = hx->t;
    const int rank = (int)x->dims.size();
    if (rank > 8) { set_error("%s: rank %d not supported (up to 8)", name, rank); return nullptr; }
    std::vector<unsigned char> red((size_t)rank, all ? 1 : 0);
    if (!all) {
        if (n_axes <= 0 || !axes) { set_error("%s requires at least one dimension", name); return nullptr; }      // sum.rs:226
        for (int i = 0; i < n_axes; ++i) {
            if (axes[i] >= (unsigned long long)rank) { set_error("%s dim %llu out of bounds for rank %d", name, axes[i], rank); return nullptr; }   // sum.rs:228-235
            red[axes[i]] = 1;
        }
    }
    // output shape: a reduced axis becomes 1 (keepdim) or disappears; nothing left means [1] (sum.rs:236-249)
    std::vector<size_t> od;
    size_t factor = 1;
    for (int i = 0; i < rank; ++i) {
        if (red[i]) { factor *= x->dims[i]; if (keepdim && !all) od.push_back(1); }
        else od.push_back(x->dims[i]);
    }
    if (od.empty()) od.push_back(1);
    if ((kind == TS_REDUCE_VAR || kind == TS_REDUCE_STD) && !all && factor == 0) { set_error("reduced size must be > 0"); return nullptr; }   // std.rs:349
    const float* px = rptr(x);
    TensorP out = px ? new_tensor(c, od) : nullptr;
    if (!out) return nullptr;
    float* scratch = c->alloc.alloc(k::reduce_dims_scratch_elems() * sizeof(float));
    if (!scratch) return nullptr;
    cudaStream_t s = c->compute;
    const size_t* d = x->dims.data();
    float* o = out->st->ptr;
    TensorP mean_t;
    bool ok = true;
    switch (kind) {
        case TS_REDUCE_SUM: ok = k::reduce_dims(0, px, nullptr, o, d, rank, red.data(), scratch, s); break;
        case TS_REDUCE_MEAN:   // mean.rs:186-200: sum_dims, then mul_scalar(1 / count)
            ok = k::reduce_dims(0, px, nullptr, o, d, rank, red.data(), scratch, s) &&
                 k::scale(o, factor > 0 ? 1.0f / (float)factor : 0.0f, o, out->size, s);
            break;
        case TS_REDUCE_MAX: ok = k::reduce_dims(1, px, nullptr, o, d, rank, red.data(), scratch, s); break;
        case TS_REDUCE_MIN: ok = k::reduce_dims(2, px, nullptr, o, d, rank, red.data(), scratch, s); break;
        case TS_REDUCE_NORM:   // norm.rs: sqrt of the sum of squares
            ok = k::reduce_dims(3, px, nullptr, o, d, rank, red.data(), scratch, s) && k::unary(TS_UNARY_SQRT, o, o, out->size, 0.0f, s);
            break;
        case TS_REDUCE_VAR:
        case TS_REDUCE_STD: {
            // var.rs / std.rs: mean = sum / n, then the sum of squared deviations / n (population variance); std = sqrt
            mean_t = new_tensor(c, od);
            ok = mean_t != nullptr;
            if (ok && factor == 0) {
                ok = k::fill(mean_t->st->ptr, 0.0f, out->size, s) && k::fill(o, 0.0f, out->size, s);   // var.rs:103-105: an empty tensor gives 0
            } else if (ok) {
                ok = k::reduce_dims(0, px, nullptr, mean_t->st->ptr, d, rank, red.data(), scratch, s) &&
                     k::unary(TS_UNARY_DIV_SCALAR, mean_t->st->ptr, mean_t->st->ptr, out->size, (float)factor, s) &&
                     k::reduce_dims(4, px, mean_t->st->ptr, o, d, rank, red.data(), scratch, s) &&
                     k::unary(TS_UNARY_DIV_SCALAR, o, o, out->size, (float)factor, s);
                if (ok && kind == TS_REDUCE_STD) ok = k::unary(TS_UNARY_SQRT, o, o, out->size, 0.0f, s);
            }
            break;
        }
    }
    c->alloc.free(scratch);
    if (!ok) return nullptr;
    if (x->requires_grad) {   // registered whenever the input requires a gradient, as in the reference (sum.rs:292-301)
        Node nd;
        nd.op = Op::ReduceDims;
        nd.code = kind;
        nd.inputs = {x->id};
        nd.needs = {true};
        nd.dims0 = x->dims;
        nd.perm.assign(red.begin(), red.end());
        if (kind >= TS_REDUCE_MAX) { nd.s0.set(x); nd.s1.set(out); }
        if (mean_t) nd.s2.set(mean_t);
        record(out, std::move(nd));
    }
    return wrap(out);
}
TS_API ts_tensor* ts_tensor_reduce_dims(ts_tensor* x, int kind, const unsigned long long* dims, int n_dims, int keepdim) {
    return reduce_dims_op(x, kind, dims, n_dims, keepdim != 0, false);
}
TS_API ts_tensor* ts_tensor_reduce_all(ts_tensor* x, int kind) {
    if (kind == TS_REDUCE_SUM) return ts_tensor_sum(x);
    if (kind == TS_REDUCE_MEAN) return ts_tensor_mean(x);
    return reduce_dims_op(x, kind, nullptr, 0, false, true);
}

TS_API ts_tensor* ts_tensor_pow_scalar(ts_tensor* hx, float exponent) {
    if (!hx) { set_error("pow_scalar: null tensor"); return nullptr; }
    if (exponent != 2.0f) return unary_op(hx, TS_UNARY_POW_SCALAR, exponent, "pow_scalar");
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP x = hx->t;
    TensorP out;
    if (fusion_enabled() && x->pending_ew && x->pending_ew->kind == PendingEw::Diff) {
        out = std::make_shared<TensorImpl>(x->dims);   // (a - b)^2, still deferred
        out->pending_ew.reset(new PendingEw{PendingEw::SqDiff, x->pending_ew->a, x->pending_ew->b});
        register_pending(out);
    } else {
        const float* px = rptr(x);
        out = px ? new_tensor(c, x->dims) : nullptr;
        if (!out || !k::square(px, out->st->ptr, out->size, c->compute)) return nullptr;
    }
    if (grad_on() && x->requires_grad) {
        Node nd;
        nd.op = Op::PowScalar;
        nd.inputs = {x->id};
        nd.needs = {true};
        nd.dims0 = x->dims;
        nd.scalar = exponent;
        nd.s0.set(x);
        record(out, std::move(nd));
    }
    return wrap(out);
}

static ts_tensor* reduce_all(ts_tensor* hx, bool mean) {
    if (!hx) { set_error("sum/mean: null tensor"); return nullptr; }
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    TensorP x = hx->t;
    TensorP out;
    if (mean && fusion_enabled() && x->pending_ew && x->pending_ew->kind == PendingEw::SqDiff) {
        // mean((a - b)^2) straight from a and b: the same two-stage tree as sum() over the squared differences
        const float *pa = rptr(x->pending_ew->a), *pb = rptr(x->pending_ew->b);
        out = (pa && pb) ? new_tensor(c, {1}) : nullptr;
        if (!out || !k::mse_loss(pa, pb, out->st->ptr, x->size, c->reduce_scratch, c->compute)) return nullptr;
    } else {
        const float* px = rptr(x);
        out = px ? new_tensor(c, {1}) : nullptr;
        if (!out || !k::sum(px, out->st->ptr, x->size, mean, c->reduce_scratch, c->compute)) return nullptr;
    }
    // The reference registers these nodes even under NoGradTrack (reductions/sum.rs:131, mean.rs:99).
    if (x->requires_grad) {
        Node nd;
        nd.op = mean ? Op::ReduceMean : Op::ReduceSum;
        nd.inputs = {x->id};
        nd.needs = {true};
        nd.dims0 = x->dims;
        record(out, std::move(nd));
    }
    return wrap(out);
}
TS_API ts_tensor* ts_tensor_sum(ts_tensor* x) { return reduce_all(x, false); }
TS_API ts_tensor* ts_tensor_mean(ts_tensor* x) { return reduce_all(x, true); }

// ====================================================================== C ABI: gradtrack
TS_API bool ts_tensor_backward(ts_tensor* t, ts_tensor* grad_output) {
    if (!t) { set_error("backward: null tensor"); return false; }
    return ts::backward(t->t, grad_output ? grad_output->t : nullptr);
}
TS_API ts_tensor* ts_tensor_grad_by_value(const ts_tensor* t) {
    if (!t) return nullptr;
    TensorP g = grad_lookup(t->t->id);
    if (!g) return nullptr;
    if (!materialize(g)) return nullptr;
    auto r = g_dp.red.find(t->t->id);
    if (r != g_dp.red.end() || g_dp.comm_outstanding) {
        // a gradient handed to the caller must be the sum over ranks, whole: a reduce-scattered one is gathered first
        // (a collective: every rank has to ask for it)
        DeviceCtx* c = ctx();
        if (!c) return nullptr;
        if (r != g_dp.red.end() && !dp_gather_grad(c, r->second)) return nullptr;
        if (!dp_join(c)) return nullptr;
    }
    return wrap(reshaped_alias(g, t->t->dims));
}
TS_API void ts_clear_gradients(void) {
    if (g_dp.grads_outstanding) {
        // Gradient buffers go back to the allocator below and are reused in compute-stream order: the compute stream
        // waits for the communication stream's last use of them (a sum, or the sharded Adam update).  The all-gathers
        // of updated parameters that follow on the communication stream are not waited for here.
        DeviceCtx* c = ctx();
        if (c) dp_join_grads(c);
    }
    g_dp.red.clear();
    g_graph.ops.clear();
    g_graph.grads.clear();
    g_graph.bias_grad_ready.clear();
}
TS_API void ts_no_grad_push(void) { ++g_no_grad_depth; }
TS_API void ts_no_grad_pop(void) { if (g_no_grad_depth > 0) --g_no_grad_depth; }
TS_API bool ts_is_grad_enabled(void) { return grad_on(); }
TS_API unsigned long long ts_tape_len(void) { return g_graph.ops.size(); }

// ====================================================================== C ABI: Adam
TS_API ts_adam* ts_adam_new(float lr, float beta1, float beta2, float eps, float weight_decay) {
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    ts_adam* o = new ts_adam();
    o->lr = lr; o->beta1 = beta1; o->beta2 = beta2; o->eps = eps; o->wd = weight_decay;
    o->c = c;
    g_adams.insert(o);
    return o;
}
TS_API ts_adam* ts_adam_new_amsgrad(float lr, float beta1, float beta2, float eps, float weight_decay, int amsgrad) {
    ts_adam* o = ts_adam_new(lr, beta1, beta2, eps, weight_decay);
    if (o) o->amsgrad = amsgrad != 0;
    return o;
}
TS_API void ts_adam_free(ts_adam* o) {
    if (!o) return;
    g_adams.erase(o);
    if (o->c) {
        if (g_dp.comm_outstanding) dp_join(o->c);   // the sharded update reads its chunk map on the communication stream
        o->c->alloc.free(o->whole.dev);
        o->c->alloc.free(o->sliced.dev);
    }
    delete o;
}
TS_API bool ts_adam_add_parameter(ts_adam* o, const ts_tensor* p) {
    if (!o || !p) { set_error("add_parameter: null argument"); return false; }
    if (!p->t->requires_grad) { set_error("add_parameter: parameter must require gradients"); return false; }   // adam/mod.rs:287-300
    if (o->states.count(p->t->id)) return true;
    AdamState st;
    st.n = p->t->size;
    st.m = new_storage(o->c, st.n);
    st.v = new_storage(o->c, st.n);
    if (!st.m || !st.v) return false;
    if (!k::fill(st.m->ptr, 0.0f, st.n, o->c->compute) || !k::fill(st.v->ptr, 0.0f, st.n, o->c->compute)) return false;
    if (o->amsgrad) {
        // the reference starts v_hat_max as a copy of the first v_hat (adam/mod.rs:535-537); zero gives the same maxima
        st.vmax = new_storage(o->c, st.n);
        if (!st.vmax || !k::fill(st.vmax->ptr, 0.0f, st.n, o->c->compute)) return false;
    }
    o->states[p->t->id] = st;
    o->order.push_back(p->t->id);
    return true;
}

TS_API bool ts_adam_step(ts_adam* o, ts_tensor* const* params, int n, float grad_scale) {
    if (!o || (n > 0 && !params)) { set_error("adam step: null argument"); return false; }
    DeviceCtx* c = o->c;
    // Everything is validated before any counter moves: a call that fails leaves step_count and the per-parameter
    // steps where they were, so later bias corrections are not shifted by it.
    for (int i = 0; i < n; ++i) {
        if (!params[i]) { set_error("adam step: null parameter at index %d", i); return false; }
        const TensorP& p = params[i]->t;
        if (!o->states.count(p->id)) {   // adam/mod.rs:489-492 asserts
            set_error("adam step: parameter %llu is not linked to the optimizer; call add_parameter first", (unsigned long long)p->id);
            return false;
        }
        TensorP g = grad_lookup(p->id);
        if (g && g->size != p->size) { set_error("adam step: gradient and parameter sizes differ for %llu", (unsigned long long)p->id); return false; }
        if (is_view(p)) { set_error("adam step: parameter %llu is a transposed view; optimise the tensor it was taken from", (unsigned long long)p->id); return false; }
    }
    struct Item { TensorP p; AdamState* st; k::AdamTensor rec; bool from_dp = false, sliced = false; size_t lo = 0, cnt = 0; uint64_t id = 0; };
    std::vector<Item> whole, sliced;
    std::string skipped;
    const bool write_tf32 = matmul_precision() == 1;
    for (int i = 0; i < n; ++i) {
        TensorP p = params[i]->t;
        AdamState& st = o->states.find(p->id)->second;
        TensorP g = grad_lookup(p->id);
        if (!g) {   // adam/mod.rs:494-497, 1039-1042: reported and skipped
            skipped += (skipped.empty() ? "" : ", ") + std::to_string(p->id);
            continue;
        }
        auto red = g_dp.red.find(p->id);
        const bool from_dp = red != g_dp.red.end() && g_graph.grads.find(p->id) == g_graph.grads.end();
        // a gradient that is being summed on the communication stream is read there or behind its event: no wait here
        const float* gp = from_dp ? red->second.buf->st->ptr : rptr(g);
        float* pp = const_cast<float*>(rptr(p));
        if (!gp || !pp) return false;
        Item it;
        it.p = p; it.st = &st; it.id = p->id; it.from_dp = from_dp;
        it.sliced = from_dp && red->second.sliced;
        if (it.sliced) { it.lo = red->second.lo; it.cnt = red->second.cnt; }
        // TF32 mode: a parameter that feeds tensor-core GEMMs keeps a copy rounded to TF32 beside it; the update
        // writes that copy too, so the next forward finds it current instead of running a rounding pass
        float* tf = (write_tf32 && p->st->tf32_copy) ? p->st->tf32_copy : nullptr;
        if (it.sliced && !dp_gather_tf32_enabled()) tf = nullptr;   // the rounded copy is then remade locally after the gather
        const size_t lo = it.lo, cnt = it.sliced ? it.cnt : p->size;
        it.rec = k::AdamTensor{pp + lo, gp + lo, st.m->ptr + lo, st.v->ptr + lo, (unsigned long long)cnt,
                               o->amsgrad ? st.vmax->ptr + lo : nullptr, tf ? tf + lo : nullptr};
        (it.sliced ? sliced : whole).push_back(it);
    }
    if (whole.empty() && sliced.empty() && !dp_join(c)) return false;
    o->step_count += 1;   // adam/mod.rs:1037
    // bias corrections in f64 from the f32-rounded betas, then to f32: adam/mod.rs:526-531, :793
    const float stepf = (float)o->step_count;
    const float bc1 = (float)(1.0 - std::pow((double)o->beta1, (double)stepf));
    const float bc2 = (float)(1.0 - std::pow((double)o->beta2, (double)stepf));
    const float f1 = 1.0f / bc1, f2 = 1.0f / bc2;
    if (!whole.empty() || !sliced.empty()) {
        {   // deferred operations that read a parameter must see its value from before this step
            std::unordered_set<const Storage*> written;
            for (auto& it : whole) written.insert(it.p->st.get());
            for (auto& it : sliced) written.insert(it.p->st.get());
            if (!flush_pending(written)) return false;
        }
        // The pointer tables go to the kernel by value: the host may be several steps ahead of the GPU, and a table
        // staged in reused host memory would be overwritten before the queued copy reads it.
        auto chunks_for = [&](ChunkCache& cache, const std::vector<Item>& items) -> bool {
            std::vector<unsigned long long> sizes;
            for (auto& it : items) sizes.push_back(it.rec.n);
            if (sizes == cache.sizes && cache.dev) return true;
            const int nc = k::adam_chunk_count(sizes.data(), (int)sizes.size());
            const size_t bytes = k::adam_chunk_bytes(nc);
            std::vector<char> host(bytes);
            k::adam_build_chunks(sizes.data(), (int)sizes.size(), host.data());
            if (g_dp.comm_outstanding && !dp_join(c)) return false;   // the old map may still be read on the communication stream
            c->alloc.free(cache.dev);
            cache.dev = c->alloc.alloc(bytes ? bytes : 16);
            if (!cache.dev) return false;
            TS_CHECK(cudaMemcpyAsync(cache.dev, host.data(), bytes, cudaMemcpyHostToDevice, c->compute));
            TS_CHECK(cudaStreamSynchronize(c->compute));
            cache.n = nc;
            cache.sizes = sizes;
            return true;
        };
        auto table_of = [](const std::vector<Item>& items) {
            std::vector<k::AdamTensor> t;
            for (auto& it : items) t.push_back(it.rec);
            return t;
        };
        if (!sliced.empty()) {
            // Sharded update on the communication stream, behind the reduce-scatters that produce its gradients and
            // behind everything the compute stream has queued so far (the backward GEMMs still read the parameters):
            // one launch over this rank's slice of every tensor, then the all-gathers of the updated parameters in the
            // order the next forward needs them.  Each parameter's storage carries an event that its next reader waits
            // for, so the gathers of the later layers overlap the next forward's first GEMMs.
            NcclApi* nc = nccl_api();
            if (!nc || !dp_healthy() || !chunks_for(o->sliced, sliced) || !dp_comm_after_compute(c)) return false;
            const std::vector<k::AdamTensor> tab = table_of(sliced);
            if (!k::adam_launch(tab.data(), (int)tab.size(), o->sliced.dev, o->lr, o->beta1, o->beta2, o->eps, o->wd, f1, f2, grad_scale,
                                c->comm))
                return false;
            if (!dp_mark_grads(c)) return false;     // the gradient buffers are free for reuse once this kernel has run
            for (auto& it : sliced) {
                Storage* ps = it.p->st.get();
                if (!dp_nccl_ok(nc, nc->AllGather(ps->ptr + it.lo, ps->ptr, it.cnt, ncclFloat32, g_dp.comm, c->comm), "ncclAllGather")) return false;
                if (it.rec.tf32_out &&
                    !dp_nccl_ok(nc, nc->AllGather(ps->tf32_copy + it.lo, ps->tf32_copy, it.cnt, ncclFloat32, g_dp.comm, c->comm), "ncclAllGather"))
                    return false;
                if (ps->ready) { cudaEventDestroy(ps->ready); ps->ready = nullptr; }   // rptr above already waited for it
                TS_CHECK(cudaEventCreateWithFlags(&ps->ready, cudaEventDisableTiming));
                TS_CHECK(cudaEventRecord(ps->ready, c->comm));
                it.st->sharded = true; it.st->lo = it.lo; it.st->cnt = it.cnt;
            }
            g_dp.comm_outstanding = true;
        }
        if (!whole.empty()) {
            // Replicated update on the compute stream, one launch for all of these tensors, behind the all-reduces of
            // their own gradients only (the reduce-scatter of the first layer's weights, enqueued last, is not waited for).
            if (!chunks_for(o->whole, whole)) return false;
            for (auto& it : whole) {
                if (it.from_dp) TS_CHECK(cudaStreamWaitEvent(c->compute, g_dp.done_event[it.id], 0));
                if (it.st->sharded && !gather_adam_state(c, *it.st)) return false;   // earlier steps updated a slice only
            }
            const std::vector<k::AdamTensor> tab = table_of(whole);
            if (!k::adam_launch(tab.data(), (int)tab.size(), o->whole.dev, o->lr, o->beta1, o->beta2, o->eps, o->wd, f1, f2, grad_scale,
                                c->compute))
                return false;
        }
        for (auto* items : {&whole, &sliced})
            for (auto& it : *items) {
                Storage* ps = it.p->st.get();
                it.st->step += 1;
                ps->version++;
                ps->tf32_clean = false;
                if (it.rec.tf32_out) ps->tf32_copy_version = ps->version;
            }
    }
    if (!skipped.empty()) {
        set_error("adam step: parameter(s) %s have no gradient and were skipped", skipped.c_str());
    } else {
        set_error("%s", "");
    }
    return true;
}

TS_API void ts_adam_zero_grad(ts_adam* o, ts_tensor* const* params, int n) {
    (void)o; (void)params; (void)n;
    ts_clear_gradients();   // adam/mod.rs:1061-1068 clears the whole thread-local graph
}
TS_API float ts_adam_learning_rate(const ts_adam* o) { return o ? o->lr : 0.0f; }
TS_API void ts_adam_set_learning_rate(ts_adam* o, float lr) { if (o) o->lr = lr; }
TS_API unsigned long long ts_adam_step_count(const ts_adam* o) { return o ? o->step_count : 0; }

static ts_tensor* state_view(const ts_adam* o, const ts_tensor* p, int which) {
    if (!o || !p) return nullptr;
    auto it = o->states.find(p->t->id);
    if (it == o->states.end()) return nullptr;
    StorageP st = which == 0 ? it->second.m : which == 1 ? it->second.v : it->second.vmax;
    if (!st) return nullptr;
    // under data parallelism with sharded updates the moments are whole only after a gather (a collective call)
    if (it->second.sharded && !gather_adam_state(o->c, const_cast<AdamState&>(it->second))) return nullptr;
    auto t = std::make_shared<TensorImpl>(p->t->dims);
    t->st = st;
    return wrap(t);
}
// Checkpoint support (optimizers/adam/serialization.rs:692-752, mod.rs:396-458 relink_parameters): the moments are
// reached through the state views above; these set and read the counters.
TS_API void ts_adam_set_step_count(ts_adam* o, unsigned long long n) { if (o) o->step_count = n; }
TS_API unsigned long long ts_adam_param_step(const ts_adam* o, const ts_tensor* p) {
    if (!o || !p) return 0;
    auto it = o->states.find(p->t->id);
    return it == o->states.end() ? 0 : it->second.step;
}
TS_API bool ts_adam_set_param_step(ts_adam* o, const ts_tensor* p, unsigned long long n) {
    if (!o || !p) { set_error("ts_adam_set_param_step: null argument"); return false; }
    auto it = o->states.find(p->t->id);
    if (it == o->states.end()) { set_error("ts_adam_set_param_step: parameter is not linked to the optimizer"); return false; }
    it->second.step = n;
    return true;
}
TS_API ts_tensor* ts_adam_state_m(const ts_adam* o, const ts_tensor* p) { return state_view(o, p, 0); }
TS_API ts_tensor* ts_adam_state_v(const ts_adam* o, const ts_tensor* p) { return state_view(o, p, 1); }
TS_API ts_tensor* ts_adam_state_v_hat_max(const ts_adam* o, const ts_tensor* p) { return state_view(o, p, 2); }

// ====================================================================== C ABI: data parallel
TS_API bool ts_dp_get_unique_id(unsigned char id_out[TS_DP_UNIQUE_ID_BYTES]) {
    static_assert(sizeof(ncclUniqueId) == TS_DP_UNIQUE_ID_BYTES, "NCCL unique id size");
    if (!id_out) { set_error("ts_dp_get_unique_id: null buffer"); return false; }
    NcclApi* nc = nccl_api();
    if (!nc) return false;
    ncclUniqueId id;
    ncclResult_t r = nc->GetUniqueId(&id);
    if (r != ncclSuccess) { set_error("ncclGetUniqueId failed: %s", nc->GetErrorString(r)); return false; }
    memcpy(id_out, &id, sizeof(id));
    return true;
}
// ncclCommInitRank blocks until every rank has called it.  It runs on a helper thread so that a rank that never joins
// costs a bounded wait and an error instead of a hang; a helper that is still blocked when the wait runs out is left
// behind (there is no communicator yet to abort) and cleans up after itself should it ever return.
struct InitState {
    std::mutex mu;
    std::condition_variable cv;
    bool done = false, abandoned = false;
    ncclResult_t result = ncclSuccess;
    ncclComm_t comm = nullptr;
};
TS_API bool ts_dp_init_with_timeout(const unsigned char id_in[TS_DP_UNIQUE_ID_BYTES], int rank, int world, double timeout_seconds) {
    NcclApi* nc = nccl_api();
    if (!nc) return false;
    DeviceCtx* c = nc->fake ? nullptr : ctx();
    if (!nc->fake && !c) return false;
    if (!id_in || world < 1 || rank < 0 || rank >= world) { set_error("ts_dp_init: bad arguments (rank %d, world %d)", rank, world); return false; }
    if (g_dp.comm) { set_error("ts_dp_init: already initialised on this thread"); return false; }
    g_dp.rank = rank; g_dp.world = world; g_dp.failed = false;
    if (world == 1) return true;
    ncclUniqueId id;
    memcpy(&id, id_in, sizeof(id));
    auto st = std::make_shared<InitState>();
    const int device = c ? c->device : -1;
    std::thread([st, nc, id, rank, world, device] {
        if (device >= 0) cudaSetDevice(device);
        ncclComm_t comm = nullptr;
        ncclResult_t r = nc->CommInitRank(&comm, world, id, rank);
        std::lock_guard<std::mutex> lk(st->mu);
        if (st->abandoned) { if (r == ncclSuccess && comm) nc->CommAbort(comm); return; }
        st->result = r; st->comm = comm; st->done = true;
        st->cv.notify_all();
    }).detach();
    std::unique_lock<std::mutex> lk(st->mu);
    const bool in_time = timeout_seconds <= 0 ? (st->cv.wait(lk, [&] { return st->done; }), true)
                                              : st->cv.wait_for(lk, std::chrono::duration<double>(timeout_seconds), [&] { return st->done; });
    if (!in_time) {
        st->abandoned = true;
        g_dp.rank = 0; g_dp.world = 1;
        set_error("ts_dp_init: the rendezvous of %d ranks did not complete within %.1f s (rank %d waited; a rank never joined)", world,
                  timeout_seconds, rank);
        return false;
    }
    if (st->result != ncclSuccess) {
        g_dp.rank = 0; g_dp.world = 1;
        set_error("ncclCommInitRank failed: %s", nc->GetErrorString(st->result));
        return false;
    }
    g_dp.comm = st->comm;
    if (c) {
        // NCCL's kernels need SMs of their own: the GEMM kernels are persistent, one CTA per SM with all of its shared
        // memory, so a collective that starts beside one would wait for a whole CTA to retire (or, started first, make
        // GEMM CTAs queue behind it and stretch that launch by a wave).  TS_DP_RESERVE_SMS SMs are kept out of the GEMM grids.
        int reserve = 0;
        if (const char* e = getenv("TS_DP_RESERVE_SMS")) reserve = atoi(e);
        if (reserve < 0) reserve = 0;
        if (reserve > c->sm_count / 2) reserve = c->sm_count / 2;
        c->sm_reserved = reserve & ~1;   // the two-CTA kernel takes SMs in pairs
    }
    return true;
}
TS_API bool ts_dp_init(const unsigned char id_in[TS_DP_UNIQUE_ID_BYTES], int rank, int world) {
    double t = 300.0;   // TS_DP_INIT_TIMEOUT (seconds; 0 = wait for ever)
    if (const char* e = getenv("TS_DP_INIT_TIMEOUT")) t = atof(e);
    return ts_dp_init_with_timeout(id_in, rank, world, t);
}
// Which elements of an n-element gradient a rank owns after the cross-rank sum (1: a slice, 0: all of it); for tests.
TS_API int ts_debug_dp_shard_plan(unsigned long long n, int world, int rank, unsigned long long* lo, unsigned long long* count) {
    size_t l = 0, c = 0;
    const bool sliced = ts::dp_shard_plan((size_t)n, (size_t)(world > 0 ? world : 1), (size_t)(rank > 0 ? rank : 0), &l, &c);
    if (lo) *lo = l;
    if (count) *count = c;
    return sliced ? 1 : 0;
}
// True while the communicator reports no asynchronous error.  On an error (a peer that died, a transport fault) the
// communicator is aborted, so that nothing can block on it any more, and this and every later collective call fail.
TS_API bool ts_dp_healthy(void) { return dp_healthy(); }
// Test hook: replaces NCCL by an in-process stand-in that moves no data (see the modes above); mode < 0 removes it.
TS_API void ts_dp_install_fake_nccl(int mode) {
    std::lock_guard<std::mutex> lk(g_nccl_mu);
    if (mode < 0) { g_nccl = NcclApi(); return; }
    g_fake_mode.store(mode);
    g_nccl.GetUniqueId = fake_get_unique_id; g_nccl.CommInitRank = fake_comm_init_rank; g_nccl.AllReduce = fake_all_reduce;
    g_nccl.ReduceScatter = fake_reduce_scatter; g_nccl.AllGather = fake_all_gather; g_nccl.CommGetAsyncError = fake_async_error;
    g_nccl.CommAbort = fake_abort; g_nccl.CommDestroy = fake_destroy; g_nccl.GetErrorString = fake_error_string;
    g_nccl.ok = g_nccl.fake = true;
}
TS_API int ts_dp_fake_nccl_aborts(void) { return g_fake_aborts.load(); }
TS_API void ts_dp_finalize(void) {
    DeviceCtx* c = ctx_if_initialized();
    if (c && g_dp.comm && !g_dp.failed) {
        // optimizer moments that are current on their owner's slice only are made whole while the ranks can still talk
        for (ts_adam* o : g_adams)
            for (auto& kv : o->states)
                if (kv.second.sharded) gather_adam_state(c, kv.second);
    }
    if (c) { cudaStreamSynchronize(c->comm); cudaStreamSynchronize(c->compute); }
    if (g_dp.comm) { if (NcclApi* nc = nccl_api()) nc->CommDestroy(g_dp.comm); g_dp.comm = nullptr; }
    if (c) c->sm_reserved = 0;
    if (g_dp.ev_compute) {
        cudaEventDestroy(g_dp.ev_compute); cudaEventDestroy(g_dp.ev_comm); cudaEventDestroy(g_dp.ev_grads);
        g_dp.ev_compute = g_dp.ev_comm = g_dp.ev_grads = nullptr;
    }
    for (auto& kv : g_dp.done_event) cudaEventDestroy(kv.second);
    g_dp.done_event.clear();
    g_dp.red.clear();
    g_dp.retired.clear();
    g_dp.params.clear();
    g_dp.rank = 0; g_dp.world = 1; g_dp.comm_outstanding = g_dp.grads_outstanding = g_dp.failed = false;
}
TS_API int ts_dp_world_size(void) { return g_dp.world; }
TS_API int ts_dp_rank(void) { return g_dp.rank; }
TS_API bool ts_dp_register_parameters(ts_tensor* const* params, int n) {
    if (n > 0 && !params) { set_error("ts_dp_register_parameters: null argument"); return false; }
    g_dp.params.clear();
    for (int i = 0; i < n; ++i) {
        if (!params[i]) { set_error("ts_dp_register_parameters: null parameter at index %d", i); return false; }
        g_dp.params.insert(params[i]->t->id);
    }
    return true;
}
TS_API bool ts_dp_all_reduce(float* data, unsigned long long size) {
    DeviceCtx* c = ctx();
    if (!c) return false;
    if (!data && size) { set_error("ts_dp_all_reduce: null data"); return false; }
    if (!dp_all_reduce_async(c, data, size)) return false;
    return dp_join(c);
}
