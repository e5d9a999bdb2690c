// Internal declarations shared by the translation units of libtrain_station_b200.so.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#define TS_API extern "C" __attribute__((visibility("default")))

namespace ts {

// ---------------------------------------------------------------- errors
void set_error(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
const char* last_error();
bool cuda_ok(cudaError_t e, const char* what);  // records the error text when e != success

#define TS_CHECK(expr)                                   \
    do {                                                 \
        if (!::ts::cuda_ok((expr), #expr)) return false; \
    } while (0)

// ---------------------------------------------------------------- allocator
// Size-bucketed caching allocator.  Blocks are reused in stream order on the compute
// stream; a block used on another stream must be fenced by the caller with an event.
class Allocator {
public:
    float* alloc(size_t bytes);
    void free(float* p);
    void release_cached();
    void stats(unsigned long long* in_use, unsigned long long* reserved, unsigned long long* peak,
               unsigned long long* driver_allocs, unsigned long long* hits);
    void set_limit(size_t bytes) { limit_ = bytes; }
    ~Allocator();

private:
    static size_t round_size(size_t bytes);
    std::mutex mu_;
    std::multimap<size_t, void*> cache_;            // free blocks by size
    std::unordered_map<void*, size_t> live_;        // handed-out blocks
    size_t in_use_ = 0, reserved_ = 0, peak_ = 0, limit_ = 0;
    unsigned long long driver_allocs_ = 0, hits_ = 0;
};

// ---------------------------------------------------------------- per-device context
struct DeviceCtx {
    int device = -1;
    int sm_count = 0;
    int sm_reserved = 0;              // SMs the persistent GEMM kernels leave free (for NCCL's CTAs under data parallelism)
    cudaStream_t compute = nullptr;   // every engine kernel runs here
    cudaStream_t copy = nullptr;      // asynchronous uploads
    cudaStream_t comm = nullptr;      // NCCL
    Allocator alloc;
    float* reduce_scratch = nullptr;  // partial sums of sum()/mean()
    int* tile_counter = nullptr;      // device word: the next tile of a GEMM whose tiles are handed out dynamically
    int* error_flag = nullptr;        // device word set by kernels whose bounded waits gave up
    int* error_flag_host = nullptr;   // pinned mirror
};

DeviceCtx* ctx();                     // context of this thread's current device, or nullptr (error set)
DeviceCtx* ctx_if_initialized();      // the same, but never creates one (no allocation); nullptr when absent
int current_device();
bool set_device(int dev);
cudaStream_t pick_stream(void* user_stream);  // NULL -> compute stream of the current device

// ---------------------------------------------------------------- launch accounting
enum ProfClass { kProfGemmTc = 0, kProfGemmFp32 = 1, kProfElementwise = 2, kProfReduce = 3, kProfAdam = 4, kProfClasses = 5 };
// Counts the launch and, when profiling is on, brackets the enclosed launches with two events.
struct ProfScope {
    ProfScope(ProfClass cls, cudaStream_t s, double work, int launches = 1);
    ~ProfScope();
    ProfClass cls;
    cudaStream_t stream;
    cudaEvent_t start = nullptr;
    double work;
};

// While one of these is alive on a thread, ProfScope only counts launches: it creates and records no events even
// when profiling is on.  For entry points that promise not to allocate (event creation allocates).
struct ProfSuspend {
    ProfSuspend();
    ~ProfSuspend();
    bool was_on;
};

int matmul_precision();
bool fusion_enabled();

// ---------------------------------------------------------------- programmatic dependent launch
// A step of a small network is a chain of twenty-odd kernels of a few microseconds each, every one waiting for the one
// before it; between two of them the GPU sits idle while the next grid is set up.  Kernels launched through launch_dep()
// carry the programmatic-stream-serialization attribute: their CTAs may be placed on the SMs while the kernel before
// them is still running, and they call grid_dependency_sync() before they touch global memory, which waits until
// everything launched before them has completed and its writes are visible, so the order of the stream's results is
// unchanged.  The same call then lets the grid behind them be set up in turn.  A kernel launched the ordinary way, or
// following one that never makes the call, simply starts when its predecessor has finished.  TS_PDL=0 launches
// everything the ordinary way.
bool dependent_launch_enabled();
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
template <typename... KArgs, typename... Args>
inline void launch_dep(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = dependent_launch_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);   // the caller reads cudaGetLastError()
}
#endif

// ---------------------------------------------------------------- kernels (device pointers)
namespace k {
constexpr size_t kReduceScratchElems = 4096;

bool binary(int op, const float* a, const float* b, float* o, size_t n, cudaStream_t s);  // 0 add 1 sub 2 mul 3 div
// the same four ops over a broadcast shape `dims` (outermost first); stride_a / stride_b are the operands' element
// strides along those axes, 0 where an operand is stretched
bool binary_bcast(int op, const float* a, const float* b, float* o, const size_t* dims, int rank, const size_t* stride_a,
                  const size_t* stride_b, cudaStream_t s);
bool binary_bcast_bwd(int op, const float* a, const float* b, const float* go, float* ga, float* gb, const size_t* dims, int rank,
                      const size_t* stride_a, const size_t* stride_b, cudaStream_t s);
bool bias_act(const float* z, const float* bias, float* o, size_t rows, size_t cols, bool relu, cudaStream_t s);
bool add_scalar_bcast(const float* a, const float* scalar_dev, float* o, size_t n, cudaStream_t s);
bool relu(const float* x, float* o, size_t n, cudaStream_t s);
bool relu_bwd(const float* ref, const float* go, float* gi, size_t n, cudaStream_t s);
bool square(const float* x, float* o, size_t n, cudaStream_t s);
bool square_bwd(const float* x, const float* go, float* gi, size_t n, cudaStream_t s);
bool mul_bwd(const float* a, const float* b, const float* go, float* ga, float* gb, size_t n, cudaStream_t s);
bool div_bwd(const float* a, const float* b, const float* go, float* ga, float* gb, size_t n, cudaStream_t s);
bool scale(const float* x, float alpha, float* o, size_t n, cudaStream_t s);
bool fill(float* o, float v, size_t n, cudaStream_t s);
// out[i] = part[i] + part[n + i] + ... + part[(slabs - 1) * n + i], added in that order (split-K partial products)
bool sum_slabs(const float* part, float* out, size_t n, size_t slabs, cudaStream_t s);
bool fill_from_scalar(float* o, const float* scalar, float scale, size_t n, cudaStream_t s);
bool sqdiff(const float* a, const float* b, float* o, size_t n, cudaStream_t s);   // (a - b)^2, both steps rounded
// gi = (scale * (*upstream)) * (2 * x): ReduceMean / ReduceSum backward followed by PowScalar(2) backward.
bool square_bwd_scalar(const float* x, const float* upstream, float scale, float* gi, size_t n, cudaStream_t s);
// gy = ((inv_n) * (*upstream)) * (2 * (y - t)): ReduceMean -> PowScalar(2) -> Sub in one pass.
// round_tf32: store the result rounded to the nearest TF32 value (it feeds tensor-core GEMMs directly).
bool mse_grad(const float* y, const float* t, const float* upstream, float inv_n, float* gy, size_t n, bool round_tf32, cudaStream_t s);
// op codes: enum ts_unary_op of the public header; p is the slope, scalar or exponent
bool unary(int op, const float* x, float* o, size_t n, float p, cudaStream_t s);
bool unary_bwd(int op, const float* saved, const float* go, float* gi, size_t n, float p, cudaStream_t s);
bool softmax(const float* x, float* y, size_t outer, size_t reduce, size_t inner, cudaStream_t s);
bool softmax_bwd(const float* y, const float* go, float* gi, size_t outer, size_t reduce, size_t inner, cudaStream_t s);
// out = in with its axes permuted: output axis i is input axis perm[i]; dims are the input's (rank <= 8)
bool permute(const float* in, float* out, const size_t* dims, const int* perm, int rank, cudaStream_t s);
// Reduction over the axes flagged in `reduced` (one byte per input axis).  op: 0 sum, 1 max, 2 min, 3 sum of squares,
// 4 sum of squared deviations from aux[output], 5 count of elements equal to aux[output].  scratch: reduce_dims_scratch_elems().
size_t reduce_dims_scratch_elems();
bool reduce_dims(int op, const float* x, const float* aux, float* out, const size_t* dims, int rank, const unsigned char* reduced,
                 float* scratch, cudaStream_t s);
// mode: 0 sum, 1 mean (scale = 1/count), 2 max/min (a1 extremum, a2 tie count), 3 norm (a1), 4 var (a1 mean, scale 2/n),
// 5 std (a1 mean, a2 std, scale 1/n)
bool reduce_dims_backward(int mode, const float* x, const float* a1, const float* a2, const float* go, float* gi, const size_t* dims,
                          int rank, const unsigned char* reduced, bool go_is_scalar, float scale, cudaStream_t s);
bool sum(const float* x, float* out, size_t n, bool mean, float* scratch, cudaStream_t s);
// loss[0] = mean((y-t)^2) without materialising the difference.
bool mse_loss(const float* y, const float* t, float* out, size_t n, float* scratch, cudaStream_t s);
size_t colsum_scratch_elems(size_t rows, size_t cols);
bool colsum(const float* g, float* out, size_t rows, size_t cols, float* scratch, cudaStream_t s);
// out[j] = partial[0][j] + partial[1][j] + ... in that order: the second stage of a column sum on its own
bool colsum_finish(const float* partial, float* out, size_t cols, size_t partial_rows, cudaStream_t s);
bool relu_bwd_colsum(const float* ref, const float* go, float* gi, float* bias_grad, size_t rows, size_t cols,
                     float* scratch, cudaStream_t s);
// mse_grad (elementwise.cu) over a [rows x cols] prediction plus, from the same pass, the column sums of the stored
// gradient: the gradient of the bias that was added to make the prediction.
bool mse_grad_colsum(const float* y, const float* t, const float* upstream, float inv_n, float* gy, float* bias_grad, size_t rows,
                     size_t cols, bool round_tf32, float* scratch, cudaStream_t s);

struct AdamTensor {
    float* p;
    const float* g;
    float* m;
    float* v;
    unsigned long long n;
    float* vmax = nullptr;   // AMSGrad: running maximum of the bias-corrected second moment; null = plain Adam
    float* tf32_out = nullptr;   // when set: also receives the updated parameter rounded to the nearest TF32 value
};
int adam_chunk_count(const unsigned long long* sizes, int n);
size_t adam_chunk_bytes(int n_chunks);
void adam_build_chunks(const unsigned long long* sizes, int n, void* host_out);
bool adam_launch_range(const AdamTensor* tensors, int first, int last, const void* chunks_dev, float lr, float beta1, float beta2,
                       float eps, float wd, float f1, float f2, float grad_scale, cudaStream_t s);
// tensors is a HOST array: the records are passed to the kernel by value (captured at enqueue time).
bool adam_launch(const AdamTensor* tensors, int n, const void* chunks_dev, float lr, float beta1, float beta2, float eps, float wd,
                 float f1, float f2, float grad_scale, cudaStream_t s);

struct GemmArgs {
    const float* a;
    const float* b;
    float* c;
    size_t m, n, k;
    bool trans_a, trans_b;
    const float* bias;   // [n] or null
    bool relu;
    const float* mask;   // [m,n] or null
    bool round_tf32 = false;   // tensor-core path only: store the result rounded to nearest TF32
    // 3xTF32: when both are set, a and b hold the TF32-exact high parts and these the low parts
    const float* a_lo = nullptr;
    const float* b_lo = nullptr;
    // When set ([n], device): also receives the column sums of the stored result (after bias / ReLU / mask / rounding):
    // from the tensor-core kernels' epilogue, or by a separate pass after an FP32-kernel product.
    float* colsum_out = nullptr;
    float* colsum_partial = nullptr;   // internal: the epilogue's per-32-row partial sums
    // FP32 kernel only: `batch` independent products in one launch (grid z); entry z reads a + z * batch_stride_a and
    // b + z * batch_stride_b (a stride of 0 repeats the operand) and writes c + z * m * n.  No bias / mask with batch > 1.
    size_t batch = 1, batch_stride_a = 0, batch_stride_b = 0;
};
// hi = x rounded to nearest TF32, lo = (x - hi) rounded to nearest TF32: x = hi + lo to about 2^-22 relative.
bool split_tf32(const float* x, float* hi, float* lo, size_t n, cudaStream_t s);
// out = x rounded to the nearest TF32 value (10 explicit mantissa bits, ties away from zero).
bool round_to_tf32(const float* x, float* o, size_t n, cudaStream_t s);
bool sgemm(const GemmArgs& g, cudaStream_t s);                       // FFMA, reference summation order
bool gemm_tc_supported(const GemmArgs& g);
bool gemm_tc(const GemmArgs& g, bool split3, DeviceCtx* c, cudaStream_t s);  // tcgen05 TF32 / 3xTF32
bool gemm(const GemmArgs& g, int precision, DeviceCtx* c, cudaStream_t s);   // dispatch
// Products with one dimension of at most 16 (a 10-class output layer, its weight and input gradients) in the modes
// without a fixed summation order: FFMA kernels laid out along the long dimensions (thin_gemm.cu).
// Where a product goes (host arithmetic only; needs no device): the kernels act on these, ts_debug_gemm_route reports them.
enum GemmRouteKind { kRouteFp32 = 0, kRouteFp32SplitK = 1, kRouteThinNN = 2, kRouteThinTN = 3, kRouteThinNT = 4, kRouteTc128 = 5,
                     kRouteTc256 = 6, kRouteTcPairs = 7, kRouteTcSplitK128 = 8, kRouteTcSplitK256 = 9 };
struct TcRoute { int kind; size_t splits; size_t kb_per_split; };
struct GemmRoute { int kind; size_t splits; size_t kb_per_split; };
TcRoute tc_route(const GemmArgs& g, int sm_count);
GemmRoute gemm_route(const GemmArgs& g, int precision, int sm_count);
int gemm_thin_kind(const GemmArgs& g);      // 0 none, 1 thin_n_nn, 2 thin_n_tn, 3 thin_k_nt
bool gemm_thin_supported(const GemmArgs& g);
bool gemm_thin_rounds(const GemmArgs& g);   // ... and this one would honour round_tf32
bool gemm_thin(const GemmArgs& g, DeviceCtx* c, cudaStream_t s);
}  // namespace k

}  // namespace ts
