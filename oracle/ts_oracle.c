/*
 * CPU oracle for the train-station training-step hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing that ships may call into this file: it is the
 * checker for the CUDA path (tests/, the smoke check) and the timed CPU baseline of
 * the benchmark.  It restates, in plain C with AVX2 intrinsics, the arithmetic of the
 * reference's single-threaded CPU code, operation order included, so that results can
 * be compared bit for bit where the reference performs one IEEE operation per element
 * and within a stated tolerance where summation order differs.
 *
 * Parity pin: the reference is Rust and cannot be compiled in this environment, so
 * this restatement is pinned by (1) the literal known-answer values of the reference's
 * own unit tests and doc-tests (tests/golden/reference_known_answers.json) and (2) the
 * reference's LibTorch differential procedures replayed with PyTorch
 * (tests/golden/torch_differential.npz).  2-D matmul with k > 128 or n > 128 is
 * "parity unpinned": the reference's blocked driver hands sub-block pointers to
 * micro-kernels that use the block width as the row stride
 * (tensor/ops/matmul/kernels.rs:1111-1131 vs :274-307), so no passing reference test
 * covers such shapes; here the row strides are those of the parent matrices, which is
 * the documented contract C = A.B.
 *
 * Build: gcc -O3 -mavx2 -mfma -ffp-contract=off -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: Rust never fuses a*b+c, so neither may this file,
 * except where the reference itself calls _mm256_fmadd_ps.
 */
#include <immintrin.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORA_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ matmul */

/* Block sizes: tensor/ops/matmul/config.rs:122-156 (MatmulConfig::for_dimensions). */
static void ora_block_sizes(size_t m, size_t n, size_t k, size_t *bm, size_t *bn, size_t *bk) {
    size_t mx = m > n ? m : n;
    if (k > mx) mx = k;
    size_t cm, cn, ck;
    if (mx <= 32) { cm = 32; cn = 32; ck = 32; }
    else if (mx <= 64) { cm = 64; cn = 64; ck = 64; }
    else if (mx <= 128) { cm = 64; cn = 128; ck = 128; }
    else { cm = 128; cn = 128; ck = 128; }
    *bm = cm < m ? cm : m;
    *bn = cn < n ? cn : n;
    *bk = ck < k ? ck : k;
}

/*
 * One row strip of R rows (R = 1, 2 or 4) of a block: for every 8-column group one
 * accumulator per row runs the chain acc = fma(A[i,p], B[p,j..j+8], acc) over p
 * ascending (kernels.rs:278-305 one row, :378-385 two rows, :474-497 four rows); the
 * jb mod 8 trailing columns use a rounded multiply followed by an add
 * (kernels.rs:312-335, :393-407, :507-521).  lda/ldb/ldc are the parent strides.
 */
static inline void ora_strip(const float *a, const float *b, float *c, int rows, size_t jb,
                             size_t kb, size_t lda, size_t ldb, size_t ldc, int first) {
    size_t n_simd = jb / 8 * 8;
    for (size_t j = 0; j < n_simd; j += 8) {
        __m256 acc[4];
        for (int r = 0; r < rows; ++r)
            acc[r] = first ? _mm256_setzero_ps() : _mm256_loadu_ps(c + (size_t)r * ldc + j);
        for (size_t p = 0; p < kb; ++p) {
            __m256 bv = _mm256_loadu_ps(b + p * ldb + j);
            for (int r = 0; r < rows; ++r)
                acc[r] = _mm256_fmadd_ps(_mm256_set1_ps(a[(size_t)r * lda + p]), bv, acc[r]);
        }
        for (int r = 0; r < rows; ++r) _mm256_storeu_ps(c + (size_t)r * ldc + j, acc[r]);
    }
    for (size_t j = n_simd; j < jb; ++j) {
        for (int r = 0; r < rows; ++r) {
            float sum = first ? 0.0f : c[(size_t)r * ldc + j];
            for (size_t p = 0; p < kb; ++p) sum += a[(size_t)r * lda + p] * b[p * ldb + j];
            c[(size_t)r * ldc + j] = sum;
        }
    }
}

/*
 * Size-class dispatch of one block: kernels.rs:168-203.  With blocks of at most 128
 * only the first three arms are reachable from the blocked driver.
 */
static void ora_block(const float *a, const float *b, float *c, size_t ib, size_t jb, size_t kb,
                      size_t lda, size_t ldb, size_t ldc, int first) {
    size_t mx = ib > jb ? ib : jb; if (kb > mx) mx = kb;
    size_t mn = ib < jb ? ib : jb; if (kb < mn) mn = kb;
    int rows = (mx <= 64 && mn <= 32) ? 1 : (mx <= 128 && mn <= 64) ? 2 : 4;
    size_t i = 0;
    for (; i + rows <= ib; i += rows)
        ora_strip(a + i * lda, b, c + i * ldc, rows, jb, kb, lda, ldb, ldc, first);
    for (; i < ib; ++i)  /* leftover rows go through the one-row kernel, :410-421, :524-535 */
        ora_strip(a + i * lda, b, c + i * ldc, 1, jb, kb, lda, ldb, ldc, first);
}

/*
 * C[m,n] = A[m,k] . B[k,n], row-major f32.  Blocked driver: kernels.rs:1092-1134
 * (k-blocks outermost; the first k-block initialises C, later ones accumulate
 * through it), with the leading-dimension defect repaired.
 */
ORA_API void ora_matmul(const float *a, const float *b, float *c, size_t m, size_t n, size_t k) {
    if (m == 0 || n == 0) return;
    if (k == 0) { memset(c, 0, m * n * sizeof(float)); return; }
    size_t bm, bn, bk;
    ora_block_sizes(m, n, k, &bm, &bn, &bk);
    for (size_t kk = 0; kk < k; kk += bk) {
        size_t kb = (kk + bk < k ? kk + bk : k) - kk;
        for (size_t ii = 0; ii < m; ii += bm) {
            size_t ib = (ii + bm < m ? ii + bm : m) - ii;
            for (size_t jj = 0; jj < n; jj += bn) {
                size_t jb = (jj + bn < n ? jj + bn : n) - jj;
                ora_block(a + ii * k + kk, b + kk * n + jj, c + ii * n + jj, ib, jb, kb, k, n, n,
                          kk == 0);
            }
        }
    }
}

/* The naive triple loop the reference's tests and its FFI placeholder use as truth:
 * kernels.rs:1148-1158 (reference_matmul), cuda/cuda_wrapper.cpp:81-94. */
ORA_API void ora_matmul_naive(const float *a, const float *b, float *c, size_t m, size_t n,
                              size_t k) {
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) {
            float s = 0.0f;
            for (size_t p = 0; p < k; ++p) s += a[i * k + p] * b[p * n + j];
            c[i * n + j] = s;
        }
}

/* Materialised transpose: t() is a strided view (transform/transpose.rs:181-184) that
 * matmul makes contiguous before multiplying (matmul/mod.rs:586-595). */
ORA_API void ora_transpose(const float *src, float *dst, size_t rows, size_t cols) {
    for (size_t i = 0; i < rows; ++i)
        for (size_t j = 0; j < cols; ++j) dst[j * rows + i] = src[i * cols + j];
}

/* ------------------------------------------------------------- elementwise */

/* add.rs:329-379, sub.rs:369-420, mul.rs:359-400, div.rs:347-420: one IEEE op per element. */
ORA_API void ora_add(const float *a, const float *b, float *o, size_t n) {
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        _mm256_storeu_ps(o + i, _mm256_add_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i)));
    for (; i < n; ++i) o[i] = a[i] + b[i];
}
ORA_API void ora_sub(const float *a, const float *b, float *o, size_t n) {
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        _mm256_storeu_ps(o + i, _mm256_sub_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i)));
    for (; i < n; ++i) o[i] = a[i] - b[i];
}
ORA_API void ora_mul(const float *a, const float *b, float *o, size_t n) {
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        _mm256_storeu_ps(o + i, _mm256_mul_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i)));
    for (; i < n; ++i) o[i] = a[i] * b[i];
}
ORA_API void ora_div(const float *a, const float *b, float *o, size_t n) {
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        _mm256_storeu_ps(o + i, _mm256_div_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i)));
    for (; i < n; ++i) o[i] = a[i] / b[i];
}

/* Row broadcast: out[i,j] = z[i,j] + b[j].  The reference materialises b to [rows,cols]
 * (broadcasting.rs:422-478) and then adds; the value per element is the same single add. */
ORA_API void ora_add_row(const float *z, const float *b, float *o, size_t rows, size_t cols) {
    for (size_t i = 0; i < rows; ++i) ora_add(z + i * cols, b, o + i * cols, cols);
}

/* relu.rs:175-215: _mm256_max_ps(x, 0) -- NaN -> 0 and -0 -> +0 because maxps returns
 * its second operand when the compare is unordered or the operands are equal. */
ORA_API void ora_relu(const float *x, float *o, size_t n) {
    __m256 z = _mm256_setzero_ps();
    size_t i = 0;
    for (; i + 8 <= n; i += 8) _mm256_storeu_ps(o + i, _mm256_max_ps(_mm256_loadu_ps(x + i), z));
    for (; i < n; ++i) o[i] = x[i] > 0.0f ? x[i] : 0.0f; /* scalar tail, relu.rs:260-271 */
}
/* grad_fn/ops/relu.rs:4-16 */
ORA_API void ora_relu_bwd(const float *x, const float *go, float *gi, size_t n) {
    for (size_t i = 0; i < n; ++i) gi[i] = x[i] > 0.0f ? go[i] : 0.0f;
}
/* pow.rs:195-240: exponent 2.0 takes the x*x path. */
ORA_API void ora_square(const float *x, float *o, size_t n) { ora_mul(x, x, o, n); }
/* grad_fn/ops/pow.rs:5-27 with exponent 2: gi = go * (2 * powf(x, 1)) */
ORA_API void ora_square_bwd(const float *x, const float *go, float *gi, size_t n) {
    for (size_t i = 0; i < n; ++i) gi[i] = go[i] * (2.0f * x[i]);
}
/* grad_fn/ops/mul.rs:4-49: (go*b, go*a) */
ORA_API void ora_mul_bwd(const float *a, const float *b, const float *go, float *ga, float *gb,
                         size_t n) {
    for (size_t i = 0; i < n; ++i) { ga[i] = go[i] * b[i]; gb[i] = go[i] * a[i]; }
}
/* grad_fn/ops/div.rs:4-49: (go / b, -((go*a) / (b*b))) */
ORA_API void ora_div_bwd(const float *a, const float *b, const float *go, float *ga, float *gb,
                         size_t n) {
    for (size_t i = 0; i < n; ++i) {
        ga[i] = go[i] / b[i];
        gb[i] = -((go[i] * a[i]) / (b[i] * b[i]));
    }
}
/* grad_fn/ops/sub.rs:26-31: second gradient is the negated clone. */
ORA_API void ora_neg(const float *x, float *o, size_t n) {
    for (size_t i = 0; i < n; ++i) o[i] = -x[i];
}
ORA_API void ora_fill(float *o, float v, size_t n) {
    for (size_t i = 0; i < n; ++i) o[i] = v;
}

/* -------------------------------------------------------------- reductions */

/* reductions/sum.rs:93-105: one f32 accumulator, acc += ((x0+x1)+x2)+x3 per trip. */
ORA_API float ora_sum(const float *x, size_t n) {
    float acc = 0.0f;
    size_t i = 0;
    for (; i + 4 <= n; i += 4) acc += x[i] + x[i + 1] + x[i + 2] + x[i + 3];
    for (; i < n; ++i) acc += x[i];
    return acc;
}
/* reductions/mean.rs:48-95 */
ORA_API float ora_mean(const float *x, size_t n) {
    if (n == 0) return 0.0f;
    return ora_sum(x, n) / (float)n;
}
/* sum_dims(&[0]) on [rows, cols] (reductions/sum.rs:255-290): elements are visited in
 * flat order, so each column accumulates its rows in ascending order from 0.0. */
ORA_API void ora_colsum(const float *g, float *o, size_t rows, size_t cols) {
    for (size_t j = 0; j < cols; ++j) o[j] = 0.0f;
    for (size_t i = 0; i < rows; ++i)
        for (size_t j = 0; j < cols; ++j) o[j] += g[i * cols + j];
}

/* ------------------------------------------------------------------- Adam */

/*
 * One Adam update of one tensor: optimizers/adam/mod.rs:485-556 with the helpers at
 * :635-700 (m), :710-775 (v), :791-840 (bias correction), :914-1010 (update).
 * step is the optimizer's global step count after the increment (:507,:1037).
 * Elements below size/8*8 follow the 8-wide bodies, the rest the scalar tails; the two
 * differ in how (1-beta2)*g*g associates.
 */
ORA_API void ora_adam_update(float *p, const float *g_in, float *m, float *v, size_t n, float lr,
                             float beta1, float beta2, float eps, float weight_decay,
                             uint64_t step) {
    float stepf = (float)step;
    float bc1 = (float)(1.0 - pow((double)beta1, (double)stepf));
    float bc2 = (float)(1.0 - pow((double)beta2, (double)stepf));
    float f1 = 1.0f / bc1, f2 = 1.0f / bc2;
    float c1 = 1.0f - beta1, c2 = 1.0f - beta2;
    size_t body = n / 8 * 8;
    for (size_t i = 0; i < n; ++i) {
        float g = g_in[i];
        if (weight_decay > 0.0f) g = g + weight_decay * p[i]; /* :567-620 */
        float mi = (beta1 * m[i]) + (c1 * g);
        float vi = i < body ? (beta2 * v[i]) + (c2 * (g * g)) : (beta2 * v[i]) + ((c2 * g) * g);
        m[i] = mi;
        v[i] = vi;
        float mh = mi * f1, vh = vi * f2;
        p[i] = p[i] - ((lr * mh) / (sqrtf(vh) + eps));
    }
}

/* ------------------------------------------------- whole MLP training step */

/*
 * The canonical loop (examples/neural_networks/feedforward_network.rs:473-488):
 * per layer z = h.matmul(w).add_tensor(b), relu between layers (and after the last
 * layer iff relu_last), then a loss, backward(), Adam step.  loss_kind: 0 = sum(y),
 * 1 = mean(y), 2 = mean((y - target)^2).  Gradients are written to gw[l]/gb[l] (and
 * gx when x_requires_grad) exactly as the GradFns of gradtrack/grad_fn/ would:
 * ReduceSum/ReduceMean fill, PowScalar, Sub, Relu, Add with sum_dims for the bias,
 * MatMul with materialised transposes (grad_fn/ops/matmul.rs:68-80).
 * as_written != 0 additionally performs the work the reference does around the arithmetic, so
 * that timing reflects it: the deep copies of saved and multiplied operands
 * (matmul/mod.rs:296-297,586-595), the element-by-element materialisation of the broadcast
 * bias (broadcasting.rs:452-477) and the coordinate-walk contiguous() of the transposed
 * operands in backward (transform/contiguous.rs:283-345).  Values are identical either way.
 * Returns the loss.  dims has layers+1 entries.
 */
typedef struct {
    int layers;
    const size_t *dims;
    size_t batch;
    float **w, **b;       /* parameters, updated in place when do_adam */
    float **gw, **gb;     /* gradients out */
    float **mw, **vw, **mb, **vb; /* Adam state */
    const float *x, *target;
    float *gx;            /* may be NULL */
    float *y_out;         /* may be NULL: receives the network output [batch, dims[layers]] */
    int loss_kind, relu_last, as_written, do_adam;
    float lr, beta1, beta2, eps, weight_decay;
    uint64_t step;
} ora_mlp_args;

static float *ora_alloc(size_t n) {
    void *p = NULL;
    if (posix_memalign(&p, 64, (n ? n : 1) * sizeof(float)) != 0) abort();
    return (float *)p;
}
static void ora_touch_copy(const float *src, size_t n) { /* a deep copy that is then dropped */
    float *t = ora_alloc(n);
    memcpy(t, src, n * sizeof(float));
    __asm__ volatile("" : : "r"(t) : "memory");
    free(t);
}

/* A small heap vector per element, as Rust's `vec![0; rank]` inside the reference's copy loops: allocated, used and
 * dropped for every single element.  The barrier keeps the compiler from folding the allocation away. */
static size_t *ora_index_vec(int rank) {
    size_t *v = (size_t *)calloc((size_t)rank, sizeof(size_t));
    if (!v) abort();
    __asm__ volatile("" : : "r"(v) : "memory");
    return v;
}
/* broadcasting.rs:452-477 (broadcast_copy_data, general path): for each element of the stretched result a fresh
 * index vector, one div/mod per axis from the innermost outwards, then the offset through the broadcast strides
 * (0 on stretched axes).  This is how the reference materialises the [rows, cols] copy of a bias row. */
static void ora_broadcast_copy_walk(const float *src, float *dst, const size_t *bdims, const size_t *bstrides,
                                    int rank, size_t total) {
    for (size_t i = 0; i < total; ++i) {
        size_t *idx = ora_index_vec(rank);
        size_t t = i;
        for (int d = rank - 1; d >= 0; --d) { idx[d] = t % bdims[d]; t /= bdims[d]; }
        size_t off = 0;
        for (int d = 0; d < rank; ++d)
            if (bstrides[d] > 0) off += idx[d] * bstrides[d];
        dst[i] = src[off];
        free(idx);
    }
}
/* transform/contiguous.rs:283-322 (copy_to_contiguous_large) with linear_to_coords (:337-345): blocks of 1024
 * destination elements, four per trip, each converting its linear index to coordinates in a fresh vector and
 * taking the source offset through the view's strides.  This is the materialised transpose matmul makes of
 * `w.t()` and `a.t()` in backward (matmul/mod.rs:586-595, grad_fn/ops/matmul.rs:68-80). */
static void ora_contiguous_walk(const float *src, float *dst, const size_t *dims, const size_t *strides, int rank,
                                size_t total) {
    const size_t block = 1024;
    for (size_t start = 0; start < total; start += block) {
        size_t end = start + block < total ? start + block : total;
        for (size_t i = start; i < end; ++i) {      /* the 4-way unrolling changes no access, only loop overhead */
            size_t *c = ora_index_vec(rank);
            size_t t = i;
            for (int d = rank - 1; d >= 0; --d) { c[d] = t % dims[d]; t /= dims[d]; }
            size_t off = 0;
            for (int d = 0; d < rank; ++d) off += c[d] * strides[d];
            dst[i] = src[off];
            free(c);
        }
    }
}
/* dst[cols][rows] = src[rows][cols]^T the way the reference does it: a stride-swapped view made contiguous */
static void ora_transpose_as_written(const float *src, float *dst, size_t rows, size_t cols) {
    size_t dims[2] = {cols, rows}, strides[2] = {1, cols};
    ora_contiguous_walk(src, dst, dims, strides, 2, rows * cols);
}

ORA_API float ora_mlp_step(ora_mlp_args *A) {
    int L = A->layers;
    size_t B = A->batch;
    const size_t *d = A->dims;
    float **z = (float **)calloc((size_t)L, sizeof(float *));   /* pre-activations */
    float **h = (float **)calloc((size_t)L + 1, sizeof(float *)); /* layer inputs */
    h[0] = (float *)A->x;
    for (int l = 0; l < L; ++l) {
        size_t K = d[l], N = d[l + 1];
        float *mm = ora_alloc(B * N);
        if (A->as_written) { ora_touch_copy(h[l], B * K); ora_touch_copy(A->w[l], K * N);
                             ora_touch_copy(h[l], B * K); ora_touch_copy(A->w[l], K * N); }
        ora_matmul(h[l], A->w[l], mm, B, N, K);
        z[l] = ora_alloc(B * N);
        if (A->as_written) {
            /* add_tensor of [B,N] and [N] (add.rs:107-146 -> broadcasting.rs:299-333): the full-size operand is
             * deep-copied, the bias is materialised to [B,N] element by element, then the same-shape add runs */
            float *bb = ora_alloc(B * N);
            size_t bdims[2] = {B, N}, bstr[2] = {0, 1};
            ora_touch_copy(mm, B * N);
            ora_broadcast_copy_walk(A->b[l], bb, bdims, bstr, 2, B * N);
            ora_add(mm, bb, z[l], B * N); free(bb);
        } else ora_add_row(mm, A->b[l], z[l], B, N);
        free(mm);
        int act = (l + 1 < L) || A->relu_last;
        if (act) { h[l + 1] = ora_alloc(B * N); ora_relu(z[l], h[l + 1], B * N); }
        else h[l + 1] = z[l];
    }
    size_t NO = d[L], tot = B * NO;
    float *y = h[L];
    if (A->y_out) memcpy(A->y_out, y, tot * sizeof(float));
    float loss;
    float *gy = ora_alloc(tot);
    if (A->loss_kind == 0) { loss = ora_sum(y, tot); ora_fill(gy, 1.0f, tot); }
    else if (A->loss_kind == 1) {
        loss = ora_mean(y, tot);
        ora_fill(gy, (1.0f / (float)tot) * 1.0f, tot); /* grad_fn/reductions/mean.rs:10-19 */
    } else {
        float *diff = ora_alloc(tot), *sq = ora_alloc(tot);
        ora_sub(y, A->target, diff, tot);
        ora_square(diff, sq, tot);
        loss = ora_mean(sq, tot);
        float *gsq = ora_alloc(tot);
        ora_fill(gsq, (1.0f / (float)tot) * 1.0f, tot);
        ora_square_bwd(diff, gsq, gy, tot); /* Sub passes the gradient to its left input unchanged */
        free(diff); free(sq); free(gsq);
    }
    /* backward */
    float *g = gy; /* gradient w.r.t. h[L] */
    for (int l = L - 1; l >= 0; --l) {
        size_t K = d[l], N = d[l + 1];
        int act = (l + 1 < L) || A->relu_last;
        float *gz;
        if (act) { gz = ora_alloc(B * N); ora_relu_bwd(z[l], g, gz, B * N); free(g); }
        else gz = g;
        ora_colsum(gz, A->gb[l], B, N);
        /* dW = h^T . gz */
        float *ht = ora_alloc(K * B);
        if (A->as_written) ora_transpose_as_written(h[l], ht, B, K); else ora_transpose(h[l], ht, B, K);
        if (A->as_written) { ora_touch_copy(ht, K * B); ora_touch_copy(gz, B * N); }
        ora_matmul(ht, gz, A->gw[l], K, N, B);
        free(ht);
        float *gprev = NULL;
        if (l > 0 || A->gx) {
            float *wt = ora_alloc(N * K);
            if (A->as_written) ora_transpose_as_written(A->w[l], wt, K, N); else ora_transpose(A->w[l], wt, K, N);
            gprev = (l > 0) ? ora_alloc(B * K) : A->gx;
            if (A->as_written) { ora_touch_copy(gz, B * N); ora_touch_copy(wt, N * K); }
            ora_matmul(gz, wt, gprev, B, K, N);
            free(wt);
        }
        free(gz);
        g = gprev;
    }
    for (int l = 0; l < L; ++l) {
        int act = (l + 1 < L) || A->relu_last;
        if (act) free(h[l + 1]);
        free(z[l]);
    }
    free(z); free(h);
    if (A->do_adam) {
        for (int l = 0; l < L; ++l) {
            ora_adam_update(A->w[l], A->gw[l], A->mw[l], A->vw[l], d[l] * d[l + 1], A->lr, A->beta1,
                            A->beta2, A->eps, A->weight_decay, A->step);
            ora_adam_update(A->b[l], A->gb[l], A->mb[l], A->vb[l], d[l + 1], A->lr, A->beta1,
                            A->beta2, A->eps, A->weight_decay, A->step);
        }
    }
    return loss;
}
