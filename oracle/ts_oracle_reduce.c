/*
 * CPU oracle, part 4: reductions over axes (and the whole-tensor max / min / norm / var / std) with their
 * backward passes.
 *
 * TEST INFRASTRUCTURE ONLY, like ts_oracle.c: the checker of the device library, never a product path.
 *
 * Restated from tensor/reductions/{sum,mean,max,min,norm,var,std}.rs and the files of gradtrack/grad_fn/reductions/ in the
 * reference's order of accumulation: the *_dims forms walk the input in linear order and add each element into
 * its output slot; the whole-tensor forms are single sequential chains (norm and std add groups of four).
 * Pinned by the literal values of the reference's unit tests (tests/golden/reference_known_answers.json) and by
 * f64 evaluations in tests/test_oracle_reduce.py.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#define ORA_API __attribute__((visibility("default")))

enum { R_SUM = 0, R_MEAN = 1, R_MAX = 2, R_MIN = 3, R_NORM = 4, R_VAR = 5, R_STD = 6 };

/* output offset of input element `lin`: the kept coordinates, in order, under the output's contiguous strides
 * (sum.rs:262-285; identical with and without keepdim because extent-1 axes do not move an offset) */
static size_t out_offset(size_t lin, const size_t *dims, int rank, const unsigned char *red) {
    size_t coords[8];
    for (int i = rank - 1; i >= 0; --i) {
        size_t s = dims[i];
        coords[i] = s ? lin % s : 0;
        if (s) lin /= s;
    }
    size_t off = 0;
    for (int i = 0; i < rank; ++i)
        if (!red[i]) off = off * dims[i] + coords[i];
    return off;
}
static size_t count_out(const size_t *dims, int rank, const unsigned char *red, size_t *factor) {
    size_t n = 1, f = 1;
    for (int i = 0; i < rank; ++i) { if (red[i]) f *= dims[i]; else n *= dims[i]; }
    if (factor) *factor = f;
    return n;
}

/* forward over axes.  out: n_out elements; mean_out (n_out, may be NULL): the per-output mean of var / std. */
ORA_API int ora_reduce_dims(int kind, const float *x, float *out, float *mean_out, const size_t *dims, int rank,
                            const unsigned char *red) {
    size_t factor, n_out = count_out(dims, rank, red, &factor), n = n_out * factor;
    if (rank < 1 || rank > 8) return -2;
    for (size_t o = 0; o < n_out; ++o) out[o] = kind == R_MAX ? -INFINITY : kind == R_MIN ? INFINITY : 0.0f;
    if (kind == R_SUM || kind == R_MEAN) {                 /* sum.rs:250-290; mean.rs:186-200 */
        for (size_t i = 0; i < n; ++i) out[out_offset(i, dims, rank, red)] += x[i];
        if (kind == R_MEAN) {
            float scale = factor > 0 ? 1.0f / (float)factor : 0.0f;
            for (size_t o = 0; o < n_out; ++o) out[o] = out[o] * scale;
        }
    } else if (kind == R_MAX) {                            /* max.rs:90-130: `if val > cur` */
        for (size_t i = 0; i < n; ++i) { size_t o = out_offset(i, dims, rank, red); if (x[i] > out[o]) out[o] = x[i]; }
    } else if (kind == R_MIN) {
        for (size_t i = 0; i < n; ++i) { size_t o = out_offset(i, dims, rank, red); if (x[i] < out[o]) out[o] = x[i]; }
    } else if (kind == R_NORM) {                           /* norm.rs:202-290 */
        for (size_t i = 0; i < n; ++i) { float v = x[i]; out[out_offset(i, dims, rank, red)] += v * v; }
        for (size_t o = 0; o < n_out; ++o) out[o] = sqrtf(out[o]);
    } else if (kind == R_VAR || kind == R_STD) {           /* var.rs:294-420, std.rs:316-440: two passes, divide by the count */
        float *mu = mean_out ? mean_out : (float *)malloc((n_out ? n_out : 1) * sizeof(float));
        for (size_t o = 0; o < n_out; ++o) mu[o] = 0.0f;
        for (size_t i = 0; i < n; ++i) mu[out_offset(i, dims, rank, red)] += x[i];
        for (size_t o = 0; o < n_out; ++o) mu[o] /= (float)factor;
        for (size_t i = 0; i < n; ++i) { size_t o = out_offset(i, dims, rank, red); float d = x[i] - mu[o]; out[o] += d * d; }
        for (size_t o = 0; o < n_out; ++o) { out[o] /= (float)factor; if (kind == R_STD) out[o] = sqrtf(out[o]); }
        if (!mean_out) free(mu);
    } else return -2;
    return 0;
}

/* whole-tensor forms, result one value (max.rs:30-60, min.rs:39-70, norm.rs:80-125, var.rs:101-165, std.rs:102-175) */
ORA_API float ora_reduce_all(int kind, const float *x, size_t n, float *mean_out) {
    if (kind == R_MAX) { float m = -INFINITY; for (size_t i = 0; i < n; ++i) if (x[i] > m) m = x[i]; return m; }
    if (kind == R_MIN) { float m = INFINITY; for (size_t i = 0; i < n; ++i) if (x[i] < m) m = x[i]; return m; }
    if (kind == R_NORM) {
        float s = 0.0f;
        size_t i = 0;
        for (; i + 4 <= n; i += 4) s += x[i] * x[i] + x[i + 1] * x[i + 1] + x[i + 2] * x[i + 2] + x[i + 3] * x[i + 3];
        for (; i < n; ++i) s += x[i] * x[i];
        return sqrtf(s);
    }
    if (n == 0) { if (mean_out) *mean_out = 0.0f; return 0.0f; }
    float mean = 0.0f, var = 0.0f;
    if (kind == R_VAR) {                 /* plain sequential chains */
        for (size_t i = 0; i < n; ++i) mean += x[i];
        mean /= (float)n;
        for (size_t i = 0; i < n; ++i) { float d = x[i] - mean; var += d * d; }
        var /= (float)n;
        if (mean_out) *mean_out = mean;
        return var;
    }
    size_t i = 0;                        /* std: groups of four */
    for (; i + 4 <= n; i += 4) mean += x[i] + x[i + 1] + x[i + 2] + x[i + 3];
    for (; i < n; ++i) mean += x[i];
    mean /= (float)n;
    for (i = 0; i + 4 <= n; i += 4) {
        float a = x[i] - mean, b = x[i + 1] - mean, c = x[i + 2] - mean, d = x[i + 3] - mean;
        var += a * a + b * b + c * c + d * d;
    }
    for (; i < n; ++i) { float d = x[i] - mean; var += d * d; }
    var /= (float)n;
    if (mean_out) *mean_out = mean;
    return sqrtf(var);
}

/* backward (the files of gradtrack/grad_fn/reductions/).  y: the forward result (n_out values), mean: per-output means for
 * var / std, go: n_out values or one value when go_is_scalar.  A whole-tensor reduction is `red` all ones. */
ORA_API int ora_reduce_dims_backward(int kind, const float *x, const float *y, const float *mean, const float *go, float *gi,
                                     const size_t *dims, int rank, const unsigned char *red, int go_is_scalar) {
    size_t factor, n_out = count_out(dims, rank, red, &factor), n = n_out * factor;
    float *counts = NULL;
    if (kind == R_MAX || kind == R_MIN) {          /* max.rs:40-75: ties share the gradient equally */
        counts = (float *)calloc(n_out ? n_out : 1, sizeof(float));
        for (size_t i = 0; i < n; ++i) { size_t o = out_offset(i, dims, rank, red); if (x[i] == y[o]) counts[o] += 1.0f; }
    }
    const float inv = factor > 0 ? 1.0f / (float)factor : 0.0f;
    const float inv2 = factor > 0 ? 2.0f / (float)factor : 0.0f;
    for (size_t i = 0; i < n; ++i) {
        size_t o = out_offset(i, dims, rank, red);
        float up = go_is_scalar ? go[0] : go[o];
        float g;
        switch (kind) {
            case R_SUM: g = up; break;
            case R_MEAN: g = up * inv; break;
            case R_MAX:
            case R_MIN: g = x[i] == y[o] ? (counts[o] > 0.0f ? up / counts[o] : 0.0f) : 0.0f; break;
            case R_NORM: g = y[o] > 0.0f ? x[i] * (up / y[o]) : 0.0f; break;
            case R_VAR: g = (x[i] - mean[o]) * (up * inv2); break;
            case R_STD: g = y[o] > 0.0f ? (x[i] - mean[o]) * (up * inv / y[o]) : 0.0f; break;
            default: free(counts); return -2;
        }
        gi[i] = g;
    }
    free(counts);
    return 0;
}
