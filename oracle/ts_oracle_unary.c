/*
 * CPU oracle, part 2: the unary / scalar elementwise ops and softmax that sit next to the
 * training-step hot path (the ops every example network of the reference uses besides ReLU).
 *
 * TEST INFRASTRUCTURE ONLY, like ts_oracle.c: the checker of the CUDA kernels, never a
 * product path.
 *
 * Parity pin: the reference is Rust; f32::exp / ln / tanh / powf lower to the platform
 * libm (expf, logf, tanhf, powf of glibc on x86_64 Linux), which is what this file calls,
 * and sqrt is the correctly rounded IEEE operation in both.  Every other step is one
 * rounded f32 operation written in the reference's association order (-ffp-contract=off).
 * Pinned by the literal known answers of the reference's unit tests
 * (tests/golden/reference_known_answers.json) and by its LibTorch differential procedures
 * replayed with PyTorch (tests/golden/torch_unary.npz).
 */
#include <math.h>
#include <stddef.h>

#define ORA_API __attribute__((visibility("default")))

/* Operation codes shared with include/train_station_b200.h (ts_unary_op). */
enum {
    ORA_EXP = 0, ORA_LOG = 1, ORA_SQRT = 2, ORA_TANH = 3, ORA_SIGMOID = 4, ORA_LEAKY_RELU = 5,
    ORA_ADD_SCALAR = 6, ORA_SUB_SCALAR = 7, ORA_MUL_SCALAR = 8, ORA_DIV_SCALAR = 9, ORA_POW_SCALAR = 10
};

/* Forward.  Returns 0, or -1 where the reference panics (log of x <= 0: tensor/ops/log.rs:68-107;
 * division by a zero scalar: tensor/ops/div.rs:511-514); `out` is still filled with the IEEE result. */
ORA_API int ora_unary(int op, const float *x, float *out, size_t n, float p) {
    int status = 0;
    for (size_t i = 0; i < n; ++i) {
        const float v = x[i];
        float y;
        switch (op) {
            case ORA_EXP: y = expf(v); break;                               /* tensor/ops/exp.rs:148-163 */
            case ORA_LOG: if (!(v > 0.0f)) status = -1; y = logf(v); break; /* tensor/ops/log.rs:68-107 */
            case ORA_SQRT: y = sqrtf(v); break;                             /* tensor/ops/sqrt.rs:136-280 */
            case ORA_TANH: y = tanhf(v); break;                             /* tensor/ops/tanh.rs:174-190 */
            case ORA_SIGMOID:                                               /* tensor/ops/sigmoid.rs:90-110 */
                if (v >= 0.0f) { float z = expf(-v); y = 1.0f / (1.0f + z); }
                else { float z = expf(v); y = z / (1.0f + z); }
                break;
            case ORA_LEAKY_RELU: y = v > 0.0f ? v : p * v; break;           /* tensor/ops/leaky_relu.rs:124-330 */
            case ORA_ADD_SCALAR: y = v + p; break;                          /* tensor/ops/add.rs:450 ff. */
            case ORA_SUB_SCALAR: y = v - p; break;                          /* tensor/ops/sub.rs:504 ff. */
            case ORA_MUL_SCALAR: y = v * p; break;                          /* tensor/ops/mul.rs:495 ff. */
            case ORA_DIV_SCALAR: if (p == 0.0f) status = -1; y = v / p; break; /* tensor/ops/div.rs:511-575 */
            case ORA_POW_SCALAR:                                            /* tensor/ops/pow.rs:125-160, :446-462 */
                if (p == 2.0f) y = v * v;
                else if (p == 0.5f) y = sqrtf(v);
                else y = powf(v, p);
                break;
            default: return -2;
        }
        out[i] = y;
    }
    return status;
}

/* Backward.  `saved` is what the reference's GradFn keeps: the OUTPUT for exp, sqrt, tanh and sigmoid,
 * the INPUT for log, leaky_relu and pow_scalar; unused for the scalar ops. */
ORA_API int ora_unary_backward(int op, const float *saved, const float *go, float *gi, size_t n, float p) {
    for (size_t i = 0; i < n; ++i) {
        const float g = go[i];
        const float s = saved ? saved[i] : 0.0f;
        float r;
        switch (op) {
            case ORA_EXP: r = g * s; break;                                  /* grad_fn/ops/exp.rs:3-6 */
            case ORA_LOG: { float inv = 1.0f / s; r = g * inv; break; }      /* grad_fn/ops/log.rs:3-17 */
            case ORA_SQRT: { float inv = 1.0f / s; float sc = inv * 0.5f; r = g * sc; break; } /* grad_fn/ops/sqrt.rs:3-20 */
            case ORA_TANH: { float tt = s * s; r = g * (1.0f - tt); break; } /* grad_fn/ops/tanh.rs:4-17 */
            case ORA_SIGMOID: { float gs = g * s; r = gs * (1.0f - s); break; } /* grad_fn/ops/sigmoid.rs:4-17 */
            case ORA_LEAKY_RELU: r = s > 0.0f ? g : p * g; break;            /* grad_fn/ops/leaky_relu.rs:4-25 */
            case ORA_ADD_SCALAR:
            case ORA_SUB_SCALAR: r = g; break;                               /* grad_fn/ops/add.rs:9-11, sub.rs:9-11 */
            case ORA_MUL_SCALAR: r = g * p; break;                           /* grad_fn/ops/mul.rs:11-14 */
            case ORA_DIV_SCALAR: r = g / p; break;                           /* grad_fn/ops/div.rs:11-14 */
            case ORA_POW_SCALAR: {                                           /* grad_fn/ops/pow.rs:5-27 */
                float local = p == 0.0f ? 0.0f : p * powf(s, p - 1.0f);
                r = g * local;
                break;
            }
            default: return -2;
        }
        gi[i] = r;
    }
    return 0;
}

/* softmax over the middle axis of [outer, reduce, inner]: tensor/ops/softmax.rs:110-158.
 * max, e = exp(x - max) with a sequential f32 sum, then e * (1 / sum). */
ORA_API void ora_softmax(const float *x, float *y, size_t outer, size_t reduce, size_t inner) {
    for (size_t o = 0; o < outer; ++o)
        for (size_t i = 0; i < inner; ++i) {
            const size_t base = o * reduce * inner + i;
            float mx = -INFINITY;
            for (size_t j = 0; j < reduce; ++j) {
                float v = x[base + j * inner];
                if (v > mx) mx = v;
            }
            float sum = 0.0f;
            for (size_t j = 0; j < reduce; ++j) {
                float e = expf(x[base + j * inner] - mx);
                y[base + j * inner] = e;
                sum += e;
            }
            const float inv = 1.0f / sum;
            for (size_t j = 0; j < reduce; ++j) y[base + j * inner] *= inv;
        }
}

/* grad_fn/ops/softmax.rs:4-35: dot = sum_j go*y (sequential), gi = y * (go - dot). */
ORA_API void ora_softmax_backward(const float *y, const float *go, float *gi, size_t outer, size_t reduce, size_t inner) {
    for (size_t o = 0; o < outer; ++o)
        for (size_t i = 0; i < inner; ++i) {
            const size_t base = o * reduce * inner + i;
            float dot = 0.0f;
            for (size_t j = 0; j < reduce; ++j) {
                float pr = go[base + j * inner] * y[base + j * inner];
                dot += pr;
            }
            for (size_t j = 0; j < reduce; ++j) gi[base + j * inner] = y[base + j * inner] * (go[base + j * inner] - dot);
        }
}
