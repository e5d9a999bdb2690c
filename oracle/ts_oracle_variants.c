/*
 * CPU oracle, part 3: the AMSGrad branch of Adam and the seeded normal initialiser.
 *
 * TEST INFRASTRUCTURE ONLY, like ts_oracle.c: the checker of the device library, never a product path.
 *
 * Parity pin: restated from the reference's source.  AMSGrad is pinned by the reference's LibTorch
 * procedure replayed with PyTorch (tests/golden/torch_differential.npz, the adam*_amsgrad cases).  randn
 * has no literal values in the reference's tests (they check reproducibility and moments only): its
 * integer generator is pinned here by values worked out with arbitrary-precision integers in
 * tests/test_oracle_variants.py, and the float stage calls the same libm (logf, sqrtf, cosf) that Rust's
 * f32::ln / sqrt / cos lower to on x86_64 Linux.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

#define ORA_API __attribute__((visibility("default")))

/*
 * optimizers/adam/mod.rs:485-556 with config.amsgrad: after the moment updates and the bias corrections,
 * v_hat_max = max(v_hat_max, v_hat) elementwise (`if a > b { a } else { b }`, :846-900) on the
 * BIAS-CORRECTED second moment, and the update divides by sqrt(v_hat_max) + eps.  The reference creates
 * v_hat_max as a copy of the first v_hat; a zero-initialised buffer gives the same maxima because v_hat >= 0.
 * Body/tail association of (1-beta2)*g*g as in ora_adam_update (:761-772).
 */
ORA_API void ora_adam_update_amsgrad(float *p, const float *g_in, float *m, float *v, float *vmax, size_t n,
                                     float lr, float beta1, float beta2, float eps, float weight_decay,
                                     uint64_t step) {
    float stepf = (float)step;
    float bc1 = (float)(1.0 - pow((double)beta1, (double)stepf));
    float bc2 = (float)(1.0 - pow((double)beta2, (double)stepf));
    float f1 = 1.0f / bc1, f2 = 1.0f / bc2;
    float c1 = 1.0f - beta1, c2 = 1.0f - beta2;
    size_t body = n / 8 * 8;
    for (size_t i = 0; i < n; ++i) {
        float g = g_in[i];
        if (weight_decay > 0.0f) g = g + weight_decay * p[i];
        float mi = (beta1 * m[i]) + (c1 * g);
        float vi = i < body ? (beta2 * v[i]) + (c2 * (g * g)) : (beta2 * v[i]) + ((c2 * g) * g);
        m[i] = mi;
        v[i] = vi;
        float mh = mi * f1, vh = vi * f2;
        float a = vmax[i];
        float mx = a > vh ? a : vh;
        vmax[i] = mx;
        p[i] = p[i] - ((lr * mh) / (sqrtf(mx) + eps));
    }
}

/*
 * tensor/init/random.rs:473-616.  XorShiftRng: state = seed; next_u64 is xorshift64 with shifts 13, 7, 17
 * (:524-529); next_f32 puts the low 23 bits under exponent field 126 (:557-563), i.e. a value in
 * [0.5, 1) although the comment there says [0, 1); next_normal draws u1 then u2 and returns
 * sqrt(-2 ln u1) * cos(2 pi u2), replacing NaN or infinity by 0 (:592-616).  The u1 clamps (:598-604)
 * can never fire for values in [0.5, 1) and are kept for fidelity.  A zero seed leaves the state at
 * zero for ever (every draw is 0.5), as in the reference.
 */
static inline uint64_t ora_xorshift_next(uint64_t *s) {
    *s ^= *s << 13;
    *s ^= *s >> 7;
    *s ^= *s << 17;
    return *s;
}
static inline float ora_next_f32(uint64_t *s) {
    uint32_t bits = (uint32_t)(ora_xorshift_next(s) & 0x7FFFFFu) | (126u << 23);
    union { uint32_t u; float f; } c;
    c.u = bits;
    return c.f;
}
ORA_API void ora_xorshift_u64(uint64_t seed, uint64_t *out, size_t n) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; ++i) out[i] = ora_xorshift_next(&s);
}
ORA_API void ora_randn(float *out, size_t n, uint64_t seed) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; ++i) {
        float u1 = ora_next_f32(&s);
        float u2 = ora_next_f32(&s);
        if (u1 <= 0.0f) u1 = 1e-7f;
        else if (u1 >= 1.0f) u1 = 1.0f - 1e-7f;
        float r = sqrtf(-2.0f * logf(u1));
        float c = cosf((2.0f * 3.14159265358979323846f) * u2);
        float z = r * c;
        out[i] = (isnan(z) || isinf(z)) ? 0.0f : z;
    }
}
