/*
 * CPU restatement of oxidizr's data-parallel optimizer step.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is the checker for the CUDA path and the
 * timed CPU baseline; nothing in the product library links, loads or calls it.
 *
 * PARITY STATUS
 *   The reference is Rust and its arithmetic for this path lives in the
 *   un-vendored crates boostr 0.10.0 / numr 0.14.0 (Cargo.lock:281-284, 2075-2078),
 *   whose source is not available and which cannot be built without a Rust
 *   toolchain. This restatement therefore follows the reference's own call
 *   sites, documentation and tests:
 *     - pinned by known answers in the reference's tests (see tests/test_oracle_pins.py):
 *       the sum over ranks, the unscale, the value-clamp / norm-clip ordering and
 *       the returned norm, the non-finite rule, the zero-gradient decay behaviour,
 *       skip_all == weight_decay 0, and the skip semantics;
 *     - PARITY UNPINNED (no reference test fixes a number): the exact AdamW update
 *       form (eps placement, decay order), the clip coefficient's epsilon, and the
 *       accumulation type of the sum of squares. Each is a named switch below with
 *       the conventional default.
 *
 * The structure is deliberately the reference's: one pass per operation, per
 * tensor (cast, scale, square-sum, clamp, scale, AdamW), parallelised over the
 * host cores with OpenMP as boostr/numr's CPU backend is with rayon.
 *
 * Build: gcc -O3 -march=native -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
 * -ffp-contract=off matters: every f32 operation below rounds once, exactly as
 * the CUDA kernels' explicit round-to-nearest intrinsics do.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_F32 0
#define ORC_BF16 1
#define ORC_F16 2

/* ---- scalar conversions ------------------------------------------------ */

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even, NaN stays NaN (quiet), as half 2.7.1's bf16::from_f32 does */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            man &= 0x3ffu;
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even f32 -> f16 with overflow to inf and gradual underflow */
static inline uint16_t f32_to_f16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((a >> 13) & 0x3ffu));
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u); /* >= 65536 or inf */
    if (a < 0x33000000u) return (uint16_t)sign;              /* < 2^-25 rounds to 0 */
    int32_t exp = (int32_t)(a >> 23) - 127;
    uint32_t man = (a & 0x7fffffu) | 0x800000u;
    uint32_t shift, half;
    if (exp < -14) { /* subnormal result */
        shift = (uint32_t)(13 + (-14 - exp));
        half = 0;
    } else {
        shift = 13;
        half = (uint32_t)(exp + 15) << 10;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (q & 1u))) q++;
    if (exp < -14) return (uint16_t)(sign | q); /* q may carry into the normal range: correct */
    /* q includes the hidden bit at position 10; adding carries into the exponent correctly */
    uint32_t r = half + (q - 0x400u);
    if (r >= 0x7c00u) r = 0x7c00u;
    return (uint16_t)(sign | r);
}

static inline float load_as_f32(const void* p, int dtype, size_t i) {
    switch (dtype) {
        case ORC_BF16: return bf16_to_f32(((const uint16_t*)p)[i]);
        case ORC_F16: return f16_to_f32(((const uint16_t*)p)[i]);
        default: return ((const float*)p)[i];
    }
}

/* conversion helpers exported for the tests */
void orc_f32_to_bf16(const float* in, uint16_t* out, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = f32_to_bf16(in[i]);
}
void orc_f32_to_f16(const float* in, uint16_t* out, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = f32_to_f16(in[i]);
}
void orc_widen(const void* in, int dtype, float* out, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = load_as_f32(in, dtype, i);
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n > 0 ? n : 1);
#else
    (void)n;
#endif
}

/* ---- one pass per operation, as the reference issues them --------------- */

/*
 * Sum of one tensor's gradient over `world` ranks: widen each rank's values to
 * f32 and add them in rank order 0..world-1. Never divided by the world size.
 * Follows src/dp/reduce.rs:11-29 ("The sum is never divided by the world size",
 * "After the call every gradient is f32"); known answer src/dp/reduce.rs:88-121.
 */
void orc_sum_ranks(const void* const* rank_grads, int world, int dtype, size_t n, float* out) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float s = load_as_f32(rank_grads[0], dtype, i);
        for (int r = 1; r < world; r++) s = s + load_as_f32(rank_grads[r], dtype, i);
        out[i] = s;
    }
}

/*
 * Unscale of one gradient: widen to f32 first, then multiply by 1/scale, the
 * reciprocal formed in f64 and applied as an f32 scalar.
 * Follows src/loss_scale/scaler.rs:63-87 (inv_scale at :73, cast at :82, mul_scalar at :84).
 */
void orc_unscale(const void* in, int dtype, size_t n, double scale, float* out) {
    const float inv = (float)(1.0 / scale);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = load_as_f32(in, dtype, i) * inv;
}

/*
 * Sum of squares of one f32 tensor. Each square is formed in f32 (so a value
 * above ~1.8e19 squares to +inf: src/grad_clip.rs:85 "each square still fits in
 * f32, so the raw norm is finite") and the squares accumulate in f64.
 * SWITCH (parity unpinned): the accumulation type; f64 here.
 * The chunking is fixed, so the result does not depend on the thread count.
 */
double orc_sumsq(const float* g, size_t n) {
    const size_t CH = 1u << 16;
    size_t nch = (n + CH - 1) / CH;
    double total = 0.0;
    double* part = (double*)malloc((nch ? nch : 1) * sizeof(double));
#pragma omp parallel for schedule(static)
    for (size_t c = 0; c < nch; c++) {
        size_t lo = c * CH, hi = lo + CH < n ? lo + CH : n;
        double s = 0.0;
        for (size_t i = lo; i < hi; i++) {
            float q = g[i] * g[i];
            s += (double)q;
        }
        part[c] = s;
    }
    for (size_t c = 0; c < nch; c++) total += part[c];
    free(part);
    return total;
}

/* Clamp every element to [-v, v]; NaN stays NaN. boostr clip_grad_value, called at src/grad_clip.rs:53. */
void orc_clamp(float* g, size_t n, double v) {
    const float hi = (float)v, lo = -(float)v;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float x = g[i];
        x = x > hi ? hi : x;
        x = x < lo ? lo : x;
        g[i] = x;
    }
}

/* In-place scale by an f32 coefficient: the rescale half of boostr clip_grad_norm (src/grad_clip.rs:55). */
void orc_scale(float* g, size_t n, float c) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) g[i] = g[i] * c;
}

/*
 * The per-step scalars of AdamW, prepared in f64 and rounded to f32 once.
 * t is the 1-based count of APPLIED steps (src/trainer.rs:906-908, tests/loss_scale.rs:118-176).
 */
typedef struct {
    float beta1, one_minus_beta1, beta2, one_minus_beta2;
    float eps;
    float bias2_sqrt;  /* sqrt(1 - beta2^t) */
    float step_size;   /* lr*lr_scale / (1 - beta1^t)            (eps_mode 0)
                          lr*lr_scale * sqrt(1-beta2^t)/(1-beta1^t) (eps_mode 1) */
    float decay_mul;   /* 1 - lr*lr_scale*weight_decay ; exactly 1.0f when weight_decay == 0 */
    int32_t decay_after; /* SWITCH: 0 = decay first (default), 1 = decay after the Adam term */
    int32_t eps_mode;    /* SWITCH: 0 = sqrt(v)/sqrt(bc2) + eps (default), 1 = sqrt(v) + eps */
} orc_adam_scalars;

void orc_adam_prepare(double lr, double lr_scale, double beta1, double beta2, double eps, double weight_decay,
                      uint64_t t, int32_t decay_after, int32_t eps_mode, orc_adam_scalars* out) {
    double bc1 = 1.0 - pow(beta1, (double)t);
    double bc2 = 1.0 - pow(beta2, (double)t);
    double lr_t = lr * lr_scale;
    out->beta1 = (float)beta1;
    out->one_minus_beta1 = (float)(1.0 - beta1);
    out->beta2 = (float)beta2;
    out->one_minus_beta2 = (float)(1.0 - beta2);
    out->eps = (float)eps;
    out->bias2_sqrt = (float)sqrt(bc2);
    out->step_size = eps_mode == 0 ? (float)(lr_t / bc1) : (float)(lr_t * sqrt(bc2) / bc1);
    out->decay_mul = (float)(1.0 - lr_t * weight_decay);
    out->decay_after = decay_after;
    out->eps_mode = eps_mode;
}

/*
 * AdamW with decoupled weight decay on one tensor (boostr optimizer::AdamW, called at
 * src/trainer.rs:649, configured at src/trainer.rs:184-193 with the zero-decay group of
 * src/weight_decay/plan.rs:113-122). p is the f32 master; `work` receives the
 * narrowed working weight (models/llama-3.2-1b.yaml:54-57) or is NULL for f32 params.
 * Pinned only relationally: tests/weight_decay.rs:102-147 and :165-187.
 */
void orc_adamw(float* p, float* m, float* v, const float* g, size_t n, const orc_adam_scalars* s, void* work,
               int work_dtype) {
    const orc_adam_scalars k = *s;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float pi = p[i], gi = g[i];
        if (!k.decay_after) pi = pi * k.decay_mul;
        float t1 = k.beta1 * m[i];
        float t2 = k.one_minus_beta1 * gi;
        float mi = t1 + t2;
        float gg = gi * gi;
        float t3 = k.beta2 * v[i];
        float t4 = k.one_minus_beta2 * gg;
        float vi = t3 + t4;
        float root = sqrtf(vi);
        float denom = k.eps_mode == 0 ? (root / k.bias2_sqrt) + k.eps : root + k.eps;
        float q = mi / denom;
        float u = k.step_size * q;
        pi = pi - u;
        if (k.decay_after) pi = pi * k.decay_mul;
        p[i] = pi;
        m[i] = mi;
        v[i] = vi;
        if (work) {
            if (work_dtype == ORC_BF16) ((uint16_t*)work)[i] = f32_to_bf16(pi);
            else if (work_dtype == ORC_F16) ((uint16_t*)work)[i] = f32_to_f16(pi);
            else ((float*)work)[i] = pi;
        }
    }
}

/*
 * One call of boostr clip_grad_norm as oxidizr uses it (compute_grad_norm, src/prelude.rs:13): measure the global
 * L2 norm of the gradients as they are now, and when it is finite and above `max_norm` scale every gradient in place
 * by the f32 coefficient max_norm / (norm + eps). Returns the measured norm. Called for the max-norm clip
 * (src/grad_clip.rs:55) and, with the target as the limit, for the optional second clip (src/trainer.rs:635-645).
 * SWITCH (parity unpinned): eps, 1e-6 by default.
 */
static double clip_norm_pass(size_t T, const size_t* numel, float* const* g, const uint8_t* present, double max_norm,
                             double eps, double* coef) {
    double ss = 0.0;
    for (size_t i = 0; i < T; i++)
        if (present[i]) ss += orc_sumsq(g[i], numel[i]);
    double norm = sqrt(ss);
    if (isfinite(norm) && norm > max_norm) {
        float c = (float)(max_norm / (norm + eps));
        for (size_t i = 0; i < T; i++)
            if (present[i]) orc_scale(g[i], numel[i], c);
        *coef *= (double)c;
    }
    return norm;
}

/*
 * clip_gradients (src/grad_clip.rs:36-56) over T f32 gradients in place (present[i] == 0: tensor i has none):
 * with a value clip, the raw norm first; a non-finite raw norm returns as is, before any clamp; else clamp every
 * element, then the norm clip. Returns the norm the norm clip measured; *coef is multiplied by the coefficient applied.
 * orc_step calls this function, and the reference's known answers (src/grad_clip.rs:82-143) are checked on it.
 */
double orc_clip_gradients(size_t T, const size_t* numel, float* const* g, const uint8_t* present, double max_grad_value,
                          double max_grad_norm, double clip_eps, double* coef) {
    int value_clip = max_grad_value == max_grad_value;
    if (value_clip) {
        double raw = 0.0;
        for (size_t i = 0; i < T; i++)
            if (present[i]) raw += orc_sumsq(g[i], numel[i]);
        raw = sqrt(raw);
        if (!isfinite(raw)) return raw;
        for (size_t i = 0; i < T; i++)
            if (present[i]) orc_clamp(g[i], numel[i], max_grad_value);
    }
    return clip_norm_pass(T, numel, g, present, max_grad_norm, clip_eps, coef);
}

/* ---- the whole post-accumulation step, src/trainer.rs:515-695 ------------ */

typedef struct {
    double lr, beta1, beta2, eps, weight_decay;
    double max_grad_norm;
    double max_grad_value;   /* NaN: off */
    double target_grad_norm; /* NaN: off */
    double loss_scale;       /* NaN or 0: no scaler (bf16 / f32 runs) */
    double clip_eps;         /* SWITCH: 1e-6 (default) or 0 */
    int32_t decay_after, eps_mode;
    int32_t spike_skip; /* the spike guard's verdict for this step (src/metrics/state.rs:79-86) */
    int32_t absent_mode; /* SWITCH: 0 = a tensor with no gradient is left untouched (default) */
} orc_hyper;

typedef struct {
    double grad_norm;     /* the norm the norm clip measured (src/grad_clip.rs:28-35) */
    double reported_norm; /* what training_step returns (src/trainer.rs:629-632, 657-661) */
    double clip_coef;     /* product of the coefficients applied to the gradients */
    int32_t overflow;     /* !grad_norm.is_finite()   (src/trainer.rs:619) */
    int32_t applied;      /* optimizer.step ran       (src/trainer.rs:649) */
    uint64_t timestep;    /* applied steps after this one */
} orc_result;

/*
 * One optimizer step over T tensors.
 *   rank_grads[r*T + i]: rank r's gradient of tensor i in `grad_dtype`, or NULL when that rank produced none.
 *   A tensor with no gradient on any rank has none after the sum (src/dp/reduce.rs:20) and is
 *   skipped by every later pass (src/loss_scale/scaler.rs:75-77).
 *   scratch: n_total f32 values of working space for the f32 gradients.
 *   group_wd[i]: NaN = the base weight_decay, else the group's override (0.0 for the no-decay group).
 */
void orc_step(size_t T, const size_t* numel, const void* const* rank_grads, int world, int grad_dtype,
              float* const* master, float* const* exp_avg, float* const* exp_avg_sq, void* const* work, int work_dtype,
              const double* lr_scale, const double* group_wd, uint64_t timestep, const orc_hyper* h, float* scratch,
              orc_result* res) {
    float** g = (float**)malloc(T * sizeof(float*));
    uint8_t* present = (uint8_t*)calloc(T, 1);
    const void** per_rank = (const void**)malloc((size_t)world * sizeof(void*));
    size_t off = 0;

    /* A2: the gradient sum over ranks (src/trainer.rs:520-527). World 1 keeps the tensors as they are. */
    for (size_t i = 0; i < T; i++) {
        g[i] = scratch + off;
        off += numel[i];
        int have = 0;
        for (int r = 0; r < world; r++) have |= rank_grads[(size_t)r * T + i] != NULL;
        present[i] = (uint8_t)have;
        if (!have) continue;
        if (world == 1) {
            orc_widen(rank_grads[i], grad_dtype, g[i], numel[i]);
        } else {
            /* a rank without this gradient contributes zeros */
            int nr = 0;
            for (int r = 0; r < world; r++)
                if (rank_grads[(size_t)r * T + i]) per_rank[nr++] = rank_grads[(size_t)r * T + i];
            orc_sum_ranks(per_rank, nr, grad_dtype, numel[i], g[i]);
        }
    }

    /* A3: unscale (src/trainer.rs:573-575). */
    int scaled = h->loss_scale == h->loss_scale && h->loss_scale != 0.0;
    if (scaled) {
        for (size_t i = 0; i < T; i++)
            if (present[i]) orc_unscale(g[i], ORC_F32, numel[i], h->loss_scale, g[i]);
    }

    /* A4: clip_gradients (src/grad_clip.rs:36-56). */
    double coef = 1.0;
    double norm = orc_clip_gradients(T, numel, g, present, h->max_grad_value, h->max_grad_norm, h->clip_eps, &coef);

    /* A5: the skip decision (src/trainer.rs:611-633). */
    int overflow = !isfinite(norm);
    res->grad_norm = norm;
    res->overflow = overflow;
    res->applied = 0;
    res->timestep = timestep;
    res->reported_norm = norm;
    if (!overflow && !h->spike_skip) {
        /* A6: optional tighter clip (src/trainer.rs:635-645). */
        double eff = norm < h->max_grad_norm ? norm : h->max_grad_norm;
        int has_target = h->target_grad_norm == h->target_grad_norm;
        if (has_target && eff > h->target_grad_norm && eff > 1e-8) {
            /* the same utility once more, on the gradients as the first clip left them: it measures them AGAIN
               and rescales by target / (measured + eps). After a max-norm clip the measured norm is about
               max * norm / (norm + eps), a little under max, so this is not target / (max + eps). */
            (void)clip_norm_pass(T, numel, g, present, h->target_grad_norm, h->clip_eps, &coef);
        }
        /* A7: optimizer.step (src/trainer.rs:649). */
        uint64_t t = timestep + 1;
        for (size_t i = 0; i < T; i++) {
            if (!present[i]) continue;
            double wd = group_wd[i] == group_wd[i] ? group_wd[i] : h->weight_decay;
            orc_adam_scalars s;
            orc_adam_prepare(h->lr, lr_scale[i], h->beta1, h->beta2, h->eps, wd, t, h->decay_after, h->eps_mode, &s);
            orc_adamw(master[i], exp_avg[i], exp_avg_sq[i], g[i], numel[i], &s, work ? work[i] : NULL, work_dtype);
        }
        res->applied = 1;
        res->timestep = t;
        double rep = norm < h->max_grad_norm ? norm : h->max_grad_norm;
        if (has_target && h->target_grad_norm < rep) rep = h->target_grad_norm;
        res->reported_norm = rep;
    }
    res->clip_coef = coef;
    free(per_rank);
    free(present);
    free(g);
}
