/*
 * CPU oracle for the MoE expert-FFN path.  TEST INFRASTRUCTURE ONLY: this file
 * is the checker the CUDA path is compared with and the timed CPU baseline; no
 * product code path may call it.
 *
 * It restates, in plain C, the arithmetic of the reference engine's CPU int4
 * path.  Every function names the reference file:line it follows (paths are
 * relative to the reference project root).  The reference is Rust and cannot be
 * built where this oracle is built, so the restatement is pinned against the
 * reference's own known-answer tests instead (see tests/test_oracle_golden.py).
 *
 * Floating point rules shared with the CUDA kernels: IEEE fp32, no FMA
 * contraction (build with -ffp-contract=off), operations evaluated left to
 * right exactly as written in the reference, round-to-nearest-even.
 *
 * exp():  the reference calls Rust's f32::exp (the platform libm expf).  The
 * oracle and the CUDA kernels both use exp32(v) = (float)exp((double)v), the
 * correctly rounded fp32 exponential up to a ~2^-29 double-rounding chance, so
 * that the two sides agree by construction.  po_set_exp_mode(1) switches the
 * oracle to libm expf so the size of that deviation can be counted.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#if defined(__x86_64__)
#include <immintrin.h>
#endif
#ifdef _OPENMP
#include <omp.h>
#endif

#define PO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ utils */

static int g_exp_mode = 0; /* 0 = (float)exp((double)v), 1 = expf(v) */

PO_API void po_set_exp_mode(int mode) { g_exp_mode = mode; }
PO_API int po_get_exp_mode(void) { return g_exp_mode; }

static inline float exp32(float v) {
    if (g_exp_mode == 1) return expf(v);
    return (float)exp((double)v);
}

/* 64-bit LCG of the reference's fixtures:
 * crates/peregrine-model/src/testkit.rs:10-16 and
 * crates/peregrine-kernels/src/idot.rs:558-572. */
PO_API uint64_t po_lcg_next(uint64_t *state) {
    *state = *state * 6364136223846793005ULL + 1442695040888963407ULL;
    return *state;
}
/* testkit.rs:13-15: (s >> 40) / 2^24 * 2 - 1 */
PO_API void po_lcg_fill_f32(uint64_t *state, float *out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        uint64_t s = po_lcg_next(state);
        out[i] = (float)(s >> 40) / (float)(1ULL << 24) * 2.0f - 1.0f;
    }
}
/* idot.rs:566-568: ((s >> 33) as i32 % 255 - 127) as i8 */
PO_API void po_lcg_fill_i8_127(uint64_t *state, int8_t *out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        uint64_t s = po_lcg_next(state);
        int32_t v = (int32_t)(uint32_t)(s >> 33);
        out[i] = (int8_t)(v % 255 - 127);
    }
}
/* idot.rs:569-571: (s >> 40) as i32 % 16 - 8 */
PO_API void po_lcg_fill_nib(uint64_t *state, int32_t *out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        uint64_t s = po_lcg_next(state);
        out[i] = (int32_t)(uint32_t)(s >> 40) % 16 - 8;
    }
}

/* idot.rs:574-586 (test helper pack_i4); same nibble rule as
 * crates/peregrine-core/src/pack.rs:505-511. */
PO_API void po_pack_i4(const int32_t *vals, size_t n, uint8_t *out) {
    memset(out, 0, (n + 1) / 2);
    for (size_t i = 0; i < n; ++i) {
        uint8_t b = (uint8_t)(vals[i] + 8) & 0x0F;
        out[i >> 1] |= (i & 1) ? (uint8_t)(b << 4) : b;
    }
}

/* ------------------------------------------------- activation quantisation */

/* crates/peregrine-kernels/src/quant.rs:14-33 */
PO_API float po_qrow_i8(const float *x, int8_t *q, size_t n) {
    float amax = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float a = fabsf(x[i]);
        if (a > amax) amax = a;
    }
    float s = amax / 127.0f;
    if (s < 1e-12f) s = 1e-12f;
    float inv = 1.0f / s;
    for (size_t i = 0; i < n; ++i) q[i] = (int8_t)nearbyintf(x[i] * inv);
    return s;
}

/* --------------------------------------------------------- integer dots */

/* crates/peregrine-kernels/src/idot.rs:24-32 */
PO_API int32_t po_dot_i4i8_scalar(const uint8_t *w4, const int8_t *x, size_t n) {
    int32_t sum = 0;
    for (size_t i = 0; i < n; ++i) {
        uint8_t byte = w4[i >> 1];
        int32_t nib = (i & 1) ? (int32_t)(byte >> 4) : (int32_t)(byte & 0x0F);
        sum += (nib - 8) * (int32_t)x[i];
    }
    return sum;
}

#if defined(__x86_64__)
/* crates/peregrine-kernels/src/idot.rs:214-239 (maddubs sign trick over 32
 * nibbles per step, scalar tail).  Integer sums are exact, so the result equals
 * the scalar kernel bit for bit. */
__attribute__((target("avx2"))) static int32_t dot_i4i8_avx2(const uint8_t *w4, const int8_t *x, size_t n) {
    const __m128i nibmask = _mm_set1_epi8(0x0F);
    const __m256i eight = _mm256_set1_epi8(8);
    const __m256i one16 = _mm256_set1_epi16(1);
    __m256i acc = _mm256_setzero_si256();
    size_t i = 0;
    for (; i + 32 <= n; i += 32) {
        __m128i packed = _mm_loadu_si128((const __m128i *)(w4 + (i >> 1)));
        __m128i even = _mm_and_si128(packed, nibmask);
        __m128i odd = _mm_and_si128(_mm_srli_epi16(packed, 4), nibmask);
        __m256i w = _mm256_set_m128i(_mm_unpackhi_epi8(even, odd), _mm_unpacklo_epi8(even, odd));
        w = _mm256_sub_epi8(w, eight);
        __m256i xv = _mm256_loadu_si256((const __m256i *)(x + i));
        __m256i prod16 = _mm256_maddubs_epi16(_mm256_sign_epi8(w, w), _mm256_sign_epi8(xv, w));
        acc = _mm256_add_epi32(acc, _mm256_madd_epi16(prod16, one16));
    }
    __m128i s = _mm_add_epi32(_mm256_castsi256_si128(acc), _mm256_extracti128_si256(acc, 1));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xB1));
    int32_t sum = _mm_cvtsi128_si32(s);
    if (i < n) sum += po_dot_i4i8_scalar(w4 + (i >> 1), x + i, n - i);
    return sum;
}
#endif

static int g_simd = -1; /* -1 = undecided, 0 = scalar, 1 = avx2 */

PO_API int po_simd_tier(void) {
    if (g_simd < 0) {
#if defined(__x86_64__)
        g_simd = __builtin_cpu_supports("avx2") ? 1 : 0;
#else
        g_simd = 0;
#endif
    }
    return g_simd;
}
/* force the tier: 0 scalar, 1 avx2 (ignored if unsupported), -1 auto */
PO_API void po_force_simd(int tier) {
    g_simd = -1;
    int best = po_simd_tier();
    if (tier >= 0 && tier <= best) g_simd = tier;
}

/* crates/peregrine-kernels/src/idot.rs:56-65 (runtime dispatch) */
PO_API int32_t po_dot_i4i8(const uint8_t *w4, const int8_t *x, size_t n) {
#if defined(__x86_64__)
    if (po_simd_tier() == 1) return dot_i4i8_avx2(w4, x, n);
#endif
    return po_dot_i4i8_scalar(w4, x, n);
}

/* crates/peregrine-kernels/src/idot.rs:78-92 (scalar inner dot) and :98-110
 * (dispatched inner dot).  `simd` selects which.  When `blocks` is not NULL the
 * per-group int32 accumulators are written there (ceil(n/gs) values): these are
 * the values the CUDA kernels must reproduce bit for bit. */
static float dot_i4i8_grouped_impl(const uint8_t *w4, const int8_t *x, const float *scales, size_t n, size_t gs,
                                   int simd, int32_t *blocks) {
    float acc = 0.0f;
    size_t g = 0;
    for (size_t start = 0; start < n; start += gs, ++g) {
        size_t len = n - start < gs ? n - start : gs;
        int32_t d = simd ? po_dot_i4i8(w4 + (start >> 1), x + start, len)
                         : po_dot_i4i8_scalar(w4 + (start >> 1), x + start, len);
        if (blocks) blocks[g] = d;
        acc += scales[g] * (float)d;
    }
    return acc;
}
PO_API float po_dot_i4i8_grouped_scalar(const uint8_t *w4, const int8_t *x, const float *scales, size_t n, size_t gs) {
    return dot_i4i8_grouped_impl(w4, x, scales, n, gs, 0, NULL);
}
PO_API float po_dot_i4i8_grouped(const uint8_t *w4, const int8_t *x, const float *scales, size_t n, size_t gs) {
    return dot_i4i8_grouped_impl(w4, x, scales, n, gs, 1, NULL);
}

/* ------------------------------------------------------------- matmuls */

/* crates/peregrine-kernels/src/matmul.rs:18-30 — strictly sequential fp32 */
PO_API void po_matmul_f32(float *y, const float *x, const float *w, size_t s_n, size_t d_n, size_t o_n) {
    for (size_t s = 0; s < s_n; ++s) {
        const float *xs = x + s * d_n;
        for (size_t o = 0; o < o_n; ++o) {
            const float *wo = w + o * d_n;
            float acc = 0.0f;
            for (size_t d = 0; d < d_n; ++d) acc += xs[d] * wo[d];
            y[s * o_n + o] = acc;
        }
    }
}

/* crates/peregrine-kernels/src/matmul.rs:75-87 — per-row scale:
 * y = ((float)dot * scale[o]) * sx[s].  `acc_i32` (may be NULL) receives the
 * whole-row int32 dot, [S*O]. */
PO_API void po_matmul_i4_idot(float *y, const int8_t *xq, const float *sx, const uint8_t *q4, const float *scale,
                              size_t s_n, size_t i_n, size_t o_n, int32_t *acc_i32) {
    size_t rb = (i_n + 1) / 2;
    for (size_t o = 0; o < o_n; ++o) {
        const uint8_t *w = q4 + o * rb;
        float sc = scale[o];
        for (size_t s = 0; s < s_n; ++s) {
            int32_t di = po_dot_i4i8(w, xq + s * i_n, i_n);
            if (acc_i32) acc_i32[s * o_n + o] = di;
            float d = (float)di;
            y[s * o_n + o] = d * sc * sx[s];
        }
    }
}

/* crates/peregrine-kernels/src/matmul.rs:93-106 — group scales:
 * y = grouped_dot * sx[s].  `blocks` (may be NULL) receives the per-group int32
 * accumulators, [S*O*ng]. */
PO_API void po_matmul_i4g_idot(float *y, const int8_t *xq, const float *sx, const uint8_t *q4, const float *scale,
                               size_t s_n, size_t i_n, size_t o_n, size_t gs, int32_t *blocks) {
    size_t rb = (i_n + 1) / 2;
    size_t ng = (i_n + gs - 1) / gs;
    for (size_t o = 0; o < o_n; ++o) {
        const uint8_t *w = q4 + o * rb;
        const float *sc = scale + o * ng;
        for (size_t s = 0; s < s_n; ++s) {
            float d = dot_i4i8_grouped_impl(w, xq + s * i_n, sc, i_n, gs, 1,
                                            blocks ? blocks + (s * o_n + o) * ng : NULL);
            y[s * o_n + o] = d * sx[s];
        }
    }
}

/* One quantised weight matrix as the reference's QtWeight holds it
 * (crates/peregrine-model/src/weight.rs:20-34): fmt 2 = per-row int4
 * (scale[O]), fmt 4 = grouped int4 (scale[O*ng], gs), fmt 0 = f32 [O,I]. */
typedef struct {
    const void *q;
    const float *scale;
    int32_t fmt;
    int32_t gs;
    int32_t i_n;
    int32_t o_n;
} PoWeight;

/* crates/peregrine-model/src/weight.rs:126-145 (format dispatch of apply) with
 * matmul.rs:109-124, 138-145 (quantise rows, then integer matmul).  The row
 * threading of weight.rs:213-237 only splits rows across workers and does not
 * change any element's arithmetic, so it is not restated here. */
static void weight_apply(const PoWeight *w, const float *x, size_t s_n, float *y, int8_t *xq, float *sx) {
    size_t i_n = (size_t)w->i_n, o_n = (size_t)w->o_n;
    if (w->fmt == 0) {
        po_matmul_f32(y, x, (const float *)w->q, s_n, i_n, o_n);
        return;
    }
    for (size_t s = 0; s < s_n; ++s) sx[s] = po_qrow_i8(x + s * i_n, xq + s * i_n, i_n);
    if (w->fmt == 2)
        po_matmul_i4_idot(y, xq, sx, (const uint8_t *)w->q, w->scale, s_n, i_n, o_n, NULL);
    else
        po_matmul_i4g_idot(y, xq, sx, (const uint8_t *)w->q, w->scale, s_n, i_n, o_n, (size_t)w->gs, NULL);
}

PO_API void po_weight_apply(const PoWeight *w, const float *x, size_t s_n, float *y) {
    int8_t *xq = (int8_t *)malloc(s_n * (size_t)w->i_n + 1);
    float *sx = (float *)malloc((s_n + 1) * sizeof(float));
    weight_apply(w, x, s_n, y, xq, sx);
    free(xq);
    free(sx);
}

/* -------------------------------------------------------- elementwise */

/* crates/peregrine-model/src/math.rs:103-105 */
PO_API float po_sigmoidf(float x) { return 1.0f / (1.0f + exp32(-x)); }
/* crates/peregrine-model/src/math.rs:108-110 */
PO_API float po_siluf(float x) { return x / (1.0f + exp32(-x)); }
/* crates/peregrine-model/src/math.rs:114-118 */
PO_API void po_silu_mul(float *g, const float *u, size_t n) {
    for (size_t i = 0; i < n; ++i) g[i] = po_siluf(g[i]) * u[i];
}

/* crates/peregrine-model/src/math.rs:9-25 — f64 sum of squares */
PO_API void po_rmsnorm(float *out, const float *x, const float *w, size_t d, float eps) {
    if (d == 0) return;
    double ms = 0.0;
    for (size_t i = 0; i < d; ++i) ms += (double)x[i] * (double)x[i];
    float r = 1.0f / sqrtf((float)(ms / (double)d) + eps);
    for (size_t i = 0; i < d; ++i) out[i] = x[i] * r * w[i];
}

/* crates/peregrine-model/src/sample.rs:21-32 */
PO_API int32_t po_argmax(const float *lo, size_t n) {
    size_t b = 0;
    while (b < n && isnan(lo[b])) ++b;
    if (b >= n) return 0;
    for (size_t i = b + 1; i < n; ++i)
        if (lo[i] > lo[b]) b = i;
    return (int32_t)b;
}

/* ------------------------------------------------------------ SwiGLU */

/* crates/peregrine-model/src/mlp.rs:21-26.  `h_out` (may be NULL) receives the
 * SwiGLU intermediate [s_n, I] that the down projection re-quantises. */
PO_API void po_swiglu(const PoWeight *gate, const PoWeight *up, const PoWeight *down, const float *x, size_t s_n,
                      float *y, float *h_out) {
    size_t in = (size_t)gate->i_n, mid = (size_t)gate->o_n;
    size_t widest = in > mid ? in : mid;
    float *g = (float *)malloc(s_n * mid * sizeof(float) + 4);
    float *u = (float *)malloc(s_n * mid * sizeof(float) + 4);
    int8_t *xq = (int8_t *)malloc(s_n * widest + 1);
    float *sx = (float *)malloc((s_n + 1) * sizeof(float));
    weight_apply(gate, x, s_n, g, xq, sx);
    weight_apply(up, x, s_n, u, xq, sx);
    po_silu_mul(g, u, s_n * mid);
    if (h_out) memcpy(h_out, g, s_n * mid * sizeof(float));
    weight_apply(down, g, s_n, y, xq, sx);
    free(g);
    free(u);
    free(xq);
    free(sx);
}

/* -------------------------------------------------------------- router */

/* crates/peregrine-model/src/router.rs:52-150 with min_share = 0 (the
 * reference default; the negligible-tail truncation of :175-205 is an opt-in
 * knob that changes token values and is outside this path).
 * `logits_out` (may be NULL) receives the raw fp32 logits [S*E] before the
 * sigmoid.  The pool splits of :63-77 only partition outputs and leave each
 * element's left-to-right sum unchanged. */
PO_API void po_route(const float *x, const float *router_w, const float *router_bias, size_t s_n, size_t d_n,
                     size_t e_n, size_t k, int norm_topk, float routed_scale, int32_t *idx, float *w, int32_t *keff,
                     float *logits_out) {
    float *logits = (float *)malloc((s_n * e_n + 1) * sizeof(float));
    float *choice = (float *)malloc((e_n + 1) * sizeof(float));
#ifdef _OPENMP
#pragma omp parallel for schedule(static) if (s_n * d_n * e_n >= (1u << 20))
#endif
    for (long so = 0; so < (long)(s_n * e_n); ++so) {
        size_t s = (size_t)so / e_n, o = (size_t)so % e_n;
        const float *xs = x + s * d_n, *wo = router_w + o * d_n;
        float acc = 0.0f;
        for (size_t d = 0; d < d_n; ++d) acc += xs[d] * wo[d];
        logits[so] = acc;
    }
    if (logits_out) memcpy(logits_out, logits, s_n * e_n * sizeof(float));
    for (size_t s = 0; s < s_n; ++s) {
        float *logit = logits + s * e_n;
        for (size_t e = 0; e < e_n; ++e) {
            logit[e] = po_sigmoidf(logit[e]);
            choice[e] = logit[e] + router_bias[e];
        }
        int32_t *ib = idx + s * k;
        float *wb = w + s * k;
        size_t kept = k;
        for (size_t kk = 0; kk < k; ++kk) {
            int32_t best = -1;
            float bv = -INFINITY;
            for (size_t e = 0; e < e_n; ++e) {
                int taken = 0;
                for (size_t j = 0; j < kk; ++j)
                    if (ib[j] == (int32_t)e) { taken = 1; break; }
                if (taken) continue;
                if (choice[e] > bv) { bv = choice[e]; best = (int32_t)e; }
            }
            if (best < 0) { kept = kk; break; }
            ib[kk] = best;
            wb[kk] = logit[best];
        }
        for (size_t slot = kept; slot < k; ++slot) { ib[slot] = 0; wb[slot] = 0.0f; }
        keff[s] = (int32_t)kept;
        if (norm_topk) {
            float sm = 0.0f;
            for (size_t j = 0; j < k; ++j) sm += wb[j];
            sm += 1e-20f;
            for (size_t j = 0; j < k; ++j) wb[j] /= sm;
        }
        for (size_t j = 0; j < k; ++j) wb[j] *= routed_scale;
    }
    free(logits);
    free(choice);
}

/* crates/peregrine-model/src/router.rs:420-430 — distinct experts in
 * first-seen order (s ascending, kk ascending).  Returns the count. */
PO_API size_t po_batch_union(const int32_t *idx, const int32_t *keff, size_t s_n, size_t k, size_t e_n,
                             int32_t *uniq) {
    uint8_t *seen = (uint8_t *)calloc(e_n + 1, 1);
    size_t n = 0;
    for (size_t s = 0; s < s_n; ++s)
        for (size_t kk = 0; kk < (size_t)(keff[s] > 0 ? keff[s] : 0) && kk < k; ++kk) {
            int32_t e = idx[s * k + kk];
            if (e < 0 || (size_t)e >= e_n) continue;
            if (!seen[e]) { seen[e] = 1; uniq[n++] = e; }
        }
    free(seen);
    return n;
}

/* crates/peregrine-cuda/src/lib.rs:585-610 (ReduceLayout::build): counting sort
 * of y-row indices by destination row, ascending within each row.  Returns 0
 * when a destination is out of range. */
PO_API int po_reduce_layout(const int32_t *dst, size_t total, size_t s_n, int32_t *row_ptr, int32_t *row_idx) {
    for (size_t k = 0; k < total; ++k)
        if (dst[k] < 0 || (size_t)dst[k] >= s_n) return 0;
    memset(row_ptr, 0, (s_n + 1) * sizeof(int32_t));
    for (size_t k = 0; k < total; ++k) row_ptr[dst[k] + 1] += 1;
    for (size_t s = 0; s < s_n; ++s) row_ptr[s + 1] += row_ptr[s];
    int32_t *fill = (int32_t *)malloc((s_n + 1) * sizeof(int32_t));
    memcpy(fill, row_ptr, (s_n + 1) * sizeof(int32_t));
    for (size_t k = 0; k < total; ++k) row_idx[fill[dst[k]]++] = (int32_t)k;
    free(fill);
    return 1;
}

/* ----------------------------------------------------------- MoE layer */

/* crates/peregrine-model/src/mlp.rs:46-128 (resident MoE forward); the GPU-lane
 * variant crates/peregrine-model/src/concurrent.rs:1246-1265, 1866-1929 follows
 * the same order rule.  experts[e*3+{0,1,2}] = gate, up, down of expert e;
 * shared (may be NULL) points at 3 weights.  Threads (when > 1) compute distinct
 * experts in parallel as mlp.rs:102-110 does; the scatter stays serial in
 * batch-union order, so the result does not depend on the thread count.
 * Optional taps: idx/w/keff [S*k],[S*k],[S], union_out [E] with *n_union. */
PO_API void po_moe_forward(const float *x, const float *router_w, const float *router_bias, const PoWeight *experts,
                           size_t e_n, const PoWeight *shared, size_t s_n, size_t hidden, size_t k, int norm_topk,
                           float routed_scale, int threads, float *out, int32_t *idx_out, float *w_out,
                           int32_t *keff_out, int32_t *union_out, int32_t *n_union_out) {
    int32_t *idx = (int32_t *)malloc((s_n * k + 1) * sizeof(int32_t));
    float *w = (float *)malloc((s_n * k + 1) * sizeof(float));
    int32_t *keff = (int32_t *)malloc((s_n + 1) * sizeof(int32_t));
    po_route(x, router_w, router_bias, s_n, hidden, e_n, k, norm_topk, routed_scale, idx, w, keff, NULL);
    int32_t *uniq = (int32_t *)malloc((e_n + 1) * sizeof(int32_t));
    size_t nu = po_batch_union(idx, keff, s_n, k, e_n, uniq);
    if (idx_out) memcpy(idx_out, idx, s_n * k * sizeof(int32_t));
    if (w_out) memcpy(w_out, w, s_n * k * sizeof(float));
    if (keff_out) memcpy(keff_out, keff, s_n * sizeof(int32_t));
    if (union_out) memcpy(union_out, uniq, nu * sizeof(int32_t));
    if (n_union_out) *n_union_out = (int32_t)nu;

    /* plans in union order; rows ascending s, one row per (s, expert) */
    int32_t *slot_of = (int32_t *)malloc((e_n + 1) * sizeof(int32_t));
    for (size_t e = 0; e < e_n; ++e) slot_of[e] = -1;
    for (size_t p = 0; p < nu; ++p) slot_of[uniq[p]] = (int32_t)p;
    int32_t *cnt = (int32_t *)calloc(nu + 1, sizeof(int32_t));
    int32_t *rows = (int32_t *)malloc((nu * s_n + 1) * sizeof(int32_t));
    float *rw = (float *)malloc((nu * s_n + 1) * sizeof(float));
    for (size_t s = 0; s < s_n; ++s) {
        size_t ke = (size_t)(keff[s] > 0 ? keff[s] : 0);
        if (ke > k) ke = k;
        for (size_t kk = 0; kk < ke; ++kk) {
            int32_t e = idx[s * k + kk];
            if (e < 0 || (size_t)e >= e_n) continue;
            int32_t p = slot_of[e];
            if (p < 0) continue;
            if (cnt[p] > 0 && rows[(size_t)p * s_n + cnt[p] - 1] == (int32_t)s) continue;
            rows[(size_t)p * s_n + cnt[p]] = (int32_t)s;
            rw[(size_t)p * s_n + cnt[p]] = w[s * k + kk];
            cnt[p] += 1;
        }
    }
    float **hs = (float **)calloc(nu + 1, sizeof(float *));
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1) if (threads > 1 && nu >= 2)
#endif
    for (long p = 0; p < (long)nu; ++p) {
        size_t nr = (size_t)cnt[p];
        if (nr == 0) continue;
        float *xg = (float *)malloc(nr * hidden * sizeof(float));
        for (size_t ri = 0; ri < nr; ++ri)
            memcpy(xg + ri * hidden, x + (size_t)rows[(size_t)p * s_n + ri] * hidden, hidden * sizeof(float));
        hs[p] = (float *)malloc(nr * hidden * sizeof(float));
        const PoWeight *ex = experts + (size_t)uniq[p] * 3;
        po_swiglu(ex, ex + 1, ex + 2, xg, nr, hs[p], NULL);
        free(xg);
    }
    memset(out, 0, s_n * hidden * sizeof(float));
    for (size_t p = 0; p < nu; ++p) {
        for (size_t ri = 0; ri < (size_t)cnt[p]; ++ri) {
            float *dst = out + (size_t)rows[p * s_n + ri] * hidden;
            const float *src = hs[p] + ri * hidden;
            float wgt = rw[p * s_n + ri];
            for (size_t d = 0; d < hidden; ++d) dst[d] += wgt * src[d];
        }
        free(hs[p]);
    }
    if (shared) {
        float *sh = (float *)malloc(s_n * hidden * sizeof(float));
        po_swiglu(shared, shared + 1, shared + 2, x, s_n, sh, NULL);
        for (size_t z = 0; z < s_n * hidden; ++z) out[z] += sh[z];
        free(sh);
    }
    free(hs);
    free(idx);
    free(w);
    free(keff);
    free(uniq);
    free(slot_of);
    free(cnt);
    free(rows);
    free(rw);
}

/* --------------------------------------------------------- quantisers */

/* crates/peregrine-core/src/pack.rs:492-512 */
PO_API void po_quant_i4(const float *w, size_t o, size_t i, uint8_t *q, float *sc) {
    size_t rb = (i + 1) / 2;
    memset(q, 0, o * rb);
    for (size_t oo = 0; oo < o; ++oo) {
        const float *row = w + oo * i;
        float amax = 0.0f;
        for (size_t ii = 0; ii < i; ++ii) amax = fmaxf(amax, fabsf(row[ii]));
        float s = fmaxf(amax / 7.0f, 1e-12f);
        sc[oo] = s;
        for (size_t ii = 0; ii < i; ++ii) {
            float r = nearbyintf(row[ii] / s);
            if (r < -8.0f) r = -8.0f;
            if (r > 7.0f) r = 7.0f;
            uint8_t b = (uint8_t)((int32_t)r + 8) & 0x0F;
            q[oo * rb + (ii >> 1)] |= (ii & 1) ? (uint8_t)(b << 4) : b;
        }
    }
}

/* crates/peregrine-core/src/pack.rs:518-542 */
PO_API void po_quant_i4_grouped(const float *w, size_t o, size_t i, size_t gs, uint8_t *q, float *sc) {
    size_t rb = (i + 1) / 2, ng = (i + gs - 1) / gs;
    memset(q, 0, o * rb);
    for (size_t oo = 0; oo < o; ++oo) {
        const float *row = w + oo * i;
        for (size_t g = 0; g < ng; ++g) {
            size_t s0 = g * gs, e0 = (g + 1) * gs < i ? (g + 1) * gs : i;
            float amax = 0.0f;
            for (size_t ii = s0; ii < e0; ++ii) amax = fmaxf(amax, fabsf(row[ii]));
            float scale = fmaxf(amax / 7.0f, 1e-12f);
            sc[oo * ng + g] = scale;
            for (size_t ii = s0; ii < e0; ++ii) {
                float r = nearbyintf(row[ii] / scale);
                if (r < -8.0f) r = -8.0f;
                if (r > 7.0f) r = 7.0f;
                uint8_t b = (uint8_t)((int32_t)r + 8) & 0x0F;
                q[oo * rb + (ii >> 1)] |= (ii & 1) ? (uint8_t)(b << 4) : b;
            }
        }
    }
}

PO_API int po_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
