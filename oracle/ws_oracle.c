/*
 * CPU oracle (test infrastructure only; see ws_oracle.h).
 *
 * Every function follows the reference file:line named beside it.  Build with
 * -O2 -ffp-contract=off and without -ffast-math: the reference defines
 * sequential f32 accumulation as normative (crates/weightstream-ref/src/num.rs:1-15),
 * so no fused multiply-add and no re-association may be introduced.
 */
#include "ws_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* crates/weightstream-core/src/quant.rs:11-13 (E2M1 table, index = 4-bit code) */
static const float FP4_TABLE[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                    0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

float wso_fp4_to_f32(uint8_t nibble) { return FP4_TABLE[nibble & 0x0F]; }

/* crates/weightstream-core/src/quant.rs:26-39: finite-only E4M3, bias 7,
 * S.1111.111 = NaN, subnormal step 1/512. */
float wso_e4m3_to_f32(uint8_t b) {
    float sign = (b & 0x80) ? -1.0f : 1.0f;
    int e = (b >> 3) & 0x0F;
    int m = b & 0x07;
    if (e == 0x0F && m == 0x07) return NAN;
    if (e == 0) return sign * (float)m * (1.0f / 512.0f);
    return sign * ldexpf(1.0f, e - 7) * (1.0f + (float)m / 8.0f);
}

/* crates/weightstream-core/src/quant.rs:43-48 */
float wso_e8m0_to_f32(uint8_t b) {
    if (b == 0xFF) return NAN;
    return ldexpf(1.0f, (int)b - 127);
}

/* crates/weightstream-core/src/quant.rs:63-73: ceil(log2 x) from the exponent
 * field; +1 when any mantissa bit is set. */
int32_t wso_log2_ceil(float x) {
    uint32_t bits = f2u(x);
    int32_t e = (int32_t)((bits >> 23) & 0xFF) - 127;
    return (bits & 0x7FFFFF) ? e + 1 : e;
}

/* crates/weightstream-core/src/quant.rs:77-79 (f32::exp2 of an integer is exact) */
float wso_pow2i(int32_t e) { return ldexpf(1.0f, e); }

/* crates/weightstream-core/src/quant.rs:85-87 */
float wso_ue8m0_round_scale(float amax, float fp_max) {
    return wso_pow2i(wso_log2_ceil(amax / fp_max));
}

/* crates/weightstream-core/src/quant.rs:91-93 */
float wso_bf16_to_f32(uint16_t bits) { return u2f((uint32_t)bits << 16); }

/* crates/weightstream-core/src/quant.rs:97-101 (round to nearest even) */
uint16_t wso_f32_to_bf16(float v) {
    uint32_t bits = f2u(v);
    uint32_t round = ((bits >> 16) & 1u) + 0x7FFFu;
    return (uint16_t)((bits + round) >> 16);
}

/* Which byte a magnitude in [7.5/512, 8/512) -- the top of the subnormal range, which
 * rounds up to the smallest normal 2^-6 -- encodes to.  The reference has two answers:
 *   0 (default): 0x08, the byte of 2^-6 (E=1, M=0).  This is what the reference's device
 *      encoder returns (crates/weightstream-cuda/kernels/common.cuh:26), what its comment at
 *      crates/weightstream-core/src/quant.rs:121 says it means, and what round-to-nearest-even
 *      onto the E4M3 grid is.
 *   1: 0x38, the byte of 1.0, which is what crates/weightstream-core/src/quant.rs:121
 *      returns as written ("sign | 0x38"); no reference test reaches that branch
 *      (quant.rs:285-306 only round-trips exact grid points and three ties below it).
 * Everything else in the encoder is identical in both modes. */
static int g_e4m3_literal_quant_rs = 0;
void wso_set_e4m3_literal(int on) { g_e4m3_literal_quant_rs = on ? 1 : 0; }
int wso_get_e4m3_literal(void) { return g_e4m3_literal_quant_rs; }

/* crates/weightstream-core/src/quant.rs:106-137: RNE onto the E4M3 grid,
 * saturating at +-448, NaN -> S.1111.111. nearbyintf under the default rounding
 * mode is round-half-to-even, as round_ties_even is.  Line 121 is followed in the
 * sense of the mode above. */
uint8_t wso_f32_to_e4m3(float v) {
    uint32_t bits = f2u(v);
    uint8_t sign = (uint8_t)((bits >> 24) & 0x80);
    if (isnan(v)) return sign | 0x7F;
    float a = fabsf(v);
    if (a >= 448.0f) return sign | 0x7E;
    if (a < wso_pow2i(-6)) {
        float q = a * 512.0f;
        int m = (int)nearbyintf(q);
        if (m == 8) return sign | (g_e4m3_literal_quant_rs ? 0x38 : 0x08); /* 2^-6: E=1, M=0 */
        return sign | (uint8_t)m;
    }
    int e = (int)((bits >> 23) & 0xFF) - 127;
    float q = a * wso_pow2i(3 - e);
    int m8 = (int)nearbyintf(q);
    int ef, mant;
    if (m8 == 16) { ef = e + 8; mant = 0; } else { ef = e + 7; mant = m8 - 8; }
    return sign | (uint8_t)(ef << 3) | (uint8_t)mant;
}

/* crates/weightstream-core/src/quant.rs:141-163: thresholds encode ties-to-even
 * on the E2M1 grid; saturates at +-6. */
uint8_t wso_f32_to_e2m1(float v) {
    uint8_t sign = (f2u(v) >> 31) ? 0x8 : 0x0;
    float a = fabsf(v);
    uint8_t code;
    if (a <= 0.25f) code = 0;
    else if (a < 0.75f) code = 1;
    else if (a <= 1.25f) code = 2;
    else if (a < 1.75f) code = 3;
    else if (a <= 2.5f) code = 4;
    else if (a < 3.5f) code = 5;
    else if (a <= 5.0f) code = 6;
    else code = 7;
    return sign | code;
}

static inline float clampf(float v, float lo, float hi) {
    /* f32::clamp: NaN stays NaN */
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

/* crates/weightstream-ref/src/actquant.rs:21-45 */
void wso_fp8_snap(float *x, size_t n, size_t block) {
    for (size_t g = 0; g + block <= n; g += block) {
        float amax = 0.0f;
        for (size_t i = 0; i < block; i++) {
            float a = fabsf(x[g + i]);
            if (a > amax) amax = a;
        }
        if (amax < 1e-4f) amax = 1e-4f;
        float s = wso_pow2i(wso_log2_ceil(amax / 448.0f));
        for (size_t i = 0; i < block; i++) {
            float q = clampf(x[g + i] / s, -448.0f, 448.0f);
            x[g + i] = wso_e4m3_to_f32(wso_f32_to_e4m3(q)) * s;
        }
    }
}

/* Storage form: crates/weightstream-cuda/kernels/actquant.cu:47-83 (block 32). */
void wso_fp8_act_emit(const float *x, size_t n, uint8_t *q, uint8_t *sexp) {
    for (size_t g = 0; g + 32 <= n; g += 32) {
        float amax = 0.0f;
        for (size_t i = 0; i < 32; i++) {
            float a = fabsf(x[g + i]);
            if (a > amax) amax = a;
        }
        if (amax < 1e-4f) amax = 1e-4f;
        int32_t e = wso_log2_ceil(amax / 448.0f);
        float s = wso_pow2i(e);
        sexp[g / 32] = (uint8_t)(e + 127);
        for (size_t i = 0; i < 32; i++)
            q[g + i] = wso_f32_to_e4m3(clampf(x[g + i] / s, -448.0f, 448.0f));
    }
}

/* crates/weightstream-ref/src/store.rs:359-390, generalised over the block shape
 * and the scale type; uses the true block amax (the reference's per-row overwrite
 * of a 32x32 block's scale is a generator quirk, not part of the GEMV contract). */
void wso_encode_fp8(const float *vals, size_t rows, size_t cols, int scale_kind,
                    size_t bn, size_t bk, uint8_t *w, void *scales) {
    size_t sr = (rows + bn - 1) / bn, sc = (cols + bk - 1) / bk;
    for (size_t rb = 0; rb < sr; rb++) {
        for (size_t cb = 0; cb < sc; cb++) {
            size_t r1 = (rb + 1) * bn < rows ? (rb + 1) * bn : rows;
            size_t c1 = (cb + 1) * bk < cols ? (cb + 1) * bk : cols;
            float amax = 1e-4f;
            for (size_t r = rb * bn; r < r1; r++)
                for (size_t c = cb * bk; c < c1; c++) {
                    float a = fabsf(vals[r * cols + c]);
                    if (a > amax) amax = a;
                }
            float s;
            if (scale_kind == 0) {
                int32_t e = wso_log2_ceil(amax / 448.0f);
                s = wso_pow2i(e);
                ((uint8_t *)scales)[rb * sc + cb] = (uint8_t)(e + 127);
            } else {
                s = amax / 448.0f;
                ((float *)scales)[rb * sc + cb] = s;
            }
            for (size_t r = rb * bn; r < r1; r++)
                for (size_t c = cb * bk; c < c1; c++)
                    w[r * cols + c] =
                        wso_f32_to_e4m3(clampf(vals[r * cols + c] / s, -448.0f, 448.0f));
        }
    }
}

/* crates/weightstream-ref/src/store.rs:392-419 */
void wso_encode_fp4(const float *vals, size_t rows, size_t cols, uint8_t *w,
                    uint8_t *scales) {
    size_t sc = (cols + 31) / 32;
    memset(w, 0, rows * cols / 2);
    for (size_t r = 0; r < rows; r++) {
        for (size_t kb = 0; kb < sc; kb++) {
            size_t c1 = kb * 32 + 32 < cols ? kb * 32 + 32 : cols;
            float amax = 6.0f * wso_pow2i(-126);
            for (size_t c = kb * 32; c < c1; c++) {
                float a = fabsf(vals[r * cols + c]);
                if (a > amax) amax = a;
            }
            int32_t e = wso_log2_ceil(amax / 6.0f);
            float s = wso_pow2i(e);
            scales[r * sc + kb] = (uint8_t)(e + 127);
            for (size_t c = kb * 32; c < c1; c++) {
                uint8_t q = wso_f32_to_e2m1(clampf(vals[r * cols + c] / s, -6.0f, 6.0f));
                size_t idx = r * (cols / 2) + c / 2;
                if (c % 2 == 0) w[idx] = (uint8_t)((w[idx] & 0xF0) | (q & 0x0F));
                else w[idx] = (uint8_t)((w[idx] & 0x0F) | (q << 4));
            }
        }
    }
}

static inline float scale_at(const void *scales, int scale_kind, size_t idx) {
    return scale_kind == 0 ? wso_e8m0_to_f32(((const uint8_t *)scales)[idx])
                           : ((const float *)scales)[idx];
}

/* crates/weightstream-ref/src/actquant.rs:114-138.  Per 32-wide K block:
 * blk += qa[c] * (e4m3(w) * s_b), then acc += blk, sequentially. */
void wso_fp8_gemv(const uint8_t *w, size_t ldw, const void *scales, int scale_kind,
                  size_t bn, size_t bk, size_t scale_ld, size_t rows, size_t cols,
                  size_t row0, size_t k0, const float *x, size_t ldx, size_t M,
                  float *y, size_t ldy, int threads) {
    size_t kb_n = cols / 32;
    float *qa = (float *)malloc(sizeof(float) * (cols ? cols : 1));
    for (size_t m = 0; m < M; m++) {
        memcpy(qa, x + m * ldx, sizeof(float) * cols);
        wso_fp8_snap(qa, cols, 32);
        float *ym = y + m * ldy;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#endif
        for (long n = 0; n < (long)rows; n++) {
            const uint8_t *row = w + (size_t)n * ldw;
            size_t srow = ((row0 + (size_t)n) / bn) * scale_ld;
            float acc = 0.0f;
            for (size_t kb = 0; kb < kb_n; kb++) {
                float s_b = scale_at(scales, scale_kind, srow + (k0 + kb * 32) / bk);
                float blk = 0.0f;
                for (size_t j = 0; j < 32; j++) {
                    size_t c = kb * 32 + j;
                    blk += qa[c] * (wso_e4m3_to_f32(row[c]) * s_b);
                }
                acc += blk;
            }
            ym[n] = acc;
        }
    }
    free(qa);
}

/* crates/weightstream-ref/src/actquant.rs:144-173 */
void wso_fp4_gemv(const uint8_t *w, const uint8_t *scales, size_t rows, size_t cols,
                  const float *x, size_t ldx, size_t M, float *y, size_t ldy,
                  int threads) {
    size_t kb_n = cols / 32, half = cols / 2;
    float *qa = (float *)malloc(sizeof(float) * (cols ? cols : 1));
    for (size_t m = 0; m < M; m++) {
        memcpy(qa, x + m * ldx, sizeof(float) * cols);
        wso_fp8_snap(qa, cols, 32);
        float *ym = y + m * ldy;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#endif
        for (long n = 0; n < (long)rows; n++) {
            const uint8_t *row = w + (size_t)n * half;
            float acc = 0.0f;
            for (size_t kb = 0; kb < kb_n; kb++) {
                float s_b = wso_e8m0_to_f32(scales[(size_t)n * kb_n + kb]);
                float blk = 0.0f;
                for (size_t j = 0; j < 32; j++) {
                    size_t c = kb * 32 + j;
                    uint8_t byte = row[c / 2];
                    float v = (c % 2 == 0) ? FP4_TABLE[byte & 0x0F] : FP4_TABLE[byte >> 4];
                    blk += qa[c] * (v * s_b);
                }
                acc += blk;
            }
            ym[n] = acc;
        }
    }
    free(qa);
}

/* crates/weightstream-ref/src/moe.rs:75-84 (ascending expert id, plain sum),
 * :150/:201 (routing weight multiplied into the hidden before quantisation),
 * :203-207 (w2 GEMV). */
void wso_moe_down_combine(const uint8_t *w2, const uint8_t *s2, size_t n, size_t k,
                          int32_t e_start, int32_t e_len, const float *h,
                          const int32_t *route_ids, const float *route_w, size_t M,
                          size_t top_k, float *y, int threads) {
    size_t wbytes = n * k / 2, sbytes = n * (k / 32);
    float *hw = (float *)malloc(sizeof(float) * k);
    float *ye = (float *)malloc(sizeof(float) * n);
    size_t *order = (size_t *)malloc(sizeof(size_t) * (top_k ? top_k : 1));
    for (size_t t = 0; t < M; t++) {
        float *yt = y + t * n;
        for (size_t d = 0; d < n; d++) yt[d] = 0.0f;
        /* stable insertion sort of the slots by expert id */
        size_t cnt = 0;
        for (size_t s = 0; s < top_k; s++) {
            int32_t e = route_ids[t * top_k + s];
            if (e < e_start || e >= e_start + e_len) continue;
            size_t p = cnt++;
            while (p > 0 && route_ids[t * top_k + order[p - 1]] > e) { order[p] = order[p - 1]; p--; }
            order[p] = s;
        }
        for (size_t i = 0; i < cnt; i++) {
            size_t r = t * top_k + order[i];
            size_t le = (size_t)(route_ids[r] - e_start);
            for (size_t j = 0; j < k; j++) hw[j] = h[r * k + j] * route_w[r];
            wso_fp4_gemv(w2 + le * wbytes, s2 + le * sbytes, n, k, hw, k, 1, ye, n, threads);
            for (size_t d = 0; d < n; d++) yt[d] += ye[d];
        }
    }
    free(hw); free(ye); free(order);
}

/* crates/weightstream-transport/src/ring.rs:399-408: acc = slot0; acc += slot r. */
void wso_allreduce_fold(const float *partials, size_t nranks, size_t len, float *out) {
    for (size_t i = 0; i < len; i++) {
        float acc = partials[i];
        for (size_t r = 1; r < nranks; r++) acc += partials[r * len + i];
        out[i] = acc;
    }
}

/* crates/weightstream-transport/src/ring.rs:426-432 */
void wso_allgather(const float *contribs, size_t nranks, size_t len, float *out) {
    memcpy(out, contribs, sizeof(float) * nranks * len);
}

/* crates/weightstream-ref/src/sample.rs:13-23: strict >, first maximum wins,
 * all -inf (or NaN) -> 0. */
uint32_t wso_argmax(const float *logits, size_t n) {
    size_t best = 0;
    float bv = -INFINITY;
    for (size_t i = 0; i < n; i++)
        if (logits[i] > bv) { bv = logits[i]; best = i; }
    return (uint32_t)best;
}

int wso_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
