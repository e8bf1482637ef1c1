/*
 * CPU oracle for the tensor-parallel reduction path of msuiche/weightstream.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference's
 * CPU arithmetic (the Rust crates weightstream-core and weightstream-ref, and the
 * rank-ordered fold of weightstream-transport). It is the checker for the CUDA
 * library, never a fallback for it: only the test-suite, the smoke check and the
 * benchmark's cpu_baseline / reference arm may load it.
 *
 * Parity status: pinned against every known-answer value the reference's own
 * unit tests hold for these functions (see the per-function citations), with one
 * recorded departure: the E4M3 encoder's answer for |v| in [7.5/512, 8/512), where the
 * reference's CPU and device encoders disagree (wso_set_e4m3_literal below); the
 * 128x128-fp32-scale FP8 form, the FP8 lm_head and world sizes other than 4 are
 * not covered by any reference test and are pinned by this restatement only.
 * The Rust original cannot be compiled in the build environment (no cargo/rustc).
 */
#ifndef WS_ORACLE_H
#define WS_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- quant primitives: crates/weightstream-core/src/quant.rs ---- */
float    wso_e4m3_to_f32(uint8_t b);                 /* quant.rs:26  */
float    wso_e8m0_to_f32(uint8_t b);                 /* quant.rs:43  */
float    wso_fp4_to_f32(uint8_t nibble);             /* quant.rs:11  */
int32_t  wso_log2_ceil(float x);                     /* quant.rs:63  */
float    wso_pow2i(int32_t e);                       /* quant.rs:77  */
float    wso_ue8m0_round_scale(float amax, float fp_max); /* quant.rs:85 */
float    wso_bf16_to_f32(uint16_t bits);             /* quant.rs:91  */
uint16_t wso_f32_to_bf16(float v);                   /* quant.rs:97  */
uint8_t  wso_f32_to_e4m3(float v);                   /* quant.rs:106 */
/* quant.rs:121 as written returns the byte of 1.0 for |v| in [7.5/512, 8/512); the reference's
 * device encoder (kernels/common.cuh:26) returns the byte of 2^-6.  0 (default) follows the device
 * encoder, 1 follows quant.rs:121 to the letter.  Process-wide; not thread-safe to flip mid-call. */
void     wso_set_e4m3_literal(int on);
int      wso_get_e4m3_literal(void);
uint8_t  wso_f32_to_e2m1(float v);                   /* quant.rs:141 */

/* ---- activation quantisation: crates/weightstream-ref/src/actquant.rs:21-57 ---- */
void wso_fp8_snap(float *x, size_t n, size_t block);
/* Storage form of the same quantisation (kernels/actquant.cu:47-83): E4M3 byte
 * per element and one UE8M0 exponent byte per 32 elements. */
void wso_fp8_act_emit(const float *x, size_t n, uint8_t *q, uint8_t *sexp);

/* ---- weight encoders: crates/weightstream-ref/src/store.rs:359-419 ----
 * scale_kind 0: one UE8M0 byte per (bn x bk) block, scale = 2^ceil(log2(amax/448))
 *               with amax floored at 1e-4 (the reference's rule, but with the true
 *               block amax instead of the last row's).
 * scale_kind 1: one fp32 per block, scale = amax/448 (amax floored at 1e-4). */
void wso_encode_fp8(const float *vals, size_t rows, size_t cols, int scale_kind,
                    size_t bn, size_t bk, uint8_t *w, void *scales);
void wso_encode_fp4(const float *vals, size_t rows, size_t cols, uint8_t *w,
                    uint8_t *scales);

/* ---- block-scaled GEMV: crates/weightstream-ref/src/actquant.rs:114-173 ----
 * y[m, n] for m < M.  x is fp32 [M, ldx]; only the first `cols` of each row are
 * used.  The weight shard is rows x cols with byte stride ldw; `row0`/`k0` are the
 * shard's offsets inside the full tensor and only select scale blocks:
 * scale(n, c) = scales[((row0+n)/bn) * scale_ld + (k0+c)/bk].
 * threads <= 1 runs single-threaded (the reference); > 1 splits output rows with
 * OpenMP, which keeps each dot product's order and so its bits. */
void wso_fp8_gemv(const uint8_t *w, size_t ldw, const void *scales, int scale_kind,
                  size_t bn, size_t bk, size_t scale_ld, size_t rows, size_t cols,
                  size_t row0, size_t k0, const float *x, size_t ldx, size_t M,
                  float *y, size_t ldy, int threads);
/* FP4: w is [rows, cols/2] packed (low nibble = even K), scales [rows, cols/32]. */
void wso_fp4_gemv(const uint8_t *w, const uint8_t *scales, size_t rows, size_t cols,
                  const float *x, size_t ldx, size_t M, float *y, size_t ldy,
                  int threads);

/* ---- MoE down-projection + combine: crates/weightstream-ref/src/moe.rs:75-84, :150, :203-207 ----
 * For each token t < M: y[t] = sum over its routes whose expert id lies in
 * [e_start, e_start+e_len), in ascending expert id, of
 * fp4_gemv(W2[e], fp8_act(h[t*top_k+slot] * weight[t*top_k+slot])).
 * h is fp32 [M*top_k, K] (already widened from bf16 by the caller).
 * w2 / s2 hold the e_len local experts back to back. */
void wso_moe_down_combine(const uint8_t *w2, const uint8_t *s2, size_t n, size_t k,
                          int32_t e_start, int32_t e_len, const float *h,
                          const int32_t *route_ids, const float *route_w, size_t M,
                          size_t top_k, float *y, int threads);

/* ---- collectives: crates/weightstream-transport/src/ring.rs:399-408, :426-432 ---- */
void wso_allreduce_fold(const float *partials, size_t nranks, size_t len, float *out);
void wso_allgather(const float *contribs, size_t nranks, size_t len, float *out);

/* ---- sampling: crates/weightstream-ref/src/sample.rs:13-23 ---- */
uint32_t wso_argmax(const float *logits, size_t n);

int wso_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
