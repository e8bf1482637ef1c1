/*
 * ws_tp.h -- C ABI of the B200 (sm_100a) tensor-parallel reduction library.
 *
 * One `ws_tp_t` is one rank's endpoint of a tensor-parallel group of 1, 2, 4 or 8
 * ranks on one NVLink/NVSwitch node.  The fused operators below run the
 * row-parallel block-scaled GEMM of a reduction point and the fp32 exchange that
 * follows it in ONE kernel: partial sums are stored straight into every peer's
 * memory and summed in rank order 0,1,..,R-1, so every rank ends with identical
 * bits.  They replace, in msuiche/weightstream, the GEMM launches of
 * `crates/weightstream-gpu/src/engine.rs` together with the host-side
 * `trait Collectives` (`engine.rs:287-294`) that `crates/weightstream-transport`
 * implements over RoCE (`src/ring.rs:395-437`).
 *
 * Conventions
 *  - every function returns a `ws_status_t` (0 = ok, negative = error); nothing
 *    aborts the process or throws.  `ws_tp_last_error` gives the text.
 *  - all device work is enqueued on the caller's stream (`void*` = cudaStream_t);
 *    the device-resident entry points never synchronise.  A peer that does not
 *    arrive within `wait_ms` makes the kernel record WS_ERR_TIMEOUT in a status
 *    word and return (fail-stop, as `ring.rs:439-458`); `ws_tp_check` reads it.
 *  - ranks are lock-step SPMD: every rank issues the same sequence of fused
 *    operators / collectives on its endpoint (`ring.rs:334-337`).
 *  - per-rank slicing keeps the reference's contract `rank*len/world`
 *    (`engine.rs:1477-1480` K slices, `:1194-1195` experts, `:3107-3108` vocab).
 */
#ifndef WS_TP_H
#define WS_TP_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WS_MAX_WORLD 8
#define WS_IPC_HANDLE_BYTES 128

typedef int32_t ws_status_t;
enum {
    WS_OK = 0,
    WS_ERR_INVALID = -1,      /* bad argument: shape, alignment, shard bounds   */
    WS_ERR_CUDA = -2,         /* a CUDA runtime / driver call failed             */
    WS_ERR_TIMEOUT = -3,      /* a peer's partial did not arrive within wait_ms  */
    WS_ERR_SEQUENCE = -4,     /* ranks disagree on the step count (host check, or a peer's
                                 partial tagged with a later step: ring.rs:488-499)          */
    WS_ERR_CAPACITY = -5,     /* the step exceeds what the endpoint was sized for */
    WS_ERR_UNSUPPORTED = -6
};

enum { WS_SCALE_UE8M0 = 0, WS_SCALE_F32 = 1 };   /* weight-scale element type */
enum { WS_ACT_BF16 = 0, WS_ACT_F32 = 1 };        /* activation element type   */

typedef struct ws_tp ws_tp_t;

typedef struct {
    int32_t max_m;          /* most activation rows (tokens) in one fused step           */
    int32_t max_n;          /* widest reduced output row (model dim)                     */
    int32_t max_vocab;      /* full vocabulary for the lm_head gather (0 = not used)     */
    int32_t wait_ms;        /* bound on every wait for a peer; <= 0 selects 2000 ms      */
    int32_t num_ctas;       /* persistent CTAs per rank; 0 = one per SM                  */
    int32_t reserved[3];
} ws_tp_config_t;

typedef struct { uint8_t bytes[WS_IPC_HANDLE_BYTES]; } ws_ipc_handle_t;

/* ---- endpoint life cycle: replaces tp4::join + Ring::new
 *      (crates/weightstream-gpu/src/tp4.rs:191-312, crates/weightstream-transport/src/ring.rs:115-217) */
ws_status_t ws_tp_create(int32_t world, int32_t rank, int32_t device,
                         const ws_tp_config_t *cfg, ws_tp_t **out);
ws_status_t ws_tp_destroy(ws_tp_t *tp);
/* One process per rank: export this rank's exchange memory, then hand every
 * rank's handle (index = rank) to ws_tp_connect_ipc.  The caller moves the
 * bytes between processes (the reference does the same over its TCP control
 * plane, crates/weightstream-transport/src/ctrl.rs:12-29). */
ws_status_t ws_tp_export_handle(ws_tp_t *tp, ws_ipc_handle_t *out);
ws_status_t ws_tp_connect_ipc(ws_tp_t *tp, const ws_ipc_handle_t *handles, int32_t n);
/* The same exchange without a host framework: the ranks trade their handles over TCP (rank 0 listens on
 * host:port, the others connect, retrying until timeout_ms has passed) and every rank connects as by
 * ws_tp_connect_ipc.  Replaces, for this purpose, the reference's TCP control plane
 * (crates/weightstream-transport/src/ctrl.rs:12-29, group bring-up in
 * crates/weightstream-gpu/src/tp4.rs:191-312).  WS_ERR_TIMEOUT when a rank does not show up,
 * WS_ERR_INVALID when a rank reports another world size, a rank number twice or one out of range. */
ws_status_t ws_tp_connect_tcp(ws_tp_t *tp, int32_t rank, int32_t world, const char *host, int32_t port, int32_t timeout_ms);
/* The rendezvous by itself (no device involved): every rank contributes `len` bytes and receives all
 * ranks' bytes in rank order in `out` (world * len bytes). */
ws_status_t ws_tcp_allgather(int32_t rank, int32_t world, const char *host, int32_t port, const void *in, void *out,
                             int32_t len, int32_t timeout_ms);
/* One process driving all ranks (several devices with peer access, or several
 * virtual ranks on one device for single-GPU testing). */
ws_status_t ws_tp_connect_local(ws_tp_t *const *ranks, int32_t n);

/* Synchronise `stream`, then report the status word the kernels wrote. */
ws_status_t ws_tp_check(ws_tp_t *tp, void *stream);
/* Replaces Collectives::stats (engine.rs:291-293). */
const char *ws_tp_last_error(ws_tp_t *tp);
ws_status_t ws_tp_stats(ws_tp_t *tp, uint64_t *steps, uint64_t *launches);
int32_t ws_tp_num_ctas(ws_tp_t *tp);

/* ---- FP8 row-parallel GEMM + all-reduce -------------------------------------------------
 * Replaces emit8 + gemm_q8(wo_b) + Collectives::allreduce at the attention output
 * projection (engine.rs:3988-4029; batched form :6158-6181) and the same triple
 * for a K-sharded shared-expert down projection (reference CPU form
 * crates/weightstream-ref/src/moe.rs:245-249).
 *
 * out[m, n] = sum over ranks r (in rank order) of
 *             sum_k fp8_act(x_r)[m, k] * e4m3(w_r[n, k]) * scale_r(n, k)
 * where fp8_act is the reference's dynamic per-32 activation quantisation
 * (crates/weightstream-ref/src/actquant.rs:21-57) applied in the kernel prologue, and
 * scale_r(n, k) = scales[((row0 + n) / block_n) * scale_ld + (k0 + k) / block_k]. */
typedef struct {
    const void *x;            /* [m, k] activations of this rank's K slice, row stride ldx (elements) */
    int64_t ldx;
    int32_t x_dtype;          /* WS_ACT_BF16 or WS_ACT_F32                                            */
    int32_t m, n, k;          /* k = this rank's slice length (multiple of 32)                        */
    const uint8_t *w;         /* E4M3 bytes [n, k], row stride ldw bytes (multiple of 16)             */
    int64_t ldw;
    const void *scales;       /* scale matrix this rank holds                                         */
    int64_t scale_ld;         /* elements per scale row                                               */
    int32_t scale_kind;       /* WS_SCALE_UE8M0 (reference: 32x32) or WS_SCALE_F32 (128x128)          */
    int32_t block_n, block_k; /* scale block shape; powers of two, block_n >= 16, block_k >= 32       */
    int64_t row0, k0;         /* offset of w[0,0] inside the held scale matrix (row0 multiple of 16)  */
    float *out;               /* [m, n] fp32, row stride n                                            */
} ws_fp8_gemm_args_t;

ws_status_t ws_fp8_rowpar_gemm_allreduce(ws_tp_t *tp, const ws_fp8_gemm_args_t *args, void *stream);
/* Same step for n endpoints held by one process (args[i] and streams[i] belong to ranks[i]). */
ws_status_t ws_fp8_rowpar_gemm_allreduce_group(ws_tp_t *const *ranks, int32_t n,
                                               const ws_fp8_gemm_args_t *args, void *const *streams);

/* ---- MoE routed-expert down projection + combine + all-reduce ---------------------------
 * Replaces emit8 + moe_grouped_tl(Down) + moe_combine_f32 + Collectives::allreduce
 * (engine.rs:4207-4239, :4513-4522; reference CPU form moe.rs:75-84, :150, :203-207).
 * For token t: out[t] = sum over ranks of the sum, in ascending expert id, over the
 * routes of t whose expert is local, of fp4_gemv(W2[e], fp8_act(h[route] * weight[route])).
 * The routing weight multiplies the hidden BEFORE quantisation (moe.rs:99-102). */
typedef struct {
    const void *h;            /* [m*top_k, k] hidden of every route (row = t*top_k + slot)    */
    int64_t ldh;
    int32_t h_dtype;
    int32_t m, n, k, top_k;
    const int32_t *route_ids; /* device [m, top_k] global expert ids, -1 = empty slot         */
    const float *route_w;     /* device [m, top_k]                                            */
    const uint8_t *w2;        /* local slab [e_len][n][k/2] packed E2M1, low nibble = even K  */
    const uint8_t *s2;        /* [e_len][n][k/32] UE8M0                                       */
    int32_t e_start, e_len;   /* this rank owns experts [e_start, e_start+e_len)              */
    float *out;               /* [m, n] fp32                                                  */
} ws_moe_down_args_t;

ws_status_t ws_moe_down_combine_allreduce(ws_tp_t *tp, const ws_moe_down_args_t *args, void *stream);
ws_status_t ws_moe_down_combine_allreduce_group(ws_tp_t *const *ranks, int32_t n,
                                                const ws_moe_down_args_t *args, void *const *streams);

/* ---- vocab-sharded lm_head + all-gather + argmax ------------------------------------------
 * Replaces bf16_gemv(head) + Collectives::allgather + argmax_rows
 * (engine.rs:2647-2667, :2687-2703; tie rule crates/weightstream-ref/src/sample.rs:13-23:
 * the lowest index among equal maxima wins, all -inf gives 0).
 * `g` describes this rank's vocab shard (g.n = local rows, g.out unused);
 * `vocab_row0` is the shard's first global row and `vocab` the full size. */
typedef struct {
    ws_fp8_gemm_args_t g;
    int64_t vocab_row0;
    int32_t vocab;
    int32_t reserved;
    float *logits;            /* [m, vocab] fp32 or NULL when only the argmax is wanted */
    uint32_t *argmax;         /* [m] or NULL                                            */
} ws_lm_head_args_t;

ws_status_t ws_lm_head_allgather_argmax(ws_tp_t *tp, const ws_lm_head_args_t *args, void *stream);
ws_status_t ws_lm_head_allgather_argmax_group(ws_tp_t *const *ranks, int32_t n,
                                              const ws_lm_head_args_t *args, void *const *streams);

/* ---- bare collectives on device buffers: Collectives::allreduce / ::allgather
 *      (engine.rs:287-290, ring.rs:395-437) without the host round trip ------------------- */
ws_status_t ws_allreduce_f32(ws_tp_t *tp, const float *in, float *out, int64_t len, void *stream);
ws_status_t ws_allgather_f32(ws_tp_t *tp, const float *in, float *out, int64_t len, void *stream);
ws_status_t ws_allreduce_f32_group(ws_tp_t *const *ranks, int32_t n, const float *const *in,
                                   float *const *out, int64_t len, void *const *streams);
ws_status_t ws_allgather_f32_group(ws_tp_t *const *ranks, int32_t n, const float *const *in,
                                   float *const *out, int64_t len, void *const *streams);

/* ---- host-buffer forms: the exact shape of the reference trait (host slice in, host
 *      result out, error = abort the decode).  They copy, launch, synchronise and check. --- */
ws_status_t ws_allreduce_f32_host(ws_tp_t *tp, const float *in, float *out, int64_t len);
ws_status_t ws_allgather_f32_host(ws_tp_t *tp, const float *in, float *out, int64_t len);
ws_status_t ws_fp8_rowpar_gemm_allreduce_host(ws_tp_t *tp, const ws_fp8_gemm_args_t *dev_weights,
                                              const void *x_host, float *out_host);

/* ---- activation quantisation alone: act_quant_fp8_emit
 *      (crates/weightstream-cuda/kernels/actquant.cu:47-83), bit-exact with
 *      crates/weightstream-ref/src/actquant.rs:21-57.  q [m, k] E4M3, sexp [m, k/32] UE8M0. */
ws_status_t ws_act_quant_fp8(const void *x, int64_t ldx, int32_t x_dtype, int32_t m, int32_t k,
                             uint8_t *q, uint8_t *sexp, void *stream);

/* Scheduling knob with no counterpart in the reference: 1 (default) deals the output rows
 * that do not fill whole 16-row tiles on every CTA out row by row, so that every SM streams
 * the same number of bytes; 0 hands each leftover tile to one CTA whole. */
ws_status_t ws_tp_set_split(ws_tp_t *tp, int32_t on);
/* Kernel choice, also without counterpart in the reference.  0 (default) automatic: FP8 steps run
 * one or two activation rows on CUDA cores and three or more (and shards from 128 MB) on the
 * block-scaled tcgen05 kernel; the MoE step runs on its tcgen05 kernel when the shape fits it
 * (k <= 4096, one rank per launch), else on its CUDA-core decode form.  1: the mma.sync
 * formulations.  2: the tcgen05 kernels wherever the shape fits.  3: the CUDA-core kernels (MoE: the
 * decode form).  All choices give results within the same tolerance of the reference arithmetic;
 * ranks of one group must make the same choice. */
ws_status_t ws_tp_set_kernel(ws_tp_t *tp, int32_t which);

/* ---- FP8 GEMM for callers that must not allocate ------------------------------------------
 * No counterpart in the reference.  Some hosts embed this library where device memory may
 * not be allocated on their behalf: a runtime that hands out one fixed arena at start-up and
 * forbids cudaMalloc afterwards, code running inside a memory-pool or capture-style region
 * where an allocation is an error, or a plug-in that has no endpoint (ws_tp_create allocates
 * the exchange region).  This is the single-rank form of ws_fp8_rowpar_gemm_allreduce (same
 * arguments, same kernel, out = the whole sum since there is one rank) whose scratch -- the
 * kernel's status word, step counter and arrival counters -- is a fixed array inside
 * the library image (WS_STATIC_SCRATCH_BYTES per GPU that loads the library, held until the
 * process exits).  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *  - limits: m <= WS_STATIC_MAX_M and n <= WS_STATIC_MAX_N; beyond them WS_ERR_CAPACITY with a
 *    message in `err` (optional buffer of err_len bytes).
 *  - the first call on a device looks the array's device address up and raises the kernel's
 *    shared-memory limit; make that first call before any stream capture begins.
 *  - all calls on a device share the one array, which keeps the previous call's contents; the
 *    entry point clears the counters and the status word on `stream` before the kernel.  Two
 *    calls that overlap on the GPU (different streams, no ordering) race on it.
 *  - both functions make `device` the calling thread's current device and leave it so.
 *  - the launch is asynchronous and returns WS_OK once enqueued.  A bounded wait inside the kernel
 *    that gives up (a weight tile that never lands) is recorded in the array's status word, which
 *    the next call clears: call ws_fp8_gemm_static_scratch_check after the launch -- it
 *    synchronises `stream`, reads the word (4 bytes, no allocation) and returns WS_OK or the
 *    recorded error with its text in `err` -- before trusting `out`. */
#define WS_STATIC_MAX_M 8
#define WS_STATIC_MAX_N 1048576
#define WS_STATIC_SCRATCH_BYTES 1024
ws_status_t ws_fp8_gemm_static_scratch(const ws_fp8_gemm_args_t *args, int32_t device, void *stream,
                                       char *err, size_t err_len);
ws_status_t ws_fp8_gemm_static_scratch_check(int32_t device, void *stream, char *err, size_t err_len);

const char *ws_version(void);

#ifdef __cplusplus
}
#endif
#endif
