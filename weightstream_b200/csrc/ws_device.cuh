// Device-side building blocks shared by the sm_100a kernels: PTX wrappers
// (mbarrier, TMA tile loads, ldmatrix, FP8 tensor-core MMA, system-scope flags),
// the bit-exact activation quantiser and the exchange layout.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ws_tp.h"

namespace ws {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + one TMA producer warp
constexpr int kBoxBytes = 2048;                  // one TMA box: 16 rows x 128 bytes
constexpr int kBoxesPerStage = 16;
constexpr int kStageBytes = kBoxBytes * kBoxesPerStage;  // 32 KB
constexpr int kMaxStages = 16;
constexpr int kMaxCtas = 160;    // persistent CTAs per rank (one per SM on B200: 148)
constexpr int kMaxShared = 160;  // further counter / flag slots per rank (status word and step counter follow them)
constexpr int kGroupRows = 16;   // MMA M: output rows per group

// Error detail codes written to the device status word (high byte) with WS_ERR_*.
enum : uint32_t {
    kStatOk = 0,
    kStatTimeoutPeerA = 0x01000000u,  // waiting for a peer CTA's owned-rows flag
    kStatTimeoutTma = 0x03000000u,    // a weight tile never landed in shared memory
    kStatTimeoutGather = 0x04000000u,
    kStatRunAhead = 0x05000000u       // a peer's word or flag carries a later step than this rank's
};

// ---------------------------------------------------------------- exchange layout
// Every rank allocates one region with this layout; peers map it and store into it.
struct SymLayout {
    int64_t flags_off;   // u32  [2 banks][R src][kMaxCtas + kMaxShared]
    int64_t pairs_off;   // u64  [2][R][kMaxCtas][max_m]      (argmax candidates)
    int64_t slotf_off;   // f32  [2][R][max_m*max_n]  plain-float slots (flag-synchronised exchanges: gather, MMA-form MoE, tcgen05 kernel)
    int64_t slota_off;   // u64  [2][R][max_m*max_n]  {step sequence, fp32 bits} words of the all-reduce
    int64_t gather_off;  // f32  [2][max_m*max_vocab]
    int64_t total;
    int32_t max_m, max_n, max_vocab, world;
};

__host__ __device__ inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

__host__ inline SymLayout make_layout(int world, int max_m, int max_n, int max_vocab) {
    SymLayout L{};
    L.world = world; L.max_m = max_m; L.max_n = max_n; L.max_vocab = max_vocab;
    int64_t o = 0;
    L.flags_off = o;  o += align_up((int64_t)2 * world * (kMaxCtas + kMaxShared) * 4, 256);
    L.pairs_off = o;  o += align_up((int64_t)2 * world * kMaxCtas * max_m * 8, 256);
    L.slotf_off = o;  o += align_up((int64_t)2 * world * max_m * max_n * 4, 256);
    L.slota_off = o;  o += align_up((int64_t)2 * world * max_m * max_n * 8, 256);
    L.gather_off = o; o += align_up((int64_t)2 * max_m * (int64_t)max_vocab * 4, 256);
    L.total = o;
    return L;
}

// What one (possibly virtual) rank needs inside a kernel to reach its group.
struct RankCtx {
    char *sym[WS_MAX_WORLD];  // sym[p] = rank p's exchange region as mapped here
    uint32_t *counters;       // local: [kMaxShared] arrival counters (self-resetting)
    uint32_t *status;         // local: first error wins
    uint32_t *step_ctr;       // local: [0] steps completed by this rank, [1] CTAs done with the current step, [2] CTAs that reported to the host
    uint64_t *host_done;      // host-buffer calls: a word in pinned host memory the last CTA sets (see host_done_signal); else null
    int32_t rank;
    int32_t pad;
};

// ---------------------------------------------------------------- small PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(20000u)  // the thread may sleep until the phase completes (at most ~20 us per probe)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after two seconds of wall time (globaltimer), records why, and lets the
// caller unwind instead of spinning forever.  Once any wait of the launch has failed (the status
// word is set) every later wait that is not satisfied at once returns false immediately, so a
// kernel with hundreds of stage waits ends in one time-out, not hundreds.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t *status) {
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (*(volatile uint32_t *)status != 0u) return false;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*(volatile uint32_t *)status != 0u) return false;
        if (globaltimer_ns() - t0 > 2000000000ull) break;
    }
    atomicCAS(status, 0u, kStatTimeoutTma | (uint32_t)(-WS_ERR_TIMEOUT));
    return false;
}

// Position in a ring of `n` stages, advanced without the division and remainder that
// (item % n, item / n) would cost per stage and warp.
struct RingPos {
    int s = 0;        // stage
    uint32_t ph = 0;  // parity of the number of completed laps
    __device__ __forceinline__ void next(int n) {
        if (++s == n) {
            s = 0;
            ph ^= 1u;
        }
    }
};

// 2-D TMA tile load global -> shared, completion on an mbarrier (no multicast).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int32_t x,
                                            int32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1,
                                            uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8, f32) = A(16x32 e4m3, row) * B(32x8 e4m3, col); accumulator starts at zero.
__device__ __forceinline__ void mma_e4m3_16x8x32(float (&d)[4], uint32_t a0, uint32_t a1,
                                                 uint32_t a2, uint32_t a3, uint32_t b0,
                                                 uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// Explicit shared-state-space loads: pointers carved out of the dynamic shared-memory block are
// generic to the compiler, and generic loads take the slower L1 path.
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds_u64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}

__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}

// ---- CUDA-core dot products (decode rows with one or two tokens)
// Two E4M3 bytes (the low 16 bits of v) -> f16x2, exact.
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t v) {
    uint32_t r;
    asm("{.reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t;}" : "=r"(r) : "r"(v));
    return r;
}
// Two E2M1 codes (the low byte of v; low nibble -> low half) -> f16x2, exact.
__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t v) {
    uint32_t r;
    asm("{.reg .b8 b; .reg .b16 t; cvt.u16.u32 t, %1; cvt.u8.u16 b, t; cvt.rn.f16x2.e2m1x2 %0, b;}" : "=r"(r) : "r"(v));
    return r;
}
// f16x2 -> two f32 (exact).
__device__ __forceinline__ float2 f16x2_to_f32x2(uint32_t v) {
    float2 r;
    asm("{.reg .f16 l, h; mov.b32 {l, h}, %2; cvt.f32.f16 %0, l; cvt.f32.f16 %1, h;}" : "=f"(r.x), "=f"(r.y) : "r"(v));
    return r;
}
// Two E4M3 bytes, the low (H = 0) or high (H = 1) half of v, -> f16x2 (exact).  The half is
// named by a register unpack so that the conversion can take it as an operand modifier.
template <int H>
__device__ __forceinline__ uint32_t e4m3x2_half_to_f16x2(uint32_t v) {
    uint32_t r;
    if (H == 0) asm("{.reg .b16 l, h; mov.b32 {l, h}, %1; cvt.rn.f16x2.e4m3x2 %0, l;}" : "=r"(r) : "r"(v));
    else        asm("{.reg .b16 l, h; mov.b32 {l, h}, %1; cvt.rn.f16x2.e4m3x2 %0, h;}" : "=r"(r) : "r"(v));
    return r;
}
// Two E2M1 codes, byte B of v (low nibble -> low half), -> f16x2 (exact).
template <int B>
__device__ __forceinline__ uint32_t e2m1x2_byte_to_f16x2(uint32_t v) {
    uint32_t r;
    if (B == 0) asm("{.reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b0;}" : "=r"(r) : "r"(v));
    if (B == 1) asm("{.reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b1;}" : "=r"(r) : "r"(v));
    if (B == 2) asm("{.reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b2;}" : "=r"(r) : "r"(v));
    if (B == 3) asm("{.reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b3;}" : "=r"(r) : "r"(v));
    return r;
}
// s += a.lo * b.lo + a.hi * b.hi with f16 operands and fp32 accumulation: the products of two
// 4-significant-bit values are exact, every add rounds once in fp32.
__device__ __forceinline__ void fma2_f16(float &s, uint32_t a, uint32_t b) {
    asm("{.reg .f16 a0, a1, b0, b1; mov.b32 {a0, a1}, %1; mov.b32 {b0, b1}, %2;"
        " fma.rn.f32.f16 %0, a0, b0, %0; fma.rn.f32.f16 %0, a1, b1, %0;}"
        : "+f"(s) : "r"(a), "r"(b));
}

template <int N>
__device__ __forceinline__ void consumer_bar_n() {  // the N consumer threads only
    asm volatile("bar.sync 1, %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void consumer_bar() {  // the consumer warps only
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// ---------------------------------------------------------------- system-scope flags
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_volatile_u64(const uint64_t *p) {
    uint64_t v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// A tag that is ahead of this rank's step: the peer ran on without this rank (the reference aborts
// on an immediate whose sequence is neither this step's nor an earlier one,
// crates/weightstream-transport/src/ring.rs:488-499).  Tags compare modulo 2^32.
__device__ __forceinline__ bool tag_ahead(uint32_t tag, uint32_t seq) { return (int32_t)(tag - seq) > 0; }
__device__ __forceinline__ void record_run_ahead(uint32_t *status) {
    atomicCAS(status, 0u, kStatRunAhead | (uint32_t)(-WS_ERR_SEQUENCE));
}

// Poll `flag` until it carries `seq`.  Every wait is bounded by `timeout_ns`: on
// expiry the first error is recorded in *status and the caller returns normally
// (fail-stop at the host, never a trap or an endless spin).  A flag from a later step is an
// error of its own (WS_ERR_SEQUENCE) and ends the wait at once.
__device__ __forceinline__ bool wait_flag(const uint32_t *flag, uint32_t seq, uint64_t timeout_ns,
                                          uint32_t *status, uint32_t code) {
    uint32_t f = ld_acquire_sys(flag);
    if (f == seq) return true;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 32; ++i) {
            f = ld_acquire_sys(flag);
            if (f == seq) return true;
        }
        if (tag_ahead(f, seq)) {
            record_run_ahead(status);
            return false;
        }
        if (globaltimer_ns() - t0 > timeout_ns) {
            atomicCAS(status, 0u, code | (uint32_t)(-WS_ERR_TIMEOUT));
            return false;
        }
        if (*(volatile uint32_t *)status != 0u) return false;  // someone else already failed
    }
}

// All-reduce words.  A partial sum travels as one 64-bit word {step sequence, fp32 bits}; a
// naturally aligned 64-bit store is single-copy atomic, so the value and its tag arrive together
// and the receiver needs neither a fence on the sender nor a separate flag: it polls the word
// until the tag is this step's.  One NVLink store latency instead of store, fence, flag.
__device__ __forceinline__ void st_word_sys(uint64_t *p, uint32_t seq, float v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(((uint64_t)seq << 32) | __float_as_uint(v)) : "memory");
}
__device__ __forceinline__ uint64_t ld_word_sys(const uint64_t *p) {
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// Bounded like wait_flag (time-out and run-ahead detection); returns 0 when the wait gave up (the
// status word then says why).
__device__ __forceinline__ float wait_word(const uint64_t *p, uint32_t seq, uint64_t timeout_ns, uint32_t *status,
                                           uint32_t code) {
    uint64_t w = ld_word_sys(p);
    if ((uint32_t)(w >> 32) == seq) return __uint_as_float((uint32_t)w);
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 32; ++i) {
            w = ld_word_sys(p);
            if ((uint32_t)(w >> 32) == seq) return __uint_as_float((uint32_t)w);
        }
        if (tag_ahead((uint32_t)(w >> 32), seq)) {
            record_run_ahead(status);
            return 0.0f;
        }
        if (globaltimer_ns() - t0 > timeout_ns) {
            atomicCAS(status, 0u, code | (uint32_t)(-WS_ERR_TIMEOUT));
            return 0.0f;
        }
        if (*(volatile uint32_t *)status != 0u) return 0.0f;  // someone else already failed
    }
}

// The ranks' words of one output, added in rank order.  All of them are requested before the first is
// looked at, so that words that have already arrived cost one memory round trip together, not one each
// (measured: eight dependent polls of local memory are ~5 us of an 8-rank step); a word that is not
// there yet is then waited for on its own.
__device__ __forceinline__ float fold_words(const uint64_t *slots, size_t astride, size_t off, int world, uint32_t seq,
                                            uint64_t timeout_ns, uint32_t *status, uint32_t code) {
    uint64_t w[WS_MAX_WORLD];
#pragma unroll
    for (int rr = 0; rr < WS_MAX_WORLD; ++rr)
        if (rr < world) w[rr] = ld_word_sys(slots + (size_t)rr * astride + off);
    float s = 0.0f;
#pragma unroll
    for (int rr = 0; rr < WS_MAX_WORLD; ++rr)
        if (rr < world) {
            const float v = (uint32_t)(w[rr] >> 32) == seq ? __uint_as_float((uint32_t)w[rr])
                                                            : wait_word(slots + (size_t)rr * astride + off, seq, timeout_ns, status, code);
            s = rr == 0 ? v : s + v;
        }
    return s;
}

// ---------------------------------------------------------------- step sequence
// The step number that tags flags and selects the slot bank lives in device memory, so a
// captured CUDA graph can be replayed: every CTA reads it when the kernel starts, and the last
// CTA to finish publishes the next value for the kernel that follows on the stream.
__device__ __forceinline__ uint32_t step_begin(const RankCtx &X) {
    return *reinterpret_cast<volatile uint32_t *>(X.step_ctr) + 1u;
}
__device__ __forceinline__ void step_end(const RankCtx &X, uint32_t seq, uint32_t ncta) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t prev = atomicAdd(X.step_ctr + 1, 1u);
        if (prev + 1u == ncta) {
            X.step_ctr[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(X.step_ctr) = seq;
        }
    }
}

// Host-buffer calls write their results straight into pinned host memory and the host waits on one
// word there instead of on the stream.  Every CTA, once all of its threads have stored their results,
// fences at system scope (its stores have then reached host memory: a PCIe round trip, ~3 us) and
// counts itself in; the CTA that counts last stores {1, status word}.  That store is issued after every
// CTA's fence has completed, so the host cannot see it before the results, and needs no second fence.
__device__ __forceinline__ void host_done_signal(const RankCtx &X, uint32_t ncta) {
    if (X.host_done == nullptr) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t prev = atomicAdd(X.step_ctr + 2, 1u);
        if (prev + 1u == ncta) {
            X.step_ctr[2] = 0u;
            __threadfence();  // the count is read before the word is written
            const uint64_t word = ((uint64_t)1 << 32) | *reinterpret_cast<volatile uint32_t *>(X.status);
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(X.host_done), "l"(word) : "memory");
        }
    }
}

// ---------------------------------------------------------------- activation quantiser
// The reference's dynamic FP8 activation quantisation, bit for bit
// (crates/weightstream-ref/src/actquant.rs:21-45; device twin
// crates/weightstream-cuda/kernels/actquant.cu:47-83): per 32 contiguous values,
// amax floored at 1e-4, scale 2^ceil(log2(amax/448)) taken from the exponent and
// mantissa bits of the quotient, value/scale rounded to nearest even onto the
// E4M3 grid with saturation at +-448.
__device__ __forceinline__ int act_scale_exp(float amax) {
    amax = fmaxf(amax, 1e-4f);
    const uint32_t bits = __float_as_uint(__fdiv_rn(amax, 448.0f));
    return (int)((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFF) ? 1 : 0);
}
__device__ __forceinline__ float pow2_f32(int e) {  // 2^e for any e: inf above 127, subnormal/0 below -126
    if (e > 127) return __uint_as_float(0x7F800000u);
    if (e >= -126) return __uint_as_float((uint32_t)(e + 127) << 23);
    return e >= -149 ? __uint_as_float(1u << (e + 149)) : 0.0f;
}
// Two floats -> two E4M3 bytes (lo = a, hi = b), RNE, saturating, NaN -> 0x7F.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float a, float b) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(b), "f"(a));
    return r;
}
// Eight values held by one lane (a quarter of a 32-block spread over 4 adjacent
// lanes): returns the block exponent and the eight E4M3 bytes in k order.
__device__ __forceinline__ void act_quant8(const float (&v)[8], int &e, uint32_t &lo, uint32_t &hi) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    e = act_scale_exp(amax);
    const float inv = e > 127 ? 0.0f : pow2_f32(-e);  // an infinite block scale divides everything to zero
    lo = cvt_e4m3x2(v[0] * inv, v[1] * inv) | (cvt_e4m3x2(v[2] * inv, v[3] * inv) << 16);
    hi = cvt_e4m3x2(v[4] * inv, v[5] * inv) | (cvt_e4m3x2(v[6] * inv, v[7] * inv) << 16);
}

// Load eight consecutive activations (bf16 or f32) as floats, zero beyond `valid`.
__device__ __forceinline__ void load_act8(const void *base, int x_dtype, int64_t elem_off, bool valid,
                                          float (&v)[8]) {
    if (!valid) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        return;
    }
    if (x_dtype == WS_ACT_BF16) {
        const uint4 r = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(base) + elem_off));
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    } else {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem_off));
        const float4 b = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem_off) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

}  // namespace ws
