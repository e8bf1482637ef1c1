// Bare collectives on device buffers and the stand-alone activation quantiser.
#pragma once

#include "ws_device.cuh"

namespace ws {

// Host-buffer calls with small inputs: the activations come out of the pinned host buffer (device-
// readable under unified addressing) into device memory, 16 bytes per thread.  The step's main kernel
// may become resident at once; it waits for this grid before it reads the activations.
struct StageParams {
    const uint4 *src;
    uint4 *dst;
    int64_t n16;
};
__global__ void __launch_bounds__(256) stage_in_kernel(const __grid_constant__ StageParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < p.n16) p.dst[i] = p.src[i];
}

struct CollRank {
    const float *in;
    float *out;
    RankCtx ctx;
};
struct CollParams {
    int64_t len;
    int32_t world, gather;
    uint32_t pad0_, pad;
    uint64_t timeout_ns;
    SymLayout lay;
    CollRank r[WS_MAX_WORLD];
};

// One-shot all-reduce / all-gather: every rank stores its vector into slot [rank] of
// every peer and then adds (rank order 0..R-1, crates/weightstream-transport/src/ring.rs:399-408)
// or concatenates (ring.rs:426-432) the slots.
__device__ __forceinline__ void coll_body(const CollParams &p, const uint32_t seq) {
    const int vr = blockIdx.y, cta = blockIdx.x, ncta = gridDim.x, tid = threadIdx.x;
    const CollRank &A = p.r[vr];
    const RankCtx &X = A.ctx;
    const int64_t a = (int64_t)cta * p.len / ncta, b = (int64_t)(cta + 1) * p.len / ncta;
    if (p.world == 1) {
        for (int64_t i = a + tid; i < b; i += blockDim.x) A.out[i] = A.in[i];
        return;
    }
    const uint32_t bank = seq & 1u;
    const size_t astride = (size_t)p.lay.max_m * p.lay.max_n;
    if (!p.gather) {  // all-reduce: tagged words, see st_word_sys
        for (int pr = 0; pr < p.world; ++pr) {
            uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[pr] + p.lay.slota_off) + ((size_t)bank * p.world + X.rank) * astride;
            for (int64_t i = a + tid; i < b; i += blockDim.x) st_word_sys(dst + i, seq, A.in[i]);
        }
        const uint64_t *slots = reinterpret_cast<const uint64_t *>(X.sym[X.rank] + p.lay.slota_off) + (size_t)bank * p.world * astride;
        for (int64_t i = a + tid; i < b; i += blockDim.x) {
            const float s = fold_words(slots, astride, (size_t)i, p.world, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
            A.out[i] = s;
        }
        return;
    }
    // all-gather: plain stores into the (float-addressed) slots, one released flag per CTA and peer
    const int nflag = kMaxCtas + kMaxShared;
    for (int pr = 0; pr < p.world; ++pr) {
        float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.slotf_off) + ((size_t)bank * p.world + X.rank) * astride;
        for (int64_t i = a + tid; i < b; i += blockDim.x) dst[i] = A.in[i];
    }
    __syncthreads();  // the st.release.sys below is cumulative over the stores this barrier ordered
    if (tid < p.world) {
        uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[tid] + p.lay.flags_off) + ((size_t)bank * p.world + X.rank) * nflag;
        st_release_sys(f + cta, seq);
    }
    const uint32_t *myflags = reinterpret_cast<const uint32_t *>(X.sym[X.rank] + p.lay.flags_off) + (size_t)bank * p.world * nflag;
    if (tid < p.world) wait_flag(myflags + (size_t)tid * nflag + cta, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
    __syncthreads();
    const float *slots = reinterpret_cast<const float *>(X.sym[X.rank] + p.lay.slotf_off) + (size_t)bank * p.world * astride;
    for (int r = 0; r < p.world; ++r)
        for (int64_t i = a + tid; i < b; i += blockDim.x) A.out[(int64_t)r * p.len + i] = __ldcg(slots + r * astride + i);
}

__global__ void __launch_bounds__(256) coll_kernel(const __grid_constant__ CollParams p) {
    const RankCtx &X = p.r[blockIdx.y].ctx;
    const uint32_t seq = step_begin(X);
    coll_body(p, seq);
    step_end(X, seq, gridDim.x);
}

// x [m, k] (bf16 or f32) -> q [m, k] E4M3 bytes, sexp [m, k/32] UE8M0 bytes.
__global__ void __launch_bounds__(256) act_quant_kernel(const void *x, int64_t ldx, int x_dtype, int m, int k,
                                                         uint8_t *q, uint8_t *sexp) {
    const int chunks_per_row = k >> 3;
    const int64_t total = (int64_t)m * chunks_per_row;
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = c < total;
    const int tok = valid ? (int)(c / chunks_per_row) : 0;
    const int ch = valid ? (int)(c - (int64_t)tok * chunks_per_row) : 0;
    float v[8];
    load_act8(x, x_dtype, (int64_t)tok * ldx + ch * 8, valid, v);
    int e;
    uint32_t lo, hi;
    act_quant8(v, e, lo, hi);
    if (valid) {
        *reinterpret_cast<uint2 *>(q + (int64_t)tok * k + ch * 8) = make_uint2(lo, hi);
        if ((ch & 3) == 0) sexp[(int64_t)tok * (k >> 5) + (ch >> 2)] = (uint8_t)(e + 127);
    }
}

}  // namespace ws
