// FP8 E4M3 row-parallel decode GEMM on the 5th-generation tensor cores (tcgen05 + TMEM),
// fused with its exchange (sm_100a).  Up to 8 activation rows per launch.
//
// One persistent CTA per SM owns a contiguous range of output rows and streams their weights
// over the full local K, so every row is a complete dot product inside one CTA.  The range is
// walked in chunks of at most 128 rows = the M of one UMMA tile (rows past the range are
// computed on whatever lies in shared memory and never read back).  Per 128-byte K slab one
// TMA box (chunk rows x 128 bytes, 128B swizzle) lands in the stage ring; one thread issues
// four tcgen05.mma.kind::f8f6f4 (M=128, N=16, K=32): K=32 is exactly one block of the
// reference's activation quantisation, and each of the four writes its own group of TMEM
// columns with a zero accumulator.  Four epilogue warps read the columns back (tcgen05.ld) and
// add d * (s_act * s_w) in fp32 registers -- activation scales per 32, weight scales per block,
// any scale format -- while the next slab's MMAs run into the other TMEM buffers.
//
// The activations (quantised in the prologue exactly as the reference does) are the B operand:
// 8 token rows x 128 bytes per slab in the canonical 128B-swizzled K-major layout; the
// descriptor's 8-row stride is 0, so MMA columns 8..15 repeat tokens 0..7 and are ignored.
//
// Exchange and lm_head mode are those of the mma.sync kernel (ws_fp8_kernel.cuh): partial rows
// are stored into every peer's slot, one flag per CTA and peer, rank-ordered add; or gather +
// argmax candidates.
#pragma once

#include <math.h>

#include "ws_device.cuh"
#include "ws_fp8_kernel.cuh"

namespace ws {

constexpr int kUmmaThreads = 192;   // warp 0: TMA, warp 1: MMA issue + TMEM owner, warps 2-5: epilogue
constexpr int kUmmaSlabCols = 64;   // TMEM columns one slab needs: 4 K-blocks x 16 MMA columns
constexpr int kUmmaTmemCols = 512;  // all of it: a TMEM buffer holds the accumulators of one whole stage
constexpr int kUmmaMaxBufs = 8;

struct alignas(64) UmmaParams {
    CUtensorMap tmap[WS_MAX_WORLD];  // per rank: weight shard [n][k bytes], box 128 bytes x chunk_rows, 128B swizzle
    int32_t m, n, k, x_dtype, scale_kind, bn, bk;
    int32_t world, mode, vocab, gather_logits;
    int32_t bk_shift, bn_shift;
    int32_t chunk_rows, nchunk;      // rows per chunk (<= 128) and chunks per CTA
    int32_t slabs_per_stage, nstages, pitch;  // pitch = bytes one slab occupies in a stage (chunk rows padded to 8)
    int32_t skb, nslot_max;
    uint64_t timeout_ns;
    SymLayout lay;
    Fp8RankArgs r[WS_MAX_WORLD];
};

struct UmmaSmem {
    int32_t stages, q, sa, sw, bars, misc, total;
};
__host__ __device__ inline UmmaSmem umma_smem_layout(int nstages, int slabs_per_stage, int pitch, int kslabs,
                                                     int nslot_max, int skb) {
    UmmaSmem s{};
    int o = 0;
    s.stages = o; o += (int)align_up((int64_t)nstages * slabs_per_stage * pitch, 1024);
    s.q = o;      o += kslabs * 1024;              // 8 tokens x 128 bytes per slab (also the MMA's read-past area)
    if (kslabs * 1024 < 16384) o += 16384 - kslabs * 1024;
    s.sa = o;     o += kslabs * 4 * 8 * 4;
    s.sw = o;     o += (int)align_up((int64_t)nslot_max * skb * 4, 16);
    s.bars = o;   o += (2 * kMaxStages + kUmmaMaxBufs) * 8;
    s.misc = o;   o += 64 + 4 * 8 * 8;             // TMEM base, per-warp argmax candidates
    s.total = o;
    return s;
}

// ---- tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] = A[smem] * B[smem], E4M3 x E4M3 -> F32, accumulator not read (a fresh sum per K block).
__device__ __forceinline__ void umma_f8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(0u), "r"(0u)
        : "memory");
}
// Issue (do not wait for) the load of 8 consecutive columns of this warp's 32 TMEM lanes.
__device__ __forceinline__ void tmem_ld8_issue(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
// Wait for every TMEM load issued so far.  The registers pass through the statement so that no
// use of them can be scheduled before the wait.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                   "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                   "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}
// Shared-memory matrix descriptor: K-major, 128B swizzle, 8-row groups `sbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);         // start address, 16-byte units
    d |= (uint64_t)1 << 16;                           // leading byte offset: unused with 128B swizzle, K-major
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;      // stride between 8-row groups
    d |= (uint64_t)1 << 46;                           // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                           // SWIZZLE_128B
    return d;
}
constexpr uint32_t kUmmaIdesc = (1u << 4)      // D = F32
                                | (0u << 7)    // A = E4M3
                                | (0u << 10)   // B = E4M3
                                | (2u << 17)   // N = 16
                                | (8u << 24);  // M = 128

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 2, 128;" ::: "memory"); }   // warps 2-5
__device__ __forceinline__ void quant_bar() { asm volatile("bar.sync 3, 160;" ::: "memory"); } // warps 1-5

__global__ void __launch_bounds__(kUmmaThreads, 1) fp8_umma_kernel(const __grid_constant__ UmmaParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);

    const int vr = blockIdx.y, cta = blockIdx.x, ncta = gridDim.x;
    const Fp8RankArgs &A = p.r[vr];
    const RankCtx &X = A.ctx;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t seq = step_begin(X);

    const int kslabs = (p.k + 127) >> 7;
    const int kb32 = p.k >> 5;
    const int SL = p.slabs_per_stage, NS = p.nstages;
    // rows of this CTA: [row_a, row_b), walked in p.nchunk chunks of p.chunk_rows
    const int row_a = (int)((int64_t)cta * p.n / ncta), row_b = (int)((int64_t)(cta + 1) * p.n / ncta);

    const UmmaSmem S = umma_smem_layout(NS, SL, p.pitch, kslabs, p.nslot_max, p.skb);
    uint8_t *q_s = smem + S.q;
    float *sa_s = reinterpret_cast<float *>(smem + S.sa);
    float *sw_s = reinterpret_cast<float *>(smem + S.sw);
    uint32_t *misc_s = reinterpret_cast<uint32_t *>(smem + S.misc);
    const uint32_t stage0 = smem_u32(smem + S.stages);
    // full[s]: the stage's TMA bytes landed.  done[s]: every MMA of the stage completed (ONE
    // tcgen05.commit per stage) -- the producer reads it as "stage free", the epilogue as
    // "accumulators ready".  tempty[b]: TMEM buffer b has been drained.
    const uint32_t full0 = smem_u32(smem + S.bars), done0 = full0 + kMaxStages * 8;
    const uint32_t tempty0 = done0 + kMaxStages * 8;
    const int NB = kUmmaTmemCols / (SL * kUmmaSlabCols);  // TMEM buffers (host keeps SL <= 4, so NB >= 2)
    const uint32_t stage_bytes = (uint32_t)(SL * p.pitch);

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(done0 + s * 8, 1);
        }
        for (int b = 0; b < kUmmaMaxBufs; ++b) mbar_init(tempty0 + b * 8, 4);  // one arrival per epilogue warp
        mbar_fence_init();
    }
    if (warp == 1) {  // TMEM: allocated and freed by the same warp
        tmem_alloc(smem_u32(misc_s), kUmmaTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(misc_s);
    const uint32_t bank = seq & 1u;
    const int nflag = kMaxCtas + kMaxShared;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int item = 0;
            for (int c = 0; c < p.nchunk; ++c) {
                const int r0 = row_a + c * p.chunk_rows;
                for (int s0 = 0; s0 < kslabs; s0 += SL) {
                    const int nsl = min(SL, kslabs - s0);
                    const int s = item % NS;
                    mbar_wait(done0 + s * 8, (((uint32_t)(item / NS)) & 1u) ^ 1u, X.status);
                    mbar_arrive_expect_tx(full0 + s * 8, (uint32_t)(nsl * p.chunk_rows * 128));
                    for (int j = 0; j < nsl; ++j)
                        tma_load_2d(stage0 + s * stage_bytes + j * p.pitch, &p.tmap[vr], (s0 + j) * 128, r0, full0 + s * 8);
                    ++item;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ prologue (warps 1-5)
        // weight scales of this CTA's rows as fp32, then the activation quantisation into the
        // MMA's B layout: slab s, token t, 16-byte chunk c at q_s + s*1024 + t*128 + ((c ^ t) << 4).
        const int qt = tid - 32;
        const int64_t kcol0 = A.k0 >> p.bk_shift;
        const int64_t srow_lo = (A.row0 + row_a) >> p.bn_shift;
        const int nslot = row_b > row_a ? (int)(((A.row0 + row_b - 1) >> p.bn_shift) - srow_lo + 1) : 0;
        const int ncols = (int)(((A.k0 + p.k - 1) >> p.bk_shift) - kcol0 + 1);
        for (int i = qt; i < nslot * ncols; i += 160) {
            const int sl = i / ncols, c = i - sl * ncols;
            const int64_t idx = (srow_lo + sl) * A.scale_ld + kcol0 + c;
            float s;
            if (p.scale_kind == WS_SCALE_UE8M0) {
                const uint32_t b = __ldg(static_cast<const uint8_t *>(A.scales) + idx);
                s = (b == 0xFFu) ? __uint_as_float(0x7FC00000u)
                                 : (b == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(b << 23));
            } else {
                s = __ldg(static_cast<const float *>(A.scales) + idx);
            }
            sw_s[sl * p.skb + c] = s;
        }
        // Only the m token rows the launch carries are written: the MMA columns of the other
        // tokens are computed on whatever the rows hold and are never read back.
        const int chunks_per_row = kslabs * 16;  // 8-element chunks over the padded K
        const int total = p.m * chunks_per_row;
        const int total_up = (total + 31) & ~31;
        for (int c0 = qt; c0 < total_up; c0 += 8 * 160) {  // eight loads in flight per thread
            float v[8][8];
            int tok[8], ch[8];
            bool valid[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int c = c0 + u * 160;
                tok[u] = c / chunks_per_row;
                ch[u] = c - tok[u] * chunks_per_row;
                valid[u] = c < total && ch[u] * 8 < p.k;
                load_act8(A.x, p.x_dtype, (int64_t)tok[u] * A.ldx + ch[u] * 8, valid[u], v[u]);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int c = c0 + u * 160;
                if (c >= total_up) break;  // warp-uniform
                int e;
                uint32_t lo, hi;
                act_quant8(v[u], e, lo, hi);
                if (c < total) {
                    const int slab = ch[u] >> 4, c16 = (ch[u] & 15) >> 1, half = ch[u] & 1;
                    *reinterpret_cast<uint2 *>(q_s + slab * 1024 + tok[u] * 128 + ((c16 ^ tok[u]) << 4) + half * 8) =
                        valid[u] ? make_uint2(lo, hi) : make_uint2(0u, 0u);
                    if ((ch[u] & 3) == 0) sa_s[(ch[u] >> 2) * 8 + tok[u]] = valid[u] ? pow2_f32(e) : 0.0f;
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA
        quant_bar();

        if (warp == 1) {
            // -------------------------------------------------------- MMA issue (one thread)
            if (lane == 0) {
                int item = 0;
                for (int c = 0; c < p.nchunk; ++c) {
                    for (int s0 = 0; s0 < kslabs; s0 += SL, ++item) {
                        const int nsl = min(SL, kslabs - s0);
                        const int s = item % NS, tb = item % NB;
                        mbar_wait(tempty0 + tb * 8, (((uint32_t)(item / NB)) & 1u) ^ 1u, X.status);
                        mbar_wait(full0 + s * 8, ((uint32_t)(item / NS)) & 1u, X.status);
                        tc_fence_after();
                        for (int j = 0; j < nsl; ++j) {
                            const int slab = s0 + j;
                            const uint32_t a_addr = stage0 + s * stage_bytes + j * p.pitch;
                            const uint32_t b_addr = smem_u32(q_s) + slab * 1024;
                            const int nblk = min(4, kb32 - slab * 4);
                            for (int b = 0; b < nblk; ++b)
                                umma_f8_ss(tmem_base + (tb * SL + j) * kUmmaSlabCols + b * 16,
                                           umma_desc(a_addr + b * 32, 1024), umma_desc(b_addr + b * 32, 0), kUmmaIdesc);
                        }
                        umma_commit(done0 + s * 8);  // stage consumed and its accumulators complete
                    }
                }
            }
            __syncwarp();
        } else {
            // -------------------------------------------------------- epilogue warps 2-5
            const int et = tid - 64;                     // 0..127
            const int quad = warp & 3;                   // TMEM lanes this warp may read
            const int rc = quad * 32 + lane;             // row inside the chunk = TMEM lane
            const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
            const int kofs = (int)(A.k0 - kcol0 * p.bk);
            const bool solo = p.mode == kModeAllReduce && p.world == 1;
            const size_t astride = (size_t)p.lay.max_m * p.lay.max_n;
            float cbv[8];
            uint32_t cbi[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) { cbv[t] = -INFINITY; cbi[t] = 0xFFFFFFFFu; }
            int item0 = 0;  // first stage item of the current chunk
            for (int c = 0; c < p.nchunk; ++c) {
                const int row = row_a + c * p.chunk_rows + rc;
                const bool mine = rc < p.chunk_rows && row < row_b;
                const float *swrow = sw_s + (mine ? (int)(((A.row0 + row) >> p.bn_shift) - srow_lo) : 0) * p.skb;
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                // Drain one slab: its four K blocks are loaded with one wait, and the loads of the
                // next slab are in flight while this slab's products are added.
                uint32_t cur[32], nxt[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) cur[i] = nxt[i] = 0u;
                // slab `sl` of this chunk lives in stage item (item0 + sl / SL), TMEM buffer item % NB
                auto issue_slab = [&](int sl, uint32_t (&r)[32]) {
                    const int item = item0 + sl / SL, j = sl % SL;
                    if (j == 0) {
                        mbar_wait(done0 + (item % NS) * 8, ((uint32_t)(item / NS)) & 1u, X.status);
                        tc_fence_after();
                    }
                    const int nblk = min(4, kb32 - sl * 4);
                    const uint32_t col = tlane + ((item % NB) * SL + j) * kUmmaSlabCols;
#pragma unroll
                    for (int b = 0; b < 4; ++b)
                        if (b < nblk) tmem_ld8_issue(col + b * 16, *reinterpret_cast<uint32_t (*)[8]>(&r[b * 8]));
                };
                auto loaded_slab = [&](int sl) {  // after the wait: the last slab of a stage frees its TMEM buffer
                    if ((sl % SL) == SL - 1 || sl == kslabs - 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty0 + ((item0 + sl / SL) % NB) * 8);
                    }
                };
                auto add_slab = [&](int slab, const uint32_t (&r)[32]) {
                    const int nblk = min(4, kb32 - slab * 4);
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        if (b >= nblk) break;
                        const int kb = slab * 4 + b;
                        const float sw = swrow[(kofs + kb * 32) >> p.bk_shift];
                        const float4 s0 = *reinterpret_cast<const float4 *>(sa_s + kb * 8);
                        const float4 s1 = *reinterpret_cast<const float4 *>(sa_s + kb * 8 + 4);
                        acc[0] = fmaf(__uint_as_float(r[b * 8 + 0]), s0.x * sw, acc[0]);
                        acc[1] = fmaf(__uint_as_float(r[b * 8 + 1]), s0.y * sw, acc[1]);
                        acc[2] = fmaf(__uint_as_float(r[b * 8 + 2]), s0.z * sw, acc[2]);
                        acc[3] = fmaf(__uint_as_float(r[b * 8 + 3]), s0.w * sw, acc[3]);
                        acc[4] = fmaf(__uint_as_float(r[b * 8 + 4]), s1.x * sw, acc[4]);
                        acc[5] = fmaf(__uint_as_float(r[b * 8 + 5]), s1.y * sw, acc[5]);
                        acc[6] = fmaf(__uint_as_float(r[b * 8 + 6]), s1.z * sw, acc[6]);
                        acc[7] = fmaf(__uint_as_float(r[b * 8 + 7]), s1.w * sw, acc[7]);
                    }
                };
                issue_slab(0, cur);
                tmem_ld_wait(cur);
                loaded_slab(0);
                for (int slab = 0; slab < kslabs; slab += 2) {
                    // cur holds slab; fetch slab+1 into nxt while adding cur, then the other way round
                    if (slab + 1 < kslabs) issue_slab(slab + 1, nxt);
                    add_slab(slab, cur);
                    if (slab + 1 < kslabs) {
                        tmem_ld_wait(nxt);
                        loaded_slab(slab + 1);
                        if (slab + 2 < kslabs) issue_slab(slab + 2, cur);
                        add_slab(slab + 1, nxt);
                        if (slab + 2 < kslabs) {
                            tmem_ld_wait(cur);
                            loaded_slab(slab + 2);
                        }
                    }
                }
                item0 += (kslabs + SL - 1) / SL;
                // publish this chunk's rows
                if (mine) {
                    if (solo) {
#pragma unroll
                        for (int t = 0; t < 8; ++t)
                            if (t < p.m) A.out[(size_t)t * p.n + row] = acc[t];
                    } else if (p.mode == kModeAllReduce) {
                        for (int pr = 0; pr < p.world; ++pr) {
                            float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.slotf_off) +
                                         ((size_t)bank * p.world + X.rank) * astride;
#pragma unroll
                            for (int t = 0; t < 8; ++t)
                                if (t < p.m) dst[(size_t)t * p.n + row] = acc[t];
                        }
                    } else {
                        if (p.gather_logits)
                            for (int pr = 0; pr < p.world; ++pr) {
                                float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.gather_off) +
                                             (size_t)bank * p.lay.max_m * (size_t)p.lay.max_vocab;
#pragma unroll
                                for (int t = 0; t < 8; ++t)
                                    if (t < p.m) dst[(size_t)t * p.lay.max_vocab + A.vocab_row0 + row] = acc[t];
                            }
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            const uint32_t idx = (uint32_t)(A.vocab_row0 + row);
                            if (t < p.m && acc[t] > -INFINITY && cand_better(acc[t], idx, cbv[t], cbi[t])) { cbv[t] = acc[t]; cbi[t] = idx; }
                        }
                    }
                }
            }

            // ---- exchange (the 128 epilogue threads)
            const uint32_t *myflags = solo ? nullptr
                                           : reinterpret_cast<const uint32_t *>(X.sym[X.rank] + p.lay.flags_off) +
                                                 (size_t)bank * p.world * nflag;
            if (!solo && p.mode == kModeAllReduce) {
                epi_bar();  // the st.release.sys below is cumulative over the stores this barrier ordered
                if (et < p.world) {
                    uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[et] + p.lay.flags_off) +
                                  ((size_t)bank * p.world + X.rank) * nflag;
                    st_release_sys(f + cta, seq);
                    wait_flag(myflags + (size_t)et * nflag + cta, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
                }
                epi_bar();
                const float *slots = reinterpret_cast<const float *>(X.sym[X.rank] + p.lay.slotf_off) +
                                     (size_t)bank * p.world * astride;
                for (int c = 0; c < p.nchunk; ++c) {
                    const int row = row_a + c * p.chunk_rows + rc;
                    if (rc < p.chunk_rows && row < row_b)
                        for (int t = 0; t < p.m; ++t) {
                            const size_t off = (size_t)t * p.n + row;
                            float s = __ldcg(slots + off);
                            for (int rr = 1; rr < p.world; ++rr) s += __ldcg(slots + rr * astride + off);
                            A.out[off] = s;
                        }
                }
            } else if (p.mode == kModeLmHead) {
                // best (value, lowest index) of this CTA's rows per token -> every peer's candidate table
                float *cv_s = reinterpret_cast<float *>(misc_s + 16);       // [4 warps][8 tokens]
                uint32_t *ci_s = misc_s + 16 + 32;
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    float bv = cbv[t];
                    uint32_t bi = cbi[t];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                        if (cand_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                    }
                    if (lane == 0) { cv_s[quad * 8 + t] = bv; ci_s[quad * 8 + t] = bi; }
                }
                epi_bar();
                if (et < p.m) {
                    float bv = cv_s[et];
                    uint32_t bi = ci_s[et];
                    for (int w = 1; w < 4; ++w)
                        if (cand_better(cv_s[w * 8 + et], ci_s[w * 8 + et], bv, bi)) { bv = cv_s[w * 8 + et]; bi = ci_s[w * 8 + et]; }
                    for (int pr = 0; pr < p.world; ++pr) {
                        uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[pr] + p.lay.pairs_off) +
                                        (((size_t)bank * p.world + X.rank) * kMaxCtas + cta) * p.lay.max_m + et;
                        *dst = ((uint64_t)__float_as_uint(bv) << 32) | bi;
                    }
                }
                epi_bar();  // the st.release.sys below is cumulative over the stores this barrier ordered
                if (et < p.world) {
                    uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[et] + p.lay.flags_off) +
                                  ((size_t)bank * p.world + X.rank) * nflag;
                    st_release_sys(f + cta, seq);
                }
                const bool copies = p.gather_logits && A.logits != nullptr;
                if (copies || cta == 0) {
                    // every CTA of every rank has published (its flag follows all of its stores)
                    for (int i = et; i < p.world * ncta; i += 128)
                        wait_flag(myflags + (size_t)(i / ncta) * nflag + (i % ncta), seq, p.timeout_ns, X.status,
                                  kStatTimeoutGather);
                    epi_bar();
                    if (copies) {
                        const float *gl = reinterpret_cast<const float *>(X.sym[X.rank] + p.lay.gather_off) +
                                          (size_t)bank * p.lay.max_m * (size_t)p.lay.max_vocab;
                        const int64_t per = ((int64_t)p.vocab + ncta - 1) / ncta;
                        const int64_t v0 = (int64_t)cta * per, v1 = min((int64_t)p.vocab, v0 + per);
                        for (int t = 0; t < p.m; ++t)
                            for (int64_t v = v0 + et; v < v1; v += 128)
                                A.logits[(size_t)t * p.vocab + v] = __ldcg(gl + (size_t)t * p.lay.max_vocab + v);
                    }
                    if (cta == 0 && A.argmax != nullptr) {
                        const uint64_t *pairs = reinterpret_cast<const uint64_t *>(X.sym[X.rank] + p.lay.pairs_off) +
                                                (size_t)bank * p.world * kMaxCtas * p.lay.max_m;
                        for (int t = warp - 2; t < p.m; t += 4) {
                            float bv = -INFINITY;
                            uint32_t bi = 0xFFFFFFFFu;
                            for (int i = lane; i < p.world * ncta; i += 32) {
                                const uint64_t pr = ld_volatile_u64(pairs + ((size_t)(i / ncta) * kMaxCtas + (i % ncta)) * p.lay.max_m + t);
                                const float v = __uint_as_float((uint32_t)(pr >> 32));
                                const uint32_t idx = (uint32_t)pr;
                                if (cand_better(v, idx, bv, bi)) { bv = v; bi = idx; }
                            }
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) {
                                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                                const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                                if (cand_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                            }
                            if (lane == 0) A.argmax[t] = (bi == 0xFFFFFFFFu) ? 0u : bi;
                        }
                    }
                }
            }
        }
    }

    // ---- teardown: every TMEM read and MMA has completed once all threads are here
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kUmmaTmemCols);
    }
    if (p.world > 1 || p.mode == kModeLmHead) step_end(X, seq, gridDim.x);
}

}  // namespace ws
