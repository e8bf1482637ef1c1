// FP8 E4M3 row-parallel GEMM on the 5th-generation tensor cores with block scaling
// (tcgen05.mma.kind::mxf8f6f4.block_scale, accumulators in tensor memory), fused with its
// exchange (sm_100a).  One pass over the weights for up to 64 activation rows.
//
// Two kernels per step:
//
//   act_prep_kernel   quantises the activations once per step exactly as the reference does
//                     (crates/weightstream-ref/src/actquant.rs:21-57): E4M3 bytes [mp][k] and the
//                     per-32 UE8M0 exponents in the layout the MMA's scale operand wants (one 512-byte
//                     atom per 128-wide K slab: byte (t & 31) * 16 + (t >> 5) * 4 + j holds the exponent
//                     of token t, K block 4 * slab + j).  Both stay in L2 for the main kernel.
//   fp8_bs_kernel     persistent, one CTA per SM.  A CTA owns a contiguous range of output rows,
//                     walked in chunks of at most 128 rows = the M of one MMA tile, and streams their
//                     weights over the whole local K, so every output is a complete dot product
//                     inside one CTA.  Per 128-byte K slab the producer warp lands, in one stage of a
//                     shared-memory ring: the weight rows (TMA box, 128B swizzle), the quantised
//                     activations of all tokens (TMA box from the prep kernel's buffer) and their
//                     scale atom (bulk copy).  One thread copies the atom into tensor memory
//                     (tcgen05.cp) and issues four MMAs (M=128, N=tokens, K=32): the activations'
//                     per-32 scales ride the MMA's scale operand, the weight operand's scale is 2^0,
//                     and the four K blocks accumulate in tensor memory.  The weights' own scales are
//                     fp32 per (block_n x block_k) block, which no MMA scale format can carry, so
//                     four epilogue warps read each slab's accumulators back (tcgen05.ld) and add
//                     them, times the fp32 weight scale, to their registers while the next slabs'
//                     MMAs run into the other accumulator buffers.
//
// Rows past a chunk's end are computed on whatever follows in shared memory and never read back.
// Exchange and lm_head mode are those of the decode kernel (ws_fp8_kernel.cuh): tagged 64-bit
// words stored into every peer's slots and folded in rank order, or gather + argmax candidates.
#pragma once

#include <math.h>

#include "ws_device.cuh"
#include "ws_fp8_kernel.cuh"

namespace ws {

constexpr int kBsThreads = 192;      // warp 0: producer, warp 1: MMA issue + TMEM owner, warps 2-5: epilogue
constexpr int kBsTmemCols = 512;
constexpr int kBsMaxAcc = 8;         // accumulator buffers in tensor memory
constexpr int kBsMaxTokens = 64;     // activation rows one launch takes
constexpr int kBsAtomBytes = 512;    // one scale atom: 128 rows x 4 K blocks

// ---------------------------------------------------------------- activation prep
struct ActPrepRank {
    const void *x;
    uint8_t *xq;   // [mp][k] E4M3
    uint8_t *sfb;  // [k / 128][512] scale atoms
    int64_t ldx;
};
struct ActPrepParams {
    int32_t m, mp, k, x_dtype;
    ActPrepRank r[WS_MAX_WORLD];
};

__global__ void __launch_bounds__(256) act_prep_kernel(const __grid_constant__ ActPrepParams p) {
    // The step that follows may become resident at once (it streams weights until its own wait);
    // the activations come from earlier work on the stream.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const ActPrepRank &A = p.r[blockIdx.y];
    const int chunks_per_row = p.k >> 3;
    const int64_t total = (int64_t)p.mp * chunks_per_row;
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool in = c < total;
    const int tok = in ? (int)(c / chunks_per_row) : 0;
    const int ch = in ? (int)(c - (int64_t)tok * chunks_per_row) : 0;
    const bool valid = in && tok < p.m;
    float v[8];
    load_act8(A.x, p.x_dtype, (int64_t)tok * A.ldx + ch * 8, valid, v);
    int e;
    uint32_t lo, hi;
    act_quant8(v, e, lo, hi);  // the four lanes of a 32-block are adjacent threads of one warp
    if (in) {
        *reinterpret_cast<uint2 *>(A.xq + (int64_t)tok * p.k + ch * 8) = valid ? make_uint2(lo, hi) : make_uint2(0u, 0u);
        if ((ch & 3) == 0) {
            const int kb = ch >> 2;
            const int eb = valid ? min(max(e + 127, 0), 255) : 127;
            A.sfb[(size_t)(kb >> 2) * kBsAtomBytes + (tok & 31) * 16 + (tok >> 5) * 4 + (kb & 3)] = (uint8_t)eb;
        }
    }
}

// ---------------------------------------------------------------- main kernel
struct alignas(64) BsParams {
    CUtensorMap tmap_w[WS_MAX_WORLD];  // weight shard [n][k bytes], box 128 bytes x chunk_rows, 128B swizzle
    CUtensorMap tmap_x[WS_MAX_WORLD];  // quantised activations [mp][k bytes], box 128 bytes x mp, 128B swizzle
    int32_t m, mp, n, k, bn_shift, bk_shift;
    int32_t world, mode, vocab, gather_logits;
    int32_t chunk_rows, nchunk;        // rows per chunk (<= 128) and chunks per CTA
    int32_t slabs_per_stage, nstages;
    int32_t a_pitch, b_pitch;          // bytes one slab's weights / activations occupy in a stage (multiples of 1024)
    int32_t skb, nslot_max, nacc, l2_prefetch;
    uint64_t timeout_ns;
    SymLayout lay;
    Fp8RankArgs r[WS_MAX_WORLD];       // x is unused here; scales/out/logits/argmax/row0/k0/ctx as in the decode kernel
    const uint8_t *sfb[WS_MAX_WORLD];  // the prep kernel's scale atoms
    const uint8_t *w[WS_MAX_WORLD];    // weight shard base and row stride (L2 prefetch only; the data path uses tmap_w)
    int64_t ldw[WS_MAX_WORLD];
};

struct BsSmem {
    int32_t a, b, sf, sfa, sw, cand, bars, misc, total;
};
__host__ __device__ inline BsSmem bs_smem_layout(int nstages, int slabs_per_stage, int a_pitch, int b_pitch, int nslot_max,
                                                 int skb, int mp) {
    BsSmem s{};
    const int nsl = nstages * slabs_per_stage;
    int o = 0;
    s.a = o;    o += nsl * a_pitch;
    s.b = o;    o += nsl * b_pitch;
    // an MMA reads 128 rows of its weight slab whatever the chunk holds: keep 16 KB readable behind the last one
    if (nsl * b_pitch < 16384) o += 16384 - nsl * b_pitch;
    s.sf = o;   o += nsl * kBsAtomBytes;
    s.sfa = o;  o += kBsAtomBytes;
    s.sw = o;   o += (int)align_up((int64_t)nslot_max * skb * 4, 16);
    s.cand = o; o += 4 * mp * 8;                         // lm_head: per epilogue warp and token (value, index)
    s.bars = o; o += (2 * kMaxStages + 2 * kBsMaxAcc) * 8;
    s.misc = o; o += 64;
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
// Shared-memory matrix descriptor, K-major: 128B swizzle with 8-row groups `sbo` bytes apart
// (operands), or no swizzle (scale atoms: 8-row x 16-byte core matrices `sbo` bytes apart).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t sbo, bool swizzle128) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);         // start address, 16-byte units
    if (swizzle128) d |= (uint64_t)1 << 16;           // leading byte offset: unused with 128B swizzle, K-major
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;      // stride between 8-row groups
    d |= (uint64_t)1 << 46;                           // descriptor version of sm_100
    if (swizzle128) d |= (uint64_t)2 << 61;           // SWIZZLE_128B
    return d;
}
// Instruction descriptor of the block-scaled MMA: E4M3 x E4M3, UE8M0 scales, M = 128, N = n;
// sfa / sfb pick the byte (K block of the slab) inside the scale operands' 32-bit columns.
__device__ __forceinline__ uint32_t bs_idesc(int n, int sfa, int sfb) {
    return ((uint32_t)sfb << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | (8u << 24) |
           ((uint32_t)sfa << 29);
}
// D[tmem] (+)= A[smem] * B[smem] with per-32 scales from tensor memory.
__device__ __forceinline__ void umma_bs_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa,
                                           uint32_t tsfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
        : "memory");
}
// One 512-byte scale atom (32 rows x 16 bytes) -> 4 columns of all 128 TMEM lanes.
__device__ __forceinline__ void tmem_cp_atom(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// N consecutive columns of this warp's 32 TMEM lanes -> registers; the wait is part of the same
// statement, so no use of the registers can be scheduled before the data has arrived.
#define WS_R4(a, i) "=r"(a[i]), "=r"(a[i + 1]), "=r"(a[i + 2]), "=r"(a[i + 3])
#define WS_R16(a, i) WS_R4(a, i), WS_R4(a, i + 4), WS_R4(a, i + 8), WS_R4(a, i + 12)
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[N]);
template <>
__device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : WS_R16(r, 0) : "r"(taddr) : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : WS_R16(r, 0), WS_R16(r, 16) : "r"(taddr) : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_cols<64>(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,"
        "%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : WS_R16(r, 0), WS_R16(r, 16), WS_R16(r, 32), WS_R16(r, 48) : "r"(taddr) : "memory");
}
#undef WS_R16
#undef WS_R4

__device__ __forceinline__ void bs_epi_bar() { asm volatile("bar.sync 2, 128;" ::: "memory"); }  // warps 2-5

template <int MP>
__global__ void __launch_bounds__(kBsThreads, 1) fp8_bs_kernel(const __grid_constant__ BsParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);

    const int vr = blockIdx.y, cta = blockIdx.x, ncta = gridDim.x;
    const Fp8RankArgs &A = p.r[vr];
    const RankCtx &X = A.ctx;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int kslabs = p.k >> 7;
    const int SL = p.slabs_per_stage, NS = p.nstages, NB = p.nacc;
    const int row_a = (int)((int64_t)cta * p.n / ncta), row_b = (int)((int64_t)(cta + 1) * p.n / ncta);
    const int items_per_chunk = (kslabs + SL - 1) / SL;

    const BsSmem S = bs_smem_layout(NS, SL, p.a_pitch, p.b_pitch, p.nslot_max, p.skb, MP);
    float *sw_s = reinterpret_cast<float *>(smem + S.sw);
    uint32_t *misc_s = reinterpret_cast<uint32_t *>(smem + S.misc);
    const uint32_t a0 = smem_u32(smem + S.a), b0 = smem_u32(smem + S.b), sf0 = smem_u32(smem + S.sf);
    // full[s]: the stage's bytes landed.  done[s]: every MMA that reads the stage completed.
    // accfull[b] / accempty[b]: accumulator buffer b holds a finished slab / has been read back.
    const uint32_t full0 = smem_u32(smem + S.bars), done0 = full0 + kMaxStages * 8;
    const uint32_t accfull0 = done0 + kMaxStages * 8, accempty0 = accfull0 + kBsMaxAcc * 8;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(done0 + s * 8, 1);
        }
        for (int b = 0; b < kBsMaxAcc; ++b) {
            mbar_init(accfull0 + b * 8, 1);
            mbar_init(accempty0 + b * 8, 4);  // one arrival per epilogue warp
        }
        mbar_fence_init();
    }
    if (warp == 1) {  // tensor memory: allocated and freed by the same warp
        tmem_alloc(smem_u32(misc_s), kBsTmemCols);
        tmem_relinquish();
    }
    if (warp >= 2) {  // the weight operand's scale atom: 2^0 everywhere
        uint32_t *sfa = reinterpret_cast<uint32_t *>(smem + S.sfa);
        sfa[tid - 64] = 0x7F7F7F7Fu;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(misc_s);
    // tensor-memory columns: NB accumulator buffers of MP columns, then NB x 4 activation-scale columns
    // (one scale atom per buffer), then the 4 weight-scale columns
    const uint32_t t_sfb0 = tmem_base + (uint32_t)(NB * MP);
    const uint32_t t_sfa = t_sfb0 + (uint32_t)(NB * 4);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            // Weights are static: the first ring's worth streams before the wait on the prep kernel;
            // the activations and their scales follow once it has finished.
            const int total_items = p.nchunk * items_per_chunk;
            auto issue_w = [&](int it) {
                const int c = it / items_per_chunk, s0 = (it - c * items_per_chunk) * SL;
                const int nsl = min(SL, kslabs - s0), s = it % NS;
                const int r0 = row_a + c * p.chunk_rows;
                for (int j = 0; j < nsl; ++j)
                    tma_load_2d(a0 + (s * SL + j) * p.a_pitch, &p.tmap_w[vr], (s0 + j) * 128, r0, full0 + s * 8);
            };
            auto issue_x = [&](int it) {
                const int c = it / items_per_chunk, s0 = (it - c * items_per_chunk) * SL;
                const int nsl = min(SL, kslabs - s0), s = it % NS;
                for (int j = 0; j < nsl; ++j) {
                    tma_load_2d(b0 + (s * SL + j) * p.b_pitch, &p.tmap_x[vr], (s0 + j) * 128, 0, full0 + s * 8);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(sf0 + (s * SL + j) * kBsAtomBytes), "l"(p.sfb[vr] + (size_t)(s0 + j) * kBsAtomBytes),
                                   "r"((uint32_t)kBsAtomBytes), "r"(full0 + s * 8) : "memory");
                }
            };
            auto expect = [&](int it) {
                const int c = it / items_per_chunk, s0 = (it - c * items_per_chunk) * SL;
                const int nsl = min(SL, kslabs - s0);
                mbar_arrive_expect_tx(full0 + (it % NS) * 8, (uint32_t)(nsl * (p.chunk_rows * 128 + MP * 128 + kBsAtomBytes)));
            };
            const int first = min(NS, total_items);
            for (int it = 0; it < first; ++it) {
                expect(it);
                issue_w(it);
            }
            if (p.l2_prefetch) {  // the rest of this CTA's weights start towards L2 while the predecessor finishes
                for (int c = 0; c < p.nchunk; ++c) {
                    const int r0 = row_a + c * p.chunk_rows, r1 = min(row_b, r0 + p.chunk_rows);
                    for (int r = r0; r < r1; ++r)
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;"
                                     ::"l"(p.w[vr] + (size_t)r * (size_t)p.ldw[vr]), "r"((uint32_t)p.k) : "memory");
                }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int it = 0; it < first; ++it) issue_x(it);
            for (int item = first; item < total_items; ++item) {
                const int s = item % NS;
                if (!mbar_wait(done0 + s * 8, (((uint32_t)(item / NS)) & 1u) ^ 1u, X.status)) break;
                expect(item);
                issue_w(item);
                issue_x(item);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issue (one thread)
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0) {
            tmem_cp_atom(t_sfa, umma_desc(smem_u32(smem + S.sfa), 128, false));
            int item = 0, slab_no = 0;
            bool ok = true;
            for (int c = 0; c < p.nchunk && ok; ++c) {
                for (int s0 = 0; s0 < kslabs && ok; s0 += SL, ++item) {
                    const int nsl = min(SL, kslabs - s0), s = item % NS;
                    if (!mbar_wait(full0 + s * 8, ((uint32_t)(item / NS)) & 1u, X.status)) { ok = false; break; }
                    tc_fence_after();
                    for (int j = 0; j < nsl; ++j, ++slab_no) {
                        const int tb = slab_no % NB;
                        if (!mbar_wait(accempty0 + tb * 8, (((uint32_t)(slab_no / NB)) & 1u) ^ 1u, X.status)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t t_acc = tmem_base + (uint32_t)(tb * MP);
                        const uint32_t t_sfb = t_sfb0 + (uint32_t)(tb * 4);
                        tmem_cp_atom(t_sfb, umma_desc(sf0 + (s * SL + j) * kBsAtomBytes, 128, false));
                        const uint32_t a_addr = a0 + (s * SL + j) * p.a_pitch, b_addr = b0 + (s * SL + j) * p.b_pitch;
#pragma unroll
                        for (int b = 0; b < 4; ++b)
                            umma_bs_ss(t_acc, umma_desc(a_addr + b * 32, 1024, true), umma_desc(b_addr + b * 32, 1024, true),
                                       bs_idesc(MP, 0, b), t_sfa, t_sfb, b ? 1u : 0u);
                        umma_commit(accfull0 + tb * 8);  // this slab's accumulators are complete
                    }
                    umma_commit(done0 + s * 8);          // ... and the stage may be refilled
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue warps 2-5
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t seq = step_begin(X);
        const uint32_t bank = seq & 1u;
        const int et = tid - 64;                     // 0..127
        const int quad = warp & 3;                   // TMEM lanes this warp may read
        const int rc = quad * 32 + lane;             // row inside the chunk = TMEM lane
        const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
        // weight scales of this CTA's rows as fp32: sw_s[slot][column]
        const int64_t kcol0 = A.k0 >> p.bk_shift;
        const int64_t srow_lo = (A.row0 + row_a) >> p.bn_shift;
        const int nslot = row_b > row_a ? (int)(((A.row0 + row_b - 1) >> p.bn_shift) - srow_lo + 1) : 0;
        const int ncols = (int)(((A.k0 + p.k - 1) >> p.bk_shift) - kcol0 + 1);
        for (int i = et; i < nslot * ncols; i += 128) {
            const int sl = i / ncols, c = i - sl * ncols;
            sw_s[sl * p.skb + c] = __ldg(static_cast<const float *>(A.scales) + (srow_lo + sl) * A.scale_ld + kcol0 + c);
        }
        bs_epi_bar();
        const int kofs = (int)(A.k0 - kcol0 * ((int64_t)1 << p.bk_shift));
        const bool solo = p.mode == kModeAllReduce && p.world == 1;
        const size_t astride = (size_t)p.lay.max_m * p.lay.max_n;
        const int nflag = kMaxCtas + kMaxShared;
        float *cv_s = reinterpret_cast<float *>(smem + S.cand);        // [4 warps][MP]
        uint32_t *ci_s = reinterpret_cast<uint32_t *>(smem + S.cand) + 4 * MP;
        if (p.mode == kModeLmHead)
            for (int i = lane; i < MP; i += 32) { cv_s[(warp - 2) * MP + i] = -INFINITY; ci_s[(warp - 2) * MP + i] = 0xFFFFFFFFu; }
        int slab_no = 0;
        bool ok = true;
        for (int c = 0; c < p.nchunk; ++c) {
            const int row = row_a + c * p.chunk_rows + rc;
            const bool mine = rc < p.chunk_rows && row < row_b;
            // a warp none of whose rows are real only keeps the accumulator buffers moving
            const bool wactive = quad * 32 < p.chunk_rows && row_a + c * p.chunk_rows + quad * 32 < row_b;
            const float *swrow = sw_s + (mine ? (int)(((A.row0 + row) >> p.bn_shift) - srow_lo) : 0) * p.skb;
            float acc[MP];
#pragma unroll
            for (int i = 0; i < MP; ++i) acc[i] = 0.0f;
            for (int sl = 0; sl < kslabs; ++sl, ++slab_no) {
                const int tb = slab_no % NB;
                if (ok && !mbar_wait(accfull0 + tb * 8, ((uint32_t)(slab_no / NB)) & 1u, X.status)) ok = false;
                tc_fence_after();
                if (wactive && ok) {
                    const float sw = swrow[(kofs + sl * 128) >> p.bk_shift];
                    uint32_t r[MP];
                    tmem_ld_cols<MP>(tlane + (uint32_t)(tb * MP), r);  // returns once the values are in registers
#pragma unroll
                    for (int i = 0; i < MP; ++i) acc[i] = fmaf(__uint_as_float(r[i]), sw, acc[i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(accempty0 + tb * 8);
            }
            // ---- this chunk's rows are final
            if (mine) {
                if (solo) {
#pragma unroll
                    for (int t = 0; t < MP; ++t)
                        if (t < p.m) A.out[(size_t)t * p.n + row] = acc[t];
                } else if (p.mode == kModeAllReduce) {
                    for (int pr = 0; pr < p.world; ++pr) {
                        uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[pr] + p.lay.slota_off) + ((size_t)bank * p.world + X.rank) * astride;
#pragma unroll
                        for (int t = 0; t < MP; ++t)
                            if (t < p.m) st_word_sys(dst + (size_t)t * p.n + row, seq, acc[t]);
                    }
                } else if (p.gather_logits) {
                    for (int pr = 0; pr < p.world; ++pr) {
                        float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.gather_off) + (size_t)bank * p.lay.max_m * (size_t)p.lay.max_vocab;
#pragma unroll
                        for (int t = 0; t < MP; ++t)
                            if (t < p.m) dst[(size_t)t * p.lay.max_vocab + A.vocab_row0 + row] = acc[t];
                    }
                }
            }
            if (p.mode == kModeLmHead && wactive) {
                // best (value, lowest index) of this warp's rows per token, merged into the warp's running best
                const uint32_t idx = (uint32_t)(A.vocab_row0 + row);
#pragma unroll
                for (int t = 0; t < MP; ++t) {
                    if (t >= p.m) break;
                    float bv = (mine && acc[t] > -INFINITY) ? acc[t] : -INFINITY;
                    uint32_t bi = (mine && acc[t] > -INFINITY) ? idx : 0xFFFFFFFFu;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                        if (cand_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                    }
                    if (lane == 0 && cand_better(bv, bi, cv_s[(warp - 2) * MP + t], ci_s[(warp - 2) * MP + t])) {
                        cv_s[(warp - 2) * MP + t] = bv;
                        ci_s[(warp - 2) * MP + t] = bi;
                    }
                }
            }
        }

        // ---- exchange (the 128 epilogue threads)
        const uint32_t *myflags = solo ? nullptr
                                       : reinterpret_cast<const uint32_t *>(X.sym[X.rank] + p.lay.flags_off) + (size_t)bank * p.world * nflag;
        if (!solo && p.mode == kModeAllReduce) {
            // fold the same rows in rank order as the ranks' words arrive
            const uint64_t *slots = reinterpret_cast<const uint64_t *>(X.sym[X.rank] + p.lay.slota_off) + (size_t)bank * p.world * astride;
            for (int c = 0; c < p.nchunk; ++c) {
                const int row = row_a + c * p.chunk_rows + rc;
                if (rc < p.chunk_rows && row < row_b)
                    for (int t = 0; t < p.m; ++t) {
                        const size_t off = (size_t)t * p.n + row;
                        float s = wait_word(slots + off, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
                        for (int rr = 1; rr < p.world; ++rr)
                            s += wait_word(slots + rr * astride + off, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
                        A.out[off] = s;
                    }
            }
        } else if (p.mode == kModeLmHead) {
            bs_epi_bar();
            if (et < p.m) {  // this CTA's candidate per token -> every peer's candidate table
                float bv = cv_s[et];
                uint32_t bi = ci_s[et];
                for (int w = 1; w < 4; ++w)
                    if (cand_better(cv_s[w * MP + et], ci_s[w * MP + et], bv, bi)) { bv = cv_s[w * MP + et]; bi = ci_s[w * MP + et]; }
                for (int pr = 0; pr < p.world; ++pr) {
                    uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[pr] + p.lay.pairs_off) +
                                    (((size_t)bank * p.world + X.rank) * kMaxCtas + cta) * p.lay.max_m + et;
                    *dst = ((uint64_t)__float_as_uint(bv) << 32) | bi;
                }
            }
            bs_epi_bar();  // the st.release.sys below is cumulative over the stores this barrier ordered
            if (et < p.world) {
                uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[et] + p.lay.flags_off) + ((size_t)bank * p.world + X.rank) * nflag;
                st_release_sys(f + cta, seq);
            }
            const bool copies = p.gather_logits && A.logits != nullptr;
            if (copies || cta == 0) {
                // every CTA of every rank has published (its flag follows all of its stores)
                for (int i = et; i < p.world * ncta; i += 128)
                    wait_flag(myflags + (size_t)(i / ncta) * nflag + (i % ncta), seq, p.timeout_ns, X.status, kStatTimeoutGather);
                bs_epi_bar();
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

    // ---- teardown: every TMEM read and MMA has completed once all threads are here
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kBsTmemCols);
    }
    if (p.world > 1 || p.mode == kModeLmHead) step_end(X, step_begin(X), gridDim.x);
}

}  // namespace ws
