// MXFP4 routed-expert down projection + top-k combine fused with its exchange on the 5th-generation
// tensor cores (sm_100a): tcgen05.mma.kind::mxf8f6f4.block_scale computes exactly this step's product,
// E2M1 weights x E4M3 activations with a UE8M0 scale per 32 values on BOTH operands, so a pass
// accumulates over all of K in tensor memory and the SMs only move bytes.
//
// Two kernels per step:
//
//   moe_bs_prep_kernel  one block per route: its position among the rank's routes sorted by expert
//                       (a pass = one local expert with up to 16 of its routes as MMA columns, experts
//                       in ascending id as crates/weightstream-ref/src/moe.rs:75-84 adds them),
//                       hidden x routing-weight quantised as the reference does (moe.rs:150, then
//                       actquant.rs:21-57) into E4M3 rows at that position, and the per-32 exponents
//                       into the pass's 512-byte scale atoms (one per 128-wide K slab: byte
//                       (t & 31) * 16 + (t >> 5) * 4 + j = exponent of column t, K block j).
//   moe_bs_kernel       persistent CTA pairs (clusters of 2), one pair per tile of ~97 output rows,
//                       each CTA of a pair streams half of K of every pass: with a lone CTA's ~48
//                       rows under half of the MMA's 128 rows would be real, and the tensor pipe
//                       needs the same ~35 ns per K=32 MMA however few are.  Warp 0 lane 0 streams,
//                       per 128-wide K slab, the expert's rows (TMA, 4-bit codes unpacked by the
//                       copy into the 16-bytes-per-16-codes form the MMA reads), the pass's
//                       activation rows (TMA) and their scale atom (bulk copy).  Four warps turn the
//                       weights' UE8M0 bytes (4 consecutive bytes per row and slab in the reference's
//                       [expert][row][k/32] layout) into scale atoms in shared memory, one pass ahead.
//                       Warp 1 lane 0 copies both atoms of a slab into tensor memory and issues its
//                       four MMAs; one commit per stage frees it, one per pass hands the accumulator
//                       (16 columns, double-buffered) to the four epilogue warps, which add column t
//                       to the shared-memory sums of the token that route belongs to.  After the last
//                       pass the second CTA hands its sums to the first through distributed shared
//                       memory; that one adds them after its own and stores the rows or exchanges them.
//
// Exchange: as in the FP8 kernels (partials stored to every peer as tagged words, folded in rank order).
#pragma once

#include <math.h>

#include "ws_device.cuh"
#include "ws_fp8_bs_kernel.cuh"      // tcgen05 / cluster wrappers, kBsAtomBytes, kBsMmaRows
#include "ws_moe_gemv_kernel.cuh"    // MoePass, kMoeMaxRoutes, kMoeMaxExperts

namespace ws {

constexpr int kMoeBsCols = 16;        // routes of one expert per pass = N of the MMA
constexpr int kMoeBsThreads = 320;    // warp 0 producer, 1 MMA issue, 2-5 epilogue, 6-9 weight-scale atoms
constexpr int kMoeBsMaxSlabs = 16;    // K slabs one CTA walks per pass (k <= 4096 with pairs)

// Per-endpoint scratch written by moe_bs_prep_kernel and read by moe_bs_kernel.
// The activations of a pass are stored as the main kernel's shared memory wants them, so that ONE bulk
// copy fills a stage: per pass and group of `sl` K slabs, sl tiles of 16 rows x 128 bytes (128B-swizzled
// K-major, the layout a TMA box would produce) followed by their sl scale atoms.
constexpr int kMoeBsXTile = kMoeBsCols * 128;                 // 2048
constexpr int kMoeBsXSlab = kMoeBsXTile + kBsAtomBytes;       // 2560 bytes of a stage per slab
struct MoeBsWork {
    int64_t hdr, pass, stok, xs, total;  // byte offsets
};
__host__ __device__ inline MoeBsWork moe_bs_work_layout(int k) {
    MoeBsWork w{};
    int64_t o = 0;
    w.hdr = o;  o += 64;
    w.pass = o; o += (int64_t)kMoeMaxRoutes * sizeof(MoePass);
    w.stok = o; o += align_up((int64_t)(kMoeMaxRoutes + kMoeBsCols) * 2, 256);
    w.xs = o;   o += (int64_t)kMoeMaxRoutes * (k / 128) * kMoeBsXSlab;  // [pass][slab group][tiles | atoms]
    w.total = o;
    return w;
}

struct MoeBsPrepParams {
    int32_t m, k, top_k, h_dtype;
    int32_t sl, pad0;  // K slabs per stage of the main kernel (a group of the layout above)
    MoePrepRank r[WS_MAX_WORLD];
};

__device__ __forceinline__ int block_sum_256(int v, int *red_s) {  // all 256 threads get the sum
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red_s[warp] = v;
    __syncthreads();
    int s = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red_s[w];
    return s;
}

__global__ void __launch_bounds__(256) moe_bs_prep_kernel(const __grid_constant__ MoeBsPrepParams p) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const MoePrepRank &A = p.r[blockIdx.y];
    const int NR = p.m * p.top_k, tid = threadIdx.x;
    const MoeBsWork W = moe_bs_work_layout(p.k);
    __shared__ int32_t cnt_s[kMoeMaxExperts];
    __shared__ int red_s[8];
    for (int i = tid; i < A.e_len; i += blockDim.x) cnt_s[i] = 0;
    __syncthreads();
    for (int i = tid; i < NR; i += blockDim.x) {
        const int e = A.route_ids[i] - A.e_start;
        if (e >= 0 && e < A.e_len) atomicAdd(&cnt_s[e], 1);
    }
    __syncthreads();
    if ((int)blockIdx.x == NR) {  // the extra block: how many passes the step has
        int np = 0;
        for (int e = tid; e < A.e_len; e += blockDim.x) np += (cnt_s[e] + kMoeBsCols - 1) / kMoeBsCols;
        np = block_sum_256(np, red_s);
        if (tid == 0) *reinterpret_cast<int32_t *>(A.work + W.hdr) = np;
        return;
    }
    const int route = blockIdx.x;
    const int e = A.route_ids[route] - A.e_start;
    if (e < 0 || e >= A.e_len) return;  // another rank's expert (or none)
    // position among the rank's routes sorted by (expert, route), rank among the expert's routes,
    // and the passes of the experts before this one
    int pos = 0, rnk = 0, pb = 0;
    for (int i = tid; i < NR; i += blockDim.x) {
        const int ei = A.route_ids[i] - A.e_start;
        if (ei < 0 || ei >= A.e_len) continue;
        if (ei < e || (ei == e && i < route)) ++pos;
        if (ei == e && i < route) ++rnk;
    }
    for (int i = tid; i < e; i += blockDim.x) pb += (cnt_s[i] + kMoeBsCols - 1) / kMoeBsCols;
    pos = block_sum_256(pos, red_s);
    rnk = block_sum_256(rnk, red_s);
    pb = block_sum_256(pb, red_s);
    const int pass = pb + rnk / kMoeBsCols, t = rnk % kMoeBsCols;
    if (tid == 0) {
        if (t == 0) {
            MoePass ps;
            ps.expert = (uint16_t)e;
            ps.first = (uint16_t)pos;
            ps.nr = (uint16_t)min(kMoeBsCols, cnt_s[e] - rnk);
            ps.pad = 0;
            reinterpret_cast<MoePass *>(A.work + W.pass)[pass] = ps;
        }
        reinterpret_cast<uint16_t *>(A.work + W.stok)[pos] = (uint16_t)(route / p.top_k);
    }
    const float w = A.route_w[route];
    uint8_t *xs = A.work + W.xs + (size_t)pass * (p.k >> 7) * kMoeBsXSlab;
    const int group_bytes = p.sl * kMoeBsXSlab;
    for (int c = tid; c < (p.k >> 3); c += blockDim.x) {  // the four chunks of a 32-block are adjacent lanes
        float v[8];
        load_act8(A.h, p.h_dtype, (int64_t)route * A.ldh + c * 8, true, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= w;
        int ex;
        uint32_t lo, hi;
        act_quant8(v, ex, lo, hi);
        // 8 values = half of a 16-byte chunk of row t of the slab's tile; chunk cc sits at (cc ^ (t & 7))
        const int slab = c >> 4, cc = (c >> 1) & 7, half = c & 1;
        uint8_t *grp = xs + (size_t)(slab / p.sl) * group_bytes;
        const int j = slab % p.sl;
        *reinterpret_cast<uint2 *>(grp + j * kMoeBsXTile + t * 128 + ((cc ^ (t & 7)) << 4) + half * 8) = make_uint2(lo, hi);
        if ((c & 3) == 0)
            grp[p.sl * kMoeBsXTile + j * kBsAtomBytes + t * 16 + ((c >> 2) & 3)] = (uint8_t)min(max(ex + 127, 0), 255);
    }
}

// ------------------------------------------------------------------------------------------
struct MoeBsRank {
    const uint8_t *s2;    // [e_len][n][k/32] UE8M0
    const uint8_t *work;  // MoeBsWork
    float *out;           // [m][n]
    int32_t e_start, e_len;
    RankCtx ctx;
};

struct alignas(64) MoeBsParams {
    CUtensorMap tmap_w[WS_MAX_WORLD];  // expert slab as [e_len][n][k] 4-bit codes; boxes of 128 codes x tile_rows x 1, unpacked, 128B swizzle
    int32_t m, n, k, world;
    int32_t tile_rows, a_pitch, slabs_per_stage, nstages;
    int32_t tmem_cols, pad0;
    uint64_t timeout_ns;
    SymLayout lay;
    MoeBsRank r[WS_MAX_WORLD];
};

struct MoeBsSmem {
    int32_t a, b, sfa, acc, rx, bars, misc, total;
};
__host__ __device__ inline MoeBsSmem moe_bs_smem_layout(int nstages, int slabs_per_stage, int a_pitch, int m, int nslab_cta) {
    MoeBsSmem s{};
    const int nsl = nstages * slabs_per_stage;
    const int b_bytes = nsl * kMoeBsXSlab;  // per stage: its slabs' activation tiles, then their scale atoms (one bulk copy)
    int o = 0;
    s.a = o;    o += nsl * a_pitch;
    s.b = o;    o += b_bytes;
    if (b_bytes < kBsMmaRows * 128) o += kBsMmaRows * 128 - b_bytes;  // an MMA reads 128 rows behind the last weight slab
    s.sfa = o;  o += 2 * nslab_cta * kBsAtomBytes;                      // weight-scale atoms of two passes
    s.acc = o;  o += m * kBsMmaRows * 4;                                // sums of (token, row)
    s.rx = o;   o += m * kBsMmaRows * 4;                                // the partner's, at the end
    s.bars = o; o += (2 * kMaxStages + 8) * 8;
    s.misc = o; o += 64;
    s.total = o;
    return s;
}

// 3-D TMA tile load (codes, rows, expert), completion on an mbarrier.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}

// Instruction descriptor: E2M1 weights (format code 5) x E4M3 activations, UE8M0 scales, M = 128, N = 16.
__device__ __forceinline__ uint32_t moe_bs_idesc(int sf_id) {
    return ((uint32_t)sf_id << 4) | (5u << 7) | (0u << 10) | ((uint32_t)(kMoeBsCols >> 3) << 17) | (1u << 23) | (8u << 24) |
           ((uint32_t)sf_id << 29);
}

__global__ void __launch_bounds__(kMoeBsThreads, 1) moe_bs_kernel(const __grid_constant__ MoeBsParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);

    const int vr = blockIdx.y, cta = blockIdx.x, ncta = gridDim.x;
    const MoeBsRank &A = p.r[vr];
    const RankCtx &X = A.ctx;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t crank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
    const int part = cta >> 1, TR = p.tile_rows;
    const int row0 = part * TR;                                     // this pair's rows [row0, row0 + TR)
    const int KS = p.k >> 7;
    const int k_lo = (int)crank * KS / 2, k_hi = ((int)crank + 1) * KS / 2;
    const int NSLAB = k_hi - k_lo;                                  // slabs this CTA walks per pass
    const int SL = p.slabs_per_stage, NS = p.nstages;
    const int IP = (NSLAB + SL - 1) / SL;                           // stage items per pass

    const MoeBsSmem S = moe_bs_smem_layout(NS, SL, p.a_pitch, p.m, NSLAB);
    const MoeBsWork W = moe_bs_work_layout(p.k);
    float *acc_s = reinterpret_cast<float *>(smem + S.acc);
    uint32_t *misc_s = reinterpret_cast<uint32_t *>(smem + S.misc);
    const uint32_t a0 = smem_u32(smem + S.a), b0 = smem_u32(smem + S.b), sfa0 = smem_u32(smem + S.sfa);
    const uint32_t stage_x = (uint32_t)(SL * kMoeBsXSlab);  // a stage's activation tiles and scale atoms
    // full[s]: a stage's bytes landed; done[s]: its MMAs have completed (stage free); accfull[g] /
    // accempty[g]: a pass's accumulator is complete (and its scale columns free again) / has been read;
    // sfafull[g]: the weight scales of a pass are in tensor memory.
    const uint32_t full0 = smem_u32(smem + S.bars), done0 = full0 + kMaxStages * 8;
    const uint32_t accfull0 = done0 + kMaxStages * 8, accempty0 = accfull0 + 16, sfafull0 = accempty0 + 16;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(done0 + s * 8, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accfull0 + b * 8, 1);
            mbar_init(accempty0 + b * 8, 4);    // one arrival per epilogue warp
            mbar_init(sfafull0 + b * 8, 1);     // the commit that follows the scale warps' copies
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(misc_s), (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    for (int i = tid; i < p.m * kBsMmaRows; i += kMoeBsThreads) acc_s[i] = 0.0f;
    if (tid == 0) misc_s[8] = 0u;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(misc_s);
    // tensor-memory columns: two accumulators of 16, then per pass buffer and slab 4 activation-scale
    // and 4 weight-scale columns
    const uint32_t t_sc0 = tmem_base + 2u * kMoeBsCols;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // everything below depends on the prep kernel's pass table
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int npass = *reinterpret_cast<const volatile int32_t *>(A.work + W.hdr);
    const MoePass *passes = reinterpret_cast<const MoePass *>(A.work + W.pass);

    if (warp == 0) {
        // ------------------------------------------------------------ producer (one thread)
        if (lane == 0) {
            // the unpacking copy counts the packed bytes it read (64 per row), not the 128 it wrote
            const uint32_t slab_tx = (uint32_t)(TR * 64 + kMoeBsXSlab);
            RingPos st;
            int item = 0;
            for (int ps = 0; ps < npass; ++ps) {
                const MoePass P = passes[ps];
                const uint8_t *xs = A.work + W.xs + ((size_t)ps * KS + k_lo) * kMoeBsXSlab;  // this CTA's slab groups of the pass
                for (int i = 0; i < IP; ++i, ++item, st.next(NS)) {
                    const int s = st.s, j0 = i * SL, nsl = min(SL, NSLAB - j0);
                    if (item >= NS && !mbar_wait(done0 + s * 8, st.ph ^ 1u, X.status)) { ps = npass; break; }
                    mbar_arrive_expect_tx(full0 + s * 8, (uint32_t)nsl * slab_tx);
                    for (int j = 0; j < nsl; ++j)
                        tma_load_3d(a0 + (s * SL + j) * p.a_pitch, &p.tmap_w[vr], (k_lo + j0 + j) * 128, row0, (int)P.expert, full0 + s * 8);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(b0 + s * stage_x), "l"(xs + (size_t)i * stage_x), "r"(stage_x), "r"(full0 + s * 8) : "memory");
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issue (one thread)
        if (lane == 0) {
            const uint32_t id0 = moe_bs_idesc(0), id1 = moe_bs_idesc(1), id2 = moe_bs_idesc(2), id3 = moe_bs_idesc(3);
            const uint32_t a_lo0 = umma_desc_lo(a0), b_lo0 = umma_desc_lo(b0);
            const uint32_t a_step = (uint32_t)p.a_pitch >> 4, b_step = (uint32_t)kMoeBsXTile >> 4;
            const uint64_t sf_desc0 = umma_desc(b0 + (uint32_t)(SL * kMoeBsXTile), 128, false);  // a stage's atoms follow its tiles
            const uint32_t sf_step = (uint32_t)kBsAtomBytes >> 4;
            RingPos st;
            bool ok = true;
            for (int ps = 0; ps < npass && ok; ++ps) {
                const int g = ps & 1;
                const uint32_t lap = (uint32_t)(ps >> 1) & 1u;
                if (!mbar_wait(sfafull0 + g * 8, lap, X.status) || !mbar_wait(accempty0 + g * 8, lap ^ 1u, X.status)) break;
                tc_fence_after();
                const uint32_t t_acc = tmem_base + (uint32_t)(g * kMoeBsCols);
                uint32_t t_sc = t_sc0 + (uint32_t)(g * NSLAB * 8);
                bool first = true;
                for (int i = 0; i < IP; ++i, st.next(NS)) {
                    const int s = st.s, nsl = min(SL, NSLAB - i * SL);
                    if (!mbar_wait(full0 + s * 8, st.ph, X.status)) { ok = false; break; }
                    tc_fence_after();
                    uint32_t a_lo = a_lo0 + (uint32_t)(s * SL) * a_step, b_lo = b_lo0 + (uint32_t)s * (stage_x >> 4);
                    uint64_t sf_desc = sf_desc0 + (uint64_t)((uint32_t)s * (stage_x >> 4));
                    for (int j = 0; j < nsl; ++j) {
                        tmem_cp_atom(t_sc, sf_desc);          // the activations' scales of this slab (the weights' are there already)
                        if (first) umma_bs_ss<false>(t_acc, a_lo, b_lo, kUmmaDescHiSw128, kUmmaDescHiSw128, id0, t_sc + 4, t_sc);
                        else umma_bs_ss<true>(t_acc, a_lo, b_lo, kUmmaDescHiSw128, kUmmaDescHiSw128, id0, t_sc + 4, t_sc);
                        umma_bs_ss<true>(t_acc, a_lo + 2, b_lo + 2, kUmmaDescHiSw128, kUmmaDescHiSw128, id1, t_sc + 4, t_sc);
                        umma_bs_ss<true>(t_acc, a_lo + 4, b_lo + 4, kUmmaDescHiSw128, kUmmaDescHiSw128, id2, t_sc + 4, t_sc);
                        umma_bs_ss<true>(t_acc, a_lo + 6, b_lo + 6, kUmmaDescHiSw128, kUmmaDescHiSw128, id3, t_sc + 4, t_sc);
                        first = false;
                        a_lo += a_step; b_lo += b_step; sf_desc += sf_step;
                        t_sc += 8;
                    }
                    umma_commit(done0 + s * 8);  // the stage may be refilled
                }
                if (!ok) break;
                umma_commit(accfull0 + g * 8);   // the pass's sums are complete; its scale columns may be rewritten
            }
        }
        __syncwarp();
    } else if (warp >= 6) {
        // ------------------------------------------------------------ weight scales, one pass ahead
        // The expert's UE8M0 bytes of this CTA's rows and K half become scale atoms in shared memory
        // (thread = row), and one thread copies them into the pass's tensor-memory columns: the
        // MMA-issuing thread only waits for that commit.
        const int r = tid - 192;  // 0..127: row of the tile = lane of the atom
        const int row = row0 + r;
        const bool real = r < TR && row < p.n;
        const int kb32 = p.k >> 5;
        const uint64_t sfa_desc0 = umma_desc(sfa0, 128, false);
        for (int ps = 0; ps < npass; ++ps) {
            const int g = ps & 1;
            const uint32_t lap = (uint32_t)(ps >> 1) & 1u;
            // the pass that used these columns and this buffer last (ps - 2) has completed; a wait that
            // gave up is told to all four warps at the barrier below, so that they leave the loop together
            if (ps >= 2 && !mbar_wait(accfull0 + g * 8, lap ^ 1u, X.status)) misc_s[8] = 1u;
            const int e = passes[ps].expert;
            uint8_t *dst = smem + S.sfa + (size_t)(g * NSLAB) * kBsAtomBytes + (r & 31) * 16 + (r >> 5) * 4;
            const uint32_t *src = reinterpret_cast<const uint32_t *>(A.s2 + ((size_t)e * p.n + (real ? row : 0)) * kb32) + k_lo;
            for (int j = 0; j < NSLAB; ++j)
                *reinterpret_cast<uint32_t *>(dst + (size_t)j * kBsAtomBytes) = real ? __ldg(src + j) : 0x7F7F7F7Fu;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 3, 128;" ::: "memory");
            if (*reinterpret_cast<volatile uint32_t *>(misc_s + 8) != 0u) break;
            if (r == 0) {
                tc_fence_after();
                const uint32_t t_sfa = t_sc0 + (uint32_t)(g * NSLAB * 8) + 4u;
                for (int j = 0; j < NSLAB; ++j)
                    tmem_cp_atom(t_sfa + (uint32_t)(j * 8), sfa_desc0 + (uint64_t)((uint32_t)(g * NSLAB + j) * ((uint32_t)kBsAtomBytes >> 4)));
                umma_commit(sfafull0 + g * 8);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps 2-5
        const int quad = warp & 3;
        const int rc = quad * 32 + lane;  // row inside the tile = TMEM lane
        const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint16_t *stok = reinterpret_cast<const uint16_t *>(A.work + W.stok);
        bool ok = true;
        for (int ps = 0; ps < npass; ++ps) {
            const int g = ps & 1;
            const uint32_t lap = (uint32_t)(ps >> 1) & 1u;
            const MoePass P = passes[ps];
            if (ok && !mbar_wait(accfull0 + g * 8, lap, X.status)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t v[kMoeBsCols];
            tmem_ld_cols<kMoeBsCols>(tlane + (uint32_t)(g * kMoeBsCols), v);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(accempty0 + g * 8);
#pragma unroll
            for (int t = 0; t < kMoeBsCols; ++t)
                if (t < (int)P.nr) acc_s[(int)stok[P.first + t] * kBsMmaRows + rc] += __uint_as_float(v[t]);
        }
    }

    // ---- the pair's halves of K: the second CTA's sums go to the first
    __syncthreads();
    float *rx_s = reinterpret_cast<float *>(smem + S.rx);
    if (crank == 1) {
        const uint32_t dst = mapa_u32(smem_u32(rx_s), 0u);
        for (int i = tid; i < p.m * kBsMmaRows; i += kMoeBsThreads) st_cluster_f32(dst + (uint32_t)i * 4u, acc_s[i]);
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");

    const bool solo = p.world == 1;
    if (crank == 0) {
        const uint32_t seq = step_begin(X);
        const uint32_t bank = seq & 1u;
        const size_t astride = (size_t)p.lay.max_m * p.lay.max_n;
        // K half 0 (own) + K half 1 (the partner's), in that order; thread -> (token, row)
        for (int i = tid; i < p.m * kBsMmaRows; i += kMoeBsThreads) {
            const int tok = i >> 7, rc = i & 127, row = row0 + rc;
            if (rc >= TR || row >= p.n) continue;
            const float v = acc_s[i] + rx_s[i];
            if (solo) {
                A.out[(size_t)tok * p.n + row] = v;
            } else {
                for (int pr = 0; pr < p.world; ++pr) {
                    uint64_t *dstw = reinterpret_cast<uint64_t *>(X.sym[pr] + p.lay.slota_off) + ((size_t)bank * p.world + X.rank) * astride;
                    st_word_sys(dstw + (size_t)tok * p.n + row, seq, v);
                }
            }
        }
        if (!solo) {  // fold the same rows in rank order as the ranks' words arrive
            const uint64_t *slots = reinterpret_cast<const uint64_t *>(X.sym[X.rank] + p.lay.slota_off) + (size_t)bank * p.world * astride;
            for (int i = tid; i < p.m * kBsMmaRows; i += kMoeBsThreads) {
                const int tok = i >> 7, rc = i & 127, row = row0 + rc;
                if (rc >= TR || row >= p.n) continue;
                const size_t off = (size_t)tok * p.n + row;
                A.out[off] = fold_words(slots, astride, off, p.world, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
            }
        }
    }

    // ---- teardown
    tc_fence_before();
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
    if (p.world > 1) step_end(X, step_begin(X), gridDim.x);
}

}  // namespace ws
