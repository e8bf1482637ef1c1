// FP8 E4M3 row-parallel decode GEMM fused with its exchange (sm_100a).
//
// One persistent CTA per SM.  Every output row is a complete dot product inside ONE CTA:
// a CTA owns floor(n/16/ncta) whole 16-row tiles plus a ragged share (at most 16 rows) of the
// rows that are left over, so all SMs stream the same number of bytes and nothing is combined
// across CTAs.  Weight tiles arrive by TMA into a ring of 32 KB stages filled by one producer
// warp: 16-row x 128-byte boxes for whole tiles, 8/4/2/1-row boxes for the ragged rows, all
// 128B-swizzled.  The prologue quantises the activations exactly as the reference does; eight
// consumer warps then multiply the staged rows with them and apply the activation- and
// weight-block scales per 32-wide K block in fp32.  Two formulations of that product:
//   GT = 1, 2 (one or two activation rows): CUDA cores.  A lane owns 16 bytes of a row
//     (128-bit shared load), converts them to f16 pairs and accumulates exact products in fp32
//     (fma.rn.f32.f16); the eight lanes of a row are combined by shuffles at the end of a tile.
//     About 1.5 lane-instructions per weight byte, so HBM, not issue, bounds it.
//   GT = 0 (three to eight rows): the FP8 tensor-core MMA m16n8k32, one per 32-wide K block.
//     Its issue rate caps streaming near 70 % of HBM bandwidth, which is why it is not used
//     for the narrow cases.
//
// Exchange (world > 1): a thread stores its rows' fp32 partials into slot [my rank] of every
// peer's exchange memory as 64-bit {step, value} words and then adds the same rows' words of all
// ranks in rank order as they arrive, so all ranks produce identical bits.
//
// lm_head mode: rows are vocabulary entries; instead of a sum every rank's rows are gathered
// (stored into every peer's logits buffer) and each CTA publishes its best (value, lowest
// index) candidate per token; CTA 0 merges them.
#pragma once

#include <math.h>

#include "ws_device.cuh"

namespace ws {

enum { kModeAllReduce = 0, kModeLmHead = 1 };

struct Fp8RankArgs {
    const void *x;
    const void *scales;
    float *out;        // all-reduce mode: [m, n]
    float *logits;     // lm_head mode: [m, vocab] or null
    uint32_t *argmax;  // lm_head mode: [m] or null
    int64_t ldx, scale_ld, row0, k0, vocab_row0;
    RankCtx ctx;
};

struct alignas(64) Fp8Params {
    // TMA descriptors first: the TMA unit fetches them from the parameter block, and they are
    // fetched fastest from its first bytes.  Per rank: weight shard [n rows][k bytes] as boxes of
    // 128 bytes x 16 rows ([0]) and x `gran` rows ([1]), 128B swizzle.
    CUtensorMap tmap[WS_MAX_WORLD][2];
    int32_t m, n, k, x_dtype, scale_kind, bn, bk;
    int32_t world, mode, vocab, mp, nstages, nslot_max, skb;
    int32_t gather_logits, ragged;   // ragged = 0: leftover tiles go whole to the first CTAs
    int32_t bk_shift, bn_shift;      // log2 of the scale block edges
    int32_t part_rows, gran;         // partial rows reserved per token; row granularity (1,2,4,8) of the ragged share
    int32_t stage_bytes, l2_prefetch;  // bytes of one weight stage: a whole number of 2 KB boxes (fp8_stage_boxes); see below
    uint64_t timeout_ns;
    SymLayout lay;
    Fp8RankArgs r[WS_MAX_WORLD];
    // l2_prefetch: once the stage ring is full for the first time, the producer asks L2 for the rest
    // of this CTA's rows (weights are static), so that HBM keeps streaming while the predecessor on
    // the stream finishes and this kernel quantises its activations.  Needs the plain addresses:
    const uint8_t *w[WS_MAX_WORLD];
    int64_t ldw[WS_MAX_WORLD];
};

// Consumer warps per CTA.  Sixteen warps instead of eight changed neither formulation's time by
// more than 2 % on B200, so both run eight.
__host__ __device__ constexpr int fp8_consumer_warps(int) { return kConsumerWarps; }
__host__ __device__ constexpr int fp8_threads(int gt) { return (fp8_consumer_warps(gt) + 1) * 32; }  // + the TMA producer warp

struct Fp8Smem {  // byte offsets from the 1024-aligned base
    int32_t stages, q, sa, sw, red, part, bars, misc, total;
};

// gt: 0 for the MMA formulation (activations kept as E4M3 bytes, [kb][tok][32]), else the number
// of activation rows of the CUDA-core formulation (kept as f16, [tok][kbox*128]).
// Boxes (16 rows x 128 bytes) per stage: a tile's kbox boxes are cut into equal stages of at most
// kBoxesPerStage, so that no stage travels half empty (7168 columns = 56 boxes: four stages of 14
// instead of 16 + 16 + 16 + 8).
__host__ __device__ inline int fp8_stage_boxes(int kbox) {
    const int per_tile = (kbox + kBoxesPerStage - 1) / kBoxesPerStage;
    return (kbox + per_tile - 1) / per_tile;
}

__host__ __device__ inline Fp8Smem fp8_smem_layout(int nstages, int kbox, int mp, int nslot_max, int skb,
                                                   int m, int part_rows, int gt) {
    Fp8Smem s{};
    int o = 0;
    s.stages = o; o += nstages * fp8_stage_boxes(kbox) * kBoxBytes;
    s.q = o;      o += gt > 0 ? kbox * 128 * 2 * gt : kbox * 4 * mp * 32;
    s.sa = o;     o += kbox * 4 * (mp > 8 ? mp : 8) * 4;
    s.sw = o;     o += ((nslot_max * skb * 4 + 15) / 16) * 16;
    s.red = o;    o += 2 * fp8_consumer_warps(gt) * 128 * 4;
    s.part = o;   o += ((m * part_rows * 4 + 15) / 16) * 16;
    s.bars = o;   o += 2 * kMaxStages * 8;
    s.misc = o;   o += 128;
    s.total = o;
    return s;
}

// Row schedule shared by host and device.  Whole tiles: CTA c owns tiles [c*Gm, (c+1)*Gm).
// Leftover rows [Gm*ncta*16, n), in units of `gran` rows: CTA c takes units [c*U/ncta, (c+1)*U/ncta)
// (ragged), or, when ragged is off, CTA c < Rg takes leftover tile c whole.
struct RowPlan {
    int Gm, lb, e0, e1;  // whole tiles per CTA; first leftover row; this CTA's extra rows [e0, e1)
};
__host__ __device__ inline RowPlan row_plan(int n, int ncta, int cta, int ragged, int gran) {
    RowPlan r{};
    const int G = n / kGroupRows;
    r.Gm = G / ncta;
    r.lb = r.Gm * ncta * kGroupRows;
    const int L = n - r.lb;
    if (ragged) {
        const int U = L / gran;
        r.e0 = r.lb + gran * (int)((int64_t)cta * U / ncta);
        r.e1 = r.lb + gran * (int)((int64_t)(cta + 1) * U / ncta);
    } else {
        r.e0 = r.lb + cta * kGroupRows;
        r.e1 = r.e0 + kGroupRows;
        if (r.e0 >= n) r.e0 = r.e1 = n;
    }
    return r;
}

__device__ __forceinline__ bool cand_better(float v, uint32_t i, float bv, uint32_t bi) {
    return v > bv || (v == bv && i < bi);
}

template <int GT>
__device__ __forceinline__ void fp8_rowpar_kernel_body(const Fp8Params &p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);

    constexpr int CW = fp8_consumer_warps(GT), CT = CW * 32;  // consumer warps / threads of this formulation
    const int vr = blockIdx.y, cta = blockIdx.x, ncta = gridDim.x;
    const Fp8RankArgs &A = p.r[vr];
    const RankCtx &X = A.ctx;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int kbox = (p.k + 127) >> 7;
    const int kb32 = p.k >> 5;  // real 32-wide K blocks
    const RowPlan R = row_plan(p.n, ncta, cta, p.ragged, p.gran);
    // tiles of this CTA: Gm whole ones, then the extra rows cut at 16-row boundaries (so that a
    // tile never straddles a weight-scale block); tile t covers rows [trow(t), trow(t) + tcnt(t))
    const int xa = R.e0, xb = R.e1;
    const int xmid = min(xb, (xa / kGroupRows + 1) * kGroupRows);
    const int nx = xb > xa ? (xb > xmid ? 2 : 1) : 0;
    const int ntile = R.Gm + nx;
    auto trow = [&](int t) { return t < R.Gm ? (cta * R.Gm + t) * kGroupRows : (t == R.Gm ? xa : xmid); };
    auto tcnt = [&](int t) { return t < R.Gm ? kGroupRows : (t == R.Gm ? xmid - xa : xb - xmid); };
    // A tile of cnt rows is staged with a row pitch of tpad(cnt) (next power of two), so that a
    // stage always carries 16-32 KB: one box column = tpad rows x 128 bytes.
    auto tpad = [](int cnt) { return cnt > 8 ? 16 : cnt > 4 ? 8 : cnt > 2 ? 4 : cnt > 1 ? 2 : 1; };

    const Fp8Smem S = fp8_smem_layout(p.nstages, kbox, p.mp, p.nslot_max, p.skb, p.m, p.part_rows, GT);
    uint8_t *q_s = smem + S.q;
    float *sa_s = reinterpret_cast<float *>(smem + S.sa);
    float *sw_s = reinterpret_cast<float *>(smem + S.sw);
    float *red_s = reinterpret_cast<float *>(smem + S.red);
    float *part_s = reinterpret_cast<float *>(smem + S.part);  // [tok][part_rows], tile t at t*16
    const uint32_t stage0 = smem_u32(smem + S.stages);
    const uint32_t full0 = smem_u32(smem + S.bars), empty0 = full0 + kMaxStages * 8;
    const int NS = p.nstages;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(empty0 + s * 8, CW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    const int nflag = kMaxCtas + kMaxShared;
    // Let the next kernel on the stream begin (it only prefetches weights until its own wait).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == CW) {
        // ------------------------------------------------------------ TMA producer warp
        RingPos rp;
        int issued = 0;
        bool prefetched = !p.l2_prefetch;
        auto prefetch_rest = [&]() {  // every row of this CTA after its first tile, one request per row
            for (int t = 1; t < ntile; ++t)
                for (int r = lane; r < tcnt(t); r += 32)
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;"
                                 ::"l"(p.w[vr] + (size_t)(trow(t) + r) * (size_t)p.ldw[vr]), "r"((uint32_t)(p.k & ~15)) : "memory");
            prefetched = true;
        };
        for (int t = 0; t < ntile; ++t) {
            const int r0 = trow(t), cnt = tcnt(t);
            const int pad = tpad(cnt), cols = p.stage_bytes / (pad * 128);  // box columns one stage holds
            for (int b0 = 0; b0 < kbox; b0 += cols) {
                const int nb = min(cols, kbox - b0);
                const int s = rp.s;
                if (!mbar_wait(empty0 + s * 8, rp.ph ^ 1u, X.status)) return;  // a wait gave up: stop streaming
                if (lane == 0) mbar_arrive_expect_tx(full0 + s * 8, (uint32_t)(nb * cnt * 128));
                __syncwarp();
                for (int col = lane; col < nb; col += 32) {
                    const uint32_t dst = stage0 + s * p.stage_bytes + col * pad * 128;
                    if (cnt == kGroupRows) {  // a whole tile is one 16-row box, a ragged one is cnt/gran small boxes
                        tma_load_2d(dst, &p.tmap[vr][0], (b0 + col) * 128, r0, full0 + s * 8);
                    } else {
                        for (int done = 0; done < cnt; done += p.gran)
                            tma_load_2d(dst + done * 128, &p.tmap[vr][1], (b0 + col) * 128, r0 + done, full0 + s * 8);
                    }
                }
                rp.next(NS);
                if (!prefetched && ++issued >= NS) prefetch_rest();
            }
        }
        if (!prefetched) prefetch_rest();
        return;
    }

    // ---------------------------------------------------------------- consumer warps
    // Everything below may read what the previous kernel on the stream wrote (activations, the
    // step sequence, exchange slots): wait for it.  The producer warp above streams weights,
    // which are static, and does not wait.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t seq = step_begin(X);
    const uint32_t bank = seq & 1u;
    // Prologue: weight scales of the rows this CTA touches (loads issued first, stored last, so
    // their latency overlaps the activation loads), then the activation quantisation.
    // q_s[kb][tok][32] holds E4M3 bytes, sa_s[kb][tok(sast)] the block scale 2^e.
    const int sast = p.mp > 8 ? p.mp : 8;  // tokens per K block in sa_s
    const int64_t kcol0 = A.k0 >> p.bk_shift;
    const int64_t srow_lo = (A.row0 + (int64_t)cta * R.Gm * kGroupRows) >> p.bn_shift;
    const int nslotA = R.Gm ? (int)(((A.row0 + (int64_t)(cta + 1) * R.Gm * kGroupRows - 1) >> p.bn_shift) - srow_lo + 1) : 0;
    auto slot_of = [&](int t) {
        return t < R.Gm ? (int)(((A.row0 + (int64_t)trow(t)) >> p.bn_shift) - srow_lo) : nslotA + (t - R.Gm);
    };
    {
        const int ncols = (int)(((A.k0 + p.k - 1) >> p.bk_shift) - kcol0 + 1);
        const int nsw = (nslotA + nx) * ncols;
        auto load_scale = [&](int i) -> float {
            const int sl = i / ncols, c = i - sl * ncols;
            const int64_t srow = sl < nslotA ? srow_lo + sl : (A.row0 + (int64_t)trow(R.Gm + sl - nslotA)) >> p.bn_shift;
            const int64_t idx = srow * A.scale_ld + kcol0 + c;
            if (p.scale_kind == WS_SCALE_UE8M0) {
                const uint32_t b = __ldg(static_cast<const uint8_t *>(A.scales) + idx);
                return (b == 0xFFu) ? __uint_as_float(0x7FC00000u)
                                    : (b == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(b << 23));
            }
            return __ldg(static_cast<const float *>(A.scales) + idx);
        };
        auto sw_index = [&](int i) { return (i / ncols) * p.skb + (i - (i / ncols) * ncols); };
        float pre[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = tid + u * CT;
            pre[u] = i < nsw ? load_scale(i) : 0.0f;
        }
        for (int i = tid; i < kbox * 4 * sast; i += CT)  // tokens the launch does not carry
            if ((i % sast) >= p.m) sa_s[i] = 0.0f;
        const int chunks_per_row = kbox * 16;  // 8-element chunks over the padded K
        const int total = p.mp * chunks_per_row;
        // four chunks per thread and pass: all loads are in flight before the first is used
        for (int c0 = tid; c0 < ((total + 31) & ~31); c0 += 4 * CT) {
            float v[4][8];
            int tok[4], ch[4];
            bool valid[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * CT;
                tok[u] = p.mp == 1 ? 0 : c / chunks_per_row;
                ch[u] = c - tok[u] * chunks_per_row;
                valid[u] = (c < total) && (tok[u] < p.m) && (ch[u] * 8 < p.k);
                load_act8(A.x, p.x_dtype, (int64_t)tok[u] * A.ldx + ch[u] * 8, valid[u], v[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * CT;
                if (c >= ((total + 31) & ~31)) break;  // warp-uniform
                int e;
                uint32_t lo, hi;
                act_quant8(v[u], e, lo, hi);
                if (c < total) {
                    const int kb = ch[u] >> 2;
                    if constexpr (GT > 0) {  // f16 copies of the quantised values (exact)
                        uint4 hv = make_uint4(0u, 0u, 0u, 0u);
                        if (valid[u])
                            hv = make_uint4(e4m3x2_to_f16x2(lo), e4m3x2_to_f16x2(lo >> 16), e4m3x2_to_f16x2(hi),
                                            e4m3x2_to_f16x2(hi >> 16));
                        *reinterpret_cast<uint4 *>(q_s + ((size_t)tok[u] * chunks_per_row + ch[u]) * 16) = hv;
                    } else {
                        *reinterpret_cast<uint2 *>(q_s + ((size_t)(kb * p.mp + tok[u]) * 32 + (ch[u] & 3) * 8)) =
                            valid[u] ? make_uint2(lo, hi) : make_uint2(0u, 0u);
                    }
                    if ((ch[u] & 3) == 0) sa_s[kb * sast + tok[u]] = valid[u] ? pow2_f32(e) : 0.0f;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = tid + u * CT;
            if (i < nsw) sw_s[sw_index(i)] = pre[u];
        }
        for (int i = tid + 4 * CT; i < nsw; i += CT) sw_s[sw_index(i)] = load_scale(i);
    }
    consumer_bar_n<CT>();

    const int g = lane >> 2, tq = lane & 3;
    const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;  // ldmatrix source row of this lane
    const int lm_hi = lane >> 4;                            // 0: k 0..15 of the block, 1: k 16..31
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int item = 0;
    RingPos rp;
    int redbuf = 0;

    const int kofs = (int)(A.k0 - kcol0 * p.bk);  // k0 modulo the scale block
    // shared-space addresses of this lane's operands of K block 0 (advanced per block below)
    // More than eight activation rows ("wide"): warp w takes rows 8w..8w+7 of the activations
    // (MMA columns) for every box of a tile, so each warp owns a 16 x 8 block of the output and
    // nothing is combined across warps; the weights are staged once for all rows.
    const bool wide = p.mp > 8;
    const int tg = wide ? warp : 0;                 // this warp's group of eight activation rows
    const bool tg_active = !wide || tg * 8 < p.mp;
    const uint32_t q_lane = smem_u32(q_s) + (uint32_t)((tg * 8 + g) * 32 + tq * 4);
    const uint32_t q_step = (uint32_t)(p.mp * 32);
    const uint32_t sa_lane = smem_u32(sa_s) + (uint32_t)((tg * 8 + tq * 2) * 4);
    const uint32_t sa_step = (uint32_t)(sast * 4);
    const bool has_b = tg * 8 + g < p.mp;
    auto mma_step = [&](uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, int kb, uint32_t swrow) {
        uint32_t b0r = 0, b1r = 0;
        if (has_b) {
            b0r = lds_u32(q_lane + kb * q_step);
            b1r = lds_u32(q_lane + kb * q_step + 16);
        }
        float d[4];
        mma_e4m3_16x8x32(d, a0, a1, a2, a3, b0r, b1r);
        const float2 sa = lds_f32x2(sa_lane + kb * sa_step);
        const float sw = lds_f32(swrow + (uint32_t)(((kofs + kb * 32) >> p.bk_shift) * 4));
        const float f0 = sa.x * sw, f1 = sa.y * sw;
        acc[0] = fmaf(d[0], f0, acc[0]);
        acc[1] = fmaf(d[1], f1, acc[1]);
        acc[2] = fmaf(d[2], f0, acc[2]);
        acc[3] = fmaf(d[3], f1, acc[3]);
    };
    auto run_item = [&](int b0, int nb, int slot, int pad) {
        const int s = rp.s;
        const bool landed = mbar_wait(full0 + s * 8, rp.ph, X.status);  // false: a wait gave up, the step is void
        const uint32_t sbase = stage0 + s * p.stage_bytes;
        const uint32_t swrow = smem_u32(sw_s) + (uint32_t)(slot * p.skb * 4);
        for (int bi = wide ? 0 : warp; bi < nb && tg_active && landed; bi += wide ? 1 : CW) {
            const int box = b0 + bi;
            const uint32_t bbase = sbase + bi * pad * 128 + lm_row * 128;
            const uint32_t sw7 = (uint32_t)((bi * pad + lm_row) & 7);  // 128B-swizzle phase of this row's address
            if (box * 4 + 4 <= kb32) {  // full box: issue the four fragment loads together
                uint32_t a[4][4];
#pragma unroll
                for (int kq = 0; kq < 4; ++kq)
                    ldmatrix_x4(bbase + ((((uint32_t)(kq << 1) | lm_hi) ^ sw7) << 4), a[kq][0], a[kq][1], a[kq][2], a[kq][3]);
#pragma unroll
                for (int kq = 0; kq < 4; ++kq) mma_step(a[kq][0], a[kq][1], a[kq][2], a[kq][3], box * 4 + kq, swrow);
            } else {
                for (int kq = 0; kq < 4 && box * 4 + kq < kb32; ++kq) {
                    uint32_t a0, a1, a2, a3;
                    ldmatrix_x4(bbase + ((((uint32_t)(kq << 1) | lm_hi) ^ sw7) << 4), a0, a1, a2, a3);
                    mma_step(a0, a1, a2, a3, box * 4 + kq, swrow);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + s * 8);
        ++item;
        rp.next(NS);
    };
    // Sum the consumer warps' accumulators in warp order; thread t < 128 ends with
    // the value of (row = t & 15, tok = t >> 4).
    auto reduce_warps = [&]() -> float {
        float *rb = red_s + (redbuf * CW + warp) * 128;
        rb[(2 * tq) * 16 + g] = acc[0];
        rb[(2 * tq + 1) * 16 + g] = acc[1];
        rb[(2 * tq) * 16 + g + 8] = acc[2];
        rb[(2 * tq + 1) * 16 + g + 8] = acc[3];
        consumer_bar_n<CT>();
        float v = 0.0f;
        if (tid < 128) {
            const float *r0 = red_s + redbuf * CW * 128 + tid;
            v = r0[0];
#pragma unroll
            for (int w = 1; w < CW; ++w) v += r0[w * 128];
        }
        redbuf ^= 1;
        return v;
    };

    // ---- CUDA-core formulation.  Lane = (row 4j + rsub of the tile, 16-byte chunk cch of the box);
    // accv[tok][j] collects this lane's share of row 4j + rsub over every box its warp visits.
    // Weights become f16 pairs, the activations are kept as f16 pairs, their exact products are
    // summed in fp32 by mixed-precision FMAs (measured: 45 weight bytes per clock and SM, against
    // 31 with conversions to f32 and packed fp32 FMAs), and the block scale multiplies each
    // 16-element partial sum.
    constexpr int GTn = GT > 0 ? GT : 1;
    float accv[GTn][4];
    const int rsub = lane >> 3, cch = lane & 7;
    // whole tiles: row 4j + rsub sits at j * 512 + its swizzled chunk; the swizzle phase (row & 7)
    // only depends on the parity of j
    const uint32_t off_e = (uint32_t)(rsub * 128 + ((cch ^ rsub) << 4));
    const uint32_t off_o = (uint32_t)((rsub + 4) * 128 + ((cch ^ rsub ^ 4) << 4));
    auto dot16 = [&](const uint4 w, const uint32_t (&xh)[GTn][8], const float (&f)[GTn], int j) {
        const uint32_t h0 = e4m3x2_half_to_f16x2<0>(w.x), h1 = e4m3x2_half_to_f16x2<1>(w.x);
        const uint32_t h2 = e4m3x2_half_to_f16x2<0>(w.y), h3 = e4m3x2_half_to_f16x2<1>(w.y);
        const uint32_t h4 = e4m3x2_half_to_f16x2<0>(w.z), h5 = e4m3x2_half_to_f16x2<1>(w.z);
        const uint32_t h6 = e4m3x2_half_to_f16x2<0>(w.w), h7 = e4m3x2_half_to_f16x2<1>(w.w);
#pragma unroll
        for (int tk = 0; tk < GTn; ++tk) {
            float s0 = 0.0f, s1 = 0.0f;
            fma2_f16(s0, h0, xh[tk][0]); fma2_f16(s1, h1, xh[tk][1]);
            fma2_f16(s0, h2, xh[tk][2]); fma2_f16(s1, h3, xh[tk][3]);
            fma2_f16(s0, h4, xh[tk][4]); fma2_f16(s1, h5, xh[tk][5]);
            fma2_f16(s0, h6, xh[tk][6]); fma2_f16(s1, h7, xh[tk][7]);
            accv[tk][j] = fmaf(s0 + s1, f[tk], accv[tk][j]);
        }
    };
    auto run_item_gemv = [&](int b0, int nb, int slot, int pad) {
        const int s = rp.s;
        const bool landed = mbar_wait(full0 + s * 8, rp.ph, X.status);  // false: a wait gave up, the step is void
        const uint32_t sbase = stage0 + s * p.stage_bytes;
        const uint32_t swrow = smem_u32(sw_s) + (uint32_t)(slot * p.skb * 4);
        const uint32_t xbase = smem_u32(q_s) + (uint32_t)(cch * 32);
        for (int bi = warp; bi < nb && landed; bi += CW) {
            const int box = b0 + bi;
            const int kb = box * 4 + (cch >> 1);  // the 32-wide K block of this lane's chunk
            const float sw = kb < kb32 ? lds_f32(swrow + (uint32_t)(((kofs + kb * 32) >> p.bk_shift) * 4)) : 0.0f;
            uint32_t xh[GTn][8];
            float f[GTn];
#pragma unroll
            for (int tk = 0; tk < GTn; ++tk) {
                const uint32_t xa = xbase + (uint32_t)((tk * kbox + box) * 256);
                const uint4 x0 = lds_u128(xa), x1 = lds_u128(xa + 16);
                xh[tk][0] = x0.x; xh[tk][1] = x0.y; xh[tk][2] = x0.z; xh[tk][3] = x0.w;
                xh[tk][4] = x1.x; xh[tk][5] = x1.y; xh[tk][6] = x1.z; xh[tk][7] = x1.w;
                f[tk] = kb < kb32 ? lds_f32(smem_u32(sa_s) + (uint32_t)((kb * sast + tk) * 4)) * sw : 0.0f;
            }
            const uint32_t bbase = sbase + bi * pad * 128;
            if (pad == kGroupRows) {  // whole tile: four rows per lane, straight-line
                const uint4 wa = lds_u128(bbase + off_e), wb = lds_u128(bbase + off_o);
                const uint4 wc = lds_u128(bbase + 1024 + off_e), wd = lds_u128(bbase + 1024 + off_o);
                dot16(wa, xh, f, 0);
                dot16(wb, xh, f, 1);
                dot16(wc, xh, f, 2);
                dot16(wd, xh, f, 3);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (4 * j < pad) {  // warp-uniform: rows the stage holds
                        const int r = 4 * j + rsub;
                        dot16(lds_u128(bbase + r * 128 + ((uint32_t)(cch ^ ((bi * pad + r) & 7)) << 4)), xh, f, j);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + s * 8);
        ++item;
        rp.next(NS);
    };
    // Combine the eight lanes of each row, then the warps in warp order (same result layout as
    // reduce_warps: thread t < 128 ends with row t & 15 of token t >> 4).
    auto reduce_gemv = [&]() -> float {
        float *rb = red_s + (redbuf * CW + warp) * 128;
#pragma unroll
        for (int tk = 0; tk < GTn; ++tk)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float v = accv[tk][j];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if (cch == 0) rb[tk * 16 + 4 * j + rsub] = v;
            }
        consumer_bar_n<CT>();
        float v = 0.0f;
        if (tid < 16 * GTn) {
            const float *r0 = red_s + redbuf * CW * 128 + tid;
            v = r0[0];
#pragma unroll
            for (int w = 1; w < CW; ++w) v += r0[w * 128];
        }
        redbuf ^= 1;
        return v;
    };

    const int row_t = tid & 15, tok_t = tid >> 4;  // meaningful for tid < 128
    const bool solo = (p.mode == kModeAllReduce && p.world == 1);
    const int PR = p.part_rows;

    for (int t = 0; t < ntile; ++t) {
        const int slot = slot_of(t);
        const int pad = tpad(tcnt(t)), cols = p.stage_bytes / (pad * 128);
        float v;
        if constexpr (GT > 0) {
#pragma unroll
            for (int tk = 0; tk < GTn; ++tk) accv[tk][0] = accv[tk][1] = accv[tk][2] = accv[tk][3] = 0.0f;
            for (int b0 = 0; b0 < kbox; b0 += cols) run_item_gemv(b0, min(cols, kbox - b0), slot, pad);
            v = reduce_gemv();
        } else {
            acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
            for (int b0 = 0; b0 < kbox; b0 += cols) run_item(b0, min(cols, kbox - b0), slot, pad);
            if (wide) {  // the accumulator fragment is final: rows g, g + 8 x tokens 8 tg + 2 tq, + 1
                const int tk0 = tg * 8 + 2 * tq;
                if (tk0 < p.m) {
                    part_s[tk0 * PR + t * kGroupRows + g] = acc[0];
                    part_s[tk0 * PR + t * kGroupRows + g + 8] = acc[2];
                }
                if (tk0 + 1 < p.m) {
                    part_s[(tk0 + 1) * PR + t * kGroupRows + g] = acc[1];
                    part_s[(tk0 + 1) * PR + t * kGroupRows + g + 8] = acc[3];
                }
                continue;
            }
            v = reduce_warps();
        }
        if (tid < 128 && tok_t < p.m) part_s[tok_t * PR + t * kGroupRows + row_t] = v;
    }
    consumer_bar_n<CT>();  // part_s complete

    // Visit every (token, valid row) of this CTA: fn(tok, global row, value index in part_s).
    auto for_rows = [&](auto fn) {
        for (int i = tid; i < ntile * p.m * kGroupRows; i += CT) {
            const int t = i / (p.m * kGroupRows), j = i - t * (p.m * kGroupRows);
            const int tok = j >> 4, r = j & 15;
            if (r < tcnt(t)) fn(tok, trow(t) + r, tok * PR + t * kGroupRows + r);
        }
    };

    if (solo) {
        for_rows([&](int tok, int row, int pi) { A.out[(size_t)tok * p.n + row] = part_s[pi]; });
        return;
    }
    const uint32_t *myflags = reinterpret_cast<const uint32_t *>(X.sym[X.rank] + p.lay.flags_off) +
                              (size_t)bank * p.world * nflag;

    if (p.mode == kModeAllReduce) {
        // every thread sends its rows' partials to all ranks as tagged words, then folds the same
        // rows in rank order as the ranks' words arrive: no barrier, fence or flag in between
        const size_t astride = (size_t)p.lay.max_m * p.lay.max_n;
        for (int pr = 0; pr < p.world; ++pr) {
            uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[pr] + p.lay.slota_off) + ((size_t)bank * p.world + X.rank) * astride;
            for_rows([&](int tok, int row, int pi) { st_word_sys(dst + (size_t)tok * p.n + row, seq, part_s[pi]); });
        }
        const uint64_t *slots = reinterpret_cast<const uint64_t *>(X.sym[X.rank] + p.lay.slota_off) +
                                (size_t)bank * p.world * astride;
        for_rows([&](int tok, int row, int) {
            const size_t off = (size_t)tok * p.n + row;
            A.out[off] = fold_words(slots, astride, off, p.world, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
        });
        return;
    }

    // ---- lm_head: gather rows, publish candidates, final argmax
    if (p.gather_logits) {
        for (int pr = 0; pr < p.world; ++pr) {
            float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.gather_off) +
                         (size_t)bank * p.lay.max_m * (size_t)p.lay.max_vocab;
            for_rows([&](int tok, int row, int pi) { dst[(size_t)tok * p.lay.max_vocab + A.vocab_row0 + row] = part_s[pi]; });
        }
    }
    for (int tok = warp; tok < p.m; tok += CW) {  // a warp per token
        float bv = -INFINITY;
        uint32_t bi = 0xFFFFFFFFu;
        for (int i = lane; i < ntile * kGroupRows; i += 32) {
            const int t = i >> 4, r = i & 15;
            if (r >= tcnt(t)) continue;
            const float v = part_s[tok * PR + i];
            const uint32_t idx = (uint32_t)(A.vocab_row0 + trow(t) + r);
            if (v > -INFINITY && cand_better(v, idx, bv, bi)) { bv = v; bi = idx; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (cand_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane < p.world) {
            uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[lane] + p.lay.pairs_off) +
                            (((size_t)bank * p.world + X.rank) * kMaxCtas + cta) * p.lay.max_m + tok;
            *dst = ((uint64_t)__float_as_uint(bv) << 32) | bi;
        }
    }
    consumer_bar_n<CT>();  // the st.release.sys below is cumulative over the stores this barrier ordered
    if (tid < p.world) {
        uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[tid] + p.lay.flags_off) +
                      ((size_t)bank * p.world + X.rank) * nflag;
        st_release_sys(f + cta, seq);
    }
    const bool copies = p.gather_logits && A.logits != nullptr;
    if (!copies && cta != 0) return;
    // every CTA of every rank has published (its flag follows all of its stores)
    for (int i = tid; i < p.world * ncta; i += CT)
        wait_flag(myflags + (size_t)(i / ncta) * nflag + (i % ncta), seq, p.timeout_ns, X.status, kStatTimeoutGather);
    consumer_bar_n<CT>();
    if (copies) {
        const float *gl = reinterpret_cast<const float *>(X.sym[X.rank] + p.lay.gather_off) +
                          (size_t)bank * p.lay.max_m * (size_t)p.lay.max_vocab;
        const int64_t per = ((int64_t)p.vocab + ncta - 1) / ncta;
        const int64_t v0 = (int64_t)cta * per, v1 = min((int64_t)p.vocab, v0 + per);
        for (int tok = 0; tok < p.m; ++tok)
            for (int64_t v = v0 + tid; v < v1; v += CT)
                A.logits[(size_t)tok * p.vocab + v] = __ldcg(gl + (size_t)tok * p.lay.max_vocab + v);
    }
    if (cta == 0 && A.argmax != nullptr) {
        const uint64_t *pairs = reinterpret_cast<const uint64_t *>(X.sym[X.rank] + p.lay.pairs_off) +
                                (size_t)bank * p.world * kMaxCtas * p.lay.max_m;
        for (int tok = warp; tok < p.m; tok += CW) {
            float bv = -INFINITY;
            uint32_t bi = 0xFFFFFFFFu;
            for (int i = lane; i < p.world * ncta; i += 32) {
                const uint64_t pr = ld_volatile_u64(pairs + ((size_t)(i / ncta) * kMaxCtas + (i % ncta)) * p.lay.max_m + tok);
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
            if (lane == 0) A.argmax[tok] = (bi == 0xFFFFFFFFu) ? 0u : bi;
        }
    }
}

template <int GT>
__global__ void __launch_bounds__(fp8_threads(GT), 1) fp8_rowpar_kernel(const __grid_constant__ Fp8Params p) {
    const RankCtx &X = p.r[blockIdx.y].ctx;
    fp8_rowpar_kernel_body<GT>(p);
    if (p.world > 1 || p.mode == kModeLmHead) {  // a lone all-reduce rank exchanges nothing
        // step_begin again: the value is unchanged until the last CTA publishes the next one below
        step_end(X, step_begin(X), gridDim.x);
    }
    host_done_signal(X, gridDim.x);
}

}  // namespace ws
