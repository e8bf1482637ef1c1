// FP8 E4M3 row-parallel decode GEMM fused with its exchange (sm_100a).
//
// One persistent CTA per SM.  Output rows are cut into groups of 16 (one MMA M
// tile).  Each CTA OWNS floor(G/ncta) whole groups and streams their weights
// over the full local K; the G mod ncta leftover groups are cut along K into
// 128-byte boxes shared out over all CTAs, so that every SM streams the same
// number of bytes.  Weight tiles arrive by TMA (128B-swizzled 16x128 boxes, a
// 32 KB stage ring filled by one producer warp); eight consumer warps feed them
// straight to the FP8 tensor-core MMA against activations that the prologue
// quantised exactly as the reference does, and apply activation- and
// weight-block scales per 32-wide K block in fp32.
//
// Exchange (world > 1): a CTA stores its owned rows' fp32 partials into slot
// [my rank] of every peer's exchange memory and then releases one flag per peer;
// it waits for the same CTA of every rank and adds the slots in rank order, so
// all ranks produce identical bits.  K-split groups are first combined locally
// in fixed order by the last CTA to arrive, then exchanged the same way.
//
// lm_head mode: rows are vocabulary entries; instead of a sum every rank's rows
// are gathered (stored into every peer's logits buffer) and each CTA publishes
// its best (value, lowest index) candidate per token; CTA 0 merges them.
#pragma once

#include <math.h>

#include "ws_device.cuh"

namespace ws {

enum { kModeAllReduce = 0, kModeLmHead = 1 };

struct alignas(64) Fp8RankArgs {
    CUtensorMap tmap;  // weight shard [n rows][k bytes], box 128 x 16, swizzle 128B
    const void *x;
    const void *scales;
    float *out;        // all-reduce mode: [m, n]
    float *logits;     // lm_head mode: [m, vocab] or null
    uint32_t *argmax;  // lm_head mode: [m] or null
    int64_t ldx, scale_ld, row0, k0, vocab_row0;
    RankCtx ctx;
};

struct Fp8Params {
    int32_t m, n, k, x_dtype, scale_kind, bn, bk;
    int32_t world, mode, vocab, mp, nstages, nslot_max, skb;
    int32_t gather_logits, split;
    int32_t bk_shift, bn_shift;  // log2 of the scale block edges
    uint32_t seq, pad1;
    uint64_t timeout_ns;
    SymLayout lay;
    Fp8RankArgs r[WS_MAX_WORLD];
};

struct Fp8Smem {  // byte offsets from the 1024-aligned base
    int32_t stages, q, sa, sw, red, part, bars, misc, total;
};

__host__ __device__ inline Fp8Smem fp8_smem_layout(int nstages, int kbox, int mp, int nslot_max, int skb,
                                                   int m, int owned_rows) {
    Fp8Smem s{};
    int o = 0;
    s.stages = o; o += nstages * kStageBytes;
    s.q = o;      o += kbox * 4 * mp * 32;
    s.sa = o;     o += kbox * 4 * 8 * 4;
    s.sw = o;     o += ((nslot_max * skb * 4 + 15) / 16) * 16;
    s.red = o;    o += 2 * kConsumerWarps * 128 * 4;
    s.part = o;   o += ((m * owned_rows * 4 + 15) / 16) * 16;
    s.bars = o;   o += 2 * kMaxStages * 8;
    s.misc = o;   o += 128;
    s.total = o;
    return s;
}

// Split schedule of the leftover groups: unit u = j * kbox + box; CTA c takes
// units [c*U/ncta, (c+1)*U/ncta); unit u therefore belongs to CTA owner_of(u).
__host__ __device__ __forceinline__ int64_t unit_begin(int c, int64_t U, int ncta) {
    return (int64_t)c * U / ncta;
}
__host__ __device__ __forceinline__ int owner_of(int64_t u, int64_t U, int ncta) {
    return (int)(((u + 1) * ncta + U - 1) / U) - 1;
}

__device__ __forceinline__ bool cand_better(float v, uint32_t i, float bv, uint32_t bi) {
    return v > bv || (v == bv && i < bi);
}

__global__ void __launch_bounds__(kThreads, 1) fp8_rowpar_kernel(const __grid_constant__ Fp8Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);

    const int vr = blockIdx.y, cta = blockIdx.x, ncta = gridDim.x;
    const Fp8RankArgs &A = p.r[vr];
    const RankCtx &X = A.ctx;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int kbox = (p.k + 127) >> 7;
    const int kb32 = p.k >> 5;  // real 32-wide K blocks
    const int G = (p.n + kGroupRows - 1) / kGroupRows;
    const int Gm = G / ncta;
    const int Rg = G - Gm * ncta;
    const int g0 = cta * Gm;
    const int extra = (!p.split && cta < Rg) ? 1 : 0;  // unsplit leftover: one more owned group
    const int n_own = Gm + extra;
    const int owned_rows = (Gm + ((!p.split && Rg) ? 1 : 0)) * kGroupRows;  // part_s row stride
    auto group_of = [&](int gi) { return gi < Gm ? g0 + gi : Gm * ncta + cta; };
    const int64_t U = p.split ? (int64_t)Rg * kbox : 0;
    const int64_t u0 = unit_begin(cta, U, ncta), u1 = unit_begin(cta + 1, U, ncta);
    const int jfirst = (u1 > u0) ? (int)(u0 / kbox) : 0;
    const int nruns = (u1 > u0) ? (int)((u1 - 1) / kbox) - jfirst + 1 : 0;

    const Fp8Smem S = fp8_smem_layout(p.nstages, kbox, p.mp, p.nslot_max, p.skb, p.m, owned_rows);
    uint8_t *q_s = smem + S.q;
    float *sa_s = reinterpret_cast<float *>(smem + S.sa);
    float *sw_s = reinterpret_cast<float *>(smem + S.sw);
    float *red_s = reinterpret_cast<float *>(smem + S.red);
    float *part_s = reinterpret_cast<float *>(smem + S.part);
    uint32_t *misc_s = reinterpret_cast<uint32_t *>(smem + S.misc);  // [0]=last flag, [8..15]/[16..23] candidates
    float *cand_v = reinterpret_cast<float *>(misc_s + 8);
    uint32_t *cand_i = misc_s + 16;
    const uint32_t stage0 = smem_u32(smem + S.stages);
    const uint32_t full0 = smem_u32(smem + S.bars), empty0 = full0 + kMaxStages * 8;
    const int NS = p.nstages;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(empty0 + s * 8, kConsumerWarps);
        }
        mbar_fence_init();
        prefetch_tmap(&A.tmap);
    }
    if (tid < 8) {
        cand_v[tid] = -INFINITY;
        cand_i[tid] = 0xFFFFFFFFu;
    }
    __syncthreads();

    const uint32_t bank = p.seq & 1u;
    const int nflag = kMaxCtas + kMaxShared;

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ TMA producer warp
        int item = 0;
        auto issue = [&](int rowbase, int b0, int nb) {
            const int s = item % NS;
            const uint32_t ph = (uint32_t)(item / NS) & 1u;
            mbar_wait(empty0 + s * 8, ph ^ 1u, X.status);
            if (lane == 0) mbar_arrive_expect_tx(full0 + s * 8, (uint32_t)nb * kBoxBytes);
            __syncwarp();
            if (lane < nb)
                tma_load_2d(stage0 + s * kStageBytes + lane * kBoxBytes, &A.tmap, (b0 + lane) * 128, rowbase,
                            full0 + s * 8);
            ++item;
        };
        for (int gi = 0; gi < n_own; ++gi)
            for (int b0 = 0; b0 < kbox; b0 += kBoxesPerStage)
                issue(group_of(gi) * kGroupRows, b0, min(kBoxesPerStage, kbox - b0));
        for (int r = 0; r < nruns; ++r) {
            const int j = jfirst + r;
            const int ba = (int)(max(u0, (int64_t)j * kbox) - (int64_t)j * kbox);
            const int bb = (int)(min(u1, (int64_t)(j + 1) * kbox) - (int64_t)j * kbox);
            for (int b0 = ba; b0 < bb; b0 += kBoxesPerStage)
                issue((Gm * ncta + j) * kGroupRows, b0, min(kBoxesPerStage, bb - b0));
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps
    // Prologue 1: quantise this rank's activations into shared memory.
    // q_s[kb][tok][32] holds E4M3 bytes, sa_s[kb][tok(8)] the block scale 2^e.
    {
        for (int i = tid; i < kbox * 4 * 8; i += kConsumerThreads) sa_s[i] = 0.0f;
        consumer_bar();
        const int chunks_per_row = kbox * 16;  // 8-element chunks over the padded K
        const int total = p.mp * chunks_per_row;
        for (int c = tid; c < ((total + 31) & ~31); c += kConsumerThreads) {
            const int tok = c / chunks_per_row, ch = c - tok * chunks_per_row;
            const int kk = ch * 8;
            const bool valid = (c < total) && (tok < p.m) && (kk < p.k);
            float v[8];
            load_act8(A.x, p.x_dtype, (int64_t)tok * A.ldx + kk, valid, v);
            int e;
            uint32_t lo, hi;
            act_quant8(v, e, lo, hi);
            if (c < total) {
                const int kb = ch >> 2;
                *reinterpret_cast<uint2 *>(q_s + ((size_t)(kb * p.mp + tok) * 32 + (ch & 3) * 8)) =
                    valid ? make_uint2(lo, hi) : make_uint2(0u, 0u);
                if ((ch & 3) == 0 && valid) sa_s[kb * 8 + tok] = pow2_f32(e);
            }
        }
    }
    // Prologue 2: weight scales of the rows this CTA touches, as fp32.
    const int64_t kcol0 = A.k0 >> p.bk_shift;
    const int64_t srow_lo = (A.row0 + (int64_t)g0 * kGroupRows) >> p.bn_shift;
    const int nslotA = Gm ? (int)(((A.row0 + (int64_t)(g0 + Gm) * kGroupRows - 1) >> p.bn_shift) - srow_lo + 1) : 0;
    {
        const int ncols = (int)(((A.k0 + p.k - 1) >> p.bk_shift) - kcol0 + 1);
        const int nslots = nslotA + extra + nruns;
        for (int i = tid; i < nslots * ncols; i += kConsumerThreads) {
            const int sl = i / ncols, c = i - sl * ncols;
            const int lg = (extra && sl == nslotA) ? Gm * ncta + cta : Gm * ncta + jfirst + (sl - nslotA - extra);
            const int64_t srow = sl < nslotA ? srow_lo + sl : (A.row0 + (int64_t)lg * kGroupRows) >> p.bn_shift;
            const int64_t idx = srow * A.scale_ld + kcol0 + c;
            float s;
            if (p.scale_kind == WS_SCALE_UE8M0) {
                const uint32_t b = static_cast<const uint8_t *>(A.scales)[idx];
                s = (b == 0xFFu) ? __uint_as_float(0x7FC00000u)
                                 : (b == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(b << 23));
            } else {
                s = static_cast<const float *>(A.scales)[idx];
            }
            sw_s[sl * p.skb + c] = s;
        }
    }
    consumer_bar();

    const int g = lane >> 2, tq = lane & 3;
    const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;  // ldmatrix source row of this lane
    const int lm_hi = lane >> 4;                            // 0: k 0..15 of the block, 1: k 16..31
    float acc[4];
    int item = 0;
    int redbuf = 0;

    const int kofs = (int)(A.k0 - kcol0 * p.bk);  // k0 modulo the scale block
    auto mma_step = [&](uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, int kb, const float *swrow) {
        uint32_t b0r = 0, b1r = 0;
        if (g < p.mp) {
            const uint8_t *qp = q_s + ((size_t)(kb * p.mp + g) * 32 + tq * 4);
            b0r = *reinterpret_cast<const uint32_t *>(qp);
            b1r = *reinterpret_cast<const uint32_t *>(qp + 16);
        }
        float d[4];
        mma_e4m3_16x8x32(d, a0, a1, a2, a3, b0r, b1r);
        const float2 sa = *reinterpret_cast<const float2 *>(sa_s + kb * 8 + tq * 2);
        const float sw = swrow[(kofs + kb * 32) >> p.bk_shift];
        const float f0 = sa.x * sw, f1 = sa.y * sw;
        acc[0] = fmaf(d[0], f0, acc[0]);
        acc[1] = fmaf(d[1], f1, acc[1]);
        acc[2] = fmaf(d[2], f0, acc[2]);
        acc[3] = fmaf(d[3], f1, acc[3]);
    };
    auto run_item = [&](int b0, int nb, int slot) {
        const int s = item % NS;
        mbar_wait(full0 + s * 8, (uint32_t)(item / NS) & 1u, X.status);
        const uint32_t sbase = stage0 + s * kStageBytes;
        const float *swrow = sw_s + slot * p.skb;
        const uint32_t sw7 = (uint32_t)(lm_row & 7);
        for (int bi = warp; bi < nb; bi += kConsumerWarps) {
            const int box = b0 + bi;
            const uint32_t bbase = sbase + bi * kBoxBytes + lm_row * 128;
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
    };
    // Sum the eight warps' accumulators in warp order; thread t < 128 ends with
    // the value of (row = t & 15, tok = t >> 4).
    auto reduce_warps = [&]() -> float {
        float *rb = red_s + (redbuf * kConsumerWarps + warp) * 128;
        rb[(2 * tq) * 16 + g] = acc[0];
        rb[(2 * tq + 1) * 16 + g] = acc[1];
        rb[(2 * tq) * 16 + g + 8] = acc[2];
        rb[(2 * tq + 1) * 16 + g + 8] = acc[3];
        consumer_bar();
        float v = 0.0f;
        if (tid < 128) {
            const float *r0 = red_s + redbuf * kConsumerWarps * 128 + tid;
            v = r0[0];
#pragma unroll
            for (int w = 1; w < kConsumerWarps; ++w) v += r0[w * 128];
        }
        redbuf ^= 1;
        return v;
    };

    const int row_t = tid & 15, tok_t = tid >> 4;  // meaningful for tid < 128
    const int nrow_own = n_own * kGroupRows;
    const bool solo = (p.mode == kModeAllReduce && p.world == 1);

    // ---- owned groups
    for (int gi = 0; gi < n_own; ++gi) {
        acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
        const int slot = gi < Gm ? (int)(((A.row0 + (int64_t)(g0 + gi) * kGroupRows) >> p.bn_shift) - srow_lo) : nslotA;
        for (int b0 = 0; b0 < kbox; b0 += kBoxesPerStage) run_item(b0, min(kBoxesPerStage, kbox - b0), slot);
        const float v = reduce_warps();
        if (tid < 128 && tok_t < p.m) part_s[tok_t * owned_rows + gi * kGroupRows + row_t] = v;
    }

    // ---- K-split leftover groups: contribution -> local scratch -> last arriver folds
    int fin[kMaxRuns];  // leftover groups this CTA finalised (it exchanges them below)
    int nfin = 0;
    for (int r = 0; r < nruns; ++r) {
        const int j = jfirst + r;
        const int ba = (int)(max(u0, (int64_t)j * kbox) - (int64_t)j * kbox);
        const int bb = (int)(min(u1, (int64_t)(j + 1) * kbox) - (int64_t)j * kbox);
        acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
        for (int b0 = ba; b0 < bb; b0 += kBoxesPerStage) run_item(b0, min(kBoxesPerStage, bb - b0), nslotA + extra + r);
        const float v = reduce_warps();
        if (tid < 128) {
            X.contrib[((size_t)cta * kMaxRuns + r) * (8 * kGroupRows) + tid] = v;
            __threadfence();
        }
        consumer_bar();
        const int c_lo = owner_of((int64_t)j * kbox, U, ncta);
        const int c_hi = owner_of((int64_t)(j + 1) * kbox - 1, U, ncta);
        const uint32_t expect = (U >= ncta) ? (uint32_t)(c_hi - c_lo + 1) : (uint32_t)kbox;
        if (tid == 0) {
            const uint32_t prev = atomicAdd(X.counters + j, 1u);
            misc_s[0] = (prev + 1u == expect) ? 1u : 0u;
            if (prev + 1u == expect) X.counters[j] = 0u;  // ready for the next step
        }
        consumer_bar();
        const bool last = misc_s[0] != 0u;
        consumer_bar();  // misc_s[0] may be rewritten by the next run
        if (!last) continue;
        __threadfence();
        float sum = 0.0f;
        if (tid < 128) {
            // contributions in CTA (= K) order; loads are issued eight at a time, adds stay ordered
            for (int c = c_lo; c <= c_hi; c += 8) {
                float v[8];
                bool has[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int cc = c + i;
                    const int64_t cb = unit_begin(cc, U, ncta);
                    has[i] = cc <= c_hi && unit_begin(cc + 1, U, ncta) > cb;
                    const int jf = (int)(cb / kbox);
                    v[i] = has[i] ? __ldcg(X.contrib + ((size_t)cc * kMaxRuns + (j - jf)) * (8 * kGroupRows) + tid) : 0.0f;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (has[i]) sum += v[i];
            }
        }
        // `sum` is this rank's partial of leftover group j at (row_t, tok_t)
        const int row = (Gm * ncta + j) * kGroupRows + row_t;
        const bool ok = tid < 128 && tok_t < p.m && row < p.n;
        if (p.mode == kModeAllReduce) {
            if (ok) {
                if (p.world == 1) {
                    A.out[(size_t)tok_t * p.n + row] = sum;
                } else {
                    for (int pr = 0; pr < p.world; ++pr) {
                        float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.slotb_off) +
                                     (((size_t)bank * p.world + X.rank) * kMaxShared + j) *
                                         ((size_t)p.lay.max_m * kGroupRows);
                        dst[tok_t * kGroupRows + row_t] = sum;
                    }
                }
            }
        } else {
            if (ok && p.gather_logits) {
                for (int pr = 0; pr < p.world; ++pr) {
                    float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.gather_off) +
                                 ((size_t)bank * p.lay.max_m + tok_t) * (size_t)p.lay.max_vocab;
                    dst[A.vocab_row0 + row] = sum;
                }
            }
            // best of the 16 rows of each token (16 adjacent lanes), merged into cand_*
            float bv = (ok && sum > -INFINITY) ? sum : -INFINITY;
            uint32_t bi = (ok && sum > -INFINITY) ? (uint32_t)(A.vocab_row0 + row) : 0xFFFFFFFFu;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (cand_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            if (tid < 128 && row_t == 0 && tok_t < p.m && cand_better(bv, bi, cand_v[tok_t], cand_i[tok_t])) {
                cand_v[tok_t] = bv;
                cand_i[tok_t] = bi;
            }
        }
        fin[nfin++] = j;
    }

    // ---- publish owned rows
    if (solo) {
        for (int i = tid; i < p.m * nrow_own; i += kConsumerThreads) {
            const int tok = i / nrow_own, r = i - tok * nrow_own;
            A.out[(size_t)tok * p.n + group_of(r >> 4) * kGroupRows + (r & 15)] = part_s[tok * owned_rows + r];
        }
        return;
    }
    consumer_bar();  // part_s and cand_* complete

    if (p.mode == kModeAllReduce) {
        for (int pr = 0; pr < p.world; ++pr) {
            float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.slota_off) +
                         ((size_t)bank * p.world + X.rank) * ((size_t)p.lay.max_m * p.lay.max_n);
            for (int i = tid; i < p.m * nrow_own; i += kConsumerThreads) {
                const int tok = i / nrow_own, r = i - tok * nrow_own;
                dst[(size_t)tok * p.n + group_of(r >> 4) * kGroupRows + (r & 15)] = part_s[tok * owned_rows + r];
            }
        }
        __threadfence_system();
        consumer_bar();
        if (tid < p.world) {
            uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[tid] + p.lay.flags_off) +
                          ((size_t)bank * p.world + X.rank) * nflag;
            st_release_sys(f + cta, p.seq);
        }
        if (warp == 1) {
            for (int i = lane; i < nfin * p.world; i += 32) {
                uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[i % p.world] + p.lay.flags_off) +
                              ((size_t)bank * p.world + X.rank) * nflag;
                st_release_sys(f + kMaxCtas + fin[i / p.world], p.seq);
            }
        }
        // wait for every rank, then fold in rank order
        const uint32_t *myflags = reinterpret_cast<const uint32_t *>(X.sym[X.rank] + p.lay.flags_off) +
                                  (size_t)bank * p.world * nflag;
        if (tid < p.world)
            wait_flag(myflags + (size_t)tid * nflag + cta, p.seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
        if (warp == 1)
            for (int i = lane; i < nfin * p.world; i += 32)
                wait_flag(myflags + (size_t)(i % p.world) * nflag + kMaxCtas + fin[i / p.world], p.seq,
                          p.timeout_ns, X.status, kStatTimeoutPeerB);
        consumer_bar();
        const size_t astride = (size_t)p.lay.max_m * p.lay.max_n;
        const float *slots = reinterpret_cast<const float *>(X.sym[X.rank] + p.lay.slota_off) +
                             (size_t)bank * p.world * astride;
        for (int i = tid; i < p.m * nrow_own; i += kConsumerThreads) {
            const int tok = i / nrow_own, r = i - tok * nrow_own;
            const size_t off = (size_t)tok * p.n + group_of(r >> 4) * kGroupRows + (r & 15);
            float s = __ldcg(slots + off);
            for (int rr = 1; rr < p.world; ++rr) s += __ldcg(slots + rr * astride + off);
            A.out[off] = s;
        }
        const size_t bstride = (size_t)kMaxShared * p.lay.max_m * kGroupRows;
        const float *slotb = reinterpret_cast<const float *>(X.sym[X.rank] + p.lay.slotb_off) +
                             (size_t)bank * p.world * bstride;
        for (int f = 0; f < nfin; ++f) {
            const int j = fin[f];
            const int row = (Gm * ncta + j) * kGroupRows + row_t;
            if (tid < 128 && tok_t < p.m && row < p.n) {
                const size_t off = (size_t)j * p.lay.max_m * kGroupRows + tok_t * kGroupRows + row_t;
                float s = __ldcg(slotb + off);
                for (int rr = 1; rr < p.world; ++rr) s += __ldcg(slotb + rr * bstride + off);
                A.out[(size_t)tok_t * p.n + row] = s;
            }
        }
        return;
    }

    // ---- lm_head: gather rows, publish candidates, final argmax
    if (p.gather_logits) {
        for (int pr = 0; pr < p.world; ++pr) {
            float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.gather_off) +
                         (size_t)bank * p.lay.max_m * (size_t)p.lay.max_vocab;
            for (int i = tid; i < p.m * nrow_own; i += kConsumerThreads) {
                const int tok = i / nrow_own, r = i - tok * nrow_own;
                dst[(size_t)tok * p.lay.max_vocab + A.vocab_row0 + group_of(r >> 4) * kGroupRows + (r & 15)] =
                    part_s[tok * owned_rows + r];
            }
        }
    }
    for (int tok = warp; tok < p.m; tok += kConsumerWarps) {  // a warp per token
        float bv = -INFINITY;
        uint32_t bi = 0xFFFFFFFFu;
        for (int r = lane; r < nrow_own; r += 32) {
            const float v = part_s[tok * owned_rows + r];
            const int row = group_of(r >> 4) * kGroupRows + (r & 15);
            const uint32_t idx = (uint32_t)(A.vocab_row0 + row);
            if (row < p.n && v > -INFINITY && cand_better(v, idx, bv, bi)) { bv = v; bi = idx; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (cand_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (cand_better(cand_v[tok], cand_i[tok], bv, bi)) { bv = cand_v[tok]; bi = cand_i[tok]; }
        if (lane < p.world) {
            uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[lane] + p.lay.pairs_off) +
                            (((size_t)bank * p.world + X.rank) * kMaxCtas + cta) * p.lay.max_m + tok;
            *dst = ((uint64_t)__float_as_uint(bv) << 32) | bi;
        }
    }
    __threadfence_system();
    consumer_bar();
    if (tid < p.world) {
        uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[tid] + p.lay.flags_off) +
                      ((size_t)bank * p.world + X.rank) * nflag;
        st_release_sys(f + cta, p.seq);
    }
    const bool copies = p.gather_logits && A.logits != nullptr;
    if (!copies && cta != 0) return;
    // every CTA of every rank has published (its flag follows all of its stores)
    const uint32_t *myflags = reinterpret_cast<const uint32_t *>(X.sym[X.rank] + p.lay.flags_off) +
                              (size_t)bank * p.world * nflag;
    for (int i = tid; i < p.world * ncta; i += kConsumerThreads)
        wait_flag(myflags + (size_t)(i / ncta) * nflag + (i % ncta), p.seq, p.timeout_ns, X.status,
                  kStatTimeoutGather);
    consumer_bar();
    if (copies) {
        const float *gl = reinterpret_cast<const float *>(X.sym[X.rank] + p.lay.gather_off) +
                          (size_t)bank * p.lay.max_m * (size_t)p.lay.max_vocab;
        const int64_t per = ((int64_t)p.vocab + ncta - 1) / ncta;
        const int64_t v0 = (int64_t)cta * per, v1 = min((int64_t)p.vocab, v0 + per);
        for (int tok = 0; tok < p.m; ++tok)
            for (int64_t v = v0 + tid; v < v1; v += kConsumerThreads)
                A.logits[(size_t)tok * p.vocab + v] = __ldcg(gl + (size_t)tok * p.lay.max_vocab + v);
    }
    if (cta == 0 && A.argmax != nullptr) {
        const uint64_t *pairs = reinterpret_cast<const uint64_t *>(X.sym[X.rank] + p.lay.pairs_off) +
                                (size_t)bank * p.world * kMaxCtas * p.lay.max_m;
        for (int tok = warp; tok < p.m; tok += kConsumerWarps) {
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

}  // namespace ws
