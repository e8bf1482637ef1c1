// MXFP4 routed-expert down projection + top-k combine fused with its exchange
// (sm_100a).  Same persistent structure as the FP8 kernel: 16-row groups owned by
// CTAs, leftover groups cut along (pass, K box), weights streamed by TMA, partial
// sums stored into every peer and added in rank order.
//
// A "pass" is one local expert that at least one token selected, with up to eight
// of its routes as the eight MMA columns (an expert with more routes takes several
// passes).  Passes run in ascending expert id, so a token's experts are added in
// the reference's order (crates/weightstream-ref/src/moe.rs:75-84).  Before each
// pass the consumers quantise hidden * routing-weight for its routes exactly as
// the reference does (moe.rs:150 then actquant.rs:21-57).
//
// E2M1 -> E4M3 without a table: both formats keep subnormals the same way, so the
// three magnitude bits of an E2M1 code, shifted left by two, ARE the E4M3 code of
// value * 2^-6.  The 2^6 is folded into the activation block scale.
#pragma once

#include <math.h>

#include "ws_device.cuh"
#include "ws_fp8_kernel.cuh"  // unit_begin / owner_of

namespace ws {

constexpr int kMoeMaxRoutes = 512;
constexpr int kMoeMaxExperts = 512;
constexpr int kMoeMaxTopK = 8;

struct alignas(64) MoeRankArgs {
    CUtensorMap tmap;  // slab as [e_len*n rows][k/2 bytes], box 128 x 16, swizzle 128B
    const void *h;
    const int32_t *route_ids;
    const float *route_w;
    const uint8_t *s2;
    float *out;
    int64_t ldh;
    int32_t e_start, e_len;
    RankCtx ctx;
};

struct MoeParams {
    int32_t m, n, k, top_k, h_dtype, world, nstages, stage_boxes, split, pad0;
    uint32_t pad0_, pad1;
    uint64_t timeout_ns;
    SymLayout lay;
    MoeRankArgs r[WS_MAX_WORLD];
};

struct MoeSmem {
    int32_t stages, q, sa, red, part, yroute, ids, wts, cnt, pstart, pass_e, pass_n, pass_r, bars, misc, total;
    int32_t stage_bytes, scale_off;
};

__host__ __device__ inline MoeSmem moe_smem_layout(int nstages, int stage_boxes, int k, int m, int top_k,
                                                   int e_len, int owned_rows) {
    MoeSmem s{};
    const int kb32 = k / 32;
    s.scale_off = stage_boxes * kBoxBytes;  // weight-scale bytes of the item follow its boxes
    s.stage_bytes = (int)align_up(s.scale_off + kGroupRows * kb32, 1024);
    int o = 0;
    s.stages = o; o += nstages * s.stage_bytes;
    s.q = o;      o += kb32 * 8 * 32;
    s.sa = o;     o += kb32 * 8 * 4;
    s.red = o;    o += 2 * kConsumerWarps * 128 * 4;
    s.part = o;   o += (int)align_up((int64_t)m * owned_rows * 4, 16);
    s.yroute = o; o += (int)align_up((int64_t)m * top_k * kGroupRows * 4, 16);  // per-route sums of a leftover group
    s.ids = o;    o += (int)align_up((int64_t)m * top_k * 4, 16);
    s.wts = o;    o += (int)align_up((int64_t)m * top_k * 4, 16);
    s.cnt = o;    o += (int)align_up((int64_t)e_len * 4, 16);
    s.pstart = o; o += (int)align_up((int64_t)(e_len + 1) * 4, 16);
    s.pass_e = o; o += (int)align_up((int64_t)m * top_k * 2, 16);
    s.pass_n = o; o += (int)align_up((int64_t)m * top_k, 16);
    s.pass_r = o; o += (int)align_up((int64_t)m * top_k * 8 * 2, 16);
    s.bars = o;   o += 2 * kMaxStages * 8;
    s.misc = o;   o += 64 + (kMaxCtas + 8) * 4;
    s.total = o;
    return s;
}

// 8 packed E2M1 codes -> two words of E4M3 bytes (value * 2^-6):
// even nibbles (elements 0,2,4,6) and odd nibbles (elements 1,3,5,7).
__device__ __forceinline__ void fp4x8_to_e4m3(uint32_t w, uint32_t &even, uint32_t &odd) {
    even = ((w << 2) & 0x1C1C1C1Cu) | ((w << 4) & 0x80808080u);
    odd = ((w >> 2) & 0x1C1C1C1Cu) | (w & 0x80808080u);
}
__device__ __forceinline__ float e8m0_f32(uint32_t b) {
    return (b == 0xFFu) ? __uint_as_float(0x7FC00000u)
                        : (b == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(b << 23));
}

__device__ __forceinline__ void moe_down_kernel_body(const MoeParams &p, const uint32_t seq) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);

    const int vr = blockIdx.y, cta = blockIdx.x, ncta = gridDim.x;
    const MoeRankArgs &A = p.r[vr];
    const RankCtx &X = A.ctx;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int kbytes = p.k >> 1;
    const int kbox = (kbytes + 127) >> 7;  // 128-byte boxes = 256 K elements
    const int kb32 = p.k >> 5;
    const int NR = p.m * p.top_k;
    const int G = p.n / kGroupRows;
    const int Gm = G / ncta;
    const int Rg = G - Gm * ncta;
    const int extra = (!p.split && cta < Rg) ? 1 : 0;  // unsplit leftover: one more owned group
    const int n_own = Gm + extra;
    const int owned_rows = (Gm + ((!p.split && Rg) ? 1 : 0)) * kGroupRows;  // part_s row stride (uniform)
    auto group_of = [&](int gi) { return gi < Gm ? cta * Gm + gi : Gm * ncta + cta; };

    const MoeSmem S = moe_smem_layout(p.nstages, p.stage_boxes, p.k, p.m, p.top_k, A.e_len, owned_rows);
    uint8_t *q_s = smem + S.q;
    float *sa_s = reinterpret_cast<float *>(smem + S.sa);
    float *red_s = reinterpret_cast<float *>(smem + S.red);
    float *part_s = reinterpret_cast<float *>(smem + S.part);
    int32_t *ids_s = reinterpret_cast<int32_t *>(smem + S.ids);
    float *wts_s = reinterpret_cast<float *>(smem + S.wts);
    int32_t *cnt_s = reinterpret_cast<int32_t *>(smem + S.cnt);
    int32_t *pstart_s = reinterpret_cast<int32_t *>(smem + S.pstart);
    uint16_t *pass_e = reinterpret_cast<uint16_t *>(smem + S.pass_e);
    uint8_t *pass_n = smem + S.pass_n;
    uint16_t *pass_r = reinterpret_cast<uint16_t *>(smem + S.pass_r);
    volatile uint32_t *misc_s = reinterpret_cast<volatile uint32_t *>(smem + S.misc);
    const uint32_t stage0 = smem_u32(smem + S.stages);
    const uint32_t full0 = smem_u32(smem + S.bars), empty0 = full0 + kMaxStages * 8;
    const int NS = p.nstages;
    const int SB = p.stage_boxes;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(empty0 + s * 8, kConsumerWarps);
        }
        mbar_fence_init();
        prefetch_tmap(&A.tmap);
    }
    // ---- pass table (every CTA builds the same one): all threads, including the producer
    for (int i = tid; i < A.e_len; i += kThreads) cnt_s[i] = 0;
    for (int i = tid; i < p.m * owned_rows; i += kThreads) part_s[i] = 0.0f;
    __syncthreads();
    for (int i = tid; i < NR; i += kThreads) {
        const int e = A.route_ids[i];
        ids_s[i] = e;
        wts_s[i] = A.route_w[i];
        if (e >= A.e_start && e < A.e_start + A.e_len) atomicAdd(&cnt_s[e - A.e_start], 1);
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scan of passes per expert, 32 lanes x contiguous chunks
        const int per = (A.e_len + 31) / 32;
        const int a = lane * per, b = min(A.e_len, a + per);
        int sum = 0;
        for (int e = a; e < b; ++e) sum += (cnt_s[e] + 7) >> 3;
        int incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        int run = incl - sum;
        for (int e = a; e < b; ++e) {
            pstart_s[e] = run;
            run += (cnt_s[e] + 7) >> 3;
        }
        if (lane == 31) pstart_s[A.e_len] = incl;
    }
    __syncthreads();
    const int NP = pstart_s[A.e_len];
    for (int e = tid; e < A.e_len; e += kThreads) {
        const int c = cnt_s[e];
        if (c == 0) continue;
        const int ps = pstart_s[e];
        for (int q = 0; q < (c + 7) >> 3; ++q) {
            pass_e[ps + q] = (uint16_t)e;
            pass_n[ps + q] = (uint8_t)min(8, c - q * 8);
        }
        int idx = 0;
        for (int r = 0; r < NR; ++r)
            if (ids_s[r] == e + A.e_start) {
                pass_r[(ps + (idx >> 3)) * 8 + (idx & 7)] = (uint16_t)r;
                ++idx;
            }
    }
    __syncthreads();

    // leftover schedule: unit u = (j*NP + pass)*kbox + box
    const int64_t U = p.split ? (int64_t)Rg * NP * kbox : 0;
    int32_t *ub_s = reinterpret_cast<int32_t *>(smem + S.misc + 64);  // ub_s[c] = first split unit of CTA c
    for (int c = tid; c <= ncta; c += kThreads) ub_s[c] = (int32_t)unit_begin(c, U, ncta);
    __syncthreads();
    const int64_t u0 = unit_begin(cta, U, ncta), u1 = unit_begin(cta + 1, U, ncta);
    const int64_t pair0 = (u1 > u0) ? u0 / kbox : 0;
    const int nruns = (u1 > u0) ? (int)((u1 - 1) / kbox - pair0) + 1 : 0;
    const uint32_t bank = seq & 1u;
    const int nflag = kMaxCtas + kMaxShared;
    const uint32_t scale_item_bytes = (uint32_t)(kGroupRows * kb32);

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ TMA producer warp
        int item = 0;
        auto issue = [&](int e, int group, int b0, int nb) {
            const int s = item % NS;
            const uint32_t ph = (uint32_t)(item / NS) & 1u;
            mbar_wait(empty0 + s * 8, ph ^ 1u, X.status);
            const int64_t row = (int64_t)e * p.n + (int64_t)group * kGroupRows;
            if (lane == 0) {
                mbar_arrive_expect_tx(full0 + s * 8, (uint32_t)nb * kBoxBytes + scale_item_bytes);
                // the 16 rows' UE8M0 bytes are contiguous in the slab
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                    ::"r"(stage0 + s * S.stage_bytes + S.scale_off), "l"(A.s2 + row * kb32),
                      "r"(scale_item_bytes), "r"(full0 + s * 8)
                    : "memory");
            }
            __syncwarp();
            if (lane < nb)
                tma_load_2d(stage0 + s * S.stage_bytes + lane * kBoxBytes, &A.tmap, (b0 + lane) * 128, (int32_t)row,
                            full0 + s * 8);
            ++item;
        };
        for (int ps = 0; ps < NP; ++ps)
            for (int gi = 0; gi < n_own; ++gi)
                for (int b0 = 0; b0 < kbox; b0 += SB) issue(pass_e[ps], group_of(gi), b0, min(SB, kbox - b0));
        for (int r = 0; r < nruns; ++r) {
            const int64_t pair = pair0 + r;
            const int j = (int)(pair / NP), ps = (int)(pair - (int64_t)j * NP);
            const int ba = (int)(max(u0, pair * kbox) - pair * kbox);
            const int bb = (int)(min(u1, (pair + 1) * kbox) - pair * kbox);
            for (int b0 = ba; b0 < bb; b0 += SB) issue(pass_e[ps], Gm * ncta + j, b0, min(SB, bb - b0));
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps
    const int g = lane >> 2, tq = lane & 3;
    const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int lm_hi = lane >> 4;
    float acc[4];
    int item = 0, redbuf = 0;

    // Quantise hidden * routing weight of the (<= 8) routes of pass `ps` into q_s / sa_s.
    auto prep_pass = [&](int ps) {
        consumer_bar();  // every warp is done with the previous pass's q_s
        const int nr = pass_n[ps];
        const int chunks_per_row = kb32 * 4;
        for (int c = tid; c < 8 * chunks_per_row; c += kConsumerThreads) {
            const int col = c / chunks_per_row, ch = c - col * chunks_per_row;
            const bool valid = col < nr;
            const int route = valid ? pass_r[ps * 8 + col] : 0;
            float v[8];
            load_act8(A.h, p.h_dtype, (int64_t)route * A.ldh + ch * 8, valid, v);
            const float w = valid ? wts_s[route] : 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= w;
            int e;
            uint32_t lo, hi;
            act_quant8(v, e, lo, hi);
            const int kb = ch >> 2;
            uint2 st = make_uint2(0u, 0u);
            if (valid) st = make_uint2(__byte_perm(lo, hi, 0x6420), __byte_perm(lo, hi, 0x7531));
            *reinterpret_cast<uint2 *>(q_s + ((size_t)(kb * 8 + col) * 32 + (ch & 3) * 8)) = st;
            if ((ch & 3) == 0) sa_s[kb * 8 + col] = valid ? pow2_f32(e + 6) : 0.0f;
        }
        consumer_bar();
    };

    auto run_item = [&](int b0, int nb) {
        const int s = item % NS;
        mbar_wait(full0 + s * 8, (uint32_t)(item / NS) & 1u, X.status);
        const uint32_t sbase = stage0 + s * S.stage_bytes;
        const uint8_t *sc = smem + S.stages + (size_t)s * S.stage_bytes + S.scale_off;
        for (int bi = warp; bi < nb; bi += kConsumerWarps) {
            const int box = b0 + bi;
            const uint32_t bbase = sbase + bi * kBoxBytes + lm_row * 128;
            // UE8M0 bytes of the box's eight K blocks, rows g and g+8
            const uint64_t sc0 = *reinterpret_cast<const uint64_t *>(sc + g * kb32 + box * 8);
            const uint64_t sc1 = *reinterpret_cast<const uint64_t *>(sc + (g + 8) * kb32 + box * 8);
#pragma unroll
            for (int kp = 0; kp < 4; ++kp) {  // two 32-wide K blocks (two 16-byte chunks) per step
                const int kb = box * 8 + kp * 2;
                if (kb >= kb32) break;
                uint32_t w00, w10, w01, w11;  // (rows g / g+8) x (block kb / kb+1)
                ldmatrix_x4(bbase + ((((kp << 1) | lm_hi) ^ (lm_row & 7)) << 4), w00, w10, w01, w11);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int kbh = kb + h;
                    if (kbh >= kb32) break;
                    uint32_t a0, a1, a2, a3;
                    fp4x8_to_e4m3(h ? w01 : w00, a0, a2);
                    fp4x8_to_e4m3(h ? w11 : w10, a1, a3);
                    const uint2 b = *reinterpret_cast<const uint2 *>(q_s + ((size_t)(kbh * 8 + g) * 32 + tq * 8));
                    float d[4];
                    mma_e4m3_16x8x32(d, a0, a1, a2, a3, b.x, b.y);
                    const float2 sa = *reinterpret_cast<const float2 *>(sa_s + kbh * 8 + tq * 2);
                    const float s0 = e8m0_f32((uint32_t)(sc0 >> ((kp * 2 + h) * 8)) & 0xFFu);
                    const float s1 = e8m0_f32((uint32_t)(sc1 >> ((kp * 2 + h) * 8)) & 0xFFu);
                    acc[0] = fmaf(d[0], sa.x * s0, acc[0]);
                    acc[1] = fmaf(d[1], sa.y * s0, acc[1]);
                    acc[2] = fmaf(d[2], sa.x * s1, acc[2]);
                    acc[3] = fmaf(d[3], sa.y * s1, acc[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + s * 8);
        ++item;
    };
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

    const int row_t = tid & 15, col_t = tid >> 4;  // reduce threads: tid < 128
    const bool solo = p.world == 1;

    // ---- owned groups, passes in ascending expert id
    for (int ps = 0; ps < NP; ++ps) {
        if (n_own == 0) break;
        prep_pass(ps);
        const int nr = pass_n[ps];
        for (int gi = 0; gi < n_own; ++gi) {
            acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
            for (int b0 = 0; b0 < kbox; b0 += SB) run_item(b0, min(SB, kbox - b0));
            const float v = reduce_warps();
            if (tid < 128 && col_t < nr) {
                const int tok = pass_r[ps * 8 + col_t] / p.top_k;
                part_s[tok * owned_rows + gi * kGroupRows + row_t] += v;
            }
        }
    }

    // ---- leftover groups split over (pass, K box): contributions, last arriver folds
    int fin[kMaxRuns];
    int nfin = 0;
    for (int r = 0; r < nruns;) {
        const int j = (int)((pair0 + r) / NP);
        int r_end = r;  // runs [r, r_end) belong to leftover group j
        while (r_end < nruns && (int)((pair0 + r_end) / NP) == j) ++r_end;
        for (; r < r_end; ++r) {
            const int64_t pair = pair0 + r;
            const int ps = (int)(pair - (int64_t)j * NP);
            const int ba = (int)(max(u0, pair * kbox) - pair * kbox);
            const int bb = (int)(min(u1, (pair + 1) * kbox) - pair * kbox);
            prep_pass(ps);
            acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
            for (int b0 = ba; b0 < bb; b0 += SB) run_item(b0, min(SB, bb - b0));
            const float v = reduce_warps();
            if (tid < 128) X.contrib[((size_t)cta * kMaxRuns + r) * (8 * kGroupRows) + tid] = v;
        }
        if (tid < 128) __threadfence();
        consumer_bar();
        const int c_lo = owner_of((int64_t)j * NP * kbox, U, ncta);
        const int c_hi = owner_of((int64_t)(j + 1) * NP * kbox - 1, U, ncta);
        uint32_t expect = 0;  // CTAs that hold at least one unit of group j
        for (int c = c_lo; c <= c_hi; ++c) expect += ub_s[c + 1] > ub_s[c] ? 1u : 0u;
        if (tid == 0) {
            const uint32_t prev = atomicAdd(X.counters + j, 1u);
            misc_s[0] = (prev + 1u == expect) ? 1u : 0u;
            if (prev + 1u == expect) X.counters[j] = 0u;
        }
        consumer_bar();
        const bool last = misc_s[0] != 0u;
        consumer_bar();
        if (last) fin[nfin++] = j;
    }
    // A rank none of whose experts was selected still owes its (zero) leftover partials.
    const bool empty_rank = p.split && NP == 0 && cta < Rg;
    if (empty_rank) fin[nfin++] = cta;

    // Fold the leftover groups this CTA arrived last at.
    for (int f = 0; f < nfin; ++f) {
        const int j = fin[f];
        __threadfence();
        // Phase 1: per route, add the K-split contributions in K order.
        float *yroute = reinterpret_cast<float *>(smem + S.yroute);  // [NR][16]
        for (int ps = 0; ps < NP; ++ps) {
            const int64_t pair = (int64_t)j * NP + ps;
            const int ca = owner_of(pair * kbox, U, ncta), cb = owner_of((pair + 1) * kbox - 1, U, ncta);
            if (tid < 128 && col_t < pass_n[ps]) {
                float sum = 0.0f;
                for (int c = ca; c <= cb; ++c) {
                    const int cu0 = ub_s[c];
                    if (ub_s[c + 1] == cu0) continue;
                    const int ridx = (int)(pair - (int64_t)((uint32_t)cu0 / (uint32_t)kbox));
                    sum += ld_volatile_f32(X.contrib + ((size_t)c * kMaxRuns + ridx) * (8 * kGroupRows) + tid);
                }
                yroute[(size_t)pass_r[ps * 8 + col_t] * kGroupRows + row_t] = sum;
            }
        }
        consumer_bar();
        // Phase 2: per token, add its local routes in ascending expert id.
        for (int tok = tid >> 4; tok < p.m; tok += kConsumerThreads / 16) {
            float sum = 0.0f;
            int prev_e = -1;
            for (int it = 0; it < p.top_k; ++it) {
                int best = -1, best_e = 0x7FFFFFFF;
                for (int s = 0; s < p.top_k; ++s) {
                    const int e = ids_s[tok * p.top_k + s];
                    if (e >= A.e_start && e < A.e_start + A.e_len && e > prev_e && e < best_e) { best = s; best_e = e; }
                }
                if (best < 0) break;
                sum += yroute[(size_t)(tok * p.top_k + best) * kGroupRows + row_t];
                prev_e = best_e;
            }
            const int row = (Gm * ncta + j) * kGroupRows + row_t;
            if (solo) {
                A.out[(size_t)tok * p.n + row] = sum;
            } else {
                for (int pr = 0; pr < p.world; ++pr) {
                    float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.slotb_off) +
                                 (((size_t)bank * p.world + X.rank) * kMaxShared + j) * ((size_t)p.lay.max_m * kGroupRows);
                    dst[tok * kGroupRows + row_t] = sum;
                }
            }
        }
        consumer_bar();  // yroute is reused by the next leftover group
    }

    // ---- publish owned rows
    consumer_bar();
    if (solo) {
        for (int i = tid; i < p.m * n_own * kGroupRows; i += kConsumerThreads) {
            const int tok = i / (n_own * kGroupRows), r = i - tok * (n_own * kGroupRows);
            A.out[(size_t)tok * p.n + group_of(r >> 4) * kGroupRows + (r & 15)] = part_s[tok * owned_rows + r];
        }
        return;
    }
    for (int pr = 0; pr < p.world; ++pr) {
        float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.slota_off) +
                     ((size_t)bank * p.world + X.rank) * ((size_t)p.lay.max_m * p.lay.max_n);
        for (int i = tid; i < p.m * n_own * kGroupRows; i += kConsumerThreads) {
            const int tok = i / (n_own * kGroupRows), r = i - tok * (n_own * kGroupRows);
            dst[(size_t)tok * p.n + group_of(r >> 4) * kGroupRows + (r & 15)] = part_s[tok * owned_rows + r];
        }
    }
    __threadfence_system();
    consumer_bar();
    if (tid < p.world) {
        uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[tid] + p.lay.flags_off) +
                      ((size_t)bank * p.world + X.rank) * nflag;
        st_release_sys(f + cta, seq);
    }
    if (warp == 1) {
        for (int i = lane; i < nfin * p.world; i += 32) {
            uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[i % p.world] + p.lay.flags_off) +
                          ((size_t)bank * p.world + X.rank) * nflag;
            st_release_sys(f + kMaxCtas + fin[i / p.world], seq);
        }
    }
    const uint32_t *myflags = reinterpret_cast<const uint32_t *>(X.sym[X.rank] + p.lay.flags_off) +
                              (size_t)bank * p.world * nflag;
    if (tid < p.world)
        wait_flag(myflags + (size_t)tid * nflag + cta, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
    if (warp == 1)
        for (int i = lane; i < nfin * p.world; i += 32)
            wait_flag(myflags + (size_t)(i % p.world) * nflag + kMaxCtas + fin[i / p.world], seq, p.timeout_ns,
                      X.status, kStatTimeoutPeerB);
    consumer_bar();
    const size_t astride = (size_t)p.lay.max_m * p.lay.max_n;
    const float *slots = reinterpret_cast<const float *>(X.sym[X.rank] + p.lay.slota_off) +
                         (size_t)bank * p.world * astride;
    for (int i = tid; i < p.m * n_own * kGroupRows; i += kConsumerThreads) {
        const int tok = i / (n_own * kGroupRows), r = i - tok * (n_own * kGroupRows);
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
        for (int tok = tid >> 4; tok < p.m; tok += kConsumerThreads / 16) {
            const size_t off = (size_t)j * p.lay.max_m * kGroupRows + tok * kGroupRows + row_t;
            float s = __ldcg(slotb + off);
            for (int rr = 1; rr < p.world; ++rr) s += __ldcg(slotb + rr * bstride + off);
            A.out[(size_t)tok * p.n + (Gm * ncta + j) * kGroupRows + row_t] = s;
        }
    }
}

__global__ void __launch_bounds__(kThreads, 1) moe_down_kernel(const __grid_constant__ MoeParams p) {
    const RankCtx &X = p.r[blockIdx.y].ctx;
    const uint32_t seq = step_begin(X);
    moe_down_kernel_body(p, seq);
    step_end(X, seq, gridDim.x);
}

}  // namespace ws
