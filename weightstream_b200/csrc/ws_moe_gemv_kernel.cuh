// MXFP4 routed-expert down projection + top-k combine fused with its exchange: decode form
// (sm_100a, CUDA cores).
//
// In decode an expert is selected by one or two tokens, so every weight byte is used once or
// twice: the step is a set of matrix-vector products and HBM bandwidth is the bound.  Two
// kernels per step:
//
//   moe_prep_kernel   one block per route quantises hidden * routing-weight exactly as the
//                     reference does (crates/weightstream-ref/src/moe.rs:150, then
//                     actquant.rs:21-57) and stores the quantised values as f16 (exact) with the
//                     per-32 block scales; one more block sorts the routes by expert and writes
//                     the pass table.  Done once per step, not once per CTA.
//   moe_gemv_kernel   persistent, one CTA per SM.  A CTA owns a contiguous range of output rows
//                     and walks the passes (local experts in ascending id, as moe.rs:75-84 adds
//                     them).  Per pass the producer warp streams the expert's rows of that range
//                     (TMA, 128B swizzle), their UE8M0 scale bytes and the pass's activations
//                     (bulk copies) into shared-memory rings.  Sixteen consumer warps: a lane owns
//                     one 32-wide K block (16 bytes of E2M1 codes) of every row its warp visits,
//                     keeps that block's activations in registers (f16 pairs) for the whole pass,
//                     converts the codes to f16 pairs and accumulates the exact products in fp32
//                     (fma.rn.f32.f16); a row's
//                     lanes are combined by shuffles and lane 0 adds the result to the
//                     accumulator of (K slice, token, row), which only ever this warp touches:
//                     no barrier between passes, deterministic order.
//
// Exchange: as in the FP8 kernel (partials stored to every peer as tagged words, folded in rank
// order).
#pragma once

#include <math.h>

#include <type_traits>

#include "ws_device.cuh"
#include "ws_moe_kernel.cuh"  // kMoeMaxRoutes, kMoeMaxExperts, e8m0_f32

namespace ws {

constexpr int kMoeGemvWarps = 16;
constexpr int kMoeGemvThreads = (kMoeGemvWarps + 1) * 32;  // + the producer warp
constexpr int kMoeRoutesPerPass = 4;                        // more routes of one expert take further passes
constexpr int kMoeXSlots = 8;                               // activation ring: two full passes
constexpr int kMoeMaxPanelRows = 64;

struct MoePass {
    uint16_t expert;  // local expert index
    uint16_t first;   // index of its first route in the sorted route list
    uint16_t nr;      // routes in this pass (1..kMoeRoutesPerPass)
    uint16_t pad;
};

// Per-endpoint scratch written by moe_prep_kernel and read by moe_gemv_kernel.
struct MoeWork {
    int64_t hdr, pass, sorted, stok, sa, xq, total;  // byte offsets
};
__host__ __device__ inline MoeWork moe_work_layout(int k) {
    MoeWork w{};
    int64_t o = 0;
    w.hdr = o;    o += 64;
    w.pass = o;   o += (int64_t)kMoeMaxRoutes * sizeof(MoePass);
    w.sorted = o; o += align_up((int64_t)kMoeMaxRoutes * 2, 64);
    w.stok = o;   o += align_up((int64_t)kMoeMaxRoutes * 2, 64);
    w.sa = o;     o += (int64_t)kMoeMaxRoutes * (k / 32) * 4;
    w.xq = o;     o += (int64_t)kMoeMaxRoutes * k * 2;
    w.total = o;
    return w;
}

struct MoePrepRank {
    const void *h;
    const int32_t *route_ids;
    const float *route_w;
    uint8_t *work;
    int64_t ldh;
    int32_t e_start, e_len;
};
struct MoePrepParams {
    int32_t m, k, top_k, h_dtype;
    MoePrepRank r[WS_MAX_WORLD];
};

__global__ void __launch_bounds__(256) moe_prep_kernel(const __grid_constant__ MoePrepParams p) {
    // the hidden states and routes come from earlier work on the stream; the step that follows
    // may start streaming as soon as this grid is resident
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const MoePrepRank &A = p.r[blockIdx.y];
    const int NR = p.m * p.top_k, tid = threadIdx.x;
    const MoeWork W = moe_work_layout(p.k);
    if ((int)blockIdx.x < NR) {
        const int route = blockIdx.x;
        const int e = A.route_ids[route];
        if (e < A.e_start || e >= A.e_start + A.e_len) return;  // another rank's expert
        const float w = A.route_w[route];
        uint8_t *xq = A.work + W.xq + (size_t)route * p.k * 2;
        float *sa = reinterpret_cast<float *>(A.work + W.sa) + (size_t)route * (p.k >> 5);
        for (int c = tid; c < (p.k >> 3); c += blockDim.x) {
            float v[8];
            load_act8(A.h, p.h_dtype, (int64_t)route * A.ldh + c * 8, true, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= w;
            int ex;
            uint32_t lo, hi;
            act_quant8(v, ex, lo, hi);
            *reinterpret_cast<uint4 *>(xq + (size_t)c * 16) =
                make_uint4(e4m3x2_to_f16x2(lo), e4m3x2_to_f16x2(lo >> 16), e4m3x2_to_f16x2(hi), e4m3x2_to_f16x2(hi >> 16));
            if ((c & 3) == 0) sa[c >> 2] = pow2_f32(ex);
        }
        return;
    }
    // ---- the last block: routes sorted by expert (stable), then the pass table
    __shared__ int32_t ids_s[kMoeMaxRoutes];
    __shared__ int32_t cnt_s[kMoeMaxExperts];
    __shared__ int32_t rstart_s[kMoeMaxExperts + 1];  // first sorted index of an expert's routes
    __shared__ int32_t pstart_s[kMoeMaxExperts + 1];  // first pass of an expert
    for (int i = tid; i < A.e_len; i += blockDim.x) cnt_s[i] = 0;
    __syncthreads();
    for (int i = tid; i < NR; i += blockDim.x) {
        const int e = A.route_ids[i] - A.e_start;
        ids_s[i] = e;
        if (e >= 0 && e < A.e_len) atomicAdd(&cnt_s[e], 1);
    }
    __syncthreads();
    if (tid < 32) {  // two exclusive scans over the experts, 32 lanes x contiguous chunks
        const int per = (A.e_len + 31) / 32;
        const int a = tid * per, b = min(A.e_len, a + per);
        int sr = 0, sp = 0;
        for (int e = a; e < b; ++e) {
            sr += cnt_s[e];
            sp += (cnt_s[e] + kMoeRoutesPerPass - 1) / kMoeRoutesPerPass;
        }
        int ir = sr, ip = sp;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int tr = __shfl_up_sync(0xffffffffu, ir, o), tpp = __shfl_up_sync(0xffffffffu, ip, o);
            if (tid >= o) { ir += tr; ip += tpp; }
        }
        int rr = ir - sr, rp = ip - sp;
        for (int e = a; e < b; ++e) {
            rstart_s[e] = rr;
            pstart_s[e] = rp;
            rr += cnt_s[e];
            rp += (cnt_s[e] + kMoeRoutesPerPass - 1) / kMoeRoutesPerPass;
        }
        if (tid == 31) {
            rstart_s[A.e_len] = ir;
            pstart_s[A.e_len] = ip;
        }
    }
    __syncthreads();
    MoePass *pass = reinterpret_cast<MoePass *>(A.work + W.pass);
    uint16_t *sorted = reinterpret_cast<uint16_t *>(A.work + W.sorted);
    uint16_t *stok = reinterpret_cast<uint16_t *>(A.work + W.stok);  // the routes' tokens, same order
    for (int e = tid; e < A.e_len; e += blockDim.x) {
        const int c = cnt_s[e];
        if (c == 0) continue;
        int idx = rstart_s[e];
        for (int r = 0; r < NR; ++r)
            if (ids_s[r] == e) {
                sorted[idx] = (uint16_t)r;
                stok[idx] = (uint16_t)(r / p.top_k);
                ++idx;
            }
        for (int q = 0; q * kMoeRoutesPerPass < c; ++q) {
            MoePass ps;
            ps.expert = (uint16_t)e;
            ps.first = (uint16_t)(rstart_s[e] + q * kMoeRoutesPerPass);
            ps.nr = (uint16_t)min(kMoeRoutesPerPass, c - q * kMoeRoutesPerPass);
            ps.pad = 0;
            pass[pstart_s[e] + q] = ps;
        }
    }
    if (tid == 0) *reinterpret_cast<int32_t *>(A.work + W.hdr) = pstart_s[A.e_len];
}

// ------------------------------------------------------------------------------------------
struct MoeGemvRank {
    const uint8_t *s2;
    const uint8_t *work;
    float *out;
    float *acc_g;  // [nslice][m][n] accumulators when they do not fit shared memory
    int32_t e_start, e_len;
    RankCtx ctx;
};

struct alignas(64) MoeGemvParams {
    CUtensorMap tmap[WS_MAX_WORLD][2];  // slab as [e_len*n rows][k/2 bytes]; boxes of 128 bytes x 16 rows / x gran rows
    int32_t m, n, k, top_k, world, nstages, gran, panel_rows;
    int32_t rows_pitch, stage_bytes, scale_off, acc_global;
    int32_t acc_rows, pad0;  // rows per CTA the shared-memory accumulators are laid out for
    uint64_t timeout_ns;
    SymLayout lay;
    MoeGemvRank r[WS_MAX_WORLD];
};

struct MoeGemvSmem {
    int32_t stages, xring, acc, pass, sorted, stok, bars, total;
    int32_t xbytes;
};
__host__ __device__ inline int moe_gemv_slices(int k) { return (k / 32 + 31) / 32; }  // warps along K
__host__ __device__ inline MoeGemvSmem moe_gemv_smem(int nstages, int stage_bytes, int k, int m, int acc_rows,
                                                     int acc_global) {
    MoeGemvSmem s{};
    int o = 0;
    s.stages = o; o += nstages * stage_bytes;
    s.xbytes = (int)align_up((int64_t)k * 2 + (k / 32) * 4, 128);
    s.xring = o;  o += kMoeXSlots * s.xbytes;
    s.acc = o;    o += acc_global ? 0 : (int)align_up((int64_t)moe_gemv_slices(k) * m * acc_rows * 4, 16);
    s.pass = o;   o += kMoeMaxRoutes * (int)sizeof(MoePass);
    s.sorted = o; o += kMoeMaxRoutes * 2;
    s.stok = o;   o += kMoeMaxRoutes * 2;
    s.bars = o;   o += (2 * kMaxStages + 2 * kMoeXSlots) * 8;
    s.total = o;
    return s;
}

// Rows of CTA `cta`: units of `gran` rows dealt out evenly.
__host__ __device__ inline void moe_gemv_rows(int n, int gran, int ncta, int cta, int &a, int &b) {
    const int U = n / gran;
    a = gran * (int)((int64_t)cta * U / ncta);
    b = gran * (int)((int64_t)(cta + 1) * U / ncta);
}

// 16 bytes of E2M1 codes (32 values, low nibble first) times 32 activations (16 f16 pairs):
// the codes become f16 pairs, the products of a 2-bit and a 4-bit significand are exact, the
// sums are fp32 (mixed-precision FMA).  Measured on B200: 28 weight bytes per clock and SM,
// against 16 with conversions to f32 and packed fp32 FMAs.
template <int RT>
__device__ __forceinline__ void dot32_e2m1(const uint4 w, const uint32_t (&xa)[16], const uint32_t (&xb)[16], float &da,
                                           float &db) {
    float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t h0 = e2m1x2_byte_to_f16x2<0>(ww[i]), h1 = e2m1x2_byte_to_f16x2<1>(ww[i]);
        const uint32_t h2 = e2m1x2_byte_to_f16x2<2>(ww[i]), h3 = e2m1x2_byte_to_f16x2<3>(ww[i]);
        fma2_f16(a0, h0, xa[4 * i + 0]); fma2_f16(a1, h1, xa[4 * i + 1]);
        fma2_f16(a0, h2, xa[4 * i + 2]); fma2_f16(a1, h3, xa[4 * i + 3]);
        if (RT == 2) {  // a second route of the same expert shares the converted codes
            fma2_f16(b0, h0, xb[4 * i + 0]); fma2_f16(b1, h1, xb[4 * i + 1]);
            fma2_f16(b0, h2, xb[4 * i + 2]); fma2_f16(b1, h3, xb[4 * i + 3]);
        }
    }
    da = a0 + a1;
    db = b0 + b1;
}

// Four per-lane partial sums (one per row) -> their 32-lane sums: lanes are folded 4 -> 2 -> 1
// values per lane, then three plain steps (6 shuffles instead of 20).  The lane with
// (lane & 7) == 0 ends with the sum of row 2 * bit4(lane) + bit3(lane).
__device__ __forceinline__ float fold4(const float (&v)[4], bool hi16, bool hi8) {
    float k0 = hi16 ? v[2] : v[0], k1 = hi16 ? v[3] : v[1];
    k0 += __shfl_xor_sync(0xffffffffu, hi16 ? v[0] : v[2], 16);
    k1 += __shfl_xor_sync(0xffffffffu, hi16 ? v[1] : v[3], 16);
    float k = hi8 ? k1 : k0;
    k += __shfl_xor_sync(0xffffffffu, hi8 ? k0 : k1, 8);
    k += __shfl_xor_sync(0xffffffffu, k, 4);
    k += __shfl_xor_sync(0xffffffffu, k, 2);
    k += __shfl_xor_sync(0xffffffffu, k, 1);
    return k;
}

__device__ __forceinline__ void moe_gemv_body(const MoeGemvParams &p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);

    const int vr = blockIdx.y, cta = blockIdx.x, ncta = gridDim.x;
    const MoeGemvRank &A = p.r[vr];
    const RankCtx &X = A.ctx;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int CW = kMoeGemvWarps, CT = CW * 32;

    const int kbytes = p.k >> 1, kbox = kbytes >> 7, kb32 = p.k >> 5;
    const int NS = p.nstages;
    const int nslice = moe_gemv_slices(p.k);
    int row_a, row_b;
    moe_gemv_rows(p.n, p.gran, ncta, cta, row_a, row_b);
    const int rows_cta = row_b - row_a;
    const int npanel = (rows_cta + p.panel_rows - 1) / p.panel_rows;

    const MoeGemvSmem S = moe_gemv_smem(NS, p.stage_bytes, p.k, p.m, p.acc_rows, p.acc_global);
    const MoeWork W = moe_work_layout(p.k);
    MoePass *pass_s = reinterpret_cast<MoePass *>(smem + S.pass);
    uint16_t *sorted_s = reinterpret_cast<uint16_t *>(smem + S.sorted);
    uint16_t *stok_s = reinterpret_cast<uint16_t *>(smem + S.stok);
    const uint32_t stage0 = smem_u32(smem + S.stages), xring0 = smem_u32(smem + S.xring);
    const uint32_t full0 = smem_u32(smem + S.bars), empty0 = full0 + kMaxStages * 8;
    const uint32_t xfull0 = empty0 + kMaxStages * 8, xempty0 = xfull0 + kMoeXSlots * 8;
    // accumulators of (K slice, token, row): shared memory, or global when m is large
    float *acc_base = p.acc_global ? A.acc_g + row_a : reinterpret_cast<float *>(smem + S.acc);
    const size_t acc_stride = p.acc_global ? (size_t)p.n : (size_t)p.acc_rows;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(empty0 + s * 8, CW);
        }
        for (int s = 0; s < kMoeXSlots; ++s) {
            mbar_init(xfull0 + s * 8, 1);
            mbar_init(xempty0 + s * 8, CW);
        }
        mbar_fence_init();
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // pass table, activations and the step sequence come from earlier work on the stream
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t seq = step_begin(X);
    const int NP = *reinterpret_cast<const int32_t *>(A.work + W.hdr);
    {
        const uint2 *src = reinterpret_cast<const uint2 *>(A.work + W.pass);
        for (int i = tid; i < NP; i += kMoeGemvThreads) reinterpret_cast<uint2 *>(pass_s)[i] = src[i];
        const uint16_t *ss = reinterpret_cast<const uint16_t *>(A.work + W.sorted);
        const uint16_t *st = reinterpret_cast<const uint16_t *>(A.work + W.stok);
        for (int i = tid; i < p.m * p.top_k; i += kMoeGemvThreads) {
            sorted_s[i] = ss[i];
            stok_s[i] = st[i];
        }
    }
    // zero this CTA's accumulators
    if (p.acc_global) {
        for (int i = tid; i < nslice * p.m * rows_cta; i += kMoeGemvThreads)
            acc_base[(size_t)(i / rows_cta) * acc_stride + (i % rows_cta)] = 0.0f;
    } else {
        for (int i = tid; i < nslice * p.m * p.acc_rows; i += kMoeGemvThreads) acc_base[i] = 0.0f;
    }
    __syncthreads();

    const uint32_t bank = seq & 1u;
    const int nflag = kMaxCtas + kMaxShared;
    const uint32_t colpitch = (uint32_t)(p.rows_pitch * 128);

    if (warp == CW) {
        // ------------------------------------------------------------ producer warp
        int xi = 0;
        RingPos rp;
        for (int pn = 0; pn < npanel; ++pn) {
            const int r0 = row_a + pn * p.panel_rows, rows = min(p.panel_rows, row_b - r0);
            const int nb16 = rows >> 4, nbg = (rows & 15) / p.gran, nbox = nb16 + nbg;
            for (int ps = 0; ps < NP; ++ps, rp.next(NS)) {
                const MoePass P = pass_s[ps];
                for (int j = 0; j < P.nr; ++j, ++xi) {  // the pass's activations, one ring slot per route
                    const int xs = xi % kMoeXSlots;
                    if (!mbar_wait(xempty0 + xs * 8, (((uint32_t)(xi / kMoeXSlots)) & 1u) ^ 1u, X.status)) return;
                    if (lane == 0) {
                        const int route = sorted_s[P.first + j];
                        const uint32_t dst = xring0 + xs * S.xbytes;
                        mbar_arrive_expect_tx(xfull0 + xs * 8, (uint32_t)(p.k * 2 + kb32 * 4));
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(dst), "l"(A.work + W.xq + (size_t)route * p.k * 2), "r"((uint32_t)(p.k * 2)),
                                       "r"(xfull0 + xs * 8) : "memory");
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(dst + p.k * 2), "l"(A.work + W.sa + (size_t)route * kb32 * 4), "r"((uint32_t)(kb32 * 4)),
                                       "r"(xfull0 + xs * 8) : "memory");
                    }
                    __syncwarp();
                }
                const int s = rp.s;
                const int64_t erow = (int64_t)P.expert * p.n + r0;
                if (!mbar_wait(empty0 + s * 8, rp.ph ^ 1u, X.status)) return;  // a wait gave up: stop streaming
                const uint32_t sbase = stage0 + s * p.stage_bytes;
                if (lane == 0) {
                    mbar_arrive_expect_tx(full0 + s * 8, (uint32_t)(rows * (kbytes + kb32)));
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(sbase + p.scale_off), "l"(A.s2 + erow * kb32), "r"((uint32_t)(rows * kb32)),
                                   "r"(full0 + s * 8) : "memory");
                }
                __syncwarp();
                for (int i = lane; i < kbox * nbox; i += 32) {
                    const int b = i / nbox, j = i - b * nbox;
                    if (j < nb16)
                        tma_load_2d(sbase + b * colpitch + j * 2048, &p.tmap[vr][0], b * 128, (int32_t)(erow + j * 16), full0 + s * 8);
                    else
                        tma_load_2d(sbase + b * colpitch + (nb16 * 16 + (j - nb16) * p.gran) * 128, &p.tmap[vr][1], b * 128,
                                    (int32_t)(erow + nb16 * 16 + (j - nb16) * p.gran), full0 + s * 8);
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps
    // Lane = one 32-wide K block c of the rows its warp visits; warps = K slices x row groups.
    const int ng = CW / nslice;                  // row groups
    const int kslice = warp % nslice, rg = warp / nslice;
    const bool wactive = rg < ng;                // warps beyond ng * nslice only keep the barriers moving
    const int c = kslice * 32 + lane;
    const bool lvalid = c < kb32;
    const int cs = lvalid ? c : 0;               // idle lanes read block 0 and multiply by zero
    const uint32_t lane_col = (uint32_t)((cs >> 3) * colpitch);
    const int cc = cs & 7;
    int xi = 0;
    RingPos rp;
    for (int pn = 0; pn < npanel; ++pn) {
        const int r0 = pn * p.panel_rows, rows = min(p.panel_rows, rows_cta - r0);  // r0 relative to row_a
        for (int ps = 0; ps < NP; ++ps, rp.next(NS)) {
            const MoePass P = pass_s[ps];
            const int s = rp.s;
            const uint32_t sbase = stage0 + s * p.stage_bytes;
            bool landed = false;
            const bool hi16 = (lane & 16) != 0, hi8 = (lane & 8) != 0;
            const int jrow = (hi16 ? 2 : 0) + (hi8 ? 1 : 0);
            // this lane's 32 quantised activations (f16 pairs) and block scale of the next route
            auto take_route = [&](int j, uint32_t (&xh)[16], float &sa, int &tok) {
                const int xs = xi % kMoeXSlots;
                tok = stok_s[P.first + j];
                mbar_wait(xfull0 + xs * 8, ((uint32_t)(xi / kMoeXSlots)) & 1u, X.status);
                const uint32_t xa = xring0 + xs * S.xbytes;
                sa = lvalid ? lds_f32(xa + p.k * 2 + cs * 4) : 0.0f;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint4 v = lds_u128(xa + cs * 64 + q * 16);
                    xh[q * 4 + 0] = v.x; xh[q * 4 + 1] = v.y; xh[q * 4 + 2] = v.z; xh[q * 4 + 3] = v.w;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(xempty0 + xs * 8);  // the values are in registers
                ++xi;
            };
            // rows of this warp, four at a time, against one route or two routes of the expert
            auto rows_pass = [&](auto rt_c, const uint32_t (&xa)[16], const uint32_t (&xb)[16], float sa, float sb2, int ta,
                                 int tb) {
                constexpr int RT = decltype(rt_c)::value;
                float *acc_a = acc_base + ((size_t)kslice * p.m + ta) * acc_stride + r0;
                float *acc_b = acc_base + ((size_t)kslice * p.m + tb) * acc_stride + r0;
                for (int rb = rg; rb < rows; rb += 4 * ng) {
                    float va[4], vb[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int r = rb + j * ng;
                        va[j] = vb[j] = 0.0f;
                        if (r < rows) {  // warp-uniform
                            const uint4 w = lds_u128(sbase + lane_col + r * 128 + ((uint32_t)(cc ^ (r & 7)) << 4));
                            const float sw = e8m0_f32(lds_u8(sbase + p.scale_off + r * kb32 + cs));
                            float da, db;
                            dot32_e2m1<RT>(w, xa, xb, da, db);
                            va[j] = da * (sa * sw);
                            if (RT == 2) vb[j] = db * (sb2 * sw);
                        }
                    }
                    const int r = rb + jrow * ng;
                    const float ka = fold4(va, hi16, hi8);
                    if ((lane & 7) == 0 && r < rows) atomicAdd(acc_a + r, ka);  // only this warp ever adds to this address
                    if (RT == 2) {
                        const float kb2 = fold4(vb, hi16, hi8);
                        if ((lane & 7) == 0 && r < rows) atomicAdd(acc_b + r, kb2);
                    }
                }
            };
            for (int j = 0; j < P.nr;) {
                const int rt = P.nr - j >= 2 ? 2 : 1;
                uint32_t xa[16], xb[16];
                float sa, sb2 = 0.0f;
                int ta, tb = 0;
                take_route(j, xa, sa, ta);
                if (rt == 2) take_route(j + 1, xb, sb2, tb);
                if (!landed) {
                    mbar_wait(full0 + s * 8, rp.ph, X.status);
                    landed = true;
                }
                if (wactive) {
                    if (rt == 2) rows_pass(std::integral_constant<int, 2>{}, xa, xb, sa, sb2, ta, tb);
                    else         rows_pass(std::integral_constant<int, 1>{}, xa, xa, sa, sa, ta, ta);
                }
                j += rt;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + s * 8);
        }
    }
    consumer_bar_n<CT>();  // accumulators complete

    // Value of (token, row r of this CTA): the K slices in ascending order.
    auto value = [&](int tok, int r) {
        float v = 0.0f;
        for (int ks = 0; ks < nslice; ++ks) {
            const float *a = acc_base + ((size_t)ks * p.m + tok) * acc_stride + r;
            v += p.acc_global ? __ldcg(a) : *a;
        }
        return v;
    };
    const bool solo = p.world == 1;
    if (solo) {
        for (int i = tid; i < p.m * rows_cta; i += CT) {
            const int tok = i / rows_cta, r = i - tok * rows_cta;
            A.out[(size_t)tok * p.n + row_a + r] = value(tok, r);
        }
        return;
    }
    // tagged-word exchange, as in the FP8 kernel: send, then fold the same rows in rank order
    const size_t astride = (size_t)p.lay.max_m * p.lay.max_n;
    for (int i = tid; i < p.m * rows_cta; i += CT) {
        const int tok = i / rows_cta, r = i - tok * rows_cta;
        const float v = value(tok, r);
        for (int pr = 0; pr < p.world; ++pr) {
            uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[pr] + p.lay.slota_off) + ((size_t)bank * p.world + X.rank) * astride;
            st_word_sys(dst + (size_t)tok * p.n + row_a + r, seq, v);
        }
    }
    const uint64_t *slots = reinterpret_cast<const uint64_t *>(X.sym[X.rank] + p.lay.slota_off) + (size_t)bank * p.world * astride;
    for (int i = tid; i < p.m * rows_cta; i += CT) {
        const int tok = i / rows_cta, r = i - tok * rows_cta;
        const size_t off = (size_t)tok * p.n + row_a + r;
        const float s = fold_words(slots, astride, off, p.world, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
        A.out[off] = s;
    }
}

__global__ void __launch_bounds__(kMoeGemvThreads, 1) moe_gemv_kernel(const __grid_constant__ MoeGemvParams p) {
    const RankCtx &X = p.r[blockIdx.y].ctx;
    moe_gemv_body(p);
    if (p.world > 1) step_end(X, step_begin(X), gridDim.x);
}

}  // namespace ws
