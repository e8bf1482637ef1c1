// MXFP4 routed-expert down projection + top-k combine fused with its exchange (sm_100a).
//
// Same persistent structure as the FP8 kernel (ws_fp8_kernel.cuh): a CTA owns whole 16-row
// tiles plus a ragged share of the leftover rows, every output row is complete inside one
// CTA, weights are streamed by TMA, partial sums are stored into every peer and added in
// rank order.
//
// A "pass" is one local expert that at least one token selected, with up to eight of its
// routes as the eight MMA columns (an expert with more routes takes several passes).  Passes
// run in ascending expert id, so a token's experts are added in the reference's order
// (crates/weightstream-ref/src/moe.rs:75-84).  Before each pass the consumers quantise
// hidden * routing-weight for its routes exactly as the reference does (moe.rs:150 then
// actquant.rs:21-57), while the producer warp keeps streaming the pass's weights.
//
// E2M1 -> E4M3 without a table: both formats keep subnormals the same way, so the three
// magnitude bits of an E2M1 code, shifted left by two, ARE the E4M3 code of value * 2^-6.
// The 2^6 is folded into the activation block scale.
#pragma once

#include <math.h>

#include "ws_device.cuh"
#include "ws_fp8_kernel.cuh"  // RowPlan

namespace ws {

constexpr int kMoeMaxRoutes = 512;
constexpr int kMoeMaxExperts = 512;
constexpr int kMoeMaxTopK = 8;

struct MoeRankArgs {
    const void *h;
    const int32_t *route_ids;
    const float *route_w;
    const uint8_t *s2;
    float *out;
    int64_t ldh;
    int32_t e_start, e_len;
    RankCtx ctx;
};

struct alignas(64) MoeParams {
    CUtensorMap tmap[WS_MAX_WORLD][2];  // slab as [e_len*n rows][k/2 bytes]; boxes 128 bytes x 16 rows / x gran rows
    int32_t m, n, k, top_k, h_dtype, world, nstages, tiles_per_item;
    int32_t ragged, gran, part_rows, pad0;
    uint64_t timeout_ns;
    SymLayout lay;
    MoeRankArgs r[WS_MAX_WORLD];
};

struct MoeSmem {
    int32_t stages, q, sa, red, part, ids, wts, cnt, pstart, pass_e, pass_n, pass_r, bars, total;
    int32_t stage_bytes, scale_off, tile_bytes;
};

__host__ __device__ inline MoeSmem moe_smem_layout(int nstages, int tiles_per_item, int k, int m, int top_k,
                                                   int e_len, int part_rows) {
    MoeSmem s{};
    const int kb32 = k / 32;
    const int kbox = (k / 2 + 127) / 128;
    s.tile_bytes = kbox * kBoxBytes;                       // one 16-row tile over the whole K
    s.scale_off = tiles_per_item * s.tile_bytes;           // the tiles' weight-scale bytes follow the boxes
    s.stage_bytes = (int)align_up(s.scale_off + tiles_per_item * kGroupRows * kb32, 1024);
    int o = 0;
    s.stages = o; o += nstages * s.stage_bytes;
    s.q = o;      o += kb32 * 8 * 32;
    s.sa = o;     o += kb32 * 8 * 4;
    s.red = o;    o += 2 * 2 * kConsumerWarps * 128 * 4;   // double buffered, two tiles per item
    s.part = o;   o += (int)align_up((int64_t)m * part_rows * 4, 16);
    s.ids = o;    o += (int)align_up((int64_t)m * top_k * 4, 16);
    s.wts = o;    o += (int)align_up((int64_t)m * top_k * 4, 16);
    s.cnt = o;    o += (int)align_up((int64_t)e_len * 4, 16);
    s.pstart = o; o += (int)align_up((int64_t)(e_len + 1) * 4, 16);
    s.pass_e = o; o += (int)align_up((int64_t)m * top_k * 2, 16);
    s.pass_n = o; o += (int)align_up((int64_t)m * top_k, 16);
    s.pass_r = o; o += (int)align_up((int64_t)m * top_k * 8 * 2, 16);
    s.bars = o;   o += 2 * kMaxStages * 8;
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

__device__ __forceinline__ void moe_down_body(const MoeParams &p) {
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
    const int TPI = p.tiles_per_item;
    // tiles of this CTA, as in the FP8 kernel: Gm whole ones, then the ragged rows cut at a 16-row boundary
    const RowPlan R = row_plan(p.n, ncta, cta, p.ragged, p.gran);
    const int xa = R.e0, xb = R.e1;
    const int xmid = min(xb, (xa / kGroupRows + 1) * kGroupRows);
    const int nx = xb > xa ? (xb > xmid ? 2 : 1) : 0;
    const int ntile = R.Gm + nx;
    auto trow = [&](int t) { return t < R.Gm ? (cta * R.Gm + t) * kGroupRows : (t == R.Gm ? xa : xmid); };
    auto tcnt = [&](int t) { return t < R.Gm ? kGroupRows : (t == R.Gm ? xmid - xa : xb - xmid); };
    const int PR = p.part_rows;

    const MoeSmem S = moe_smem_layout(p.nstages, TPI, p.k, p.m, p.top_k, A.e_len, PR);
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
    const uint32_t stage0 = smem_u32(smem + S.stages);
    const uint32_t full0 = smem_u32(smem + S.bars), empty0 = full0 + kMaxStages * 8;
    const int NS = p.nstages;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(empty0 + s * 8, kConsumerWarps);
        }
        mbar_fence_init();
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // routes, hidden states and the step sequence come from earlier work on the stream
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t seq = step_begin(X);

    // ---- pass table (every CTA builds the same one): all threads, including the producer
    for (int i = tid; i < A.e_len; i += kThreads) cnt_s[i] = 0;
    for (int i = tid; i < p.m * PR; i += kThreads) part_s[i] = 0.0f;
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

    const uint32_t bank = seq & 1u;
    const int nflag = kMaxCtas + kMaxShared;

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ TMA producer warp
        int item = 0;
        for (int ps = 0; ps < NP; ++ps) {
            const int64_t erow = (int64_t)pass_e[ps] * p.n;
            for (int t0 = 0; t0 < ntile; t0 += TPI, ++item) {
                const int nt = min(TPI, ntile - t0);
                const int s = item % NS;
                if (!mbar_wait(empty0 + s * 8, (((uint32_t)(item / NS)) & 1u) ^ 1u, X.status)) return;
                uint32_t bytes = 0;
                for (int j = 0; j < nt; ++j) bytes += (uint32_t)(tcnt(t0 + j) * (kbox * 128 + kb32));
                if (lane == 0) {
                    mbar_arrive_expect_tx(full0 + s * 8, bytes);
                    for (int j = 0; j < nt; ++j)  // the rows' UE8M0 bytes are contiguous in the slab
                        asm volatile(
                            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                            ::"r"(stage0 + s * S.stage_bytes + S.scale_off + j * kGroupRows * kb32),
                              "l"(A.s2 + (erow + trow(t0 + j)) * kb32), "r"((uint32_t)(tcnt(t0 + j) * kb32)),
                              "r"(full0 + s * 8)
                            : "memory");
                }
                __syncwarp();
                for (int i = lane; i < nt * kbox; i += 32) {
                    const int j = i / kbox, b = i - j * kbox;
                    const int r0 = trow(t0 + j), cnt = tcnt(t0 + j);
                    const uint32_t dst = stage0 + s * S.stage_bytes + j * S.tile_bytes + b * kBoxBytes;
                    if (cnt == kGroupRows) {
                        tma_load_2d(dst, &p.tmap[vr][0], b * 128, (int32_t)(erow + r0), full0 + s * 8);
                    } else {
                        for (int done = 0; done < cnt; done += p.gran)
                            tma_load_2d(dst + done * 128, &p.tmap[vr][1], b * 128, (int32_t)(erow + r0 + done), full0 + s * 8);
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps
    const int g = lane >> 2, tq = lane & 3;
    const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int lm_hi = lane >> 4;
    float acc[2][4];
    int item = 0, redbuf = 0;

    // Quantise hidden * routing weight of the (<= 8) routes of pass `ps` into q_s / sa_s.
    auto prep_pass = [&](int ps) {
        consumer_bar();  // every warp is done with the previous pass's q_s
        const int nr = pass_n[ps];
        const int chunks_per_row = kb32 * 4;
        const int total = nr * chunks_per_row;  // only the routes the pass carries
        for (int c0 = tid; c0 < ((total + 31) & ~31); c0 += 4 * kConsumerThreads) {
            float v[4][8];
            int col[4], ch[4];
            bool valid[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {  // four loads in flight per thread
                const int c = c0 + u * kConsumerThreads;
                col[u] = c / chunks_per_row;
                ch[u] = c - col[u] * chunks_per_row;
                valid[u] = c < total;
                const int route = valid[u] ? pass_r[ps * 8 + col[u]] : 0;
                load_act8(A.h, p.h_dtype, (int64_t)route * A.ldh + ch[u] * 8, valid[u], v[u]);
                const float w = valid[u] ? wts_s[route] : 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) v[u][i] *= w;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * kConsumerThreads;
                if (c >= ((total + 31) & ~31)) break;  // warp-uniform
                int e;
                uint32_t lo, hi;
                act_quant8(v[u], e, lo, hi);
                if (valid[u]) {
                    const int kb = ch[u] >> 2;
                    *reinterpret_cast<uint2 *>(q_s + ((size_t)(kb * 8 + col[u]) * 32 + (ch[u] & 3) * 8)) =
                        make_uint2(__byte_perm(lo, hi, 0x6420), __byte_perm(lo, hi, 0x7531));
                    if ((ch[u] & 3) == 0) sa_s[kb * 8 + col[u]] = pow2_f32(e + 6);
                }
            }
        }
        // columns the pass does not carry: zero scale and zero data, so they add nothing
        for (int i = tid; i < kb32 * (8 - nr); i += kConsumerThreads) {
            const int kb = i / (8 - nr), col = nr + i % (8 - nr);
            sa_s[kb * 8 + col] = 0.0f;
            uint4 *z = reinterpret_cast<uint4 *>(q_s + (size_t)(kb * 8 + col) * 32);
            z[0] = make_uint4(0u, 0u, 0u, 0u);
            z[1] = make_uint4(0u, 0u, 0u, 0u);
        }
        consumer_bar();
    };

    const uint32_t q_lane = smem_u32(q_s) + (uint32_t)(g * 32 + tq * 8);
    const uint32_t sa_lane = smem_u32(sa_s) + (uint32_t)(tq * 8);
    // One stage item: `nt` tiles of this pass, each kbox boxes wide; pair (tile j, box b) -> warps round robin.
    auto run_item = [&](int nt) {
        const int s = item % NS;
        mbar_wait(full0 + s * 8, ((uint32_t)(item / NS)) & 1u, X.status);
        const uint32_t sbase = stage0 + s * S.stage_bytes;
        const uint32_t scbase = sbase + S.scale_off;
        for (int pi = warp; pi < nt * kbox; pi += kConsumerWarps) {
            const int j = pi / kbox, box = pi - j * kbox;
            const uint32_t bbase = sbase + j * S.tile_bytes + box * kBoxBytes + lm_row * 128;
            const uint32_t sc = scbase + j * kGroupRows * kb32 + box * 8;
            // UE8M0 bytes of the box's eight K blocks, rows g and g+8
            const uint2 sc0v = lds_u64(sc + g * kb32), sc1v = lds_u64(sc + (g + 8) * kb32);
            const uint64_t sc0 = ((uint64_t)sc0v.y << 32) | sc0v.x, sc1 = ((uint64_t)sc1v.y << 32) | sc1v.x;
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
                    const uint2 b = lds_u64(q_lane + kbh * 256);
                    float d[4];
                    mma_e4m3_16x8x32(d, a0, a1, a2, a3, b.x, b.y);
                    const float2 sa = lds_f32x2(sa_lane + kbh * 32);
                    const float s0 = e8m0_f32((uint32_t)(sc0 >> ((kp * 2 + h) * 8)) & 0xFFu);
                    const float s1 = e8m0_f32((uint32_t)(sc1 >> ((kp * 2 + h) * 8)) & 0xFFu);
                    float *a = acc[j & 1];
                    a[0] = fmaf(d[0], sa.x * s0, a[0]);
                    a[1] = fmaf(d[1], sa.y * s0, a[1]);
                    a[2] = fmaf(d[2], sa.x * s1, a[2]);
                    a[3] = fmaf(d[3], sa.y * s1, a[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + s * 8);
        ++item;
    };
    // Sum the warps' accumulators of both tiles of the item in warp order; thread t < 128 ends
    // with (row = t & 15, column = t >> 4) of tile 0, thread 128 + t of tile 1.
    auto reduce_warps = [&]() -> float {
        float *rb = red_s + ((size_t)redbuf * 2 * kConsumerWarps + warp) * 128;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float *r = rb + (size_t)j * kConsumerWarps * 128;
            r[(2 * tq) * 16 + g] = acc[j][0];
            r[(2 * tq + 1) * 16 + g] = acc[j][1];
            r[(2 * tq) * 16 + g + 8] = acc[j][2];
            r[(2 * tq + 1) * 16 + g + 8] = acc[j][3];
        }
        consumer_bar();
        const float *r0 = red_s + ((size_t)redbuf * 2 + (tid >> 7)) * kConsumerWarps * 128 + (tid & 127);
        float v = r0[0];
#pragma unroll
        for (int w = 1; w < kConsumerWarps; ++w) v += r0[w * 128];
        redbuf ^= 1;
        return v;
    };

    const int row_t = tid & 15, col_t = (tid >> 4) & 7, tile_t = tid >> 7;  // reduce-thread roles
    const bool solo = p.world == 1;

    // ---- passes in ascending expert id
    for (int ps = 0; ps < NP; ++ps) {
        prep_pass(ps);
        const int nr = pass_n[ps];
        for (int t0 = 0; t0 < ntile; t0 += TPI) {
            const int nt = min(TPI, ntile - t0);
#pragma unroll
            for (int j = 0; j < 2; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
            run_item(nt);
            const float v = reduce_warps();
            if (tile_t < nt && col_t < nr) {
                const int tok = pass_r[ps * 8 + col_t] / p.top_k;
                part_s[tok * PR + (t0 + tile_t) * kGroupRows + row_t] += v;
            }
        }
    }
    consumer_bar();  // part_s complete

    // Visit every (token, valid row) of this CTA: fn(tok, global row, index in part_s).
    auto for_rows = [&](auto fn) {
        for (int i = tid; i < ntile * p.m * kGroupRows; i += kConsumerThreads) {
            const int t = i / (p.m * kGroupRows), j = i - t * (p.m * kGroupRows);
            const int tok = j >> 4, r = j & 15;
            if (r < tcnt(t)) fn(tok, trow(t) + r, tok * PR + t * kGroupRows + r);
        }
    };
    if (solo) {
        for_rows([&](int tok, int row, int pi) { A.out[(size_t)tok * p.n + row] = part_s[pi]; });
        return;
    }
    const size_t astride = (size_t)p.lay.max_m * p.lay.max_n;
    for (int pr = 0; pr < p.world; ++pr) {
        float *dst = reinterpret_cast<float *>(X.sym[pr] + p.lay.slotf_off) + ((size_t)bank * p.world + X.rank) * astride;
        for_rows([&](int tok, int row, int pi) { dst[(size_t)tok * p.n + row] = part_s[pi]; });
    }
    consumer_bar();  // the st.release.sys below is cumulative over the stores this barrier ordered
    if (tid < p.world) {
        uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[tid] + p.lay.flags_off) + ((size_t)bank * p.world + X.rank) * nflag;
        st_release_sys(f + cta, seq);
        const uint32_t *myflags = reinterpret_cast<const uint32_t *>(X.sym[X.rank] + p.lay.flags_off) +
                                  (size_t)bank * p.world * nflag;
        wait_flag(myflags + (size_t)tid * nflag + cta, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
    }
    consumer_bar();
    const float *slots = reinterpret_cast<const float *>(X.sym[X.rank] + p.lay.slotf_off) + (size_t)bank * p.world * astride;
    for_rows([&](int tok, int row, int) {
        const size_t off = (size_t)tok * p.n + row;
        float s = __ldcg(slots + off);
        for (int rr = 1; rr < p.world; ++rr) s += __ldcg(slots + rr * astride + off);
        A.out[off] = s;
    });
}

__global__ void __launch_bounds__(kThreads, 1) moe_down_kernel(const __grid_constant__ MoeParams p) {
    const RankCtx &X = p.r[blockIdx.y].ctx;
    moe_down_body(p);
    if (p.world > 1) step_end(X, step_begin(X), gridDim.x);
}

}  // namespace ws
