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
//   fp8_bs_kernel     persistent, one CTA per SM.  The rows are cut into tiles of at most 128 rows (the
//                     M of the MMA) that deal out evenly, and a CTA streams the weights of its tiles over
//                     the whole local K, so every output is a complete dot product inside one CTA.  Per
//                     128-byte K slab the producer warp lands, in one stage of a shared-memory ring: the
//                     tile's weight rows (TMA box, 128B swizzle), the quantised activations of all
//                     tokens (TMA box from the prep kernel's buffer) and their scale atom (bulk copy).
//                     One thread copies the atom into tensor memory (tcgen05.cp) and issues four MMAs
//                     (M=128, N=tokens, K=32): the activations' per-32 scales ride the MMA's scale
//                     operand, the weight operand's scale is 2^0, and the four K blocks accumulate in
//                     tensor memory.  The weights' own scales are fp32 per (block_n x block_k) block,
//                     which no MMA scale format can carry, so every slab gets its own accumulator
//                     buffer and four epilogue warps read a stage's buffers back (tcgen05.ld) and add
//                     them, times the fp32 weight scale, to their registers while the next stages'
//                     MMAs run into the other buffers.
//
// Measured on B200 and kept in mind above: the tensor pipe needs 30-45 ns per K=32 MMA at M=128 however
// few of the rows are real (M=64 is not available with block scaling); a tcgen05.commit stalls the
// issuing thread for ~160 ns; handing partial sums from one CTA to another through L2 (a split of K
// across CTAs) costs 3-5 us, more than it saves on these shapes.
//
// MMA rows past a tile's end are computed on whatever follows in shared memory and never read back.
// Exchange and lm_head mode are those of the decode kernel (ws_fp8_kernel.cuh): tagged 64-bit
// words stored into every peer's slots and folded in rank order, or argmax candidates merged per rank.
#pragma once

#include <math.h>

#include "ws_device.cuh"
#include "ws_fp8_kernel.cuh"

namespace ws {

// Threads of a CTA.  Warp 0: producer, warp 1: MMA issue (and owner of the tensor memory), then the
// epilogue warps: four (one per 32-lane quarter of the tensor memory, all token columns) for up to 32
// tokens, eight (two per quarter, half of the token columns each) for 64, where reading the
// accumulators back is what a stage waits for (measured on B200, 64 rows: lm_head 324 -> 249 us;
// with 32 rows eight warps were 3 % slower than four).
__host__ __device__ constexpr int bs_epi_warps(int mp) { return mp >= 64 ? 8 : 4; }
__host__ __device__ constexpr int bs_threads(int mp) { return 64 + 32 * bs_epi_warps(mp); }
constexpr int kBsMaxAcc = 8;         // accumulator groups in tensor memory (a group = one stage's slabs)
constexpr int kBsMaxTokens = 128;    // activation rows one launch takes (16, 32, 64 or 128 MMA columns)
constexpr int kBsAtomBytes = 512;    // one scale atom: 128 rows x 4 K blocks
constexpr int kBsMmaRows = 128;      // M of the MMA; a tile of output rows holds at most as many

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
    CUtensorMap tmap_w[WS_MAX_WORLD];  // weight shard [n][k bytes], box 128 bytes x tile_rows, 128B swizzle
    CUtensorMap tmap_x[WS_MAX_WORLD];  // quantised activations [mp][k bytes], box 128 bytes x mp, 128B swizzle
    int32_t m, mp, n, k, bn_shift, bk_shift;
    int32_t world, mode, vocab, tmem_cols;  // tmem_cols: tensor-memory columns to allocate (512, or at most 256 when two CTAs share an SM)
    int32_t owner_reduce;              // all-reduce by owners: tile t is folded by rank t % world, which sends the sums back
    int32_t csize;                     // 1, or 2: CTA pairs (a cluster) share a tile, each streams half of K
    int32_t tile_rows, ntiles;         // output rows per tile (<= 128) and tiles of the shard
    int32_t slabs_per_stage, nstages;
    int32_t a_pitch, b_pitch;          // bytes one slab's weights / activations occupy in a stage (multiples of 1024)
    int32_t skb, nslot_max, nacc;
    uint64_t timeout_ns;
    SymLayout lay;
    Fp8RankArgs r[WS_MAX_WORLD];       // x is unused here; scales/out/logits/argmax/row0/k0/ctx as in the decode kernel
    const uint8_t *sfb[WS_MAX_WORLD];  // the prep kernel's scale atoms
};

struct BsSmem {
    int32_t a, b, sf, sfa, sw, cand, rx, bars, misc, total;
};
__host__ __device__ inline BsSmem bs_smem_layout(int nstages, int slabs_per_stage, int a_pitch, int b_pitch, int nslot_max,
                                                 int skb, int mp, int rx_rows) {
    BsSmem s{};
    const int nsl = nstages * slabs_per_stage;
    const int b_bytes = nsl * b_pitch;
    int o = 0;
    s.a = o;    o += nsl * a_pitch;
    s.b = o;    o += b_bytes;
    // an MMA reads 128 rows of its weight slab however many the tile holds: keep 16 KB readable behind the last one
    if (b_bytes < kBsMmaRows * 128) o += kBsMmaRows * 128 - b_bytes;
    s.sf = o;   o += nsl * kBsAtomBytes;
    s.sfa = o;  o += kBsAtomBytes;
    s.sw = o;   o += (int)align_up((int64_t)nslot_max * skb * 4, 16);
    s.cand = o; o += bs_epi_warps(mp) * mp * 8;          // lm_head: per epilogue warp and token (value, index)
    s.rx = o;   o += rx_rows * kBsMmaRows * 4;           // CTA pairs: the partner's partial sums of one tile, [token][row]
    s.bars = o; o += (2 * kMaxStages + kBsMaxAcc + 2) * 8;
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
// D[tmem] (+)= A[smem] * B[smem] with per-32 scales from tensor memory.  The descriptors arrive as
// their 32-bit halves: the upper half is the same for every operand tile, the lower one advances by
// two (32 bytes) per K block, so the single issuing thread spends two adds per MMA on them.
template <bool ACCUMULATE>
__device__ __forceinline__ void umma_bs_ss(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t a_hi, uint32_t b_hi,
                                           uint32_t idesc, uint32_t tsfa, uint32_t tsfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %4};\n\t"
        "setp.ne.b32 p, %8, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], da, db, %5, [%6], [%7], p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(a_hi), "r"(b_hi), "r"(idesc), "r"(tsfa), "r"(tsfb), "n"(ACCUMULATE ? 1 : 0)
        : "memory");
}
// Halves of the 128B-swizzled K-major operand descriptor (see umma_desc): 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
constexpr uint32_t kUmmaDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
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

// ---- distributed shared memory of a CTA pair
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t cta_rank) {  // the same address in CTA `cta_rank` of the cluster
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar) {  // releases this thread's earlier stores to the cluster
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// Wait on an own barrier that the partner CTA arrives on; bounded like mbar_wait.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, uint32_t *status) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((++spins & 63u) == 0u) {
            if (*(volatile uint32_t *)status != 0u) return false;
            if (globaltimer_ns() - t0 > 2000000000ull) break;
        }
    }
    atomicCAS(status, 0u, kStatTimeoutTma | (uint32_t)(-WS_ERR_TIMEOUT));
    return false;
}

template <int THREADS>
__device__ __forceinline__ void bs_epi_bar_n() {  // the epilogue warps
    asm volatile("bar.sync 2, %0;" ::"n"(THREADS) : "memory");
}

// The sequence of stage items of one CTA.  The shard's rows are cut into tiles of tile_rows rows
// (at most 128, the M of the MMA; chosen so that the tiles deal out evenly) and CTA c takes tiles
// [c * T / ncta, (c + 1) * T / ncta) whole, so every output row is a complete dot product inside one
// CTA and nothing is combined across CTAs.  An item is up to SL consecutive K slabs of one tile.
// With CTA pairs (csize = 2) the tiles are dealt out to the pairs and each CTA of a pair walks one
// half of every tile's K slabs; the second CTA hands its sums to the first through the pair's
// distributed shared memory (see the epilogue).
struct BsWalk {
    int t, t1, s, K0, K1, SL;  // tiles [t, t1), slabs [K0, K1) of each
    __device__ __forceinline__ BsWalk(int ntiles, int part, int nparts, int k0, int k1, int sl) : s(k0), K0(k0), K1(k1), SL(sl) {
        t = (int)((int64_t)ntiles * part / nparts);
        t1 = (int)((int64_t)ntiles * (part + 1) / nparts);
        if (k1 <= k0) t1 = t;
    }
    // next item: tile, first slab, slab count; false when the CTA's tiles are used up
    __device__ __forceinline__ bool next(int &tile, int &s0, int &nsl) {
        if (t >= t1) return false;
        tile = t;
        s0 = s;
        nsl = min(SL, K1 - s);
        s += nsl;
        if (s == K1) {
            s = K0;
            ++t;
        }
        return true;
    }
};

template <int MP>
__global__ void __launch_bounds__(bs_threads(MP), 1) fp8_bs_kernel(const __grid_constant__ BsParams p) {
    constexpr int EW = bs_epi_warps(MP), ET = EW * 32;  // epilogue warps / threads
    constexpr int CP = MP * 4 / EW;                      // token columns one epilogue thread holds
    auto bs_epi_bar = [] { bs_epi_bar_n<ET>(); };
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);

    const int vr = blockIdx.y, cta = blockIdx.x, ncta = gridDim.x;
    const Fp8RankArgs &A = p.r[vr];
    const RankCtx &X = A.ctx;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int KS = p.k >> 7;                                // slabs per tile
    // CTA pairs: which half of K is this CTA's, and which pair of how many it belongs to
    uint32_t crank = 0;
    if (p.csize == 2) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
    const int part = p.csize == 2 ? cta >> 1 : cta, nparts = p.csize == 2 ? ncta >> 1 : ncta;
    const int k_lo = (int)crank * KS / p.csize, k_hi = ((int)crank + 1) * KS / p.csize;
    const int SL = p.slabs_per_stage, NS = p.nstages, NB = p.nacc;
    const int ntiles = p.ntiles, TR = p.tile_rows;

    const BsSmem S = bs_smem_layout(NS, SL, p.a_pitch, p.b_pitch, p.nslot_max, p.skb, MP, p.csize == 2 ? p.m : 0);
    float *sw_s = reinterpret_cast<float *>(smem + S.sw);
    uint32_t *misc_s = reinterpret_cast<uint32_t *>(smem + S.misc);
    const uint32_t a0 = smem_u32(smem + S.a), b0 = smem_u32(smem + S.b), sf0 = smem_u32(smem + S.sf);
    // full[s]: the stage's bytes landed.  done[s]: every MMA that reads the stage has completed (ONE
    // tcgen05.commit per stage: a commit stalls the issuing thread for ~160 ns, so it is not spent per
    // slab) -- the producer reads it as "stage free", the epilogue as "this stage's accumulators are
    // ready".  A stage's slabs accumulate into the SL buffers of accumulator group g = item mod NB;
    // accempty[g]: the group has been read back.
    const uint32_t full0 = smem_u32(smem + S.bars), done0 = full0 + kMaxStages * 8;
    const uint32_t accempty0 = done0 + kMaxStages * 8;
    const uint32_t rxfull = accempty0 + kBsMaxAcc * 8, rxempty = rxfull + 8;  // CTA pairs: the partner's sums of a tile have arrived / been read

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(done0 + s * 8, 1);
        }
        for (int b = 0; b < kBsMaxAcc; ++b) mbar_init(accempty0 + b * 8, EW);  // one arrival per epilogue warp
        mbar_init(rxfull, ET);   // every epilogue thread of the partner arrives after its stores
        mbar_init(rxempty, ET);
        mbar_fence_init();
    }
    if (warp == 1) {  // tensor memory: allocated and freed by the same warp
        tmem_alloc(smem_u32(misc_s), (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    if (warp >= 2 && warp < 6) {  // the weight operand's scale atom: 2^0 everywhere (128 threads x 4 bytes)
        uint32_t *sfa = reinterpret_cast<uint32_t *>(smem + S.sfa);
        sfa[tid - 64] = 0x7F7F7F7Fu;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (p.csize == 2) {  // the partner's barriers are initialised before anything is sent to them
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(misc_s);
    // tensor-memory columns: NB groups x SL accumulator buffers of MP columns, then 4 activation-scale
    // columns (one scale atom) per buffer, then the 4 weight-scale columns
    const uint32_t t_sfb0 = tmem_base + (uint32_t)(NB * SL * MP);
    const uint32_t t_sfa = t_sfb0 + (uint32_t)(NB * SL * 4);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------ producer (one thread)
        if (lane == 0) {
            // Weights are static: the first ring's worth streams before the wait on the prep kernel;
            // the activations and their scales follow once it has finished.
            const uint32_t slab_tx = (uint32_t)(TR * 128 + MP * 128 + kBsAtomBytes);
            auto issue_w = [&](int s, int tile, int s0, int nsl) {
                mbar_arrive_expect_tx(full0 + s * 8, (uint32_t)nsl * slab_tx);
                for (int j = 0; j < nsl; ++j)
                    tma_load_2d(a0 + (s * SL + j) * p.a_pitch, &p.tmap_w[vr], (s0 + j) * 128, tile * TR, full0 + s * 8);
            };
            auto issue_x = [&](int s, int s0, int nsl) {
                for (int j = 0; j < nsl; ++j) {
                    tma_load_2d(b0 + (s * SL + j) * p.b_pitch, &p.tmap_x[vr], (s0 + j) * 128, 0, full0 + s * 8);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(sf0 + (s * SL + j) * kBsAtomBytes), "l"(p.sfb[vr] + (size_t)(s0 + j) * kBsAtomBytes),
                                   "r"((uint32_t)kBsAtomBytes), "r"(full0 + s * 8) : "memory");
                }
            };
            int tile, s0, nsl;
            {   // first lap of the ring: weights at once
                BsWalk w(ntiles, part, nparts, k_lo, k_hi, SL);
                for (int item = 0; item < NS && w.next(tile, s0, nsl); ++item) issue_w(item, tile, s0, nsl);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            BsWalk w(ntiles, part, nparts, k_lo, k_hi, SL);
            RingPos st;
            for (int item = 0; w.next(tile, s0, nsl); ++item, st.next(NS)) {
                const int s = st.s;
                if (item >= NS) {
                    if (!mbar_wait(done0 + s * 8, st.ph ^ 1u, X.status)) break;
                    issue_w(s, tile, s0, nsl);
                }
                issue_x(s, s0, nsl);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issue (one thread)
        // A second issuing thread (stage items taken in turn, so that one thread's waits and commit hide
        // behind the other's MMAs) was ~7% faster on one-row steps, but a launch that streamed a
        // [129280, 7168] shard partly out of L2 (weights written just before) then ended in "unspecified
        // launch failure" in most attempts, in a different CTA and stage item each time, and never with
        // one thread; the barrier hand-offs are the same either way, so the cause is not known.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0) {
            tmem_cp_atom(t_sfa, umma_desc(smem_u32(smem + S.sfa), 128, false));
            // Everything the loop needs per MMA is an add away: descriptor halves per stage slot, the
            // four instruction descriptors (one per K block of a slab), ring positions kept incrementally.
            const uint32_t id0 = bs_idesc(MP, 0, 0), id1 = bs_idesc(MP, 0, 1), id2 = bs_idesc(MP, 0, 2), id3 = bs_idesc(MP, 0, 3);
            const uint32_t a_lo0 = umma_desc_lo(a0), b_lo0 = umma_desc_lo(b0);
            const uint32_t a_step = (uint32_t)p.a_pitch >> 4, b_step = (uint32_t)p.b_pitch >> 4;
            const uint64_t sf_desc0 = umma_desc(sf0, 128, false);
            const uint32_t sf_step = (uint32_t)kBsAtomBytes >> 4;
            BsWalk w(ntiles, part, nparts, k_lo, k_hi, SL);
            RingPos st, ag;  // stage ring, accumulator-group ring
            int tile, s0, nsl;
            for (int item = 0; w.next(tile, s0, nsl); ++item, st.next(NS), ag.next(NB)) {
                const int s = st.s, g = ag.s;
                if (!mbar_wait(full0 + s * 8, st.ph, X.status) || !mbar_wait(accempty0 + g * 8, ag.ph ^ 1u, X.status)) break;
                tc_fence_after();
                uint32_t a_lo = a_lo0 + (uint32_t)(s * SL) * a_step, b_lo = b_lo0 + (uint32_t)(s * SL) * b_step;
                uint64_t sf_desc = sf_desc0 + (uint64_t)((uint32_t)(s * SL) * sf_step);
                uint32_t t_acc = tmem_base + (uint32_t)(g * SL * MP), t_sfb = t_sfb0 + (uint32_t)(g * SL * 4);
                for (int j = 0; j < nsl; ++j) {
                    tmem_cp_atom(t_sfb, sf_desc);
                    umma_bs_ss<false>(t_acc, a_lo, b_lo, kUmmaDescHiSw128, kUmmaDescHiSw128, id0, t_sfa, t_sfb);
                    umma_bs_ss<true>(t_acc, a_lo + 2, b_lo + 2, kUmmaDescHiSw128, kUmmaDescHiSw128, id1, t_sfa, t_sfb);
                    umma_bs_ss<true>(t_acc, a_lo + 4, b_lo + 4, kUmmaDescHiSw128, kUmmaDescHiSw128, id2, t_sfa, t_sfb);
                    umma_bs_ss<true>(t_acc, a_lo + 6, b_lo + 6, kUmmaDescHiSw128, kUmmaDescHiSw128, id3, t_sfa, t_sfb);
                    a_lo += a_step; b_lo += b_step; sf_desc += sf_step;
                    t_acc += MP; t_sfb += 4;
                }
                umma_commit(done0 + s * 8);  // the stage may be refilled and its accumulators read
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue warps
        const int et = tid - 64;                     // 0..ET-1
        const int ew = warp - 2;                     // 0..EW-1
        const int quad = warp & 3;                   // TMEM lanes this warp may read: its index modulo 4
        const int rc = quad * 32 + lane;             // row inside the tile = TMEM lane
        const int col0 = (ew >> 2) * CP;             // first token column of this thread
        const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
        const int t_lo = (int)((int64_t)ntiles * part / nparts), t_hi = (int)((int64_t)ntiles * (part + 1) / nparts) - 1;  // this CTA's tiles
        // weight scales of the rows this CTA touches as fp32: sw_s[slot][column].  They are static, so
        // they are fetched before the wait on the predecessor.
        const int64_t kcol0 = A.k0 >> p.bk_shift;
        const int row_lo = t_lo * TR, row_hi = min(p.n, (t_hi + 1) * TR);
        const int64_t srow_lo = (A.row0 + row_lo) >> p.bn_shift;
        const int nslot = row_hi > row_lo ? (int)(((A.row0 + row_hi - 1) >> p.bn_shift) - srow_lo + 1) : 0;
        const int ncols = (int)(((A.k0 + p.k - 1) >> p.bk_shift) - kcol0 + 1);
        for (int i = et; i < nslot * ncols; i += ET) {
            const int sl = i / ncols, c = i - sl * ncols;
            sw_s[sl * p.skb + c] = __ldg(static_cast<const float *>(A.scales) + (srow_lo + sl) * A.scale_ld + kcol0 + c);
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t seq = step_begin(X);
        const uint32_t bank = seq & 1u;
        bs_epi_bar();
        const int kofs = (int)(A.k0 - kcol0 * ((int64_t)1 << p.bk_shift));
        const bool solo = p.mode == kModeAllReduce && p.world == 1;
        const size_t astride = (size_t)p.lay.max_m * p.lay.max_n;
        const int nflag = kMaxCtas + kMaxShared;
        float *cv_s = reinterpret_cast<float *>(smem + S.cand);        // [EW warps][MP]; a warp fills its own columns
        uint32_t *ci_s = reinterpret_cast<uint32_t *>(smem + S.cand) + EW * MP;
        if (p.mode == kModeLmHead)
            for (int i = lane; i < MP; i += 32) { cv_s[ew * MP + i] = -INFINITY; ci_s[ew * MP + i] = 0xFFFFFFFFu; }

        // A finished tile: its rows go to the output or to the peers; of an lm_head tile the candidates are kept.
        auto finalize = [&](const float (&v)[CP], int tile) {  // v[i]: token col0 + i
            const int row = tile * TR + rc;
            const bool mine = rc < TR && row < p.n;
            if (mine) {
                if (solo) {
#pragma unroll
                    for (int i = 0; i < CP; ++i)
                        if (col0 + i < p.m) A.out[(size_t)(col0 + i) * p.n + row] = v[i];
                } else if (p.mode == kModeAllReduce) {
                    // every rank gets the partial sums, or (many rows, many ranks) only the tile's owner
                    const int pr0 = p.owner_reduce ? tile % p.world : 0, pr1 = p.owner_reduce ? pr0 + 1 : p.world;
                    for (int pr = pr0; pr < pr1; ++pr) {
                        uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[pr] + p.lay.slota_off) + ((size_t)bank * p.world + X.rank) * astride;
#pragma unroll
                        for (int i = 0; i < CP; ++i)
                            if (col0 + i < p.m) st_word_sys(dst + (size_t)(col0 + i) * p.n + row, seq, v[i]);
                    }
                }
            }
            if (p.mode == kModeLmHead) {
                // best (value, lowest index) of this warp's rows per token, merged into the warp's running best
                const uint32_t idx = (uint32_t)(A.vocab_row0 + row);
#pragma unroll
                for (int i = 0; i < CP; ++i) {
                    const int t = col0 + i;
                    if (t >= p.m) break;
                    float bv = (mine && v[i] > -INFINITY) ? v[i] : -INFINITY;
                    uint32_t bi = (mine && v[i] > -INFINITY) ? idx : 0xFFFFFFFFu;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                        if (cand_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                    }
                    if (lane == 0 && cand_better(bv, bi, cv_s[ew * MP + t], ci_s[ew * MP + t])) {
                        cv_s[ew * MP + t] = bv;
                        ci_s[ew * MP + t] = bi;
                    }
                }
            }
        };

        BsWalk w(ntiles, part, nparts, k_lo, k_hi, SL);
        RingPos st, ag;  // stage ring, accumulator-group ring
        bool ok = true;
        int tile, s0, nsl, ntile_done = 0;
        float acc[CP];
        const float *swrow = sw_s;
        while (w.next(tile, s0, nsl)) {
            if (s0 == k_lo) {  // a new tile
#pragma unroll
                for (int i = 0; i < CP; ++i) acc[i] = 0.0f;
                const int row = min(tile * TR + min(rc, TR - 1), p.n - 1);
                swrow = sw_s + (int)(((A.row0 + row) >> p.bn_shift) - srow_lo) * p.skb;
            }
            const int g = ag.s;
            if (ok && !mbar_wait(done0 + st.s * 8, st.ph, X.status)) ok = false;
            ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below need the whole warp
            tc_fence_after();
            if (ok) {
                for (int j = 0; j < nsl; ++j) {
                    const float sw = swrow[(kofs + (s0 + j) * 128) >> p.bk_shift];
                    uint32_t r[CP];
                    tmem_ld_cols<CP>(tlane + (uint32_t)((g * SL + j) * MP + col0), r);  // returns once the values are in registers
#pragma unroll
                    for (int i = 0; i < CP; ++i) acc[i] = fmaf(__uint_as_float(r[i]), sw, acc[i]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(accempty0 + g * 8);
            st.next(NS);
            ag.next(NB);
            if (s0 + nsl == k_hi) {  // this CTA's slabs of the tile are done
                if (p.csize == 1) {
                    finalize(acc, tile);
                } else if (crank == 1) {
                    // second CTA of the pair: hand the sums to the first one, into its shared memory
                    if (ntile_done > 0) mbar_wait_cluster(rxempty, (uint32_t)(ntile_done - 1) & 1u, X.status);  // the previous tile's have been read
                    const uint32_t dst = mapa_u32(smem_u32(smem + S.rx) + (uint32_t)rc * 4u, 0u);
#pragma unroll
                    for (int i = 0; i < CP; ++i)
                        if (col0 + i < p.m) st_cluster_f32(dst + (uint32_t)((col0 + i) * kBsMmaRows * 4), acc[i]);
                    mbar_arrive_cluster(mapa_u32(rxfull, 0u));
                } else {
                    // first CTA: K half 0 (own) + K half 1 (the partner's), in that order
                    mbar_wait_cluster(rxfull, (uint32_t)ntile_done & 1u, X.status);
                    const float *rx = reinterpret_cast<const float *>(smem + S.rx) + rc;
#pragma unroll
                    for (int i = 0; i < CP; ++i)
                        if (col0 + i < p.m) acc[i] += rx[(col0 + i) * kBsMmaRows];
                    mbar_arrive_cluster(mapa_u32(rxempty, 1u));
                    finalize(acc, tile);
                }
                ++ntile_done;
            }
        }

        // ---- exchange (the epilogue threads)
        const uint32_t *myflags = solo ? nullptr
                                       : reinterpret_cast<const uint32_t *>(X.sym[X.rank] + p.lay.flags_off) + (size_t)bank * p.world * nflag;
        if (!solo && p.mode == kModeAllReduce) {
            // fold the rows of the tiles this CTA finished, in rank order, as the ranks' words arrive
            const uint64_t *slots = reinterpret_cast<const uint64_t *>(X.sym[X.rank] + p.lay.slota_off) + (size_t)bank * p.world * astride;
            for (int t = t_lo; t <= t_hi && crank == 0; ++t) {  // in a pair the first CTA finished the tiles
                const int row = t * TR + rc;
                if (rc >= TR || row >= p.n) continue;
                // 16 tokens at a time: their words of one rank are all requested before the first is
                // looked at (one memory round trip per batch, not per word); a word that has not
                // arrived yet is then waited for on its own.  Ranks are added in rank order.
                const int tend = min(p.m, col0 + CP);  // this thread's token columns
                // Fold by owners: the sums of tile t are formed on rank t % world only (in rank order, as
                // everywhere) and travel back in that rank's own slot at every peer, so all ranks end up
                // with the same bits and each partial sum crosses the links once instead of world - 1 times.
                const int owner = p.owner_reduce ? t % p.world : X.rank;
                for (int tok0 = col0; tok0 < tend; tok0 += 16) {
                    float sum[16];
                    const int rr0 = owner == X.rank ? 0 : owner, rr1 = owner == X.rank ? p.world : owner + 1;
                    for (int rr = rr0; rr < rr1; ++rr) {
                        const uint64_t *src = slots + rr * astride + (size_t)tok0 * p.n + row;
                        uint64_t w[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (tok0 + i < tend) w[i] = ld_word_sys(src + (size_t)i * p.n);
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (tok0 + i < tend) {
                                const float v = (uint32_t)(w[i] >> 32) == seq
                                                    ? __uint_as_float((uint32_t)w[i])
                                                    : wait_word(src + (size_t)i * p.n, seq, p.timeout_ns, X.status, kStatTimeoutPeerA);
                                sum[i] = rr == rr0 ? v : sum[i] + v;
                            }
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (tok0 + i < tend) A.out[(size_t)(tok0 + i) * p.n + row] = sum[i];
                    if (p.owner_reduce && owner == X.rank)
                        for (int pr = 0; pr < p.world; ++pr) {
                            if (pr == X.rank) continue;
                            uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[pr] + p.lay.slota_off) +
                                            ((size_t)bank * p.world + X.rank) * astride + (size_t)tok0 * p.n + row;
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (tok0 + i < tend) st_word_sys(dst + (size_t)i * p.n, seq, sum[i]);
                        }
                }
            }
        } else if (p.mode == kModeLmHead) {
            // Only the argmax is wanted.  The CTAs of a rank leave their candidates in the rank's own
            // table; the CTA that arrives last merges them into ONE (value, lowest index) per token,
            // sends it to every peer and merges the ranks' candidates: one 64-bit store and one flag
            // per peer and step instead of one per CTA.
            bs_epi_bar();
            uint64_t *table = reinterpret_cast<uint64_t *>(X.sym[X.rank] + p.lay.pairs_off) + (size_t)bank * p.world * kMaxCtas * p.lay.max_m;
            if (et < p.m) {  // token et: the four warps (one per lane quarter) that hold its column
                const int w0 = (et / CP) * 4;
                float bv = cv_s[w0 * MP + et];
                uint32_t bi = ci_s[w0 * MP + et];
                for (int w = w0 + 1; w < w0 + 4; ++w)
                    if (cand_better(cv_s[w * MP + et], ci_s[w * MP + et], bv, bi)) { bv = cv_s[w * MP + et]; bi = ci_s[w * MP + et]; }
                table[((size_t)X.rank * kMaxCtas + cta) * p.lay.max_m + et] = ((uint64_t)__float_as_uint(bv) << 32) | bi;
            }
            volatile uint32_t *last_s = misc_s + 4;
            bs_epi_bar();
            if (et == 0) {
                __threadfence();
                const bool last = atomicAdd(X.counters, 1u) + 1u == (uint32_t)ncta;
                if (last) {
                    X.counters[0] = 0u;  // ready for the next step
                    __threadfence();
                }
                *last_s = last ? 1u : 0u;
            }
            bs_epi_bar();
            if (*last_s) {
                constexpr int kRankRow = kMaxCtas - 1;  // table row of a rank's merged candidate (a rank runs fewer CTAs than that)
                auto merge = [&](int t, int count, auto entry) {  // warp-wide: best of `count` table entries of token t
                    float bv = -INFINITY;
                    uint32_t bi = 0xFFFFFFFFu;
                    for (int i = lane; i < count; i += 32) {
                        const uint64_t pr = ld_volatile_u64(entry(i) + t);
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
                    return ((uint64_t)__float_as_uint(bv) << 32) | bi;
                };
                for (int t = ew; t < p.m; t += EW) {
                    const uint64_t best = merge(t, ncta, [&](int i) { return table + ((size_t)X.rank * kMaxCtas + i) * p.lay.max_m; });
                    if (lane < p.world) {
                        uint64_t *dst = reinterpret_cast<uint64_t *>(X.sym[lane] + p.lay.pairs_off) +
                                        (((size_t)bank * p.world + X.rank) * kMaxCtas + kRankRow) * p.lay.max_m + t;
                        *dst = best;
                    }
                }
                bs_epi_bar();  // the st.release.sys below is cumulative over the stores this barrier ordered
                if (et < p.world) {
                    uint32_t *f = reinterpret_cast<uint32_t *>(X.sym[et] + p.lay.flags_off) + ((size_t)bank * p.world + X.rank) * nflag;
                    st_release_sys(f + kMaxCtas + 1, seq);
                    wait_flag(myflags + (size_t)et * nflag + kMaxCtas + 1, seq, p.timeout_ns, X.status, kStatTimeoutGather);
                }
                bs_epi_bar();
                if (A.argmax != nullptr)
                    for (int t = ew; t < p.m; t += EW) {
                        const uint64_t best = merge(t, p.world, [&](int i) { return table + ((size_t)i * kMaxCtas + kRankRow) * p.lay.max_m; });
                        if (lane == 0) A.argmax[t] = ((uint32_t)best == 0xFFFFFFFFu) ? 0u : (uint32_t)best;
                    }
            }
        }
    }

    // ---- teardown: every TMEM read and MMA has completed once all threads are here
    tc_fence_before();
    __syncthreads();
    if (p.csize == 2) {  // neither CTA of a pair leaves while the other may still write to or signal it
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
    if (p.world > 1 || p.mode == kModeLmHead) step_end(X, step_begin(X), gridDim.x);
    host_done_signal(X, gridDim.x);
}

}  // namespace ws
