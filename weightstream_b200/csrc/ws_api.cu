// Host side of the C ABI declared in include/ws_tp.h: endpoint life cycle, peer
// mapping, argument validation, tensor-map construction and kernel launches.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/ws_tp.h"
#include "ws_device.cuh"
#include "ws_fp8_kernel.cuh"
#include "ws_fp8_bs_kernel.cuh"
#include "ws_misc_kernels.cuh"
#include "ws_moe_kernel.cuh"
#include "ws_moe_gemv_kernel.cuh"
#include "ws_moe_bs_kernel.cuh"

using namespace ws;

struct ws_tp {
    int world = 1, rank = 0, device = 0;
    ws_tp_config_t cfg{};
    SymLayout lay{};
    char *sym = nullptr;                 // this rank's exchange region
    char *peers[WS_MAX_WORLD] = {};      // every rank's region as mapped in this process
    bool opened[WS_MAX_WORLD] = {};      // mapped through an IPC handle (must be closed)
    bool connected = false;
    uint32_t *counters = nullptr;
    uint32_t *status = nullptr;
    uint64_t step = 0, launches = 0;
    int sm_count = 0, ncta = 0;
    uint64_t timeout_ns = 0;
    int split = 1;
    int pdl = 1;         // programmatic dependent launch for the FP8 mma.sync kernel
    int kernel_sel = 0;  // 0: automatic (CUDA cores for 1-2 rows, block-scaled tcgen05 above), 1: mma.sync, 2: tcgen05 whenever the shape fits
    // host-buffer entry points
    cudaStream_t hstream = nullptr;
    void *pin = nullptr;
    size_t pin_bytes = 0;
    void *dev_stage = nullptr;
    size_t dev_stage_bytes = 0;
    // host-buffer FP8 step replayed as one CUDA graph (copy in, kernel(s), copy out, status out)
    struct HostGraph {
        ws_fp8_gemm_args_t key{};
        void *pin = nullptr, *dev = nullptr;
        int kernel_sel = 0, split = 0, pdl = 0;
        uint64_t steps = 0, launches = 0, used = 0;
        cudaGraphExec_t exec = nullptr;
    };
    std::unordered_map<uint64_t, HostGraph> hgraphs;  // keyed by a hash of the argument set
    uint64_t *pin_done = nullptr;       // pinned: {1, device status} once a host-buffer call's last kernel has finished
    uint64_t *host_done_arm = nullptr;  // set while a host-buffer call enqueues: its last kernel reports to this word
    uint64_t hgraph_clock = 0;
    // MoE decode step: routes quantised once per step, pass table, large-m accumulators
    uint8_t *moe_work = nullptr;
    size_t moe_work_bytes = 0;
    float *moe_acc = nullptr;
    size_t moe_acc_bytes = 0;
    // block-scaled tcgen05 step: the step's quantised activations [64][k] and their scale atoms
    int moe_bs = 1;  // 0: the MoE step stays on the CUDA-core decode form
    uint8_t *bs_work = nullptr;
    size_t bs_work_bytes = 0;
    std::string err;
};

namespace {

constexpr int kSmemBudget = 227 * 1024 - 1024;  // opt-in maximum minus alignment slack
constexpr int kHalfSmemBudget = 113 * 1024 - 1024;  // what lets two CTAs share an SM (228 KB, 1 KB reserved per CTA)

ws_status_t fail(ws_tp *tp, ws_status_t code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (tp) tp->err = buf;
    return code;
}

#define WS_CUDA(tp, call)                                                                   \
    do {                                                                                    \
        cudaError_t e_ = (call);                                                            \
        if (e_ != cudaSuccess)                                                              \
            return fail(tp, WS_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_));   \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Row-major byte matrix [rows][row_bytes] with stride `ld` bytes, boxes of 128 bytes x box_rows, 128B swizzle.
ws_status_t make_tmap(ws_tp *tp, CUtensorMap *map, const void *base, uint64_t rows, uint64_t row_bytes,
                      uint64_t ld, uint32_t box_rows = kGroupRows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(tp, WS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld & 15))
        return fail(tp, WS_ERR_INVALID, "weight base and row stride must be multiples of 16 bytes");
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {ld};
    cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(tp, WS_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return WS_OK;
}

// Expert slab [experts][rows][k] of packed 4-bit codes (row stride k/2 bytes), boxes of 128 codes x
// box_rows x 1 expert; the copy unpacks 16 codes (8 bytes) into 16 bytes of shared memory, the form
// tcgen05.mma.kind::mxf8f6f4 reads 4-bit operands in; 128B swizzle.
ws_status_t make_tmap_fp4(ws_tp *tp, CUtensorMap *map, const void *base, uint64_t experts, uint64_t rows, uint64_t k,
                          uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(tp, WS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 31) || (k & 255))
        return fail(tp, WS_ERR_INVALID, "expert slab must be 32-byte aligned with k a multiple of 256");
    cuuint64_t dims[3] = {k, rows, experts};
    cuuint64_t strides[2] = {k / 2, rows * (k / 2)};
    cuuint32_t box[3] = {128, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(tp, WS_ERR_CUDA, "cuTensorMapEncodeTiled (4-bit) failed (%d)", (int)r);
    return WS_OK;
}

// Row granularity of the ragged share of leftover rows: small when each CTA gets a row or two
// (balance matters, few boxes), larger when it gets many (fewer, bigger TMA boxes).
int ragged_granularity(int n, int ncta) {
    const int Gm = n / kGroupRows / ncta;
    const int L = n - Gm * ncta * kGroupRows;
    const int per = L / ncta;  // whole rows per CTA
    return per >= 8 ? 4 : per >= 4 ? 2 : 1;
}

// Text for a non-zero device status word (detail code in the high byte, -WS_ERR_* in the low byte).
std::string describe_status(uint32_t st, uint64_t timeout_ns) {
    const uint32_t where = st >> 24;
    char buf[256];
    if (where == (kStatRunAhead >> 24)) {
        snprintf(buf, sizeof buf, "collective out of sequence: a peer's partial carries a later step than this rank's; "
                                  "fail-stop, results invalid");
    } else {
        const char *what = where == 1   ? "a peer CTA's partial"
                           : where == 3 ? "a weight tile (TMA)"
                           : where == 4 ? "the gather of every rank"
                                        : "an unknown event";
        snprintf(buf, sizeof buf, "wait for %s timed out after %llu ms; fail-stop, results invalid", what,
                 (unsigned long long)(timeout_ns / 1000000ull));
    }
    return buf;
}

RankCtx make_ctx(const ws_tp *tp) {
    RankCtx c{};
    for (int i = 0; i < WS_MAX_WORLD; ++i) c.sym[i] = tp->peers[i];
    c.counters = tp->counters;
    c.status = tp->status;
    c.step_ctr = tp->counters + kMaxShared + 2;
    c.rank = tp->rank;
    c.host_done = nullptr;
    return c;
}

template <typename K>
ws_status_t set_smem(ws_tp *tp, K kernel) {
    WS_CUDA(tp, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    return WS_OK;
}

template <typename P>
ws_status_t launch(ws_tp *tp, void (*kernel)(P), const P &params, int ncta, int nvr, int threads, size_t smem,
                   cudaStream_t stream, bool pdl = false, bool waits_on_peers = true, int cluster = 1) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)ncta, (unsigned)nvr, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.numAttrs = 1;
    if (cluster > 1) {  // CTA pairs sharing distributed shared memory (never together with virtual ranks)
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = (unsigned)cluster;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    if (nvr > 1 && waits_on_peers) {
        // Virtual ranks sharing one device wait on one another inside the kernel: they must be
        // co-resident, which a cooperative launch guarantees (or refuses).
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
    } else {
        // Programmatic dependent launch: the kernel may start while its predecessor on the stream
        // is still finishing; it streams (static) weights at once and executes griddepcontrol.wait
        // before it touches anything the predecessor may have written.
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    }
    cfg.attrs = attr;
    WS_CUDA(tp, cudaLaunchKernelEx(&cfg, kernel, params));
    tp->launches++;
    return WS_OK;
}

// Common checks for a group call; returns the CTA count to use.
ws_status_t group_prelude(ws_tp *const *ranks, int n, int *ncta, bool *same_device) {
    if (!ranks || n < 1 || n > WS_MAX_WORLD) return WS_ERR_INVALID;
    ws_tp *t0 = ranks[0];
    if (!t0) return WS_ERR_INVALID;
    bool same = true;
    for (int i = 0; i < n; ++i) {
        ws_tp *t = ranks[i];
        if (!t) return fail(t0, WS_ERR_INVALID, "null endpoint %d", i);
        if (t->world > 1 && !t->connected) return fail(t0, WS_ERR_INVALID, "endpoint %d is not connected", i);
        if (t->step != t0->step) return fail(t0, WS_ERR_SEQUENCE, "endpoints disagree on the step count");
        if (t->device != t0->device) same = false;
    }
    if (n > 1) {
        if (n != t0->world) return fail(t0, WS_ERR_INVALID, "a group call needs all %d ranks", t0->world);
        for (int i = 0; i < n; ++i)
            if (ranks[i]->rank != i) return fail(t0, WS_ERR_INVALID, "ranks[] must be ordered by rank");
    }
    if (!same)  // kernels that wait on one another must not be separate launches on one GPU
        for (int i = 0; i < n; ++i)
            for (int j = i + 1; j < n; ++j)
                if (ranks[i]->device == ranks[j]->device)
                    return fail(t0, WS_ERR_UNSUPPORTED, "ranks %d and %d share device %d while others do not", i, j,
                                ranks[i]->device);
    int c = t0->ncta;
    if (n > 1 && same) c = std::min(c, t0->sm_count / n);
    if (c < 1) return fail(t0, WS_ERR_CAPACITY, "no CTAs left per virtual rank");
    *ncta = c;
    *same_device = same;
    return WS_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------
extern "C" {

const char *ws_version(void) { return "weightstream_b200 0.1 (sm_100a)"; }

ws_status_t ws_tp_create(int32_t world, int32_t rank, int32_t device, const ws_tp_config_t *cfg, ws_tp_t **out) {
    if (!out || !cfg) return WS_ERR_INVALID;
    *out = nullptr;
    if (!(world == 1 || world == 2 || world == 4 || world == 8) || rank < 0 || rank >= world) return WS_ERR_INVALID;
    if (cfg->max_m < 1 || cfg->max_n < 16 || cfg->max_vocab < 0) return WS_ERR_INVALID;
    ws_tp *tp = new ws_tp();
    tp->world = world;
    tp->rank = rank;
    tp->device = device;
    tp->cfg = *cfg;
    tp->timeout_ns = (uint64_t)(cfg->wait_ms > 0 ? cfg->wait_ms : 2000) * 1000000ull;
    auto bail = [&](ws_status_t s) {
        ws_tp_destroy(tp);
        return s;
    };
    if (cudaSetDevice(device) != cudaSuccess) return bail(WS_ERR_CUDA);
    if (cudaDeviceGetAttribute(&tp->sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        return bail(WS_ERR_CUDA);
    tp->ncta = cfg->num_ctas > 0 ? std::min(cfg->num_ctas, tp->sm_count) : tp->sm_count;
    if (tp->ncta > kMaxCtas) tp->ncta = kMaxCtas;
    tp->lay = make_layout(world, cfg->max_m, cfg->max_n, cfg->max_vocab);
    if (cudaMalloc(&tp->sym, (size_t)tp->lay.total) != cudaSuccess) return bail(WS_ERR_CUDA);
    if (cudaMemset(tp->sym, 0, (size_t)tp->lay.total) != cudaSuccess) return bail(WS_ERR_CUDA);
    if (cudaMalloc(&tp->counters, (kMaxShared + 8) * sizeof(uint32_t)) != cudaSuccess) return bail(WS_ERR_CUDA);
    if (cudaMemset(tp->counters, 0, (kMaxShared + 8) * sizeof(uint32_t)) != cudaSuccess) return bail(WS_ERR_CUDA);
    tp->status = tp->counters + kMaxShared;
    if (cudaStreamCreateWithFlags(&tp->hstream, cudaStreamNonBlocking) != cudaSuccess) return bail(WS_ERR_CUDA);
    if (cudaDeviceSynchronize() != cudaSuccess) return bail(WS_ERR_CUDA);
    tp->peers[rank] = tp->sym;
    if (world == 1) tp->connected = true;
    if (set_smem(tp, moe_gemv_kernel) != WS_OK || set_smem(tp, fp8_rowpar_kernel<0>) != WS_OK || set_smem(tp, fp8_rowpar_kernel<1>) != WS_OK ||
        set_smem(tp, fp8_rowpar_kernel<2>) != WS_OK || set_smem(tp, moe_down_kernel) != WS_OK ||
        set_smem(tp, fp8_bs_kernel<16>) != WS_OK || set_smem(tp, fp8_bs_kernel<32>) != WS_OK ||
        set_smem(tp, fp8_bs_kernel<64>) != WS_OK || set_smem(tp, fp8_bs_kernel<128>) != WS_OK || set_smem(tp, moe_bs_kernel) != WS_OK ||
        cudaFuncSetAttribute(moe_bs_prep_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess ||
        // The prep kernel uses no shared memory, but a main-kernel CTA (which needs almost all of an SM's)
        // cannot move onto an SM whose L1/shared split must first change, and that has to wait for the prep
        // blocks there to leave: measured 2.5-4.5 us of late CTAs.  With the same preference nothing changes.
        cudaFuncSetAttribute(act_prep_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess ||
        cudaFuncSetAttribute(stage_in_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
        return bail(WS_ERR_CUDA);
    *out = tp;
    return WS_OK;
}

ws_status_t ws_tp_destroy(ws_tp_t *tp) {
    if (!tp) return WS_OK;
    cudaSetDevice(tp->device);
    for (int i = 0; i < WS_MAX_WORLD; ++i)
        if (tp->opened[i] && tp->peers[i]) cudaIpcCloseMemHandle(tp->peers[i]);
    if (tp->hstream) cudaStreamDestroy(tp->hstream);
    if (tp->pin) cudaFreeHost(tp->pin);
    if (tp->dev_stage) cudaFree(tp->dev_stage);
    for (auto &g : tp->hgraphs)
        if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
    if (tp->pin_done) cudaFreeHost(tp->pin_done);
    if (tp->moe_work) cudaFree(tp->moe_work);
    if (tp->moe_acc) cudaFree(tp->moe_acc);
    if (tp->bs_work) cudaFree(tp->bs_work);
    if (tp->sym) cudaFree(tp->sym);
    if (tp->counters) cudaFree(tp->counters);
    delete tp;
    return WS_OK;
}

ws_status_t ws_tp_export_handle(ws_tp_t *tp, ws_ipc_handle_t *out) {
    if (!tp || !out) return WS_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) + 16 <= WS_IPC_HANDLE_BYTES, "handle does not fit");
    memset(out, 0, sizeof *out);
    WS_CUDA(tp, cudaSetDevice(tp->device));
    cudaIpcMemHandle_t h;
    WS_CUDA(tp, cudaIpcGetMemHandle(&h, tp->sym));
    memcpy(out->bytes, &h, sizeof h);
    int64_t total = tp->lay.total;
    int32_t meta[2] = {tp->world, tp->rank};
    memcpy(out->bytes + sizeof h, &total, 8);
    memcpy(out->bytes + sizeof h + 8, meta, 8);
    return WS_OK;
}

ws_status_t ws_tp_connect_ipc(ws_tp_t *tp, const ws_ipc_handle_t *handles, int32_t n) {
    if (!tp || !handles || n != tp->world) return WS_ERR_INVALID;
    WS_CUDA(tp, cudaSetDevice(tp->device));
    for (int r = 0; r < n; ++r) {
        cudaIpcMemHandle_t h;
        int64_t total;
        int32_t meta[2];
        memcpy(&h, handles[r].bytes, sizeof h);
        memcpy(&total, handles[r].bytes + sizeof h, 8);
        memcpy(meta, handles[r].bytes + sizeof h + 8, 8);
        if (total != tp->lay.total || meta[0] != tp->world || meta[1] != r)
            return fail(tp, WS_ERR_INVALID, "handle %d describes a different group (world/rank/layout)", r);
        if (r == tp->rank) continue;
        void *p = nullptr;
        WS_CUDA(tp, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        tp->peers[r] = static_cast<char *>(p);
        tp->opened[r] = true;
    }
    tp->connected = true;
    return WS_OK;
}

ws_status_t ws_tp_connect_local(ws_tp_t *const *ranks, int32_t n) {
    if (!ranks || n < 1 || n > WS_MAX_WORLD) return WS_ERR_INVALID;
    for (int i = 0; i < n; ++i)
        if (!ranks[i] || ranks[i]->world != n || ranks[i]->rank != i || ranks[i]->lay.total != ranks[0]->lay.total)
            return fail(ranks[0], WS_ERR_INVALID, "ranks[] must hold the n endpoints of one group, ordered by rank");
    for (int i = 0; i < n; ++i) {
        ws_tp *a = ranks[i];
        WS_CUDA(a, cudaSetDevice(a->device));
        for (int j = 0; j < n; ++j) {
            ws_tp *b = ranks[j];
            if (a->device != b->device) {
                int can = 0;
                WS_CUDA(a, cudaDeviceCanAccessPeer(&can, a->device, b->device));
                if (!can) return fail(a, WS_ERR_UNSUPPORTED, "device %d cannot map device %d", a->device, b->device);
                cudaError_t e = cudaDeviceEnablePeerAccess(b->device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
                else if (e != cudaSuccess) return fail(a, WS_ERR_CUDA, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
            }
            a->peers[j] = b->sym;
        }
        a->connected = true;
    }
    return WS_OK;
}

ws_status_t ws_tp_check(ws_tp_t *tp, void *stream) {
    if (!tp) return WS_ERR_INVALID;
    WS_CUDA(tp, cudaSetDevice(tp->device));
    WS_CUDA(tp, cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    uint32_t st = 0;
    WS_CUDA(tp, cudaMemcpy(&st, tp->status, 4, cudaMemcpyDeviceToHost));
    if (st == 0) return WS_OK;
    WS_CUDA(tp, cudaMemset(tp->status, 0, 4));
    return fail(tp, -(ws_status_t)(st & 0xFFu), "rank %d: %s", tp->rank, describe_status(st, tp->timeout_ns).c_str());
}

const char *ws_tp_last_error(ws_tp_t *tp) { return tp ? tp->err.c_str() : "null endpoint"; }

ws_status_t ws_tp_stats(ws_tp_t *tp, uint64_t *steps, uint64_t *launches) {
    if (!tp) return WS_ERR_INVALID;
    if (steps) *steps = tp->step;
    if (launches) *launches = tp->launches;
    return WS_OK;
}

int32_t ws_tp_num_ctas(ws_tp_t *tp) { return tp ? tp->ncta : 0; }

// ------------------------------------------------------------------------------ FP8 GEMM
static ws_status_t validate_fp8(ws_tp *tp, const ws_fp8_gemm_args_t &a, bool lm_head) {
    if (!a.x || !a.w || !a.scales) return fail(tp, WS_ERR_INVALID, "null x / w / scales");
    if (a.m < 1 || a.n < 16 || a.k < 32) return fail(tp, WS_ERR_INVALID, "bad shape m=%d n=%d k=%d", a.m, a.n, a.k);
    if (a.k % 32) return fail(tp, WS_ERR_INVALID, "k=%d is not a multiple of the 32-wide activation block", a.k);
    if (a.n % 16) return fail(tp, WS_ERR_INVALID, "n=%d is not a multiple of 16", a.n);
    if (a.x_dtype != WS_ACT_BF16 && a.x_dtype != WS_ACT_F32) return fail(tp, WS_ERR_INVALID, "bad x_dtype");
    const int xa = a.x_dtype == WS_ACT_BF16 ? 8 : 4;
    if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (a.ldx % xa) || a.ldx < a.k)
        return fail(tp, WS_ERR_INVALID, "x must be 16-byte aligned with ldx >= k and ldx a multiple of %d", xa);
    if (a.scale_kind != WS_SCALE_UE8M0 && a.scale_kind != WS_SCALE_F32) return fail(tp, WS_ERR_INVALID, "bad scale_kind");
    if (a.block_n < 16 || (a.block_n & (a.block_n - 1)) || a.block_k < 32 || (a.block_k & (a.block_k - 1)))
        return fail(tp, WS_ERR_INVALID, "scale block %dx%d: block_n must be a power of two >= 16, block_k >= 32", a.block_n, a.block_k);
    if (a.row0 < 0 || a.k0 < 0 || a.row0 % 16) return fail(tp, WS_ERR_INVALID, "row0 must be a non-negative multiple of 16");
    if ((a.k0 + a.k - 1) / a.block_k >= a.scale_ld) return fail(tp, WS_ERR_INVALID, "k slice reaches past scale_ld");
    if (a.ldw < a.k) return fail(tp, WS_ERR_INVALID, "ldw < k");
    if (!lm_head && !a.out) return fail(tp, WS_ERR_INVALID, "null out");
    if (a.k > 32768) return fail(tp, WS_ERR_CAPACITY, "k=%d exceeds the decode kernel's shared-memory plan", a.k);
    return WS_OK;
}

// Plan of the block-scaled tcgen05 path for one fused step; ok = false when the shape does not fit it
// (it needs fp32 weight scales whose K blocks are whole 128-wide slabs, and k a multiple of 128).
struct BsPlan {
    bool ok;
    int mp, tile_rows, ntiles, a_pitch, b_pitch, slabs_per_stage, nstages, nslot_max, nacc;
    int csize;  // 2: CTA pairs share a tile, each CTA streams half of K (tiles of a lone CTA would fill under half of the MMA's rows)
    int ncta;   // CTAs the plan is for (even with pairs)
    int tmem_cols;  // tensor-memory columns the CTA allocates (a power of two)
    size_t smem;
};
static BsPlan bs_plan(const ws_fp8_gemm_args_t &a, int mt, int skb, int ncta, bool pairs_allowed) {
    BsPlan u{};
    if (a.scale_kind != WS_SCALE_F32 || a.block_k % 128 || a.k % 128 || mt > kBsMaxTokens) return u;
    u.mp = mt <= 16 ? 16 : mt <= 32 ? 32 : mt <= 64 ? 64 : 128;
    // tiles of equal height that deal out evenly: a CTA's share of the rows, cut into as few pieces
    // of at most 128 rows as possible
    const int kslabs = a.k / 128;
    // The tensor pipe spends the same time on an MMA however few of its 128 rows are real.  When a
    // CTA's share of the rows fills under half of them, two CTAs share a tile and split K instead.
    u.csize = (pairs_allowed && ncta >= 2 && kslabs >= 2 && (a.n + ncta - 1) / ncta <= kBsMmaRows / 2) ? 2 : 1;
    u.ncta = u.csize == 2 ? ncta & ~1 : ncta;
    const int nparts = u.ncta / u.csize;
    const int crmax = (a.n + nparts - 1) / nparts;
    const int pieces = (crmax + kBsMmaRows - 1) / kBsMmaRows;
    u.tile_rows = (crmax + pieces - 1) / pieces;
    u.ntiles = (a.n + u.tile_rows - 1) / u.tile_rows;
    const int tiles_per_cta = (u.ntiles + nparts - 1) / nparts;
    u.a_pitch = (u.tile_rows + 7) / 8 * 8 * 128;
    u.b_pitch = u.mp * 128;
    const int slab_bytes = u.a_pitch + u.b_pitch + kBsAtomBytes;
    // slabs per stage: one MMA commit (a ~160 ns stall of the issuing thread) per stage, so several
    // slabs share it; bounded by the stage size and by tensor memory (each slab has its own
    // accumulator buffer: groups x slabs x (mp + 4) + 8 columns of 512, at least two groups)
    u.nslot_max = (tiles_per_cta * u.tile_rows) / a.block_n + 2;
    const int rx_rows = u.csize == 2 ? mt : 0;
    // Half an SM (shared memory and tensor memory) when the tokens are few and the CTA's whole share of
    // the weights fits such a ring (TP-8 shards): the next step's CTA is then resident beside this one
    // (one CTA per SM and step) and loads all of its weights under this step's exchange and exit.
    // Measured on B200, K/rank 1024, 8 rows: 7.7 us per step against 10.6.  Larger shares lose more to
    // the shallower ring than they gain (K/rank 8192: 19.3 against 17.8 us).
    const bool small = u.mp == 16 && (int64_t)a.n * a.k / u.ncta * u.csize <= ((int64_t)2 << 20);
    for (int half = small ? 1 : 0; half >= 0; --half) {
        const int budget = half ? kHalfSmemBudget : kSmemBudget, tmem = half ? 256 : 512;
        const int stage_target = half ? 32 * 1024 : 56 * 1024;
        u.slabs_per_stage = std::max(1, std::min({4, stage_target / slab_bytes, (tmem - 8) / (2 * (u.mp + 4)), kslabs}));
        u.nacc = std::min((int)kBsMaxAcc, (tmem - 8) / (u.slabs_per_stage * (u.mp + 4)));
        int ns = kMaxStages;  // the most stages whose layout fits
        while (ns >= 2 && bs_smem_layout(ns, u.slabs_per_stage, u.a_pitch, u.b_pitch, u.nslot_max, skb, u.mp, rx_rows).total + 1024 > budget) --ns;
        const int items = tiles_per_cta * ((kslabs / u.csize + u.slabs_per_stage - 1) / u.slabs_per_stage);
        ns = std::min(ns, std::min((int)kMaxStages, std::max(2, items)));
        u.nstages = ns;
        // the epilogue and the producer wait on the same per-stage barrier: the MMA thread must not get a
        // whole lap of the stage ring ahead of the epilogue, which holds when groups <= stages
        u.nacc = std::max(1, std::min(u.nacc, ns));
        u.ok = ns >= 2;
        if (!u.ok || (half && items > ns)) continue;  // half an SM only when the CTA's whole share of the weights fits the ring
        u.smem = (size_t)bs_smem_layout(ns, u.slabs_per_stage, u.a_pitch, u.b_pitch, u.nslot_max, skb, u.mp, rx_rows).total + 1024;
        int cols = 32;
        while (cols < u.nacc * u.slabs_per_stage * (u.mp + 4) + 4) cols *= 2;
        u.tmem_cols = half ? std::min(cols, 256) : 512;
        break;
    }
    return u;
}

static ws_status_t ensure_bs_scratch(ws_tp *tp, size_t bytes) {
    WS_CUDA(tp, cudaSetDevice(tp->device));
    if (bytes > tp->bs_work_bytes) {
        // graphs of earlier host-buffer calls hold the old buffer's address: they go with it
        for (auto &g : tp->hgraphs)
            if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
        tp->hgraphs.clear();
        if (tp->bs_work) cudaFree(tp->bs_work);
        tp->bs_work = nullptr;
        tp->bs_work_bytes = 0;
        WS_CUDA(tp, cudaMalloc(&tp->bs_work, bytes));
        WS_CUDA(tp, cudaMemset(tp->bs_work, 0, bytes));
        tp->bs_work_bytes = bytes;
    }
    return WS_OK;
}

// A tensor map over a row-major byte matrix with boxes of 128 bytes x box_rows, 128B swizzle (see make_tmap).
// One fused step over at most 64 activation rows on the block-scaled tcgen05 path: the prep
// kernel (activation quantisation once per step) followed by the persistent MMA kernel.
static ws_status_t bs_step(ws_tp *const *ranks, int n, const ws_fp8_gemm_args_t *args, const ws_lm_head_args_t *lm,
                           int m0, int mt, void *const *streams, int ncta, bool same_device, const BsPlan &u, int skb, bool last) {
    ws_tp *t0 = ranks[0];
    const ws_fp8_gemm_args_t &a0 = lm ? lm[0].g : args[0];
    BsParams p{};
    p.m = mt; p.mp = u.mp; p.n = a0.n; p.k = a0.k; p.world = t0->world;
    for (p.bk_shift = 0; (1 << p.bk_shift) < a0.block_k; ++p.bk_shift) {}
    for (p.bn_shift = 0; (1 << p.bn_shift) < a0.block_n; ++p.bn_shift) {}
    p.mode = lm ? kModeLmHead : kModeAllReduce;
    p.vocab = lm ? lm[0].vocab : 0;
    p.tile_rows = u.tile_rows; p.ntiles = u.ntiles; p.a_pitch = u.a_pitch; p.b_pitch = u.b_pitch;
    p.slabs_per_stage = u.slabs_per_stage; p.nstages = u.nstages; p.nslot_max = u.nslot_max; p.skb = skb; p.nacc = u.nacc;
    p.csize = u.csize;
    p.tmem_cols = u.tmem_cols;
    // 32 rows and more on four ranks and more: all-to-all of every partial sum costs more link time than the second hop
    p.owner_reduce = (t0->world >= 4 && u.mp >= 32) ? 1 : 0;
    ncta = u.ncta;
    p.timeout_ns = t0->timeout_ns;
    p.lay = t0->lay;
    ActPrepParams q{};
    q.m = mt; q.mp = u.mp; q.k = a0.k; q.x_dtype = a0.x_dtype;
    // scratch of one endpoint: quantised activations and their scale atoms
    const size_t xq_bytes = align_up((int64_t)kBsMaxTokens * a0.k, 256), sf_bytes = (size_t)(a0.k / 128) * kBsAtomBytes;

    for (int i = 0; i < n; ++i) {
        ws_tp *t = ranks[i];
        const ws_fp8_gemm_args_t &a = lm ? lm[i].g : args[i];
        ws_status_t s = ensure_bs_scratch(t, xq_bytes + sf_bytes);
        if (s == WS_OK) s = make_tmap(t, &p.tmap_w[i], a.w, (uint64_t)a.n, (uint64_t)a.k, (uint64_t)a.ldw, (uint32_t)u.tile_rows);
        uint8_t *const xq = t->bs_work;
        if (s == WS_OK) s = make_tmap(t, &p.tmap_x[i], xq, (uint64_t)u.mp, (uint64_t)a.k, (uint64_t)a.k, (uint32_t)u.mp);
        if (s != WS_OK) { t0->err = t->err; return s; }
        Fp8RankArgs &r = p.r[i];
        const size_t xes = a.x_dtype == WS_ACT_BF16 ? 2 : 4;
        r.x = nullptr;
        r.scales = a.scales;
        r.out = lm ? nullptr : a.out + (size_t)m0 * a.n;
        r.logits = nullptr;
        r.argmax = lm && lm[i].argmax ? lm[i].argmax + m0 : nullptr;
        r.ldx = a.ldx; r.scale_ld = a.scale_ld; r.row0 = a.row0; r.k0 = a.k0;
        r.vocab_row0 = lm ? lm[i].vocab_row0 : 0;
        r.ctx = make_ctx(t);
        if (last) r.ctx.host_done = t->host_done_arm;
        p.sfb[i] = xq + xq_bytes;
        q.r[i].x = static_cast<const char *>(a.x) + (size_t)m0 * a.ldx * xes;
        q.r[i].xq = xq;
        q.r[i].sfb = xq + xq_bytes;
        q.r[i].ldx = a.ldx;
    }
    for (int i = 0; i < n; ++i) ranks[i]->step++;
    void (*const kernel)(BsParams) = u.mp == 16 ? fp8_bs_kernel<16> : u.mp == 32 ? fp8_bs_kernel<32>
                                     : u.mp == 64 ? fp8_bs_kernel<64> : fp8_bs_kernel<128>;
    const int prep_blocks = (int)(((int64_t)u.mp * (a0.k / 8) + 255) / 256);
    if (same_device) {
        WS_CUDA(t0, cudaSetDevice(t0->device));
        cudaStream_t cs = static_cast<cudaStream_t>(streams ? streams[0] : nullptr);
        ws_status_t s = launch(t0, act_prep_kernel, q, prep_blocks, n, 256, 0, cs, t0->pdl != 0, false);
        if (s != WS_OK) return s;
        return launch(t0, kernel, p, ncta, n, bs_threads(u.mp), u.smem, cs, t0->pdl != 0, true, u.csize);
    }
    for (int i = 0; i < n; ++i) {
        BsParams pi = p;
        pi.r[0] = p.r[i];
        pi.tmap_w[0] = p.tmap_w[i];
        pi.tmap_x[0] = p.tmap_x[i];
        pi.sfb[0] = p.sfb[i];
        ActPrepParams qi = q;
        qi.r[0] = q.r[i];
        WS_CUDA(ranks[i], cudaSetDevice(ranks[i]->device));
        cudaStream_t cs = static_cast<cudaStream_t>(streams ? streams[i] : nullptr);
        ws_status_t s = launch(ranks[i], act_prep_kernel, qi, prep_blocks, 1, 256, 0, cs, t0->pdl != 0, false);
        if (s == WS_OK) s = launch(ranks[i], kernel, pi, ncta, 1, bs_threads(u.mp), u.smem, cs, t0->pdl != 0, true, u.csize);
        if (s != WS_OK) { t0->err = ranks[i]->err; return s; }
    }
    return WS_OK;
}

// Whether rows [.., +mt) of this step go to the block-scaled tcgen05 path: always when the caller
// selected it; by default from three rows up, and for one or two rows when the shard is large enough
// for its streaming rate to outweigh the second launch (measured on B200, M=1: 927 MB 153 against
// 208 us on CUDA cores; 58.7 MB 17.7 against 17.2 us, 14.7 MB 8.8 against 6.8 us, 7.3 MB 12.8 against 5.9 us).
// A step that also gathers the logits stays on the CUDA-core kernel: the tensor-memory kernel leaves
// only the argmax candidates (the decode loop's form of the call).
static bool bs_wanted(const ws_tp *t0, int mt, const ws_fp8_gemm_args_t &a, bool gathers_logits, bool lm_head = false) {
    if (gathers_logits) return false;
    if (t0->kernel_sel == 2) return true;
    if (t0->kernel_sel != 0) return false;
    // an argmax-only lm_head step also saves the exchange of one candidate per CTA (this kernel sends one per rank)
    // two rows: the CUDA-core kernel needs 23 us for a 58.7 MB shard, this one 17.8 (it is the same for 2 to 8 rows)
    if (mt == 2 && (int64_t)a.n * a.k >= ((int64_t)32 << 20)) return true;
    return mt >= 3 || (int64_t)a.n * a.k >= ((int64_t)(lm_head ? 32 : 128) << 20);
}

// Activation rows the next launch takes: up to 64 when their quantised copies fit in shared
// memory beside at least three weight stages (the weights are then streamed once for all of
// them), else 8.
static int fp8_rows_per_launch(const ws_tp *t0, const ws_fp8_gemm_args_t &a, int ncta, int rem, bool gathers_logits, bool lm_head = false) {
    {   // the tensor-memory path streams the weights once for up to 64 rows
        const int mt = std::min(rem, (int)kBsMaxTokens);
        const int skb = (int)((a.k0 + a.k - 1) / a.block_k - a.k0 / a.block_k + 1);
        if (bs_wanted(t0, mt, a, gathers_logits, lm_head) && bs_plan(a, mt, skb, ncta, false).ok) return mt;
    }
    if (rem <= 8) return rem;
    const int kbox = (a.k + 127) / 128;
    const int Gm = a.n / kGroupRows / ncta;
    const int skb = (int)((a.k0 + a.k - 1) / a.block_k - a.k0 / a.block_k + 1);
    for (int mp = std::min(64, (rem + 7) / 8 * 8); mp > 8; mp -= 8) {
        const int m = std::min(rem, mp);
        const Fp8Smem fixed = fp8_smem_layout(0, kbox, mp, (Gm * kGroupRows) / a.block_n + 4, skb, m, (Gm + 2) * kGroupRows, 0);
        if ((kSmemBudget - fixed.total) / (fp8_stage_boxes(kbox) * kBoxBytes) >= 3) return m;
    }
    return 8;
}

// One fused step over the activation rows [m0, m0 + mt) (mt from fp8_rows_per_launch).
static ws_status_t fp8_step(ws_tp *const *ranks, int n, const ws_fp8_gemm_args_t *args, const ws_lm_head_args_t *lm,
                            int m0, int mt, void *const *streams, int ncta, bool same_device, bool last) {
    ws_tp *t0 = ranks[0];
    const ws_fp8_gemm_args_t &a0 = lm ? lm[0].g : args[0];
    bool gathers_logits = false;
    for (int i = 0; lm && i < n; ++i) gathers_logits |= lm[i].logits != nullptr;
    if (bs_wanted(t0, mt, a0, gathers_logits, lm != nullptr)) {  // tensor-memory path whenever the shape fits it
        int64_t skb_u = 1;
        for (int i = 0; i < n; ++i) {
            const ws_fp8_gemm_args_t &a = lm ? lm[i].g : args[i];
            skb_u = std::max<int64_t>(skb_u, (a.k0 + a.k - 1) / a.block_k - a.k0 / a.block_k + 1);
        }
        const BsPlan u = bs_plan(a0, mt, (int)skb_u, ncta, n == 1);  // CTA pairs need a cluster launch, virtual ranks a cooperative one
        if (u.ok) return bs_step(ranks, n, args, lm, m0, mt, streams, ncta, same_device, u, (int)skb_u, last);
    }
    Fp8Params p{};
    p.m = mt; p.n = a0.n; p.k = a0.k; p.x_dtype = a0.x_dtype; p.scale_kind = a0.scale_kind;
    p.bn = a0.block_n; p.bk = a0.block_k; p.world = t0->world;
    for (p.bk_shift = 0; (1 << p.bk_shift) < p.bk; ++p.bk_shift) {}
    for (p.bn_shift = 0; (1 << p.bn_shift) < p.bn; ++p.bn_shift) {}
    p.mode = lm ? kModeLmHead : kModeAllReduce;
    p.vocab = lm ? lm[0].vocab : 0;
    p.gather_logits = 0;
    p.mp = mt <= 1 ? 1 : mt <= 2 ? 2 : mt <= 4 ? 4 : (mt + 7) / 8 * 8;
    p.timeout_ns = t0->timeout_ns;
    p.lay = t0->lay;
    const int kbox = (p.k + 127) / 128;
    const int Gm = p.n / kGroupRows / ncta;
    int64_t skb = 1;
    for (int i = 0; i < n; ++i) {
        const ws_fp8_gemm_args_t &a = lm ? lm[i].g : args[i];
        skb = std::max<int64_t>(skb, (a.k0 + a.k - 1) / a.block_k - a.k0 / a.block_k + 1);
        if (lm && lm[i].logits) p.gather_logits = 1;
    }
    p.skb = (int)skb;
    // Ragged leftover rows pay off when a CTA holds only a few tiles (7168 rows: 3 tiles + 1 row instead
    // of 4 tiles on four CTAs); with many tiles per CTA one whole extra tile is within 2 % of balance.
    p.ragged = (t0->split && Gm < 8) ? 1 : 0;
    p.gran = ragged_granularity(p.n, ncta);
    p.nslot_max = (Gm * kGroupRows) / p.bn + 2 + 2;
    p.part_rows = (Gm + 2) * kGroupRows;  // whole tiles + at most two ragged tiles
    // One or two activation rows: CUDA-core dot products; more: the tensor-core MMA.
    const int gt = (t0->kernel_sel != 1 && mt <= 2) ? mt : 0;
    void (*const kernel)(Fp8Params) = gt == 1 ? fp8_rowpar_kernel<1> : gt == 2 ? fp8_rowpar_kernel<2> : fp8_rowpar_kernel<0>;
    const Fp8Smem fixed = fp8_smem_layout(0, kbox, p.mp, p.nslot_max, p.skb, p.m, p.part_rows, gt);
    p.stage_bytes = fp8_stage_boxes(kbox) * kBoxBytes;
    int ns = (kSmemBudget - fixed.total) / p.stage_bytes;
    if (ns > kMaxStages) ns = kMaxStages;
    if (ns < 2) return fail(t0, WS_ERR_CAPACITY, "shapes m=%d n=%d k=%d leave no room for the weight stage ring", p.m, p.n, p.k);
    p.nstages = ns;
    const size_t smem = (size_t)fp8_smem_layout(ns, kbox, p.mp, p.nslot_max, p.skb, p.m, p.part_rows, gt).total + 1024;

    for (int i = 0; i < n; ++i) {
        ws_tp *t = ranks[i];
        const ws_fp8_gemm_args_t &a = lm ? lm[i].g : args[i];
        Fp8RankArgs &r = p.r[i];
        for (int b = 0; b < 2; ++b) {
            ws_status_t s = make_tmap(t, &p.tmap[i][b], a.w, (uint64_t)a.n, (uint64_t)a.k, (uint64_t)a.ldw,
                                      b ? (uint32_t)p.gran : (uint32_t)kGroupRows);
            if (s != WS_OK) { t0->err = t->err; return s; }
        }
        const size_t xes = a.x_dtype == WS_ACT_BF16 ? 2 : 4;
        r.x = static_cast<const char *>(a.x) + (size_t)m0 * a.ldx * xes;
        r.scales = a.scales;
        r.out = lm ? nullptr : a.out + (size_t)m0 * a.n;
        r.logits = lm && lm[i].logits ? lm[i].logits + (size_t)m0 * lm[i].vocab : nullptr;
        r.argmax = lm && lm[i].argmax ? lm[i].argmax + m0 : nullptr;
        r.ldx = a.ldx; r.scale_ld = a.scale_ld; r.row0 = a.row0; r.k0 = a.k0;
        r.vocab_row0 = lm ? lm[i].vocab_row0 : 0;
        r.ctx = make_ctx(t);
        if (last) r.ctx.host_done = t->host_done_arm;
        p.w[i] = a.w;
        p.ldw[i] = a.ldw;
    }
    // as in the tensor-memory path: only when a second CTA can be resident beside the predecessor's
    p.l2_prefetch = (2 * smem <= (size_t)227 * 1024 && (size_t)p.n * p.k <= ((size_t)64 << 20)) ? 1 : 0;
    // every endpoint advances by one step
    for (int i = 0; i < n; ++i) ranks[i]->step++;
    if (same_device) {
        WS_CUDA(t0, cudaSetDevice(t0->device));
        return launch(t0, kernel, p, ncta, n, fp8_threads(gt), smem, static_cast<cudaStream_t>(streams ? streams[0] : nullptr), t0->pdl != 0);
    }
    for (int i = 0; i < n; ++i) {  // one launch per device, each sees itself as virtual rank 0
        Fp8Params q = p;
        q.r[0] = p.r[i];
        q.tmap[0][0] = p.tmap[i][0];
        q.tmap[0][1] = p.tmap[i][1];
        q.w[0] = p.w[i];
        q.ldw[0] = p.ldw[i];
        WS_CUDA(ranks[i], cudaSetDevice(ranks[i]->device));
        ws_status_t s = launch(ranks[i], kernel, q, ncta, 1, fp8_threads(gt), smem,
                               static_cast<cudaStream_t>(streams ? streams[i] : nullptr), t0->pdl != 0);
        if (s != WS_OK) { t0->err = ranks[i]->err; return s; }
    }
    return WS_OK;
}

ws_status_t ws_fp8_rowpar_gemm_allreduce_group(ws_tp_t *const *ranks, int32_t n, const ws_fp8_gemm_args_t *args,
                                               void *const *streams) {
    int ncta;
    bool same;
    ws_status_t s = group_prelude(ranks, n, &ncta, &same);
    if (s != WS_OK) return s;
    ws_tp *t0 = ranks[0];
    if (!args) return fail(t0, WS_ERR_INVALID, "null args");
    for (int i = 0; i < n; ++i) {
        s = validate_fp8(t0, args[i], false);
        if (s != WS_OK) return s;
        if (args[i].m != args[0].m || args[i].n != args[0].n || args[i].k != args[0].k ||
            args[i].block_n != args[0].block_n || args[i].block_k != args[0].block_k ||
            args[i].scale_kind != args[0].scale_kind || args[i].x_dtype != args[0].x_dtype)
            return fail(t0, WS_ERR_INVALID, "ranks must pass equal shapes and formats");
    }
    if (args[0].m > t0->cfg.max_m || args[0].n > t0->cfg.max_n)
        return fail(t0, WS_ERR_CAPACITY, "m=%d n=%d exceed the endpoint's max_m=%d max_n=%d", args[0].m, args[0].n,
                    t0->cfg.max_m, t0->cfg.max_n);
    for (int m0 = 0; m0 < args[0].m;) {
        const int mt = fp8_rows_per_launch(t0, args[0], ncta, args[0].m - m0, false);
        s = fp8_step(ranks, n, args, nullptr, m0, mt, streams, ncta, same, m0 + mt >= args[0].m);
        if (s != WS_OK) return s;
        m0 += mt;
    }
    return WS_OK;
}

ws_status_t ws_fp8_rowpar_gemm_allreduce(ws_tp_t *tp, const ws_fp8_gemm_args_t *args, void *stream) {
    ws_tp_t *r[1] = {tp};
    void *s[1] = {stream};
    return ws_fp8_rowpar_gemm_allreduce_group(r, 1, args, s);
}

ws_status_t ws_lm_head_allgather_argmax_group(ws_tp_t *const *ranks, int32_t n, const ws_lm_head_args_t *args,
                                              void *const *streams) {
    int ncta;
    bool same;
    ws_status_t s = group_prelude(ranks, n, &ncta, &same);
    if (s != WS_OK) return s;
    ws_tp *t0 = ranks[0];
    if (!args) return fail(t0, WS_ERR_INVALID, "null args");
    bool any_logits = false;
    for (int i = 0; i < n; ++i) {
        s = validate_fp8(t0, args[i].g, true);
        if (s != WS_OK) return s;
        const ws_fp8_gemm_args_t &g = args[i].g, &g0 = args[0].g;
        if (g.m != g0.m || g.n != g0.n || g.k != g0.k || g.block_n != g0.block_n || g.block_k != g0.block_k ||
            g.scale_kind != g0.scale_kind || g.x_dtype != g0.x_dtype || args[i].vocab != args[0].vocab)
            return fail(t0, WS_ERR_INVALID, "ranks must pass equal shapes and formats");
        if (args[i].vocab_row0 < 0 || args[i].vocab_row0 + g.n > args[i].vocab)
            return fail(t0, WS_ERR_INVALID, "vocab shard [%lld, +%d) lies outside vocab %d",
                        (long long)args[i].vocab_row0, g.n, args[i].vocab);
        any_logits |= args[i].logits != nullptr;
    }
    if (args[0].g.m > t0->cfg.max_m) return fail(t0, WS_ERR_CAPACITY, "m=%d exceeds max_m=%d", args[0].g.m, t0->cfg.max_m);
    if (any_logits && args[0].vocab > t0->cfg.max_vocab)
        return fail(t0, WS_ERR_CAPACITY, "vocab=%d exceeds the endpoint's max_vocab=%d", args[0].vocab, t0->cfg.max_vocab);
    for (int m0 = 0; m0 < args[0].g.m;) {
        const int mt = fp8_rows_per_launch(t0, args[0].g, ncta, args[0].g.m - m0, any_logits, true);
        s = fp8_step(ranks, n, nullptr, args, m0, mt, streams, ncta, same, m0 + mt >= args[0].g.m);
        if (s != WS_OK) return s;
        m0 += mt;
    }
    return WS_OK;
}

ws_status_t ws_lm_head_allgather_argmax(ws_tp_t *tp, const ws_lm_head_args_t *args, void *stream) {
    ws_tp_t *r[1] = {tp};
    void *s[1] = {stream};
    return ws_lm_head_allgather_argmax_group(r, 1, args, s);
}


// ------------------------------------------------------------------------------ MoE down
static ws_status_t ensure_moe_scratch(ws_tp *tp, size_t work_bytes, size_t acc_bytes) {
    WS_CUDA(tp, cudaSetDevice(tp->device));
    if (work_bytes > tp->moe_work_bytes) {
        if (tp->moe_work) cudaFree(tp->moe_work);
        tp->moe_work = nullptr;
        tp->moe_work_bytes = 0;
        WS_CUDA(tp, cudaMalloc(&tp->moe_work, work_bytes));
        tp->moe_work_bytes = work_bytes;
    }
    if (acc_bytes > tp->moe_acc_bytes) {
        if (tp->moe_acc) cudaFree(tp->moe_acc);
        tp->moe_acc = nullptr;
        tp->moe_acc_bytes = 0;
        WS_CUDA(tp, cudaMalloc(&tp->moe_acc, acc_bytes));
        tp->moe_acc_bytes = acc_bytes;
    }
    return WS_OK;
}

// Plan of the MoE step on the tcgen05 path; ok = false when the shape does not fit it (CTA pairs split K
// in halves of at most 16 slabs, a pair's rows are one MMA tile, the per-token sums live in shared memory).
struct MoeBsPlan {
    bool ok;
    int ncta, tile_rows, a_pitch, slabs_per_stage, nstages, tmem_cols;
    size_t smem;
};
static MoeBsPlan moe_bs_plan(const ws_moe_down_args_t &a, int ncta) {
    MoeBsPlan u{};
    u.ncta = ncta & ~1;
    const int nparts = u.ncta / 2, kslabs = a.k / 128;
    if (nparts < 1 || a.k % 256 || kslabs / 2 > kMoeBsMaxSlabs || a.m > 64) return u;  // 64 tokens: their sums fill 64 KB of shared memory
    u.tile_rows = (a.n + nparts - 1) / nparts;
    if (u.tile_rows > kBsMmaRows) return u;
    u.a_pitch = (u.tile_rows + 7) / 8 * 8 * 128;
    const int nslab = kslabs / 2;
    // a stage = 4 slabs (2 when the half of K is not a multiple of 4): one commit and one activation copy per stage
    if (nslab % 2) return u;
    u.slabs_per_stage = nslab % 4 ? 2 : 4;
    int ns = kMaxStages;
    while (ns >= 2 && moe_bs_smem_layout(ns, u.slabs_per_stage, u.a_pitch, a.m, nslab).total + 1024 > kSmemBudget) --ns;
    u.nstages = ns;
    int cols = 32;
    while (cols < 2 * kMoeBsCols + 2 * nslab * 8) cols *= 2;
    u.tmem_cols = cols;
    u.ok = ns >= 2 && cols <= 512;
    if (u.ok) u.smem = (size_t)moe_bs_smem_layout(ns, u.slabs_per_stage, u.a_pitch, a.m, nslab).total + 1024;
    return u;
}

// The MoE step on the block-scaled tcgen05 path: prep kernel, then the persistent CTA pairs.  One rank
// per launch (a cluster launch cannot also be the cooperative launch virtual ranks need).
static ws_status_t moe_bs_step(ws_tp *const *ranks, int n, const ws_moe_down_args_t *args, void *const *streams,
                               const MoeBsPlan &u) {
    ws_tp *t0 = ranks[0];
    const ws_moe_down_args_t &a0 = args[0];
    MoeBsParams p{};
    p.m = a0.m; p.n = a0.n; p.k = a0.k; p.world = t0->world;
    p.tile_rows = u.tile_rows; p.a_pitch = u.a_pitch; p.slabs_per_stage = u.slabs_per_stage; p.nstages = u.nstages;
    p.tmem_cols = u.tmem_cols;
    p.timeout_ns = t0->timeout_ns;
    p.lay = t0->lay;
    MoeBsPrepParams q{};
    q.m = a0.m; q.k = a0.k; q.top_k = a0.top_k; q.h_dtype = a0.h_dtype; q.sl = u.slabs_per_stage;
    const MoeBsWork W = moe_bs_work_layout(a0.k);
    const int nblk = a0.m * a0.top_k + 1;
    for (int i = 0; i < n; ++i) ranks[i]->step++;
    for (int i = 0; i < n; ++i) {
        ws_tp *t = ranks[i];
        const ws_moe_down_args_t &a = args[i];
        ws_status_t s = ensure_moe_scratch(t, (size_t)W.total, 0);
        if (s == WS_OK) s = make_tmap_fp4(t, &p.tmap_w[0], a.w2, (uint64_t)a.e_len, (uint64_t)a.n, (uint64_t)a.k, (uint32_t)u.tile_rows);
        if (s != WS_OK) { t0->err = t->err; return s; }
        MoeBsRank &r = p.r[0];
        r.s2 = a.s2; r.work = t->moe_work; r.out = a.out; r.e_start = a.e_start; r.e_len = a.e_len;
        r.ctx = make_ctx(t);
        MoePrepRank &pr = q.r[0];
        pr.h = a.h; pr.route_ids = a.route_ids; pr.route_w = a.route_w; pr.work = t->moe_work;
        pr.ldh = a.ldh; pr.e_start = a.e_start; pr.e_len = a.e_len;
        WS_CUDA(t, cudaSetDevice(t->device));
        cudaStream_t cs = static_cast<cudaStream_t>(streams ? streams[i] : nullptr);
        s = launch(t, moe_bs_prep_kernel, q, nblk, 1, 256, 0, cs, t0->pdl != 0, false);
        if (s == WS_OK) s = launch(t, moe_bs_kernel, p, u.ncta, 1, kMoeBsThreads, u.smem, cs, t0->pdl != 0, true, 2);
        if (s != WS_OK) { t0->err = t->err; return s; }
    }
    return WS_OK;
}

// Decode form of the MoE step: the prep kernel (activation quantisation once per route, pass
// table) followed by the persistent matrix-vector kernel.  Arguments are already validated.
static ws_status_t moe_gemv_step(ws_tp *const *ranks, int n, const ws_moe_down_args_t *args, void *const *streams,
                                 int ncta, bool same) {
    ws_tp *t0 = ranks[0];
    const ws_moe_down_args_t &a0 = args[0];
    MoeGemvParams p{};
    p.m = a0.m; p.n = a0.n; p.k = a0.k; p.top_k = a0.top_k; p.world = t0->world;
    p.timeout_ns = t0->timeout_ns;
    p.lay = t0->lay;
    const int kbytes = p.k / 2, kbox = kbytes / 128, kb32 = p.k / 32;
    const int nslice = moe_gemv_slices(p.k);
    // rows are dealt out in units whose scale bytes are a multiple of 16 (they travel by bulk copy)
    p.gran = 1;
    while ((p.gran * kb32) % 16) p.gran *= 2;
    int rows_max = 0;
    for (int c = 0; c < ncta; ++c) {
        int a, b;
        moe_gemv_rows(p.n, p.gran, ncta, c, a, b);
        rows_max = std::max(rows_max, b - a);
    }
    if (rows_max < 1) rows_max = p.gran;
    p.acc_rows = rows_max;
    p.acc_global = (size_t)nslice * p.m * rows_max * 4 > 16384 ? 1 : 0;
    auto stage_bytes = [&](int pr) { return (int)align_up((int64_t)kbox * ((pr + 7) / 8 * 8) * 128 + (int64_t)pr * kb32, 1024); };
    const int fixed = moe_gemv_smem(0, 0, p.k, p.m, p.acc_rows, p.acc_global).total;
    // one stage holds a CTA's whole row range of one expert when three of them fit; otherwise
    // the range is walked in panels of a multiple of 16 rows
    p.panel_rows = rows_max;
    if (3 * stage_bytes(p.panel_rows) > kSmemBudget - fixed) {
        p.panel_rows = (rows_max + 15) / 16 * 16;
        while (p.panel_rows > 16 && 3 * stage_bytes(p.panel_rows) > kSmemBudget - fixed) p.panel_rows -= 16;
    }
    p.stage_bytes = stage_bytes(p.panel_rows);
    p.rows_pitch = (p.panel_rows + 7) / 8 * 8;
    p.scale_off = kbox * p.rows_pitch * 128;
    int ns = (kSmemBudget - fixed) / p.stage_bytes;
    if (ns > kMaxStages) ns = kMaxStages;
    if (ns < 2) return fail(t0, WS_ERR_CAPACITY, "shapes m=%d n=%d k=%d leave no room for the weight stage ring", p.m, p.n, p.k);
    p.nstages = ns;
    const size_t smem = (size_t)moe_gemv_smem(ns, p.stage_bytes, p.k, p.m, p.acc_rows, p.acc_global).total + 1024;

    MoePrepParams q{};
    q.m = p.m; q.k = p.k; q.top_k = p.top_k; q.h_dtype = a0.h_dtype;
    const size_t work_bytes = (size_t)moe_work_layout(p.k).total;
    const size_t acc_bytes = p.acc_global ? (size_t)nslice * p.m * p.n * 4 : 0;
    for (int i = 0; i < n; ++i) {
        const ws_moe_down_args_t &a = args[i];
        ws_status_t s = ensure_moe_scratch(ranks[i], work_bytes, acc_bytes);
        if (s != WS_OK) { t0->err = ranks[i]->err; return s; }
        for (int b = 0; b < 2; ++b) {
            s = make_tmap(ranks[i], &p.tmap[i][b], a.w2, (uint64_t)a.e_len * a.n, (uint64_t)kbytes, (uint64_t)kbytes,
                          b ? (uint32_t)p.gran : (uint32_t)kGroupRows);
            if (s != WS_OK) { t0->err = ranks[i]->err; return s; }
        }
        MoeGemvRank &r = p.r[i];
        r.s2 = a.s2; r.work = ranks[i]->moe_work; r.out = a.out; r.acc_g = ranks[i]->moe_acc;
        r.e_start = a.e_start; r.e_len = a.e_len;
        r.ctx = make_ctx(ranks[i]);
        MoePrepRank &pr = q.r[i];
        pr.h = a.h; pr.route_ids = a.route_ids; pr.route_w = a.route_w; pr.work = ranks[i]->moe_work;
        pr.ldh = a.ldh; pr.e_start = a.e_start; pr.e_len = a.e_len;
    }
    for (int i = 0; i < n; ++i) ranks[i]->step++;
    const int nblk = p.m * p.top_k + 1;
    if (same) {
        WS_CUDA(t0, cudaSetDevice(t0->device));
        cudaStream_t cs = static_cast<cudaStream_t>(streams ? streams[0] : nullptr);
        ws_status_t s = launch(t0, moe_prep_kernel, q, nblk, n, 256, 0, cs, t0->pdl != 0, false);
        if (s != WS_OK) return s;
        return launch(t0, moe_gemv_kernel, p, ncta, n, kMoeGemvThreads, smem, cs, t0->pdl != 0);
    }
    for (int i = 0; i < n; ++i) {
        MoeGemvParams pi = p;
        pi.r[0] = p.r[i];
        pi.tmap[0][0] = p.tmap[i][0];
        pi.tmap[0][1] = p.tmap[i][1];
        MoePrepParams qi = q;
        qi.r[0] = q.r[i];
        WS_CUDA(ranks[i], cudaSetDevice(ranks[i]->device));
        cudaStream_t cs = static_cast<cudaStream_t>(streams ? streams[i] : nullptr);
        ws_status_t s = launch(ranks[i], moe_prep_kernel, qi, nblk, 1, 256, 0, cs, t0->pdl != 0, false);
        if (s == WS_OK) s = launch(ranks[i], moe_gemv_kernel, pi, ncta, 1, kMoeGemvThreads, smem, cs, t0->pdl != 0);
        if (s != WS_OK) { t0->err = ranks[i]->err; return s; }
    }
    return WS_OK;
}

ws_status_t ws_moe_down_combine_allreduce_group(ws_tp_t *const *ranks, int32_t n, const ws_moe_down_args_t *args,
                                                void *const *streams) {
    int ncta;
    bool same;
    ws_status_t s = group_prelude(ranks, n, &ncta, &same);
    if (s != WS_OK) return s;
    ws_tp *t0 = ranks[0];
    if (!args) return fail(t0, WS_ERR_INVALID, "null args");
    const ws_moe_down_args_t &a0 = args[0];
    for (int i = 0; i < n; ++i) {
        const ws_moe_down_args_t &a = args[i];
        if (!a.h || !a.route_ids || !a.route_w || !a.w2 || !a.s2 || !a.out) return fail(t0, WS_ERR_INVALID, "null argument");
        if (a.m < 1 || a.top_k < 1 || a.top_k > kMoeMaxTopK || a.m * a.top_k > kMoeMaxRoutes)
            return fail(t0, WS_ERR_CAPACITY, "m*top_k = %d*%d exceeds %d routes per step", a.m, a.top_k, kMoeMaxRoutes);
        if (a.n % 16 || a.k % 256 || a.k < 256) return fail(t0, WS_ERR_INVALID, "n must be a multiple of 16 and k of 256");
        if (a.e_len < 1 || a.e_len > kMoeMaxExperts || a.e_start < 0) return fail(t0, WS_ERR_INVALID, "bad local expert range");
        if ((int64_t)a.e_len * a.n >= (1ll << 31)) return fail(t0, WS_ERR_CAPACITY, "expert slab has too many rows");
        const int ha = a.h_dtype == WS_ACT_BF16 ? 8 : 4;
        if ((reinterpret_cast<uintptr_t>(a.h) & 15) || (a.ldh % ha) || a.ldh < a.k)
            return fail(t0, WS_ERR_INVALID, "h must be 16-byte aligned with ldh >= k and ldh a multiple of %d", ha);
        if (reinterpret_cast<uintptr_t>(a.s2) & 15) return fail(t0, WS_ERR_INVALID, "s2 must be 16-byte aligned");
        if (a.m != a0.m || a.n != a0.n || a.k != a0.k || a.top_k != a0.top_k || a.h_dtype != a0.h_dtype)
            return fail(t0, WS_ERR_INVALID, "ranks must pass equal shapes and formats");
    }
    if (a0.m > t0->cfg.max_m || a0.n > t0->cfg.max_n)
        return fail(t0, WS_ERR_CAPACITY, "m=%d n=%d exceed the endpoint's max_m=%d max_n=%d", a0.m, a0.n, t0->cfg.max_m, t0->cfg.max_n);

    int e_len_all = args[0].e_len;
    for (int i = 0; i < n; ++i)
        if (args[i].e_len != e_len_all) return fail(t0, WS_ERR_INVALID, "ranks must hold equally many experts");
    if (t0->kernel_sel != 1 && (n == 1 || !same) && (reinterpret_cast<uintptr_t>(a0.w2) & 31) == 0) {  // tcgen05 form
        const MoeBsPlan u = moe_bs_plan(a0, ncta);
        // measured on B200 (384 experts of 7168x2048, top-6), tcgen05 against the CUDA-core decode form:
        // 1 token 19.5 against 23.6 us, 8 tokens 95 against 130, 64 tokens 495 against 841
        if (u.ok && t0->moe_bs) return moe_bs_step(ranks, n, args, streams, u);
    }
    if (t0->kernel_sel != 1 && a0.k <= 32 * 32 * kMoeGemvWarps)  // decode form: CUDA-core matrix-vector products
        return moe_gemv_step(ranks, n, args, streams, ncta, same);

    MoeParams p{};
    p.m = a0.m; p.n = a0.n; p.k = a0.k; p.top_k = a0.top_k; p.h_dtype = a0.h_dtype; p.world = t0->world;
    p.timeout_ns = t0->timeout_ns;
    p.lay = t0->lay;
    const int kbox = (p.k / 2 + 127) / 128, kb32 = p.k / 32;
    p.tiles_per_item = kbox * kBoxBytes <= kStageBytes / 2 ? 2 : 1;  // keep a stage near 32 KB
    const int Gm = p.n / kGroupRows / ncta;
    p.ragged = (t0->split && Gm < 8) ? 1 : 0;
    p.gran = ragged_granularity(p.n, ncta);
    // the rows' scale bytes travel by bulk copy: sizes and addresses must be multiples of 16 bytes
    while (p.gran < kGroupRows && (p.gran * kb32) % 16) p.gran *= 2;
    if (p.gran >= kGroupRows) { p.ragged = 0; p.gran = 1; }
    p.part_rows = (Gm + 2) * kGroupRows;
    int e_len_max = 0;
    for (int i = 0; i < n; ++i) e_len_max = std::max(e_len_max, args[i].e_len);
    const MoeSmem fixed = moe_smem_layout(0, p.tiles_per_item, p.k, p.m, p.top_k, e_len_max, p.part_rows);
    int ns = (kSmemBudget - fixed.total) / fixed.stage_bytes;
    if (ns > kMaxStages) ns = kMaxStages;
    if (ns < 2)
        return fail(t0, WS_ERR_CAPACITY, "shapes m=%d n=%d k=%d leave no room for the weight stage ring", p.m, p.n, p.k);
    p.nstages = ns;
    const size_t smem = (size_t)moe_smem_layout(ns, p.tiles_per_item, p.k, p.m, p.top_k, e_len_max, p.part_rows).total + 1024;
    for (int i = 0; i < n; ++i) {
        const ws_moe_down_args_t &a = args[i];
        if (a.e_len != e_len_max) return fail(t0, WS_ERR_INVALID, "ranks must hold equally many experts");
        for (int b = 0; b < 2; ++b) {
            s = make_tmap(ranks[i], &p.tmap[i][b], a.w2, (uint64_t)a.e_len * a.n, (uint64_t)a.k / 2, (uint64_t)a.k / 2,
                          b ? (uint32_t)p.gran : (uint32_t)kGroupRows);
            if (s != WS_OK) { t0->err = ranks[i]->err; return s; }
        }
        MoeRankArgs &r = p.r[i];
        r.h = a.h; r.route_ids = a.route_ids; r.route_w = a.route_w; r.s2 = a.s2; r.out = a.out;
        r.ldh = a.ldh; r.e_start = a.e_start; r.e_len = a.e_len;
        r.ctx = make_ctx(ranks[i]);
    }
    for (int i = 0; i < n; ++i) ranks[i]->step++;
    if (same) {
        WS_CUDA(t0, cudaSetDevice(t0->device));
        return launch(t0, moe_down_kernel, p, ncta, n, kThreads, smem, static_cast<cudaStream_t>(streams ? streams[0] : nullptr),
                      t0->pdl != 0);
    }
    for (int i = 0; i < n; ++i) {
        MoeParams q = p;
        q.r[0] = p.r[i];
        q.tmap[0][0] = p.tmap[i][0];
        q.tmap[0][1] = p.tmap[i][1];
        WS_CUDA(ranks[i], cudaSetDevice(ranks[i]->device));
        s = launch(ranks[i], moe_down_kernel, q, ncta, 1, kThreads, smem, static_cast<cudaStream_t>(streams ? streams[i] : nullptr),
                   t0->pdl != 0);
        if (s != WS_OK) { t0->err = ranks[i]->err; return s; }
    }
    return WS_OK;
}

ws_status_t ws_moe_down_combine_allreduce(ws_tp_t *tp, const ws_moe_down_args_t *args, void *stream) {
    ws_tp_t *r[1] = {tp};
    void *s[1] = {stream};
    return ws_moe_down_combine_allreduce_group(r, 1, args, s);
}

// ------------------------------------------------------------------------------ collectives
static ws_status_t coll_group(ws_tp_t *const *ranks, int n, const float *const *in, float *const *out, int64_t len,
                              void *const *streams, int gather) {
    int ncta;
    bool same;
    ws_status_t s = group_prelude(ranks, n, &ncta, &same);
    if (s != WS_OK) return s;
    ws_tp *t0 = ranks[0];
    if (!in || !out || len < 1) return fail(t0, WS_ERR_INVALID, "collective input len %lld not in 1..", (long long)len);
    if (len > (int64_t)t0->cfg.max_m * t0->cfg.max_n)
        return fail(t0, WS_ERR_CAPACITY, "collective input len %lld not in 1..=%lld", (long long)len,
                    (long long)t0->cfg.max_m * t0->cfg.max_n);
    CollParams p{};
    p.len = len; p.world = t0->world; p.gather = gather; p.timeout_ns = t0->timeout_ns; p.lay = t0->lay;
    for (int i = 0; i < n; ++i) {
        if (!in[i] || !out[i]) return fail(t0, WS_ERR_INVALID, "null buffer");
        p.r[i].in = in[i];
        p.r[i].out = out[i];
        p.r[i].ctx = make_ctx(ranks[i]);
    }
    ncta = (int)std::min<int64_t>(ncta, std::max<int64_t>(1, len / 256));
    for (int i = 0; i < n; ++i) ranks[i]->step++;
    if (same) {
        WS_CUDA(t0, cudaSetDevice(t0->device));
        return launch(t0, coll_kernel, p, ncta, n, 256, 0, static_cast<cudaStream_t>(streams ? streams[0] : nullptr));
    }
    for (int i = 0; i < n; ++i) {
        CollParams q = p;
        q.r[0] = p.r[i];
        WS_CUDA(ranks[i], cudaSetDevice(ranks[i]->device));
        s = launch(ranks[i], coll_kernel, q, ncta, 1, 256, 0, static_cast<cudaStream_t>(streams ? streams[i] : nullptr));
        if (s != WS_OK) { t0->err = ranks[i]->err; return s; }
    }
    return WS_OK;
}

ws_status_t ws_allreduce_f32_group(ws_tp_t *const *ranks, int32_t n, const float *const *in, float *const *out,
                                   int64_t len, void *const *streams) {
    return coll_group(ranks, n, in, out, len, streams, 0);
}
ws_status_t ws_allgather_f32_group(ws_tp_t *const *ranks, int32_t n, const float *const *in, float *const *out,
                                   int64_t len, void *const *streams) {
    return coll_group(ranks, n, in, out, len, streams, 1);
}
ws_status_t ws_allreduce_f32(ws_tp_t *tp, const float *in, float *out, int64_t len, void *stream) {
    ws_tp_t *r[1] = {tp};
    void *s[1] = {stream};
    const float *i[1] = {in};
    float *o[1] = {out};
    return coll_group(r, 1, i, o, len, s, 0);
}
ws_status_t ws_allgather_f32(ws_tp_t *tp, const float *in, float *out, int64_t len, void *stream) {
    ws_tp_t *r[1] = {tp};
    void *s[1] = {stream};
    const float *i[1] = {in};
    float *o[1] = {out};
    return coll_group(r, 1, i, o, len, s, 1);
}

// ------------------------------------------------------------------------------ host-buffer forms
static ws_status_t ensure_staging(ws_tp *tp, size_t pin_bytes, size_t dev_bytes) {
    WS_CUDA(tp, cudaSetDevice(tp->device));
    if (pin_bytes > tp->pin_bytes) {
        if (tp->pin) cudaFreeHost(tp->pin);
        tp->pin = nullptr;
        tp->pin_bytes = 0;
        WS_CUDA(tp, cudaHostAlloc(&tp->pin, pin_bytes, cudaHostAllocDefault));
        tp->pin_bytes = pin_bytes;
    }
    if (dev_bytes > tp->dev_stage_bytes) {
        if (tp->dev_stage) cudaFree(tp->dev_stage);
        tp->dev_stage = nullptr;
        tp->dev_stage_bytes = 0;
        WS_CUDA(tp, cudaMalloc(&tp->dev_stage, dev_bytes));
        tp->dev_stage_bytes = dev_bytes;
    }
    return WS_OK;
}

static ws_status_t coll_host(ws_tp *tp, const float *in, float *out, int64_t len, int gather) {
    if (!tp || !in || !out || len < 1) return WS_ERR_INVALID;
    const size_t ib = (size_t)len * 4, ob = gather ? ib * tp->world : ib;
    ws_status_t s = ensure_staging(tp, ib + ob, ib + ob);
    if (s != WS_OK) return s;
    char *pin = static_cast<char *>(tp->pin), *dev = static_cast<char *>(tp->dev_stage);
    memcpy(pin, in, ib);
    WS_CUDA(tp, cudaMemcpyAsync(dev, pin, ib, cudaMemcpyHostToDevice, tp->hstream));
    s = gather ? ws_allgather_f32(tp, reinterpret_cast<float *>(dev), reinterpret_cast<float *>(dev + ib), len, tp->hstream)
               : ws_allreduce_f32(tp, reinterpret_cast<float *>(dev), reinterpret_cast<float *>(dev + ib), len, tp->hstream);
    if (s != WS_OK) return s;
    WS_CUDA(tp, cudaMemcpyAsync(pin + ib, dev + ib, ob, cudaMemcpyDeviceToHost, tp->hstream));
    s = ws_tp_check(tp, tp->hstream);
    if (s != WS_OK) return s;
    memcpy(out, pin + ib, ob);
    return WS_OK;
}
ws_status_t ws_allreduce_f32_host(ws_tp_t *tp, const float *in, float *out, int64_t len) { return coll_host(tp, in, out, len, 0); }
ws_status_t ws_allgather_f32_host(ws_tp_t *tp, const float *in, float *out, int64_t len) { return coll_host(tp, in, out, len, 1); }

// The host-buffer step is the same sequence every time a caller repeats it on one weight (copy
// the activations in, launch, copy the rows and the status word out), so it is captured once per
// distinct argument set and replayed as one graph launch; a handful of sets are kept.
static uint64_t hash_fp8_args(const ws_fp8_gemm_args_t &a, const void *pin, const void *dev, int sel) {
    uint64_t h = 0xcbf29ce484222325ull;  // FNV-1a over the fields that name a distinct step
    auto mix = [&](uint64_t v) {
        for (int i = 0; i < 8; ++i) {
            h ^= (v >> (8 * i)) & 0xFFu;
            h *= 0x100000001b3ull;
        }
    };
    mix((uint64_t)(uintptr_t)a.w); mix((uint64_t)(uintptr_t)a.scales); mix((uint64_t)a.ldw); mix((uint64_t)a.scale_ld);
    mix(((uint64_t)(uint32_t)a.m << 32) | (uint32_t)a.n); mix(((uint64_t)(uint32_t)a.k << 32) | (uint32_t)a.x_dtype);
    mix(((uint64_t)(uint32_t)a.block_n << 32) | (uint32_t)a.block_k); mix((uint64_t)a.row0); mix((uint64_t)a.k0);
    mix((uint64_t)(uintptr_t)pin); mix((uint64_t)(uintptr_t)dev); mix(((uint64_t)(uint32_t)a.scale_kind << 32) | (uint32_t)sel);
    return h;
}

static bool same_fp8_args(const ws_fp8_gemm_args_t &a, const ws_fp8_gemm_args_t &b) {
    return a.m == b.m && a.n == b.n && a.k == b.k && a.x_dtype == b.x_dtype && a.w == b.w && a.ldw == b.ldw &&
           a.scales == b.scales && a.scale_ld == b.scale_ld && a.scale_kind == b.scale_kind && a.block_n == b.block_n &&
           a.block_k == b.block_k && a.row0 == b.row0 && a.k0 == b.k0;
}

// Activations of a host-buffer call on their way in: nothing to do when the step's own prep kernel
// reads the pinned buffer, a fetching kernel for small inputs, the copy engine for large ones.
static bool host_stage_in(ws_tp *tp, char *dev, const char *pin, size_t bytes, bool direct, bool stage) {
    if (direct && !stage) return true;
    if (!direct) return cudaMemcpyAsync(dev, pin, bytes, cudaMemcpyHostToDevice, tp->hstream) == cudaSuccess;
    StageParams q{reinterpret_cast<const uint4 *>(pin), reinterpret_cast<uint4 *>(dev), (int64_t)((bytes + 15) / 16)};
    const int blocks = (int)((q.n16 + 255) / 256);
    return launch(tp, stage_in_kernel, q, blocks, 1, 256, 0, tp->hstream, tp->pdl != 0, false) == WS_OK;
}

// Wait for the word the step's last kernel sets in pinned memory, then hand the results (which the
// kernel wrote into the pinned buffer) to the caller.  The stream is asked now and then, so that a
// launch that died, or a step that ended without reporting, still ends the call.
static ws_status_t host_wait_and_copy_out(ws_tp *tp, volatile uint64_t *done, float *out_host, const char *src, size_t bytes) {
    uint64_t word = 0;
    for (uint32_t spins = 0; (word = *done) == 0; ++spins) {
        if ((spins & 0xFFFu) == 0xFFFu) {
            if (cudaStreamQuery(tp->hstream) == cudaErrorNotReady) continue;
            word = *done;  // the stream has drained (or died): whatever the kernel wrote is there now
            break;
        }
#if defined(__x86_64__)
        __builtin_ia32_pause();
#endif
    }
    if (word == 0 || (uint32_t)word != 0u) {  // no report, or a device code: the check turns it into status + message
        const ws_status_t s = ws_tp_check(tp, tp->hstream);
        if (s != WS_OK) return s;
    }
    memcpy(out_host, src, bytes);
    return WS_OK;
}

ws_status_t ws_fp8_rowpar_gemm_allreduce_host(ws_tp_t *tp, const ws_fp8_gemm_args_t *dw, const void *x_host, float *out_host) {
    if (!tp || !dw || !x_host || !out_host) return WS_ERR_INVALID;
    const size_t es = dw->x_dtype == WS_ACT_BF16 ? 2 : 4;
    const size_t xb = (size_t)dw->m * dw->k * es, xb_al = (xb + 255) / 256 * 256, ob = (size_t)dw->m * dw->n * 4;
    ws_status_t s = ensure_staging(tp, xb_al + ob, xb_al);
    if (s != WS_OK) return s;
    if (!tp->pin_done) WS_CUDA(tp, cudaHostAlloc(reinterpret_cast<void **>(&tp->pin_done), 64, cudaHostAllocDefault));
    char *pin = static_cast<char *>(tp->pin), *dev = static_cast<char *>(tp->dev_stage);
    // The activations are copied in; the results are written by the kernel straight into the pinned
    // buffer (it is mapped into the device's address space), and the last CTA sets *pin_done: no copy
    // back and no wait on the stream stand between the last store and the host.
    ws_fp8_gemm_args_t a = *dw;
    a.x = dev;
    a.ldx = dw->k;
    a.out = reinterpret_cast<float *>(pin + xb_al);
    volatile uint64_t *done = tp->pin_done;

    // Up to 64 KB of activations: no copy engine on the way in either.  A kernel fetches them from the
    // pinned buffer over PCIe (a few us for 16 KB) while the main kernel, launched with it from one graph
    // and already resident, streams its first weights: the tensor-memory path's prep kernel reads them in
    // place; for the CUDA-core path a small kernel brings them into device memory.  Either way the step
    // runs on the kernel a device-buffer call with these arguments runs on, so the results are the same bits.
    bool direct = false, stage = false;
    if (xb <= 64 * 1024) {
        int ncta = 0;
        bool same = true;
        ws_tp *self[1] = {tp};
        if (validate_fp8(tp, a, false) == WS_OK && group_prelude(self, 1, &ncta, &same) == WS_OK) {
            const int skb = (int)((dw->k0 + dw->k - 1) / dw->block_k - dw->k0 / dw->block_k + 1);
            const int mt = fp8_rows_per_launch(tp, a, ncta, a.m, false);
            direct = true;
            stage = !(bs_wanted(tp, mt, a, false) && bs_plan(a, mt, skb, ncta, true).ok);
            if (!stage) a.x = pin;
        }
    }

    ws_tp::HostGraph *hit = nullptr;
    const uint64_t hkey = hash_fp8_args(a, pin, dev, tp->kernel_sel * 4 + tp->split * 2 + tp->pdl);
    {
        auto it = tp->hgraphs.find(hkey);
        if (it != tp->hgraphs.end()) {
            ws_tp::HostGraph &g = it->second;
            if (g.exec && g.pin == pin && g.dev == dev && g.kernel_sel == tp->kernel_sel && g.split == tp->split &&
                g.pdl == tp->pdl && same_fp8_args(g.key, a)) {
                hit = &g;
            } else {  // a hash collision or a re-sized staging buffer: the stale graph goes
                if (g.exec) cudaGraphExecDestroy(g.exec);
                tp->hgraphs.erase(it);
            }
        }
    }
    tp->host_done_arm = tp->pin_done;
    if (!hit) {  // capture; any failure falls back to plain enqueueing below
        const uint64_t step0 = tp->step, launches0 = tp->launches;
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        bool ok = cudaStreamBeginCapture(tp->hstream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        if (ok) {
            ok = host_stage_in(tp, dev, pin, xb, direct, stage);
            ok = ok && ws_fp8_rowpar_gemm_allreduce(tp, &a, tp->hstream) == WS_OK;
            const bool ended = cudaStreamEndCapture(tp->hstream, &graph) == cudaSuccess && graph != nullptr;
            ok = ok && ended && cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
            if (graph) cudaGraphDestroy(graph);
        }
        const uint64_t steps = tp->step - step0, launches = tp->launches - launches0;
        tp->step = step0;  // nothing ran yet: the replay below (or the fallback) counts the step
        tp->launches = launches0;
        cudaGetLastError();
        if (ok && exec) {
            if (tp->hgraphs.size() >= 1024) {  // one per weight a caller cycles through; evict the least recently used
                auto old = tp->hgraphs.begin();
                for (auto it = tp->hgraphs.begin(); it != tp->hgraphs.end(); ++it)
                    if (it->second.used < old->second.used) old = it;
                if (old->second.exec) cudaGraphExecDestroy(old->second.exec);
                tp->hgraphs.erase(old);
            }
            ws_tp::HostGraph *slot = &tp->hgraphs[hkey];
            slot->key = a; slot->pin = pin; slot->dev = dev;
            slot->kernel_sel = tp->kernel_sel; slot->split = tp->split; slot->pdl = tp->pdl;
            slot->steps = steps; slot->launches = launches; slot->exec = exec;
            hit = slot;
        }
    }
    memcpy(pin, x_host, xb);
    *done = 0;
    if (hit) {
        hit->used = ++tp->hgraph_clock;
        s = cudaGraphLaunch(hit->exec, tp->hstream) == cudaSuccess ? WS_OK : WS_ERR_CUDA;
        if (s == WS_OK) {
            tp->step += hit->steps;
            tp->launches += hit->launches;
        }
    } else {
        s = host_stage_in(tp, dev, pin, xb, direct, stage) ? WS_OK : WS_ERR_CUDA;
        if (s == WS_OK) s = ws_fp8_rowpar_gemm_allreduce(tp, &a, tp->hstream);
    }
    tp->host_done_arm = nullptr;
    if (s != WS_OK) {
        if (s == WS_ERR_CUDA) return fail(tp, WS_ERR_CUDA, "enqueueing the host-buffer step failed: %s", cudaGetErrorString(cudaGetLastError()));
        return s;
    }
    return host_wait_and_copy_out(tp, done, out_host, pin + xb_al, ob);
}

// ------------------------------------------------------------------------------ act quant
ws_status_t ws_act_quant_fp8(const void *x, int64_t ldx, int32_t x_dtype, int32_t m, int32_t k, uint8_t *q,
                             uint8_t *sexp, void *stream) {
    if (!x || !q || !sexp || m < 1 || k < 32 || k % 32) return WS_ERR_INVALID;
    const int xa = x_dtype == WS_ACT_BF16 ? 8 : 4;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7) || ldx % xa || ldx < k) return WS_ERR_INVALID;
    const int64_t total = (int64_t)m * (k / 8);
    const unsigned blocks = (unsigned)((total + 255) / 256);
    act_quant_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, ldx, x_dtype, m, k, q, sexp);
    return cudaGetLastError() == cudaSuccess ? WS_OK : WS_ERR_CUDA;
}

// 0 (default): automatic; 1: the mma.sync kernels; 2: the block-scaled tcgen05 kernels wherever the shape
// fits; 3: the CUDA-core kernels (FP8: as automatic for one or two rows, mma.sync beyond; MoE: the decode form).
ws_status_t ws_tp_set_kernel(ws_tp_t *tp, int32_t which) {
    if (!tp || which < 0 || which > 3) return WS_ERR_INVALID;
    tp->kernel_sel = which;
    tp->moe_bs = which == 3 ? 0 : 1;
    return WS_OK;
}

// 1 (default): leftover rows are dealt out row by row; 0: each leftover tile goes to one CTA whole.
ws_status_t ws_tp_set_split(ws_tp_t *tp, int32_t on) {
    if (!tp) return WS_ERR_INVALID;
    tp->split = on ? 1 : 0;
    return WS_OK;
}


// ------------------------------------------------------------------------------ no allocation
// Scratch for ws_fp8_gemm_static_scratch: what the kernel keeps in device memory outside its
// operands (arrival counters, the status word, the step counter).  It lives in the library
// image, so every GPU that loads the library holds these bytes until the process exits.
constexpr size_t kStaticScratchBytes = WS_STATIC_SCRATCH_BYTES;
static_assert((kMaxShared + 8) * sizeof(uint32_t) <= kStaticScratchBytes, "the static scratch is too small for the kernel's counters");
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kStaticMaxDevices = 64;
unsigned char *g_static_scratch_addr[kStaticMaxDevices] = {};
int g_static_sm_count[kStaticMaxDevices] = {};
std::mutex g_static_mutex;

void set_err(char *err, size_t len, const char *fmt, ...) {
    if (!err || !len) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, len, fmt, ap);
    va_end(ap);
}
}  // namespace

ws_status_t ws_fp8_gemm_static_scratch(const ws_fp8_gemm_args_t *a, int32_t device, void *stream, char *err,
                                       size_t err_len) {
    if (err && err_len) err[0] = 0;
    if (!a) { set_err(err, err_len, "null args"); return WS_ERR_INVALID; }
    if (device < 0 || device >= kStaticMaxDevices) { set_err(err, err_len, "device %d out of range", device); return WS_ERR_INVALID; }
    ws_tp probe_err;  // only carries validate_fp8's message; owns no device memory
    ws_status_t st = validate_fp8(&probe_err, *a, false);
    if (st != WS_OK) { set_err(err, err_len, "%s", probe_err.err.c_str()); return st; }
    if (a->m > WS_STATIC_MAX_M) {
        set_err(err, err_len, "m=%d exceeds the %d activation rows the static scratch is laid out for", a->m, WS_STATIC_MAX_M);
        return WS_ERR_CAPACITY;
    }
    if (a->n > WS_STATIC_MAX_N) {
        set_err(err, err_len, "n=%d exceeds the static-scratch limit of %d output rows", a->n, WS_STATIC_MAX_N);
        return WS_ERR_CAPACITY;
    }
    cudaError_t ce = cudaSetDevice(device);
    if (ce != cudaSuccess) { set_err(err, err_len, "cudaSetDevice(%d): %s", device, cudaGetErrorString(ce)); return WS_ERR_CUDA; }
    {   // set-up, once per device, with that device current: the array's name is only a host-side
        // stand-in, the address a kernel may use comes from cudaGetSymbolAddress
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!g_static_scratch_addr[device]) {
            void *ptr = nullptr;
            ce = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (ce != cudaSuccess || !ptr) {
                set_err(err, err_len, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(ce));
                return WS_ERR_CUDA;
            }
            int sms = 0;
            ce = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
            if (ce == cudaSuccess) ce = cudaFuncSetAttribute(fp8_rowpar_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (ce != cudaSuccess) { set_err(err, err_len, "device set-up: %s", cudaGetErrorString(ce)); return WS_ERR_CUDA; }
            g_static_sm_count[device] = sms;
            g_static_scratch_addr[device] = static_cast<unsigned char *>(ptr);
        }
    }
    unsigned char *base = g_static_scratch_addr[device];
    const int ncta = std::min(g_static_sm_count[device], (int)kMaxCtas);
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    // counters, status word and step counter must start at zero
    ce = cudaMemsetAsync(base, 0, (kMaxShared + 8) * sizeof(uint32_t), cs);
    if (ce != cudaSuccess) { set_err(err, err_len, "cudaMemsetAsync: %s", cudaGetErrorString(ce)); return WS_ERR_CUDA; }

    Fp8Params p{};
    p.m = a->m; p.n = a->n; p.k = a->k; p.x_dtype = a->x_dtype; p.scale_kind = a->scale_kind;
    p.bn = a->block_n; p.bk = a->block_k; p.world = 1; p.mode = kModeAllReduce;
    for (p.bk_shift = 0; (1 << p.bk_shift) < p.bk; ++p.bk_shift) {}
    for (p.bn_shift = 0; (1 << p.bn_shift) < p.bn; ++p.bn_shift) {}
    p.mp = p.m <= 1 ? 1 : p.m <= 2 ? 2 : p.m <= 4 ? 4 : 8;
    p.timeout_ns = 2000000000ull;
    const int kbox = (p.k + 127) / 128;
    const int Gm = p.n / kGroupRows / ncta;
    p.skb = (int)((a->k0 + a->k - 1) / a->block_k - a->k0 / a->block_k + 1);
    p.nslot_max = (Gm * kGroupRows) / p.bn + 2 + 2;
    p.ragged = Gm < 8 ? 1 : 0;
    p.gran = ragged_granularity(p.n, ncta);
    p.part_rows = (Gm + 2) * kGroupRows;
    const Fp8Smem fixed = fp8_smem_layout(0, kbox, p.mp, p.nslot_max, p.skb, p.m, p.part_rows, 0);
    p.stage_bytes = fp8_stage_boxes(kbox) * kBoxBytes;
    int ns = std::min((kSmemBudget - fixed.total) / p.stage_bytes, (int)kMaxStages);
    if (ns < 2) { set_err(err, err_len, "shapes m=%d n=%d k=%d leave no room for the weight stage ring", p.m, p.n, p.k); return WS_ERR_CAPACITY; }
    p.nstages = ns;
    const size_t smem = (size_t)fp8_smem_layout(ns, kbox, p.mp, p.nslot_max, p.skb, p.m, p.part_rows, 0).total + 1024;
    Fp8RankArgs &r = p.r[0];
    for (int b = 0; b < 2; ++b) {
        st = make_tmap(&probe_err, &p.tmap[0][b], a->w, (uint64_t)a->n, (uint64_t)a->k, (uint64_t)a->ldw,
                       b ? (uint32_t)p.gran : (uint32_t)kGroupRows);
        if (st != WS_OK) { set_err(err, err_len, "%s", probe_err.err.c_str()); return st; }
    }
    r.x = a->x; r.scales = a->scales; r.out = a->out;
    r.ldx = a->ldx; r.scale_ld = a->scale_ld; r.row0 = a->row0; r.k0 = a->k0;
    r.ctx.counters = reinterpret_cast<uint32_t *>(base);
    r.ctx.status = r.ctx.counters + kMaxShared;
    r.ctx.step_ctr = r.ctx.counters + kMaxShared + 2;
    r.ctx.rank = 0;
    fp8_rowpar_kernel<0><<<dim3((unsigned)ncta, 1, 1), kThreads, smem, cs>>>(p);
    ce = cudaGetLastError();
    if (ce != cudaSuccess) { set_err(err, err_len, "kernel launch: %s", cudaGetErrorString(ce)); return WS_ERR_CUDA; }
    return WS_OK;
}

// Completion check for ws_fp8_gemm_static_scratch: the kernel records a bounded wait that gave up
// in the scratch array's status word; this reads it back (no allocation: a stream synchronise and
// a 4-byte copy into a local) and turns it into a status, as ws_tp_check does for an endpoint.
ws_status_t ws_fp8_gemm_static_scratch_check(int32_t device, void *stream, char *err, size_t err_len) {
    if (err && err_len) err[0] = 0;
    if (device < 0 || device >= kStaticMaxDevices) { set_err(err, err_len, "device %d out of range", device); return WS_ERR_INVALID; }
    unsigned char *base;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        base = g_static_scratch_addr[device];
    }
    if (!base) { set_err(err, err_len, "ws_fp8_gemm_static_scratch has not run on device %d", device); return WS_ERR_INVALID; }
    cudaError_t ce = cudaSetDevice(device);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    uint32_t st = 0;
    if (ce == cudaSuccess) ce = cudaMemcpy(&st, base + kMaxShared * sizeof(uint32_t), sizeof st, cudaMemcpyDeviceToHost);
    if (ce != cudaSuccess) { set_err(err, err_len, "reading the status word: %s", cudaGetErrorString(ce)); return WS_ERR_CUDA; }
    if (st == 0) return WS_OK;
    set_err(err, err_len, "%s", describe_status(st, 2000000000ull).c_str());
    return -(ws_status_t)(st & 0xFFu);
}

}  // extern "C"
