// C ABI of libtalu_gaf.so (declared in include/talu_gaf.h): context, weight
// upload / tensor-parallel sharding, dispatch of the matmul operator, NCCL
// exchange for row-parallel outputs.  No CPU fallback: every compute entry
// point needs a CUDA device and fails with a status code otherwise.
#include "../../include/talu_gaf.h"
#include "gaf_internal.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <thread>
#include <vector>

using namespace tgaf;

// ---------------------------------------------------------------------------
// NCCL, bound at run time (the library is usable single-GPU without it)
// ---------------------------------------------------------------------------
namespace {

struct NcclUniqueId {
    char internal[TGAF_COMM_ID_BYTES];
};
typedef void *NcclComm;
enum { kNcclSuccess = 0, kNcclInProgress = 7, kNcclSum = 0, kNcclMin = 3, kNcclUint8 = 1, kNcclInt32 = 2, kNcclFloat32 = 7, kNcclBfloat16 = 9 };

struct NcclApi {
    void *handle = nullptr;
    int (*GetUniqueId)(NcclUniqueId *) = nullptr;
    int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*CommAbort)(NcclComm) = nullptr;
    int (*CommGetAsyncError)(NcclComm, int *) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool ok = false;
    std::string why;
};

NcclApi &nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api;
    tried = true;
    // TGAF_NCCL_LIBRARY names another build of the collective library (same C API)
    const char *names[] = {getenv("TGAF_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n || !n[0]) continue;
        api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) break;
    }
    if (!api.handle) {
        api.why = "libnccl.so.2 not found";
        return api;
    }
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(api.handle, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(api.handle, "ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(api.handle, "ncclCommDestroy"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(dlsym(api.handle, "ncclCommAbort"));
    api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(dlsym(api.handle, "ncclCommGetAsyncError"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(api.handle, "ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(api.handle, "ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(api.handle, "ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.GetErrorString;
    if (!api.ok) api.why = "libnccl is missing a required symbol";
    return api;
}

}  // namespace

// ---------------------------------------------------------------------------
// objects
// ---------------------------------------------------------------------------
struct tgaf_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 148;
    Scratch scratch = {nullptr, 0, nullptr, 0, nullptr, 0};
    GemvTuning tune = {0, 1, 0, 0, 0, 0, 2, nullptr, nullptr};
    // staging for the *_host entry points
    void *stage_x = nullptr;
    size_t stage_x_bytes = 0;
    void *stage_y = nullptr;
    size_t stage_y_bytes = 0;
    unsigned int *d_error_word = nullptr;
    // queued host-buffer calls: copies run on their own streams around the kernels, over a small ring of
    // staging buffers (tgaf_linear_bf16_host_async)
    static constexpr int kPipe = 4;
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
    void *pipe_x[kPipe] = {nullptr, nullptr, nullptr, nullptr};
    void *pipe_y[kPipe] = {nullptr, nullptr, nullptr, nullptr};
    size_t pipe_x_bytes[kPipe] = {0, 0, 0, 0}, pipe_y_bytes[kPipe] = {0, 0, 0, 0};
    cudaEvent_t ev_x_ready[kPipe] = {nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t ev_k_done[kPipe] = {nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t ev_y_done[kPipe] = {nullptr, nullptr, nullptr, nullptr};
    uint64_t pipe_calls = 0;
    // FFN operator: intermediate activations and the two-operation kernel's arrival counters
    void *ffn_mid = nullptr;
    size_t ffn_mid_bytes = 0;
    unsigned int *d_grid_bar = nullptr;
    // tensor-core GEMM: one fp32 partial tile per CTA and the flags that announce them
    float *gemm_ws = nullptr;
    size_t gemm_ws_bytes = 0;
    unsigned int *gemm_flags = nullptr;
    size_t gemm_flag_count = 0;
    std::vector<tgaf_batch *> batches;   // live launch lists (their counters are reset after an abandoned launch)
    NcclComm comm = nullptr;
    uint32_t comm_rank = 0, comm_size = 1;
    PeerComm peer = {{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr}, 0, 1, false};
    int peer_allreduce = 1;  // small tiles go through the peer-memory kernel when the mapping exists
    uint32_t gemm_min_m = 17;  // activation rows from which the tensor-core GEMM takes over from the decode GEMVs
    int fused_allreduce = 1; // tgaf_linear_bf16_allreduce sums inside the GEMV when it can
    int ffn_one_launch = 1;  // tgaf_ffn_swiglu_bf16 runs both linears in one kernel when it can
    int peer_pdl = 0;        // programmatic stream serialization for the all-reduce kernel (measured slower)
    int peer_expect_absent_rank = 0;  // diagnostic: the all-reduce kernel also waits for a rank that does not exist
    uint32_t comm_timeout_ms = 30000; // wall-clock limit of tgaf_synchronize while a communicator exists (0 = wait for ever)
    // tensor maps of raw-pointer weights (tgaf_gaffine_u*_matvec_f32), keyed on pointers and dimensions
    static constexpr int kRawCache = 32;
    WeightView raw_cache[kRawCache];
    int raw_cache_used = 0, raw_cache_next = 0;
    char err[512] = {0};
};

namespace {
void peer_teardown(tgaf_ctx *ctx);
}

// A launch list of device-buffer linears (tgaf_batch_*): one kernel launch when the list qualifies, the calls one
// after the other otherwise.
struct tgaf_batch {
    GemvList *list = nullptr;
    unsigned long long *tagged = nullptr;   // the list's own split-K words (its operations overlap in time)
    size_t tagged_bytes = 0;
    uint32_t m = 0;
    std::vector<const tgaf_weight *> weights;
    std::vector<const void *> xs;
    std::vector<void *> ys;
    std::vector<uint8_t> deps, reduce;
};

// A recorded list of queued host-buffer calls (tgaf_host_batch_*): the CUDA graph of their copies and kernels.
struct tgaf_host_batch {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint32_t count = 0;
    // staged form: all activations in one device block, all outputs in another, one launch list between the copies
    tgaf_batch *inner = nullptr;
    uint8_t *d_x = nullptr, *d_y = nullptr;
};

struct tgaf_weight {
    WeightView v;
    bool owns = false;
    uint64_t full_N = 0, full_K = 0;
    uint32_t shard_kind = 0, tp_rank = 0, tp_size = 1;
};

namespace {

int32_t fail(tgaf_ctx *ctx, int32_t status, const char *fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof ctx->err, fmt, ap);
        va_end(ap);
    }
    return status;
}

int32_t cuda_fail(tgaf_ctx *ctx, cudaError_t e, const char *what) {
    const int32_t st = (e == cudaErrorMemoryAllocation) ? TGAF_ERR_OUT_OF_MEMORY : TGAF_ERR_CUDA;
    return fail(ctx, st, "%s: %s", what, cudaGetErrorString(e));
}

#define TGAF_CUDA(ctx, call)                                  \
    do {                                                      \
        cudaError_t e__ = (call);                             \
        if (e__ != cudaSuccess) return cuda_fail(ctx, e__, #call); \
    } while (0)

// Shape rules of the reference (gaffine_u4_matvec.zig:99-113, engine.zig:8229-8233,
// transforms.zig:158-185).
bool shape_ok(uint64_t N, uint64_t K, uint32_t group, uint32_t bits, uint32_t sdtype) {
    if (bits != 4 && bits != 8) return false;
    const uint32_t vpw = 32u / bits;
    if (N == 0 || K == 0 || group == 0) return false;
    if (K % vpw != 0 || group % vpw != 0) return false;
    if (K % group != 0) return false;
    if (sdtype != TGAF_SCALES_F16 && sdtype != TGAF_SCALES_BF16) return false;
    if (K / group > 1024) return false;               // MAX_SUPPORTED_GAFFINE_GROUPS
    if (N > 0x7FFFFFFFull || K > 0x7FFFFFFFull) return false;
    if (K * bits / 8 > 0xFFFFFFFFull) return false;
    return true;
}

int32_t ensure_scratch(tgaf_ctx *ctx, size_t partial_bytes, size_t counters, size_t tagged_bytes = 0) {
    if (tagged_bytes > ctx->scratch.tagged_bytes) {
        TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->scratch.tagged) cudaFree(ctx->scratch.tagged);
        ctx->scratch.tagged = nullptr;
        ctx->scratch.tagged_bytes = 0;
        size_t want = tagged_bytes < (size_t(2) << 20) ? (size_t(2) << 20) : tagged_bytes;
        TGAF_CUDA(ctx, cudaMalloc(reinterpret_cast<void **>(&ctx->scratch.tagged), want));
        TGAF_CUDA(ctx, cudaMemsetAsync(ctx->scratch.tagged, 0, want, ctx->stream));  // no tag is set
        ctx->scratch.tagged_bytes = want;
    }
    if (partial_bytes > ctx->scratch.partial_bytes) {
        // previous launches may still be using the old buffer
        TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->scratch.partials) cudaFree(ctx->scratch.partials);
        ctx->scratch.partials = nullptr;
        ctx->scratch.partial_bytes = 0;
        size_t want = partial_bytes < (size_t(8) << 20) ? (size_t(8) << 20) : partial_bytes;
        TGAF_CUDA(ctx, cudaMalloc(&ctx->scratch.partials, want));
        ctx->scratch.partial_bytes = want;
    }
    if (counters > ctx->scratch.counter_count) {
        TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->scratch.counters) cudaFree(ctx->scratch.counters);
        ctx->scratch.counters = nullptr;
        ctx->scratch.counter_count = 0;
        size_t want = counters < 65536 ? 65536 : counters;
        TGAF_CUDA(ctx, cudaMalloc(&ctx->scratch.counters, want * sizeof(unsigned int)));
        TGAF_CUDA(ctx, cudaMemsetAsync(ctx->scratch.counters, 0, want * sizeof(unsigned int), ctx->stream));
        ctx->scratch.counter_count = want;
    }
    return TGAF_OK;
}

int32_t ensure_stage(tgaf_ctx *ctx, void **buf, size_t *have, size_t need) {
    if (need <= *have) return TGAF_OK;
    TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (*buf) cudaFree(*buf);
    *buf = nullptr;
    *have = 0;
    size_t want = need < (size_t(1) << 20) ? (size_t(1) << 20) : need;
    TGAF_CUDA(ctx, cudaMalloc(buf, want));
    *have = want;
    return TGAF_OK;
}

// The operator: picks the kernel for (shape, M) and enqueues it.
// `reduce`: also sum y over the communicator's ranks (inside the GEMV when it can, else a separate all-reduce).
int32_t allreduce_device(tgaf_ctx *ctx, void *d_buf, uint64_t count, uint32_t dtype);

int32_t linear_device(tgaf_ctx *ctx, const WeightView &w, const void *x, uint32_t M, void *y, bool f32, bool reduce = false) {
    // the next-weight hint belongs to exactly one call, whichever kernel that call ends up on
    const WeightView *hint = ctx->tune.next;
    ctx->tune.next = nullptr;
    if (!x || !y) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null activation or output pointer");
    if (M == 0) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "M must be > 0");
    const size_t elt = f32 ? 4 : 2;
    TGAF_CUDA(ctx, cudaSetDevice(ctx->device));  // scratch growth and launches below belong to the context's device

    if (!f32 && gemm_tc_eligible(w, M, ctx->gemm_min_m)) {
        if (!ctx->gemm_ws) {
            // first GEMM on this context: the split-tile workspace (38 MB on 148 SMs) and its flags
            const size_t wb = gemm_tc_workspace_bytes(ctx->sm_count), fc = gemm_tc_flag_count(ctx->sm_count);
            TGAF_CUDA(ctx, cudaMalloc(reinterpret_cast<void **>(&ctx->gemm_flags), fc * sizeof(unsigned int)));
            ctx->gemm_flag_count = fc;
            TGAF_CUDA(ctx, cudaMemsetAsync(ctx->gemm_flags, 0, fc * sizeof(unsigned int), ctx->stream));
            TGAF_CUDA(ctx, cudaMalloc(reinterpret_cast<void **>(&ctx->gemm_ws), wb));
            ctx->gemm_ws_bytes = wb;
        }
        cudaError_t e = gemm_tc(w, x, y, M, ctx->stream, ctx->sm_count, ctx->d_error_word, ctx->gemm_ws, ctx->gemm_ws_bytes,
                                ctx->gemm_flags, ctx->gemm_flag_count);
        if (e == cudaSuccess)
            return reduce ? allreduce_device(ctx, y, static_cast<uint64_t>(M) * w.N, TGAF_DTYPE_BF16) : TGAF_OK;
        if (e != cudaErrorNotSupported) return cuda_fail(ctx, e, "gemm_tc");
    }

    if (!ctx->tune.force_generic && gemv_mma_eligible(w, x, y, f32)) {
        // rows in chunks of 16; each chunk streams the weights once
        const uint32_t step = gemv_mma_max_rows(w, f32);
        for (uint32_t m0 = 0; m0 < M; m0 += step) {
            const uint32_t mc = (M - m0) < step ? (M - m0) : step;
            const size_t need = gemv_mma_scratch_bytes(w, mc, ctx->tune, ctx->sm_count);
            int32_t st = ensure_scratch(ctx, need, gemv_mma_counter_count(w),
                                        gemv_tagged_bytes(w, mc, f32, ctx->tune, ctx->sm_count));
            if (st != TGAF_OK) return st;
            const void *xp = static_cast<const uint8_t *>(x) + static_cast<size_t>(m0) * w.K * elt;
            void *yp = static_cast<uint8_t *>(y) + static_cast<size_t>(m0) * w.N * elt;
            GemvTuning t = ctx->tune;
            t.next = m0 + step >= M ? hint : nullptr;  // the last chunk is the one the next launch follows
            t.fuse = nullptr;
            if (reduce && M <= 16u && ctx->peer.ok && ctx->fused_allreduce) {
                t.fuse = &ctx->peer;
                if (gemv_fused_eligible(w, mc, f32, t)) {
                    cudaError_t e = gemv_mma(w, xp, yp, mc, f32, ctx->scratch, t, ctx->stream, ctx->sm_count, ctx->d_error_word);
                    if (e == cudaSuccess) return TGAF_OK;  // y is already the sum over the ranks
                    if (e != cudaErrorNotSupported) return cuda_fail(ctx, e, "fused gemv launch");
                }
                t.fuse = nullptr;
            }
            cudaError_t e = gemv_mma(w, xp, yp, mc, f32, ctx->scratch, t, ctx->stream, ctx->sm_count,
                                     ctx->d_error_word);
            if (e != cudaSuccess) return cuda_fail(ctx, e, "gemv_mma launch");
        }
        return reduce ? allreduce_device(ctx, y, static_cast<uint64_t>(M) * w.N, f32 ? TGAF_DTYPE_F32 : TGAF_DTYPE_BF16) : TGAF_OK;
    }
    cudaError_t e = gemv_generic(w, x, y, M, f32, ctx->stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "gemv_generic launch");
    return reduce ? allreduce_device(ctx, y, static_cast<uint64_t>(M) * w.N, f32 ? TGAF_DTYPE_F32 : TGAF_DTYPE_BF16) : TGAF_OK;
}

int32_t linear_host(tgaf_ctx *ctx, const tgaf_weight *w, const void *xh, uint32_t M, void *yh, bool f32, bool wait = true) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!w || !xh || !yh || M == 0) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null pointer or M == 0");
    const size_t elt = f32 ? 4 : 2;
    const size_t xb = static_cast<size_t>(M) * w->v.K * elt, yb = static_cast<size_t>(M) * w->v.N * elt;
    TGAF_CUDA(ctx, cudaSetDevice(ctx->device));
    int32_t st = ensure_stage(ctx, &ctx->stage_x, &ctx->stage_x_bytes, xb);
    if (st != TGAF_OK) return st;
    st = ensure_stage(ctx, &ctx->stage_y, &ctx->stage_y_bytes, yb);
    if (st != TGAF_OK) return st;
    TGAF_CUDA(ctx, cudaMemcpyAsync(ctx->stage_x, xh, xb, cudaMemcpyHostToDevice, ctx->stream));
    st = linear_device(ctx, w->v, ctx->stage_x, M, ctx->stage_y, f32);
    if (st != TGAF_OK) return st;
    TGAF_CUDA(ctx, cudaMemcpyAsync(yh, ctx->stage_y, yb, cudaMemcpyDeviceToHost, ctx->stream));
    if (wait) TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return TGAF_OK;
}

int32_t raw_matvec(tgaf_ctx *ctx, uint32_t bits, const float *input, const uint32_t *packed,
                   const uint16_t *scales, const uint16_t *biases, float *out, uint32_t in_dim,
                   uint32_t out_dim, uint32_t group_size, uint32_t sdtype, uint32_t batch_rows) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    // validateArgs, core/src/compute/cuda/gaffine_u4_matvec.zig:99-113
    const uint32_t vpw = 32u / bits;
    if (in_dim == 0 || out_dim == 0 || group_size == 0 || batch_rows == 0)
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "zero dimension");
    if (in_dim % vpw != 0 || group_size % vpw != 0)
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "in_dim and group_size must be multiples of %u", vpw);
    if (in_dim % group_size != 0) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "in_dim %% group_size != 0");
    if (sdtype != TGAF_SCALES_F16 && sdtype != TGAF_SCALES_BF16)
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "bad scales dtype tag %u", sdtype);
    if (!input || !packed || !scales || !biases || !out)
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null device pointer");
    WeightView v;
    v.packed = reinterpret_cast<const uint8_t *>(packed);
    v.scales = scales;
    v.biases = biases;
    v.N = out_dim;
    v.K = in_dim;
    v.group = group_size;
    v.bits = bits;
    v.sdtype = sdtype;
    v.row_bytes = in_dim / vpw * 4u;
    v.groups = in_dim / group_size;
    // a decoder calls this once per token and weight with the same pointers: encode the tensor maps once
    for (int i = 0; i < ctx->raw_cache_used; ++i) {
        const WeightView &c = ctx->raw_cache[i];
        if (c.packed == v.packed && c.scales == v.scales && c.biases == v.biases && c.N == v.N && c.K == v.K &&
            c.group == v.group && c.bits == v.bits && c.sdtype == v.sdtype)
            return linear_device(ctx, c, input, batch_rows, out, true);
    }
    attach_packed_tmap(v);
    const int slot = ctx->raw_cache_used < tgaf_ctx::kRawCache ? ctx->raw_cache_used++ : (ctx->raw_cache_next++ % tgaf_ctx::kRawCache);
    ctx->raw_cache[slot] = v;
    return linear_device(ctx, ctx->raw_cache[slot], input, batch_rows, out, true);
}

}  // namespace

// ---------------------------------------------------------------------------
// exported functions
// ---------------------------------------------------------------------------
namespace {

// Unmaps the peers' regions and frees the local one.  Safe at any time after the stream is idle: a rank's
// last all-reduce returns only after every peer's last push into this rank's region has arrived.
void peer_teardown(tgaf_ctx *ctx) {
    PeerComm &pc = ctx->peer;
    for (uint32_t r = 0; r < static_cast<uint32_t>(kPeerMaxRanks); ++r) {
        if (!pc.region[r]) continue;
        if (r == pc.rank)
            cudaFree(pc.region[r]);
        else
            cudaIpcCloseMemHandle(pc.region[r]);
        pc.region[r] = nullptr;
    }
    pc.ok = false;
}

// Maps every rank's all-reduce region into this process (CUDA IPC; the handles travel by ncclAllGather).
// Any failure, on any rank, leaves ALL ranks on the NCCL path: the outcome is agreed by an all-reduce(min).
void peer_setup(tgaf_ctx *ctx, NcclApi &api) {
    PeerComm &pc = ctx->peer;
    pc.rank = ctx->comm_rank;
    pc.size = ctx->comm_size;
    pc.ok = false;
    if (!api.AllGather || pc.size < 1 || pc.size > static_cast<uint32_t>(kPeerMaxRanks)) return;
    const char *env = getenv("TGAF_PEER_ALLREDUCE");
    const bool wanted = !(env && env[0] == '0');
    int good = wanted ? 1 : 0;
    cudaIpcMemHandle_t mine;
    memset(&mine, 0, sizeof mine);
    void *local = nullptr;
    if (good && cudaMalloc(&local, peer_region_bytes()) != cudaSuccess) good = 0, local = nullptr;
    if (good && cudaMemset(local, 0, peer_region_bytes()) != cudaSuccess) good = 0;
    if (good && cudaIpcGetMemHandle(&mine, local) != cudaSuccess) good = 0;
    cudaGetLastError();
    // exchange {handle, good} of every rank
    constexpr size_t kRec = sizeof(cudaIpcMemHandle_t) + 8;
    uint8_t host[kPeerMaxRanks * kRec];
    memset(host, 0, sizeof host);
    uint8_t *d_all = nullptr;
    if (cudaMalloc(reinterpret_cast<void **>(&d_all), pc.size * kRec) != cudaSuccess) {
        // cannot even exchange: every rank must still enter the collectives below, so use no device scratch
        d_all = nullptr;
    }
    bool exchanged = false;
    if (d_all) {
        memcpy(host + pc.rank * kRec, &mine, sizeof mine);
        host[pc.rank * kRec + sizeof mine] = static_cast<uint8_t>(good);
        cudaMemcpy(d_all + pc.rank * kRec, host + pc.rank * kRec, kRec, cudaMemcpyHostToDevice);
        cudaDeviceSynchronize();  // the memset of the region is complete before anybody learns its handle
        if (api.AllGather(d_all + pc.rank * kRec, d_all, kRec, kNcclUint8, ctx->comm, ctx->stream) == kNcclSuccess &&
            cudaStreamSynchronize(ctx->stream) == cudaSuccess &&
            cudaMemcpy(host, d_all, pc.size * kRec, cudaMemcpyDeviceToHost) == cudaSuccess)
            exchanged = true;
    }
    if (!exchanged) good = 0;
    for (uint32_t r = 0; good && r < pc.size; ++r)
        if (!host[r * kRec + sizeof mine]) good = 0;
    if (good) {
        for (uint32_t r = 0; r < pc.size; ++r) {
            if (r == pc.rank) {
                pc.region[r] = local;
                continue;
            }
            cudaIpcMemHandle_t h;
            memcpy(&h, host + r * kRec, sizeof h);
            void *ptr = nullptr;
            if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                cudaGetLastError();
                good = 0;
                break;
            }
            pc.region[r] = ptr;
        }
    }
    // second agreement: did every rank map every region?
    if (d_all && exchanged) {
        int32_t flag = good;
        cudaMemcpy(d_all, &flag, sizeof flag, cudaMemcpyHostToDevice);
        if (api.AllReduce(d_all, d_all, 1, kNcclInt32, kNcclMin, ctx->comm, ctx->stream) == kNcclSuccess &&
            cudaStreamSynchronize(ctx->stream) == cudaSuccess &&
            cudaMemcpy(&flag, d_all, sizeof flag, cudaMemcpyDeviceToHost) == cudaSuccess)
            good = flag;
        else
            good = 0;
    }
    if (d_all) cudaFree(d_all);
    if (good) {
        pc.ok = true;
    } else {
        if (!pc.region[pc.rank] && local) cudaFree(local);
        peer_teardown(ctx);
    }
}

}  // namespace

extern "C" {

int32_t tgaf_abi_version(void) { return TGAF_ABI_VERSION; }

const char *tgaf_status_string(int32_t status) {
    switch (status) {
        case TGAF_OK: return "ok";
        case TGAF_ERR_INVALID_ARGUMENT: return "invalid argument";
        case TGAF_ERR_CUDA: return "CUDA error";
        case TGAF_ERR_OUT_OF_MEMORY: return "out of device memory";
        case TGAF_ERR_NCCL: return "NCCL error";
        case TGAF_ERR_UNSUPPORTED: return "unsupported";
        case TGAF_ERR_TIMEOUT: return "timeout";
        case TGAF_ERR_DEVICE_FLAG: return "device-side wait ran out";
        default: return "unknown status";
    }
}

int32_t tgaf_ctx_create(int32_t device_ordinal, void *stream, tgaf_ctx **out_ctx) {
    if (!out_ctx) return TGAF_ERR_INVALID_ARGUMENT;
    *out_ctx = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) return TGAF_ERR_CUDA;
    if (device_ordinal < 0 || device_ordinal >= count) return TGAF_ERR_INVALID_ARGUMENT;
    tgaf_ctx *ctx = new (std::nothrow) tgaf_ctx();
    if (!ctx) return TGAF_ERR_OUT_OF_MEMORY;
    ctx->device = device_ordinal;
    if (cudaSetDevice(device_ordinal) != cudaSuccess) {
        delete ctx;
        return TGAF_ERR_CUDA;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) {
        delete ctx;
        return TGAF_ERR_CUDA;
    }
    if (prop.major != 10) {  // the kernels are sm_100a only; nothing else is compiled in
        delete ctx;
        return TGAF_ERR_UNSUPPORTED;
    }
    ctx->sm_count = prop.multiProcessorCount;
    if (stream) {
        ctx->stream = static_cast<cudaStream_t>(stream);
    } else {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete ctx;
            return TGAF_ERR_CUDA;
        }
        ctx->owns_stream = true;
    }
    if (cudaMalloc(&ctx->d_error_word, sizeof(unsigned int)) != cudaSuccess ||
        cudaMemsetAsync(ctx->d_error_word, 0, sizeof(unsigned int), ctx->stream) != cudaSuccess) {
        tgaf_ctx_destroy(ctx);
        return TGAF_ERR_CUDA;
    }
    // split-K scratch up front so that steady-state calls never allocate
    if (ensure_scratch(ctx, size_t(8) << 20, 65536) != TGAF_OK) {
        tgaf_ctx_destroy(ctx);
        return TGAF_ERR_OUT_OF_MEMORY;
    }
    *out_ctx = ctx;
    return TGAF_OK;
}

int32_t tgaf_ctx_destroy(tgaf_ctx *ctx) {
    if (!ctx) return TGAF_OK;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->comm) {
        // tearing a context down must never block (ncclCommDestroy waits for anything that still refers
        // to the communicator, e.g. a captured graph the caller has not released): abort instead
        NcclApi &api = nccl_api();
        if (api.ok && api.CommAbort) api.CommAbort(ctx->comm);
        ctx->comm = nullptr;
    }
    peer_teardown(ctx);
    while (!ctx->batches.empty()) tgaf_batch_destroy(ctx, ctx->batches.back());   // launch lists the caller left behind
    if (ctx->scratch.partials) cudaFree(ctx->scratch.partials);
    if (ctx->scratch.counters) cudaFree(ctx->scratch.counters);
    if (ctx->scratch.tagged) cudaFree(ctx->scratch.tagged);
    if (ctx->stage_x) cudaFree(ctx->stage_x);
    if (ctx->stage_y) cudaFree(ctx->stage_y);
    if (ctx->d_error_word) cudaFree(ctx->d_error_word);
    for (int i = 0; i < tgaf_ctx::kPipe; ++i) {
        if (ctx->pipe_x[i]) cudaFree(ctx->pipe_x[i]);
        if (ctx->pipe_y[i]) cudaFree(ctx->pipe_y[i]);
        if (ctx->ev_x_ready[i]) cudaEventDestroy(ctx->ev_x_ready[i]);
        if (ctx->ev_k_done[i]) cudaEventDestroy(ctx->ev_k_done[i]);
        if (ctx->ev_y_done[i]) cudaEventDestroy(ctx->ev_y_done[i]);
    }
    if (ctx->h2d_stream) cudaStreamDestroy(ctx->h2d_stream);
    if (ctx->d2h_stream) cudaStreamDestroy(ctx->d2h_stream);
    if (ctx->ffn_mid) cudaFree(ctx->ffn_mid);
    if (ctx->d_grid_bar) cudaFree(ctx->d_grid_bar);
    if (ctx->gemm_ws) cudaFree(ctx->gemm_ws);
    if (ctx->gemm_flags) cudaFree(ctx->gemm_flags);
    if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return TGAF_OK;
}

int32_t tgaf_ctx_set_stream(tgaf_ctx *ctx, void *stream) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!stream) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "stream must not be NULL");
    TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    ctx->owns_stream = false;
    ctx->stream = static_cast<cudaStream_t>(stream);
    return TGAF_OK;
}

int32_t tgaf_watchdog_wait(const tgaf_watch_fns *fns, void *user, uint32_t timeout_ms) {
    if (!fns || !fns->work_done) return TGAF_ERR_INVALID_ARGUMENT;
    const auto t0 = std::chrono::steady_clock::now();
    for (uint64_t it = 0;; ++it) {
        const int32_t done = fns->work_done(user);
        if (done > 0) return TGAF_OK;
        if (done < 0) return TGAF_ERR_CUDA;
        if (fns->async_error && fns->async_error(user) != 0) {
            if (fns->abort_comm) fns->abort_comm(user);
            return TGAF_ERR_NCCL;
        }
        const auto waited = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
        if (timeout_ms != 0 && waited >= static_cast<int64_t>(timeout_ms) * 1000) {
            if (fns->abort_comm) fns->abort_comm(user);
            return TGAF_ERR_TIMEOUT;
        }
        // a decode step is tens of microseconds: poll flat out for the first 2 ms, then yield between polls
        if (waited > 2000) std::this_thread::sleep_for(std::chrono::microseconds(it & 63 ? 50 : 500));
    }
}

namespace {
// tgaf_synchronize with a communicator: the stream may hold a collective that never completes when a rank is
// missing or has failed, so the wait polls instead of blocking and gives the communicator up at the limit.
struct CommWatch {
    tgaf_ctx *ctx;
    cudaError_t stream_error;
    int nccl_error;
};
int32_t watch_work_done(void *user) {
    CommWatch *cw = static_cast<CommWatch *>(user);
    cudaStream_t streams[3] = {cw->ctx->stream, cw->ctx->h2d_stream, cw->ctx->d2h_stream};
    for (cudaStream_t st : streams) {
        if (st == nullptr) continue;  // the copy streams exist only after a queued host-buffer call
        const cudaError_t e = cudaStreamQuery(st);
        if (e == cudaErrorNotReady) return 0;
        if (e != cudaSuccess) {
            cw->stream_error = e;
            return -1;
        }
    }
    return 1;
}
int32_t watch_async_error(void *user) {
    CommWatch *cw = static_cast<CommWatch *>(user);
    NcclApi &api = nccl_api();
    if (!cw->ctx->comm || !api.CommGetAsyncError) return 0;
    int async_err = 0;
    if (api.CommGetAsyncError(cw->ctx->comm, &async_err) != kNcclSuccess) async_err = -1;
    if (async_err == kNcclInProgress) async_err = 0;  // a non-blocking communicator still setting up
    cw->nccl_error = async_err;
    return async_err;
}
void watch_abort(void *user) {
    CommWatch *cw = static_cast<CommWatch *>(user);
    NcclApi &api = nccl_api();
    if (cw->ctx->comm && api.CommAbort) api.CommAbort(cw->ctx->comm);  // the library's kernels leave the stream
    cw->ctx->comm = nullptr;
    cw->ctx->comm_size = 1;
    cw->ctx->comm_rank = 0;
}
}  // namespace

int32_t tgaf_synchronize(tgaf_ctx *ctx) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    TGAF_CUDA(ctx, cudaSetDevice(ctx->device));
    if (ctx->comm && ctx->comm_timeout_ms != 0) {
        CommWatch cw = {ctx, cudaSuccess, 0};
        const tgaf_watch_fns fns = {watch_work_done, watch_async_error, watch_abort};
        const int32_t st = tgaf_watchdog_wait(&fns, &cw, ctx->comm_timeout_ms);
        if (st == TGAF_ERR_CUDA) return cuda_fail(ctx, cw.stream_error, "cudaStreamQuery");
        if (st != TGAF_OK) {
            // the communicator is gone; this library's own kernels give their waits up by themselves (bounded polls)
            cudaStreamSynchronize(ctx->stream);
            peer_teardown(ctx);
            if (st == TGAF_ERR_TIMEOUT)
                return fail(ctx, TGAF_ERR_TIMEOUT, "the stream did not finish within %u ms (a rank missing?): communicator aborted", ctx->comm_timeout_ms);
            NcclApi &api = nccl_api();
            return fail(ctx, TGAF_ERR_NCCL, "asynchronous communicator error (%s): communicator aborted",
                        cw.nccl_error > 0 && api.GetErrorString ? api.GetErrorString(cw.nccl_error) : "query failed");
        }
    }
    TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->d2h_stream) {  // queued host-buffer calls: their last copies run on the copy streams
        TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->h2d_stream));
        TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->d2h_stream));
    }
    unsigned int flag = 0;
    TGAF_CUDA(ctx, cudaMemcpy(&flag, ctx->d_error_word, sizeof flag, cudaMemcpyDeviceToHost));
    if (flag != 0) {
        cudaMemset(ctx->d_error_word, 0, sizeof flag);
        // an abandoned launch may have left arrival counters half way
        if (ctx->scratch.counters) cudaMemset(ctx->scratch.counters, 0, ctx->scratch.counter_count * sizeof(unsigned int));
        if (ctx->scratch.tagged) cudaMemset(ctx->scratch.tagged, 0, ctx->scratch.tagged_bytes);  // ... or tags set
        if (ctx->d_grid_bar) cudaMemset(ctx->d_grid_bar, 0, 4 * sizeof(unsigned int));
        if (ctx->gemm_flags) cudaMemset(ctx->gemm_flags, 0, ctx->gemm_flag_count * sizeof(unsigned int));
        for (tgaf_batch *b : ctx->batches) {
            if (b->list) gemv_list_reset(b->list);
            if (b->tagged) cudaMemset(b->tagged, 0, b->tagged_bytes);
        }
        return fail(ctx, TGAF_ERR_DEVICE_FLAG, "a kernel gave up a bounded wait (code 0x%x)", flag);
    }
    return TGAF_OK;
}

const char *tgaf_last_error(const tgaf_ctx *ctx) { return ctx ? ctx->err : "null context"; }

int32_t tgaf_ctx_set_option(tgaf_ctx *ctx, const char *name, int64_t value) {
    if (!ctx || !name) return TGAF_ERR_INVALID_ARGUMENT;
    if (!strcmp(name, "gemv_ctas")) {
        // the split-K collection and the two-operation launch wait on other CTAs of the same grid, so every
        // CTA must be resident at once: one per SM at most
        if (value < 0 || value > ctx->sm_count)
            return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "gemv_ctas must be 0 (one per SM) or 1..%d", ctx->sm_count);
        ctx->tune.ctas = static_cast<int>(value);
    } else if (!strcmp(name, "pdl")) {
        ctx->tune.pdl = value != 0;
    } else if (!strcmp(name, "force_generic")) {
        ctx->tune.force_generic = value != 0;
    } else if (!strcmp(name, "imma_small")) {
        ctx->tune.imma_small = value != 0;
    } else if (!strcmp(name, "no_dp4a")) {
        ctx->tune.no_dp4a = value != 0;
    } else if (!strcmp(name, "gemm_min_m")) {
        if (value < 1 || value > 17) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "gemm_min_m must be in [1, 17]");
        ctx->gemm_min_m = static_cast<uint32_t>(value);
    } else if (!strcmp(name, "peer_allreduce")) {
        ctx->peer_allreduce = value != 0;
    } else if (!strcmp(name, "ffn_one_launch")) {
        ctx->ffn_one_launch = value != 0;
    } else if (!strcmp(name, "fused_allreduce")) {
        ctx->fused_allreduce = value != 0;
    } else if (!strcmp(name, "peer_pdl")) {
        ctx->peer_pdl = value != 0;
    } else if (!strcmp(name, "prefetch_units")) {
        if (value < 0 || value > 4096) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "prefetch_units out of range");
        ctx->tune.prefetch_units = static_cast<int>(value);
    } else if (!strcmp(name, "wait_limit")) {
        if (value < 0 || value > (int64_t(1) << 30)) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "wait_limit out of range");
        ctx->tune.wait_limit = static_cast<int>(value);
    } else if (!strcmp(name, "peer_expect_absent_rank")) {
        ctx->peer_expect_absent_rank = value != 0;
    } else if (!strcmp(name, "comm_timeout_ms")) {
        if (value < 0 || value > 3600000) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "comm_timeout_ms out of range");
        ctx->comm_timeout_ms = static_cast<uint32_t>(value);
    } else {
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "unknown option '%s'", name);
    }
    return TGAF_OK;
}

int32_t tgaf_weight_upload(tgaf_ctx *ctx, const void *packed, const void *scales, const void *biases,
                           uint64_t N, uint64_t K, uint32_t group_size, uint32_t bits,
                           uint32_t scales_dtype, uint32_t shard_kind, uint32_t tp_rank,
                           uint32_t tp_size, tgaf_weight **out_weight) {
    if (!out_weight) return TGAF_ERR_INVALID_ARGUMENT;
    *out_weight = nullptr;
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!packed || !scales || !biases) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null weight pointer");
    if (bits != 4 && bits != 8) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "bits must be 4 or 8");
    if (shard_kind > TGAF_SHARD_ROW) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "bad shard kind %u", shard_kind);
    if (shard_kind == TGAF_SHARD_NONE) {
        tp_rank = 0;
        tp_size = 1;
    }
    if (tp_size == 0 || tp_rank >= tp_size) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "bad tp rank %u of %u", tp_rank, tp_size);
    const uint32_t vpw = 32u / bits;
    if (group_size == 0 || K == 0 || N == 0 || K % vpw != 0 || group_size % vpw != 0 || K % group_size != 0)
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "bad shape N=%llu K=%llu G=%u bits=%u",
                    (unsigned long long)N, (unsigned long long)K, group_size, bits);

    uint64_t n_local = N, k_local = K, n0 = 0, k0 = 0;
    if (shard_kind == TGAF_SHARD_COL) {
        if (N % tp_size != 0) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "N=%llu not divisible by %u ranks", (unsigned long long)N, tp_size);
        n_local = N / tp_size;
        n0 = n_local * tp_rank;
    } else if (shard_kind == TGAF_SHARD_ROW) {
        // cut on group boundaries (vpw divides the group)
        if (K % (static_cast<uint64_t>(tp_size) * group_size) != 0)
            return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "K=%llu not divisible by ranks*group = %u*%u",
                        (unsigned long long)K, tp_size, group_size);
        k_local = K / tp_size;
        k0 = k_local * tp_rank;
    }
    if (!shape_ok(n_local, k_local, group_size, bits, scales_dtype))
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "shape rejected: N=%llu K=%llu G=%u bits=%u sdtype=%u (K/G <= 1024)",
                    (unsigned long long)n_local, (unsigned long long)k_local, group_size, bits, scales_dtype);

    tgaf_weight *w = new (std::nothrow) tgaf_weight();
    if (!w) return fail(ctx, TGAF_ERR_OUT_OF_MEMORY, "host allocation failed");
    w->owns = true;
    w->full_N = N;
    w->full_K = K;
    w->shard_kind = shard_kind;
    w->tp_rank = tp_rank;
    w->tp_size = tp_size;
    WeightView &v = w->v;
    v.N = static_cast<uint32_t>(n_local);
    v.K = static_cast<uint32_t>(k_local);
    v.group = group_size;
    v.bits = bits;
    v.sdtype = scales_dtype;
    v.row_bytes = static_cast<uint32_t>(k_local * bits / 8);
    v.groups = static_cast<uint32_t>(k_local / group_size);

    const size_t full_row_bytes = K * bits / 8, full_groups = K / group_size;
    const size_t pbytes = static_cast<size_t>(v.N) * v.row_bytes;
    const size_t sbytes = static_cast<size_t>(v.N) * v.groups * 2;
    uint8_t *dp = nullptr, *ds = nullptr, *db = nullptr;
    cudaSetDevice(ctx->device);
    cudaError_t e = cudaMalloc(&dp, pbytes);
    if (e == cudaSuccess) e = cudaMalloc(&ds, sbytes);
    if (e == cudaSuccess) e = cudaMalloc(&db, sbytes);
    if (e == cudaSuccess) {
        // host sources may be unaligned mmap views: they are copied as bytes
        const uint8_t *hp = static_cast<const uint8_t *>(packed) + n0 * full_row_bytes + k0 * bits / 8;
        const uint8_t *hs = static_cast<const uint8_t *>(scales) + (n0 * full_groups + k0 / group_size) * 2;
        const uint8_t *hb = static_cast<const uint8_t *>(biases) + (n0 * full_groups + k0 / group_size) * 2;
        e = cudaMemcpy2DAsync(dp, v.row_bytes, hp, full_row_bytes, v.row_bytes, v.N, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess)
            e = cudaMemcpy2DAsync(ds, v.groups * 2, hs, full_groups * 2, v.groups * 2, v.N, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess)
            e = cudaMemcpy2DAsync(db, v.groups * 2, hb, full_groups * 2, v.groups * 2, v.N, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);  // the host buffers are the caller's again
    }
    if (e != cudaSuccess) {
        if (dp) cudaFree(dp);
        if (ds) cudaFree(ds);
        if (db) cudaFree(db);
        delete w;
        return cuda_fail(ctx, e, "weight upload");
    }
    v.packed = dp;
    v.scales = reinterpret_cast<uint16_t *>(ds);
    v.biases = reinterpret_cast<uint16_t *>(db);
    attach_packed_tmap(v);
    *out_weight = w;
    return TGAF_OK;
}

int32_t tgaf_weight_wrap_device(tgaf_ctx *ctx, const void *d_packed, const void *d_scales, const void *d_biases,
                                uint64_t N, uint64_t K, uint32_t group_size, uint32_t bits,
                                uint32_t scales_dtype, tgaf_weight **out_weight) {
    if (!out_weight) return TGAF_ERR_INVALID_ARGUMENT;
    *out_weight = nullptr;
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!d_packed || !d_scales || !d_biases) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null weight pointer");
    if (!shape_ok(N, K, group_size, bits, scales_dtype))
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "shape rejected: N=%llu K=%llu G=%u bits=%u sdtype=%u",
                    (unsigned long long)N, (unsigned long long)K, group_size, bits, scales_dtype);
    tgaf_weight *w = new (std::nothrow) tgaf_weight();
    if (!w) return fail(ctx, TGAF_ERR_OUT_OF_MEMORY, "host allocation failed");
    w->owns = false;
    w->full_N = N;
    w->full_K = K;
    WeightView &v = w->v;
    v.packed = static_cast<const uint8_t *>(d_packed);
    v.scales = static_cast<const uint16_t *>(d_scales);
    v.biases = static_cast<const uint16_t *>(d_biases);
    v.N = static_cast<uint32_t>(N);
    v.K = static_cast<uint32_t>(K);
    v.group = group_size;
    v.bits = bits;
    v.sdtype = scales_dtype;
    v.row_bytes = static_cast<uint32_t>(K * bits / 8);
    v.groups = static_cast<uint32_t>(K / group_size);
    attach_packed_tmap(v);
    *out_weight = w;
    return TGAF_OK;
}

int32_t tgaf_hint_next_weight(tgaf_ctx *ctx, const tgaf_weight *next) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    ctx->tune.next = next ? &next->v : nullptr;
    return TGAF_OK;
}

int32_t tgaf_weight_free(tgaf_ctx *ctx, tgaf_weight *w) {
    if (!w) return TGAF_OK;
    if (ctx && ctx->tune.next == &w->v) ctx->tune.next = nullptr;
    if (w->owns) {
        if (ctx) {
            cudaSetDevice(ctx->device);
            cudaStreamSynchronize(ctx->stream);
        }
        cudaFree(const_cast<uint8_t *>(w->v.packed));
        cudaFree(const_cast<uint16_t *>(w->v.scales));
        cudaFree(const_cast<uint16_t *>(w->v.biases));
    }
    delete w;
    return TGAF_OK;
}

int32_t tgaf_weight_dims(const tgaf_weight *w, uint64_t *n_local, uint64_t *k_local, uint32_t *group_size,
                         uint32_t *bits) {
    if (n_local) *n_local = 0;
    if (k_local) *k_local = 0;
    if (group_size) *group_size = 0;
    if (bits) *bits = 0;
    if (!w) return TGAF_ERR_INVALID_ARGUMENT;
    if (n_local) *n_local = w->v.N;
    if (k_local) *k_local = w->v.K;
    if (group_size) *group_size = w->v.group;
    if (bits) *bits = w->v.bits;
    return TGAF_OK;
}

int32_t tgaf_linear_bf16(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16, uint32_t M, void *y_bf16) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!w) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null weight");
    return linear_device(ctx, w->v, x_bf16, M, y_bf16, false);
}

int32_t tgaf_linear_f32(tgaf_ctx *ctx, const tgaf_weight *w, const float *x, uint32_t M, float *y) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!w) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null weight");
    return linear_device(ctx, w->v, x, M, y, true);
}

// the reference's Linear.forward with its optional bias: matmul, then addBiasRows
static int32_t linear_bias(tgaf_ctx *ctx, const tgaf_weight *w, const void *x, uint32_t M, const float *bias, void *y, bool f32) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!w) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null weight");
    const int32_t st = linear_device(ctx, w->v, x, M, y, f32);
    if (st != TGAF_OK || !bias) return st;
    cudaError_t e = add_bias_rows(y, bias, M, w->v.N, f32, ctx->stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "bias rows launch");
    return TGAF_OK;
}

int32_t tgaf_linear_bf16_bias(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16, uint32_t M, const float *d_bias, void *y_bf16) {
    return linear_bias(ctx, w, x_bf16, M, d_bias, y_bf16, false);
}

int32_t tgaf_linear_f32_bias(tgaf_ctx *ctx, const tgaf_weight *w, const float *x, uint32_t M, const float *d_bias, float *y) {
    return linear_bias(ctx, w, x, M, d_bias, y, true);
}

int32_t tgaf_linear_bf16_fixed_scratch(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16, uint32_t M,
                                       void *y_bf16) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!w || !x_bf16 || !y_bf16) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null pointer");
    if (M == 0) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "M must be > 0");
    // nothing below allocates: no cudaMalloc / cudaFree, no growth of the context's scratch
    TGAF_CUDA(ctx, cudaSetDevice(ctx->device));
    const WeightView &v = w->v;
    ctx->tune.next = nullptr;  // a pending next-weight hint is dropped: this variant does not prefetch
    if (ctx->tune.force_generic || !gemv_mma_eligible(v, x_bf16, y_bf16, false)) {
        // shapes outside the fast path use the kernel that needs no scratch at all
        cudaError_t e = gemv_generic(v, x_bf16, y_bf16, M, false, ctx->stream);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "gemv_generic launch");
        return TGAF_OK;
    }
    for (uint32_t m0 = 0; m0 < M; m0 += 16u) {
        const uint32_t mc = (M - m0) < 16u ? (M - m0) : 16u;
        const void *xp = static_cast<const uint8_t *>(x_bf16) + static_cast<size_t>(m0) * v.K * 2u;
        void *yp = static_cast<uint8_t *>(y_bf16) + static_cast<size_t>(m0) * v.N * 2u;
        size_t need = 0;
        cudaError_t e = gemv_mma_static(v, xp, yp, mc, false, ctx->tune, ctx->stream, ctx->sm_count, ctx->device,
                                        ctx->d_error_word, &need);
        if (e == cudaErrorMemoryAllocation)
            return fail(ctx, TGAF_ERR_UNSUPPORTED,
                        "this problem needs %zu bytes of split-K scratch (or more than 8192 row groups); the fixed "
                        "scratch holds %zu bytes - use tgaf_linear_bf16",
                        need, gemv_static_scratch_capacity());
        if (e != cudaSuccess) return cuda_fail(ctx, e, "fixed-scratch gemv launch");
    }
    return TGAF_OK;
}

int32_t tgaf_linear_bf16_host(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16_host, uint32_t M,
                              void *y_bf16_host) {
    return linear_host(ctx, w, x_bf16_host, M, y_bf16_host, false);
}

int32_t tgaf_linear_bf16_host_async(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16_host, uint32_t M,
                                    void *y_bf16_host) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!w || !x_bf16_host || !y_bf16_host || M == 0) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null pointer or M == 0");
    cudaSetDevice(ctx->device);
    if (!ctx->h2d_stream) {
        TGAF_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
        TGAF_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));
        for (int i = 0; i < tgaf_ctx::kPipe; ++i) {
            TGAF_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_x_ready[i], cudaEventDisableTiming));
            TGAF_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_k_done[i], cudaEventDisableTiming));
            TGAF_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_y_done[i], cudaEventDisableTiming));
        }
    }
    const int slot = static_cast<int>(ctx->pipe_calls % tgaf_ctx::kPipe);
    const bool reused = ctx->pipe_calls >= static_cast<uint64_t>(tgaf_ctx::kPipe);
    const size_t xb = static_cast<size_t>(M) * w->v.K * 2u, yb = static_cast<size_t>(M) * w->v.N * 2u;
    if (xb > ctx->pipe_x_bytes[slot] || yb > ctx->pipe_y_bytes[slot]) {
        // growing a staging buffer: nothing may still be using the old one
        TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->h2d_stream));
        TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        TGAF_CUDA(ctx, cudaStreamSynchronize(ctx->d2h_stream));
        if (xb > ctx->pipe_x_bytes[slot]) {
            if (ctx->pipe_x[slot]) cudaFree(ctx->pipe_x[slot]);
            ctx->pipe_x[slot] = nullptr, ctx->pipe_x_bytes[slot] = 0;
            const size_t want = xb < (size_t(256) << 10) ? (size_t(256) << 10) : xb;
            TGAF_CUDA(ctx, cudaMalloc(&ctx->pipe_x[slot], want));
            ctx->pipe_x_bytes[slot] = want;
        }
        if (yb > ctx->pipe_y_bytes[slot]) {
            if (ctx->pipe_y[slot]) cudaFree(ctx->pipe_y[slot]);
            ctx->pipe_y[slot] = nullptr, ctx->pipe_y_bytes[slot] = 0;
            const size_t want = yb < (size_t(256) << 10) ? (size_t(256) << 10) : yb;
            TGAF_CUDA(ctx, cudaMalloc(&ctx->pipe_y[slot], want));
            ctx->pipe_y_bytes[slot] = want;
        }
    }
    // x: host -> slot, once the kernel that last read this slot is done
    if (reused) TGAF_CUDA(ctx, cudaStreamWaitEvent(ctx->h2d_stream, ctx->ev_k_done[slot], 0));
    TGAF_CUDA(ctx, cudaMemcpyAsync(ctx->pipe_x[slot], x_bf16_host, xb, cudaMemcpyHostToDevice, ctx->h2d_stream));
    TGAF_CUDA(ctx, cudaEventRecord(ctx->ev_x_ready[slot], ctx->h2d_stream));
    // kernel: after x has landed and the slot's previous y has left
    TGAF_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_x_ready[slot], 0));
    if (reused) TGAF_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_y_done[slot], 0));
    int32_t st = linear_device(ctx, w->v, ctx->pipe_x[slot], M, ctx->pipe_y[slot], false);
    if (st != TGAF_OK) return st;
    TGAF_CUDA(ctx, cudaEventRecord(ctx->ev_k_done[slot], ctx->stream));
    // y: slot -> host
    TGAF_CUDA(ctx, cudaStreamWaitEvent(ctx->d2h_stream, ctx->ev_k_done[slot], 0));
    TGAF_CUDA(ctx, cudaMemcpyAsync(y_bf16_host, ctx->pipe_y[slot], yb, cudaMemcpyDeviceToHost, ctx->d2h_stream));
    TGAF_CUDA(ctx, cudaEventRecord(ctx->ev_y_done[slot], ctx->d2h_stream));
    ++ctx->pipe_calls;
    return TGAF_OK;
}

int32_t tgaf_linear_bf16_host_async_batch(tgaf_ctx *ctx, uint32_t count, const tgaf_weight *const *weights,
                                          const void *const *xs_bf16_host, const uint32_t *ms, void *const *ys_bf16_host) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (count == 0) return TGAF_OK;
    if (!weights || !xs_bf16_host || !ms || !ys_bf16_host) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null array");
    for (uint32_t i = 0; i < count; ++i) {
        // the list is the layer order: each launch also warms L2 with the head of the following weight
        if (i + 1u < count && weights[i + 1u]) ctx->tune.next = &weights[i + 1u]->v;
        const int32_t st = tgaf_linear_bf16_host_async(ctx, weights[i], xs_bf16_host[i], ms[i], ys_bf16_host[i]);
        if (st != TGAF_OK) return st;
    }
    return TGAF_OK;
}

namespace {

// Copies `count` buffers between host and the device block, merging neighbours that are adjacent on both sides
// (a decoder that keeps its activations in one page-locked block pays for one copy, not one per linear).
// The allocation [base, base + size) that holds a page-locked host pointer; false for pageable memory.
bool host_allocation_of(const void *p, uintptr_t *base, size_t *size) {
    typedef CUresult (*RangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);
    static RangeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<RangeFn>(sym);
    }
    if (!fn) return false;
    CUdeviceptr b = 0;
    size_t n = 0;
    if (fn(&b, &n, reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS) return false;
    *base = static_cast<uintptr_t>(b), *size = n;
    return true;
}

cudaError_t copy_runs(uint32_t count, const std::vector<size_t> &dev_off, const std::vector<size_t> &bytes, uint8_t *dev,
                      const void *const *host, bool to_device, cudaStream_t stream) {
    uint32_t i = 0;
    while (i < count) {
        uint32_t j = i + 1u;
        size_t run = bytes[i];
        // neighbours in address space may still be two allocations, which one copy must not span
        uintptr_t base = 0;
        size_t span = 0;
        const bool known = host_allocation_of(host[i], &base, &span);
        while (known && j < count && static_cast<const uint8_t *>(host[j]) == static_cast<const uint8_t *>(host[i]) + run &&
               dev_off[j] == dev_off[i] + run && reinterpret_cast<uintptr_t>(host[j]) + bytes[j] <= base + span) {
            run += bytes[j];
            ++j;
        }
        void *h = const_cast<void *>(host[i]);
        const cudaError_t e = to_device ? cudaMemcpyAsync(dev + dev_off[i], h, run, cudaMemcpyHostToDevice, stream)
                                        : cudaMemcpyAsync(h, dev + dev_off[i], run, cudaMemcpyDeviceToHost, stream);
        if (e != cudaSuccess) return e;
        i = j;
    }
    return cudaSuccess;
}

void host_batch_free(tgaf_ctx *ctx, tgaf_host_batch *b) {
    if (b->exec) cudaGraphExecDestroy(b->exec);
    if (b->graph) cudaGraphDestroy(b->graph);
    if (b->inner) tgaf_batch_destroy(ctx, b->inner);
    if (b->d_x) cudaFree(b->d_x);
    if (b->d_y) cudaFree(b->d_y);
    delete b;
}

// The staged form of a recorded host list: x block up, ONE launch list (or, with sums over the ranks on a
// communicator without peer memory, its calls one after the other), y block down.  Returns TGAF_OK with *out == nullptr
// when the list is not of that kind (different m per call, or no single launch to gain).
int32_t host_batch_staged(tgaf_ctx *ctx, uint32_t count, const tgaf_weight *const *weights, const void *const *xs_host,
                          const uint32_t *ms, void *const *ys_host, const uint8_t *reduce, tgaf_host_batch **out) {
    *out = nullptr;
    bool any_reduce = false;
    for (uint32_t i = 0; i < count; ++i) {
        if (!weights[i] || !xs_host[i] || !ys_host[i] || ms[i] == 0) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null entry %u or M == 0", i);
        if (ms[i] != ms[0]) {
            if (reduce) return fail(ctx, TGAF_ERR_UNSUPPORTED, "a host batch with sums over the ranks needs the same M in every call");
            return TGAF_OK;
        }
        if (reduce && reduce[i]) any_reduce = true;
    }
    const uint32_t m = ms[0];
    std::vector<size_t> xoff(count), yoff(count), xb(count), yb(count);
    size_t xt = 0, yt = 0;
    for (uint32_t i = 0; i < count; ++i) {
        xb[i] = static_cast<size_t>(m) * weights[i]->v.K * 2u, yb[i] = static_cast<size_t>(m) * weights[i]->v.N * 2u;
        xoff[i] = xt, yoff[i] = yt;
        xt += (xb[i] + 15u) & ~size_t(15), yt += (yb[i] + 15u) & ~size_t(15);
    }
    tgaf_host_batch *b = new (std::nothrow) tgaf_host_batch();
    if (!b) return fail(ctx, TGAF_ERR_OUT_OF_MEMORY, "host batch");
    b->count = count;
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&b->d_x), xt);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&b->d_y), yt);
    if (e != cudaSuccess) {
        host_batch_free(ctx, b);
        return cuda_fail(ctx, e, "host batch staging");
    }
    std::vector<const void *> dx(count);
    std::vector<void *> dy(count);
    for (uint32_t i = 0; i < count; ++i) dx[i] = b->d_x + xoff[i], dy[i] = b->d_y + yoff[i];
    int32_t st = tgaf_batch_create(ctx, count, weights, dx.data(), m, dy.data(), nullptr, any_reduce ? reduce : nullptr, &b->inner);
    if (st != TGAF_OK) {
        host_batch_free(ctx, b);
        return st;
    }
    if (!b->inner->list && !any_reduce) {   // nothing to gain: the queued form overlaps its copies with its kernels
        host_batch_free(ctx, b);
        return TGAF_OK;
    }
    auto enqueue = [&]() -> int32_t {
        cudaError_t ce = copy_runs(count, xoff, xb, b->d_x, xs_host, true, ctx->stream);
        if (ce != cudaSuccess) return cuda_fail(ctx, ce, "host batch upload");
        const int32_t rs = tgaf_batch_run(ctx, b->inner);
        if (rs != TGAF_OK) return rs;
        ce = copy_runs(count, yoff, yb, b->d_y, ys_host, false, ctx->stream);
        if (ce != cudaSuccess) return cuda_fail(ctx, ce, "host batch download");
        return TGAF_OK;
    };
    st = enqueue();   // once for real: scratch, kernel attributes
    if (st == TGAF_OK) st = tgaf_synchronize(ctx);
    if (st != TGAF_OK) {
        host_batch_free(ctx, b);
        return st;
    }
    e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        host_batch_free(ctx, b);
        return cuda_fail(ctx, e, "cudaStreamBeginCapture");
    }
    st = enqueue();
    cudaGraph_t graph = nullptr;
    const cudaError_t e_end = cudaStreamEndCapture(ctx->stream, &graph);
    if (st == TGAF_OK && (e_end != cudaSuccess || !graph)) st = cuda_fail(ctx, e_end, "capturing the host batch");
    if (st == TGAF_OK) {
        b->graph = graph;
        e = cudaGraphInstantiate(&b->exec, graph, 0);
        if (e != cudaSuccess) st = cuda_fail(ctx, e, "cudaGraphInstantiate");
    } else if (graph) {
        cudaGraphDestroy(graph);
    }
    if (st != TGAF_OK) {
        cudaGetLastError();
        host_batch_free(ctx, b);
        return st;
    }
    *out = b;
    return TGAF_OK;
}

}  // namespace

int32_t tgaf_host_batch_create_reduce(tgaf_ctx *ctx, uint32_t count, const tgaf_weight *const *weights,
                                      const void *const *xs_bf16_host, const uint32_t *ms, void *const *ys_bf16_host,
                                      const uint8_t *reduce, tgaf_host_batch **out_batch) {
    if (out_batch) *out_batch = nullptr;
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!out_batch || count == 0 || !weights || !xs_bf16_host || !ms || !ys_bf16_host)
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null array or empty list");
    cudaSetDevice(ctx->device);
    if (ctx->stream == cudaStreamLegacy || ctx->stream == cudaStreamPerThread || ctx->stream == nullptr)
        return fail(ctx, TGAF_ERR_UNSUPPORTED, "recording needs a context on a stream of its own (the default streams cannot be captured)");
    {
        const int32_t sst = host_batch_staged(ctx, count, weights, xs_bf16_host, ms, ys_bf16_host, reduce, out_batch);
        if (sst != TGAF_OK || *out_batch) return sst;
    }
    // 1. once for real: every staging buffer, scratch area and kernel attribute the list needs exists afterwards
    ctx->pipe_calls = 0;
    int32_t st = tgaf_linear_bf16_host_async_batch(ctx, count, weights, xs_bf16_host, ms, ys_bf16_host);
    if (st != TGAF_OK) return st;
    st = tgaf_synchronize(ctx);
    if (st != TGAF_OK) return st;
    // 2. the same list into a graph; the copy streams join the capture through the events and are joined back
    tgaf_host_batch *b = new (std::nothrow) tgaf_host_batch();
    if (!b) return fail(ctx, TGAF_ERR_OUT_OF_MEMORY, "host batch");
    b->count = count;
    ctx->pipe_calls = 0;  // every replay starts on staging slot 0; replays run one after another on the stream
    cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        delete b;
        return cuda_fail(ctx, e, "cudaStreamBeginCapture");
    }
    // fork: the upload stream enters the capture by depending on the captured stream's start
    e = cudaEventRecord(ctx->ev_y_done[tgaf_ctx::kPipe - 1], ctx->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->h2d_stream, ctx->ev_y_done[tgaf_ctx::kPipe - 1], 0);
    st = e == cudaSuccess ? tgaf_linear_bf16_host_async_batch(ctx, count, weights, xs_bf16_host, ms, ys_bf16_host) : TGAF_OK;
    if (st == TGAF_OK && e == cudaSuccess) {
        // join: the last copies of every staging slot
        const uint32_t used = count < static_cast<uint32_t>(tgaf_ctx::kPipe) ? count : static_cast<uint32_t>(tgaf_ctx::kPipe);
        for (uint32_t i = 0; i < used && e == cudaSuccess; ++i) e = cudaStreamWaitEvent(ctx->stream, ctx->ev_y_done[i], 0);
        if (e == cudaSuccess) e = cudaEventRecord(ctx->ev_x_ready[0], ctx->h2d_stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->stream, ctx->ev_x_ready[0], 0);
    }
    cudaGraph_t graph = nullptr;
    const cudaError_t e_end = cudaStreamEndCapture(ctx->stream, &graph);
    ctx->pipe_calls = 0;
    if (st != TGAF_OK || e != cudaSuccess || e_end != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        delete b;
        cudaGetLastError();
        if (st != TGAF_OK) return st;
        return cuda_fail(ctx, e != cudaSuccess ? e : e_end, "capturing the host batch");
    }
    b->graph = graph;
    e = cudaGraphInstantiate(&b->exec, graph, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(graph);
        delete b;
        return cuda_fail(ctx, e, "cudaGraphInstantiate");
    }
    *out_batch = b;
    return TGAF_OK;
}

int32_t tgaf_host_batch_create(tgaf_ctx *ctx, uint32_t count, const tgaf_weight *const *weights,
                               const void *const *xs_bf16_host, const uint32_t *ms, void *const *ys_bf16_host,
                               tgaf_host_batch **out_batch) {
    return tgaf_host_batch_create_reduce(ctx, count, weights, xs_bf16_host, ms, ys_bf16_host, nullptr, out_batch);
}

int32_t tgaf_host_batch_uses_one_launch(const tgaf_host_batch *batch) { return batch && batch->inner && batch->inner->list ? 1 : 0; }

int32_t tgaf_host_batch_submit(tgaf_ctx *ctx, tgaf_host_batch *batch) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!batch || !batch->exec) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null batch");
    cudaSetDevice(ctx->device);
    TGAF_CUDA(ctx, cudaGraphLaunch(batch->exec, ctx->stream));
    return TGAF_OK;
}

int32_t tgaf_host_batch_destroy(tgaf_ctx *ctx, tgaf_host_batch *batch) {
    if (!batch) return TGAF_OK;
    if (ctx) {
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
    }
    host_batch_free(ctx, batch);
    return TGAF_OK;
}

int32_t tgaf_batch_create(tgaf_ctx *ctx, uint32_t count, const tgaf_weight *const *weights, const void *const *xs_bf16,
                          uint32_t m, void *const *ys_bf16, const uint8_t *depends, const uint8_t *reduce,
                          tgaf_batch **out_batch) {
    if (out_batch) *out_batch = nullptr;
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!out_batch || count == 0 || !weights || !xs_bf16 || !ys_bf16 || m == 0)
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null array, empty list or m == 0");
    bool any_reduce = false;
    for (uint32_t i = 0; i < count; ++i) {
        if (!weights[i] || !xs_bf16[i] || !ys_bf16[i]) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null entry %u", i);
        if (reduce && reduce[i]) any_reduce = true;
    }
    if (depends && depends[0]) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "the first operation has no predecessor to depend on");
    if (any_reduce && !ctx->comm) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "no communicator: call tgaf_comm_init first");
    TGAF_CUDA(ctx, cudaSetDevice(ctx->device));
    tgaf_batch *b = new (std::nothrow) tgaf_batch();
    if (!b) return fail(ctx, TGAF_ERR_OUT_OF_MEMORY, "batch");
    b->m = m;
    std::vector<const WeightView *> views(count);
    std::vector<const PeerComm *> fuse(count, nullptr);
    for (uint32_t i = 0; i < count; ++i) {
        b->weights.push_back(weights[i]);
        b->xs.push_back(xs_bf16[i]);
        b->ys.push_back(ys_bf16[i]);
        b->deps.push_back(depends ? depends[i] : 0);
        b->reduce.push_back(reduce ? reduce[i] : 0);
        views[i] = &weights[i]->v;
        if (b->reduce[i]) fuse[i] = &ctx->peer;
    }
    // one launch when every operation is on the M <= 4 kernel's ground (and every sum over the ranks can ride in it)
    bool one_launch = gemv_list_eligible(views.data(), count, m, ctx->tune);
    if (any_reduce && !(ctx->peer.ok && ctx->fused_allreduce)) one_launch = false;
    if (one_launch) {
        const size_t words = gemv_list_tagged_words(views.data(), count, m, ctx->tune, ctx->sm_count);
        b->tagged_bytes = words * 8u < 256u ? 256u : words * 8u;
        cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&b->tagged), b->tagged_bytes);
        if (e == cudaSuccess) e = cudaMemsetAsync(b->tagged, 0, b->tagged_bytes, ctx->stream);
        if (e == cudaSuccess)
            e = gemv_list_create(views.data(), b->xs.data(), b->ys.data(), b->deps.data(), any_reduce ? fuse.data() : nullptr, count, m,
                                 b->tagged, ctx->tune, ctx->sm_count, ctx->d_error_word, ctx->stream, &b->list);
        if (e != cudaSuccess && e != cudaErrorNotSupported) {
            if (b->tagged) cudaFree(b->tagged);
            delete b;
            return cuda_fail(ctx, e, "building the launch list");
        }
        if (e == cudaErrorNotSupported) {   // e.g. a buffer that is not 16-byte aligned: the calls run one by one
            cudaGetLastError();
            if (b->tagged) cudaFree(b->tagged);
            b->tagged = nullptr, b->tagged_bytes = 0, b->list = nullptr;
        }
    }
    ctx->batches.push_back(b);
    *out_batch = b;
    return TGAF_OK;
}

int32_t tgaf_batch_run(tgaf_ctx *ctx, tgaf_batch *batch) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!batch) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null batch");
    TGAF_CUDA(ctx, cudaSetDevice(ctx->device));
    if (batch->list) {
        ctx->tune.next = nullptr;
        cudaError_t e = gemv_list_launch(batch->list, ctx->tune, ctx->stream);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "launch list");
        return TGAF_OK;
    }
    const uint32_t n = static_cast<uint32_t>(batch->weights.size());
    for (uint32_t i = 0; i < n; ++i) {
        if (i + 1u < n) ctx->tune.next = &batch->weights[i + 1u]->v;   // the list is the call order
        const int32_t st = linear_device(ctx, batch->weights[i]->v, batch->xs[i], batch->m, batch->ys[i], false, batch->reduce[i] != 0);
        if (st != TGAF_OK) return st;
    }
    return TGAF_OK;
}

int32_t tgaf_batch_uses_one_launch(const tgaf_batch *batch) { return batch && batch->list ? 1 : 0; }

int32_t tgaf_batch_destroy(tgaf_ctx *ctx, tgaf_batch *batch) {
    if (!batch) return TGAF_OK;
    if (ctx) {
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        for (size_t i = 0; i < ctx->batches.size(); ++i)
            if (ctx->batches[i] == batch) {
                ctx->batches.erase(ctx->batches.begin() + static_cast<long>(i));
                break;
            }
    }
    if (batch->list) gemv_list_destroy(batch->list);
    if (batch->tagged) cudaFree(batch->tagged);
    delete batch;
    return TGAF_OK;
}

int32_t tgaf_linear_f32_host(tgaf_ctx *ctx, const tgaf_weight *w, const float *x_host, uint32_t M, float *y_host) {
    return linear_host(ctx, w, x_host, M, y_host, true);
}

int32_t tgaf_gaffine_u4_matvec_f32(tgaf_ctx *ctx, const float *input, const uint32_t *packed_weight,
                                   const uint16_t *scales, const uint16_t *biases, float *out, uint32_t in_dim,
                                   uint32_t out_dim, uint32_t group_size, uint32_t scales_dtype_tag,
                                   uint32_t batch_rows) {
    return raw_matvec(ctx, 4, input, packed_weight, scales, biases, out, in_dim, out_dim, group_size,
                      scales_dtype_tag, batch_rows);
}

int32_t tgaf_gaffine_u8_matvec_f32(tgaf_ctx *ctx, const float *input, const uint32_t *packed_weight,
                                   const uint16_t *scales, const uint16_t *biases, float *out, uint32_t in_dim,
                                   uint32_t out_dim, uint32_t group_size, uint32_t scales_dtype_tag,
                                   uint32_t batch_rows) {
    return raw_matvec(ctx, 8, input, packed_weight, scales, biases, out, in_dim, out_dim, group_size,
                      scales_dtype_tag, batch_rows);
}

int32_t tgaf_dequant_f32(tgaf_ctx *ctx, const tgaf_weight *w, float *d_out) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!w || !d_out) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null pointer");
    TGAF_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaError_t e = dequant_f32(w->v, d_out, ctx->stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "dequant launch");
    return TGAF_OK;
}

int32_t tgaf_dequant_f32_host(tgaf_ctx *ctx, const tgaf_weight *w, float *h_out) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!w || !h_out) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null pointer");
    TGAF_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t bytes = static_cast<size_t>(w->v.N) * w->v.K * sizeof(float);
    float *d = nullptr;
    TGAF_CUDA(ctx, cudaMalloc(&d, bytes));
    cudaError_t e = dequant_f32(w->v, d, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_out, d, bytes, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(d);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "dequant to host");
    return TGAF_OK;
}

int32_t tgaf_embedding_lookup_f32(tgaf_ctx *ctx, const tgaf_weight *w, const uint32_t *token_ids, uint32_t count,
                                  float multiplier, float *d_out) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!w || !token_ids || !d_out) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null pointer");
    if (count == 0) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "count must be > 0");
    TGAF_CUDA(ctx, cudaSetDevice(ctx->device));
    for (uint32_t i = 0; i < count; ++i)
        if (token_ids[i] >= w->v.N)
            return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "token id %u at position %u is outside the table of %u rows",
                        token_ids[i], i, w->v.N);
    const size_t bytes = static_cast<size_t>(count) * sizeof(uint32_t);
    int32_t st = ensure_stage(ctx, &ctx->stage_x, &ctx->stage_x_bytes, bytes);
    if (st != TGAF_OK) return st;
    TGAF_CUDA(ctx, cudaMemcpyAsync(ctx->stage_x, token_ids, bytes, cudaMemcpyHostToDevice, ctx->stream));
    cudaError_t e = gather_dequant_f32(w->v, static_cast<const uint32_t *>(ctx->stage_x), count, multiplier, d_out,
                                       ctx->stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "embedding lookup launch");
    return TGAF_OK;
}

int32_t tgaf_comm_make_id(uint8_t id[TGAF_COMM_ID_BYTES]) {
    if (!id) return TGAF_ERR_INVALID_ARGUMENT;
    memset(id, 0, TGAF_COMM_ID_BYTES);
    NcclApi &api = nccl_api();
    if (!api.ok) return TGAF_ERR_NCCL;
    NcclUniqueId uid;
    if (api.GetUniqueId(&uid) != kNcclSuccess) return TGAF_ERR_NCCL;
    memcpy(id, uid.internal, TGAF_COMM_ID_BYTES);
    return TGAF_OK;
}

int32_t tgaf_comm_init(tgaf_ctx *ctx, const uint8_t id[TGAF_COMM_ID_BYTES], uint32_t rank, uint32_t nranks) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!id || nranks == 0 || rank >= nranks) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "bad rank %u of %u", rank, nranks);
    if (ctx->comm) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "communicator already initialised");
    NcclApi &api = nccl_api();
    if (!api.ok) return fail(ctx, TGAF_ERR_NCCL, "NCCL unavailable: %s", api.why.c_str());
    NcclUniqueId uid;
    memcpy(uid.internal, id, TGAF_COMM_ID_BYTES);
    cudaSetDevice(ctx->device);
    int rc = api.CommInitRank(&ctx->comm, static_cast<int>(nranks), uid, static_cast<int>(rank));
    if (rc != kNcclSuccess) {
        ctx->comm = nullptr;
        return fail(ctx, TGAF_ERR_NCCL, "ncclCommInitRank: %s", api.GetErrorString(rc));
    }
    ctx->comm_rank = rank;
    ctx->comm_size = nranks;
    peer_setup(ctx, api);
    return TGAF_OK;
}

int32_t tgaf_comm_destroy(tgaf_ctx *ctx) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!ctx->comm) return TGAF_OK;
    NcclApi &api = nccl_api();
    cudaStreamSynchronize(ctx->stream);
    peer_teardown(ctx);
    if (api.ok) api.CommDestroy(ctx->comm);
    ctx->comm = nullptr;
    ctx->comm_size = 1;
    ctx->comm_rank = 0;
    return TGAF_OK;
}

// FFN operator.  reduce: sum the result over the communicator's ranks (row-parallel down projection).
static int32_t ffn_swiglu(tgaf_ctx *ctx, const tgaf_weight *wgu, const tgaf_weight *wd, const void *x, uint32_t M, void *y,
                          bool reduce, uint32_t act = TGAF_ACT_SILU) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (act != TGAF_ACT_SILU && act != TGAF_ACT_GELU) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "bad activation %u", act);
    if (!wgu || !wd || !x || !y || M == 0) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null pointer or M == 0");
    const WeightView &w1 = wgu->v, &w2 = wd->v;
    if (w1.N != 2u * w2.K)
        return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "gate|up has %u rows, down has %u columns (need rows = 2 x columns)", w1.N, w2.K);
    if (reduce && !ctx->comm) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "no communicator: call tgaf_comm_init first");
    cudaSetDevice(ctx->device);
    const WeightView *hint = ctx->tune.next;
    ctx->tune.next = nullptr;
    const uint32_t d_ff = w2.K;
    // intermediate: fp32 [M][2 d_ff] for the one-launch path; bf16 [M][2 d_ff] + bf16 [M][d_ff] otherwise
    const size_t mid_need = static_cast<size_t>(M) * 2u * d_ff * 4u;
    int32_t st = ensure_stage(ctx, &ctx->ffn_mid, &ctx->ffn_mid_bytes, mid_need);
    if (st != TGAF_OK) return st;
    if (!ctx->d_grid_bar) {
        TGAF_CUDA(ctx, cudaMalloc(reinterpret_cast<void **>(&ctx->d_grid_bar), 4 * sizeof(unsigned int)));
        TGAF_CUDA(ctx, cudaMemsetAsync(ctx->d_grid_bar, 0, 4 * sizeof(unsigned int), ctx->stream));
    }
    GemvTuning t = ctx->tune;
    t.fuse = (reduce && ctx->peer.ok && ctx->fused_allreduce) ? &ctx->peer : nullptr;
    const bool peer_ready = !reduce || (t.fuse && gemv_fused_eligible(w2, M, false, t));
    if (ctx->ffn_one_launch && !ctx->tune.force_generic && peer_ready && gemv_ffn_eligible(w1, w2, x, y, M, t)) {
        st = ensure_scratch(ctx, 0, 0, gemv_ffn_tagged_bytes(w1, w2, M, t, ctx->sm_count));
        if (st != TGAF_OK) return st;
        cudaError_t e = gemv_ffn_swiglu(w1, w2, x, static_cast<float *>(ctx->ffn_mid), y, M, act, ctx->scratch, ctx->d_grid_bar, t,
                                        ctx->stream, ctx->sm_count, ctx->d_error_word);
        if (e == cudaSuccess) return TGAF_OK;
        if (e != cudaErrorNotSupported) return cuda_fail(ctx, e, "ffn launch");
    }
    // two linears with the activation in between
    uint8_t *gu = static_cast<uint8_t *>(ctx->ffn_mid);
    uint8_t *h = gu + static_cast<size_t>(M) * 2u * d_ff * 2u;
    ctx->tune.next = &w2;
    st = linear_device(ctx, w1, x, M, gu, false);
    if (st != TGAF_OK) return st;
    cudaError_t e = swiglu_bf16(gu, h, M, d_ff, act, ctx->stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "swiglu launch");
    ctx->tune.next = hint;
    return linear_device(ctx, w2, h, M, y, false, reduce);
}

int32_t tgaf_ffn_swiglu_bf16(tgaf_ctx *ctx, const tgaf_weight *w_gate_up, const tgaf_weight *w_down, const void *x_bf16,
                             uint32_t m, void *y_bf16) {
    return ffn_swiglu(ctx, w_gate_up, w_down, x_bf16, m, y_bf16, false);
}

int32_t tgaf_ffn_gated_bf16(tgaf_ctx *ctx, const tgaf_weight *w_gate_up, const tgaf_weight *w_down, const void *x_bf16,
                            uint32_t m, uint32_t activation, void *y_bf16) {
    return ffn_swiglu(ctx, w_gate_up, w_down, x_bf16, m, y_bf16, false, activation);
}

int32_t tgaf_ffn_swiglu_bf16_allreduce(tgaf_ctx *ctx, const tgaf_weight *w_gate_up, const tgaf_weight *w_down,
                                       const void *x_bf16, uint32_t m, void *y_bf16) {
    return ffn_swiglu(ctx, w_gate_up, w_down, x_bf16, m, y_bf16, true);
}

int32_t tgaf_comm_uses_peer_memory(const tgaf_ctx *ctx) { return ctx && ctx->peer.ok ? 1 : 0; }

int32_t tgaf_allreduce(tgaf_ctx *ctx, void *d_buf, uint64_t count, uint32_t dtype) {
    return allreduce_device(ctx, d_buf, count, dtype);
}

int32_t tgaf_linear_bf16_allreduce(tgaf_ctx *ctx, const tgaf_weight *w, const void *x_bf16, uint32_t m, void *y_bf16) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!w) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null weight");
    if (!ctx->comm) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "no communicator: call tgaf_comm_init first");
    cudaSetDevice(ctx->device);
    return linear_device(ctx, w->v, x_bf16, m, y_bf16, false, true);
}

}  // extern "C"

namespace {
int32_t allreduce_device(tgaf_ctx *ctx, void *d_buf, uint64_t count, uint32_t dtype) {
    if (!ctx) return TGAF_ERR_INVALID_ARGUMENT;
    if (!d_buf || count == 0) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "null buffer or zero count");
    if (dtype != TGAF_DTYPE_F32 && dtype != TGAF_DTYPE_BF16) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "bad dtype %u", dtype);
    if (!ctx->comm) return fail(ctx, TGAF_ERR_INVALID_ARGUMENT, "no communicator: call tgaf_comm_init first");
    if (ctx->peer.ok && ctx->peer_allreduce) {
        // decode-sized tiles: one kernel over NVLink peer memory; anything else falls through to NCCL
        cudaError_t e = peer_allreduce(ctx->peer, d_buf, count, dtype == TGAF_DTYPE_F32, ctx->tune.pdl != 0 && ctx->peer_pdl != 0, ctx->stream,
                                       ctx->d_error_word, static_cast<uint32_t>(ctx->tune.wait_limit), ctx->peer_expect_absent_rank != 0);
        if (e == cudaSuccess) return TGAF_OK;
        if (e != cudaErrorNotSupported) return cuda_fail(ctx, e, "peer all-reduce launch");
    }
    NcclApi &api = nccl_api();
    int rc = api.AllReduce(d_buf, d_buf, count, dtype == TGAF_DTYPE_F32 ? kNcclFloat32 : kNcclBfloat16, kNcclSum,
                           ctx->comm, ctx->stream);
    if (rc != kNcclSuccess) return fail(ctx, TGAF_ERR_NCCL, "ncclAllReduce: %s", api.GetErrorString(rc));
    return TGAF_OK;
}
}  // namespace
