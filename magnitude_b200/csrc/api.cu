// C-ABI layer: contexts, weight handles, route selection, host-buffer path, NCCL exchange.
// Everything behind `extern "C"` returns a status; no exception leaves this file.
#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <chrono>
#include <future>
#include <memory>
#include <mutex>
#include <new>
#include <thread>
#include <vector>

#include "common.cuh"
#include "kernels.h"

using namespace b200q;

// ---------------------------------------------------------------------------------------------
// NCCL through dlopen: the library must load on machines without NCCL, and inside a Python
// process it must share the NCCL that process already loaded.
// ---------------------------------------------------------------------------------------------
namespace {

struct NcclUniqueId { char internal[128]; };
typedef void *NcclComm;
struct NcclApi {
    void *handle = nullptr;
    int (*GetUniqueId)(NcclUniqueId *) = nullptr;
    int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*CommAbort)(NcclComm) = nullptr;
    int (*CommGetAsyncError)(NcclComm, int *) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
};
constexpr int kNcclFloat32 = 7, kNcclBfloat16 = 9, kNcclSum = 0, kNcclInProgress = 7;

NcclApi *nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char *n : names) {
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (api.handle) {
            api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
            api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
            api.AllReduce = (decltype(api.AllReduce))dlsym(api.handle, "ncclAllReduce");
            api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
            api.CommAbort = (decltype(api.CommAbort))dlsym(api.handle, "ncclCommAbort");
            api.CommGetAsyncError = (decltype(api.CommGetAsyncError))dlsym(api.handle, "ncclCommGetAsyncError");
            api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
            if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.CommDestroy) {
                dlclose(api.handle);
                api.handle = nullptr;
            }
        }
    });
    return api.handle ? &api : nullptr;
}

int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

}  // namespace

struct b200q_ctx {
    int device = 0;
    int sm_count = 0;
    size_t smem_optin = 0;
    size_t smem_sm = 0;
    int *status_dev = nullptr;
    char err[512] = {0};
    int last_route = B200Q_ROUTE_NONE;
    int last_launches = 0;
    bool poisoned = false;
    // host-buffer path
    cudaStream_t hstream = nullptr;
    void *hx_dev = nullptr;
    size_t hx_bytes = 0;
    void *hy_dev = nullptr;
    size_t hy_bytes = 0;
    // prefill path: bf16 copy of fp32 activations
    void *gemm_scratch = nullptr;
    size_t gemm_scratch_bytes = 0;
    float *gemm_part = nullptr;       // K-split partial products of skinny batches (allocated on first use)
    // skinny route (2..16 rows): chunk sums, row-block counters, job table
    uint8_t *sk_ws = nullptr;
    size_t sk_ws_bytes = 0;
    uint64_t tp_timeout_ms = 60000;   // host deadline of b200q_tp_init
    bool peer_stale = false;          // a peer exchange timed out: the ranks' call counters no longer agree
    bool peer_ipc = true;             // peer buffers were mapped through CUDA IPC (else given as pointers)
    int skinny_min_m = 3;             // smallest M that takes the skinny route (smaller batches: the dp4a kernel)
    int gemm_bn = 0, gemm_debug = 0, gemm_pair = 0, gemm_ksplit = 1;
    // tunables (environment overrides for experiments)
    int gemv_warps = 0, gemv_depth = 0, gemv_grid = 0, gemv_smem = 0, gemv_rows = 0, gemv_debug = 0, gemv_pdl = 1, gemv_teams = 2, gemv_xprep = 1, gemv_nap = 0;
    // tensor parallel
    NcclComm comm = nullptr;
    int tp_rank = 0, tp_world = 1;
    // peer exchange (CUDA IPC): own buffer, every rank's buffer as mapped here
    uint8_t *peer_local = nullptr;
    uint8_t *peer_base[kPeerMaxWorld] = {nullptr};
    int peer_rank = -1, peer_world = 0;
};

struct b200q_plan {
    b200q_ctx *ctx = nullptr;
    int device = 0;                   // the context's device, kept here: the plan may outlive the context
    std::vector<StreamJob> jobs;
    StreamJob *jobs_dev = nullptr;
    uint8_t *xq_dev = nullptr;        // fixed-point activation images of the jobs (filled by the prep launch of every run)
    bool has_xq = false;
    int M = 0;
    // plans on the skinny route (3..16 rows by default): groups of products run by the skinny kernel, one launch pair per group
    std::vector<SkinnySet *> sets;
    uint8_t *sk_ws = nullptr;
    uint8_t *sk_jobs = nullptr;
};

struct b200q_weight {
    b200q_ctx *ctx = nullptr;
    int device = 0;                   // the context's device, kept here: the weight may outlive the context
    int type = 0;
    int64_t N = 0, K = 0, Kpad = 0;
    int64_t row_bytes = 0;
    size_t gguf_bytes = 0, device_bytes = 0;
    uint8_t *dev = nullptr;
};

namespace {

b200q_status fail(b200q_ctx *ctx, b200q_status code, const char *fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

b200q_status cuda_fail(b200q_ctx *ctx, cudaError_t e, const char *what) {
    const b200q_status code = (e == cudaErrorMemoryAllocation) ? B200Q_ERR_OVERLOADED : B200Q_ERR_BACKEND;
    return fail(ctx, code, "%s: %s", what, cudaGetErrorString(e));
}

#define CU_TRY(ctx, expr)                                          \
    do {                                                           \
        cudaError_t e__ = (expr);                                  \
        if (e__ != cudaSuccess) return cuda_fail(ctx, e__, #expr); \
    } while (0)

bool known_type(int t) { return t == QT_MXFP4 || t == QT_Q4_0 || t == QT_Q8_0 || t == QT_Q4_K || t == QT_Q5_K || t == QT_Q6_K; }
bool act_type(int t) { return t == B200Q_TYPE_F32 || t == B200Q_TYPE_BF16; }
size_t act_size(int t) { return t == B200Q_TYPE_BF16 ? 2 : 4; }

void split_even(int64_t units, int rank, int world, int64_t *b, int64_t *e) {
    const int64_t base = units / world, rem = units % world;
    *b = rank * base + (rank < rem ? rank : rem);
    *e = *b + base + (rank < rem ? 1 : 0);
}

b200q_status make_weight(b200q_ctx *ctx, int type, int64_t N, int64_t Kfull, const uint8_t *gguf,
                         int64_t r0, int64_t r1, int64_t k0, int64_t k1, b200q_weight **out) {
    const int64_t n = r1 - r0, k = k1 - k0;
    const int64_t sb0 = k0 / SB, sb1 = (k1 + SB - 1) / SB;
    b200q_weight *w = new (std::nothrow) b200q_weight();
    if (!w) return fail(ctx, B200Q_ERR_OVERLOADED, "out of host memory");
    w->ctx = ctx;
    w->device = ctx->device;
    w->type = type;
    w->N = n;
    w->K = k;
    w->Kpad = (sb1 - sb0) * SB;
    w->row_bytes = row_bytes_for(type, sb1 - sb0);
    w->gguf_bytes = (size_t)(n * (k / gguf_block_elems(type)) * gguf_block_bytes(type));
    w->device_bytes = (size_t)(padded_rows(n) * w->row_bytes);   // whole 4-row groups, zero padded
    if (n > 0 && k > 0) {
        std::vector<uint8_t> staged;
        try {
            staged.assign(w->device_bytes, 0);
        } catch (...) {
            const size_t need = w->device_bytes;
            delete w;
            return fail(ctx, B200Q_ERR_OVERLOADED, "out of host memory staging %zu bytes", need);
        }
        // rows are independent: re-lay them on a few threads
        const int nt = (int)std::min<int64_t>(8, std::max<int64_t>(1, n / 256));
        std::vector<std::thread> th;
        for (int t = 0; t < nt; ++t) {
            const int64_t a = n * t / nt, b = n * (t + 1) / nt;
            uint8_t *dst = staged.data();
            th.emplace_back([=] { repack_host(type, Kfull, gguf, r0, n, sb0, sb1, dst, a, b); });
        }
        for (auto &t : th) t.join();
        cudaError_t e = cudaMalloc(&w->dev, w->device_bytes + 256);
        if (e == cudaSuccess) e = cudaMemcpy(w->dev, staged.data(), w->device_bytes, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemset(w->dev + w->device_bytes, 0, 256);
        if (e != cudaSuccess) {
            if (w->dev) cudaFree(w->dev);
            delete w;
            return cuda_fail(ctx, e, "weight upload");
        }
    }
    *out = w;
    return B200Q_OK;
}

b200q_status check_ctx(b200q_ctx *ctx) {
    if (!ctx) return B200Q_ERR_INVALID_CONFIG;
    if (ctx->poisoned) return fail(ctx, B200Q_ERR_STOPPED, "context stopped after a device error");
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaSetDevice");
    // a launch is checked with cudaGetLastError(): an error some earlier, unrelated runtime call of the
    // process left behind (they are not sticky) must not be taken for this call's
    (void)cudaGetLastError();
    return B200Q_OK;
}

void fill_job(StreamJob &J, const b200q_weight *const *w, int nw, const void *x, int x_dtype, int64_t ldx,
              void *const *y, int y_dtype, const int64_t *ldy, int flags) {
    J = StreamJob{};
    J.nseg = nw;
    for (int i = 0; i < nw; ++i) {
        J.seg[i].w = w[i]->dev;
        J.seg[i].y = y[i];
        J.seg[i].ldy = ldy[i];
        J.seg[i].n = (int)w[i]->N;
    }
    J.qt = w[0]->type;
    J.K = (int)w[0]->K;
    J.Kpad = (int)w[0]->Kpad;
    J.row_bytes = w[0]->row_bytes;
    J.x = x;
    J.ldx = ldx;
    J.x_is_bf16 = x_dtype == B200Q_TYPE_BF16;
    const size_t xelt = act_size(x_dtype);
    J.x_vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((ldx * xelt) % 16 == 0);
    J.y_is_bf16 = y_dtype == B200Q_TYPE_BF16;
    J.flags = flags;
    J.team = 0;
    J.xq = nullptr;
    stream_job_finish(J);
}

b200q_status run_stream(b200q_ctx *ctx, const StreamJob *jobs_host, const StreamJob *jobs_dev, int njobs, int M,
                        cudaStream_t st) {
    StreamLaunch a{};
    a.jobs_host = jobs_host;
    a.jobs_dev = jobs_dev;
    a.njobs = njobs;
    a.M = M;
    a.status = ctx->status_dev;
    a.counter = reinterpret_cast<unsigned *>(ctx->status_dev) + 16;   // its own 64-byte line
    a.sm_count = ctx->sm_count;
    a.smem_limit = (ctx->gemv_smem > 0 && (size_t)ctx->gemv_smem < ctx->smem_optin) ? (size_t)ctx->gemv_smem : ctx->smem_optin;
    a.warps = ctx->gemv_warps;
    a.depth = ctx->gemv_depth;
    a.grid = ctx->gemv_grid;
    a.debug = ctx->gemv_debug;
    a.pdl = ctx->gemv_pdl;
    a.teams = ctx->gemv_teams;
    a.producer_nap = ctx->gemv_nap;
    a.peer_rank = ctx->peer_rank;
    a.peer_world = ctx->peer_world;
    for (int r = 0; r < kPeerMaxWorld; ++r) a.peer_base[r] = ctx->peer_base[r];
    cudaError_t e = stream_launch(a, st);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "streaming kernel launch");
    return B200Q_OK;
}

b200q_status run_gemv(b200q_ctx *ctx, const b200q_weight *const *w, int nw, const void *x, int x_dtype,
                      int M, int64_t ldx, void *const *y, int y_dtype, const int64_t *ldy,
                      cudaStream_t st) {
    StreamJob J;
    fill_job(J, w, nw, x, x_dtype, ldx, y, y_dtype, ldy, 0);
    return run_stream(ctx, &J, nullptr, 1, M, st);
}

// prefill route: one activation conversion per weight set and one tensor-core launch per weight
b200q_status run_gemm(b200q_ctx *ctx, const b200q_weight *w, const void *x, int x_dtype, int64_t M, int64_t ldx,
                      void *y, int y_dtype, int64_t ldy, cudaStream_t st, int *launches, bool x_already_converted) {
    // Both tensor-core operands are fp16: the activations are converted into context-owned scratch
    // memory first (once for all the weights of a set, which share them).
    if (!x_already_converted) {
        const size_t need = gemm_x_scratch_bytes((int)M, (int)w->K);
        if (need > ctx->gemm_scratch_bytes) {
            if (ctx->gemm_scratch) {
                CU_TRY(ctx, cudaStreamSynchronize(st));   // earlier launches may still read the old buffer
                cudaFree(ctx->gemm_scratch);
                ctx->gemm_scratch = nullptr;
                ctx->gemm_scratch_bytes = 0;
            }
            CU_TRY(ctx, cudaMalloc(&ctx->gemm_scratch, need));
            ctx->gemm_scratch_bytes = need;
        }
        cudaError_t e = gemm_convert_x(x, x_dtype == B200Q_TYPE_BF16, ldx, ctx->gemm_scratch, (int)M, (int)w->K, st);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "activation conversion launch");
        ++*launches;
    }
    const void *xb = ctx->gemm_scratch;
    const long long ldb = (w->K + 7) & ~int64_t(7);
    GemmLaunch a{};
    a.qt = w->type;
    a.w = w->dev;
    a.N = (int)w->N;
    a.K = (int)w->K;
    a.Kpad = (int)w->Kpad;
    a.x = xb;
    a.ldx = ldb;
    a.M = (int)M;
    a.y = y;
    a.ldy = ldy;
    a.y_is_bf16 = y_dtype == B200Q_TYPE_BF16;
    a.status = ctx->status_dev;
    a.sm_count = ctx->sm_count;
    a.bn_override = ctx->gemm_bn;
    a.debug = ctx->gemm_debug;
    a.pair = ctx->gemm_pair;
    if (M < 128 && !ctx->gemm_part && ctx->gemm_ksplit) {
        void *ptr = nullptr;
        if (cudaMalloc(&ptr, kGemmPartBytes) == cudaSuccess) ctx->gemm_part = reinterpret_cast<float *>(ptr);
        else cudaGetLastError();      // no workspace: the product runs unsplit
    }
    a.part = ctx->gemm_ksplit ? ctx->gemm_part : nullptr;
    a.part_bytes = kGemmPartBytes;
    cudaError_t e = gemm_launch(a, st);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "tensor-core GEMM launch");
    ++*launches;
    return B200Q_OK;
}

// skinny route: 2..16 activation rows, mma.sync on exact integer weights (skinny.cu); all weights of
// the call share x, type and K
b200q_status run_skinny(b200q_ctx *ctx, const b200q_weight *const *w, int nw, const void *x, int x_dtype, int M,
                        int64_t ldx, void *const *y, int y_dtype, const int64_t *ldy, cudaStream_t st) {
    SkinnyProduct prods[4];
    int n = 0;
    size_t need = 0;
    for (int i = 0; i < nw; ++i) {
        if (w[i]->N == 0) continue;
        SkinnyProduct &a = prods[n++];
        a.qt = w[i]->type;
        a.w = w[i]->dev;
        a.N = (int)w[i]->N;
        a.K = (int)w[i]->K;
        a.Kpad = (int)w[i]->Kpad;
        a.x = x;
        a.ldx = ldx;
        a.x_is_bf16 = x_dtype == B200Q_TYPE_BF16;
        a.y = y[i];
        a.ldy = ldy[i];
        a.y_is_bf16 = y_dtype == B200Q_TYPE_BF16;
        a.M = M;
        need += skinny_part_bytes(a);
    }
    if (n == 0) return B200Q_OK;
    if (need > ctx->sk_ws_bytes) {
        if (ctx->sk_ws) {
            CU_TRY(ctx, cudaStreamSynchronize(st));   // earlier launches may still use the old buffer
            cudaFree(ctx->sk_ws);
            ctx->sk_ws = nullptr;
            ctx->sk_ws_bytes = 0;
        }
        const size_t grow = std::max(need, size_t(4) << 20);
        CU_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&ctx->sk_ws), grow));
        ctx->sk_ws_bytes = grow;
    }
    SkinnyBuffers buf{};
    buf.ws = ctx->sk_ws;
    buf.ws_bytes = ctx->sk_ws_bytes;
    buf.jobs_dev = nullptr;      // at most four products: their descriptions travel in the kernel parameters
    buf.status = ctx->status_dev;
    buf.sm_count = ctx->sm_count;
    buf.smem_limit = ctx->smem_optin;
    cudaError_t e = skinny_run(prods, n, buf, st, &ctx->last_launches);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "skinny kernel launch");
    return B200Q_OK;
}

b200q_status validate_mm(b200q_ctx *ctx, const b200q_weight *w, const void *x, int x_dtype, int64_t M,
                         int64_t ldx, const void *y, int y_dtype, int64_t ldy) {
    if (!w) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "null weight");
    if (w->ctx != ctx) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "weight belongs to another context");
    if (!act_type(x_dtype) || !act_type(y_dtype))
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "activation/output dtype must be F32 (0) or BF16 (30)");
    if (M < 0) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "M < 0");
    if (M > 0 && ((!x && w->K > 0) || (!y && w->N > 0)))
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "null activation or output pointer");
    if (ldx < w->K || ldy < w->N) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "leading dimension smaller than the row");
    return B200Q_OK;
}

// One weight set (1..4 weights sharing x), any M: picks the route and launches.
b200q_status matmul_any(b200q_ctx *ctx, const b200q_weight *const *w, int nw, const void *x, int x_dtype,
                        int64_t M, int64_t ldx, void *const *y, int y_dtype, const int64_t *ldy,
                        cudaStream_t st) {
    ctx->last_route = B200Q_ROUTE_NONE;
    ctx->last_launches = 0;
    if (M == 0) return B200Q_OK;
    bool any_rows = false;
    for (int i = 0; i < nw; ++i) any_rows |= w[i]->N > 0;
    if (!any_rows) return B200Q_OK;
    if (w[0]->K == 0) {   // empty contraction: the product is all zeros
        for (int i = 0; i < nw; ++i)
            for (int64_t m = 0; m < M; ++m)
                CU_TRY(ctx, cudaMemsetAsync((char *)y[i] + m * ldy[i] * act_size(y_dtype), 0,
                                            w[i]->N * act_size(y_dtype), st));
        return B200Q_OK;
    }
    const int mt = gemv_max_m();
    if (M >= ctx->skinny_min_m && M <= skinny_max_m()) {
        // verify / small continuous batches: one pass over the packed weights, exact bf16 activations
        ctx->last_route = B200Q_ROUTE_SKINNY;
        const bool f32 = x_dtype != B200Q_TYPE_BF16;
        const int step = f32 ? 8 : 16;     // fp32 rows take two token slots each (high and low halves)
        for (int64_t m0 = 0; m0 < M; m0 += step) {
            const int mc = (int)std::min<int64_t>(step, M - m0);
            void *yy[4];
            for (int i = 0; i < nw; ++i) yy[i] = (char *)y[i] + m0 * ldy[i] * act_size(y_dtype);
            const void *xx = (const char *)x + m0 * ldx * act_size(x_dtype);
            b200q_status s = run_skinny(ctx, w, nw, xx, x_dtype, mc, ldx, yy, y_dtype, ldy, st);
            if (s != B200Q_OK) return s;
        }
        return B200Q_OK;
    }
    if (M > mt) {   // prefill / verify batches: tensor cores, one launch per weight
        ctx->last_route = B200Q_ROUTE_GEMM;
        bool converted = false;
        for (int i = 0; i < nw; ++i) {
            if (w[i]->N == 0) continue;
            b200q_status s = run_gemm(ctx, w[i], x, x_dtype, M, ldx, y[i], y_dtype, ldy[i], st, &ctx->last_launches, converted);
            if (s != B200Q_OK) return s;
            converted = true;
        }
        return B200Q_OK;
    }
    ctx->last_route = B200Q_ROUTE_GEMV;
    for (int64_t m0 = 0; m0 < M; m0 += mt) {
        const int mc = (int)std::min<int64_t>(mt, M - m0);
        void *yy[4];
        for (int i = 0; i < nw; ++i) yy[i] = (char *)y[i] + m0 * ldy[i] * act_size(y_dtype);
        const void *xx = (const char *)x + m0 * ldx * act_size(x_dtype);
        b200q_status s = run_gemv(ctx, w, nw, xx, x_dtype, mc, ldx, yy, y_dtype, ldy, st);
        if (s != B200Q_OK) return s;
        ctx->last_launches++;
    }
    return B200Q_OK;
}

b200q_status ensure_host_path(b200q_ctx *ctx, size_t xb, size_t yb) {
    if (!ctx->hstream) CU_TRY(ctx, cudaStreamCreateWithFlags(&ctx->hstream, cudaStreamNonBlocking));
    if (xb > ctx->hx_bytes) {
        if (ctx->hx_dev) cudaFree(ctx->hx_dev);
        ctx->hx_dev = nullptr;
        ctx->hx_bytes = 0;
        CU_TRY(ctx, cudaMalloc(&ctx->hx_dev, xb));
        ctx->hx_bytes = xb;
    }
    if (yb > ctx->hy_bytes) {
        if (ctx->hy_dev) cudaFree(ctx->hy_dev);
        ctx->hy_dev = nullptr;
        ctx->hy_bytes = 0;
        CU_TRY(ctx, cudaMalloc(&ctx->hy_dev, yb));
        ctx->hy_bytes = yb;
    }
    return B200Q_OK;
}

// A plan on the skinny route (3..16 activation rows by default): consecutive products of one block type form a group that one
// skinny launch runs (a job that reads what earlier jobs wrote starts a new group, so stream order
// provides the dependency); the plan owns the groups' images, chunk sums, counters and job tables.
b200q_status plan_create_skinny(b200q_ctx *ctx, b200q_plan *pl, const b200q_job *jobs, int n_jobs, int M) {
    struct Group { std::vector<SkinnyProduct> prods; };
    std::vector<Group> groups;
    for (int i = 0; i < n_jobs; ++i) {
        const b200q_job &j = jobs[i];
        if (j.n_weights < 1 || j.n_weights > 4) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: 1..4 weights", i);
        if (j.flags & B200Q_JOB_SUM_RANKS)
            return fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: sums over ranks inside the launch need M <= %d", i, gemv_max_m());
        if (j.x_dtype != B200Q_TYPE_BF16 && M > 8)
            return fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: plans of more than 8 rows take bf16 activations", i);
        for (int k = 0; k < j.n_weights; ++k) {
            b200q_status s = validate_mm(ctx, j.w[k], j.x_dev, j.x_dtype, M, j.ldx, j.y_dev[k], j.y_dtype, j.ldy[k]);
            if (s == B200Q_OK && (j.w[k]->type != j.w[0]->type || j.w[k]->K != j.w[0]->K))
                s = fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: weights of one job must share type and K", i);
            if (s != B200Q_OK) return s;
        }
        if (j.w[0]->K == 0) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: K = 0 is not allowed in a plan", i);
        const bool waits = (j.flags & B200Q_JOB_WAITS_FOR_EARLIER) != 0;
        for (int k = 0; k < j.n_weights; ++k) {
            const b200q_weight *w = j.w[k];
            if (w->N == 0) continue;
            SkinnyProduct a{};
            a.qt = w->type;
            a.w = w->dev;
            a.N = (int)w->N;
            a.K = (int)w->K;
            a.Kpad = (int)w->Kpad;
            a.x = j.x_dev;
            a.ldx = j.ldx;
            a.x_is_bf16 = j.x_dtype == B200Q_TYPE_BF16;
            a.y = j.y_dev[k];
            a.ldy = j.ldy[k];
            a.y_is_bf16 = j.y_dtype == B200Q_TYPE_BF16;
            a.M = M;
            const bool fresh = groups.empty() || (waits && k == 0) || groups.back().prods[0].qt != a.qt ||
                               groups.back().prods[0].x_is_bf16 != a.x_is_bf16 ||
                               (int)groups.back().prods.size() >= skinny_max_products();
            if (fresh) groups.emplace_back();
            groups.back().prods.push_back(a);
        }
    }
    size_t ws = 0;
    for (const Group &g : groups)
        for (const SkinnyProduct &a : g.prods) ws += skinny_part_bytes(a);
    if (groups.empty()) return B200Q_OK;
    CU_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->sk_ws), std::max<size_t>(ws, 256)));
    CU_TRY(ctx, cudaMalloc(reinterpret_cast<void **>(&pl->sk_jobs), groups.size() * skinny_job_table_bytes()));
    size_t ws_off = 0;
    for (size_t gi = 0; gi < groups.size(); ++gi) {
        const Group &g = groups[gi];
        size_t gws = 0;
        for (const SkinnyProduct &a : g.prods) gws += skinny_part_bytes(a);
        SkinnyBuffers buf{};
        buf.ws = pl->sk_ws + ws_off;
        buf.ws_bytes = gws;
        buf.jobs_dev = pl->sk_jobs + gi * skinny_job_table_bytes();
        buf.status = ctx->status_dev;
        buf.sm_count = ctx->sm_count;
        buf.smem_limit = ctx->smem_optin;
        SkinnySet *set = nullptr;
        cudaError_t e = skinny_set_create(g.prods.data(), (int)g.prods.size(), buf, &set);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "skinny plan group");
        pl->sets.push_back(set);
        ws_off += gws;
    }
    return B200Q_OK;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
extern "C" {

const char *b200q_version(void) { return "0.1.0"; }

int64_t b200q_tensor_storage_bytes(int32_t type, int64_t n_elements) {
    if (n_elements < 0) return -1;
    if (type == B200Q_TYPE_F32) return n_elements * 4;
    if (type == B200Q_TYPE_BF16) return n_elements * 2;
    if (!known_type(type)) return -1;
    const int64_t be = gguf_block_elems(type);
    if (n_elements % be) return -1;
    return n_elements / be * gguf_block_bytes(type);
}

b200q_status b200q_ctx_create(int32_t device, b200q_ctx **out) {
    if (!out) return B200Q_ERR_INVALID_CONFIG;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return B200Q_ERR_BACKEND;   // no CUDA device: there is no CPU fallback
    }
    if (device < 0 || device >= count) return B200Q_ERR_INVALID_CONFIG;
    b200q_ctx *ctx = new (std::nothrow) b200q_ctx();
    if (!ctx) return B200Q_ERR_OVERLOADED;
    ctx->device = device;
    cudaDeviceProp prop;
    if ((e = cudaSetDevice(device)) != cudaSuccess || (e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) {
        delete ctx;
        return B200Q_ERR_BACKEND;
    }
    if (prop.major != 10) {   // the kernels are sm_100a only
        delete ctx;
        return B200Q_ERR_BACKEND;
    }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    ctx->smem_sm = prop.sharedMemPerMultiprocessor;
    if ((e = cudaMalloc(&ctx->status_dev, 256)) != cudaSuccess || (e = cudaMemset(ctx->status_dev, 0, 256)) != cudaSuccess) {
        delete ctx;
        return e == cudaErrorMemoryAllocation ? B200Q_ERR_OVERLOADED : B200Q_ERR_BACKEND;
    }
    ctx->gemv_warps = env_int("B200Q_GEMV_WARPS", 0);
    ctx->gemv_depth = env_int("B200Q_GEMV_DEPTH", 0);
    ctx->gemv_grid = env_int("B200Q_GEMV_GRID", 0);
    ctx->gemv_smem = env_int("B200Q_GEMV_SMEM", 0);
    ctx->gemv_rows = env_int("B200Q_GEMV_ROWS", 0);
#ifdef B200Q_TIMING_EXPERIMENTS      // pipeline parts switched off for timing: results are invalid, never in a shipped build
    ctx->gemv_debug = env_int("B200Q_GEMV_DEBUG", 0);
    ctx->gemm_debug = env_int("B200Q_GEMM_DEBUG", 0);
#endif
    ctx->gemv_pdl = env_int("B200Q_GEMV_PDL", 1);
    ctx->gemv_teams = env_int("B200Q_GEMV_TEAMS", 2);
    ctx->gemv_xprep = env_int("B200Q_GEMV_XPREP", 1);
    ctx->gemv_nap = env_int("B200Q_GEMV_NAP", 0);
    ctx->gemm_bn = env_int("B200Q_GEMM_BN", 0);
    ctx->gemm_pair = env_int("B200Q_GEMM_PAIR", 1);
    ctx->gemm_ksplit = env_int("B200Q_GEMM_KSPLIT", 1);
    *out = ctx;
    return B200Q_OK;
}

void b200q_ctx_destroy(b200q_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->comm) {
        NcclApi *api = nccl_api();
        if (api) api->CommDestroy(ctx->comm);
    }
    b200q_peer_detach(ctx);
    if (ctx->peer_local) cudaFree(ctx->peer_local);
    if (ctx->hstream) cudaStreamDestroy(ctx->hstream);
    if (ctx->hx_dev) cudaFree(ctx->hx_dev);
    if (ctx->hy_dev) cudaFree(ctx->hy_dev);
    if (ctx->gemm_scratch) cudaFree(ctx->gemm_scratch);
    if (ctx->gemm_part) cudaFree(ctx->gemm_part);
    if (ctx->sk_ws) cudaFree(ctx->sk_ws);
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    delete ctx;
}

b200q_status b200q_ctx_set_option(b200q_ctx *ctx, int32_t option, int64_t value) {
    if (!ctx) return B200Q_ERR_INVALID_CONFIG;
    switch (option) {
    case B200Q_OPT_SKINNY_MIN_M:
        if (value < 2 || value > skinny_max_m() + 1) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "SKINNY_MIN_M must be 2..%d", skinny_max_m() + 1);
        ctx->skinny_min_m = (int)value;
        return B200Q_OK;
    case B200Q_OPT_WAIT_LIMIT_MS: {
        if (value < 1 || value > 600000) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "WAIT_LIMIT_MS must be 1..600000");
        b200q_status s = check_ctx(ctx);
        if (s != B200Q_OK) return s;
        const unsigned long long ns = (unsigned long long)value * 1000000ull;
        CU_TRY(ctx, gemv_set_wait_limit_ns(ns));
        CU_TRY(ctx, skinny_set_wait_limit_ns(ns));
        CU_TRY(ctx, gemm_set_wait_limit_ns(ns));
        CU_TRY(ctx, peer_set_wait_limit_ns(ns));
        return B200Q_OK;
    }
    case B200Q_OPT_TP_INIT_TIMEOUT_MS:
        if (value < 1) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "TP_INIT_TIMEOUT_MS must be positive");
        ctx->tp_timeout_ms = (uint64_t)value;
        return B200Q_OK;
    default:
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "unknown option %d", option);
    }
}

b200q_status b200q_last_error(const b200q_ctx *ctx, char *buf, size_t n) {
    if (!ctx || !buf || n == 0) return B200Q_ERR_INVALID_CONFIG;
    snprintf(buf, n, "%s", ctx->err);
    return B200Q_OK;
}

b200q_status b200q_last_route(const b200q_ctx *ctx, int32_t *route, int32_t *launches) {
    if (!ctx) return B200Q_ERR_INVALID_CONFIG;
    if (route) *route = ctx->last_route;
    if (launches) *launches = ctx->last_launches;
    return B200Q_OK;
}

b200q_status b200q_sync(b200q_ctx *ctx, void *stream, uint64_t timeout_ms) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t e = cudaStreamQuery(st);
        if (e == cudaSuccess) break;
        if (e != cudaErrorNotReady) {
            ctx->poisoned = true;
            return cuda_fail(ctx, e, "stream");
        }
        NcclApi *api = ctx->comm ? nccl_api() : nullptr;
        if (api && api->CommGetAsyncError) {      // a collective that failed on some rank never finishes: ask NCCL
            int async_err = 0;
            if (api->CommGetAsyncError(ctx->comm, &async_err) == 0 && async_err != 0 && async_err != kNcclInProgress) {
                if (api->CommAbort) api->CommAbort(ctx->comm);
                ctx->comm = nullptr;
                ctx->tp_world = 1;
                return fail(ctx, B200Q_ERR_BACKEND, "NCCL reported an asynchronous error (%s); the communicator was aborted",
                            api->GetErrorString ? api->GetErrorString(async_err) : "error");
            }
        }
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (timeout_ms && (uint64_t)ms > timeout_ms) {
            if (api && api->CommAbort) {          // the deadline passed with a communicator attached: its kernels are
                api->CommAbort(ctx->comm);        // told to stop, so the stream can drain and the context be reused
                ctx->comm = nullptr;
                ctx->tp_world = 1;
                return fail(ctx, B200Q_ERR_TIMEOUT, "stream not finished after %llu ms; the NCCL communicator was aborted", (unsigned long long)timeout_ms);
            }
            return fail(ctx, B200Q_ERR_TIMEOUT, "stream not finished after %llu ms", (unsigned long long)timeout_ms);
        }
        std::this_thread::yield();
    }
    int status = 0;
    CU_TRY(ctx, cudaMemcpy(&status, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
    if (status != DEV_OK) {
        cudaMemset(ctx->status_dev, 0, sizeof(int));
        if (ctx->peer_world > 1) ctx->peer_stale = true;     // some rank may have skipped an exchange: counters disagree
        return fail(ctx, B200Q_ERR_TIMEOUT, "a kernel gave up a bounded wait (device status %d); results are invalid", status);
    }
    return B200Q_OK;
}

// -- weights ----------------------------------------------------------------------------------

b200q_status b200q_shard_range(int32_t type, int64_t N, int64_t K, int32_t split, int32_t rank,
                               int32_t world, int64_t align_rows, int64_t *begin, int64_t *end) {
    if (!begin || !end || !known_type(type) || N < 0 || K < 0 || world < 1 || rank < 0 || rank >= world)
        return B200Q_ERR_INVALID_CONFIG;
    if (K % gguf_block_elems(type)) return B200Q_ERR_INVALID_CONFIG;
    if (split == B200Q_SPLIT_COLUMN) {
        const int64_t al = align_rows > 1 ? align_rows : 1;
        if (N % al) return B200Q_ERR_INVALID_CONFIG;
        split_even(N / al, rank, world, begin, end);
        *begin *= al;
        *end *= al;
    } else if (split == B200Q_SPLIT_ROW) {
        split_even((K + SB - 1) / SB, rank, world, begin, end);
        *begin = std::min<int64_t>(K, *begin * SB);
        *end = std::min<int64_t>(K, *end * SB);
    } else {
        return B200Q_ERR_INVALID_CONFIG;
    }
    return B200Q_OK;
}

int64_t b200q_layout_row_bytes(int32_t type, int64_t K) {
    if (!known_type(type) || K < 0 || K % gguf_block_elems(type)) return -1;
    return row_bytes_for(type, (K + SB - 1) / SB);
}

b200q_status b200q_layout_pack(int32_t type, int64_t N, int64_t K, const void *packed_host,
                               size_t bytes, void *out_host, size_t out_bytes) {
    const int64_t rb = b200q_layout_row_bytes(type, K);
    if (rb < 0 || N < 0) return B200Q_ERR_INVALID_CONFIG;
    if ((int64_t)bytes != b200q_tensor_storage_bytes(type, N * K) || (int64_t)out_bytes != padded_rows(N) * rb)
        return B200Q_ERR_INVALID_CONFIG;
    if (N * K == 0) return B200Q_OK;
    if (!packed_host || !out_host) return B200Q_ERR_INVALID_CONFIG;
    memset(out_host, 0, out_bytes);
    repack_host(type, K, (const uint8_t *)packed_host, 0, N, 0, (K + SB - 1) / SB, (uint8_t *)out_host, 0, N);
    return B200Q_OK;
}

b200q_status b200q_weight_upload_shard(b200q_ctx *ctx, int32_t type, int64_t N, int64_t K,
                                       const void *packed_host, size_t bytes, int32_t split,
                                       int32_t rank, int32_t world, int64_t align_rows,
                                       b200q_weight **out) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (!out) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "null out pointer");
    *out = nullptr;
    if (!known_type(type)) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "unsupported ggml type id %d (8=Q8_0, 12=Q4_K, 14=Q6_K)", type);
    if (N < 0 || K < 0) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "negative shape");
    if (K % gguf_block_elems(type))
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "K=%lld is not a multiple of the %d-weight block", (long long)K, gguf_block_elems(type));
    if (N > 0x7FFFFFF0ll || K > 0x3FFFFF00ll) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "shape too large");
    const int64_t want = b200q_tensor_storage_bytes(type, N * K);
    if ((int64_t)bytes != want)
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "byte count %zu does not match the tensor (%lld expected)", bytes, (long long)want);
    if (want > 0 && !packed_host) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "null weight pointer");
    int64_t r0 = 0, r1 = N, k0 = 0, k1 = K;
    if (world != 1 || rank != 0) {
        int64_t b, e;
        if (b200q_shard_range(type, N, K, split, rank, world, align_rows, &b, &e) != B200Q_OK)
            return fail(ctx, B200Q_ERR_INVALID_CONFIG, "bad shard request (split %d rank %d world %d align %lld)", split, rank, world, (long long)align_rows);
        if (split == B200Q_SPLIT_COLUMN) { r0 = b; r1 = e; } else { k0 = b; k1 = e; }
    }
    return make_weight(ctx, type, N, K, (const uint8_t *)packed_host, r0, r1, k0, k1, out);
}

b200q_status b200q_weight_upload(b200q_ctx *ctx, int32_t type, int64_t N, int64_t K,
                                 const void *packed_host, size_t bytes, b200q_weight **out) {
    return b200q_weight_upload_shard(ctx, type, N, K, packed_host, bytes, B200Q_SPLIT_COLUMN, 0, 1, 0, out);
}

b200q_status b200q_weight_clone(b200q_ctx *ctx, const b200q_weight *w, b200q_weight **out) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (!w || !out || w->ctx != ctx) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "bad clone arguments");
    b200q_weight *c = new (std::nothrow) b200q_weight(*w);
    if (!c) return fail(ctx, B200Q_ERR_OVERLOADED, "out of host memory");
    c->dev = nullptr;
    if (w->dev) {
        cudaError_t e = cudaMalloc(&c->dev, w->device_bytes + 256);
        if (e == cudaSuccess) e = cudaMemcpy(c->dev, w->dev, w->device_bytes + 256, cudaMemcpyDeviceToDevice);
        if (e != cudaSuccess) {
            if (c->dev) cudaFree(c->dev);
            delete c;
            return cuda_fail(ctx, e, "weight clone");
        }
    }
    *out = c;
    return B200Q_OK;
}

b200q_status b200q_weight_info(const b200q_weight *w, int32_t *type, int64_t *N, int64_t *K,
                               size_t *gguf_bytes, size_t *device_bytes) {
    if (!w) return B200Q_ERR_INVALID_CONFIG;
    if (type) *type = w->type;
    if (N) *N = w->N;
    if (K) *K = w->K;
    if (gguf_bytes) *gguf_bytes = w->gguf_bytes;
    if (device_bytes) *device_bytes = w->device_bytes;
    return B200Q_OK;
}

void b200q_weight_destroy(b200q_weight *w) {
    if (!w) return;
    if (w->dev) {
        cudaSetDevice(w->device);     // not through w->ctx: the context may be gone already
        cudaFree(w->dev);
    }
    delete w;
}

b200q_status b200q_dequantize(b200q_ctx *ctx, const b200q_weight *w, float *out_dev, void *stream) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (!w || w->ctx != ctx) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "bad weight");
    if (w->N == 0 || w->K == 0) return B200Q_OK;
    if (!out_dev) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "null output pointer");
    cudaError_t e = dequant_launch(w->type, w->dev, w->N, w->K, w->Kpad, w->row_bytes, out_dev, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "dequantize launch");
    return B200Q_OK;
}

// -- projection -------------------------------------------------------------------------------

b200q_status b200q_matmul(b200q_ctx *ctx, const b200q_weight *w, const void *x_dev, int32_t x_dtype,
                          int64_t M, int64_t ldx, void *y_dev, int32_t y_dtype, int64_t ldy,
                          void *stream) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if ((s = validate_mm(ctx, w, x_dev, x_dtype, M, ldx, y_dev, y_dtype, ldy)) != B200Q_OK) return s;
    return matmul_any(ctx, &w, 1, x_dev, x_dtype, M, ldx, &y_dev, y_dtype, &ldy, (cudaStream_t)stream);
}

b200q_status b200q_matmul_multi(b200q_ctx *ctx, const b200q_weight *const *w, int32_t n_weights,
                                const void *x_dev, int32_t x_dtype, int64_t M, int64_t ldx,
                                void *const *y_dev, int32_t y_dtype, const int64_t *ldy, void *stream) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (!w || !y_dev || !ldy || n_weights < 1 || n_weights > 4)
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "matmul_multi takes 1..4 weights");
    for (int i = 0; i < n_weights; ++i) {
        if ((s = validate_mm(ctx, w[i], x_dev, x_dtype, M, ldx, y_dev[i], y_dtype, ldy[i])) != B200Q_OK) return s;
        if (w[i]->type != w[0]->type || w[i]->K != w[0]->K)
            return fail(ctx, B200Q_ERR_INVALID_CONFIG, "weights of one launch must share type and K");
    }
    return matmul_any(ctx, w, n_weights, x_dev, x_dtype, M, ldx, y_dev, y_dtype, ldy, (cudaStream_t)stream);
}

b200q_status b200q_matmul_multi_host(b200q_ctx *ctx, const b200q_weight *const *w, int32_t n_weights,
                                     const void *x_host, int32_t x_dtype, int64_t M, int64_t ldx,
                                     void *const *y_host, int32_t y_dtype, const int64_t *ldy) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (!w || !y_host || !ldy || n_weights < 1 || n_weights > 4)
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "matmul_multi takes 1..4 weights");
    for (int i = 0; i < n_weights; ++i) {
        if ((s = validate_mm(ctx, w[i], x_host, x_dtype, M, ldx, y_host[i], y_dtype, ldy[i])) != B200Q_OK) return s;
        if (w[i]->type != w[0]->type || w[i]->K != w[0]->K)
            return fail(ctx, B200Q_ERR_INVALID_CONFIG, "weights of one launch must share type and K");
    }
    if (M == 0) return B200Q_OK;
    const size_t xs = act_size(x_dtype), ys = act_size(y_dtype);
    const size_t xb = (size_t)((M - 1) * ldx + w[0]->K) * xs;
    size_t yoff[4], yb = 0;
    for (int i = 0; i < n_weights; ++i) {
        yoff[i] = yb;
        yb += (((size_t)((M - 1) * ldy[i] + w[i]->N) * ys) + 255) & ~size_t(255);
    }
    if ((s = ensure_host_path(ctx, xb, yb)) != B200Q_OK) return s;
    cudaStream_t st = ctx->hstream;
    CU_TRY(ctx, cudaMemcpyAsync(ctx->hx_dev, x_host, xb, cudaMemcpyHostToDevice, st));
    void *yd[4];
    for (int i = 0; i < n_weights; ++i) yd[i] = (char *)ctx->hy_dev + yoff[i];
    if ((s = matmul_any(ctx, w, n_weights, ctx->hx_dev, x_dtype, M, ldx, yd, y_dtype, ldy, st)) != B200Q_OK) return s;
    for (int i = 0; i < n_weights; ++i)
        if (w[i]->N > 0)
            CU_TRY(ctx, cudaMemcpyAsync(y_host[i], yd[i], (size_t)((M - 1) * ldy[i] + w[i]->N) * ys, cudaMemcpyDeviceToHost, st));
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        ctx->poisoned = true;
        return cuda_fail(ctx, e, "host-path synchronize");
    }
    return B200Q_OK;
}

b200q_status b200q_matmul_host(b200q_ctx *ctx, const b200q_weight *w, const void *x_host,
                               int32_t x_dtype, int64_t M, int64_t ldx, void *y_host,
                               int32_t y_dtype, int64_t ldy) {
    return b200q_matmul_multi_host(ctx, &w, 1, x_host, x_dtype, M, ldx, &y_host, y_dtype, &ldy);
}

b200q_status b200q_matmul_prefill_noalloc(b200q_ctx *ctx, const b200q_weight *w, const void *x_dev,
                                          int32_t x_dtype, int64_t M, int64_t ldx, void *y_dev, int32_t y_dtype,
                                          int64_t ldy, void *stream) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if ((s = validate_mm(ctx, w, x_dev, x_dtype, M, ldx, y_dev, y_dtype, ldy)) != B200Q_OK) return s;
    if (M == 0 || w->N == 0) return B200Q_OK;
    if (w->K == 0) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "K = 0 is not supported by this entry point");
    const size_t need = (size_t)M * (size_t)((w->K + 7) & ~int64_t(7));
    if (need > gemm_static_scratch_elems())
        return fail(ctx, B200Q_ERR_INVALID_CONFIG,
                    "M x K = %lld x %lld needs %zu scratch elements, the built-in scratch holds %zu (8 MiB of 16-bit values)",
                    (long long)M, (long long)w->K, need, gemm_static_scratch_elems());
    GemmLaunch a{};
    a.qt = w->type;
    a.w = w->dev;
    a.N = (int)w->N;
    a.K = (int)w->K;
    a.Kpad = (int)w->Kpad;
    a.x = x_dev;
    a.ldx = ldx;
    a.M = (int)M;
    a.y = y_dev;
    a.ldy = ldy;
    a.y_is_bf16 = y_dtype == B200Q_TYPE_BF16;
    a.status = ctx->status_dev;
    a.sm_count = ctx->sm_count;
    a.bn_override = ctx->gemm_bn;
    a.debug = ctx->gemm_debug;
    a.pair = ctx->gemm_pair;
    cudaError_t e = gemm_launch_static(a, x_dtype == B200Q_TYPE_BF16, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "prefill launch (built-in scratch)");
    ctx->last_route = B200Q_ROUTE_GEMM;
    ctx->last_launches = 2;
    return B200Q_OK;
}

// -- decode plans -------------------------------------------------------------------------------

b200q_status b200q_plan_create(b200q_ctx *ctx, const b200q_job *jobs, int32_t n_jobs, int64_t M,
                               b200q_plan **out) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (!out) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "null out pointer");
    *out = nullptr;
    if (!jobs || n_jobs < 1) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "a plan needs at least one job");
    if (M < 1 || M > skinny_max_m()) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "plans take 1..%d activation rows", skinny_max_m());
    for (int i = 0; i < n_jobs; ++i)
        if (jobs[i].reserved != 0) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: the reserved field must be 0 (zero-initialise b200q_job)", i);
    b200q_plan *pl = new (std::nothrow) b200q_plan();
    if (!pl) return fail(ctx, B200Q_ERR_OVERLOADED, "out of host memory");
    pl->ctx = ctx;
    pl->device = ctx->device;
    pl->M = (int)M;
    bool rank_sums = false;      // ... or another epilogue only the streaming kernel has
    for (int i = 0; i < n_jobs; ++i)
        rank_sums |= (jobs[i].flags & (B200Q_JOB_SUM_RANKS | B200Q_JOB_SWIGLU | B200Q_JOB_ACCUMULATE)) != 0 || jobs[i].norm_weight != nullptr;
    // 3 or more rows run on the skinny kernel, like single calls; plans that add partial sums over
    // ranks inside the launch stay on the streaming kernel (up to 4 rows)
    if (M > gemv_max_m() || (M >= ctx->skinny_min_m && !rank_sums)) {
        if (rank_sums) {
            delete pl;
            return fail(ctx, B200Q_ERR_INVALID_CONFIG, "rank sums, SWIGLU, ACCUMULATE and fused-norm jobs need a streaming plan (M <= %d)", gemv_max_m());
        }
        s = plan_create_skinny(ctx, pl, jobs, n_jobs, (int)M);
        if (s != B200Q_OK) {
            b200q_plan_destroy(pl);
            return s;
        }
        *out = pl;
        return B200Q_OK;
    }
    for (int i = 0; i < n_jobs; ++i) {
        const b200q_job &j = jobs[i];
        if (j.n_weights < 1 || j.n_weights > 4) {
            delete pl;
            return fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: 1..4 weights", i);
        }
        const bool glu = (j.flags & B200Q_JOB_SWIGLU) != 0;
        if (glu && (j.n_weights != 2 || !j.w[0] || !j.w[1] || j.w[0]->N != j.w[1]->N || (j.flags & B200Q_JOB_SUM_RANKS))) {
            delete pl;
            return fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: SWIGLU takes two weights of equal shape (gate, up) and no rank sum", i);
        }
        bool rows = false;
        for (int k = 0; k < j.n_weights; ++k) {
            const int ky = glu ? 0 : k;      // SWIGLU writes y_dev[0] only
            s = validate_mm(ctx, j.w[k], j.x_dev, j.x_dtype, M, j.ldx, j.y_dev[ky], j.y_dtype, j.ldy[ky]);
            if (s == B200Q_OK && (j.w[k]->type != j.w[0]->type || j.w[k]->K != j.w[0]->K))
                s = fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: weights of one job must share type and K", i);
            if (s != B200Q_OK) {
                delete pl;
                return s;
            }
            rows |= j.w[k]->N > 0;
        }
        if (j.w[0]->K == 0) {
            delete pl;
            return fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: K = 0 is not allowed in a plan", i);
        }
        if (!rows) continue;   // nothing to compute
        int jflags = (j.flags & B200Q_JOB_WAITS_FOR_EARLIER) && !pl->jobs.empty() ? STREAM_JOB_WAITS : 0;
        if (j.flags & B200Q_JOB_SUM_RANKS) {
            if (j.n_weights != 1 || j.y_dtype != B200Q_TYPE_F32 || M * j.w[0]->N > kPeerSlotFloats) {
                delete pl;
                return fail(ctx, B200Q_ERR_INVALID_CONFIG,
                            "job %d: a rank sum takes one weight, fp32 output and at most %d outputs", i, kPeerSlotFloats);
            }
            jflags |= STREAM_JOB_SUM_RANKS;
        }
        if (glu) jflags |= STREAM_JOB_SWIGLU;
        if (j.flags & B200Q_JOB_ACCUMULATE) jflags |= STREAM_JOB_ACCUM;
        StreamJob J;
        fill_job(J, j.w, j.n_weights, j.x_dev, j.x_dtype, j.ldx, j.y_dev, j.y_dtype, j.ldy, jflags);
        if (j.norm_weight) {
            if (!(j.norm_eps >= 0.f) || (reinterpret_cast<uintptr_t>(j.norm_weight) & 3)) {
                delete pl;
                return fail(ctx, B200Q_ERR_INVALID_CONFIG, "job %d: norm_weight must be 4-byte aligned and norm_eps >= 0", i);
            }
            J.gamma = j.norm_weight;
            J.norm_eps = j.norm_eps;
        }
        pl->jobs.push_back(J);
    }
    if (pl->jobs.size() >= 2 && ctx->gemv_xprep) {
        // activations that no job of the plan writes are converted to fixed point once per run by a
        // small launch of its own, instead of by every CTA
        size_t total = 0;
        for (const StreamJob &J : pl->jobs)
            if (!(J.flags & STREAM_JOB_WAITS)) total += stream_xq_bytes(J, (int)M);
        if (total > 0 && cudaMalloc(reinterpret_cast<void **>(&pl->xq_dev), total) == cudaSuccess) {
            size_t off = 0;
            for (StreamJob &J : pl->jobs) {
                if (J.flags & STREAM_JOB_WAITS) continue;
                J.xq = pl->xq_dev + off;
                off += stream_xq_bytes(J, (int)M);
            }
            pl->has_xq = true;
        } else {
            cudaGetLastError();
        }
    }
    if (!pl->jobs.empty()) {
        stream_assign_teams(pl->jobs.data(), (int)pl->jobs.size());
        const size_t bytes = pl->jobs.size() * sizeof(StreamJob);
        cudaError_t e = cudaMalloc(&pl->jobs_dev, bytes);
        if (e == cudaSuccess) e = cudaMemcpy(pl->jobs_dev, pl->jobs.data(), bytes, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            if (pl->jobs_dev) cudaFree(pl->jobs_dev);
            delete pl;
            return cuda_fail(ctx, e, "plan upload");
        }
    }
    *out = pl;
    return B200Q_OK;
}

b200q_status b200q_plan_run(b200q_ctx *ctx, b200q_plan *plan, void *stream) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (!plan || plan->ctx != ctx) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "bad plan");
    ctx->last_route = B200Q_ROUTE_NONE;
    ctx->last_launches = 0;
    if (!plan->sets.empty()) {
        for (const SkinnySet *set : plan->sets) {
            cudaError_t e = skinny_set_launch(set, (cudaStream_t)stream);
            if (e != cudaSuccess) return cuda_fail(ctx, e, "skinny plan launch");
            ctx->last_launches += skinny_set_launches(set);
        }
        ctx->last_route = B200Q_ROUTE_SKINNY;
        return B200Q_OK;
    }
    if (plan->jobs.empty()) return B200Q_OK;
    if (ctx->peer_stale && ctx->peer_world > 1) {
        for (const StreamJob &J : plan->jobs)
            if (J.flags & STREAM_JOB_SUM_RANKS)
                return fail(ctx, B200Q_ERR_STOPPED, "a peer exchange timed out earlier: detach and attach the peers again on every rank");
    }
    if (plan->has_xq) {
        cudaError_t e = stream_xprep_launch(plan->jobs_dev, (int)plan->jobs.size(), plan->M, (cudaStream_t)stream);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "activation prep launch");
    }
    s = run_stream(ctx, plan->jobs.data(), plan->jobs_dev, (int)plan->jobs.size(), plan->M, (cudaStream_t)stream);
    if (s != B200Q_OK) return s;
    ctx->last_route = B200Q_ROUTE_GEMV;
    ctx->last_launches = plan->has_xq ? 2 : 1;
    return B200Q_OK;
}

void b200q_plan_destroy(b200q_plan *plan) {
    if (!plan) return;
    cudaSetDevice(plan->device);      // not through plan->ctx: the context may be gone already
    if (plan->jobs_dev) cudaFree(plan->jobs_dev);
    if (plan->xq_dev) cudaFree(plan->xq_dev);
    for (SkinnySet *set : plan->sets) skinny_set_destroy(set);
    if (plan->sk_ws) cudaFree(plan->sk_ws);
    if (plan->sk_jobs) cudaFree(plan->sk_jobs);
    delete plan;
}

// -- tensor parallel --------------------------------------------------------------------------

b200q_status b200q_tp_unique_id(void *id_out_128) {
    if (!id_out_128) return B200Q_ERR_INVALID_CONFIG;
    NcclApi *api = nccl_api();
    if (!api) return B200Q_ERR_BACKEND;
    NcclUniqueId id;
    if (api->GetUniqueId(&id) != 0) return B200Q_ERR_BACKEND;
    memcpy(id_out_128, &id, sizeof(id));
    return B200Q_OK;
}

b200q_status b200q_tp_init(b200q_ctx *ctx, int32_t rank, int32_t world, const void *id_128) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (world < 1 || rank < 0 || rank >= world || !id_128)
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "bad rank/world (%d/%d) or null id", rank, world);
    if (ctx->comm) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "communicator already initialised");
    NcclApi *api = nccl_api();
    if (!api) return fail(ctx, B200Q_ERR_BACKEND, "libnccl.so.2 could not be loaded");
    NcclUniqueId id;
    memcpy(&id, id_128, sizeof(id));
    // The rendezvous blocks until every rank has joined.  It runs on a helper thread so that this call
    // can give up at the deadline (a rank that never joins must not hang the executor: the reference
    // kills and replaces a backend that misses its one absolute deadline,
    // design/icn/calibration-model-assessment.md:164-177); the helper is then left to finish or fail
    // on its own and its communicator, if it ever gets one, is aborted.
    struct InitState {
        std::promise<int> done;
        NcclComm comm = nullptr;
        std::atomic<bool> abandoned{false};
    };
    auto state = std::make_shared<InitState>();
    std::future<int> fut = state->done.get_future();
    const int device = ctx->device;
    std::thread([state, api, world, id, rank, device] {
        cudaSetDevice(device);
        NcclComm c = nullptr;
        const int rc = api->CommInitRank(&c, world, id, rank);
        state->comm = c;
        if (state->abandoned.load() && rc == 0 && c) {
            if (api->CommAbort) api->CommAbort(c);
            else api->CommDestroy(c);
        }
        state->done.set_value(rc);
    }).detach();
    if (fut.wait_for(std::chrono::milliseconds(ctx->tp_timeout_ms)) != std::future_status::ready) {
        state->abandoned.store(true);
        return fail(ctx, B200Q_ERR_TIMEOUT, "ncclCommInitRank did not finish within %llu ms (rank %d of %d)",
                    (unsigned long long)ctx->tp_timeout_ms, rank, world);
    }
    const int rc = fut.get();
    if (rc != 0) {
        ctx->comm = nullptr;
        return fail(ctx, B200Q_ERR_BACKEND, "ncclCommInitRank: %s", api->GetErrorString ? api->GetErrorString(rc) : "error");
    }
    ctx->comm = state->comm;
    ctx->tp_rank = rank;
    ctx->tp_world = world;
    return B200Q_OK;
}

b200q_status b200q_allreduce(b200q_ctx *ctx, void *y_dev, int64_t count, int32_t dtype, void *stream) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (!act_type(dtype) || count < 0 || (count > 0 && !y_dev))
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "bad all-reduce arguments");
    if (count == 0) return B200Q_OK;
    if (ctx->peer_world > 1 && dtype == B200Q_TYPE_F32 && count <= kPeerSlotFloats &&
        !(reinterpret_cast<uintptr_t>(y_dev) & 3)) {
        if (ctx->peer_stale)
            return fail(ctx, B200Q_ERR_STOPPED, "a peer exchange timed out earlier: detach and attach the peers again on every rank");
        CU_TRY(ctx, cudaSetDevice(ctx->device));
        PeerLaunch a{};
        a.y = reinterpret_cast<float *>(y_dev);
        a.count = (int)count;
        a.rank = ctx->peer_rank;
        a.world = ctx->peer_world;
        for (int r = 0; r < ctx->peer_world; ++r) a.base[r] = ctx->peer_base[r];
        a.status = ctx->status_dev;
        cudaError_t e = peer_allreduce_launch(a, (cudaStream_t)stream);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "peer all-reduce launch");
        return B200Q_OK;
    }
    if (!ctx->comm) {
        if (ctx->tp_world == 1 && ctx->peer_world <= 1) return B200Q_OK;   // single rank: the sum is the input
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "no exchange path for this call: b200q_tp_init has not been called"
                                                   " (the peer path takes fp32 vectors of up to %d elements)", kPeerSlotFloats);
    }
    NcclApi *api = nccl_api();
    int rc = api->AllReduce(y_dev, y_dev, (size_t)count, dtype == B200Q_TYPE_BF16 ? kNcclBfloat16 : kNcclFloat32,
                            kNcclSum, ctx->comm, (cudaStream_t)stream);
    if (rc != 0) return fail(ctx, B200Q_ERR_BACKEND, "ncclAllReduce: %s", api->GetErrorString ? api->GetErrorString(rc) : "error");
    return B200Q_OK;
}

b200q_status b200q_tp_finalize(b200q_ctx *ctx) {
    if (!ctx) return B200Q_ERR_INVALID_CONFIG;
    if (ctx->comm) {
        cudaSetDevice(ctx->device);
        NcclApi *api = nccl_api();
        if (api) api->CommDestroy(ctx->comm);
        ctx->comm = nullptr;
    }
    ctx->tp_world = 1;
    ctx->tp_rank = 0;
    return B200Q_OK;
}

b200q_status b200q_peer_export(b200q_ctx *ctx, void *handle_out_64) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (!handle_out_64) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "null handle buffer");
    static_assert(sizeof(cudaIpcMemHandle_t) == B200Q_PEER_HANDLE_BYTES, "handle size");
    static_assert(kPeerSlotFloats == B200Q_PEER_MAX_COUNT, "peer vector limit");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    if (!ctx->peer_local) {
        void *ptr = nullptr;
        cudaError_t e = cudaMalloc(&ptr, kPeerBufferBytes);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "exchange buffer");
        e = cudaMemset(ptr, 0, kPeerBufferBytes);
        if (e != cudaSuccess) {
            cudaFree(ptr);
            return cuda_fail(ctx, e, "exchange buffer clear");
        }
        ctx->peer_local = reinterpret_cast<uint8_t *>(ptr);
    }
    cudaIpcMemHandle_t h;
    CU_TRY(ctx, cudaIpcGetMemHandle(&h, ctx->peer_local));
    memcpy(handle_out_64, &h, sizeof(h));
    return B200Q_OK;
}

b200q_status b200q_peer_attach(b200q_ctx *ctx, int32_t rank, int32_t world, const void *handles) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world || !handles)
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "bad peer arguments (rank %d of %d, at most %d ranks)", rank, world, kPeerMaxWorld);
    if (!ctx->peer_local) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "b200q_peer_export has not been called");
    if (ctx->peer_world > 0) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "peers are already attached");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    for (int r = 0; r < world; ++r) {
        if (r == rank) {
            ctx->peer_base[r] = ctx->peer_local;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, reinterpret_cast<const char *>(handles) + (size_t)r * sizeof(h), sizeof(h));
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < r; ++q)
                if (q != rank && ctx->peer_base[q]) cudaIpcCloseMemHandle(ctx->peer_base[q]);
            for (int q = 0; q < kPeerMaxWorld; ++q) ctx->peer_base[q] = nullptr;
            return cuda_fail(ctx, e, "mapping a peer's exchange buffer");
        }
        ctx->peer_base[r] = reinterpret_cast<uint8_t *>(ptr);
    }
    ctx->peer_rank = rank;
    ctx->peer_world = world;
    ctx->peer_ipc = true;
    ctx->peer_stale = false;
    return B200Q_OK;
}

b200q_status b200q_peer_buffer(b200q_ctx *ctx, void **buffer_out) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (!buffer_out) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "null out pointer");
    char handle[B200Q_PEER_HANDLE_BYTES];
    if ((s = b200q_peer_export(ctx, handle)) != B200Q_OK) return s;     // allocates and clears the buffer on first use
    *buffer_out = ctx->peer_local;
    return B200Q_OK;
}

b200q_status b200q_peer_attach_buffers(b200q_ctx *ctx, int32_t rank, int32_t world, void *const *buffers) {
    b200q_status s = check_ctx(ctx);
    if (s != B200Q_OK) return s;
    if (world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world || !buffers)
        return fail(ctx, B200Q_ERR_INVALID_CONFIG, "bad peer arguments (rank %d of %d, at most %d ranks)", rank, world, kPeerMaxWorld);
    if (!ctx->peer_local) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "b200q_peer_buffer has not been called");
    if (ctx->peer_world > 0) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "peers are already attached");
    if (buffers[rank] != ctx->peer_local) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "buffers[rank] must be this context's own buffer");
    for (int r = 0; r < world; ++r) {
        if (!buffers[r]) return fail(ctx, B200Q_ERR_INVALID_CONFIG, "null buffer of rank %d", r);
        ctx->peer_base[r] = reinterpret_cast<uint8_t *>(buffers[r]);
    }
    ctx->peer_rank = rank;
    ctx->peer_world = world;
    ctx->peer_ipc = false;
    ctx->peer_stale = false;
    return B200Q_OK;
}

b200q_status b200q_peer_detach(b200q_ctx *ctx) {
    if (!ctx) return B200Q_ERR_INVALID_CONFIG;
    cudaSetDevice(ctx->device);
    if (ctx->peer_ipc)
        for (int r = 0; r < ctx->peer_world; ++r)
            if (r != ctx->peer_rank && ctx->peer_base[r]) cudaIpcCloseMemHandle(ctx->peer_base[r]);
    for (int r = 0; r < kPeerMaxWorld; ++r) ctx->peer_base[r] = nullptr;
    // the next attachment starts from call number zero on every rank: clear what this one left behind
    if (ctx->peer_local && ctx->peer_world > 0) cudaMemset(ctx->peer_local, 0, kPeerBufferBytes);
    ctx->peer_rank = -1;
    ctx->peer_world = 0;
    ctx->peer_ipc = true;
    ctx->peer_stale = false;
    return B200Q_OK;
}

}  // extern "C"
