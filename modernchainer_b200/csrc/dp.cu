// Data-parallel gradient exchange: one process per GPU, NCCL all-reduce (sum) over buckets
// of the flat gradient arena, launched on a communication stream as soon as the tape walker
// has finished the last parameter of a bucket, so the exchange overlaps the rest of
// backward.  The reference has no distributed training; the only contract is that N ranks
// with batch B each behave like one device with batch N*B (losses are batch means, so the
// summed gradient is divided by N inside the optimizer's unscale factor).
//
// NCCL is resolved with dlopen at mcb_dp_init, so the library loads on hosts without it.
#include <dlfcn.h>
#include <nccl.h>

#include "handles.h"

using namespace mcbag;

namespace {

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

NcclApi &api() {
    static NcclApi a;
    if (!a.lib) {
        a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!a.lib) a.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (a.lib) {
            a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(a.lib, "ncclGetUniqueId");
            a.CommInitRank = (decltype(a.CommInitRank))dlsym(a.lib, "ncclCommInitRank");
            a.AllReduce = (decltype(a.AllReduce))dlsym(a.lib, "ncclAllReduce");
            a.CommDestroy = (decltype(a.CommDestroy))dlsym(a.lib, "ncclCommDestroy");
            a.GetErrorString = (decltype(a.GetErrorString))dlsym(a.lib, "ncclGetErrorString");
            a.ok = a.GetUniqueId && a.CommInitRank && a.AllReduce && a.CommDestroy && a.GetErrorString;
        }
    }
    return a;
}

struct DpState {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ready = nullptr, done = nullptr;
    std::vector<char> launched; // per bucket, this round
    bool round_active = false;
    // MCB_DP_TRACE (diagnostic, tape path only): per bucket, when it became ready and when its all-reduce ended
    bool trace = false;
    std::vector<cudaEvent_t> t_ready, t_end;
    std::vector<int> t_bucket;
};

mcb_status nccl_check(mcb_ctx *ctx, ncclResult_t r, const char *what) {
    if (r == ncclSuccess) return MCB_OK;
    return mcb_fail(ctx, MCB_BACKEND, "nccl %s: %s", what, api().GetErrorString ? api().GetErrorString(r) : "error");
}

mcb_status launch_bucket(Arena *a, int b) {
    mcb_ctx *ctx = a->ctx;
    DpState *dp = (DpState *)ctx->dp;
    if (dp->launched[b]) return MCB_OK;
    dp->launched[b] = 1;
    // everything that produced this bucket's gradients is already enqueued on the compute stream
    MCB_CUDA(ctx, cudaEventRecord(dp->ready, ctx->stream));
    MCB_CUDA(ctx, cudaStreamWaitEvent(dp->comm_stream, dp->ready, 0));
    float *g = (float *)a->g->p + a->bucket_begin[b];
    size_t count = (size_t)(a->bucket_end[b] - a->bucket_begin[b]);
    const bool trace = dp->trace && ctx->capture_id == 0;
    if (trace) {
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, dp->comm_stream);
        dp->t_ready.push_back(e0);
        dp->t_end.push_back(e1);
        dp->t_bucket.push_back(b);
    }
    mcb_status st = nccl_check(ctx, api().AllReduce(g, g, count, ncclFloat, ncclSum, dp->comm, dp->comm_stream), "all-reduce");
    if (trace) cudaEventRecord(dp->t_end.back(), dp->comm_stream);
    return st;
}

} // namespace

namespace mcbag {

mcb_status arena_grad_ready(Arena *a, int idx) {
    if (!a->dp_attached) return MCB_OK;
    DpState *dp = (DpState *)a->ctx->dp;
    dp->round_active = true;
    int b = a->bucket_of[idx];
    if (--a->bucket_pending[b] == 0) return launch_bucket(a, b);
    return MCB_OK;
}

mcb_status arena_wait_comm(Arena *a) {
    if (!a->dp_attached) return MCB_OK;
    mcb_ctx *ctx = a->ctx;
    DpState *dp = (DpState *)ctx->dp;
    if (!dp->round_active) return MCB_OK;
    // buckets whose parameters did not all receive a gradient still have to take part,
    // or the ranks' collectives would not match
    for (size_t b = 0; b < a->bucket_begin.size(); ++b) MCB_TRY(launch_bucket(a, (int)b));
    cudaEvent_t tail = nullptr;
    if (dp->trace && !dp->t_ready.empty()) { // where the compute stream's own backward work ends
        cudaEventCreate(&tail);
        cudaEventRecord(tail, ctx->stream);
    }
    MCB_CUDA(ctx, cudaEventRecord(dp->done, dp->comm_stream));
    MCB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, dp->done, 0));
    if (tail) {
        cudaStreamSynchronize(dp->comm_stream);
        cudaStreamSynchronize(ctx->stream);
        if (dp->rank == 0) {
            for (size_t i = 0; i < dp->t_ready.size(); ++i) {
                float r = 0, e = 0;
                cudaEventElapsedTime(&r, dp->t_ready[0], dp->t_ready[i]);
                cudaEventElapsedTime(&e, dp->t_ready[0], dp->t_end[i]);
                fprintf(stderr, "dp trace: bucket %d (%.1f MB) ready %.3f ms, reduced %.3f ms\n", dp->t_bucket[i],
                        (a->bucket_end[dp->t_bucket[i]] - a->bucket_begin[dp->t_bucket[i]]) * 4e-6, r, e);
            }
            float t = 0;
            cudaEventElapsedTime(&t, dp->t_ready[0], tail);
            fprintf(stderr, "dp trace: compute stream reaches the optimizer at %.3f ms\n", t);
        }
        for (cudaEvent_t e : dp->t_ready) cudaEventDestroy(e);
        for (cudaEvent_t e : dp->t_end) cudaEventDestroy(e);
        cudaEventDestroy(tail);
        dp->t_ready.clear();
        dp->t_end.clear();
        dp->t_bucket.clear();
    }
    dp->round_active = false;
    std::fill(dp->launched.begin(), dp->launched.end(), 0);
    a->bucket_pending = a->bucket_size;
    return MCB_OK;
}

double arena_grad_divisor(Arena *a) {
    if (!a->dp_attached) return 1.0;
    return 1.0 / (double)((DpState *)a->ctx->dp)->world;
}

} // namespace mcbag

extern "C" {

mcb_status mcb_dp_plan_buckets(const int64_t *sizes, int32_t n, int64_t bucket_elems, int32_t *bucket_of,
                               int32_t *n_buckets_out) {
    if (n < 0 || (n > 0 && (!sizes || !bucket_of)) || bucket_elems <= 0) return MCB_INVALID_ARGUMENT;
    int32_t b = 0;
    int64_t fill = 0;
    for (int32_t i = n - 1; i >= 0; --i) {
        if (fill > 0 && fill + sizes[i] > bucket_elems) {
            ++b;
            fill = 0;
        }
        bucket_of[i] = b;
        fill += sizes[i];
    }
    if (n_buckets_out) *n_buckets_out = n > 0 ? b + 1 : 0;
    return MCB_OK;
}

mcb_status mcb_dp_unique_id(void *host_id_out_128) {
    if (!api().ok) return MCB_BACKEND;
    ncclUniqueId id;
    if (api().GetUniqueId(&id) != ncclSuccess) return MCB_BACKEND;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    memcpy(host_id_out_128, &id, 128);
    return MCB_OK;
}

mcb_status mcb_dp_init(mcb_ctx *ctx, int32_t rank, int32_t world, const void *host_id_128) {
    MCB_CHECK_CTX(ctx);
    if (!api().ok) return mcb_fail(ctx, MCB_BACKEND, "libnccl.so.2 could not be loaded");
    if (ctx->dp) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "data-parallel state already initialised");
    if (world < 1 || rank < 0 || rank >= world) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "bad rank/world");
    DpState *dp = new DpState();
    dp->rank = rank;
    dp->world = world;
    ncclUniqueId id;
    memcpy(&id, host_id_128, 128);
    MCB_CUDA(ctx, cudaSetDevice(ctx->device));
    mcb_status st = nccl_check(ctx, api().CommInitRank(&dp->comm, world, id, rank), "comm init");
    if (st != MCB_OK) {
        delete dp;
        return st;
    }
    int lo, hi;
    MCB_CUDA(ctx, cudaDeviceGetStreamPriorityRange(&lo, &hi));
    MCB_CUDA(ctx, cudaStreamCreateWithPriority(&dp->comm_stream, cudaStreamNonBlocking, hi));
    MCB_CUDA(ctx, cudaEventCreateWithFlags(&dp->ready, cudaEventDisableTiming));
    MCB_CUDA(ctx, cudaEventCreateWithFlags(&dp->done, cudaEventDisableTiming));
    dp->trace = getenv("MCB_DP_TRACE") != nullptr;
    ctx->dp = dp;
    return MCB_OK;
}

mcb_status mcb_dp_attach(mcb_ctx *ctx, mcb_arena *arena, int64_t bucket_bytes) {
    MCB_CHECK_CTX(ctx);
    if (!ctx->dp) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "call mcb_dp_init first");
    DpState *dp = (DpState *)ctx->dp;
    Arena *a = arena->a;
    int n = (int)a->vars.size();
    // plan over the slots in arena order (the arena places matrices before vectors), so that every
    // bucket is one contiguous range; walking from the arena's end meets the vectors (small, final
    // only late in backward), then the last layers' matrices, which are the first to be ready
    std::vector<int> order(n);
    for (int i = 0; i < n; ++i) order[i] = i;
    std::sort(order.begin(), order.end(), [&](int x, int y) { return a->off[x] < a->off[y]; });
    std::vector<int64_t> sizes(n);
    for (int j = 0; j < n; ++j) sizes[j] = (j + 1 < n ? a->off[order[j + 1]] : a->total) - a->off[order[j]]; // padded slot sizes
    std::vector<int32_t> bo(n);
    int32_t nb = 0;
    MCB_TRY(mcb_dp_plan_buckets(sizes.data(), n, bucket_bytes / 4 > 0 ? bucket_bytes / 4 : 1, bo.data(), &nb));
    a->bucket_of.assign(n, 0);
    a->bucket_begin.assign(nb, INT64_MAX);
    a->bucket_end.assign(nb, 0);
    a->bucket_size.assign(nb, 0);
    for (int j = 0; j < n; ++j) {
        int b = bo[j], i = order[j];
        a->bucket_of[i] = b;
        a->bucket_begin[b] = std::min(a->bucket_begin[b], a->off[i]);
        a->bucket_end[b] = std::max(a->bucket_end[b], a->off[i] + sizes[j]);
        a->bucket_size[b] += 1;
    }
    a->bucket_pending = a->bucket_size;
    dp->launched.assign(nb, 0);
    a->dp_attached = dp->world > 1;
    return MCB_OK;
}

mcb_status mcb_dp_allreduce_f32(mcb_ctx *ctx, float *buf, int64_t n, int32_t op_max) {
    MCB_CHECK_CTX(ctx);
    if (!ctx->dp) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "call mcb_dp_init first");
    DpState *dp = (DpState *)ctx->dp;
    return nccl_check(ctx, api().AllReduce(buf, buf, (size_t)n, ncclFloat, op_max ? ncclMax : ncclSum, dp->comm, ctx->stream), "all-reduce");
}

mcb_status mcb_dp_shutdown(mcb_ctx *ctx) {
    MCB_CHECK_CTX(ctx);
    if (!ctx->dp) return MCB_OK;
    DpState *dp = (DpState *)ctx->dp;
    cudaStreamSynchronize(dp->comm_stream);
    cudaStreamSynchronize(ctx->stream);
    api().CommDestroy(dp->comm);
    cudaEventDestroy(dp->ready);
    cudaEventDestroy(dp->done);
    cudaStreamDestroy(dp->comm_stream);
    delete dp;
    ctx->dp = nullptr;
    return MCB_OK;
}

} // extern "C"
