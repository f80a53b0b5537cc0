// Data-parallel gradient exchange: one process per GPU, NCCL all-reduce (sum) over buckets
// of the flat gradient arena, launched on a communication stream as soon as the tape walker
// has finished the last parameter of a bucket, so the exchange overlaps the rest of
// backward.  The reference has no distributed training; the only contract is that N ranks
// with batch B each behave like one device with batch N*B (losses are batch means, so the
// summed gradient is divided by N inside the optimizer's unscale factor).
//
// Two layers:
//   * the ROUND LOGIC (which bucket is ready, one backward pass per optimizer step, what happens
//     when the transport reports an error or a peer never shows up) is plain host code over a
//     small transport interface (DpOps).  It never blocks without a limit: a failed or timed-out
//     exchange aborts the communicator, marks the state as failed and every later call returns
//     MCB_BACKEND, so a rank whose peer died leaves its training loop with an error instead of
//     waiting in the optimizer for ever.
//   * the NCCL TRANSPORT binds that interface to ncclAllReduce on a high-priority stream.  NCCL is
//     resolved with dlopen at mcb_dp_init, so the library loads on hosts without it.
// A second transport, the test double behind mcb_dp_sim_*, records what the round logic asks for and
// can be told to fail, so the failure paths are tested on a host without any GPU.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <functional>
#include <future>
#include <thread>

#include "handles.h"

using namespace mcbag;

namespace {

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
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
            a.CommAbort = (decltype(a.CommAbort))dlsym(a.lib, "ncclCommAbort");
            a.CommGetAsyncError = (decltype(a.CommGetAsyncError))dlsym(a.lib, "ncclCommGetAsyncError");
            a.GetErrorString = (decltype(a.GetErrorString))dlsym(a.lib, "ncclGetErrorString");
            a.ok = a.GetUniqueId && a.CommInitRank && a.AllReduce && a.CommDestroy && a.CommAbort && a.CommGetAsyncError && a.GetErrorString;
        }
    }
    return a;
}

// What the round logic needs from a transport.  Every call returns at once (it enqueues or queries).
struct DpOps {
    std::function<mcb_status(Arena *, int)> enqueue;  // order bucket b's all-reduce behind the work enqueued so far
    std::function<mcb_status()> join;                 // make the compute stream wait for every all-reduce enqueued so far
    std::function<int()> async_error;                 // 0 = none; else the transport's error code (sticky)
    std::function<bool()> idle;                       // true when nothing enqueued is still running
    std::function<void()> abort;                      // tear the communicator down so that nothing keeps waiting for a peer
    std::function<const char *(int)> error_string;
};

struct DpState {
    DpOps ops;
    int rank = 0, world = 1;
    std::vector<char> launched; // per bucket, this round
    bool round_active = false;  // a backward pass has produced gradients that the optimizer has not consumed yet
    bool failed = false;        // sticky: the communicator was aborted
    int64_t timeout_ms = 300000;
    // NCCL transport
    ncclComm_t comm = nullptr;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ready = nullptr, done = nullptr;
    // MCB_DP_TRACE (diagnostic, tape path only): per bucket, when it became ready and when its all-reduce ended
    bool trace = false;
    std::vector<cudaEvent_t> t_ready, t_end;
    std::vector<int> t_bucket;
};

mcb_status nccl_check(mcb_ctx *ctx, ncclResult_t r, const char *what) {
    if (r == ncclSuccess) return MCB_OK;
    return mcb_fail(ctx, MCB_BACKEND, "nccl %s: %s", what, api().GetErrorString ? api().GetErrorString(r) : "error");
}

// ------------------------------------------------------------------ round logic (no CUDA, no NCCL)
mcb_status dp_fail(mcb_ctx *ctx, DpState *dp, const char *why, int code) {
    if (!dp->failed) {
        dp->failed = true;
        if (dp->ops.abort) dp->ops.abort();
    }
    const char *es = (code && dp->ops.error_string) ? dp->ops.error_string(code) : "";
    return mcb_fail(ctx, MCB_BACKEND, "data-parallel exchange failed (%s%s%s); the communicator was aborted, create a new one to continue", why,
                    es[0] ? ": " : "", es);
}

mcb_status dp_check_alive(mcb_ctx *ctx, DpState *dp) {
    if (dp->failed) return mcb_fail(ctx, MCB_BACKEND, "data-parallel communicator was aborted after an earlier failure");
    return MCB_OK;
}

mcb_status dp_launch_bucket(Arena *a, DpState *dp, int b) {
    mcb_ctx *ctx = a->ctx;
    if (dp->launched[b]) return MCB_OK;
    MCB_TRY(dp_check_alive(ctx, dp));
    dp->launched[b] = 1;
    mcb_status st = dp->ops.enqueue(a, b);
    if (st != MCB_OK) {
        std::string msg = ctx->last_error;
        dp_fail(ctx, dp, "enqueue", 0);
        return mcb_fail(ctx, MCB_BACKEND, "%s; the communicator was aborted", msg.c_str());
    }
    // an error another rank or the network raised since the last call shows up here, before more work piles up behind it
    if (int e = dp->ops.async_error()) return dp_fail(ctx, dp, "asynchronous error", e);
    return MCB_OK;
}

mcb_status dp_grad_ready(Arena *a, DpState *dp, int idx) {
    MCB_TRY(dp_check_alive(a->ctx, dp));
    dp->round_active = true;
    int b = a->bucket_of[idx];
    if (--a->bucket_pending[b] == 0) return dp_launch_bucket(a, dp, b);
    return MCB_OK;
}

void dp_reset_round(Arena *a, DpState *dp) {
    dp->round_active = false;
    std::fill(dp->launched.begin(), dp->launched.end(), 0);
    a->bucket_pending = a->bucket_size;
}

// what the optimizer does first: every bucket takes part (also those whose parameters did not all
// receive a gradient, or the ranks' collectives would not match), then the compute stream waits
mcb_status dp_finish_round(Arena *a, DpState *dp) {
    if (!dp->round_active) return MCB_OK;
    for (size_t b = 0; b < a->bucket_begin.size(); ++b) MCB_TRY(dp_launch_bucket(a, dp, (int)b));
    MCB_TRY(dp->ops.join());
    dp_reset_round(a, dp);
    return MCB_OK;
}

// A second backward pass before the optimizer has consumed the first one would add local gradients into buckets
// that are already summed over the ranks (and possibly still being reduced), and would not be exchanged itself:
// the replicas would drift apart silently.  It is refused before any kernel is enqueued.
mcb_status dp_backward_begin(Arena *a, DpState *dp) {
    MCB_TRY(dp_check_alive(a->ctx, dp));
    if (dp->round_active)
        return mcb_fail(a->ctx, MCB_UNSUPPORTED,
                        "data-parallel arena: one backward pass per optimizer step (gradients of the previous pass are already being all-reduced); "
                        "run the optimizer or zero_grad first, or accumulate on a single rank");
    return MCB_OK;
}

// zero_grad with a round open: the gradients are discarded, but their all-reduces may still run; the compute
// stream waits for them before anything writes the arena again, and the round starts over
mcb_status dp_abandon_round(Arena *a, DpState *dp) {
    if (!dp->round_active) return MCB_OK;
    if (dp->failed) {
        dp_reset_round(a, dp);
        return MCB_OK;
    }
    return dp_finish_round(a, dp);
}

// Bounded host-side wait for everything enqueued (what a synchronising call uses instead of an unbounded
// stream synchronise): polls completion and the transport's error word; on an error or when `timeout_ms`
// pass it aborts the communicator, which releases the streams, and returns MCB_BACKEND.
mcb_status dp_host_wait(mcb_ctx *ctx, DpState *dp, int64_t timeout_ms) {
    MCB_TRY(dp_check_alive(ctx, dp));
    const auto t0 = std::chrono::steady_clock::now();
    for (unsigned spin = 0;; ++spin) {
        if (dp->ops.idle()) return MCB_OK;
        if (int e = dp->ops.async_error()) return dp_fail(ctx, dp, "asynchronous error", e);
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms >= timeout_ms) return dp_fail(ctx, dp, "timed out waiting for the gradient all-reduce: a peer rank did not take part", 0);
        if (ms >= 20) std::this_thread::sleep_for(std::chrono::microseconds(200)); // a healthy step ends within the spinning phase
        (void)spin;
    }
}

// FNV-1a over the bucket layout: ranks whose plans differ would pair up all-reduces of different sizes
uint64_t plan_checksum(const std::vector<int64_t> &begin, const std::vector<int64_t> &end, int world) {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](uint64_t v) {
        for (int i = 0; i < 8; ++i) {
            h ^= (v >> (8 * i)) & 0xffu;
            h *= 1099511628211ull;
        }
    };
    mix((uint64_t)world);
    mix((uint64_t)begin.size());
    for (size_t b = 0; b < begin.size(); ++b) {
        mix((uint64_t)begin[b]);
        mix((uint64_t)end[b]);
    }
    return h;
}

void plan_arena(Arena *a, int64_t bucket_elems, std::vector<int32_t> *bo_out, int32_t *nb_out) {
    int n = (int)a->off.size();
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
    mcb_dp_plan_buckets(sizes.data(), n, bucket_elems > 0 ? bucket_elems : 1, bo.data(), &nb);
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
    if (bo_out) *bo_out = bo;
    if (nb_out) *nb_out = nb;
}

// ------------------------------------------------------------------ NCCL transport
void bind_nccl(mcb_ctx *ctx, DpState *dp) {
    dp->ops.enqueue = [ctx, dp](Arena *a, int b) -> mcb_status {
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
    };
    dp->ops.join = [ctx, dp]() -> mcb_status {
        MCB_CUDA(ctx, cudaEventRecord(dp->done, dp->comm_stream));
        MCB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, dp->done, 0));
        return MCB_OK;
    };
    dp->ops.async_error = [ctx, dp]() -> int {
        if (ctx->capture_id) return 0; // nothing runs while a step is being recorded
        ncclResult_t r = ncclSuccess;
        if (api().CommGetAsyncError(dp->comm, &r) != ncclSuccess) return (int)ncclSystemError;
        return (r == ncclSuccess || r == ncclInProgress) ? 0 : (int)r;
    };
    dp->ops.idle = [ctx, dp]() -> bool {
        return cudaStreamQuery(dp->comm_stream) == cudaSuccess && cudaStreamQuery(ctx->stream) == cudaSuccess;
    };
    dp->ops.abort = [dp]() {
        if (dp->comm) api().CommAbort(dp->comm); // ends the collectives in flight on this rank; the streams drain
        dp->comm = nullptr;
    };
    dp->ops.error_string = [](int code) -> const char * { return api().GetErrorString((ncclResult_t)code); };
}

void dp_trace_report(Arena *a, DpState *dp) {
    mcb_ctx *ctx = a->ctx;
    cudaEvent_t tail = nullptr;
    cudaEventCreate(&tail);
    cudaEventRecord(tail, ctx->stream); // where the compute stream's own backward work ends
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

} // namespace

namespace mcbag {

mcb_status arena_grad_ready(Arena *a, int idx) {
    if (!a->dp_attached) return MCB_OK;
    return dp_grad_ready(a, (DpState *)a->ctx->dp, idx);
}

mcb_status arena_wait_comm(Arena *a) {
    if (!a->dp_attached) return MCB_OK;
    DpState *dp = (DpState *)a->ctx->dp;
    if (!dp->round_active) return dp_check_alive(a->ctx, dp);
    const bool report = dp->trace && !dp->t_ready.empty();
    // launch what is missing first, so that the trace sees every bucket
    for (size_t b = 0; b < a->bucket_begin.size(); ++b) MCB_TRY(dp_launch_bucket(a, dp, (int)b));
    if (report) dp_trace_report(a, dp);
    return dp_finish_round(a, dp);
}

mcb_status arena_backward_begin(Arena *a) {
    if (!a->dp_attached) return MCB_OK;
    return dp_backward_begin(a, (DpState *)a->ctx->dp);
}

mcb_status arena_abandon_round(Arena *a) {
    if (!a->dp_attached) return MCB_OK;
    return dp_abandon_round(a, (DpState *)a->ctx->dp);
}

double arena_grad_divisor(Arena *a) {
    if (!a->dp_attached) return 1.0;
    return 1.0 / (double)((DpState *)a->ctx->dp)->world;
}

} // namespace mcbag

// runtime.cu calls this from its synchronising entry points while a data-parallel state exists
extern "C" mcb_status mcb_dp_bounded_wait(mcb_ctx *ctx) {
    DpState *dp = (DpState *)ctx->dp;
    if (!dp || dp->world <= 1 || ctx->capture_id) return MCB_OK;
    if (dp->failed) return MCB_OK; // the streams were released by the abort; the caller's own synchronise returns
    return dp_host_wait(ctx, dp, dp->timeout_ms);
}

// Waits for one event of the compute stream.  With collectives possibly in flight the wait is bounded and watches the
// communicator for asynchronous errors, like every other host wait of the data-parallel path.
extern "C" mcb_status mcb_dp_wait_event(mcb_ctx *ctx, void *event) {
    cudaEvent_t ev = (cudaEvent_t)event;
    DpState *dp = (DpState *)ctx->dp;
    if (!dp || dp->world <= 1 || dp->failed) {
        MCB_CUDA(ctx, cudaEventSynchronize(ev));
        return MCB_OK;
    }
    MCB_TRY(dp_check_alive(ctx, dp));
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const cudaError_t q = cudaEventQuery(ev);
        if (q == cudaSuccess) return MCB_OK;
        if (q != cudaErrorNotReady) return mcb_cuda_check(ctx, q, "waiting for a step's result");
        if (int e = dp->ops.async_error()) return dp_fail(ctx, dp, "asynchronous error", e);
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms >= dp->timeout_ms) return dp_fail(ctx, dp, "timed out waiting for a step that holds gradient all-reduces: a peer rank did not take part", 0);
        if (ms >= 20) std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

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

mcb_status mcb_dp_check_plan_checksums(const uint64_t *checksums, int32_t world) {
    if (!checksums || world < 1) return MCB_INVALID_ARGUMENT;
    for (int32_t r = 1; r < world; ++r)
        if (checksums[r] != checksums[0]) return MCB_INVALID_ARGUMENT;
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
    if (const char *t = getenv("MCB_DP_TIMEOUT_MS")) dp->timeout_ms = atoll(t) > 0 ? atoll(t) : dp->timeout_ms;
    ncclUniqueId id;
    memcpy(&id, host_id_128, 128);
    MCB_CUDA(ctx, cudaSetDevice(ctx->device));
    // The rendezvous blocks until every rank has called it.  It runs on a helper thread so that a rank that
    // never joins costs this rank a timeout, not its life; on a timeout the helper is left behind (it owns
    // nothing but its own arguments) and the context stays usable without data parallelism.
    struct InitJob {
        std::promise<ncclResult_t> done;
        ncclComm_t comm = nullptr;
    };
    auto job = std::make_shared<InitJob>();
    std::future<ncclResult_t> fut = job->done.get_future();
    const int device = ctx->device;
    std::thread([job, world, id, rank, device]() {
        cudaSetDevice(device);
        ncclResult_t r = api().CommInitRank(&job->comm, world, id, rank);
        job->done.set_value(r);
    }).detach();
    if (fut.wait_for(std::chrono::milliseconds(dp->timeout_ms)) != std::future_status::ready) {
        delete dp;
        return mcb_fail(ctx, MCB_BACKEND, "nccl comm init: rendezvous of %d ranks timed out after %lld ms (a rank did not join)", world,
                        (long long)dp->timeout_ms);
    }
    mcb_status st = nccl_check(ctx, fut.get(), "comm init");
    if (st != MCB_OK) {
        delete dp;
        return st;
    }
    dp->comm = job->comm;
    int lo, hi;
    MCB_CUDA(ctx, cudaDeviceGetStreamPriorityRange(&lo, &hi));
    MCB_CUDA(ctx, cudaStreamCreateWithPriority(&dp->comm_stream, cudaStreamNonBlocking, hi));
    MCB_CUDA(ctx, cudaEventCreateWithFlags(&dp->ready, cudaEventDisableTiming));
    MCB_CUDA(ctx, cudaEventCreateWithFlags(&dp->done, cudaEventDisableTiming));
    dp->trace = getenv("MCB_DP_TRACE") != nullptr;
    bind_nccl(ctx, dp);
    ctx->dp = dp;
    return MCB_OK;
}

mcb_status mcb_dp_set_timeout_ms(mcb_ctx *ctx, int64_t timeout_ms) {
    MCB_CHECK_CTX(ctx);
    if (!ctx->dp) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "call mcb_dp_init first");
    if (timeout_ms <= 0) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "timeout must be positive");
    ((DpState *)ctx->dp)->timeout_ms = timeout_ms;
    return MCB_OK;
}

mcb_status mcb_dp_attach(mcb_ctx *ctx, mcb_arena *arena, int64_t bucket_bytes) {
    MCB_CHECK_CTX(ctx);
    if (!ctx->dp) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "call mcb_dp_init first");
    DpState *dp = (DpState *)ctx->dp;
    MCB_TRY(dp_check_alive(ctx, dp));
    Arena *a = arena->a;
    int32_t nb = 0;
    plan_arena(a, bucket_bytes / 4, nullptr, &nb);
    dp->launched.assign(nb, 0);
    a->dp_attached = dp->world > 1;
    if (!a->dp_attached) return MCB_OK;
    // Every rank must have cut its arena into the same buckets, or all-reduces of different sizes would be paired.
    // The ranks compare a checksum of their plans: max and min of its four 16-bit pieces (exact in f32) must agree.
    const uint64_t cs = plan_checksum(a->bucket_begin, a->bucket_end, dp->world);
    float h[8];
    for (int i = 0; i < 4; ++i) {
        h[i] = (float)((cs >> (16 * i)) & 0xffffu);
        h[4 + i] = -h[i];
    }
    void *d = nullptr;
    MCB_TRY(mcb_alloc(ctx, sizeof(h), &d));
    mcb_status st = mcb_memcpy_h2d(ctx, d, h, sizeof(h));
    if (st == MCB_OK) st = nccl_check(ctx, api().AllReduce(d, d, 8, ncclFloat, ncclMax, dp->comm, ctx->stream), "bucket-plan check");
    if (st == MCB_OK) st = dp_host_wait(ctx, dp, dp->timeout_ms);
    float r[8] = {0};
    if (st == MCB_OK) st = mcb_memcpy_d2h(ctx, r, d, sizeof(r));
    mcb_free(ctx, d);
    MCB_TRY(st);
    for (int i = 0; i < 4; ++i)
        if (r[i] != -r[4 + i]) {
            a->dp_attached = false;
            return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "data-parallel attach: the ranks planned different gradient buckets (different models or bucket sizes)");
        }
    return MCB_OK;
}

mcb_status mcb_dp_allreduce_f32(mcb_ctx *ctx, float *buf, int64_t n, int32_t op_max) {
    MCB_CHECK_CTX(ctx);
    if (!ctx->dp) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "call mcb_dp_init first");
    DpState *dp = (DpState *)ctx->dp;
    MCB_TRY(dp_check_alive(ctx, dp));
    mcb_status st = nccl_check(ctx, api().AllReduce(buf, buf, (size_t)n, ncclFloat, op_max ? ncclMax : ncclSum, dp->comm, ctx->stream), "all-reduce");
    if (st != MCB_OK) {
        dp_fail(ctx, dp, "enqueue", 0);
        return st;
    }
    if (int e = dp->ops.async_error()) return dp_fail(ctx, dp, "asynchronous error", e);
    return MCB_OK;
}

mcb_status mcb_dp_shutdown(mcb_ctx *ctx) {
    MCB_CHECK_CTX(ctx);
    if (!ctx->dp) return MCB_OK;
    DpState *dp = (DpState *)ctx->dp;
    mcb_status st = MCB_OK;
    if (!dp->failed) st = dp_host_wait(ctx, dp, dp->timeout_ms); // bounded; aborts the communicator when it runs out
    cudaStreamSynchronize(dp->comm_stream);
    cudaStreamSynchronize(ctx->stream);
    if (dp->comm) {
        mcb_status d = nccl_check(ctx, api().CommDestroy(dp->comm), "comm destroy");
        if (st == MCB_OK) st = d;
    }
    cudaEventDestroy(dp->ready);
    cudaEventDestroy(dp->done);
    cudaStreamDestroy(dp->comm_stream);
    delete dp;
    ctx->dp = nullptr;
    return st;
}

// ------------------------------------------------------------------ test double: the round logic over a recording transport
// Host only (no device, no NCCL).  The simulated arena has `n` parameter slots of the given padded sizes, planned into
// buckets exactly like mcb_dp_attach plans a real one.
struct mcb_dp_sim {
    mcb_ctx ctx;
    Arena arena;
    DpState dp;
    std::vector<int> log;     // buckets in the order their all-reduce was enqueued
    int joins = 0, aborted = 0;
    int fail_enqueue_at = -1; // enqueue of this bucket returns an error (the rank failed before it could take part)
    int async_error_after = -1, polls = 0; // the transport reports an asynchronous error from this many polls on
    bool never_idle = false;  // a peer never joins: the collectives never complete
};

mcb_status mcb_dp_sim_create(const int64_t *slot_sizes, int32_t n, int64_t bucket_elems, int32_t world, mcb_dp_sim **out) {
    if (!slot_sizes || n <= 0 || bucket_elems <= 0 || world < 1 || !out) return MCB_INVALID_ARGUMENT;
    auto *s = new mcb_dp_sim();
    s->arena.ctx = &s->ctx;
    int64_t off = 0;
    for (int32_t i = 0; i < n; ++i) {
        s->arena.off.push_back(off);
        s->arena.size.push_back(slot_sizes[i]);
        off += slot_sizes[i];
    }
    s->arena.total = off;
    int32_t nb = 0;
    plan_arena(&s->arena, bucket_elems, nullptr, &nb);
    s->arena.dp_attached = true;
    s->dp.world = world;
    s->dp.launched.assign(nb, 0);
    s->dp.ops.enqueue = [s](Arena *, int b) -> mcb_status {
        if (b == s->fail_enqueue_at) return mcb_fail(&s->ctx, MCB_BACKEND, "simulated transport: enqueue of bucket %d failed", b);
        s->log.push_back(b);
        return MCB_OK;
    };
    s->dp.ops.join = [s]() -> mcb_status {
        s->joins++;
        return MCB_OK;
    };
    s->dp.ops.async_error = [s]() -> int { return (s->async_error_after >= 0 && s->polls++ >= s->async_error_after) ? 7 : 0; };
    s->dp.ops.idle = [s]() -> bool { return !s->never_idle; };
    s->dp.ops.abort = [s]() { s->aborted++; };
    s->dp.ops.error_string = [](int) -> const char * { return "simulated remote error"; };
    *out = s;
    return MCB_OK;
}
void mcb_dp_sim_release(mcb_dp_sim *s) { delete s; }
mcb_status mcb_dp_sim_backward_begin(mcb_dp_sim *s) { return dp_backward_begin(&s->arena, &s->dp); }
mcb_status mcb_dp_sim_grad_ready(mcb_dp_sim *s, int32_t param) {
    if (param < 0 || param >= (int32_t)s->arena.off.size()) return MCB_INVALID_ARGUMENT;
    return dp_grad_ready(&s->arena, &s->dp, param);
}
mcb_status mcb_dp_sim_finish(mcb_dp_sim *s) { return s->dp.round_active ? dp_finish_round(&s->arena, &s->dp) : dp_check_alive(&s->ctx, &s->dp); }
mcb_status mcb_dp_sim_zero_grad(mcb_dp_sim *s) { return dp_abandon_round(&s->arena, &s->dp); }
mcb_status mcb_dp_sim_host_wait(mcb_dp_sim *s, int32_t timeout_ms) { return dp_host_wait(&s->ctx, &s->dp, timeout_ms); }
void mcb_dp_sim_inject(mcb_dp_sim *s, int32_t what, int32_t value) {
    if (what == 0) s->fail_enqueue_at = value;
    else if (what == 1) s->async_error_after = value;
    else if (what == 2) s->never_idle = value != 0;
}
int32_t mcb_dp_sim_log(mcb_dp_sim *s, int32_t *buckets_out, int32_t max) {
    for (int32_t i = 0; i < max && i < (int32_t)s->log.size(); ++i) buckets_out[i] = s->log[i];
    return (int32_t)s->log.size();
}
int32_t mcb_dp_sim_bucket_of(mcb_dp_sim *s, int32_t param) { return s->arena.bucket_of[param]; }
int32_t mcb_dp_sim_buckets(mcb_dp_sim *s) { return (int32_t)s->arena.bucket_begin.size(); }
int32_t mcb_dp_sim_joins(mcb_dp_sim *s) { return s->joins; }
int32_t mcb_dp_sim_aborted(mcb_dp_sim *s) { return s->aborted; }
uint64_t mcb_dp_sim_plan_checksum(mcb_dp_sim *s) { return plan_checksum(s->arena.bucket_begin, s->arena.bucket_end, s->dp.world); }
const char *mcb_dp_sim_last_error(mcb_dp_sim *s) { return s->ctx.last_error.c_str(); }

} // extern "C"
