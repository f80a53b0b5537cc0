// Runtime: context, stream, caching allocator, copies, events, error word.
// Replaces CudaRuntime / CudaPool / CudaStorage of the reference
// (crates/modern-chainer-cuda/src/backend.rs:13-191,269-451).
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

mcb_status mcb_fail(mcb_ctx *ctx, mcb_status st, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) ctx->last_error = buf;
    return st;
}

mcb_status mcb_cuda_check(mcb_ctx *ctx, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return MCB_OK;
    // same text shape as the reference's Error::Backend(format!("cuda {context}: {error}"))
    return mcb_fail(ctx, MCB_BACKEND, "cuda %s: %s", what, cudaGetErrorString(e));
}

static size_t round_size(size_t bytes) {
    // 512 B granularity below 1 MiB, 2 MiB granularity above: few distinct bucket sizes,
    // every block 256-byte aligned (cudaMalloc alignment) so vector access is always legal.
    if (bytes == 0) bytes = 1;
    if (bytes < (1u << 20)) return (bytes + 511) & ~size_t(511);
    return (bytes + (2u << 20) - 1) & ~size_t((2u << 20) - 1);
}

// One thread samples (wall-clock ns, SM cycle counter) every `interval_ns` for `duration_ns`
// (both bounded by the host).  Consecutive samples give the SM clock that kernels running
// beside it on other streams actually saw, at a far finer grain than driver polling.
__global__ void clock_trace_kernel(unsigned long long *buf, int cap, unsigned long long duration_ns, unsigned long long interval_ns) {
    unsigned long long t0, t, next;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    next = t0;
    int n = 0;
    for (;;) {
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        if (t >= next) {
            if (n < cap) {
                buf[1 + 2 * n] = t;
                buf[2 + 2 * n] = (unsigned long long)clock64();
                ++n;
            }
            next += interval_ns;
        }
        if (t - t0 >= duration_ns || n >= cap) break;
        __nanosleep(200);
    }
    buf[0] = (unsigned long long)n;
}

// the environment names of McbKnob, in its order
static const char *const kKnobNames[K_COUNT] = {
    "MCB_UNFUSED_BWD", "MCB_LN_NO_AUX", "MCB_UNFUSED_ADD_LN", "MCB_UNFUSED_QKV", "MCB_CONV_DIRECT", "MCB_FLASH_LEGACY", "MCB_FLASH_LEGACY_BWD",
    "MCB_SGEMM_NO_SPLIT", "MCB_LN_NO_BULK", "MCB_SCE_NO_STREAM", "MCB_TC_EPI", "MCB_TC_EPI_KB", "MCB_TC_STAGES", "MCB_TC_DIRECT_OUT", "MCB_TC_BN",
    "MCB_TC_PAIR", "MCB_TC_SPLIT_TAIL", "MCB_GRAPH_INFO", "MCB_DETERMINISTIC", "MCB_NO_DEP_LAUNCH", "MCB_FLASH_DQ_RECOMPUTE", "MCB_FLASH_BWD_ONE_JOB"};

extern "C" {

int32_t mcb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

mcb_status mcb_ctx_create(int32_t ordinal, mcb_ctx **out) {
    if (!out) return MCB_INVALID_ARGUMENT;
    *out = nullptr;
    int n = mcb_device_count();
    if (ordinal < 0 || ordinal >= n) return MCB_BACKEND; // no device: there is no CPU fallback
    mcb_ctx *ctx = new mcb_ctx();
    ctx->device = ordinal;
    cudaError_t e = cudaSetDevice(ordinal);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->d_err, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(ctx->d_err, 0, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->tc_fix_cnt, mcb_ctx::kTcFixCntBytes);
    if (e == cudaSuccess) e = cudaMemset(ctx->tc_fix_cnt, 0, mcb_ctx::kTcFixCntBytes);
    cudaDeviceProp prop;
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, ordinal);
    if (e != cudaSuccess) {
        fprintf(stderr, "mcb_ctx_create: %s\n", cudaGetErrorString(e));
        delete ctx;
        return MCB_BACKEND;
    }
    ctx->sm_count = prop.multiProcessorCount;
    // MCB_SM_LIMIT: size persistent grids for fewer SMs (leaves room for communication kernels that run beside the step)
    if (const char *lim = getenv("MCB_SM_LIMIT")) {
        int v = atoi(lim);
        if (v >= 8 && v < ctx->sm_count) ctx->sm_count = v;
    }
    for (int k = 0; k < K_COUNT; ++k) {
        const char *v = getenv(kKnobNames[k]);
        ctx->knobs[k] = !v ? -1 : ((*v >= '0' && *v <= '9') ? atoi(v) : 1);
    }
    ctx->dep_launch = !knob_on(ctx, K_NO_DEP_LAUNCH); // test knob: plain stream-ordered launches
    *out = ctx;
    return MCB_OK;
}

mcb_status mcb_set_knob(mcb_ctx *ctx, const char *name, int32_t value) {
    MCB_CHECK_CTX(ctx);
    if (!name) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "mcb_set_knob: no name");
    for (int k = 0; k < K_COUNT; ++k)
        if (!strcmp(name, kKnobNames[k])) {
            ctx->knobs[k] = value < 0 ? -1 : value;
            if (k == K_NO_DEP_LAUNCH) ctx->dep_launch = value < 0;
            return MCB_OK;
        }
    return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "mcb_set_knob: unknown knob %s", name);
}

void mcb_ctx_destroy(mcb_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto &kv : ctx->free_blocks) cudaFree(kv.second);
    for (auto &kv : ctx->live) cudaFree(kv.first);
    if (ctx->scratch) cudaFree(ctx->scratch);
    for (void *p : ctx->retired_scratch) cudaFree(p);
    for (auto &kv : ctx->graph_free)
        for (auto &b : kv.second) cudaFree(b.second);
    if (ctx->trace_stream) {
        cudaStreamSynchronize(ctx->trace_stream);
        cudaStreamDestroy(ctx->trace_stream);
    }
    if (ctx->trace_buf) cudaFree(ctx->trace_buf);
    cudaFree(ctx->d_err);
    cudaFree(ctx->tc_fix_cnt);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char *mcb_last_error(mcb_ctx *ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

mcb_status mcb_alloc(mcb_ctx *ctx, size_t bytes, void **out) {
    MCB_CHECK_CTX(ctx);
    if (!out) return MCB_INVALID_ARGUMENT;
    size_t sz = round_size(bytes);
    std::lock_guard<std::mutex> lk(ctx->mu);
    void *p = nullptr;
    if (ctx->capture_id) {
        // blocks this step already owns first (a second capture of the same step finds the first one's blocks)
        auto &own = ctx->graph_free[ctx->capture_id];
        auto g = own.find(sz);
        if (g != own.end()) {
            p = g->second;
            own.erase(g);
            ctx->live[p] = sz;
            *out = p;
            return MCB_OK;
        }
    }
    auto it = ctx->free_blocks.find(sz);
    if (it != ctx->free_blocks.end()) {
        p = it->second;
        ctx->free_blocks.erase(it);
    } else {
        cudaSetDevice(ctx->device);
        cudaError_t e = cudaMalloc(&p, sz);
        if (e != cudaSuccess && ctx->capture_id) return mcb_cuda_check(ctx, e, "alloc during stream capture");
        if (e != cudaSuccess) {
            // release cached blocks once and retry before giving up
            cudaGetLastError();
            cudaStreamSynchronize(ctx->stream);
            for (auto &kv : ctx->free_blocks) cudaFree(kv.second);
            ctx->free_blocks.clear();
            e = cudaMalloc(&p, sz);
            if (e != cudaSuccess) return mcb_cuda_check(ctx, e, "alloc");
        }
        ctx->allocated_bytes += (int64_t)sz;
    }
    if (ctx->capture_id) ctx->graph_owner[p] = ctx->capture_id;
    ctx->live[p] = sz;
    *out = p;
    return MCB_OK;
}

mcb_status mcb_free(mcb_ctx *ctx, void *ptr) {
    MCB_CHECK_CTX(ctx);
    if (!ptr) return MCB_OK;
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->live.find(ptr);
    if (it == ctx->live.end()) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "free of a pointer this context did not allocate");
    // single stream: work already enqueued on the block finishes before any later user starts
    auto own = ctx->graph_owner.find(ptr);
    if (own == ctx->graph_owner.end() && ctx->capture_id) own = ctx->graph_owner.emplace(ptr, ctx->capture_id).first;
    if (own != ctx->graph_owner.end()) ctx->graph_free[own->second].emplace(it->second, ptr); // recorded kernels know this address
    else ctx->free_blocks.emplace(it->second, ptr);
    ctx->live.erase(it);
    return MCB_OK;
}

// A static step is gone: its parked blocks return to the general pool, live ones become ordinary blocks.
void mcb_release_capture_blocks(mcb_ctx *ctx, int capture_id) {
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto f = ctx->graph_free.find(capture_id);
    if (f != ctx->graph_free.end()) {
        for (auto &kv : f->second) ctx->free_blocks.emplace(kv.first, kv.second);
        ctx->graph_free.erase(f);
    }
    for (auto it = ctx->graph_owner.begin(); it != ctx->graph_owner.end();) {
        if (it->second == capture_id) it = ctx->graph_owner.erase(it);
        else ++it;
    }
}

mcb_status mcb_host_alloc(size_t bytes, void **host_out) {
    if (!host_out) return MCB_INVALID_ARGUMENT;
    return cudaMallocHost(host_out, bytes ? bytes : 1) == cudaSuccess ? MCB_OK : MCB_BACKEND;
}
mcb_status mcb_host_free(void *host_ptr) { return cudaFreeHost(host_ptr) == cudaSuccess ? MCB_OK : MCB_BACKEND; }

mcb_status mcb_memcpy_h2d(mcb_ctx *ctx, void *dst, const void *host_src, size_t bytes) {
    MCB_CHECK_CTX(ctx);
    if (bytes == 0) return MCB_OK;
    MCB_CUDA(ctx, cudaMemcpyAsync(dst, host_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return MCB_OK;
}

extern "C" mcb_status mcb_dp_bounded_wait(mcb_ctx *ctx); // dp.cu

static mcb_status take_device_error(mcb_ctx *ctx) {
    unsigned int err = 0;
    // With data-parallel collectives possibly in flight, an unbounded stream synchronise would wait for ever for a
    // peer that died: wait with a limit first (an expired limit aborts the communicator, which releases the stream).
    mcb_status dp_st = ctx->dp ? mcb_dp_bounded_wait(ctx) : MCB_OK;
    MCB_CUDA(ctx, cudaMemcpyAsync(&err, ctx->d_err, sizeof(err), cudaMemcpyDeviceToHost, ctx->stream));
    MCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (dp_st != MCB_OK) return dp_st;
    if (err) {
        MCB_CUDA(ctx, cudaMemsetAsync(ctx->d_err, 0, sizeof(err), ctx->stream));
        if (err & MCB_DEVERR_TIMEOUT) {
            // a GEMM that gave up may have left its split-tail counters half counted
            MCB_CUDA(ctx, cudaMemsetAsync(ctx->tc_fix_cnt, 0, mcb_ctx::kTcFixCntBytes, ctx->stream));
            return mcb_fail(ctx, MCB_BACKEND, "device-side wait timed out");
        }
        if (err & MCB_DEVERR_LABEL) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "class index negative or out of range");
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "embedding index negative or out of range");
    }
    return MCB_OK;
}

mcb_status mcb_memcpy_d2h(mcb_ctx *ctx, void *host_dst, const void *src, size_t bytes) {
    MCB_CHECK_CTX(ctx);
    if (bytes) MCB_CUDA(ctx, cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return take_device_error(ctx);
}

mcb_status mcb_memcpy_d2h_async(mcb_ctx *ctx, void *host_dst, const void *src, size_t bytes) {
    MCB_CHECK_CTX(ctx);
    if (bytes) MCB_CUDA(ctx, cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return MCB_OK;
}

mcb_status mcb_memcpy_d2d(mcb_ctx *ctx, void *dst, const void *src, size_t bytes) {
    MCB_CHECK_CTX(ctx);
    if (bytes) MCB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return MCB_OK;
}

mcb_status mcb_memset(mcb_ctx *ctx, void *dst, int32_t byte, size_t bytes) {
    MCB_CHECK_CTX(ctx);
    if (bytes) MCB_CUDA(ctx, cudaMemsetAsync(dst, byte, bytes, ctx->stream));
    return MCB_OK;
}

mcb_status mcb_sync(mcb_ctx *ctx) {
    MCB_CHECK_CTX(ctx);
    return take_device_error(ctx);
}

void *mcb_stream(mcb_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }
int64_t mcb_launch_count(mcb_ctx *ctx) { return ctx ? ctx->launches : 0; }
int64_t mcb_allocated_bytes(mcb_ctx *ctx) { return ctx ? ctx->allocated_bytes : 0; }

mcb_status mcb_event_create(mcb_ctx *ctx, void **event_out) {
    MCB_CHECK_CTX(ctx);
    cudaEvent_t ev;
    MCB_CUDA(ctx, cudaEventCreate(&ev));
    *event_out = (void *)ev;
    return MCB_OK;
}
mcb_status mcb_event_record(mcb_ctx *ctx, void *event) {
    MCB_CHECK_CTX(ctx);
    MCB_CUDA(ctx, cudaEventRecord((cudaEvent_t)event, ctx->stream));
    return MCB_OK;
}
mcb_status mcb_event_elapsed_ms(mcb_ctx *ctx, void *start, void *stop, float *ms_out) {
    MCB_CHECK_CTX(ctx);
    MCB_CUDA(ctx, cudaEventSynchronize((cudaEvent_t)stop));
    MCB_CUDA(ctx, cudaEventElapsedTime(ms_out, (cudaEvent_t)start, (cudaEvent_t)stop));
    return MCB_OK;
}
mcb_status mcb_event_destroy(mcb_ctx *ctx, void *event) {
    MCB_CHECK_CTX(ctx);
    MCB_CUDA(ctx, cudaEventDestroy((cudaEvent_t)event));
    return MCB_OK;
}

mcb_status mcb_prof_enable(mcb_ctx *ctx, int32_t on) {
    MCB_CHECK_CTX(ctx);
    MCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (auto &r : ctx->prof) {
        ctx->ev_pool.push_back(r.a);
        ctx->ev_pool.push_back(r.b);
    }
    ctx->prof.clear();
    ctx->prof_on = on != 0;
    return MCB_OK;
}

mcb_status mcb_prof_read(mcb_ctx *ctx, int32_t klass, int64_t *launches_out, double *ms_out, double *flops_out,
                         double *bytes_out) {
    MCB_CHECK_CTX(ctx);
    MCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    int64_t n = 0;
    double ms = 0.0, fl = 0.0, by = 0.0;
    for (auto &r : ctx->prof) {
        if (r.klass != klass) continue;
        float t = 0.0f;
        MCB_CUDA(ctx, cudaEventElapsedTime(&t, r.a, r.b));
        ++n;
        ms += t;
        fl += r.flops;
        by += r.bytes;
    }
    if (launches_out) *launches_out = n;
    if (ms_out) *ms_out = ms;
    if (flops_out) *flops_out = fl;
    if (bytes_out) *bytes_out = by;
    return MCB_OK;
}

mcb_status mcb_clock_trace_start(mcb_ctx *ctx, int32_t duration_us, int32_t interval_us) {
    MCB_CHECK_CTX(ctx);
    if (duration_us < 1 || duration_us > 5000000 || interval_us < 1)
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "clock trace: duration 1..5000000 us and interval >= 1 us");
    int cap = duration_us / interval_us + 2;
    if (cap > 1 << 20) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "clock trace: more than 2^20 samples");
    MCB_CUDA(ctx, cudaSetDevice(ctx->device));
    if (!ctx->trace_stream) MCB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->trace_stream, cudaStreamNonBlocking));
    MCB_CUDA(ctx, cudaStreamSynchronize(ctx->trace_stream));
    if (cap > ctx->trace_cap) {
        if (ctx->trace_buf) cudaFree(ctx->trace_buf);
        ctx->trace_buf = nullptr;
        ctx->trace_cap = 0;
        MCB_CUDA(ctx, cudaMalloc(&ctx->trace_buf, (size_t)(1 + 2 * cap) * sizeof(unsigned long long)));
        ctx->trace_cap = cap;
    }
    MCB_CUDA(ctx, cudaMemsetAsync(ctx->trace_buf, 0, sizeof(unsigned long long), ctx->trace_stream));
    clock_trace_kernel<<<1, 1, 0, ctx->trace_stream>>>(ctx->trace_buf, cap, (unsigned long long)duration_us * 1000ull,
                                                      (unsigned long long)interval_us * 1000ull);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_clock_trace_read(mcb_ctx *ctx, double *mhz_out, int32_t max_out, int32_t *n_out) {
    MCB_CHECK_CTX(ctx);
    if (!ctx->trace_stream || !ctx->trace_buf) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "clock trace was not started");
    MCB_CUDA(ctx, cudaStreamSynchronize(ctx->trace_stream));
    std::vector<unsigned long long> h((size_t)1 + 2 * ctx->trace_cap);
    MCB_CUDA(ctx, cudaMemcpy(h.data(), ctx->trace_buf, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    int n = (int)h[0], w = 0;
    for (int i = 1; i < n && w < max_out; ++i) {
        unsigned long long dt = h[1 + 2 * i] - h[1 + 2 * (i - 1)], dc = h[2 + 2 * i] - h[2 + 2 * (i - 1)];
        if (dt == 0) continue;
        if (mhz_out) mhz_out[w] = (double)dc / (double)dt * 1000.0;
        ++w;
    }
    if (n_out) *n_out = w;
    return MCB_OK;
}

mcb_status mcb_set_compute_type(mcb_ctx *ctx, int32_t compute) {
    MCB_CHECK_CTX(ctx);
    if (compute != MCB_COMPUTE_F32 && compute != MCB_COMPUTE_BF16 && compute != MCB_COMPUTE_F16)
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "unknown compute type %d", compute);
    ctx->compute = compute;
    return MCB_OK;
}

} // extern "C"

mcb_status mcb_scratch(mcb_ctx *ctx, size_t bytes, void **out) {
    if (bytes > ctx->scratch_bytes) {
        // the old block may still be read by enqueued kernels: hand it to the pool (stream-ordered reuse)
        size_t want = round_size(bytes < (4u << 20) ? (4u << 20) : bytes);
        void *p = nullptr;
        cudaSetDevice(ctx->device);
        MCB_CUDA(ctx, cudaMalloc(&p, want));
        if (ctx->scratch) {
            std::lock_guard<std::mutex> lk(ctx->mu);
            // a captured step may have recorded the old address: park it instead of recycling it
            if (ctx->static_steps > 0 || ctx->capture_id) ctx->retired_scratch.push_back(ctx->scratch);
            else ctx->free_blocks.emplace(round_size(ctx->scratch_bytes), ctx->scratch);
        }
        ctx->scratch = p;
        ctx->scratch_bytes = want;
        ctx->allocated_bytes += (int64_t)want;
    }
    *out = ctx->scratch;
    return MCB_OK;
}

static cudaEvent_t prof_event(mcb_ctx *ctx) {
    if (!ctx->ev_pool.empty()) {
        cudaEvent_t e = ctx->ev_pool.back();
        ctx->ev_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

ProfScope::ProfScope(mcb_ctx *c, int klass, double flops, double bytes) : ctx(c) {
    if (!c || !c->prof_on) return;
    mcb_ctx::ProfRec r;
    r.klass = klass;
    r.a = prof_event(c);
    r.b = prof_event(c);
    r.flops = flops;
    r.bytes = bytes;
    cudaEventRecord(r.a, c->stream);
    idx = (int)c->prof.size();
    c->prof.push_back(r);
}

ProfScope::~ProfScope() {
    if (idx >= 0) cudaEventRecord(ctx->prof[idx].b, ctx->stream);
}
