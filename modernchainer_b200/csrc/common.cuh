// Shared definitions for the sm_100a training-step library: context, allocator,
// status handling and small device helpers (vector access, reductions).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/mcb.h"

// Device error word bits (surfaced as MCB_INVALID_ARGUMENT by synchronising calls).
#define MCB_DEVERR_LABEL 1u   // class label negative or >= classes
#define MCB_DEVERR_INDEX 2u   // embedding index negative or >= vocab
#define MCB_DEVERR_TIMEOUT 4u // a bounded device-side wait gave up

struct mcb_ctx {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    unsigned int *d_err = nullptr;        // device error word
    std::string last_error;
    std::mutex mu;
    // caching allocator: exact-rounded size -> free blocks
    std::multimap<size_t, void *> free_blocks;
    std::unordered_map<void *, size_t> live;
    int64_t allocated_bytes = 0;
    int64_t launches = 0;
    int compute = MCB_COMPUTE_F32;
    // lazily grown scratch for reductions that need partial sums
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    // data-parallel state (owned by dp.cu)
    void *dp = nullptr;
    // optional per-kernel-class timing (mcb_prof_*): event pairs around launches
    bool prof_on = false;
    struct ProfRec {
        int klass;
        cudaEvent_t a, b;
        double flops, bytes;
    };
    std::vector<ProfRec> prof;
    std::vector<cudaEvent_t> ev_pool;
    // Stream capture of a static training step (static_step.cu).  While capture_id != 0 every block
    // that is allocated or freed becomes the property of that step: the recorded kernels hold its
    // address, so it may be reused inside the same step's captures but never handed to anyone else
    // until the step is released.
    int capture_id = 0;
    int next_capture_id = 1;
    int static_steps = 0; // live static steps: while > 0 an outgrown scratch buffer is parked, not freed
    std::unordered_map<void *, int> graph_owner;
    std::unordered_map<int, std::multimap<size_t, void *>> graph_free;
    std::vector<void *> retired_scratch;
    // SM clock trace (mcb_clock_trace_*): a one-thread sampler kernel on its own stream
    cudaStream_t trace_stream = nullptr;
    unsigned long long *trace_buf = nullptr; // [0] = samples written, then (globaltimer ns, clock64) pairs
    int trace_cap = 0;
    // Programmatic dependent launch: kernels launched through mcb_launch_dep may be scheduled while the
    // previous kernel of the stream drains; they call dep_wait() before touching global memory.
    bool dep_launch = true;
    // counters of the tensor-core GEMM's in-kernel split-tail fix-up (148 tiles x 2 pair halves x 8 warps x 2); zero
    // between launches: the slice that finishes a tile resets them
    unsigned *tc_fix_cnt = nullptr;
    static constexpr size_t kTcFixCntBytes = 148 * 2 * 8 * 2 * sizeof(unsigned);
    // Test and tuning knobs (McbKnob): -1 = not set.  Each is read from the environment once, when the context is created;
    // afterwards only mcb_set_knob changes it, for this context alone.  No entry point reads the environment.
    int knobs[32];
};

enum McbKnob {
    K_UNFUSED_BWD, K_LN_NO_AUX, K_UNFUSED_ADD_LN, K_UNFUSED_QKV, K_CONV_DIRECT, K_FLASH_LEGACY, K_FLASH_LEGACY_BWD, K_SGEMM_NO_SPLIT,
    K_LN_NO_BULK, K_SCE_NO_STREAM, K_TC_EPI, K_TC_EPI_KB, K_TC_STAGES, K_TC_DIRECT_OUT, K_TC_BN, K_TC_PAIR, K_TC_SPLIT_TAIL,
    K_GRAPH_INFO, K_DETERMINISTIC, K_NO_DEP_LAUNCH, K_FLASH_DQ_RECOMPUTE, K_FLASH_BWD_ONE_JOB, K_COUNT
};
static_assert(K_COUNT <= 32, "mcb_ctx::knobs is too small");
inline bool knob_on(const mcb_ctx *ctx, McbKnob k) { return ctx->knobs[k] >= 0; } // flag knobs: set at all
inline int knob_val(const mcb_ctx *ctx, McbKnob k, int unset) { return ctx->knobs[k] >= 0 ? ctx->knobs[k] : unset; }

// RAII timing scope: when profiling is on, brackets the launches made inside it with events
// on the context's stream and books `flops` / `bytes` (algorithmic work) to class `klass`.
struct ProfScope {
    mcb_ctx *ctx;
    int idx = -1;
    ProfScope(mcb_ctx *c, int klass, double flops, double bytes);
    ~ProfScope();
};

mcb_status mcb_fail(mcb_ctx *ctx, mcb_status st, const char *fmt, ...);
mcb_status mcb_cuda_check(mcb_ctx *ctx, cudaError_t e, const char *what);
// scratch buffer of at least `bytes` (stable until a larger request)
mcb_status mcb_scratch(mcb_ctx *ctx, size_t bytes, void **out);

#define MCB_CHECK_CTX(ctx)                                                                                           \
    do {                                                                                                             \
        if (!(ctx)) return MCB_INVALID_ARGUMENT;                                                                     \
    } while (0)
#define MCB_CUDA(ctx, expr)                                                                                          \
    do {                                                                                                             \
        cudaError_t e__ = (expr);                                                                                    \
        if (e__ != cudaSuccess) return mcb_cuda_check(ctx, e__, #expr);                                              \
    } while (0)
#define MCB_TRY(expr)                                                                                                \
    do {                                                                                                             \
        mcb_status s__ = (expr);                                                                                     \
        if (s__ != MCB_OK) return s__;                                                                               \
    } while (0)
// call after every kernel launch
#define MCB_LAUNCHED(ctx)                                                                                            \
    do {                                                                                                             \
        (ctx)->launches++;                                                                                           \
        cudaError_t e__ = cudaGetLastError();                                                                        \
        if (e__ != cudaSuccess) return mcb_cuda_check(ctx, e__, "kernel launch");                                    \
    } while (0)

static inline size_t mcb_dtype_size(int dt) {
    switch (dt) {
    case MCB_F32: return 4;
    case MCB_I64: return 8;
    case MCB_I32: return 4;
    case MCB_U8: return 1;
    case MCB_F16: return 2;
    case MCB_BF16: return 2;
    default: return 0;
    }
}

// the 16-bit storage types a low-precision step can use
static inline bool mcb_is_lp(int dt) { return dt == MCB_BF16 || dt == MCB_F16; }

static inline int mcb_grid_for(mcb_ctx *ctx, int64_t work_items, int per_block, int max_waves = 8) {
    int64_t blocks = (work_items + per_block - 1) / per_block;
    int64_t cap = (int64_t)ctx->sm_count * max_waves;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

#ifdef __CUDACC__
// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched with mcb_launch_dep may become resident while the preceding kernel of the stream is
// still running its last CTAs (that kernel must have passed dep_trigger() in every CTA, or finished).
// Contract for such a kernel: EVERY thread calls dep_wait() before its first access to global memory
// (reads and writes: the predecessor may still be reading what this kernel overwrites); only index
// arithmetic, barrier initialisation and shared/tensor-memory set-up may come before.  dep_wait() returns
// once all preceding kernels have completed and their writes are visible, so the stream stays in order;
// what overlaps is launch latency, the prologue and the tail of the previous grid.  Both calls are no-ops
// in a kernel launched the ordinary way.
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dep_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t mcb_launch_dep(mcb_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = ctx->dep_launch ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------------ device helpers
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// block-wide sum; `red` is shared float[32]; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float *red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float *red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

// storage-type adapters: load/store one element or a group of 4 as f32
template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float ld(const float *p, int64_t i) { return p[i]; }
    static __device__ __forceinline__ void st(float *p, int64_t i, float v) { p[i] = v; }
    static __device__ __forceinline__ float4 ld4(const float *p, int64_t i4) {
        return reinterpret_cast<const float4 *>(p)[i4];
    }
    static __device__ __forceinline__ void st4(float *p, int64_t i4, float4 v) { reinterpret_cast<float4 *>(p)[i4] = v; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(const __nv_bfloat16 *p, int64_t i) { return __bfloat162float(p[i]); }
    static __device__ __forceinline__ void st(__nv_bfloat16 *p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float4 ld4(const __nv_bfloat16 *p, int64_t i4) {
        uint2 raw = reinterpret_cast<const uint2 *>(p)[i4];
        __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&raw.x);
        __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162 *>(&raw.y);
        float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
        return make_float4(fa.x, fa.y, fb.x, fb.y);
    }
    static __device__ __forceinline__ void st4(__nv_bfloat16 *p, int64_t i4, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned int *>(&a);
        raw.y = *reinterpret_cast<unsigned int *>(&b);
        reinterpret_cast<uint2 *>(p)[i4] = raw;
    }
};

template <> struct Elem<__half> {
    static __device__ __forceinline__ float ld(const __half *p, int64_t i) { return __half2float(p[i]); }
    static __device__ __forceinline__ void st(__half *p, int64_t i, float v) { p[i] = __float2half_rn(v); }
    static __device__ __forceinline__ float4 ld4(const __half *p, int64_t i4) {
        uint2 raw = reinterpret_cast<const uint2 *>(p)[i4];
        float2 fa = __half22float2(*reinterpret_cast<__half2 *>(&raw.x)), fb = __half22float2(*reinterpret_cast<__half2 *>(&raw.y));
        return make_float4(fa.x, fa.y, fb.x, fb.y);
    }
    static __device__ __forceinline__ void st4(__half *p, int64_t i4, float4 v) {
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned int *>(&a);
        raw.y = *reinterpret_cast<unsigned int *>(&b);
        reinterpret_cast<uint2 *>(p)[i4] = raw;
    }
};

// The two 16-bit storage types (bf16, f16) as pairs packed in one 32-bit word, both rounded to
// nearest even from f32: what the kernels that are written once for both formats use.
template <typename T> struct Lp;
template <> struct Lp<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t pack2(float a, float b) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    static __device__ __forceinline__ float2 unpack2(uint32_t w) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&w)); }
};
template <> struct Lp<__half> {
    static __device__ __forceinline__ uint32_t pack2(float a, float b) {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    static __device__ __forceinline__ float2 unpack2(uint32_t w) { return __half22float2(*reinterpret_cast<__half2 *>(&w)); }
};

static inline bool mcb_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// integer label / index fetch for I64, I32, U8 storage
__device__ __forceinline__ long long load_index(const void *p, int dt, int64_t i) {
    if (dt == MCB_I64) return reinterpret_cast<const long long *>(p)[i];
    if (dt == MCB_I32) return (long long)reinterpret_cast<const int *>(p)[i];
    return (long long)reinterpret_cast<const unsigned char *>(p)[i];
}
#endif
