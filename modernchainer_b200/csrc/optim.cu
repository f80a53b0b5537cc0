// Optimizer kernels: Adam (reference-shaped out-of-place form and the fused in-place
// flat-arena form with unscale, skip flag and bf16 shadow write) and the inf/nan scan.
// Pure HBM streaming: 128-bit accesses, grid = multiple of the SM count.
#include "common.cuh"
#include "internal.h"

namespace {

constexpr int kThreads = 256;

struct AdamK {
    float b1, b2, omb1, omb2, bc1, bc2, lr, eps, inv_scale;
    // the rest of the optimizer family on the same flat pass (optim/src/lib.rs:23-51, 122-233)
    float wd = 0.0f;   // AdamW: (f32)(weight_decay * lr), applied to the parameter value before the step
    float nlr = 0.0f;  // SGD forms: (f32)(-lr)
    float mom = 0.0f;  // MomentumSGD: (f32)momentum
    int first = 0;     // MomentumSGD: no velocity yet, so velocity = gradient
    int shadow_f16 = 0; // the 16-bit copy of the parameters is f16 (else bf16)
};

// Rust f32::powi: repeated squaring in f32 (the reference computes 1 - beta^t this way,
// crates/modern-chainer-cpu/src/kernels.rs:667-668)
float powi_f32(float base, int32_t e) {
    uint32_t n = (uint32_t)e;
    float r = 1.0f, b = base;
    for (;;) {
        if (n & 1u) r *= b;
        n >>= 1;
        if (!n) break;
        b *= b;
    }
    return r;
}

AdamK make_k(double lr, double beta1, double beta2, double eps, int32_t step, double inv_scale) {
    AdamK k;
    k.b1 = (float)beta1;
    k.b2 = (float)beta2;
    k.omb1 = 1.0f - k.b1;
    k.omb2 = 1.0f - k.b2;
    k.bc1 = 1.0f - powi_f32(k.b1, step);
    k.bc2 = 1.0f - powi_f32(k.b2, step);
    k.lr = (float)lr;
    k.eps = (float)eps;
    k.inv_scale = (float)inv_scale;
    return k;
}

// same operation order as the reference: nm = b1*m + (1-b1)*g; nv = b2*v + ((1-b2)*g)*g;
// p - lr*(nm/bc1)/(sqrt(nv/bc2)+eps).  No FMA contraction so f32 results match the CPU.
__device__ __forceinline__ void adam_one(const AdamK &k, float g, float &p, float &m, float &v) {
    float nm = __fadd_rn(__fmul_rn(k.b1, m), __fmul_rn(k.omb1, g));
    float nv = __fadd_rn(__fmul_rn(k.b2, v), __fmul_rn(__fmul_rn(k.omb2, g), g));
    float m_hat = __fdiv_rn(nm, k.bc1);
    float v_hat = __fdiv_rn(nv, k.bc2);
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(k.lr, m_hat), __fadd_rn(__fsqrt_rn(v_hat), k.eps)));
    m = nm;
    v = nv;
}

__global__ void adam_update_kernel(const float *__restrict__ p, const float *__restrict__ g,
                                   const float *__restrict__ m, const float *__restrict__ v, float *__restrict__ np,
                                   float *__restrict__ nm, float *__restrict__ nv, long long n, AdamK k) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float pp = p[i], mm = m[i], vv = v[i];
        adam_one(k, g[i], pp, mm, vv);
        np[i] = pp;
        nm[i] = mm;
        nv[i] = vv;
    }
}

// 16-bit copy of the updated parameters for the low-precision GEMMs: bf16, or f16 when the step runs under f16 autocast
__device__ __forceinline__ void store_shadow4(__nv_bfloat16 *shadow, long long j, float4 v, int f16) {
    if (f16) Elem<__half>::st4(reinterpret_cast<__half *>(shadow), j, v);
    else Elem<__nv_bfloat16>::st4(shadow, j, v);
}
__device__ __forceinline__ void store_shadow(__nv_bfloat16 *shadow, long long j, float v, int f16) {
    if (f16) reinterpret_cast<__half *>(shadow)[j] = __float2half_rn(v);
    else shadow[j] = __float2bfloat16_rn(v);
}

// One element of the other update rules, in the reference's operation order and without FMA:
//   AdamW        : next = adam(p, ...); p' = next - p * (f32)(wd * lr)          (lib.rs:196-211)
//   SGD          : p' = p + g * (f32)(-lr)                                      (lib.rs:38-41)
//   MomentumSGD  : vel' = vel * (f32)mom + g (vel' = g on the first step); p' = p + vel' * (f32)(-lr)  (lib.rs:141-150)
template <int KIND> __device__ __forceinline__ void opt_one(const AdamK &k, float g, float &p, float &m, float &v) {
    if (KIND == MCB_OPT_ADAM) {
        adam_one(k, g, p, m, v);
    } else if (KIND == MCB_OPT_ADAMW) {
        float decay = __fmul_rn(p, k.wd);
        adam_one(k, g, p, m, v);
        p = __fsub_rn(p, decay);
    } else if (KIND == MCB_OPT_SGD) {
        p = __fadd_rn(p, __fmul_rn(g, k.nlr));
    } else {
        float vel = k.first ? g : __fadd_rn(__fmul_rn(m, k.mom), g);
        m = vel;
        p = __fadd_rn(p, __fmul_rn(vel, k.nlr));
    }
}

// SGD touches only p and g, MomentumSGD p, g and the velocity (kept where Adam keeps m)
template <typename GT, int KIND>
__global__ void __launch_bounds__(kThreads)
sgd_flat_kernel(float *__restrict__ p, const GT *__restrict__ g, float *__restrict__ m, __nv_bfloat16 *__restrict__ shadow, long long n,
                AdamK k, const float *__restrict__ inv_scale_dev, const int *__restrict__ skip, const int *__restrict__ step_dev, int vec) {
    if (skip && *skip) return;
    if (inv_scale_dev) k.inv_scale *= inv_scale_dev[0];
    if (step_dev) k.first = step_dev[0] == 0; // device-resident count of applied steps (replayed graphs)
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    long long n4 = vec ? (n >> 2) : 0;
    float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long j = i; j < n4; j += stride) {
        float4 pp = reinterpret_cast<float4 *>(p)[j], gg = Elem<GT>::ld4(g, j);
        float4 mm = KIND == MCB_OPT_MOMENTUM_SGD ? reinterpret_cast<float4 *>(m)[j] : zero, vv = zero;
        opt_one<KIND>(k, gg.x * k.inv_scale, pp.x, mm.x, vv.x);
        opt_one<KIND>(k, gg.y * k.inv_scale, pp.y, mm.y, vv.y);
        opt_one<KIND>(k, gg.z * k.inv_scale, pp.z, mm.z, vv.z);
        opt_one<KIND>(k, gg.w * k.inv_scale, pp.w, mm.w, vv.w);
        reinterpret_cast<float4 *>(p)[j] = pp;
        if (KIND == MCB_OPT_MOMENTUM_SGD) reinterpret_cast<float4 *>(m)[j] = mm;
        if (shadow) store_shadow4(shadow, j, pp, k.shadow_f16);
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride) {
        float pp = p[j], mm = KIND == MCB_OPT_MOMENTUM_SGD ? m[j] : 0.0f, vv = 0.0f;
        opt_one<KIND>(k, Elem<GT>::ld(g, j) * k.inv_scale, pp, mm, vv);
        p[j] = pp;
        if (KIND == MCB_OPT_MOMENTUM_SGD) m[j] = mm;
        if (shadow) store_shadow(shadow, j, pp, k.shadow_f16);
    }
}

template <typename GT, int KIND = MCB_OPT_ADAM>
__global__ void __launch_bounds__(kThreads)
adam_flat_kernel(float *__restrict__ p, const GT *__restrict__ g, float *__restrict__ m, float *__restrict__ v,
                 __nv_bfloat16 *__restrict__ shadow, long long n, AdamK k, const float *__restrict__ inv_scale_dev,
                 const int *__restrict__ skip, const int *__restrict__ step_dev, int vec) {
    if (skip && *skip) return;
    if (inv_scale_dev) k.inv_scale *= inv_scale_dev[0];
    if (step_dev) { // bias correction from the device-resident count of applied steps
        unsigned t = (unsigned)(step_dev[0] + 1);
        float r1 = 1.0f, r2 = 1.0f, b1 = k.b1, b2 = k.b2;
        for (;;) {
            if (t & 1u) {
                r1 = __fmul_rn(r1, b1);
                r2 = __fmul_rn(r2, b2);
            }
            t >>= 1;
            if (!t) break;
            b1 = __fmul_rn(b1, b1);
            b2 = __fmul_rn(b2, b2);
        }
        k.bc1 = 1.0f - r1;
        k.bc2 = 1.0f - r2;
    }
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    long long n4 = vec ? (n >> 2) : 0;
    for (long long j = i; j < n4; j += stride) {
        float4 pp = reinterpret_cast<float4 *>(p)[j], mm = reinterpret_cast<float4 *>(m)[j];
        float4 vv = reinterpret_cast<float4 *>(v)[j], gg = Elem<GT>::ld4(g, j);
        opt_one<KIND>(k, gg.x * k.inv_scale, pp.x, mm.x, vv.x);
        opt_one<KIND>(k, gg.y * k.inv_scale, pp.y, mm.y, vv.y);
        opt_one<KIND>(k, gg.z * k.inv_scale, pp.z, mm.z, vv.z);
        opt_one<KIND>(k, gg.w * k.inv_scale, pp.w, mm.w, vv.w);
        reinterpret_cast<float4 *>(p)[j] = pp;
        reinterpret_cast<float4 *>(m)[j] = mm;
        reinterpret_cast<float4 *>(v)[j] = vv;
        if (shadow) store_shadow4(shadow, j, pp, k.shadow_f16);
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride) {
        float pp = p[j], mm = m[j], vv = v[j];
        opt_one<KIND>(k, Elem<GT>::ld(g, j) * k.inv_scale, pp, mm, vv);
        p[j] = pp;
        m[j] = mm;
        v[j] = vv;
        if (shadow) store_shadow(shadow, j, pp, k.shadow_f16);
    }
}

// inf/nan scan: exponent all ones.  f32: (bits & 0x7F800000) == 0x7F800000; bf16 likewise on 16 bits.
__global__ void check_finite_f32_kernel(const float *__restrict__ g, long long n, int *__restrict__ flag, int vec) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    unsigned bad = 0;
    long long n4 = vec ? (n >> 2) : 0;
    for (long long j = i; j < n4; j += stride) {
        uint4 b = reinterpret_cast<const uint4 *>(g)[j];
        bad |= ((b.x & 0x7F800000u) == 0x7F800000u) | ((b.y & 0x7F800000u) == 0x7F800000u) |
               ((b.z & 0x7F800000u) == 0x7F800000u) | ((b.w & 0x7F800000u) == 0x7F800000u);
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride)
        bad |= ((__float_as_uint(g[j]) & 0x7F800000u) == 0x7F800000u);
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicExch(flag, 1);
}
// 16-bit gradients: `em` is the exponent mask of the format (bf16 0x7F80, f16 0x7C00)
__global__ void check_finite_bf16_kernel(const unsigned short *__restrict__ g, long long n, int *__restrict__ flag, int vec, unsigned em) {
    const unsigned emh = em << 16;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    unsigned bad = 0;
    long long n8 = vec ? (n >> 3) : 0;
    for (long long j = i; j < n8; j += stride) {
        uint4 b = reinterpret_cast<const uint4 *>(g)[j];
        unsigned w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int q = 0; q < 4; ++q)
            bad |= ((w[q] & em) == em) | ((w[q] & emh) == emh);
    }
    for (long long j = (n8 << 3) + i; j < n; j += stride) bad |= ((g[j] & em) == em);
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicExch(flag, 1);
}

} // namespace

extern "C" {

mcb_status mcb_adam_update(mcb_ctx *ctx, const float *p, const float *g, const float *m, const float *v,
                           float *new_p, float *new_m, float *new_v, int64_t n, double lr, double beta1,
                           double beta2, double eps, int32_t step) {
    MCB_CHECK_CTX(ctx);
    if (step < 1) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "adam step must be >= 1");
    if (n == 0) return MCB_OK;
    AdamK k = make_k(lr, beta1, beta2, eps, step, 1.0);
    adam_update_kernel<<<mcb_grid_for(ctx, n, kThreads), kThreads, 0, ctx->stream>>>(p, g, m, v, new_p, new_m, new_v, n, k);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_adam_flat(mcb_ctx *ctx, float *p, const void *g, int32_t g_dt, float *m, float *v, void *p_bf16,
                         int64_t n, double lr, double beta1, double beta2, double eps, int32_t step,
                         double inv_scale, const int32_t *skip_flag) {
    MCB_CHECK_CTX(ctx);
    return mcb_adam_flat_ex(ctx, p, g, g_dt, m, v, p_bf16, n, lr, beta1, beta2, eps, step, inv_scale, nullptr, skip_flag, nullptr);
}

mcb_status mcb_check_finite(mcb_ctx *ctx, const void *g, int32_t g_dt, int64_t n, int32_t *flag) {
    MCB_CHECK_CTX(ctx);
    if (n == 0) return MCB_OK;
    int vec = mcb_aligned16(g);
    ProfScope prof(ctx, MCB_PROF_OPTIMIZER, 0.0, (double)n * (mcb_is_lp(g_dt) ? 2.0 : 4.0));
    if (g_dt == MCB_F32)
        check_finite_f32_kernel<<<mcb_grid_for(ctx, (n + 3) / 4, kThreads, 8), kThreads, 0, ctx->stream>>>((const float *)g, n, flag, vec);
    else if (mcb_is_lp(g_dt))
        check_finite_bf16_kernel<<<mcb_grid_for(ctx, (n + 7) / 8, kThreads, 8), kThreads, 0, ctx->stream>>>((const unsigned short *)g, n, flag, vec,
                                                                                                          g_dt == MCB_BF16 ? 0x7F80u : 0x7C00u);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "check_finite supports f32, bf16 and f16");
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

} // extern "C"

mcb_status mcb_adam_flat_ex(mcb_ctx *ctx, float *p, const void *g, int32_t g_dt, float *m, float *v, void *p_bf16,
                            int64_t n, double lr, double beta1, double beta2, double eps, int32_t step,
                            double inv_scale, const float *inv_scale_dev, const int32_t *skip_flag, const int32_t *step_dev) {
    return mcb_opt_flat(ctx, MCB_OPT_ADAM, p, g, g_dt, m, v, p_bf16, n, lr, beta1, beta2, eps, 0.0, step, inv_scale, inv_scale_dev, skip_flag,
                        step_dev);
}

namespace {
template <typename GT>
void launch_opt(mcb_ctx *ctx, int kind, int grid, float *p, const GT *g, float *m, float *v, __nv_bfloat16 *sh, long long n, const AdamK &k,
                const float *inv_scale_dev, const int32_t *skip, const int32_t *step_dev, int vec) {
    cudaStream_t s = ctx->stream;
    if (kind == MCB_OPT_ADAM) adam_flat_kernel<GT, MCB_OPT_ADAM><<<grid, kThreads, 0, s>>>(p, g, m, v, sh, n, k, inv_scale_dev, skip, step_dev, vec);
    else if (kind == MCB_OPT_ADAMW) adam_flat_kernel<GT, MCB_OPT_ADAMW><<<grid, kThreads, 0, s>>>(p, g, m, v, sh, n, k, inv_scale_dev, skip, step_dev, vec);
    else if (kind == MCB_OPT_SGD) sgd_flat_kernel<GT, MCB_OPT_SGD><<<grid, kThreads, 0, s>>>(p, g, m, sh, n, k, inv_scale_dev, skip, step_dev, vec);
    else sgd_flat_kernel<GT, MCB_OPT_MOMENTUM_SGD><<<grid, kThreads, 0, s>>>(p, g, m, sh, n, k, inv_scale_dev, skip, step_dev, vec);
}
__global__ void increment_i32_kernel(int *p) {
    if (threadIdx.x == 0 && blockIdx.x == 0) p[0] += 1;
}
} // namespace

mcb_status mcb_increment_i32(mcb_ctx *ctx, int32_t *counter) {
    increment_i32_kernel<<<1, 32, 0, ctx->stream>>>(counter);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

// One fused in-place pass of any optimizer of the family over a flat range.  For the SGD forms
// `beta1` carries the momentum, `v` is unused and `m` holds the velocity; `step` is the 1-based
// count of this update (bias correction for Adam/AdamW, "no velocity yet" when 1 for MomentumSGD).
mcb_status mcb_opt_flat(mcb_ctx *ctx, int32_t kind, float *p, const void *g, int32_t g_dt, float *m, float *v, void *p_bf16, int64_t n,
                        double lr, double beta1, double beta2, double eps, double weight_decay, int32_t step, double inv_scale,
                        const float *inv_scale_dev, const int32_t *skip_flag, const int32_t *step_dev, int32_t shadow_dt) {
    if (kind < MCB_OPT_ADAM || kind > MCB_OPT_MOMENTUM_SGD) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "unknown optimizer kind %d", kind);
    if (step < 1) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "optimizer step must be >= 1");
    if (n == 0) return MCB_OK;
    const bool adam = kind == MCB_OPT_ADAM || kind == MCB_OPT_ADAMW;
    AdamK k = make_k(lr, adam ? beta1 : 0.9, adam ? beta2 : 0.999, eps, step, inv_scale);
    k.wd = (float)(weight_decay * lr);
    k.nlr = (float)(-lr);
    k.mom = (float)beta1;
    k.first = step == 1;
    k.shadow_f16 = shadow_dt == MCB_F16;
    int vec = mcb_aligned16(p) && mcb_aligned16(g) && (!m || mcb_aligned16(m)) && (!v || mcb_aligned16(v)) && (!p_bf16 || mcb_aligned16(p_bf16));
    int grid = mcb_grid_for(ctx, (n + 3) / 4, kThreads, 8);
    // algorithmic bytes per parameter: read and write p plus the state the rule keeps, read g (+ the bf16 shadow)
    double state_bytes = adam ? 16.0 : (kind == MCB_OPT_MOMENTUM_SGD ? 8.0 : 0.0);
    ProfScope prof(ctx, MCB_PROF_OPTIMIZER, 0.0, (double)n * (8.0 + state_bytes + (mcb_is_lp(g_dt) ? 2.0 : 4.0) + (p_bf16 ? 2.0 : 0.0)));
    if (g_dt == MCB_F32) launch_opt<float>(ctx, kind, grid, p, (const float *)g, m, v, (__nv_bfloat16 *)p_bf16, n, k, inv_scale_dev, skip_flag, step_dev, vec);
    else if (g_dt == MCB_BF16)
        launch_opt<__nv_bfloat16>(ctx, kind, grid, p, (const __nv_bfloat16 *)g, m, v, (__nv_bfloat16 *)p_bf16, n, k, inv_scale_dev, skip_flag, step_dev, vec);
    else if (g_dt == MCB_F16)
        launch_opt<__half>(ctx, kind, grid, p, (const __half *)g, m, v, (__nv_bfloat16 *)p_bf16, n, k, inv_scale_dev, skip_flag, step_dev, vec);
    else return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "optimizer grads must be f32, bf16 or f16");
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

// ------------------------------------------------------------------ clip_grad_norm (optim/src/lib.rs:216-243)
namespace {
// per-block sum of g^2: the square in f32 (as ops.mul does), the sum in f64
__global__ void sumsq_partial_kernel(const float *__restrict__ g, long long n, double *__restrict__ partial) {
    __shared__ double red[kThreads / 32];
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    double acc = 0.0;
    for (; i < n; i += stride) {
        float x = g[i];
        acc += (double)__fmul_rn(x, x);
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < kThreads / 32; ++w) t += red[w];
        partial[blockIdx.x] = t;
    }
}
// out[0] = norm, out[1] = factor (max_norm / norm when the norm exceeds max_norm and is positive, else 1).
// `mean_factor` turns the norm of a gradient that is still a SUM over data-parallel ranks into the norm of the
// mean the optimizer will use (1 / world; 1 on a single rank): the limit applies to the mean, and the factor
// max_norm / norm scales the sum and the mean alike.
__global__ void clip_final_kernel(const double *__restrict__ partial, int count, double max_norm, double mean_factor, double *__restrict__ out) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    double t = 0.0;
    for (int i = 0; i < count; ++i) t += partial[i];
    double norm = sqrt(t) * mean_factor;
    out[0] = norm;
    out[1] = (norm > max_norm && norm > 0.0) ? max_norm / norm : 1.0;
}
__global__ void scale_by_clip_kernel(float *__restrict__ g, long long n, const double *__restrict__ clip) {
    double f = clip[1];
    if (f == 1.0) return; // within the limit: gradients stay untouched (no pass over memory)
    float ff = (float)f;  // Ops::scale narrows the factor to f32 first
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) g[i] = __fmul_rn(g[i], ff);
}
} // namespace

int mcb_sumsq_blocks(mcb_ctx *ctx, int64_t n) { return mcb_grid_for(ctx, n > 0 ? n : 1, kThreads, 4); }
mcb_status mcb_sumsq_partial(mcb_ctx *ctx, const float *g, int64_t n, double *partial, int blocks) {
    ProfScope prof(ctx, MCB_PROF_OPTIMIZER, 0.0, 4.0 * (double)n);
    sumsq_partial_kernel<<<blocks, kThreads, 0, ctx->stream>>>(g, n, partial);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}
mcb_status mcb_clip_finalize(mcb_ctx *ctx, const double *partial, int count, double max_norm, double *out2, double mean_factor) {
    clip_final_kernel<<<1, 32, 0, ctx->stream>>>(partial, count, max_norm, mean_factor, out2);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}
mcb_status mcb_scale_by_clip(mcb_ctx *ctx, float *g, int64_t n, const double *clip2) {
    if (n == 0) return MCB_OK;
    ProfScope prof(ctx, MCB_PROF_OPTIMIZER, 0.0, 8.0 * (double)n);
    scale_by_clip_kernel<<<mcb_grid_for(ctx, n, kThreads, 8), kThreads, 0, ctx->stream>>>(g, n, clip2);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

namespace {
// GradScaler::step bookkeeping (crates/modern-chainer-optim/src/amp.rs:66-86) on the device
__global__ void scaler_update_kernel(float *sf, int *si, float growth, float backoff, int interval) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int found = si[1];
    si[2] = found;
    if (!found) si[3] += 1; // applied steps
    if (found) {
        sf[0] = fmaxf(sf[0] * backoff, 1.0f);
        si[0] = 0;
    } else {
        si[0] += 1;
        if (si[0] >= interval) {
            sf[0] *= growth;
            si[0] = 0;
        }
    }
    sf[1] = 1.0f / sf[0];
    si[1] = 0;
}
} // namespace

mcb_status mcb_scaler_update(mcb_ctx *ctx, float *state_f, int *state_i, float growth, float backoff, int interval) {
    scaler_update_kernel<<<1, 32, 0, ctx->stream>>>(state_f, state_i, growth, backoff, interval);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}
