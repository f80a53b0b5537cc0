// Optimizer kernels: Adam (reference-shaped out-of-place form and the fused in-place
// flat-arena form with unscale, skip flag and bf16 shadow write) and the inf/nan scan.
// Pure HBM streaming: 128-bit accesses, grid = multiple of the SM count.
#include "common.cuh"
#include "internal.h"

namespace {

constexpr int kThreads = 256;

struct AdamK {
    float b1, b2, omb1, omb2, bc1, bc2, lr, eps, inv_scale;
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

template <typename GT>
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
        adam_one(k, gg.x * k.inv_scale, pp.x, mm.x, vv.x);
        adam_one(k, gg.y * k.inv_scale, pp.y, mm.y, vv.y);
        adam_one(k, gg.z * k.inv_scale, pp.z, mm.z, vv.z);
        adam_one(k, gg.w * k.inv_scale, pp.w, mm.w, vv.w);
        reinterpret_cast<float4 *>(p)[j] = pp;
        reinterpret_cast<float4 *>(m)[j] = mm;
        reinterpret_cast<float4 *>(v)[j] = vv;
        if (shadow) Elem<__nv_bfloat16>::st4(shadow, j, pp);
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride) {
        float pp = p[j], mm = m[j], vv = v[j];
        adam_one(k, Elem<GT>::ld(g, j) * k.inv_scale, pp, mm, vv);
        p[j] = pp;
        m[j] = mm;
        v[j] = vv;
        if (shadow) shadow[j] = __float2bfloat16_rn(pp);
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
__global__ void check_finite_bf16_kernel(const unsigned short *__restrict__ g, long long n, int *__restrict__ flag, int vec) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    unsigned bad = 0;
    long long n8 = vec ? (n >> 3) : 0;
    for (long long j = i; j < n8; j += stride) {
        uint4 b = reinterpret_cast<const uint4 *>(g)[j];
        unsigned w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int q = 0; q < 4; ++q)
            bad |= ((w[q] & 0x7F80u) == 0x7F80u) | ((w[q] & 0x7F800000u) == 0x7F800000u);
    }
    for (long long j = (n8 << 3) + i; j < n; j += stride) bad |= ((g[j] & 0x7F80u) == 0x7F80u);
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
    ProfScope prof(ctx, MCB_PROF_OPTIMIZER, 0.0, (double)n * (g_dt == MCB_BF16 ? 2.0 : 4.0));
    if (g_dt == MCB_F32)
        check_finite_f32_kernel<<<mcb_grid_for(ctx, (n + 3) / 4, kThreads, 8), kThreads, 0, ctx->stream>>>((const float *)g, n, flag, vec);
    else if (g_dt == MCB_BF16)
        check_finite_bf16_kernel<<<mcb_grid_for(ctx, (n + 7) / 8, kThreads, 8), kThreads, 0, ctx->stream>>>((const unsigned short *)g, n, flag, vec);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "check_finite supports f32 and bf16");
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

} // extern "C"

mcb_status mcb_adam_flat_ex(mcb_ctx *ctx, float *p, const void *g, int32_t g_dt, float *m, float *v, void *p_bf16,
                            int64_t n, double lr, double beta1, double beta2, double eps, int32_t step,
                            double inv_scale, const float *inv_scale_dev, const int32_t *skip_flag, const int32_t *step_dev) {
    if (step < 1) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "adam step must be >= 1");
    if (n == 0) return MCB_OK;
    AdamK k = make_k(lr, beta1, beta2, eps, step, inv_scale);
    int vec = mcb_aligned16(p) && mcb_aligned16(g) && mcb_aligned16(m) && mcb_aligned16(v) && (!p_bf16 || mcb_aligned16(p_bf16));
    int grid = mcb_grid_for(ctx, (n + 3) / 4, kThreads, 8);
    // algorithmic bytes per parameter: read p, m, v, g; write p, m, v (+ the bf16 shadow)
    ProfScope prof(ctx, MCB_PROF_OPTIMIZER, 0.0, (double)n * (24.0 + (g_dt == MCB_BF16 ? 2.0 : 4.0) + (p_bf16 ? 2.0 : 0.0)));
    if (g_dt == MCB_F32)
        adam_flat_kernel<float><<<grid, kThreads, 0, ctx->stream>>>(p, (const float *)g, m, v, (__nv_bfloat16 *)p_bf16, n, k, inv_scale_dev, skip_flag, step_dev, vec);
    else if (g_dt == MCB_BF16)
        adam_flat_kernel<__nv_bfloat16><<<grid, kThreads, 0, ctx->stream>>>(p, (const __nv_bfloat16 *)g, m, v, (__nv_bfloat16 *)p_bf16, n, k, inv_scale_dev, skip_flag, step_dev, vec);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "adam grads must be f32 or bf16");
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
