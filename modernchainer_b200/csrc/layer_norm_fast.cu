// LayerNorm forward / backward for rows of up to 1024 elements (dim % 4 == 0): one warp per
// row with the whole row held in registers, so x (and g) are read from HBM exactly once and
// the row statistics cost only warp shuffles.  The dgamma / dbeta column sums are carried in
// per-lane registers across the rows a warp sweeps, folded through shared memory once per
// block in a fixed warp order, and finished by a second kernel over the per-block partials
// (deterministic, no float atomics).  Wider or unaligned rows use the generic kernels in reduce.cu.
#include "common.cuh"
#include "internal.h"

namespace {

constexpr int kWarps = 8;

template <typename T> __device__ __forceinline__ float4 ld4_or_zero(const T *p, int idx, int dim4) {
    return idx < dim4 ? Elem<T>::ld4(p, idx) : make_float4(0.f, 0.f, 0.f, 0.f);
}

template <typename OutT, int NV>
__global__ void __launch_bounds__(kWarps * 32) ln_fwd_reg_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                                                                  const float *__restrict__ beta, float eps, OutT *__restrict__ out,
                                                                  float *__restrict__ mean_out, float *__restrict__ rstd_out,
                                                                  long long rows, int dim) {
    int lane = threadIdx.x & 31;
    long long warp = (long long)blockIdx.x * kWarps + (threadIdx.x >> 5);
    long long nwarps = (long long)gridDim.x * kWarps;
    int dim4 = dim >> 2;
    float inv_dim = 1.0f / (float)dim;
    float4 ga[NV], be[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        ga[j] = ld4_or_zero(gamma, lane + 32 * j, dim4);
        be[j] = ld4_or_zero(beta, lane + 32 * j, dim4);
    }
    // the next row of this warp is fetched while the current one is reduced and written, so two
    // rows' loads are in flight per warp (one block per SM is resident: latency, not bandwidth, binds)
    float4 v[NV];
    if (warp < rows) {
#pragma unroll
        for (int j = 0; j < NV; ++j) v[j] = ld4_or_zero(x + warp * dim, lane + 32 * j, dim4);
    }
    for (long long r = warp; r < rows; r += nwarps) {
        float4 nx[NV];
        const long long rn = r + nwarps;
        if (rn < rows) {
#pragma unroll
            for (int j = 0; j < NV; ++j) nx[j] = ld4_or_zero(x + rn * dim, lane + 32 * j, dim4);
        }
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        float mean = warp_sum(sum) * inv_dim;
        float var = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j)
            if (lane + 32 * j < dim4) {
                float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                var += (a * a + b * b) + (c * c + d * d);
            }
        var = warp_sum(var) * inv_dim;
        float rstd = 1.0f / sqrtf(var + eps);
        if (lane == 0) {
            if (mean_out) mean_out[r] = mean;
            if (rstd_out) rstd_out[r] = rstd;
        }
        OutT *d = out + r * dim;
#pragma unroll
        for (int j = 0; j < NV; ++j)
            if (lane + 32 * j < dim4)
                Elem<OutT>::st4(d, lane + 32 * j,
                                make_float4((v[j].x - mean) * rstd * ga[j].x + be[j].x, (v[j].y - mean) * rstd * ga[j].y + be[j].y,
                                            (v[j].z - mean) * rstd * ga[j].z + be[j].z, (v[j].w - mean) * rstd * ga[j].w + be[j].w));
        if (rn < rows) {
#pragma unroll
            for (int j = 0; j < NV; ++j) v[j] = nx[j];
        }
    }
}

// upstream gradient as loaded (bf16 stays packed while it waits in the prefetch registers)
template <typename T> struct RawG;
template <> struct RawG<float> {
    typedef float4 type;
    static __device__ __forceinline__ type load(const float *p, int idx, int dim4) { return ld4_or_zero(p, idx, dim4); }
    static __device__ __forceinline__ float4 unpack(type r) { return r; }
};
template <> struct RawG<__nv_bfloat16> {
    typedef uint2 type;
    static __device__ __forceinline__ type load(const __nv_bfloat16 *p, int idx, int dim4) {
        return idx < dim4 ? reinterpret_cast<const uint2 *>(p)[idx] : make_uint2(0u, 0u);
    }
    static __device__ __forceinline__ float4 unpack(type r) {
        float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&r.x));
        float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&r.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
};

// `addend` (optional, may alias dx): a gradient already pending for the same input; dx is written as
// addend + dx, which saves the separate fan-in add over the residual stream.
template <typename GT, int NV>
__global__ void __launch_bounds__(kWarps * 32) ln_bwd_reg_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                                                                  const GT *__restrict__ g, float eps, const float *__restrict__ mean_in,
                                                                  const float *__restrict__ rstd_in, const float *addend, float *dx,
                                                                  float *__restrict__ partial, long long rows, int dim) {
    __shared__ float acc[2 * 32 * NV * 4];
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    long long warp = (long long)blockIdx.x * kWarps + w;
    long long nwarps = (long long)gridDim.x * kWarps;
    int dim4 = dim >> 2;
    float fdim = (float)dim, inv_dim = 1.0f / fdim;
    float4 ga[NV], dga[NV], dbe[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        ga[j] = ld4_or_zero(gamma, lane + 32 * j, dim4);
        dga[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        dbe[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // rows are software-pipelined: the next row's x and g are requested before the current row is
    // reduced, so each warp keeps two rows of loads in flight (one block per SM fits: latency binds)
    float4 v[NV];
    typename RawG<GT>::type graw[NV];
    if (warp < rows) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            v[j] = ld4_or_zero(x + warp * dim, lane + 32 * j, dim4);
            graw[j] = RawG<GT>::load(g + warp * dim, lane + 32 * j, dim4);
        }
    }
    for (long long r = warp; r < rows; r += nwarps) {
        float4 nx[NV], gv[NV], ad[NV];
        typename RawG<GT>::type ng[NV];
        const long long rn = r + nwarps;
        if (rn < rows) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                nx[j] = ld4_or_zero(x + rn * dim, lane + 32 * j, dim4);
                ng[j] = RawG<GT>::load(g + rn * dim, lane + 32 * j, dim4);
            }
        }
        if (addend) {
#pragma unroll
            for (int j = 0; j < NV; ++j) ad[j] = ld4_or_zero(addend + r * dim, lane + 32 * j, dim4);
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) gv[j] = RawG<GT>::unpack(graw[j]);
        float mean, rstd;
        if (mean_in && rstd_in) {
            mean = mean_in[r];
            rstd = rstd_in[r];
        } else {
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < NV; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
            mean = warp_sum(sum) * inv_dim;
            float var = 0.0f;
#pragma unroll
            for (int j = 0; j < NV; ++j)
                if (lane + 32 * j < dim4) {
                    float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                    var += (a * a + b * b) + (c * c + d * d);
                }
            rstd = 1.0f / sqrtf(warp_sum(var) * inv_dim + eps);
        }
        float sum_dy = 0.0f, sum_dy_norm = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            // v becomes the normalised value; lanes past the row end hold zeros in gv, so they add nothing
            v[j].x = (v[j].x - mean) * rstd;
            v[j].y = (v[j].y - mean) * rstd;
            v[j].z = (v[j].z - mean) * rstd;
            v[j].w = (v[j].w - mean) * rstd;
            float4 dy = make_float4(gv[j].x * ga[j].x, gv[j].y * ga[j].y, gv[j].z * ga[j].z, gv[j].w * ga[j].w);
            sum_dy += (dy.x + dy.y) + (dy.z + dy.w);
            sum_dy_norm += (dy.x * v[j].x + dy.y * v[j].y) + (dy.z * v[j].z + dy.w * v[j].w);
            dga[j].x += gv[j].x * v[j].x;
            dga[j].y += gv[j].y * v[j].y;
            dga[j].z += gv[j].z * v[j].z;
            dga[j].w += gv[j].w * v[j].w;
            dbe[j].x += gv[j].x;
            dbe[j].y += gv[j].y;
            dbe[j].z += gv[j].z;
            dbe[j].w += gv[j].w;
        }
        sum_dy = warp_sum(sum_dy);
        sum_dy_norm = warp_sum(sum_dy_norm);
        float k = rstd * inv_dim;
        float *d = dx + r * dim;
#pragma unroll
        for (int j = 0; j < NV; ++j)
            if (lane + 32 * j < dim4) {
                float4 o;
                o.x = (fdim * gv[j].x * ga[j].x - sum_dy - v[j].x * sum_dy_norm) * k;
                o.y = (fdim * gv[j].y * ga[j].y - sum_dy - v[j].y * sum_dy_norm) * k;
                o.z = (fdim * gv[j].z * ga[j].z - sum_dy - v[j].z * sum_dy_norm) * k;
                o.w = (fdim * gv[j].w * ga[j].w - sum_dy - v[j].w * sum_dy_norm) * k;
                if (addend) { // gradient already pending for this input (residual branch): dx joins it
                    o.x += ad[j].x;
                    o.y += ad[j].y;
                    o.z += ad[j].z;
                    o.w += ad[j].w;
                }
                reinterpret_cast<float4 *>(d)[lane + 32 * j] = o;
            }
        if (rn < rows) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                v[j] = nx[j];
                graw[j] = ng[j];
            }
        }
    }
    // fold the warps' register sums in warp order 0..7 (fixed order: run-to-run identical results)
    float4 *acc_g = reinterpret_cast<float4 *>(acc), *acc_b = acc_g + 32 * NV;
    for (int turn = 0; turn < kWarps; ++turn) {
        if (w == turn) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                int idx = lane + 32 * j;
                if (turn == 0) {
                    acc_g[idx] = dga[j];
                    acc_b[idx] = dbe[j];
                } else {
                    float4 a = acc_g[idx], b = acc_b[idx];
                    acc_g[idx] = make_float4(a.x + dga[j].x, a.y + dga[j].y, a.z + dga[j].z, a.w + dga[j].w);
                    acc_b[idx] = make_float4(b.x + dbe[j].x, b.y + dbe[j].y, b.z + dbe[j].z, b.w + dbe[j].w);
                }
            }
        }
        __syncthreads();
    }
    float *dst = partial + (size_t)blockIdx.x * 2 * dim;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        dst[c] = acc[c];
        dst[dim + c] = acc[32 * NV * 4 + c];
    }
}

__global__ void ln_params_final_kernel(const float *__restrict__ partial, int blocks, int dim, float *__restrict__ dgamma,
                                       float *__restrict__ dbeta) {
    // block (32, 32): 32 of the 2*dim columns, 32 interleaved groups of per-block partials, fixed order;
    // the few loads of a thread are independent, so the kernel costs about one memory round trip
    __shared__ float red[32][33];
    int j = blockIdx.x * 32 + threadIdx.x;
    float t = 0.0f;
    if (j < 2 * dim) {
#pragma unroll 4
        for (int b = threadIdx.y; b < blocks; b += 32) t += partial[(size_t)b * 2 * dim + j];
    }
    red[threadIdx.y][threadIdx.x] = t;
    __syncthreads();
    if (threadIdx.y == 0 && j < 2 * dim) {
        float u = 0.0f;
#pragma unroll
        for (int y = 0; y < 32; ++y) u += red[y][threadIdx.x];
        if (j < dim) dgamma[j] = u;
        else dbeta[j - dim] = u;
    }
}

int pick_nv(int64_t dim) {
    int64_t need = (dim / 4 + 31) / 32;
    const int opts[6] = {1, 2, 3, 4, 6, 8};
    for (int i = 0; i < 6; ++i)
        if (need <= opts[i]) return opts[i];
    return 0;
}

template <typename OutT>
void launch_fwd(int nv, int grid, cudaStream_t s, const float *x, const float *gamma, const float *beta, float eps, OutT *out, float *mean,
                float *rstd, long long rows, int dim) {
    switch (nv) {
    case 1: ln_fwd_reg_kernel<OutT, 1><<<grid, kWarps * 32, 0, s>>>(x, gamma, beta, eps, out, mean, rstd, rows, dim); break;
    case 2: ln_fwd_reg_kernel<OutT, 2><<<grid, kWarps * 32, 0, s>>>(x, gamma, beta, eps, out, mean, rstd, rows, dim); break;
    case 3: ln_fwd_reg_kernel<OutT, 3><<<grid, kWarps * 32, 0, s>>>(x, gamma, beta, eps, out, mean, rstd, rows, dim); break;
    case 4: ln_fwd_reg_kernel<OutT, 4><<<grid, kWarps * 32, 0, s>>>(x, gamma, beta, eps, out, mean, rstd, rows, dim); break;
    case 6: ln_fwd_reg_kernel<OutT, 6><<<grid, kWarps * 32, 0, s>>>(x, gamma, beta, eps, out, mean, rstd, rows, dim); break;
    default: ln_fwd_reg_kernel<OutT, 8><<<grid, kWarps * 32, 0, s>>>(x, gamma, beta, eps, out, mean, rstd, rows, dim); break;
    }
}
template <typename GT>
void launch_bwd(int nv, int grid, cudaStream_t s, const float *x, const float *gamma, const GT *g, float eps, const float *mean,
                const float *rstd, const float *addend, float *dx, float *partial, long long rows, int dim) {
    switch (nv) {
    case 1: ln_bwd_reg_kernel<GT, 1><<<grid, kWarps * 32, 0, s>>>(x, gamma, g, eps, mean, rstd, addend, dx, partial, rows, dim); break;
    case 2: ln_bwd_reg_kernel<GT, 2><<<grid, kWarps * 32, 0, s>>>(x, gamma, g, eps, mean, rstd, addend, dx, partial, rows, dim); break;
    case 3: ln_bwd_reg_kernel<GT, 3><<<grid, kWarps * 32, 0, s>>>(x, gamma, g, eps, mean, rstd, addend, dx, partial, rows, dim); break;
    case 4: ln_bwd_reg_kernel<GT, 4><<<grid, kWarps * 32, 0, s>>>(x, gamma, g, eps, mean, rstd, addend, dx, partial, rows, dim); break;
    case 6: ln_bwd_reg_kernel<GT, 6><<<grid, kWarps * 32, 0, s>>>(x, gamma, g, eps, mean, rstd, addend, dx, partial, rows, dim); break;
    default: ln_bwd_reg_kernel<GT, 8><<<grid, kWarps * 32, 0, s>>>(x, gamma, g, eps, mean, rstd, addend, dx, partial, rows, dim); break;
    }
}

bool eligible(int64_t dim, const void *a, const void *b, const void *c, const void *d) {
    return dim % 4 == 0 && dim <= 1024 && mcb_aligned16(a) && mcb_aligned16(b) && mcb_aligned16(c) && mcb_aligned16(d);
}

} // namespace

// Returns MCB_UNSUPPORTED (and launches nothing) when the shape is outside the register-resident range.
mcb_status mcb_ln_fast_forward(mcb_ctx *ctx, const float *x, const float *gamma, const float *beta, double eps, void *out, int32_t out_dt,
                               float *mean, float *rstd, int64_t rows, int64_t dim) {
    if (!eligible(dim, x, gamma, beta, out)) return MCB_UNSUPPORTED;
    if (out_dt != MCB_F32 && out_dt != MCB_BF16) return MCB_UNSUPPORTED; // f16 rows take the generic kernel
    if (out_dt == MCB_BF16 && (dim % 8)) return MCB_UNSUPPORTED; // 8-byte bf16x4 stores need even row starts of 8 bytes: dim*2 % 8 == 0 holds; keep 16 B rows
    int nv = pick_nv(dim);
    int grid = mcb_grid_for(ctx, rows, kWarps, 2); // few persistent warps: gamma / beta are fetched once per warp, not once per row
    if (out_dt == MCB_F32) launch_fwd<float>(nv, grid, ctx->stream, x, gamma, beta, (float)eps, (float *)out, mean, rstd, rows, (int)dim);
    else launch_fwd<__nv_bfloat16>(nv, grid, ctx->stream, x, gamma, beta, (float)eps, (__nv_bfloat16 *)out, mean, rstd, rows, (int)dim);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_ln_fast_backward(mcb_ctx *ctx, const float *x, const float *gamma, const void *g, int32_t g_dt, double eps, const float *mean,
                                const float *rstd, const float *addend, float *dx, float *dgamma, float *dbeta, int64_t rows, int64_t dim) {
    if (!eligible(dim, x, gamma, g, dx) || rows == 0 || (addend && !mcb_aligned16(addend))) return MCB_UNSUPPORTED;
    if (g_dt == MCB_BF16 && (dim % 8)) return MCB_UNSUPPORTED;
    if (g_dt != MCB_F32 && g_dt != MCB_BF16) return MCB_UNSUPPORTED; // f16 gradients take the generic kernel
    int nv = pick_nv(dim);
    int grid = mcb_grid_for(ctx, rows, kWarps, 2);
    void *scratch;
    MCB_TRY(mcb_scratch(ctx, sizeof(float) * (size_t)grid * 2 * dim, &scratch));
    if (g_dt == MCB_F32) launch_bwd<float>(nv, grid, ctx->stream, x, gamma, (const float *)g, (float)eps, mean, rstd, addend, dx, (float *)scratch, rows, (int)dim);
    else launch_bwd<__nv_bfloat16>(nv, grid, ctx->stream, x, gamma, (const __nv_bfloat16 *)g, (float)eps, mean, rstd, addend, dx, (float *)scratch, rows, (int)dim);
    MCB_LAUNCHED(ctx);
    ln_params_final_kernel<<<(int)((2 * dim + 31) / 32), dim3(32, 32), 0, ctx->stream>>>((const float *)scratch, grid, (int)dim, dgamma, dbeta);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}
