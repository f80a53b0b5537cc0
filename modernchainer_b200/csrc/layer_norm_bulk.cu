// LayerNorm forward / backward as a bulk-copy pipeline (rows of up to 1024 elements, dim % 8 == 0).
//
// One persistent CTA per SM: a producer thread streams blocks of eight (forward) or seven (backward) consecutive rows (x, and for
// backward g and the pending gradient) from HBM into a ring of shared-memory stages with
// cp.async.bulk (rows are contiguous, so each operand of a block is ONE copy and no tensor map is
// needed); one compute warp per row takes its row from the stage, reduces it with warp shuffles and
// writes the result straight from registers.  The ring keeps 100-180 KB of loads in flight per SM
// without holding them in registers, which is what bounded the register-resident kernels
// (layer_norm_fast.cu: 255 registers, one block per SM, 3.4 TB/s).  Every mbarrier wait is bounded.
// dgamma / dbeta: per-lane register sums over the rows a warp handles, folded through shared memory in
// a fixed warp order, finished by ln_bulk_params_final over the per-CTA partials (no float atomics).  Backward can
// also leave dx rounded to bf16 and the column sums of those values for the Linear backward that reads dx next.
#include <type_traits>

#include "common.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

namespace {

using namespace tcptx;

// rows per stage = compute warps.  Seven for backward, so that the block is eight warps with the producer: a ninth
// warp puts three warps on one SM sub-partition, whose 16 K registers then cap every thread at 168, which the backward
// kernel with by-products exceeds
constexpr int kRowsBwd = 7;
constexpr int kRowsFwd = 8;                  // the forward kernel needs 112 registers: nine warps are fine
constexpr int kThreadsBwd = (kRowsBwd + 1) * 32; // + the producer warp
constexpr int kThreadsFwd = (kRowsFwd + 1) * 32;
constexpr int kMaxStages = 6;
constexpr unsigned kSmemBudget = 200u * 1024u;

struct LnBulkArgs {
    const float *x, *gamma, *beta;
    const void *g;       // backward: upstream gradient (f32 or bf16)
    const float *mean_in, *rstd_in;
    const float *addend; // backward: gradient already pending for x (may alias dx), or null
    void *out;           // forward: y (f32 or bf16); backward: dx (f32)
    float *mean_out, *rstd_out;
    float *partial;      // backward: [grid][2][dim], or [grid][3][dim] with dx_bf16
    int f16;             // the 16-bit operands (out, res, g, dx_bf16) are f16 instead of bf16
    __nv_bfloat16 *dx_bf16; // backward, optional: dx rounded to bf16 (what the backward GEMMs of the Linear feeding this
                            // residual stream read); the third partial row then holds the column sums of those rounded values
    float *sum_out;      // forward with a residual operand (g): x + g, written beside the normalised rows
    long long rows;
    int dim;
    int stages;
    unsigned stage_bytes, off_g, off_ad;
    float eps;
    unsigned int *err;
};

__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gsrc, unsigned bytes, unsigned long long *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :
                 : "r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// 16-bit operands are bf16 or, when `f16` is set (LnBulkArgs::f16, the same for every thread), IEEE f16;
// the kernels are compiled once for "a 16-bit type" (the template parameter stays __nv_bfloat16)
__device__ __forceinline__ float4 unpack4(float4 r, int) { return r; }
__device__ __forceinline__ float4 unpack4(uint2 r, int f16) {
    float2 a, b;
    if (f16) {
        a = Lp<__half>::unpack2(r.x);
        b = Lp<__half>::unpack2(r.y);
    } else {
        a = Lp<__nv_bfloat16>::unpack2(r.x);
        b = Lp<__nv_bfloat16>::unpack2(r.y);
    }
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ uint2 pack4(float4 v, int f16) {
    return f16 ? make_uint2(Lp<__half>::pack2(v.x, v.y), Lp<__half>::pack2(v.z, v.w))
               : make_uint2(Lp<__nv_bfloat16>::pack2(v.x, v.y), Lp<__nv_bfloat16>::pack2(v.z, v.w));
}
template <typename T> struct Raw4 { typedef float4 type; };
template <> struct Raw4<__nv_bfloat16> { typedef uint2 type; };

__device__ __forceinline__ void store4(float *p, int idx, float4 v, int) { reinterpret_cast<float4 *>(p)[idx] = v; }
__device__ __forceinline__ void store4(__nv_bfloat16 *p, int idx, float4 v, int f16) { reinterpret_cast<uint2 *>(p)[idx] = pack4(v, f16); }

// The producer: one thread walks this CTA's row blocks and fills the ring.  NOPS operands per stage.
template <int NOPS, int kRows>
__device__ __forceinline__ void produce(const LnBulkArgs &a, unsigned char *smem, unsigned long long *full, unsigned long long *empty,
                                        volatile int *abort_flag, const void *const (&src)[3], const unsigned (&elem)[3],
                                        const unsigned (&off)[3]) {
    const long long nblk = (a.rows + kRows - 1) / kRows;
    unsigned it = 0;
    for (long long blk = blockIdx.x; blk < nblk; blk += gridDim.x, ++it) {
        const int s = (int)(it % (unsigned)a.stages);
        const unsigned use = it / (unsigned)a.stages;
        if (use > 0 && !mbar_wait(&empty[s], (use - 1) & 1u, abort_flag, a.err)) return;
        const long long r0 = blk * kRows;
        const unsigned nr = (unsigned)min((long long)kRows, a.rows - r0);
        unsigned total = 0;
#pragma unroll
        for (int o = 0; o < NOPS; ++o)
            if (src[o]) total += nr * (unsigned)a.dim * elem[o];
        mbar_expect_tx(&full[s], total);
        unsigned char *stage = smem + (size_t)s * a.stage_bytes;
#pragma unroll
        for (int o = 0; o < NOPS; ++o)
            if (src[o])
                bulk_load(stage + off[o], (const unsigned char *)src[o] + (size_t)r0 * a.dim * elem[o], nr * (unsigned)a.dim * elem[o], &full[s]);
    }
}

template <int kRows> __device__ __forceinline__ void ring_init(const LnBulkArgs &a, unsigned long long *full, unsigned long long *empty, volatile int *abort_flag) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kRows);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    dep_wait(); // global memory is touched only from here on
    dep_trigger();
}

// ResT = void: y = LN(x).  Otherwise the residual add of a pre-norm block rides along: s = x + g (g of type
// ResT) is written to sum_out and y = LN(s), in the arithmetic of the separate add and LayerNorm kernels.
template <typename OutT, int NV, typename ResT>
__global__ void __launch_bounds__(kThreadsFwd, 1) ln_fwd_bulk_kernel(const LnBulkArgs a) {
    constexpr int kRows = kRowsFwd;
    constexpr bool kRes = !std::is_same<ResT, void>::value;
    typedef typename std::conditional<kRes, ResT, float>::type RT;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned long long *full = (unsigned long long *)(smem + (size_t)a.stages * a.stage_bytes), *empty = full + kMaxStages;
    volatile int *abort_flag = (volatile int *)(empty + kMaxStages);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ring_init<kRows>(a, full, empty, abort_flag);
    if (warp == kRows) {
        if (lane == 0) {
            const void *const src[3] = {a.x, kRes ? a.g : nullptr, nullptr};
            const unsigned elem[3] = {4u, (unsigned)sizeof(RT), 0u}, off[3] = {0u, a.off_g, 0u};
            produce<2, kRows>(a, smem, full, empty, abort_flag, src, elem, off);
        }
        return;
    }
    const int dim4 = a.dim >> 2;
    const float inv_dim = 1.0f / (float)a.dim;
    float4 ga[NV], be[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int idx = lane + 32 * j;
        ga[j] = idx < dim4 ? reinterpret_cast<const float4 *>(a.gamma)[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
        be[j] = idx < dim4 ? reinterpret_cast<const float4 *>(a.beta)[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const long long nblk = (a.rows + kRows - 1) / kRows;
    unsigned it = 0;
    for (long long blk = blockIdx.x; blk < nblk; blk += gridDim.x, ++it) {
        const int s = (int)(it % (unsigned)a.stages);
        const unsigned ph = (it / (unsigned)a.stages) & 1u;
        const long long r = blk * kRows + warp;
        if (!mbar_wait(&full[s], ph, abort_flag, a.err)) break;
        if (r < a.rows) {
            const float4 *sx = reinterpret_cast<const float4 *>(smem + (size_t)s * a.stage_bytes + (size_t)warp * a.dim * 4);
            float4 v[NV];
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int idx = lane + 32 * j;
                v[j] = idx < dim4 ? sx[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
                if (kRes && idx < dim4) {
                    const typename Raw4<RT>::type *sg =
                        reinterpret_cast<const typename Raw4<RT>::type *>(smem + (size_t)s * a.stage_bytes + a.off_g + (size_t)warp * a.dim * sizeof(RT));
                    const float4 t = unpack4(sg[idx], a.f16);
                    v[j] = make_float4(v[j].x + t.x, v[j].y + t.y, v[j].z + t.z, v[j].w + t.w);
                    reinterpret_cast<float4 *>(a.sum_out + r * a.dim)[idx] = v[j];
                }
                sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
            }
            const float mean = warp_sum(sum) * inv_dim;
            float var = 0.0f;
#pragma unroll
            for (int j = 0; j < NV; ++j)
                if (lane + 32 * j < dim4) {
                    const float p = v[j].x - mean, q = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                    var += (p * p + q * q) + (c * c + d * d);
                }
            var = warp_sum(var) * inv_dim;
            const float rstd = 1.0f / sqrtf(var + a.eps);
            if (lane == 0) {
                if (a.mean_out) a.mean_out[r] = mean;
                if (a.rstd_out) a.rstd_out[r] = rstd;
            }
            OutT *d = (OutT *)a.out + r * a.dim;
#pragma unroll
            for (int j = 0; j < NV; ++j)
                if (lane + 32 * j < dim4)
                    store4(d, lane + 32 * j,
                           make_float4((v[j].x - mean) * rstd * ga[j].x + be[j].x, (v[j].y - mean) * rstd * ga[j].y + be[j].y,
                                       (v[j].z - mean) * rstd * ga[j].z + be[j].z, (v[j].w - mean) * rstd * ga[j].w + be[j].w), a.f16);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
}

// (256 threads: the variant with by-products needs about 200 registers)
template <typename GT, int NV, bool AUX>
__global__ void __maxnreg__(216) ln_bwd_bulk_kernel(const LnBulkArgs a) {
    constexpr int kRows = kRowsBwd;
    constexpr int kVec = AUX ? 3 : 2; // dgamma, dbeta (, column sums of the bf16 copy of dx)
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ float acc[kVec * 32 * NV * 4];
    unsigned long long *full = (unsigned long long *)(smem + (size_t)a.stages * a.stage_bytes), *empty = full + kMaxStages;
    volatile int *abort_flag = (volatile int *)(empty + kMaxStages);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ring_init<kRows>(a, full, empty, abort_flag);
    const int dim4 = a.dim >> 2;
    float4 dga[NV], dbe[NV], dcs[AUX ? NV : 1];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        dga[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        dbe[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (AUX) dcs[AUX ? j : 0] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (warp == kRows) {
        if (lane == 0) {
            const void *const src[3] = {a.x, a.g, a.addend};
            const unsigned elem[3] = {4u, (unsigned)sizeof(GT), 4u}, off[3] = {0u, a.off_g, a.off_ad};
            produce<3, kRows>(a, smem, full, empty, abort_flag, src, elem, off);
        }
    } else {
        const float fdim = (float)a.dim, inv_dim = 1.0f / fdim;
        float4 ga[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int idx = lane + 32 * j;
            ga[j] = idx < dim4 ? reinterpret_cast<const float4 *>(a.gamma)[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const bool have_stats = a.mean_in && a.rstd_in;
        const long long nblk = (a.rows + kRows - 1) / kRows;
        unsigned it = 0;
        for (long long blk = blockIdx.x; blk < nblk; blk += gridDim.x, ++it) {
            const int s = (int)(it % (unsigned)a.stages);
            const unsigned ph = (it / (unsigned)a.stages) & 1u;
            const long long r = blk * kRows + warp;
            float mean = 0.0f, rstd = 0.0f; // requested before the wait: the two scalars arrive while the stage fills
            if (have_stats && r < a.rows) {
                mean = __ldg(a.mean_in + r);
                rstd = __ldg(a.rstd_in + r);
            }
            if (!mbar_wait(&full[s], ph, abort_flag, a.err)) break;
            if (r < a.rows) {
                const unsigned char *stage = smem + (size_t)s * a.stage_bytes;
                const float4 *sx = reinterpret_cast<const float4 *>(stage + (size_t)warp * a.dim * 4);
                const typename Raw4<GT>::type *sg = reinterpret_cast<const typename Raw4<GT>::type *>(stage + a.off_g + (size_t)warp * a.dim * sizeof(GT));
                const float4 *sa = reinterpret_cast<const float4 *>(stage + a.off_ad + (size_t)warp * a.dim * 4);
                float4 v[NV], gv[NV];
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    const int idx = lane + 32 * j;
                    if (idx < dim4) {
                        v[j] = sx[idx];
                        gv[j] = unpack4(sg[idx], a.f16);
                    } else {
                        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                        gv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                if (!have_stats) {
                    float sum = 0.0f;
#pragma unroll
                    for (int j = 0; j < NV; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
                    mean = warp_sum(sum) * inv_dim;
                    float var = 0.0f;
#pragma unroll
                    for (int j = 0; j < NV; ++j)
                        if (lane + 32 * j < dim4) {
                            const float p = v[j].x - mean, q = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                            var += (p * p + q * q) + (c * c + d * d);
                        }
                    rstd = 1.0f / sqrtf(warp_sum(var) * inv_dim + a.eps);
                }
                float sum_dy = 0.0f, sum_dy_norm = 0.0f;
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    // v becomes the normalised value; lanes past the row end hold zeros in gv, so they add nothing
                    v[j].x = (v[j].x - mean) * rstd;
                    v[j].y = (v[j].y - mean) * rstd;
                    v[j].z = (v[j].z - mean) * rstd;
                    v[j].w = (v[j].w - mean) * rstd;
                    const float4 dy = make_float4(gv[j].x * ga[j].x, gv[j].y * ga[j].y, gv[j].z * ga[j].z, gv[j].w * ga[j].w);
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
                const float k = rstd * inv_dim;
                float *d = (float *)a.out + r * a.dim;
#pragma unroll
                for (int j = 0; j < NV; ++j)
                    if (lane + 32 * j < dim4) {
                        float4 o;
                        o.x = (fdim * gv[j].x * ga[j].x - sum_dy - v[j].x * sum_dy_norm) * k;
                        o.y = (fdim * gv[j].y * ga[j].y - sum_dy - v[j].y * sum_dy_norm) * k;
                        o.z = (fdim * gv[j].z * ga[j].z - sum_dy - v[j].z * sum_dy_norm) * k;
                        o.w = (fdim * gv[j].w * ga[j].w - sum_dy - v[j].w * sum_dy_norm) * k;
                        if (a.addend) { // gradient already pending for this input (residual branch): dx joins it
                            const float4 ad = sa[lane + 32 * j];
                            o.x += ad.x;
                            o.y += ad.y;
                            o.z += ad.z;
                            o.w += ad.w;
                        }
                        reinterpret_cast<float4 *>(d)[lane + 32 * j] = o;
                        if (AUX) { // the bf16 copy the next Linear's backward GEMMs read, and the column sums of exactly those values
                            const uint2 h = pack4(o, a.f16);
                            reinterpret_cast<uint2 *>(a.dx_bf16 + r * a.dim)[lane + 32 * j] = h;
                            const float4 back = unpack4(h, a.f16);
                            float4 &cs = dcs[AUX ? j : 0];
                            cs.x += back.x;
                            cs.y += back.y;
                            cs.z += back.z;
                            cs.w += back.w;
                        }
                    }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
    }
    // fold the compute warps' register sums in warp order 0..7 (fixed order: run-to-run identical results)
    float4 *acc_g = reinterpret_cast<float4 *>(acc), *acc_b = acc_g + 32 * NV;
    for (int turn = 0; turn < kRows; ++turn) {
        if (warp == turn) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int idx = lane + 32 * j;
                if (turn == 0) {
                    acc_g[idx] = dga[j];
                    acc_b[idx] = dbe[j];
                    if (AUX) acc_b[32 * NV + idx] = dcs[AUX ? j : 0];
                } else {
                    const float4 p = acc_g[idx], q = acc_b[idx];
                    acc_g[idx] = make_float4(p.x + dga[j].x, p.y + dga[j].y, p.z + dga[j].z, p.w + dga[j].w);
                    acc_b[idx] = make_float4(q.x + dbe[j].x, q.y + dbe[j].y, q.z + dbe[j].z, q.w + dbe[j].w);
                    if (AUX) {
                        const float4 t = acc_b[32 * NV + idx], u = dcs[AUX ? j : 0];
                        acc_b[32 * NV + idx] = make_float4(t.x + u.x, t.y + u.y, t.z + u.z, t.w + u.w);
                    }
                }
            }
        }
        __syncthreads();
    }
    float *dst = a.partial + (size_t)blockIdx.x * kVec * a.dim;
    for (int c = threadIdx.x; c < a.dim; c += blockDim.x) {
        dst[c] = acc[c];
        dst[a.dim + c] = acc[32 * NV * 4 + c];
        if (AUX) dst[2 * a.dim + c] = acc[2 * 32 * NV * 4 + c];
    }
}

__global__ void ln_bulk_params_final(const float *__restrict__ partial, int blocks, int dim, float *__restrict__ dgamma, float *__restrict__ dbeta,
                                     float *__restrict__ colsum) {
    // block (32, 32): 32 of the nvec*dim columns (nvec = 3 with `colsum`), 32 interleaved groups of per-CTA partials, fixed order
    const int nvec = colsum ? 3 : 2;
    __shared__ float red[32][33];
    const int j = blockIdx.x * 32 + threadIdx.x;
    dep_wait();
    dep_trigger();
    float t = 0.0f;
    if (j < nvec * dim) {
#pragma unroll 4
        for (int b = threadIdx.y; b < blocks; b += 32) t += partial[(size_t)b * nvec * dim + j];
    }
    red[threadIdx.y][threadIdx.x] = t;
    __syncthreads();
    if (threadIdx.y == 0 && j < nvec * dim) {
        float u = 0.0f;
#pragma unroll
        for (int y = 0; y < 32; ++y) u += red[y][threadIdx.x];
        if (j < dim) dgamma[j] = u;
        else if (j < 2 * dim) dbeta[j - dim] = u;
        else colsum[j - 2 * dim] = u;
    }
}

int pick_nv(int64_t dim) {
    const int64_t need = (dim / 4 + 31) / 32;
    const int opts[6] = {1, 2, 3, 4, 6, 8};
    for (int i = 0; i < 6; ++i)
        if (need <= opts[i]) return opts[i];
    return 0;
}

unsigned round128(size_t v) { return (unsigned)((v + 127) & ~(size_t)127); }

// stages that fit the shared-memory budget; 0 = use another kernel
int plan_stages(unsigned stage_bytes) {
    int st = (int)(kSmemBudget / stage_bytes);
    if (st > kMaxStages) st = kMaxStages;
    return st >= 2 ? st : 0;
}

template <typename K> mcb_status launch(mcb_ctx *ctx, K kernel, const LnBulkArgs &a, int grid, const char *what) {
    const int kThreads = what[0] == 'f' ? kThreadsFwd : kThreadsBwd;
    const size_t smem = (size_t)a.stages * a.stage_bytes + 2 * kMaxStages * sizeof(unsigned long long) + 16;
    MCB_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MCB_CUDA(ctx, mcb_launch_dep(ctx, kernel, dim3(grid), dim3(kThreads), smem, a));
    MCB_LAUNCHED(ctx);
    (void)what;
    return MCB_OK;
}

template <typename OutT, typename ResT> mcb_status launch_fwd(mcb_ctx *ctx, int nv, const LnBulkArgs &a, int grid) {
    switch (nv) {
    case 1: return launch(ctx, ln_fwd_bulk_kernel<OutT, 1, ResT>, a, grid, "fwd");
    case 2: return launch(ctx, ln_fwd_bulk_kernel<OutT, 2, ResT>, a, grid, "fwd");
    case 3: return launch(ctx, ln_fwd_bulk_kernel<OutT, 3, ResT>, a, grid, "fwd");
    case 4: return launch(ctx, ln_fwd_bulk_kernel<OutT, 4, ResT>, a, grid, "fwd");
    case 6: return launch(ctx, ln_fwd_bulk_kernel<OutT, 6, ResT>, a, grid, "fwd");
    default: return launch(ctx, ln_fwd_bulk_kernel<OutT, 8, ResT>, a, grid, "fwd");
    }
}
template <typename GT, bool AUX> mcb_status launch_bwd_aux(mcb_ctx *ctx, int nv, const LnBulkArgs &a, int grid) {
    switch (nv) {
    case 1: return launch(ctx, ln_bwd_bulk_kernel<GT, 1, AUX>, a, grid, "bwd");
    case 2: return launch(ctx, ln_bwd_bulk_kernel<GT, 2, AUX>, a, grid, "bwd");
    case 3: return launch(ctx, ln_bwd_bulk_kernel<GT, 3, AUX>, a, grid, "bwd");
    case 4: return launch(ctx, ln_bwd_bulk_kernel<GT, 4, AUX>, a, grid, "bwd");
    case 6: return launch(ctx, ln_bwd_bulk_kernel<GT, 6, AUX>, a, grid, "bwd");
    default: return launch(ctx, ln_bwd_bulk_kernel<GT, 8, AUX>, a, grid, "bwd");
    }
}
template <typename GT> mcb_status launch_bwd(mcb_ctx *ctx, int nv, const LnBulkArgs &a, int grid) {
    return a.dx_bf16 ? launch_bwd_aux<GT, true>(ctx, nv, a, grid) : launch_bwd_aux<GT, false>(ctx, nv, a, grid);
}

bool eligible(int64_t rows, int64_t dim, const void *p0, const void *p1, const void *p2, const void *p3) {
    // bulk copies need 16-byte aligned row starts for every operand (bf16 rows: dim % 8 == 0); small problems
    // do not fill a persistent grid and stay on the register-resident kernels
    return dim % 8 == 0 && dim >= 128 && dim <= 1024 && rows >= 8 * 148 && mcb_aligned16(p0) && mcb_aligned16(p1) && mcb_aligned16(p2) &&
           mcb_aligned16(p3);
}

} // namespace

mcb_status mcb_ln_bulk_forward(mcb_ctx *ctx, const float *x, const float *gamma, const float *beta, double eps, void *out, int32_t out_dt,
                               float *mean, float *rstd, int64_t rows, int64_t dim) {
    if (!eligible(rows, dim, x, gamma, beta, out) || knob_on(ctx, K_LN_NO_BULK)) return MCB_UNSUPPORTED;
    LnBulkArgs a = {};
    a.x = x; a.gamma = gamma; a.beta = beta; a.out = out; a.mean_out = mean; a.rstd_out = rstd;
    a.rows = rows; a.dim = (int)dim; a.eps = (float)eps; a.err = ctx->d_err;
    a.stage_bytes = round128((size_t)kRowsFwd * dim * 4);
    a.stages = plan_stages(a.stage_bytes);
    if (!a.stages) return MCB_UNSUPPORTED;
    const int64_t nblk = (rows + kRowsFwd - 1) / kRowsFwd;
    const int grid = (int)(nblk < ctx->sm_count ? nblk : ctx->sm_count);
    const int nv = pick_nv(dim);
    if (out_dt == MCB_F32) return launch_fwd<float, void>(ctx, nv, a, grid);
    if (!mcb_is_lp(out_dt)) return MCB_UNSUPPORTED;
    a.f16 = out_dt == MCB_F16;
    return launch_fwd<__nv_bfloat16, void>(ctx, nv, a, grid);
}

// sum = x + res (res f32 or bf16), out = LayerNorm(sum): the residual add and the LayerNorm that follows it in a
// pre-norm block, in one pass over the rows.  Same arithmetic as mcb_add_typed followed by mcb_layer_norm.
mcb_status mcb_ln_bulk_add_forward(mcb_ctx *ctx, const float *x, const void *res, int32_t res_dt, const float *gamma, const float *beta, double eps,
                                   float *sum, void *out, int32_t out_dt, float *mean, float *rstd, int64_t rows, int64_t dim) {
    if (!eligible(rows, dim, x, gamma, beta, out) || !mcb_aligned16(res) || !mcb_aligned16(sum) || knob_on(ctx, K_LN_NO_BULK)) return MCB_UNSUPPORTED;
    if ((res_dt != MCB_F32 && !mcb_is_lp(res_dt)) || (out_dt != MCB_F32 && !mcb_is_lp(out_dt))) return MCB_UNSUPPORTED;
    if (mcb_is_lp(res_dt) && mcb_is_lp(out_dt) && res_dt != out_dt) return MCB_UNSUPPORTED; // one 16-bit format per launch
    LnBulkArgs a = {};
    a.x = x; a.g = res; a.gamma = gamma; a.beta = beta; a.out = out; a.sum_out = sum; a.mean_out = mean; a.rstd_out = rstd;
    a.rows = rows; a.dim = (int)dim; a.eps = (float)eps; a.err = ctx->d_err;
    a.f16 = res_dt == MCB_F16 || out_dt == MCB_F16;
    a.off_g = round128((size_t)kRowsFwd * dim * 4);
    a.stage_bytes = a.off_g + round128((size_t)kRowsFwd * dim * (mcb_is_lp(res_dt) ? 2 : 4));
    a.stages = plan_stages(a.stage_bytes);
    if (!a.stages) return MCB_UNSUPPORTED;
    const int64_t nblk = (rows + kRowsFwd - 1) / kRowsFwd;
    const int grid = (int)(nblk < ctx->sm_count ? nblk : ctx->sm_count);
    const int nv = pick_nv(dim);
    if (out_dt == MCB_F32) {
        if (res_dt == MCB_F32) return launch_fwd<float, float>(ctx, nv, a, grid);
        return launch_fwd<float, __nv_bfloat16>(ctx, nv, a, grid);
    }
    if (res_dt == MCB_F32) return launch_fwd<__nv_bfloat16, float>(ctx, nv, a, grid);
    return launch_fwd<__nv_bfloat16, __nv_bfloat16>(ctx, nv, a, grid);
}

mcb_status mcb_ln_bulk_backward(mcb_ctx *ctx, const float *x, const float *gamma, const void *g, int32_t g_dt, double eps, const float *mean,
                                const float *rstd, const float *addend, float *dx, float *dgamma, float *dbeta, int64_t rows, int64_t dim,
                                void *dx_bf16, float *dx_colsum, int32_t aux_dt) {
    if (g_dt != MCB_F32 && !mcb_is_lp(g_dt)) return MCB_UNSUPPORTED;
    if (dx_bf16 && mcb_is_lp(g_dt) && aux_dt != g_dt) return MCB_UNSUPPORTED; // one 16-bit format per launch
    if (!eligible(rows, dim, x, gamma, g, dx) || (addend && !mcb_aligned16(addend)) || knob_on(ctx, K_LN_NO_BULK)) return MCB_UNSUPPORTED;
    if ((dx_bf16 != nullptr) != (dx_colsum != nullptr) || (dx_bf16 && !mcb_aligned16(dx_bf16))) return MCB_UNSUPPORTED;
    LnBulkArgs a = {};
    a.x = x; a.gamma = gamma; a.g = g; a.mean_in = mean; a.rstd_in = rstd; a.addend = addend; a.out = dx;
    a.dx_bf16 = (__nv_bfloat16 *)dx_bf16;
    a.rows = rows; a.dim = (int)dim; a.eps = (float)eps; a.err = ctx->d_err;
    a.f16 = g_dt == MCB_F16 || (dx_bf16 && aux_dt == MCB_F16);
    const size_t gsz = mcb_is_lp(g_dt) ? 2 : 4;
    a.off_g = round128((size_t)kRowsBwd * dim * 4);
    a.off_ad = a.off_g + round128((size_t)kRowsBwd * dim * gsz);
    a.stage_bytes = a.off_ad + (addend ? round128((size_t)kRowsBwd * dim * 4) : 0u);
    a.stages = plan_stages(a.stage_bytes);
    if (!a.stages) return MCB_UNSUPPORTED;
    const int64_t nblk = (rows + kRowsBwd - 1) / kRowsBwd;
    const int grid = (int)(nblk < ctx->sm_count ? nblk : ctx->sm_count);
    void *scratch;
    MCB_TRY(mcb_scratch(ctx, sizeof(float) * (size_t)grid * (dx_bf16 ? 3 : 2) * dim, &scratch));
    a.partial = (float *)scratch;
    const int nv = pick_nv(dim);
    if (g_dt == MCB_F32) MCB_TRY(launch_bwd<float>(ctx, nv, a, grid));
    else MCB_TRY(launch_bwd<__nv_bfloat16>(ctx, nv, a, grid));
    MCB_CUDA(ctx, mcb_launch_dep(ctx, ln_bulk_params_final, dim3((unsigned)(((dx_bf16 ? 3 : 2) * dim + 31) / 32)), dim3(32, 32), 0, (const float *)scratch, grid,
                                 (int)dim, dgamma, dbeta, dx_colsum));
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}
