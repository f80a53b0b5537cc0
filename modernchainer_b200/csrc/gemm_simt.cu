// Exact-f32 GEMM family (FFMA, no tensor cores): the MCB_COMPUTE_F32 path behind
// Ops::matmul / linear / linear_backward, and the batched products of the f32 attention.
// One kernel with generic element strides covers NN / NT / TN operands, so no transpose is
// ever materialised (the reference builds grad^T with transpose2d_f32 in every
// linear_backward, crates/modern-chainer-cuda/src/ops.rs:833-843).
#include "common.cuh"
#include "internal.h"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, kThreads = 256;

__global__ void __launch_bounds__(kThreads) sgemm_kernel(SgemmParams p) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    int bz = blockIdx.z;
    long long bo = bz / p.batch_inner, bi = bz % p.batch_inner;
    const float *A = p.a + bo * p.a_bo + bi * p.a_bi;
    const float *B = p.b + bo * p.b_bo + bi * p.b_bi;
    float *C = p.c + bo * p.c_bo + bi * p.c_bi;
    int tid = threadIdx.x;
    int tx = tid % (BN / TN), ty = tid / (BN / TN);
    long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;
    // split reduction (single problems that would fill only a few SMs): slice blockIdx.z of the k range, partial result to a
    // workspace of p.splits [m, n] matrices that sgemm_reduce_kernel adds in slice order
    long long k_begin = 0, k_end = p.k;
    if (p.splits > 1) {
        const long long per = ((p.k + p.splits - 1) / p.splits + BK - 1) / BK * BK;
        k_begin = (long long)bz * per;
        k_end = k_begin + per < p.k ? k_begin + per : p.k;
        A = p.a;
        B = p.b;
        C = p.ws + (long long)bz * p.m * p.n;
    }
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    bool a_k_contig = (p.as1 == 1), b_n_contig = (p.bs1 == 1);
    for (long long k0 = k_begin; k0 < k_end; k0 += BK) {
#pragma unroll
        for (int l = 0; l < (BM * BK) / kThreads; ++l) {
            int e = tid + l * kThreads;
            int i, d;
            if (a_k_contig) { d = e % BK; i = e / BK; } else { i = e % BM; d = e / BM; }
            long long gi = m0 + i, gd = k0 + d;
            As[d][i] = (gi < p.m && gd < k_end) ? A[gi * p.as0 + gd * p.as1] : 0.0f;
        }
#pragma unroll
        for (int l = 0; l < (BN * BK) / kThreads; ++l) {
            int e = tid + l * kThreads;
            int j, d;
            if (b_n_contig) { j = e % BN; d = e / BN; } else { d = e % BK; j = e / BK; }
            long long gj = n0 + j, gd = k0 + d;
            Bs[d][j] = (gj < p.n && gd < k_end) ? B[gd * p.bs0 + gj * p.bs1] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int d = 0; d < BK; ++d) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[d][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[d][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        long long gi = m0 + ty * TM + i;
        if (gi >= p.m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            long long gj = n0 + tx * TN + j;
            if (gj >= p.n) continue;
            if (p.splits > 1) { // raw partial sum; scale, bias and activation follow the reduction
                C[gi * p.n + gj] = acc[i][j];
                continue;
            }
            float v = acc[i][j] * p.alpha;
            if (p.bias) v += p.bias[gj];
            if (p.act == MCB_ACT_RELU) v = v > 0.0f ? v : 0.0f;
            else if (p.act == MCB_ACT_GELU) {
                float v3 = v * v * v;
                v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v3)));
            }
            float *dst = C + gi * p.ldc + gj;
            *dst = p.accumulate ? (*dst + v) : v;
        }
    }
}

__global__ void sgemm_reduce_kernel(SgemmParams p) {
    long long total = p.m * p.n;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        float v = 0.0f;
        for (int s = 0; s < p.splits; ++s) v += p.ws[(long long)s * total + i]; // fixed order: same bits every run
        v *= p.alpha;
        const long long gi = i / p.n, gj = i - gi * p.n;
        if (p.bias) v += p.bias[gj];
        if (p.act == MCB_ACT_RELU) v = v > 0.0f ? v : 0.0f;
        else if (p.act == MCB_ACT_GELU) {
            float v3 = v * v * v;
            v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v3)));
        }
        float *dst = p.c + gi * p.ldc + gj;
        *dst = p.accumulate ? (*dst + v) : v;
    }
}

} // namespace

mcb_status mcb_sgemm(mcb_ctx *ctx, const SgemmParams &p_in) {
    SgemmParams p = p_in;
    if (p.m == 0 || p.n == 0 || p.batch == 0) return MCB_OK;
    if (p.batch > 65535) return mcb_fail(ctx, MCB_UNSUPPORTED, "sgemm batch > 65535");
    ProfScope prof(ctx, MCB_PROF_GEMM_F32, 2.0 * (double)p.m * (double)p.n * (double)p.k * (double)p.batch,
                   4.0 * (double)p.batch * ((double)p.m * p.k + (double)p.n * p.k + (double)p.m * p.n));
    dim3 grid((unsigned)((p.n + BN - 1) / BN), (unsigned)((p.m + BM - 1) / BM), (unsigned)p.batch);
    // A single skinny product (a classifier head, a weight gradient with few rows) would occupy a handful of SMs for the
    // whole reduction: cut the reduction into slices, one block each, and add the slices afterwards in a fixed order.
    const long long tiles = (long long)grid.x * grid.y;
    p.splits = 1;
    if (p.batch == 1 && tiles * 2 <= ctx->sm_count && p.k >= 512 && !knob_on(ctx, K_SGEMM_NO_SPLIT)) {
        long long s = (2ll * ctx->sm_count) / tiles;
        if (s > p.k / 128) s = p.k / 128;
        if (s > 64) s = 64;
        if (s >= 2) {
            void *ws;
            MCB_TRY(mcb_scratch(ctx, sizeof(float) * (size_t)s * (size_t)p.m * (size_t)p.n, &ws));
            p.splits = (int)s;
            p.ws = (float *)ws;
            grid.z = (unsigned)s;
        }
    }
    sgemm_kernel<<<grid, kThreads, 0, ctx->stream>>>(p);
    MCB_LAUNCHED(ctx);
    if (p.splits > 1) {
        sgemm_reduce_kernel<<<mcb_grid_for(ctx, p.m * p.n, 256, 4), 256, 0, ctx->stream>>>(p);
        MCB_LAUNCHED(ctx);
    }
    return MCB_OK;
}

static SgemmParams plain(const float *a, long long as0, long long as1, const float *b, long long bs0, long long bs1,
                         float *c, long long m, long long n, long long k) {
    SgemmParams p;
    p.a = a; p.b = b; p.c = c;
    p.m = m; p.n = n; p.k = k;
    p.as0 = as0; p.as1 = as1; p.bs0 = bs0; p.bs1 = bs1; p.ldc = n;
    return p;
}

extern "C" {

mcb_status mcb_matmul(mcb_ctx *ctx, const float *a, const float *b, float *c, int64_t m, int64_t k, int64_t n) {
    MCB_CHECK_CTX(ctx);
    if (k == 0) return mcb_memset(ctx, c, 0, sizeof(float) * m * n);
    return mcb_sgemm(ctx, plain(a, k, 1, b, n, 1, c, m, n, k));
}

mcb_status mcb_linear(mcb_ctx *ctx, const float *x, const float *w, const float *bias, float *y, int64_t m,
                      int64_t k, int64_t n, int32_t act) {
    MCB_CHECK_CTX(ctx);
    SgemmParams p = plain(x, k, 1, w, 1, k, y, m, n, k);
    p.bias = bias;
    p.act = act;
    return mcb_sgemm(ctx, p);
}

mcb_status mcb_linear_backward(mcb_ctx *ctx, const float *g, const float *x, const float *w, float *dx, float *dw,
                               float *db, int64_t m, int64_t k, int64_t n) {
    MCB_CHECK_CTX(ctx);
    if (dx) MCB_TRY(mcb_sgemm(ctx, plain(g, n, 1, w, k, 1, dx, m, k, n)));      // dx[m,k] = g[m,n] w[n,k]
    if (dw) MCB_TRY(mcb_sgemm(ctx, plain(g, 1, n, x, k, 1, dw, n, k, m)));      // dw[n,k] = g^T[n,m] x[m,k]
    if (db) MCB_TRY(mcb_col_sum(ctx, g, MCB_F32, m, n, db));
    return MCB_OK;
}

} // extern "C"
