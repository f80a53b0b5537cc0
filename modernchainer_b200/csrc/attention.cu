// Multi-head attention forward / backward on the device (the reference runs this as a
// single-threaded host loop on every backend, autograd/src/host_ops.rs:779-968).
//
// Layout: q, k, v, out, grads are [n, seq, dim] with head h in columns h*hd .. (h+1)*hd.
// The probabilities P[n, heads, seq, seq] are materialised in f32 scratch: scores by a
// strided batched GEMM that reads the heads where they lie, a row softmax with the causal
// mask and the 1/sqrt(hd) scale fused, then P V.  Backward recomputes P the same way.
// bf16 tensors are widened to f32 scratch first, so both storage types share one exact-f32
// arithmetic path.
#include "common.cuh"
#include "internal.h"

namespace {

// in-place: row <- softmax(scale * row) over unmasked keys; masked entries become exactly 0.
// lse (optional) receives max + log(sum) of the scaled scores.
__global__ void attn_softmax_kernel(float *__restrict__ p, float *__restrict__ lse, int seq, float scale, int causal) {
    __shared__ float red[32];
    long long row = blockIdx.x; // (n*heads + h)*seq + q
    int q = (int)(row % seq);
    float *r = p + row * seq;
    int limit = causal ? q + 1 : seq;
    float mx = -INFINITY;
    for (int j = threadIdx.x; j < limit; j += blockDim.x) mx = fmaxf(mx, r[j] * scale);
    mx = block_max(mx, red);
    float sum = 0.0f;
    for (int j = threadIdx.x; j < limit; j += blockDim.x) sum += expf(r[j] * scale - mx);
    sum = block_sum(sum, red);
    for (int j = threadIdx.x; j < seq; j += blockDim.x) r[j] = (j < limit) ? expf(r[j] * scale - mx) / sum : 0.0f;
    if (lse && threadIdx.x == 0) lse[row] = mx + logf(sum);
}

// in-place on dp: ds = p * (dp - sum_k p*dp)
__global__ void attn_dsoftmax_kernel(const float *__restrict__ p, float *__restrict__ dp, int seq) {
    __shared__ float red[32];
    long long row = blockIdx.x;
    const float *pr = p + row * seq;
    float *dr = dp + row * seq;
    float dot = 0.0f;
    for (int j = threadIdx.x; j < seq; j += blockDim.x) dot += pr[j] * dr[j];
    dot = block_sum(dot, red);
    for (int j = threadIdx.x; j < seq; j += blockDim.x) dr[j] = pr[j] * (dr[j] - dot);
}

struct Tmp {
    mcb_ctx *ctx;
    std::vector<void *> ptrs;
    explicit Tmp(mcb_ctx *c) : ctx(c) {}
    ~Tmp() {
        for (void *p : ptrs) mcb_free(ctx, p);
    }
    mcb_status get(size_t bytes, void **out) {
        mcb_status s = mcb_alloc(ctx, bytes, out);
        if (s == MCB_OK) ptrs.push_back(*out);
        return s;
    }
};

// returns an f32 view of `x` (widening bf16 into scratch when needed)
mcb_status as_f32(mcb_ctx *ctx, Tmp &tmp, const void *x, int dt, long long n, const float **out) {
    if (dt == MCB_F32) {
        *out = (const float *)x;
        return MCB_OK;
    }
    void *buf;
    MCB_TRY(tmp.get(sizeof(float) * n, &buf));
    MCB_TRY(mcb_cast(ctx, x, dt, buf, MCB_F32, n));
    *out = (const float *)buf;
    return MCB_OK;
}

SgemmParams head_gemm(long long n, long long heads, long long seq, long long dim) {
    SgemmParams p;
    p.batch = n * heads;
    p.batch_inner = heads;
    (void)seq;
    (void)dim;
    return p;
}

mcb_status probs(mcb_ctx *ctx, const float *q, const float *k, float *P, float *lse, long long n, long long seq,
                 long long dim, long long heads, int causal) {
    long long hd = dim / heads;
    SgemmParams p = head_gemm(n, heads, seq, dim);
    p.a = q; p.b = k; p.c = P;
    p.m = seq; p.n = seq; p.k = hd;
    p.as0 = dim; p.as1 = 1;       // Q[i, d]
    p.bs0 = 1; p.bs1 = dim;       // K^T[d, j] = K[j, d]
    p.ldc = seq;
    p.a_bo = seq * dim; p.a_bi = hd;
    p.b_bo = seq * dim; p.b_bi = hd;
    p.c_bo = heads * seq * seq; p.c_bi = seq * seq;
    MCB_TRY(mcb_sgemm(ctx, p));
    float scale = 1.0f / sqrtf((float)hd);
    int threads = seq >= 512 ? 256 : (seq >= 64 ? 64 : 32);
    attn_softmax_kernel<<<(unsigned)(n * heads * seq), threads, 0, ctx->stream>>>(P, lse, (int)seq, scale, causal);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

} // namespace

extern "C" {

mcb_status mcb_attention(mcb_ctx *ctx, const void *q, const void *k, const void *v, void *out, float *lse, int64_t n,
                         int64_t seq, int64_t dim, int64_t heads, int32_t causal, int32_t dt) {
    MCB_CHECK_CTX(ctx);
    if (heads <= 0 || dim % heads != 0) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "attention dimension must divide heads");
    if (dt != MCB_F32 && !mcb_is_lp(dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "attention supports f32, bf16 and f16");
    if (n == 0 || seq == 0 || dim == 0) return MCB_OK;
    long long hd = dim / heads, total = n * seq * dim;
    // algorithmic flops: 4 N H S^2 hd forward, 10 N H S^2 hd backward (halved under a causal mask)
    ProfScope prof(ctx, MCB_PROF_ATTENTION, 4.0 * (double)n * heads * seq * seq * hd * (causal ? 0.5 : 1.0),
                   (double)total * (mcb_is_lp(dt) ? 2.0 : 4.0) * 4.0);
    if (mcb_flash_supported(dim, heads, dt)) {
        void *lse_buf = lse;
        Tmp own(ctx);
        if (!lse_buf) MCB_TRY(own.get(sizeof(float) * n * heads * seq, &lse_buf));
        return mcb_flash_forward(ctx, q, k, v, out, (float *)lse_buf, n, seq, dim, heads, causal, dim, dim, dt);
    }
    Tmp tmp(ctx);
    const float *qf, *kf, *vf;
    MCB_TRY(as_f32(ctx, tmp, q, dt, total, &qf));
    MCB_TRY(as_f32(ctx, tmp, k, dt, total, &kf));
    MCB_TRY(as_f32(ctx, tmp, v, dt, total, &vf));
    void *P;
    MCB_TRY(tmp.get(sizeof(float) * n * heads * seq * seq, &P));
    MCB_TRY(probs(ctx, qf, kf, (float *)P, lse, n, seq, dim, heads, causal));
    float *of = (float *)out;
    void *obuf = nullptr;
    if (dt != MCB_F32) {
        MCB_TRY(tmp.get(sizeof(float) * total, &obuf));
        of = (float *)obuf;
    }
    SgemmParams p = head_gemm(n, heads, seq, dim);
    p.a = (const float *)P; p.b = vf; p.c = of;
    p.m = seq; p.n = hd; p.k = seq;
    p.as0 = seq; p.as1 = 1;
    p.bs0 = dim; p.bs1 = 1;
    p.ldc = dim;
    p.a_bo = heads * seq * seq; p.a_bi = seq * seq;
    p.b_bo = seq * dim; p.b_bi = hd;
    p.c_bo = seq * dim; p.c_bi = hd;
    MCB_TRY(mcb_sgemm(ctx, p));
    if (dt != MCB_F32) MCB_TRY(mcb_cast(ctx, of, MCB_F32, out, dt, total));
    return MCB_OK;
}

mcb_status mcb_attention_backward(mcb_ctx *ctx, const void *q, const void *k, const void *v, const void *out,
                                  const void *gout, const float *lse, void *dq, void *dk, void *dv, int64_t n,
                                  int64_t seq, int64_t dim, int64_t heads, int32_t causal, int32_t dt) {
    MCB_CHECK_CTX(ctx);
    (void)out;
    (void)lse;
    if (heads <= 0 || dim % heads != 0) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "attention dimension must divide heads");
    if (dt != MCB_F32 && !mcb_is_lp(dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "attention supports f32, bf16 and f16");
    if (n == 0 || seq == 0 || dim == 0) return MCB_OK;
    long long hd = dim / heads, total = n * seq * dim;
    // algorithmic flops: 4 N H S^2 hd forward, 10 N H S^2 hd backward (halved under a causal mask)
    ProfScope prof(ctx, MCB_PROF_ATTENTION, 10.0 * (double)n * heads * seq * seq * hd * (causal ? 0.5 : 1.0),
                   (double)total * (mcb_is_lp(dt) ? 2.0 : 4.0) * 8.0);
    if (mcb_flash_supported(dim, heads, dt) && out && lse)
        return mcb_flash_backward(ctx, q, k, v, out, gout, lse, dq, dk, dv, n, seq, dim, heads, causal, dim, dim, dim, nullptr, 0, nullptr, dt);
    float scale = 1.0f / sqrtf((float)hd);
    Tmp tmp(ctx);
    const float *qf, *kf, *vf, *gf;
    MCB_TRY(as_f32(ctx, tmp, q, dt, total, &qf));
    MCB_TRY(as_f32(ctx, tmp, k, dt, total, &kf));
    MCB_TRY(as_f32(ctx, tmp, v, dt, total, &vf));
    MCB_TRY(as_f32(ctx, tmp, gout, dt, total, &gf));
    void *P, *dP;
    MCB_TRY(tmp.get(sizeof(float) * n * heads * seq * seq, &P));
    MCB_TRY(tmp.get(sizeof(float) * n * heads * seq * seq, &dP));
    MCB_TRY(probs(ctx, qf, kf, (float *)P, nullptr, n, seq, dim, heads, causal));
    float *dqf = (float *)dq, *dkf = (float *)dk, *dvf = (float *)dv;
    if (dt != MCB_F32) {
        void *b;
        MCB_TRY(tmp.get(sizeof(float) * total, &b)); dqf = (float *)b;
        MCB_TRY(tmp.get(sizeof(float) * total, &b)); dkf = (float *)b;
        MCB_TRY(tmp.get(sizeof(float) * total, &b)); dvf = (float *)b;
    }
    long long pb_o = heads * seq * seq, pb_i = seq * seq, xb_o = seq * dim, xb_i = hd;
    // dP[q,k] = sum_d g[q,d] v[k,d]
    SgemmParams p = head_gemm(n, heads, seq, dim);
    p.a = gf; p.b = vf; p.c = (float *)dP;
    p.m = seq; p.n = seq; p.k = hd;
    p.as0 = dim; p.as1 = 1; p.bs0 = 1; p.bs1 = dim; p.ldc = seq;
    p.a_bo = xb_o; p.a_bi = xb_i; p.b_bo = xb_o; p.b_bi = xb_i; p.c_bo = pb_o; p.c_bi = pb_i;
    MCB_TRY(mcb_sgemm(ctx, p));
    // dV[k,d] = sum_q P[q,k] g[q,d]   (before dP is overwritten by dS; P is still intact)
    p = head_gemm(n, heads, seq, dim);
    p.a = (const float *)P; p.b = gf; p.c = dvf;
    p.m = seq; p.n = hd; p.k = seq;
    p.as0 = 1; p.as1 = seq; p.bs0 = dim; p.bs1 = 1; p.ldc = dim;
    p.a_bo = pb_o; p.a_bi = pb_i; p.b_bo = xb_o; p.b_bi = xb_i; p.c_bo = xb_o; p.c_bi = xb_i;
    MCB_TRY(mcb_sgemm(ctx, p));
    int threads = seq >= 512 ? 256 : (seq >= 64 ? 64 : 32);
    attn_dsoftmax_kernel<<<(unsigned)(n * heads * seq), threads, 0, ctx->stream>>>((const float *)P, (float *)dP, (int)seq);
    MCB_LAUNCHED(ctx);
    // dQ[q,d] = scale * sum_k dS[q,k] K[k,d]
    p = head_gemm(n, heads, seq, dim);
    p.a = (const float *)dP; p.b = kf; p.c = dqf;
    p.m = seq; p.n = hd; p.k = seq;
    p.as0 = seq; p.as1 = 1; p.bs0 = dim; p.bs1 = 1; p.ldc = dim;
    p.a_bo = pb_o; p.a_bi = pb_i; p.b_bo = xb_o; p.b_bi = xb_i; p.c_bo = xb_o; p.c_bi = xb_i;
    p.alpha = scale;
    MCB_TRY(mcb_sgemm(ctx, p));
    // dK[k,d] = scale * sum_q dS[q,k] Q[q,d]
    p.a = (const float *)dP; p.b = qf; p.c = dkf;
    p.as0 = 1; p.as1 = seq;
    MCB_TRY(mcb_sgemm(ctx, p));
    if (dt != MCB_F32) {
        MCB_TRY(mcb_cast(ctx, dqf, MCB_F32, dq, dt, total));
        MCB_TRY(mcb_cast(ctx, dkf, MCB_F32, dk, dt, total));
        MCB_TRY(mcb_cast(ctx, dvf, MCB_F32, dv, dt, total));
    }
    return MCB_OK;
}

} // extern "C"
