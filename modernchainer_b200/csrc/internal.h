// Prototypes shared between the translation units of the library (not part of the C ABI).
#pragma once
#include "common.cuh"

// Strided / batched exact-f32 GEMM:
//   C[z][i*ldc + j] (+)= alpha * sum_d A[z][i*as0 + d*as1] * B[z][d*bs0 + j*bs1] (+ bias[j]) -> act
// Batch index z in [0, batch) is split as (z / batch_inner, z % batch_inner) with separate
// strides, so a [n, seq, heads*hd] tensor can be walked per (sample, head) without a copy.
struct SgemmParams {
    const float *a = nullptr, *b = nullptr;
    float *c = nullptr;
    const float *bias = nullptr;
    long long m = 0, n = 0, k = 0;
    long long as0 = 0, as1 = 0, bs0 = 0, bs1 = 0, ldc = 0;
    long long batch = 1, batch_inner = 1;
    long long a_bo = 0, a_bi = 0, b_bo = 0, b_bi = 0, c_bo = 0, c_bi = 0;
    float alpha = 1.0f;
    int act = MCB_ACT_NONE;
    int accumulate = 0;
    // set by mcb_sgemm, not by callers: reduction slices and their workspace (splits x [m, n])
    int splits = 1;
    float *ws = nullptr;
};
mcb_status mcb_sgemm(mcb_ctx *ctx, const SgemmParams &p);

// Tensor-core GEMM with explicit leading dimensions and (sample, head) batching; see gemm_tc.cu.
struct TcGemmParams {
    const void *a = nullptr, *b = nullptr; // both of type in_dt
    int in_dt = MCB_BF16;                  // MCB_BF16 or MCB_F16
    void *d = nullptr;
    const float *bias = nullptr;
    int a_mn_major = 0, b_mn_major = 0;
    int out_dt = MCB_BF16; // MCB_F32 or in_dt
    long long m = 0, n = 0, k = 0;
    long long lda = 0, ldb = 0, ldd = 0; // elements between consecutive rows of the stored matrices
    int accumulate = 0;
    int split_k = 1;
    int bn = 0; // tile width 128 / 192 / 256, 0 = choose
    int pair = -1; // 1 = two CTAs share a 256-row tile (cta_group::2), 0 = one CTA per 128-row tile, -1 = choose
    int act = MCB_ACT_NONE;
    void *d_pre = nullptr; // optional second output: value before the activation (same dtype/ld as d)
    // optional side job: fill zero_bytes (a multiple of 16) at zero_ptr (16-byte aligned) with zeros while the first tiles are
    // in flight (the epilogue warps have nothing to do until then).  The tape uses it to clear the output of the split
    // weight-gradient GEMM that follows a data-gradient GEMM, instead of a fill of its own.
    void *zero_ptr = nullptr;
    size_t zero_bytes = 0;
    int split_tail = -1;   // 1 = cut the tiles of a mostly empty last wave along K (f32 workspace + finishing kernel), 0 = never, -1 = choose
};
mcb_status mcb_tc_gemm(mcb_ctx *ctx, const TcGemmParams &p);
// tile width and reduction split for an [m, n] output reduced over k (see gemm_tc.cu)
void mcb_tc_plan(mcb_ctx *ctx, int64_t m, int64_t n, int64_t k, bool allow_split, bool atomic_out, int fixed_split, int *bn_out,
                 int *split_out);

// flash_attn.cu: fused bf16 attention, head_dim 64
bool mcb_flash_supported(int64_t dim, int64_t heads, int32_t dt);
mcb_status mcb_flash_forward(mcb_ctx *ctx, const void *q, const void *k, const void *v, void *out, float *lse, int64_t n, int64_t seq,
                             int64_t dim, int64_t heads, int32_t causal, int64_t ldi, int64_t ldo, int32_t dt = MCB_BF16);
// bias_partial (optional): see mcb_flash_tc_backward; *bias_done says whether it was filled
mcb_status mcb_flash_backward(mcb_ctx *ctx, const void *q, const void *k, const void *v, const void *out, const void *gout, const float *lse,
                              void *dq, void *dk, void *dv, int64_t n, int64_t seq, int64_t dim, int64_t heads, int32_t causal,
                              int64_t ldi, int64_t ldo, int64_t ldg, float *bias_partial = nullptr, int64_t bias_ld = 0, int *bias_done = nullptr,
                              int32_t dt = MCB_BF16); // dt: MCB_BF16 or MCB_F16, the type of every 16-bit tensor of the call
// flash_tc.cu: the same forward on tcgen05 / TMEM; MCB_UNSUPPORTED (nothing launched) outside its range
mcb_status mcb_flash_tc_forward(mcb_ctx *ctx, const void *q, const void *k, const void *v, void *out, float *lse, int64_t n, int64_t seq,
                                int64_t dim, int64_t heads, int32_t causal, int64_t ldi, int64_t ldo, int32_t dt = MCB_BF16);
// flash_tc_bwd.cu: dq, dk, dv on tcgen05 / TMEM; `delta` = rowsum(O * dO) per (sample, head, row)
mcb_status mcb_flash_tc_backward(mcb_ctx *ctx, const void *q, const void *k, const void *v, const void *gout, const float *lse, const float *delta,
                                 void *dq, void *dk, void *dv, int64_t n, int64_t seq, int64_t dim, int64_t heads, int32_t causal, int64_t ldi,
                                 int64_t ldo, int64_t ldg, float *bias_partial = nullptr, int64_t bias_ld = 0, int32_t dt = MCB_BF16);
// rows of the bias by-product of mcb_flash_tc_backward: [mcb_flash_bias_rows(n, seq)][bias_ld] partial column sums of dq | dk | dv
// (columns 0, dim, 2 dim); 0 when the tcgen05 kernels would decline the shape
int64_t mcb_flash_bias_rows(int64_t n, int64_t seq);
// layer_norm_fast.cu: register-resident rows; MCB_UNSUPPORTED (nothing launched) outside their range
mcb_status mcb_ln_fast_forward(mcb_ctx *ctx, const float *x, const float *gamma, const float *beta, double eps, void *out, int32_t out_dt,
                               float *mean, float *rstd, int64_t rows, int64_t dim);
mcb_status mcb_ln_fast_backward(mcb_ctx *ctx, const float *x, const float *gamma, const void *g, int32_t g_dt, double eps, const float *mean,
                                const float *rstd, const float *addend, float *dx, float *dgamma, float *dbeta, int64_t rows, int64_t dim);
// layer_norm_bulk.cu: the same two passes as a persistent bulk-copy pipeline through shared memory, for
// problems with enough rows to fill every SM; MCB_UNSUPPORTED (nothing launched) otherwise
mcb_status mcb_ln_bulk_forward(mcb_ctx *ctx, const float *x, const float *gamma, const float *beta, double eps, void *out, int32_t out_dt,
                               float *mean, float *rstd, int64_t rows, int64_t dim);
// sum = x + res (res f32 or bf16) and out = LayerNorm(sum) in one pass
mcb_status mcb_ln_bulk_add_forward(mcb_ctx *ctx, const float *x, const void *res, int32_t res_dt, const float *gamma, const float *beta, double eps,
                                   float *sum, void *out, int32_t out_dt, float *mean, float *rstd, int64_t rows, int64_t dim);
// dx_bf16 / dx_colsum (both or neither): also leaves dx rounded to bf16 and the column sums of those rounded values
mcb_status mcb_ln_bulk_backward(mcb_ctx *ctx, const float *x, const float *gamma, const void *g, int32_t g_dt, double eps, const float *mean,
                                const float *rstd, const float *addend, float *dx, float *dgamma, float *dbeta, int64_t rows, int64_t dim,
                                void *dx_bf16 = nullptr, float *dx_colsum = nullptr, int32_t aux_dt = MCB_BF16); // aux_dt: 16-bit format of dx_bf16
// reduce.cu: LayerNorm backward that writes dx as addend + dx when `addend` is given (may alias dx);
// MCB_UNSUPPORTED (nothing launched) where only the plain form exists
mcb_status mcb_layer_norm_backward_ex(mcb_ctx *ctx, const float *x, const float *gamma, const void *g, int32_t g_dt, double eps,
                                      const float *mean, const float *rstd, const float *addend, float *dx, float *dgamma,
                                      float *dbeta, int64_t rows, int64_t dim);
// conv_tc.cu: convolution as column matrix + tensor-core GEMMs at f32 accuracy (f16 hi/lo pieces); _eligible says whether a
// problem is large and regular enough for it
bool mcb_conv_tc_eligible(mcb_ctx *ctx, int64_t n, int64_t c, int64_t h, int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride, int64_t pad);
mcb_status mcb_conv_tc_forward(mcb_ctx *ctx, const float *x, const float *w, const float *bias, float *out, int64_t n, int64_t c, int64_t h,
                               int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride, int64_t pad);
mcb_status mcb_conv_tc_backward(mcb_ctx *ctx, const float *x, const float *w, const float *g, float *dx, float *dw, int64_t n, int64_t c, int64_t h,
                                int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride, int64_t pad);
// reduce.cu: row softmax (mode 0), its backward from x (1) or from the forward's output y (2)
mcb_status mcb_softmax_rows(mcb_ctx *ctx, int mode, const float *a, const float *b, float *out, int64_t rows, int64_t cols);
// reduce.cu
mcb_status mcb_sce_grad(mcb_ctx *ctx, const void *logits, void *out, int32_t dt, const void *labels, int32_t label_dt,
                        int64_t n, int64_t c, float *loss_out, const float *upstream, float *stats_out = nullptr,
                        const float *stats_in = nullptr); // stats: [n][2] row maximum and sum of exp, passed from the loss pass to the gradient pass
mcb_status mcb_sum_scaled(mcb_ctx *ctx, const float *x, int64_t n, double scale, float *out);
// elementwise.cu
// out[i] = (*scalar) * factor for all i (broadcast of a device scalar)
mcb_status mcb_fill_from_scalar(mcb_ctx *ctx, float *out, const float *scalar, double factor, int64_t n);
// out = x * (*scalar); x/out f32 or bf16
mcb_status mcb_mul_scalar_ptr(mcb_ctx *ctx, const void *x, const float *scalar, void *out, int64_t n, int32_t dt);
// out = a + b with per-operand storage types (f32 or bf16), same shape
mcb_status mcb_add_typed(mcb_ctx *ctx, const void *a, int32_t a_dt, const void *b, int32_t b_dt, void *out, int32_t out_dt, int64_t n);
// one pass producing a bf16 [rows, cols] matrix and its column sums (of the rounded values):
// mode 0: out = bf16(a), a f32;  mode 1: out = gelu'(a) * b;  mode 2: out = relu'(a) * b (a, b bf16).
// Returns MCB_UNSUPPORTED (nothing launched) unless cols % 8 == 0 and all pointers are 16-byte aligned.
mcb_status mcb_map_colsum(mcb_ctx *ctx, int mode, const void *a, const void *b, void *out_bf16, int64_t rows, int64_t cols,
                          float *colsum_out, int32_t lp_dt = MCB_BF16); // lp_dt: the 16-bit type of out (and of a, b in modes 1, 2)
bool mcb_map_colsum_supported(const void *a, const void *b, const void *out, int64_t cols);
// reduce.cu: out[col] = sum of `parts` rows of partial[parts, cols], fixed order
mcb_status mcb_partial_sum_final(mcb_ctx *ctx, const float *partial, int parts, int64_t cols, float *out);
// optim.cu
mcb_status mcb_adam_flat_ex(mcb_ctx *ctx, float *p, const void *g, int32_t g_dt, float *m, float *v, void *p_bf16,
                            int64_t n, double lr, double beta1, double beta2, double eps, int32_t step,
                            double inv_scale, const float *inv_scale_dev, const int32_t *skip_flag, const int32_t *step_dev);
// any optimizer of the family (MCB_OPT_*) as one fused in-place pass; see optim.cu
mcb_status mcb_opt_flat(mcb_ctx *ctx, int32_t kind, float *p, const void *g, int32_t g_dt, float *m, float *v, void *p_bf16, int64_t n,
                        double lr, double beta1, double beta2, double eps, double weight_decay, int32_t step, double inv_scale,
                        const float *inv_scale_dev, const int32_t *skip_flag, const int32_t *step_dev,
                        int32_t shadow_dt = MCB_BF16); // shadow_dt: format of the 16-bit parameter copy p_bf16 (MCB_BF16 or MCB_F16)
// *counter += 1 on the stream (device-resident step count of a replayed graph without a GradScaler)
mcb_status mcb_increment_i32(mcb_ctx *ctx, int32_t *counter);
// runtime.cu: blocks owned by a released static step go back to the general pool
extern "C" void mcb_release_capture_blocks(mcb_ctx *ctx, int capture_id);
// global-norm clipping in three launches: per-block sums of squares (f64), {norm, factor}, conditional scale
int mcb_sumsq_blocks(mcb_ctx *ctx, int64_t n);
mcb_status mcb_sumsq_partial(mcb_ctx *ctx, const float *g, int64_t n, double *partial, int blocks);
mcb_status mcb_clip_finalize(mcb_ctx *ctx, const double *partial, int count, double max_norm, double *out2, double mean_factor = 1.0);
mcb_status mcb_scale_by_clip(mcb_ctx *ctx, float *g, int64_t n, const double *clip2);
// scaler state on the device: {scale, inv_scale} floats then {growth_tracker, found_inf, last_found_inf, applied_steps} ints
mcb_status mcb_scaler_update(mcb_ctx *ctx, float *state_f, int *state_i, float growth, float backoff, int interval);
