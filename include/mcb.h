/*
 * mcb.h -- C ABI of the B200 (sm_100a) training-step backend for ModernChainer.
 *
 * The library replaces the CUDA backend's kernel layer (NVRTC kernel string +
 * cuBLAS/cuBLASLt call sites) and the host logic above it that made a fast
 * path impossible (tape walker accumulation, per-tensor Adam, host-side
 * inf/nan scan).  Three groups of entry points:
 *
 *   1. runtime        -- context, stream, caching allocator, copies, error word
 *                        (replaces CudaRuntime / CudaPool / CudaStorage,
 *                        crates/modern-chainer-cuda/src/backend.rs:138-191,269-451)
 *   2. ops            -- one function per `Ops<CudaBackend>` method on the training
 *                        path, raw device pointers + extents
 *                        (trait: crates/modern-chainer-core/src/storage.rs:31-414,
 *                        CUDA impl: crates/modern-chainer-cuda/src/ops.rs:600-1925)
 *   3. tape / optim   -- handles that mirror `Variable`, `F::*`, `Optimizer`,
 *                        `GradScaler` and the nn modules, so a binding can forward
 *                        the reference's public API call-for-call
 *                        (crates/modern-chainer-autograd/src/{variable,node,ops,host_ops}.rs,
 *                        crates/modern-chainer-optim/src/{lib,amp}.rs,
 *                        crates/modern-chainer-nn/src/lib.rs)
 *
 * Conventions: every function returns an mcb_status (0 = ok; codes map 1:1 onto
 * the variants of core::Error, crates/modern-chainer-core/src/error.rs:8-40) and
 * records a message retrievable with mcb_last_error().  All tensors are
 * contiguous row-major.  Pointers are DEVICE pointers unless a parameter name
 * starts with `host_`.  The library borrows caller buffers for the duration of
 * the enqueue only.  All work is enqueued on the context's stream and returns
 * immediately; faults found on the device (label / token id out of range) are
 * written to an error word that the next synchronising call (mcb_sync,
 * mcb_memcpy_d2h, mcb_var_* read-backs) returns as MCB_INVALID_ARGUMENT.
 * There is no CPU fallback: every compute entry point fails with MCB_BACKEND
 * when no CUDA device is usable.
 */
#ifndef MCB_H
#define MCB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t mcb_status;
enum {
    MCB_OK = 0,
    MCB_SHAPE_MISMATCH = 1,
    MCB_BROADCAST = 2,
    MCB_DTYPE_MISMATCH = 3,
    MCB_UNSUPPORTED_DTYPE = 4,
    MCB_INVALID_ARGUMENT = 5,
    MCB_OUT_OF_BOUNDS = 6,
    MCB_UNSUPPORTED = 7,
    MCB_BACKEND = 8,
    MCB_IO = 9
};

/* crates/modern-chainer-core/src/dtype.rs:4-13 */
enum { MCB_F32 = 0, MCB_I64 = 1, MCB_I32 = 2, MCB_U8 = 3, MCB_F16 = 4, MCB_BF16 = 5 };

/* GEMM arithmetic (ComputeType, crates/modern-chainer-cuda/src/backend.rs:109-136).
 * MCB_COMPUTE_F32: exact-f32 FMA kernel.  MCB_COMPUTE_BF16 / MCB_COMPUTE_F16: tcgen05
 * tensor-core kernel, operands rounded to nearest even to bf16 / IEEE f16, f32 accumulate
 * in TMEM (the reference's ComputeType::Bf16 / ::F16; its Tf32 default has no counterpart:
 * MCB_COMPUTE_F32 is exact). */
enum { MCB_COMPUTE_F32 = 0, MCB_COMPUTE_BF16 = 1, MCB_COMPUTE_F16 = 2 };

enum { MCB_ADD = 0, MCB_SUB = 1, MCB_MUL = 2, MCB_DIV = 3 };
enum { MCB_EXP = 0, MCB_LOG = 1, MCB_SIGMOID = 2, MCB_SQRT = 3, MCB_SILU = 4, MCB_ABS = 5, MCB_NEG = 6 };
enum { MCB_ACT_NONE = 0, MCB_ACT_RELU = 1, MCB_ACT_GELU = 2 };

typedef struct mcb_ctx mcb_ctx;

/* ------------------------------------------------------------------ runtime */
/* CudaBackend::new(ordinal), crates/modern-chainer-cuda/src/backend.rs:460-468 */
mcb_status mcb_ctx_create(int32_t ordinal, mcb_ctx **out);
void mcb_ctx_destroy(mcb_ctx *ctx);
/* Test and tuning knobs.  Each has the name of an environment variable (MCB_DETERMINISTIC, MCB_UNFUSED_BWD,
 * MCB_CONV_DIRECT, MCB_TC_BN ...); the environment is read ONCE, when the context is created, and no entry point
 * reads it afterwards.  mcb_set_knob changes one knob of one context: value >= 0 sets it, value < 0 clears it.
 * MCB_DETERMINISTIC makes a step reproducible bit for bit from run to run: the embedding gradient is added in
 * position order (the order of crates/modern-chainer-cpu/src/kernels.rs:1783-1815) instead of by float atomics,
 * tensor-core GEMMs run without split reductions (whose slices meet the output in arrival order), and max-pool
 * gradients of overlapping windows are gathered per input element.  It costs time, not accuracy. */
mcb_status mcb_set_knob(mcb_ctx *ctx, const char *name, int32_t value);
const char *mcb_last_error(mcb_ctx *ctx);
/* number of usable CUDA devices (0 when the driver is missing); probe(), cuda/src/lib.rs:54-66 */
int32_t mcb_device_count(void);
/* CudaPool allocate / Drop, backend.rs:13-107,401-431: size-bucketed free lists */
mcb_status mcb_alloc(mcb_ctx *ctx, size_t bytes, void **out);
mcb_status mcb_free(mcb_ctx *ctx, void *ptr);
mcb_status mcb_host_alloc(size_t bytes, void **host_out); /* pinned host memory */
mcb_status mcb_host_free(void *host_ptr);
/* Tensor::from_bytes / to_bytes, backend.rs:269-399 */
mcb_status mcb_memcpy_h2d(mcb_ctx *ctx, void *dst, const void *host_src, size_t bytes);
mcb_status mcb_memcpy_d2h(mcb_ctx *ctx, void *host_dst, const void *src, size_t bytes); /* synchronises */
mcb_status mcb_memcpy_d2h_async(mcb_ctx *ctx, void *host_dst, const void *src, size_t bytes);
mcb_status mcb_memcpy_d2d(mcb_ctx *ctx, void *dst, const void *src, size_t bytes);
mcb_status mcb_memset(mcb_ctx *ctx, void *dst, int32_t byte, size_t bytes);
/* CudaBackend::synchronize, backend.rs:478-483; also returns and clears the device error word */
mcb_status mcb_sync(mcb_ctx *ctx);
void *mcb_stream(mcb_ctx *ctx); /* the cudaStream_t all work is enqueued on */
int64_t mcb_launch_count(mcb_ctx *ctx); /* kernels launched by this library on this context so far */
int64_t mcb_allocated_bytes(mcb_ctx *ctx);
/* device-side timing on the context's stream */
mcb_status mcb_event_create(mcb_ctx *ctx, void **event_out);
mcb_status mcb_event_record(mcb_ctx *ctx, void *event);
mcb_status mcb_event_elapsed_ms(mcb_ctx *ctx, void *start, void *stop, float *ms_out); /* synchronises on stop */
mcb_status mcb_event_destroy(mcb_ctx *ctx, void *event);
/* Per-kernel-class device timing for benchmarks (no counterpart in the reference, which times
 * with Instant + synchronize, crates/modern-chainer/examples/cuda_bench.rs:6-33).  While enabled,
 * every launch group is bracketed by two events on the context's stream.  mcb_prof_read
 * synchronises and returns, for one class, the launch groups seen, their summed device time and
 * the algorithmic flops / bytes they were booked with. */
enum { MCB_PROF_GEMM_TC = 0, MCB_PROF_GEMM_F32 = 1, MCB_PROF_ATTENTION = 2, MCB_PROF_OPTIMIZER = 3,
       MCB_PROF_NORM = 4, MCB_PROF_LOSS = 5, MCB_PROF_ELEMENTWISE = 6, MCB_PROF_REDUCE = 7, MCB_PROF_EMBEDDING = 8,
       MCB_PROF_CONV = 9, MCB_PROF_CLASSES = 10 };
mcb_status mcb_prof_enable(mcb_ctx *ctx, int32_t on); /* enabling also clears earlier records */
mcb_status mcb_prof_read(mcb_ctx *ctx, int32_t klass, int64_t *launches_out, double *ms_out, double *flops_out,
                         double *bytes_out);
/* SM clock trace for benchmarks (no counterpart in the reference).  _start launches a one-thread
 * sampler on a stream of its own that records (wall-clock ns, SM cycle counter) every interval_us
 * for duration_us (at most 5 s) and then ends by itself; kernels launched meanwhile on the
 * context's stream run beside it.  _read waits for the sampler and returns the SM clock in MHz
 * between consecutive samples (up to max_out values). */
mcb_status mcb_clock_trace_start(mcb_ctx *ctx, int32_t duration_us, int32_t interval_us);
mcb_status mcb_clock_trace_read(mcb_ctx *ctx, double *mhz_out, int32_t max_out, int32_t *n_out);
/* CudaBackend::set_compute_type, backend.rs:489-497 */
mcb_status mcb_set_compute_type(mcb_ctx *ctx, int32_t compute);

/* ------------------------------------------------------------------ ops: elementwise */
/* Ops::add/sub/mul/div with NumPy broadcast, storage.rs:40-56; CUDA ops.rs:86-115,601-643 */
mcb_status mcb_binary(mcb_ctx *ctx, int32_t op, const float *a, const int64_t *a_dims, int32_t a_rank,
                      const float *b, const int64_t *b_dims, int32_t b_rank, float *out);
/* in-place gradient accumulation dst += src (replaces the out-of-place add of
 * autograd/src/variable.rs:196,212); dt = MCB_F32 or MCB_BF16 for both */
mcb_status mcb_add_inplace(mcb_ctx *ctx, void *dst, const void *src, int64_t n, int32_t dt);
/* Ops::scale, ops.rs:920-936: factor narrowed to f32 first */
mcb_status mcb_scale(mcb_ctx *ctx, const float *x, double factor, float *out, int64_t n);
mcb_status mcb_fill(mcb_ctx *ctx, float *out, float value, int64_t n); /* ones_like/full_like, ops.rs:938-952 */
mcb_status mcb_unary(mcb_ctx *ctx, int32_t op, const float *x, float *out, int64_t n); /* ops.rs:645-709 */
/* Ops::relu / relu_backward, ops.rs:649-659; dt selects f32 or bf16 storage for x, g, out */
mcb_status mcb_relu(mcb_ctx *ctx, const void *x, void *out, int64_t n, int32_t dt);
mcb_status mcb_relu_backward(mcb_ctx *ctx, const void *x, const void *g, void *out, int64_t n, int32_t dt);
/* Ops::gelu (ops.rs:665) and the fused backward that replaces the ~25-op chain of
 * autograd/src/ops.rs:646-676 */
mcb_status mcb_gelu(mcb_ctx *ctx, const void *x, void *out, int64_t n, int32_t dt);
mcb_status mcb_gelu_backward(mcb_ctx *ctx, const void *x, const void *g, void *out, int64_t n, int32_t dt);
/* Ops::cast, ops.rs:322-417; f32<->bf16/f16 with round-to-nearest-even (core/src/dtype.rs:75-150) */
mcb_status mcb_cast(mcb_ctx *ctx, const void *src, int32_t src_dt, void *dst, int32_t dst_dt, int64_t n);
/* Ops::transpose2d, storage.rs / cpu/src/kernels.rs:306-330: out[c, r] = a[r, c] for a [rows, cols] f32 matrix */
mcb_status mcb_transpose2d(mcb_ctx *ctx, const float *a, float *out, int64_t rows, int64_t cols);
/* permute_data, autograd/src/host_ops.rs:703-735: output dim d takes source axis axes[d]; axes must be a
 * permutation of 0..rank-1 ("invalid permute axes" otherwise), rank <= 8 */
mcb_status mcb_permute(mcb_ctx *ctx, const float *a, const int64_t *dims, int32_t rank, const int32_t *axes, float *out);

/* ------------------------------------------------------------------ ops: reductions */
/* Ops::sum_all, ops.rs:872-891: deterministic two-stage reduction, f64 final sum */
mcb_status mcb_sum_all(mcb_ctx *ctx, const float *x, int64_t n, float *out);
/* Ops::sum_to, ops.rs:893-918 (all shapes on device, including the bias path [rows,cols]->[cols]) */
mcb_status mcb_sum_to(mcb_ctx *ctx, const float *a, const int64_t *a_dims, int32_t a_rank, const int64_t *t_dims,
                      int32_t t_rank, float *out);
/* column sums of a [rows,cols] matrix stored as f32 or bf16, f32 result (bias gradient) */
mcb_status mcb_col_sum(mcb_ctx *ctx, const void *a, int32_t dt, int64_t rows, int64_t cols, float *out);
/* Ops::softmax_last_dim / _backward, ops.rs:1314-1374 */
mcb_status mcb_softmax(mcb_ctx *ctx, const float *x, float *out, int64_t rows, int64_t cols);
mcb_status mcb_softmax_backward(mcb_ctx *ctx, const float *x, const float *g, float *out, int64_t rows,
                                int64_t cols);
/* the same gradient from the forward's OUTPUT y instead of its input (what a tape that keeps y uses: no
 * exponentials, dx = y (g - sum(y g))) */
mcb_status mcb_softmax_backward_from_output(mcb_ctx *ctx, const float *y, const float *g, float *out, int64_t rows,
                                            int64_t cols);
/* Ops::layer_norm / layer_norm_backward, ops.rs:1200-1305.  x is f32; out_dt selects the
 * storage of the normalised output (f32, or bf16 when it only feeds a bf16 GEMM).
 * mean/rstd ([rows] f32, may be NULL) are saved by forward and reused by backward. */
mcb_status mcb_layer_norm(mcb_ctx *ctx, const float *x, const float *gamma, const float *beta, double eps, void *out,
                          int32_t out_dt, float *mean, float *rstd, int64_t rows, int64_t dim);
mcb_status mcb_layer_norm_backward(mcb_ctx *ctx, const float *x, const float *gamma, const void *g, int32_t g_dt,
                                   double eps, const float *mean, const float *rstd, float *dx, float *dgamma,
                                   float *dbeta, int64_t rows, int64_t dim);
/* LayerNorm backward for callers that must not allocate device memory.  It has no counterpart in
 * the reference.  Some hosts give a plugin a stream and a fixed set of buffers and rule out
 * cudaMalloc / cudaFree for good: a control loop with a latency budget, a process whose device
 * memory is carved up once at start-up, a section that is being recorded and may not touch the
 * address space.  mcb_layer_norm_backward is unusable there because its per-block partial sums of
 * dgamma / dbeta live in scratch memory the context allocates on demand.  This variant keeps those
 * partial sums in a 2 MiB array that is part of the library image (every GPU that loads the
 * library holds it until the process exits).  It takes no context, allocates nothing, and calls no
 * allocating routine.  It always runs the general row-sweeping kernel on at most 64 blocks (the
 * array has room for 64 partial results), not the pipelined kernels that mcb_layer_norm_backward
 * picks for most shapes: same results up to the order of the f32 partial sums, but at 8192 x 768 it
 * occupies fewer than half of the SMs.  It is for callers that cannot allocate, not a fast path.
 *   stream      the cudaStream_t to enqueue on; its device must be the current device
 *   arguments   as mcb_layer_norm_backward; mean / rstd may be NULL (recomputed from x)
 *   limit       dim <= 4096; larger dims return MCB_INVALID_ARGUMENT and enqueue nothing
 * The first call on each device looks up the array's device address and raises the kernel's
 * shared-memory limit; make that first call before any stream capture begins.  All calls share
 * the one array: two calls that can overlap on the GPU (different streams, no ordering between
 * them) race on it and must be serialised by the caller.  The array keeps whatever the previous
 * call left, which is harmless: each call overwrites every slot it later reads.
 * The message for a failed call is returned by mcb_noalloc_last_error() (per host thread). */
mcb_status mcb_layer_norm_backward_noalloc(void *stream, const float *x, const float *gamma, const void *g,
                                           int32_t g_dt, double eps, const float *mean, const float *rstd, float *dx,
                                           float *dgamma, float *dbeta, int64_t rows, int64_t dim);
const char *mcb_noalloc_last_error(void);
/* Ops::softmax_cross_entropy / _backward, ops.rs:1039-1119; labels I64, I32 or U8.
 * loss_out: one f32 on the device. */
mcb_status mcb_softmax_cross_entropy(mcb_ctx *ctx, const float *logits, const void *labels, int32_t label_dt,
                                     int64_t n, int64_t c, float *loss_out);
mcb_status mcb_softmax_cross_entropy_backward(mcb_ctx *ctx, const float *logits, const void *labels,
                                              int32_t label_dt, int64_t n, int64_t c, float *out);
/* fused forward+backward over one pass of the logits (f32 or bf16): writes the mean loss and
 * overwrites `logits` with (softmax - onehot) / n * (*upstream), `upstream` a device f32
 * (NULL = 1).  Replaces forward + backward + scale of autograd/src/ops.rs:328-350. */
mcb_status mcb_softmax_ce_fused(mcb_ctx *ctx, void *logits, int32_t logits_dt, const void *labels, int32_t label_dt,
                                int64_t n, int64_t c, float *loss_out, const float *upstream);
/* Ops::embedding / embedding_backward, ops.rs:1121-1198; ids I64, I32 or U8 */
mcb_status mcb_embedding(mcb_ctx *ctx, const void *ids, int32_t id_dt, int64_t n, const float *weight, int64_t vocab,
                         int64_t dim, float *out);
mcb_status mcb_embedding_backward(mcb_ctx *ctx, const void *ids, int32_t id_dt, int64_t n, const void *g,
                                  int32_t g_dt, int64_t vocab, int64_t dim, float *out, int32_t accumulate);

/* ------------------------------------------------------------------ ops: GEMM family */
/* Ops::matmul, ops.rs:711-760: c[m,n] = a[m,k] b[k,n] */
mcb_status mcb_matmul(mcb_ctx *ctx, const float *a, const float *b, float *c, int64_t m, int64_t k, int64_t n);
/* Ops::linear / linear_activation, ops.rs:762-831: y[m,n] = act(x[m,k] w[n,k]^T + bias[n]), f32 storage */
mcb_status mcb_linear(mcb_ctx *ctx, const float *x, const float *w, const float *bias, float *y, int64_t m,
                      int64_t k, int64_t n, int32_t act);
/* Ops::linear_backward / linear_backward_with_bias, ops.rs:833-843: any of dx, dw, db may be NULL */
mcb_status mcb_linear_backward(mcb_ctx *ctx, const float *g, const float *x, const float *w, float *dx, float *dw,
                               float *db, int64_t m, int64_t k, int64_t n);
/* The tensor-core GEMM behind the bf16 / f16 compute types (replaces mixed_linear / mixed_matmul,
 * ops.rs:419-597).  D[M,N] (+)= A * B with f32 accumulation in TMEM.  mcb_gemm_lowp takes the
 * operands' 16-bit type (MCB_BF16 or MCB_F16) as in_dt; mcb_gemm_bf16 is the same call with MCB_BF16.
 *   A: bf16, a_mn_major=0 -> stored [M,K] (K contiguous); 1 -> stored [K,M] (M contiguous)
 *   B: bf16, b_mn_major=0 -> stored [N,K] (K contiguous); 1 -> stored [K,N] (N contiguous)
 *   D: [M,N] row-major, out_dt MCB_F32 or MCB_BF16; bias (f32 [N]) may be NULL
 *   accumulate!=0: D += result (f32 only, atomic adds, used with split_k > 1 for weight gradients)
 * M,N,K and the leading dimensions must be multiples of 8. */
mcb_status mcb_gemm_bf16(mcb_ctx *ctx, const void *a, int32_t a_mn_major, const void *b, int32_t b_mn_major, void *d,
                         int32_t out_dt, const float *bias, int64_t m, int64_t n, int64_t k, int32_t accumulate,
                         int32_t split_k);
mcb_status mcb_gemm_lowp(mcb_ctx *ctx, int32_t in_dt, const void *a, int32_t a_mn_major, const void *b, int32_t b_mn_major, void *d,
                         int32_t out_dt, const float *bias, int64_t m, int64_t n, int64_t k, int32_t accumulate,
                         int32_t split_k);

/* ------------------------------------------------------------------ ops: attention / conv */
/* MultiHeadAttentionOp, autograd/src/host_ops.rs:779-968 (a host loop in the reference).
 * q,k,v,out: [n, seq, dim], head h in columns h*hd..(h+1)*hd.  dt = MCB_F32 or MCB_BF16.
 * lse: [n, heads, seq] f32 row log-sum-exp saved for backward. */
mcb_status mcb_attention(mcb_ctx *ctx, const void *q, const void *k, const void *v, void *out, float *lse, int64_t n,
                         int64_t seq, int64_t dim, int64_t heads, int32_t causal, int32_t dt);
mcb_status mcb_attention_backward(mcb_ctx *ctx, const void *q, const void *k, const void *v, const void *out,
                                  const void *gout, const float *lse, void *dq, void *dk, void *dv, int64_t n,
                                  int64_t seq, int64_t dim, int64_t heads, int32_t causal, int32_t dt);
/* Conv2dOp / Pool2dOp (max), autograd/src/host_ops.rs:40-180,341-476; NCHW f32 */
mcb_status mcb_conv2d(mcb_ctx *ctx, const float *x, const float *w, const float *bias, float *out, int64_t n,
                      int64_t c, int64_t h, int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride,
                      int64_t pad);
mcb_status mcb_conv2d_backward(mcb_ctx *ctx, const float *x, const float *w, const float *g, float *dx, float *dw,
                               float *db, int64_t n, int64_t c, int64_t h, int64_t wd, int64_t o, int64_t kh,
                               int64_t kw, int64_t stride, int64_t pad);
mcb_status mcb_max_pool2d(mcb_ctx *ctx, const float *x, float *out, int64_t n, int64_t c, int64_t h, int64_t w,
                          int64_t kernel, int64_t stride, int64_t pad);
mcb_status mcb_max_pool2d_backward(mcb_ctx *ctx, const float *x, const float *g, float *dx, int64_t n, int64_t c,
                                   int64_t h, int64_t w, int64_t kernel, int64_t stride, int64_t pad);

/* ------------------------------------------------------------------ ops: optimizer */
/* Ops::adam_update, ops.rs:973-1037 (out-of-place, one tensor).  step >= 1. */
mcb_status mcb_adam_update(mcb_ctx *ctx, const float *p, const float *g, const float *m, const float *v,
                           float *new_p, float *new_m, float *new_v, int64_t n, double lr, double beta1,
                           double beta2, double eps, int32_t step);
/* Fused optimizer pass over a flat arena (replaces one launch + three allocations per
 * parameter tensor, optim/src/lib.rs:85-115, and the separate unscale pass of
 * optim/src/amp.rs:50-62).  In place on p, m, v.  g is f32 or bf16 and is multiplied by
 * inv_scale first.  p_bf16 (may be NULL) receives a bf16 copy of the updated parameters.
 * skip_flag (device int32, may be NULL): when non-zero the kernel changes nothing. */
mcb_status mcb_adam_flat(mcb_ctx *ctx, float *p, const void *g, int32_t g_dt, float *m, float *v, void *p_bf16,
                         int64_t n, double lr, double beta1, double beta2, double eps, int32_t step,
                         double inv_scale, const int32_t *skip_flag);
/* GradScaler::has_non_finite_grad, optim/src/amp.rs:88-107, on the device: sets *flag to 1
 * when any entry of g (f32 or bf16) is inf or nan; never clears it. */
mcb_status mcb_check_finite(mcb_ctx *ctx, const void *g, int32_t g_dt, int64_t n, int32_t *flag);

/* ------------------------------------------------------------------ tape / optim handles */
typedef struct mcb_var mcb_var;
typedef struct mcb_adam mcb_adam;
typedef struct mcb_scaler mcb_scaler;
typedef struct mcb_arena mcb_arena;
typedef struct mcb_model mcb_model;

/* Variable::new / Variable::constant, autograd/src/variable.rs:36-42.  host_data is copied. */
mcb_status mcb_var_new(mcb_ctx *ctx, const void *host_data, int32_t dtype, const int64_t *dims, int32_t rank,
                       int32_t requires_grad, mcb_var **out);
void mcb_var_release(mcb_var *v);
mcb_status mcb_var_rank(mcb_var *v, int32_t *rank_out);
mcb_status mcb_var_dims(mcb_var *v, int64_t *dims_out);
mcb_status mcb_var_dtype(mcb_var *v, int32_t *dtype_out);
mcb_status mcb_var_data(mcb_var *v, void *host_out);                   /* f32 (bf16 widened) or raw ints */
mcb_status mcb_var_grad(mcb_var *v, float *host_out, int32_t *has_grad); /* host_out may be NULL to query */
mcb_status mcb_var_set_data(mcb_var *v, const void *host_data);
mcb_status mcb_var_set_grad(mcb_var *v, const float *host_grad); /* NULL clears */
mcb_status mcb_var_cleargrad(mcb_var *v);
mcb_status mcb_var_requires_grad(mcb_var *v, int32_t *out);
mcb_status mcb_var_is_leaf(mcb_var *v, int32_t *out);
mcb_status mcb_var_unchain_backward(mcb_var *v);
/* Variable::backward, autograd/src/variable.rs:150-207 */
mcb_status mcb_var_backward(mcb_var *v);
/* no_grad, autograd/src/lib.rs:20-60: per host thread, like the reference's thread-local cell */
void mcb_set_grad_enabled(int32_t enabled);
int32_t mcb_is_grad_enabled(void);
/* autocast, core/src/autocast.rs:6-44: MCB_BF16 or MCB_F16 lowers linear / matmul / attention of the calling
 * host thread to that type (operands rounded to nearest even, f32 accumulate); -1 disables.  LayerNorm,
 * softmax, the loss and every reduction stay in f32. */
void mcb_set_autocast(int32_t dtype_or_minus1);
int32_t mcb_get_autocast(void); /* the calling thread's autocast type, or -1 */

/* F::*, autograd/src/ops.rs:356-415,579-612,888-936 and host_ops.rs:594-990 */
mcb_status mcb_f_binary(int32_t op, mcb_var *a, mcb_var *b, mcb_var **out);
mcb_status mcb_f_scale(mcb_var *x, double factor, mcb_var **out);
mcb_status mcb_f_unary(int32_t op, mcb_var *x, mcb_var **out);
mcb_status mcb_f_relu(mcb_var *x, mcb_var **out);
mcb_status mcb_f_gelu(mcb_var *x, mcb_var **out);
mcb_status mcb_f_sum(mcb_var *x, mcb_var **out);
mcb_status mcb_f_mean(mcb_var *x, mcb_var **out);
mcb_status mcb_f_matmul(mcb_var *a, mcb_var *b, mcb_var **out);
mcb_status mcb_f_linear(mcb_var *x, mcb_var *w, mcb_var *bias_or_null, mcb_var **out);
mcb_status mcb_f_linear_activation(mcb_var *x, mcb_var *w, mcb_var *bias_or_null, int32_t act, mcb_var **out);
mcb_status mcb_f_softmax(mcb_var *x, mcb_var **out);
mcb_status mcb_f_layer_norm(mcb_var *x, mcb_var *gamma, mcb_var *beta, double eps, mcb_var **out);
mcb_status mcb_f_softmax_cross_entropy(mcb_var *logits, mcb_var *target, mcb_var **out);
mcb_status mcb_f_embedding(mcb_var *ids, mcb_var *weight, mcb_var **out);
mcb_status mcb_f_reshape(mcb_var *x, const int64_t *dims, int32_t rank, mcb_var **out);
/* Transpose2d, autograd/src/ops.rs:235-255 (2-D only; backward transposes the gradient) and
 * PermuteOp, autograd/src/host_ops.rs:690-777 (backward applies the inverse permutation) */
mcb_status mcb_f_transpose(mcb_var *x, mcb_var **out);
mcb_status mcb_f_permute(mcb_var *x, const int32_t *axes, int32_t rank, mcb_var **out);
mcb_status mcb_f_multi_head_attention(mcb_var *q, mcb_var *k, mcb_var *v, int64_t heads, int32_t causal,
                                      mcb_var **out);
mcb_status mcb_f_conv2d(mcb_var *x, mcb_var *w, mcb_var *bias_or_null, int64_t stride, int64_t pad, mcb_var **out);
mcb_status mcb_f_max_pool2d(mcb_var *x, int64_t kernel, int64_t stride, int64_t pad, mcb_var **out);

/* Flat parameter arena: moves the listed parameters into one contiguous p / grad / m / v
 * allocation (plus a bf16 shadow of p) so the optimizer and the gradient allreduce run over
 * flat ranges.  The variables keep working as before (their data become views). */
mcb_status mcb_arena_create(mcb_ctx *ctx, mcb_var **params, int32_t n, mcb_arena **out);
void mcb_arena_release(mcb_arena *a);
mcb_status mcb_arena_numel(mcb_arena *a, int64_t *out);

/* zero_grad, optim/src/lib.rs:17-21 */
mcb_status mcb_zero_grad(mcb_var **params, int32_t n);
/* Adam::new / Optimizer::update, optim/src/lib.rs:53-120 */
mcb_status mcb_adam_create(mcb_ctx *ctx, double lr, double beta1, double beta2, double eps, mcb_adam **out);
void mcb_adam_release(mcb_adam *opt);
mcb_status mcb_adam_step(mcb_adam *opt, mcb_var **params, int32_t n);
/* GradScaler, optim/src/amp.rs:8-113.  The scale, the growth tracker and the found-inf flag
 * live on the device so a step needs no host synchronisation; mcb_scaler_step reads the
 * flag back (one 4-byte copy) to return `applied` like the reference's bool. */
mcb_status mcb_scaler_create(mcb_ctx *ctx, double init_scale, double growth_factor, double backoff_factor,
                             int32_t growth_interval, mcb_scaler **out);
void mcb_scaler_release(mcb_scaler *s);
mcb_status mcb_scaler_scale_loss(mcb_scaler *s, mcb_var *loss, mcb_var **out);
mcb_status mcb_scaler_step(mcb_scaler *s, mcb_adam *opt, mcb_var **params, int32_t n, int32_t *applied);
mcb_status mcb_scaler_step_async(mcb_scaler *s, mcb_adam *opt, mcb_var **params, int32_t n);
mcb_status mcb_scaler_state(mcb_scaler *s, double *scale_out, int32_t *growth_tracker_out, int32_t *last_found_inf);

/* The rest of the Optimizer family on the same fused flat pass (optim/src/lib.rs:23-51 SGD, 122-160
 * MomentumSGD, 162-214 AdamW).  The handle is the mcb_adam type so that mcb_adam_step, mcb_scaler_step and
 * mcb_adam_release work for every kind.  `beta1` carries the momentum for MomentumSGD; unused fields are
 * ignored.  AdamW subtracts (f32)(weight_decay*lr) * p_old after the Adam step, as the reference does. */
enum { MCB_OPT_ADAM = 0, MCB_OPT_ADAMW = 1, MCB_OPT_SGD = 2, MCB_OPT_MOMENTUM_SGD = 3 };
mcb_status mcb_opt_create(mcb_ctx *ctx, int32_t kind, double lr, double beta1, double beta2, double eps, double weight_decay,
                          mcb_adam **out);
/* learning rate used by the following steps (the schedules below are stateless functions of the step) */
mcb_status mcb_opt_set_lr(mcb_adam *opt, double lr);
mcb_status mcb_opt_get_lr(mcb_adam *opt, double *lr_out);
/* clip_grad_norm, optim/src/lib.rs:216-243: global L2 norm over every listed parameter that has a gradient
 * (squares in f32, sums in f64), gradients scaled in place by (f32)(max_norm/norm) when norm > max_norm;
 * *norm_out receives the pre-clip norm (one 8-byte read-back).  max_norm <= 0 is InvalidArgument. */
mcb_status mcb_clip_grad_norm(mcb_var **params, int32_t n, double max_norm, double *norm_out);
/* LR schedules, optim/src/lib.rs:245-326 (pure host functions of the step) */
double mcb_lr_linear_warmup_cosine(uint64_t step, uint64_t warmup_steps, uint64_t total_steps, double base_lr, double min_lr);
double mcb_lr_step(uint64_t step, double base_lr, uint64_t step_size, double gamma);
double mcb_lr_polynomial(uint64_t step, double base_lr, uint64_t total_steps, double power, double min_lr);

/* he_normal, core/src/init.rs:6-11 over Rng (core/src/rng.rs:14-56): the values nn::Linear / Conv2d / Embedding
 * start from for a given seed, so that a link built above this library is bit-identical to the reference's.
 * Host function (no context, no device). */
mcb_status mcb_he_normal(float *host_out, int64_t n, int64_t fan_in, uint64_t seed);

/* Training checkpoint in the reference's `.mcn` container (crates/modern-chainer-serial/src/lib.rs:12-115:
 * "MCHN0001", u32 count, per entry name / dtype tag / rank / u64 dims / u64 byte length / bytes, little-endian).
 * Entries: `name` (f32 value) for every listed parameter; with `opt`: `name.opt_m`, `name.opt_v` (f32) and
 * `name.opt_t` (i64 [1]); with `scaler`: `grad_scaler.state` (f32 {scale, inv_scale}) and `grad_scaler.counters`
 * (i32 {growth_tracker, found_inf, last_found_inf, applied_steps}).  Both calls synchronise.  Load checks every
 * entry (presence, dtype, shape) before it changes anything; a file that is not .mcn is InvalidArgument
 * ("not a Modern Chainer .mcn file", lib.rs:41), an unreadable one Io. */
mcb_status mcb_checkpoint_save(mcb_ctx *ctx, const char *path, const char *const *names, mcb_var **params, int32_t n,
                               mcb_adam *opt_or_null, mcb_scaler *scaler_or_null);
mcb_status mcb_checkpoint_load(mcb_ctx *ctx, const char *path, const char *const *names, mcb_var **params, int32_t n,
                               mcb_adam *opt_or_null, mcb_scaler *scaler_or_null);

/* Whole-step CUDA Graph (cuda/src/graph.rs:261-603 GraphLinearTrainer, cuda/src/static_run.rs:1875-2096
 * CudaStaticStep / LinearMseAdamStep): zero_grad + model loss (+ GradScaler scaling) + backward + optimizer update
 * recorded once from the tape and replayed with a single launch.  Inputs live in fixed device buffers; _run copies
 * host_x / host_y into them first (either may be NULL when the caller filled the buffers returned by _inputs).
 * autocast_dt is -1 (f32) or MCB_BF16.  Declared after mcb_model below. */
typedef struct mcb_static_step mcb_static_step;

/* The benchmark models, built from the nn initialisers (nn/src/lib.rs:38-73,141-147,185-191,
 * 246-271) and, for the decoder, the layout of llm/src/decoder.rs:98-140.
 *   kind 0: MLP  cfg = {in, hidden, out}
 *   kind 1: pre-LN encoder block  cfg = {d_model, heads, d_ff, causal}
 *   kind 2: CNN  cfg = {in_channels, c1, c2, height_width, classes}
 *   kind 3: decoder  cfg = {vocab, d_model, heads, d_ff, layers, seed} */
mcb_status mcb_model_create(mcb_ctx *ctx, int32_t kind, const int64_t *cfg, int32_t n_cfg, mcb_model **out);
void mcb_model_release(mcb_model *m);
mcb_status mcb_model_num_params(mcb_model *m, int32_t *out);
mcb_status mcb_model_param(mcb_model *m, int32_t index, mcb_var **out); /* a new reference; release it */
/* forward to the scalar loss: (x f32, labels int) for kinds 0,2; (x, target f32) for 1; (ids, targets int) for 3 */
mcb_status mcb_model_loss(mcb_model *m, mcb_var *input, mcb_var *target, mcb_var **loss_out);

/* static (graph-captured) training step; see the note at the typedef above.  Creating one changes no parameter
 * (capture records, it does not execute).  Per-kernel timing must be off.  With a data-parallel arena the bucket
 * all-reduces are part of the graph; run at least one ordinary step first so that NCCL has set up its connections. */
mcb_status mcb_static_step_create(mcb_model *model, mcb_adam *opt, mcb_scaler *scaler_or_null, int32_t autocast_dt,
                                  const int64_t *x_dims, int32_t x_rank, int32_t x_dt, const int64_t *y_dims, int32_t y_rank,
                                  int32_t y_dt, mcb_static_step **out);
mcb_status mcb_static_step_inputs(mcb_static_step *s, void **x_dev_out, void **y_dev_out);
mcb_status mcb_static_step_run(mcb_static_step *s, const void *host_x_or_null, const void *host_y_or_null);
mcb_status mcb_static_step_loss(mcb_static_step *s, float *loss_out); /* synchronises; the unscaled loss of the last run */
/* Pipelined form for loops that read every step's loss.  Launches this step, queues the copy of ITS loss to pinned
 * host memory behind it, and returns the loss of the PREVIOUS pipelined run (*have_prev_out = 0 on the first call),
 * waiting only for that one: the device always has the next step queued, where run + loss leaves it idle while the
 * host launches.  The host buffers of call i may be rewritten once call i + 1 has returned.  mcb_static_step_drain
 * returns the loss of the last pipelined run (*have_out = 0 if none is outstanding).  The waits are bounded like
 * every host wait of the data-parallel path when collectives are in flight. */
mcb_status mcb_static_step_run_pipelined(mcb_static_step *s, const void *host_x_or_null, const void *host_y_or_null,
                                         float *prev_loss_out, int32_t *have_prev_out);
mcb_status mcb_static_step_drain(mcb_static_step *s, float *loss_out, int32_t *have_out);
mcb_status mcb_static_step_launches(mcb_static_step *s, int64_t *kernels_per_step_out);
void mcb_static_step_release(mcb_static_step *s);

/* ------------------------------------------------------------------ data parallel */
/* No counterpart in the reference (it has no distributed training).  One process per GPU.
 * nccl_unique_id: the 128 bytes of an ncclUniqueId created by mcb_dp_unique_id on rank 0
 * and shared by the launcher.  After mcb_dp_attach every backward pass over the arena's
 * parameters all-reduces the gradient arena in buckets on a communication stream as soon
 * as the last gradient of a bucket is final, and the optimizer waits for them.  Gradients
 * are summed; the 1/world factor is folded into the optimizer's unscale factor (and into
 * the norm mcb_clip_grad_norm measures), so N ranks at batch B behave like one at batch N*B.
 *
 * Rules and failure behaviour:
 *   - ONE backward pass per optimizer step on an attached arena.  A second mcb_var_backward before
 *     the optimizer (or mcb_zero_grad) has closed the round returns MCB_UNSUPPORTED and enqueues
 *     nothing: its gradients would be added into buckets that are already summed over the ranks
 *     and would never be exchanged themselves.
 *   - mcb_dp_attach compares a checksum of the bucket plan across ranks and returns
 *     MCB_INVALID_ARGUMENT when they differ.
 *   - No call waits without a limit.  mcb_dp_init gives up after the timeout when a rank does not
 *     join; synchronising calls (mcb_sync, mcb_memcpy_d2h, read-backs) poll instead of blocking
 *     while collectives may be in flight.  An error reported by NCCL, a failed enqueue or an
 *     expired timeout ABORTS the communicator (ncclCommAbort), after which every data-parallel
 *     call on the context returns MCB_BACKEND: the caller leaves its loop, calls mcb_dp_shutdown
 *     and may rebuild the group.  Default timeout 300 s; MCB_DP_TIMEOUT_MS or mcb_dp_set_timeout_ms. */
mcb_status mcb_dp_unique_id(void *host_id_out_128);
mcb_status mcb_dp_init(mcb_ctx *ctx, int32_t rank, int32_t world, const void *host_id_128);
mcb_status mcb_dp_set_timeout_ms(mcb_ctx *ctx, int64_t timeout_ms);
mcb_status mcb_dp_attach(mcb_ctx *ctx, mcb_arena *arena, int64_t bucket_bytes);
mcb_status mcb_dp_allreduce_f32(mcb_ctx *ctx, float *buf, int64_t n, int32_t op_max); /* on the compute stream */
mcb_status mcb_dp_shutdown(mcb_ctx *ctx);
/* host-only helper (no GPU needed): splits `n` tensors of `sizes` elements, walked from last to
 * first, into buckets of at most bucket_elems; bucket_of[i] receives the bucket index of tensor i */
mcb_status mcb_dp_plan_buckets(const int64_t *sizes, int32_t n, int64_t bucket_elems, int32_t *bucket_of,
                               int32_t *n_buckets_out);
/* host-only: MCB_OK when the `world` plan checksums (one per rank) agree, else MCB_INVALID_ARGUMENT */
mcb_status mcb_dp_check_plan_checksums(const uint64_t *checksums, int32_t world);

/* Host-only model of one rank's data-parallel round logic over a recording transport (no device, no NCCL):
 * the code that decides when a bucket's all-reduce starts, refuses a second backward pass, and turns
 * transport errors and timeouts into an abort is the code the GPU path runs; only the transport differs.
 * For tests of the failure paths, which must not be provoked on a GPU.
 *   _create      `n` parameter slots of the given (padded) sizes, planned into buckets like mcb_dp_attach does
 *   _backward_begin / _grad_ready(param) / _finish (the optimizer's first act) / _zero_grad / _host_wait
 *   _inject      what = 0: the enqueue of bucket `value` fails (this rank broke before it could take part);
 *                what = 1: the transport reports an asynchronous error from its `value`-th poll on (a peer
 *                          or the network failed); what = 2: value != 0: collectives never complete (a peer
 *                          never joined)
 *   _log         buckets in the order their all-reduce was enqueued; returns how many */
typedef struct mcb_dp_sim mcb_dp_sim;
mcb_status mcb_dp_sim_create(const int64_t *slot_sizes, int32_t n, int64_t bucket_elems, int32_t world, mcb_dp_sim **out);
void mcb_dp_sim_release(mcb_dp_sim *s);
mcb_status mcb_dp_sim_backward_begin(mcb_dp_sim *s);
mcb_status mcb_dp_sim_grad_ready(mcb_dp_sim *s, int32_t param);
mcb_status mcb_dp_sim_finish(mcb_dp_sim *s);
mcb_status mcb_dp_sim_zero_grad(mcb_dp_sim *s);
mcb_status mcb_dp_sim_host_wait(mcb_dp_sim *s, int32_t timeout_ms);
void mcb_dp_sim_inject(mcb_dp_sim *s, int32_t what, int32_t value);
int32_t mcb_dp_sim_log(mcb_dp_sim *s, int32_t *buckets_out, int32_t max);
int32_t mcb_dp_sim_bucket_of(mcb_dp_sim *s, int32_t param);
int32_t mcb_dp_sim_buckets(mcb_dp_sim *s);
int32_t mcb_dp_sim_joins(mcb_dp_sim *s);
int32_t mcb_dp_sim_aborted(mcb_dp_sim *s);
uint64_t mcb_dp_sim_plan_checksum(mcb_dp_sim *s);
const char *mcb_dp_sim_last_error(mcb_dp_sim *s);

#ifdef __cplusplus
}
#endif
#endif /* MCB_H */
