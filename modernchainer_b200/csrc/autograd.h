// Internal C++ types behind the tape / optimizer handles of the C ABI.
#pragma once
#include <algorithm>
#include <functional>
#include <memory>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "internal.h"

namespace mcbag {

// device allocation returned to the context's pool when the last tensor drops it
struct Buf {
    mcb_ctx *ctx;
    void *p;
    Buf(mcb_ctx *c, void *ptr) : ctx(c), p(ptr) {}
    ~Buf() { mcb_free(ctx, p); }
    Buf(const Buf &) = delete;
    Buf &operator=(const Buf &) = delete;
};

struct GradAux;

struct Tensor {
    std::shared_ptr<Buf> buf;
    void *ptr = nullptr;
    int dt = MCB_F32;
    std::vector<int64_t> shape;
    bool defined = false;
    // Optional by-products of the kernel that wrote an f32 gradient: the same values rounded to bf16 and their
    // column sums.  Valid only while the values are unchanged: whoever modifies the tensor in place drops it.
    std::shared_ptr<GradAux> aux;
    int64_t numel() const;
};

struct GradAux {
    Tensor bf16;   // same shape, bf16
    Tensor colsum; // [last dim], f32: column sums of the bf16 values
};

struct Node;
struct Arena;

struct VarImpl {
    mcb_ctx *ctx = nullptr;
    Tensor data;
    Tensor grad;
    bool has_grad = false;
    bool requires_grad = false;
    std::shared_ptr<Node> node;
    // flat arena binding (parameters only)
    Arena *arena = nullptr;
    int arena_idx = -1;
    bool slot_claimed = false;
};
using Var = std::shared_ptr<VarImpl>;

using BackwardFn = std::function<mcb_status(const Tensor &g, std::vector<Tensor> &input_grads)>;
struct Node {
    const char *name = "";
    std::vector<Var> inputs;
    BackwardFn backward;
};

struct Arena {
    mcb_ctx *ctx = nullptr;
    int64_t total = 0;
    std::shared_ptr<Buf> p, g, m, v, shadow;
    std::vector<Var> vars;
    std::vector<int64_t> off, size;
    std::vector<int32_t> step;
    bool shadow_valid = false;
    int shadow_dt = MCB_BF16; // format of the 16-bit copy: MCB_BF16 or MCB_F16
    std::vector<VarImpl *> claimed;
    // data-parallel bucketing (filled by mcb_dp_attach)
    std::vector<int> bucket_of;            // per parameter
    std::vector<int64_t> bucket_begin, bucket_end; // element ranges in the arena
    std::vector<int> bucket_pending, bucket_size;   // parameters still missing / total per bucket
    bool dp_attached = false;
    bool comm_in_flight = false;
};

bool grad_enabled();
int autocast();

mcb_status new_tensor(mcb_ctx *ctx, int dt, const std::vector<int64_t> &shape, Tensor *out);
Tensor view(const Tensor &t, const std::vector<int64_t> &shape);
mcb_status to_dtype(mcb_ctx *ctx, const Tensor &t, int dt, Tensor *out);
Var make_var(mcb_ctx *ctx, const Tensor &data, bool requires_grad);
mcb_status backward(const Var &root);

mcb_status f_binary(int op, const Var &a, const Var &b, Var *out);
mcb_status f_scale(const Var &x, double factor, Var *out);
mcb_status f_scale_by_device(const Var &x, const float *scalar, std::shared_ptr<Buf> keep, Var *out);
mcb_status f_unary(int op, const Var &x, Var *out);
mcb_status f_relu(const Var &x, Var *out);
mcb_status f_gelu(const Var &x, Var *out);
mcb_status f_sum(const Var &x, Var *out);
mcb_status f_mean(const Var &x, Var *out);
mcb_status f_matmul(const Var &a, const Var &b, Var *out);
mcb_status f_linear(const Var &x, const Var &w, const Var &b, Var *out);
mcb_status f_linear_activation(const Var &x, const Var &w, const Var &b, int act, Var *out);
mcb_status f_softmax(const Var &x, Var *out);
mcb_status f_layer_norm(const Var &x, const Var &gamma, const Var &beta, double eps, Var *out);
mcb_status f_softmax_cross_entropy(const Var &logits, const Var &target, Var *out);
mcb_status f_sce_consuming(const Var &logits, const Var &target, Var *out);
mcb_status f_embedding(const Var &ids, const Var &weight, Var *out);
mcb_status f_reshape(const Var &x, const std::vector<int64_t> &shape, Var *out);
mcb_status f_permute(const Var &x, const std::vector<int32_t> &axes, Var *out);
mcb_status f_transpose(const Var &x, Var *out);
mcb_status f_multi_head_attention(const Var &q, const Var &k, const Var &v, int64_t heads, bool causal, Var *out);
mcb_status f_conv2d(const Var &x, const Var &w, const Var &b, int64_t stride, int64_t pad, Var *out);
mcb_status f_max_pool2d(const Var &x, int64_t kernel, int64_t stride, int64_t pad, Var *out);

mcb_status arena_create(mcb_ctx *ctx, const std::vector<Var> &params, Arena **out);
void arena_release(Arena *a);
mcb_status arena_refresh_shadow(Arena *a, int dt = -1);
// data-parallel hooks (dp.cu): a parameter's gradient is final / wait for the buckets in flight /
// factor that turns the summed gradient into the mean over ranks
mcb_status arena_grad_ready(Arena *a, int idx);
mcb_status arena_wait_comm(Arena *a);
mcb_status arena_backward_begin(Arena *a); // refuses a second backward pass before the optimizer on a data-parallel arena
mcb_status arena_abandon_round(Arena *a);  // zero_grad while all-reduces of dropped gradients may still run
double arena_grad_divisor(Arena *a);

mcb_status zero_grad(const std::vector<Var> &params);

struct AdamState {
    Tensor m, v;
    int32_t t = 0;
};
struct AdamOpt {
    mcb_ctx *ctx = nullptr;
    double lr = 1e-3, beta1 = 0.9, beta2 = 0.999, eps = 1e-8;
    int kind = MCB_OPT_ADAM;      // MCB_OPT_*: Adam, AdamW, SGD, MomentumSGD (beta1 = momentum) on the same flat pass
    double weight_decay = 0.0;    // AdamW only
    std::unordered_map<VarImpl *, AdamState> state;
    mcb_status update(const std::vector<Var> &params, const float *inv_scale_dev = nullptr, double inv_scale_host = 1.0,
                      const int32_t *skip = nullptr, const int32_t *step_dev = nullptr);
    void rollback_step(const std::vector<Var> &params);
    void rollback_steps(const std::vector<Var> &params, int64_t k); // every listed parameter, k steps (not below zero)
    ~AdamOpt();
};

struct Scaler {
    mcb_ctx *ctx = nullptr;
    double growth = 2.0, backoff = 0.5;
    int interval = 2000;
    std::shared_ptr<Buf> state; // {scale, inv_scale} f32, {growth_tracker, found_inf, last_found_inf, applied_steps} i32
    // Steps taken without reading the outcome back (mcb_scaler_step_async, replays of a captured step) advance the
    // host's per-parameter step counts even when the device skipped them.  issued_since counts the steps whose
    // outcome the host has booked as applied since the last reconciliation; applied_seen is the device's count of
    // applied steps at that point: the difference of the two growths is the number of skipped steps still to undo.
    int64_t issued_since = 0;
    int32_t applied_seen = 0;
    float *state_f() const { return (float *)state->p; }
    int *state_i() const { return (int *)((float *)state->p + 2); }
};
mcb_status scaler_create(mcb_ctx *ctx, double init_scale, double growth, double backoff, int interval, Scaler **out);
mcb_status scaler_step(Scaler *s, AdamOpt *opt, const std::vector<Var> &params, bool sync, int32_t *applied);
// reads the device's count of applied steps (synchronises) and takes the skipped steps off the host's step counts
mcb_status scaler_reconcile(Scaler *s, AdamOpt *opt, const std::vector<Var> &params);

struct Model {
    mcb_ctx *ctx = nullptr;
    int kind = 0;
    std::vector<int64_t> cfg;
    std::vector<Var> params;
    static mcb_status create(mcb_ctx *ctx, int kind, const std::vector<int64_t> &cfg, Model **out);
    mcb_status loss(const Var &input, const Var &target, Var *out);
};

void set_grad_enabled(bool on);
void set_autocast(int dt);

} // namespace mcbag
