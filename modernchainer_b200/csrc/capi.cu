// extern "C" surface of the tape / optimizer / model handles (declared in include/mcb.h).
#include <cstring>

#include "handles.h"

using namespace mcbag;

static mcb_status wrap(mcb_status st, const Var &v, mcb_var **out) {
    if (st != MCB_OK) return st;
    *out = new mcb_var{v};
    return MCB_OK;
}
static std::vector<Var> collect(mcb_var **params, int32_t n) {
    std::vector<Var> v;
    v.reserve(n);
    for (int32_t i = 0; i < n; ++i) v.push_back(params[i]->v);
    return v;
}

extern "C" {

mcb_status mcb_var_new(mcb_ctx *ctx, const void *host_data, int32_t dtype, const int64_t *dims, int32_t rank,
                       int32_t requires_grad, mcb_var **out) {
    MCB_CHECK_CTX(ctx);
    if (rank < 0 || rank > 8 || !out) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "rank must be in 0..8");
    if (mcb_dtype_size(dtype) == 0) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "unknown dtype %d", dtype);
    std::vector<int64_t> shape(dims, dims + rank);
    Tensor t;
    MCB_TRY(new_tensor(ctx, dtype, shape, &t));
    if (host_data && t.numel()) MCB_TRY(mcb_memcpy_h2d(ctx, t.ptr, host_data, (size_t)t.numel() * mcb_dtype_size(dtype)));
    MCB_TRY(mcb_sync(ctx)); // the caller may release host_data as soon as this returns
    bool rg = requires_grad && (dtype == MCB_F32 || dtype == MCB_BF16 || dtype == MCB_F16);
    *out = new mcb_var{make_var(ctx, t, rg)};
    return MCB_OK;
}

void mcb_var_release(mcb_var *v) { delete v; }

mcb_status mcb_var_rank(mcb_var *v, int32_t *rank_out) {
    *rank_out = (int32_t)v->v->data.shape.size();
    return MCB_OK;
}
mcb_status mcb_var_dims(mcb_var *v, int64_t *dims_out) {
    for (size_t i = 0; i < v->v->data.shape.size(); ++i) dims_out[i] = v->v->data.shape[i];
    return MCB_OK;
}
mcb_status mcb_var_dtype(mcb_var *v, int32_t *dtype_out) {
    *dtype_out = v->v->data.dt;
    return MCB_OK;
}

mcb_status mcb_var_data(mcb_var *v, void *host_out) {
    mcb_ctx *ctx = v->v->ctx;
    const Tensor &d = v->v->data;
    if (d.dt == MCB_BF16 || d.dt == MCB_F16) {
        Tensor f;
        MCB_TRY(to_dtype(ctx, d, MCB_F32, &f));
        return mcb_memcpy_d2h(ctx, host_out, f.ptr, sizeof(float) * f.numel());
    }
    return mcb_memcpy_d2h(ctx, host_out, d.ptr, (size_t)d.numel() * mcb_dtype_size(d.dt));
}

mcb_status mcb_var_grad(mcb_var *v, float *host_out, int32_t *has_grad) {
    mcb_ctx *ctx = v->v->ctx;
    if (has_grad) *has_grad = v->v->has_grad ? 1 : 0;
    if (!v->v->has_grad || !host_out) return MCB_OK;
    if (v->v->arena) MCB_TRY(arena_wait_comm(v->v->arena));
    Tensor f;
    MCB_TRY(to_dtype(ctx, v->v->grad, MCB_F32, &f));
    return mcb_memcpy_d2h(ctx, host_out, f.ptr, sizeof(float) * f.numel());
}

mcb_status mcb_var_set_data(mcb_var *v, const void *host_data) {
    mcb_ctx *ctx = v->v->ctx;
    Tensor &d = v->v->data;
    MCB_TRY(mcb_memcpy_h2d(ctx, d.ptr, host_data, (size_t)d.numel() * mcb_dtype_size(d.dt)));
    if (v->v->arena) v->v->arena->shadow_valid = false;
    return mcb_sync(ctx);
}

mcb_status mcb_var_set_grad(mcb_var *v, const float *host_grad) {
    mcb_ctx *ctx = v->v->ctx;
    v->v->has_grad = false;
    v->v->grad = Tensor();
    if (!host_grad) return MCB_OK;
    Tensor g;
    if (v->v->arena) {
        g.buf = v->v->arena->g;
        g.ptr = (float *)v->v->arena->g->p + v->v->arena->off[v->v->arena_idx];
        g.dt = MCB_F32;
        g.shape = v->v->data.shape;
        g.defined = true;
    } else {
        MCB_TRY(new_tensor(ctx, MCB_F32, v->v->data.shape, &g));
    }
    MCB_TRY(mcb_memcpy_h2d(ctx, g.ptr, host_grad, sizeof(float) * g.numel()));
    MCB_TRY(mcb_sync(ctx));
    v->v->grad = g;
    v->v->has_grad = true;
    return MCB_OK;
}

mcb_status mcb_var_cleargrad(mcb_var *v) {
    v->v->has_grad = false;
    v->v->grad = Tensor();
    return MCB_OK;
}
mcb_status mcb_var_requires_grad(mcb_var *v, int32_t *out) {
    *out = v->v->requires_grad;
    return MCB_OK;
}
mcb_status mcb_var_is_leaf(mcb_var *v, int32_t *out) {
    *out = v->v->node == nullptr;
    return MCB_OK;
}
mcb_status mcb_var_unchain_backward(mcb_var *v) {
    v->v->node.reset();
    return MCB_OK;
}
mcb_status mcb_var_backward(mcb_var *v) { return backward(v->v); }

void mcb_set_grad_enabled(int32_t enabled) { set_grad_enabled(enabled != 0); }
int32_t mcb_is_grad_enabled(void) { return grad_enabled() ? 1 : 0; }
void mcb_set_autocast(int32_t dt) { set_autocast((dt == MCB_BF16 || dt == MCB_F16) ? dt : -1); }
int32_t mcb_get_autocast(void) { return autocast(); }

mcb_status mcb_f_binary(int32_t op, mcb_var *a, mcb_var *b, mcb_var **out) {
    if (op < MCB_ADD || op > MCB_DIV) return mcb_fail(a->v->ctx, MCB_INVALID_ARGUMENT, "unknown binary op %d", op);
    Var r;
    return wrap(f_binary(op, a->v, b->v, &r), r, out);
}
mcb_status mcb_f_scale(mcb_var *x, double factor, mcb_var **out) {
    Var r;
    return wrap(f_scale(x->v, factor, &r), r, out);
}
mcb_status mcb_f_unary(int32_t op, mcb_var *x, mcb_var **out) {
    Var r;
    return wrap(f_unary(op, x->v, &r), r, out);
}
mcb_status mcb_f_relu(mcb_var *x, mcb_var **out) {
    Var r;
    return wrap(f_relu(x->v, &r), r, out);
}
mcb_status mcb_f_gelu(mcb_var *x, mcb_var **out) {
    Var r;
    return wrap(f_gelu(x->v, &r), r, out);
}
mcb_status mcb_f_sum(mcb_var *x, mcb_var **out) {
    Var r;
    return wrap(f_sum(x->v, &r), r, out);
}
mcb_status mcb_f_mean(mcb_var *x, mcb_var **out) {
    Var r;
    return wrap(f_mean(x->v, &r), r, out);
}
mcb_status mcb_f_matmul(mcb_var *a, mcb_var *b, mcb_var **out) {
    Var r;
    return wrap(f_matmul(a->v, b->v, &r), r, out);
}
mcb_status mcb_f_linear(mcb_var *x, mcb_var *w, mcb_var *bias, mcb_var **out) {
    Var r;
    return wrap(f_linear(x->v, w->v, bias ? bias->v : Var(), &r), r, out);
}
mcb_status mcb_f_linear_activation(mcb_var *x, mcb_var *w, mcb_var *bias, int32_t act, mcb_var **out) {
    Var r;
    return wrap(f_linear_activation(x->v, w->v, bias ? bias->v : Var(), act, &r), r, out);
}
mcb_status mcb_f_softmax(mcb_var *x, mcb_var **out) {
    Var r;
    return wrap(f_softmax(x->v, &r), r, out);
}
mcb_status mcb_f_layer_norm(mcb_var *x, mcb_var *gamma, mcb_var *beta, double eps, mcb_var **out) {
    Var r;
    return wrap(f_layer_norm(x->v, gamma->v, beta->v, eps, &r), r, out);
}
mcb_status mcb_f_softmax_cross_entropy(mcb_var *logits, mcb_var *target, mcb_var **out) {
    Var r;
    return wrap(f_softmax_cross_entropy(logits->v, target->v, &r), r, out);
}
mcb_status mcb_f_embedding(mcb_var *ids, mcb_var *weight, mcb_var **out) {
    Var r;
    return wrap(f_embedding(ids->v, weight->v, &r), r, out);
}
mcb_status mcb_f_reshape(mcb_var *x, const int64_t *dims, int32_t rank, mcb_var **out) {
    Var r;
    return wrap(f_reshape(x->v, std::vector<int64_t>(dims, dims + rank), &r), r, out);
}
mcb_status mcb_f_transpose(mcb_var *x, mcb_var **out) {
    Var r;
    return wrap(f_transpose(x->v, &r), r, out);
}
mcb_status mcb_f_permute(mcb_var *x, const int32_t *axes, int32_t rank, mcb_var **out) {
    Var r;
    if (rank < 0 || (rank > 0 && !axes)) return MCB_INVALID_ARGUMENT;
    return wrap(f_permute(x->v, std::vector<int32_t>(axes, axes + rank), &r), r, out);
}
mcb_status mcb_f_multi_head_attention(mcb_var *q, mcb_var *k, mcb_var *v, int64_t heads, int32_t causal, mcb_var **out) {
    Var r;
    return wrap(f_multi_head_attention(q->v, k->v, v->v, heads, causal != 0, &r), r, out);
}
mcb_status mcb_f_conv2d(mcb_var *x, mcb_var *w, mcb_var *bias, int64_t stride, int64_t pad, mcb_var **out) {
    Var r;
    return wrap(f_conv2d(x->v, w->v, bias ? bias->v : Var(), stride, pad, &r), r, out);
}
mcb_status mcb_f_max_pool2d(mcb_var *x, int64_t kernel, int64_t stride, int64_t pad, mcb_var **out) {
    Var r;
    return wrap(f_max_pool2d(x->v, kernel, stride, pad, &r), r, out);
}

mcb_status mcb_arena_create(mcb_ctx *ctx, mcb_var **params, int32_t n, mcb_arena **out) {
    MCB_CHECK_CTX(ctx);
    Arena *a = nullptr;
    MCB_TRY(arena_create(ctx, collect(params, n), &a));
    *out = new mcb_arena{a};
    return MCB_OK;
}
void mcb_arena_release(mcb_arena *a) {
    if (!a) return;
    arena_release(a->a);
    delete a;
}
mcb_status mcb_arena_numel(mcb_arena *a, int64_t *out) {
    *out = a->a->total;
    return MCB_OK;
}

mcb_status mcb_zero_grad(mcb_var **params, int32_t n) {
    MCB_TRY(zero_grad(collect(params, n)));
    return MCB_OK;
}

mcb_status mcb_adam_create(mcb_ctx *ctx, double lr, double beta1, double beta2, double eps, mcb_adam **out) {
    MCB_CHECK_CTX(ctx);
    mcb_adam *o = new mcb_adam();
    o->opt.ctx = ctx;
    o->opt.lr = lr;
    o->opt.beta1 = beta1;
    o->opt.beta2 = beta2;
    o->opt.eps = eps;
    *out = o;
    return MCB_OK;
}
void mcb_adam_release(mcb_adam *opt) { delete opt; }
mcb_status mcb_adam_step(mcb_adam *opt, mcb_var **params, int32_t n) { return opt->opt.update(collect(params, n)); }

mcb_status mcb_opt_create(mcb_ctx *ctx, int32_t kind, double lr, double beta1, double beta2, double eps, double weight_decay,
                          mcb_adam **out) {
    MCB_CHECK_CTX(ctx);
    if (kind < MCB_OPT_ADAM || kind > MCB_OPT_MOMENTUM_SGD) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "unknown optimizer kind %d", kind);
    mcb_adam *o = new mcb_adam();
    o->opt.ctx = ctx;
    o->opt.kind = kind;
    o->opt.lr = lr;
    o->opt.beta1 = beta1;
    o->opt.beta2 = beta2;
    o->opt.eps = eps;
    o->opt.weight_decay = kind == MCB_OPT_ADAMW ? weight_decay : 0.0;
    *out = o;
    return MCB_OK;
}
mcb_status mcb_opt_set_lr(mcb_adam *opt, double lr) {
    if (!opt) return MCB_INVALID_ARGUMENT;
    opt->opt.lr = lr;
    return MCB_OK;
}
mcb_status mcb_opt_get_lr(mcb_adam *opt, double *lr_out) {
    if (!opt || !lr_out) return MCB_INVALID_ARGUMENT;
    *lr_out = opt->opt.lr;
    return MCB_OK;
}

mcb_status mcb_clip_grad_norm(mcb_var **params, int32_t n, double max_norm, double *norm_out) {
    std::vector<Var> ps = collect(params, n);
    mcb_ctx *ctx = nullptr;
    for (auto &p : ps)
        if (p) ctx = p->ctx;
    if (!ctx) {
        if (norm_out) *norm_out = 0.0;
        return max_norm > 0.0 ? MCB_OK : MCB_INVALID_ARGUMENT;
    }
    if (!(max_norm > 0.0)) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "max_norm must be positive");
    // gradient ranges: the whole flat arena in one piece when every parameter of it is listed and has a gradient
    struct Range {
        float *g;
        int64_t n;
    };
    std::vector<Range> ranges;
    Arena *a = ps[0]->arena;
    bool flat = a && ps.size() == a->vars.size();
    for (size_t i = 0; i < ps.size() && flat; ++i) flat = ps[i]->arena == a && ps[i]->arena_idx == (int)i && ps[i]->has_grad;
    std::vector<Tensor> keep;
    // Gradients on a data-parallel arena are sums over the ranks until the optimizer folds 1 / world into its
    // unscale factor; the norm reported and compared here is that of the mean, so N ranks at batch B clip like
    // one rank at batch N * B.  (A list that mixes arenas with different divisors is not meaningful; the
    // divisor of the first parameter's arena is used.)
    const double mean_factor = a ? arena_grad_divisor(a) : 1.0;
    if (flat) {
        MCB_TRY(arena_wait_comm(a));
        ranges.push_back({(float *)a->g->p, a->total}); // padding between slots is zero
    } else {
        for (auto &p : ps) {
            if (!p->has_grad) continue;
            if (p->arena) MCB_TRY(arena_wait_comm(p->arena));
            if (p->grad.dt != MCB_F32) { // clip in f32, as the reference's gradients are
                Tensor gf;
                MCB_TRY(to_dtype(ctx, p->grad, MCB_F32, &gf));
                p->grad = gf;
            }
            ranges.push_back({(float *)p->grad.ptr, p->grad.numel()});
        }
    }
    int total_blocks = 0;
    std::vector<int> blocks(ranges.size());
    for (size_t i = 0; i < ranges.size(); ++i) {
        blocks[i] = mcb_sumsq_blocks(ctx, ranges[i].n);
        if (!flat && blocks[i] > 64) blocks[i] = 64;
        total_blocks += blocks[i];
    }
    void *scratch;
    MCB_TRY(mcb_scratch(ctx, sizeof(double) * (size_t)(total_blocks + 2), &scratch));
    double *partial = (double *)scratch, *clip = partial + total_blocks;
    int at = 0;
    for (size_t i = 0; i < ranges.size(); ++i) {
        MCB_TRY(mcb_sumsq_partial(ctx, ranges[i].g, ranges[i].n, partial + at, blocks[i]));
        at += blocks[i];
    }
    MCB_TRY(mcb_clip_finalize(ctx, partial, total_blocks, max_norm, clip, mean_factor));
    for (auto &r : ranges) MCB_TRY(mcb_scale_by_clip(ctx, r.g, r.n, clip));
    if (norm_out) MCB_TRY(mcb_memcpy_d2h(ctx, norm_out, clip, sizeof(double)));
    return MCB_OK;
}

namespace {
// f64::powi as compiler-rt computes it (binary exponentiation), so StepLR matches gamma.powi(e) bit for bit
double powi_f64(double a, int32_t b) {
    const bool recip = b < 0;
    double r = 1.0;
    for (;;) {
        if (b & 1) r *= a;
        b /= 2;
        if (b == 0) break;
        a *= a;
    }
    return recip ? 1.0 / r : r;
}
} // namespace

double mcb_lr_linear_warmup_cosine(uint64_t step, uint64_t warmup_steps, uint64_t total_steps, double base_lr, double min_lr) {
    if (step < warmup_steps) {
        if (warmup_steps == 0) return base_lr;
        return base_lr * (double)step / (double)warmup_steps;
    }
    if (step >= total_steps) return min_lr;
    uint64_t span = total_steps - warmup_steps;
    double denom = (double)(span < 1 ? 1 : span);
    double progress = (double)(step - warmup_steps) / denom;
    double c = cos(3.14159265358979323846 * progress) * 0.5 + 0.5;
    return min_lr + (base_lr - min_lr) * c;
}
double mcb_lr_step(uint64_t step, double base_lr, uint64_t step_size, double gamma) {
    uint64_t ss = step_size < 1 ? 1 : step_size;
    return base_lr * powi_f64(gamma, (int32_t)(step / ss));
}
double mcb_lr_polynomial(uint64_t step, double base_lr, uint64_t total_steps, double power, double min_lr) {
    if (step == 0) return base_lr;
    double progress = (double)step / (double)(total_steps < 1 ? 1 : total_steps);
    progress = progress < 0.0 ? 0.0 : (progress > 1.0 ? 1.0 : progress);
    return min_lr + (base_lr - min_lr) * pow(1.0 - progress, power);
}

mcb_status mcb_scaler_create(mcb_ctx *ctx, double init_scale, double growth_factor, double backoff_factor,
                             int32_t growth_interval, mcb_scaler **out) {
    MCB_CHECK_CTX(ctx);
    Scaler *s = nullptr;
    MCB_TRY(scaler_create(ctx, init_scale, growth_factor, backoff_factor, growth_interval, &s));
    *out = new mcb_scaler{s};
    return MCB_OK;
}
void mcb_scaler_release(mcb_scaler *s) {
    if (!s) return;
    delete s->s;
    delete s;
}
mcb_status mcb_scaler_scale_loss(mcb_scaler *s, mcb_var *loss, mcb_var **out) {
    Var r;
    return wrap(f_scale_by_device(loss->v, s->s->state_f(), s->s->state, &r), r, out);
}
mcb_status mcb_scaler_step(mcb_scaler *s, mcb_adam *opt, mcb_var **params, int32_t n, int32_t *applied) {
    return scaler_step(s->s, &opt->opt, collect(params, n), true, applied);
}
mcb_status mcb_scaler_step_async(mcb_scaler *s, mcb_adam *opt, mcb_var **params, int32_t n) {
    return scaler_step(s->s, &opt->opt, collect(params, n), false, nullptr);
}
mcb_status mcb_scaler_state(mcb_scaler *s, double *scale_out, int32_t *growth_tracker_out, int32_t *last_found_inf) {
    struct {
        float f[2];
        int i[4];
    } st;
    MCB_TRY(mcb_memcpy_d2h(s->s->ctx, &st, s->s->state->p, sizeof(st)));
    if (scale_out) *scale_out = st.f[0];
    if (growth_tracker_out) *growth_tracker_out = st.i[0];
    if (last_found_inf) *last_found_inf = st.i[2];
    return MCB_OK;
}

mcb_status mcb_model_create(mcb_ctx *ctx, int32_t kind, const int64_t *cfg, int32_t n_cfg, mcb_model **out) {
    MCB_CHECK_CTX(ctx);
    Model *m = nullptr;
    MCB_TRY(Model::create(ctx, kind, std::vector<int64_t>(cfg, cfg + n_cfg), &m));
    *out = new mcb_model{m};
    return MCB_OK;
}
void mcb_model_release(mcb_model *m) {
    if (!m) return;
    delete m->m;
    delete m;
}
mcb_status mcb_model_num_params(mcb_model *m, int32_t *out) {
    *out = (int32_t)m->m->params.size();
    return MCB_OK;
}
mcb_status mcb_model_param(mcb_model *m, int32_t index, mcb_var **out) {
    if (index < 0 || index >= (int32_t)m->m->params.size()) return mcb_fail(m->m->ctx, MCB_OUT_OF_BOUNDS, "parameter index out of range");
    *out = new mcb_var{m->m->params[index]};
    return MCB_OK;
}
mcb_status mcb_model_loss(mcb_model *m, mcb_var *input, mcb_var *target, mcb_var **loss_out) {
    Var r;
    return wrap(m->m->loss(input->v, target->v, &r), r, loss_out);
}

} // extern "C"
