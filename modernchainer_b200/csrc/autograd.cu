// Host side of the training step: define-by-run tape, the F.* operator table, the flat
// parameter arena, Adam, GradScaler and the benchmark models.
//
// Mirrors the reference's public surface (Variable / F::* / Optimizer::update /
// GradScaler::step; crates/modern-chainer-autograd/src/{variable,node,ops,host_ops}.rs,
// crates/modern-chainer-optim/src/{lib,amp}.rs, crates/modern-chainer-nn/src/lib.rs) with a
// different engine underneath:
//   * fan-in gradients are accumulated in place when the pending tensor is uniquely owned
//     (the reference allocates a new tensor per add, variable.rs:196,212);
//   * gradients are kept on leaves only, not on every intermediate;
//   * parameter gradients are produced straight into a flat arena when possible, and the
//     walker reports each finished parameter so gradient buckets can be all-reduced while
//     the rest of backward still runs;
//   * no step of backward reads a value back to the host (the reference synchronises in
//     SoftmaxCrossEntropy::backward, Sum/Mean::backward and every sum_to that is not the
//     bias case, ops.rs:268-301,346-348 and cuda/src/ops.rs:893-918);
//   * reshape is a view (a download/upload round trip in the reference, host_ops.rs:659-703).
#include <cmath>
#include <cstring>
#include <functional>
#include <memory>
#include <unordered_map>
#include <unordered_set>

#include "autograd.h"

namespace mcbag {

// Grad mode and autocast are per host thread, as in the reference (thread-local cells in
// crates/modern-chainer-autograd/src/lib.rs:20-22 and crates/modern-chainer-core/src/autocast.rs:6-8):
// two threads driving two contexts do not see each other's no_grad / autocast scopes.
static thread_local bool g_grad_enabled = true;
static thread_local int g_autocast = -1;

bool grad_enabled() { return g_grad_enabled; }
int autocast() { return g_autocast; }
void set_grad_enabled(bool on) { g_grad_enabled = on; }
void set_autocast(int dt) { g_autocast = dt; }

// ------------------------------------------------------------------ tensors
int64_t Tensor::numel() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
}

mcb_status new_tensor(mcb_ctx *ctx, int dt, const std::vector<int64_t> &shape, Tensor *out) {
    Tensor t;
    t.dt = dt;
    t.shape = shape;
    void *p = nullptr;
    MCB_TRY(mcb_alloc(ctx, (size_t)t.numel() * mcb_dtype_size(dt), &p));
    t.buf = std::make_shared<Buf>(ctx, p);
    t.ptr = p;
    t.defined = true;
    *out = t;
    return MCB_OK;
}

Tensor view(const Tensor &t, const std::vector<int64_t> &shape) {
    Tensor v = t;
    v.shape = shape;
    return v;
}

// returns `t` itself when it already has storage type `dt`, else a converted copy
mcb_status to_dtype(mcb_ctx *ctx, const Tensor &t, int dt, Tensor *out) {
    if (t.dt == dt) {
        *out = t;
        return MCB_OK;
    }
    if (t.dt != MCB_F32 && dt != MCB_F32) { // bf16 <-> f16: through f32 (every bf16 and f16 value is exact in f32)
        Tensor f;
        MCB_TRY(new_tensor(ctx, MCB_F32, t.shape, &f));
        MCB_TRY(mcb_cast(ctx, t.ptr, t.dt, f.ptr, MCB_F32, t.numel()));
        MCB_TRY(new_tensor(ctx, dt, t.shape, out));
        return mcb_cast(ctx, f.ptr, MCB_F32, out->ptr, dt, t.numel());
    }
    MCB_TRY(new_tensor(ctx, dt, t.shape, out));
    return mcb_cast(ctx, t.ptr, t.dt, out->ptr, dt, t.numel());
}

static bool is_float(int dt) { return dt == MCB_F32 || dt == MCB_BF16 || dt == MCB_F16; }
static bool is_lp(int dt) { return dt == MCB_BF16 || dt == MCB_F16; }
// storage type of the sum of two gradients: f32 unless both are the same 16-bit type
static int sum_dtype(int a, int b) { return (is_lp(a) && a == b) ? a : MCB_F32; }

// ------------------------------------------------------------------ apply
Var make_var(mcb_ctx *ctx, const Tensor &data, bool requires_grad) {
    Var v = std::make_shared<VarImpl>();
    v->ctx = ctx;
    v->data = data;
    v->requires_grad = requires_grad;
    return v;
}

// wraps an op result: attaches the node only when grad mode is on and an input needs it
static Var apply(mcb_ctx *ctx, const char *name, const Tensor &out, const std::vector<Var> &inputs, BackwardFn bwd) {
    bool need = false;
    for (auto &i : inputs) need = need || i->requires_grad;
    Var v = make_var(ctx, out, g_grad_enabled && need);
    if (v->requires_grad) {
        auto n = std::make_shared<Node>();
        n->name = name;
        n->inputs = inputs;
        n->backward = std::move(bwd);
        v->node = n;
    }
    return v;
}

// ------------------------------------------------------------------ arena helpers
static Tensor slot_view(const Var &v) {
    Arena *a = v->arena;
    Tensor t;
    t.buf = a->g;
    t.ptr = (float *)a->g->p + a->off[v->arena_idx];
    t.dt = MCB_F32;
    t.shape = v->data.shape;
    t.defined = true;
    return t;
}

// Where an op should write the gradient of input `v`: the arena slot when it is still empty
// and nobody claimed it during this backward pass, otherwise a fresh tensor.
static mcb_status grad_dst(const Var &v, Tensor *out, bool *direct) {
    if (v->arena && !v->has_grad && !v->slot_claimed) {
        v->slot_claimed = true;
        v->arena->claimed.push_back(v.get());
        *out = slot_view(v);
        *direct = true;
        return MCB_OK;
    }
    *direct = false;
    return new_tensor(v->ctx, MCB_F32, v->data.shape, out);
}

// While a node's backward runs, the walker exposes, per input, the gradient that is already
// waiting for that input if the walker holds its only reference.  An op that can add into such
// a tensor in place returns it as the input's gradient and the walker skips its own fan-in add.
static thread_local const std::vector<const Tensor *> *g_pending = nullptr; // set by the walker of this thread around each node's backward
static const Tensor *pending_grad(size_t input) {
    if (!g_pending || input >= g_pending->size()) return nullptr;
    return (*g_pending)[input];
}

// ------------------------------------------------------------------ backward walker
static mcb_status accumulate_leaf(const Var &v, const Tensor &g) {
    mcb_ctx *ctx = v->ctx;
    if (v->arena) {
        Tensor slot = slot_view(v);
        Tensor gf;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        if (!v->has_grad) {
            if (gf.ptr != slot.ptr) MCB_TRY(mcb_memcpy_d2d(ctx, slot.ptr, gf.ptr, sizeof(float) * slot.numel()));
        } else {
            MCB_TRY(mcb_add_inplace(ctx, slot.ptr, gf.ptr, slot.numel(), MCB_F32));
        }
        v->grad = slot;
        v->has_grad = true;
        return arena_grad_ready(v->arena, v->arena_idx);
    }
    if (!v->has_grad) {
        v->grad = g;
        v->has_grad = true;
        return MCB_OK;
    }
    if (v->grad.buf && v->grad.buf.use_count() == 1 && v->grad.dt == g.dt) {
        return mcb_add_inplace(ctx, v->grad.ptr, g.ptr, g.numel(), g.dt);
    }
    Tensor sum;
    int dt = sum_dtype(v->grad.dt, g.dt);
    MCB_TRY(new_tensor(ctx, dt, g.shape, &sum));
    MCB_TRY(mcb_add_typed(ctx, v->grad.ptr, v->grad.dt, g.ptr, g.dt, sum.ptr, dt, g.numel()));
    v->grad = sum;
    return MCB_OK;
}

mcb_status backward(const Var &root) {
    if (!root->requires_grad || !g_grad_enabled) return MCB_OK;
    mcb_ctx *ctx = root->ctx;
    // iterative post-order DFS (same visiting rule as Variable::backward, variable.rs:158-175)
    std::vector<Var> order;
    std::unordered_set<VarImpl *> seen;
    std::vector<std::pair<Var, bool>> stack;
    // How many node inputs each leaf feeds.  The visiting order puts the leaves last, but a leaf's gradient is
    // final as soon as its last consumer has run: it is stored then (same value, same order of additions), so a
    // data-parallel bucket can start its all-reduce while the rest of backward still runs.
    std::unordered_map<VarImpl *, int> leaf_uses;
    stack.emplace_back(root, false);
    while (!stack.empty()) {
        auto top = stack.back();
        stack.pop_back();
        if (top.second) {
            order.push_back(top.first);
            continue;
        }
        if (!seen.insert(top.first.get()).second) continue;
        stack.emplace_back(top.first, true);
        if (top.first->node)
            for (auto &in : top.first->node->inputs) {
                stack.emplace_back(in, false);
                if (!in->node && in->requires_grad) ++leaf_uses[in.get()];
            }
    }
    // a data-parallel arena takes one backward pass per optimizer step: refused here, before anything is enqueued
    {
        std::vector<Arena *> begun;
        for (auto &lu : leaf_uses) {
            Arena *a = lu.first->arena;
            if (!a || std::find(begun.begin(), begun.end(), a) != begun.end()) continue;
            begun.push_back(a);
            MCB_TRY(arena_backward_begin(a));
        }
    }
    std::unordered_map<VarImpl *, Tensor> grads;
    {
        Tensor seed;
        MCB_TRY(new_tensor(ctx, MCB_F32, root->data.shape, &seed));
        MCB_TRY(mcb_fill(ctx, (float *)seed.ptr, 1.0f, seed.numel()));
        if (root->data.dt != MCB_F32) {
            Tensor s2;
            MCB_TRY(to_dtype(ctx, seed, root->data.dt, &s2));
            seed = s2;
        }
        grads[root.get()] = seed;
    }
    std::vector<Arena *> touched;
    mcb_status st = MCB_OK;
    auto store_leaf = [&](const Var &leaf, const Tensor &g) -> mcb_status {
        if (leaf->arena && std::find(touched.begin(), touched.end(), leaf->arena) == touched.end()) touched.push_back(leaf->arena);
        return accumulate_leaf(leaf, g);
    };
    // a node is done with (it ran, or no gradient reached it): leaves it was the last consumer of are stored now
    auto release_inputs = [&](const Var &v) -> mcb_status {
        for (const Var &in : v->node->inputs) {
            if (in->node || !in->requires_grad) continue;
            auto u = leaf_uses.find(in.get());
            if (u == leaf_uses.end() || --u->second > 0) continue;
            auto e = grads.find(in.get());
            if (e == grads.end()) continue;
            Tensor g = e->second;
            grads.erase(e);
            MCB_TRY(store_leaf(in, g));
        }
        return MCB_OK;
    };
    for (auto it = order.rbegin(); it != order.rend() && st == MCB_OK; ++it) {
        const Var &v = *it;
        auto f = grads.find(v.get());
        if (f == grads.end()) {
            if (v->node) st = release_inputs(v);
            continue;
        }
        Tensor g = f->second;
        grads.erase(f);
        if (!v->node) {
            st = store_leaf(v, g);
            continue;
        }
        std::vector<Tensor> in_grads(v->node->inputs.size());
        std::vector<const Tensor *> pending(v->node->inputs.size(), nullptr);
        for (size_t i = 0; i < pending.size(); ++i) {
            const Var &in = v->node->inputs[i];
            if (!in->requires_grad || in.get() == v.get()) continue;
            bool repeated = false; // the same variable twice among the inputs: no in-place target
            for (size_t j = 0; j < pending.size(); ++j) repeated |= (j != i && v->node->inputs[j].get() == in.get());
            auto e = grads.find(in.get());
            if (!repeated && e != grads.end() && e->second.buf && e->second.buf.use_count() == 1) pending[i] = &e->second;
        }
        g_pending = &pending;
        st = v->node->backward(g, in_grads);
        g_pending = nullptr;
        if (st != MCB_OK) break;
        g = Tensor(); // drop our reference so a pending tensor can be uniquely owned
        for (size_t i = 0; i < in_grads.size(); ++i) {
            const Var &in = v->node->inputs[i];
            if (!in_grads[i].defined || !in->requires_grad) continue;
            auto e = grads.find(in.get());
            if (e == grads.end()) {
                grads.emplace(in.get(), in_grads[i]);
                continue;
            }
            Tensor &cur = e->second;
            if (in_grads[i].ptr == cur.ptr && in_grads[i].buf == cur.buf) { // the op already added into the pending tensor
                cur.aux = in_grads[i].aux; // by-products of the kernel that wrote the new values (or none)
                in_grads[i] = Tensor();
                continue;
            }
            Tensor add = in_grads[i];
            in_grads[i] = Tensor();
            if (cur.buf && cur.buf.use_count() == 1 && cur.dt == add.dt) {
                st = mcb_add_inplace(ctx, cur.ptr, add.ptr, cur.numel(), cur.dt);
                cur.aux.reset(); // the values changed
            } else if (add.buf && add.buf.use_count() == 1 && cur.dt == add.dt) {
                st = mcb_add_inplace(ctx, add.ptr, cur.ptr, cur.numel(), cur.dt);
                cur = add;
                cur.aux.reset();
            } else {
                Tensor sum;
                int dt = sum_dtype(cur.dt, add.dt);
                st = new_tensor(ctx, dt, cur.shape, &sum);
                if (st == MCB_OK) st = mcb_add_typed(ctx, cur.ptr, cur.dt, add.ptr, add.dt, sum.ptr, dt, cur.numel());
                cur = sum;
            }
            if (st != MCB_OK) break;
        }
        if (st == MCB_OK) st = release_inputs(v);
    }
    for (Arena *a : touched) {
        for (VarImpl *c : a->claimed) c->slot_claimed = false;
        a->claimed.clear();
    }
    return st;
}

// ------------------------------------------------------------------ F.*
static mcb_status check_same_ctx(const Var &a, const Var &b) {
    if (a->ctx != b->ctx) return mcb_fail(a->ctx, MCB_INVALID_ARGUMENT, "variables live on different contexts");
    return MCB_OK;
}

static mcb_status f32_of(const Var &v, Tensor *out) { return to_dtype(v->ctx, v->data, MCB_F32, out); }

// un-broadcast `g` to `shape` (Ops::sum_to); equal shapes alias, no copy
static mcb_status sum_to_shape(mcb_ctx *ctx, const Tensor &g, const std::vector<int64_t> &shape, Tensor *out) {
    if (g.shape == shape) {
        *out = g;
        return MCB_OK;
    }
    Tensor gf;
    MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
    MCB_TRY(new_tensor(ctx, MCB_F32, shape, out));
    return mcb_sum_to(ctx, (const float *)gf.ptr, gf.shape.data(), (int)gf.shape.size(), shape.data(), (int)shape.size(), (float *)out->ptr);
}

static mcb_status bin(mcb_ctx *ctx, int op, const Tensor &a, const Tensor &b, Tensor *out) {
    std::vector<int64_t> os;
    size_t r = std::max(a.shape.size(), b.shape.size());
    os.resize(r);
    for (size_t i = 0; i < r; ++i) {
        int64_t x = i >= r - a.shape.size() ? a.shape[i - (r - a.shape.size())] : 1;
        int64_t y = i >= r - b.shape.size() ? b.shape[i - (r - b.shape.size())] : 1;
        if (x != y && x != 1 && y != 1) return mcb_fail(ctx, MCB_BROADCAST, "shapes do not broadcast");
        os[i] = x == 1 ? y : x;
    }
    MCB_TRY(new_tensor(ctx, MCB_F32, os, out));
    return mcb_binary(ctx, op, (const float *)a.ptr, a.shape.data(), (int)a.shape.size(), (const float *)b.ptr, b.shape.data(),
                      (int)b.shape.size(), (float *)out->ptr);
}
static mcb_status scaled(mcb_ctx *ctx, const Tensor &x, double f, Tensor *out) {
    MCB_TRY(new_tensor(ctx, MCB_F32, x.shape, out));
    return mcb_scale(ctx, (const float *)x.ptr, f, (float *)out->ptr, x.numel());
}
// cast a gradient to the storage type of the input it belongs to
static mcb_status like_input(mcb_ctx *ctx, const Tensor &g, const Var &in, Tensor *out) {
    int want = is_float(in->data.dt) ? in->data.dt : MCB_F32;
    return to_dtype(ctx, g, want, out);
}
// Same, except that an f32 gradient for the bf16 output of a Linear stays f32: that op's backward
// rounds its incoming gradient to bf16 as its first step anyway (same values), and does so in the
// pass that also produces the bias gradient, so rounding here would only add a kernel.
static mcb_status like_input_lazy(mcb_ctx *ctx, const Tensor &g, const Var &in, Tensor *out) {
    if (g.dt == MCB_F32 && is_lp(in->data.dt) && in->node && !knob_on(ctx, K_UNFUSED_BWD) &&
        (!strcmp(in->node->name, "Linear") || !strcmp(in->node->name, "LinearActivation"))) {
        *out = g;
        return MCB_OK;
    }
    return like_input(ctx, g, in, out);
}

void binary_node(mcb_ctx *ctx, int op, const Var &a, const Var &b, const Tensor &res, Var *out);

mcb_status f_binary(int op, const Var &a, const Var &b, Var *out) {
    MCB_TRY(check_same_ctx(a, b));
    mcb_ctx *ctx = a->ctx;
    if (!is_float(a->data.dt) || !is_float(b->data.dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "arithmetic needs floating-point operands");
    Tensor res;
    bool mixed = (a->data.dt != MCB_F32 || b->data.dt != MCB_F32);
    if (op == MCB_ADD && a->data.shape == b->data.shape && mixed) {
        // residual add with a low-precision operand: one pass, f32 result unless both are bf16
        int odt = sum_dtype(a->data.dt, b->data.dt);
        MCB_TRY(new_tensor(ctx, odt, a->data.shape, &res));
        MCB_TRY(mcb_add_typed(ctx, a->data.ptr, a->data.dt, b->data.ptr, b->data.dt, res.ptr, odt, res.numel()));
    } else {
        Tensor af, bf;
        MCB_TRY(f32_of(a, &af));
        MCB_TRY(f32_of(b, &bf));
        MCB_TRY(bin(ctx, op, af, bf, &res));
    }
    binary_node(ctx, op, a, b, res, out);
    return MCB_OK;
}

// the tape node of a + b, a - b, a * b, a / b over an already computed result
void binary_node(mcb_ctx *ctx, int op, const Var &a, const Var &b, const Tensor &res, Var *out) {
    Var av = a, bv = b;
    *out = apply(ctx, "Binary", res, {a, b}, [ctx, op, av, bv](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        const std::vector<int64_t> &as = av->data.shape, &bs = bv->data.shape;
        Tensor ga, gb;
        if (op == MCB_ADD || op == MCB_SUB) {
            if (av->requires_grad) {
                MCB_TRY(sum_to_shape(ctx, g, as, &ga));
                MCB_TRY(like_input_lazy(ctx, ga, av, &gi[0]));
            }
            if (bv->requires_grad) {
                Tensor t = g;
                if (op == MCB_SUB) {
                    Tensor gf;
                    MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
                    MCB_TRY(scaled(ctx, gf, -1.0, &t));
                }
                MCB_TRY(sum_to_shape(ctx, t, bs, &gb));
                MCB_TRY(like_input_lazy(ctx, gb, bv, &gi[1]));
            }
            return MCB_OK;
        }
        Tensor gf, af, bf;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        MCB_TRY(f32_of(av, &af));
        MCB_TRY(f32_of(bv, &bf));
        if (op == MCB_MUL) {
            if (av->requires_grad) {
                Tensor t;
                MCB_TRY(bin(ctx, MCB_MUL, gf, bf, &t));
                MCB_TRY(sum_to_shape(ctx, t, as, &ga));
                MCB_TRY(like_input(ctx, ga, av, &gi[0]));
            }
            if (bv->requires_grad) {
                Tensor t;
                MCB_TRY(bin(ctx, MCB_MUL, gf, af, &t));
                MCB_TRY(sum_to_shape(ctx, t, bs, &gb));
                MCB_TRY(like_input(ctx, gb, bv, &gi[1]));
            }
            return MCB_OK;
        }
        // div: ga = g / b ; gb = -(g * a) / (b * b)   (autograd/src/ops.rs:97-128)
        if (av->requires_grad) {
            Tensor t;
            MCB_TRY(bin(ctx, MCB_DIV, gf, bf, &t));
            MCB_TRY(sum_to_shape(ctx, t, as, &ga));
            MCB_TRY(like_input(ctx, ga, av, &gi[0]));
        }
        if (bv->requires_grad) {
            Tensor denom, numer, q, neg;
            MCB_TRY(bin(ctx, MCB_MUL, bf, bf, &denom));
            MCB_TRY(bin(ctx, MCB_MUL, gf, af, &numer));
            MCB_TRY(bin(ctx, MCB_DIV, numer, denom, &q));
            MCB_TRY(scaled(ctx, q, -1.0, &neg));
            MCB_TRY(sum_to_shape(ctx, neg, bs, &gb));
            MCB_TRY(like_input(ctx, gb, bv, &gi[1]));
        }
        return MCB_OK;
    });
}

mcb_status f_scale(const Var &x, double factor, Var *out) {
    mcb_ctx *ctx = x->ctx;
    Tensor xf, res;
    MCB_TRY(f32_of(x, &xf));
    MCB_TRY(scaled(ctx, xf, factor, &res));
    Var xv = x;
    *out = apply(ctx, "Scale", res, {x}, [ctx, factor, xv](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gf, t;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        MCB_TRY(scaled(ctx, gf, factor, &t));
        return like_input(ctx, t, xv, &gi[0]);
    });
    return MCB_OK;
}

// y = x * (*scalar) with the scalar resident on the device (GradScaler::scale_loss without a host value)
mcb_status f_scale_by_device(const Var &x, const float *scalar, std::shared_ptr<Buf> keep, Var *out) {
    mcb_ctx *ctx = x->ctx;
    Tensor xf, res;
    MCB_TRY(f32_of(x, &xf));
    MCB_TRY(new_tensor(ctx, MCB_F32, xf.shape, &res));
    MCB_TRY(mcb_mul_scalar_ptr(ctx, xf.ptr, scalar, res.ptr, xf.numel(), MCB_F32));
    Var xv = x;
    *out = apply(ctx, "ScaleLoss", res, {x}, [ctx, scalar, keep, xv](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gf, t;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        MCB_TRY(new_tensor(ctx, MCB_F32, gf.shape, &t));
        MCB_TRY(mcb_mul_scalar_ptr(ctx, gf.ptr, scalar, t.ptr, gf.numel(), MCB_F32));
        return like_input(ctx, t, xv, &gi[0]);
    });
    return MCB_OK;
}

mcb_status f_unary(int op, const Var &x, Var *out) {
    mcb_ctx *ctx = x->ctx;
    if (op < MCB_EXP || op > MCB_NEG) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "unknown unary op %d", op);
    Tensor xf, res;
    MCB_TRY(f32_of(x, &xf));
    MCB_TRY(new_tensor(ctx, MCB_F32, xf.shape, &res));
    MCB_TRY(mcb_unary(ctx, op, (const float *)xf.ptr, (float *)res.ptr, xf.numel()));
    Var xv = x;
    *out = apply(ctx, "Unary", res, {x}, [ctx, op, xv, xf, res](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gf, t;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        switch (op) {
        case MCB_EXP: MCB_TRY(bin(ctx, MCB_MUL, gf, res, &t)); break;        // g * y
        case MCB_LOG: MCB_TRY(bin(ctx, MCB_DIV, gf, xf, &t)); break;         // g / x
        case MCB_SQRT: {                                                      // g / (2 y)
            Tensor two_y;
            MCB_TRY(scaled(ctx, res, 2.0, &two_y));
            MCB_TRY(bin(ctx, MCB_DIV, gf, two_y, &t));
            break;
        }
        case MCB_SIGMOID: {                                                   // g * y * (1 - y)
            Tensor ones, om, ym;
            MCB_TRY(new_tensor(ctx, MCB_F32, res.shape, &ones));
            MCB_TRY(mcb_fill(ctx, (float *)ones.ptr, 1.0f, ones.numel()));
            MCB_TRY(bin(ctx, MCB_SUB, ones, res, &om));
            MCB_TRY(bin(ctx, MCB_MUL, res, om, &ym));
            MCB_TRY(bin(ctx, MCB_MUL, gf, ym, &t));
            break;
        }
        case MCB_NEG: MCB_TRY(scaled(ctx, gf, -1.0, &t)); break;
        default: return mcb_fail(ctx, MCB_UNSUPPORTED, "backward of this unary op is not on the training path");
        }
        return like_input(ctx, t, xv, &gi[0]);
    });
    return MCB_OK;
}

static mcb_status f_act(const Var &x, bool gelu, Var *out) {
    mcb_ctx *ctx = x->ctx;
    if (!is_float(x->data.dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "activation needs a floating-point input");
    Tensor res;
    MCB_TRY(new_tensor(ctx, x->data.dt, x->data.shape, &res));
    MCB_TRY((gelu ? mcb_gelu : mcb_relu)(ctx, x->data.ptr, res.ptr, res.numel(), x->data.dt));
    Tensor xd = x->data;
    *out = apply(ctx, gelu ? "GELU" : "ReLU", res, {x}, [ctx, gelu, xd](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gg;
        MCB_TRY(to_dtype(ctx, g, xd.dt, &gg));
        MCB_TRY(new_tensor(ctx, xd.dt, xd.shape, &gi[0]));
        return (gelu ? mcb_gelu_backward : mcb_relu_backward)(ctx, xd.ptr, gg.ptr, gi[0].ptr, xd.numel(), xd.dt);
    });
    return MCB_OK;
}
mcb_status f_relu(const Var &x, Var *out) { return f_act(x, false, out); }
mcb_status f_gelu(const Var &x, Var *out) { return f_act(x, true, out); }

static mcb_status f_sum_mean(const Var &x, bool mean, Var *out) {
    mcb_ctx *ctx = x->ctx;
    Tensor xf, res;
    MCB_TRY(f32_of(x, &xf));
    MCB_TRY(new_tensor(ctx, MCB_F32, {}, &res));
    int64_t n = xf.numel();
    double factor = mean ? 1.0 / (double)(n > 1 ? n : 1) : 1.0;
    // Mean = sum_all then scale(1/n): the f32 sum is rounded before the scale in the reference
    if (mean) {
        Tensor s;
        MCB_TRY(new_tensor(ctx, MCB_F32, {}, &s));
        MCB_TRY(mcb_sum_all(ctx, (const float *)xf.ptr, n, (float *)s.ptr));
        MCB_TRY(mcb_scale(ctx, (const float *)s.ptr, factor, (float *)res.ptr, 1));
    } else {
        MCB_TRY(mcb_sum_all(ctx, (const float *)xf.ptr, n, (float *)res.ptr));
    }
    Var xv = x;
    *out = apply(ctx, mean ? "Mean" : "Sum", res, {x}, [ctx, factor, xv](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gf, t;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        MCB_TRY(new_tensor(ctx, MCB_F32, xv->data.shape, &t));
        MCB_TRY(mcb_fill_from_scalar(ctx, (float *)t.ptr, (const float *)gf.ptr, factor, t.numel()));
        return like_input(ctx, t, xv, &gi[0]);
    });
    return MCB_OK;
}
mcb_status f_sum(const Var &x, Var *out) { return f_sum_mean(x, false, out); }
mcb_status f_mean(const Var &x, Var *out) { return f_sum_mean(x, true, out); }

// ---- GEMM helpers ----------------------------------------------------------------------
// The 16-bit type linear / matmul / attention are lowered to, or -1: the autocast scope of this thread first
// (core/src/autocast.rs:10-44), else the context's compute type (cuda/src/backend.rs:109-136).
static int lowp_dtype(mcb_ctx *ctx) {
    if (is_lp(g_autocast)) return g_autocast;
    if (ctx->compute == MCB_COMPUTE_BF16) return MCB_BF16;
    if (ctx->compute == MCB_COMPUTE_F16) return MCB_F16;
    return -1;
}
static bool tc_shape_ok(int64_t m, int64_t n, int64_t k) { return m > 0 && (n % 8 == 0) && (k % 8 == 0) && n > 0 && k > 0; }

// 16-bit operand (type lp) for `v`: the arena's shadow copy for parameters, the tensor itself when it
// already has that type, otherwise a converted copy
static mcb_status lowp_of(const Var &v, int lp, Tensor *out) {
    if (v->data.dt == lp) {
        *out = v->data;
        return MCB_OK;
    }
    if (v->arena) {
        MCB_TRY(arena_refresh_shadow(v->arena, lp));
        Tensor t;
        t.buf = v->arena->shadow;
        t.ptr = (uint16_t *)v->arena->shadow->p + v->arena->off[v->arena_idx];
        t.dt = lp;
        t.shape = v->data.shape;
        t.defined = true;
        *out = t;
        return MCB_OK;
    }
    return to_dtype(v->ctx, v->data, lp, out);
}

static int pick_split_k(mcb_ctx *ctx, int64_t m, int64_t n, int64_t k) {
    int64_t tiles = ((m + 127) / 128) * ((n + 255) / 256);
    int64_t kb = (k + 63) / 64;
    if (tiles >= ctx->sm_count || kb < 8) return 1;
    int64_t s = (ctx->sm_count + tiles - 1) / tiles;
    if (s > kb / 4) s = kb / 4;
    if (s < 1) s = 1;
    if (s > 32) s = 32;
    return (int)s;
}

struct LinearSaved {
    Tensor x;      // activation as used by the forward GEMM (16-bit under autocast, else f32)
    Tensor pre;    // pre-activation (linear_activation only)
    bool bf16 = false; // the op ran on the tensor cores with 16-bit operands of type lp
    int lp = MCB_BF16;
    bool emulated = false; // operands rounded to lp, product on the exact-f32 kernel (shapes the tensor-core kernel declines)
    int act = MCB_ACT_NONE;
};

// shared backward of linear / linear_activation: g is the gradient w.r.t. the op output
static mcb_status linear_backward_impl(mcb_ctx *ctx, const Tensor &g_in, const LinearSaved &sv, const Var &x, const Var &w,
                                       const Var &b, std::vector<Tensor> &gi) {
    int64_t m = sv.x.numel() / sv.x.shape.back(), k = sv.x.shape.back(), n = w->data.shape[0];
    int gdt = sv.bf16 ? sv.lp : MCB_F32;
    Tensor g;
    // The bias gradient is the column sum of the bf16 gradient the GEMMs below read.  Whenever a
    // pass over that gradient is needed anyway (a cast from f32, the activation's backward), the
    // same pass leaves the column sums, and no separate reduction reads the matrix again.
    const bool fuse = !knob_on(ctx, K_UNFUSED_BWD); // test knob: separate cast / activation-backward / column-sum kernels
    const bool want_db = b && b->requires_grad;
    bool db_done = false;
    if (fuse && sv.bf16 && sv.act == MCB_ACT_NONE && g_in.dt == MCB_F32 && g_in.aux && g_in.aux->bf16.numel() == g_in.numel() && g_in.aux->bf16.dt == sv.lp &&
        g_in.aux->colsum.numel() == n && !g_in.shape.empty() && g_in.shape.back() == n) {
        // the kernel that wrote this f32 gradient (LayerNorm backward on the residual stream) already left it rounded to
        // bf16 together with the column sums of the rounded values: nothing to read again
        g = g_in.aux->bf16;
        g.shape = g_in.shape;
        if (want_db) {
            gi[2] = g_in.aux->colsum;
            db_done = true;
        }
    } else if (fuse && sv.bf16 && want_db && sv.act == MCB_ACT_NONE && g_in.dt == MCB_F32 && mcb_map_colsum_supported(g_in.ptr, nullptr, g_in.ptr, n)) {
        bool direct;
        MCB_TRY(grad_dst(b, &gi[2], &direct));
        MCB_TRY(new_tensor(ctx, sv.lp, g_in.shape, &g));
        MCB_TRY(mcb_map_colsum(ctx, 0, g_in.ptr, nullptr, g.ptr, m, n, (float *)gi[2].ptr, sv.lp));
        db_done = true;
    } else {
        MCB_TRY(to_dtype(ctx, g_in, gdt, &g));
    }
    if (sv.act != MCB_ACT_NONE) {
        Tensor gp;
        MCB_TRY(new_tensor(ctx, gdt, g.shape, &gp));
        if (fuse && sv.bf16 && want_db && mcb_map_colsum_supported(sv.pre.ptr, g.ptr, gp.ptr, n)) {
            bool direct;
            MCB_TRY(grad_dst(b, &gi[2], &direct));
            MCB_TRY(mcb_map_colsum(ctx, sv.act == MCB_ACT_GELU ? 1 : 2, sv.pre.ptr, g.ptr, gp.ptr, m, n, (float *)gi[2].ptr, sv.lp));
            db_done = true;
        } else {
            MCB_TRY((sv.act == MCB_ACT_GELU ? mcb_gelu_backward : mcb_relu_backward)(ctx, sv.pre.ptr, g.ptr, gp.ptr, g.numel(), gdt));
        }
        g = gp;
    }
    if (sv.bf16) {
        // The weight gradient first in the books: where it goes and whether its reduction is split.  A split one adds its
        // slices into an output that must be zero: the data-gradient GEMM in front of it clears that buffer on the side
        // (its epilogue warps are idle until the first tile is done), which saves a fill of its own per Linear.
        TcGemmParams pw; // dw[n,k] = g^T[n,m] * x[m,k]
        bool clear_dw = false;
        if (w->requires_grad) {
            bool direct;
            MCB_TRY(grad_dst(w, &gi[1], &direct));
            pw.in_dt = sv.lp;
            pw.a = g.ptr; pw.a_mn_major = 1; pw.lda = n;
            pw.b = sv.x.ptr; pw.b_mn_major = 1; pw.ldb = k;
            pw.d = gi[1].ptr; pw.out_dt = MCB_F32; pw.ldd = k;
            pw.m = n; pw.n = k; pw.k = m;
            mcb_tc_plan(ctx, n, k, m, true, false, 1, &pw.bn, &pw.split_k);
            if (pw.split_k > 1) {
                pw.accumulate = 1;
                clear_dw = true;
            }
        }
        if (x->requires_grad) {
            Tensor wb;
            MCB_TRY(lowp_of(w, sv.lp, &wb));
            int xdt = x->data.dt == sv.lp ? sv.lp : MCB_F32;
            MCB_TRY(new_tensor(ctx, xdt, x->data.shape, &gi[0]));
            TcGemmParams p; // dx[m,k] = g[m,n] * W[n,k]
            p.in_dt = sv.lp;
            p.a = g.ptr; p.a_mn_major = 0; p.lda = n;
            p.b = wb.ptr; p.b_mn_major = 1; p.ldb = k;
            p.d = gi[0].ptr; p.out_dt = xdt; p.ldd = k;
            p.m = m; p.n = k; p.k = n;
            if (clear_dw && m > 0 && mcb_aligned16(gi[1].ptr) && (sizeof(float) * n * k) % 16 == 0) {
                p.zero_ptr = gi[1].ptr;
                p.zero_bytes = sizeof(float) * n * k;
                clear_dw = false;
            }
            MCB_TRY(mcb_tc_gemm(ctx, p));
        }
        if (w->requires_grad) {
            if (clear_dw) MCB_TRY(mcb_memset(ctx, gi[1].ptr, 0, sizeof(float) * n * k));
            MCB_TRY(mcb_tc_gemm(ctx, pw));
        }
    } else {
        float *dx = nullptr, *dw = nullptr;
        if (x->requires_grad) {
            MCB_TRY(new_tensor(ctx, MCB_F32, x->data.shape, &gi[0]));
            dx = (float *)gi[0].ptr;
        }
        if (w->requires_grad) {
            bool direct;
            MCB_TRY(grad_dst(w, &gi[1], &direct));
            dw = (float *)gi[1].ptr;
        }
        Tensor wf = w->data;
        if (sv.emulated) { // same rounding points as the tensor-core path: gradient and weight rounded to the 16-bit type
            Tensor t;
            MCB_TRY(to_dtype(ctx, g, sv.lp, &t));
            MCB_TRY(to_dtype(ctx, t, MCB_F32, &g));
            MCB_TRY(to_dtype(ctx, w->data, sv.lp, &t));
            MCB_TRY(to_dtype(ctx, t, MCB_F32, &wf));
        }
        MCB_TRY(mcb_linear_backward(ctx, (const float *)g.ptr, (const float *)sv.x.ptr, (const float *)wf.ptr, dx, dw, nullptr, m, k, n));
        if (x->requires_grad && is_lp(x->data.dt)) {
            Tensor t;
            MCB_TRY(to_dtype(ctx, gi[0], x->data.dt, &t));
            gi[0] = t;
        }
    }
    if (want_db && !db_done) {
        bool direct;
        MCB_TRY(grad_dst(b, &gi[2], &direct));
        MCB_TRY(mcb_col_sum(ctx, g.ptr, gdt, m, n, (float *)gi[2].ptr));
    }
    return MCB_OK;
}

static mcb_status f_linear_impl(const Var &x, const Var &w, const Var &b, int act, Var *out) {
    MCB_TRY(check_same_ctx(x, w));
    mcb_ctx *ctx = x->ctx;
    if (w->data.shape.size() != 2 || x->data.shape.empty() || x->data.shape.back() != w->data.shape[1])
        return mcb_fail(ctx, MCB_SHAPE_MISMATCH, "linear: x [..., in] and weight [out, in] do not match");
    if (b && (b->data.shape.size() != 1 || b->data.shape[0] != w->data.shape[0]))
        return mcb_fail(ctx, MCB_SHAPE_MISMATCH, "linear: bias must be [out]");
    if (!is_float(x->data.dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "linear needs a floating-point input");
    int64_t k = w->data.shape[1], n = w->data.shape[0], m = x->data.numel() / (k > 0 ? k : 1);
    std::vector<int64_t> oshape = x->data.shape;
    oshape.back() = n;
    auto sv = std::make_shared<LinearSaved>();
    sv->act = act;
    const int lp = lowp_dtype(ctx);
    sv->bf16 = lp >= 0 && tc_shape_ok(m, n, k);
    sv->emulated = lp >= 0 && !sv->bf16 && m > 0 && n > 0 && k > 0;
    if (lp >= 0) sv->lp = lp;
    Tensor res;
    if (sv->bf16) {
        Tensor wb;
        MCB_TRY(to_dtype(ctx, x->data, lp, &sv->x));
        MCB_TRY(lowp_of(w, lp, &wb));
        MCB_TRY(new_tensor(ctx, lp, oshape, &res));
        TcGemmParams p; // y[m,n] = x[m,k] * W[n,k]^T + bias
        p.in_dt = lp;
        p.a = sv->x.ptr; p.lda = k;
        p.b = wb.ptr; p.ldb = k;
        p.d = res.ptr; p.out_dt = lp; p.ldd = n;
        p.bias = b ? (const float *)b->data.ptr : nullptr;
        p.m = m; p.n = n; p.k = k;
        p.act = act;
        if (act != MCB_ACT_NONE && g_grad_enabled) {
            MCB_TRY(new_tensor(ctx, lp, oshape, &sv->pre));
            p.d_pre = sv->pre.ptr;
        }
        MCB_TRY(mcb_tc_gemm(ctx, p));
    } else {
        // Shapes the tensor-core kernel declines (an extent that is not a multiple of 8) keep the lowering's
        // numerics under autocast: operands rounded to the 16-bit type, exact f32 products and sums, f32 result
        // (the reference lowers every linear under autocast, cuda/src/ops.rs:762-781).
        Tensor wf = w->data;
        if (sv->emulated) {
            Tensor t;
            MCB_TRY(to_dtype(ctx, x->data, lp, &t));
            MCB_TRY(to_dtype(ctx, t, MCB_F32, &sv->x));
            MCB_TRY(lowp_of(w, lp, &t));
            MCB_TRY(to_dtype(ctx, t, MCB_F32, &wf));
        } else {
            MCB_TRY(f32_of(x, &sv->x));
        }
        MCB_TRY(new_tensor(ctx, MCB_F32, oshape, &res));
        const float *bp = b ? (const float *)b->data.ptr : nullptr;
        if (act != MCB_ACT_NONE) {
            MCB_TRY(new_tensor(ctx, MCB_F32, oshape, &sv->pre));
            MCB_TRY(mcb_linear(ctx, (const float *)sv->x.ptr, (const float *)wf.ptr, bp, (float *)sv->pre.ptr, m, k, n, MCB_ACT_NONE));
            MCB_TRY((act == MCB_ACT_GELU ? mcb_gelu : mcb_relu)(ctx, sv->pre.ptr, res.ptr, res.numel(), MCB_F32));
        } else {
            MCB_TRY(mcb_linear(ctx, (const float *)sv->x.ptr, (const float *)wf.ptr, bp, (float *)res.ptr, m, k, n, MCB_ACT_NONE));
        }
        if (sv->emulated) { // stored like the tensor-core path stores it: result in the 16-bit type, pre-activation rounded to it
            Tensor t;
            MCB_TRY(to_dtype(ctx, res, lp, &t));
            res = t;
            if (sv->pre.defined) {
                MCB_TRY(to_dtype(ctx, sv->pre, lp, &t));
                MCB_TRY(to_dtype(ctx, t, MCB_F32, &sv->pre));
            }
        }
    }
    std::vector<Var> ins = {x, w};
    if (b) ins.push_back(b);
    Var xv = x, wv = w, bv = b;
    *out = apply(ctx, act ? "LinearActivation" : "Linear", res, ins, [ctx, sv, xv, wv, bv](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        return linear_backward_impl(ctx, g, *sv, xv, wv, bv, gi);
    });
    if (!(*out)->requires_grad) sv->pre = Tensor();
    return MCB_OK;
}
mcb_status f_linear(const Var &x, const Var &w, const Var &b, Var *out) { return f_linear_impl(x, w, b, MCB_ACT_NONE, out); }
mcb_status f_linear_activation(const Var &x, const Var &w, const Var &b, int act, Var *out) {
    if (act != MCB_ACT_RELU && act != MCB_ACT_GELU) return mcb_fail(x->ctx, MCB_INVALID_ARGUMENT, "linear_activation supports relu and gelu");
    return f_linear_impl(x, w, b, act, out);
}

mcb_status f_matmul(const Var &a, const Var &b, Var *out) {
    MCB_TRY(check_same_ctx(a, b));
    mcb_ctx *ctx = a->ctx;
    if (a->data.shape.size() != 2 || b->data.shape.size() != 2 || a->data.shape[1] != b->data.shape[0])
        return mcb_fail(ctx, MCB_SHAPE_MISMATCH, "matmul expects [m,k] x [k,n]");
    int64_t m = a->data.shape[0], k = a->data.shape[1], n = b->data.shape[1];
    Tensor af, bf, res;
    MCB_TRY(f32_of(a, &af));
    MCB_TRY(f32_of(b, &bf));
    MCB_TRY(new_tensor(ctx, MCB_F32, {m, n}, &res));
    MCB_TRY(mcb_matmul(ctx, (const float *)af.ptr, (const float *)bf.ptr, (float *)res.ptr, m, k, n));
    Var av = a, bv = b;
    *out = apply(ctx, "MatMul", res, {a, b}, [ctx, af, bf, av, bv, m, k, n](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gf;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        if (av->requires_grad) { // ga[m,k] = g[m,n] b^T[n,k]
            Tensor t;
            MCB_TRY(new_tensor(ctx, MCB_F32, {m, k}, &t));
            SgemmParams p;
            p.a = (const float *)gf.ptr; p.b = (const float *)bf.ptr; p.c = (float *)t.ptr;
            p.m = m; p.n = k; p.k = n; p.as0 = n; p.as1 = 1; p.bs0 = 1; p.bs1 = n; p.ldc = k;
            MCB_TRY(mcb_sgemm(ctx, p));
            MCB_TRY(like_input(ctx, t, av, &gi[0]));
        }
        if (bv->requires_grad) { // gb[k,n] = a^T[k,m] g[m,n]
            Tensor t;
            MCB_TRY(new_tensor(ctx, MCB_F32, {k, n}, &t));
            SgemmParams p;
            p.a = (const float *)af.ptr; p.b = (const float *)gf.ptr; p.c = (float *)t.ptr;
            p.m = k; p.n = n; p.k = m; p.as0 = 1; p.as1 = k; p.bs0 = n; p.bs1 = 1; p.ldc = n;
            MCB_TRY(mcb_sgemm(ctx, p));
            MCB_TRY(like_input(ctx, t, bv, &gi[1]));
        }
        return MCB_OK;
    });
    return MCB_OK;
}

mcb_status f_softmax(const Var &x, Var *out) {
    mcb_ctx *ctx = x->ctx;
    if (x->data.shape.size() != 2) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "softmax expects a 2-D input");
    Tensor xf, res;
    MCB_TRY(f32_of(x, &xf));
    MCB_TRY(new_tensor(ctx, MCB_F32, xf.shape, &res));
    int64_t rows = xf.shape[0], cols = xf.shape[1];
    MCB_TRY(mcb_softmax(ctx, (const float *)xf.ptr, (float *)res.ptr, rows, cols));
    Var xv = x;
    // the node keeps the probabilities it already has (the reference keeps x and rebuilds them, ops.rs:495-517)
    *out = apply(ctx, "Softmax", res, {x}, [ctx, res, xv, rows, cols](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gf, t;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        MCB_TRY(new_tensor(ctx, MCB_F32, res.shape, &t));
        MCB_TRY(mcb_softmax_backward_from_output(ctx, (const float *)res.ptr, (const float *)gf.ptr, (float *)t.ptr, rows, cols));
        return like_input(ctx, t, xv, &gi[0]);
    });
    return MCB_OK;
}

void layer_norm_node(mcb_ctx *ctx, const Var &x, const Var &gamma, const Var &beta, double eps, const Tensor &xf, const Tensor &res,
                     const Tensor &mean, const Tensor &rstd, Var *out);

mcb_status f_layer_norm(const Var &x, const Var &gamma, const Var &beta, double eps, Var *out) {
    mcb_ctx *ctx = x->ctx;
    if (x->data.shape.size() < 2) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "layer_norm expects rank >= 2");
    int64_t dim = x->data.shape.back();
    if (gamma->data.numel() != dim || beta->data.numel() != dim) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "layer_norm gamma/beta shape mismatch");
    int64_t rows = dim ? x->data.numel() / dim : 0;
    Tensor xf, res, mean, rstd;
    MCB_TRY(f32_of(x, &xf));
    int odt = is_lp(g_autocast) ? g_autocast : MCB_F32; // under autocast the result only feeds low-precision GEMMs
    MCB_TRY(new_tensor(ctx, odt, xf.shape, &res));
    MCB_TRY(new_tensor(ctx, MCB_F32, {rows}, &mean));
    MCB_TRY(new_tensor(ctx, MCB_F32, {rows}, &rstd));
    MCB_TRY(mcb_layer_norm(ctx, (const float *)xf.ptr, (const float *)gamma->data.ptr, (const float *)beta->data.ptr, eps, res.ptr, odt,
                           (float *)mean.ptr, (float *)rstd.ptr, rows, dim));
    layer_norm_node(ctx, x, gamma, beta, eps, xf, res, mean, rstd, out);
    return MCB_OK;
}

// the tape node of LayerNorm over an already computed result (xf: x as f32; mean, rstd: the row statistics)
void layer_norm_node(mcb_ctx *ctx, const Var &x, const Var &gamma, const Var &beta, double eps, const Tensor &xf, const Tensor &res,
                     const Tensor &mean, const Tensor &rstd, Var *out) {
    const int64_t dim = x->data.shape.back();
    const int64_t rows = dim ? x->data.numel() / dim : 0;
    Var xv = x, gv = gamma, bv = beta;
    // A bf16 result means the model runs under autocast: the gradient of the f32 residual stream that this backward
    // writes is then read next by the backward of a bf16 Linear, which wants it rounded to bf16 and its column sums (the
    // bias gradient).  The pipeline kernel leaves both as by-products (GradAux) and saves that Linear a pass over dx.
    const bool lowp = is_lp(res.dt);
    const int lpdt = res.dt;
    *out = apply(ctx, "LayerNorm", res, {x, gamma, beta}, [ctx, xf, mean, rstd, xv, gv, bv, eps, rows, dim, lowp, lpdt](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor dx, dg, db;
        bool d1, d2;
        MCB_TRY(grad_dst(gv, &dg, &d1));
        MCB_TRY(grad_dst(bv, &db, &d2));
        const bool fuse = !knob_on(ctx, K_UNFUSED_BWD); // test knob: separate fan-in add, cast and column sums
        const bool want_aux = fuse && lowp && xv->data.dt == MCB_F32 && (g.dt == MCB_F32 || g.dt == lpdt) && !knob_on(ctx, K_LN_NO_AUX);
        // the pipeline kernel with the by-products; MCB_UNSUPPORTED (nothing launched) where it does not apply
        auto with_aux = [&](const float *addend, float *dst, std::shared_ptr<GradAux> *aux_out) -> mcb_status {
            if (!want_aux) return MCB_UNSUPPORTED;
            auto aux = std::make_shared<GradAux>();
            MCB_TRY(new_tensor(ctx, lpdt, xf.shape, &aux->bf16));
            MCB_TRY(new_tensor(ctx, MCB_F32, {dim}, &aux->colsum));
            ProfScope prof(ctx, MCB_PROF_NORM, 0.0, (double)rows * dim * (10.0 + (is_lp(g.dt) ? 2.0 : 4.0) + (addend ? 4.0 : 0.0)) + 8.0 * rows + 12.0 * dim);
            mcb_status st = mcb_ln_bulk_backward(ctx, (const float *)xf.ptr, (const float *)gv->data.ptr, g.ptr, g.dt, eps, (const float *)mean.ptr,
                                                 (const float *)rstd.ptr, addend, dst, (float *)dg.ptr, (float *)db.ptr, rows, dim, aux->bf16.ptr,
                                                 (float *)aux->colsum.ptr, lpdt);
            if (st == MCB_OK) *aux_out = aux;
            return st;
        };
        // A gradient already waiting for x (the residual branch of a pre-norm block) takes dx in place
        const Tensor *pend = fuse ? pending_grad(0) : nullptr;
        if (pend && pend->dt == MCB_F32 && xv->data.dt == MCB_F32 && pend->numel() == xf.numel()) {
            std::shared_ptr<GradAux> aux;
            mcb_status st = with_aux((const float *)pend->ptr, (float *)pend->ptr, &aux);
            if (st == MCB_UNSUPPORTED)
                st = mcb_layer_norm_backward_ex(ctx, (const float *)xf.ptr, (const float *)gv->data.ptr, g.ptr, g.dt, eps, (const float *)mean.ptr,
                                                (const float *)rstd.ptr, (const float *)pend->ptr, (float *)pend->ptr, (float *)dg.ptr,
                                                (float *)db.ptr, rows, dim);
            if (st != MCB_UNSUPPORTED) {
                MCB_TRY(st);
                gi[0] = *pend; // same storage: the walker sees that the sum is already in place
                gi[0].aux = aux; // by-products of the new values, or none
                gi[1] = dg;
                gi[2] = db;
                return MCB_OK;
            }
        }
        MCB_TRY(new_tensor(ctx, MCB_F32, xf.shape, &dx));
        std::shared_ptr<GradAux> aux;
        mcb_status st = with_aux(nullptr, (float *)dx.ptr, &aux);
        if (st == MCB_UNSUPPORTED)
            st = mcb_layer_norm_backward(ctx, (const float *)xf.ptr, (const float *)gv->data.ptr, g.ptr, g.dt, eps, (const float *)mean.ptr,
                                         (const float *)rstd.ptr, (float *)dx.ptr, (float *)dg.ptr, (float *)db.ptr, rows, dim);
        MCB_TRY(st);
        MCB_TRY(like_input(ctx, dx, xv, &gi[0]));
        if (gi[0].ptr == dx.ptr) gi[0].aux = aux;
        gi[1] = dg;
        gi[2] = db;
        return MCB_OK;
    });
}

// sum = a + b and out = LayerNorm(sum): the residual add of a pre-norm block and the LayerNorm that reads it.
// Two tape nodes, exactly those of f_binary(MCB_ADD) and f_layer_norm; when a is an f32 residual stream and the
// shapes suit the pipeline kernel, one kernel produces both results (same arithmetic, one pass over the rows).
mcb_status f_add_layer_norm(const Var &a, const Var &b, const Var &gamma, const Var &beta, double eps, Var *sum, Var *out) {
    MCB_TRY(check_same_ctx(a, b));
    mcb_ctx *ctx = a->ctx;
    const std::vector<int64_t> &sh = a->data.shape;
    if (!knob_on(ctx, K_UNFUSED_ADD_LN) && sh.size() >= 2 && sh == b->data.shape && a->data.dt == MCB_F32 &&
        (b->data.dt == MCB_F32 || is_lp(b->data.dt)) && gamma->data.numel() == sh.back() && beta->data.numel() == sh.back() &&
        gamma->data.dt == MCB_F32 && beta->data.dt == MCB_F32) {
        const int64_t dim = sh.back(), rows = dim ? a->data.numel() / dim : 0;
        const int odt = is_lp(g_autocast) ? g_autocast : MCB_F32;
        Tensor st, res, mean, rstd;
        MCB_TRY(new_tensor(ctx, MCB_F32, sh, &st));
        MCB_TRY(new_tensor(ctx, odt, sh, &res));
        MCB_TRY(new_tensor(ctx, MCB_F32, {rows}, &mean));
        MCB_TRY(new_tensor(ctx, MCB_F32, {rows}, &rstd));
        mcb_status fused;
        {
            ProfScope prof(ctx, MCB_PROF_NORM, 0.0, (double)rows * dim * (8.0 + (is_lp(b->data.dt) ? 2.0 : 4.0) + (is_lp(odt) ? 2.0 : 4.0)) + 8.0 * rows);
            fused = mcb_ln_bulk_add_forward(ctx, (const float *)a->data.ptr, b->data.ptr, b->data.dt, (const float *)gamma->data.ptr,
                                            (const float *)beta->data.ptr, eps, (float *)st.ptr, res.ptr, odt, (float *)mean.ptr, (float *)rstd.ptr, rows, dim);
        }
        if (fused != MCB_UNSUPPORTED) {
            MCB_TRY(fused);
            binary_node(ctx, MCB_ADD, a, b, st, sum);
            layer_norm_node(ctx, *sum, gamma, beta, eps, st, res, mean, rstd, out);
            return MCB_OK;
        }
    }
    MCB_TRY(f_binary(MCB_ADD, a, b, sum));
    return f_layer_norm(*sum, gamma, beta, eps, out);
}

mcb_status f_softmax_cross_entropy(const Var &logits, const Var &target, Var *out) {
    mcb_ctx *ctx = logits->ctx;
    if (logits->data.shape.size() != 2) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "softmax_cross_entropy expects [batch, classes] logits");
    int64_t n = logits->data.shape[0], c = logits->data.shape[1];
    int ldt = target->data.dt;
    if (ldt != MCB_I64 && ldt != MCB_I32 && ldt != MCB_U8) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "labels must be i64, i32 or u8");
    if (target->data.numel() != n) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "expected %lld targets, got %lld", (long long)n, (long long)target->data.numel());
    Tensor res;
    MCB_TRY(new_tensor(ctx, MCB_F32, {}, &res));
    Tensor x = logits->data, lab = target->data;
    if (x.dt == MCB_F32) {
        MCB_TRY(mcb_softmax_cross_entropy(ctx, (const float *)x.ptr, lab.ptr, ldt, n, c, (float *)res.ptr));
    } else {
        Tensor xf;
        MCB_TRY(to_dtype(ctx, x, MCB_F32, &xf));
        MCB_TRY(mcb_softmax_cross_entropy(ctx, (const float *)xf.ptr, lab.ptr, ldt, n, c, (float *)res.ptr));
    }
    *out = apply(ctx, "SoftmaxCrossEntropy", res, {logits, target}, [ctx, x, lab, ldt, n, c](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        // (softmax - onehot)/n times the upstream scalar, read on the device (no host round trip)
        Tensor gf;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        MCB_TRY(new_tensor(ctx, x.dt, x.shape, &gi[0]));
        return mcb_sce_grad(ctx, x.ptr, gi[0].ptr, x.dt, lab.ptr, ldt, n, c, nullptr, (const float *)gf.ptr);
    });
    return MCB_OK;
}

// Loss head whose backward overwrites the logits buffer with their gradient instead of
// allocating a second [n, classes] tensor.  Used by the decoder model, whose logits nobody
// else reads: at vocabulary 32000 that buffer is the largest activation of the step.
mcb_status f_sce_consuming(const Var &logits, const Var &target, Var *out) {
    mcb_ctx *ctx = logits->ctx;
    int64_t n = logits->data.shape[0], c = logits->data.shape[1];
    int ldt = target->data.dt;
    if (ldt != MCB_I64 && ldt != MCB_I32 && ldt != MCB_U8) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "labels must be i64, i32 or u8");
    if (target->data.numel() != n) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "expected %lld targets", (long long)n);
    Tensor res;
    MCB_TRY(new_tensor(ctx, MCB_F32, {}, &res));
    Tensor x = logits->data, lab = target->data, stats;
    MCB_TRY(new_tensor(ctx, MCB_F32, {n, 2}, &stats)); // row maximum and sum of exp: the gradient pass streams the rows without reducing them again
    MCB_TRY(mcb_sce_grad(ctx, x.ptr, nullptr, x.dt, lab.ptr, ldt, n, c, (float *)res.ptr, nullptr, (float *)stats.ptr, nullptr)); // loss only
    *out = apply(ctx, "SoftmaxCrossEntropy", res, {logits, target}, [ctx, x, lab, stats, ldt, n, c](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gf;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        MCB_TRY(mcb_sce_grad(ctx, x.ptr, x.ptr, x.dt, lab.ptr, ldt, n, c, nullptr, (const float *)gf.ptr, nullptr, (const float *)stats.ptr));
        gi[0] = x;
        return MCB_OK;
    });
    return MCB_OK;
}

mcb_status f_embedding(const Var &ids, const Var &weight, Var *out) {
    MCB_TRY(check_same_ctx(ids, weight));
    mcb_ctx *ctx = ids->ctx;
    int idt = ids->data.dt;
    if (idt != MCB_I64 && idt != MCB_I32 && idt != MCB_U8) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "ids must be i64, i32 or u8");
    if (weight->data.shape.size() != 2) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "embedding weight must be [vocab, dim]");
    if (ids->data.shape.size() != 1 && ids->data.shape.size() != 2) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "ids must have rank 1 or 2");
    int64_t vocab = weight->data.shape[0], dim = weight->data.shape[1], n = ids->data.numel();
    std::vector<int64_t> os = ids->data.shape;
    os.push_back(dim);
    Tensor res;
    MCB_TRY(new_tensor(ctx, MCB_F32, os, &res));
    MCB_TRY(mcb_embedding(ctx, ids->data.ptr, idt, n, (const float *)weight->data.ptr, vocab, dim, (float *)res.ptr));
    Tensor idt_t = ids->data;
    Var wv = weight;
    *out = apply(ctx, "Embedding", res, {ids, weight}, [ctx, idt_t, wv, vocab, dim, n](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        bool direct;
        MCB_TRY(grad_dst(wv, &gi[1], &direct));
        return mcb_embedding_backward(ctx, idt_t.ptr, idt_t.dt, n, g.ptr, g.dt, vocab, dim, (float *)gi[1].ptr, 0);
    });
    return MCB_OK;
}

mcb_status f_reshape(const Var &x, const std::vector<int64_t> &shape_in, Var *out) {
    mcb_ctx *ctx = x->ctx;
    std::vector<int64_t> shape = shape_in;
    int64_t known = 1, infer = -1;
    for (size_t i = 0; i < shape.size(); ++i) {
        if (shape[i] == -1) {
            if (infer >= 0) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "reshape: more than one -1");
            infer = (int64_t)i;
        } else known *= shape[i];
    }
    if (infer >= 0) shape[infer] = known ? x->data.numel() / known : 0;
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    if (n != x->data.numel()) return mcb_fail(ctx, MCB_SHAPE_MISMATCH, "reshape changes the element count");
    std::vector<int64_t> in_shape = x->data.shape;
    *out = apply(ctx, "Reshape", view(x->data, shape), {x}, [in_shape](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        gi[0] = view(g, in_shape);
        return MCB_OK;
    });
    return MCB_OK;
}

// shared by transpose and permute: f32 gather with the given axes; backward = inverse permutation
static mcb_status permute_tensor(mcb_ctx *ctx, const Tensor &x, const std::vector<int32_t> &axes, Tensor *out) {
    std::vector<int64_t> oshape(axes.size());
    for (size_t i = 0; i < axes.size(); ++i) oshape[i] = x.shape[axes[i]];
    Tensor xf;
    MCB_TRY(to_dtype(ctx, x, MCB_F32, &xf));
    MCB_TRY(new_tensor(ctx, MCB_F32, oshape, out));
    if (axes.size() == 2 && axes[0] == 1 && axes[1] == 0)
        return mcb_transpose2d(ctx, (const float *)xf.ptr, (float *)out->ptr, x.shape[0], x.shape[1]);
    return mcb_permute(ctx, (const float *)xf.ptr, x.shape.data(), (int32_t)axes.size(), axes.data(), (float *)out->ptr);
}

mcb_status f_permute(const Var &x, const std::vector<int32_t> &axes, Var *out) {
    mcb_ctx *ctx = x->ctx;
    if (!is_float(x->data.dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "permute needs a floating-point input");
    if (axes.size() != x->data.shape.size()) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "permute rank mismatch");
    if (axes.size() > 8) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "permute supports up to 8 dimensions");
    std::vector<int32_t> inverse(axes.size(), -1);
    for (size_t i = 0; i < axes.size(); ++i) {
        if (axes[i] < 0 || (size_t)axes[i] >= axes.size() || inverse[axes[i]] >= 0) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "invalid permute axes");
        inverse[axes[i]] = (int32_t)i;
    }
    Tensor res;
    MCB_TRY(permute_tensor(ctx, x->data, axes, &res));
    Var xv = x;
    *out = apply(ctx, "Permute", res, {x}, [ctx, inverse, xv](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor t;
        MCB_TRY(permute_tensor(ctx, g, inverse, &t));
        return like_input(ctx, t, xv, &gi[0]);
    });
    return MCB_OK;
}

mcb_status f_transpose(const Var &x, Var *out) {
    if (x->data.shape.size() != 2) return mcb_fail(x->ctx, MCB_INVALID_ARGUMENT, "transpose2d expects a 2-D tensor, got rank %d", (int)x->data.shape.size());
    mcb_status st = f_permute(x, {1, 0}, out);
    if (st == MCB_OK && (*out)->node) (*out)->node->name = "Transpose";
    return st;
}

mcb_status f_multi_head_attention(const Var &q, const Var &k, const Var &v, int64_t heads, bool causal, Var *out) {
    mcb_ctx *ctx = q->ctx;
    if (q->data.shape.size() != 3) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "attention expects [N, S, D]");
    if (k->data.shape != q->data.shape || v->data.shape != q->data.shape) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "attention q/k/v shape mismatch");
    int64_t n = q->data.shape[0], s = q->data.shape[1], d = q->data.shape[2];
    if (heads <= 0 || d % heads) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "attention dimension must divide heads");
    int dt = (is_lp(q->data.dt) && k->data.dt == q->data.dt && v->data.dt == q->data.dt) ? q->data.dt : MCB_F32;
    Tensor qt, kt, vt, res, lse;
    MCB_TRY(to_dtype(ctx, q->data, dt, &qt));
    MCB_TRY(to_dtype(ctx, k->data, dt, &kt));
    MCB_TRY(to_dtype(ctx, v->data, dt, &vt));
    MCB_TRY(new_tensor(ctx, dt, q->data.shape, &res));
    MCB_TRY(new_tensor(ctx, MCB_F32, {n, heads, s}, &lse));
    MCB_TRY(mcb_attention(ctx, qt.ptr, kt.ptr, vt.ptr, res.ptr, (float *)lse.ptr, n, s, d, heads, causal, dt));
    Var qv = q, kv = k, vv = v;
    *out = apply(ctx, "MultiHeadAttention", res, {q, k, v}, [ctx, qt, kt, vt, res, lse, qv, kv, vv, n, s, d, heads, causal, dt](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gg, dq, dk, dv;
        MCB_TRY(to_dtype(ctx, g, dt, &gg));
        MCB_TRY(new_tensor(ctx, dt, qt.shape, &dq));
        MCB_TRY(new_tensor(ctx, dt, qt.shape, &dk));
        MCB_TRY(new_tensor(ctx, dt, qt.shape, &dv));
        MCB_TRY(mcb_attention_backward(ctx, qt.ptr, kt.ptr, vt.ptr, res.ptr, gg.ptr, (const float *)lse.ptr, dq.ptr, dk.ptr, dv.ptr, n, s, d, heads, causal, dt));
        MCB_TRY(like_input(ctx, dq, qv, &gi[0]));
        MCB_TRY(like_input(ctx, dk, kv, &gi[1]));
        MCB_TRY(like_input(ctx, dv, vv, &gi[2]));
        return MCB_OK;
    });
    return MCB_OK;
}

// ---- fused self-attention block input: q/k/v projections as ONE GEMM, attention on the packed result
// y = MHA(x Wq^T + bq, x Wk^T + bk, x Wv^T + bv) for x [n*s, d].  Possible when the three weights (and the
// three biases) lie back to back in a parameter arena, which mcb_arena_create arranges: the GEMM then reads
// one [3d, d] operand, the attention kernels read q, k, v as column blocks of the [n*s, 3d] result (row pitch
// 3d), and backward needs one dgrad GEMM (K = 3d) instead of three plus two fan-in additions, one wgrad GEMM
// into the three adjacent gradient slots, and one bias column sum.  Returns MCB_UNSUPPORTED (nothing
// enqueued) when the layout or the dtype does not allow it; callers then compose the unfused ops.
static bool adjacent(const Var &a, const Var &b) {
    return a->arena && a->arena == b->arena && a->arena->off[b->arena_idx] == a->arena->off[a->arena_idx] + a->data.numel() &&
           a->data.numel() % 64 == 0;
}

mcb_status f_qkv_attention(const Var &x, const Var &wq, const Var &bq, const Var &wk, const Var &bk, const Var &wv, const Var &bv,
                           int64_t n, int64_t s, int64_t heads, bool causal, Var *out) {
    mcb_ctx *ctx = x->ctx;
    const int lp = lowp_dtype(ctx);
    if (lp < 0 || x->data.shape.size() != 2) return MCB_UNSUPPORTED;
    if (knob_on(ctx, K_UNFUSED_QKV)) return MCB_UNSUPPORTED; // test knob: run the composed ops instead
    int64_t d = x->data.shape[1], m = x->data.shape[0];
    if (m != n * s || !mcb_flash_supported(d, heads, lp) || !tc_shape_ok(m, 3 * d, d)) return MCB_UNSUPPORTED;
    for (const Var &w : {wq, wk, wv})
        if (w->data.shape != std::vector<int64_t>{d, d}) return MCB_UNSUPPORTED;
    for (const Var &b : {bq, bk, bv})
        if (!b || b->data.shape != std::vector<int64_t>{d}) return MCB_UNSUPPORTED;
    if (!adjacent(wq, wk) || !adjacent(wk, wv) || !adjacent(bq, bk) || !adjacent(bk, bv)) return MCB_UNSUPPORTED;
    Tensor xb, wb, qkv, o, lse;
    MCB_TRY(to_dtype(ctx, x->data, lp, &xb));
    MCB_TRY(lowp_of(wq, lp, &wb)); // shadow of wq; wk and wv follow it in memory
    MCB_TRY(new_tensor(ctx, lp, {m, 3 * d}, &qkv));
    MCB_TRY(new_tensor(ctx, lp, {m, d}, &o));
    MCB_TRY(new_tensor(ctx, MCB_F32, {n, heads, s}, &lse));
    {
        TcGemmParams p; // qkv[m, 3d] = x[m, d] * Wqkv[3d, d]^T + bqkv
        p.in_dt = lp;
        p.a = xb.ptr; p.lda = d;
        p.b = wb.ptr; p.ldb = d;
        p.d = qkv.ptr; p.out_dt = lp; p.ldd = 3 * d;
        p.bias = (const float *)bq->data.ptr;
        p.m = m; p.n = 3 * d; p.k = d;
        MCB_TRY(mcb_tc_gemm(ctx, p));
    }
    const uint16_t *qp = (const uint16_t *)qkv.ptr;
    {
        ProfScope prof(ctx, MCB_PROF_ATTENTION, 4.0 * (double)n * heads * s * s * 64 * (causal ? 0.5 : 1.0), 8.0 * (double)m * d);
        MCB_TRY(mcb_flash_forward(ctx, qp, qp + d, qp + 2 * d, o.ptr, (float *)lse.ptr, n, s, d, heads, causal, 3 * d, d, lp));
    }
    Var xv = x, wqv = wq, wkv = wk, wvv = wv, bqv = bq, bkv = bk, bvv = bv;
    *out = apply(ctx, "QkvAttention", o, {x, wq, bq, wk, bk, wv, bv},
                 [=](const Tensor &g_in, std::vector<Tensor> &gi) -> mcb_status {
        Tensor g, dqkv, bias_part;
        int bias_done = 0;
        MCB_TRY(to_dtype(ctx, g_in, lp, &g));
        MCB_TRY(new_tensor(ctx, lp, {m, 3 * d}, &dqkv));
        uint16_t *dp = (uint16_t *)dqkv.ptr;
        const uint16_t *qp = (const uint16_t *)qkv.ptr; // the closure owns qkv, o and lse until backward has run
        {
            ProfScope prof(ctx, MCB_PROF_ATTENTION, 10.0 * (double)n * heads * s * s * 64 * (causal ? 0.5 : 1.0), 16.0 * (double)m * d);
            // the attention backward kernels can leave per-warp column sums of dq | dk | dv (the rounded values they write): the bias
            // gradients then need only the final reduction over those rows instead of another pass over dqkv
            const int64_t brows = knob_on(ctx, K_UNFUSED_BWD) ? 0 : mcb_flash_bias_rows(n, s);
            if (brows > 0) MCB_TRY(new_tensor(ctx, MCB_F32, {brows, 3 * d}, &bias_part));
            MCB_TRY(mcb_flash_backward(ctx, qp, qp + d, qp + 2 * d, o.ptr, g.ptr, (const float *)lse.ptr, dp, dp + d, dp + 2 * d, n, s, d, heads,
                                       causal, 3 * d, d, 3 * d, brows > 0 ? (float *)bias_part.ptr : nullptr, 3 * d, &bias_done, lp));
        }
        // weight gradients: one [3d, d] product, straight into the three adjacent arena slots when they are free
        bool dq_, dk_, dv_;
        Tensor tw[3], tb[3];
        Var ws[3] = {wqv, wkv, wvv}, bs[3] = {bqv, bkv, bvv};
        bool all_free = true;
        for (int i = 0; i < 3; ++i) all_free = all_free && !ws[i]->has_grad && !ws[i]->slot_claimed && !bs[i]->has_grad && !bs[i]->slot_claimed;
        Tensor dw, db;
        if (all_free) {
            MCB_TRY(grad_dst(wqv, &tw[0], &dq_));
            MCB_TRY(grad_dst(wkv, &tw[1], &dk_));
            MCB_TRY(grad_dst(wvv, &tw[2], &dv_));
            MCB_TRY(grad_dst(bqv, &tb[0], &dq_));
            MCB_TRY(grad_dst(bkv, &tb[1], &dk_));
            MCB_TRY(grad_dst(bvv, &tb[2], &dv_));
            dw = tw[0];
            db = tb[0];
        } else {
            MCB_TRY(new_tensor(ctx, MCB_F32, {3 * d, d}, &dw));
            MCB_TRY(new_tensor(ctx, MCB_F32, {3 * d}, &db));
            for (int i = 0; i < 3; ++i) {
                tw[i] = dw;
                tw[i].ptr = (float *)dw.ptr + i * d * d;
                tw[i].shape = {d, d};
                tb[i] = db;
                tb[i].ptr = (float *)db.ptr + i * d;
                tb[i].shape = {d};
            }
        }
        TcGemmParams pw; // dWqkv[3d, d] = dqkv^T[3d, m] * x[m, d]
        pw.in_dt = lp;
        pw.a = dqkv.ptr; pw.a_mn_major = 1; pw.lda = 3 * d;
        pw.b = xb.ptr; pw.b_mn_major = 1; pw.ldb = d;
        pw.d = dw.ptr; pw.out_dt = MCB_F32; pw.ldd = d;
        pw.m = 3 * d; pw.n = d; pw.k = m;
        mcb_tc_plan(ctx, pw.m, pw.n, pw.k, true, false, 1, &pw.bn, &pw.split_k);
        bool clear_dw = false; // a split reduction adds its slices into a zero output: cleared by the GEMM in front where there is one
        if (pw.split_k > 1) {
            pw.accumulate = 1;
            clear_dw = true;
        }
        if (xv->requires_grad) {
            int xdt = xv->data.dt == lp ? lp : MCB_F32;
            MCB_TRY(new_tensor(ctx, xdt, xv->data.shape, &gi[0]));
            TcGemmParams p; // dx[m, d] = dqkv[m, 3d] * Wqkv[3d, d]
            p.in_dt = lp;
            p.a = dqkv.ptr; p.lda = 3 * d;
            p.b = wb.ptr; p.b_mn_major = 1; p.ldb = d;
            p.d = gi[0].ptr; p.out_dt = xdt; p.ldd = d;
            p.m = m; p.n = d; p.k = 3 * d;
            if (clear_dw && m > 0 && mcb_aligned16(dw.ptr)) {
                p.zero_ptr = dw.ptr;
                p.zero_bytes = sizeof(float) * 3 * d * d;
                clear_dw = false;
            }
            MCB_TRY(mcb_tc_gemm(ctx, p));
        }
        if (clear_dw) MCB_TRY(mcb_memset(ctx, dw.ptr, 0, sizeof(float) * 3 * d * d));
        MCB_TRY(mcb_tc_gemm(ctx, pw));
        if (bias_done) MCB_TRY(mcb_partial_sum_final(ctx, (const float *)bias_part.ptr, (int)bias_part.shape[0], 3 * d, (float *)db.ptr));
        else MCB_TRY(mcb_col_sum(ctx, dqkv.ptr, lp, m, 3 * d, (float *)db.ptr));
        gi[1] = tw[0]; gi[3] = tw[1]; gi[5] = tw[2];
        gi[2] = tb[0]; gi[4] = tb[1]; gi[6] = tb[2];
        return MCB_OK;
    });
    return MCB_OK;
}

mcb_status f_conv2d(const Var &x, const Var &w, const Var &b, int64_t stride, int64_t pad, Var *out) {
    mcb_ctx *ctx = x->ctx;
    if (x->data.shape.size() != 4 || w->data.shape.size() != 4) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "conv2d expects [N,C,H,W] and [O,C,KH,KW]");
    int64_t n = x->data.shape[0], c = x->data.shape[1], h = x->data.shape[2], wd = x->data.shape[3];
    int64_t o = w->data.shape[0], kh = w->data.shape[2], kw = w->data.shape[3];
    if (c != w->data.shape[1]) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "conv2d channel mismatch");
    if (b && b->data.numel() != o) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "conv2d bias size mismatch");
    if (stride <= 0 || h + 2 * pad < kh || wd + 2 * pad < kw) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "conv2d: kernel larger than the padded input");
    int64_t oh = (h + 2 * pad - kh) / stride + 1, ow = (wd + 2 * pad - kw) / stride + 1;
    Tensor xf, res;
    MCB_TRY(f32_of(x, &xf));
    MCB_TRY(new_tensor(ctx, MCB_F32, {n, o, oh, ow}, &res));
    MCB_TRY(mcb_conv2d(ctx, (const float *)xf.ptr, (const float *)w->data.ptr, b ? (const float *)b->data.ptr : nullptr, (float *)res.ptr, n, c, h, wd, o, kh, kw, stride, pad));
    std::vector<Var> ins = {x, w};
    if (b) ins.push_back(b);
    Var xv = x, wv = w, bv = b;
    *out = apply(ctx, "Conv2d", res, ins, [=](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gf;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        float *dx = nullptr, *dw = nullptr, *db = nullptr;
        bool direct;
        if (xv->requires_grad) {
            MCB_TRY(new_tensor(ctx, MCB_F32, xf.shape, &gi[0]));
            dx = (float *)gi[0].ptr;
        }
        if (wv->requires_grad) {
            MCB_TRY(grad_dst(wv, &gi[1], &direct));
            dw = (float *)gi[1].ptr;
        }
        if (bv && bv->requires_grad) {
            MCB_TRY(grad_dst(bv, &gi[2], &direct));
            db = (float *)gi[2].ptr;
        }
        return mcb_conv2d_backward(ctx, (const float *)xf.ptr, (const float *)wv->data.ptr, (const float *)gf.ptr, dx, dw, db, n, c, h, wd, o, kh, kw, stride, pad);
    });
    return MCB_OK;
}

mcb_status f_max_pool2d(const Var &x, int64_t kernel, int64_t stride, int64_t pad, Var *out) {
    mcb_ctx *ctx = x->ctx;
    if (x->data.shape.size() != 4) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "pool2d expects [N,C,H,W]");
    int64_t n = x->data.shape[0], c = x->data.shape[1], h = x->data.shape[2], w = x->data.shape[3];
    if (stride <= 0 || h + 2 * pad < kernel || w + 2 * pad < kernel) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "pool2d: window larger than the padded input");
    int64_t oh = (h + 2 * pad - kernel) / stride + 1, ow = (w + 2 * pad - kernel) / stride + 1;
    Tensor xf, res;
    MCB_TRY(f32_of(x, &xf));
    MCB_TRY(new_tensor(ctx, MCB_F32, {n, c, oh, ow}, &res));
    MCB_TRY(mcb_max_pool2d(ctx, (const float *)xf.ptr, (float *)res.ptr, n, c, h, w, kernel, stride, pad));
    *out = apply(ctx, "Pool2d", res, {x}, [=](const Tensor &g, std::vector<Tensor> &gi) -> mcb_status {
        Tensor gf;
        MCB_TRY(to_dtype(ctx, g, MCB_F32, &gf));
        MCB_TRY(new_tensor(ctx, MCB_F32, xf.shape, &gi[0]));
        return mcb_max_pool2d_backward(ctx, (const float *)xf.ptr, (const float *)gf.ptr, (float *)gi[0].ptr, n, c, h, w, kernel, stride, pad);
    });
    return MCB_OK;
}

// ------------------------------------------------------------------ arena
static int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

mcb_status arena_create(mcb_ctx *ctx, const std::vector<Var> &params, Arena **out) {
    auto a = std::make_unique<Arena>();
    a->ctx = ctx;
    int64_t off = 0;
    for (auto &p : params) {
        if (p->arena) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "a parameter already belongs to an arena");
        if (p->data.dt != MCB_F32) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "arena parameters must be f32");
    }
    // Layout: all matrices (rank >= 2) in list order, then all vectors in list order.  Slots are
    // padded to 64 elements (256 bytes) so vector access and TMA bases stay legal.  With the
    // biases out of the way, consecutive weight matrices of equal width (the q, k, v projections)
    // sit back to back and can be read as one [3d, d] operand; their biases likewise as one [3d].
    a->off.assign(params.size(), 0);
    a->size.assign(params.size(), 0);
    for (int pass = 0; pass < 2; ++pass)
        for (size_t i = 0; i < params.size(); ++i) {
            bool matrix = params[i]->data.shape.size() >= 2;
            if (matrix != (pass == 0)) continue;
            a->off[i] = off;
            a->size[i] = params[i]->data.numel();
            off += align_up(params[i]->data.numel(), 64);
        }
    a->total = off;
    auto mk = [&](size_t bytes, std::shared_ptr<Buf> *b) -> mcb_status {
        void *p = nullptr;
        MCB_TRY(mcb_alloc(ctx, bytes ? bytes : 16, &p));
        *b = std::make_shared<Buf>(ctx, p);
        return mcb_memset(ctx, p, 0, bytes);
    };
    MCB_TRY(mk(sizeof(float) * off, &a->p));
    MCB_TRY(mk(sizeof(float) * off, &a->g));
    MCB_TRY(mk(sizeof(float) * off, &a->m));
    MCB_TRY(mk(sizeof(float) * off, &a->v));
    MCB_TRY(mk(2 * (size_t)off, &a->shadow));
    for (size_t i = 0; i < params.size(); ++i) {
        auto &p = params[i];
        float *dst = (float *)a->p->p + a->off[i];
        MCB_TRY(mcb_memcpy_d2d(ctx, dst, p->data.ptr, sizeof(float) * a->size[i]));
        Tensor t;
        t.buf = a->p;
        t.ptr = dst;
        t.dt = MCB_F32;
        t.shape = p->data.shape;
        t.defined = true;
        bool had = p->has_grad;
        Tensor old_grad = p->grad;
        p->data = t;
        p->arena = a.get();
        p->arena_idx = (int)i;
        p->has_grad = false;
        p->grad = Tensor();
        if (had) MCB_TRY(accumulate_leaf(p, old_grad));
        a->vars.push_back(p);
        a->step.push_back(0);
    }
    a->shadow_valid = false;
    *out = a.release();
    return MCB_OK;
}

void arena_release(Arena *a) {
    if (!a) return;
    for (auto &v : a->vars) {
        v->arena = nullptr; // data/grad views keep the buffers alive through their shared_ptr
        v->arena_idx = -1;
    }
    delete a;
}

// The arena's 16-bit copy of the parameters in format `dt` (MCB_BF16 or MCB_F16; -1 keeps the current one):
// rebuilt when it is stale or held the other format; the fused optimizer pass rewrites it in its current format.
mcb_status arena_refresh_shadow(Arena *a, int dt) {
    if (dt >= 0 && dt != a->shadow_dt) {
        a->shadow_dt = dt;
        a->shadow_valid = false;
    }
    if (a->shadow_valid) return MCB_OK;
    MCB_TRY(mcb_cast(a->ctx, a->p->p, MCB_F32, a->shadow->p, a->shadow_dt, a->total));
    a->shadow_valid = true;
    return MCB_OK;
}

// ------------------------------------------------------------------ optimizers
mcb_status zero_grad(const std::vector<Var> &params) {
    Arena *last = nullptr;
    for (auto &p : params) {
        p->has_grad = false;
        p->grad = Tensor();
        if (p->arena && p->arena != last) { // gradients of an open data-parallel round are dropped: wait for their all-reduces, start over
            last = p->arena;
            MCB_TRY(arena_abandon_round(last));
        }
    }
    return MCB_OK;
}

mcb_status AdamOpt::update(const std::vector<Var> &params, const float *inv_scale_dev, double inv_scale_host, const int32_t *skip,
                           const int32_t *step_dev) {
    // arena fast path: every listed parameter lives in one arena, all have gradients and equal step counts
    Arena *a = params.empty() ? nullptr : params[0]->arena;
    bool flat = a != nullptr && params.size() == a->vars.size();
    if (flat) {
        for (size_t i = 0; i < params.size() && flat; ++i)
            flat = params[i]->arena == a && params[i]->arena_idx == (int)i && params[i]->has_grad && a->step[i] == a->step[0];
    }
    if (flat) {
        MCB_TRY(arena_wait_comm(a));
        double inv = inv_scale_host * arena_grad_divisor(a);
        int32_t t = a->step[0] + 1;
        MCB_TRY(mcb_opt_flat(ctx, kind, (float *)a->p->p, a->g->p, MCB_F32, (float *)a->m->p, (float *)a->v->p, a->shadow->p, a->total, lr, beta1,
                             beta2, eps, weight_decay, t, inv, inv_scale_dev, skip, step_dev, a->shadow_dt));
        // the step counter advances on the host even if the device skips: a skipped step must not
        // count, so callers that pass `skip` roll it back through rollback_step() once they know
        for (auto &s : a->step) s = t;
        a->shadow_valid = true;
        return MCB_OK;
    }
    for (auto &p : params) {
        if (!p->has_grad) continue; // parameters without a gradient are skipped (optim/src/lib.rs:87-89)
        if (p->arena) {
            Arena *pa = p->arena;
            MCB_TRY(arena_wait_comm(pa));
            int i = p->arena_idx;
            int32_t t = ++pa->step[i];
            int64_t off = pa->off[i];
            MCB_TRY(mcb_opt_flat(ctx, kind, (float *)pa->p->p + off, (float *)pa->g->p + off, MCB_F32, (float *)pa->m->p + off, (float *)pa->v->p + off,
                                 (uint16_t *)pa->shadow->p + off, pa->size[i], lr, beta1, beta2, eps, weight_decay, t,
                                 inv_scale_host * arena_grad_divisor(pa), inv_scale_dev, skip, step_dev, pa->shadow_dt));
            continue;
        }
        AdamState &st = state[p.get()];
        if (!st.m.defined) {
            MCB_TRY(new_tensor(ctx, MCB_F32, p->data.shape, &st.m));
            MCB_TRY(new_tensor(ctx, MCB_F32, p->data.shape, &st.v));
            MCB_TRY(mcb_memset(ctx, st.m.ptr, 0, sizeof(float) * st.m.numel()));
            MCB_TRY(mcb_memset(ctx, st.v.ptr, 0, sizeof(float) * st.v.numel()));
        }
        st.t += 1;
        Tensor gf;
        MCB_TRY(to_dtype(ctx, p->grad, MCB_F32, &gf));
        MCB_TRY(mcb_opt_flat(ctx, kind, (float *)p->data.ptr, gf.ptr, MCB_F32, (float *)st.m.ptr, (float *)st.v.ptr, nullptr, p->data.numel(), lr, beta1,
                             beta2, eps, weight_decay, st.t, inv_scale_host, inv_scale_dev, skip, step_dev));
    }
    return MCB_OK;
}

void AdamOpt::rollback_step(const std::vector<Var> &params) {
    for (auto &p : params) {
        if (!p->has_grad) continue;
        if (p->arena) {
            if (p->arena->step[p->arena_idx] > 0) p->arena->step[p->arena_idx]--;
        } else {
            auto it = state.find(p.get());
            if (it != state.end() && it->second.t > 0) it->second.t--;
        }
    }
}

void AdamOpt::rollback_steps(const std::vector<Var> &params, int64_t k) {
    std::vector<Arena *> done;
    for (auto &p : params) {
        if (p->arena) {
            int32_t &t = p->arena->step[p->arena_idx];
            t = (int32_t)std::max<int64_t>(0, (int64_t)t - k);
        } else {
            auto it = state.find(p.get());
            if (it != state.end()) it->second.t = (int32_t)std::max<int64_t>(0, (int64_t)it->second.t - k);
        }
    }
}

AdamOpt::~AdamOpt() {}

mcb_status scaler_create(mcb_ctx *ctx, double init_scale, double growth, double backoff, int interval, Scaler **out) {
    auto s = std::make_unique<Scaler>();
    s->ctx = ctx;
    s->growth = growth;
    s->backoff = backoff;
    s->interval = interval;
    void *p = nullptr;
    MCB_TRY(mcb_alloc(ctx, 64, &p));
    s->state = std::make_shared<Buf>(ctx, p);
    float sc = (float)(init_scale < 1.0 ? 1.0 : init_scale); // with_scale clamps to >= 1 (amp.rs:27-30)
    struct {
        float f[2];
        int i[4];
    } init = {{sc, 1.0f / sc}, {0, 0, 0, 0}};
    MCB_TRY(mcb_memcpy_h2d(ctx, p, &init, sizeof(init)));
    MCB_TRY(mcb_sync(ctx)); // `init` is a stack object
    *out = s.release();
    return MCB_OK;
}

static mcb_status scaler_check(Scaler *s, const std::vector<Var> &params) {
    mcb_ctx *ctx = s->ctx;
    int *flag = s->state_i() + 1;
    Arena *a = params.empty() ? nullptr : params[0]->arena;
    bool flat = a != nullptr && params.size() == a->vars.size();
    for (size_t i = 0; i < params.size() && flat; ++i) flat = params[i]->arena == a && params[i]->has_grad;
    if (flat) {
        MCB_TRY(arena_wait_comm(a));
        return mcb_check_finite(ctx, a->g->p, MCB_F32, a->total, flag);
    }
    for (auto &p : params) {
        if (!p->has_grad) continue;
        if (p->arena) MCB_TRY(arena_wait_comm(p->arena));
        MCB_TRY(mcb_check_finite(ctx, p->grad.ptr, p->grad.dt, p->grad.numel(), flag));
    }
    return MCB_OK;
}

mcb_status scaler_step(Scaler *s, AdamOpt *opt, const std::vector<Var> &params, bool sync, int32_t *applied) {
    mcb_ctx *ctx = s->ctx;
    // 1. inf/nan scan of the scaled gradients (before unscale, like has_non_finite_grad)
    MCB_TRY(scaler_check(s, params));
    // 2. unscale fused into the optimizer pass; the kernel changes nothing when the flag is set
    // async: the device-resident count of applied steps drives the bias correction, so a skipped
    // step does not advance it even though the host never learns about the skip
    MCB_TRY(opt->update(params, s->state_f() + 1, 1.0, s->state_i() + 1, sync ? nullptr : s->state_i() + 3));
    // 3. backoff / growth bookkeeping on the device
    MCB_TRY(mcb_scaler_update(ctx, s->state_f(), s->state_i(), (float)s->growth, (float)s->backoff, s->interval));
    if (!sync) {
        s->issued_since++; // booked as applied; scaler_reconcile corrects the host counts if the device skipped it
        return MCB_OK;
    }
    int found = 0;
    MCB_TRY(mcb_memcpy_d2h(ctx, &found, s->state_i() + 2, sizeof(int)));
    if (found) {
        opt->rollback_step(params);
        MCB_TRY(zero_grad(params)); // the reference clears the gradients of a skipped step (amp.rs:71-76)
    } else {
        s->issued_since++;
    }
    if (applied) *applied = found ? 0 : 1;
    return MCB_OK;
}

mcb_status scaler_reconcile(Scaler *s, AdamOpt *opt, const std::vector<Var> &params) {
    int32_t applied_now = 0;
    MCB_TRY(mcb_memcpy_d2h(s->ctx, &applied_now, s->state_i() + 3, sizeof(int32_t)));
    const int64_t skipped = s->issued_since - ((int64_t)applied_now - s->applied_seen);
    if (skipped > 0 && opt) opt->rollback_steps(params, skipped);
    s->issued_since = 0;
    s->applied_seen = applied_now;
    return MCB_OK;
}

// ------------------------------------------------------------------ initialisers and models
// xorshift64* with polar Box-Muller, the reference's parameter RNG (core/src/rng.rs:14-56)
struct Rng {
    uint64_t state;
    bool has_spare = false;
    double spare = 0.0;
    explicit Rng(uint64_t seed) : state((seed * 0x9E3779B97F4A7C15ull) | 1ull) {}
    uint64_t next_u64() {
        uint64_t x = state;
        x ^= x >> 12;
        x ^= x << 25;
        x ^= x >> 27;
        state = x;
        return x * 0x2545F4914F6CDD1Dull;
    }
    double next_f64() { return (double)(next_u64() >> 11) * (1.0 / 9007199254740992.0); }
    double normal() {
        if (has_spare) {
            has_spare = false;
            return spare;
        }
        for (;;) {
            double u = 2.0 * next_f64() - 1.0, v = 2.0 * next_f64() - 1.0, s = u * u + v * v;
            if (s > 0.0 && s < 1.0) {
                double f = std::sqrt(-2.0 * std::log(s) / s);
                spare = v * f;
                has_spare = true;
                return u * f;
            }
        }
    }
    void fill(std::vector<float> &out, double mean, double std) {
        for (auto &o : out) o = (float)(mean + std * normal());
    }
};

static mcb_status param_from_host(mcb_ctx *ctx, const std::vector<float> &h, const std::vector<int64_t> &shape, Var *out) {
    Tensor t;
    MCB_TRY(new_tensor(ctx, MCB_F32, shape, &t));
    MCB_TRY(mcb_memcpy_h2d(ctx, t.ptr, h.data(), sizeof(float) * h.size()));
    MCB_TRY(mcb_sync(ctx)); // the host vector is released by the caller
    *out = make_var(ctx, t, true);
    return MCB_OK;
}
static mcb_status he_param(mcb_ctx *ctx, const std::vector<int64_t> &shape, int64_t fan_in, uint64_t seed, Var *out) {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    std::vector<float> h((size_t)n);
    Rng r(seed);
    r.fill(h, 0.0, std::sqrt(2.0 / (double)(fan_in > 1 ? fan_in : 1)));
    return param_from_host(ctx, h, shape, out);
}
static mcb_status const_param(mcb_ctx *ctx, int64_t n, float value, Var *out) {
    std::vector<float> h((size_t)n, value);
    return param_from_host(ctx, h, {n}, out);
}

struct LinearL {
    Var w, b;
    mcb_status init(mcb_ctx *ctx, int64_t in, int64_t outf, uint64_t seed) {
        MCB_TRY(he_param(ctx, {outf, in}, in, seed, &w));
        return const_param(ctx, outf, 0.0f, &b);
    }
};

mcb_status Model::create(mcb_ctx *ctx, int kind, const std::vector<int64_t> &cfg, Model **out) {
    auto m = std::make_unique<Model>();
    m->ctx = ctx;
    m->kind = kind;
    m->cfg = cfg;
    auto need = [&](size_t n) -> mcb_status { return cfg.size() >= n ? MCB_OK : mcb_fail(ctx, MCB_INVALID_ARGUMENT, "model config too short"); };
    auto lin = [&](int64_t in, int64_t o, uint64_t seed) -> mcb_status {
        LinearL l;
        MCB_TRY(l.init(ctx, in, o, seed));
        m->params.push_back(l.w);
        m->params.push_back(l.b);
        return MCB_OK;
    };
    auto ln = [&](int64_t d) -> mcb_status {
        Var g, b;
        MCB_TRY(const_param(ctx, d, 1.0f, &g));
        MCB_TRY(const_param(ctx, d, 0.0f, &b));
        m->params.push_back(g);
        m->params.push_back(b);
        return MCB_OK;
    };
    if (kind == 0) { // MLP: Linear seeds 0, 1
        MCB_TRY(need(3));
        MCB_TRY(lin(cfg[0], cfg[1], 0));
        MCB_TRY(lin(cfg[1], cfg[2], 1));
    } else if (kind == 1) { // encoder block: ln1, MHA(q,k,v,o seeds 1..4), ln2, ffn seeds 5, 6
        MCB_TRY(need(4));
        int64_t d = cfg[0], ff = cfg[2];
        MCB_TRY(ln(d));
        for (uint64_t s = 1; s <= 4; ++s) MCB_TRY(lin(d, d, s));
        MCB_TRY(ln(d));
        MCB_TRY(lin(d, ff, 5));
        MCB_TRY(lin(ff, d, 6));
    } else if (kind == 2) { // CNN: conv seeds 0, 1 (fan_in = C*KH*KW), fc seed 2
        MCB_TRY(need(5));
        int64_t cin = cfg[0], c1 = cfg[1], c2 = cfg[2], hw = cfg[3], classes = cfg[4];
        Var w, b;
        MCB_TRY(he_param(ctx, {c1, cin, 3, 3}, cin * 9, 0, &w));
        MCB_TRY(const_param(ctx, c1, 0.0f, &b));
        m->params.push_back(w);
        m->params.push_back(b);
        MCB_TRY(he_param(ctx, {c2, c1, 3, 3}, c1 * 9, 1, &w));
        MCB_TRY(const_param(ctx, c2, 0.0f, &b));
        m->params.push_back(w);
        m->params.push_back(b);
        MCB_TRY(lin(c2 * (hw / 4) * (hw / 4), classes, 2));
    } else if (kind == 3) { // decoder: one RNG stream in the order of Decoder::new (llm/src/decoder.rs:98-140)
        MCB_TRY(need(6));
        int64_t vocab = cfg[0], d = cfg[1], ff = cfg[3], layers = cfg[4];
        Rng rng((uint64_t)cfg[5]);
        auto mat = [&](int64_t r, int64_t c, double std) -> mcb_status {
            std::vector<float> h((size_t)(r * c));
            rng.fill(h, 0.0, std);
            Var v;
            MCB_TRY(param_from_host(ctx, h, {r, c}, &v));
            m->params.push_back(v);
            return MCB_OK;
        };
        auto vec = [&](int64_t n, float val) -> mcb_status {
            Var v;
            MCB_TRY(const_param(ctx, n, val, &v));
            m->params.push_back(v);
            return MCB_OK;
        };
        MCB_TRY(mat(vocab, d, 0.02));
        double sd = std::sqrt(2.0 / (double)d), sff = std::sqrt(2.0 / (double)ff);
        for (int64_t l = 0; l < layers; ++l) {
            MCB_TRY(vec(d, 1.0f)); MCB_TRY(vec(d, 0.0f));            // ln1
            for (int i = 0; i < 4; ++i) { MCB_TRY(mat(d, d, sd)); MCB_TRY(vec(d, 0.0f)); } // q k v o
            MCB_TRY(vec(d, 1.0f)); MCB_TRY(vec(d, 0.0f));            // ln2
            MCB_TRY(mat(ff, d, sd)); MCB_TRY(vec(ff, 0.0f));         // w1 b1
            MCB_TRY(mat(d, ff, sff)); MCB_TRY(vec(d, 0.0f));         // w2 b2
        }
        MCB_TRY(vec(d, 1.0f)); MCB_TRY(vec(d, 0.0f));                // ln_f
        MCB_TRY(mat(vocab, d, 0.02));                                // lm_head (untied, no bias)
    } else {
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "unknown model kind %d", kind);
    }
    *out = m.release();
    return MCB_OK;
}

mcb_status Model::loss(const Var &input, const Var &target, Var *out) {
    const std::vector<Var> &P = params;
    const double eps = 1e-5;
    if (kind == 0) {
        Var h, a, logits;
        MCB_TRY(f_linear(input, P[0], P[1], &h));
        MCB_TRY(f_relu(h, &a));
        MCB_TRY(f_linear(a, P[2], P[3], &logits));
        return f_softmax_cross_entropy(logits, target, out);
    }
    if (kind == 1) {
        int64_t heads = cfg[1];
        bool causal = cfg[3] != 0;
        if (input->data.shape.size() != 3) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "encoder block expects [N, S, D]");
        int64_t b = input->data.shape[0], s = input->data.shape[1], d = input->data.shape[2];
        Var n1, flat, q, k, v, q3, k3, v3, att, att2, o, o3, x1, n2, flat2, h, f2, f3, y, diff, sq;
        MCB_TRY(f_layer_norm(input, P[0], P[1], eps, &n1));
        MCB_TRY(f_reshape(n1, {b * s, d}, &flat));
        mcb_status fused = f_qkv_attention(flat, P[2], P[3], P[4], P[5], P[6], P[7], b, s, heads, causal, &att2);
        if (fused == MCB_UNSUPPORTED) {
            MCB_TRY(f_linear(flat, P[2], P[3], &q));
            MCB_TRY(f_linear(flat, P[4], P[5], &k));
            MCB_TRY(f_linear(flat, P[6], P[7], &v));
            MCB_TRY(f_reshape(q, {b, s, d}, &q3));
            MCB_TRY(f_reshape(k, {b, s, d}, &k3));
            MCB_TRY(f_reshape(v, {b, s, d}, &v3));
            MCB_TRY(f_multi_head_attention(q3, k3, v3, heads, causal, &att));
            MCB_TRY(f_reshape(att, {b * s, d}, &att2));
        } else {
            MCB_TRY(fused);
        }
        MCB_TRY(f_linear(att2, P[8], P[9], &o));
        MCB_TRY(f_reshape(o, {b, s, d}, &o3));
        MCB_TRY(f_binary(MCB_ADD, input, o3, &x1));
        MCB_TRY(f_layer_norm(x1, P[10], P[11], eps, &n2));
        MCB_TRY(f_reshape(n2, {b * s, d}, &flat2));
        MCB_TRY(f_linear_activation(flat2, P[12], P[13], MCB_ACT_GELU, &h));
        MCB_TRY(f_linear(h, P[14], P[15], &f2));
        MCB_TRY(f_reshape(f2, {b, s, d}, &f3));
        MCB_TRY(f_binary(MCB_ADD, x1, f3, &y));
        MCB_TRY(f_binary(MCB_SUB, y, target, &diff));
        MCB_TRY(f_binary(MCB_MUL, diff, diff, &sq));
        return f_mean(sq, out);
    }
    if (kind == 2) {
        Var c1, r1, p1, c2, r2, p2, flat, logits;
        MCB_TRY(f_conv2d(input, P[0], P[1], 1, 1, &c1));
        MCB_TRY(f_relu(c1, &r1));
        MCB_TRY(f_max_pool2d(r1, 2, 2, 0, &p1));
        MCB_TRY(f_conv2d(p1, P[2], P[3], 1, 1, &c2));
        MCB_TRY(f_relu(c2, &r2));
        MCB_TRY(f_max_pool2d(r2, 2, 2, 0, &p2));
        MCB_TRY(f_reshape(p2, {p2->data.shape[0], -1}, &flat));
        MCB_TRY(f_linear(flat, P[4], P[5], &logits));
        return f_softmax_cross_entropy(logits, target, out);
    }
    // decoder (forward order of llm/src/decoder.rs:213-241, training form: full sequence, causal)
    int64_t heads = cfg[2], layers = cfg[4];
    if (input->data.shape.size() != 2) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "decoder expects ids [N, S]");
    int64_t b = input->data.shape[0], s = input->data.shape[1], d = cfg[1];
    Var ids, tgt, x;
    MCB_TRY(f_reshape(input, {b * s}, &ids));
    MCB_TRY(f_reshape(target, {b * s}, &tgt));
    MCB_TRY(f_embedding(ids, P[0], &x));
    size_t pi = 1;
    // every residual add is followed by the LayerNorm of the next sub-block (or the final one), so the two are
    // issued together (f_add_layer_norm); n1 carries the normalised input of the coming attention sub-block
    Var n1;
    if (layers > 0) MCB_TRY(f_layer_norm(x, P[pi + 0], P[pi + 1], eps, &n1));
    for (int64_t l = 0; l < layers; ++l, pi += 16) {
        Var q, k, v, q3, k3, v3, att, att2, o, x1, n2, h, f2, x2;
        mcb_status fused = f_qkv_attention(n1, P[pi + 2], P[pi + 3], P[pi + 4], P[pi + 5], P[pi + 6], P[pi + 7], b, s, heads, true, &att2);
        if (fused == MCB_UNSUPPORTED) {
            MCB_TRY(f_linear(n1, P[pi + 2], P[pi + 3], &q));
            MCB_TRY(f_linear(n1, P[pi + 4], P[pi + 5], &k));
            MCB_TRY(f_linear(n1, P[pi + 6], P[pi + 7], &v));
            MCB_TRY(f_reshape(q, {b, s, d}, &q3));
            MCB_TRY(f_reshape(k, {b, s, d}, &k3));
            MCB_TRY(f_reshape(v, {b, s, d}, &v3));
            MCB_TRY(f_multi_head_attention(q3, k3, v3, heads, true, &att));
            MCB_TRY(f_reshape(att, {b * s, d}, &att2));
        } else {
            MCB_TRY(fused);
        }
        MCB_TRY(f_linear(att2, P[pi + 8], P[pi + 9], &o));
        MCB_TRY(f_add_layer_norm(x, o, P[pi + 10], P[pi + 11], eps, &x1, &n2));
        MCB_TRY(f_linear_activation(n2, P[pi + 12], P[pi + 13], MCB_ACT_GELU, &h));
        MCB_TRY(f_linear(h, P[pi + 14], P[pi + 15], &f2));
        // the LayerNorm that reads x2: the next layer's first one, or the final one (same slots of the next group)
        MCB_TRY(f_add_layer_norm(x1, f2, P[pi + 16], P[pi + 17], eps, &x2, &n1));
        x = x2;
    }
    Var nf = n1, logits;
    if (layers == 0) MCB_TRY(f_layer_norm(x, P[pi + 0], P[pi + 1], eps, &nf));
    MCB_TRY(f_linear(nf, P[pi + 2], nullptr, &logits));
    return f_sce_consuming(logits, tgt, out);
}

} // namespace mcbag

// He-normal values exactly as the reference's links draw them (core/src/init.rs:6-11 over the
// xorshift64* / polar Box-Muller generator of core/src/rng.rs:14-56); a host function.
extern "C" mcb_status mcb_he_normal(float *host_out, int64_t n, int64_t fan_in, uint64_t seed) {
    if (n < 0 || (n > 0 && !host_out)) return MCB_INVALID_ARGUMENT;
    std::vector<float> h((size_t)n);
    mcbag::Rng r(seed);
    r.fill(h, 0.0, std::sqrt(2.0 / (double)(fan_in > 1 ? fan_in : 1)));
    if (n) memcpy(host_out, h.data(), sizeof(float) * (size_t)n);
    return MCB_OK;
}
