// Whole-step CUDA Graph: zero_grad, forward, (loss scaling,) backward and the optimizer update of
// one model, recorded once from the ordinary tape and replayed with one launch per step.
// Follows the reference's static training steps (cuda/src/graph.rs:261-603 GraphLinearTrainer,
// cuda/src/static_run.rs:1875-2096 CudaStaticStep / LinearMseAdamStep): fixed input buffers,
// in-place optimizer, device-resident step counter, replay without host arguments.
//
// How the tape becomes a graph:
//  * the step is run twice under stream capture.  Kernels do not execute while capturing, so
//    neither run changes a parameter.  The first run only serves the host-side lazy work
//    (function attributes, scratch sizing) and fills the step's private block pool; its graph is
//    dropped.  The second run finds every buffer size in that pool and is the one instantiated.
//  * every block allocated or freed while capturing belongs to the step until it is released
//    (runtime.cu), because the recorded kernels carry its address.
//  * bias correction and "first momentum step" read a device counter of applied steps (the
//    GradScaler's, or one owned by the step), so the host value baked into the kernel arguments
//    at capture time is not used.
#include "handles.h"

using namespace mcbag;

struct mcb_static_step {
    mcb_ctx *ctx = nullptr;
    Model *model = nullptr;
    AdamOpt *opt = nullptr;
    Scaler *scaler = nullptr;
    int autocast_dt = -1;
    int capture_id = 0;
    Tensor x, y, loss;     // fixed input buffers and the (unscaled) scalar loss
    Tensor counter;        // applied steps, when no GradScaler keeps one
    int32_t host_step_after = 0; // the host's step count as the last replay (or the creation) left it
    cudaGraphExec_t exec = nullptr;
    int64_t launches_per_step = 0;
    // pipelined runs: the loss of run i goes to pinned slot i & 1 behind the graph; run i + 1 returns it
    float *h_loss = nullptr;
    cudaEvent_t loss_ev[2] = {nullptr, nullptr};
    int64_t piped = 0; // pipelined runs whose loss has been requested so far
    bool loss_pending = false;
};

extern "C" mcb_status mcb_dp_wait_event(mcb_ctx *ctx, void *event); // dp.cu

namespace {

size_t dt_size(int dt) {
    switch (dt) {
    case MCB_F32: return 4;
    case MCB_I64: return 8;
    case MCB_I32: return 4;
    case MCB_U8: return 1;
    case MCB_F16: return 2;
    case MCB_BF16: return 2;
    default: return 0;
    }
}

// one recorded pass of the step on the context's stream (which is capturing)
mcb_status record(mcb_static_step *s) {
    mcb_ctx *ctx = s->ctx;
    s->loss = Tensor(); // the first pass's loss block returns to the step's pool, so both passes allocate alike
    Var xv = make_var(ctx, s->x, false), yv = make_var(ctx, s->y, false), loss;
    zero_grad(s->model->params);
    int prev = autocast();
    set_autocast(s->autocast_dt);
    mcb_status st = s->model->loss(xv, yv, &loss);
    set_autocast(prev);
    MCB_TRY(st);
    // keep the loss where replays will write it; the first capture decides the address, the
    // second must land on the same one (same allocation sequence, same private pool)
    s->loss = loss->data;
    Var root = loss;
    if (s->scaler) MCB_TRY(f_scale_by_device(loss, s->scaler->state_f(), s->scaler->state, &root));
    MCB_TRY(backward(root));
    if (s->scaler) {
        MCB_TRY(scaler_step(s->scaler, s->opt, s->model->params, false, nullptr));
    } else {
        MCB_TRY(s->opt->update(s->model->params, nullptr, 1.0, nullptr, (const int32_t *)s->counter.ptr));
        MCB_TRY(mcb_increment_i32(ctx, (int32_t *)s->counter.ptr));
    }
    return MCB_OK;
}

// host-side step counters advance with every recorded or replayed step; a capture must leave them as it found them
std::vector<std::vector<int32_t>> save_steps(Model *m, AdamOpt *opt, std::vector<int32_t> *per_var) {
    std::vector<std::vector<int32_t>> out;
    std::vector<Arena *> seen;
    for (auto &p : m->params) {
        if (p->arena && std::find(seen.begin(), seen.end(), p->arena) == seen.end()) {
            seen.push_back(p->arena);
            out.push_back(p->arena->step);
        }
        auto it = opt->state.find(p.get());
        per_var->push_back(it == opt->state.end() ? 0 : it->second.t);
    }
    return out;
}
void restore_steps(Model *m, AdamOpt *opt, const std::vector<std::vector<int32_t>> &saved, const std::vector<int32_t> &per_var) {
    std::vector<Arena *> seen;
    size_t k = 0, i = 0;
    for (auto &p : m->params) {
        if (p->arena && std::find(seen.begin(), seen.end(), p->arena) == seen.end()) {
            seen.push_back(p->arena);
            p->arena->step = saved[k++];
        }
        auto it = opt->state.find(p.get());
        if (it != opt->state.end()) it->second.t = per_var[i];
        ++i;
    }
}
// the optimizer's step count as the host knows it (largest over the model's parameters)
int32_t host_step(Model *m, AdamOpt *opt) {
    int32_t t0 = 0;
    for (auto &p : m->params) {
        if (p->arena) t0 = std::max(t0, p->arena->step[p->arena_idx]);
        else {
            auto it = opt->state.find(p.get());
            if (it != opt->state.end()) t0 = std::max(t0, it->second.t);
        }
    }
    return t0;
}
void bump_steps(Model *m, AdamOpt *opt) {
    std::vector<Arena *> seen;
    for (auto &p : m->params) {
        if (p->arena) {
            if (std::find(seen.begin(), seen.end(), p->arena) == seen.end()) {
                seen.push_back(p->arena);
                for (auto &t : p->arena->step) ++t;
            }
        } else {
            auto it = opt->state.find(p.get());
            if (it != opt->state.end()) ++it->second.t;
        }
    }
}

} // namespace

extern "C" {

mcb_status mcb_static_step_create(mcb_model *model, mcb_adam *opt, mcb_scaler *scaler, int32_t autocast_dt, const int64_t *x_dims, int32_t x_rank,
                                  int32_t x_dt, const int64_t *y_dims, int32_t y_rank, int32_t y_dt, mcb_static_step **out) {
    if (!model || !opt || !out) return MCB_INVALID_ARGUMENT;
    mcb_ctx *ctx = model->m->ctx;
    MCB_CHECK_CTX(ctx);
    if (ctx->prof_on) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "static step: switch per-kernel timing off before capturing");
    if (ctx->capture_id) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "static step: another capture is in progress");
    if (dt_size(x_dt) == 0 || dt_size(y_dt) == 0 || x_rank < 0 || y_rank < 0) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "static step: bad input description");
    if (autocast_dt != -1 && autocast_dt != MCB_BF16 && autocast_dt != MCB_F16)
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "static step: autocast must be -1 (off), bf16 or f16");
    // Data-parallel arenas are captured too: the bucket all-reduces are enqueued on the communication stream
    // behind an event of the capturing stream, which pulls that stream into the capture, and the optimizer's
    // wait on the communication stream joins it back.  NCCL must have run one eager step first (its lazy
    // connection set-up is not capturable), which any warm-up step provides.
    auto s = std::make_unique<mcb_static_step>();
    s->ctx = ctx;
    s->model = model->m;
    s->opt = &opt->opt;
    s->scaler = scaler ? scaler->s : nullptr;
    s->autocast_dt = autocast_dt;
    MCB_TRY(new_tensor(ctx, x_dt, std::vector<int64_t>(x_dims, x_dims + x_rank), &s->x));
    MCB_TRY(new_tensor(ctx, y_dt, std::vector<int64_t>(y_dims, y_dims + y_rank), &s->y));
    MCB_TRY(mcb_memset(ctx, s->x.ptr, 0, dt_size(x_dt) * (size_t)s->x.numel()));
    MCB_TRY(mcb_memset(ctx, s->y.ptr, 0, dt_size(y_dt) * (size_t)s->y.numel()));
    if (!s->scaler) {
        MCB_TRY(new_tensor(ctx, MCB_I32, {1}, &s->counter));
        // continue the bias correction where the optimizer stands (0 for a fresh one)
        int32_t t0 = host_step(s->model, s->opt);
        MCB_TRY(mcb_memcpy_h2d(ctx, s->counter.ptr, &t0, sizeof(t0)));
        MCB_TRY(mcb_sync(ctx)); // t0 is a stack object
        s->host_step_after = t0;
    }
    // device state that the tape creates or refreshes lazily must exist before recording: a capture only
    // records the zero-fill / refresh kernels, it does not run them
    for (auto &p : s->model->params) {
        if (p->arena) {
            MCB_TRY(arena_refresh_shadow(p->arena, autocast_dt));
        } else {
            AdamState &as = s->opt->state[p.get()];
            if (!as.m.defined) {
                MCB_TRY(new_tensor(ctx, MCB_F32, p->data.shape, &as.m));
                MCB_TRY(new_tensor(ctx, MCB_F32, p->data.shape, &as.v));
                MCB_TRY(mcb_memset(ctx, as.m.ptr, 0, sizeof(float) * as.m.numel()));
                MCB_TRY(mcb_memset(ctx, as.v.ptr, 0, sizeof(float) * as.v.numel()));
            }
        }
    }
    MCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    s->capture_id = ctx->next_capture_id++;
    ctx->static_steps++;
    cudaGraph_t graph = nullptr;
    mcb_status st = MCB_OK;
    void *loss_ptr_first = nullptr;
    for (int pass = 0; pass < 2 && st == MCB_OK; ++pass) {
        std::vector<int32_t> per_var;
        auto saved = save_steps(s->model, s->opt, &per_var);
        int64_t launches0 = ctx->launches;
        ctx->capture_id = s->capture_id;
        cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed);
        if (e != cudaSuccess) {
            ctx->capture_id = 0;
            st = mcb_cuda_check(ctx, e, "begin stream capture");
            break;
        }
        st = record(s.get());
        cudaGraph_t g = nullptr;
        e = cudaStreamEndCapture(ctx->stream, &g);
        ctx->capture_id = 0;
        restore_steps(s->model, s->opt, saved, per_var);
        s->launches_per_step = ctx->launches - launches0;
        if (st == MCB_OK && e != cudaSuccess) st = mcb_cuda_check(ctx, e, "end stream capture");
        if (st != MCB_OK) {
            if (g) cudaGraphDestroy(g);
            break;
        }
        if (pass == 0) {
            loss_ptr_first = s->loss.ptr;
            cudaGraphDestroy(g);
        } else {
            graph = g;
        }
    }
    if (st == MCB_OK && knob_on(ctx, K_GRAPH_INFO)) { // diagnostic: how many recorded edges are programmatic (dependent launch)
        size_t ne = 0, prog = 0;
        if (cudaGraphGetEdges_v2(graph, nullptr, nullptr, nullptr, &ne) == cudaSuccess && ne) {
            std::vector<cudaGraphNode_t> from(ne), to(ne);
            std::vector<cudaGraphEdgeData> ed(ne);
            if (cudaGraphGetEdges_v2(graph, from.data(), to.data(), ed.data(), &ne) == cudaSuccess)
                for (size_t i = 0; i < ne; ++i) prog += ed[i].type == cudaGraphDependencyTypeProgrammatic;
        }
        fprintf(stderr, "static step graph: %zu edges, %zu programmatic\n", ne, prog);
        // node kinds, and the bytes the fill nodes clear: fills and copies do not show in a kernel launch list
        size_t nn = 0;
        if (cudaGraphGetNodes(graph, nullptr, &nn) == cudaSuccess && nn) {
            std::vector<cudaGraphNode_t> nodes(nn);
            size_t kernels = 0, fills = 0, copies = 0, other = 0;
            double fill_bytes = 0.0;
            if (cudaGraphGetNodes(graph, nodes.data(), &nn) == cudaSuccess)
                for (size_t i = 0; i < nn; ++i) {
                    cudaGraphNodeType t;
                    if (cudaGraphNodeGetType(nodes[i], &t) != cudaSuccess) continue;
                    if (t == cudaGraphNodeTypeKernel) ++kernels;
                    else if (t == cudaGraphNodeTypeMemcpy) ++copies;
                    else if (t == cudaGraphNodeTypeMemset) {
                        ++fills;
                        cudaMemsetParams mp;
                        if (cudaGraphMemsetNodeGetParams(nodes[i], &mp) == cudaSuccess) fill_bytes += (double)mp.width * mp.elementSize * (mp.height ? mp.height : 1);
                    } else ++other;
                }
            fprintf(stderr, "static step graph: %zu kernel, %zu fill (%.1f MB), %zu copy, %zu other nodes\n", kernels, fills, fill_bytes / 1e6, copies, other);
        }
        (void)cudaGetLastError();
    }
    if (st == MCB_OK) {
        cudaError_t e = cudaGraphInstantiate(&s->exec, graph, 0);
        if (e != cudaSuccess) st = mcb_cuda_check(ctx, e, "graph instantiate");
    }
    if (graph) cudaGraphDestroy(graph);
    (void)loss_ptr_first;
    // the tape marked gradients as present although nothing ran: a step that was only recorded leaves none
    zero_grad(s->model->params);
    if (st != MCB_OK) {
        ctx->static_steps--;
        s->x = Tensor();
        s->y = Tensor();
        s->loss = Tensor();
        s->counter = Tensor();
        mcb_release_capture_blocks(ctx, s->capture_id);
        return st;
    }
    *out = s.release();
    return MCB_OK;
}

mcb_status mcb_static_step_inputs(mcb_static_step *s, void **x_dev_out, void **y_dev_out) {
    if (!s) return MCB_INVALID_ARGUMENT;
    if (x_dev_out) *x_dev_out = s->x.ptr;
    if (y_dev_out) *y_dev_out = s->y.ptr;
    return MCB_OK;
}

mcb_status mcb_static_step_run(mcb_static_step *s, const void *host_x, const void *host_y) {
    if (!s) return MCB_INVALID_ARGUMENT;
    mcb_ctx *ctx = s->ctx;
    MCB_CHECK_CTX(ctx);
    if (host_x) MCB_TRY(mcb_memcpy_h2d(ctx, s->x.ptr, host_x, dt_size(s->x.dt) * (size_t)s->x.numel()));
    if (host_y) MCB_TRY(mcb_memcpy_h2d(ctx, s->y.ptr, host_y, dt_size(s->y.dt) * (size_t)s->y.numel()));
    if (!s->scaler) {
        // The bias correction of a step without a GradScaler reads the step's own device counter.  A checkpoint
        // load or an eager optimizer update since the last replay moved the host's count: the counter follows.
        const int32_t t_now = host_step(s->model, s->opt);
        if (t_now != s->host_step_after) {
            MCB_TRY(mcb_memcpy_h2d(ctx, s->counter.ptr, &t_now, sizeof(t_now)));
            MCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream)); // t_now is a stack object; this path is rare
        }
        s->host_step_after = t_now + 1;
    } else {
        s->scaler->issued_since++; // outcome not read back: see scaler_reconcile
    }
    MCB_CUDA(ctx, cudaGraphLaunch(s->exec, ctx->stream));
    ctx->launches += s->launches_per_step;
    bump_steps(s->model, s->opt);
    // the replay wrote every parameter's gradient and the weights: same host-side marks as the tape step leaves
    for (auto &p : s->model->params) {
        if (p->arena) {
            p->has_grad = true;
            p->arena->shadow_valid = true;
        }
    }
    return MCB_OK;
}

static mcb_status take_pending_loss(mcb_static_step *s, float *loss_out, int32_t *have_out) {
    if (have_out) *have_out = s->loss_pending ? 1 : 0;
    if (!s->loss_pending) return MCB_OK;
    const int slot = (int)((s->piped - 1) & 1);
    MCB_TRY(mcb_dp_wait_event(s->ctx, s->loss_ev[slot]));
    if (loss_out) *loss_out = s->h_loss[slot];
    s->loss_pending = false;
    return MCB_OK;
}

mcb_status mcb_static_step_run_pipelined(mcb_static_step *s, const void *host_x, const void *host_y, float *prev_loss_out,
                                         int32_t *have_prev_out) {
    if (!s) return MCB_INVALID_ARGUMENT;
    mcb_ctx *ctx = s->ctx;
    MCB_CHECK_CTX(ctx);
    if (!s->h_loss) {
        MCB_CUDA(ctx, cudaHostAlloc((void **)&s->h_loss, 2 * sizeof(float), cudaHostAllocDefault));
        for (int i = 0; i < 2; ++i) MCB_CUDA(ctx, cudaEventCreateWithFlags(&s->loss_ev[i], cudaEventDisableTiming));
    }
    // this step first, so that the device has it queued while the host waits for the one before
    MCB_TRY(mcb_static_step_run(s, host_x, host_y));
    const int slot = (int)(s->piped & 1);
    const bool had = s->loss_pending;
    MCB_CUDA(ctx, cudaMemcpyAsync(&s->h_loss[slot], s->loss.ptr, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    MCB_CUDA(ctx, cudaEventRecord(s->loss_ev[slot], ctx->stream));
    s->piped++;
    s->loss_pending = true;
    float prev = 0.0f;
    if (had) { // the previous run's loss: its copy sits in the other slot, behind the previous graph
        MCB_TRY(mcb_dp_wait_event(ctx, s->loss_ev[slot ^ 1]));
        prev = s->h_loss[slot ^ 1];
    }
    if (have_prev_out) *have_prev_out = had ? 1 : 0;
    if (prev_loss_out && had) *prev_loss_out = prev;
    return MCB_OK;
}

mcb_status mcb_static_step_drain(mcb_static_step *s, float *loss_out, int32_t *have_out) {
    if (!s) return MCB_INVALID_ARGUMENT;
    MCB_CHECK_CTX(s->ctx);
    return take_pending_loss(s, loss_out, have_out);
}

mcb_status mcb_static_step_loss(mcb_static_step *s, float *loss_out) {
    if (!s || !loss_out) return MCB_INVALID_ARGUMENT;
    return mcb_memcpy_d2h(s->ctx, loss_out, s->loss.ptr, sizeof(float));
}

mcb_status mcb_static_step_launches(mcb_static_step *s, int64_t *kernels_per_step_out) {
    if (!s || !kernels_per_step_out) return MCB_INVALID_ARGUMENT;
    *kernels_per_step_out = s->launches_per_step;
    return MCB_OK;
}

void mcb_static_step_release(mcb_static_step *s) {
    if (!s) return;
    mcb_ctx *ctx = s->ctx;
    cudaStreamSynchronize(ctx->stream);
    if (s->exec) cudaGraphExecDestroy(s->exec);
    if (s->h_loss) cudaFreeHost(s->h_loss);
    for (int i = 0; i < 2; ++i)
        if (s->loss_ev[i]) cudaEventDestroy(s->loss_ev[i]);
    s->x = Tensor();
    s->y = Tensor();
    s->loss = Tensor();
    s->counter = Tensor();
    mcb_release_capture_blocks(ctx, s->capture_id);
    ctx->static_steps--;
    delete s;
}

} // extern "C"
