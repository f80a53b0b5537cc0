// Training checkpoints in the reference's `.mcn` container (crates/modern-chainer-serial/src/lib.rs:12-115):
//   "MCHN0001", u32 entry count, then per entry: u32 name length + UTF-8 name, u8 dtype tag
//   (0 f32, 1 f64, 2 f16, 3 bf16, 4 i32, 5 i64, 6 u8, 7 bool), u32 rank, u64 dims, u64 byte
//   length, raw little-endian bytes.
// A checkpoint holds, for every parameter `name`: the f32 value under `name`; with an optimizer
// its state under `name.opt_m`, `name.opt_v` (f32, same shape; the velocity of MomentumSGD lives in
// opt_m) and `name.opt_t` (i64 [1], updates applied so far); with a GradScaler `grad_scaler.state`
// (f32 {scale, inv_scale}) and `grad_scaler.counters` (i32 {growth_tracker, found_inf,
// last_found_inf, applied_steps}).  Parameters that live in a flat arena are read and written
// as one device copy per array (values, m, v), not one per tensor.
#include <cstdio>
#include <map>
#include <string>

#include "handles.h"

using namespace mcbag;

namespace {

enum { TAG_F32 = 0, TAG_I32 = 4, TAG_I64 = 5 };

struct Entry {
    std::string name;
    uint8_t tag = 0;
    std::vector<uint64_t> dims;
    std::vector<unsigned char> bytes;
};

void put_u32(std::vector<unsigned char> &o, uint32_t v) {
    for (int i = 0; i < 4; ++i) o.push_back((unsigned char)(v >> (8 * i)));
}
void put_u64(std::vector<unsigned char> &o, uint64_t v) {
    for (int i = 0; i < 8; ++i) o.push_back((unsigned char)(v >> (8 * i)));
}

bool write_entry(FILE *f, const Entry &e) {
    std::vector<unsigned char> h;
    put_u32(h, (uint32_t)e.name.size());
    h.insert(h.end(), e.name.begin(), e.name.end());
    h.push_back(e.tag);
    put_u32(h, (uint32_t)e.dims.size());
    for (uint64_t d : e.dims) put_u64(h, d);
    put_u64(h, (uint64_t)e.bytes.size());
    if (fwrite(h.data(), 1, h.size(), f) != h.size()) return false;
    return e.bytes.empty() || fwrite(e.bytes.data(), 1, e.bytes.size(), f) == e.bytes.size();
}

bool get(FILE *f, void *dst, size_t n) { return n == 0 || fread(dst, 1, n, f) == n; }
bool get_u32(FILE *f, uint32_t *v) {
    unsigned char b[4];
    if (!get(f, b, 4)) return false;
    *v = (uint32_t)b[0] | ((uint32_t)b[1] << 8) | ((uint32_t)b[2] << 16) | ((uint32_t)b[3] << 24);
    return true;
}
bool get_u64(FILE *f, uint64_t *v) {
    unsigned char b[8];
    if (!get(f, b, 8)) return false;
    *v = 0;
    for (int i = 0; i < 8; ++i) *v |= (uint64_t)b[i] << (8 * i);
    return true;
}

size_t tag_size(uint8_t tag) {
    switch (tag) {
    case 0: return 4;
    case 1: return 8;
    case 2: return 2;
    case 3: return 2;
    case 4: return 4;
    case 5: return 8;
    case 6: return 1;
    case 7: return 1;
    default: return 0;
    }
}

mcb_status read_file_unchecked(mcb_ctx *ctx, const char *path, std::map<std::string, Entry> *out, std::vector<std::string> *order);

// The file is untrusted input: sizes are checked against the bytes that are really there before anything is
// allocated, products are checked for overflow, and an allocation failure becomes MCB_IO instead of leaving through
// the C boundary as an exception.
mcb_status read_file(mcb_ctx *ctx, const char *path, std::map<std::string, Entry> *out, std::vector<std::string> *order) {
    try {
        return read_file_unchecked(ctx, path, out, order);
    } catch (const std::exception &e) {
        return mcb_fail(ctx, MCB_IO, "reading %s failed: %s", path, e.what());
    }
}

mcb_status read_file_unchecked(mcb_ctx *ctx, const char *path, std::map<std::string, Entry> *out, std::vector<std::string> *order) {
    FILE *f = fopen(path, "rb");
    if (!f) return mcb_fail(ctx, MCB_IO, "cannot open %s", path);
    uint64_t file_size = 0;
    if (fseek(f, 0, SEEK_END) == 0) {
        long sz = ftell(f);
        file_size = sz > 0 ? (uint64_t)sz : 0;
    }
    rewind(f);
    char magic[8];
    uint32_t count = 0;
    mcb_status st = MCB_OK;
    if (!get(f, magic, 8) || memcmp(magic, "MCHN0001", 8) != 0) st = mcb_fail(ctx, MCB_INVALID_ARGUMENT, "not a Modern Chainer .mcn file");
    else if (!get_u32(f, &count)) st = mcb_fail(ctx, MCB_IO, "truncated .mcn header");
    for (uint32_t i = 0; i < count && st == MCB_OK; ++i) {
        Entry e;
        uint32_t nlen = 0, rank = 0;
        uint64_t blen = 0;
        if (!get_u32(f, &nlen) || nlen > (1u << 20)) {
            st = mcb_fail(ctx, MCB_IO, "truncated .mcn entry");
            break;
        }
        e.name.resize(nlen);
        if (!get(f, &e.name[0], nlen) || !get(f, &e.tag, 1) || !get_u32(f, &rank) || rank > 64) {
            st = mcb_fail(ctx, MCB_IO, "truncated .mcn entry");
            break;
        }
        if (tag_size(e.tag) == 0) {
            st = mcb_fail(ctx, MCB_INVALID_ARGUMENT, "unknown dtype tag %d", (int)e.tag);
            break;
        }
        e.dims.resize(rank);
        uint64_t numel = 1;
        bool ok = true, overflow = false;
        for (uint32_t d = 0; d < rank && ok; ++d) {
            ok = get_u64(f, &e.dims[d]);
            if (ok && e.dims[d] != 0 && numel > UINT64_MAX / e.dims[d]) overflow = true;
            numel = overflow ? 0 : numel * e.dims[d];
        }
        if (ok && !overflow && numel > UINT64_MAX / tag_size(e.tag)) overflow = true;
        if (!ok || overflow || !get_u64(f, &blen) || blen != numel * tag_size(e.tag)) {
            st = mcb_fail(ctx, MCB_IO, "entry %s: byte length does not match its shape", e.name.c_str());
            break;
        }
        const long here = ftell(f);
        if (here < 0 || blen > file_size - (uint64_t)here) { // more bytes announced than the file still holds
            st = mcb_fail(ctx, MCB_IO, "truncated .mcn entry %s", e.name.c_str());
            break;
        }
        if (out->count(e.name)) {
            st = mcb_fail(ctx, MCB_INVALID_ARGUMENT, "entry %s appears twice", e.name.c_str());
            break;
        }
        e.bytes.resize(blen);
        if (!get(f, e.bytes.data(), blen)) {
            st = mcb_fail(ctx, MCB_IO, "truncated .mcn entry %s", e.name.c_str());
            break;
        }
        if (order) order->push_back(e.name);
        (*out)[e.name] = std::move(e);
    }
    fclose(f);
    return st;
}

Entry f32_entry(const std::string &name, const std::vector<int64_t> &shape, const float *host, int64_t n) {
    Entry e;
    e.name = name;
    e.tag = TAG_F32;
    for (int64_t d : shape) e.dims.push_back((uint64_t)d);
    e.bytes.resize(sizeof(float) * (size_t)n);
    if (n) memcpy(e.bytes.data(), host, e.bytes.size());
    return e;
}

bool same_shape(const Entry &e, const std::vector<int64_t> &shape) {
    if (e.dims.size() != shape.size()) return false;
    for (size_t i = 0; i < shape.size(); ++i)
        if (e.dims[i] != (uint64_t)shape[i]) return false;
    return true;
}

// host copies of an arena's arrays, fetched once
struct ArenaHost {
    std::vector<float> p, m, v;
};

} // namespace

extern "C" {

mcb_status mcb_checkpoint_save(mcb_ctx *ctx, const char *path, const char *const *names, mcb_var **params, int32_t n, mcb_adam *opt,
                               mcb_scaler *scaler) {
    MCB_CHECK_CTX(ctx);
    if (!path || n < 0 || (n > 0 && (!names || !params))) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "checkpoint_save: bad arguments");
    MCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (scaler && opt) {
        // steps whose outcome was never read back (async scaler steps, graph replays) were booked as applied on the
        // host; the device knows how many were skipped: opt_t below is the number of APPLIED steps, the value the
        // reference's per-parameter t holds (a skipped step does not advance it, optim/src/amp.rs:66-76)
        std::vector<Var> listed;
        for (int32_t i = 0; i < n; ++i) listed.push_back(params[i]->v);
        MCB_TRY(scaler_reconcile(scaler->s, &opt->opt, listed));
    }
    std::map<Arena *, ArenaHost> arenas;
    std::vector<Entry> entries;
    for (int32_t i = 0; i < n; ++i) {
        const Var &v = params[i]->v;
        if (v->data.dt != MCB_F32) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "checkpoint_save: parameter %s is not f32", names[i]);
        int64_t cnt = v->data.numel();
        const float *hp = nullptr, *hm = nullptr, *hv = nullptr;
        std::vector<float> tp, tm, tv;
        int64_t t = 0;
        if (v->arena) {
            Arena *a = v->arena;
            auto it = arenas.find(a);
            if (it == arenas.end()) {
                MCB_TRY(arena_wait_comm(a));
                ArenaHost h;
                h.p.resize(a->total);
                MCB_TRY(mcb_memcpy_d2h(ctx, h.p.data(), a->p->p, sizeof(float) * a->total));
                if (opt) {
                    h.m.resize(a->total);
                    h.v.resize(a->total);
                    MCB_TRY(mcb_memcpy_d2h(ctx, h.m.data(), a->m->p, sizeof(float) * a->total));
                    MCB_TRY(mcb_memcpy_d2h(ctx, h.v.data(), a->v->p, sizeof(float) * a->total));
                }
                it = arenas.emplace(a, std::move(h)).first;
            }
            int64_t off = a->off[v->arena_idx];
            hp = it->second.p.data() + off;
            if (opt) {
                hm = it->second.m.data() + off;
                hv = it->second.v.data() + off;
                t = a->step[v->arena_idx];
            }
        } else {
            tp.resize(cnt);
            MCB_TRY(mcb_memcpy_d2h(ctx, tp.data(), v->data.ptr, sizeof(float) * cnt));
            hp = tp.data();
            if (opt) {
                auto st = opt->opt.state.find(v.get());
                tm.assign(cnt, 0.0f);
                tv.assign(cnt, 0.0f);
                if (st != opt->opt.state.end() && st->second.m.defined) {
                    MCB_TRY(mcb_memcpy_d2h(ctx, tm.data(), st->second.m.ptr, sizeof(float) * cnt));
                    MCB_TRY(mcb_memcpy_d2h(ctx, tv.data(), st->second.v.ptr, sizeof(float) * cnt));
                    t = st->second.t;
                }
                hm = tm.data();
                hv = tv.data();
            }
        }
        std::string name = names[i];
        entries.push_back(f32_entry(name, v->data.shape, hp, cnt));
        if (opt) {
            entries.push_back(f32_entry(name + ".opt_m", v->data.shape, hm, cnt));
            entries.push_back(f32_entry(name + ".opt_v", v->data.shape, hv, cnt));
            Entry te;
            te.name = name + ".opt_t";
            te.tag = TAG_I64;
            te.dims = {1};
            te.bytes.resize(8);
            memcpy(te.bytes.data(), &t, 8);
            entries.push_back(te);
        }
    }
    if (scaler) {
        float sf[2];
        int32_t si[4];
        MCB_TRY(mcb_memcpy_d2h(ctx, sf, scaler->s->state_f(), sizeof(sf)));
        MCB_TRY(mcb_memcpy_d2h(ctx, si, scaler->s->state_i(), sizeof(si)));
        entries.push_back(f32_entry("grad_scaler.state", {2}, sf, 2));
        Entry ce;
        ce.name = "grad_scaler.counters";
        ce.tag = TAG_I32;
        ce.dims = {4};
        ce.bytes.resize(sizeof(si));
        memcpy(ce.bytes.data(), si, sizeof(si));
        entries.push_back(ce);
    }
    FILE *f = fopen(path, "wb");
    if (!f) return mcb_fail(ctx, MCB_IO, "cannot create %s", path);
    std::vector<unsigned char> head(8);
    memcpy(head.data(), "MCHN0001", 8);
    put_u32(head, (uint32_t)entries.size());
    bool ok = fwrite(head.data(), 1, head.size(), f) == head.size();
    for (size_t i = 0; i < entries.size() && ok; ++i) ok = write_entry(f, entries[i]);
    ok = (fclose(f) == 0) && ok;
    if (!ok) return mcb_fail(ctx, MCB_IO, "short write to %s", path);
    return MCB_OK;
}

mcb_status mcb_checkpoint_load(mcb_ctx *ctx, const char *path, const char *const *names, mcb_var **params, int32_t n, mcb_adam *opt,
                               mcb_scaler *scaler) {
    MCB_CHECK_CTX(ctx);
    if (!path || n < 0 || (n > 0 && (!names || !params))) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "checkpoint_load: bad arguments");
    std::map<std::string, Entry> file;
    MCB_TRY(read_file(ctx, path, &file, nullptr));
    // check everything before touching device memory, so a bad file leaves the model as it was
    for (int32_t i = 0; i < n; ++i) {
        const Var &v = params[i]->v;
        std::string name = names[i];
        const char *suffix[4] = {"", ".opt_m", ".opt_v", ".opt_t"};
        for (int k = 0; k < (opt ? 4 : 1); ++k) {
            auto it = file.find(name + suffix[k]);
            if (it == file.end()) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "checkpoint has no entry %s%s", names[i], suffix[k]);
            if (k < 3 && (it->second.tag != TAG_F32 || !same_shape(it->second, v->data.shape)))
                return mcb_fail(ctx, MCB_SHAPE_MISMATCH, "checkpoint entry %s%s does not match the parameter's f32 shape", names[i], suffix[k]);
            if (k == 3 && (it->second.tag != TAG_I64 || it->second.bytes.size() != 8))
                return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "checkpoint entry %s.opt_t must be one i64", names[i]);
        }
        if (v->data.dt != MCB_F32) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "checkpoint_load: parameter %s is not f32", names[i]);
    }
    if (scaler) {
        auto a = file.find("grad_scaler.state"), b = file.find("grad_scaler.counters");
        if (a == file.end() || b == file.end() || a->second.bytes.size() != 8 || b->second.bytes.size() != 16 || a->second.tag != TAG_F32 ||
            b->second.tag != TAG_I32)
            return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "checkpoint has no usable grad_scaler entries");
    }
    MCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    std::map<Arena *, ArenaHost> arenas;
    for (int32_t i = 0; i < n; ++i) {
        const Var &v = params[i]->v;
        std::string name = names[i];
        int64_t cnt = v->data.numel();
        const Entry &ep = file[name];
        int64_t t = 0;
        if (opt) memcpy(&t, file[name + ".opt_t"].bytes.data(), 8);
        if (t < 0 || t > INT32_MAX) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "checkpoint entry %s.opt_t is out of range", names[i]);
        if (v->arena) {
            Arena *a = v->arena;
            auto it = arenas.find(a);
            if (it == arenas.end()) {
                // start from the current contents so that slots of parameters not listed keep their values
                ArenaHost h;
                h.p.resize(a->total);
                MCB_TRY(mcb_memcpy_d2h(ctx, h.p.data(), a->p->p, sizeof(float) * a->total));
                if (opt) {
                    h.m.resize(a->total);
                    h.v.resize(a->total);
                    MCB_TRY(mcb_memcpy_d2h(ctx, h.m.data(), a->m->p, sizeof(float) * a->total));
                    MCB_TRY(mcb_memcpy_d2h(ctx, h.v.data(), a->v->p, sizeof(float) * a->total));
                }
                it = arenas.emplace(a, std::move(h)).first;
            }
            int64_t off = a->off[v->arena_idx];
            if (cnt) memcpy(it->second.p.data() + off, ep.bytes.data(), sizeof(float) * cnt);
            if (opt) {
                if (cnt) memcpy(it->second.m.data() + off, file[name + ".opt_m"].bytes.data(), sizeof(float) * cnt);
                if (cnt) memcpy(it->second.v.data() + off, file[name + ".opt_v"].bytes.data(), sizeof(float) * cnt);
                a->step[v->arena_idx] = (int32_t)t;
            }
        } else {
            MCB_TRY(mcb_memcpy_h2d(ctx, v->data.ptr, ep.bytes.data(), sizeof(float) * cnt));
            if (opt) {
                AdamState &st = opt->opt.state[v.get()];
                if (!st.m.defined) {
                    MCB_TRY(new_tensor(ctx, MCB_F32, v->data.shape, &st.m));
                    MCB_TRY(new_tensor(ctx, MCB_F32, v->data.shape, &st.v));
                }
                MCB_TRY(mcb_memcpy_h2d(ctx, st.m.ptr, file[name + ".opt_m"].bytes.data(), sizeof(float) * cnt));
                MCB_TRY(mcb_memcpy_h2d(ctx, st.v.ptr, file[name + ".opt_v"].bytes.data(), sizeof(float) * cnt));
                st.t = (int32_t)t;
            }
        }
    }
    for (auto &kv : arenas) {
        Arena *a = kv.first;
        MCB_TRY(mcb_memcpy_h2d(ctx, a->p->p, kv.second.p.data(), sizeof(float) * a->total));
        if (opt) {
            MCB_TRY(mcb_memcpy_h2d(ctx, a->m->p, kv.second.m.data(), sizeof(float) * a->total));
            MCB_TRY(mcb_memcpy_h2d(ctx, a->v->p, kv.second.v.data(), sizeof(float) * a->total));
        }
        a->shadow_valid = false; // the bf16 copy of the weights is rebuilt on next use
    }
    if (scaler) {
        MCB_TRY(mcb_memcpy_h2d(ctx, scaler->s->state_f(), file["grad_scaler.state"].bytes.data(), 8));
        MCB_TRY(mcb_memcpy_h2d(ctx, scaler->s->state_i(), file["grad_scaler.counters"].bytes.data(), 16));
        int32_t counters[4];
        memcpy(counters, file["grad_scaler.counters"].bytes.data(), 16);
        scaler->s->issued_since = 0; // the loaded step counts are counts of applied steps
        scaler->s->applied_seen = counters[3];
    }
    MCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MCB_OK;
}

} // extern "C"
