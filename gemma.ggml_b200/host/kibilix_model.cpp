// kibilix_model.cpp — see kibilix_model.h
#include "kibilix_model.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "seq_cache.h"

#define KB_OP(name, expr)                        \
    do {                                         \
        ggb_prof_start(name);                    \
        const int rc__ = (expr);                 \
        ggb_prof_stop(name);                     \
        if (rc__ != 0) return fail(rc__, #expr); \
    } while (0)

#define KB_TRY(expr)                             \
    do {                                         \
        const int rc__ = (expr);                 \
        if (rc__ != 0) return fail(rc__, #expr); \
    } while (0)

static const float kExpertAlpha = 1.702f; // the experts' gate is g * sigmoid(1.702 g)

int kibilix_model::fail(int rc, const std::string &what) {
    if (err_.empty() || rc != GGB_ERR_ARG) err_ = what + ": " + ggb_last_error();
    return rc;
}

// ------------------------------------------------------------------------------------------------ configuration
int kb_parse_config(const json_value &j, const safetensors_file *file, kb_config *c, std::string *err) {
    auto bad = [&](const std::string &m) {
        if (err) *err = "config.json: " + m;
        return -1;
    };
    c->vocab = (int)j.integer("vocab", 0);
    c->width = (int)j.integer("width", 0);
    if (c->vocab <= 0 || c->width <= 0) return bad("vocab and width must be positive");
    if (const json_value *n = j.get("norm")) c->eps = (float)n->number("eps", 1e-6);
    c->residual_mult = (float)j.number("residual_mult", 1.0);
    c->streams = (int)j.integer("streams", 0);
    if (c->streams < 0 || c->streams > 16) return bad("streams must be between 1 and 16");
    if (const json_value *e = j.get("embedding"))
        if (const json_value *b = e->get("bigram")) {
            c->buckets = b->integer("buckets", 0);
            c->mul_prev = b->integer("mul_prev", 0);
            c->mul_cur = b->integer("mul_cur", 0);
            if (c->buckets <= 0) return bad("embedding.bigram.buckets must be positive");
        }
    const json_value *layers = j.get("layers");
    if (!layers || layers->kind != json_value::ARR || layers->arr.empty()) return bad("'layers' must be a list");
    const int64_t W = c->width;
    for (size_t i = 0; i < layers->arr.size(); i++) {
        const json_value &L = layers->arr[i];
        const std::string where = "layer " + std::to_string(i) + ": ";
        const std::string type = L.string("type", "");
        const json_value *m = L.get("mixer");
        if (!m) return bad(where + "no 'mixer'");
        kb_layer_cfg l;
        const int heads = (int)m->integer("heads", 0), dim = (int)m->integer("dim", 0);
        const int kv_heads = (int)m->integer("kv_heads", heads), vdim = (int)m->integer("vdim", dim);
        if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0)
            return bad(where + "mixer sizes must be positive and kv_heads must divide heads");
        if (type == "attention") {
            l.type = 0;
            kb_attn_cfg &a = l.attn;
            a.heads = heads, a.kv_heads = kv_heads, a.dim = dim, a.vdim = vdim;
            a.scale = (float)m->number("scale", 1.0 / std::sqrt((double)dim));
            a.softcap = (float)m->number("softcap", 0.0);
            if (a.softcap < 0.f) return bad(where + "softcap must be positive");
            if (const json_value *k = m->get("mask")) a.chunk = k->integer("size", 0);
            if (a.chunk < 0) return bad(where + "mask.size must be positive");
            if (dim % 2 || vdim % 2) return bad(where + "dim and vdim must be even");
            if (vdim > 256) return bad(where + "vdim above 256 is not built");
            if (const json_value *ro = m->get("rot")) {
                a.rot.dims = (int)ro->integer("dims", dim);
                a.rot.base = ro->number("base", 10000.0);
                if (a.rot.dims < 0 || a.rot.dims > dim || a.rot.dims % 2) return bad(where + "rot.dims must be even and at most dim");
                if (const json_value *s = ro->get("scaling")) {
                    a.rot.banded = true;
                    a.rot.factor = s->number("factor", 1.0);
                    a.rot.low = s->number("low", 1.0);
                    a.rot.high = s->number("high", 4.0);
                    a.rot.original = s->number("original", 0.0);
                    if (!(a.rot.factor > 0.0) || !(a.rot.original > 0.0) || !(a.rot.low > 0.0) || !(a.rot.high > a.rot.low))
                        return bad(where + "rot.scaling needs factor > 0, original > 0 and high > low > 0");
                }
            }
        } else if (type == "channel_delta") {
            l.type = 1;
            kb_delta_cfg &d = l.delta;
            d.heads = heads, d.kv_heads = kv_heads, d.dim = dim, d.vdim = vdim;
            const std::string p = "l" + std::to_string(i) + ".mix.";
            d.conv = (int)m->integer("conv", 0);
            if (d.conv == 0) { // not configured: as many taps as the file's tensor has, one (of weight 1: no convolution) without it
                const st_tensor *cw = file ? file->find(p + "q.conv") : nullptr;
                d.conv = cw && cw->shape.size() == 2 ? (int)cw->shape[1] : 1;
            }
            if (d.conv < 1 || d.conv > 8) return bad(where + "conv must be between 1 and 8 taps");
            if (dim > 256) return bad(where + "dim above 256 is not built");
            // the inner sizes of the two low-rank projections are the tensors' shapes; without a file, a quarter of the key size
            d.a_rank = d.g_rank = (int)m->integer("rank", std::max(8, (dim / 4 + 7) / 8 * 8));
            if (file) {
                const st_tensor *a1 = file->find(p + "a1"), *g1 = file->find(p + "g1");
                if (!a1 || !g1 || a1->shape.size() != 2 || g1->shape.size() != 2 || a1->shape[1] != W || g1->shape[1] != W)
                    return bad(where + "tensors '" + p + "a1' and '" + p + "g1' must be [rank, width]");
                d.a_rank = (int)a1->shape[0];
                d.g_rank = (int)g1->shape[0];
            }
            if (d.a_rank <= 0 || d.g_rank <= 0) return bad(where + "the low-rank projections need a positive rank");
        } else {
            return bad(where + "unknown mixer type '" + type + "'");
        }
        if (const json_value *f = L.get("mlp")) {
            const std::string kind = f->string("kind", "");
            if (kind == "dense") {
                l.ff_kind = 1;
                l.ff = (int)f->integer("ff", 0);
                if (l.ff <= 0) return bad(where + "ff must be positive");
            } else if (kind == "moe") {
                l.ff_kind = 2;
                const json_value *e = f->get("expert"), *r = f->get("router");
                if (!e || !r) return bad(where + "a mixture of experts needs 'expert' and 'router'");
                kb_moe_cfg &x = l.moe;
                x.ff = (int)e->integer("ff", 0);
                x.limit = e->get("limit") ? (float)e->number("limit", 0.0) : INFINITY; // not configured: nothing is clamped
                x.experts = (int)r->integer("experts", 0);
                x.identity = (int)r->integer("identity", 0);
                x.top = (int)r->integer("top", 0);
                if (x.ff <= 0 || x.experts <= 0 || x.identity < 0 || x.top <= 0 || x.top > x.experts + x.identity)
                    return bad(where + "experts, ff and top must be positive and top at most experts + identity");
                if (!(x.limit > 0.f)) return bad(where + "expert.limit must be positive");
                if (x.experts + x.identity > 4096) return bad(where + "more than 4096 experts are not built");
            } else {
                return bad(where + "unknown mlp kind '" + kind + "'");
            }
        }
        c->layers.push_back(l);
    }
    const int n = (int)c->layers.size();
    c->loop_start = c->loop_stop = 0;
    c->loop_times = 1;
    if (const json_value *lp = j.get("loop")) {
        c->loop_start = (int)lp->integer("start", 0);
        c->loop_stop = (int)lp->integer("stop", c->loop_start);
        c->loop_times = (int)lp->integer("times", 1);
        if (c->loop_start < 0 || c->loop_stop < c->loop_start || c->loop_stop > n || c->loop_times < 1)
            return bad("loop needs 0 <= start <= stop <= layers and times >= 1");
    }
    c->runs.clear();
    for (int i = 0; i < c->loop_start; i++) c->runs.push_back(i);
    for (int t = 0; t < c->loop_times; t++)
        for (int i = c->loop_start; i < c->loop_stop; i++) c->runs.push_back(i);
    for (int i = c->loop_stop; i < n; i++) c->runs.push_back(i);
    return 0;
}

// ------------------------------------------------------------------------------------------------ weights
int kibilix_model::upload_matrix(const std::vector<float> &host, void **dev) {
    const size_t n = host.size();
    void *d = nullptr;
    KB_TRY(ggb_buffer_alloc(std::max<size_t>(n, 8) * ggb_dtype_size(dt_), &d));
    owned_.push_back(d);
    if (dt_ == GGB_TYPE_BF16) {
        std::vector<uint16_t> h(n);
        for (size_t i = 0; i < n; i++) h[i] = f32_to_bf16(host[i]);
        KB_TRY(ggb_upload(d, h.data(), n * 2));
        KB_TRY(ggb_sync());
    } else {
        KB_TRY(ggb_upload(d, host.data(), n * 4));
        KB_TRY(ggb_sync());
    }
    weight_bytes_ += n * ggb_dtype_size(dt_);
    *dev = d;
    return 0;
}

int kibilix_model::upload_f32(const std::vector<float> &host, float **dev) {
    void *d = nullptr;
    KB_TRY(ggb_buffer_alloc(std::max<size_t>(host.size(), 4) * 4, &d));
    owned_.push_back(d);
    KB_TRY(ggb_upload(d, host.data(), host.size() * 4));
    KB_TRY(ggb_sync());
    weight_bytes_ += host.size() * 4;
    *dev = (float *)d;
    return 0;
}

// the stream weights of one sublayer; a model without streams gets the one-stream form of the plain residual sum
int kibilix_model::load_hyper(weight_source &src, const std::string &name, kb_hyper_w *w) {
    const int S = S_;
    const float m = cfg_.residual_mult;
    std::vector<float> in(1, 1.f), mix(1, 1.f), out(1, 1.f);
    if (cfg_.streams > 0) {
        if (src.get(name + ".in", 1, S, 0.3f, 1.0f / (float)S, &in)) return GGB_ERR_ARG;
        if (src.get(name + ".out", 1, S, 0.3f, 1.0f, &out)) return GGB_ERR_ARG;
        if (src.get(name + ".mix", S, S, 0.3f / (float)S, 0.f, &mix)) return GGB_ERR_ARG;
        if (!src.file)
            for (int s = 0; s < S; s++) mix[(size_t)s * S + s] += 1.0f; // random weights: near the identity
    }
    for (float &v : out) v = m * v;
    KB_TRY(upload_f32(in, &w->in));
    KB_TRY(upload_f32(mix, &w->mix));
    KB_TRY(upload_f32(out, &w->coef));
    return 0;
}

int kibilix_model::load(const safetensors_file *file, uint64_t seed) {
    const kb_config &c = cfg_;
    const int64_t W = c.width, V = c.vocab;
    weight_source src{file, seed, &err_};
    std::vector<float> a, b;
#define KB_GET(...)                                   \
    do {                                              \
        if (src.get(__VA_ARGS__)) return GGB_ERR_ARG; \
    } while (0)
#define KB_F32(name, n, amp, mean, dst)    \
    do {                                   \
        KB_GET(name, 1, n, amp, mean, &a); \
        KB_TRY(upload_f32(a, dst));        \
    } while (0)
    const float aw = std::sqrt(3.0f / (float)W);
    auto amp = [](int64_t fan_in) { return std::sqrt(3.0f / (float)fan_in); };
    KB_GET("embed", V, W, 1.7f, 0.f, &a);
    KB_TRY(upload_matrix(a, &embed_));
    if (c.buckets > 0) {
        KB_GET("bigram", c.buckets + 1, W, 1.0f, 0.f, &a);
        KB_TRY(upload_matrix(a, &bigram_));
    }
    KB_GET("head", V, W, aw, 0.f, &a);
    KB_TRY(upload_matrix(a, &head_));
    KB_F32("final.norm", W, 0.1f, 1.0f, &final_norm_);
    KB_TRY(upload_f32(std::vector<float>((size_t)S_, 1.0f), &ones_));
    lw_.assign(c.layers.size(), kb_layer_w());
    // stacks `name` (rows x W) below what `stack` already holds; returns the row it starts at
    std::vector<float> stack;
    auto push = [&](const std::string &name, int64_t rows, float amplitude, int64_t *at) -> int {
        *at = (int64_t)(stack.size() / (size_t)W);
        if (src.get(name, rows, W, amplitude, 0.f, &b)) return GGB_ERR_ARG;
        stack.insert(stack.end(), b.begin(), b.end());
        return 0;
    };
    for (size_t li = 0; li < c.layers.size(); li++) {
        const kb_layer_cfg &l = c.layers[li];
        kb_layer_w &w = lw_[li];
        const std::string p = "l" + std::to_string(li) + ".";
        KB_F32(p + "norm1", W, 0.1f, 1.0f, &w.norm1);
        KB_TRY(load_hyper(src, p + "hc1", &w.hc1));
        stack.clear();
        if (l.type == 0) {
            const kb_attn_cfg &A = l.attn;
            const int64_t H = A.heads, G = A.kv_heads, D = A.dim, Dv = A.vdim;
            KB_TRY(push(p + "mix.q", H * D, aw, &w.o_q));
            KB_TRY(push(p + "mix.k", G * D, aw, &w.o_k));
            KB_TRY(push(p + "mix.v", G * Dv, aw, &w.o_v));
            KB_GET(p + "mix.o", W, H * Dv, amp(H * Dv), 0.f, &a);
            KB_TRY(upload_matrix(a, &w.o));
        } else {
            const kb_delta_cfg &R = l.delta;
            const int64_t H = R.heads, G = R.kv_heads, D = R.dim, Dv = R.vdim;
            KB_TRY(push(p + "mix.q", G * D, aw, &w.o_q));
            KB_TRY(push(p + "mix.k", G * D, aw, &w.o_k));
            KB_TRY(push(p + "mix.v", H * Dv, aw, &w.o_v));
            KB_TRY(push(p + "mix.b", H, aw, &w.o_b));
            int64_t o_g1 = 0;
            KB_TRY(push(p + "mix.a1", R.a_rank, aw, &w.o_a1));
            KB_TRY(push(p + "mix.g1", R.g_rank, aw, &o_g1));
            // the three convolutions side by side, as their channels lie in the stacked product
            std::vector<float> cw;
            if (R.conv == 1 && file && !file->find(p + "mix.q.conv")) { // no convolution: one tap of weight 1
                cw.assign((size_t)(2 * G * D + H * Dv), 1.0f);
            } else {
                KB_GET(p + "mix.q.conv", G * D, R.conv, 0.5f, 0.f, &a);
                cw.insert(cw.end(), a.begin(), a.end());
                KB_GET(p + "mix.k.conv", G * D, R.conv, 0.5f, 0.f, &a);
                cw.insert(cw.end(), a.begin(), a.end());
                KB_GET(p + "mix.v.conv", H * Dv, R.conv, 0.5f, 0.f, &a);
                cw.insert(cw.end(), a.begin(), a.end());
            }
            KB_TRY(upload_f32(cw, &w.conv));
            KB_F32(p + "mix.A_log", H, 1.0f, -1.0f, &w.A_log);
            KB_F32(p + "mix.dt_bias", H * D, 1.0f, 0.f, &w.dt_bias);
            KB_F32(p + "mix.norm", Dv, 0.1f, 1.0f, &w.onorm);
            KB_GET(p + "mix.a2", H * D, R.a_rank, amp(R.a_rank), 0.f, &a);
            KB_TRY(upload_matrix(a, &w.a2));
            KB_GET(p + "mix.g2", H * Dv, R.g_rank, amp(R.g_rank), 0.f, &a);
            KB_TRY(upload_matrix(a, &w.g2));
            KB_GET(p + "mix.o", W, H * Dv, amp(H * Dv), 0.f, &a);
            KB_TRY(upload_matrix(a, &w.o));
        }
        w.n_proj = ((int64_t)(stack.size() / (size_t)W) + 31) / 32 * 32; // whole tiles for the tensor-core product
        stack.resize((size_t)(w.n_proj * W), 0.f);
        KB_TRY(upload_matrix(stack, &w.proj));
        if (l.ff_kind) {
            KB_F32(p + "norm2", W, 0.1f, 1.0f, &w.norm2);
            KB_TRY(load_hyper(src, p + "hc2", &w.hc2));
        }
        if (l.ff_kind == 1) {
            KB_GET(p + "mlp.up", l.ff, W, aw, 0.f, &a);
            KB_TRY(upload_matrix(a, &w.up));
            KB_GET(p + "mlp.down", W, l.ff, amp(l.ff), 0.f, &a);
            KB_TRY(upload_matrix(a, &w.down));
        } else if (l.ff_kind == 2) {
            const kb_moe_cfg &E = l.moe;
            const std::string f = p + "mlp.";
            std::vector<float> gu, dn;
            gu.reserve((size_t)E.experts * 2 * (size_t)E.ff * (size_t)W);
            dn.reserve((size_t)E.experts * (size_t)E.ff * (size_t)W);
            for (int e = 0; e < E.experts; e++) {
                const std::string q = f + "e" + std::to_string(e) + ".";
                KB_GET(q + "gate", E.ff, W, aw, 0.f, &a);
                gu.insert(gu.end(), a.begin(), a.end());
                KB_GET(q + "up", E.ff, W, aw, 0.f, &a);
                gu.insert(gu.end(), a.begin(), a.end());
                KB_GET(q + "down", W, E.ff, amp(E.ff), 0.f, &a);
                dn.insert(dn.end(), a.begin(), a.end());
            }
            KB_TRY(upload_matrix(gu, &w.e_gate_up));
            KB_TRY(upload_matrix(dn, &w.e_down));
            KB_GET(f + "router", E.experts + E.identity, W, aw, 0.f, &a);
            KB_TRY(upload_f32(a, &w.router));
            KB_F32(f + "correction", E.experts + E.identity, 0.1f, 0.f, &w.correction);
        }
    }
#undef KB_GET
#undef KB_F32
    // every layer RUN has a cache array or a piece of the state block of its own
    int n_cache = 0;
    int64_t st = 4; // number 0 of the block: the previous token
    auto take = [&](int64_t n) {
        const int64_t at = st;
        st += (n + 3) / 4 * 4;
        return at;
    };
    runs_.clear();
    bool bounded = true;
    lookback_ = 0;
    for (int li : c.runs) {
        const kb_layer_cfg &l = c.layers[(size_t)li];
        kb_run r;
        r.layer = li;
        if (l.type == 0) {
            r.cache_index = n_cache++;
            if (l.attn.chunk <= 0) bounded = false;
            lookback_ = std::max(lookback_, l.attn.chunk);
        } else {
            const kb_delta_cfg &R = l.delta;
            const int64_t C = 2 * (int64_t)R.kv_heads * R.dim + (int64_t)R.heads * R.vdim;
            if (R.conv > 1) r.s_conv = take((int64_t)(R.conv - 1) * C);
            r.s_S = take((int64_t)R.heads * R.dim * R.vdim);
        }
        runs_.push_back(r);
    }
    state_elems_ = st;
    // pages behind the widest chunk are never read again; one layer that sees everything keeps everything
    if (!bounded || n_cache == 0) lookback_ = 0;
    return 0;
}

lm_model *kibilix_model::create(const std::string &dir, const json_value &cfg, const lm_load_options &opt, std::string *err) {
    kibilix_model *m = new kibilix_model();
    safetensors_file file;
    m->dt_ = opt.dtype;
    if (opt.max_portion > 0) m->max_T_ = opt.max_portion;
    int rc = 0;
    if (!ggb_dtype_size(m->dt_)) rc = -1, m->err_ = "Kibilix runs in bfloat16 or float32";
    if (!rc && !opt.random_weights) rc = file.open(dir + "/model.safetensors", &m->err_);
    if (!rc) rc = kb_parse_config(cfg, opt.random_weights ? nullptr : &file, &m->cfg_, &m->err_);
    if (!rc) {
        m->S_ = std::max(m->cfg_.streams, 1);
        rc = m->load(opt.random_weights ? nullptr : &file, opt.seed);
    }
    if (rc) {
        if (err) *err = m->err_;
        delete m;
        return nullptr;
    }
    return m;
}

kibilix_model::~kibilix_model() {
    ggb_sync();
    for (step_graph &g : graphs_) ggb_graph_free(g.graph);
    for (void *p : owned_) ggb_buffer_free(p);
}

std::vector<int64_t> kibilix_model::cache_row_elems() const {
    std::vector<int64_t> v;
    for (const kb_run &r : runs_) {
        const kb_layer_cfg &l = cfg_.layers[(size_t)r.layer];
        if (l.type == 0) v.push_back(ggb_window_cache_ld(l.attn.kv_heads, l.attn.dim, l.attn.vdim));
    }
    return v;
}

// ------------------------------------------------------------------------------------------------ buffers
int kibilix_model::alloc_scratch() {
    const kb_config &c = cfg_;
    const int64_t T = max_T_, W = c.width;
    int64_t npr = 0, ncv = 0, nq = 0, nao = 0, nlr = 0, nda = 0, nro = 0, ff = 0, slots = 0, gu = 0, ffs = 0, ints = 0, n_exp = 0;
    int hmax = 1;
    for (size_t li = 0; li < c.layers.size(); li++) {
        const kb_layer_cfg &l = c.layers[li];
        npr = std::max(npr, lw_[li].n_proj);
        if (l.type == 0) {
            nq = std::max(nq, (int64_t)l.attn.heads * l.attn.dim);
            nao = std::max(nao, (int64_t)l.attn.heads * l.attn.vdim);
            hmax = std::max(hmax, l.attn.heads);
        } else {
            const kb_delta_cfg &R = l.delta;
            ncv = std::max(ncv, 2 * (int64_t)R.kv_heads * R.dim + (int64_t)R.heads * R.vdim);
            nlr = std::max(nlr, (int64_t)R.a_rank + R.g_rank);
            nda = std::max(nda, (int64_t)R.heads * R.dim);
            nro = std::max(nro, (int64_t)R.heads * R.vdim);
        }
        if (l.ff_kind == 1) ff = std::max(ff, (int64_t)l.ff);
        if (l.ff_kind == 2) {
            const int all = l.moe.experts + l.moe.identity;
            slots = std::max(slots, T * l.moe.top);
            gu = std::max(gu, T * l.moe.top * 2 * l.moe.ff);
            ffs = std::max(ffs, T * l.moe.top * l.moe.ff);
            ints = std::max(ints, (int64_t)ggb_moe_group_ints(T * l.moe.top, all));
            n_exp = std::max(n_exp, (int64_t)all);
        }
    }
    const size_t es = ggb_dtype_size(dt_);
    auto alloc = [&](size_t bytes, void **p) -> int {
        KB_TRY(ggb_buffer_alloc(std::max<size_t>(bytes, 16), p));
        owned_.push_back(*p);
        return 0;
    };
#define KB_ALLOC(ptr, bytes) KB_TRY(alloc((size_t)(bytes), (void **)&(ptr)))
    KB_ALLOC(ids_, T * 4);
    KB_ALLOC(want_, T * 4);
    KB_ALLOC(pos0_, 16);
    KB_ALLOC(x0_, T * W * 4);
    KB_ALLOC(xs_, T * S_ * W * 4);
    KB_ALLOC(h_, T * W * es);
    KB_ALLOC(pr_, T * npr * 4);
    KB_ALLOC(cv_, T * ncv * 4);
    KB_ALLOC(qr_, T * nq * 4);
    KB_ALLOC(ao_, T * nao * es);
    KB_ALLOC(wa_, ggb_window_attn_scratch_bytes(hmax));
    KB_ALLOC(lr_, T * nlr * es);
    KB_ALLOC(da_, T * nda * 4);
    KB_ALLOC(dg_, T * nro * 4);
    KB_ALLOC(ro_, T * nro * 4);
    KB_ALLOC(gd_, T * nro * es);
    KB_ALLOC(ya_, T * W * 4);
    KB_ALLOC(yb_, T * W * 4);
    KB_ALLOC(gu_, std::max(gu, T * ff) * 4);
    KB_ALLOC(act_, std::max(ffs, T * ff) * es);
    KB_ALLOC(y2_, slots * W * 4);
    KB_ALLOC(route_z_, T * n_exp * 4);
    KB_ALLOC(route_i_, slots * 4);
    KB_ALLOC(route_w_, slots * 4);
    KB_ALLOC(group_ws_, ints * 4);
    KB_ALLOC(hw_, T * W * es);
    KB_ALLOC(logits_, T * (int64_t)c.vocab * 4);
#undef KB_ALLOC
    return 0;
}

int kibilix_model::bind_cache(paged_cache *cache, int64_t max_positions) {
    cache_ = cache;
    max_pos_ = max_positions;
    if ((int)cache_row_elems().size() != cache->n_layers()) return fail(GGB_ERR_ARG, "the cache has another number of layers than the model");
    if (cache->state_elems() < state_elems_) return fail(GGB_ERR_ARG, "the cache keeps less state per sequence than the model needs");
    for (size_t li = 0; li < cfg_.layers.size(); li++) {
        const kb_layer_cfg &l = cfg_.layers[li];
        if (l.type != 0 || l.attn.rot.dims <= 0) continue;
        const std::string k = l.attn.rot.key();
        if (!rot_tables_.count(k)) {
            float *d = nullptr;
            KB_TRY(upload_f32(rot_table(l.attn.rot, max_positions), &d));
            rot_tables_[k] = d;
        }
        lw_[li].cs = rot_tables_[k];
    }
    return alloc_scratch();
}

// ------------------------------------------------------------------------------------------------ one portion
int kibilix_model::emit(int T, const int32_t *table, float *state, int n_want) {
    const kb_config &c = cfg_;
    const int64_t W = c.width, t = T;
    const int B = cache_->page_size();
    const size_t es = ggb_dtype_size(dt_);
    if (c.buckets > 0)
        KB_OP("op_rows", ggb_op_embed_bigram(dt_, embed_, bigram_, ids_, t, W, c.buckets, c.mul_prev, c.mul_cur, pos0_, (int32_t *)state, x0_));
    else
        KB_OP("op_rows", ggb_op_embed_rows(dt_, embed_, ids_, t, W, x0_));
    // a sublayer's output waits for the next pass over the streams: that pass renews them and reads the next sublayer's
    // input out in one launch
    // (experts: their weighted sum is taken in that launch too, from the slot rows)
    const float *start = x0_, *y = nullptr;
    const kb_hyper_w *from = nullptr;
    const kb_moe_cfg *slots = nullptr;
    auto streams = [&](const float *in, const float *nw, const int32_t *rows, int64_t n, float *u_out, void *h) -> int {
        if (slots)
            KB_OP("op_residual", ggb_op_hyper_mix_moe(dt_, xs_, y2_, group_ws_, route_w_, route_i_, t, slots->top, slots->experts + slots->identity,
                                                      slots->identity, h_, from->mix, from->coef, S_, in, nw, c.eps, W, n, rows, u_out, h));
        else
            KB_OP("op_residual", ggb_op_hyper_mix(dt_, xs_, start, y, from ? from->mix : nullptr, from ? from->coef : nullptr, S_, in, nw, c.eps, W, n,
                                                  rows, u_out, h));
        start = nullptr, y = nullptr, from = nullptr, slots = nullptr;
        return 0;
    };
    for (size_t ri = 0; ri < runs_.size(); ri++) {
        const kb_run &r = runs_[ri];
        const kb_layer_cfg &l = c.layers[(size_t)r.layer];
        const kb_layer_w &w = lw_[(size_t)r.layer];
        const int64_t N = w.n_proj;
        KB_TRY(streams(w.hc1.in, w.norm1, nullptr, t, nullptr, h_));
        KB_OP("op_linear", ggb_op_linear(dt_, w.proj, N, W, h_, W, t, pr_, N));
        if (l.type == 0) {
            const kb_attn_cfg &A = l.attn;
            void *cache = cache_->layer(r.cache_index);
            const int64_t HV = (int64_t)A.heads * A.vdim;
            KB_OP("op_attn_prep", ggb_op_masked_qkv_store(dt_, pr_ + w.o_q, pr_ + w.o_k, pr_ + w.o_v, N, t, A.heads, A.kv_heads, A.dim, A.vdim, nullptr,
                                                          nullptr, c.eps, A.rot.dims, 1, w.cs, nullptr, A.scale, pos0_, table, B, cache, qr_));
            KB_OP("op_attn", ggb_op_masked_attn(dt_, qr_, cache, table, B, pos0_, t, A.heads, A.kv_heads, A.dim, A.vdim, A.chunk, 1, A.softcap, nullptr,
                                                ao_, wa_));
            KB_OP("op_linear", ggb_op_linear(dt_, w.o, W, HV, ao_, HV, t, ya_, W));
        } else {
            const kb_delta_cfg &R = l.delta;
            const int64_t GD = (int64_t)R.kv_heads * R.dim, HD = (int64_t)R.heads * R.dim, RV = (int64_t)R.heads * R.vdim, C = 2 * GD + RV;
            const int64_t LR = (int64_t)R.a_rank + R.g_rank;
            KB_OP("op_conv", ggb_op_causal_conv(dt_, pr_ + w.o_q, N, t, C, w.conv, R.conv, 0, 1, R.conv > 1 ? state + r.s_conv : nullptr, cv_, C, nullptr));
            // the second halves of the two low-rank projections read the first halves in the matrices' type; the fused form
            // hands the recurrence the decays themselves
            const bool fused = ggb_lowrank_pair_fits(dt_, R.a_rank, R.g_rank) != 0;
            if (fused) {
                KB_OP("op_linear", ggb_op_lowrank_pair(dt_, pr_ + w.o_a1, N, t, w.a2, HD, R.a_rank, w.g2, RV, R.g_rank, w.A_log, w.dt_bias, R.dim, da_, dg_));
            } else {
                KB_OP("op_act", ggb_op_act_rows(dt_, pr_ + w.o_a1, N, t, LR, 0, lr_));
                KB_OP("op_linear", ggb_op_linear(dt_, w.a2, HD, R.a_rank, lr_, LR, t, da_, HD));
                KB_OP("op_linear", ggb_op_linear(dt_, w.g2, RV, R.g_rank, (const char *)lr_ + (size_t)R.a_rank * es, LR, t, dg_, RV));
            }
            KB_OP("op_recurrence", ggb_op_channel_delta(cv_, cv_ + GD, cv_ + 2 * GD, C, pr_ + w.o_b, N, da_, HD, fused ? 1 : 0, t, R.heads, R.kv_heads, R.dim,
                                                        R.vdim, w.A_log, w.dt_bias, state + r.s_S, ro_, RV));
            KB_OP("op_norm", ggb_op_norm_gate(dt_, ro_, RV, dg_, RV, t, R.heads, R.vdim, w.onorm, R.vdim, c.eps, 0, gd_));
            KB_OP("op_linear", ggb_op_linear(dt_, w.o, W, RV, gd_, RV, t, ya_, W));
        }
        y = ya_, from = &w.hc1;
        if (l.ff_kind) {
            KB_TRY(streams(w.hc2.in, w.norm2, nullptr, t, nullptr, h_));
            if (l.ff_kind == 1) {
                KB_OP("op_linear", ggb_op_linear_relu2(dt_, w.up, l.ff, W, h_, W, t, gu_, act_));
                KB_OP("op_linear", ggb_op_linear(dt_, w.down, W, l.ff, act_, l.ff, t, yb_, W));
            } else {
                const kb_moe_cfg &E = l.moe;
                const int all = E.experts + E.identity;
                // a step of few slots: the router lists the slots itself and every slot is a mat-vec with the gate folded in
                const bool step = ggb_moe_step_form(t * E.top) != 0;
                KB_OP("op_moe", ggb_op_moe_route_softmax(dt_, h_, W, t, w.router, w.correction, all, E.top, route_z_, route_i_, route_w_, group_ws_));
                if (step) {
                    KB_OP("op_moe_linear", ggb_op_moe_linear_identity(dt_, w.e_gate_up, E.ff, W, h_, W, 1, t, E.top, all, E.identity, group_ws_, 3, E.limit,
                                                                      kExpertAlpha, act_, E.ff));
                } else {
                    KB_OP("op_moe", ggb_op_moe_group_identity(route_i_, t, E.top, all, E.identity, group_ws_));
                    KB_OP("op_moe_linear", ggb_op_moe_linear_identity(dt_, w.e_gate_up, 2 * (int64_t)E.ff, W, h_, W, 1, t, E.top, all, E.identity, group_ws_, 0,
                                                                      0.f, 0.f, gu_, 2 * (int64_t)E.ff));
                    KB_OP("op_act", ggb_op_glu_clamp(dt_, gu_, E.ff, t * E.top, E.limit, kExpertAlpha, act_));
                }
                KB_OP("op_moe_linear", ggb_op_moe_linear_identity(dt_, w.e_down, W, E.ff, act_, E.ff, 0, t, E.top, all, E.identity, group_ws_, 0, 0.f, 0.f,
                                                                  y2_, W));
                if (E.top <= 64) slots = &E; // the weighted sum waits for the next pass over the streams
                else KB_OP("op_moe", ggb_op_moe_combine_identity(dt_, y2_, group_ws_, route_w_, route_i_, t, E.top, all, E.identity, W, h_, yb_));
            }
            y = yb_, from = &w.hc2;
        }
        if (capture_ && cap_) KB_TRY(streams(ones_, nullptr, nullptr, t, cap_ + ri * (size_t)max_T_ * (size_t)W, nullptr));
    }
    if (n_want > 0) {
        // the last sublayer's output enters on the way: only the wanted rows are computed, nothing is written back
        KB_TRY(streams(ones_, final_norm_, want_, n_want, nullptr, hw_));
        KB_OP("op_linear", ggb_op_linear(dt_, head_, c.vocab, W, hw_, W, n_want, logits_, c.vocab));
    }
    return 0;
}

int kibilix_model::forward(const lm_portion &p, const int32_t *want, int n_want) {
    if (!cache_) return fail(GGB_ERR_ARG, "forward before bind_cache");
    if (p.T <= 0 || p.T > max_T_ || n_want < 0 || n_want > p.T || p.pos0 < 0 || p.pos0 + p.T > max_pos_ || !p.state_dev) {
        err_ = "forward: a portion of " + std::to_string(p.T) + " tokens at position " + std::to_string(p.pos0) + " does not fit";
        return GGB_ERR_ARG;
    }
    for (int i = 0; i < p.T; i++)
        if (p.tokens[i] < 0 || p.tokens[i] >= cfg_.vocab) {
            err_ = "forward: token " + std::to_string(p.tokens[i]) + " is outside the vocabulary";
            return GGB_ERR_ARG;
        }
    const int32_t pos0 = (int32_t)p.pos0;
    KB_TRY(ggb_upload(ids_, p.tokens, (size_t)p.T * 4));
    KB_TRY(ggb_upload(pos0_, &pos0, 4));
    if (n_want) KB_TRY(ggb_upload(want_, want, (size_t)n_want * 4));
    const int64_t l0 = ggb_launch_count();
    if (capture_) {
        if (!cap_) {
            void *d = nullptr;
            KB_TRY(ggb_buffer_alloc(runs_.size() * (size_t)max_T_ * (size_t)cfg_.width * 4, &d));
            owned_.push_back(d);
            cap_ = (float *)d;
        }
        cap_T_ = p.T;
    }
    if (p.T == 1 && use_graphs_ && !capture_ && !getenv("GGB_NO_STEP_GRAPH")) {
        ggb_graph *g = nullptr;
        for (const step_graph &sg : graphs_)
            if (sg.table == p.block_table_dev && sg.state == p.state_dev && sg.n_want == n_want) g = sg.graph;
        if (!g) {
            KB_TRY(ggb_capture_begin());
            const int rc = emit(1, p.block_table_dev, p.state_dev, n_want);
            const int rc2 = ggb_capture_end(&g);
            if (rc) return rc;
            if (rc2) return fail(rc2, "ggb_capture_end");
            if (graphs_.size() >= 32) {
                ggb_graph_free(graphs_.front().graph);
                graphs_.erase(graphs_.begin());
            }
            graphs_.push_back(step_graph{p.block_table_dev, p.state_dev, n_want, g});
        }
        KB_TRY(ggb_graph_launch(g));
    } else {
        KB_TRY(emit(p.T, p.block_table_dev, p.state_dev, n_want));
    }
    kernels_last_ = (int)(ggb_launch_count() - l0);
    return 0;
}

int kibilix_model::get_capture(int run, float *host, int64_t n) const {
    if (!cap_ || run < 0 || run >= (int)runs_.size() || n > (int64_t)cap_T_ * cfg_.width) return GGB_ERR_ARG;
    return ggb_download(host, cap_ + (size_t)run * (size_t)max_T_ * (size_t)cfg_.width, (size_t)n * 4);
}

namespace {
struct register_kibilix {
    register_kibilix() { lm_register("Kibilix", &kibilix_model::create); }
} g_register_kibilix;
} // namespace
