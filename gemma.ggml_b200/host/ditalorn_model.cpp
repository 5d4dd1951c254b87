// ditalorn_model.cpp — see ditalorn_model.h
#include "ditalorn_model.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "lm_weights.h"
#include "seq_cache.h"

#define DL_OP(name, expr)                        \
    do {                                         \
        ggb_prof_start(name);                    \
        const int rc__ = (expr);                 \
        ggb_prof_stop(name);                     \
        if (rc__ != 0) return fail(rc__, #expr); \
    } while (0)

#define DL_TRY(expr)                             \
    do {                                         \
        const int rc__ = (expr);                 \
        if (rc__ != 0) return fail(rc__, #expr); \
    } while (0)

int ditalorn_model::fail(int rc, const std::string &what) {
    if (err_.empty() || rc != GGB_ERR_ARG) err_ = what + ": " + ggb_last_error();
    return rc;
}

// ------------------------------------------------------------------------------------------------ configuration
int dl_parse_config(const json_value &j, const safetensors_file *file, dl_config *c, std::string *err) {
    auto bad = [&](const std::string &m) {
        if (err) *err = "config.json: " + m;
        return -1;
    };
    // a size the configuration leaves out: dimension `axis` of a tensor, 0 when there is neither
    auto shape_of = [&](const std::string &name, size_t axis) -> long long {
        const st_tensor *t = file ? file->find(name) : nullptr;
        return t && t->shape.size() > axis ? (long long)t->shape[axis] : 0;
    };
    c->vocab = (int)j.integer("vocab", shape_of("embed", 0));
    c->width = (int)j.integer("width", shape_of("embed", 1));
    if (c->vocab <= 0 || c->width <= 0) return bad("vocab and width must be positive");
    c->max_positions = j.integer("max_positions", shape_of("pos", 0));
    if (file && shape_of("pos", 0) > 0) c->max_positions = std::min<int64_t>(c->max_positions, shape_of("pos", 0));
    if (c->max_positions <= 0) return bad("max_positions must be positive");
    if (const json_value *n = j.get("norm")) c->eps = (float)n->number("eps", 1e-5);
    if (const json_value *e = j.get("embedding")) c->embed_scale = (float)e->number("scale", 1.0);
    const json_value *layers = j.get("layers");
    if (!layers || layers->kind != json_value::ARR || layers->arr.empty()) return bad("'layers' must be a list");
    for (size_t i = 0; i < layers->arr.size(); i++) {
        const json_value &L = layers->arr[i];
        const std::string where = "layer " + std::to_string(i) + ": ", p = "l" + std::to_string(i) + ".mix.";
        const std::string type = L.string("type", "");
        const json_value *m = L.get("mixer");
        if (!m) return bad(where + "no 'mixer'");
        dl_layer_cfg l;
        if (type == "attention") {
            l.type = 0;
            dl_attn_cfg &a = l.attn;
            a.heads = (int)m->integer("heads", 0);
            a.kv_heads = (int)m->integer("kv_heads", a.heads);
            a.dim = (int)m->integer("dim", a.heads > 0 ? shape_of(p + "q", 0) / a.heads : 0);
            a.vdim = (int)m->integer("vdim", a.kv_heads > 0 && shape_of(p + "v", 0) ? shape_of(p + "v", 0) / a.kv_heads : a.dim);
            a.conv = (int)m->integer("conv", shape_of(p + "q.conv", 1));
            a.scale = (float)m->number("scale", 1.0);
            if (const json_value *t = m->get("q_temp")) {
                a.temp_coef = (float)t->number("coef", 0.0);
                a.temp_every = (int)t->integer("every", 0);
                if (a.temp_every <= 0) return bad(where + "q_temp.every must be positive");
            }
            if (a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads || a.dim <= 0 || a.vdim <= 0)
                return bad(where + "sizes must be positive and kv_heads must divide heads");
            if (a.conv < 0 || a.conv > 8) return bad(where + "conv must have at most 8 taps");
            if (a.vdim > 256) return bad(where + "vdim above 256 is not built");
        } else if (type == "latent_attention") {
            l.type = 1;
            dl_latent_cfg &a = l.latent;
            a.heads = (int)m->integer("heads", 0);
            a.q_rank = (int)m->integer("q_rank", shape_of(p + "dq", 0));
            a.kv_rank = (int)m->integer("kv_rank", shape_of(p + "dkv", 0));
            a.dim = (int)m->integer("dim", a.heads > 0 ? shape_of(p + "uq", 0) / a.heads : 0);
            a.vdim = (int)m->integer("vdim", a.heads > 0 && shape_of(p + "uv", 0) ? shape_of(p + "uv", 0) / a.heads : a.dim);
            a.scale = (float)m->number("scale", 1.0);
            if (const json_value *k = m->get("mask")) a.window = k->integer("size", 0);
            if (a.heads <= 0 || a.q_rank <= 0 || a.kv_rank <= 0 || a.dim <= 0 || a.vdim <= 0 || a.window < 0)
                return bad(where + "sizes must be positive");
            if (a.kv_rank > 1024) return bad(where + "kv_rank above 1024 is not built");
        } else {
            return bad(where + "unknown mixer type '" + type + "'");
        }
        if (const json_value *f = L.get("mlp")) {
            const std::string kind = f->string("kind", "moe");
            if (kind != "moe") return bad(where + "unknown mlp kind '" + kind + "'");
            dl_moe_cfg &e = l.moe;
            const std::string q = "l" + std::to_string(i) + ".mlp.";
            if (const json_value *x = f->get("expert")) e.ff = (int)x->integer("ff", 0);
            if (e.ff <= 0) e.ff = (int)shape_of(q + "e0.gate", 0);
            const json_value *r = f->get("router");
            if (!r) return bad(where + "a mixture of experts needs a 'router'");
            e.experts = (int)r->integer("experts", shape_of(q + "router", 0));
            e.top = (int)r->integer("top", 0);
            if (const json_value *g = r->get("groups")) {
                e.groups = (int)g->integer("count", 1);
                e.keep = (int)g->integer("keep", e.groups);
            }
            if (e.ff <= 0 || e.experts <= 0 || e.top <= 0 || e.top > e.experts) return bad(where + "ff, experts and top must be positive, top at most experts");
            if (e.groups <= 0 || e.experts % e.groups || e.keep <= 0 || e.keep > e.groups || e.top > e.keep * (e.experts / e.groups))
                return bad(where + "groups.count must divide the experts and the groups that stay must hold 'top' experts");
        }
        c->layers.push_back(l);
    }
    return 0;
}

// ------------------------------------------------------------------------------------------------ weights
int ditalorn_model::upload_matrix(const std::vector<float> &host, void **dev) {
    const size_t n = host.size();
    void *d = nullptr;
    DL_TRY(ggb_buffer_alloc(std::max<size_t>(n, 8) * ggb_dtype_size(dt_), &d));
    owned_.push_back(d);
    if (dt_ == GGB_TYPE_BF16) {
        std::vector<uint16_t> h(n);
        for (size_t i = 0; i < n; i++) h[i] = f32_to_bf16(host[i]);
        DL_TRY(ggb_upload(d, h.data(), n * 2));
        DL_TRY(ggb_sync());
    } else {
        DL_TRY(ggb_upload(d, host.data(), n * 4));
        DL_TRY(ggb_sync());
    }
    weight_bytes_ += n * ggb_dtype_size(dt_);
    *dev = d;
    return 0;
}

int ditalorn_model::upload_f32(const std::vector<float> &host, float **dev) {
    void *d = nullptr;
    DL_TRY(ggb_buffer_alloc(std::max<size_t>(host.size(), 4) * 4, &d));
    owned_.push_back(d);
    DL_TRY(ggb_upload(d, host.data(), host.size() * 4));
    DL_TRY(ggb_sync());
    weight_bytes_ += host.size() * 4;
    *dev = (float *)d;
    return 0;
}

int ditalorn_model::load(const safetensors_file *file, uint64_t seed) {
    const dl_config &c = cfg_;
    const int64_t W = c.width, V = c.vocab;
    weight_source src{file, seed, &err_};
    std::vector<float> a, b;
#define DL_GET(...)                                   \
    do {                                              \
        if (src.get(__VA_ARGS__)) return GGB_ERR_ARG; \
    } while (0)
#define DL_F32(name, n, amp, mean, dst)    \
    do {                                   \
        DL_GET(name, 1, n, amp, mean, &a); \
        DL_TRY(upload_f32(a, dst));        \
    } while (0)
    // a layer norm's weight is stored around zero and multiplies as 1 + w
#define DL_NORM(name, dst)                  \
    do {                                    \
        DL_GET(name, 1, W, 0.1f, 0.f, &a);  \
        for (float &v : a) v = 1.0f + v;    \
        DL_TRY(upload_f32(a, dst));         \
    } while (0)
    const float aw = std::sqrt(3.0f / (float)W);
    auto amp = [](int64_t fan_in) { return std::sqrt(3.0f / (float)fan_in); };
    DL_GET("embed", V, W, 1.7f / std::max(1.0f, c.embed_scale), 0.f, &a);
    DL_TRY(upload_matrix(a, &embed_));
    DL_GET("pos", c.max_positions, W, 0.5f, 0.f, &a);
    DL_TRY(upload_matrix(a, &pos_));
    DL_NORM("final.norm", &final_norm_);
    lw_.assign(c.layers.size(), dl_layer_w());
    int n_cache = 0;
    int64_t st = 0;
    std::vector<float> stack;
    auto push = [&](const std::string &name, int64_t rows, float amplitude) -> int {
        if (src.get(name, rows, W, amplitude, 0.f, &b)) return GGB_ERR_ARG;
        stack.insert(stack.end(), b.begin(), b.end());
        return 0;
    };
    for (size_t li = 0; li < c.layers.size(); li++) {
        const dl_layer_cfg &l = c.layers[li];
        dl_layer_w &w = lw_[li];
        const std::string p = "l" + std::to_string(li) + ".", m = p + "mix.";
        DL_NORM(p + "norm1", &w.norm1);
        DL_NORM(p + "norm1b", &w.norm1b);
        stack.clear();
        w.cache_index = n_cache++;
        if (l.type == 0) {
            const dl_attn_cfg &A = l.attn;
            const int64_t HD = (int64_t)A.heads * A.dim, GD = (int64_t)A.kv_heads * A.dim, GV = (int64_t)A.kv_heads * A.vdim, C = HD + GD + GV;
            DL_TRY(push(m + "q", HD, aw));
            DL_TRY(push(m + "k", GD, aw));
            DL_TRY(push(m + "v", GV, aw));
            std::vector<float> bias, cw;
            DL_GET(m + "q.b", 1, HD, 0.2f, 0.f, &a);
            bias.insert(bias.end(), a.begin(), a.end());
            DL_GET(m + "k.b", 1, GD, 0.2f, 0.f, &a);
            bias.insert(bias.end(), a.begin(), a.end());
            DL_GET(m + "v.b", 1, GV, 0.2f, 0.f, &a);
            bias.insert(bias.end(), a.begin(), a.end());
            DL_TRY(upload_f32(bias, &w.proj_b));
            if (A.conv >= 1) { // the three convolutions side by side, as their channels lie in the stacked product
                DL_GET(m + "q.conv", HD, A.conv, 0.5f, 0.f, &a);
                cw.insert(cw.end(), a.begin(), a.end());
                DL_GET(m + "k.conv", GD, A.conv, 0.5f, 0.f, &a);
                cw.insert(cw.end(), a.begin(), a.end());
                DL_GET(m + "v.conv", GV, A.conv, 0.5f, 0.f, &a);
                cw.insert(cw.end(), a.begin(), a.end());
                w.s_tail = st;
                st += ((int64_t)(A.conv - 1) * C + 3) / 4 * 4;
            } else { // no convolution: one tap of weight one, the biased projection as it is
                cw.assign((size_t)C, 1.0f);
            }
            DL_TRY(upload_f32(cw, &w.conv));
            DL_F32(m + "r1", A.heads, 0.4f, 0.5f, &w.r1);
            DL_F32(m + "r2", A.heads, 0.4f, 0.5f, &w.r2);
            DL_F32(m + "pb", A.heads, 1.0f, -2.0f, &w.pb);
            DL_GET(m + "o", W, (int64_t)A.heads * A.vdim, amp((int64_t)A.heads * A.vdim), 0.f, &a);
            DL_TRY(upload_matrix(a, &w.o));
            DL_F32(m + "o.b", W, 0.1f, 0.f, &w.o_b);
        } else {
            const dl_latent_cfg &A = l.latent;
            const int64_t HD = (int64_t)A.heads * A.dim, HV = (int64_t)A.heads * A.vdim;
            DL_TRY(push(m + "dq", A.q_rank, aw));
            DL_TRY(push(m + "dkv", A.kv_rank, aw));
            DL_TRY(push(m + "g", A.heads, aw));
            DL_F32(m + "dq.norm", A.q_rank, 0.1f, 1.0f, &w.dq_norm);
            DL_F32(m + "dkv.norm", A.kv_rank, 0.1f, 1.0f, &w.dkv_norm);
            DL_GET(m + "uq", HD, A.q_rank, amp(A.q_rank), 0.f, &a);
            DL_TRY(upload_matrix(a, &w.uq));
            DL_GET(m + "uk", HD, A.kv_rank, amp(A.kv_rank), 0.f, &a);
            DL_TRY(upload_matrix(a, &w.uk));
            DL_GET(m + "uv", HV, A.kv_rank, amp(A.kv_rank), 0.f, &b);
            DL_TRY(upload_matrix(b, &w.uv));
            a.insert(a.end(), b.begin(), b.end());
            DL_TRY(upload_matrix(a, &w.ukv));
            DL_GET(m + "o", W, HV, amp(HV), 0.f, &a);
            DL_TRY(upload_matrix(a, &w.o));
        }
        w.n_proj = ((int64_t)(stack.size() / (size_t)W) + 31) / 32 * 32; // whole tiles for the tensor-core product
        stack.resize((size_t)(w.n_proj * W), 0.f);
        DL_TRY(upload_matrix(stack, &w.proj));
        if (l.moe.experts > 0) {
            const dl_moe_cfg &E = l.moe;
            const std::string f = p + "mlp.";
            DL_NORM(p + "norm2", &w.norm2);
            DL_NORM(p + "norm2b", &w.norm2b);
            std::vector<float> gu, dn;
            gu.reserve((size_t)E.experts * 2 * (size_t)E.ff * (size_t)W);
            dn.reserve((size_t)E.experts * (size_t)E.ff * (size_t)W);
            for (int e = 0; e < E.experts; e++) {
                const std::string q = f + "e" + std::to_string(e) + ".";
                DL_GET(q + "gate", E.ff, W, aw, 0.f, &a);
                gu.insert(gu.end(), a.begin(), a.end());
                DL_GET(q + "up", E.ff, W, aw, 0.f, &a);
                gu.insert(gu.end(), a.begin(), a.end());
                DL_GET(q + "down", W, E.ff, amp(E.ff), 0.f, &a);
                dn.insert(dn.end(), a.begin(), a.end());
            }
            DL_TRY(upload_matrix(gu, &w.e_gate_up));
            DL_TRY(upload_matrix(dn, &w.e_down));
            DL_GET(f + "router", E.experts, W, aw, 0.f, &a);
            DL_TRY(upload_f32(a, &w.router));
            DL_F32(f + "correction", E.experts, 0.1f, 0.f, &w.correction);
        }
    }
#undef DL_GET
#undef DL_F32
#undef DL_NORM
    state_elems_ = st;
    // pages behind the widest window are never read again; one layer that sees everything keeps everything
    lookback_ = 0;
    for (const dl_layer_cfg &l : c.layers) {
        if (l.type == 0 || l.latent.window <= 0) {
            lookback_ = 0;
            break;
        }
        lookback_ = std::max(lookback_, l.latent.window);
    }
    return 0;
}

lm_model *ditalorn_model::create(const std::string &dir, const json_value &cfg, const lm_load_options &opt, std::string *err) {
    ditalorn_model *m = new ditalorn_model();
    safetensors_file file;
    m->dt_ = opt.dtype;
    if (opt.max_portion > 0) m->max_T_ = opt.max_portion;
    int rc = 0;
    if (!ggb_dtype_size(m->dt_)) rc = -1, m->err_ = "Ditalorn runs in bfloat16 or float32";
    if (!rc && !opt.random_weights) rc = file.open(dir + "/model.safetensors", &m->err_);
    if (!rc) rc = dl_parse_config(cfg, opt.random_weights ? nullptr : &file, &m->cfg_, &m->err_);
    if (!rc) rc = m->load(opt.random_weights ? nullptr : &file, opt.seed);
    if (rc) {
        if (err) *err = m->err_;
        delete m;
        return nullptr;
    }
    return m;
}

ditalorn_model::~ditalorn_model() {
    ggb_sync();
    for (step_graph &g : graphs_) ggb_graph_free(g.graph);
    for (void *p : owned_) ggb_buffer_free(p);
}

std::vector<int64_t> ditalorn_model::cache_row_elems() const {
    std::vector<int64_t> v;
    for (const dl_layer_cfg &l : cfg_.layers)
        v.push_back(l.type == 0 ? ggb_window_cache_ld(l.attn.kv_heads, l.attn.dim, l.attn.vdim) : ggb_latent_cache_ld(l.latent.kv_rank, 0));
    return v;
}

// ------------------------------------------------------------------------------------------------ buffers
int ditalorn_model::alloc_scratch() {
    const dl_config &c = cfg_;
    const int64_t T = max_T_, W = c.width;
    int64_t npr = 0, ncv = 0, nq = 0, nqa = 0, nhr = 0, nao = 0, nrq = 0, slots = 0, gu = 0, ffs = 0, ints = 0, top = 0, n_exp = 0;
    int hmax = 1;
    for (size_t li = 0; li < c.layers.size(); li++) {
        const dl_layer_cfg &l = c.layers[li];
        npr = std::max(npr, lw_[li].n_proj);
        if (l.type == 0) {
            const dl_attn_cfg &A = l.attn;
            ncv = std::max(ncv, (int64_t)A.heads * A.dim + (int64_t)A.kv_heads * (A.dim + A.vdim));
            nq = std::max(nq, (int64_t)A.heads * A.dim);
            nao = std::max(nao, (int64_t)A.heads * A.vdim);
            hmax = std::max(hmax, A.heads);
        } else {
            const dl_latent_cfg &A = l.latent;
            nq = std::max(nq, (int64_t)A.heads * A.dim);
            nqa = std::max(nqa, (int64_t)A.heads * A.kv_rank);
            nhr = std::max(nhr, (int64_t)A.heads * (A.kv_rank + 2));
            nao = std::max(nao, (int64_t)A.heads * A.vdim);
            nrq = std::max(nrq, (int64_t)A.q_rank);
        }
        if (l.moe.experts > 0) {
            slots = std::max(slots, T * l.moe.top);
            gu = std::max(gu, T * l.moe.top * 2 * l.moe.ff);
            ffs = std::max(ffs, T * l.moe.top * l.moe.ff);
            ints = std::max(ints, (int64_t)ggb_moe_group_ints(T * l.moe.top, l.moe.experts));
            top = std::max(top, (int64_t)l.moe.top);
            n_exp = std::max(n_exp, (int64_t)l.moe.experts);
        }
    }
    part_rows_ = std::max<int64_t>(T, 320);
    const size_t es = ggb_dtype_size(dt_);
    // the materialised form of the latent attention: room for the widest visible range of a portion, if that is modest
    int64_t ldkv = 0, rmax = 0;
    kv_rows_ = 0;
    for (const dl_layer_cfg &l : c.layers)
        if (l.type == 1) {
            const dl_latent_cfg &A = l.latent;
            const int64_t rows = std::min<int64_t>(max_pos_, A.window > 0 ? A.window + T : max_pos_);
            if (!materialise(A, (int)T)) continue;
            kv_rows_ = std::max(kv_rows_, rows);
            ldkv = std::max(ldkv, ggb_window_cache_ld(A.heads, A.dim, A.vdim));
            rmax = std::max(rmax, (int64_t)A.kv_rank);
        }
    if ((size_t)kv_rows_ * (size_t)ldkv * (4 + es) > ((size_t)512 << 20)) kv_rows_ = 0; // too much: the absorbed form everywhere
    auto alloc = [&](size_t bytes, void **p) -> int {
        DL_TRY(ggb_buffer_alloc(std::max<size_t>(bytes, 16), p));
        owned_.push_back(*p);
        return 0;
    };
#define DL_ALLOC(ptr, bytes) DL_TRY(alloc((size_t)(bytes), (void **)&(ptr)))
    DL_ALLOC(ids_, T * 4);
    DL_ALLOC(want_, T * 4);
    DL_ALLOC(iota_, T * 4);
    DL_ALLOC(pos0_, 16);
    DL_ALLOC(x_, T * W * 4);
    DL_ALLOC(h_, T * W * es);
    DL_ALLOC(pr_, T * npr * 4);
    DL_ALLOC(cv_, T * ncv * 4);
    DL_ALLOC(q_, T * nq * 4);
    DL_ALLOC(cq_, T * nrq * es);
    DL_ALLOC(qa_, T * nqa * 4);
    DL_ALLOC(part_, part_rows_ * nhr * 4);
    DL_ALLOC(sa_, ggb_sigmoid_attn_scratch_bytes(hmax));
    DL_ALLOC(ao_, T * nao * es);
    DL_ALLOC(ya_, T * W * 4);
    DL_ALLOC(route_i_, T * top * 4);
    DL_ALLOC(route_w_, T * top * 4);
    DL_ALLOC(route_z_, T * n_exp * 4);
    DL_ALLOC(group_ws_, ints * 4);
    DL_ALLOC(gu_, gu * 4);
    DL_ALLOC(act_, ffs * es);
    DL_ALLOC(y2_, slots * W * 4);
    DL_ALLOC(xw_, T * W * 4);
    DL_ALLOC(hw_, T * W * es);
    DL_ALLOC(logits_, T * (int64_t)c.vocab * 4);
    DL_ALLOC(posrel_, c.layers.size() * 4);
    if (kv_rows_ > 0) {
        DL_ALLOC(crows_, kv_rows_ * rmax * es);
        DL_ALLOC(kv_, kv_rows_ * ldkv * es);
        if (dt_ == GGB_TYPE_BF16) DL_ALLOC(kvf_, kv_rows_ * ldkv * 4);
        const int64_t np = kv_rows_ / cache_->page_size() + 2;
        DL_ALLOC(page_iota_, np * 4);
        std::vector<int32_t> pi((size_t)np);
        for (int64_t i = 0; i < np; i++) pi[(size_t)i] = (int32_t)i;
        DL_TRY(ggb_upload(page_iota_, pi.data(), (size_t)np * 4));
    }
#undef DL_ALLOC
    std::vector<int32_t> iota((size_t)T);
    for (int64_t i = 0; i < T; i++) iota[(size_t)i] = (int32_t)i;
    DL_TRY(ggb_upload(iota_, iota.data(), (size_t)T * 4));
    DL_TRY(ggb_sync());
    return 0;
}

int ditalorn_model::bind_cache(paged_cache *cache, int64_t max_positions) {
    cache_ = cache;
    max_pos_ = std::min(max_positions, cfg_.max_positions); // the learned position rows end there
    if ((int)cache_row_elems().size() != cache->n_layers()) return fail(GGB_ERR_ARG, "the cache has another number of layers than the model");
    if (cache->state_elems() < state_elems_) return fail(GGB_ERR_ARG, "the cache keeps less state per sequence than the model needs");
    return alloc_scratch();
}

// The absorbed form scores against the latent (2 R multiply-adds per key and head, twice); the materialised form multiplies
// the visible latents by [W_uk; W_uv] once per portion (a tensor-core product) and then pays D + Dv per key and head in the
// window attention kernel.  Portions take the second when heads are short beside the latent; steps always take the first.
bool ditalorn_model::materialise(const dl_latent_cfg &a, int T) const {
    return T >= 32 && a.vdim % 2 == 0 && a.vdim <= 256 && 4 * (int64_t)(a.dim + a.vdim) <= 5 * (int64_t)a.kv_rank && !getenv("GGB_LATENT_ABSORBED");
}

// ------------------------------------------------------------------------------------------------ one portion
int ditalorn_model::emit(int T, int64_t pos0, int ns, const int32_t *table, float *state, int n_want) {
    const dl_config &c = cfg_;
    const int64_t W = c.width, t = T;
    const int B = cache_->page_size();
    // the embedding and the first layer's norm in one pass
    DL_OP("op_rows", ggb_op_embed_pos(dt_, embed_, pos_, ids_, pos0_, t, W, c.embed_scale, x_, lw_[0].norm1, c.eps, h_));
    for (size_t li = 0; li < c.layers.size(); li++) {
        const dl_layer_cfg &l = c.layers[li];
        const dl_layer_w &w = lw_[li];
        const int64_t N = w.n_proj;
        void *cache = cache_->layer(w.cache_index);
        const bool ff = l.moe.experts > 0, last = li + 1 == c.layers.size();
        const float *next_norm = last ? nullptr : lw_[li + 1].norm1; // the norm in front of the next layer's mixer
        // every projection that reads the mixer's input in one product
        DL_OP("op_linear", ggb_op_linear(dt_, w.proj, N, W, h_, W, t, pr_, N));
        const float *mixer_bias = nullptr;
        if (l.type == 0) {
            const dl_attn_cfg &A = l.attn;
            const int64_t HD = (int64_t)A.heads * A.dim, GD = (int64_t)A.kv_heads * A.dim, GV = (int64_t)A.kv_heads * A.vdim, C = HD + GD + GV;
            DL_OP("op_conv", ggb_op_causal_conv_bias(dt_, pr_, N, t, C, w.conv, w.proj_b, std::max(A.conv, 1), 0, 0, A.conv > 1 ? state + w.s_tail : nullptr, cv_, C,
                                                     nullptr));
            DL_OP("op_attn_prep", ggb_op_sigmoid_qkv_store(dt_, cv_, cv_ + HD, cv_ + HD + GD, C, t, A.heads, A.kv_heads, A.dim, A.vdim, A.temp_coef,
                                                           A.temp_every, c.eps, A.scale, pos0_, table, B, cache, q_));
            DL_OP("op_sigmoid_attn", ggb_op_sigmoid_attn(dt_, q_, cache, table, B, pos0_, t, A.heads, A.kv_heads, A.dim, A.vdim, 0, w.r1, w.r2, w.pb, ao_, sa_));
            DL_OP("op_linear", ggb_op_linear(dt_, w.o, W, (int64_t)A.heads * A.vdim, ao_, (int64_t)A.heads * A.vdim, t, ya_, W));
            mixer_bias = w.o_b;
        } else {
            const dl_latent_cfg &A = l.latent;
            const int H = A.heads, D = A.dim, Dv = A.vdim, R = A.kv_rank, Rq = A.q_rank;
            DL_OP("op_norm", ggb_op_rms_norm2(dt_, pr_, N, w.dq_norm, 1, nullptr, 0, c.eps, Rq, t, cq_, nullptr));
            DL_OP("op_linear", ggb_op_linear(dt_, w.uq, (int64_t)H * D, Rq, cq_, Rq, t, q_, (int64_t)H * D));
            DL_OP("op_attn_prep", ggb_op_latent_kv_store(dt_, pr_ + Rq, N, t, R, 0, 0, w.dkv_norm, c.eps, nullptr, pos0_, table, B, cache));
            const int64_t first = A.window > 0 ? std::max<int64_t>(0, pos0 - A.window + 1) : 0, n_vis = pos0 + T - first;
            if (kv_rows_ >= n_vis && materialise(A, T)) {
                const int64_t ldkv = ggb_window_cache_ld(H, D, Dv);
                DL_OP("op_attn_prep", ggb_op_latent_expand(dt_, cache, table, B, first, n_vis, R, 0, w.ukv, (int64_t)H * (D + Dv), crows_, kvf_, kv_, ldkv));
                DL_OP("op_attn_prep", ggb_op_scale(q_, A.scale, t * H * D, q_));
                DL_OP("op_attn", ggb_op_window_attn(dt_, q_, kv_, page_iota_, B, posrel_ + li, t, H, H, D, Dv, A.window, nullptr, ao_, nullptr));
                DL_OP("op_attn_out", ggb_op_head_gate(dt_, ao_, t, H, Dv, pr_ + Rq + R, N));
            } else {
                DL_OP("op_attn_prep", ggb_op_latent_q_absorb(dt_, q_, (int64_t)H * D, t, H, D, 0, 0, nullptr, pos0_, w.uk, R, A.scale, qa_));
                DL_OP("op_attn", ggb_op_latent_attn_window(dt_, qa_, cache, table, B, pos0_, t, H, R, 0, A.window, ns, part_));
                DL_OP("op_attn_out", ggb_op_latent_attn_out_gated(dt_, part_, ns, nullptr, w.uv, t, H, R, Dv, pr_ + Rq + R, N, ao_));
            }
            DL_OP("op_linear", ggb_op_linear(dt_, w.o, W, (int64_t)H * Dv, ao_, (int64_t)H * Dv, t, ya_, W));
        }
        // x += norm1b(mixer), and the norm in front of what reads x next, in one pass
        const float *after = ff ? w.norm2 : next_norm;
        DL_OP("op_residual", ggb_op_norm_add_norm(dt_, ya_, mixer_bias, w.norm1b, c.eps, W, t, x_, after, after ? h_ : nullptr));
        if (ff) {
            const dl_moe_cfg &E = l.moe;
            // a step of few slots: the router lists the slots itself and every slot is a mat-vec with the gate folded in
            const bool step = ggb_moe_step_form(t * E.top) != 0;
            DL_OP("op_moe", ggb_op_moe_route_sigmoid(dt_, h_, W, t, w.router, w.correction, E.experts, E.top, E.groups, E.keep, route_z_, route_i_, route_w_,
                                                     group_ws_));
            if (step) {
                DL_OP("op_moe_linear", ggb_op_moe_linear(dt_, w.e_gate_up, E.ff, W, h_, W, 1, t, E.top, E.experts, group_ws_, 2, act_, E.ff));
            } else {
                DL_OP("op_moe", ggb_op_moe_group(route_i_, t, E.top, E.experts, group_ws_));
                DL_OP("op_moe_linear", ggb_op_moe_linear(dt_, w.e_gate_up, 2 * (int64_t)E.ff, W, h_, W, 1, t, E.top, E.experts, group_ws_, 0, gu_, 2 * (int64_t)E.ff));
                DL_OP("op_act", ggb_op_glu_bias(dt_, gu_, E.ff, t * E.top, nullptr, nullptr, 1, act_));
            }
            DL_OP("op_moe_linear", ggb_op_moe_linear(dt_, w.e_down, W, E.ff, act_, E.ff, 0, t, E.top, E.experts, group_ws_, 0, y2_, W));
            // the weighted sum of the slots, x += norm2b(.), and the norm in front of the next layer, in one pass
            if (E.top <= GGB_MOE_COMBINE_NORM_MAX_TOP) {
                DL_OP("op_residual", ggb_op_moe_combine_norm(dt_, y2_, group_ws_, route_w_, t, E.top, E.experts, W, w.norm2b, c.eps, x_, next_norm, next_norm ? h_ : nullptr));
            } else {
                DL_OP("op_moe", ggb_op_moe_combine(y2_, group_ws_, route_w_, t, E.top, E.experts, W, ya_));
                DL_OP("op_residual", ggb_op_norm_add_norm(dt_, ya_, nullptr, w.norm2b, c.eps, W, t, x_, next_norm, next_norm ? h_ : nullptr));
            }
        }
        if (capture_ && cap_) DL_OP("op_rows", ggb_op_gather_rows_f32(x_, iota_, t, W, cap_ + li * (size_t)max_T_ * (size_t)W));
    }
    if (n_want > 0) {
        DL_OP("op_rows", ggb_op_gather_rows_f32(x_, want_, n_want, W, xw_));
        DL_OP("op_norm", ggb_op_rms_norm2(dt_, xw_, W, final_norm_, 1, nullptr, 0, c.eps, W, n_want, hw_, nullptr));
        DL_OP("op_linear", ggb_op_linear(dt_, embed_, c.vocab, W, hw_, W, n_want, logits_, c.vocab));
    }
    return 0;
}

int ditalorn_model::forward(const lm_portion &p, const int32_t *want, int n_want) {
    if (!cache_) return fail(GGB_ERR_ARG, "forward before bind_cache");
    if (p.T <= 0 || p.T > max_T_ || n_want < 0 || n_want > p.T || p.pos0 < 0 || p.pos0 + p.T > max_pos_ || (state_elems_ > 0 && !p.state_dev)) {
        err_ = "forward: a portion of " + std::to_string(p.T) + " tokens at position " + std::to_string(p.pos0) + " does not fit (" +
               std::to_string(max_pos_) + " positions)";
        return GGB_ERR_ARG;
    }
    for (int i = 0; i < p.T; i++)
        if (p.tokens[i] < 0 || p.tokens[i] >= cfg_.vocab) {
            err_ = "forward: token " + std::to_string(p.tokens[i]) + " is outside the vocabulary";
            return GGB_ERR_ARG;
        }
    const int32_t pos0 = (int32_t)p.pos0;
    DL_TRY(ggb_upload(ids_, p.tokens, (size_t)p.T * 4));
    DL_TRY(ggb_upload(pos0_, &pos0, 4));
    if (n_want) DL_TRY(ggb_upload(want_, want, (size_t)n_want * 4));
    if (p.T > 1) { // the portion's position counted from the first one a latent layer's window shows (materialised form)
        std::vector<int32_t> rel(cfg_.layers.size(), 0);
        for (size_t li = 0; li < cfg_.layers.size(); li++) {
            const dl_layer_cfg &l = cfg_.layers[li];
            if (l.type == 1) rel[li] = (int32_t)(p.pos0 - (l.latent.window > 0 ? std::max<int64_t>(0, p.pos0 - l.latent.window + 1) : 0));
        }
        DL_TRY(ggb_upload(posrel_, rel.data(), rel.size() * 4));
    }
    // splits of a latent layer's visible positions (the widest window bounds them): enough CTAs for a short portion, one
    // split once the tokens fill the GPU
    int64_t n_vis = 1;
    for (const dl_layer_cfg &l : cfg_.layers)
        if (l.type == 1) n_vis = std::max(n_vis, l.latent.window > 0 ? std::min<int64_t>(p.pos0 + p.T, l.latent.window + p.T + 30) : p.pos0 + p.T);
    int64_t ns = std::min<int64_t>((n_vis + (p.T <= 8 ? 31 : 127)) / (p.T <= 8 ? 32 : 128), std::max<int64_t>(1, 296 / p.T));
    ns = std::max<int64_t>(1, std::min<int64_t>(ns, 64));
    if (p.T == 1) { // powers of two: the captured one-token step changes rarely
        int64_t q = 1;
        while (q < ns) q *= 2;
        ns = q;
    }
    while (ns > 1 && ns * p.T > part_rows_) ns--;
    const int64_t l0 = ggb_launch_count();
    if (capture_) {
        if (!cap_) {
            void *d = nullptr;
            DL_TRY(ggb_buffer_alloc(cfg_.layers.size() * (size_t)max_T_ * (size_t)cfg_.width * 4, &d));
            owned_.push_back(d);
            cap_ = (float *)d;
        }
        cap_T_ = p.T;
    }
    if (p.T == 1 && use_graphs_ && !capture_ && !getenv("GGB_NO_STEP_GRAPH")) {
        ggb_graph *g = nullptr;
        for (const step_graph &sg : graphs_)
            if (sg.table == p.block_table_dev && sg.state == p.state_dev && sg.n_split == (int)ns && sg.n_want == n_want) g = sg.graph;
        if (!g) {
            DL_TRY(ggb_capture_begin());
            const int rc = emit(1, p.pos0, (int)ns, p.block_table_dev, p.state_dev, n_want);
            const int rc2 = ggb_capture_end(&g);
            if (rc) return rc;
            if (rc2) return fail(rc2, "ggb_capture_end");
            if (graphs_.size() >= 32) {
                ggb_graph_free(graphs_.front().graph);
                graphs_.erase(graphs_.begin());
            }
            graphs_.push_back(step_graph{p.block_table_dev, p.state_dev, (int)ns, n_want, g});
        }
        DL_TRY(ggb_graph_launch(g));
    } else {
        DL_TRY(emit(p.T, p.pos0, (int)ns, p.block_table_dev, p.state_dev, n_want));
    }
    kernels_last_ = (int)(ggb_launch_count() - l0);
    return 0;
}

int ditalorn_model::get_capture(int layer, float *host, int64_t n) const {
    if (!cap_ || layer < 0 || layer >= (int)cfg_.layers.size() || n > (int64_t)cap_T_ * cfg_.width) return GGB_ERR_ARG;
    return ggb_download(host, cap_ + (size_t)layer * (size_t)max_T_ * (size_t)cfg_.width, (size_t)n * 4);
}

namespace {
struct register_ditalorn {
    register_ditalorn() { lm_register("Ditalorn", &ditalorn_model::create); }
} g_register_ditalorn;
} // namespace
