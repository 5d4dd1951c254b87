// capi.cpp — flat C entry points over gemma_model so tests / bench.py can drive the host side with
// ctypes (the reference drives its model from app::run, ref: src/app.cpp:30-44).
#include <cstdio>
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "gemma_model.h"
#include "gguf_loader.h"
#include "lm_engine.h"
#include "begupel_model.h"
#include "ditalorn_model.h"
#include "kibilix_model.h"
#include "safolorn_model.h"
#include "tensor_dump.h"

extern "C" {

void *gm_create(const gemma_config *cfg) { return new gemma_model(*cfg); }
void gm_free(void *m) { delete (gemma_model *)m; }
int gm_init_tensor_parallel(void *m, int rank, int size) { return ((gemma_model *)m)->init_tensor_parallel(rank, size); }
// host-only: fills out[18] = {valid, head0, heads, kv_head0, kv_heads, kv_replicated, q.row0, q.nrows, k.row0, k.nrows,
// o.row0, o.nrows, gate_up.row0, gate_up.nrows, down.row0, down.nrows, logits.row0, logits.nrows}
int gm_tp_plan(const gemma_config *cfg, int rank, int size, int64_t *out) {
    const tp_plan p = make_tp_plan(*cfg, rank, size);
    const int64_t v[18] = {p.valid, p.head0, p.heads, p.kv_head0, p.kv_heads, p.kv_replicated, p.q.row0, p.q.nrows,
                           p.k.row0, p.k.nrows, p.o.row0, p.o.nrows, p.gate_up.row0, p.gate_up.nrows, p.down.row0,
                           p.down.nrows, p.logits.row0, p.logits.nrows};
    for (int i = 0; i < 18; i++) out[i] = v[i];
    return p.valid ? 0 : -2;
}
int gm_init_synthetic_weights(void *m) { return ((gemma_model *)m)->init_synthetic_weights(); }
int gm_set_tensor(void *m, int tensor_id, const void *host, int64_t nbytes) {
    return ((gemma_model *)m)->set_tensor(tensor_id, host, nbytes);
}
int gm_set_tensor_typed(void *m, int tensor_id, int type, const void *host, int64_t nbytes) {
    return ((gemma_model *)m)->set_tensor_typed(tensor_id, type, host, nbytes);
}
int gm_kquant_mode(void *m) { return ((gemma_model *)m)->kquant_mode() ? 1 : 0; }
int gm_init_kv_cache(void *m) { return ((gemma_model *)m)->init_kv_cache(); }
int gm_fill_kv_cache_synthetic(void *m, uint64_t seed) { return ((gemma_model *)m)->fill_kv_cache_synthetic(seed); }
int gm_build_compute_graph(void *m, int capture_acts, int fused) {
    return ((gemma_model *)m)->build_compute_graph(capture_acts != 0, fused != 0);
}
void *gm_decoder(void *m) { return ((gemma_model *)m)->decoder(); }
int gm_is_fused(void *m) { return ((gemma_model *)m)->is_fused() ? 1 : 0; }
int gm_decode_step(void *m, int32_t token, int32_t pos, int32_t *next) {
    return ((gemma_model *)m)->decode_step(token, pos, next);
}
int gm_set_state(void *m, int32_t token, int32_t pos, int32_t pos_step) {
    return ((gemma_model *)m)->set_state(token, pos, pos_step);
}
int gm_run_steps(void *m, int steps) { return ((gemma_model *)m)->run_steps(steps); }
int gm_run_steps_profiled(void *m, int steps) { return ((gemma_model *)m)->run_steps_profiled(steps); }
int gm_get_state(void *m, int32_t *token, int32_t *pos) { return ((gemma_model *)m)->get_state(token, pos); }
int gm_generate(void *m, const int32_t *prompt, int n_prompt, int n_decode, int32_t *out, int *n_out, double *prefill_ms,
                double *decode_ms) {
    std::vector<token_id> p(prompt, prompt + n_prompt), o;
    const int rc = ((gemma_model *)m)->generate(p, n_decode, o, prefill_ms, decode_ms);
    if (rc) return rc;
    if (n_out) *n_out = (int)o.size();
    memcpy(out, o.data(), o.size() * sizeof(int32_t));
    return 0;
}
// ---- GGUF loader + tokenizer.  gm_gguf_probe parses a file on the host only (no GPU needed).
static thread_local std::string g_capi_err;
const char *gm_last_error() { return g_capi_err.c_str(); }
int gm_gguf_probe(const char *path, gemma_config *cfg, int32_t *n_tensors, int32_t *n_kv, int32_t *n_tokens, int32_t *bos, int32_t *eos) {
    gguf_file f;
    if (f.open(path) != 0) { g_capi_err = f.error(); return -1; }
    if (gguf_gemma_config(f, 0, cfg, &g_capi_err) != 0) return -2;
    gemma_tokenizer tok;
    const bool has_tok = gguf_gemma_tokenizer(f, &tok) == 0;
    if (n_tensors) *n_tensors = (int32_t)f.tensors().size();
    if (n_kv) *n_kv = (int32_t)f.n_kv();
    if (n_tokens) *n_tokens = has_tok ? (int32_t)tok.tokens.size() : 0;
    if (bos) *bos = tok.special_bos_id;
    if (eos) *eos = tok.special_eos_id;
    return 0;
}
// detokenise with the vocabulary of a GGUF file (host only): "▁" -> " ", leading "<bos>" dropped; returns the length
int gm_gguf_detokenize(const char *path, const int32_t *ids, int n, char *buf, int cap) {
    gguf_file f;
    if (f.open(path) != 0) { g_capi_err = f.error(); return -1; }
    gemma_tokenizer tok;
    if (gguf_gemma_tokenizer(f, &tok) != 0) { g_capi_err = "no tokenizer.ggml.tokens in the file"; return -2; }
    const std::string t = tok.tokens_text(std::vector<token_id>(ids, ids + n));
    if (buf && cap > 0) {
        const size_t k = t.size() < (size_t)cap - 1 ? t.size() : (size_t)cap - 1;
        memcpy(buf, t.data(), k);
        buf[k] = 0;
    }
    return (int)t.size();
}
void *gm_load_model_from_file(const char *path, int32_t n_ctx) {
    gemma_model *m = gemma_model::load_model_from_file(path, n_ctx, &g_capi_err);
    return m;
}
int gm_get_config(void *m, gemma_config *cfg) {
    *cfg = ((gemma_model *)m)->config();
    return 0;
}
int gm_begin_one_round_inference(void *m, const int32_t *prompt, int n_prompt, int max_tokens, int32_t *out, int *n_out,
                                 char *text, int text_cap, double *prefill_ms, double *decode_ms) {
    std::vector<token_id> p(prompt, prompt + n_prompt), o;
    std::string t;
    const int rc = ((gemma_model *)m)->begin_one_round_inference(p, max_tokens, o, text ? &t : nullptr, prefill_ms, decode_ms);
    if (rc) return rc;
    if (n_out) *n_out = (int)o.size();
    memcpy(out, o.data(), o.size() * sizeof(int32_t));
    if (text && text_cap > 0) {
        const size_t k = t.size() < (size_t)text_cap - 1 ? t.size() : (size_t)text_cap - 1;
        memcpy(text, t.data(), k);
        text[k] = 0;
    }
    return 0;
}
int gm_prefill(void *m, const int32_t *tokens, int T, int32_t pos0, int32_t *next) {
    return ((gemma_model *)m)->prefill(tokens, T, pos0, next);
}
int gm_get_prefill_logits(void *m, int row, float *host) { return ((gemma_model *)m)->get_prefill_logits(row, host); }
double gm_last_prefill_gemm_flops(void *m) { return ((gemma_model *)m)->last_prefill_gemm_flops(); }
int gm_get_logits(void *m, float *host) { return ((gemma_model *)m)->get_logits(host); }
int gm_get_capture(void *m, const char *name, int layer, float *host, int64_t n) {
    return ((gemma_model *)m)->get_capture(name, layer, host, n);
}
int gm_get_kv(void *m, int layer, void *k_host, void *v_host) { return ((gemma_model *)m)->get_kv(layer, k_host, v_host); }
int gm_kernels_per_step(void *m) { return ((gemma_model *)m)->kernels_per_step(); }
uint64_t gm_weight_bytes(void *m) { return (uint64_t)((gemma_model *)m)->weight_bytes(); }

// ---- the serving engine over the architecture registry (host/lm_engine.h): a model folder with config.json and
// model.safetensors (or a configuration text with random weights), sequences by name, steps of token portions
void *lm_engine_open(const char *dir, const char *config_text, int dtype, int64_t max_tokens, int page_size, int max_seqs,
                     int max_portion, int random_weights, uint64_t seed) {
    lm_load_options opt;
    opt.dtype = dtype;
    opt.max_tokens = max_tokens;
    opt.max_portion = max_portion;
    opt.random_weights = random_weights != 0;
    opt.seed = seed;
    lm_model *m = config_text && *config_text ? lm_load_config(config_text, dir ? dir : "", opt, &g_capi_err)
                                              : lm_load(dir ? dir : "", opt, &g_capi_err);
    if (!m) return nullptr;
    lm_engine *e = new lm_engine();
    if (e->init(m, max_tokens, page_size, max_seqs)) {
        g_capi_err = e->error();
        delete e;
        return nullptr;
    }
    return e;
}
void lm_engine_close(void *e) { delete (lm_engine *)e; }
const char *lm_engine_error(void *e) { return ((lm_engine *)e)->error().c_str(); }
int lm_engine_vocab(void *e) { return ((lm_engine *)e)->model()->vocab(); }
const char *lm_engine_architecture(void *e) { return ((lm_engine *)e)->model()->architecture(); }
// entries: ids[i], tokens[i][n_tokens[i]], want[i][n_want[i]]; logits_out receives sum(n_want) rows of vocab floats
int lm_engine_step(void *e, int n_entries, const char *const *ids, const int32_t *const *tokens, const int32_t *n_tokens,
                   const int32_t *const *want, const int32_t *n_want, int n_end, const char *const *end_ids, float *logits_out) {
    std::vector<lm_entry> es((size_t)n_entries);
    for (int i = 0; i < n_entries; i++) {
        es[(size_t)i].id = ids[i];
        es[(size_t)i].tokens.assign(tokens[i], tokens[i] + n_tokens[i]);
        es[(size_t)i].want.assign(want[i], want[i] + n_want[i]);
    }
    std::vector<std::string> end;
    for (int i = 0; i < n_end; i++) end.push_back(end_ids[i]);
    std::vector<float> logits;
    const int rc = ((lm_engine *)e)->step(es, end, &logits);
    if (rc) return rc;
    if (logits_out && !logits.empty()) memcpy(logits_out, logits.data(), logits.size() * 4);
    return 0;
}
int lm_engine_generate(void *e, const char *id, const int32_t *prompt, int n_prompt, int n_new, int32_t *out) {
    std::vector<int32_t> o;
    const int rc = ((lm_engine *)e)->generate(id, std::vector<int32_t>(prompt, prompt + n_prompt), n_new, &o);
    if (rc) return rc;
    memcpy(out, o.data(), o.size() * 4);
    return 0;
}
// out[6] = {live sequences, free pages, pages, page size, kernels of the last forward call, weight bytes}
int lm_engine_stats(void *e, int64_t *out) {
    lm_engine *g = (lm_engine *)e;
    out[0] = g->live_seqs();
    out[1] = g->cache()->free_pages();
    out[2] = g->cache()->n_pages();
    out[3] = g->cache()->page_size();
    out[4] = g->model()->kernels_last_forward();
    out[5] = (int64_t)g->model()->weight_bytes();
    return 0;
}
int64_t lm_engine_seq_len(void *e, const char *id) { return ((lm_engine *)e)->seq_len(id); }
// pages of a live sequence (host copy): returns their number, fills at most cap
int lm_engine_seq_pages(void *e, const char *id, int32_t *out, int cap) { return ((lm_engine *)e)->seq_pages(id, out, cap); }
int lm_engine_capture(void *e, int on) { return ((lm_engine *)e)->model()->set_capture(on != 0); }
int lm_engine_use_graphs(void *e, int on) { return ((lm_engine *)e)->model()->set_use_graphs(on != 0); }
int lm_engine_get_capture(void *e, int layer, float *host, int64_t n) { return ((lm_engine *)e)->model()->get_capture(layer, host, n); }
// pages a live sequence holds now (trimmed ones not counted); -1: no such sequence
int lm_engine_seq_live_pages(void *e, const char *id) { return ((lm_engine *)e)->seq_live_pages(id); }
// host only: parses a Safolorn configuration text; out[5] = {layers, caching layers, vocab, width, side dim}; -1 and
// gm_last_error() when the configuration is refused
int sf_config_probe(const char *text, int64_t *out) {
    json_value j;
    sf_config c;
    if (!json_parser(text, strlen(text)).parse(&j, &g_capi_err)) return -1;
    if (sf_parse_config(j, &c, &g_capi_err)) return -1;
    int64_t own = 0;
    for (const auto &l : c.layers) own += l.kv_from < 0;
    out[0] = (int64_t)c.layers.size(); out[1] = own; out[2] = c.vocab; out[3] = c.width; out[4] = c.side_dim;
    return 0;
}
// host only: parses a Begupel configuration text; out[6] = {layers, layers with a window cache, vocab, width, norm groups,
// taps of the input convolution}; -1 and gm_last_error() when the configuration is refused
int bg_config_probe(const char *text, int64_t *out) {
    json_value j;
    bg_config c;
    if (!json_parser(text, strlen(text)).parse(&j, &g_capi_err)) return -1;
    if (bg_parse_config(j, &c, &g_capi_err)) return -1;
    int64_t win = 0;
    for (const auto &l : c.layers) win += l.type == 1;
    out[0] = (int64_t)c.layers.size(); out[1] = win; out[2] = c.vocab; out[3] = c.width; out[4] = c.groups; out[5] = c.taps;
    return 0;
}
// host only: parses a Ditalorn configuration text; out[8] = {layers, attention layers, latent layers, layers with experts,
// vocab, width, positions, widest window (0: some layer sees everything)}; -1 and gm_last_error() when it is refused
int dl_config_probe(const char *text, int64_t *out) {
    json_value j;
    dl_config c;
    if (!json_parser(text, strlen(text)).parse(&j, &g_capi_err)) return -1;
    if (dl_parse_config(j, nullptr, &c, &g_capi_err)) return -1;
    int64_t attn = 0, lat = 0, moe = 0, win = 0;
    bool bounded = true;
    for (const auto &l : c.layers) {
        attn += l.type == 0;
        lat += l.type == 1;
        moe += l.moe.experts > 0;
        if (l.type == 0 || l.latent.window <= 0) bounded = false;
        else win = std::max<int64_t>(win, l.latent.window);
    }
    out[0] = (int64_t)c.layers.size(); out[1] = attn; out[2] = lat; out[3] = moe; out[4] = c.vocab; out[5] = c.width;
    out[6] = c.max_positions; out[7] = bounded ? win : 0;
    return 0;
}
// host only: parses a Kibilix configuration text; out[8] = {layers, layer runs, attention runs, channel_delta runs, layers with
// experts, vocab, width, streams}; -1 and gm_last_error() when it is refused
int kb_config_probe(const char *text, int64_t *out) {
    json_value j;
    kb_config c;
    if (!json_parser(text, strlen(text)).parse(&j, &g_capi_err)) return -1;
    if (kb_parse_config(j, nullptr, &c, &g_capi_err)) return -1;
    int64_t attn = 0, delta = 0, moe = 0;
    for (int li : c.runs) {
        attn += c.layers[(size_t)li].type == 0;
        delta += c.layers[(size_t)li].type == 1;
    }
    for (const auto &l : c.layers) moe += l.ff_kind == 2;
    out[0] = (int64_t)c.layers.size(); out[1] = (int64_t)c.runs.size(); out[2] = attn; out[3] = delta; out[4] = moe; out[5] = c.vocab;
    out[6] = c.width; out[7] = c.streams;
    return 0;
}
// host only: a tensor of a .safetensors file: returns its number of dimensions (shape[0 .. 8) filled, *nbytes, dtype text),
// -1 when the file cannot be read, -2 when the tensor is not there
int st_probe(const char *path, const char *name, int64_t *shape, int64_t *nbytes, char *dtype, int dtype_cap, int64_t *n_tensors) {
    safetensors_file f;
    if (f.open(path, &g_capi_err)) return -1;
    if (n_tensors) *n_tensors = (int64_t)f.tensors().size();
    const st_tensor *t = f.find(name);
    if (!t) return -2;
    for (size_t i = 0; i < t->shape.size() && i < 8; i++) shape[i] = t->shape[i];
    if (nbytes) *nbytes = (int64_t)t->nbytes;
    if (dtype) snprintf(dtype, (size_t)dtype_cap, "%s", t->dtype.c_str());
    return (int)t->shape.size();
}
// the registered architecture names, comma separated
int lm_architectures_csv(char *buf, int cap) {
    std::string s;
    for (const auto &a : lm_architectures()) s += (s.empty() ? "" : ",") + a;
    snprintf(buf, (size_t)cap, "%s", s.c_str());
    return (int)s.size();
}

// ---- tensor_dump (ref: src/tensor_dump.h): host-side parity harness
void td_set_dir(const char *dir) { set_tensor_dump_dir(dir); }
int td_dump_ptr_data(const char *name, const void *ptr, uint64_t size, int target) {
    return dump_ptr_data(name, ptr, (size_t)size, target ? tensor_dump_mode::target : tensor_dump_mode::source) ? 0 : -1;
}
// a named intermediate of the model's last step, fetched from the device and dumped as "<name>-<layer>_source|_target"
int td_dump_capture(void *m, const char *name, int layer, int64_t n, int target) {
    std::vector<float> h((size_t)n);
    const int rc = ((gemma_model *)m)->get_capture(name, layer, h.data(), n);
    if (rc) return rc;
    const std::string file = std::string(name) + "-" + std::to_string(layer);
    return dump_ptr_data(file.c_str(), h.data(), h.size() * 4, target ? tensor_dump_mode::target : tensor_dump_mode::source) ? 0 : -1;
}
int td_compare_tensors(const char *name) { return compare_tensors(name) ? 1 : 0; }
// out[5] = {n, n_diff, max_abs, max_rel, max_target}; returns 0 if both files exist with equal fp32 sizes
int td_compare_tensors_report(const char *name, double *out) {
    tensor_compare_report r;
    if (!compare_tensors_report(name, &r)) return -1;
    out[0] = (double)r.n; out[1] = (double)r.n_diff; out[2] = r.max_abs; out[3] = r.max_rel; out[4] = r.max_target;
    return 0;
}

} // extern "C"
