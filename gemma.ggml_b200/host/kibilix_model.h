// kibilix_model.h — the Kibilix decoder: a hashed bigram row added to the token embedding; pre-norm layers whose residual
// is several streams (hyper-connections: a sublayer reads a weighted sum of the streams and its output enters all of
// them while they are mixed among themselves); two kinds of mixer in any order: "attention" (grouped-query soft-max
// attention inside chunks of consecutive positions, rotary positions in the halves layout with frequencies rescaled by
// wavelength, soft-capped scores) and "channel_delta" (a gated delta rule with short convolutions, unit q / k, and one
// decay per head and key channel from a low-rank projection; per-head RMS norm and a low-rank sigmoid gate on the way
// out); a squared-ReLU dense feed-forward or a mixture of clamped gated experts with a soft-max router over all
// experts, a choice correction and identity experts; a block of consecutive layers may run several times with the
// same weights.  Every size and constant comes from config.json or a tensor's shape.
//
// What a sequence carries: rows [k | v] of every attention layer RUN in the engine's paged cache (a layer that runs three
// times owns three arrays; pages behind the widest chunk go back to the pool while the sequence lives), and one block of
// fp32 state in the cache's per-sequence storage: the previous token and, per channel_delta run, the convolutions' tail
// and the matrices S.  The residual streams belong to a token and are not carried.
//
// The class lowers a portion of tokens to ggb_op_* operators (dense.cu, recurrent.cu, window_attention.cu, moe.cu), as
// the other designs do; positions, page tables and state are read on the device, so the one-token step is captured into
// a CUDA graph per sequence slot and replayed.
#pragma once

#include <map>
#include <string>
#include <vector>

#include "ggml_b200.h"
#include "lm_model.h"
#include "lm_weights.h"
#include "rotary.h"
#include "safetensors.h"

struct kb_attn_cfg {
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
    int64_t chunk = 0;    // 0: every earlier position
    float scale = 1.0f;
    float softcap = 0.0f; // 0: scores as they are
    rot_spec rot;         // dims 0: none
};

struct kb_delta_cfg {
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0, conv = 1;
    int a_rank = 0, g_rank = 0; // inner sizes of the decay's and the gate's projections (from the tensors' shapes)
};

struct kb_moe_cfg {
    int experts = 0, identity = 0, top = 0, ff = 0; // `experts` have matrices, `identity` more hand their input through
    float limit = 0.f;
};

struct kb_layer_cfg {
    int type = 0;    // 0 attention, 1 channel_delta
    kb_attn_cfg attn;
    kb_delta_cfg delta;
    int ff_kind = 0; // 0 none, 1 dense, 2 experts
    int ff = 0;      // dense
    kb_moe_cfg moe;
};

struct kb_config {
    int vocab = 0, width = 0;
    float eps = 1e-6f, residual_mult = 1.0f;
    int streams = 0; // 0: one residual, x += m * sublayer(norm(x))
    int64_t buckets = 0, mul_prev = 0, mul_cur = 0; // buckets 0: no bigram table
    int loop_start = 0, loop_stop = 0, loop_times = 1;
    std::vector<kb_layer_cfg> layers;
    std::vector<int> runs; // the layer of every layer run, in order (a looped layer appears once per pass)
};
// file: where the ranks of the low-rank projections are read from (null: a default from the key size)
int kb_parse_config(const json_value &j, const safetensors_file *file, kb_config *c, std::string *err);

struct kb_hyper_w { // one sublayer's stream weights: read-out, mix [from][to], m * out
    float *in = nullptr, *mix = nullptr, *coef = nullptr;
};

struct kb_layer_w {
    float *norm1 = nullptr, *norm2 = nullptr;
    kb_hyper_w hc1, hc2;
    void *proj = nullptr; // every matrix that reads the mixer's input, stacked (rows padded to a multiple of 32)
    int64_t n_proj = 0;
    int64_t o_q = 0, o_k = 0, o_v = 0, o_b = 0, o_a1 = 0; // a1 | g1 are neighbours
    void *o = nullptr;
    const float *cs = nullptr;                                                  // attention
    float *conv = nullptr, *A_log = nullptr, *dt_bias = nullptr, *onorm = nullptr; // channel_delta
    void *a2 = nullptr, *g2 = nullptr;
    void *up = nullptr, *down = nullptr;                                        // dense feed-forward
    void *e_gate_up = nullptr, *e_down = nullptr;                               // experts
    float *router = nullptr, *correction = nullptr;
};

struct kb_run {
    int layer = 0;
    int cache_index = -1;         // attention
    int64_t s_conv = 0, s_S = 0;  // channel_delta: offsets (fp32 numbers) into the sequence's state block
};

class kibilix_model : public lm_model {
  public:
    static lm_model *create(const std::string &dir, const json_value &cfg, const lm_load_options &opt, std::string *err);
    ~kibilix_model() override;

    const char *architecture() const override { return "Kibilix"; }
    int vocab() const override { return cfg_.vocab; }
    int dtype() const override { return dt_; }
    std::vector<int64_t> cache_row_elems() const override;
    int64_t state_elems() const override { return state_elems_; }
    int64_t cache_lookback() const override { return lookback_; }
    int bind_cache(paged_cache *cache, int64_t max_positions) override;
    int max_portion() const override { return max_T_; }
    int forward(const lm_portion &p, const int32_t *want, int n_want) override;
    const float *logits_dev() const override { return logits_; }
    std::string last_error() const override { return err_; }
    int set_capture(bool on) override {
        capture_ = on;
        return 0;
    }
    int set_use_graphs(bool on) override {
        use_graphs_ = on;
        return 0;
    }
    int get_capture(int run, float *host, int64_t n) const override; // the sum of the streams after layer run `run`
    size_t weight_bytes() const override { return weight_bytes_; }
    int kernels_last_forward() const override { return kernels_last_; }
    const kb_config &config() const { return cfg_; }

  private:
    kibilix_model() {}
    int load(const safetensors_file *file, uint64_t seed);
    int load_hyper(weight_source &src, const std::string &name, kb_hyper_w *w);
    int alloc_scratch();
    int emit(int T, const int32_t *table_dev, float *state, int n_want);
    int upload_matrix(const std::vector<float> &host, void **dev);
    int upload_f32(const std::vector<float> &host, float **dev);
    int fail(int rc, const std::string &what);

    kb_config cfg_;
    int S_ = 1; // streams the kernels see (a plain residual is one stream)
    int dt_ = GGB_TYPE_BF16;
    int max_T_ = 1024;
    std::string err_;
    std::vector<kb_layer_w> lw_;
    std::vector<kb_run> runs_;
    void *embed_ = nullptr, *bigram_ = nullptr, *head_ = nullptr;
    float *final_norm_ = nullptr, *ones_ = nullptr;
    size_t weight_bytes_ = 0;
    int64_t state_elems_ = 0, lookback_ = 0;
    std::vector<void *> owned_;
    paged_cache *cache_ = nullptr;
    int64_t max_pos_ = 0;
    std::map<std::string, float *> rot_tables_;
    int32_t *ids_ = nullptr, *pos0_ = nullptr, *want_ = nullptr, *route_i_ = nullptr, *group_ws_ = nullptr;
    float *x0_ = nullptr, *xs_ = nullptr, *pr_ = nullptr, *cv_ = nullptr, *qr_ = nullptr, *da_ = nullptr, *dg_ = nullptr, *ro_ = nullptr,
          *ya_ = nullptr, *yb_ = nullptr, *gu_ = nullptr, *y2_ = nullptr, *route_z_ = nullptr, *route_w_ = nullptr, *logits_ = nullptr,
          *cap_ = nullptr, *wa_ = nullptr;
    void *h_ = nullptr, *ao_ = nullptr, *lr_ = nullptr, *gd_ = nullptr, *act_ = nullptr, *hw_ = nullptr;
    bool capture_ = false, use_graphs_ = true;
    int cap_T_ = 0, kernels_last_ = 0;
    struct step_graph {
        const int32_t *table;
        const float *state;
        int n_want;
        ggb_graph *graph;
    };
    std::vector<step_graph> graphs_;
};
