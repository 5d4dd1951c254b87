// ditalorn_model.h — the Ditalorn decoder: token embedding times a constant plus a learned position row; layers with a
// norm on both sides of every sublayer (x += norm1b(mixer(norm1 x)), x += norm2b(ff(norm2 x)), RMS norms whose weight is
// stored around zero); two kinds of mixer in any order the configuration lists:
//   "attention"        — grouped heads, biased q / k / v projections, a short causal convolution over time on every
//                        channel of them, a query temperature that grows with the position, values divided by their root
//                        mean square, and unnormalised weights sigmoid(q.k scale - r1 ln(1 + r2 (i - j)) + pb) over
//                        every earlier position;
//   "latent_attention" — queries and keys / values through normed latents, only the key / value latent cached, soft-max
//                        over a sliding window, no positions, a sigmoid gate per head on the output;
// a mixture of experts (sigmoid scores, a choice correction, groups of experts of which the best stay, SiLU-gated
// experts, weights not renormalised) or no feed-forward; logits against the embedding table itself.  Every size and
// constant comes from config.json or a tensor's shape.
//
// What a sequence carries: one row per position and caching layer in the engine's paged cache ([k | unit v] of an
// attention layer, the latent of a latent layer), and one block of fp32 state: the last taps - 1 biased projections of
// every attention layer's convolutions.
//
// The class lowers a portion of tokens to ggb_op_* operators, as safolorn_model and begupel_model do; positions, page
// tables and state are read on the device, so the one-token step is captured into a CUDA graph and replayed.
#pragma once

#include <string>
#include <vector>

#include "ggml_b200.h"
#include "lm_model.h"
#include "safetensors.h"

struct dl_attn_cfg { // "attention"
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
    int conv = 0;          // taps; 0: no convolution
    int temp_every = 0;    // 0: no query temperature
    float temp_coef = 0.f, scale = 1.f;
};

struct dl_latent_cfg { // "latent_attention"
    int heads = 0, dim = 0, vdim = 0, kv_rank = 0, q_rank = 0;
    int64_t window = 0; // 0: every earlier position
    float scale = 1.f;
};

struct dl_moe_cfg {
    int experts = 0, top = 0, groups = 1, keep = 1, ff = 0; // experts == 0: the layer has no feed-forward
};

struct dl_layer_cfg {
    int type = 0; // 0 attention, 1 latent_attention
    dl_attn_cfg attn;
    dl_latent_cfg latent;
    dl_moe_cfg moe;
};

struct dl_config {
    int vocab = 0, width = 0;
    int64_t max_positions = 0;
    float eps = 1e-5f, embed_scale = 1.f;
    std::vector<dl_layer_cfg> layers;
};
// fills *c from a parsed config.json; sizes the configuration leaves out are taken from the tensors' shapes when a file
// is given; 0 or -1 with *err
int dl_parse_config(const json_value &j, const safetensors_file *file, dl_config *c, std::string *err);

struct dl_layer_w {
    float *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr; // as they multiply: 1 + stored
    void *proj = nullptr; // every matrix that reads the mixer's input, stacked (rows padded to a multiple of 32)
    int64_t n_proj = 0;
    void *o = nullptr;
    // attention
    float *proj_b = nullptr, *conv = nullptr, *r1 = nullptr, *r2 = nullptr, *pb = nullptr, *o_b = nullptr;
    int64_t s_tail = 0; // offset of the convolutions' tail in the sequence's state block
    // latent attention
    float *dq_norm = nullptr, *dkv_norm = nullptr;
    void *uq = nullptr, *uk = nullptr, *uv = nullptr;
    void *ukv = nullptr; // [W_uk; W_uv] stacked: keys and values of every head in one product (portions, materialised form)
    int cache_index = -1;
    // experts: [E][2 ff][W] (gate rows, then up rows), [E][W][ff]
    void *e_gate_up = nullptr, *e_down = nullptr;
    float *router = nullptr, *correction = nullptr;
};

class ditalorn_model : public lm_model {
  public:
    static lm_model *create(const std::string &dir, const json_value &cfg, const lm_load_options &opt, std::string *err);
    ~ditalorn_model() override;

    const char *architecture() const override { return "Ditalorn"; }
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
    int get_capture(int layer, float *host, int64_t n) const override;
    size_t weight_bytes() const override { return weight_bytes_; }
    int kernels_last_forward() const override { return kernels_last_; }
    const dl_config &config() const { return cfg_; }

  private:
    ditalorn_model() {}
    int load(const safetensors_file *file, uint64_t seed);
    int alloc_scratch();
    int emit(int T, int64_t pos0, int n_split, const int32_t *table_dev, float *state, int n_want);
    bool materialise(const dl_latent_cfg &a, int T) const; // which form of the latent attention a portion of T tokens takes
    int upload_matrix(const std::vector<float> &host, void **dev);
    int upload_f32(const std::vector<float> &host, float **dev);
    int fail(int rc, const std::string &what);

    dl_config cfg_;
    int dt_ = GGB_TYPE_BF16;
    int max_T_ = 1024;
    std::string err_;
    std::vector<dl_layer_w> lw_;
    void *embed_ = nullptr, *pos_ = nullptr;
    float *final_norm_ = nullptr;
    size_t weight_bytes_ = 0;
    int64_t state_elems_ = 0, lookback_ = 0;
    std::vector<void *> owned_;
    paged_cache *cache_ = nullptr;
    int64_t max_pos_ = 0;
    int32_t *ids_ = nullptr, *pos0_ = nullptr, *want_ = nullptr, *iota_ = nullptr, *route_i_ = nullptr, *group_ws_ = nullptr;
    float *x_ = nullptr, *pr_ = nullptr, *cv_ = nullptr, *q_ = nullptr, *qa_ = nullptr, *part_ = nullptr, *sa_ = nullptr, *ya_ = nullptr,
          *gu_ = nullptr, *y2_ = nullptr, *route_w_ = nullptr, *route_z_ = nullptr, *xw_ = nullptr, *logits_ = nullptr, *cap_ = nullptr;
    void *h_ = nullptr, *cq_ = nullptr, *ao_ = nullptr, *act_ = nullptr, *hw_ = nullptr;
    // the materialised form: gathered latents, keys | values of the visible range (fp32 scratch, then the storage type),
    // an identity page table, the portion's position counted from the first visible one (per layer)
    void *crows_ = nullptr, *kv_ = nullptr;
    float *kvf_ = nullptr;
    int32_t *page_iota_ = nullptr, *posrel_ = nullptr;
    int64_t kv_rows_ = 0;
    int64_t part_rows_ = 0;
    bool capture_ = false, use_graphs_ = true;
    int cap_T_ = 0, kernels_last_ = 0;
    struct step_graph {
        const int32_t *table;
        const float *state;
        int n_split, n_want;
        ggb_graph *graph;
    };
    std::vector<step_graph> graphs_;
};
