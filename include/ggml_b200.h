/*
 * ggml_b200.h — the C-ABI CUDA layer (libggb_cuda.so) that replaces the reference's OpenCL
 * offload: src/opencl.{h,cpp} (device runtime) and src/kernals.cl (kernels), and is what
 * the rewired src/hpc.cpp dispatch and the graph builder of src/gemma_model.cpp call.
 *
 * Plain C: pointers, sizes, ints.  No torch / C++ types.  Every entry returns GGB_OK (0) or a
 * negative ggb_status; ggb_last_error() gives the text (the reference exits the process on
 * error, src/opencl.cpp:13-17 — a library cannot, so failures are returned and are loud).
 * There is no CPU fallback anywhere below this header: with no CUDA device ggb_init fails.
 *
 * Unless stated otherwise "device pointer" arguments come from ggb_buffer_alloc and every
 * ggb_op_* call is ASYNCHRONOUS on the library's stream; ggb_sync() waits
 * (ref: wait_queue_finish, src/opencl.h:37).
 */
#ifndef GGML_B200_H
#define GGML_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    GGB_OK = 0,
    GGB_ERR_CUDA = -1,        /* a CUDA runtime call failed */
    GGB_ERR_ARG = -2,         /* bad argument / unsupported shape */
    GGB_ERR_NOT_INIT = -3,    /* ggb_init not called or failed */
    GGB_ERR_UNSUPPORTED = -4, /* tensor type without a kernel (ref: "kernel is null", src/hpc.cpp:162-166) */
    GGB_ERR_NCCL = -5
} ggb_status;

/* ggml_type values the path uses (upstream enum ids; ref: src/hpc.cpp:132-143) */
enum { GGB_TYPE_F32 = 0, GGB_TYPE_F16 = 1, GGB_TYPE_Q4_0 = 2, GGB_TYPE_Q8_0 = 8,
       GGB_TYPE_Q4_K = 12, GGB_TYPE_Q6_K = 14, GGB_TYPE_Q8_K = 15, GGB_TYPE_BF16 = 30 }; /* ggml_type ids */

/* Arithmetic: every result of the Q4_0 / Q8_0 decode path and of the K-quant operators is BIT-IDENTICAL to the scalar
 * ggml code the reference's CPU path runs (one fp32 accumulator per row, blocks in order; double accumulators where
 * ggml has them) - there is no kernel-specific summation order.  The constants below are tiling
 * parameters only: blocks per K segment of the decode kernel's pass stream, threads of the rms_norm partial sums
 * (double: insensitive to their grouping at fp32 precision), positions per attention item. */
#define GGB_DEV_SEG_BLOCKS 64
#define GGB_DEV_NORM_THREADS 256
#define GGB_DEV_ATTN_CHUNK 32

/* ------------------------------------------------------------------ runtime
 * replaces: init_opencl / set_platform_and_device / setup_opencl_env / build_all_kernels
 * (src/opencl.h:22-30, src/opencl.cpp:161-245, 350-356), print_now_using (:100),
 * wait_queue_finish (:309), release_opencl_env (:247). */
int ggb_init(int device);
int ggb_shutdown(void);
const char *ggb_last_error(void);
int ggb_device_info(char *buf, size_t buflen); /* name, SMs, memory, compute capability */
int ggb_sm_count(void);
int ggb_sync(void);
void *ggb_stream(void); /* the cudaStream_t all ops are enqueued on */
int64_t ggb_launch_count(void); /* kernels launched (or replayed via graphs) since init */

/* replaces: create_buffer / release_buffer_in_set (src/opencl.h:35,38; src/opencl.cpp:313-348).
 * Buffers are device-resident and live until freed (the reference re-wraps host memory per
 * mul_mat call, src/hpc.cpp:168-170,196 — only viable on a zero-copy iGPU). */
int ggb_buffer_alloc(size_t bytes, void **dptr);
int ggb_buffer_free(void *dptr);
int ggb_buffer_memset(void *dptr, int value, size_t bytes);
int ggb_upload(void *dst_dev, const void *src_host, size_t bytes);   /* async if src is pinned */
int ggb_download(void *dst_host, const void *src_dev, size_t bytes); /* synchronous */
int ggb_host_alloc(size_t bytes, void **hptr); /* pinned host memory */
int ggb_host_free(void *hptr);

/* replaces the profiling probes (src/profiling.h:10-57: _start_recording/_stop_recording/
 * _print_profiling_result) with cudaEvent pairs keyed by the same kind of name strings. */
int ggb_prof_enable(int on);
int ggb_prof_start(const char *name);
int ggb_prof_stop(const char *name);
int ggb_prof_reset(void);
/* total ms and call count accumulated under `name` (resolves pending events; syncs) */
int ggb_prof_get(const char *name, double *total_ms, int64_t *calls);
int ggb_prof_report(char *buf, size_t buflen);

/* CUDA-graph capture of a sequence of ggb_op_* calls (one decode step) */
typedef struct ggb_graph ggb_graph;
int ggb_capture_begin(void);
int ggb_capture_end(ggb_graph **out);
int ggb_graph_launch(ggb_graph *g);
int ggb_graph_free(ggb_graph *g);
int ggb_graph_kernel_count(const ggb_graph *g);

/* ------------------------------------------------------------------ weights
 * A quantised matrix [rows][cols] uploaded ONCE and repacked to the device layout
 * (SoA: one plane of 16 B (Q4_0) / 32 B (Q8_0) quant payloads, one plane of fp16 scales). */
typedef struct ggb_weight ggb_weight;
int ggb_weight_upload(int type, int64_t rows, int64_t cols, const void *host_blocks, int64_t nb01,
                      ggb_weight **out);
/* synthetic matrix generated and quantised on the device (SURVEY.md §8d generator):
 * value(row, col) = synth(seed, tensor_id, row*cols + col) * sigma; bit-identical to the oracle's. */
int ggb_weight_synth(int type, int64_t rows, int64_t cols, uint64_t seed, uint64_t tensor_id, float sigma,
                     ggb_weight **out);
/* rows [row0, row0+nrows) of an existing weight as a new handle (no copy) — TP row shards */
int ggb_weight_slice(const ggb_weight *w, int64_t row0, int64_t nrows, ggb_weight **out);
int ggb_weight_download(const ggb_weight *w, void *host_blocks); /* back to ggml AoS blocks */
int ggb_weight_free(ggb_weight *w);
int64_t ggb_weight_rows(const ggb_weight *w);
int64_t ggb_weight_cols(const ggb_weight *w);
int ggb_weight_type(const ggb_weight *w);
size_t ggb_weight_algorithmic_bytes(const ggb_weight *w); /* rows * cols/32 * (18|34) */
/* f32 vector filled with bias + synth()*sigma (norm weights) */
int ggb_vector_synth(float *dst_dev, int64_t n, uint64_t seed, uint64_t tensor_id, float sigma, float bias);

/* ------------------------------------------------------------------ drop-in mul_mat
 * replaces: extern "C" void mul_mat(...) (src/hpc.h:22-32, src/hpc.cpp:216-277) — same
 * fields, HOST pointers, synchronous: on return all of dst is written.  src0_data/dst_data
 * are src0->data / dst->data of the ggml tensors; vec_dot is gone (the kernel is chosen by
 * src0_type).  wdata = src1 already converted by ggml's INIT stage to rows of `row_size` bytes in the
 * type's vec_dot_type: Q8_0 for Q4_0 / Q8_0 weights, Q8_K for Q4_K / Q6_K (the types the reference's
 * own kernels cover, src/hpc.cpp:132-143), F16 for F16.  Any other src0_type returns
 * GGB_ERR_UNSUPPORTED (the host mirror host/hpc.cpp then runs the caller's vec_dot, as the reference's
 * CPU share does).  src0 is uploaded (Q4_0 / Q8_0: repacked) on first use and cached by
 * (pointer, shape); call ggb_mul_mat_forget(ptr) if the host copy changes. */
int ggb_mul_mat(int64_t ne01, int64_t ne11, int64_t ne12, int64_t nb01, int64_t ne1, int64_t nb1, int64_t nb2,
                size_t row_size, int64_t shared_edge, const void *src0_data, void *dst_data, int src0_type,
                const char *wdata);
int ggb_mul_mat_forget(const void *src0_data);

/* ------------------------------------------------------------------ device operators
 * One entry per graph node kind the builder emits (ref: src/gemma_model.cpp:438-530, 665-747),
 * plus the fused forms the decode step uses.  All pointers are device pointers. */

/* planar Q8_0 activations: per row `cols` int8 followed by cols/32 fp16 scales */
size_t ggb_q8_row_bytes(int64_t cols);
/* K1 — quantize_row_q8_0 (ggml mul_mat INIT stage): T rows of `cols` floats -> planar Q8_0 */
int ggb_op_quantize_q8_0(const float *x, int64_t cols, int64_t T, void *q8);
int ggb_op_q8_to_blocks(const void *q8, int64_t cols, int64_t T, void *blocks);   /* planar -> ggml AoS (34 B) */
int ggb_op_q8_from_blocks(const void *blocks, int64_t cols, int64_t T, int64_t row_size, void *q8);

/* K-quants.  Blocks stay in ggml's AoS layout on the device.
 * ggb_type_row_bytes: bytes of one row of `cols` elements in `type` (0 for an unknown type).
 * ggb_op_quantize_q8_K: [UPSTREAM] quantize_row_q8_K (block: src/kernals.cl:29-34), rows x cols floats ->
 *   rows x cols/256 block_q8_K (292 B), bit-exact.
 * ggb_op_mul_mat_blocks: dst[t][row] = vec_dot(w row, act row t) for type Q4_K / Q6_K (act = Q8_K rows) or F16
 *   (act = fp16 rows); replaces matrix_multiply_q4_K / _q6_K / _f16 (src/kernals.cl:166-265) - which only
 *   compared against the CPU result - with kernels that produce it, in the scalar code's summation order. */
size_t ggb_type_row_bytes(int type, int64_t cols);
int ggb_op_quantize_q8_K(const float *x, int64_t cols, int64_t rows, void *out);
int ggb_op_mul_mat_blocks(int type, const void *w, int64_t rows, int64_t nb01, int64_t K, const void *act,
                          int64_t row_size, int64_t T, float *dst, int64_t dst_stride);
/* Q4_K weights that stay on the device: ggb_op_q4k_repack re-lays a matrix out once (same 144 B per super-block, the
 * nibbles that share a lane-sum index adjacent), ggb_op_mul_mat_q4k_packed is the mat-vec on that layout (same bits as
 * ggb_op_mul_mat_blocks / src/kernals.cl:48-111, ~4x its throughput).  ggb_mul_mat uses it for its cached src0. */
int ggb_op_q4k_repack(const void *raw, int64_t rows, int64_t nb01, int64_t K, void *packed);
int ggb_op_mul_mat_q4k_packed(const void *packed, int64_t rows, int64_t K, const void *act, int64_t row_size, int64_t T,
                              float *dst, int64_t dst_stride);
/* the same for Q6_K: codes expanded to int8 (q - 32) in the transposed arrangement; ggb_q6k_packed_bytes = size of the
 * packed matrix (274 B per super-block, rows padded to 16 B) */
/* the packed mat-vecs on an fp32 activation row x[t][K]: the kernel quantises the row to Q8_K itself while it stages it
 * (ggml's INIT stage of the mul_mat node fused into the COMPUTE stage; same bits as quantize + packed mat-vec) */
int ggb_op_mul_mat_kq_packed_f32(int type, const void *packed, int64_t rows, int64_t K, const float *x, int64_t T, float *dst,
                                 int64_t dst_stride);
/* get_rows on ggml's AoS K-quant blocks (embedding lookup): y[t] = dequantize_row(raw row ids[t]) * scale */
int ggb_op_get_rows_blocks(int type, const void *raw, int64_t n_rows, int64_t nb01, int64_t K, const int32_t *ids, int64_t T,
                           float scale, float *y);
size_t ggb_q6k_packed_bytes(int64_t rows, int64_t K);
int ggb_op_q6k_repack(const void *raw, int64_t rows, int64_t nb01, int64_t K, void *packed);
int ggb_op_mul_mat_q6k_packed(const void *packed, int64_t rows, int64_t K, const void *act, int64_t row_size, int64_t T,
                              float *dst, int64_t dst_stride);

/* K2/K3 — dst[t][row] = dot(w[row], q8[t]) (+ residual[t][row]); dst row pitch dst_stride floats */
int ggb_op_mul_mat_q8(const ggb_weight *w, const void *q8, int64_t T, float *dst, int64_t dst_stride,
                      const float *residual);
/* up to 3 weights sharing one activation row, one launch (Q/K/V) */
int ggb_op_mul_mat_q8_multi(int n, const ggb_weight *const *w, const void *q8, float *const *dst);
/* FFN front half: q8_out = quantize( gelu(gate·x) * (up·x) ); act_f32 optional (dump) */
int ggb_op_ffn_gate_up(const ggb_weight *gate, const ggb_weight *up, const void *q8, void *q8_out,
                       float *act_f32);

/* row-shard form (tensor parallel): this rank's rows write their int8 codes to out_qs and their fp16 block
 * scales to out_d — the caller passes pointers already offset into the gathered planar row */
int ggb_op_ffn_gate_up_shard(const ggb_weight *gate, const ggb_weight *up, const void *q8, void *out_qs, void *out_d,
                             float *act_f32);

/* K5 — rms_norm (+ weight mul when w != NULL) over T rows of E floats; y and/or q8 may be NULL */
int ggb_op_rms_norm(const float *x, const float *w, float eps, int64_t E, int64_t T, float *y, void *q8);
/* element-wise nodes */
int ggb_op_add(const float *a, const float *b, int64_t n, float *y);
int ggb_op_mul(const float *a, const float *b, int64_t n, float *y);
int ggb_op_scale(const float *x, float s, int64_t n, float *y);
int ggb_op_gelu(const float *x, int64_t n, float *y);
/* soft_max_ext(x*scale + mask), max_bias 0 (standalone node, REF semantics except the
 * double sum is a 256-way strided reduction); rows of nc floats; mask may be NULL */
int ggb_op_soft_max_ext(const float *x, const float *mask, float scale, int64_t nc, int64_t nrows, float *y);
/* K6 — rope NEOX on [n_heads][n_dims] rows for T tokens with positions pos[T] (device int32) */
int ggb_op_rope_neox(const float *x, const int32_t *pos, int n_dims, int n_heads, int64_t T, float *y);
/* K8 — get_rows(token_embd, ids) * scale */
int ggb_op_get_rows(const ggb_weight *table, const int32_t *ids, int64_t T, float scale, float *y);
/* K9 — first maximum (strict >); result index written to *out (device int32) */
int ggb_op_argmax(const float *x, int64_t n, int32_t *out);
int ggb_op_cpy_f32_f16(const float *x, int64_t n, void *y_f16);

/* rope tables (host libm recurrence, uploaded once); must be called before rope / decode ops */
int ggb_rope_table_init(int n_ctx, int n_dims, float freq_base);

/* K6 fused: q <- rope(q)*q_scale in place; kcache[pos] <- f16(rope(k)); vcache[pos] <- f16(v).
 * caches are position-major fp16 [n_ctx][Hkv*d]; *pos is a device int32 */
int ggb_op_rope_kv_store(float *q, const float *k, const float *v, const int32_t *pos, int H, int Hkv, int d,
                         float q_scale, void *kcache, void *vcache);
/* the same for T tokens (prefill): q [T][H*d], k / v [T][Hkv*d], pos[T] (device int32); one launch instead of
 * rope(q), scale(q), rope(k) and the two F32->F16 copies */
int ggb_op_rope_kv_store_batch(float *q, const float *k, const float *v, const int32_t *pos, int64_t T, int H, int Hkv,
                               int d, float q_scale, void *kcache, void *vcache);
/* K4 — split-K decode attention over positions [0, *pos]; scratch from ggb_attn_scratch_bytes.
 * out f32 [H*d] and/or q8 (planar, cols = H*d) */
size_t ggb_attn_scratch_bytes(int H, int d, int n_ctx);
int ggb_op_attn_decode(const float *q, const void *kcache, const void *vcache, const int32_t *pos, int H, int Hkv,
                       int d, int n_ctx, void *scratch, float *out, void *q8_out);

/* decode-step glue kept on the device so a captured step can be replayed:
 * state[0] = current token id, state[1] = its position, state[2] = position increment per step
 * (1 for generation; 0 pins n_kv for fixed-context bandwidth measurements) */
int ggb_op_embed_token(const ggb_weight *table, const int32_t *state, float scale, float *y);
/* state[0] <- argmax(logits), state[1] += state[2], history[state[1]] <- token (history may be NULL) */
int ggb_op_sample_greedy(const float *logits, int64_t n, int32_t *state, int32_t *history, void *scratch);
size_t ggb_sample_scratch_bytes(int64_t n);
/* tensor-parallel greedy sampling: each rank publishes (fp32 value, int32 global index) of the first maximum of
 * its logits shard (8 bytes), the candidates are allgathered, then the first maximum over ranks is taken */
int ggb_op_argmax_shard(const float *x, int64_t n, int32_t index_offset, void *cand_out, void *scratch);
int ggb_op_sample_from_candidates(const void *cands, int n_cands, int32_t *state, int32_t *history);

/* ------------------------------------------------------------------ prefill (mul_mat with col_num = T > 1)
 * K10 — C[T][N] = A[T][K] (bf16) x dequant(W[N][K])^T (+ residual): dequant -> bf16 tcgen05 GEMM with TMEM
 * accumulators (csrc/prefill.cu).  replaces: mul_mat with ne11 = T (src/hpc.cpp:216-277) for the graph nodes
 * at src/gemma_model.cpp:692-696, 493, 446-450, 740.  K %% 64 == 0, N %% 32 == 0; workspace (optional,
 * ggb_gemm_workspace_bytes) enables the K-split used for small N. */
size_t ggb_gemm_workspace_bytes(int64_t T, int64_t N, int64_t K);
int ggb_op_gemm_bf16(const ggb_weight *w, const void *a_bf16, int64_t T, float *c, int64_t ldc, const float *resid,
                     void *workspace, size_t workspace_bytes);
/* the same for up to 3 matrices that share the A operand (Q | K | V of src/gemma_model.cpp:692-696, gate | up of
 * :446-447) in ONE launch: c[i] / ldc[i] are the outputs of w[i].  workspace: ggb_gemm_workspace_bytes(T, sum of the
 * row counts rounded up to 256 each, K). */
int ggb_op_gemm_bf16_multi(int n, const ggb_weight *const *w, const void *a_bf16, int64_t T, float *const *c,
                           const int64_t *ldc, void *workspace, size_t workspace_bytes);
int ggb_op_cvt_f32_bf16(const float *x, int64_t n, void *y_bf16);
/* fused producers of the GEMM's bf16 A operand: rms_norm(x) * w, and gelu(gate) * up (graph_build_norm /
 * graph_build_ffn, src/gemma_model.cpp:438-452) */
int ggb_op_rms_norm_bf16(const float *x, const float *w, float eps, int64_t E, int64_t T, void *y_bf16);
int ggb_op_geglu_bf16(const float *gate, const float *up, int64_t n, void *y_bf16);
/* causal attention of T query tokens at positions pos0..pos0+T-1 over the fp16 KV cache (q already roped and
 * scaled, fp32 [T][H*d]); reference node order kq -> soft_max_ext -> kqv (src/gemma_model.cpp:454-489) */
/* out (fp32) and / or out_bf16 (the o-projection's A operand, same rounding as ggb_op_cvt_f32_bf16) may be NULL */
int ggb_op_attn_prefill(const float *q, const void *kcache, const void *vcache, int64_t T, int pos0, int H, int Hkv, int d,
                        float *out, void *out_bf16);

/* ------------------------------------------------------------------ plain bf16 / fp32 matrices (csrc/dense.cu)
 * Operators of models whose matrices are stored unquantised, row-major [out][in] and applied as W x.  `dt` is
 * GGB_TYPE_BF16 (matrices and the activations that feed them are bf16, products accumulate in fp32) or GGB_TYPE_F32
 * (true fp32 everywhere, no reduced-precision matrix mode).  The residual stream, norms, soft-max and every other
 * reduction are fp32 in both.  Pointers typed void* are in `dt`. */
size_t ggb_dtype_size(int dt);
/* c[t][n] (fp32) = sum_k a[t][k] w[n][k]: a streaming mat-vec for T <= 8, the tcgen05 GEMM for aligned bf16 shapes
 * (K %% 64 == 0, N %% 32 == 0, lda == K, T >= 64), a shared-memory tile kernel for every other shape */
int ggb_op_linear(int dt, const void *w, int64_t N, int64_t K, const void *a, int64_t lda, int64_t T, float *c, int64_t ldc);
/* y = x / sqrt(mean(x^2) + eps) * w for up to two weights of the same rows (the root mean square is computed once);
 * w_stride 0: the weight is one number, 1: a vector of E; y1 / y2 ([T][E] in dt) may be NULL */
int ggb_op_rms_norm2(int dt, const float *x, int64_t ldx, const float *w1, int w1_stride, const float *w2, int w2_stride, float eps,
                     int64_t E, int64_t T, void *y1, void *y2);
int ggb_op_gather_rows_f32(const float *x, const int32_t *rows, int64_t n_rows, int64_t E, float *y);
int ggb_op_embed_rows(int dt, const void *table, const int32_t *ids, int64_t T, int64_t E, float *y);
/* gu rows = [gate F | up F]: g = min(gate, limit), u = clamp(up, -limit, limit), y = g * sigmoid(alpha g) * (u + 1) */
int ggb_op_glu_clamp(int dt, const float *gu, int64_t F, int64_t T, float limit, float alpha, void *y);
/* x <- x + a (+ f, may be NULL); with sd > 0 then the per-token side input: e = side_embed[ids[t]][e_off .. e_off + sd),
 * y = w_proj (gelu_tanh(w_gate x) * e), x <- x + y / sqrt(mean(y^2) + eps) * nw */
int ggb_op_residual_side(int dt, float *x, const float *a, const float *f, int64_t W, int64_t T, const int32_t *ids, const void *side_embed,
                         int64_t e_ld, int64_t e_off, int sd, const void *w_gate, const void *w_proj, const float *nw, float eps);
int ggb_op_cvt_bf16_f32(const void *x_bf16, int64_t n, float *y);

/* token embedding with a hashed bigram table: y[t] = table[ids[t]] + bigram[row_t], row_t = (prev_t * mul_prev +
 * ids[t] * mul_cur) mod buckets with prev_t = ids[t - 1] and, for t = 0, the sequence's carried *prev_state; the first
 * token of a sequence (*pos0 + t == 0) takes row `buckets` (the table has buckets + 1 rows).  *prev_state <- ids[T - 1]. */
int ggb_op_embed_bigram(int dt, const void *table, const void *bigram, const int32_t *ids, int64_t T, int64_t E, int64_t buckets,
                        int64_t mul_prev, int64_t mul_cur, const int32_t *pos0, int32_t *prev_state, float *y);
/* v = sa a (+ sb b) (+ bias); n = v cut into `groups` equal consecutive parts, each divided by its own
 * sqrt(mean(part^2) + eps), times w.  With x (fp32): x += n and y (dt, may be NULL) = the new x; without x: y = n. */
int ggb_op_group_norm_add(int dt, const float *a, float sa, const float *b, float sb, const float *bias, const float *w, int groups,
                          float eps, int64_t E, int64_t T, float *x, void *y);
/* gu rows = [gate F | up F] (fp32): y = act(gate + bg) * (up + bu); biases may be NULL; act 0: relu, 1: silu, 2: gelu_tanh */
int ggb_op_glu_bias(int dt, const float *gu, int64_t F, int64_t T, const float *bg, const float *bu, int act, void *y);
/* x <- cap * tanh(x / cap) */
int ggb_op_softcap(float *x, int64_t n, float cap);
/* o rows = [n_groups][gs] fp32 (row stride ldo): y = o / sqrt(mean over the group (o^2) + eps) * w[i %% w_period] *
 * act(gate) with gate fp32 rows of stride ldg; act 0: sigmoid, 1: silu; y in dt, dense [T][n_groups * gs] */
int ggb_op_norm_gate(int dt, const float *o, int64_t ldo, const float *gate, int64_t ldg, int64_t T, int n_groups, int gs, const float *w,
                     int w_period, float eps, int act, void *y);
/* token embedding with learned positions: y[t] = table[ids[t]] * scale + pos_table[*pos0 + t] (pos_table may be NULL);
 * with yn also the first layer's norm in the same pass: yn (dt) = y / sqrt(mean(y^2) + eps) * wn */
int ggb_op_embed_pos(int dt, const void *table, const void *pos_table, const int32_t *ids, const int32_t *pos0, int64_t T, int64_t E,
                     float scale, float *y, const float *wn, float eps, void *yn);
/* norms on both sides of a sublayer in one pass over the row: v = a (+ bias); x += v / sqrt(mean(v^2) + eps) * wa; then,
 * with y, y (dt) = x / sqrt(mean(x^2) + eps) * wy: the input of the next sublayer.  Weights as they multiply (a weight
 * stored around zero is handed in as 1 + w). */
int ggb_op_norm_add_norm(int dt, const float *a, const float *bias, const float *wa, float eps, int64_t E, int64_t T, float *x,
                         const float *wy, void *y);

/* Several residual streams (hyper-connections): xs [T][S][W] fp32 holds S copies of the residual per token.  One pass:
 * with x0 ([T][W]) every stream starts as that row; with y ([T][W], a sublayer's output) all streams are renewed at once from
 * the old ones, x_t <- sum_s mix[s * S + t] x_s + coef[t] y; with in_w the sum u = sum_s in_w[s] x_s is read out as fp32
 * (u_out, may be NULL) and / or normed in dt (h = u / sqrt(mean(u^2) + eps) * nw, may be NULL).  rows (device int32, may be
 * NULL): only the tokens rows[0 .. T) are read out (outputs dense in that order) and xs is left as it was: what y brings
 * enters on the way.  One stream with mix = in_w = {1} is the plain residual sum. */
int ggb_op_hyper_mix(int dt, float *xs, const float *x0, const float *y, const float *mix, const float *coef, int S, const float *in_w,
                     const float *nw, float eps, int64_t W, int64_t T, const int32_t *rows, float *u_out, void *h);
/* the same where the sublayer was a mixture of experts whose weighted sum has not been taken yet: y[t] = sum_k wt[t][k] *
 * (row of slot k in y2, or the token's row of h_in (dt, what the experts read) where idx[t][k] is an identity expert); ws, wt,
 * idx, n_exp, n_identity as for ggb_op_moe_combine_identity, T_slots the number of tokens the slot lists were made for (with
 * rows, T counts the rows read out).  h_in may be the buffer h is written to.  At most 64 slots a token. */
int ggb_op_hyper_mix_moe(int dt, float *xs, const float *y2, const int32_t *ws, const float *wt, const int32_t *idx, int64_t T_slots, int top, int n_exp,
                         int n_identity, const void *h_in, const float *mix, const float *coef, int S, const float *in_w, const float *nw, float eps,
                         int64_t W, int64_t T, const int32_t *rows, float *u_out, void *h);
/* y (dt, dense [T][N]) = relu(a w^T)^2: a feed-forward's first product with its activation.  One launch (the mat-vec or the
 * tile kernel with the activation as its epilogue) except for the shapes the tensor cores take, which go through scratch
 * (fp32 [T][N]; NULL: never) and ggb_op_act_rows */
int ggb_op_linear_relu2(int dt, const void *w, int64_t N, int64_t K, const void *a, int64_t lda, int64_t T, float *scratch, void *y);
/* y (dt, dense [T][F]) = act(x), x fp32 rows of stride ldx; act 0: as it is, 1: relu(x)^2 */
int ggb_op_act_rows(int dt, const float *x, int64_t ldx, int64_t T, int64_t F, int act, void *y);

/* ------------------------------------------------------------------ recurrent mixers (csrc/recurrent.cu)
 * State that a sequence carries from token to token (fp32, one block per sequence, handed in by the caller): tails of
 * causal convolutions and the matrices S [heads][D][Dv] of linear-attention recurrences.
 *
 * causal convolution over time on each channel: with xx = tail (the taps - 1 inputs before this portion; zeros at a
 * sequence's start) followed by x, y[t][c] = (add_input ? x[t][c] : 0) + sum_j w[c][j] xx[t + j][c] (the last tap weighs
 * the current token); act 1: y = silu(y).  y is fp32 (y_f32, row stride ldy) and / or dt (y_dt, dense [T][C]).  tail
 * [(taps - 1)][C] is replaced by the last taps - 1 inputs.  taps <= 8. */
int ggb_op_causal_conv(int dt, const float *x, int64_t ldx, int64_t T, int64_t C, const float *w, int taps, int add_input, int act,
                       float *tail, float *y_f32, int64_t ldy, void *y_dt);
/* the same on the input x + bias[c] (a projection's bias added on the way in; the tail keeps the biased values; bias may be NULL) */
int ggb_op_causal_conv_bias(int dt, const float *x, int64_t ldx, int64_t T, int64_t C, const float *w, const float *bias, int taps,
                            int add_input, int act, float *tail, float *y_f32, int64_t ldy, void *y_dt);
/* lightning attention: q, k [T][H * D], v [T][H * Dv] raw projections (row stride ld); per head with q = silu(q),
 * k = silu(k), v = silu(v): S <- decay[h] S + k v^T, o = S^T q.  state [H][D][Dv] in / out, o fp32 [T][H * Dv]. */
int ggb_op_lightning_attn(const float *q, const float *k, const float *v, int64_t ld, int64_t T, int H, int D, int Dv, const float *decay,
                          float *state, float *o, int64_t ldo);
/* gated delta rule: q, k [T][G * D] and v [T][H * Dv] (after their convolutions and activations; row stride ld), b, a
 * [T][H] raw projections (row stride ld_ba); head h uses q / k head h / (H / G).  qn = q / sqrt(sum q^2 + 1e-6) * D^(-1/2),
 * kn = k / sqrt(sum k^2 + 1e-6), beta = sigmoid(b), g = exp(-exp(A_log[h]) softplus(a + dt_bias[h]));
 * S <- g S; u = beta (v - S^T kn); S <- S + kn u^T; o = S^T qn.  state [H][D][Dv] in / out, o fp32 [T][H * Dv]. */
int ggb_op_gated_delta(const float *q, const float *k, const float *v, int64_t ld, const float *b, const float *a, int64_t ld_ba, int64_t T,
                       int H, int G, int D, int Dv, const float *A_log, const float *dt_bias, float *state, float *o, int64_t ldo);

/* the gated delta rule with one decay per head and key channel: a [T][H * D] raw rows (row stride ld_a), dt_bias [H * D],
 * b [T][H] (row stride ld_b); g[h][d] = exp(-exp(A_log[h]) softplus(a[h][d] + dt_bias[h][d])) multiplies row d of the head's
 * S [D][Dv] before the token's write; everything else as ggb_op_gated_delta */
int ggb_op_channel_delta(const float *q, const float *k, const float *v, int64_t ld, const float *b, int64_t ld_b, const float *a, int64_t ld_a,
                         int decays, int64_t T, int H, int G, int D, int Dv, const float *A_log, const float *dt_bias, float *state, float *o,
                         int64_t ldo);
/* decays 1 above: `a` already holds g (A_log and dt_bias unused), e.g. from the operator below.
 * The second halves of two low-rank projections in one launch: x rows = [a1 (Ka) | g1 (Kg)] fp32 (row stride ldx), rounded
 * to dt on the way in; a[t][n] = w_a[n] . a1[t] (Na outputs, w_a [Na][Ka] in dt) and g[t][n] = w_g[n] . g1[t] (Ng outputs), fp32,
 * dense.  With A_log (then dt_bias [Na], heads of D outputs): a leaves as exp(-exp(A_log[n / D]) softplus(a + dt_bias[n])), the
 * decays of ggb_op_channel_delta.  ggb_lowrank_pair_fits: 0 when the inner sizes are too large for the kernel's shared memory
 * (callers then use ggb_op_act_rows and ggb_op_linear). */
int ggb_lowrank_pair_fits(int dt, int Ka, int Kg);
int ggb_op_lowrank_pair(int dt, const float *x, int64_t ldx, int64_t T, const void *w_a, int64_t Na, int Ka, const void *w_g, int64_t Ng, int Kg,
                        const float *A_log, const float *dt_bias, int D, float *a, float *g);

/* ------------------------------------------------------------------ sliding-window attention (csrc/window_attention.cu)
 * Grouped-query soft-max attention over a paged cache whose row per position is [k (G * D) | v (G * Dv)] in dt,
 * ggb_window_cache_ld numbers apart (pages as in the latent cache).  Values are stored rotated by their own position
 * (pairs (2m, 2m + 1) over all Dv, table cos_sin_v) and a head's output is turned back by the reader's position.
 * cos_sin tables: [positions][pairs][2] fp32.
 *
 * qkv_store: q [T][H * D], k [T][G * D], v [T][G * Dv] raw projections (row stride ld).  With qn_w / kn_w the whole q / k
 * row is divided by its root mean square and multiplied by that weight first.  Pairs (2i, 2i + 1), 2i < rot_dims, of every
 * head of q and k are turned by the position (cos_sin_k); q times scale -> q_out fp32 [T][H * D]; k and v (cos_sin_v may
 * be NULL: stored as they are) -> the cache row of position *pos0 + t. */
int64_t ggb_window_cache_ld(int G, int D, int Dv);
int ggb_op_window_qkv_store(int dt, const float *q, const float *k, const float *v, int64_t ld, int64_t T, int H, int G, int D, int Dv,
                            const float *qn_w, const float *kn_w, float eps, int rot_dims, const float *cos_sin_k, const float *cos_sin_v,
                            float scale, const int32_t *pos0, const int32_t *block_table, int block_size, void *cache, float *q_out);
/* token t at position i = *pos0 + t sees the keys j with 0 <= i - j < window (window <= 0: every j <= i); query head h
 * reads key / value head h / (H / G); out (dt) [T][H * Dv].  scratch (ggb_window_attn_scratch_bytes, may be NULL): lets
 * a step of few tokens spread a (token, head)'s keys over several CTAs */
size_t ggb_window_attn_scratch_bytes(int H);
int ggb_op_window_attn(int dt, const float *q, const void *cache, const int32_t *block_table, int block_size, const int32_t *pos0, int64_t T,
                       int H, int G, int D, int Dv, int64_t window, const float *cos_sin_v, void *out, float *scratch);

/* The same two operators with every choice an argument.  rot_halves 1: the rotated pair m < rot_dims / 2 of a head is
 * (m, m + rot_dims / 2) instead of (2m, 2m + 1) (the table's entry m turns it either way).  chunked 1: `window` is a chunk
 * size and the query at position i sees the keys j <= i with floor(j / window) == floor(i / window), chunks counted from
 * position 0 of the sequence.  softcap > 0: a score s enters the soft-max as softcap * tanh(s / softcap). */
int ggb_op_masked_qkv_store(int dt, const float *q, const float *k, const float *v, int64_t ld, int64_t T, int H, int G, int D, int Dv,
                            const float *qn_w, const float *kn_w, float eps, int rot_dims, int rot_halves, const float *cos_sin_k,
                            const float *cos_sin_v, float scale, const int32_t *pos0, const int32_t *block_table, int block_size, void *cache,
                            float *q_out);
int ggb_op_masked_attn(int dt, const float *q, const void *cache, const int32_t *block_table, int block_size, const int32_t *pos0, int64_t T,
                       int H, int G, int D, int Dv, int64_t window, int chunked, float softcap, const float *cos_sin_v, void *out,
                       float *scratch);

/* ------------------------------------------------------------------ sigmoid attention (csrc/sigmoid_attention.cu)
 * Grouped-query attention with unnormalised weights over the same paged rows [k (G * D) | v (G * Dv)] (ggb_window_cache_ld):
 * the weight of key j for the query at position i is sigmoid(q . k - r1[h] ln(1 + r2[h] (i - j)) + pb[h]), the output
 * the plain weighted sum of the values.
 *
 * qkv_store: q [T][H * D], k [T][G * D], v [T][G * Dv] fp32 (row stride ld).  q times its temperature
 * 1 + temp_coef ln(floor((p + 1) / temp_every) + 1) at position p (temp_every 0: none) times scale -> q_out fp32
 * [T][H * D]; k and every value head divided by its root mean square (vnorm_eps < 0: as it is) -> the cache row. */
int ggb_op_sigmoid_qkv_store(int dt, const float *q, const float *k, const float *v, int64_t ld, int64_t T, int H, int G, int D, int Dv,
                             float temp_coef, int temp_every, float vnorm_eps, float scale, const int32_t *pos0, const int32_t *block_table,
                             int block_size, void *cache, float *q_out);
/* token t at position i = *pos0 + t sees j <= i (window > 0: 0 <= i - j < window); r1 / r2 (both or neither) and pb are
 * per-head fp32 and may be NULL; out (dt) [T][H * Dv].  scratch (ggb_sigmoid_attn_scratch_bytes, may be NULL): lets a
 * step of few tokens spread a (token, head)'s keys over several CTAs */
size_t ggb_sigmoid_attn_scratch_bytes(int H);
int ggb_op_sigmoid_attn(int dt, const float *q, const void *cache, const int32_t *block_table, int block_size, const int32_t *pos0, int64_t T,
                        int H, int G, int D, int Dv, int64_t window, const float *r1, const float *r2, const float *pb, void *out,
                        float *scratch);

/* ------------------------------------------------------------------ latent attention (csrc/latent_attention.cu)
 * The cache of a layer holds one row [c (R) | kr (Dr)] per position, ggb_latent_cache_ld(R, Dr) numbers apart, in pages
 * of block_size positions: position j is row block_table[j / block_size] * block_size + j %% block_size.  The step's
 * tokens sit at positions *pos0 + t (pos0 and block_table are device int32: a captured step replays elsewhere).
 * cos_sin: [positions][rot_dims / 2][2] fp32, pairs (2i, 2i+1) of the first rot_dims rotated numbers are turned. */
int64_t ggb_latent_cache_ld(int R, int Dr);
/* d rows = [R latent | Dr key part] (fp32, the down-projection's output): cache row <- [rms(d[:R]) * norm_w | rot(d[R:])] */
int ggb_op_latent_kv_store(int dt, const float *d, int64_t ldd, int64_t T, int R, int Dr, int rot_dims, const float *norm_w, float eps,
                           const float *cos_sin, const int32_t *pos0, const int32_t *block_table, int block_size, void *cache);
/* q rows hold per head D unrotated then Dr rotated numbers; qa[t][h] = [w_uk_h^T q_unrot | rot(q_rot)] * scale, R + Dr fp32 */
int ggb_op_latent_q_absorb(int dt, const float *q, int64_t ldq, int64_t T, int H, int D, int Dr, int rot_dims, const float *cos_sin,
                           const int32_t *pos0, const void *w_uk, int R, float scale, float *qa);
/* causal soft-max attention of T tokens over the cache, the visible positions of a token cut into n_split parts:
 * part[t][split][h] = {running max, sum, sum_j p_j c_j (R)} */
size_t ggb_latent_attn_scratch_bytes(int64_t T, int H, int R, int n_split);
int ggb_op_latent_attn(int dt, const float *qa, const void *cache, const int32_t *block_table, int block_size, const int32_t *pos0,
                       int64_t T, int H, int R, int Dr, int n_split, float *part);
/* merges the parts with the per-head sink (one more exp(sink_h) in the denominator, no value) and applies w_uv:
 * out[t][h * Dv ..] (dt) = w_uv_h (sum_j p_j c_j) */
int ggb_op_latent_attn_out(int dt, const float *part, int n_split, const float *sink, const void *w_uv, int64_t T, int H, int R, int Dv,
                           void *out);
/* the same over a sliding window: the token at position i sees the keys j with 0 <= i - j < window (window <= 0: every
 * j <= i); the splits deal the tiles from the first visible one */
int ggb_op_latent_attn_window(int dt, const float *qa, const void *cache, const int32_t *block_table, int block_size, const int32_t *pos0,
                              int64_t T, int H, int R, int Dr, int64_t window, int n_split, float *part);
/* The materialised form, for portions whose window is short beside the latent: the latents of positions [first, first + n)
 * are gathered (c_rows, dt [n][R]) and multiplied by w_ukv = [W_uk; W_uv] ([N][R], N = H (D + Dv)): kv (dt, row pitch ld_kv)
 * holds rows [k (H D) | v (H Dv)], which ggb_op_window_attn reads as a cache of H key heads through an identity page table
 * and positions counted from `first`.  kv_f32 ([n][ld_kv] fp32) is scratch for the bf16 type. */
int ggb_op_latent_expand(int dt, const void *cache, const int32_t *block_table, int block_size, int64_t first, int64_t n, int R, int Dr,
                         const void *w_ukv, int64_t N, void *c_rows, float *kv_f32, void *kv, int64_t ld_kv);
/* x (dt, [T][H * Dv], in place): head h of token t times sigmoid(gate[t * ldg + h]) */
int ggb_op_head_gate(int dt, void *x, int64_t T, int H, int Dv, const float *gate, int64_t ldg);
/* the merge without a sink (sink NULL: ordinary soft-max over the keys) and / or with an output gate: head h of token t
 * is multiplied by sigmoid(gate[t * ldg + h]) (fp32 raw projections; gate NULL: none) */
int ggb_op_latent_attn_out_gated(int dt, const float *part, int n_split, const float *sink, const void *w_uv, int64_t T, int H, int R, int Dv,
                                 const float *gate, int64_t ldg, void *out);

/* ------------------------------------------------------------------ mixture of experts (csrc/moe.cu)
 * route: fp32 logits w_router h + bias, the `top` largest (ties: lower index), weights = soft-max over the chosen.
 * group: sorts the T * top slots by expert into `ws` (ggb_moe_group_ints int32).  moe_linear: per expert
 * c[sorted row] = a[row] w_e^T with w = [n_exp][N][K]; gather: a is indexed by token (first product), else by sorted
 * row; act 1: c = relu(.)^2 in dt, act 0: c fp32.  combine: out[t] = sum_s wt[t][s] y[sorted row of slot s]. */
int ggb_op_moe_route(int dt, const void *h, int64_t W, int64_t T, const float *w_router, const float *bias, int n_exp, int top,
                     float *logits /* scratch [T][n_exp] */, int32_t *idx, float *wt);
/* route with sigmoid scores: s = sigmoid(w_router h) in fp32; the choice score of an expert is s + correction (may be
 * NULL); the experts form n_groups equal groups of neighbours, a group's score is the sum of its two largest choice
 * scores, and only the `keep` best groups can be chosen from (ties: the lower index, for groups and experts); the `top`
 * largest choice scores win and the weights are their s, not renormalised */
int ggb_op_moe_route_sigmoid(int dt, const void *h, int64_t W, int64_t T, const float *w_router, const float *correction, int n_exp, int top,
                             int n_groups, int keep, float *logits /* scratch [T][n_exp] */, int32_t *idx, float *wt, int32_t *ws);
/* 1 when a step of n_slots = T * top slots takes the mat-vec form of the grouped products.  Then route_sigmoid, given ws
 * (ggb_moe_group_ints), also lists the slots there in the same launch and ggb_op_moe_group may be left out, and
 * moe_linear takes act 2: w = [n_exp][2 N][K] (N gate rows, then N up rows), c (dt) = silu(gate) * up. */
int ggb_moe_step_form(int64_t n_slots);
int ggb_moe_max_tiles(int64_t n_slots, int n_exp);
size_t ggb_moe_group_ints(int64_t n_slots, int n_exp);
int ggb_op_moe_group(const int32_t *idx, int64_t T, int top, int n_exp, int32_t *ws);
int ggb_op_moe_linear(int dt, const void *w, int64_t N, int64_t K, const void *a, int64_t lda, int gather, int64_t T, int top, int n_exp,
                      const int32_t *ws, int act, void *c, int64_t ldc);
int ggb_op_moe_combine(const float *y, const int32_t *ws, const float *wt, int64_t T, int top, int n_exp, int64_t W, float *out);
/* combine and the norms on both sides of the sublayer (ggb_op_norm_add_norm) in one pass: v = sum_s wt[t][s] y[slot s];
 * x += v / rms(v) * wa; out (dt, may be NULL) = x / rms(x) * wy */
#define GGB_MOE_COMBINE_NORM_MAX_TOP 64 /* more slots per token: ggb_op_moe_combine, then ggb_op_norm_add_norm */
int ggb_op_moe_combine_norm(int dt, const float *y, const int32_t *ws, const float *wt, int64_t T, int top, int n_exp, int64_t W, const float *wa,
                            float eps, float *x, const float *wy, void *out);

/* route with soft-max scores over ALL experts: s = softmax(w_router h) in fp32; the `top` largest s + correction (may be
 * NULL) win (ties: the lower index); the weights are the chosen experts' s divided by their sum (+ 1e-20).  ws as for
 * ggb_op_moe_route_sigmoid. */
int ggb_op_moe_route_softmax(int dt, const void *h, int64_t W, int64_t T, const float *w_router, const float *correction, int n_exp, int top,
                             float *logits /* scratch [T][n_exp] */, int32_t *idx, float *wt, int32_t *ws);
/* Identity experts: the last n_identity of the n_exp experts have no matrices and hand their input through.  Their slots
 * are grouped like the others but no product touches them (w holds n_exp - n_identity experts), and the weighted sum takes
 * the token's row of h (dt, [T][W]: what the experts read) in their place.  moe_linear act 3 (steps of at most 16 slots):
 * w = [experts][2 N][K] (N gate rows, then N up rows), c (dt) = g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit),
 * u = clamp(up, -limit, limit). */
int ggb_op_moe_group_identity(const int32_t *idx, int64_t T, int top, int n_exp, int n_identity, int32_t *ws);
int ggb_op_moe_linear_identity(int dt, const void *w, int64_t N, int64_t K, const void *a, int64_t lda, int gather, int64_t T, int top, int n_exp,
                               int n_identity, const int32_t *ws, int act, float limit, float alpha, void *c, int64_t ldc);
int ggb_op_moe_combine_identity(int dt, const float *y, const int32_t *ws, const float *wt, const int32_t *idx, int64_t T, int top, int n_exp,
                                int n_identity, int64_t W, const void *h, float *out);

/* ------------------------------------------------------------------ fused decode step
 * The whole per-token node list (ref: src/gemma_model.cpp:665-747) as ONE persistent cooperative
 * kernel: weights and KV stream through a shared-memory ring fed by TMA bulk copies (csrc/decoder.cu).
 * Bit-identical to the ggb_op_* sequence and to the scalar ggml order of the reference's CPU path. */
typedef struct {
    int32_t n_embd, n_layer, n_head, n_head_kv, head_dim, n_ff, n_vocab, n_ctx;
    float eps;
    int32_t pad_;
} ggb_decoder_dims;
typedef struct {
    const float *attn_norm, *ffn_norm;
    const ggb_weight *attn_q, *attn_k, *attn_v, *attn_output, *ffn_gate, *ffn_up, *ffn_down;
    void *k_cache, *v_cache; /* fp16, position-major [n_ctx][n_head_kv*head_dim] */
} ggb_decoder_layer;
typedef struct {
    int32_t *state;   /* [token, pos, pos_step] */
    int32_t *history; /* [n_ctx + 2] or NULL */
    float *sa_out, *l_out; /* [n_layer][n_embd] */
    float *kqv;            /* [n_layer][n_head*head_dim] */
    float *ffn_act;        /* [n_layer][n_ff] or NULL (dump of gelu(gate)*up) */
    float *result_norm;    /* [n_embd] */
    float *logits;         /* [n_vocab] */
} ggb_decoder_io;
typedef struct ggb_decoder ggb_decoder;
/* GGB_ERR_UNSUPPORTED when the shape is outside the fused kernel's envelope (callers then use ggb_op_*) */
int ggb_decoder_create(const ggb_decoder_dims *dims, const ggb_decoder_layer *layers, const ggb_weight *token_embd,
                       const float *output_norm, const ggb_decoder_io *io, ggb_decoder **out);
/* tensor-parallel form (one process per GPU, ggb_comm_init done): the phases that carry the bytes (GATE_UP, DOWN,
 * LOGITS) are split by output rows over `size` ranks and push their flagged 8-byte output words into EVERY rank's
 * buffers with peer stores over NVLink (cudaIpc mappings exchanged at create time) — the all-gather is fused into
 * the producing epilogue, no NCCL call on the token path.  The attention block (QKV, scores, soft-max * V, O) is
 * sharded by KV head when n_head and n_head_kv divide by `size` (each rank's cache then holds only its heads:
 * [n_ctx][ggb_decoder_kv_heads_local * head_dim]) and replicated otherwise.  Bit-identical to the single-GPU kernel. */
int ggb_decoder_kv_heads_local(int n_head, int n_head_kv, int size);
int ggb_decoder_create_tp(const ggb_decoder_dims *dims, const ggb_decoder_layer *layers, const ggb_weight *token_embd,
                          const float *output_norm, const ggb_decoder_io *io, int rank, int size, ggb_decoder **out);
int ggb_decoder_step(ggb_decoder *d); /* enqueue one token; capturable into a ggb_graph */
int ggb_decoder_free(ggb_decoder *d);
/* run ONE traced step: stamps[n_phases][grid][4] %globaltimer values in ns (phase start, after the
 * prologue = inputs arrived, end, end), kinds[n_phases] phase kinds (0 QKV, 1 SCORE, 2 PV, 3 O,
 * 4 GATE_UP, 5 DOWN, 6 LOGITS, 7 SAMPLE) */
int ggb_decoder_trace(ggb_decoder *d, long long *stamps, int32_t *kinds, int max_phases, int *n_phases, int *grid);
/* 1 if the kernel computes the soft-max exp (double exp -> fp32 -> fp16) instead of reading the reference's fp16 table:
 * (2: fp32 expf, 1: double exp; 0: table lookup); enabled only when an exhaustive check at create time found the computed
 * form identical to the table for every non-NaN fp16 input */
int ggb_decoder_exp_computed(const ggb_decoder *d);
/* what THIS rank streams per token: bytes of its pass streams (its row shards plus the phases it runs replicated) and
 * the KV heads whose cache it reads - the per-GPU roofline of a tensor-parallel run is computed from these */
long long ggb_decoder_stream_bytes(const ggb_decoder *d);
int ggb_decoder_kv_heads(const ggb_decoder *d);

/* ------------------------------------------------------------------ multi-GPU (row-sharded TP)
 * one process per GPU; the 128-byte NCCL unique id is created on rank 0 and shipped by the
 * caller (torch.distributed / any transport). */
int ggb_comm_unique_id(void *id128);
int ggb_comm_init(const void *id128, int rank, int world);
int ggb_comm_destroy(void);
int ggb_comm_rank(void);
int ggb_comm_size(void);
/* allgather of `bytes` per rank, in place layout: recv[rank*bytes .. ) */
int ggb_op_allgather(const void *send, void *recv, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* GGML_B200_H */
