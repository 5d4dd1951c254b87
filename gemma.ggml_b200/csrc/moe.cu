// moe.cu — mixture of experts: the router (fp32 logits, the `top` largest, soft-max over the chosen ones only), the
// grouping of (token, slot) pairs by expert, the two grouped products (dense.cu: linear_tile_kernel, GROUPED) and the
// weighted sum.  A token's result does not depend on which other tokens share the step: every slot is computed by
// itself in k order and the `top` slot outputs are added in slot order.
#include <cuda_bf16.h>

#include <algorithm>
#include <math.h>

#include "common.cuh"
#include "dense.cuh"

namespace {

// one warp: w . h in fp32, the same order of sums wherever it is called from
template <typename E>
__device__ __forceinline__ float router_dot(const E *__restrict__ hr, const float *__restrict__ wr, int64_t W, int lane) {
    float s = 0.f;
    if (W % 4 == 0) {
#pragma unroll 4
        for (int64_t k = (int64_t)lane * 4; k < W; k += 128) {
            const float4 wv = *reinterpret_cast<const float4 *>(wr + k);
            s = fmaf(wv.x, to_f32(hr[k]), s);
            s = fmaf(wv.y, to_f32(hr[k + 1]), s);
            s = fmaf(wv.z, to_f32(hr[k + 2]), s);
            s = fmaf(wv.w, to_f32(hr[k + 3]), s);
        }
    } else {
        for (int64_t k = lane; k < W; k += 32) s = fmaf(wr[k], to_f32(hr[k]), s);
    }
    return warp_sum_f32(s);
}

// router logits: a warp per (token, expert), z[t][e] = w[e] . h[t] + b[e] in fp32
template <typename E>
__global__ void __launch_bounds__(256) moe_logits_kernel(const E *__restrict__ h, int64_t W, int64_t T, const float *__restrict__ w,
                                                         const float *__restrict__ b, int n_exp, float *__restrict__ z) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= T * n_exp) return;
    const int64_t t = i / n_exp;
    const int e = (int)(i - t * n_exp);
    const float s = router_dot(h + t * W, w + (int64_t)e * W, W, lane);
    if (lane == 0) z[i] = s + (b ? b[e] : 0.f);
}

// one warp per token: `top` rounds of arg-max over its logits (ties: the lower index), soft-max over the chosen
__global__ void __launch_bounds__(32) moe_select_kernel(const float *__restrict__ zg, int n_exp, int top, int32_t *__restrict__ idx,
                                                        float *__restrict__ wt) {
    extern __shared__ float z[]; // [n_exp] logits, then [top] chosen values
    float *sel = z + n_exp;
    const int64_t t = blockIdx.x;
    const int lane = threadIdx.x;
    for (int e = lane; e < n_exp; e += 32) z[e] = zg[t * n_exp + e];
    __syncwarp();
    for (int k = 0; k < top; k++) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < n_exp; e += 32) {
            const float v = z[e];
            if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            idx[t * top + k] = bi;
            sel[k] = bv;
            z[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        float m = sel[0], sum = 0.f; // sel[0] is the largest
        for (int k = 0; k < top; k++) {
            sel[k] = expf(sel[k] - m);
            sum += sel[k];
        }
        for (int k = 0; k < top; k++) wt[t * top + k] = sel[k] / sum;
    }
}

// one warp per token, sigmoid scores with a choice correction and groups: s = sigmoid(z); the choice score of expert e is
// s_e + corr_e; the experts form n_groups equal groups of neighbours, a group's score is the sum of its two largest
// choice scores, and only experts of the `keep` best groups (ties: the lower group) can be chosen; among them the `top`
// largest choice scores win (ties: the lower index).  The weight of a chosen expert is its plain s, not renormalised.
// one warp; sc holds the logits on entry (the scores afterwards), ch and gsc are scratch
__device__ __forceinline__ void select_sigmoid_warp(float *sc, float *ch, float *gsc, const float *__restrict__ corr, int n_exp, int top, int n_groups,
                                                    int keep, int64_t t, int lane, int32_t *__restrict__ idx, float *__restrict__ wt) {
    const int gs = n_exp / n_groups;
    for (int e = lane; e < n_exp; e += 32) {
        const float s = 1.0f / (1.0f + expf(-sc[e]));
        sc[e] = s;
        ch[e] = s + (corr ? corr[e] : 0.f);
    }
    __syncwarp();
    if (keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) { // the two largest of the group, in index order
            float a = -INFINITY, b = -INFINITY;
            for (int e = g * gs; e < (g + 1) * gs; e++) {
                const float v = ch[e];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            gsc[g] = gs > 1 ? a + b : a;
        }
        __syncwarp();
        // a group stays when fewer than `keep` groups come before it in the order (larger score, then lower index)
        for (int g = lane; g < n_groups; g += 32) {
            int before = 0;
            for (int o = 0; o < n_groups; o++) before += (gsc[o] > gsc[g]) || (gsc[o] == gsc[g] && o < g);
            if (before >= keep)
                for (int e = g * gs; e < (g + 1) * gs; e++) ch[e] = -INFINITY;
        }
        __syncwarp();
    }
    for (int k = 0; k < top; k++) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < n_exp; e += 32) {
            const float v = ch[e];
            if (!isnan(sc[e]) && sc[e] >= 0.f && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            idx[t * top + k] = bi;
            wt[t * top + k] = sc[bi];
            sc[bi] = -1.0f; // taken: a score is never negative otherwise
        }
        __syncwarp();
    }
}

// one warp per token, soft-max scores over ALL experts with a choice correction: s = softmax(z); the `top` largest
// s_e + corr_e win (ties: the lower index); the weight of a chosen expert is its s divided by the chosen ones' sum
// (+ 1e-20).  sc holds the logits on entry (the scores afterwards), ch is scratch.
__device__ __forceinline__ void select_softmax_warp(float *sc, float *ch, const float *__restrict__ corr, int n_exp, int top, int64_t t, int lane,
                                                    int32_t *__restrict__ idx, float *__restrict__ wt) {
    float m = -INFINITY;
    for (int e = lane; e < n_exp; e += 32) m = fmaxf(m, sc[e]);
    m = warp_max_f32(m);
    float sum = 0.f;
    for (int e = lane; e < n_exp; e += 32) {
        const float p = expf(sc[e] - m);
        sc[e] = p;
        sum += p;
    }
    sum = warp_sum_f32(sum);
    for (int e = lane; e < n_exp; e += 32) {
        const float p = sc[e] / sum;
        sc[e] = p;
        ch[e] = p + (corr ? corr[e] : 0.f);
    }
    __syncwarp();
    float chosen = 0.f; // lane 0: sum of the chosen scores, in slot order
    for (int k = 0; k < top; k++) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < n_exp; e += 32) {
            const float v = ch[e];
            if (sc[e] >= 0.f && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            idx[t * top + k] = bi;
            wt[t * top + k] = sc[bi];
            chosen += sc[bi];
            sc[bi] = -1.0f; // taken: a score is never negative otherwise
        }
        __syncwarp();
    }
    if (lane == 0) {
        chosen += 1e-20f;
        for (int k = 0; k < top; k++) wt[t * top + k] = wt[t * top + k] / chosen;
    }
}

__global__ void __launch_bounds__(32) moe_select_softmax_kernel(const float *__restrict__ zg, const float *__restrict__ corr, int n_exp, int top,
                                                                int32_t *__restrict__ idx, float *__restrict__ wt) {
    extern __shared__ float sm[]; // [n_exp] scores, [n_exp] choice scores
    for (int e = threadIdx.x; e < n_exp; e += 32) sm[e] = zg[(int64_t)blockIdx.x * n_exp + e];
    __syncwarp();
    select_softmax_warp(sm, sm + n_exp, corr, n_exp, top, blockIdx.x, threadIdx.x, idx, wt);
}

__global__ void __launch_bounds__(32) moe_select_sigmoid_kernel(const float *__restrict__ zg, const float *__restrict__ corr, int n_exp, int top,
                                                                int n_groups, int keep, int32_t *__restrict__ idx, float *__restrict__ wt) {
    extern __shared__ float sm[]; // [n_exp] scores, [n_exp] choice scores, [n_groups] group scores
    for (int e = threadIdx.x; e < n_exp; e += 32) sm[e] = zg[(int64_t)blockIdx.x * n_exp + e];
    __syncwarp();
    select_sigmoid_warp(sm, sm + n_exp, sm + 2 * n_exp, corr, n_exp, top, n_groups, keep, blockIdx.x, threadIdx.x, idx, wt);
}

// few tokens (a step): logits and choice in ONE launch.  CTA (token, y) computes the logits of experts 8 y .. 8 y + 7, a warp
// each, so that the router's rows are read by many SMs; the CTA that finishes last for its token (a counter per token, put
// back to zero by that CTA) reads all logits back and chooses.  With row_src the slots are also listed as the mat-vec form
// of the grouped products reads them (slot s = row s: no order is needed there), which stands in for moe_group_kernel.
// SOFTMAX: the rule of select_softmax_warp instead (n_groups and keep unused)
constexpr int kRouteStepTokens = 32, kRouteStepWarps = 8;
__device__ unsigned int g_route_done[kRouteStepTokens];

template <typename E, bool SOFTMAX>
__global__ void __launch_bounds__(32 * kRouteStepWarps) moe_route_sigmoid_step_kernel(const E *__restrict__ h, int64_t W, const float *__restrict__ w,
                                                                     const float *__restrict__ corr, int n_exp, int top, int n_groups, int keep,
                                                                     float *zg, int32_t *__restrict__ idx, float *__restrict__ wt,
                                                                     int32_t *__restrict__ row_src, int32_t *__restrict__ inv,
                                                                     int32_t *__restrict__ row_expert) {
    extern __shared__ float sm[];
    __shared__ bool last;
    const int64_t t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = (int)blockIdx.y * kRouteStepWarps + warp;
    if (e < n_exp) {
        const float s = router_dot(h + t * W, w + (int64_t)e * W, W, lane);
        if (lane == 0) {
            zg[t * n_exp + e] = s;
            __threadfence(); // the logit is visible before this CTA is counted
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(&g_route_done[t], 1u) == gridDim.y - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    for (int i = threadIdx.x; i < n_exp; i += blockDim.x) sm[i] = __ldcg(zg + t * n_exp + i); // other CTAs wrote them: not through L1
    if (threadIdx.x == 0) g_route_done[t] = 0; // the next launch starts from zero
    __syncthreads();
    if (warp != 0) return;
    if (SOFTMAX) select_softmax_warp(sm, sm + n_exp, corr, n_exp, top, t, lane, idx, wt);
    else select_sigmoid_warp(sm, sm + n_exp, sm + 2 * n_exp, corr, n_exp, top, n_groups, keep, t, lane, idx, wt);
    __syncwarp();
    if (row_src)
        for (int k = lane; k < top; k += 32) {
            const int64_t s = t * top + k;
            row_src[s] = (int32_t)t;
            inv[s] = (int32_t)s;
            row_expert[s] = idx[s];
        }
}

// one CTA: counts per expert, offsets, the list of 64-row tiles, and the sorted order of the n = T * top slots
// experts n_real .. n_exp - 1 have no matrices (identity experts): their slots are sorted like the others but get no tile
__global__ void __launch_bounds__(1024) moe_group_kernel(const int32_t *__restrict__ idx, int n, int top, int n_exp, int n_real, int32_t *offsets,
                                                         int32_t *row_src, int32_t *inv, int32_t *tile_expert, int32_t *tile_row0,
                                                         int32_t *n_tiles, int32_t *row_expert) {
    extern __shared__ int32_t cnt[]; // [n_exp] counts, then cursors
    for (int e = threadIdx.x; e < n_exp; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int s = threadIdx.x; s < n; s += blockDim.x) atomicAdd(&cnt[idx[s]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, nt = 0;
        for (int e = 0; e < n_exp; e++) {
            const int c = cnt[e];
            offsets[e] = off;
            cnt[e] = off;
            for (int r = off; e < n_real && r < off + c; r += 64) {
                tile_expert[nt] = e;
                tile_row0[nt] = r;
                nt++;
            }
            off += c;
        }
        offsets[n_exp] = off;
        *n_tiles = nt;
    }
    __syncthreads();
    for (int s = threadIdx.x; s < n; s += blockDim.x) {
        const int p = atomicAdd(&cnt[idx[s]], 1);
        row_src[p] = s / top;
        row_expert[p] = idx[s];
        inv[s] = p;
    }
}

// few slots (decode): a warp per (sorted row, output) streams the expert's weight row with 16-byte loads
template <typename E, int ACT>
__global__ void __launch_bounds__(256) moe_vec_kernel(const E *__restrict__ w, int64_t N, int64_t K, const E *__restrict__ a, int64_t lda,
                                                      const int32_t *__restrict__ row_src, const int32_t *__restrict__ row_expert,
                                                      float *__restrict__ c, E *__restrict__ c_act, int64_t ldc, int vec, int n_real, float limit,
                                                      float alpha) {
    constexpr int VE = 16 / (int)sizeof(E);
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int row = blockIdx.y;
    if (n >= N || row_expert[row] >= n_real) return; // an expert without matrices: nothing to compute
    // ACT 2: an expert's matrix holds N gate rows, then N up rows; output n is silu(gate_n) * up_n
    // ACT 3: the same rows; g = min(gate_n, limit), u = clamp(up_n, -limit, limit), output g * sigmoid(alpha g) * (u + 1)
    constexpr bool GATED = ACT == 2 || ACT == 3;
    const E *wr = w + ((int64_t)row_expert[row] * (GATED ? 2 * N : N) + n) * K;
    const E *wu = wr + N * K;
    const E *ar = a + (int64_t)(row_src ? row_src[row] : row) * lda;
    float acc = 0.f, up = 0.f;
    if (vec) {
#pragma unroll 4
        for (int64_t k = (int64_t)lane * VE; k < K; k += 32 * VE) {
            const uint4 wv = ldg_stream_u4(wr + k), av = *reinterpret_cast<const uint4 *>(ar + k);
            const E *we = reinterpret_cast<const E *>(&wv), *ae = reinterpret_cast<const E *>(&av);
#pragma unroll
            for (int u = 0; u < VE; u++) acc = fmaf(to_f32(we[u]), to_f32(ae[u]), acc);
            if (GATED) {
                const uint4 uv = ldg_stream_u4(wu + k);
                const E *ue = reinterpret_cast<const E *>(&uv);
#pragma unroll
                for (int u = 0; u < VE; u++) up = fmaf(to_f32(ue[u]), to_f32(ae[u]), up);
            }
        }
    } else {
        for (int64_t k = lane; k < K; k += 32) {
            acc = fmaf(to_f32(wr[k]), to_f32(ar[k]), acc);
            if (GATED) up = fmaf(to_f32(wu[k]), to_f32(ar[k]), up);
        }
    }
    acc = warp_sum_f32(acc);
    if (GATED) up = warp_sum_f32(up);
    if (lane == 0) {
        if (ACT == 1) c_act[(int64_t)row * ldc + n] = from_f32<E>(acc > 0.f ? acc * acc : 0.f);
        else if (ACT == 2) c_act[(int64_t)row * ldc + n] = from_f32<E>(acc / (1.0f + expf(-acc)) * up);
        else if (ACT == 3) {
            const float g = fminf(acc, limit), u = fminf(fmaxf(up, -limit), limit);
            c_act[(int64_t)row * ldc + n] = from_f32<E>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
        }
        else c[(int64_t)row * ldc + n] = acc;
    }
}

// rows of A in sorted-slot order (the tensor-core product reads its operand contiguously): y[i] = a[row_src[i]], 16 bytes a thread
__global__ void moe_gather_kernel(const uint4 *__restrict__ a, int64_t row_u4, const int32_t *__restrict__ row_src, uint4 *__restrict__ y) {
    const uint4 *src = a + (int64_t)row_src[blockIdx.x] * row_u4;
    for (int64_t i = threadIdx.x; i < row_u4; i += blockDim.x) y[(int64_t)blockIdx.x * row_u4 + i] = src[i];
}

__global__ void moe_combine_kernel(const float *__restrict__ y, const int32_t *__restrict__ inv, const float *__restrict__ wt, int top,
                                   int64_t W, float *__restrict__ out) {
    const int64_t t = blockIdx.x;
    for (int64_t i = threadIdx.x; i < W; i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; k++) s = fmaf(wt[t * top + k], y[(int64_t)inv[t * top + k] * W + i], s);
        out[t * W + i] = s;
    }
}

// the same with experts that hand their input through: a slot whose expert is n_real or later adds wt * h[t]
template <typename E>
__global__ void moe_combine_identity_kernel(const float *__restrict__ y, const int32_t *__restrict__ inv, const float *__restrict__ wt,
                                            const int32_t *__restrict__ idx, int top, int n_real, int64_t W, const E *__restrict__ h,
                                            float *__restrict__ out) {
    const int64_t t = blockIdx.x;
    for (int64_t i = threadIdx.x; i < W; i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; k++) {
            const float v = idx[t * top + k] < n_real ? y[(int64_t)inv[t * top + k] * W + i] : to_f32(h[t * W + i]);
            s = fmaf(wt[t * top + k], v, s);
        }
        out[t * W + i] = s;
    }
}

} // namespace

extern "C" {

#define GGB_CHECK_DT(dt) GGB_CHECK_ARG((dt) == GGB_TYPE_BF16 || (dt) == GGB_TYPE_F32, "dtype %d is neither bf16 nor f32", (int)(dt))

int ggb_op_moe_route(int dt, const void *h, int64_t W, int64_t T, const float *w_router, const float *bias, int n_exp, int top,
                     float *logits, int32_t *idx, float *wt) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(h && w_router && idx && wt && W > 0 && T > 0 && n_exp > 0 && top > 0 && top <= n_exp && n_exp <= 8192,
                  "moe_route: bad arguments");
    GGB_CHECK_ARG(logits != nullptr, "moe_route: needs T * n_exp floats for the logits");
    const size_t smem = (size_t)(n_exp + top) * 4;
    const unsigned blocks = (unsigned)((T * n_exp + 7) / 8);
    if (dt == GGB_TYPE_BF16)
        moe_logits_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>((const __nv_bfloat16 *)h, W, T, w_router, bias, n_exp, logits);
    else
        moe_logits_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>((const float *)h, W, T, w_router, bias, n_exp, logits);
    GGB_LAUNCH_CHECK();
    moe_select_kernel<<<(unsigned)T, 32, smem, ggb_cuda_stream()>>>(logits, n_exp, top, idx, wt);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_moe_step_form(int64_t n_slots) { return n_slots <= 16; }

int ggb_op_moe_route_sigmoid(int dt, const void *h, int64_t W, int64_t T, const float *w_router, const float *correction, int n_exp, int top,
                             int n_groups, int keep, float *logits, int32_t *idx, float *wt, int32_t *ws) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(h && w_router && idx && wt && logits && W > 0 && T > 0 && n_exp > 0 && top > 0 && n_exp <= 4096, "moe_route_sigmoid: bad arguments");
    GGB_CHECK_ARG(n_groups > 0 && n_exp % n_groups == 0 && keep > 0 && keep <= n_groups && top <= keep * (n_exp / n_groups),
                  "moe_route_sigmoid: %d experts in %d groups of which %d stay cannot give %d experts", n_exp, n_groups, keep, top);
    const size_t smem = (size_t)(2 * n_exp + n_groups) * 4;
    if (T <= 32) { // a step: one launch, and the slot lists of the mat-vec form with it
        const int64_t n = T * top;
        const int mt = ggb_moe_max_tiles(n, n_exp);
        const bool lists = ws && ggb_moe_step_form(n);
        int32_t *row_src = lists ? ws + n_exp + 1 : nullptr, *inv = lists ? row_src + n : nullptr, *row_expert = lists ? inv + n + 2 * mt + 1 : nullptr;
        if (dt == GGB_TYPE_BF16)
            moe_route_sigmoid_step_kernel<__nv_bfloat16, false><<<dim3((unsigned)T, (unsigned)((n_exp + kRouteStepWarps - 1) / kRouteStepWarps)), 32 * kRouteStepWarps, smem, ggb_cuda_stream()>>>((const __nv_bfloat16 *)h, W, w_router, correction, n_exp, top, n_groups,
                                                                                         keep, logits, idx, wt, row_src, inv, row_expert);
        else
            moe_route_sigmoid_step_kernel<float, false><<<dim3((unsigned)T, (unsigned)((n_exp + kRouteStepWarps - 1) / kRouteStepWarps)), 32 * kRouteStepWarps, smem, ggb_cuda_stream()>>>((const float *)h, W, w_router, correction, n_exp, top, n_groups, keep,
                                                                                         logits, idx, wt, row_src, inv, row_expert);
        GGB_LAUNCH_CHECK();
        return GGB_OK;
    }
    const unsigned blocks = (unsigned)((T * n_exp + 7) / 8);
    if (dt == GGB_TYPE_BF16)
        moe_logits_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>((const __nv_bfloat16 *)h, W, T, w_router, nullptr, n_exp, logits);
    else
        moe_logits_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>((const float *)h, W, T, w_router, nullptr, n_exp, logits);
    GGB_LAUNCH_CHECK();
    moe_select_sigmoid_kernel<<<(unsigned)T, 32, smem, ggb_cuda_stream()>>>(logits, correction, n_exp, top, n_groups,
                                                                                                         keep, idx, wt);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_moe_route_softmax(int dt, const void *h, int64_t W, int64_t T, const float *w_router, const float *correction, int n_exp, int top,
                             float *logits, int32_t *idx, float *wt, int32_t *ws) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(h && w_router && idx && wt && logits && W > 0 && T > 0 && n_exp > 0 && top > 0 && top <= n_exp && n_exp <= 4096,
                  "moe_route_softmax: bad arguments (%d of %d experts)", top, n_exp);
    const size_t smem = (size_t)(2 * n_exp) * 4;
    if (T <= 32) { // a step: one launch, and the slot lists of the mat-vec form with it
        const int64_t n = T * top;
        const int mt = ggb_moe_max_tiles(n, n_exp);
        const bool lists = ws && ggb_moe_step_form(n);
        int32_t *row_src = lists ? ws + n_exp + 1 : nullptr, *inv = lists ? row_src + n : nullptr, *row_expert = lists ? inv + n + 2 * mt + 1 : nullptr;
        if (dt == GGB_TYPE_BF16)
            moe_route_sigmoid_step_kernel<__nv_bfloat16, true><<<dim3((unsigned)T, (unsigned)((n_exp + kRouteStepWarps - 1) / kRouteStepWarps)), 32 * kRouteStepWarps, smem, ggb_cuda_stream()>>>(
                (const __nv_bfloat16 *)h, W, w_router, correction, n_exp, top, 1, 1, logits, idx, wt, row_src, inv, row_expert);
        else
            moe_route_sigmoid_step_kernel<float, true><<<dim3((unsigned)T, (unsigned)((n_exp + kRouteStepWarps - 1) / kRouteStepWarps)), 32 * kRouteStepWarps, smem, ggb_cuda_stream()>>>(
                (const float *)h, W, w_router, correction, n_exp, top, 1, 1, logits, idx, wt, row_src, inv, row_expert);
        GGB_LAUNCH_CHECK();
        return GGB_OK;
    }
    const unsigned blocks = (unsigned)((T * n_exp + 7) / 8);
    if (dt == GGB_TYPE_BF16)
        moe_logits_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>((const __nv_bfloat16 *)h, W, T, w_router, nullptr, n_exp, logits);
    else
        moe_logits_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>((const float *)h, W, T, w_router, nullptr, n_exp, logits);
    GGB_LAUNCH_CHECK();
    moe_select_softmax_kernel<<<(unsigned)T, 32, smem, ggb_cuda_stream()>>>(logits, correction, n_exp, top, idx, wt);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_moe_max_tiles(int64_t n_slots, int n_exp) { return (int)(n_slots / 64) + n_exp; }
size_t ggb_moe_group_ints(int64_t n_slots, int n_exp) {
    return (size_t)(n_exp + 1) + 3 * (size_t)n_slots + 2 * (size_t)ggb_moe_max_tiles(n_slots, n_exp) + 1;
}

static ggb_moe_groups groups_of(int32_t *ws, int64_t n, int n_exp, bool gather) {
    ggb_moe_groups g;
    const int mt = ggb_moe_max_tiles(n, n_exp);
    g.offsets = ws;
    g.row_src = gather ? ws + n_exp + 1 : nullptr;
    g.tile_expert = ws + n_exp + 1 + 2 * n;
    g.tile_row0 = g.tile_expert + mt;
    g.n_tiles = g.tile_row0 + mt;
    return g;
}

int ggb_op_moe_group(const int32_t *idx, int64_t T, int top, int n_exp, int32_t *ws) { return ggb_op_moe_group_identity(idx, T, top, n_exp, 0, ws); }

int ggb_op_moe_group_identity(const int32_t *idx, int64_t T, int top, int n_exp, int n_identity, int32_t *ws) {
    GGB_REQUIRE_INIT();
    const int64_t n = T * top;
    GGB_CHECK_ARG(idx && ws && T > 0 && top > 0 && n_exp > 0 && n_exp <= 8192 && n < (1ll << 30) && n_identity >= 0 && n_identity <= n_exp,
                  "moe_group: bad arguments");
    const int mt = ggb_moe_max_tiles(n, n_exp);
    int32_t *offsets = ws, *row_src = ws + n_exp + 1, *inv = row_src + n, *te = inv + n, *tr = te + mt, *nt = tr + mt, *re = nt + 1;
    moe_group_kernel<<<1, 1024, (size_t)n_exp * 4, ggb_cuda_stream()>>>(idx, (int)n, top, n_exp, n_exp - n_identity, offsets, row_src, inv, te, tr, nt, re);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_moe_linear(int dt, const void *w, int64_t N, int64_t K, const void *a, int64_t lda, int gather, int64_t T, int top, int n_exp,
                      const int32_t *ws, int act, void *c, int64_t ldc) {
    return ggb_op_moe_linear_identity(dt, w, N, K, a, lda, gather, T, top, n_exp, 0, ws, act, 0.f, 0.f, c, ldc);
}

int ggb_op_moe_linear_identity(int dt, const void *w, int64_t N, int64_t K, const void *a, int64_t lda, int gather, int64_t T, int top, int n_exp,
                               int n_identity, const int32_t *ws, int act, float limit, float alpha, void *c, int64_t ldc) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(w && a && ws && c && N > 0 && K > 0 && T > 0 && lda >= K && ldc >= N && act >= 0 && act <= 3 && n_identity >= 0 &&
                      n_identity < n_exp,
                  "moe_linear: bad arguments");
    GGB_CHECK_ARG(act < 2 || ggb_moe_step_form(T * top), "moe_linear: the gated forms are built for steps of at most 16 slots");
    const int n_real = n_exp - n_identity;
    const ggb_moe_groups g = groups_of(const_cast<int32_t *>(ws), T * top, n_exp, gather != 0);
    if (ggb_moe_step_form(T * top)) { // decode: every slot is a mat-vec on its expert's matrix
        const int es = dt == GGB_TYPE_BF16 ? 2 : 4;
        const int vec = K % (16 / es) == 0 && lda % (16 / es) == 0 && ((uintptr_t)w | (uintptr_t)a) % 16 == 0;
        const int32_t *row_expert = g.n_tiles + 1;
        const dim3 grid((unsigned)((N + 7) / 8), (unsigned)(T * top));
#define MV(E)                                                                                                                         \
    if (act == 3) moe_vec_kernel<E, 3><<<grid, 256, 0, ggb_cuda_stream()>>>((const E *)w, N, K, (const E *)a, lda, g.row_src, row_expert, nullptr, (E *)c, ldc, vec, n_real, limit, alpha); \
    else if (act == 2) moe_vec_kernel<E, 2><<<grid, 256, 0, ggb_cuda_stream()>>>((const E *)w, N, K, (const E *)a, lda, g.row_src, row_expert, nullptr, (E *)c, ldc, vec, n_real, 0.f, 0.f); \
    else if (act) moe_vec_kernel<E, 1><<<grid, 256, 0, ggb_cuda_stream()>>>((const E *)w, N, K, (const E *)a, lda, g.row_src, row_expert, nullptr, (E *)c, ldc, vec, n_real, 0.f, 0.f); \
    else moe_vec_kernel<E, 0><<<grid, 256, 0, ggb_cuda_stream()>>>((const E *)w, N, K, (const E *)a, lda, g.row_src, row_expert, (float *)c, nullptr, ldc, vec, n_real, 0.f, 0.f);
        if (dt == GGB_TYPE_BF16) { MV(__nv_bfloat16) } else { MV(float) }
#undef MV
        GGB_LAUNCH_CHECK();
        return GGB_OK;
    }
    // many slots, bf16, aligned shapes: the tcgen05 GEMM, one launch over (N tiles, row tiles, experts)
    if (dt == GGB_TYPE_BF16 && T * top >= 512 && ggb_gemm_grouped_bf16_fits(N, K, ldc) && lda == K && ((uintptr_t)a & 15) == 0) {
        const int64_t n = T * top;
        const void *a_sorted = a;
        if (gather) {
            static void *gbuf = nullptr;
            static size_t gbytes = 0;
            const size_t need = (size_t)n * (size_t)K * 2;
            if (need > gbytes) {
                if (gbuf) cudaFree(gbuf);
                gbuf = nullptr, gbytes = 0;
                GGB_CUDA(cudaMalloc(&gbuf, need));
                gbytes = need;
            }
            moe_gather_kernel<<<(unsigned)n, 128, 0, ggb_cuda_stream()>>>((const uint4 *)a, K / 8, g.row_src, (uint4 *)gbuf);
            GGB_LAUNCH_CHECK();
            a_sorted = gbuf;
        }
        return ggb_gemm_grouped_bf16(w, N, K, a_sorted, n, n_real, g.offsets, act ? nullptr : (float *)c, act ? c : nullptr, ldc);
    }
    return ggb_linear_grouped_launch(dt, w, N, K, a, lda, ggb_moe_max_tiles(T * top, n_exp), act ? nullptr : (float *)c, act ? c : nullptr,
                                     ldc, act, g);
}

int ggb_op_moe_combine_norm(int dt, const float *y, const int32_t *ws, const float *wt, int64_t T, int top, int n_exp, int64_t W, const float *wa,
                            float eps, float *x, const float *wy, void *out) {
    GGB_CHECK_ARG(y && ws && wt && top > 0 && n_exp > 0, "moe_combine_norm: bad arguments");
    return ggb_norm_add_norm_launch(dt, y, nullptr, ws + n_exp + 1 + T * top, wt, top, wa, eps, W, T, x, wy, out);
}

int ggb_op_moe_combine_identity(int dt, const float *y, const int32_t *ws, const float *wt, const int32_t *idx, int64_t T, int top, int n_exp,
                                int n_identity, int64_t W, const void *h, float *out) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(y && ws && wt && idx && h && out && T > 0 && top > 0 && W > 0 && n_identity >= 0 && n_identity <= n_exp,
                  "moe_combine_identity: bad arguments");
    const int32_t *inv = ws + n_exp + 1 + T * top;
    if (dt == GGB_TYPE_BF16)
        moe_combine_identity_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>(y, inv, wt, idx, top, n_exp - n_identity, W, (const __nv_bfloat16 *)h, out);
    else
        moe_combine_identity_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>(y, inv, wt, idx, top, n_exp - n_identity, W, (const float *)h, out);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_moe_combine(const float *y, const int32_t *ws, const float *wt, int64_t T, int top, int n_exp, int64_t W, float *out) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(y && ws && wt && out && T > 0 && top > 0 && W > 0, "moe_combine: bad arguments");
    const int32_t *inv = ws + n_exp + 1 + T * top;
    moe_combine_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>(y, inv, wt, top, W, out);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

} // extern "C"
