// latent_attention.cu — attention over a compressed (latent) key/value cache.
//
// A caching layer stores per position ONE row [c | kr]: the normed latent c (R numbers) and the rotated key part kr
// (Dr numbers) that all heads share.  A head's key is [W_uk_h c | kr] and its value W_uv_h c, so with
//     qa_h = [W_uk_h^T q_h(unrotated) | rot(q_h(rotated))] * scale          (ggb_op_latent_q_absorb)
// the score of head h against position j is qa_h . row_j, and the output is W_uv_h (sum_j p_j c_j)
// (ggb_op_latent_attn_out): keys and values are never materialised, every head reads the same cache rows, and a layer
// that borrows another layer's cache only brings its own W_uk / W_uv.  The soft-max carries a per-head sink: one more
// term exp(sink_h) in the denominator that has no key and no value.
//
// Scores, soft-max and the weighted sums are fp32 whatever the storage type of the cache; -fmad=false: fmaf() spelled.
// The cache is paged: position j lives in row table[j / B] * B + j % B.  Positions of a step's tokens are
// *pos0 + t with *pos0 read on the device, so a captured step can be replayed at another position.
#include <cuda_bf16.h>
#include <math.h>

#include "common.cuh"
#include "dense.cuh"

namespace {

__device__ __forceinline__ int64_t cache_row(const int32_t *table, int B, int64_t j) { return (int64_t)table[j / B] * B + j % B; }

// ---- c = rms(d[:R]) * nw, kr = rot(d[R:]) into the cache rows of the step's tokens.  One CTA per token.
// cs: [n_pos][dims / 2][2] (cos, sin) with the rotation's magnitude factor already applied.
template <typename E>
__global__ void __launch_bounds__(128) latent_kv_store_kernel(const float *__restrict__ d, int64_t ldd, int R, int Dr, int dims,
                                                              const float *__restrict__ nw, float eps, const float *__restrict__ cs,
                                                              const int32_t *__restrict__ pos0, const int32_t *__restrict__ table,
                                                              int B, E *__restrict__ cache, int64_t ldk) {
    __shared__ float red[4];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float *dr = d + (int64_t)t * ldd;
    const int64_t p = (int64_t)*pos0 + t;
    E *row = cache + cache_row(table, B, p) * ldk;
    float ss = 0.f;
    for (int i = tid; i < R; i += 128) ss = fmaf(dr[i], dr[i], ss);
    ss = warp_sum_f32(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    const float r = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)R + eps);
    for (int i = tid; i < R; i += 128) row[i] = from_f32<E>(dr[i] * r * nw[i]);
    const float *tab = cs + p * dims; // dims / 2 pairs of (cos, sin)
    for (int i = tid; i < Dr / 2 + (Dr & 1); i += 128) {
        const int i0 = 2 * i, i1 = 2 * i + 1;
        if (i1 < dims) {
            const float u = dr[R + i0], v = dr[R + i1], c = tab[2 * i], s = tab[2 * i + 1];
            row[R + i0] = from_f32<E>(u * c - v * s);
            row[R + i1] = from_f32<E>(v * c + u * s);
        } else {
            row[R + i0] = from_f32<E>(dr[R + i0]);
            if (i1 < Dr) row[R + i1] = from_f32<E>(dr[R + i1]);
        }
    }
}

// ---- qa[t][h] = [W_uk_h^T qn | rot(qr)] * scale.  q rows hold, head by head, D unrotated then Dr rotated numbers.
// A CTA takes kAbsT tokens of one head and 64 of the R outputs; its four groups of 64 threads each take a quarter of the
// D terms (loads of a group are independent and in flight together) and the quarters are added in a fixed order.
constexpr int kAbsT = 8;
template <typename E>
__global__ void __launch_bounds__(256) latent_q_absorb_kernel(const float *__restrict__ q, int64_t ldq, int64_t T, int H, int D, int Dr,
                                                              int dims, const float *__restrict__ cs, const int32_t *__restrict__ pos0,
                                                              const E *__restrict__ w_uk, int R, float scale, float *__restrict__ qa) {
    extern __shared__ float qs[]; // [kAbsT][D], then [4][kAbsT][64] partial sums
    float *ps = qs + kAbsT * D;
    const int h = blockIdx.y, tid = threadIdx.x, rl = tid & 63, dg = tid >> 6;
    const int64_t t0 = (int64_t)blockIdx.x * kAbsT;
    const int nt = (int)min((int64_t)kAbsT, T - t0);
    for (int i = tid; i < kAbsT * D; i += 256) {
        const int tt = i / D, dd = i - tt * D;
        qs[i] = tt < nt ? q[(t0 + tt) * ldq + (int64_t)h * (D + Dr) + dd] : 0.f;
    }
    __syncthreads();
    const int QK = R + Dr;
    const int r = blockIdx.z * 64 + rl;
    {
        float acc[kAbsT];
#pragma unroll
        for (int tt = 0; tt < kAbsT; tt++) acc[tt] = 0.f;
        const int dq = (D + 3) / 4, d0 = dg * dq, d1 = min(D, d0 + dq);
        if (r < R) {
            const E *wc = w_uk + (int64_t)h * D * R + r;
#pragma unroll 8
            for (int dd = d0; dd < d1; dd++) {
                const float w = to_f32(wc[(int64_t)dd * R]);
#pragma unroll
                for (int tt = 0; tt < kAbsT; tt++) acc[tt] = fmaf(qs[tt * D + dd], w, acc[tt]);
            }
        }
#pragma unroll
        for (int tt = 0; tt < kAbsT; tt++) ps[(dg * kAbsT + tt) * 64 + rl] = acc[tt];
    }
    __syncthreads();
    for (int i = tid; i < nt * 64; i += 256) {
        const int tt = i >> 6, l = i & 63, rr = blockIdx.z * 64 + l;
        if (rr < R) {
            const float v = ((ps[(0 * kAbsT + tt) * 64 + l] + ps[(1 * kAbsT + tt) * 64 + l]) + ps[(2 * kAbsT + tt) * 64 + l]) + ps[(3 * kAbsT + tt) * 64 + l];
            qa[((t0 + tt) * H + h) * QK + rr] = v * scale;
        }
    }
    if (blockIdx.z != 0) return;
    const int half = Dr / 2 + (Dr & 1);
    for (int i = tid; i < nt * half; i += 256) {
        const int tt = i / half, pi = i - tt * half;
        const int64_t t = t0 + tt, p = (int64_t)*pos0 + t;
        const float *src = q + t * ldq + (int64_t)h * (D + Dr) + D;
        float *dst = qa + (t * H + h) * QK + R;
        const int i0 = 2 * pi, i1 = i0 + 1;
        if (i1 < dims) {
            const float u = src[i0], v = src[i1], c = cs[p * dims + 2 * pi], sn = cs[p * dims + 2 * pi + 1];
            dst[i0] = (u * c - v * sn) * scale;
            dst[i1] = (v * c + u * sn) * scale;
        } else {
            dst[i0] = src[i0] * scale;
            if (i1 < Dr) dst[i1] = src[i1] * scale;
        }
    }
}

// ---- partial attention of one token over one split of its visible positions, all heads.
// A tile of 32 cache rows is staged in shared memory once per group of NW heads (one warp per head): lane j scores
// row j against the head's qa (shared memory, broadcast reads), the warp updates the running maximum / sum, and every
// lane accumulates its R / 32 coordinates of sum_j p_j c_j.  part[t][split][h] = {m, l, acc[R]}.
template <typename E> struct TileWord;
template <> struct TileWord<float> {
    static constexpr int per = 1;
    static __device__ __forceinline__ float dot(uint32_t w, const float *q, float acc) { return fmaf(__uint_as_float(w), q[0], acc); }
    // accumulator i of a lane holds coordinate coord(lane, i) of sum_j p_j c_j
    static __device__ __forceinline__ int coord(int lane, int i) { return lane + 32 * i; }
    template <int RC, int TQ>
    static __device__ __forceinline__ void pv(const uint32_t *row, int lane, int R, const float (&pj)[TQ], float (&acc)[TQ][RC]) {
#pragma unroll
        for (int i = 0; i < RC; i++)
            if (lane + 32 * i < R) {
                const float c = __uint_as_float(row[lane + 32 * i]);
#pragma unroll
                for (int u = 0; u < TQ; u++) acc[u][i] = fmaf(pj[u], c, acc[u][i]);
            }
    }
    // four words against q[0 .. 4)
    static __device__ __forceinline__ void dot4(const uint32_t *w, const float *q, float (&a)[4]) {
        const float4 q0 = *reinterpret_cast<const float4 *>(q);
        a[0] = fmaf(__uint_as_float(w[0]), q0.x, a[0]);
        a[1] = fmaf(__uint_as_float(w[1]), q0.y, a[1]);
        a[2] = fmaf(__uint_as_float(w[2]), q0.z, a[2]);
        a[3] = fmaf(__uint_as_float(w[3]), q0.w, a[3]);
    }
};
template <> struct TileWord<__nv_bfloat16> {
    static constexpr int per = 2;
    static __device__ __forceinline__ float dot(uint32_t w, const float *q, float acc) {
        acc = fmaf(__uint_as_float(w << 16), q[0], acc);
        return fmaf(__uint_as_float(w & 0xffff0000u), q[1], acc);
    }
    // a lane owns the two numbers of word lane + 32 k: accumulators 2k and 2k + 1 (one 32-bit read for both)
    static __device__ __forceinline__ int coord(int lane, int i) { return 2 * (lane + 32 * (i >> 1)) + (i & 1); }
    template <int RC, int TQ>
    static __device__ __forceinline__ void pv(const uint32_t *row, int lane, int R, const float (&pj)[TQ], float (&acc)[TQ][RC]) {
#pragma unroll
        for (int k = 0; k < RC / 2; k++) {
            const int w = lane + 32 * k;
            if (2 * w < R) { // R odd: the upper half of the last word is the first number of kr; its accumulator is not stored
                const uint32_t v = row[w];
                const float c0 = __uint_as_float(v << 16), c1 = __uint_as_float(v & 0xffff0000u);
#pragma unroll
                for (int u = 0; u < TQ; u++) {
                    acc[u][2 * k] = fmaf(pj[u], c0, acc[u][2 * k]);
                    acc[u][2 * k + 1] = fmaf(pj[u], c1, acc[u][2 * k + 1]);
                }
            }
        }
    }
    // four words (eight numbers) against q[0 .. 8)
    static __device__ __forceinline__ void dot4(const uint32_t *w, const float *q, float (&a)[4]) {
        const float4 q0 = *reinterpret_cast<const float4 *>(q), q1 = *reinterpret_cast<const float4 *>(q + 4);
        a[0] = fmaf(__uint_as_float(w[0] << 16), q0.x, a[0]);
        a[1] = fmaf(__uint_as_float(w[0] & 0xffff0000u), q0.y, a[1]);
        a[2] = fmaf(__uint_as_float(w[1] << 16), q0.z, a[2]);
        a[3] = fmaf(__uint_as_float(w[1] & 0xffff0000u), q0.w, a[3]);
        a[0] = fmaf(__uint_as_float(w[2] << 16), q1.x, a[0]);
        a[1] = fmaf(__uint_as_float(w[2] & 0xffff0000u), q1.y, a[1]);
        a[2] = fmaf(__uint_as_float(w[3] << 16), q1.z, a[2]);
        a[3] = fmaf(__uint_as_float(w[3] & 0xffff0000u), q1.w, a[3]);
    }
};

template <typename E, int RC, int TQ>
__global__ void __launch_bounds__(512) latent_attn_partial_kernel(const float *__restrict__ qa, const E *__restrict__ cache, int64_t ldk,
                                                                  const int32_t *__restrict__ table, int B, const int32_t *__restrict__ pos0,
                                                                  int T, int H, int R, int Dr, int n_split, int SW, int hpc,
                                                                  int64_t window, float *__restrict__ part) {
    // TQ consecutive tokens per CTA (portions): a warp scores and accumulates its head for all of them from ONE read of
    // every tile word; the later token's extra position is masked for the earlier one.
    extern __shared__ __align__(16) uint32_t la_smem[];
    __shared__ int64_t rowoff[32];
    constexpr int PER = TileWord<E>::per;
    const int QK = R + Dr, words = (QK + PER - 1) / PER;
    const int QKp = (words + 3) / 4 * 4 * PER; // q rows padded with zeros to whole groups of four words, 16-byte aligned
    uint32_t *tile = la_smem;                                     // [32][SW]
    float *qsm = reinterpret_cast<float *>(la_smem + 32 * SW);     // [NW][TQ][QKp]; 32 * SW words = 128 * SW bytes: 16-byte aligned
    const int NW = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * TQ, split = blockIdx.y;
    const int nq = min(TQ, T - t0);
    const int64_t n_kv0 = (int64_t)*pos0 + t0 + 1; // causal: token t0 + u sees positions < n_kv0 + u
    // tiles of 32 positions are dealt to the splits in turn: split s takes tiles s, s + n_split, ... counted from the tile
    // that holds the first position the CTA's first token sees (window > 0: token i sees i - window < j <= i)
    const int64_t jlo = window > 0 ? max((int64_t)0, n_kv0 - window) / 32 * 32 : 0;
    const int64_t j0 = jlo + (int64_t)split * 32, j1 = n_kv0 + nq - 1, jstep = (int64_t)32 * n_split;
    const int h_begin = blockIdx.z * hpc, h_end = min(H, h_begin + hpc);
    for (int h0 = h_begin; h0 < h_end; h0 += NW) {
        const int h = h0 + warp;
        const bool live = h < h_end;
        __syncthreads(); // the previous group's q and tile are no longer read
#pragma unroll
        for (int u = 0; u < TQ; u++)
            for (int k = lane; k < QKp; k += 32) // every warp stages its own head
                qsm[(warp * TQ + u) * QKp + k] = (live && u < nq && k < QK) ? qa[((int64_t)(t0 + u) * H + h) * QK + k] : 0.f;
        float m[TQ], l[TQ], acc[TQ][RC];
#pragma unroll
        for (int u = 0; u < TQ; u++) {
            m[u] = -INFINITY, l[u] = 0.f;
#pragma unroll
            for (int i = 0; i < RC; i++) acc[u][i] = 0.f;
        }
        const float *qh = qsm + warp * TQ * QKp;
        for (int64_t j = j0; j < j1; j += jstep) {
            __syncthreads();
            const int rows = (int)min((int64_t)32, j1 - j);
            // page lookups of the tile's rows side by side (one thread per row), then one flat sweep of 16-byte loads
            // over all rows: nothing in it waits for anything else (cache rows start on 16-byte boundaries)
            if (threadIdx.x < rows) rowoff[threadIdx.x] = cache_row(table, B, j + threadIdx.x) * ldk;
            __syncthreads();
            {
                const int w4n = (words + 3) / 4, total = rows * w4n;
                for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * 4) {
                    uint4 v[4];
                    int at[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int i = i0 + u * blockDim.x;
                        at[u] = -1;
                        if (i < total) {
                            const int jj = i / w4n, w4 = i - jj * w4n;
                            v[u] = reinterpret_cast<const uint4 *>(cache + rowoff[jj])[w4];
                            at[u] = jj * SW + w4 * 4;
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        if (at[u] < 0) continue;
                        const int w0 = (at[u] % SW);
                        uint32_t *dst = tile + at[u];
                        dst[0] = v[u].x;
                        if (w0 + 1 < words) dst[1] = v[u].y;
                        if (w0 + 2 < words) dst[2] = v[u].z;
                        if (w0 + 3 < words) dst[3] = v[u].w;
                    }
                }
            }
            __syncthreads();
            if (!live) continue;
            float s[TQ];
#pragma unroll
            for (int u = 0; u < TQ; u++) s[u] = -INFINITY;
            if (lane < rows) {
                const uint32_t *tr = tile + lane * SW;
                float a4[TQ][4];
#pragma unroll
                for (int u = 0; u < TQ; u++) a4[u][0] = a4[u][1] = a4[u][2] = a4[u][3] = 0.f;
                int w = 0;
#pragma unroll 2
                for (; w + 3 < words; w += 4) {
                    const uint32_t tw[4] = {tr[w], tr[w + 1], tr[w + 2], tr[w + 3]};
#pragma unroll
                    for (int u = 0; u < TQ; u++) TileWord<E>::dot4(tw, qh + u * QKp + w * PER, a4[u]);
                }
                for (; w < words; w++)
#pragma unroll
                    for (int u = 0; u < TQ; u++) a4[u][0] = TileWord<E>::dot(tr[w], qh + u * QKp + w * PER, a4[u][0]);
#pragma unroll
                for (int u = 0; u < TQ; u++)
                    if (j + lane < n_kv0 + u && u < nq && (window <= 0 || j + lane >= n_kv0 + u - window))
                        s[u] = (a4[u][0] + a4[u][1]) + (a4[u][2] + a4[u][3]);
            }
            float p[TQ];
#pragma unroll
            for (int u = 0; u < TQ; u++) {
                const float m_new = fmaxf(m[u], warp_max_f32(s[u]));
                const float base = m_new == -INFINITY ? 0.f : m_new; // nothing visible yet: exp(-inf - 0) = 0 everywhere
                const float corr = expf(m[u] - base);
                p[u] = expf(s[u] - base);
                l[u] = fmaf(l[u], corr, warp_sum_f32(p[u]));
                m[u] = m_new;
#pragma unroll
                for (int i = 0; i < RC; i++) acc[u][i] *= corr;
            }
            for (int jj = 0; jj < rows; jj++) {
                float pj[TQ];
#pragma unroll
                for (int u = 0; u < TQ; u++) pj[u] = __shfl_sync(0xffffffffu, p[u], jj);
                TileWord<E>::template pv<RC, TQ>(tile + jj * SW, lane, R, pj, acc);
            }
        }
        if (live) {
#pragma unroll
            for (int u = 0; u < TQ; u++) {
                if (u >= nq) continue;
                float *o = part + (((int64_t)(t0 + u) * n_split + split) * H + h) * (R + 2);
                if (lane == 0) {
                    o[0] = m[u];
                    o[1] = l[u];
                }
#pragma unroll
                for (int i = 0; i < RC; i++) {
                    const int r = TileWord<E>::coord(lane, i);
                    if (r < R) o[2 + r] = acc[u][i];
                }
            }
        }
    }
}

// ---- merge the splits with the sink, then out[t][h] = W_uv_h (sum_j p_j c_j).  kOutT tokens of one head per CTA.
constexpr int kOutT = 8; // tokens of one head per CTA; v_chunk outputs per CTA (every CTA of a head repeats the merge)
template <typename E>
__global__ void __launch_bounds__(256) latent_attn_out_kernel(const float *__restrict__ part, int n_split, const float *__restrict__ sink,
                                                              const E *__restrict__ w_uv, int64_t T, int H, int R, int Dv,
                                                              int v_chunk, const float *__restrict__ gate, int64_t ldg, E *__restrict__ out) {
    extern __shared__ __align__(16) float ol[]; // [kOutT][R]
    const int h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t t0 = (int64_t)blockIdx.x * kOutT;
    const int nt = (int)min((int64_t)kOutT, T - t0);
    const float sk = sink ? sink[h] : -INFINITY; // no sink: nothing beside the keys in the denominator
    float *wsm = ol + kOutT * R; // [kOutT][n_split] weight of every split: exp(m_s - M) / L
    const int64_t ps = (int64_t)H * (R + 2);
    if (warp < nt) { // one warp per token: maximum and denominator over the splits and the sink
        const float *p0 = part + (((t0 + warp) * n_split) * H + h) * (R + 2);
        float M = sk;
        for (int s = lane; s < n_split; s += 32) M = fmaxf(M, p0[s * ps]);
        M = warp_max_f32(M);
        float L = 0.f;
        for (int s = lane; s < n_split; s += 32) L = fmaf(p0[s * ps + 1], expf(p0[s * ps] - M), L);
        L = warp_sum_f32(L);
        if (sink) L += expf(sk - M);
        const float inv = 1.0f / L;
        for (int s = lane; s < n_split; s += 32) wsm[warp * n_split + s] = expf(p0[s * ps] - M) * inv;
    }
    __syncthreads();
    for (int tt = 0; tt < kOutT; tt++) {
        if (tt >= nt) {
            for (int r = tid; r < R; r += 256) ol[tt * R + r] = 0.f;
            continue;
        }
        const float *p0 = part + (((t0 + tt) * n_split) * H + h) * (R + 2) + 2;
        for (int r = tid; r < R; r += 256) {
            float a = 0.f;
#pragma unroll 16
            for (int s = 0; s < n_split; s++) a = fmaf(p0[s * ps + r], wsm[tt * n_split + s], a);
            ol[tt * R + r] = a;
        }
    }
    __syncthreads();
    const int v_end = min(Dv, ((int)blockIdx.z + 1) * v_chunk);
    for (int v = blockIdx.z * v_chunk + warp; v < v_end; v += 8) {
        const E *wr = w_uv + ((int64_t)h * Dv + v) * R;
        float acc[kOutT];
#pragma unroll
        for (int tt = 0; tt < kOutT; tt++) acc[tt] = 0.f;
        constexpr int VE = 16 / (int)sizeof(E);
        // few CTAs (decode): 16-byte loads, everything in flight at once; a full grid is better off with the conflict-free
        // 4-byte reads of shared memory
        if (v_chunk < Dv && R % VE == 0 && (reinterpret_cast<uintptr_t>(w_uv) & 15) == 0) {
#pragma unroll 4
            for (int k = lane * VE; k < R; k += 32 * VE) {
                const uint4 wv = *reinterpret_cast<const uint4 *>(wr + k);
                const E *we = reinterpret_cast<const E *>(&wv);
                float wf[VE];
#pragma unroll
                for (int u = 0; u < VE; u++) wf[u] = to_f32(we[u]);
#pragma unroll
                for (int tt = 0; tt < kOutT; tt++) { // the lane's VE numbers of a token as 16-byte shared-memory reads
#pragma unroll
                    for (int u = 0; u < VE; u += 4) {
                        const float4 o4 = *reinterpret_cast<const float4 *>(ol + tt * R + k + u);
                        acc[tt] = fmaf(wf[u], o4.x, acc[tt]);
                        acc[tt] = fmaf(wf[u + 1], o4.y, acc[tt]);
                        acc[tt] = fmaf(wf[u + 2], o4.z, acc[tt]);
                        acc[tt] = fmaf(wf[u + 3], o4.w, acc[tt]);
                    }
                }
            }
        } else {
#pragma unroll 4
            for (int k = lane; k < R; k += 32) {
                const float w = to_f32(wr[k]);
#pragma unroll
                for (int tt = 0; tt < kOutT; tt++) acc[tt] = fmaf(w, ol[tt * R + k], acc[tt]);
            }
        }
#pragma unroll
        for (int tt = 0; tt < kOutT; tt++) {
            const float s = warp_sum_f32(acc[tt]);
            if (lane == 0 && tt < nt) {
                // the head's gate: one number per (token, head), sigmoid in fp32
                const float gsc = gate ? 1.0f / (1.0f + expf(-gate[(t0 + tt) * ldg + h])) : 1.0f;
                out[(t0 + tt) * ((int64_t)H * Dv) + (int64_t)h * Dv + v] = from_f32<E>(gate ? s * gsc : s);
            }
        }
    }
}

// ---- the materialised form for portions: the latents of a range of positions as dense rows, and the gate on a head's output
template <typename E>
__global__ void latent_gather_kernel(const E *__restrict__ cache, int64_t ldk, const int32_t *__restrict__ table, int B, int64_t first, int R,
                                     E *__restrict__ out) {
    const E *row = cache + cache_row(table, B, first + blockIdx.x) * ldk;
    for (int i = threadIdx.x; i < R; i += blockDim.x) out[(int64_t)blockIdx.x * R + i] = row[i];
}

template <typename E>
__global__ void cvt_rows_kernel(const float *__restrict__ x, int64_t n, E *__restrict__ y) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = from_f32<E>(x[i]);
}

template <typename E>
__global__ void head_gate_kernel(E *__restrict__ x, int64_t T, int H, int Dv, const float *__restrict__ gate, int64_t ldg) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * H * Dv) return;
    const int64_t t = i / ((int64_t)H * Dv);
    const int h = (int)((i - t * H * Dv) / Dv);
    x[i] = from_f32<E>(to_f32(x[i]) * (1.0f / (1.0f + expf(-gate[t * ldg + h]))));
}

template <typename E>
int attn_partial_launch(const float *qa, const void *cache, int64_t ldk, const int32_t *table, int B, const int32_t *pos0, int64_t T, int H,
                        int R, int Dr, int n_split, int64_t window, float *part) {
    constexpr int PER = TileWord<E>::per;
    const int words = (R + Dr + PER - 1) / PER, SW = words | 1; // odd row pitch: lanes of a warp hit 32 different banks
    // heads per CTA: all of them (one warp each, up to 16 at a time) when many tokens share the GPU, groups of 4 when a
    // handful of tokens must fill it (the tile is then staged once per group)
    const int hpc = T >= 64 ? H : (H < 4 ? H : 4);
    const int NW = hpc < 16 ? hpc : 16;
    const int tq = (T >= 64 && R <= 512) ? 2 : 1; // two tokens per CTA for portions (their accumulators fit the registers)
    const size_t smem = (size_t)32 * SW * 4 + (size_t)NW * tq * ((words + 3) / 4 * 4) * PER * 4;
    GGB_CHECK_ARG(smem <= 200 * 1024, "latent_attn: rows of %d numbers do not fit shared memory", R + Dr);
    const dim3 grid((unsigned)((T + tq - 1) / tq), (unsigned)n_split, (unsigned)((H + hpc - 1) / hpc));
#define LA_LAUNCH(RC, TQ)                                                                                                    \
    {                                                                                                                        \
        auto k = latent_attn_partial_kernel<E, RC, TQ>;                                                                      \
        if (smem > 48 * 1024) GGB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
        k<<<grid, NW * 32, smem, ggb_cuda_stream()>>>(qa, (const E *)cache, ldk, table, B, pos0, (int)T, H, R, Dr, n_split, SW, hpc, window, part); \
    }
#define LA_CASE(RC)                       \
    {                                     \
        if (tq == 2) LA_LAUNCH(RC, 2)     \
        else LA_LAUNCH(RC, 1)             \
    }
    if (R <= 64) LA_CASE(2)
    else if (R <= 128) LA_CASE(4)
    else if (R <= 256) LA_CASE(8)
    else if (R <= 512) LA_CASE(16)
    else LA_LAUNCH(32, 1)
#undef LA_LAUNCH
#undef LA_CASE
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

} // namespace

extern "C" {

#define GGB_CHECK_DT(dt) GGB_CHECK_ARG((dt) == GGB_TYPE_BF16 || (dt) == GGB_TYPE_F32, "dtype %d is neither bf16 nor f32", (int)(dt))

int64_t ggb_latent_cache_ld(int R, int Dr) { return ((int64_t)R + Dr + 7) / 8 * 8; }

int ggb_op_latent_kv_store(int dt, const float *d, int64_t ldd, int64_t T, int R, int Dr, int rot_dims, const float *norm_w, float eps,
                           const float *cos_sin, const int32_t *pos0, const int32_t *block_table, int block_size, void *cache) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(d && norm_w && (cos_sin || !rot_dims) && pos0 && block_table && cache && T > 0 && R > 0 && Dr >= 0 && block_size > 0 &&
                      rot_dims >= 0 && rot_dims <= Dr && rot_dims % 2 == 0,
                  "latent_kv_store: bad arguments");
    const int64_t ldk = ggb_latent_cache_ld(R, Dr);
    if (dt == GGB_TYPE_BF16)
        latent_kv_store_kernel<<<(unsigned)T, 128, 0, ggb_cuda_stream()>>>(d, ldd, R, Dr, rot_dims, norm_w, eps, cos_sin, pos0, block_table,
                                                                           block_size, (__nv_bfloat16 *)cache, ldk);
    else
        latent_kv_store_kernel<<<(unsigned)T, 128, 0, ggb_cuda_stream()>>>(d, ldd, R, Dr, rot_dims, norm_w, eps, cos_sin, pos0, block_table,
                                                                           block_size, (float *)cache, ldk);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_latent_q_absorb(int dt, const float *q, int64_t ldq, int64_t T, int H, int D, int Dr, int rot_dims, const float *cos_sin,
                           const int32_t *pos0, const void *w_uk, int R, float scale, float *qa) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(q && (cos_sin || !rot_dims) && pos0 && w_uk && qa && T > 0 && H > 0 && D > 0 && R > 0 && rot_dims <= Dr && rot_dims % 2 == 0,
                  "latent_q_absorb: bad arguments");
    const dim3 grid((unsigned)((T + kAbsT - 1) / kAbsT), (unsigned)H, (unsigned)((R + 63) / 64));
    const size_t smem = (size_t)kAbsT * D * 4 + (size_t)4 * kAbsT * 64 * 4;
    GGB_CHECK_ARG(smem <= 48 * 1024, "latent_q_absorb: head dimension %d too large", D);
    if (dt == GGB_TYPE_BF16)
        latent_q_absorb_kernel<<<grid, 256, smem, ggb_cuda_stream()>>>(q, ldq, T, H, D, Dr, rot_dims, cos_sin, pos0,
                                                                       (const __nv_bfloat16 *)w_uk, R, scale, qa);
    else
        latent_q_absorb_kernel<<<grid, 256, smem, ggb_cuda_stream()>>>(q, ldq, T, H, D, Dr, rot_dims, cos_sin, pos0, (const float *)w_uk, R,
                                                                       scale, qa);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_latent_expand(int dt, const void *cache, const int32_t *block_table, int block_size, int64_t first, int64_t n, int R, int Dr,
                         const void *w_ukv, int64_t N, void *c_rows, float *kv_f32, void *kv, int64_t ld_kv) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(cache && block_table && w_ukv && c_rows && kv && block_size > 0 && first >= 0 && n > 0 && R > 0 && Dr >= 0 && N > 0 && ld_kv >= N &&
                      (dt == GGB_TYPE_F32 || kv_f32),
                  "latent_expand: bad arguments");
    const int64_t ldk = ggb_latent_cache_ld(R, Dr);
    if (dt == GGB_TYPE_BF16)
        latent_gather_kernel<<<(unsigned)n, 128, 0, ggb_cuda_stream()>>>((const __nv_bfloat16 *)cache, ldk, block_table, block_size, first, R, (__nv_bfloat16 *)c_rows);
    else
        latent_gather_kernel<<<(unsigned)n, 128, 0, ggb_cuda_stream()>>>((const float *)cache, ldk, block_table, block_size, first, R, (float *)c_rows);
    GGB_LAUNCH_CHECK();
    // keys and values of every head in one product: rows [k (H D) | v (H Dv)], the row layout of the window attention's cache
    if (dt == GGB_TYPE_F32) return ggb_op_linear(dt, w_ukv, N, R, c_rows, R, n, (float *)kv, ld_kv);
    const int rc = ggb_op_linear(dt, w_ukv, N, R, c_rows, R, n, kv_f32, ld_kv);
    if (rc) return rc;
    cvt_rows_kernel<<<(unsigned)((n * ld_kv + 255) / 256), 256, 0, ggb_cuda_stream()>>>(kv_f32, n * ld_kv, (__nv_bfloat16 *)kv);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_head_gate(int dt, void *x, int64_t T, int H, int Dv, const float *gate, int64_t ldg) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(x && gate && T > 0 && H > 0 && Dv > 0 && ldg >= H, "head_gate: bad arguments");
    const unsigned blocks = (unsigned)((T * H * Dv + 255) / 256);
    if (dt == GGB_TYPE_BF16) head_gate_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>((__nv_bfloat16 *)x, T, H, Dv, gate, ldg);
    else head_gate_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>((float *)x, T, H, Dv, gate, ldg);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

size_t ggb_latent_attn_scratch_bytes(int64_t T, int H, int R, int n_split) {
    return (size_t)T * (size_t)n_split * (size_t)H * (size_t)(R + 2) * sizeof(float);
}

int ggb_op_latent_attn(int dt, const float *qa, const void *cache, const int32_t *block_table, int block_size, const int32_t *pos0,
                       int64_t T, int H, int R, int Dr, int n_split, float *part) {
    return ggb_op_latent_attn_window(dt, qa, cache, block_table, block_size, pos0, T, H, R, Dr, 0, n_split, part);
}

int ggb_op_latent_attn_window(int dt, const float *qa, const void *cache, const int32_t *block_table, int block_size, const int32_t *pos0,
                              int64_t T, int H, int R, int Dr, int64_t window, int n_split, float *part) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(qa && cache && block_table && pos0 && part && T > 0 && H > 0 && R > 0 && R <= 1024 && Dr >= 0 && n_split > 0 &&
                      n_split <= 65535 && block_size > 0,
                  "latent_attn: bad arguments (latent size up to 1024)");
    const int64_t ldk = ggb_latent_cache_ld(R, Dr);
    if (dt == GGB_TYPE_BF16)
        return attn_partial_launch<__nv_bfloat16>(qa, cache, ldk, block_table, block_size, pos0, T, H, R, Dr, n_split, window, part);
    return attn_partial_launch<float>(qa, cache, ldk, block_table, block_size, pos0, T, H, R, Dr, n_split, window, part);
}

int ggb_op_latent_attn_out(int dt, const float *part, int n_split, const float *sink, const void *w_uv, int64_t T, int H, int R, int Dv,
                           void *out) {
    GGB_CHECK_ARG(sink != nullptr, "latent_attn_out: no sink");
    return ggb_op_latent_attn_out_gated(dt, part, n_split, sink, w_uv, T, H, R, Dv, nullptr, 0, out);
}

int ggb_op_latent_attn_out_gated(int dt, const float *part, int n_split, const float *sink, const void *w_uv, int64_t T, int H, int R, int Dv,
                                 const float *gate, int64_t ldg, void *out) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG((!gate || ldg >= H) && part && w_uv && out && T > 0 && H > 0 && R > 0 && Dv > 0 && n_split > 0, "latent_attn_out: bad arguments");
    // few tokens: spread a head's outputs over several CTAs; many tokens: the grid is large already, merge once per head
    const int v_chunk = T * H >= 1024 ? Dv : 16;
    const dim3 grid((unsigned)((T + kOutT - 1) / kOutT), (unsigned)H, (unsigned)((Dv + v_chunk - 1) / v_chunk));
    const size_t smem = (size_t)kOutT * (R + n_split) * 4;
    GGB_CHECK_ARG(smem <= 48 * 1024, "latent_attn_out: latent size %d with %d splits too large", R, n_split);
    if (dt == GGB_TYPE_BF16)
        latent_attn_out_kernel<<<grid, 256, smem, ggb_cuda_stream()>>>(part, n_split, sink, (const __nv_bfloat16 *)w_uv, T, H, R, Dv,
                                                                       v_chunk, gate, ldg, (__nv_bfloat16 *)out);
    else
        latent_attn_out_kernel<<<grid, 256, smem, ggb_cuda_stream()>>>(part, n_split, sink, (const float *)w_uv, T, H, R, Dv, v_chunk, gate, ldg, (float *)out);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

} // extern "C"
