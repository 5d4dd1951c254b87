// window_attention.cu — grouped-query soft-max attention over a sliding window of a paged cache, with rotary positions
// on queries and keys and with rotated values: the value of position j is cached turned by j, the weighted sum of a head
// is turned back by the reader's position i, so that what a head adds depends on i - j only.
//
// The cache row of a position holds [k (G * D) | v (G * Dv)] in the storage type; page tables and positions are read
// on the device (a captured one-token step replays anywhere).  Scores, soft-max and the weighted sum are fp32.
//
// qkv_store: one CTA per token: root mean square over the whole q and the whole k projection, weights, rotation, store.
// window_attn, both forms: lane = key for the scores, lane = pair of value coordinates for the weighted sum, running
// maximum and sum in registers.
//   portions (window_attn_tile_kernel): a CTA owns 32 consecutive tokens of one head, 4 per warp.  Their windows
//   overlap almost wholly, so every tile of 32 cache rows is staged once in shared memory as fp32 (row pitch odd in words:
//   lane = row reads are conflict-free) and serves all 32 queries; a K word read feeds 4 multiply-adds.
//   steps of few tokens (window_attn_kernel): 8 warps split one (token, head)'s keys, rows straight from the cache
//   (several loads in flight), parts merged through shared memory.
//
// The same kernels serve other masks and layouts, all arguments: the visible range of a query is a sliding window or the
// chunk of consecutive positions it lies in (chunks counted from position 0), a score may pass a soft cap
// cap * tanh(s / cap) before the soft-max, and the rotary pairs of q and k are neighbours (2i, 2i + 1) or halves
// (i, i + rot_dims / 2).
//
// Compiled with -fmad=false: multiply-adds are spelled fmaf().
#include <algorithm>

#include "common.cuh"
#include "dense.cuh"

namespace {

constexpr int kMaxDvRegs = 8; // value coordinates per lane: Dv <= 32 * kMaxDvRegs
constexpr int kWarps = 8;
constexpr int kMaxSplit = 16; // CTAs that share one (token, head) of a short step

// the first position the query at position i sees: everything (size <= 0), the last `size` positions, or its chunk
__device__ __forceinline__ int64_t first_visible(int64_t i, int64_t size, int chunked) {
    if (size <= 0) return 0;
    return chunked ? i - i % size : max((int64_t)0, i - size + 1);
}
__device__ __forceinline__ float soft_cap(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }

template <typename E>
__global__ void __launch_bounds__(256) window_qkv_store_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                               int64_t ld, int H, int G, int D, int Dv, const float *__restrict__ qn_w,
                                                               const float *__restrict__ kn_w, float eps, int rot_dims, int rot_halves,
                                                               const float *__restrict__ cs_k, const float *__restrict__ cs_v, float scale,
                                                               const int32_t *__restrict__ pos0, const int32_t *__restrict__ table, int B,
                                                               E *__restrict__ cache, int64_t cache_ld, float *__restrict__ q_out) {
    __shared__ float red[2][8];
    const int64_t t = blockIdx.x;
    const int64_t pos = (int64_t)*pos0 + t;
    const float *qr = q + t * ld, *kr = k + t * ld, *vr = v + t * ld;
    const int nq = H * D, nk = G * D, nv = G * Dv;
    float rq = 1.f, rk = 1.f;
    if (qn_w || kn_w) {
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) sq = fmaf(qr[i], qr[i], sq);
        for (int i = threadIdx.x; i < nk; i += blockDim.x) sk = fmaf(kr[i], kr[i], sk);
        sq = warp_sum_f32(sq);
        sk = warp_sum_f32(sk);
        if ((threadIdx.x & 31) == 0) {
            red[0][threadIdx.x >> 5] = sq;
            red[1][threadIdx.x >> 5] = sk;
        }
        __syncthreads();
        float tq = 0.f, tk = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            tq += red[0][i];
            tk += red[1][i];
        }
        if (qn_w) rq = 1.0f / sqrtf(tq / (float)nq + eps);
        if (kn_w) rk = 1.0f / sqrtf(tk / (float)nk + eps);
    }
    E *row = cache + ((int64_t)table[pos / B] * B + pos % B) * cache_ld;
    const float *ck = cs_k ? cs_k + pos * (rot_dims / 2) * 2 : nullptr;
    // pairs of q and k: pair m of a head is (2m, 2m + 1), or with rot_halves (m, m + rot_dims / 2) for the rotated pairs and
    // the neighbours behind them for the rest; pair m < rot_dims / 2 turns by the table's entry m
    for (int p = threadIdx.x; p < (nq + nk) / 2; p += blockDim.x) {
        const bool is_q = p < nq / 2;
        const int e = is_q ? 2 * p : 2 * p - nq; // even coordinate inside the projection
        const float *src = is_q ? qr : kr;
        const float *nw = is_q ? qn_w : kn_w;
        const float r = is_q ? rq : rk;
        const int d = e % D, m = d / 2;
        const bool turn = ck && d < rot_dims;
        int e0 = e, e1 = e + 1;
        if (rot_halves) {
            if (turn) e0 = e - d + m, e1 = e0 + rot_dims / 2;
            else e0 = e - d + rot_dims + 2 * (m - rot_dims / 2), e1 = e0 + 1;
        }
        float u = src[e0], w = src[e1];
        if (nw) {
            u = u * r * nw[e0];
            w = w * r * nw[e1];
        }
        if (turn) {
            const float c = ck[d], s = ck[d + 1]; // pair m: [cos, sin]
            const float u2 = u * c - w * s, w2 = w * c + u * s;
            u = u2;
            w = w2;
        }
        if (is_q) {
            q_out[t * nq + e0] = u * scale;
            q_out[t * nq + e1] = w * scale;
        } else {
            row[e0] = from_f32<E>(u);
            row[e1] = from_f32<E>(w);
        }
    }
    const float *cv = cs_v ? cs_v + pos * (Dv / 2) * 2 : nullptr;
    for (int p = threadIdx.x; p < nv / 2; p += blockDim.x) {
        const int e = 2 * p, d = e % Dv;
        float u = vr[e], w = vr[e + 1];
        if (cv) {
            const float c = cv[d], s = cv[d + 1];
            const float u2 = u * c - w * s, w2 = w * c + u * s;
            u = u2;
            w = w2;
        }
        row[nk + e] = from_f32<E>(u);
        row[nk + e + 1] = from_f32<E>(w);
    }
}

template <typename E> struct RowVec { // 16 bytes of a cache row
    static constexpr int n = 16 / (int)sizeof(E);
    uint4 raw;
    __device__ __forceinline__ float at(int i) const { return to_f32(reinterpret_cast<const E *>(&raw)[i]); }
};

// what a head's weighted sum becomes: divided by the soft-max sum, turned back by the reader's position, stored
template <typename E, int NP = kMaxDvRegs / 2>
__device__ __forceinline__ void window_finish(const float *acc, float l, int64_t i, int lane, int Dv, const float *__restrict__ cs_v, E *orow) {
    const float inv = 1.0f / l;
    const float *cv = cs_v ? cs_v + i * (Dv / 2) * 2 : nullptr;
#pragma unroll
    for (int r = 0; r < NP; r++) {
        const int c = 2 * lane + 64 * r;
        if (c < Dv) {
            float u = acc[2 * r] * inv, w = acc[2 * r + 1] * inv;
            if (cv) { // turned back: by -i
                const float cs = cv[c], sn = cv[c + 1];
                const float u2 = u * cs + w * sn, w2 = w * cs - u * sn;
                u = u2;
                w = w2;
            }
            orow[c] = from_f32<E>(u);
            orow[c + 1] = from_f32<E>(w);
        }
    }
}

constexpr int kPartW = 2 + 32 * kMaxDvRegs; // one part: running maximum, sum, weighted sum as the lanes hold it

// The CTA (token blockIdx.x, head blockIdx.y, split blockIdx.z of gridDim.z) takes the key tiles whose number is
// split * 8 + warp modulo 8 * splits, one warp a tile.  One split: the result goes to `out`; several: the CTA's merged
// part goes to `part` and window_merge_kernel finishes.
template <typename E>
__global__ void __launch_bounds__(32 * kWarps) window_attn_kernel(const float *__restrict__ q, const E *__restrict__ cache, int64_t cache_ld,
                                                                  const int32_t *__restrict__ table, int B, const int32_t *__restrict__ pos0,
                                                                  int64_t T, int H, int G, int D, int Dv, int64_t window, int chunked,
                                                                  float cap, const float *__restrict__ cs_v, E *__restrict__ out, int vec,
                                                                  float *__restrict__ part_out) {
    extern __shared__ __align__(16) float wa_smem[]; // q: [kWarps][Dp]; merge: [kWarps][kPartW]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y, g = h / (H / G);
    const int Dp = (D + 3) & ~3;
    const int64_t t = blockIdx.x;
    const bool active = t < T;
    float *sq = wa_smem + warp * Dp;
    if (active)
        for (int d = lane; d < Dp; d += 32) sq[d] = d < D ? q[(t * H + h) * D + d] : 0.f;
    __syncwarp();
    const int64_t i = (int64_t)*pos0 + (active ? t : 0);
    const int64_t jlo = first_visible(i, window, chunked);
    const int nreg = (Dv + 63) / 64; // pairs of coordinates per lane: c = 2 * lane + 64 * r
    float acc[kMaxDvRegs];
#pragma unroll
    for (int r = 0; r < kMaxDvRegs; r++) acc[r] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int64_t koff = (int64_t)g * D, voff = (int64_t)G * D + (int64_t)g * Dv;
    if (active) {
        const int64_t step = 32 * kWarps * (int64_t)gridDim.z;
        for (int64_t j0 = jlo + 32 * ((int64_t)blockIdx.z * kWarps + warp); j0 <= i; j0 += step) {
            const int64_t j = j0 + lane;
            float s = -INFINITY;
            // the lane's row of the cache, looked up once: the weighted sum below gets the other lanes' rows by shuffle
            const int64_t jc = min(j, i);
            const int64_t my_row = (int64_t)table[jc / B] * B + jc % B;
            if (j <= i) {
                const E *kr = cache + my_row * cache_ld + koff;
                float a0 = 0.f, a1 = 0.f;
                if (vec) {
                    constexpr int VN = RowVec<E>::n;
#pragma unroll 8
                    for (int d = 0; d < D; d += VN) {
                        RowVec<E> kv;
                        kv.raw = *reinterpret_cast<const uint4 *>(kr + d);
#pragma unroll
                        for (int u = 0; u < VN; u += 2) {
                            a0 = fmaf(kv.at(u), sq[d + u], a0);
                            a1 = fmaf(kv.at(u + 1), sq[d + u + 1], a1);
                        }
                    }
                } else {
                    for (int d = 0; d < D; d++) a0 = fmaf(to_f32(kr[d]), sq[d], a0);
                }
                s = soft_cap(a0 + a1, cap);
            }
            const float m_new = fmaxf(m, warp_max_f32(s)); // finite: key j0 of the tile is always visible
            const float p = j <= i ? expf(s - m_new) : 0.f;
            const float corr = expf(m - m_new);            // m = -inf at the first tile: 0
            l = l * corr + warp_sum_f32(p);
#pragma unroll
            for (int r = 0; r < kMaxDvRegs; r++) acc[r] *= corr;
            m = m_new;
            const int n_keys = (int)min((int64_t)32, i - j0 + 1);
            // rows in groups of 8: the loads of a group are independent and in flight together (a row past the last
            // visible one repeats it with weight 0)
            for (int jb = 0; jb < n_keys; jb += 8) {
                const E *vrow[8];
                float pj[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int jj = min(jb + u, n_keys - 1);
                    pj[u] = jb + u < n_keys ? __shfl_sync(0xffffffffu, p, jj) : 0.f;
                    vrow[u] = cache + __shfl_sync(0xffffffffu, my_row, jj) * cache_ld + voff;
                }
#pragma unroll
                for (int r = 0; r < kMaxDvRegs / 2; r++) {
                    const int c = 2 * lane + 64 * r;
                    if (r < nreg && c < Dv) {
                        float v0[8], v1[8];
#pragma unroll
                        for (int u = 0; u < 8; u++) {
                            v0[u] = to_f32(vrow[u][c]);
                            v1[u] = to_f32(vrow[u][c + 1]);
                        }
#pragma unroll
                        for (int u = 0; u < 8; u++) {
                            acc[2 * r] = fmaf(pj[u], v0[u], acc[2 * r]);
                            acc[2 * r + 1] = fmaf(pj[u], v1[u], acc[2 * r + 1]);
                        }
                    }
                }
            }
        }
    }
    { // merge the warps' parts: [m, l, acc...] per warp
        __syncthreads();
        float *part = wa_smem + kWarps * Dp;
        const int pw = kPartW;
        if (lane == 0) {
            part[warp * pw] = m;
            part[warp * pw + 1] = l;
        }
#pragma unroll
        for (int r = 0; r < kMaxDvRegs; r++) part[warp * pw + 2 + r * 32 + lane] = acc[r];
        __syncthreads();
        if (warp != 0) return;
        float M = -INFINITY;
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, part[w * pw]);
        l = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxDvRegs; r++) acc[r] = 0.f;
        for (int w = 0; w < kWarps; w++) {
            const float mw = part[w * pw];
            if (mw == -INFINITY) continue; // a warp without keys
            const float f = expf(mw - M);
            l = fmaf(part[w * pw + 1], f, l);
#pragma unroll
            for (int r = 0; r < kMaxDvRegs; r++) acc[r] = fmaf(part[w * pw + 2 + r * 32 + lane], f, acc[r]);
        }
        m = M;
    }
    if (gridDim.z > 1) { // M = -inf, l = 0 when the split had no tile
        float *po = part_out + ((t * H + h) * gridDim.z + blockIdx.z) * kPartW;
        if (lane == 0) {
            po[0] = m;
            po[1] = l;
        }
#pragma unroll
        for (int r = 0; r < kMaxDvRegs; r++) po[2 + r * 32 + lane] = acc[r];
        return;
    }
    window_finish(acc, l, i, lane, Dv, cs_v, out + (t * H + h) * Dv);
}

// one warp per (token, head): the splits' parts merged, then as above
template <typename E>
__global__ void __launch_bounds__(32) window_merge_kernel(const float *__restrict__ part, int n_split, const int32_t *__restrict__ pos0, int H, int Dv,
                                                         const float *__restrict__ cs_v, E *__restrict__ out) {
    const int64_t t = blockIdx.x;
    const int h = blockIdx.y, lane = threadIdx.x;
    const float *pp = part + ((t * H + h) * n_split) * kPartW;
    float M = -INFINITY;
    for (int s = 0; s < n_split; s++) M = fmaxf(M, pp[s * kPartW]);
    float l = 0.f, acc[kMaxDvRegs];
#pragma unroll
    for (int r = 0; r < kMaxDvRegs; r++) acc[r] = 0.f;
    for (int s = 0; s < n_split; s++) {
        const float ms = pp[s * kPartW];
        if (ms == -INFINITY) continue;
        const float f = expf(ms - M);
        l = fmaf(pp[s * kPartW + 1], f, l);
#pragma unroll
        for (int r = 0; r < kMaxDvRegs; r++) acc[r] = fmaf(pp[s * kPartW + 2 + r * 32 + lane], f, acc[r]);
    }
    window_finish(acc, l, (int64_t)*pos0 + t, lane, Dv, cs_v, out + (t * H + h) * Dv);
}

// ---- portions: 32 tokens of one head per CTA, tiles of 32 cache rows staged in shared memory
constexpr int kQT = 32, kQPW = kQT / kWarps; // queries per CTA and per warp

// NP: groups of 64 value coordinates (a pair per lane) the lanes accumulate, Dv <= 64 NP.  VEC: rows are staged and K rows
// read in 16-byte pieces; the K pitch kp is then a multiple of 4 words with kp / 4 odd (the eight lanes of a quarter warp, a
// row each, cover all 32 banks) and the V pitch vp a multiple of 4; otherwise kp is odd and vp even (float2 reads).
template <typename E, int NP, bool VEC>
__global__ void __launch_bounds__(32 * kWarps) window_attn_tile_kernel(const float *__restrict__ q, const E *__restrict__ cache, int64_t cache_ld,
                                                                       const int32_t *__restrict__ table, int B, const int32_t *__restrict__ pos0,
                                                                       int64_t T, int H, int G, int D, int Dv, int kp, int vp, int64_t window,
                                                                       int chunked, float cap, const float *__restrict__ cs_v, E *__restrict__ out) {
    extern __shared__ __align__(16) float wa_smem[];
    const int Dp = (D + 3) & ~3;
    float *sq = wa_smem;              // [kQT][Dp]
    float *sk = sq + kQT * Dp;        // [32][kp]
    float *sv = sk + 32 * kp;         // [32][vp]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y, g = h / (H / G);
    const int64_t t0 = (int64_t)blockIdx.x * kQT;
    const int nq = (int)min((int64_t)kQT, T - t0);
    const int64_t i0 = (int64_t)*pos0 + t0;          // position of the CTA's first query
    const int64_t i_last = i0 + nq - 1;
    for (int e = threadIdx.x; e < kQT * Dp; e += blockDim.x) {
        const int qi = e / Dp, d = e - qi * Dp;
        sq[e] = (qi < nq && d < D) ? q[((t0 + qi) * H + h) * D + d] : 0.f;
    }
    const int64_t jlo = first_visible(i0, window, chunked); // never later than a later query's first key
    float acc[kQPW][2 * NP], m[kQPW], l[kQPW];
    int64_t lo[kQPW];
#pragma unroll
    for (int a = 0; a < kQPW; a++) {
        lo[a] = first_visible(i0 + warp * kQPW + a, window, chunked);
        m[a] = -INFINITY;
        l[a] = 0.f;
#pragma unroll
        for (int r = 0; r < 2 * NP; r++) acc[a][r] = 0.f;
    }
    const int64_t koff = (int64_t)g * D, voff = (int64_t)G * D + (int64_t)g * Dv;
    const int row_elems = D + Dv;
    for (int64_t j0 = jlo; j0 <= i_last; j0 += 32) {

        __syncthreads(); // the previous tile has been consumed (and sq is written, the first time)
        const int n_rows = (int)min((int64_t)32, i_last - j0 + 1);
        // a warp stages rows warp, warp + 8, ...: 16-byte pieces of the K part and of the V part, converted to fp32
        for (int rr = warp; rr < 32; rr += kWarps) {
            const int64_t j = j0 + min(rr, n_rows - 1); // a row past the last one repeats it (masked below, weight 0)
            const E *row = cache + ((int64_t)table[j / B] * B + j % B) * cache_ld;
            if (VEC) {
                constexpr int VN = RowVec<E>::n;
                const int nk = D / VN, nv = Dv / VN;
                for (int vi = lane; vi < nk + nv; vi += 32) {
                    const bool is_k = vi < nk;
                    const int c = (is_k ? vi : vi - nk) * VN;
                    RowVec<E> x;
                    x.raw = *reinterpret_cast<const uint4 *>(row + (is_k ? koff : voff) + c);
                    float4 *dst = reinterpret_cast<float4 *>(is_k ? sk + rr * kp + c : sv + rr * vp + c);
#pragma unroll
                    for (int u = 0; u < VN; u += 4) dst[u / 4] = make_float4(x.at(u), x.at(u + 1), x.at(u + 2), x.at(u + 3));
                }
            } else {
                for (int c = lane; c < row_elems; c += 32) {
                    if (c < D) sk[rr * kp + c] = to_f32(row[koff + c]);
                    else sv[rr * vp + c - D] = to_f32(row[voff + c - D]);
                }
            }
        }
        __syncthreads();
        // scores of the warp's queries against key j0 + lane
        float s[kQPW];
#pragma unroll
        for (int a = 0; a < kQPW; a++) s[a] = 0.f;
        const float *kr = sk + lane * kp;
        const int D4 = D & ~3;
#pragma unroll 2
        for (int d = 0; d < D4; d += 4) {
            float k0, k1, k2, k3;
            if (VEC) {
                const float4 kv = *reinterpret_cast<const float4 *>(kr + d);
                k0 = kv.x, k1 = kv.y, k2 = kv.z, k3 = kv.w;
            } else {
                k0 = kr[d], k1 = kr[d + 1], k2 = kr[d + 2], k3 = kr[d + 3];
            }
#pragma unroll
            for (int a = 0; a < kQPW; a++) {
                const float4 qv = *reinterpret_cast<const float4 *>(sq + (warp * kQPW + a) * Dp + d);
                s[a] = fmaf(k0, qv.x, s[a]);
                s[a] = fmaf(k1, qv.y, s[a]);
                s[a] = fmaf(k2, qv.z, s[a]);
                s[a] = fmaf(k3, qv.w, s[a]);
            }
        }
        for (int d = D4; d < D; d++)
#pragma unroll
            for (int a = 0; a < kQPW; a++) s[a] = fmaf(kr[d], sq[(warp * kQPW + a) * Dp + d], s[a]);
        float p[kQPW];
        const int64_t j = j0 + lane;
#pragma unroll
        for (int a = 0; a < kQPW; a++) {
            const int64_t i = i0 + warp * kQPW + a;
            const bool live = warp * kQPW + a < nq;
            const bool vis = live && j <= i && j >= lo[a];
            const float sa = vis ? soft_cap(s[a], cap) : -INFINITY;
            const float m_new = fmaxf(m[a], warp_max_f32(sa));
            // a query none of whose keys lie in this tile keeps m = -inf: nothing to rescale, nothing to add
            const float corr = m_new == -INFINITY ? 1.f : expf(m[a] - m_new);
            p[a] = vis ? expf(sa - m_new) : 0.f;
            l[a] = l[a] * corr + warp_sum_f32(p[a]);
#pragma unroll
            for (int r = 0; r < 2 * NP; r++) acc[a][r] *= corr;
            m[a] = m_new;
        }
#pragma unroll 2
        for (int jj = 0; jj < n_rows; jj++) {
            float pj[kQPW];
#pragma unroll
            for (int a = 0; a < kQPW; a++) pj[a] = __shfl_sync(0xffffffffu, p[a], jj);
#pragma unroll
            for (int r = 0; r < NP; r++) {
                const int c = 2 * lane + 64 * r;
                if (c < Dv) {
                    const float2 vv = *reinterpret_cast<const float2 *>(sv + jj * vp + c);
#pragma unroll
                    for (int a = 0; a < kQPW; a++) {
                        acc[a][2 * r] = fmaf(pj[a], vv.x, acc[a][2 * r]);
                        acc[a][2 * r + 1] = fmaf(pj[a], vv.y, acc[a][2 * r + 1]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < kQPW; a++) {
        const int qi = warp * kQPW + a;
        if (qi >= nq) continue;
        window_finish<E, NP>(acc[a], l[a], i0 + qi, lane, Dv, cs_v, out + ((t0 + qi) * H + h) * Dv);
    }
}

} // namespace

extern "C" {

int64_t ggb_window_cache_ld(int G, int D, int Dv) { return (((int64_t)G * (D + Dv)) + 7) / 8 * 8; }

int ggb_op_window_qkv_store(int dt, const float *q, const float *k, const float *v, int64_t ld, int64_t T, int H, int G, int D, int Dv,
                            const float *qn_w, const float *kn_w, float eps, int rot_dims, const float *cos_sin_k, const float *cos_sin_v,
                            float scale, const int32_t *pos0, const int32_t *block_table, int block_size, void *cache, float *q_out) {
    return ggb_op_masked_qkv_store(dt, q, k, v, ld, T, H, G, D, Dv, qn_w, kn_w, eps, rot_dims, 0, cos_sin_k, cos_sin_v, scale, pos0, block_table,
                                   block_size, cache, q_out);
}

int ggb_op_masked_qkv_store(int dt, const float *q, const float *k, const float *v, int64_t ld, int64_t T, int H, int G, int D, int Dv,
                            const float *qn_w, const float *kn_w, float eps, int rot_dims, int rot_halves, const float *cos_sin_k,
                            const float *cos_sin_v, float scale, const int32_t *pos0, const int32_t *block_table, int block_size, void *cache,
                            float *q_out) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(dt == GGB_TYPE_BF16 || dt == GGB_TYPE_F32, "window_qkv_store: dtype %d is neither bf16 nor f32", dt);
    GGB_CHECK_ARG(q && k && v && pos0 && block_table && cache && q_out && T > 0 && H > 0 && G > 0 && H % G == 0 && block_size > 0,
                  "window_qkv_store: bad arguments");
    GGB_CHECK_ARG(D > 0 && D % 2 == 0 && Dv > 0 && Dv % 2 == 0 && rot_dims >= 0 && rot_dims <= D && rot_dims % 2 == 0 && (!rot_dims || cos_sin_k),
                  "window_qkv_store: head sizes %d / %d and %d rotated dimensions must be even", D, Dv, rot_dims);
    const int64_t cld = ggb_window_cache_ld(G, D, Dv);
    if (dt == GGB_TYPE_BF16)
        window_qkv_store_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>(q, k, v, ld, H, G, D, Dv, qn_w, kn_w, eps, rot_dims, rot_halves,
                                                                            rot_dims ? cos_sin_k : nullptr, cos_sin_v, scale, pos0, block_table,
                                                                            block_size, (__nv_bfloat16 *)cache, cld, q_out);
    else
        window_qkv_store_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>(q, k, v, ld, H, G, D, Dv, qn_w, kn_w, eps, rot_dims, rot_halves,
                                                                            rot_dims ? cos_sin_k : nullptr, cos_sin_v, scale, pos0, block_table,
                                                                            block_size, (float *)cache, cld, q_out);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

size_t ggb_window_attn_scratch_bytes(int H) { return (size_t)(kQT - 1) * (size_t)H * kMaxSplit * kPartW * 4; }

int ggb_op_window_attn(int dt, const float *q, const void *cache, const int32_t *block_table, int block_size, const int32_t *pos0, int64_t T,
                       int H, int G, int D, int Dv, int64_t window, const float *cos_sin_v, void *out, float *scratch) {
    return ggb_op_masked_attn(dt, q, cache, block_table, block_size, pos0, T, H, G, D, Dv, window, 0, 0.f, cos_sin_v, out, scratch);
}

int ggb_op_masked_attn(int dt, const float *q, const void *cache, const int32_t *block_table, int block_size, const int32_t *pos0, int64_t T,
                       int H, int G, int D, int Dv, int64_t window, int chunked, float softcap, const float *cos_sin_v, void *out,
                       float *scratch) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(softcap >= 0.f && (chunked == 0 || chunked == 1), "masked_attn: the soft cap must not be negative");
    GGB_CHECK_ARG(dt == GGB_TYPE_BF16 || dt == GGB_TYPE_F32, "window_attn: dtype %d is neither bf16 nor f32", dt);
    GGB_CHECK_ARG(q && cache && block_table && pos0 && out && T > 0 && H > 0 && G > 0 && H % G == 0 && block_size > 0 && D > 0 && Dv > 0 &&
                      Dv % 2 == 0 && Dv <= 32 * kMaxDvRegs,
                  "window_attn: bad arguments (value size %d, even and at most %d)", Dv, 32 * kMaxDvRegs);
    const int64_t cld = ggb_window_cache_ld(G, D, Dv);
    const int Dp = (D + 3) & ~3;
    const int es = dt == GGB_TYPE_BF16 ? 2 : 4, vn = 16 / es;
    const int vec = D % vn == 0 && ((uintptr_t)cache % 16 == 0); // rows are 8 numbers apart at least: 16-byte aligned in both types
    cudaStream_t st = ggb_cuda_stream();
    if (T >= kQT) { // a portion: tiles of cache rows staged once for 32 queries
        // 16-byte pieces need every head's keys and values to start on one: D, Dv and G * D whole pieces
        const bool tv = vec && Dv % vn == 0 && ((int64_t)G * D) % vn == 0;
        int kp = D | 1, vp = Dv + 2;
        if (tv) {
            kp = (D + 3) & ~3;
            if ((kp / 4) % 2 == 0) kp += 4;
            vp = (Dv + 3) & ~3;
        }
        const size_t smem = ((size_t)kQT * Dp + 32 * (size_t)kp + 32 * (size_t)vp) * 4;
        GGB_CHECK_ARG(smem <= 200 * 1024, "window_attn: head sizes %d / %d do not fit shared memory", D, Dv);
        const dim3 grid((unsigned)((T + kQT - 1) / kQT), (unsigned)H);
#define WT_LAUNCH(ET, NP, VEC)                                                                                               \
    {                                                                                                                        \
        auto kfn = window_attn_tile_kernel<ET, NP, VEC>;                                                                     \
        if (smem > 48 * 1024) GGB_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));    \
        kfn<<<grid, 32 * kWarps, smem, st>>>(q, (const ET *)cache, cld, block_table, block_size, pos0, T, H, G, D, Dv, kp, vp, \
                                             window, chunked, softcap, cos_sin_v, (ET *)out);                                                  \
    }
#define WT_NP(ET, VEC)                             \
    {                                              \
        if (Dv <= 64) WT_LAUNCH(ET, 1, VEC)        \
        else if (Dv <= 128) WT_LAUNCH(ET, 2, VEC)  \
        else WT_LAUNCH(ET, 4, VEC)                 \
    }
        if (dt == GGB_TYPE_BF16) {
            if (tv) WT_NP(__nv_bfloat16, true) else WT_NP(__nv_bfloat16, false)
        } else {
            if (tv) WT_NP(float, true) else WT_NP(float, false)
        }
#undef WT_NP
#undef WT_LAUNCH
    } else {
        const size_t smem = (size_t)kWarps * Dp * 4 + (size_t)kWarps * kPartW * 4;
        GGB_CHECK_ARG(smem <= 48 * 1024, "window_attn: key size %d does not fit shared memory", D);
        // a warp a tile: as many splits as the longest visible range has groups of 8 tiles (the range is bounded by the
        // window; without one, by what the scratch was sized for)
        int n_split = 1;
        if (scratch && window > 0) n_split = (int)std::min<int64_t>(kMaxSplit, ((window + 62) / 32 + kWarps - 1) / kWarps);
        else if (scratch) n_split = kMaxSplit / 2;
        const dim3 grid((unsigned)T, (unsigned)H, (unsigned)n_split);
#define WS_LAUNCH(ET)                                                                                                                        \
    window_attn_kernel<ET><<<grid, 32 * kWarps, smem, st>>>(q, (const ET *)cache, cld, block_table, block_size, pos0, T, H, G, D, Dv, window,  \
                                                            chunked, softcap, cos_sin_v, (ET *)out, vec, scratch);                                             \
    if (n_split > 1) {                                                                                                                       \
        GGB_LAUNCH_CHECK();                                                                                                                  \
        window_merge_kernel<ET><<<dim3((unsigned)T, (unsigned)H), 32, 0, st>>>(scratch, n_split, pos0, H, Dv, cos_sin_v, (ET *)out);          \
    }
        if (dt == GGB_TYPE_BF16) { WS_LAUNCH(__nv_bfloat16) } else { WS_LAUNCH(float) }
#undef WS_LAUNCH
    }
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

} // extern "C"
