// sigmoid_attention.cu — grouped-query attention whose weights are not normalised over the keys: the weight of key j for
// the query at position i >= j is
//     sigmoid(q_i . k_j * scale  -  r1_h ln(1 + r2_h (i - j))  +  pb_h),
// a head's own distance penalty and offset inside the sigmoid, and the head's output is the plain weighted sum of the
// values.  No running maximum, no denominator: parts of a key range simply add.
//
// The cache row of a position holds [k (G * D) | v (G * Dv)] in the storage type, as in window_attention.cu (same pitch,
// same pages); page tables and positions are read on the device, so a captured one-token step replays anywhere.
// Scores, the penalty, the sigmoid and the weighted sum are fp32 in both storage types.
//
// qkv_store: one CTA per token.  The query is multiplied by its temperature 1 + coef ln(floor((p + 1) / every) + 1) and
// by the score scale; each value head is divided by its root mean square before it is cached.
// sigmoid_attn, portions (sigmoid_attn_tile_kernel): a CTA owns 32 consecutive tokens of one head, 4 per warp; tiles of
// 32 cache rows are staged once in shared memory as fp32 and serve all 32 queries.  The penalty depends on i - j only:
// the 63 distances a tile can meet are computed once per tile (63 logarithms instead of 1024).
// sigmoid_attn, steps of few tokens (sigmoid_attn_step_kernel): 8 warps x up to 16 CTAs split one (token, head)'s keys a
// tile per warp; the CTAs' sums are added by sigmoid_merge_kernel in a fixed order.
//
// Compiled with -fmad=false: multiply-adds are spelled fmaf().
#include <algorithm>

#include "common.cuh"
#include "dense.cuh"

namespace {

constexpr int kMaxDvRegs = 8; // value coordinates per lane: Dv <= 32 * kMaxDvRegs
constexpr int kWarps = 8;
constexpr int kMaxSplit = 16;
constexpr int kQT = 32, kQPW = kQT / kWarps; // queries per CTA and per warp (portions)

__device__ __forceinline__ float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float penalty_f32(float r1, float r2, int64_t dist) { return dist > 0 ? r1 * log1pf(r2 * (float)dist) : 0.f; }

template <typename E> struct RowVec { // 16 bytes of a cache row
    static constexpr int n = 16 / (int)sizeof(E);
    uint4 raw;
    __device__ __forceinline__ float at(int i) const { return to_f32(reinterpret_cast<const E *>(&raw)[i]); }
};

template <typename E>
__global__ void __launch_bounds__(256) sigmoid_qkv_store_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                                int64_t ld, int H, int G, int D, int Dv, float temp_coef, int temp_every,
                                                                float vnorm_eps, float scale, const int32_t *__restrict__ pos0,
                                                                const int32_t *__restrict__ table, int B, E *__restrict__ cache, int64_t cache_ld,
                                                                float *__restrict__ q_out) {
    const int64_t t = blockIdx.x;
    const int64_t pos = (int64_t)*pos0 + t;
    const float *qr = q + t * ld, *kr = k + t * ld, *vr = v + t * ld;
    const int nq = H * D, nk = G * D, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float temp = 1.0f;
    if (temp_every > 0) temp = 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
    E *row = cache + ((int64_t)table[pos / B] * B + pos % B) * cache_ld;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) q_out[t * nq + i] = qr[i] * temp * scale;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) row[i] = from_f32<E>(kr[i]);
    for (int g = warp; g < G; g += (int)(blockDim.x >> 5)) { // a warp per value head
        const float *vg = vr + (int64_t)g * Dv;
        float r = 1.0f;
        if (vnorm_eps >= 0.f) {
            float ss = 0.f;
            for (int i = lane; i < Dv; i += 32) ss = fmaf(vg[i], vg[i], ss);
            r = 1.0f / sqrtf(warp_sum_f32(ss) / (float)Dv + vnorm_eps);
        }
        for (int i = lane; i < Dv; i += 32) row[nk + g * Dv + i] = from_f32<E>(vg[i] * r);
    }
}

// ---- steps of few tokens: CTA (token, head, split); its warps take the key tiles split * 8 + warp modulo 8 * splits
template <typename E>
__global__ void __launch_bounds__(32 * kWarps) sigmoid_attn_step_kernel(const float *__restrict__ q, const E *__restrict__ cache, int64_t cache_ld,
                                                                        const int32_t *__restrict__ table, int B, const int32_t *__restrict__ pos0,
                                                                        int H, int G, int D, int Dv, int64_t window, const float *__restrict__ r1,
                                                                        const float *__restrict__ r2, const float *__restrict__ pb,
                                                                        E *__restrict__ out, int vec, float *__restrict__ part_out) {
    extern __shared__ __align__(16) float sa_smem[]; // q: [kWarps][Dp]; sums: [kWarps][32 * kMaxDvRegs]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y, g = h / (H / G);
    const int Dp = (D + 3) & ~3;
    const int64_t t = blockIdx.x;
    float *sq = sa_smem + warp * Dp;
    for (int d = lane; d < Dp; d += 32) sq[d] = d < D ? q[(t * H + h) * D + d] : 0.f;
    __syncwarp();
    const int64_t i = (int64_t)*pos0 + t;
    const int64_t jlo = window > 0 ? max((int64_t)0, i - window + 1) : 0;
    const float hr1 = r1 ? r1[h] : 0.f, hr2 = r2 ? r2[h] : 0.f, hpb = pb ? pb[h] : 0.f;
    float acc[kMaxDvRegs];
#pragma unroll
    for (int r = 0; r < kMaxDvRegs; r++) acc[r] = 0.f;
    const int64_t koff = (int64_t)g * D, voff = (int64_t)G * D + (int64_t)g * Dv;
    const int64_t step = 32 * kWarps * (int64_t)gridDim.z;
    for (int64_t j0 = jlo + 32 * ((int64_t)blockIdx.z * kWarps + warp); j0 <= i; j0 += step) {
        const int64_t j = j0 + lane;
        const int64_t jc = min(j, i);
        const int64_t my_row = (int64_t)table[jc / B] * B + jc % B; // looked up once; the other lanes get it by shuffle
        float p = 0.f;
        if (j <= i) {
            const E *kr = cache + my_row * cache_ld + koff;
            float a0 = 0.f, a1 = 0.f;
            if (vec) {
                constexpr int VN = RowVec<E>::n;
#pragma unroll 16
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
            p = sigmoid_f32((a0 + a1) - penalty_f32(hr1, hr2, i - j) + hpb);
        }
        const int n_keys = (int)min((int64_t)32, i - j0 + 1);
        // rows in groups of 16: their loads are independent and in flight together (a row past the last visible one
        // repeats it with weight 0)
        constexpr int kRows = 16;
        for (int jb = 0; jb < n_keys; jb += kRows) {
            const E *vrow[kRows];
            float pj[kRows];
#pragma unroll
            for (int u = 0; u < kRows; u++) {
                const int jj = min(jb + u, n_keys - 1);
                pj[u] = jb + u < n_keys ? __shfl_sync(0xffffffffu, p, jj) : 0.f;
                vrow[u] = cache + __shfl_sync(0xffffffffu, my_row, jj) * cache_ld + voff;
            }
#pragma unroll
            for (int r = 0; r < kMaxDvRegs; r++) {
                const int c = lane + 32 * r;
                if (c < Dv) {
                    float vv[kRows];
#pragma unroll
                    for (int u = 0; u < kRows; u++) vv[u] = to_f32(vrow[u][c]);
#pragma unroll
                    for (int u = 0; u < kRows; u++) acc[r] = fmaf(pj[u], vv[u], acc[r]);
                }
            }
        }
    }
    // the warps' sums, added in warp order
    __syncthreads();
    float *sums = sa_smem + kWarps * Dp;
#pragma unroll
    for (int r = 0; r < kMaxDvRegs; r++) sums[(warp * kMaxDvRegs + r) * 32 + lane] = acc[r];
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int r = 0; r < kMaxDvRegs; r++) {
        float s = 0.f;
        for (int w = 0; w < kWarps; w++) s += sums[(w * kMaxDvRegs + r) * 32 + lane];
        const int c = lane + 32 * r;
        if (gridDim.z > 1) part_out[(((t * H + h) * gridDim.z + blockIdx.z) * kMaxDvRegs + r) * 32 + lane] = s;
        else if (c < Dv) out[(t * H + h) * Dv + c] = from_f32<E>(s);
    }
}

// one warp per (token, head): the splits' sums in split order
template <typename E>
__global__ void __launch_bounds__(32) sigmoid_merge_kernel(const float *__restrict__ part, int n_split, int H, int Dv, E *__restrict__ out) {
    const int64_t t = blockIdx.x;
    const int h = blockIdx.y, lane = threadIdx.x;
    const float *pp = part + ((t * H + h) * n_split) * (kMaxDvRegs * 32);
#pragma unroll
    for (int r = 0; r < kMaxDvRegs; r++) {
        const int c = lane + 32 * r;
        if (c >= Dv) continue;
        float s = 0.f;
        for (int sp = 0; sp < n_split; sp++) s += pp[(sp * kMaxDvRegs + r) * 32 + lane];
        out[(t * H + h) * Dv + c] = from_f32<E>(s);
    }
}

// ---- portions: 32 tokens of one head per CTA, tiles of 32 cache rows staged in shared memory.
// NR: groups of 32 value coordinates a lane accumulates (Dv <= 32 NR).  VEC: rows are staged and K rows read in 16-byte
// pieces; the K pitch kp is then a multiple of 4 words with kp / 4 odd, so that the eight lanes of a quarter warp, a row
// each, cover all 32 banks.
template <typename E, int NR, bool VEC>
__global__ void __launch_bounds__(32 * kWarps) sigmoid_attn_tile_kernel(const float *__restrict__ q, const E *__restrict__ cache, int64_t cache_ld,
                                                                        const int32_t *__restrict__ table, int B, const int32_t *__restrict__ pos0,
                                                                        int64_t T, int H, int G, int D, int Dv, int kp, int vp, int64_t window,
                                                                        const float *__restrict__ r1, const float *__restrict__ r2,
                                                                        const float *__restrict__ pb, E *__restrict__ out) {
    extern __shared__ __align__(16) float sa_smem[];
    __shared__ float pen[64]; // pen[31 + qi - lane]: the penalty of distance (i0 - j0) + qi - lane
    const int Dp = (D + 3) & ~3;
    float *sq = sa_smem;       // [kQT][Dp]
    float *sk = sq + kQT * Dp; // [32][kp]: lane = row reads are conflict-free
    float *sv = sk + 32 * kp;  // [32][vp]: lane = column reads
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y, g = h / (H / G);
    const int64_t t0 = (int64_t)blockIdx.x * kQT;
    const int nq = (int)min((int64_t)kQT, T - t0);
    const int64_t i0 = (int64_t)*pos0 + t0, i_last = i0 + nq - 1;
    for (int e = threadIdx.x; e < kQT * Dp; e += blockDim.x) {
        const int qi = e / Dp, d = e - qi * Dp;
        sq[e] = (qi < nq && d < D) ? q[((t0 + qi) * H + h) * D + d] : 0.f;
    }
    const float hr1 = r1 ? r1[h] : 0.f, hr2 = r2 ? r2[h] : 0.f, hpb = pb ? pb[h] : 0.f;
    const int64_t jlo = window > 0 ? max((int64_t)0, i0 - window + 1) : 0;
    float acc[kQPW][NR];
#pragma unroll
    for (int a = 0; a < kQPW; a++)
#pragma unroll
        for (int r = 0; r < NR; r++) acc[a][r] = 0.f;
    const int64_t koff = (int64_t)g * D, voff = (int64_t)G * D + (int64_t)g * Dv;
    for (int64_t j0 = jlo; j0 <= i_last; j0 += 32) {
        __syncthreads(); // the previous tile has been consumed (and sq is written, the first time)
        const int n_rows = (int)min((int64_t)32, i_last - j0 + 1);
        if (threadIdx.x < 63) pen[threadIdx.x] = penalty_f32(hr1, hr2, i0 - j0 + (int64_t)threadIdx.x - 31);
        for (int rr = warp; rr < 32; rr += kWarps) {
            const int64_t j = j0 + min(rr, n_rows - 1); // a row past the last one repeats it (weight 0 below)
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
                for (int c = lane; c < D + Dv; c += 32) {
                    if (c < D) sk[rr * kp + c] = to_f32(row[koff + c]);
                    else sv[rr * vp + c - D] = to_f32(row[voff + c - D]);
                }
            }
        }
        __syncthreads();
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
            const int qi = warp * kQPW + a;
            const int64_t i = i0 + qi;
            const bool vis = qi < nq && j <= i && (window <= 0 || i - j < window);
            p[a] = vis ? sigmoid_f32(s[a] - pen[31 + qi - lane] + hpb) : 0.f;
        }
#pragma unroll 2
        for (int jj = 0; jj < n_rows; jj++) {
            float pj[kQPW];
#pragma unroll
            for (int a = 0; a < kQPW; a++) pj[a] = __shfl_sync(0xffffffffu, p[a], jj);
#pragma unroll
            for (int r = 0; r < NR; r++) {
                const int c = lane + 32 * r;
                if (c < Dv) {
                    const float vv = sv[jj * vp + c];
#pragma unroll
                    for (int a = 0; a < kQPW; a++) acc[a][r] = fmaf(pj[a], vv, acc[a][r]);
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < kQPW; a++) {
        const int qi = warp * kQPW + a;
        if (qi >= nq) continue;
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const int c = lane + 32 * r;
            if (c < Dv) out[((t0 + qi) * H + h) * Dv + c] = from_f32<E>(acc[a][r]);
        }
    }
}

} // namespace

extern "C" {

int ggb_op_sigmoid_qkv_store(int dt, const float *q, const float *k, const float *v, int64_t ld, int64_t T, int H, int G, int D, int Dv,
                             float temp_coef, int temp_every, float vnorm_eps, float scale, const int32_t *pos0, const int32_t *block_table,
                             int block_size, void *cache, float *q_out) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(dt == GGB_TYPE_BF16 || dt == GGB_TYPE_F32, "sigmoid_qkv_store: dtype %d is neither bf16 nor f32", dt);
    GGB_CHECK_ARG(q && k && v && pos0 && block_table && cache && q_out && T > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && Dv > 0 &&
                      block_size > 0 && temp_every >= 0,
                  "sigmoid_qkv_store: bad arguments");
    const int64_t cld = ggb_window_cache_ld(G, D, Dv);
    if (dt == GGB_TYPE_BF16)
        sigmoid_qkv_store_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>(q, k, v, ld, H, G, D, Dv, temp_coef, temp_every, vnorm_eps, scale, pos0,
                                                                             block_table, block_size, (__nv_bfloat16 *)cache, cld, q_out);
    else
        sigmoid_qkv_store_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>(q, k, v, ld, H, G, D, Dv, temp_coef, temp_every, vnorm_eps, scale, pos0,
                                                                             block_table, block_size, (float *)cache, cld, q_out);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

size_t ggb_sigmoid_attn_scratch_bytes(int H) { return (size_t)(kQT - 1) * (size_t)H * kMaxSplit * kMaxDvRegs * 32 * 4; }

int ggb_op_sigmoid_attn(int dt, const float *q, const void *cache, const int32_t *block_table, int block_size, const int32_t *pos0, int64_t T,
                        int H, int G, int D, int Dv, int64_t window, const float *r1, const float *r2, const float *pb, void *out,
                        float *scratch) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(dt == GGB_TYPE_BF16 || dt == GGB_TYPE_F32, "sigmoid_attn: dtype %d is neither bf16 nor f32", dt);
    GGB_CHECK_ARG(q && cache && block_table && pos0 && out && T > 0 && H > 0 && G > 0 && H % G == 0 && block_size > 0 && D > 0 && Dv > 0 &&
                      Dv <= 32 * kMaxDvRegs && (!r1 == !r2),
                  "sigmoid_attn: bad arguments (value size %d, at most %d)", Dv, 32 * kMaxDvRegs);
    const int64_t cld = ggb_window_cache_ld(G, D, Dv);
    const int Dp = (D + 3) & ~3;
    const int es = dt == GGB_TYPE_BF16 ? 2 : 4, vn = 16 / es;
    // 16-byte pieces: rows start 8 numbers apart at least; a head's keys and values must start on such a piece too
    const int vec = D % vn == 0 && ((int64_t)G * D) % vn == 0 && ((uintptr_t)cache % 16 == 0);
    cudaStream_t st = ggb_cuda_stream();
    if (T >= kQT) {
        const bool tv = vec && Dv % vn == 0;
        int kp = D | 1, vp = Dv;
        if (tv) { // 16-byte pieces: K rows a multiple of 4 words apart with an odd number of pieces, V rows whole pieces
            kp = (D + 3) & ~3;
            if ((kp / 4) % 2 == 0) kp += 4;
            vp = (Dv + 3) & ~3;
        }
        const size_t smem = ((size_t)kQT * Dp + 32 * (size_t)kp + 32 * (size_t)vp) * 4;
        GGB_CHECK_ARG(smem <= 200 * 1024, "sigmoid_attn: head sizes %d / %d do not fit shared memory", D, Dv);
        const dim3 grid((unsigned)((T + kQT - 1) / kQT), (unsigned)H);
#define ST_LAUNCH(ET, NR, VEC)                                                                                                 \
    {                                                                                                                          \
        auto kfn = sigmoid_attn_tile_kernel<ET, NR, VEC>;                                                                      \
        if (smem > 48 * 1024) GGB_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));      \
        kfn<<<grid, 32 * kWarps, smem, st>>>(q, (const ET *)cache, cld, block_table, block_size, pos0, T, H, G, D, Dv, kp, vp, \
                                             window, r1, r2, pb, (ET *)out);                                                   \
    }
#define ST_NR(ET, VEC)                         \
    {                                          \
        if (Dv <= 64) ST_LAUNCH(ET, 2, VEC)    \
        else if (Dv <= 128) ST_LAUNCH(ET, 4, VEC) \
        else ST_LAUNCH(ET, 8, VEC)             \
    }
        if (dt == GGB_TYPE_BF16) {
            if (tv) ST_NR(__nv_bfloat16, true) else ST_NR(__nv_bfloat16, false)
        } else {
            if (tv) ST_NR(float, true) else ST_NR(float, false)
        }
#undef ST_NR
#undef ST_LAUNCH
    } else {
        const size_t smem = (size_t)kWarps * Dp * 4 + (size_t)kWarps * kMaxDvRegs * 32 * 4;
        GGB_CHECK_ARG(smem <= 48 * 1024, "sigmoid_attn: key size %d does not fit shared memory", D);
        // the grid is fixed before the position is known (a captured step): as many splits as the window has groups of 8
        // tiles, half of the most without a window
        int n_split = 1;
        if (scratch && window > 0) n_split = (int)std::min<int64_t>(kMaxSplit, ((window + 62) / 32 + kWarps - 1) / kWarps);
        else if (scratch) n_split = kMaxSplit / 2;
        const dim3 grid((unsigned)T, (unsigned)H, (unsigned)n_split);
#define SS_LAUNCH(ET)                                                                                                                       \
    sigmoid_attn_step_kernel<ET><<<grid, 32 * kWarps, smem, st>>>(q, (const ET *)cache, cld, block_table, block_size, pos0, H, G, D, Dv, window, \
                                                                  r1, r2, pb, (ET *)out, vec, scratch);                                     \
    if (n_split > 1) {                                                                                                                      \
        GGB_LAUNCH_CHECK();                                                                                                                 \
        sigmoid_merge_kernel<ET><<<dim3((unsigned)T, (unsigned)H), 32, 0, st>>>(scratch, n_split, H, Dv, (ET *)out);                         \
    }
        if (dt == GGB_TYPE_BF16) { SS_LAUNCH(__nv_bfloat16) } else { SS_LAUNCH(float) }
#undef SS_LAUNCH
    }
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

} // extern "C"
