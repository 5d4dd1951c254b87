// dense.cu — operators for models whose matrices are plain bf16 / fp32 (row-major [out][in], applied as W x):
// the linear layer in three forms (a streaming mat-vec for a handful of rows, a shared-memory tile kernel for any
// shape, and - bf16, aligned shapes - the tcgen05 GEMM of prefill.cu), RMS norms whose weight is one number or a
// vector, the clamped gated activation, embedding rows, and the residual sum with a per-token side input.
//
// `dt` is the storage type of matrices and of the activations that feed them: GGB_TYPE_BF16 (products of bf16
// values accumulated in fp32) or GGB_TYPE_F32 (everything in true fp32; no TF32 anywhere).  Norms, the residual
// stream and every reduction are fp32 in both.  The file is compiled with -fmad=false, so the fused multiply-adds
// are spelled fmaf().
#include <cuda_bf16.h>

#include "common.cuh"
#include "dense.cuh"

namespace {

// ------------------------------------------------------------------------------------------------ mat-vec
// T <= kVecT activation rows: a warp owns output row n for all of them, streams the weight row once with
// 16-byte loads and keeps T accumulators.  HBM-bound (decode).
constexpr int kVecT = 8;

// ACT 1: the output is relu(.)^2 in the matrices' type (c_act) instead of fp32 (c)
template <typename E, int TT, int ACT = 0>
__global__ void __launch_bounds__(256) linear_vec_kernel(const E *__restrict__ w, int64_t N, int64_t K, const E *__restrict__ a,
                                                         int64_t lda, float *__restrict__ c, int64_t ldc, E *__restrict__ c_act = nullptr) {
    constexpr int VE = 16 / (int)sizeof(E); // elements per 16-byte load
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) acc[t] = 0.f;
    const E *wr = w + n * K;
    const bool vec = (K % VE == 0) && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(a)) % 16 == 0) &&
                     (lda % VE == 0);
    if (vec) {
#pragma unroll 4
        for (int64_t k = (int64_t)lane * VE; k < K; k += 32 * VE) { // several 16-byte loads of the row in flight
            const uint4 wv = ldg_stream_u4(wr + k);
            const E *we = reinterpret_cast<const E *>(&wv);
            float wf[VE];
#pragma unroll
            for (int u = 0; u < VE; u++) wf[u] = to_f32(we[u]);
#pragma unroll
            for (int t = 0; t < TT; t++) {
                const uint4 av = *reinterpret_cast<const uint4 *>(a + t * lda + k);
                const E *ae = reinterpret_cast<const E *>(&av);
#pragma unroll
                for (int u = 0; u < VE; u++) acc[t] = fmaf(wf[u], to_f32(ae[u]), acc[t]);
            }
        }
    } else {
        for (int64_t k = lane; k < K; k += 32) {
            const float wf = to_f32(wr[k]);
#pragma unroll
            for (int t = 0; t < TT; t++) acc[t] = fmaf(wf, to_f32(a[t * lda + k]), acc[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
        const float s = warp_sum_f32(acc[t]);
        if (lane == 0) {
            if (ACT == 1) c_act[t * ldc + n] = from_f32<E>(s > 0.f ? s * s : 0.f);
            else c[t * ldc + n] = s;
        }
    }
}

// ------------------------------------------------------------------------------------------------ tile kernel
// C[T][N] = A[T][K] W[N][K]^T for any shape: 64 x 64 tile of C per CTA, K in steps of 16, 4 x 4 outputs per
// thread, fp32 accumulation in k order.  With `grp` the rows of A / C are the sorted slots of a mixture of experts:
// tile blockIdx.y belongs to expert grp.tile_expert[y], covers sorted rows [row0, row0 + rows), reads its A rows
// through grp.row_src and the expert's matrix w + expert * N * K.
template <typename E, bool GROUPED, int ACT>
__global__ void __launch_bounds__(256) linear_tile_kernel(const E *__restrict__ w, int64_t N, int64_t K, const E *__restrict__ a,
                                                          int64_t lda, int64_t T, float *__restrict__ c, E *__restrict__ c_act,
                                                          int64_t ldc, ggb_moe_groups grp) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float sa[BK][BM + 4], sb[BK][BN + 4];
    int64_t m0 = (int64_t)blockIdx.y * BM, m_end = T;
    if (GROUPED) {
        if ((int)blockIdx.y >= *grp.n_tiles) return;
        const int e = grp.tile_expert[blockIdx.y];
        m0 = grp.tile_row0[blockIdx.y];
        m_end = grp.offsets[e + 1];
        w += (int64_t)e * N * K;
    }
    const int64_t n0 = (int64_t)blockIdx.x * BN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    // loader: thread -> (row r = tid / 4, k quad (tid % 4) * 4) of both tiles
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const int64_t am = m0 + lr;
    const E *arow = nullptr;
    if (am < m_end) arow = a + (GROUPED && grp.row_src ? (int64_t)grp.row_src[am] : am) * lda;
    const E *wrow = n0 + lr < N ? w + (n0 + lr) * K : nullptr;
    for (int64_t k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int64_t k = k0 + lk + u;
            sa[lk + u][lr] = (arow && k < K) ? to_f32(arow[k]) : 0.f;
            sb[lk + u][lr] = (wrow && k < K) ? to_f32(wrow[k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            const float4 av = *reinterpret_cast<const float4 *>(&sa[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4 *>(&sb[kk][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= m_end) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int64_t n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (ACT == 1) { // square of relu, stored in the matrices' type (the next product's operand)
                v = v > 0.f ? v * v : 0.f;
                c_act[m * ldc + n] = from_f32<E>(v);
            } else {
                c[m * ldc + n] = v;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ norms
// y = x / sqrt(mean(x^2) + eps) * w for up to two weights of the SAME x (a layer with two parallel branches norms
// one x twice: the root mean square is computed once).  w_stride 0: the weight is one number; 1: a vector.
template <typename E>
__global__ void __launch_bounds__(256) rms_norm2_kernel(const float *__restrict__ x, int64_t ldx, const float *__restrict__ w1,
                                                        int s1, const float *__restrict__ w2, int s2, float eps, int64_t n,
                                                        E *__restrict__ y1, E *__restrict__ y2) {
    __shared__ float red[8];
    const float *xr = x + (int64_t)blockIdx.x * ldx;
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
    ss = warp_sum_f32(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];
    const float r = 1.0f / sqrtf(tot / (float)n + eps);
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = xr[i] * r;
        if (y1) y1[(int64_t)blockIdx.x * n + i] = from_f32<E>(v * w1[s1 ? i : 0]);
        if (y2) y2[(int64_t)blockIdx.x * n + i] = from_f32<E>(v * w2[s2 ? i : 0]);
    }
}

// rows of x picked by index (the positions whose logits are wanted)
__global__ void gather_rows_kernel(const float *__restrict__ x, const int32_t *__restrict__ rows, int64_t n, float *__restrict__ y) {
    const float *src = x + (int64_t)rows[blockIdx.x] * n;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) y[(int64_t)blockIdx.x * n + i] = src[i];
}

template <typename E>
__global__ void embed_rows_kernel(const E *__restrict__ table, const int32_t *__restrict__ ids, int64_t n, float *__restrict__ y) {
    const E *src = table + (int64_t)ids[blockIdx.x] * n;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) y[(int64_t)blockIdx.x * n + i] = to_f32(src[i]);
}

// g = min(gate, limit), u = clamp(up, -limit, limit); y = g * sigmoid(alpha * g) * (u + 1).  gu rows hold the gate
// half then the up half (one product with the two matrices stacked).
template <typename E>
__global__ void glu_clamp_kernel(const float *__restrict__ gu, int64_t F, int64_t T, float limit, float alpha, E *__restrict__ y) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * F) return;
    const int64_t t = i / F, f = i - t * F;
    const float g = fminf(gu[t * 2 * F + f], limit);
    const float u = fminf(fmaxf(gu[t * 2 * F + F + f], -limit), limit);
    y[i] = from_f32<E>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
}

__device__ __forceinline__ float gelu_tanh_f32(float z) {
    return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
}

// x <- x + a (+ f); then, with a side input, x <- x + rms(y) * nw, y = proj (gelu_tanh(gate x) * e), e = the token's
// slice [e_off, e_off + sd) of its side-embedding row.  A CTA takes TT tokens (x staged in shared memory, fp32) so that
// the two small matrices are read once for all of them; rows are read with 16-byte loads, several in flight.
template <typename E> struct Vec16 {
    static constexpr int n = 16 / (int)sizeof(E);
    uint4 raw;
    __device__ __forceinline__ float at(int i) const { return to_f32(reinterpret_cast<const E *>(&raw)[i]); }
};

template <typename E, int TT>
__global__ void __launch_bounds__(512) residual_side_kernel(float *__restrict__ x, const float *__restrict__ a, const float *__restrict__ f,
                                                            int64_t W, int64_t T, const int32_t *__restrict__ ids,
                                                            const E *__restrict__ side_embed, int64_t e_ld, int64_t e_off, int sd,
                                                            const E *__restrict__ w_gate, const E *__restrict__ w_proj,
                                                            const float *__restrict__ nw, float eps, int vec) {
    extern __shared__ float rs_smem[];
    float *xs = rs_smem, *ys = xs + TT * W, *gs = ys + TT * W; // [TT][W], [TT][W], [TT][sd]
    __shared__ float red[TT][16];
    constexpr int VN = Vec16<E>::n;
    const int64_t t0 = (int64_t)blockIdx.x * TT;
    const int nt = (int)min((int64_t)TT, T - t0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    for (int64_t i = tid; i < (int64_t)TT * W; i += blockDim.x) {
        const int tt = (int)(i / W);
        float v = 0.f;
        if (tt < nt) {
            const int64_t g = t0 * W + i;
            v = x[g] + (f ? a[g] + f[g] : a[g]);
            if (!sd) x[g] = v;
        }
        xs[i] = v;
    }
    if (!sd) return;
    __syncthreads();
    // gate: a warp takes GQ outputs at a time (rows i, i + nwarp, ...): their loads are independent and in flight together;
    // every row of w_gate is read once for the TT tokens
    constexpr int GQ = TT >= 4 ? 2 : 4;
    for (int i0 = warp; i0 < sd; i0 += nwarp * GQ) {
        float s[GQ][TT];
#pragma unroll
        for (int g = 0; g < GQ; g++)
#pragma unroll
            for (int tt = 0; tt < TT; tt++) s[g][tt] = 0.f;
        if (vec) {
#pragma unroll 2
            for (int64_t k = (int64_t)lane * VN; k < W; k += 32 * VN) {
                Vec16<E> v[GQ];
#pragma unroll
                for (int g = 0; g < GQ; g++) {
                    const int i = min(i0 + g * nwarp, sd - 1); // a row past the end repeats the last one; its sum is dropped
                    v[g].raw = *reinterpret_cast<const uint4 *>(w_gate + (int64_t)i * W + k);
                }
#pragma unroll
                for (int u = 0; u < VN; u++)
#pragma unroll
                    for (int tt = 0; tt < TT; tt++) {
                        const float xv = xs[tt * W + k + u];
#pragma unroll
                        for (int g = 0; g < GQ; g++) s[g][tt] = fmaf(v[g].at(u), xv, s[g][tt]);
                    }
            }
        } else {
            for (int64_t k = lane; k < W; k += 32)
#pragma unroll
                for (int g = 0; g < GQ; g++) {
                    const int i = min(i0 + g * nwarp, sd - 1);
                    const float wv = to_f32(w_gate[(int64_t)i * W + k]);
#pragma unroll
                    for (int tt = 0; tt < TT; tt++) s[g][tt] = fmaf(wv, xs[tt * W + k], s[g][tt]);
                }
        }
#pragma unroll
        for (int g = 0; g < GQ; g++) {
            const int i = i0 + g * nwarp;
#pragma unroll
            for (int tt = 0; tt < TT; tt++) {
                const float r = warp_sum_f32(s[g][tt]);
                if (lane == 0 && tt < nt && i < sd)
                    gs[tt * sd + i] = gelu_tanh_f32(r) * to_f32(side_embed[(int64_t)ids[t0 + tt] * e_ld + e_off + i]);
            }
        }
    }
    __syncthreads();
    float ss[TT];
#pragma unroll
    for (int tt = 0; tt < TT; tt++) ss[tt] = 0.f;
    for (int64_t i = tid; i < W; i += blockDim.x) { // proj: a thread per output, its row of sd numbers in 16-byte pieces
        float s[TT];
#pragma unroll
        for (int tt = 0; tt < TT; tt++) s[tt] = 0.f;
        const E *wr = w_proj + i * sd;
        if (vec) {
#pragma unroll 8
            for (int k = 0; k < sd; k += VN) {
                Vec16<E> v;
                v.raw = *reinterpret_cast<const uint4 *>(wr + k);
#pragma unroll
                for (int u = 0; u < VN; u++)
#pragma unroll
                    for (int tt = 0; tt < TT; tt++) s[tt] = fmaf(v.at(u), gs[tt * sd + k + u], s[tt]);
            }
        } else {
            for (int k = 0; k < sd; k++)
#pragma unroll
                for (int tt = 0; tt < TT; tt++) s[tt] = fmaf(to_f32(wr[k]), gs[tt * sd + k], s[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < TT; tt++) {
            ys[tt * W + i] = s[tt];
            ss[tt] = fmaf(s[tt], s[tt], ss[tt]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < TT; tt++) {
        const float r = warp_sum_f32(ss[tt]);
        if (lane == 0) red[tt][warp] = r;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; tt++) {
        float tot = 0.f;
        for (int i = 0; i < nwarp; i++) tot += red[tt][i];
        const float r = 1.0f / sqrtf(tot / (float)W + eps);
        for (int64_t i = tid; i < W; i += blockDim.x) x[(t0 + tt) * W + i] = xs[tt * W + i] + ys[tt * W + i] * r * nw[i];
    }
}

template <typename E>
__global__ void cvt_to_f32_kernel(const E *__restrict__ x, int64_t n, float *__restrict__ y) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = to_f32(x[i]);
}

template <typename E>
int linear_launch(const E *w, int64_t N, int64_t K, const E *a, int64_t lda, int64_t T, float *c, int64_t ldc) {
    cudaStream_t st = ggb_cuda_stream();
    if (T <= kVecT) {
        const dim3 grid((unsigned)((N + 7) / 8));
        switch ((int)T) {
#define VEC_CASE(TT) case TT: linear_vec_kernel<E, TT><<<grid, 256, 0, st>>>(w, N, K, a, lda, c, ldc); break;
            VEC_CASE(1) VEC_CASE(2) VEC_CASE(3) VEC_CASE(4) VEC_CASE(5) VEC_CASE(6) VEC_CASE(7) VEC_CASE(8)
#undef VEC_CASE
        }
    } else {
        const dim3 grid((unsigned)((N + 63) / 64), (unsigned)((T + 63) / 64));
        linear_tile_kernel<E, false, 0><<<grid, 256, 0, st>>>(w, N, K, a, lda, T, c, nullptr, ldc, ggb_moe_groups{});
    }
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

// y (E, [T][N]) = relu(a W^T)^2 in one launch: the mat-vec or the tile kernel with the activation as its epilogue
template <typename E>
int linear_relu2_launch(const E *w, int64_t N, int64_t K, const E *a, int64_t lda, int64_t T, E *y) {
    cudaStream_t st = ggb_cuda_stream();
    if (T <= kVecT) {
        const dim3 grid((unsigned)((N + 7) / 8));
        switch ((int)T) {
#define VEC_CASE(TT) case TT: linear_vec_kernel<E, TT, 1><<<grid, 256, 0, st>>>(w, N, K, a, lda, nullptr, N, y); break;
            VEC_CASE(1) VEC_CASE(2) VEC_CASE(3) VEC_CASE(4) VEC_CASE(5) VEC_CASE(6) VEC_CASE(7) VEC_CASE(8)
#undef VEC_CASE
        }
    } else {
        const dim3 grid((unsigned)((N + 63) / 64), (unsigned)((T + 63) / 64));
        linear_tile_kernel<E, false, 1><<<grid, 256, 0, st>>>(w, N, K, a, lda, T, nullptr, y, N, ggb_moe_groups{});
    }
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

} // namespace

// the grouped form, for moe.cu
int ggb_linear_grouped_launch(int dt, const void *w, int64_t N, int64_t K, const void *a, int64_t lda, int max_tiles, float *c,
                              void *c_act, int64_t ldc, int act, const ggb_moe_groups &grp) {
    cudaStream_t st = ggb_cuda_stream();
    const dim3 grid((unsigned)((N + 63) / 64), (unsigned)max_tiles);
#define GRP_CASE(E)                                                                                                           \
    if (act) linear_tile_kernel<E, true, 1><<<grid, 256, 0, st>>>((const E *)w, N, K, (const E *)a, lda, 0, nullptr, (E *)c_act, ldc, grp); \
    else linear_tile_kernel<E, true, 0><<<grid, 256, 0, st>>>((const E *)w, N, K, (const E *)a, lda, 0, c, nullptr, ldc, grp);
    if (dt == GGB_TYPE_BF16) { GRP_CASE(__nv_bfloat16) } else { GRP_CASE(float) }
#undef GRP_CASE
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

extern "C" {

size_t ggb_dtype_size(int dt) { return dt == GGB_TYPE_BF16 ? 2 : dt == GGB_TYPE_F32 ? 4 : 0; }

#define GGB_CHECK_DT(dt) GGB_CHECK_ARG((dt) == GGB_TYPE_BF16 || (dt) == GGB_TYPE_F32, "dtype %d is neither bf16 nor f32", (int)(dt))

int ggb_op_linear(int dt, const void *w, int64_t N, int64_t K, const void *a, int64_t lda, int64_t T, float *c, int64_t ldc) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(w && a && c && N > 0 && K > 0 && T > 0 && lda >= K && ldc >= N, "linear: bad shape N=%lld K=%lld T=%lld",
                  (long long)N, (long long)K, (long long)T);
    if (dt == GGB_TYPE_BF16) {
        if (ggb_gemm_dense_bf16_fits(N, K, T, ldc) && lda == K)
            return ggb_gemm_dense_bf16(w, N, K, a, T, c, ldc);
        return linear_launch((const __nv_bfloat16 *)w, N, K, (const __nv_bfloat16 *)a, lda, T, c, ldc);
    }
    return linear_launch((const float *)w, N, K, (const float *)a, lda, T, c, ldc);
}

int ggb_op_rms_norm2(int dt, const float *x, int64_t ldx, const float *w1, int w1_stride, const float *w2, int w2_stride, float eps,
                     int64_t E, int64_t T, void *y1, void *y2) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(x && E > 0 && T > 0 && ldx >= E && (!y1 || w1) && (!y2 || w2), "rms_norm2: bad arguments");
    if (dt == GGB_TYPE_BF16)
        rms_norm2_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>(x, ldx, w1, w1_stride, w2, w2_stride, eps, E, (__nv_bfloat16 *)y1,
                                                                     (__nv_bfloat16 *)y2);
    else
        rms_norm2_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>(x, ldx, w1, w1_stride, w2, w2_stride, eps, E, (float *)y1, (float *)y2);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_gather_rows_f32(const float *x, const int32_t *rows, int64_t n_rows, int64_t E, float *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(x && rows && y && n_rows > 0 && E > 0, "gather_rows: bad arguments");
    gather_rows_kernel<<<(unsigned)n_rows, 256, 0, ggb_cuda_stream()>>>(x, rows, E, y);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_embed_rows(int dt, const void *table, const int32_t *ids, int64_t T, int64_t E, float *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(table && ids && y && T > 0 && E > 0, "embed_rows: bad arguments");
    if (dt == GGB_TYPE_BF16) embed_rows_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>((const __nv_bfloat16 *)table, ids, E, y);
    else embed_rows_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>((const float *)table, ids, E, y);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_glu_clamp(int dt, const float *gu, int64_t F, int64_t T, float limit, float alpha, void *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(gu && y && F > 0 && T > 0, "glu_clamp: bad arguments");
    const unsigned blocks = (unsigned)((T * F + 255) / 256);
    if (dt == GGB_TYPE_BF16) glu_clamp_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>(gu, F, T, limit, alpha, (__nv_bfloat16 *)y);
    else glu_clamp_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>(gu, F, T, limit, alpha, (float *)y);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_residual_side(int dt, float *x, const float *a, const float *f, int64_t W, int64_t T, const int32_t *ids, const void *side_embed,
                         int64_t e_ld, int64_t e_off, int sd, const void *w_gate, const void *w_proj, const float *nw, float eps) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(x && a && W > 0 && T > 0 && sd >= 0, "residual_side: bad arguments");
    GGB_CHECK_ARG(!sd || (ids && side_embed && w_gate && w_proj && nw), "residual_side: a side input needs its tensors");
    // tokens per CTA: as many as shared memory holds (up to 8), one when there are too few tokens to fill the GPU
    const size_t per_token = (size_t)(2 * W + sd) * sizeof(float);
    GGB_CHECK_ARG(per_token <= 200 * 1024, "residual_side: width %lld does not fit shared memory", (long long)W);
    int tt = 8;
    while (tt > 1 && (per_token * tt > 96 * 1024 || T < (int64_t)tt * 64)) tt >>= 1;
    const size_t smem = per_token * tt;
    const int vn = dt == GGB_TYPE_BF16 ? 8 : 4;
    const int vec = sd && W % vn == 0 && sd % vn == 0 && ((uintptr_t)w_gate | (uintptr_t)w_proj) % 16 == 0;
    const unsigned grid = (unsigned)((T + tt - 1) / tt);
#define RS_LAUNCH(E, TT)                                                                                                               \
    {                                                                                                                                  \
        auto k = residual_side_kernel<E, TT>;                                                                                          \
        if (smem > 48 * 1024) GGB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                \
        k<<<grid, 512, smem, ggb_cuda_stream()>>>(x, a, f, W, T, ids, (const E *)side_embed, e_ld, e_off, sd, (const E *)w_gate,         \
                                                  (const E *)w_proj, nw, eps, vec);                                                    \
    }
#define RS_CASES(E)                          \
    switch (tt) {                            \
    case 8: RS_LAUNCH(E, 8) break;           \
    case 4: RS_LAUNCH(E, 4) break;           \
    case 2: RS_LAUNCH(E, 2) break;           \
    default: RS_LAUNCH(E, 1) break;          \
    }
    if (dt == GGB_TYPE_BF16) { RS_CASES(__nv_bfloat16) } else { RS_CASES(float) }
#undef RS_CASES
#undef RS_LAUNCH
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_cvt_bf16_f32(const void *x_bf16, int64_t n, float *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(x_bf16 && y && n > 0, "cvt_bf16_f32: bad arguments");
    cvt_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ggb_cuda_stream()>>>((const __nv_bfloat16 *)x_bf16, n, y);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

} // extern "C"

// ------------------------------------------------------------------------------------------------ grouped norms, gates, bigram rows
namespace {

__device__ __forceinline__ float block_sum_256(float v, float *red) { // all threads get the sum; blockDim.x == 256
    v = warp_sum_f32(v);
    __syncthreads(); // `red` may still be read by the previous call
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];
    return tot;
}

// one CTA per token: the embedding row plus the row of the hashed pair (previous token, token)
template <typename E>
__global__ void __launch_bounds__(256) embed_bigram_kernel(const E *__restrict__ table, const E *__restrict__ bigram,
                                                           const int32_t *__restrict__ ids, int64_t T, int64_t n, long long buckets,
                                                           long long mul_prev, long long mul_cur, const int32_t *__restrict__ pos0,
                                                           int32_t *prev_state, float *__restrict__ y) {
    const int64_t t = blockIdx.x;
    const long long id = ids[t];
    const long long prev = t > 0 ? (long long)ids[t - 1] : (long long)*prev_state;
    const long long row = ((long long)*pos0 + t == 0) ? buckets : (prev * mul_prev + id * mul_cur) % buckets;
    const E *e = table + id * n, *b = bigram + row * n;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) y[t * n + i] = to_f32(e[i]) + to_f32(b[i]);
    if (t == 0) { // only this CTA touches the carried token: it has read it above
        __syncthreads();
        if (threadIdx.x == 0) *prev_state = ids[T - 1];
    }
}

// one CTA per token; the row lives in shared memory between the two passes
template <typename E>
__global__ void __launch_bounds__(256) group_norm_add_kernel(const float *__restrict__ a, float sa, const float *__restrict__ b, float sb,
                                                             const float *__restrict__ bias, const float *__restrict__ w, int groups,
                                                             float eps, int64_t n, float *x, E *__restrict__ y) {
    extern __shared__ float gn_row[];
    __shared__ float red[8];
    const int64_t t = blockIdx.x, gs = n / groups;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = sa * a[t * n + i];
        if (b) v += sb * b[t * n + i];
        if (bias) v += bias[i];
        gn_row[i] = v;
    }
    __syncthreads();
    for (int g = 0; g < groups; g++) {
        float ss = 0.f;
        for (int64_t i = threadIdx.x; i < gs; i += blockDim.x) ss = fmaf(gn_row[g * gs + i], gn_row[g * gs + i], ss);
        const float r = 1.0f / sqrtf(block_sum_256(ss, red) / (float)gs + eps);
        for (int64_t i = g * gs + threadIdx.x; i < (g + 1) * gs; i += blockDim.x) {
            float v = gn_row[i] * r * w[i];
            if (x) {
                v += x[t * n + i];
                x[t * n + i] = v;
            }
            if (y) y[t * n + i] = from_f32<E>(v);
        }
    }
}

template <typename E>
__global__ void glu_bias_kernel(const float *__restrict__ gu, int64_t F, int64_t T, const float *__restrict__ bg, const float *__restrict__ bu,
                                int act, E *__restrict__ y) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * F) return;
    const int64_t t = i / F, f = i - t * F;
    float g = gu[t * 2 * F + f], u = gu[t * 2 * F + F + f];
    if (bg) g += bg[f];
    if (bu) u += bu[f];
    if (act == 0) g = fmaxf(g, 0.f);
    else if (act == 1) g = g / (1.0f + expf(-g));
    else g = gelu_tanh_f32(g);
    y[i] = from_f32<E>(g * u);
}

__global__ void softcap_kernel(float *x, int64_t n, float cap) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// a warp (WIDE: a CTA) per (token, group): o / rms(o) * w * act(gate)
template <typename E, bool WIDE>
__global__ void __launch_bounds__(256) norm_gate_kernel(const float *__restrict__ o, int64_t ldo, const float *__restrict__ gate, int64_t ldg,
                                                        int64_t T, int n_groups, int gs, const float *__restrict__ w, int w_period, float eps,
                                                        int act, E *__restrict__ y) {
    __shared__ float red[8];
    const int64_t item = WIDE ? (int64_t)blockIdx.x : (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= T * n_groups) return;
    const int64_t t = item / n_groups;
    const int g = (int)(item - t * n_groups), lane = WIDE ? threadIdx.x : threadIdx.x & 31, step = WIDE ? 256 : 32;
    const float *orow = o + t * ldo + (int64_t)g * gs, *grow = gate + t * ldg + (int64_t)g * gs;
    float ss = 0.f;
    for (int i = lane; i < gs; i += step) ss = fmaf(orow[i], orow[i], ss);
    const float r = 1.0f / sqrtf((WIDE ? block_sum_256(ss, red) : warp_sum_f32(ss)) / (float)gs + eps);
    for (int i = lane; i < gs; i += step) {
        const float z = grow[i];
        const float s = 1.0f / (1.0f + expf(-z));
        y[(t * n_groups + g) * gs + i] = from_f32<E>(orow[i] * r * w[(g * gs + i) % w_period] * (act == 1 ? z * s : s));
    }
}

} // namespace

extern "C" {

int ggb_op_embed_bigram(int dt, const void *table, const void *bigram, const int32_t *ids, int64_t T, int64_t E, int64_t buckets,
                        int64_t mul_prev, int64_t mul_cur, const int32_t *pos0, int32_t *prev_state, float *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(table && bigram && ids && pos0 && prev_state && y && T > 0 && E > 0 && buckets > 0, "embed_bigram: bad arguments");
    if (dt == GGB_TYPE_BF16)
        embed_bigram_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>((const __nv_bfloat16 *)table, (const __nv_bfloat16 *)bigram, ids, T, E,
                                                                        (long long)buckets, (long long)mul_prev, (long long)mul_cur, pos0,
                                                                        prev_state, y);
    else
        embed_bigram_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>((const float *)table, (const float *)bigram, ids, T, E, (long long)buckets,
                                                                        (long long)mul_prev, (long long)mul_cur, pos0, prev_state, y);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_group_norm_add(int dt, const float *a, float sa, const float *b, float sb, const float *bias, const float *w, int groups,
                          float eps, int64_t E, int64_t T, float *x, void *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(a && w && E > 0 && T > 0 && groups > 0 && E % groups == 0 && (x || y), "group_norm_add: bad arguments (width %lld, %d groups)",
                  (long long)E, groups);
    const size_t smem = (size_t)E * 4;
    GGB_CHECK_ARG(smem <= 200 * 1024, "group_norm_add: width %lld does not fit shared memory", (long long)E);
#define GN_LAUNCH(ET)                                                                                                          \
    {                                                                                                                          \
        auto k = group_norm_add_kernel<ET>;                                                                                    \
        if (smem > 48 * 1024) GGB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));        \
        k<<<(unsigned)T, 256, smem, ggb_cuda_stream()>>>(a, sa, b, sb, bias, w, groups, eps, E, x, (ET *)y);                    \
    }
    if (dt == GGB_TYPE_BF16) GN_LAUNCH(__nv_bfloat16) else GN_LAUNCH(float)
#undef GN_LAUNCH
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_glu_bias(int dt, const float *gu, int64_t F, int64_t T, const float *bg, const float *bu, int act, void *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(gu && y && F > 0 && T > 0 && act >= 0 && act <= 2, "glu_bias: bad arguments");
    const unsigned blocks = (unsigned)((T * F + 255) / 256);
    if (dt == GGB_TYPE_BF16) glu_bias_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>(gu, F, T, bg, bu, act, (__nv_bfloat16 *)y);
    else glu_bias_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>(gu, F, T, bg, bu, act, (float *)y);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_softcap(float *x, int64_t n, float cap) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(x && n > 0 && cap > 0.f, "softcap: bad arguments");
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ggb_cuda_stream()>>>(x, n, cap);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_norm_gate(int dt, const float *o, int64_t ldo, const float *gate, int64_t ldg, int64_t T, int n_groups, int gs, const float *w,
                     int w_period, float eps, int act, void *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(o && gate && w && y && T > 0 && n_groups > 0 && gs > 0 && w_period > 0 && ldo >= (int64_t)n_groups * gs &&
                      ldg >= (int64_t)n_groups * gs && (act == 0 || act == 1),
                  "norm_gate: bad arguments");
    const bool wide = gs >= 512; // a long group gets a CTA of its own
    const unsigned blocks = wide ? (unsigned)(T * n_groups) : (unsigned)((T * n_groups + 7) / 8);
#define NG_LAUNCH(ET)                                                                                                                          \
    if (wide) norm_gate_kernel<ET, true><<<blocks, 256, 0, ggb_cuda_stream()>>>(o, ldo, gate, ldg, T, n_groups, gs, w, w_period, eps, act, (ET *)y); \
    else norm_gate_kernel<ET, false><<<blocks, 256, 0, ggb_cuda_stream()>>>(o, ldo, gate, ldg, T, n_groups, gs, w, w_period, eps, act, (ET *)y);
    if (dt == GGB_TYPE_BF16) { NG_LAUNCH(__nv_bfloat16) } else { NG_LAUNCH(float) }
#undef NG_LAUNCH
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

} // extern "C"

// ------------------------------------------------------------------------------------------------ learned positions, norms on both sides of a sublayer
namespace {

__device__ __forceinline__ float block_sum_any(float v, float *red) { // all threads get the sum; blockDim.x a multiple of 32, at most 1024
    v = warp_sum_f32(v);
    __syncthreads(); // `red` may still be read by the previous call
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); i++) tot += red[i];
    return tot;
}

// one CTA per token: the embedding row times `scale` plus the (unscaled) row of the token's position
template <typename E>
__global__ void __launch_bounds__(256) embed_pos_kernel(const E *__restrict__ table, const E *__restrict__ pos_table, const int32_t *__restrict__ ids,
                                                        const int32_t *__restrict__ pos0, int64_t n, float scale, float *__restrict__ y,
                                                        const float *__restrict__ wn, float eps, E *__restrict__ yn) {
    __shared__ float red[8];
    const int64_t t = blockIdx.x;
    const E *e = table + (int64_t)ids[t] * n;
    const E *p = pos_table ? pos_table + ((int64_t)*pos0 + t) * n : nullptr;
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = to_f32(e[i]) * scale;
        if (p) v += to_f32(p[i]);
        y[t * n + i] = v;
        ss = fmaf(v, v, ss);
    }
    if (!yn) return;
    // the first layer's norm on the way out: a thread reads back what it wrote itself
    const float r = 1.0f / sqrtf(block_sum_256(ss, red) / (float)n + eps);
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) yn[t * n + i] = from_f32<E>(y[t * n + i] * r * wn[i]);
}

// one CTA per token: x += (a + bias) / rms(a + bias) * wa, then y = x / rms(x) * wy.  The row stays in shared memory
// between the passes; both root mean squares and the sum are fp32.
constexpr int kMaxCombine = GGB_MOE_COMBINE_NORM_MAX_TOP;
// With inv / wt the sublayer's output is gathered on the way in: v = sum_k wt[t][k] a[inv[t][k]] over the `top` expert
// slots of the token, added in slot order (what moe_combine_kernel computes).
template <typename E>
__global__ void __launch_bounds__(1024) norm_add_norm_kernel(const float *__restrict__ a, const float *__restrict__ bias,
                                                            const int32_t *__restrict__ inv, const float *__restrict__ wt, int top,
                                                            const float *__restrict__ wa, float eps, int64_t n, float *x,
                                                            const float *__restrict__ wy, E *__restrict__ y) {
    extern __shared__ float nn_row[];
    __shared__ float red[32];
    __shared__ float s_wt[kMaxCombine];
    __shared__ int64_t s_off[kMaxCombine];
    const int64_t t = blockIdx.x;
    if (inv) { // the token's slots, looked up once: the loads below then depend on nothing
        if ((int)threadIdx.x < top) {
            s_wt[threadIdx.x] = wt[t * top + threadIdx.x];
            s_off[threadIdx.x] = (int64_t)inv[t * top + threadIdx.x] * n;
        }
        __syncthreads();
    }
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v;
        if (inv) {
            v = 0.f;
#pragma unroll 4
            for (int k = 0; k < top; k++) v = fmaf(s_wt[k], a[s_off[k] + i], v);
        } else {
            v = a[t * n + i];
        }
        if (bias) v += bias[i];
        nn_row[i] = v;
        ss = fmaf(v, v, ss);
    }
    const float ra = 1.0f / sqrtf(block_sum_any(ss, red) / (float)n + eps);
    ss = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { // a thread reads back what it wrote itself
        const float v = x[t * n + i] + nn_row[i] * ra * wa[i];
        x[t * n + i] = v;
        nn_row[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (!y) return;
    const float rx = 1.0f / sqrtf(block_sum_any(ss, red) / (float)n + eps);
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) y[t * n + i] = from_f32<E>(nn_row[i] * rx * wy[i]);
}

} // namespace

extern "C" {

int ggb_op_embed_pos(int dt, const void *table, const void *pos_table, const int32_t *ids, const int32_t *pos0, int64_t T, int64_t E,
                     float scale, float *y, const float *wn, float eps, void *yn) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(table && ids && y && T > 0 && E > 0 && (!pos_table || pos0) && (!yn || wn), "embed_pos: bad arguments");
    if (dt == GGB_TYPE_BF16)
        embed_pos_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>((const __nv_bfloat16 *)table, (const __nv_bfloat16 *)pos_table, ids, pos0, E,
                                                                     scale, y, wn, eps, (__nv_bfloat16 *)yn);
    else
        embed_pos_kernel<<<(unsigned)T, 256, 0, ggb_cuda_stream()>>>((const float *)table, (const float *)pos_table, ids, pos0, E, scale, y, wn, eps,
                                                                     (float *)yn);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_norm_add_norm(int dt, const float *a, const float *bias, const float *wa, float eps, int64_t E, int64_t T, float *x,
                         const float *wy, void *y) {
    return ggb_norm_add_norm_launch(dt, a, bias, nullptr, nullptr, 0, wa, eps, E, T, x, wy, y);
}

} // extern "C"

int ggb_norm_add_norm_launch(int dt, const float *a, const float *bias, const int32_t *inv, const float *wt, int top, const float *wa, float eps,
                             int64_t E, int64_t T, float *x, const float *wy, void *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(a && wa && x && E > 0 && T > 0 && (!y || wy) && (!inv || (wt && top > 0 && top <= kMaxCombine)), "norm_add_norm: bad arguments");
    const size_t smem = (size_t)E * 4;
    GGB_CHECK_ARG(smem <= 200 * 1024, "norm_add_norm: width %lld does not fit shared memory", (long long)E);
    // a step of few tokens is a chain of latencies on a nearly empty GPU: a wide CTA shortens every pass over the row
    const unsigned threads = T <= 64 && E >= 2048 ? 1024 : T <= 64 && E >= 1024 ? 512 : 256;
#define NN_LAUNCH(ET)                                                                                                         \
    {                                                                                                                          \
        auto k = norm_add_norm_kernel<ET>;                                                                                     \
        if (smem > 48 * 1024) GGB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));        \
        k<<<(unsigned)T, threads, smem, ggb_cuda_stream()>>>(a, bias, inv, wt, top, wa, eps, E, x, wy, (ET *)y);                                  \
    }
    if (dt == GGB_TYPE_BF16) NN_LAUNCH(__nv_bfloat16) else NN_LAUNCH(float)
#undef NN_LAUNCH
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

// ------------------------------------------------------------------------------------------------ several residual streams, plain activations
namespace {

constexpr int kMaxStreams = 16;
constexpr int kMaxHyperTop = 64;

// a sublayer's output that is still the slot rows of a mixture of experts: y[t] = sum_k wt[t][k] (slot k's row of y2, or the
// token's row of h_in where the slot's expert is an identity expert: idx >= n_real)
template <typename E> struct hyper_slots {
    const float *y2 = nullptr;
    const int32_t *inv = nullptr, *idx = nullptr;
    const float *wt = nullptr;
    int top = 0, n_real = 0;
    const E *h_in = nullptr; // may be the buffer h is written to: a thread reads its columns before it writes them
};

// One CTA per row.  The residual is S streams x_1 .. x_S per token ([T][S][W] fp32).  In one pass over the token's columns:
//   x0:   every stream starts as the row of x0 (the embedding output) instead of what xs holds
//   y:    the sublayer's output enters, all streams at once from the old ones: x_t <- sum_s mix[s][t] x_s + coef[t] y
//         (or sl: the output is summed from its expert slots on the way in)
//   in_w: u = sum_s in_w[s] x_s is read out, as fp32 (u_out) and / or normed, u / sqrt(mean(u^2) + eps) * nw, in dt (h)
// With `rows` the CTA's token is rows[blockIdx.x] and nothing is written back to xs (a few rows read out at the end: what y
// brings enters on the way).
template <typename E, int SM, int V, int TB>
__global__ void __launch_bounds__(TB) hyper_mix_kernel(float *xs, const float *__restrict__ x0, const float *__restrict__ y,
                                                        const float *__restrict__ mix, const float *__restrict__ coef, int S,
                                                        const float *__restrict__ in_w, const float *__restrict__ nw, float eps, int64_t W,
                                                        const int32_t *__restrict__ rows, float *__restrict__ u_out, E *h, hyper_slots<E> sl) {
    extern __shared__ __align__(16) float hm_row[]; // [W] the read-out u
    __shared__ float red[32], s_mix[SM * SM], s_coef[SM], s_in[SM], s_wt[kMaxHyperTop];
    __shared__ int64_t s_row[kMaxHyperTop];
    const int64_t b = blockIdx.x, t = rows ? rows[b] : b;
    const bool renew = y || sl.y2;
    if (sl.y2 && (int)threadIdx.x < sl.top) { // the token's slots, looked up once
        const int64_t k = t * sl.top + threadIdx.x;
        s_wt[threadIdx.x] = sl.wt[k];
        s_row[threadIdx.x] = sl.idx[k] < sl.n_real ? (int64_t)sl.inv[k] * W : -1;
    }
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[(i / S) * SM + i % S] = mix ? mix[i] : 0.f;
    if ((int)threadIdx.x < S) {
        s_coef[threadIdx.x] = coef ? coef[threadIdx.x] : 0.f;
        s_in[threadIdx.x] = in_w ? in_w[threadIdx.x] : 0.f;
    }
    __syncthreads();
    float *xr = xs + t * S * W;
    float ss = 0.f;
    // V columns a thread and step (V = 4: 16-byte loads and stores, all of a column group's streams in flight together)
    for (int64_t i = (int64_t)threadIdx.x * V; i < W; i += (int64_t)blockDim.x * V) {
        float x[SM][V], yv[V];
#pragma unroll
        for (int s = 0; s < SM; s++) {
            if (s < S) {
                const float *src = x0 ? x0 + t * W + i : xr + s * W + i;
                if (V == 4) {
                    const float4 v4 = *reinterpret_cast<const float4 *>(src);
                    x[s][0] = v4.x, x[s][1 % V] = v4.y, x[s][2 % V] = v4.z, x[s][3 % V] = v4.w;
                } else {
                    x[s][0] = src[0];
                }
            } else {
#pragma unroll
                for (int c = 0; c < V; c++) x[s][c] = 0.f;
            }
        }
        if (renew) {
            if (sl.y2) {
#pragma unroll
                for (int c = 0; c < V; c++) yv[c] = 0.f;
                for (int k = 0; k < sl.top; k++) {
                    const float w = s_wt[k];
                    float sv[V];
                    if (s_row[k] >= 0) {
                        const float *src = sl.y2 + s_row[k] + i;
                        if (V == 4) {
                            const float4 v4 = *reinterpret_cast<const float4 *>(src);
                            sv[0] = v4.x, sv[1 % V] = v4.y, sv[2 % V] = v4.z, sv[3 % V] = v4.w;
                        } else {
                            sv[0] = src[0];
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < V; c++) sv[c] = to_f32(sl.h_in[t * W + i + c]);
                    }
#pragma unroll
                    for (int c = 0; c < V; c++) yv[c] = fmaf(w, sv[c], yv[c]);
                }
            } else if (V == 4) {
                const float4 v4 = *reinterpret_cast<const float4 *>(y + t * W + i);
                yv[0] = v4.x, yv[1 % V] = v4.y, yv[2 % V] = v4.z, yv[3 % V] = v4.w;
            } else {
                yv[0] = y[t * W + i];
            }
            float n[SM][V];
#pragma unroll
            for (int d = 0; d < SM; d++)
#pragma unroll
                for (int c = 0; c < V; c++) {
                    float a = 0.f;
#pragma unroll
                    for (int s = 0; s < SM; s++)
                        if (s < S) a = fmaf(s_mix[s * SM + d], x[s][c], a);
                    n[d][c] = fmaf(s_coef[d], yv[c], a);
                }
#pragma unroll
            for (int s = 0; s < SM; s++)
#pragma unroll
                for (int c = 0; c < V; c++) x[s][c] = n[s][c];
        }
        if ((renew || x0) && !rows) {
#pragma unroll
            for (int s = 0; s < SM; s++)
                if (s < S) {
                    if (V == 4) *reinterpret_cast<float4 *>(xr + s * W + i) = make_float4(x[s][0], x[s][1 % V], x[s][2 % V], x[s][3 % V]);
                    else xr[s * W + i] = x[s][0];
                }
        }
        if (in_w) {
#pragma unroll
            for (int c = 0; c < V; c++) {
                float u = 0.f;
#pragma unroll
                for (int s = 0; s < SM; s++)
                    if (s < S) u = fmaf(s_in[s], x[s][c], u);
                if (u_out) u_out[b * W + i + c] = u;
                if (h) {
                    hm_row[i + c] = u;
                    ss = fmaf(u, u, ss);
                }
            }
        }
    }
    if (!h) return;
    const float r = 1.0f / sqrtf(block_sum_any(ss, red) / (float)W + eps);
    for (int64_t i = (int64_t)threadIdx.x * V; i < W; i += (int64_t)blockDim.x * V) // a thread reads what it wrote
#pragma unroll
        for (int c = 0; c < V; c++) h[b * W + i + c] = from_f32<E>(hm_row[i + c] * r * nw[i + c]);
}

// y (dt, dense [T][F]) = act(x) for fp32 rows of stride ldx; act 0: as it is, 1: the square of relu
template <typename E>
__global__ void act_rows_kernel(const float *__restrict__ x, int64_t ldx, int64_t T, int64_t F, int act, E *__restrict__ y) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * F) return;
    const int64_t t = i / F, f = i - t * F;
    float v = x[t * ldx + f];
    if (act == 1) v = v > 0.f ? v * v : 0.f;
    y[i] = from_f32<E>(v);
}

} // namespace

extern "C" {

static int hyper_mix_launch(int dt, float *xs, const float *x0, const float *y, const float *y2, const int32_t *inv, const float *wt, const int32_t *idx,
                            int top, int n_real, const void *h_in, const float *mix, const float *coef, int S, const float *in_w, const float *nw,
                            float eps, int64_t W, int64_t T, const int32_t *rows, float *u_out, void *h) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(xs && W > 0 && T > 0 && S > 0 && S <= kMaxStreams, "hyper_mix: bad arguments (%d streams, at most %d)", S, kMaxStreams);
    GGB_CHECK_ARG((!(y || y2) || (mix && coef)) && (!(u_out || h) || in_w) && (!h || nw) && !(y && y2), "hyper_mix: an input without its weights");
    GGB_CHECK_ARG(!y2 || (inv && wt && idx && h_in && top > 0 && top <= kMaxHyperTop), "hyper_mix: expert slots without their lists (at most %d a token)", kMaxHyperTop);
    const size_t smem = h ? (size_t)W * 4 : 0;
    GGB_CHECK_ARG(smem <= 200 * 1024, "hyper_mix: width %lld does not fit shared memory", (long long)W);
    // 16-byte pieces need rows that start on one (up to 4 streams: the wider forms keep the registers of one column)
    const bool vec = W % 4 == 0 && S <= 4 && (((uintptr_t)xs | (uintptr_t)x0 | (uintptr_t)y | (uintptr_t)y2) & 15) == 0;
    // a step of few tokens is a chain of latencies on a nearly empty GPU: a wide CTA covers the row in one pass
    const int64_t per_pass = W / (vec ? 4 : 1);
    const bool wide = T <= 64 && per_pass >= 512 && S <= 4; // 512 threads: these forms keep their registers
#define HM_LAUNCH_V(ET, SM, V)                                                                                                \
    {                                                                                                                          \
        hyper_slots<ET> sl;                                                                                                    \
        sl.y2 = y2, sl.inv = inv, sl.idx = idx, sl.wt = wt, sl.top = top, sl.n_real = n_real, sl.h_in = (const ET *)h_in;       \
        auto k = hyper_mix_kernel<ET, SM, V, 256>;                                                                             \
        if (SM <= 4 && wide) k = hyper_mix_kernel<ET, (SM <= 4 ? SM : 4), V, 512>;                                             \
        if (smem > 48 * 1024) GGB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));        \
        k<<<(unsigned)T, wide ? 512 : 256, smem, ggb_cuda_stream()>>>(xs, x0, y, mix, coef, S, in_w, nw, eps, W, rows, u_out, (ET *)h, sl); \
    }
#define HM_LAUNCH(ET, SM)                       \
    {                                           \
        if (vec && SM <= 4) HM_LAUNCH_V(ET, (SM <= 4 ? SM : 4), 4) \
        else HM_LAUNCH_V(ET, SM, 1)             \
    }
#define HM_S(ET)                              \
    {                                         \
        if (S == 1) HM_LAUNCH(ET, 1)          \
        else if (S == 2) HM_LAUNCH(ET, 2)     \
        else if (S <= 4) HM_LAUNCH(ET, 4)     \
        else if (S <= 8) HM_LAUNCH(ET, 8)     \
        else HM_LAUNCH(ET, 16)                \
    }
    if (dt == GGB_TYPE_BF16) HM_S(__nv_bfloat16) else HM_S(float)
#undef HM_S
#undef HM_LAUNCH
#undef HM_LAUNCH_V
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_hyper_mix(int dt, float *xs, const float *x0, const float *y, const float *mix, const float *coef, int S, const float *in_w,
                     const float *nw, float eps, int64_t W, int64_t T, const int32_t *rows, float *u_out, void *h) {
    return hyper_mix_launch(dt, xs, x0, y, nullptr, nullptr, nullptr, nullptr, 0, 0, nullptr, mix, coef, S, in_w, nw, eps, W, T, rows, u_out, h);
}

int ggb_op_hyper_mix_moe(int dt, float *xs, const float *y2, const int32_t *ws, const float *wt, const int32_t *idx, int64_t T_slots, int top, int n_exp,
                         int n_identity, const void *h_in, const float *mix, const float *coef, int S, const float *in_w, const float *nw, float eps,
                         int64_t W, int64_t T, const int32_t *rows, float *u_out, void *h) {
    GGB_CHECK_ARG(ws && top > 0 && n_exp > 0 && n_identity >= 0 && n_identity <= n_exp && T_slots >= T, "hyper_mix_moe: bad arguments");
    return hyper_mix_launch(dt, xs, nullptr, nullptr, y2, ws + n_exp + 1 + T_slots * top, wt, idx, top, n_exp - n_identity, h_in, mix, coef, S, in_w, nw, eps, W, T,
                            rows, u_out, h);
}

int ggb_op_linear_relu2(int dt, const void *w, int64_t N, int64_t K, const void *a, int64_t lda, int64_t T, float *scratch, void *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(w && a && y && N > 0 && K > 0 && T > 0 && lda >= K, "linear_relu2: bad shape N=%lld K=%lld T=%lld", (long long)N, (long long)K, (long long)T);
    // shapes the tensor cores take: the product into scratch, then the activation; every other shape in one launch
    if (dt == GGB_TYPE_BF16 && scratch && lda == K && ggb_gemm_dense_bf16_fits(N, K, T, N)) {
        const int rc = ggb_gemm_dense_bf16(w, N, K, a, T, scratch, N);
        return rc ? rc : ggb_op_act_rows(dt, scratch, N, T, N, 1, y);
    }
    if (dt == GGB_TYPE_BF16) return linear_relu2_launch((const __nv_bfloat16 *)w, N, K, (const __nv_bfloat16 *)a, lda, T, (__nv_bfloat16 *)y);
    return linear_relu2_launch((const float *)w, N, K, (const float *)a, lda, T, (float *)y);
}

int ggb_op_act_rows(int dt, const float *x, int64_t ldx, int64_t T, int64_t F, int act, void *y) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_DT(dt);
    GGB_CHECK_ARG(x && y && T > 0 && F > 0 && ldx >= F && (act == 0 || act == 1), "act_rows: bad arguments");
    const unsigned blocks = (unsigned)((T * F + 255) / 256);
    if (dt == GGB_TYPE_BF16) act_rows_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>(x, ldx, T, F, act, (__nv_bfloat16 *)y);
    else act_rows_kernel<<<blocks, 256, 0, ggb_cuda_stream()>>>(x, ldx, T, F, act, (float *)y);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

} // extern "C"
