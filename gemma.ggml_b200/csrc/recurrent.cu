// recurrent.cu — mixers whose memory is a fixed-size state instead of a row per position: the causal convolution over
// time with a carried tail, lightning attention (a decayed sum of outer products) and the gated delta rule.  All state
// is fp32 and lives in the caller's per-sequence block; a portion of T tokens continues from the state the previous
// portion left and leaves its own, so a prompt may be cut anywhere.
//
// The two recurrences share one kernel: a CTA owns one head and a slice of CV (16 or 32) value columns (columns are independent
// in both rules), NS lanes share a column and each keeps D / NS numbers of it in registers for the whole portion.
// Per token the lanes' partial sums meet through two shuffles.  Tokens are staged through shared memory in chunks by
// four more warps, one chunk ahead of the recurrence; the staging pass also does what is per token and parallel:
// activations, unit norms, decay and step size.
//
// Compiled with -fmad=false: multiply-adds are spelled fmaf().
#include <algorithm>

#include "common.cuh"
#include "dense.cuh"

namespace {

// __frcp_rn: the correctly rounded reciprocal, one instruction sequence without the slow path of the precise division
__device__ __forceinline__ float silu_f32(float z) { return z * __frcp_rn(1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f32(float z) { return __frcp_rn(1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f32(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------------------------------------ causal convolution
constexpr int kConvMaxTaps = 8, kConvTokens = 32;

// grid (channel blocks, token chunks); a thread owns one channel of one chunk and slides a window of taps inputs along
// it.  Chunk 0 is the only reader of the old tail and its only writer (after it has the old values in registers).
template <typename E>
__global__ void __launch_bounds__(128) causal_conv_kernel(const float *__restrict__ x, int64_t ldx, int64_t T, int64_t C,
                                                          const float *__restrict__ w, const float *__restrict__ bias, int taps, int add_input,
                                                          int act, float *tail, float *__restrict__ y_f32, int64_t ldy, E *__restrict__ y_dt) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float xb = bias ? bias[c] : 0.f; // the input is x + bias; the tail keeps it so
    const int64_t t0 = (int64_t)blockIdx.y * kConvTokens, t1 = min(T, t0 + kConvTokens);
    const int nt = taps - 1;
    float wt[kConvMaxTaps], win[kConvMaxTaps], old[kConvMaxTaps];
#pragma unroll
    for (int j = 0; j < kConvMaxTaps; j++) {
        wt[j] = j < taps ? w[c * taps + j] : 0.f;
        win[j] = 0.f;
        old[j] = 0.f;
    }
    if (blockIdx.y == 0)
#pragma unroll
        for (int j = 0; j < kConvMaxTaps - 1; j++)
            if (j < nt) old[j] = tail[(int64_t)j * C + c];
    // win[j], j < taps - 1: the inputs at t0 - (taps - 1) + j
#pragma unroll
    for (int j = 0; j < kConvMaxTaps - 1; j++)
        if (j < nt) {
            const int64_t s = t0 - nt + j;
            win[j] = s >= 0 ? x[s * ldx + c] + xb : old[j]; // s < 0 only in chunk 0, where s + nt = j indexes the old tail
        }
    for (int64_t t = t0; t < t1; t++) {
        const float xv = x[t * ldx + c] + xb;
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < kConvMaxTaps - 1; j++)
            if (j < nt) acc = fmaf(wt[j], win[j], acc);
        acc = fmaf(wt[nt], xv, acc);
        if (add_input) acc += xv;
        if (act) acc = silu_f32(acc);
        if (y_f32) y_f32[t * ldy + c] = acc;
        if (y_dt) y_dt[t * C + c] = from_f32<E>(acc);
#pragma unroll
        for (int j = 0; j < kConvMaxTaps - 2; j++)
            if (j + 1 < nt) win[j] = win[j + 1];
        if (nt > 0) {
#pragma unroll
            for (int j = 0; j < kConvMaxTaps - 1; j++)
                if (j == nt - 1) win[j] = xv;
        }
    }
    if (blockIdx.y == 0) { // new tail: the last taps - 1 inputs of (old tail, x)
#pragma unroll
        for (int j = 0; j < kConvMaxTaps - 1; j++)
            if (j < nt) {
                const int64_t s = T - nt + j;
                float v = 0.f;
                if (s >= 0) v = x[s * ldx + c] + xb;
                else {
#pragma unroll
                    for (int i = 0; i < kConvMaxTaps - 1; i++)
                        if (i == (int)(s + nt)) v = old[i];
                }
                tail[(int64_t)j * C + c] = v;
            }
    }
}

// ------------------------------------------------------------------------------------------------ the recurrences
constexpr int kNS = 4;      // lanes that share a column of S
constexpr int kStageWarps = 4; // warps that stage the next chunk
constexpr int kChunk = 16;  // tokens staged at once

struct rec_args {
    const float *q, *k, *v, *b, *a;
    int64_t ld, ld_b, ld_a, T;
    int H, G, D, Dv;
    const float *decay, *A_log, *dt_bias;
    float *state, *o;
    int64_t ldo;
    int decays; // MODE 2: `a` holds the decays themselves, not the raw rows they are computed from
};

// MODE 0: lightning (q, k, v = silu of the raw rows; S <- decay S + k v^T; o = S^T q)
// MODE 1: gated delta rule (unit q and k, q * D^-1/2; S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q)
// MODE 2: the same rule with one decay per head and key channel: row d of S is multiplied by g[d]; the decays of a
//         token are staged like a q / k row
//
// CV * 4 threads run the recurrence on the chunk in one buffer while four more warps stage the next chunk into
// the other (global loads of a warp's four tokens in flight together), one barrier per chunk.
// A lane's slice of a q / k row starts DS + 4 words after its neighbour's: the four 16-byte reads of a warp fall into
// four different groups of banks (DS alone is a multiple of 8 words: all four would meet in one).
template <int DS, int CV, bool CH = false>
struct rec_smem {
    static constexpr int DP = DS * kNS;        // padded D
    static constexpr int DW = (DS + 4) * kNS;  // words of a staged row
    __device__ static __forceinline__ int at(int d) { return (d / DS) * (DS + 4) + d % DS; }
    float q[kChunk][DW], k[kChunk][DW];
    float v[kChunk][CV], g[kChunk], beta[kChunk];
    float gc[kChunk][CH ? DW : 1]; // per-channel decays
};

template <int DS, int CV, int MODE>
__device__ __forceinline__ void rec_stage(const rec_args &p, rec_smem<DS, CV, MODE == 2> &b, int64_t t0, int n, int h, int hk, int col0, int pw, int lane, float a_rate,
                                          float dtb, float q_scale) {
    constexpr int DP = DS * kNS, PL = (DP + 31) / 32, TPW = kChunk / kStageWarps; // numbers per lane and row, tokens per producer warp
    float qv[TPW][PL], kv[TPW][PL], vv[TPW], bb[TPW], aa[TPW];
    float av[MODE == 2 ? TPW : 1][MODE == 2 ? PL : 1];
#pragma unroll
    for (int u = 0; u < TPW; u++) {
        const int tt = pw + kStageWarps * u;
        const int64_t t = t0 + min(tt, n - 1); // past the chunk's end: the last token again, not stored
        const float *qr = p.q + t * p.ld + (int64_t)hk * p.D, *kr = p.k + t * p.ld + (int64_t)hk * p.D;
#pragma unroll
        for (int i = 0; i < PL; i++) {
            const int d = lane + 32 * i;
            qv[u][i] = d < p.D ? qr[d] : 0.f;
            kv[u][i] = d < p.D ? kr[d] : 0.f;
        }
        vv[u] = (lane < CV && col0 + lane < p.Dv) ? p.v[t * p.ld + (int64_t)h * p.Dv + col0 + lane] : 0.f;
        if (MODE == 1) {
            bb[u] = p.b[t * p.ld_b + h];
            aa[u] = p.a[t * p.ld_a + h];
        }
        if (MODE == 2) {
            bb[u] = p.b[t * p.ld_b + h];
            const float *ar = p.a + t * p.ld_a + (int64_t)h * p.D;
#pragma unroll
            for (int i = 0; i < PL; i++) {
                const int d = lane + 32 * i;
                av[u][i] = d < p.D ? ar[d] : 0.f;
            }
        }
    }
#pragma unroll
    for (int u = 0; u < TPW; u++) {
        const int tt = pw + kStageWarps * u;
        if (tt >= n) continue;
        float qm = 1.f, km = 1.f;
        if (MODE == 0) {
#pragma unroll
            for (int i = 0; i < PL; i++) {
                qv[u][i] = silu_f32(qv[u][i]); // silu(0) = 0: the padding stays zero
                kv[u][i] = silu_f32(kv[u][i]);
            }
            vv[u] = silu_f32(vv[u]);
        } else {
            float qs = 0.f, ks = 0.f;
#pragma unroll
            for (int i = 0; i < PL; i++) {
                qs = fmaf(qv[u][i], qv[u][i], qs);
                ks = fmaf(kv[u][i], kv[u][i], ks);
            }
            qs = warp_sum_f32(qs);
            ks = warp_sum_f32(ks);
            qm = q_scale / sqrtf(qs + 1e-6f);
            km = 1.0f / sqrtf(ks + 1e-6f);
            if (lane == 0) {
                b.beta[tt] = sigmoid_f32(bb[u]);
                if (MODE == 1) b.g[tt] = expf(-a_rate * softplus_f32(aa[u] + dtb));
            }
            if (MODE == 2) {
#pragma unroll
                for (int i = 0; i < PL; i++) {
                    const int d = lane + 32 * i;
                    if (d < DP) // rows of the padding hold zeros and stay zero
                        b.gc[tt][rec_smem<DS, CV, true>::at(d)] =
                            d >= p.D ? 1.f : p.decays ? av[u][i] : expf(-a_rate * softplus_f32(av[u][i] + p.dt_bias[(int64_t)h * p.D + d]));
                }
            }
        }
#pragma unroll
        for (int i = 0; i < PL; i++) {
            const int d = lane + 32 * i;
            if (d < DP) {
                b.q[tt][rec_smem<DS, CV, MODE == 2>::at(d)] = qv[u][i] * qm;
                b.k[tt][rec_smem<DS, CV, MODE == 2>::at(d)] = kv[u][i] * km;
            }
        }
        if (lane < CV) b.v[tt][lane] = vv[u];
    }
}

template <int DS, int CV, int MODE>
__global__ void __launch_bounds__(CV *kNS + 32 * kStageWarps) recurrence_kernel(rec_args p) {
    extern __shared__ __align__(16) unsigned char rec_raw[];
    typedef rec_smem<DS, CV, MODE == 2> smem_t;
    smem_t *buf = reinterpret_cast<smem_t *>(rec_raw);
    const int h = blockIdx.x, col0 = blockIdx.y * CV;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool producer = warp >= (CV * kNS) / 32;
    const int s = tid % kNS, cl = (tid / kNS) % CV, col = col0 + cl;
    const bool live = !producer && col < p.Dv;
    const int hk = MODE != 0 ? h / (p.H / p.G) : h; // the q / k head this head reads
    float S[DS];
    float *sp = p.state + ((int64_t)h * p.D) * p.Dv + col;
#pragma unroll
    for (int i = 0; i < DS; i++) {
        const int d = s * DS + i;
        S[i] = (live && d < p.D) ? sp[(int64_t)d * p.Dv] : 0.f;
    }
    const float decay = MODE == 0 ? p.decay[h] : 0.f;
    const float a_rate = MODE == 1 || (MODE == 2 && !p.decays) ? expf(p.A_log[h]) : 0.f, dtb = MODE == 1 ? p.dt_bias[h] : 0.f;
    const float q_scale = 1.0f / sqrtf((float)p.D);
    const int pw = warp - (CV * kNS) / 32;
    if (producer) rec_stage<DS, CV, MODE>(p, buf[0], 0, (int)min((int64_t)kChunk, p.T), h, hk, col0, pw, lane, a_rate, dtb, q_scale);
    __syncthreads();
    int cur = 0;
    for (int64_t t0 = 0; t0 < p.T; t0 += kChunk, cur ^= 1) {
        const int n = (int)min((int64_t)kChunk, p.T - t0);
        if (producer) {
            if (t0 + kChunk < p.T)
                rec_stage<DS, CV, MODE>(p, buf[cur ^ 1], t0 + kChunk, (int)min((int64_t)kChunk, p.T - t0 - kChunk), h, hk, col0, pw, lane, a_rate, dtb, q_scale);
        } else {
            const smem_t &b = buf[cur];
            for (int tt = 0; tt < n; tt++) {
                const float4 *k4 = reinterpret_cast<const float4 *>(&b.k[tt][s * (DS + 4)]);
                const float4 *q4 = reinterpret_cast<const float4 *>(&b.q[tt][s * (DS + 4)]);
                float o0 = 0.f, o1 = 0.f;
                if (MODE == 0) {
                    const float vj = b.v[tt][cl];
#pragma unroll
                    for (int i = 0; i < DS / 4; i++) {
                        const float4 kk = k4[i], qq = q4[i];
                        S[4 * i + 0] = fmaf(kk.x, vj, decay * S[4 * i + 0]);
                        S[4 * i + 1] = fmaf(kk.y, vj, decay * S[4 * i + 1]);
                        S[4 * i + 2] = fmaf(kk.z, vj, decay * S[4 * i + 2]);
                        S[4 * i + 3] = fmaf(kk.w, vj, decay * S[4 * i + 3]);
                        o0 = fmaf(S[4 * i + 0], qq.x, o0);
                        o1 = fmaf(S[4 * i + 1], qq.y, o1);
                        o0 = fmaf(S[4 * i + 2], qq.z, o0);
                        o1 = fmaf(S[4 * i + 3], qq.w, o1);
                    }
                } else {
                    const float g = MODE == 1 ? b.g[tt] : 1.f;
                    const float4 *g4 = reinterpret_cast<const float4 *>(&b.gc[MODE == 2 ? tt : 0][MODE == 2 ? s * (DS + 4) : 0]);
                    float r0 = 0.f, r1 = 0.f;
#pragma unroll
                    for (int i = 0; i < DS / 4; i++) {
                        const float4 kk = k4[i];
                        const float4 gg = MODE == 2 ? g4[i] : make_float4(g, g, g, g);
                        S[4 * i + 0] *= gg.x;
                        S[4 * i + 1] *= gg.y;
                        S[4 * i + 2] *= gg.z;
                        S[4 * i + 3] *= gg.w;
                        r0 = fmaf(S[4 * i + 0], kk.x, r0);
                        r1 = fmaf(S[4 * i + 1], kk.y, r1);
                        r0 = fmaf(S[4 * i + 2], kk.z, r0);
                        r1 = fmaf(S[4 * i + 3], kk.w, r1);
                    }
                    float r = r0 + r1;
                    r += __shfl_xor_sync(0xffffffffu, r, 1);
                    r += __shfl_xor_sync(0xffffffffu, r, 2);
                    const float u = b.beta[tt] * (b.v[tt][cl] - r);
#pragma unroll
                    for (int i = 0; i < DS / 4; i++) {
                        const float4 kk = k4[i], qq = q4[i];
                        S[4 * i + 0] = fmaf(kk.x, u, S[4 * i + 0]);
                        S[4 * i + 1] = fmaf(kk.y, u, S[4 * i + 1]);
                        S[4 * i + 2] = fmaf(kk.z, u, S[4 * i + 2]);
                        S[4 * i + 3] = fmaf(kk.w, u, S[4 * i + 3]);
                        o0 = fmaf(S[4 * i + 0], qq.x, o0);
                        o1 = fmaf(S[4 * i + 1], qq.y, o1);
                        o0 = fmaf(S[4 * i + 2], qq.z, o0);
                        o1 = fmaf(S[4 * i + 3], qq.w, o1);
                    }
                }
                float o = o0 + o1;
                o += __shfl_xor_sync(0xffffffffu, o, 1);
                o += __shfl_xor_sync(0xffffffffu, o, 2);
                if (s == 0 && live) p.o[(t0 + tt) * p.ldo + (int64_t)h * p.Dv + col] = o;
            }
        }
        __syncthreads(); // the chunk is consumed and the next one is staged
    }
#pragma unroll
    for (int i = 0; i < DS; i++) {
        const int d = s * DS + i;
        if (live && d < p.D) sp[(int64_t)d * p.Dv] = S[i];
    }
}

// ------------------------------------------------------------------------------------------------ second halves of two low-rank projections
// x rows hold the first halves [a1 (Ka) | g1 (Kg)] in fp32; CTA (x, y) owns 128 outputs of one of the two matrices and 16
// tokens: the tokens' rows wait in shared memory rounded through the matrices' type, a thread owns one output for all 16 tokens
// and streams its matrix row once in 16-byte pieces (every piece feeds 16 x 8 or 16 x 4 multiply-adds against broadcast reads).
// The decay's outputs leave as exp(-exp(A_log[head]) softplus(. + dt_bias)), the gate's as they are.
constexpr int kLrTokens = 16, kLrOut = 128;

template <typename E>
__global__ void __launch_bounds__(kLrOut) lowrank_pair_kernel(const float *__restrict__ x, int64_t ldx, int64_t T, const E *__restrict__ w_a, int64_t Na,
                                                              int Ka, const E *__restrict__ w_g, int64_t Ng, int Kg, const float *__restrict__ A_log,
                                                              const float *__restrict__ dt_bias, int D, float *__restrict__ a,
                                                              float *__restrict__ g, int vec) {
    extern __shared__ __align__(16) float lr_x[]; // [kLrTokens][Kp]
    constexpr int VE = 16 / (int)sizeof(E);
    const int blocks_a = (int)((Na + kLrOut - 1) / kLrOut);
    const bool is_a = (int)blockIdx.x < blocks_a;
    const int64_t n = (int64_t)(is_a ? blockIdx.x : blockIdx.x - blocks_a) * kLrOut + threadIdx.x, N = is_a ? Na : Ng;
    const int K = is_a ? Ka : Kg, koff = is_a ? 0 : Ka, Kp = (K + 3) & ~3;
    const int64_t t0 = (int64_t)blockIdx.y * kLrTokens;
    const int nt = (int)min((int64_t)kLrTokens, T - t0);
    for (int e = threadIdx.x; e < kLrTokens * Kp; e += blockDim.x) {
        const int tt = e / Kp, k = e - tt * Kp;
        lr_x[e] = (tt < nt && k < K) ? to_f32(from_f32<E>(x[(t0 + tt) * ldx + koff + k])) : 0.f;
    }
    __syncthreads();
    if (n >= N) return;
    const E *wr = (is_a ? w_a : w_g) + n * K;
    float acc[kLrTokens];
#pragma unroll
    for (int tt = 0; tt < kLrTokens; tt++) acc[tt] = 0.f;
    if (vec) { // K a multiple of the 16-byte piece, rows aligned
        for (int k = 0; k < K; k += VE) {
            const uint4 wv = *reinterpret_cast<const uint4 *>(wr + k);
            const E *we = reinterpret_cast<const E *>(&wv);
            float wf[VE];
#pragma unroll
            for (int u = 0; u < VE; u++) wf[u] = to_f32(we[u]);
#pragma unroll
            for (int tt = 0; tt < kLrTokens; tt++) {
#pragma unroll
                for (int u = 0; u < VE; u += 4) {
                    const float4 xv = *reinterpret_cast<const float4 *>(lr_x + tt * Kp + k + u);
                    acc[tt] = fmaf(wf[u], xv.x, acc[tt]);
                    acc[tt] = fmaf(wf[u + 1], xv.y, acc[tt]);
                    acc[tt] = fmaf(wf[u + 2], xv.z, acc[tt]);
                    acc[tt] = fmaf(wf[u + 3], xv.w, acc[tt]);
                }
            }
        }
    } else {
        for (int k = 0; k < K; k++) {
            const float wf = to_f32(wr[k]);
#pragma unroll
            for (int tt = 0; tt < kLrTokens; tt++) acc[tt] = fmaf(wf, lr_x[tt * Kp + k], acc[tt]);
        }
    }
    if (is_a && A_log) {
        const float rate = expf(A_log[n / D]), bias = dt_bias[n];
#pragma unroll
        for (int tt = 0; tt < kLrTokens; tt++) acc[tt] = expf(-rate * softplus_f32(acc[tt] + bias));
    }
    float *out = is_a ? a : g;
#pragma unroll
    for (int tt = 0; tt < kLrTokens; tt++)
        if (tt < nt) out[(t0 + tt) * N + n] = acc[tt];
}

template <int DS, int CV, int MODE>
int recurrence_launch_cv(const rec_args &p) {
    const dim3 grid((unsigned)p.H, (unsigned)((p.Dv + CV - 1) / CV));
    const size_t smem = 2 * sizeof(rec_smem<DS, CV, MODE == 2>);
    auto k = recurrence_kernel<DS, CV, MODE>;
    if (smem > 48 * 1024) GGB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k<<<grid, CV * kNS + 32 * kStageWarps, smem, ggb_cuda_stream()>>>(p);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

// value columns per CTA: 16 while that leaves a CTA per SM at most (the kernel is bound by instruction issue of the one
// CTA an SM holds, so more SMs per head is what helps), else 32
template <int DS, int MODE>
int recurrence_launch_ds(const rec_args &p) {
    if ((int64_t)p.H * ((p.Dv + 15) / 16) <= ggb_sm_count()) return recurrence_launch_cv<DS, 16, MODE>(p);
    return recurrence_launch_cv<DS, 32, MODE>(p);
}

template <int MODE>
int recurrence_launch(const rec_args &p) {
    const int ds = (p.D + kNS - 1) / kNS;
    if (ds <= 8) return recurrence_launch_ds<8, MODE>(p);
    if (ds <= 16) return recurrence_launch_ds<16, MODE>(p);
    if (ds <= 32) return recurrence_launch_ds<32, MODE>(p);
    return recurrence_launch_ds<64, MODE>(p);
}

} // namespace

extern "C" {

int ggb_op_causal_conv(int dt, const float *x, int64_t ldx, int64_t T, int64_t C, const float *w, int taps, int add_input, int act,
                       float *tail, float *y_f32, int64_t ldy, void *y_dt) {
    return ggb_op_causal_conv_bias(dt, x, ldx, T, C, w, nullptr, taps, add_input, act, tail, y_f32, ldy, y_dt);
}

int ggb_op_causal_conv_bias(int dt, const float *x, int64_t ldx, int64_t T, int64_t C, const float *w, const float *bias, int taps,
                            int add_input, int act, float *tail, float *y_f32, int64_t ldy, void *y_dt) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(dt == GGB_TYPE_BF16 || dt == GGB_TYPE_F32, "causal_conv: dtype %d is neither bf16 nor f32", dt);
    GGB_CHECK_ARG(x && w && T > 0 && C > 0 && ldx >= C && taps >= 1 && taps <= kConvMaxTaps && (taps == 1 || tail) && (y_f32 || y_dt) &&
                      (!y_f32 || ldy >= C),
                  "causal_conv: bad arguments (taps %d, at most %d)", taps, kConvMaxTaps);
    const dim3 grid((unsigned)((C + 127) / 128), (unsigned)((T + kConvTokens - 1) / kConvTokens));
    if (dt == GGB_TYPE_BF16)
        causal_conv_kernel<<<grid, 128, 0, ggb_cuda_stream()>>>(x, ldx, T, C, w, bias, taps, add_input, act, tail, y_f32, ldy, (__nv_bfloat16 *)y_dt);
    else
        causal_conv_kernel<<<grid, 128, 0, ggb_cuda_stream()>>>(x, ldx, T, C, w, bias, taps, add_input, act, tail, y_f32, ldy, (float *)y_dt);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_lowrank_pair_fits(int dt, int Ka, int Kg) { return (size_t)kLrTokens * (size_t)(std::max(Ka, Kg) + 3) * 4 <= 48 * 1024; }

int ggb_op_lowrank_pair(int dt, const float *x, int64_t ldx, int64_t T, const void *w_a, int64_t Na, int Ka, const void *w_g, int64_t Ng, int Kg,
                        const float *A_log, const float *dt_bias, int D, float *a, float *g) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(dt == GGB_TYPE_BF16 || dt == GGB_TYPE_F32, "lowrank_pair: dtype %d is neither bf16 nor f32", dt);
    GGB_CHECK_ARG(x && w_a && w_g && a && g && T > 0 && Na > 0 && Ng > 0 && Ka > 0 && Kg > 0 && ldx >= Ka + Kg && (!A_log || (dt_bias && D > 0 && Na % D == 0)),
                  "lowrank_pair: bad arguments");
    GGB_CHECK_ARG(ggb_lowrank_pair_fits(dt, Ka, Kg), "lowrank_pair: inner sizes %d / %d do not fit shared memory", Ka, Kg);
    const int ve = dt == GGB_TYPE_BF16 ? 8 : 4;
    const int vec = Ka % ve == 0 && Kg % ve == 0 && (((uintptr_t)w_a | (uintptr_t)w_g) & 15) == 0;
    const size_t smem = (size_t)kLrTokens * (size_t)((std::max(Ka, Kg) + 3) & ~3) * 4;
    const dim3 grid((unsigned)((Na + kLrOut - 1) / kLrOut + (Ng + kLrOut - 1) / kLrOut), (unsigned)((T + kLrTokens - 1) / kLrTokens));
    if (dt == GGB_TYPE_BF16)
        lowrank_pair_kernel<<<grid, kLrOut, smem, ggb_cuda_stream()>>>(x, ldx, T, (const __nv_bfloat16 *)w_a, Na, Ka, (const __nv_bfloat16 *)w_g, Ng, Kg, A_log,
                                                                      dt_bias, D, a, g, vec);
    else
        lowrank_pair_kernel<<<grid, kLrOut, smem, ggb_cuda_stream()>>>(x, ldx, T, (const float *)w_a, Na, Ka, (const float *)w_g, Ng, Kg, A_log, dt_bias, D, a, g,
                                                                      vec);
    GGB_LAUNCH_CHECK();
    return GGB_OK;
}

int ggb_op_lightning_attn(const float *q, const float *k, const float *v, int64_t ld, int64_t T, int H, int D, int Dv, const float *decay,
                          float *state, float *o, int64_t ldo) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(q && k && v && decay && state && o && T > 0 && H > 0 && D > 0 && D <= 64 * kNS && Dv > 0 && ldo >= (int64_t)H * Dv,
                  "lightning_attn: bad arguments (key size %d, at most %d)", D, 64 * kNS);
    rec_args p{q, k, v, nullptr, nullptr, ld, 0, 0, T, H, H, D, Dv, decay, nullptr, nullptr, state, o, ldo, 0};
    return recurrence_launch<0>(p);
}

int ggb_op_gated_delta(const float *q, const float *k, const float *v, int64_t ld, const float *b, const float *a, int64_t ld_ba, int64_t T,
                       int H, int G, int D, int Dv, const float *A_log, const float *dt_bias, float *state, float *o, int64_t ldo) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(q && k && v && b && a && A_log && dt_bias && state && o && T > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && D <= 64 * kNS &&
                      Dv > 0 && ldo >= (int64_t)H * Dv,
                  "gated_delta: bad arguments (heads %d over %d key heads, key size %d)", H, G, D);
    rec_args p{q, k, v, b, a, ld, ld_ba, ld_ba, T, H, G, D, Dv, nullptr, A_log, dt_bias, state, o, ldo, 0};
    return recurrence_launch<1>(p);
}

int ggb_op_channel_delta(const float *q, const float *k, const float *v, int64_t ld, const float *b, int64_t ld_b, const float *a, int64_t ld_a,
                         int decays, int64_t T, int H, int G, int D, int Dv, const float *A_log, const float *dt_bias, float *state, float *o,
                         int64_t ldo) {
    GGB_REQUIRE_INIT();
    GGB_CHECK_ARG(q && k && v && b && a && (decays || (A_log && dt_bias)) && state && o && T > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 &&
                      D <= 64 * kNS && Dv > 0 && ldo >= (int64_t)H * Dv && ld_a >= (int64_t)H * D && ld_b >= H,
                  "channel_delta: bad arguments (heads %d over %d key heads, key size %d)", H, G, D);
    rec_args p{q, k, v, b, a, ld, ld_b, ld_a, T, H, G, D, Dv, nullptr, A_log, dt_bias, state, o, ldo, decays};
    return recurrence_launch<2>(p);
}

} // extern "C"
