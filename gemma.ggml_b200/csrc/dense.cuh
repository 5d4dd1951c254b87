// dense.cuh — what the bf16 / fp32 operator files (dense.cu, latent_attention.cu, moe.cu) share.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

// Sorted-slot description of one mixture-of-experts layer on the device (built by ggb_op_moe_group): slot s of token t
// (s < top) is row `inv[t * top + s]` of the sorted order, in which the slots of expert e are rows
// [offsets[e], offsets[e + 1]); row i of the sorted order belongs to token row_src[i].  The grouped products walk a list
// of 64-row tiles, none of which crosses an expert.
struct ggb_moe_groups {
    const int32_t *offsets = nullptr;     // [E + 1]
    const int32_t *row_src = nullptr;     // [n] A row of a sorted row, or null: A is already in sorted order
    const int32_t *tile_expert = nullptr; // [max_tiles]
    const int32_t *tile_row0 = nullptr;   // [max_tiles]
    const int32_t *n_tiles = nullptr;     // [1]
};

int ggb_linear_grouped_launch(int dt, const void *w, int64_t N, int64_t K, const void *a, int64_t lda, int max_tiles, float *c,
                              void *c_act, int64_t ldc, int act, const ggb_moe_groups &grp);

// the tcgen05 GEMM of prefill.cu on plain bf16 matrices: C[T][N] (fp32) = A[T][K] W[N][K]^T
bool ggb_gemm_dense_bf16_fits(int64_t N, int64_t K, int64_t T, int64_t ldc);
int ggb_gemm_dense_bf16(const void *w, int64_t N, int64_t K, const void *a, int64_t T, float *c, int64_t ldc);

// the grouped tcgen05 form: w [n_exp][N][K] bf16, a rows in sorted-slot order, offsets [n_exp + 1] on the device;
// c fp32 or (c_act) bf16 relu(c)^2
bool ggb_gemm_grouped_bf16_fits(int64_t N, int64_t K, int64_t ldc);
int ggb_gemm_grouped_bf16(const void *w, int64_t N, int64_t K, const void *a, int64_t n_rows, int n_exp, const int32_t *offsets, float *c,
                          void *c_act, int64_t ldc);

// norms on both sides of a sublayer (ggb_op_norm_add_norm); with inv / wt the sublayer's output is the weighted sum of
// the token's `top` expert slots, gathered on the way in (moe.cu)
int ggb_norm_add_norm_launch(int dt, const float *a, const float *bias, const int32_t *inv, const float *wt, int top, const float *wa, float eps,
                             int64_t E, int64_t T, float *x, const float *wy, void *y);

#ifdef __CUDACC__
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename E> __device__ __forceinline__ E from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
#endif
