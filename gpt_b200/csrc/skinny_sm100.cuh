// Weight-streaming GEMM for decode-shaped calls (m <= 16 rows): y[m x n] = x[m x k] . W (+ bias, GELU).
//
// With so few rows the operation is bound by reading the weight matrix once from HBM (4*k*n bytes; the
// activations and outputs are negligible), so the kernel is organised around the weight stream, not around
// tensor-core tiles: every thread owns output columns, keeps one fp32 accumulator per row and column in
// registers, reads its part of the weight matrix exactly once with 16-byte loads and takes the activations from
// a shared-memory copy (broadcast reads).  The k range is split over blockIdx.y so that even a 768-column layer
// puts several hundred CTAs in flight; partial sums go to scratch and a second tiny kernel adds them in a fixed
// order and applies bias / GELU.  Plain fp32 FMAs: no TF32 rounding in either precision mode.
//
//   W_KN = true : W stored [k][n] (linear layers):   thread = 4 adjacent columns, coalesced 16-byte loads along n
//   W_KN = false: W stored [n][k] (tied un-embedding): thread = 1 column, 16-byte loads along its own row
#pragma once

#include <cuda_runtime.h>

#include "gemm_sm100.cuh"  // gelu_tanh

namespace gptb200 {

constexpr int kSkinnyThreads = 128;
constexpr int kSkinnyKChunk = 256;  // activations staged per pass: MR * 256 floats of shared memory

template <int MR, bool W_KN>
__global__ void __launch_bounds__(kSkinnyThreads)
skinny_gemm_kernel(float *__restrict__ partial, const float *__restrict__ x, const float *__restrict__ w, int M, int N, int K, int k_per_split)
{
    __shared__ __align__(16) float xs[MR][kSkinnyKChunk];
    constexpr int CPT = W_KN ? 4 : 1;  // columns per thread
    const int col = (blockIdx.x * kSkinnyThreads + threadIdx.x) * CPT;
    const int k_begin = blockIdx.y * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    const bool col_ok = col < N;  // N is a multiple of 4 on this path
    float acc[MR][CPT];
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
        for (int c = 0; c < CPT; ++c) acc[m][c] = 0.0f;

    for (int k0 = k_begin; k0 < k_end; k0 += kSkinnyKChunk) {
        const int kc = min(kSkinnyKChunk, k_end - k0);  // multiple of 4
        __syncthreads();
        for (int i = threadIdx.x; i < MR * (kSkinnyKChunk / 4); i += kSkinnyThreads) {
            const int m = i / (kSkinnyKChunk / 4), q = i % (kSkinnyKChunk / 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m < M && 4 * q < kc) v = *reinterpret_cast<const float4 *>(x + size_t(m) * K + k0 + 4 * q);
            *reinterpret_cast<float4 *>(&xs[m][4 * q]) = v;
        }
        __syncthreads();
        if (!col_ok) continue;
        if (W_KN) {
            const float *wp = w + size_t(k0) * N + col;
#pragma unroll 2
            for (int k = 0; k < kc; k += 4) {
                const float4 w0 = __ldcs(reinterpret_cast<const float4 *>(wp + size_t(k) * N));
                const float4 w1 = __ldcs(reinterpret_cast<const float4 *>(wp + size_t(k + 1) * N));
                const float4 w2 = __ldcs(reinterpret_cast<const float4 *>(wp + size_t(k + 2) * N));
                const float4 w3 = __ldcs(reinterpret_cast<const float4 *>(wp + size_t(k + 3) * N));
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const float4 xv = *reinterpret_cast<const float4 *>(&xs[m][k]);
                    acc[m][0] += xv.x * w0.x + xv.y * w1.x + xv.z * w2.x + xv.w * w3.x;
                    acc[m][1] += xv.x * w0.y + xv.y * w1.y + xv.z * w2.y + xv.w * w3.y;
                    acc[m][2] += xv.x * w0.z + xv.y * w1.z + xv.z * w2.z + xv.w * w3.z;
                    acc[m][3] += xv.x * w0.w + xv.y * w1.w + xv.z * w2.w + xv.w * w3.w;
                }
            }
        } else {
            const float *wp = w + size_t(col) * K + k0;
#pragma unroll 4
            for (int k = 0; k < kc; k += 4) {
                const float4 wv = *reinterpret_cast<const float4 *>(wp + k);  // the row's 128-byte line is reused from L1
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const float4 xv = *reinterpret_cast<const float4 *>(&xs[m][k]);
                    acc[m][0] += xv.x * wv.x + xv.y * wv.y + xv.z * wv.z + xv.w * wv.w;
                }
            }
        }
    }
    if (!col_ok) return;
    float *out = partial + size_t(blockIdx.y) * M * N;
#pragma unroll
    for (int m = 0; m < MR; ++m) {
        if (m >= M) break;
        if (W_KN)
            *reinterpret_cast<float4 *>(out + size_t(m) * N + col) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
        else
            out[size_t(m) * N + col] = acc[m][0];
    }
}

// y = sum_s partial[s] (s ascending) + bias; act = gelu_tanh(y)
__global__ void skinny_finish_kernel(float *__restrict__ y, float *__restrict__ act, const float *__restrict__ partial,
                                     const float *__restrict__ bias, int M, int N, int splits)
{
    const long long total = 1LL * M * N;
    const long long stride = 1LL * gridDim.x * blockDim.x;
    for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float s = partial[i];
        for (int p = 1; p < splits; ++p) s += partial[p * total + i];
        if (bias) s += bias[i % N];
        y[i] = s;
        if (act) act[i] = gelu_tanh(s);
    }
}

}  // namespace gptb200
