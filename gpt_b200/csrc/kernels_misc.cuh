// Small kernels beside the tcgen05 GEMM: GELU derivative, bias-gradient column sums, and a plain SIMT
// GEMM that serves shapes the TMA path cannot take (row pitches that are not a multiple of 16 bytes,
// unaligned base pointers, K == 0).  All are fp32.
#pragma once

#include <cuda_runtime.h>

#include "gemm_sm100.cuh"

namespace gptb200 {

// grad_x = grad_y * GELU'(x), same constants as the reference (linear.cu:162-187 / cpu_backend.cpp:268-287).
__device__ __forceinline__ float gelu_tanh_grad(float x)
{
    const float t = tanhf(0.79788456f * (x + 0.044715f * x * x * x));
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * (0.79788456f + 0.107032f * x * x);
}

__global__ void gelu_backward_kernel(float *__restrict__ gx, const float *__restrict__ gy, const float *__restrict__ x, long long n)
{
    const long long stride = 1LL * gridDim.x * blockDim.x;
    const long long n4 = n >> 2;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(gx) | reinterpret_cast<uintptr_t>(gy) | reinterpret_cast<uintptr_t>(x)) & 15) == 0;
    const long long tid = 1LL * blockIdx.x * blockDim.x + threadIdx.x;
    if (vec_ok) {
        for (long long i = tid; i < n4; i += stride) {
            const float4 xv = __ldcs(reinterpret_cast<const float4 *>(x) + i);
            const float4 gv = __ldcs(reinterpret_cast<const float4 *>(gy) + i);
            float4 o;
            o.x = gv.x * gelu_tanh_grad(xv.x);
            o.y = gv.y * gelu_tanh_grad(xv.y);
            o.z = gv.z * gelu_tanh_grad(xv.z);
            o.w = gv.w * gelu_tanh_grad(xv.w);
            reinterpret_cast<float4 *>(gx)[i] = o;
        }
        for (long long i = (n4 << 2) + tid; i < n; i += stride) gx[i] = gy[i] * gelu_tanh_grad(x[i]);
    } else {
        for (long long i = tid; i < n; i += stride) gx[i] = gy[i] * gelu_tanh_grad(x[i]);
    }
}

// Column sums of grad_y [M x N], stage 1: block (32, 8) covers 32 columns x one chunk of rows and writes
// one partial row into ws[chunk][N].  Stage 2 adds the chunks in a fixed order, so the result does not
// depend on scheduling.
__global__ void bias_grad_partial_kernel(float *__restrict__ ws, const float *__restrict__ gy, int M, int N, int rows_per_chunk)
{
    __shared__ float red[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    const int chunk = blockIdx.y;
    const long long r0 = 1LL * chunk * rows_per_chunk;
    const long long r1 = min(r0 + rows_per_chunk, static_cast<long long>(M));
    float s = 0.0f;
    if (col < N) {
        for (long long r = r0 + threadIdx.y; r < r1; r += 8) s += gy[r * N + col];
    }
    red[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && col < N) {
        float t = red[0][threadIdx.x];
#pragma unroll
        for (int i = 1; i < 8; ++i) t += red[i][threadIdx.x];
        ws[1LL * chunk * N + col] = t;
    }
}

__global__ void bias_grad_final_kernel(float *__restrict__ gb, const float *__restrict__ ws, int N, int chunks)
{
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= N) return;
    float s = 0.0f;
    for (int c = 0; c < chunks; ++c) s += ws[1LL * c * N + col];
    gb[col] += s;
}

// Plain tiled SIMT GEMM with arbitrary element strides: D[m][n] = sum_k A(m,k) B(k,n).
// A(m,k) = a[m * a_rs + k * a_cs], B(k,n) = b[k * b_rs + n * b_cs].  Same epilogue modes as the tcgen05
// kernel except EPI_PARTIAL.  Sums k in ascending order with separate multiply and add.
__global__ void simt_gemm_kernel(int M, int N, int K, const float *__restrict__ a, long long a_rs, long long a_cs,
                                 const float *__restrict__ b, long long b_rs, long long b_cs, float *__restrict__ out,
                                 float *__restrict__ act, const float *__restrict__ bias, long long ldo, int epi_mode)
{
    __shared__ float As[32][33];
    __shared__ float Bs[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;  // block (32, 8): each thread owns 4 rows
    const long long m_base = 1LL * blockIdx.y * 32;
    const long long n_base = 1LL * blockIdx.x * 32;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += 32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = ty + 8 * i;
            const long long m = m_base + r;
            const int k = k0 + tx;
            As[r][tx] = (m < M && k < K) ? a[m * a_rs + k * a_cs] : 0.0f;
            const int kk = k0 + r;
            const long long n = n_base + tx;
            Bs[r][tx] = (kk < K && n < N) ? b[kk * b_rs + n * b_cs] : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {
            const float bv = Bs[k][tx];
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(As[ty + 8 * i][k], bv));
        }
        __syncthreads();
    }
    const long long n = n_base + tx;
    if (n >= N) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long m = m_base + ty + 8 * i;
        if (m >= M) continue;
        float r = acc[i];
        if (epi_mode == EPI_ACCUM)
            r += out[m * ldo + n];
        else if (bias)
            r += bias[n];
        out[m * ldo + n] = r;
        if (act) act[m * ldo + n] = gelu_tanh(r);
    }
}

}  // namespace gptb200
