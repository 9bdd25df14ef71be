// LayerNorm + residual forward and backward with one warp per row (cpu_backend.cpp:142-211): for row lengths
// d = 128 * VEC (VEC <= 8, e.g. 768) a lane keeps its VEC float4 of the row in registers, so every tensor is read once,
// with 16-byte accesses, and the row statistics are warp shuffles.  The backward kernel also accumulates the
// column sums for grad_gamma / grad_beta over the rows a warp processes and leaves one partial row per block for
// layernorm_backward_params_final_kernel, which saves the separate pass over grad_y and x.  All sums are taken
// in a fixed order (results do not depend on timing).  Other row lengths use the kernels in backend_ops.cuh.
#pragma once

#include <cstddef>
#include <cuda_runtime.h>

namespace gptb200 {
namespace ops {

constexpr int kLnWarpsPerBlock = 8;

__device__ __forceinline__ float ln_warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int VEC>
__global__ void __launch_bounds__(kLnWarpsPerBlock * 32)
layernorm_forward_warp_kernel(float *__restrict__ y, float *__restrict__ means, float *__restrict__ vars, float *__restrict__ x,
                              const float *__restrict__ residual, const float *__restrict__ gamma, const float *__restrict__ beta, int rows)
{
    constexpr int D = 128 * VEC;
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kLnWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    float4 *xr = reinterpret_cast<float4 *>(x + size_t(row) * D);
    float4 v[VEC];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        v[i] = xr[lane + 32 * i];
        if (residual) {
            const float4 r = __ldg(reinterpret_cast<const float4 *>(residual + size_t(row) * D) + lane + 32 * i);
            v[i].x += r.x;
            v[i].y += r.y;
            v[i].z += r.z;
            v[i].w += r.w;
            xr[lane + 32 * i] = v[i];
        }
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = ln_warp_sum(s) / D;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
        q += (a * a + b * b) + (c * c + e * e);
    }
    const float var = ln_warp_sum(q) / D;
    if (lane == 0) {
        means[row] = mean;
        vars[row] = var;
    }
    const float sd = sqrtf(var + 1e-5f);
    float4 *yr = reinterpret_cast<float4 *>(y + size_t(row) * D);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const float4 g = __ldg(reinterpret_cast<const float4 *>(gamma) + lane + 32 * i);
        const float4 b = __ldg(reinterpret_cast<const float4 *>(beta) + lane + 32 * i);
        float4 o;
        o.x = ((v[i].x - mean) / sd) * g.x + b.x;
        o.y = ((v[i].y - mean) / sd) * g.y + b.y;
        o.z = ((v[i].z - mean) / sd) * g.z + b.z;
        o.w = ((v[i].w - mean) / sd) * g.w + b.w;
        yr[lane + 32 * i] = o;
    }
}

// grad_x for the rows of this warp (row = first, first + stride, ...), and the block's partial column sums
// ws_gamma[block][d] = sum grad_y * x_hat, ws_beta[block][d] = sum grad_y.
template <int VEC>
__global__ void __launch_bounds__(kLnWarpsPerBlock * 32)
layernorm_backward_warp_kernel(float *__restrict__ grad_x, float *__restrict__ ws_gamma, float *__restrict__ ws_beta,
                               const float *__restrict__ grad_y, const float *__restrict__ grad_residual, const float *__restrict__ x,
                               const float *__restrict__ means, const float *__restrict__ vars, const float *__restrict__ gamma, int rows)
{
    constexpr int D = 128 * VEC;
    __shared__ __align__(16) float sum_g[D], sum_b[D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float4 gam[VEC], pg[VEC], pb[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        gam[i] = __ldg(reinterpret_cast<const float4 *>(gamma) + lane + 32 * i);
        pg[i] = pb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int row = blockIdx.x * kLnWarpsPerBlock + warp; row < rows; row += gridDim.x * kLnWarpsPerBlock) {
        const float mean = means[row];
        const float inv_std = 1.0f / sqrtf(vars[row] + 1e-5f);
        float4 xh[VEC], gg[VEC];
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const float4 xv = __ldg(reinterpret_cast<const float4 *>(x + size_t(row) * D) + lane + 32 * i);
            const float4 g = __ldg(reinterpret_cast<const float4 *>(grad_y + size_t(row) * D) + lane + 32 * i);
            xh[i].x = (xv.x - mean) * inv_std;
            xh[i].y = (xv.y - mean) * inv_std;
            xh[i].z = (xv.z - mean) * inv_std;
            xh[i].w = (xv.w - mean) * inv_std;
            pg[i].x += g.x * xh[i].x;
            pg[i].y += g.y * xh[i].y;
            pg[i].z += g.z * xh[i].z;
            pg[i].w += g.w * xh[i].w;
            pb[i].x += g.x;
            pb[i].y += g.y;
            pb[i].z += g.z;
            pb[i].w += g.w;
            gg[i].x = g.x * gam[i].x;
            gg[i].y = g.y * gam[i].y;
            gg[i].z = g.z * gam[i].z;
            gg[i].w = g.w * gam[i].w;
            s1 += (gg[i].x + gg[i].y) + (gg[i].z + gg[i].w);
            s2 += (gg[i].x * xh[i].x + gg[i].y * xh[i].y) + (gg[i].z * xh[i].z + gg[i].w * xh[i].w);
        }
        s1 = ln_warp_sum(s1) / D;
        s2 = ln_warp_sum(s2) / D;
        float4 *out = reinterpret_cast<float4 *>(grad_x + size_t(row) * D);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            float4 o;
            o.x = inv_std * (gg[i].x - s1 - xh[i].x * s2);
            o.y = inv_std * (gg[i].y - s1 - xh[i].y * s2);
            o.z = inv_std * (gg[i].z - s1 - xh[i].z * s2);
            o.w = inv_std * (gg[i].w - s1 - xh[i].w * s2);
            if (grad_residual) {
                const float4 r = __ldg(reinterpret_cast<const float4 *>(grad_residual + size_t(row) * D) + lane + 32 * i);
                o.x += r.x;
                o.y += r.y;
                o.z += r.z;
                o.w += r.w;
            }
            out[lane + 32 * i] = o;
        }
    }
    // the block's column sums: warp after warp, so that the order of the additions is fixed
    for (int w = 0; w < kLnWarpsPerBlock; ++w) {
        if (warp == w) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                float4 *sg = reinterpret_cast<float4 *>(sum_g) + lane + 32 * i;
                float4 *sb = reinterpret_cast<float4 *>(sum_b) + lane + 32 * i;
                if (w == 0) {
                    *sg = pg[i];
                    *sb = pb[i];
                } else {
                    float4 a = *sg, b = *sb;
                    a.x += pg[i].x; a.y += pg[i].y; a.z += pg[i].z; a.w += pg[i].w;
                    b.x += pb[i].x; b.y += pb[i].y; b.z += pb[i].z; b.w += pb[i].w;
                    *sg = a;
                    *sb = b;
                }
            }
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < D / 4; c += blockDim.x) {
        reinterpret_cast<float4 *>(ws_gamma + size_t(blockIdx.x) * D)[c] = reinterpret_cast<const float4 *>(sum_g)[c];
        reinterpret_cast<float4 *>(ws_beta + size_t(blockIdx.x) * D)[c] = reinterpret_cast<const float4 *>(sum_b)[c];
    }
}

}  // namespace ops
}  // namespace gptb200
