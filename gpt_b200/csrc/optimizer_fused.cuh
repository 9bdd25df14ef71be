// Gradient clipping and AdamW over the whole packed parameter buffer in two launches.
//
// The reference runs one AdamW launch per parameter tensor (sixteen) after three passes over the gradients for the
// 1/accum scaling and the norm clipping (src/model/gpt.cpp:644-677, src/backend/cuda/kernels/adamw.cu:71-97,
// gradient_clip.cu:35-59).  Every one of those passes is HBM-bound.  Here
//   1. grad_sumsq_kernel reads the gradients once (16-byte loads) and leaves one partial sum of squares per block;
//   2. adamw_packed_kernel adds the partial sums in a fixed order (every block does, from L2: a few KB), derives the factor
//      inv_accum * min(1, max_norm / (norm + 1e-6)) and applies it to each gradient element on its way into the moment
//      updates, so the gradients are never rewritten; weight decay is switched per tensor through the table of segment ends.
// HBM traffic per step: 4 B/param for the norm + 28 B/param for AdamW, against 12 + 28 B/param in the unfused form.
#pragma once

#include <cuda_runtime.h>

namespace gptb200 {
namespace ops {

constexpr int kMaxParamSegments = 32;

// Tensor t covers elements [end[t-1], end[t]) of the packed buffer (end[-1] = 0); decay[t] != 0: weight decay applies.
struct ParamSegments {
    long long end[kMaxParamSegments];
    unsigned char decay[kMaxParamSegments];
    int count;
};

__global__ void grad_sumsq_kernel(float *__restrict__ partial, const float *__restrict__ g, long long n)
{
    __shared__ float red[32];
    const long long n4 = n >> 2;
    const long long per = (n4 + gridDim.x - 1) / gridDim.x;
    const long long i0 = blockIdx.x * per, i1 = min(n4, i0 + per);
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    for (long long i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const float4 v = __ldcs(reinterpret_cast<const float4 *>(g) + i);
        s0 += v.x * v.x;
        s1 += v.y * v.y;
        s2 += v.z * v.z;
        s3 += v.w * v.w;
    }
    float s = (s0 + s1) + (s2 + s3);
    if (blockIdx.x == gridDim.x - 1)   // the last up-to-three elements
        for (long long i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) s += g[i] * g[i];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += red[w];
        partial[blockIdx.x] = t;
    }
}

__device__ __forceinline__ float adamw_element(float &p, float g, float &m, float &v, float lr, float beta1, float beta2, float eps, float wd,
                                               float bc1, float bc2)
{
    m = beta1 * m + (1.0f - beta1) * g;
    v = beta2 * v + (1.0f - beta2) * g * g;
    const float m_hat = m / bc1, v_hat = v / bc2;
    p -= lr * (m_hat / (sqrtf(v_hat) + eps) + wd * p);
    return p;
}

// `partial`: the `num_partial` block sums of grad_sumsq_kernel of the gradients BEFORE the 1/accum scaling.
// `vec_ok`: every segment end is a multiple of four (16-byte accesses never straddle two tensors).
__global__ void adamw_packed_kernel(float *__restrict__ p, const float *__restrict__ g, float *__restrict__ m, float *__restrict__ v, long long n,
                                    const float *__restrict__ partial, int num_partial, float inv_accum, float max_norm, float lr, float beta1,
                                    float beta2, float eps, float wd, float bc1, float bc2, const __grid_constant__ ParamSegments seg, int vec_ok,
                                    float *__restrict__ norm_out)
{
    __shared__ float s_scale;
    if (threadIdx.x < 32) {
        // the same order in every block and every run: lane-strided partial sums, then a butterfly
        float s = 0.0f;
        for (int i = threadIdx.x; i < num_partial; i += 32) s += __ldcg(partial + i);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (threadIdx.x == 0) {
            const float norm = sqrtf(s) * inv_accum;   // norm of the scaled gradients
            s_scale = inv_accum * (norm <= max_norm ? 1.0f : max_norm / (norm + 1e-6f));
            if (blockIdx.x == 0 && norm_out) *norm_out = norm;
        }
    }
    __syncthreads();
    const float scale = s_scale;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    auto decay_of = [&](long long i) {
        int t = 0;
        while (t < seg.count - 1 && i >= seg.end[t]) ++t;
        return seg.decay[t] ? wd : 0.0f;
    };
    if (vec_ok) {
        const long long n4 = n >> 2;
        for (long long i = tid; i < n4; i += stride) {
            const float w = decay_of(i << 2);
            float4 pv = reinterpret_cast<float4 *>(p)[i], mv = reinterpret_cast<float4 *>(m)[i], vv = reinterpret_cast<float4 *>(v)[i];
            const float4 gv = __ldcs(reinterpret_cast<const float4 *>(g) + i);
            adamw_element(pv.x, gv.x * scale, mv.x, vv.x, lr, beta1, beta2, eps, w, bc1, bc2);
            adamw_element(pv.y, gv.y * scale, mv.y, vv.y, lr, beta1, beta2, eps, w, bc1, bc2);
            adamw_element(pv.z, gv.z * scale, mv.z, vv.z, lr, beta1, beta2, eps, w, bc1, bc2);
            adamw_element(pv.w, gv.w * scale, mv.w, vv.w, lr, beta1, beta2, eps, w, bc1, bc2);
            reinterpret_cast<float4 *>(p)[i] = pv;
            reinterpret_cast<float4 *>(m)[i] = mv;
            reinterpret_cast<float4 *>(v)[i] = vv;
        }
        for (long long i = (n4 << 2) + tid; i < n; i += stride) adamw_element(p[i], g[i] * scale, m[i], v[i], lr, beta1, beta2, eps, decay_of(i), bc1, bc2);
    } else {
        for (long long i = tid; i < n; i += stride) adamw_element(p[i], g[i] * scale, m[i], v[i], lr, beta1, beta2, eps, decay_of(i), bc1, bc2);
    }
}

}  // namespace ops
}  // namespace gptb200
