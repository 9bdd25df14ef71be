// Kernels of the KV-cached generation loop around the decode-shaped linear layers: the reference's inference loop has no
// KV cache (src/infer/infer.cpp:112-148 recomputes the whole prefix for every token; "TODO: Add KV Cache" at :120).  With a
// cache, a generation step is one row per sequence through every layer: the linear layers see m = batch rows (the
// weight-streaming kernels of skinny_sm100.cuh) and attention is one query against the cached keys and values.
//
// Cache layout: [layer][sequence][position][k (d_model) | v (d_model)], i.e. the k and v thirds of the reference's packed
// qkv rows ([q | k | v], heads side by side inside each third).  The current position lives in device memory (*pos) so that
// a captured step can be replayed for every position.
#pragma once

#include <cfloat>
#include <cuda_runtime.h>

namespace gptb200 {
namespace ops {

// y[b, :] = wte[tokens[b], :] + wpe[*pos, :]   (one new position per sequence)
__global__ void embedding_decode_kernel(float *__restrict__ y, const float *__restrict__ wte, const float *__restrict__ wpe,
                                        const int *__restrict__ tokens, const int *__restrict__ pos, int d)
{
    const int b = blockIdx.x;
    const int p = *pos;
    const float *te = wte + size_t(tokens[b]) * d, *pe = wpe + size_t(p) * d;
    for (int h = threadIdx.x; h < d; h += blockDim.x) y[size_t(b) * d + h] = te[h] + pe[h];
}

// Prefill: cache[b][t][:] = the k | v thirds of qkv[b][t][:] for t < seq_len (qkv rows are [q | k | v], 3 * d floats).
__global__ void kv_fill_kernel(float *__restrict__ cache, const float *__restrict__ qkv, int seq_len, int max_len, int d)
{
    const int t = blockIdx.x, b = blockIdx.y;
    const float *src = qkv + (size_t(b) * seq_len + t) * 3 * d + d;
    float *dst = cache + (size_t(b) * max_len + t) * 2 * d;
    for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) dst[i] = src[i];
}

constexpr int kDecodeAttnThreads = 128;

// One query per (sequence, head) against the cache: appends the new position's k | v (from qkv_new [batch][3 d]) at *pos,
// then y[b, h*hd + :] = softmax_{t <= pos}(q . k_t / sqrt(hd)) . v_t, the same arithmetic as the full attention operator
// (maximum subtracted, exp, sum, divide).  hd: head size, a power of two in 4 .. 128.  Block = 128 threads; shared memory =
// (max_len + hd + 128 + 64) floats.
__global__ void __launch_bounds__(kDecodeAttnThreads)
attention_decode_kernel(float *__restrict__ y, float *__restrict__ cache, const float *__restrict__ qkv_new, const int *__restrict__ pos,
                        int max_len, int d, int hd, float scale)
{
    extern __shared__ float sm[];
    float *prob = sm;                            // [max_len]
    float *q = sm + max_len;                     // [hd]
    float *part = q + hd;                        // [128 / hd][hd] partial outputs
    float *red = part + kDecodeAttnThreads;      // [64]
    const int h = blockIdx.x, b = blockIdx.y;
    const int p = *pos;                          // position of the new token
    const int tid = threadIdx.x;
    float *kv = cache + size_t(b) * max_len * 2 * d;
    const float *row = qkv_new + size_t(b) * 3 * d;
    // the new position's k and v of this head go into the cache; q into shared memory
    for (int i = tid; i < hd; i += kDecodeAttnThreads) {
        q[i] = row[h * hd + i];
        kv[size_t(p) * 2 * d + h * hd + i] = row[d + h * hd + i];
        kv[size_t(p) * 2 * d + d + h * hd + i] = row[2 * d + h * hd + i];
    }
    __syncthreads();
    float mx = -FLT_MAX;
    for (int t = tid; t <= p; t += kDecodeAttnThreads) {
        const float4 *k4 = reinterpret_cast<const float4 *>(kv + size_t(t) * 2 * d + h * hd);
        float s = 0.0f;
        for (int i = 0; i < hd / 4; ++i) {
            const float4 kk = k4[i];
            s += q[4 * i] * kk.x + q[4 * i + 1] * kk.y + q[4 * i + 2] * kk.z + q[4 * i + 3] * kk.w;
        }
        s *= scale;
        prob[t] = s;
        mx = fmaxf(mx, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    float sum = 0.0f;
    for (int t = tid; t <= p; t += kDecodeAttnThreads) {
        const float e = expf(prob[t] - mx);
        prob[t] = e;
        sum += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((tid & 31) == 0) red[32 + (tid >> 5)] = sum;
    __syncthreads();
    sum = (red[32] + red[33]) + (red[34] + red[35]);
    // output: thread (g, c) adds the positions t = g (mod groups) of column c; the groups are added in a fixed order
    const int groups = kDecodeAttnThreads / hd;
    const int c = tid % hd, g = tid / hd;
    float acc = 0.0f;
    for (int t = g; t <= p; t += groups) acc += prob[t] * kv[size_t(t) * 2 * d + d + h * hd + c];
    part[g * hd + c] = acc;
    __syncthreads();
    if (g == 0) {
        for (int i = 1; i < groups; ++i) acc += part[i * hd + c];
        y[size_t(b) * d + h * hd + c] = acc / sum;
    }
}

__global__ void advance_position_kernel(int *pos) { *pos += 1; }

}  // namespace ops
}  // namespace gptb200
