// Row kernels of the tensor-core form of causal attention (head size 64).  The products run as batched launches of the
// CTA-pair GEMM kernel on head slices of the packed qkv rows:
//   forward :  S = Q . K^T,  P = causal softmax(S / 8) in place (kernel below),  y = P . V
//   backward:  S = Q . K^T and dP = dY . V^T,  then in place P = exp(S / 8 - lse), dS = P (dP - D) / 8 (kernel below),
//              dV = P^T . dY,  dK = dS^T . Q,  dQ = dS . K
// Same arithmetic as the reference's one-kernel attention (cpu_backend.cpp:290-433, cuda/kernels/attention.cu), with the
// score matrices of all heads held in device memory between the launches: s[b][q][h][k], a row per (sequence, query, head).
#pragma once

#include <cfloat>
#include <cuda_runtime.h>

namespace gptb200 {
namespace ops {

constexpr int kScoreRowsPerBlock = 8;   // one warp per row

// In place: p[k] = exp(scale * s[k] - lse) for k <= q and 0 beyond; lse[b, q, h] = max + log(sum) over the scaled scores.
// CHUNKS = 16-byte pieces per lane (row length <= 128 * CHUNKS, a multiple of 4).
template <int CHUNKS>
__global__ void __launch_bounds__(kScoreRowsPerBlock * 32)
attention_scores_softmax_kernel(float *__restrict__ s, float *__restrict__ logsumexp, int seq_len, int num_heads, float scale, long long rows)
{
    const int lane = threadIdx.x & 31;
    const long long r = 1LL * blockIdx.x * kScoreRowsPerBlock + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int q = static_cast<int>((r / num_heads) % seq_len);
    float4 *row = reinterpret_cast<float4 *>(s + r * seq_len);
    float4 v[CHUNKS];
    float m = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
        const int c = (i * 32 + lane) * 4;
        v[i] = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        if (c <= q && c < seq_len) {
            const float4 t = row[i * 32 + lane];
            v[i].x = t.x * scale;
            if (c + 1 <= q) v[i].y = t.y * scale;
            if (c + 2 <= q) v[i].z = t.z * scale;
            if (c + 3 <= q) v[i].w = t.w * scale;
            m = fmaxf(fmaxf(m, v[i].x), fmaxf(fmaxf(v[i].y, v[i].z), v[i].w));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
        const int c = (i * 32 + lane) * 4;
        // masked entries hold -FLT_MAX: expf gives exactly 0
        if (c <= q && c < seq_len) {
            v[i].x = expf(v[i].x - m);
            v[i].y = c + 1 <= q ? expf(v[i].y - m) : 0.0f;
            v[i].z = c + 2 <= q ? expf(v[i].z - m) : 0.0f;
            v[i].w = c + 3 <= q ? expf(v[i].w - m) : 0.0f;
            sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        } else {
            v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
    if (lane == 0) logsumexp[r] = m + logf(sum);
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < seq_len) row[i * 32 + lane] = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
    }
}

// In place on both buffers: s <- p = exp(scale * s - lse) for k <= q (0 beyond); dp <- ds = p * (dp - D) * scale.
__global__ void __launch_bounds__(kScoreRowsPerBlock * 32)
attention_scores_backward_kernel(float *__restrict__ s, float *__restrict__ dp, const float *__restrict__ logsumexp, const float *__restrict__ dcache,
                                 int seq_len, int num_heads, float scale, long long rows)
{
    const int lane = threadIdx.x & 31;
    const long long r = 1LL * blockIdx.x * kScoreRowsPerBlock + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int q = static_cast<int>((r / num_heads) % seq_len);
    const float lse = __ldg(logsumexp + r), dsum = __ldg(dcache + r);
    float4 *srow = reinterpret_cast<float4 *>(s + r * seq_len);
    float4 *drow = reinterpret_cast<float4 *>(dp + r * seq_len);
    for (int c4 = lane; c4 * 4 < seq_len; c4 += 32) {
        const int c = c4 * 4;
        float4 p = make_float4(0.0f, 0.0f, 0.0f, 0.0f), g = p;
        if (c <= q) {
            const float4 t = srow[c4], d = drow[c4];
            p.x = expf(t.x * scale - lse);
            g.x = p.x * (d.x - dsum) * scale;
            if (c + 1 <= q) { p.y = expf(t.y * scale - lse); g.y = p.y * (d.y - dsum) * scale; }
            if (c + 2 <= q) { p.z = expf(t.z * scale - lse); g.z = p.z * (d.z - dsum) * scale; }
            if (c + 3 <= q) { p.w = expf(t.w * scale - lse); g.w = p.w * (d.w - dsum) * scale; }
        }
        srow[c4] = p;
        drow[c4] = g;
    }
}

}  // namespace ops
}  // namespace gptb200
