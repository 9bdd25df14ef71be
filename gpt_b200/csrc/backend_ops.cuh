// Plain fp32 CUDA kernels for the operators of the reference's backend interface that are NOT on the
// linear-layer hot path (embedding, LayerNorm + residual, causal attention, softmax, cross-entropy, AdamW,
// gradient clipping, fills).  They exist so that a whole forward/backward step can run on the GPU behind
// the same interface; they follow the arithmetic of the reference CPU backend
// (src/backend/cpu/cpu_backend.cpp) and use no library.  Reductions that feed gradients are done in a fixed
// order (two-stage partial sums), except the token-embedding scatter which uses red.global.add like the
// reference's CUDA backend (src/backend/cuda/kernels/embedding.cu:92-110).
#pragma once

#include <cfloat>
#include <cstdint>
#include <cuda_runtime.h>

namespace gptb200 {
namespace ops {

// ------------------------------------------------------------------------------------------------ helpers

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; every thread gets the result.  `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float *red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? red[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}

__device__ __forceinline__ float block_max(float v, float *red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? red[lane] : -FLT_MAX;
    t = warp_max(t);
    return t;
}

// ------------------------------------------------------------------------------------------------ fills

__global__ void fill_const_kernel(float *p, float value, size_t n)
{
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = value;
}

__device__ __forceinline__ uint32_t mix32(uint64_t x)
{
    // splitmix64 finaliser, upper half
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    x ^= x >> 31;
    return static_cast<uint32_t>(x >> 32);
}

// Counter-based normal fill (Box-Muller on two hashed uniforms per element): reproducible for a given
// (seed, offset) regardless of launch shape.
__global__ void fill_normal_kernel(float *p, float mean, float stddev, size_t n, uint64_t seed, uint64_t offset)
{
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t c = (offset + i) * 2ull;
        const float u1 = (mix32(seed ^ (c * 0xD1342543DE82EF95ull)) + 1.0f) * (1.0f / 4294967808.0f);  // (0, 1]
        const float u2 = mix32(seed ^ ((c + 1ull) * 0xD1342543DE82EF95ull)) * (1.0f / 4294967296.0f);
        p[i] = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2) * stddev + mean;
    }
}

// ------------------------------------------------------------------------------------------------ embedding

// y[r, :] = wte[token[r], :] + wpe[r % seq_len, :]          (cpu_backend.cpp:65-79)
__global__ void embedding_forward_kernel(float *__restrict__ y, const float *__restrict__ wte, const float *__restrict__ wpe,
                                         const int *__restrict__ tokens, int rows, int seq_len, int d)
{
    const int r = blockIdx.x;
    if (r >= rows) return;
    const int tok = tokens[r];
    const int s = r % seq_len;
    for (int h = threadIdx.x; h < d; h += blockDim.x) y[size_t(r) * d + h] = wte[size_t(tok) * d + h] + wpe[size_t(s) * d + h];
}

// grad_wpe[s, h] += sum_b grad_y[b, s, h]  (b ascending);  grad_wte[token, h] += grad_y[r, h] (red.add)
__global__ void embedding_backward_kernel(float *__restrict__ grad_wte, float *__restrict__ grad_wpe, const float *__restrict__ grad_y,
                                          const int *__restrict__ tokens, int batch, int seq_len, int d)
{
    const int s = blockIdx.x;
    for (int h = threadIdx.x; h < d; h += blockDim.x) {
        float acc = 0.0f;
        for (int b = 0; b < batch; ++b) {
            const size_t r = size_t(b) * seq_len + s;
            const float g = grad_y[r * d + h];
            acc += g;
            atomicAdd(grad_wte + size_t(tokens[r]) * d + h, g);
        }
        grad_wpe[size_t(s) * d + h] += acc;
    }
}

// The same with every contribution multiplied by `scale` (a data-parallel step applies the rows of all ranks, each weighted
// 1 / ranks, to gradients that were already averaged).
__global__ void embedding_backward_scaled_kernel(float *__restrict__ grad_wte, float *__restrict__ grad_wpe, const float *__restrict__ grad_y,
                                                 const int *__restrict__ tokens, int batch, int seq_len, int d, float scale)
{
    const int s = blockIdx.x;
    for (int h = threadIdx.x; h < d; h += blockDim.x) {
        float acc = 0.0f;
        for (int b = 0; b < batch; ++b) {
            const size_t r = size_t(b) * seq_len + s;
            const float g = grad_y[r * d + h] * scale;
            acc += g;
            atomicAdd(grad_wte + size_t(tokens[r]) * d + h, g);
        }
        grad_wpe[size_t(s) * d + h] += acc;
    }
}

// ------------------------------------------------------------------------------------------------ LayerNorm

// x += residual (in place); mean, biased variance; y = (x - mean) / sqrt(var + 1e-5) * gamma + beta
// (cpu_backend.cpp:142-175; `vars` holds the variance, as in the CPU backend).  One block per row.
__global__ void layernorm_forward_kernel(float *__restrict__ y, float *__restrict__ means, float *__restrict__ vars, float *__restrict__ x,
                                         const float *__restrict__ residual, const float *__restrict__ gamma,
                                         const float *__restrict__ beta, int d)
{
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    float *xr = x + r * d;
    float s = 0.0f;
    for (int h = threadIdx.x; h < d; h += blockDim.x) {
        float v = xr[h];
        if (residual) {
            v += residual[r * d + h];
            xr[h] = v;
        }
        s += v;
    }
    const float mean = block_sum(s, red) / d;
    float q = 0.0f;
    for (int h = threadIdx.x; h < d; h += blockDim.x) {
        const float diff = xr[h] - mean;
        q += diff * diff;
    }
    const float var = block_sum(q, red) / d;
    if (threadIdx.x == 0) {
        means[r] = mean;
        vars[r] = var;
    }
    const float sd = sqrtf(var + 1e-5f);
    for (int h = threadIdx.x; h < d; h += blockDim.x) y[r * d + h] = ((xr[h] - mean) / sd) * gamma[h] + beta[h];
}

// grad_x = inv_std * (gy*gamma - mean(gy*gamma) - x_hat * mean(gy*gamma*x_hat)) + grad_residual   (cpu_backend.cpp:177-211)
__global__ void layernorm_backward_dx_kernel(float *__restrict__ grad_x, const float *__restrict__ grad_y,
                                             const float *__restrict__ grad_residual, const float *__restrict__ x,
                                             const float *__restrict__ means, const float *__restrict__ vars,
                                             const float *__restrict__ gamma, int d)
{
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    const float mean = means[r];
    const float inv_std = 1.0f / sqrtf(vars[r] + 1e-5f);
    float s1 = 0.0f, s2 = 0.0f;
    for (int h = threadIdx.x; h < d; h += blockDim.x) {
        const float xh = (x[r * d + h] - mean) * inv_std;
        const float gg = grad_y[r * d + h] * gamma[h];
        s1 += gg;
        s2 += gg * xh;
    }
    s1 = block_sum(s1, red) / d;
    s2 = block_sum(s2, red) / d;
    for (int h = threadIdx.x; h < d; h += blockDim.x) {
        const float xh = (x[r * d + h] - mean) * inv_std;
        float g = inv_std * (grad_y[r * d + h] * gamma[h] - s1 - xh * s2);
        if (grad_residual) g += grad_residual[r * d + h];
        grad_x[r * d + h] = g;
    }
}

// Stage 1 of grad_gamma / grad_beta: block (32, 8) covers 32 columns x one chunk of rows.
__global__ void layernorm_backward_params_partial_kernel(float *__restrict__ ws_gamma, float *__restrict__ ws_beta,
                                                         const float *__restrict__ grad_y, const float *__restrict__ x,
                                                         const float *__restrict__ means, const float *__restrict__ vars, int rows, int d,
                                                         int rows_per_chunk)
{
    __shared__ float rg[8][33], rb[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    const int chunk = blockIdx.y;
    const int r0 = chunk * rows_per_chunk, r1 = min(r0 + rows_per_chunk, rows);
    float sg = 0.0f, sb = 0.0f;
    if (col < d) {
        for (int r = r0 + threadIdx.y; r < r1; r += 8) {
            const float inv_std = 1.0f / sqrtf(vars[r] + 1e-5f);
            const float g = grad_y[size_t(r) * d + col];
            sg += g * ((x[size_t(r) * d + col] - means[r]) * inv_std);
            sb += g;
        }
    }
    rg[threadIdx.y][threadIdx.x] = sg;
    rb[threadIdx.y][threadIdx.x] = sb;
    __syncthreads();
    if (threadIdx.y == 0 && col < d) {
        float tg = 0.0f, tb = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            tg += rg[i][threadIdx.x];
            tb += rb[i][threadIdx.x];
        }
        ws_gamma[size_t(chunk) * d + col] = tg;
        ws_beta[size_t(chunk) * d + col] = tb;
    }
}

// Stage 2: block (32, 8) covers 32 columns; the eight thread rows take every eighth partial row, then add up in a fixed order.
__global__ void layernorm_backward_params_final_kernel(float *__restrict__ grad_gamma, float *__restrict__ grad_beta,
                                                       const float *__restrict__ ws_gamma, const float *__restrict__ ws_beta, int d, int chunks)
{
    __shared__ float rg[8][33], rb[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    float sg = 0.0f, sb = 0.0f;
    if (col < d) {
        for (int c = threadIdx.y; c < chunks; c += 8) {
            sg += ws_gamma[size_t(c) * d + col];
            sb += ws_beta[size_t(c) * d + col];
        }
    }
    rg[threadIdx.y][threadIdx.x] = sg;
    rb[threadIdx.y][threadIdx.x] = sb;
    __syncthreads();
    if (threadIdx.y == 0 && col < d) {
        float tg = 0.0f, tb = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            tg += rg[i][threadIdx.x];
            tb += rb[i][threadIdx.x];
        }
        grad_gamma[col] += tg;
        grad_beta[col] += tb;
    }
}

// ------------------------------------------------------------------------------------------------ attention
//
// Causal softmax attention on the packed qkv[B, T, 3*D] layout (cpu_backend.cpp:290-433), fp32 throughout.
// A query (or key) row is owned by TPR adjacent lanes, each holding HD/TPR head dimensions in registers;
// dot products are completed with TPR-wide shuffles.  K/V (or Q/dO) rows stream through shared memory in
// tiles of kTile rows and are read as warp-wide broadcasts.

constexpr int kAttnTile = 32;
constexpr int kAttnRowsPerBlock = 64;  // rows (queries or keys) per block

// Dot product of a register array with a shared-memory row slice, with four independent partial sums so that the
// FMAs do not form one long dependency chain (the compiler may not reassociate fp32 adds on its own).
template <int DPT>
__device__ __forceinline__ float dot_partial(const float (&a)[DPT], const float *__restrict__ b)
{
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
    for (int i = 0; i < DPT; i += 4) {
        s0 += a[i] * b[i];
        if (i + 1 < DPT) s1 += a[i + 1] * b[i + 1];
        if (i + 2 < DPT) s2 += a[i + 2] * b[i + 2];
        if (i + 3 < DPT) s3 += a[i + 3] * b[i + 3];
    }
    return (s0 + s1) + (s2 + s3);
}

template <int TPR>
__device__ __forceinline__ float row_sum(float v)
{
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// y[b, s1, h*HD + :] = softmax_{s2 <= s1}(q.k / sqrt(HD)) . v ;  logsumexp[b, s1, h] = max + log(sum)
template <int HD, int TPR>
__global__ void __launch_bounds__(kAttnRowsPerBlock *TPR)
attention_forward_kernel(float *__restrict__ y, float *__restrict__ logsumexp, const float *__restrict__ qkv, int seq_len, int d_model,
                         int num_heads)
{
    constexpr int DPT = HD / TPR;
    __shared__ float ks[kAttnTile][HD];
    __shared__ float vs[kAttnTile][HD];
    const int b = blockIdx.z, h = blockIdx.y;
    const int row = blockIdx.x * kAttnRowsPerBlock + threadIdx.x / TPR;  // query index s1
    const int part = threadIdx.x % TPR;
    const int stride = 3 * d_model;
    const float scale = 1.0f / sqrtf(static_cast<float>(HD));
    const float *base = qkv + size_t(b) * seq_len * stride + h * HD;
    const bool valid = row < seq_len;

    float q[DPT], acc[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        q[i] = valid ? base[size_t(row) * stride + part * DPT + i] : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -FLT_MAX, l = 0.0f;
    const int last_row = min(seq_len, (blockIdx.x + 1) * kAttnRowsPerBlock) - 1;  // largest query in this block
    for (int t0 = 0; t0 <= last_row; t0 += kAttnTile) {
        __syncthreads();
        for (int i = threadIdx.x; i < kAttnTile * HD; i += blockDim.x) {
            const int r = i / HD, c = i % HD;
            const int s2 = t0 + r;
            ks[r][c] = s2 < seq_len ? base[size_t(s2) * stride + d_model + c] : 0.0f;
            vs[r][c] = s2 < seq_len ? base[size_t(s2) * stride + 2 * d_model + c] : 0.0f;
        }
        __syncthreads();
        const int tend = row - t0 + 1;                               // this row uses keys s2 <= row
        const int tmax = min(kAttnTile, last_row - t0 + 1);          // block-uniform bound: shuffles stay convergent
        for (int r = 0; r < tmax; ++r) {
            float sc = dot_partial<DPT>(q, &ks[r][part * DPT]);
            sc = row_sum<TPR>(sc) * scale;
            if (r >= tend) continue;
            const float m_new = fmaxf(m, sc);
            const float corr = expf(m - m_new);
            const float p = expf(sc - m_new);
            l = l * corr + p;
#pragma unroll
            for (int i = 0; i < DPT; ++i) acc[i] = acc[i] * corr + p * vs[r][part * DPT + i];
            m = m_new;
        }
    }
    if (valid) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) y[(size_t(b) * seq_len + row) * d_model + h * HD + part * DPT + i] = acc[i] / l;
        if (part == 0) logsumexp[(size_t(b) * seq_len + row) * num_heads + h] = m + logf(l);
    }
}

// D[b, s, h] = sum_d grad_y * y  (per head)
__global__ void attention_rowsum_kernel(float *__restrict__ dcache, const float *__restrict__ grad_y, const float *__restrict__ y,
                                        int rows, int d_model, int num_heads)
{
    const int hd = d_model / num_heads;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;  // (row, head)
    if (idx >= size_t(rows) * num_heads) return;
    const size_t r = idx / num_heads;
    const int h = idx % num_heads;
    float s = 0.0f;
    for (int d = 0; d < hd; ++d) s += grad_y[r * d_model + h * hd + d] * y[r * d_model + h * hd + d];
    dcache[idx] = s;
}

// grad_q[s1] = sum_{s2 <= s1} dS . k[s2],  dS = p (dP - D) / sqrt(HD), p = exp(q.k/sqrt(HD) - L), dP = dO . v
template <int HD, int TPR>
__global__ void __launch_bounds__(kAttnRowsPerBlock *TPR)
attention_backward_dq_kernel(float *__restrict__ grad_qkv, const float *__restrict__ dcache, const float *__restrict__ logsumexp,
                             const float *__restrict__ grad_y, const float *__restrict__ qkv, int seq_len, int d_model, int num_heads)
{
    constexpr int DPT = HD / TPR;
    __shared__ float ks[kAttnTile][HD];
    __shared__ float vs[kAttnTile][HD];
    const int b = blockIdx.z, h = blockIdx.y;
    const int row = blockIdx.x * kAttnRowsPerBlock + threadIdx.x / TPR;
    const int part = threadIdx.x % TPR;
    const int stride = 3 * d_model;
    const float scale = 1.0f / sqrtf(static_cast<float>(HD));
    const float *base = qkv + size_t(b) * seq_len * stride + h * HD;
    const bool valid = row < seq_len;
    float q[DPT], go[DPT], dq[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        q[i] = valid ? base[size_t(row) * stride + part * DPT + i] : 0.0f;
        go[i] = valid ? grad_y[(size_t(b) * seq_len + row) * d_model + h * HD + part * DPT + i] : 0.0f;
        dq[i] = 0.0f;
    }
    const float L = valid ? logsumexp[(size_t(b) * seq_len + row) * num_heads + h] : 0.0f;
    const float Dv = valid ? dcache[(size_t(b) * seq_len + row) * num_heads + h] : 0.0f;
    const int last_row = min(seq_len, (blockIdx.x + 1) * kAttnRowsPerBlock) - 1;
    for (int t0 = 0; t0 <= last_row; t0 += kAttnTile) {
        __syncthreads();
        for (int i = threadIdx.x; i < kAttnTile * HD; i += blockDim.x) {
            const int r = i / HD, c = i % HD;
            const int s2 = t0 + r;
            ks[r][c] = s2 < seq_len ? base[size_t(s2) * stride + d_model + c] : 0.0f;
            vs[r][c] = s2 < seq_len ? base[size_t(s2) * stride + 2 * d_model + c] : 0.0f;
        }
        __syncthreads();
        const int tend = row - t0 + 1;
        const int tmax = min(kAttnTile, last_row - t0 + 1);
        for (int r = 0; r < tmax; ++r) {
            float sc = dot_partial<DPT>(q, &ks[r][part * DPT]);
            float dp = dot_partial<DPT>(go, &vs[r][part * DPT]);
            sc = row_sum<TPR>(sc);
            dp = row_sum<TPR>(dp);
            if (r >= tend) continue;
            const float p = expf(sc * scale - L);
            const float ds = p * (dp - Dv) * scale;
#pragma unroll
            for (int i = 0; i < DPT; ++i) dq[i] += ds * ks[r][part * DPT + i];
        }
    }
    if (valid) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) grad_qkv[(size_t(b) * seq_len + row) * stride + h * HD + part * DPT + i] = dq[i];
    }
}

// grad_k[s2] = sum_{s1 >= s2} dS . q[s1],  grad_v[s2] = sum_{s1 >= s2} p . dO[s1]
template <int HD, int TPR>
__global__ void __launch_bounds__(kAttnRowsPerBlock *TPR)
attention_backward_dkv_kernel(float *__restrict__ grad_qkv, const float *__restrict__ dcache, const float *__restrict__ logsumexp,
                              const float *__restrict__ grad_y, const float *__restrict__ qkv, int seq_len, int d_model, int num_heads)
{
    constexpr int DPT = HD / TPR;
    __shared__ float qs[kAttnTile][HD];
    __shared__ float gs[kAttnTile][HD];
    __shared__ float Ls[kAttnTile], Ds[kAttnTile];
    const int b = blockIdx.z, h = blockIdx.y;
    const int row = blockIdx.x * kAttnRowsPerBlock + threadIdx.x / TPR;  // key index s2
    const int part = threadIdx.x % TPR;
    const int stride = 3 * d_model;
    const float scale = 1.0f / sqrtf(static_cast<float>(HD));
    const float *base = qkv + size_t(b) * seq_len * stride + h * HD;
    const bool valid = row < seq_len;
    float k[DPT], v[DPT], dk[DPT], dv[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        k[i] = valid ? base[size_t(row) * stride + d_model + part * DPT + i] : 0.0f;
        v[i] = valid ? base[size_t(row) * stride + 2 * d_model + part * DPT + i] : 0.0f;
        dk[i] = 0.0f;
        dv[i] = 0.0f;
    }
    const int first_row = blockIdx.x * kAttnRowsPerBlock;  // smallest key in this block
    for (int t0 = (first_row / kAttnTile) * kAttnTile; t0 < seq_len; t0 += kAttnTile) {
        __syncthreads();
        for (int i = threadIdx.x; i < kAttnTile * HD; i += blockDim.x) {
            const int r = i / HD, c = i % HD;
            const int s1 = t0 + r;
            qs[r][c] = s1 < seq_len ? base[size_t(s1) * stride + c] : 0.0f;
            gs[r][c] = s1 < seq_len ? grad_y[(size_t(b) * seq_len + s1) * d_model + h * HD + c] : 0.0f;
        }
        for (int r = threadIdx.x; r < kAttnTile; r += blockDim.x) {
            const int s1 = t0 + r;
            Ls[r] = s1 < seq_len ? logsumexp[(size_t(b) * seq_len + s1) * num_heads + h] : 0.0f;
            Ds[r] = s1 < seq_len ? dcache[(size_t(b) * seq_len + s1) * num_heads + h] : 0.0f;
        }
        __syncthreads();
        const int rbeg = max(0, first_row - t0);              // block-uniform bounds: shuffles stay convergent
        const int rend = min(kAttnTile, seq_len - t0);
        for (int r = rbeg; r < rend; ++r) {
            float sc = dot_partial<DPT>(k, &qs[r][part * DPT]);
            float dp = dot_partial<DPT>(v, &gs[r][part * DPT]);
            sc = row_sum<TPR>(sc);
            dp = row_sum<TPR>(dp);
            if (t0 + r < row) continue;                       // this key only sees queries s1 >= row
            const float p = expf(sc * scale - Ls[r]);
            const float ds = p * (dp - Ds[r]) * scale;
#pragma unroll
            for (int i = 0; i < DPT; ++i) {
                dk[i] += ds * qs[r][part * DPT + i];
                dv[i] += p * gs[r][part * DPT + i];
            }
        }
    }
    if (valid) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            grad_qkv[(size_t(b) * seq_len + row) * stride + d_model + h * HD + part * DPT + i] = dk[i];
            grad_qkv[(size_t(b) * seq_len + row) * stride + 2 * d_model + h * HD + part * DPT + i] = dv[i];
        }
    }
}

// ------------------------------------------------------------------------------------------------ softmax / cross-entropy

// y[r, :V] = softmax(x[r, :V]); y[r, V:Vp] = 0       (cpu_backend.cpp:435-472).  One block per row.
__global__ void softmax_forward_kernel(float *__restrict__ y, const float *__restrict__ x, int v, int vp)
{
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    const float *xr = x + r * vp;
    float *yr = y + r * vp;
    float m = -FLT_MAX;
    for (int i = threadIdx.x; i < v; i += blockDim.x) m = fmaxf(m, xr[i]);
    m = block_max(m, red);
    float s = 0.0f;
    for (int i = threadIdx.x; i < v; i += blockDim.x) {
        const float e = expf(xr[i] - m);
        yr[i] = e;
        s += e;
    }
    s = block_sum(s, red);
    for (int i = threadIdx.x; i < v; i += blockDim.x) yr[i] /= s;
    for (int i = v + threadIdx.x; i < vp; i += blockDim.x) yr[i] = 0.0f;
}

// The same for rows of up to THREADS * 4 * NV floats whose pitch is a multiple of 4 (16-byte aligned rows): a thread keeps its
// NV float4 of the row in registers, so the logits are read once and the probabilities written once.
template <int THREADS, int NV>
__global__ void __launch_bounds__(THREADS) softmax_forward_rowreg_kernel(float *__restrict__ y, const float *__restrict__ x, int v, int vp)
{
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    const float4 *xr = reinterpret_cast<const float4 *>(x + r * vp);
    float4 *yr = reinterpret_cast<float4 *>(y + r * vp);
    const int nvec = vp >> 2;
    float4 e[NV];
    float m = -FLT_MAX;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + THREADS * k;
        e[k] = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        if (c < nvec) {
            const float4 t = __ldg(xr + c);
            const int i = 4 * c;
            e[k].x = i < v ? t.x : -FLT_MAX;
            e[k].y = i + 1 < v ? t.y : -FLT_MAX;
            e[k].z = i + 2 < v ? t.z : -FLT_MAX;
            e[k].w = i + 3 < v ? t.w : -FLT_MAX;
        }
        m = fmaxf(m, fmaxf(fmaxf(e[k].x, e[k].y), fmaxf(e[k].z, e[k].w)));
    }
    m = block_max(m, red);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        e[k].x = e[k].x == -FLT_MAX ? 0.0f : expf(e[k].x - m);
        e[k].y = e[k].y == -FLT_MAX ? 0.0f : expf(e[k].y - m);
        e[k].z = e[k].z == -FLT_MAX ? 0.0f : expf(e[k].z - m);
        e[k].w = e[k].w == -FLT_MAX ? 0.0f : expf(e[k].w - m);
        s += (e[k].x + e[k].y) + (e[k].z + e[k].w);
    }
    s = block_sum(s, red);
    const float rs = 1.0f / s;   // one division per row: a hundred per thread would make the kernel instruction-bound
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + THREADS * k;
        if (c < nvec) yr[c] = make_float4(e[k].x * rs, e[k].y * rs, e[k].z * rs, e[k].w * rs);   // masked and padding columns: 0
    }
}

// grad_x[r, :V] = (p - onehot(label)) / rows; padding columns are left as they are   (cpu_backend.cpp:474-491)
__global__ void cross_entropy_softmax_backward_kernel(float *__restrict__ grad_x, const float *__restrict__ probs,
                                                      const int *__restrict__ labels, int rows, int v, int vp)
{
    const size_t r = blockIdx.x;
    const int label = labels[r];
    const float inv = static_cast<float>(rows);
    for (int i = threadIdx.x; i < v; i += blockDim.x) grad_x[r * vp + i] = (probs[r * vp + i] - (i == label ? 1.0f : 0.0f)) / inv;
}

// The same with 16-byte accesses (row pitch a multiple of 4); the last vector of a row is written element by element so that
// the padding columns stay untouched.
__global__ void cross_entropy_softmax_backward_vec_kernel(float *__restrict__ grad_x, const float *__restrict__ probs,
                                                          const int *__restrict__ labels, int rows, int v, int vp)
{
    const size_t r = blockIdx.x;
    const int label = labels[r];
    const float inv = 1.0f / static_cast<float>(rows);
    const float4 *p = reinterpret_cast<const float4 *>(probs + r * vp);
    float4 *g = reinterpret_cast<float4 *>(grad_x + r * vp);
    const int full = v >> 2;
    for (int c = threadIdx.x; c < full; c += blockDim.x) {
        const float4 t = __ldg(p + c);
        const int i = 4 * c;
        g[c] = make_float4((t.x - (i == label ? 1.0f : 0.0f)) * inv, (t.y - (i + 1 == label ? 1.0f : 0.0f)) * inv,
                           (t.z - (i + 2 == label ? 1.0f : 0.0f)) * inv, (t.w - (i + 3 == label ? 1.0f : 0.0f)) * inv);
    }
    for (int i = 4 * full + threadIdx.x; i < v; i += blockDim.x) grad_x[r * vp + i] = (probs[r * vp + i] - (i == label ? 1.0f : 0.0f)) * inv;
}

// Softmax, cross-entropy backward and the row's loss term in ONE pass over the logits, in place: what the reference does with
// device_softmax_forward (logits -> probabilities), device_cross_entropy_softmax_fused_backward (probabilities -> gradient)
// and device_cross_entropy_loss (cpu_backend.cpp:439-509), without the probability tensor and without a second and third
// trip through HBM.  A thread keeps its NV float4 of the row in registers: the logits are read once and overwritten by
//   x[r, i] = (softmax(x[r, :v])[i] - (i == label)) / rows   for i < v,      x[r, i] = 0   for v <= i < vp
// and row_loss[r] = -log(p[label] + 1e-8), the term that cross_entropy_loss averages.
template <int THREADS, int NV>
__global__ void __launch_bounds__(THREADS) softmax_ce_inplace_rowreg_kernel(float *__restrict__ x, float *__restrict__ row_loss,
                                                                            const int *__restrict__ labels, int rows, int v, int vp)
{
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    float4 *xr = reinterpret_cast<float4 *>(x + r * vp);
    const int nvec = vp >> 2;
    const int label = labels[r];
    float4 e[NV];
    float m = -FLT_MAX;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + THREADS * k;
        e[k] = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        if (c < nvec) {
            const float4 t = xr[c];
            const int i = 4 * c;
            e[k].x = i < v ? t.x : -FLT_MAX;
            e[k].y = i + 1 < v ? t.y : -FLT_MAX;
            e[k].z = i + 2 < v ? t.z : -FLT_MAX;
            e[k].w = i + 3 < v ? t.w : -FLT_MAX;
        }
        m = fmaxf(m, fmaxf(fmaxf(e[k].x, e[k].y), fmaxf(e[k].z, e[k].w)));
    }
    m = block_max(m, red);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        e[k].x = e[k].x == -FLT_MAX ? 0.0f : expf(e[k].x - m);
        e[k].y = e[k].y == -FLT_MAX ? 0.0f : expf(e[k].y - m);
        e[k].z = e[k].z == -FLT_MAX ? 0.0f : expf(e[k].z - m);
        e[k].w = e[k].w == -FLT_MAX ? 0.0f : expf(e[k].w - m);
        s += (e[k].x + e[k].y) + (e[k].z + e[k].w);
    }
    s = block_sum(s, red);
    const float inv = 1.0f / static_cast<float>(rows), rs = 1.0f / s;   // two divisions per row instead of two per element
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + THREADS * k;
        if (c >= nvec) continue;
        const int i = 4 * c;
        float p[4] = {e[k].x * rs, e[k].y * rs, e[k].z * rs, e[k].w * rs};
        float g[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (i + j == label) row_loss[r] = -logf(p[j] + 1e-8f);
            g[j] = i + j < v ? (p[j] - (i + j == label ? 1.0f : 0.0f)) * inv : 0.0f;
        }
        xr[c] = make_float4(g[0], g[1], g[2], g[3]);
    }
}

// The same for any row length and alignment: three passes of one block over its row (maximum, sum, write).
__global__ void softmax_ce_inplace_kernel(float *__restrict__ x, float *__restrict__ row_loss, const int *__restrict__ labels, int rows, int v, int vp)
{
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    float *xr = x + r * vp;
    const int label = labels[r];
    float m = -FLT_MAX;
    for (int i = threadIdx.x; i < v; i += blockDim.x) m = fmaxf(m, xr[i]);
    m = block_max(m, red);
    float s = 0.0f;
    for (int i = threadIdx.x; i < v; i += blockDim.x) s += expf(xr[i] - m);
    s = block_sum(s, red);
    const float inv = static_cast<float>(rows);
    for (int i = threadIdx.x; i < vp; i += blockDim.x) {
        const float p = i < v ? expf(xr[i] - m) / s : 0.0f;
        if (i == label) row_loss[r] = -logf(p + 1e-8f);
        xr[i] = i < v ? (p - (i == label ? 1.0f : 0.0f)) / inv : 0.0f;
    }
}

// loss = mean of the row terms.  Single block, fixed order per thread.
__global__ void row_loss_mean_kernel(float *__restrict__ loss, const float *__restrict__ row_loss, int rows)
{
    __shared__ float red[32];
    float s = 0.0f;
    for (int r = threadIdx.x; r < rows; r += blockDim.x) s += row_loss[r];
    s = block_sum(s, red);
    if (threadIdx.x == 0) *loss = s / static_cast<float>(rows);
}

// The loss straight from logits (no probabilities stored): per row -log(softmax[label] + 1e-8).  One block per row.
__global__ void ce_row_loss_from_logits_kernel(float *__restrict__ row_loss, const float *__restrict__ x, const int *__restrict__ labels, int v, int vp)
{
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    const float *xr = x + r * vp;
    float m = -FLT_MAX;
    for (int i = threadIdx.x; i < v; i += blockDim.x) m = fmaxf(m, xr[i]);
    m = block_max(m, red);
    float s = 0.0f;
    for (int i = threadIdx.x; i < v; i += blockDim.x) s += expf(xr[i] - m);
    s = block_sum(s, red);
    if (threadIdx.x == 0) row_loss[r] = -logf(expf(xr[labels[r]] - m) / s + 1e-8f);
}

// loss = -(1/rows) sum_r log(p[r, label[r]] + 1e-8)   (cpu_backend.cpp:493-509).  Single block, fixed order per thread.
__global__ void cross_entropy_loss_kernel(float *__restrict__ loss, const float *__restrict__ probs, const int *__restrict__ labels, int rows,
                                          int vp)
{
    __shared__ float red[32];
    float s = 0.0f;
    for (int r = threadIdx.x; r < rows; r += blockDim.x) s -= logf(probs[size_t(r) * vp + labels[r]] + 1e-8f);
    s = block_sum(s, red);
    if (threadIdx.x == 0) *loss = s / static_cast<float>(rows);
}

// ------------------------------------------------------------------------------------------------ optimiser

// AdamW with decoupled weight decay (cpu_backend.cpp:511-526); the bias-correction powers come from the host.
__global__ void adamw_kernel(float *__restrict__ p, const float *__restrict__ g, float *__restrict__ m, float *__restrict__ v, size_t n,
                             float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2)
{
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float gi = g[i];
        const float mi = beta1 * m[i] + (1.0f - beta1) * gi;
        const float vi = beta2 * v[i] + (1.0f - beta2) * gi * gi;
        m[i] = mi;
        v[i] = vi;
        const float m_hat = mi / bc1;
        const float v_hat = vi / bc2;
        p[i] -= lr * (m_hat / (sqrtf(v_hat) + eps) + wd * p[i]);
    }
}

// Gradient scaling and global-norm clipping (cpu_backend.cpp:528-556) without a host round trip:
// stage 1 scales by 1/accum_steps and writes per-block sums of squares, stage 2 adds them in order and
// stores the clip factor, stage 3 applies it when the norm exceeds max_norm.
__global__ void clip_scale_partial_kernel(float *__restrict__ g, float *__restrict__ partial, size_t n, float inv_accum)
{
    __shared__ float red[32];
    const size_t per = (n + gridDim.x - 1) / gridDim.x;
    const size_t i0 = size_t(blockIdx.x) * per, i1 = min(n, i0 + per);
    float s = 0.0f;
    for (size_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const float v = g[i] * inv_accum;
        g[i] = v;
        s += v * v;
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void clip_factor_kernel(float *__restrict__ factor, const float *__restrict__ partial, int blocks, float max_norm)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    float s = 0.0f;
    for (int i = 0; i < blocks; ++i) s += partial[i];
    const float norm = sqrtf(s);
    *factor = norm <= max_norm ? 1.0f : max_norm / (norm + 1e-6f);
}

__global__ void clip_apply_kernel(float *__restrict__ g, const float *__restrict__ factor, size_t n)
{
    const float f = *factor;
    if (f == 1.0f) return;
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) g[i] *= f;
}

}  // namespace ops
}  // namespace gptb200
