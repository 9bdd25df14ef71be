// Causal softmax attention for head size 64 on the packed qkv[B, T, 3*D] layout (cpu_backend.cpp:290-433), fp32 FMAs
// throughout, written as register-tiled block products: a block of 128 threads owns 64 query (or key) rows of one
// (batch, head) and walks over the 64-row blocks of the other side.  Every 64 x 64 x 64 block product gives each
// thread a 4 x 8 register tile (thread (ty, tx): rows 4 ty .. + 3, columns 8 tx .. + 7), fed by one 16-byte and two
// 16-byte shared-memory loads per 32 FMAs; operands that are walked along their rows are stored transposed so that
// those loads are contiguous.  The kernels for other head sizes (backend_ops.cuh) keep one row per thread group.
//
// Not part of the linear-layer path: these kernels only keep the training step's time from being dominated by
// attention once the linear layers run on the tensor cores.
#pragma once

#include <cfloat>
#include <cstddef>
#include <cuda_runtime.h>

namespace gptb200 {
namespace ops {

constexpr int kFaBlock = 64;    // rows and keys per block, and the head size
constexpr int kFaThreads = 128;
constexpr int kFaPad = 68;      // row pitch of tiles that are read down a column (keeps 16-byte alignment, spreads banks)
constexpr int kFaTile = kFaBlock * kFaBlock;   // floats

// dst[c][r] = src[(row0 + r) * stride + c]  for r, c < 64 (rows >= rows_total read as zero)
__device__ __forceinline__ void fa_load_transposed(float *dst, const float *__restrict__ src, int row0, int rows_total, size_t stride)
{
    const int r = threadIdx.x & 63;
    const bool ok = row0 + r < rows_total;
    const float4 *p = reinterpret_cast<const float4 *>(src + size_t(row0 + r) * stride);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c4 = (threadIdx.x >> 6) + 2 * i;
        const float4 v = ok ? __ldg(p + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
        dst[(4 * c4 + 0) * kFaBlock + r] = v.x;
        dst[(4 * c4 + 1) * kFaBlock + r] = v.y;
        dst[(4 * c4 + 2) * kFaBlock + r] = v.z;
        dst[(4 * c4 + 3) * kFaBlock + r] = v.w;
    }
}

// dst[r * pitch + c] = src[(row0 + r) * stride + c]
__device__ __forceinline__ void fa_load_direct(float *dst, int pitch, const float *__restrict__ src, int row0, int rows_total, size_t stride)
{
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = threadIdx.x + kFaThreads * i;
        const int r = idx >> 4, c4 = idx & 15;
        const float4 v = row0 + r < rows_total ? __ldg(reinterpret_cast<const float4 *>(src + size_t(row0 + r) * stride) + c4)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4 *>(dst + r * pitch + 4 * c4) = v;
    }
}

// acc[i][j] += sum_k a_t[k][4 ty + i] * b_t[k][8 tx + j]   (both operands stored with the reduction index first)
__device__ __forceinline__ void fa_block_product_tt(float (&acc)[4][8], const float *a_t, const float *b_t, int ty, int tx)
{
#pragma unroll 8
    for (int k = 0; k < kFaBlock; ++k) {
        const float4 a = *reinterpret_cast<const float4 *>(a_t + k * kFaBlock + 4 * ty);
        const float4 b0 = *reinterpret_cast<const float4 *>(b_t + k * kFaBlock + 8 * tx);
        const float4 b1 = *reinterpret_cast<const float4 *>(b_t + k * kFaBlock + 8 * tx + 4);
        const float av[4] = {a.x, a.y, a.z, a.w};
        const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] += av[i] * bv[j];
    }
}

// acc[i][j] += sum_k a[(4 ty + i) * kFaPad + k] * b[k][8 tx + j]   (a stored row by row with the padded pitch)
__device__ __forceinline__ void fa_block_product_nt(float (&acc)[4][8], const float *a, const float *b, int ty, int tx)
{
#pragma unroll 8
    for (int k = 0; k < kFaBlock; ++k) {
        float av[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) av[i] = a[(4 * ty + i) * kFaPad + k];
        const float4 b0 = *reinterpret_cast<const float4 *>(b + k * kFaBlock + 8 * tx);
        const float4 b1 = *reinterpret_cast<const float4 *>(b + k * kFaBlock + 8 * tx + 4);
        const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] += av[i] * bv[j];
    }
}

// value combined over the eight threads (tx = 0..7) that share a row group
__device__ __forceinline__ float fa_row_max(float v)
{
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
}

__device__ __forceinline__ float fa_row_sum(float v)
{
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v + __shfl_xor_sync(0xffffffffu, v, 4);
}

constexpr int kFaForwardSmem = (3 * kFaTile + kFaBlock * kFaPad) * 4;

// y[b, s1, h*64 + :] = softmax_{s2 <= s1}(q.k / 8) . v ;  logsumexp[b, s1, h] = max + log(sum)
// grid (row blocks, heads, batch); the row blocks with the most keys are scheduled first.
__global__ void __launch_bounds__(kFaThreads)
attention64_forward_kernel(float *__restrict__ y, float *__restrict__ logsumexp, const float *__restrict__ qkv, int seq_len, int d_model,
                           int num_heads)
{
    extern __shared__ __align__(16) float fa_smem[];
    float *q_t = fa_smem;                 // [dim][row]
    float *k_t = q_t + kFaTile;           // [dim][key]
    float *v_s = k_t + kFaTile;           // [key][dim]
    float *p_s = v_s + kFaTile;           // [row][key], padded pitch
    const int b = blockIdx.z, h = blockIdx.y;
    const int rb = gridDim.x - 1 - blockIdx.x;
    const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
    const size_t stride = 3 * size_t(d_model);
    const float *base = qkv + size_t(b) * seq_len * stride + h * kFaBlock;
    const int row0 = rb * kFaBlock;
    const float scale = 0.125f;           // 1 / sqrt(64)

    fa_load_transposed(q_t, base, row0, seq_len, stride);
    float acc[4][8], m[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m[i] = -FLT_MAX;
        l[i] = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
    }
    for (int kb = 0; kb <= rb; ++kb) {
        __syncthreads();                  // the previous block's tiles are no longer read
        fa_load_transposed(k_t, base + d_model, kb * kFaBlock, seq_len, stride);
        fa_load_direct(v_s, kFaBlock, base + 2 * d_model, kb * kFaBlock, seq_len, stride);
        __syncthreads();
        float s[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) s[i][j] = 0.0f;
        fa_block_product_tt(s, q_t, k_t, ty, tx);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = row0 + 4 * ty + i;
            float rmax = -FLT_MAX;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int key = kb * kFaBlock + 8 * tx + j;
                const bool keep = key <= row && key < seq_len;
                s[i][j] = keep ? s[i][j] * scale : -FLT_MAX;
                rmax = fmaxf(rmax, s[i][j]);
            }
            rmax = fa_row_max(rmax);
            const float m_new = fmaxf(m[i], rmax);
            const float corr = expf(m[i] - m_new);
            float rsum = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s[i][j] = s[i][j] == -FLT_MAX ? 0.0f : expf(s[i][j] - m_new);
                rsum += s[i][j];
            }
            l[i] = l[i] * corr + fa_row_sum(rsum);
            m[i] = m_new;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] *= corr;
            float *prow = p_s + (4 * ty + i) * kFaPad + 8 * tx;
            *reinterpret_cast<float4 *>(prow) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
            *reinterpret_cast<float4 *>(prow + 4) = make_float4(s[i][4], s[i][5], s[i][6], s[i][7]);
        }
        __syncwarp();                     // a row group's probabilities are written and read by the same warp
        fa_block_product_nt(acc, p_s, v_s, ty, tx);
        __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + 4 * ty + i;
        if (row >= seq_len) continue;
        const float inv = 1.0f / l[i];
        float *out = y + (size_t(b) * seq_len + row) * d_model + h * kFaBlock + 8 * tx;
        *reinterpret_cast<float4 *>(out) = make_float4(acc[i][0] * inv, acc[i][1] * inv, acc[i][2] * inv, acc[i][3] * inv);
        *reinterpret_cast<float4 *>(out + 4) = make_float4(acc[i][4] * inv, acc[i][5] * inv, acc[i][6] * inv, acc[i][7] * inv);
        if (tx == 0) logsumexp[(size_t(b) * seq_len + row) * num_heads + h] = m[i] + logf(l[i]);
    }
}

// D[b, s, h] = sum_d grad_y * y over the head's 64 dimensions: one warp per (b, s) row, 16 lanes per head.
__global__ void attention64_rowsum_kernel(float *__restrict__ dcache, const float *__restrict__ grad_y, const float *__restrict__ y,
                                          long long rows, int d_model, int num_heads)
{
    const int lane = threadIdx.x & 31;
    const long long row = (1LL * blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) return;   // whole warps leave together
    const float4 *g = reinterpret_cast<const float4 *>(grad_y + row * d_model);
    const float4 *o = reinterpret_cast<const float4 *>(y + row * d_model);
    for (int c0 = 0; c0 < d_model / 4; c0 += 32) {
        const int c = c0 + lane;
        float s = 0.0f;
        if (c < d_model / 4) {
            const float4 a = __ldg(g + c), b = __ldg(o + c);
            s = (a.x * b.x + a.y * b.y) + (a.z * b.z + a.w * b.w);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 8);
        if ((lane & 15) == 0 && c < d_model / 4) dcache[row * num_heads + c / 16] = s;
    }
}

// p = exp(s / 8 - L) and dS = p (dP - D) / 8 for a thread's 4 x 8 tile; masked entries (key > row or beyond the sequence) are 0.
__device__ __forceinline__ void fa_probabilities_and_ds(float (&s)[4][8], float (&dp)[4][8], const float (&lse)[4], const float (&dsum)[4],
                                                        int row0, int key0, int seq_len, int ty, int tx)
{
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + 4 * ty + i;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int key = key0 + 8 * tx + j;
            const bool keep = key <= row && row < seq_len;
            const float p = keep ? expf(s[i][j] * 0.125f - lse[i]) : 0.0f;
            s[i][j] = p;
            dp[i][j] = p * (dp[i][j] - dsum[i]) * 0.125f;
        }
    }
}

constexpr int kFaDqSmem = (5 * kFaTile + kFaBlock * kFaPad) * 4;
constexpr int kFaDkvSmem = 6 * kFaTile * 4;

// grad_q[s1] = sum_{s2 <= s1} dS[s1, s2] k[s2]      (grid as the forward kernel: one block per 64 query rows)
__global__ void __launch_bounds__(kFaThreads)
attention64_backward_dq_kernel(float *__restrict__ grad_qkv, const float *__restrict__ dcache, const float *__restrict__ logsumexp,
                               const float *__restrict__ grad_y, const float *__restrict__ qkv, int seq_len, int d_model, int num_heads)
{
    extern __shared__ __align__(16) float fa_smem[];
    float *q_t = fa_smem;                 // [dim][row]
    float *do_t = q_t + kFaTile;          // [dim][row]
    float *k_t = do_t + kFaTile;          // [dim][key]
    float *v_t = k_t + kFaTile;           // [dim][key]
    float *k_d = v_t + kFaTile;           // [key][dim]
    float *ds_s = k_d + kFaTile;          // [row][key], padded pitch
    const int b = blockIdx.z, h = blockIdx.y;
    const int rb = gridDim.x - 1 - blockIdx.x;
    const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
    const size_t stride = 3 * size_t(d_model);
    const float *base = qkv + size_t(b) * seq_len * stride + h * kFaBlock;
    const float *gy = grad_y + size_t(b) * seq_len * d_model + h * kFaBlock;
    const int row0 = rb * kFaBlock;

    fa_load_transposed(q_t, base, row0, seq_len, stride);
    fa_load_transposed(do_t, gy, row0, seq_len, d_model);
    float lse[4], dsum[4], acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = min(row0 + 4 * ty + i, seq_len - 1);
        lse[i] = logsumexp[(size_t(b) * seq_len + row) * num_heads + h];
        dsum[i] = dcache[(size_t(b) * seq_len + row) * num_heads + h];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
    }
    for (int kb = 0; kb <= rb; ++kb) {
        __syncthreads();
        fa_load_transposed(k_t, base + d_model, kb * kFaBlock, seq_len, stride);
        fa_load_transposed(v_t, base + 2 * d_model, kb * kFaBlock, seq_len, stride);
        fa_load_direct(k_d, kFaBlock, base + d_model, kb * kFaBlock, seq_len, stride);
        __syncthreads();
        float s[4][8], dp[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) s[i][j] = dp[i][j] = 0.0f;
        fa_block_product_tt(s, q_t, k_t, ty, tx);
        fa_block_product_tt(dp, do_t, v_t, ty, tx);
        fa_probabilities_and_ds(s, dp, lse, dsum, row0, kb * kFaBlock, seq_len, ty, tx);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float *row = ds_s + (4 * ty + i) * kFaPad + 8 * tx;
            *reinterpret_cast<float4 *>(row) = make_float4(dp[i][0], dp[i][1], dp[i][2], dp[i][3]);
            *reinterpret_cast<float4 *>(row + 4) = make_float4(dp[i][4], dp[i][5], dp[i][6], dp[i][7]);
        }
        __syncwarp();                     // a row group's dS is written and read by the same warp
        fa_block_product_nt(acc, ds_s, k_d, ty, tx);
        __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + 4 * ty + i;
        if (row >= seq_len) continue;
        float *out = grad_qkv + (size_t(b) * seq_len + row) * stride + h * kFaBlock + 8 * tx;
        *reinterpret_cast<float4 *>(out) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        *reinterpret_cast<float4 *>(out + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
}

// grad_k[s2] = sum_{s1 >= s2} dS[s1, s2] q[s1],  grad_v[s2] = sum_{s1 >= s2} p[s1, s2] dO[s1]   (one block per 64 keys)
__global__ void __launch_bounds__(kFaThreads)
attention64_backward_dkv_kernel(float *__restrict__ grad_qkv, const float *__restrict__ dcache, const float *__restrict__ logsumexp,
                                const float *__restrict__ grad_y, const float *__restrict__ qkv, int seq_len, int d_model, int num_heads)
{
    extern __shared__ __align__(16) float fa_smem[];
    float *k_t = fa_smem;                 // [dim][key]
    float *v_t = k_t + kFaTile;           // [dim][key]
    float *q_t = v_t + kFaTile;           // [dim][row]; afterwards p  [row][key]
    float *do_t = q_t + kFaTile;          // [dim][row]; afterwards dS [row][key]
    float *q_d = do_t + kFaTile;          // [row][dim]
    float *do_d = q_d + kFaTile;          // [row][dim]
    const int b = blockIdx.z, h = blockIdx.y;
    const int kb = blockIdx.x;            // the key blocks with the most query rows come first
    const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
    const size_t stride = 3 * size_t(d_model);
    const float *base = qkv + size_t(b) * seq_len * stride + h * kFaBlock;
    const float *gy = grad_y + size_t(b) * seq_len * d_model + h * kFaBlock;
    const int key0 = kb * kFaBlock;
    const int num_rb = (seq_len + kFaBlock - 1) / kFaBlock;

    fa_load_transposed(k_t, base + d_model, key0, seq_len, stride);
    fa_load_transposed(v_t, base + 2 * d_model, key0, seq_len, stride);
    float dk[4][8], dv[4][8];             // rows: keys 4 ty .. + 3, columns: dims 8 tx .. + 7
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) dk[i][j] = dv[i][j] = 0.0f;
    for (int rb = kb; rb < num_rb; ++rb) {
        const int row0 = rb * kFaBlock;
        __syncthreads();                  // p, dS, q_d, do_d of the previous block are no longer read
        fa_load_transposed(q_t, base, row0, seq_len, stride);
        fa_load_transposed(do_t, gy, row0, seq_len, d_model);
        fa_load_direct(q_d, kFaBlock, base, row0, seq_len, stride);
        fa_load_direct(do_d, kFaBlock, gy, row0, seq_len, d_model);
        float lse[4], dsum[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = min(row0 + 4 * ty + i, seq_len - 1);
            lse[i] = logsumexp[(size_t(b) * seq_len + row) * num_heads + h];
            dsum[i] = dcache[(size_t(b) * seq_len + row) * num_heads + h];
        }
        __syncthreads();
        float s[4][8], dp[4][8];          // rows: queries 4 ty .. + 3, columns: keys 8 tx .. + 7
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) s[i][j] = dp[i][j] = 0.0f;
        fa_block_product_tt(s, q_t, k_t, ty, tx);
        fa_block_product_tt(dp, do_t, v_t, ty, tx);
        fa_probabilities_and_ds(s, dp, lse, dsum, row0, key0, seq_len, ty, tx);
        __syncthreads();                  // every thread is done with q_t / do_t: they become p and dS, [row][key]
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float *prow = q_t + (4 * ty + i) * kFaBlock + 8 * tx;
            float *drow = do_t + (4 * ty + i) * kFaBlock + 8 * tx;
            *reinterpret_cast<float4 *>(prow) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
            *reinterpret_cast<float4 *>(prow + 4) = make_float4(s[i][4], s[i][5], s[i][6], s[i][7]);
            *reinterpret_cast<float4 *>(drow) = make_float4(dp[i][0], dp[i][1], dp[i][2], dp[i][3]);
            *reinterpret_cast<float4 *>(drow + 4) = make_float4(dp[i][4], dp[i][5], dp[i][6], dp[i][7]);
        }
        __syncthreads();
        fa_block_product_tt(dv, q_t, do_d, ty, tx);    // sum over rows of p[row][key] dO[row][dim]
        fa_block_product_tt(dk, do_t, q_d, ty, tx);    // sum over rows of dS[row][key] q[row][dim]
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int key = key0 + 4 * ty + i;
        if (key >= seq_len) continue;
        float *out = grad_qkv + (size_t(b) * seq_len + key) * stride + d_model + h * kFaBlock + 8 * tx;
        *reinterpret_cast<float4 *>(out) = make_float4(dk[i][0], dk[i][1], dk[i][2], dk[i][3]);
        *reinterpret_cast<float4 *>(out + 4) = make_float4(dk[i][4], dk[i][5], dk[i][6], dk[i][7]);
        out += d_model;
        *reinterpret_cast<float4 *>(out) = make_float4(dv[i][0], dv[i][1], dv[i][2], dv[i][3]);
        *reinterpret_cast<float4 *>(out + 4) = make_float4(dv[i][4], dv[i][5], dv[i][6], dv[i][7]);
    }
}

}  // namespace ops
}  // namespace gptb200
