// extern "C" entry points of the operators that are not on the linear-layer hot path (see backend_ops.cuh).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <initializer_list>

#include "ctx_internal.h"
#include "backend_ops.cuh"
#include "attention_gemm.cuh"
#include "attention_tiled.cuh"
#include "layernorm_warp.cuh"
#include "optimizer_fused.cuh"
#include "decode_ops.cuh"
#include "softmax_stream.cuh"

using namespace gptb200;

namespace {

int blocks_for(const gptb200_ctx *ctx, size_t n, int threads)
{
    const size_t want = (n + threads - 1) / threads;
    return static_cast<int>(std::max<size_t>(1, std::min<size_t>(want, size_t(ctx->num_sms) * 16)));
}

int launched(gptb200_ctx *ctx, int n = 1)
{
    ctx->launches += n;
    CUDA_TRY(ctx, cudaGetLastError());
    return GPTB200_OK;
}

template <int HD, int TPR>
int attention_forward_t(gptb200_ctx *ctx, float *y, float *lse, const float *qkv, int batch, int seq_len, int d, int heads)
{
    dim3 grid((seq_len + ops::kAttnRowsPerBlock - 1) / ops::kAttnRowsPerBlock, heads, batch);
    ops::attention_forward_kernel<HD, TPR><<<grid, ops::kAttnRowsPerBlock * TPR, 0, ctx->stream>>>(y, lse, qkv, seq_len, d, heads);
    return launched(ctx);
}

template <int HD, int TPR>
int attention_backward_t(gptb200_ctx *ctx, float *gqkv, float *dcache, const float *lse, const float *gy, const float *qkv, int batch,
                         int seq_len, int d, int heads)
{
    dim3 grid((seq_len + ops::kAttnRowsPerBlock - 1) / ops::kAttnRowsPerBlock, heads, batch);
    ops::attention_backward_dq_kernel<HD, TPR><<<grid, ops::kAttnRowsPerBlock * TPR, 0, ctx->stream>>>(gqkv, dcache, lse, gy, qkv, seq_len, d, heads);
    ops::attention_backward_dkv_kernel<HD, TPR><<<grid, ops::kAttnRowsPerBlock * TPR, 0, ctx->stream>>>(gqkv, dcache, lse, gy, qkv, seq_len, d, heads);
    return launched(ctx, 2);
}

bool aligned16_all(std::initializer_list<const void *> ptrs)
{
    for (const void *p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) & 15u) return false;
    return true;
}

// Raises the dynamic shared-memory limit of a kernel once per context (the attribute is per device).
template <typename Kernel>
cudaError_t allow_smem(gptb200_ctx *ctx, Kernel kernel, int bytes)
{
    const void *key = reinterpret_cast<const void *>(kernel);
    if (ctx->configured.count(key)) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) ctx->configured.insert(key);
    return e;
}

// Long rows of logits (16 K - 51 K floats, 16-byte aligned) and more rows than SMs: the persistent row kernels of softmax_stream.cuh.
bool row_stream_applies(const gptb200_ctx *ctx, int rows, int vocab_padded)
{
    return ctx->softmax_stream && vocab_padded % 4 == 0 && vocab_padded > 1024 * 4 * 4 && vocab_padded <= ops::kRowStreamThreads * 4 * ops::kRowStreamVecs &&
           rows > ctx->num_sms;
}

// Head size 64 with 16-byte aligned tensors: the register-tiled kernels of attention_tiled.cuh.
int attention64_forward(gptb200_ctx *ctx, float *y, float *lse, const float *qkv, int batch, int seq_len, int d, int heads)
{
    CUDA_TRY(ctx, allow_smem(ctx, ops::attention64_forward_kernel, ops::kFaForwardSmem));
    dim3 grid((seq_len + ops::kFaBlock - 1) / ops::kFaBlock, heads, batch);
    ops::attention64_forward_kernel<<<grid, ops::kFaThreads, ops::kFaForwardSmem, ctx->stream>>>(y, lse, qkv, seq_len, d, heads);
    return launched(ctx);
}

template <int VEC>
void layernorm_forward_warp(gptb200_ctx *ctx, float *y, float *means, float *vars, float *x, const float *residual, const float *gamma,
                            const float *beta, int rows)
{
    const int blocks = (rows + ops::kLnWarpsPerBlock - 1) / ops::kLnWarpsPerBlock;
    ops::layernorm_forward_warp_kernel<VEC><<<blocks, ops::kLnWarpsPerBlock * 32, 0, ctx->stream>>>(y, means, vars, x, residual, gamma, beta, rows);
}

template <int VEC>
void layernorm_backward_warp(gptb200_ctx *ctx, int blocks, float *gx, float *wg, float *wb, const float *gy, const float *gres, const float *x,
                             const float *means, const float *vars, const float *gamma, int rows)
{
    ops::layernorm_backward_warp_kernel<VEC><<<blocks, ops::kLnWarpsPerBlock * 32, 0, ctx->stream>>>(gx, wg, wb, gy, gres, x, means, vars, gamma, rows);
}

// Row lengths the one-warp-per-row LayerNorm kernels cover.
bool layernorm_warp_ok(int d) { return d % 128 == 0 && d >= 128 && d <= 1024; }

int attention64_backward(gptb200_ctx *ctx, float *gqkv, float *dcache, const float *lse, const float *gy, const float *y, const float *qkv,
                         int batch, int seq_len, int d, int heads)
{
    CUDA_TRY(ctx, allow_smem(ctx, ops::attention64_backward_dq_kernel, ops::kFaDqSmem));
    CUDA_TRY(ctx, allow_smem(ctx, ops::attention64_backward_dkv_kernel, ops::kFaDkvSmem));
    const long long rows = 1LL * batch * seq_len;
    ops::attention64_rowsum_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, ctx->stream>>>(dcache, gy, y, rows, d, heads);
    dim3 grid((seq_len + ops::kFaBlock - 1) / ops::kFaBlock, heads, batch);
    ops::attention64_backward_dq_kernel<<<grid, ops::kFaThreads, ops::kFaDqSmem, ctx->stream>>>(gqkv, dcache, lse, gy, qkv, seq_len, d, heads);
    ops::attention64_backward_dkv_kernel<<<grid, ops::kFaThreads, ops::kFaDkvSmem, ctx->stream>>>(gqkv, dcache, lse, gy, qkv, seq_len, d, heads);
    return launched(ctx, 3);
}

// Scratch of the tensor-core attention: `bytes` of device memory, kept by the context.  false (and no error left behind) when the
// device cannot give it: the caller then takes the fp32 FMA kernels, which need none.
bool attention_scratch(gptb200_ctx *ctx, size_t bytes)
{
    if (bytes <= ctx->attn_ws_bytes) return true;
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return false;   // queued launches may still use the old buffer
    if (ctx->attn_ws) cudaFree(ctx->attn_ws);
    ctx->attn_ws = nullptr;
    ctx->attn_ws_bytes = 0;
    if (cudaMalloc(&ctx->attn_ws, bytes) != cudaSuccess) {
        cudaGetLastError();
        ctx->attn_ws = nullptr;
        return false;
    }
    ctx->attn_ws_bytes = bytes;
    return true;
}

bool attention_gemm_applies(const gptb200_ctx *ctx, int seq_len, int d, int heads)
{
    const bool on = ctx->attention_gemm != 0;
    return on && d / heads == 64 && seq_len % 4 == 0 && seq_len >= 4 && seq_len <= 1024;
}

// Sequences per group of launches: bounds the scratch (one score buffer forward, two backward).  Groups small enough for the
// scores to stay in L2 were measured slower than one group (GPT-2 124M, 64 sequences of 256 tokens, TF32: forward 196 us in one
// group, 251 us in groups of 50 MB): these launches are bound by their epilogues and fixed costs, not by DRAM.
int attention_group(const gptb200_ctx *ctx, int batch, int seq_len, int heads, int buffers)
{
    const double per_seq = 4.0 * heads * seq_len * seq_len * buffers;
    const long long g = static_cast<long long>(ctx->attention_group_mb * 1048576.0 / per_seq);
    return static_cast<int>(std::max(1LL, std::min<long long>(batch, g)));
}

// Head slices of packed rows and the score buffer s[b][q][h][k] as batched operands (row pitch, head stride, sequence stride).
BatchedOperand head_slice(const float *base, bool mn, int row_floats, int seq_len) { return {base, mn, row_floats, 64, 1LL * seq_len * row_floats}; }
BatchedOperand score_rows(const float *s, bool mn, int seq_len, int heads) { return {s, mn, 1LL * heads * seq_len, seq_len, 1LL * seq_len * heads * seq_len}; }

template <typename... Args>
void launch_scores_softmax(gptb200_ctx *ctx, int T, unsigned blocks, Args... args)
{
    if (T <= 256)
        ops::attention_scores_softmax_kernel<2><<<blocks, ops::kScoreRowsPerBlock * 32, 0, ctx->stream>>>(args...);
    else if (T <= 512)
        ops::attention_scores_softmax_kernel<4><<<blocks, ops::kScoreRowsPerBlock * 32, 0, ctx->stream>>>(args...);
    else
        ops::attention_scores_softmax_kernel<8><<<blocks, ops::kScoreRowsPerBlock * 32, 0, ctx->stream>>>(args...);
}

int attention_gemm_forward(gptb200_ctx *ctx, float *y, float *lse, const float *qkv, int batch, int seq_len, int d, int heads)
{
    const int T = seq_len, G = attention_group(ctx, batch, T, heads, 1);
    if (!attention_scratch(ctx, sizeof(float) * G * T * heads * T)) return -1;
    float *s = ctx->attn_ws;
    const long long sl = 1LL * heads * T, so = 1LL * T * heads * T;
    for (int b0 = 0; b0 < batch; b0 += G) {
        const int nb = std::min(G, batch - b0);
        const float *x = qkv + 1LL * b0 * T * 3 * d;
        int rc = run_gemm_batched(ctx, s, sl, T, so, head_slice(x, false, 3 * d, T), head_slice(x + d, false, 3 * d, T), T, T, 64, heads, nb, true);   // the row kernel reads columns <= row only
        if (rc) return rc;
        const long long rows = 1LL * nb * T * heads;
        const unsigned blocks = static_cast<unsigned>((rows + ops::kScoreRowsPerBlock - 1) / ops::kScoreRowsPerBlock);
        launch_scores_softmax(ctx, T, blocks, s, lse + 1LL * b0 * T * heads, T, heads, 0.125f, rows);
        rc = launched(ctx);
        if (rc) return rc;
        rc = run_gemm_batched(ctx, y + 1LL * b0 * T * d, d, 64, 1LL * T * d, score_rows(s, false, T, heads), head_slice(x + 2 * d, true, 3 * d, T), T, 64, T, heads, nb);
        if (rc) return rc;
    }
    return GPTB200_OK;
}

int attention_gemm_backward(gptb200_ctx *ctx, float *gqkv, float *dcache, const float *lse, const float *gy, const float *y, const float *qkv, int batch,
                            int seq_len, int d, int heads)
{
    const int T = seq_len, G = attention_group(ctx, batch, T, heads, 2);
    if (!attention_scratch(ctx, 2 * sizeof(float) * G * T * heads * T)) return -1;
    float *s = ctx->attn_ws, *dp = ctx->attn_ws + 1LL * G * T * heads * T;
    ops::attention64_rowsum_kernel<<<static_cast<unsigned>((1LL * batch * T + 7) / 8), 256, 0, ctx->stream>>>(dcache, gy, y, 1LL * batch * T, d, heads);
    int rc = launched(ctx);
    if (rc) return rc;
    const long long sl = 1LL * heads * T, so = 1LL * T * heads * T, xo = 1LL * T * 3 * d;
    for (int b0 = 0; b0 < batch; b0 += G) {
        const int nb = std::min(G, batch - b0);
        const float *x = qkv + b0 * xo, *g = gy + 1LL * b0 * T * d;
        float *gx = gqkv + b0 * xo;
        rc = run_gemm_batched(ctx, s, sl, T, so, head_slice(x, false, 3 * d, T), head_slice(x + d, false, 3 * d, T), T, T, 64, heads, nb, true);   // the row kernel reads columns <= row only
        if (rc) return rc;
        rc = run_gemm_batched(ctx, dp, sl, T, so, head_slice(g, false, d, T), head_slice(x + 2 * d, false, 3 * d, T), T, T, 64, heads, nb, true);   // the row kernel reads columns <= row only
        if (rc) return rc;
        const long long rows = 1LL * nb * T * heads;
        const unsigned blocks = static_cast<unsigned>((rows + ops::kScoreRowsPerBlock - 1) / ops::kScoreRowsPerBlock);
        ops::attention_scores_backward_kernel<<<blocks, ops::kScoreRowsPerBlock * 32, 0, ctx->stream>>>(s, dp, lse + 1LL * b0 * T * heads,
                                                                                                     dcache + 1LL * b0 * T * heads, T, heads, 0.125f, rows);
        rc = launched(ctx);
        if (rc) return rc;
        // grad_v = P^T . grad_y,  grad_k = dS^T . Q,  grad_q = dS . K  (dS carries the 1 / 8)
        rc = run_gemm_batched(ctx, gx + 2 * d, 3 * d, 64, xo, score_rows(s, true, T, heads), head_slice(g, true, d, T), T, 64, T, heads, nb);
        if (rc) return rc;
        rc = run_gemm_batched(ctx, gx + d, 3 * d, 64, xo, score_rows(dp, true, T, heads), head_slice(x, true, 3 * d, T), T, 64, T, heads, nb);
        if (rc) return rc;
        rc = run_gemm_batched(ctx, gx, 3 * d, 64, xo, score_rows(dp, false, T, heads), head_slice(x + d, true, 3 * d, T), T, 64, T, heads, nb);
        if (rc) return rc;
    }
    return GPTB200_OK;
}

}  // namespace

#define NEED(ctx, cond)                                                                        \
    do {                                                                                       \
        if (!(ctx)) return GPTB200_ERR_INVALID_ARG;                                            \
        if (!(cond)) return fail(ctx, GPTB200_ERR_INVALID_ARG, "%s: invalid argument (%s)", __func__, #cond); \
    } while (0)

extern "C" {

int gptb200_fill_normal(gptb200_ctx *ctx, float *ptr, float mean, float stddev, size_t count, unsigned long long seed,
                        unsigned long long offset)
{
    NEED(ctx, ptr || count == 0);
    if (count == 0) return GPTB200_OK;
    ops::fill_normal_kernel<<<blocks_for(ctx, count, 256), 256, 0, ctx->stream>>>(ptr, mean, stddev, count, seed, offset);
    return launched(ctx);
}

int gptb200_fill_const(gptb200_ctx *ctx, float *ptr, float value, size_t count)
{
    NEED(ctx, ptr || count == 0);
    if (count == 0) return GPTB200_OK;
    ops::fill_const_kernel<<<blocks_for(ctx, count, 256), 256, 0, ctx->stream>>>(ptr, value, count);
    return launched(ctx);
}

int gptb200_embedding_forward(gptb200_ctx *ctx, float *y, const float *wte, const float *wpe, const int *tokens, int batch, int seq_len,
                              int d)
{
    NEED(ctx, batch >= 0 && seq_len >= 0 && d >= 0);
    const long long rows = 1LL * batch * seq_len;
    if (rows == 0 || d == 0) return GPTB200_OK;
    NEED(ctx, y && wte && wpe && tokens && rows <= 0x7fffffffLL);
    ops::embedding_forward_kernel<<<static_cast<unsigned>(rows), 256, 0, ctx->stream>>>(y, wte, wpe, tokens, static_cast<int>(rows), seq_len, d);
    return launched(ctx);
}

int gptb200_embedding_backward(gptb200_ctx *ctx, float *grad_wte, float *grad_wpe, const float *grad_y, const int *tokens, int batch,
                               int seq_len, int d)
{
    NEED(ctx, batch >= 0 && seq_len >= 0 && d >= 0);
    if (1LL * batch * seq_len == 0 || d == 0) return GPTB200_OK;
    NEED(ctx, grad_wte && grad_wpe && grad_y && tokens);
    ops::embedding_backward_kernel<<<seq_len, 256, 0, ctx->stream>>>(grad_wte, grad_wpe, grad_y, tokens, batch, seq_len, d);
    return launched(ctx);
}

int gptb200_embedding_backward_scaled(gptb200_ctx *ctx, float *grad_wte, float *grad_wpe, const float *grad_y, const int *tokens, int batch,
                                      int seq_len, int d, float scale)
{
    NEED(ctx, batch >= 0 && seq_len >= 0 && d >= 0);
    if (1LL * batch * seq_len == 0 || d == 0) return GPTB200_OK;
    NEED(ctx, grad_wte && grad_wpe && grad_y && tokens);
    ops::embedding_backward_scaled_kernel<<<seq_len, 256, 0, ctx->stream>>>(grad_wte, grad_wpe, grad_y, tokens, batch, seq_len, d, scale);
    return launched(ctx);
}

int gptb200_layernorm_forward(gptb200_ctx *ctx, float *y, float *means, float *vars, float *x, const float *residual, const float *gamma,
                              const float *beta, int rows, int d)
{
    NEED(ctx, rows >= 0 && d >= 0);
    if (rows == 0 || d == 0) return GPTB200_OK;
    NEED(ctx, y && means && vars && x && gamma && beta);
    if (layernorm_warp_ok(d) && aligned16_all({y, x, residual, gamma, beta})) {
        switch (d / 128) {
            case 1: layernorm_forward_warp<1>(ctx, y, means, vars, x, residual, gamma, beta, rows); break;
            case 2: layernorm_forward_warp<2>(ctx, y, means, vars, x, residual, gamma, beta, rows); break;
            case 3: layernorm_forward_warp<3>(ctx, y, means, vars, x, residual, gamma, beta, rows); break;
            case 4: layernorm_forward_warp<4>(ctx, y, means, vars, x, residual, gamma, beta, rows); break;
            case 5: layernorm_forward_warp<5>(ctx, y, means, vars, x, residual, gamma, beta, rows); break;
            case 6: layernorm_forward_warp<6>(ctx, y, means, vars, x, residual, gamma, beta, rows); break;
            case 7: layernorm_forward_warp<7>(ctx, y, means, vars, x, residual, gamma, beta, rows); break;
            default: layernorm_forward_warp<8>(ctx, y, means, vars, x, residual, gamma, beta, rows); break;
        }
        return launched(ctx);
    }
    const int threads = std::min(1024, std::max(32, ((d + 31) / 32) * 32));
    ops::layernorm_forward_kernel<<<rows, threads, 0, ctx->stream>>>(y, means, vars, x, residual, gamma, beta, d);
    return launched(ctx);
}

int gptb200_layernorm_backward(gptb200_ctx *ctx, float *grad_x, float *grad_gamma, float *grad_beta, const float *grad_y,
                               const float *grad_residual, const float *x, const float *means, const float *vars, const float *gamma,
                               int rows, int d)
{
    NEED(ctx, rows >= 0 && d >= 0);
    if (rows == 0 || d == 0) return GPTB200_OK;
    NEED(ctx, grad_x && grad_gamma && grad_beta && grad_y && x && means && vars && gamma);
    if (layernorm_warp_ok(d) && aligned16_all({grad_x, grad_y, grad_residual, x, gamma})) {
        const int blocks = std::max(1, std::min((rows + ops::kLnWarpsPerBlock - 1) / ops::kLnWarpsPerBlock, ctx->num_sms * 2));
        const int rc = ensure_workspace(ctx, size_t(2) * blocks * d * sizeof(float));
        if (rc) return rc;
        float *wg = ctx->ws, *wb = ctx->ws + size_t(blocks) * d;
        switch (d / 128) {
            case 1: layernorm_backward_warp<1>(ctx, blocks, grad_x, wg, wb, grad_y, grad_residual, x, means, vars, gamma, rows); break;
            case 2: layernorm_backward_warp<2>(ctx, blocks, grad_x, wg, wb, grad_y, grad_residual, x, means, vars, gamma, rows); break;
            case 3: layernorm_backward_warp<3>(ctx, blocks, grad_x, wg, wb, grad_y, grad_residual, x, means, vars, gamma, rows); break;
            case 4: layernorm_backward_warp<4>(ctx, blocks, grad_x, wg, wb, grad_y, grad_residual, x, means, vars, gamma, rows); break;
            case 5: layernorm_backward_warp<5>(ctx, blocks, grad_x, wg, wb, grad_y, grad_residual, x, means, vars, gamma, rows); break;
            case 6: layernorm_backward_warp<6>(ctx, blocks, grad_x, wg, wb, grad_y, grad_residual, x, means, vars, gamma, rows); break;
            case 7: layernorm_backward_warp<7>(ctx, blocks, grad_x, wg, wb, grad_y, grad_residual, x, means, vars, gamma, rows); break;
            default: layernorm_backward_warp<8>(ctx, blocks, grad_x, wg, wb, grad_y, grad_residual, x, means, vars, gamma, rows); break;
        }
        ops::layernorm_backward_params_final_kernel<<<(d + 31) / 32, dim3(32, 8), 0, ctx->stream>>>(grad_gamma, grad_beta, wg, wb, d, blocks);
        return launched(ctx, 2);
    }
    const int threads = std::min(1024, std::max(32, ((d + 31) / 32) * 32));
    ops::layernorm_backward_dx_kernel<<<rows, threads, 0, ctx->stream>>>(grad_x, grad_y, grad_residual, x, means, vars, gamma, d);
    const int col_groups = (d + 31) / 32;
    int chunks = std::max(1, std::min((ctx->num_sms * 4 + col_groups - 1) / col_groups, (rows + 63) / 64));
    const int rows_per_chunk = (rows + chunks - 1) / chunks;
    chunks = (rows + rows_per_chunk - 1) / rows_per_chunk;
    const int rc = ensure_workspace(ctx, size_t(2) * chunks * d * sizeof(float));
    if (rc) return rc;
    float *wg = ctx->ws, *wb = ctx->ws + size_t(chunks) * d;
    ops::layernorm_backward_params_partial_kernel<<<dim3(col_groups, chunks), dim3(32, 8), 0, ctx->stream>>>(wg, wb, grad_y, x, means, vars,
                                                                                                             rows, d, rows_per_chunk);
    ops::layernorm_backward_params_final_kernel<<<(d + 31) / 32, dim3(32, 8), 0, ctx->stream>>>(grad_gamma, grad_beta, wg, wb, d, chunks);
    return launched(ctx, 3);
}

int gptb200_attention_forward(gptb200_ctx *ctx, float *y, float *logsumexp, const float *qkv, int batch, int seq_len, int d, int heads)
{
    NEED(ctx, batch >= 0 && seq_len >= 0 && d >= 0 && heads > 0 && d % heads == 0);
    if (1LL * batch * seq_len * d == 0) return GPTB200_OK;
    NEED(ctx, y && logsumexp && qkv && batch <= 65535 && heads <= 65535);
    switch (d / heads) {
        case 8: return attention_forward_t<8, 1>(ctx, y, logsumexp, qkv, batch, seq_len, d, heads);
        case 16: return attention_forward_t<16, 1>(ctx, y, logsumexp, qkv, batch, seq_len, d, heads);
        case 32: return attention_forward_t<32, 1>(ctx, y, logsumexp, qkv, batch, seq_len, d, heads);
        case 64:
            if (attention_gemm_applies(ctx, seq_len, d, heads) && aligned16_all({y, qkv})) {
                const int rc = attention_gemm_forward(ctx, y, logsumexp, qkv, batch, seq_len, d, heads);
                if (rc >= 0) return rc;   // -1: no memory for the score matrices; the FMA kernels need none
            }
            if (ctx->attention_tiled && d % 4 == 0 && aligned16_all({y, qkv})) return attention64_forward(ctx, y, logsumexp, qkv, batch, seq_len, d, heads);
            return attention_forward_t<64, 2>(ctx, y, logsumexp, qkv, batch, seq_len, d, heads);
        case 128: return attention_forward_t<128, 4>(ctx, y, logsumexp, qkv, batch, seq_len, d, heads);
        default: return fail(ctx, GPTB200_ERR_INVALID_ARG, "attention: head size %d not in {8,16,32,64,128}", d / heads);
    }
}

int gptb200_attention_backward(gptb200_ctx *ctx, float *grad_qkv, float *d_cache, const float *logsumexp, const float *grad_y,
                               const float *y, const float *qkv, int batch, int seq_len, int d, int heads)
{
    NEED(ctx, batch >= 0 && seq_len >= 0 && d >= 0 && heads > 0 && d % heads == 0);
    if (1LL * batch * seq_len * d == 0) return GPTB200_OK;
    NEED(ctx, grad_qkv && d_cache && logsumexp && grad_y && y && qkv && batch <= 65535 && heads <= 65535);
    if (attention_gemm_applies(ctx, seq_len, d, heads) && aligned16_all({grad_qkv, grad_y, y, qkv})) {
        const int rc = attention_gemm_backward(ctx, grad_qkv, d_cache, logsumexp, grad_y, y, qkv, batch, seq_len, d, heads);
        if (rc >= 0) return rc;
    }
    if (d / heads == 64 && ctx->attention_tiled && d % 4 == 0 && aligned16_all({grad_qkv, grad_y, y, qkv}))
        return attention64_backward(ctx, grad_qkv, d_cache, logsumexp, grad_y, y, qkv, batch, seq_len, d, heads);
    const long long rh = 1LL * batch * seq_len * heads;
    ops::attention_rowsum_kernel<<<static_cast<unsigned>((rh + 255) / 256), 256, 0, ctx->stream>>>(d_cache, grad_y, y, batch * seq_len, d, heads);
    ctx->launches++;
    switch (d / heads) {
        case 8: return attention_backward_t<8, 1>(ctx, grad_qkv, d_cache, logsumexp, grad_y, qkv, batch, seq_len, d, heads);
        case 16: return attention_backward_t<16, 1>(ctx, grad_qkv, d_cache, logsumexp, grad_y, qkv, batch, seq_len, d, heads);
        case 32: return attention_backward_t<32, 1>(ctx, grad_qkv, d_cache, logsumexp, grad_y, qkv, batch, seq_len, d, heads);
        case 64: return attention_backward_t<64, 2>(ctx, grad_qkv, d_cache, logsumexp, grad_y, qkv, batch, seq_len, d, heads);
        case 128: return attention_backward_t<128, 4>(ctx, grad_qkv, d_cache, logsumexp, grad_y, qkv, batch, seq_len, d, heads);
        default: return fail(ctx, GPTB200_ERR_INVALID_ARG, "attention: head size %d not in {8,16,32,64,128}", d / heads);
    }
}

int gptb200_softmax_forward(gptb200_ctx *ctx, float *y, const float *x, int rows, int vocab, int vocab_padded)
{
    NEED(ctx, rows >= 0 && vocab >= 0 && vocab_padded >= vocab);
    if (rows == 0 || vocab_padded == 0) return GPTB200_OK;
    NEED(ctx, y && x);
    if (row_stream_applies(ctx, rows, vocab_padded) && aligned16_all({y, x})) {
        CUDA_TRY(ctx, allow_smem(ctx, ops::softmax_row_stream_kernel<0>, ops::kRowStreamSmem));
        ops::softmax_row_stream_kernel<0><<<std::min(rows, ctx->num_sms), ops::kRowStreamThreads, ops::kRowStreamSmem, ctx->stream>>>(
            y, const_cast<float *>(x), nullptr, nullptr, rows, vocab, vocab_padded, ctx->d_status);
    } else if (vocab_padded % 4 == 0 && vocab_padded <= 512 * 4 * 25 && vocab_padded > 1024 * 4 * 4 && aligned16_all({y, x}))
        ops::softmax_forward_rowreg_kernel<512, 25><<<rows, 512, 0, ctx->stream>>>(y, x, vocab, vocab_padded);
    else if (vocab_padded % 4 == 0 && vocab_padded <= 1024 * 4 * 4 && aligned16_all({y, x}))
        ops::softmax_forward_rowreg_kernel<1024, 4><<<rows, 1024, 0, ctx->stream>>>(y, x, vocab, vocab_padded);
    else
        ops::softmax_forward_kernel<<<rows, 1024, 0, ctx->stream>>>(y, x, vocab, vocab_padded);
    return launched(ctx);
}

int gptb200_cross_entropy_softmax_backward(gptb200_ctx *ctx, float *grad_x, const float *probs, const int *labels, int rows, int vocab,
                                           int vocab_padded)
{
    NEED(ctx, rows >= 0 && vocab >= 0 && vocab_padded >= vocab);
    if (rows == 0 || vocab == 0) return GPTB200_OK;
    NEED(ctx, grad_x && probs && labels);
    if (vocab_padded % 4 == 0 && aligned16_all({grad_x, probs}))
        ops::cross_entropy_softmax_backward_vec_kernel<<<rows, 1024, 0, ctx->stream>>>(grad_x, probs, labels, rows, vocab, vocab_padded);
    else
        ops::cross_entropy_softmax_backward_kernel<<<rows, 1024, 0, ctx->stream>>>(grad_x, probs, labels, rows, vocab, vocab_padded);
    return launched(ctx);
}

int gptb200_softmax_cross_entropy_inplace(gptb200_ctx *ctx, float *logits_inout, float *row_loss, const int *labels, int rows, int vocab,
                                          int vocab_padded)
{
    NEED(ctx, rows >= 0 && vocab >= 0 && vocab_padded >= vocab);
    if (rows == 0 || vocab_padded == 0) return GPTB200_OK;
    NEED(ctx, logits_inout && row_loss && labels);
    if (row_stream_applies(ctx, rows, vocab_padded) && aligned16_all({logits_inout})) {
        CUDA_TRY(ctx, allow_smem(ctx, ops::softmax_row_stream_kernel<1>, ops::kRowStreamSmem));
        ops::softmax_row_stream_kernel<1><<<std::min(rows, ctx->num_sms), ops::kRowStreamThreads, ops::kRowStreamSmem, ctx->stream>>>(
            nullptr, logits_inout, row_loss, labels, rows, vocab, vocab_padded, ctx->d_status);
    } else if (vocab_padded % 4 == 0 && vocab_padded <= 512 * 4 * 25 && vocab_padded > 1024 * 4 * 4 && aligned16_all({logits_inout}))
        ops::softmax_ce_inplace_rowreg_kernel<512, 25><<<rows, 512, 0, ctx->stream>>>(logits_inout, row_loss, labels, rows, vocab, vocab_padded);
    else if (vocab_padded % 4 == 0 && vocab_padded <= 1024 * 4 * 4 && aligned16_all({logits_inout}))
        ops::softmax_ce_inplace_rowreg_kernel<1024, 4><<<rows, 1024, 0, ctx->stream>>>(logits_inout, row_loss, labels, rows, vocab, vocab_padded);
    else
        ops::softmax_ce_inplace_kernel<<<rows, 1024, 0, ctx->stream>>>(logits_inout, row_loss, labels, rows, vocab, vocab_padded);
    return launched(ctx);
}

int gptb200_cross_entropy_loss_from_logits(gptb200_ctx *ctx, float *loss, float *row_loss, const float *logits, const int *labels, int rows, int vocab,
                                           int vocab_padded)
{
    NEED(ctx, rows >= 0 && vocab >= 0 && vocab_padded >= vocab && loss);
    NEED(ctx, rows == 0 || (row_loss && logits && labels));
    if (rows > 0) ops::ce_row_loss_from_logits_kernel<<<rows, 512, 0, ctx->stream>>>(row_loss, logits, labels, vocab, vocab_padded);
    ops::row_loss_mean_kernel<<<1, 1024, 0, ctx->stream>>>(loss, row_loss, rows);
    return launched(ctx, rows > 0 ? 2 : 1);
}

int gptb200_row_loss_mean(gptb200_ctx *ctx, float *loss, const float *row_loss, int rows)
{
    NEED(ctx, rows >= 0 && loss && (rows == 0 || row_loss));
    ops::row_loss_mean_kernel<<<1, 1024, 0, ctx->stream>>>(loss, row_loss, rows);
    return launched(ctx);
}

int gptb200_cross_entropy_loss(gptb200_ctx *ctx, float *loss, const float *probs, const int *labels, int rows, int vocab_padded)
{
    NEED(ctx, rows >= 0 && vocab_padded >= 0 && loss);
    NEED(ctx, rows == 0 || (probs && labels));
    ops::cross_entropy_loss_kernel<<<1, 1024, 0, ctx->stream>>>(loss, probs, labels, rows, vocab_padded);
    return launched(ctx);
}

int gptb200_adamw_step(gptb200_ctx *ctx, float *params, const float *g, float *m, float *v, size_t count, float lr, float beta1,
                       float beta2, float eps, float weight_decay, int step)
{
    NEED(ctx, count == 0 || (params && g && m && v));
    if (count == 0) return GPTB200_OK;
    const float bc1 = 1.0f - powf(beta1, static_cast<float>(step));
    const float bc2 = 1.0f - powf(beta2, static_cast<float>(step));
    ops::adamw_kernel<<<blocks_for(ctx, count, 256), 256, 0, ctx->stream>>>(params, g, m, v, count, lr, beta1, beta2, eps, weight_decay, bc1, bc2);
    return launched(ctx);
}

int gptb200_scale_and_clip_grad(gptb200_ctx *ctx, float *g, size_t count, float max_norm, int accum_steps)
{
    NEED(ctx, (count == 0 || g) && accum_steps > 0);
    if (count == 0) return GPTB200_OK;
    const int blocks = std::min<size_t>(size_t(ctx->num_sms) * 8, (count + 1023) / 1024);
    const int rc = ensure_workspace(ctx, (size_t(blocks) + 1) * sizeof(float));
    if (rc) return rc;
    float *partial = ctx->ws, *factor = ctx->ws + blocks;
    ops::clip_scale_partial_kernel<<<blocks, 256, 0, ctx->stream>>>(g, partial, count, 1.0f / static_cast<float>(accum_steps));
    ops::clip_factor_kernel<<<1, 32, 0, ctx->stream>>>(factor, partial, blocks, max_norm);
    ops::clip_apply_kernel<<<blocks_for(ctx, count, 256), 256, 0, ctx->stream>>>(g, factor, count);
    return launched(ctx, 3);
}

int gptb200_clip_adamw_packed(gptb200_ctx *ctx, float *params, const float *g, float *m, float *v, size_t count, const long long *segment_ends,
                              const unsigned char *segment_decay, int segments, float max_norm, int accum_steps, float lr, float beta1, float beta2,
                              float eps, float weight_decay, int step, float *grad_norm_dev)
{
    NEED(ctx, (count == 0 || (params && g && m && v)) && accum_steps > 0 && step > 0);
    NEED(ctx, segments >= 1 && segments <= ops::kMaxParamSegments && segment_ends && segment_decay);
    if (count == 0) return GPTB200_OK;
    ops::ParamSegments seg{};
    seg.count = segments;
    bool vec_ok = aligned16_all({params, g, m, v});
    long long prev = 0;
    for (int t = 0; t < segments; ++t) {
        NEED(ctx, segment_ends[t] >= prev);
        seg.end[t] = prev = segment_ends[t];
        seg.decay[t] = segment_decay[t];
        if (t < segments - 1 && (segment_ends[t] & 3)) vec_ok = false;
    }
    NEED(ctx, static_cast<size_t>(prev) == count);
    const int blocks = static_cast<int>(std::min<size_t>(size_t(ctx->num_sms) * 8, (count + 4095) / 4096));
    const int rc = ensure_workspace(ctx, size_t(blocks) * sizeof(float));
    if (rc) return rc;
    const float bc1 = 1.0f - powf(beta1, static_cast<float>(step));
    const float bc2 = 1.0f - powf(beta2, static_cast<float>(step));
    ops::grad_sumsq_kernel<<<blocks, 256, 0, ctx->stream>>>(ctx->ws, g, static_cast<long long>(count));
    ops::adamw_packed_kernel<<<ctx->num_sms * 8, 256, 0, ctx->stream>>>(params, g, m, v, static_cast<long long>(count), ctx->ws, blocks,
                                                                         1.0f / static_cast<float>(accum_steps), max_norm, lr, beta1, beta2, eps,
                                                                         weight_decay, bc1, bc2, seg, vec_ok ? 1 : 0, grad_norm_dev);
    return launched(ctx, 2);
}

int gptb200_embedding_decode(gptb200_ctx *ctx, float *y, const float *wte, const float *wpe, const int *tokens, const int *pos_dev, int batch, int d)
{
    NEED(ctx, batch >= 0 && d >= 0);
    if (batch == 0 || d == 0) return GPTB200_OK;
    NEED(ctx, y && wte && wpe && tokens && pos_dev);
    ops::embedding_decode_kernel<<<batch, 256, 0, ctx->stream>>>(y, wte, wpe, tokens, pos_dev, d);
    return launched(ctx);
}

int gptb200_kv_cache_fill(gptb200_ctx *ctx, float *cache, const float *qkv, int batch, int seq_len, int max_len, int d)
{
    NEED(ctx, batch >= 0 && seq_len >= 0 && seq_len <= max_len && d >= 0);
    if (batch == 0 || seq_len == 0 || d == 0) return GPTB200_OK;
    NEED(ctx, cache && qkv);
    ops::kv_fill_kernel<<<dim3(seq_len, batch), 256, 0, ctx->stream>>>(cache, qkv, seq_len, max_len, d);
    return launched(ctx);
}

int gptb200_attention_decode(gptb200_ctx *ctx, float *y, float *cache, const float *qkv_new, const int *pos_dev, int batch, int max_len, int d,
                             int heads)
{
    NEED(ctx, batch >= 0 && max_len > 0 && d > 0 && heads > 0 && d % heads == 0);
    if (batch == 0) return GPTB200_OK;
    NEED(ctx, y && cache && qkv_new && pos_dev);
    const int hd = d / heads;
    NEED(ctx, hd >= 4 && hd <= ops::kDecodeAttnThreads && (hd & (hd - 1)) == 0 && aligned16_all({cache}) && d % 4 == 0);
    const size_t smem = (size_t(max_len) + hd + ops::kDecodeAttnThreads + 64) * sizeof(float);
    NEED(ctx, smem <= 200 * 1024);
    if (smem > 48 * 1024) CUDA_TRY(ctx, allow_smem(ctx, ops::attention_decode_kernel, static_cast<int>(smem)));
    ops::attention_decode_kernel<<<dim3(heads, batch), ops::kDecodeAttnThreads, smem, ctx->stream>>>(y, cache, qkv_new, pos_dev, max_len, d, hd,
                                                                                                     1.0f / sqrtf(static_cast<float>(hd)));
    return launched(ctx);
}

int gptb200_advance_position(gptb200_ctx *ctx, int *pos_dev)
{
    NEED(ctx, pos_dev);
    ops::advance_position_kernel<<<1, 1, 0, ctx->stream>>>(pos_dev);
    return launched(ctx);
}

int gptb200_memory_info(gptb200_ctx *ctx, float *free_mb, float *total_mb)
{
    NEED(ctx, free_mb && total_mb);
    size_t f = 0, t = 0;
    CUDA_TRY(ctx, cudaMemGetInfo(&f, &t));
    *free_mb = static_cast<float>(f / (1024.0 * 1024.0));
    *total_mb = static_cast<float>(t / (1024.0 * 1024.0));
    return GPTB200_OK;
}

}  // extern "C"
