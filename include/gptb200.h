/*
 * gptb200 -- C ABI of the B200 (sm_100a) replacement for the dense linear-layer path of Filipeak/gpt.
 *
 * The reference routes these operators through a cuBLAS handle owned by its CUDA backend
 * (src/backend/cuda/core/cuda_backend.cu:4-13, src/backend/cuda/cuda_backend.h:40).  Here the handle is a
 * gptb200_ctx; each operator of the reference's IGPTBackend that belongs to the linear path has one entry
 * point with the same tensor meaning, the same overwrite/accumulate behaviour and plain pointers + ints.
 *
 * Conventions (same as the reference's interface, src/backend/backend_interface.h):
 *   - every tensor is fp32, row-major, last dimension contiguous, and lives in device memory owned by
 *     the caller; no operator allocates, frees or aliases caller memory;
 *   - `m` is batch_size * seq_len (the reference only ever uses the product);
 *   - y / act / grad_x are overwritten; grad_w / grad_b / grad_wte are accumulated into (+=);
 *   - operators are enqueued on the context's stream and return without waiting for the GPU;
 *   - every function returns 0 on success or a gptb200_status code; nothing aborts the process.
 *
 * There is no cuBLAS and no CPU fallback behind these calls.
 */
#ifndef GPTB200_H
#define GPTB200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gptb200_ctx gptb200_ctx;

typedef enum gptb200_status {
    GPTB200_OK = 0,
    GPTB200_ERR_INVALID_ARG = 1,   /* null pointer, negative dimension, m*n overflow */
    GPTB200_ERR_CUDA = 2,          /* a CUDA runtime / driver call failed; see gptb200_last_error */
    GPTB200_ERR_NO_DEVICE = 3,     /* no sm_100 device behind the requested ordinal */
    GPTB200_ERR_DEVICE_TIMEOUT = 4,/* a bounded wait inside a kernel ran out; results are invalid */
    GPTB200_ERR_WORKSPACE = 5,     /* scratch request beyond the configured limit */
    GPTB200_ERR_TOO_LARGE = 6      /* size beyond a fixed maximum of the called entry point */
} gptb200_status;

/* Precision of the tensor-core path.  Replaces cublasSetMathMode(CUBLAS_TF32_TENSOR_OP_MATH)
 * (src/backend/cuda/core/cuda_backend.cu:7). */
typedef enum gptb200_mode {
    GPTB200_MODE_3XTF32 = 0,  /* default: split operands (main term + two correction terms), fp32-level accuracy */
    GPTB200_MODE_TF32 = 1     /* single-pass TF32 */
} gptb200_mode;

/* ---- context: stands in for cublasCreate / cublasDestroy (cuda_backend.cu:6, :17) ---- */
int gptb200_ctx_create(gptb200_ctx **out, int device, void *cuda_stream, int mode);
int gptb200_ctx_destroy(gptb200_ctx *ctx);
int gptb200_ctx_set_mode(gptb200_ctx *ctx, int mode);
int gptb200_ctx_get_mode(const gptb200_ctx *ctx);
int gptb200_ctx_set_stream(gptb200_ctx *ctx, void *cuda_stream);
/* Tuning knobs, for benchmarking: key "tile_n" (0 = automatic, 128, 256), "max_splits" (0 = automatic),
 * "pair" (CTA-pair kernel with 256 x 256 tiles: 1 = always, 0 = heuristic, -1 = never),
 * "stream_k" (CTA-pair kernel: give every pair the same number of k-blocks by letting a pair's range begin and end inside a
 * tile, partial tiles summed through scratch: 1 = always, 0 = when whole tiles would leave SMs idle, -1 = never),
 * "skinny" (weight-streaming kernel for decode-shaped calls, up to 64 rows: 1 = on (default), 0 = off),
 * "skinny_rows" (most rows that kernel takes: 0 = 64 (default), 1 .. 64),
 * "skinny_cluster" (decode-shaped calls whose weight is stored [k][n]: one launch that splits k over the warps of a CTA and
 * the CTAs of a thread-block cluster and adds the parts through distributed shared memory; value = largest cluster, 0 (off:
 * k-split kernel with partial sums in scratch), 1, 2, 4, 8, 16 (default: sixteen only for layers too narrow to fill half of the
 * SMs with clusters of eight) or 32 (sixteen wherever k allows)),
 * "skinny_push" (that kernel's cluster sum: 1 = every CTA stores its part into the shared memory of the CTA that finishes it
 * (default), 0 = the finishing CTA loads the parts; same bits either way),
 * "skinny_cluster_rows" (most rows of x for which that kernel is used: default 8),
 * "skinny_tile" (more rows than the per-warp / row-wise kernels take, either weight layout: one-launch register-tiled kernel
 * whose k split also runs over a cluster: 1 = on (default), 0 = off (k-split kernel with partial sums in scratch)),
 * "skinny_tile_rows" (that kernel's row tile beyond 32 rows: 0 or 64 = one 64-row tile (default), 32 = row groups of 32),
 * "skinny_pipelined" (the k-split kernel's 16-row groups fetch weights through a shared-memory ring: 1 = on (default), 0 = off),
 * "skinny_rowwise" (decode-shaped calls whose weight is stored [n][k] - the un-embedding, grad_x: one-launch kernel, a warp
 * per pair of weight rows and group of up to 16 rows of x: 1 = on (default), 0 = off (k-split kernel)),
 * "skinny_rowwise_rows" (most rows of x for which that kernel is used: default 8; beyond, the register-tiled kernel),
 * "decode_early_launch" (inference only, 0 = off (default), 1 = on (2: also for the register-tiled kernel, measured
 * slower): the per-warp cluster kernel is launched with programmatic stream serialization, starts while the kernel before it on the stream is still running and reads w and b meanwhile - x is read and
 * y / act are written only once that kernel has completed.  The caller promises that no kernel writes weights or biases
 * immediately before a decode-shaped forward call on the same stream (an optimizer step does: leave this off when training)),
 * "skinny_fused" (the k-split kernel adds its partial sums itself instead of in a second launch: 1 = always, 0 = with at most
 * two splits (default), -1 = never; same bits either way),
 * "presplit" (3xTF32 mode, CTA-pair kernel: the bf16 correction tiles of the operand that most tiles re-read -- the weight matrix
 * in forward and grad_x, the activations in grad_w -- are written to scratch by a small kernel before the GEMM and fetched by
 * TMA, instead of being recomputed by every tile in the main loop: 0 = off (default), 1 = automatic choice of the operand,
 * 2 / 3 = always A / B; same bits either way.  Measured: 8-11 % fewer SM cycles per k-block on the GPT-2 FFN shapes but the same
 * time, because the kernel runs at the board's power limit and the clock drops by as much; one more launch per GEMM),
 * "fuse_dbias" (weight-gradient launches of the CTA-pair kernel also produce the bias gradient: 1 = on (default), 0 = the
 * separate column-sum kernels; results differ only in summation order),
 * "max_sms" (0 = all SMs; otherwise the GEMM kernels occupy at most this many, which leaves SMs to a collective that runs
 * at the same time on another stream),
 * "trace" (record a kernel-phase trace of each CTA-pair GEMM launch: 1 = on, 0 = off (default)),
 * "exact3x" (3xTF32 mode, CTA-pair kernel: form of the correction terms a_lo.b + a.b_lo -- 0 = one bf16 chain (error about 2^-20
 * per term, 8 tensor-core instructions per k-block), 1 = TF32 products of fp32 low-part tiles (2^-22, 12 instructions: 8 % slower
 * where the launch is bound by the tensor pipe or the power limit), 2 = the latter for launches of at most 6 GFLOP (default)),
 * "batched_exact3x" (the same choice for gptb200_gemm_batched and the attention products: 1 = TF32 products (default), 0 = bf16 chain),
 * "batched_chunk_kb" (3xTF32 mode, gptb200_gemm_batched and the attention products: k-blocks per hand-off of the accumulator to the
 * fp32 running sums, 1 (default) to 4, 0 = 4; the tensor core's truncating accumulation is the main error of these products),
 * "attention_gemm" (attention with head size 64 and a sequence length that is a multiple of 4, at most 1024: batched tensor-core
 * products on head slices of the packed qkv rows plus two row kernels, in the context's precision mode -- 1 = on (default),
 * 0 = the fp32 FMA kernels below; needs 2 * batch * heads * seq_len^2 floats of scratch, otherwise those kernels run too),
 * "attention_group_mb" (that form works through the sequences in groups whose score matrices take at most this many MB of
 * scratch: default 8192; fewer, larger launches are faster),
 * "attention_tiled" (attention with head size 64 on fp32 FMAs: register-tiled kernels, 1 = on (default), 0 = one row per thread group). */
int gptb200_ctx_set_option(gptb200_ctx *ctx, const char *key, int value);
/* Kernel-phase trace (option "trace" = 1): the most recent CTA-pair GEMM launch recorded the SM clock at 11 events,
 * [event][slot] with 128 slots per event.  Events 0-5 are taken in the launch's first CTA, slot = k-block (the first 128):
 * 0 loads issued, 1 conversion begins (first converter warp of the group, 3xTF32), 2 conversion published, 3 MMA thread at the
 * k-block, 4 MMA thread has the operands, 5 MMAs and commits issued.  Events 6 / 7: a tile's output begins / its stores are
 * issued (slot = tile, 3xTF32).  Events 8-10: events 0-2 in the pair's second CTA (another SM: its clock is a different
 * counter, compare durations only).  Copies up to `capacity` samples (11 * 128 in all; 0 = not recorded) after waiting for
 * the stream. */
int gptb200_ctx_read_trace(gptb200_ctx *ctx, long long *samples, int capacity);
/* Waits for the context's stream and reports a device-side timeout recorded by any earlier kernel. */
int gptb200_ctx_synchronize(gptb200_ctx *ctx);
/* Number of kernels this context has launched so far. */
long long gptb200_ctx_launch_count(const gptb200_ctx *ctx);
/* Number of tensor maps this context has encoded so far (cuTensorMapEncodeTiled calls).  Encoded maps are kept per
 * (address, extents, tile box): a call on tensors it has seen before encodes nothing. */
long long gptb200_ctx_tensor_map_encodes(const gptb200_ctx *ctx);
/* Failure-detection self-test: launches a one-CTA kernel whose bounded wait (limit_us microseconds, at most 100 ms) is on a
 * barrier that nothing signals.  The wait runs out, the kernel returns normally, and the next gptb200_ctx_synchronize reports
 * GPTB200_ERR_DEVICE_TIMEOUT (and clears the device status); the context stays usable. */
int gptb200_selftest_wait_timeout(gptb200_ctx *ctx, int limit_us);
/* The launch plan for D[m x n] = A[m x k] . B[k x n] on a GPU with num_sms SMs, without touching a GPU (host logic only,
 * default options).  plan8 = {kernel (0 none, 1 CTA-pair tcgen05, 2 one-CTA tcgen05, 3 weight streaming, 4 SIMT), tile_n,
 * tiles_m, tiles_n, split_k, k-blocks (or k elements for kernel 3) per split, CTAs, scratch KiB}.  For kernel 1 split_k is the
 * largest number of CTA pairs that work on one 256 x 256 tile (1: every pair computes whole tiles) and the next field the
 * k-blocks per CTA pair. */
int gptb200_plan_gemm(int num_sms, int m, int n, int k, int a_mn_major, int b_mn_major, int has_epilogue, int accumulate, int *plan8);
/* For a call that gptb200_plan_gemm sends to the weight-streaming kernels (kernel 3: at most 64 rows): which of them runs with
 * default options, host logic only.  w_kn_major: the weight is stored [k][n] (linear layers) rather than [n][k] (un-embedding,
 * grad_x).  plan4 = {kernel (0 k-split with scratch, 1 per-warp cluster kernel, 2 register-tiled cluster kernel, 3 warp per
 * weight-row pair), rows of x per CTA, row groups, CTAs per cluster}; clusters of 16 are assumed to be schedulable. */
int gptb200_plan_decode(int num_sms, int m, int n, int k, int w_kn_major, int has_epilogue, int *plan4);
const char *gptb200_status_string(int status);
const char *gptb200_last_error(const gptb200_ctx *ctx);

/* ---- IGPTBackend::device_linear_activation_fused_forward
 *      (backend_interface.h:120-132, cuda/kernels/linear.cu:36-66, cpu/cpu_backend.cpp:213-239)
 *   y[m x n] = x[m x k] . w[k x n] + b[n];  if activation: act = gelu_tanh(y) and y keeps the pre-activation.
 *   act may be NULL when activation == 0. */
int gptb200_linear_forward(gptb200_ctx *ctx, float *y, float *act, const float *x, const float *w, const float *b,
                           int activation, int m, int k, int n);

/* ---- IGPTBackend::device_linear_backward
 *      (backend_interface.h:134-148, cuda/kernels/linear.cu:116-159, cpu/cpu_backend.cpp:241-266)
 *   grad_x[m x k] = grad_y[m x n] . w^T;  grad_w[k x n] += x^T . grad_y;  grad_b[n] += column sums of grad_y. */
int gptb200_linear_backward(gptb200_ctx *ctx, float *grad_x, float *grad_w, float *grad_b, const float *grad_y,
                            const float *x, const float *w, int m, int k, int n);

/* The two halves of gptb200_linear_backward as separate calls (same kernels, same results): a data-parallel caller
 * issues the weight half first and all-reduces grad_w / grad_b on another stream while the input half still runs.
 * The reference has no multi-GPU path; both halves together are device_linear_backward (linear.cu:116-159). */
int gptb200_linear_backward_weights(gptb200_ctx *ctx, float *grad_w, float *grad_b, const float *grad_y, const float *x, int m, int k, int n);
int gptb200_linear_backward_input(gptb200_ctx *ctx, float *grad_x, const float *grad_y, const float *w, int m, int k, int n);

/* The input half with the GELU derivative of the layer in FRONT of this one folded into its epilogue:
 *   grad_x[m x k] = (grad_y[m x n] . w^T) * gelu_tanh'(pre_act[m x k])  element by element,
 * i.e. device_linear_backward's grad_x followed by device_activation_backward (linear.cu:116-203, gpt.cpp:565-571: the FFN's
 * down projection and its GELU) without the gradient of the activation making a round trip through HBM.  Same values as the
 * two calls up to the rounding of the derivative (fast exp / division, 1-2 ulp). */
int gptb200_linear_backward_input_gelu(gptb200_ctx *ctx, float *grad_x, const float *grad_y, const float *w, const float *pre_act, int m, int k, int n);

/* batch_inner * batch_outer independent products out[z] = a[z] . b[z] of one shape (m x n x k) in ONE launch of the CTA-pair
 * tensor-core kernel, in the context's precision mode (no counterpart in the reference, whose attention is scalar code:
 * cuda/kernels/attention.cu).  An operand is described as stored: K-major (a: [m][k], b: [n][k]) or MN-major (a: [k][m],
 * b: [k][n]); strides3 = {row pitch, distance between consecutive inner batches, distance between consecutive outer batches}
 * in floats, each a multiple of 4 and in any order of size -- which lets an operand be one head of packed rows (inner batch = head,
 * stride 64; row pitch 3 * d_model; outer batch = sequence).  Base addresses 16-byte aligned.  (a MN-major, b K-major) does not
 * occur and is refused.  out [m][n] is overwritten. */
int gptb200_gemm_batched(gptb200_ctx *ctx, float *out, const float *a, const float *b, int m, int n, int k, int a_mn_major, int b_mn_major, int batch_inner,
                         int batch_outer, const long long *a_strides3, const long long *b_strides3, const long long *out_strides3);

/* ---- IGPTBackend::device_activation_backward
 *      (backend_interface.h:150-159, cuda/kernels/linear.cu:162-203, cpu/cpu_backend.cpp:268-287)
 *   grad_x = grad_y * gelu_tanh'(x), all [m x n]. */
int gptb200_gelu_backward(gptb200_ctx *ctx, float *grad_x, const float *grad_y, const float *x, int m, int n);

/* ---- IGPTBackend::device_unembedding_forward
 *      (backend_interface.h:42-51, cuda/kernels/embedding.cu:47-63, cpu/cpu_backend.cpp:81-100)
 *   y[m x vp] = x[m x d] . wte^T, wte is [vp x d] (vp = padded vocabulary). */
int gptb200_unembed_forward(gptb200_ctx *ctx, float *y, const float *x, const float *wte, int m, int d, int vp);

/* ---- IGPTBackend::device_unembedding_backward
 *      (backend_interface.h:70-82, cuda/kernels/embedding.cu:140-170, cpu/cpu_backend.cpp:119-140)
 *   grad_x[m x d] = grad_y[m x vp] . wte;  grad_wte[vp x d] += grad_y^T . x. */
int gptb200_unembed_backward(gptb200_ctx *ctx, float *grad_x, float *grad_wte, const float *grad_y, const float *x,
                             const float *wte, int m, int d, int vp);

/* ---- memory operators of IGPTBackend (backend_interface.h:10-24, cuda/core/cuda_memory.cu:4-64) so that a
 *      host program can drive the whole path through this library: malloc / free / memset / blocking copies. */
int gptb200_malloc(gptb200_ctx *ctx, void **ptr, size_t bytes);
int gptb200_free(gptb200_ctx *ctx, void *ptr);
int gptb200_memset(gptb200_ctx *ctx, void *ptr, int value, size_t bytes);
int gptb200_memcpy_h2d(gptb200_ctx *ctx, void *dst, const void *src, size_t bytes);
int gptb200_memcpy_d2h(gptb200_ctx *ctx, void *dst, const void *src, size_t bytes);

/* ---- the remaining operators of IGPTBackend (backend_interface.h:26-40, 53-68, 84-118, 161-237), as plain
 *      kernels so that a whole training step can run behind the interface on the GPU.  They are not on the
 *      linear-layer hot path; arithmetic follows the reference CPU backend (cpu/cpu_backend.cpp).
 *      rows = batch_size * seq_len wherever only the product matters. */
int gptb200_fill_normal(gptb200_ctx *ctx, float *ptr, float mean, float stddev, size_t count, unsigned long long seed,
                        unsigned long long offset);
int gptb200_fill_const(gptb200_ctx *ctx, float *ptr, float value, size_t count);
int gptb200_embedding_forward(gptb200_ctx *ctx, float *y, const float *wte, const float *wpe, const int *tokens, int batch, int seq_len,
                              int d);
int gptb200_embedding_backward(gptb200_ctx *ctx, float *grad_wte, float *grad_wpe, const float *grad_y, const int *tokens, int batch,
                               int seq_len, int d);
/* gptb200_embedding_backward with every contribution multiplied by `scale`: a data-parallel step applies the rows of all ranks,
 * each weighted 1 / ranks, to gradients that were averaged before (no counterpart in the reference, which has one process). */
int gptb200_embedding_backward_scaled(gptb200_ctx *ctx, float *grad_wte, float *grad_wpe, const float *grad_y, const int *tokens, int batch,
                                      int seq_len, int d, float scale);
int gptb200_layernorm_forward(gptb200_ctx *ctx, float *y, float *means, float *vars, float *x, const float *residual, const float *gamma,
                              const float *beta, int rows, int d);
int gptb200_layernorm_backward(gptb200_ctx *ctx, float *grad_x, float *grad_gamma, float *grad_beta, const float *grad_y,
                               const float *grad_residual, const float *x, const float *means, const float *vars, const float *gamma,
                               int rows, int d);
int gptb200_attention_forward(gptb200_ctx *ctx, float *y, float *logsumexp, const float *qkv, int batch, int seq_len, int d, int heads);
int gptb200_attention_backward(gptb200_ctx *ctx, float *grad_qkv, float *d_cache, const float *logsumexp, const float *grad_y,
                               const float *y, const float *qkv, int batch, int seq_len, int d, int heads);
int gptb200_softmax_forward(gptb200_ctx *ctx, float *y, const float *x, int rows, int vocab, int vocab_padded);
int gptb200_cross_entropy_softmax_backward(gptb200_ctx *ctx, float *grad_x, const float *probs, const int *labels, int rows, int vocab,
                                           int vocab_padded);
int gptb200_cross_entropy_loss(gptb200_ctx *ctx, float *loss, const float *probs, const int *labels, int rows, int vocab_padded);
/* Softmax, cross-entropy backward and the loss terms in one pass over the logits, in place: the reference's
 * device_softmax_forward + device_cross_entropy_softmax_fused_backward + device_cross_entropy_loss
 * (cuda/kernels/softmax.cu:23-110, cross_entropy.cu:7-102, cpu/cpu_backend.cpp:439-509) without the probability tensor:
 *   logits_inout[r, i] becomes (softmax(logits[r, :vocab])[i] - (i == labels[r])) / rows for i < vocab and 0 in the padding
 *   columns; row_loss[r] = -log(softmax[labels[r]] + 1e-8).  gptb200_row_loss_mean averages the row terms into *loss (device
 *   memory); gptb200_cross_entropy_loss_from_logits computes row terms and loss from untouched logits. */
int gptb200_softmax_cross_entropy_inplace(gptb200_ctx *ctx, float *logits_inout, float *row_loss, const int *labels, int rows, int vocab,
                                          int vocab_padded);
int gptb200_row_loss_mean(gptb200_ctx *ctx, float *loss, const float *row_loss, int rows);
int gptb200_cross_entropy_loss_from_logits(gptb200_ctx *ctx, float *loss, float *row_loss, const float *logits, const int *labels, int rows, int vocab,
                                           int vocab_padded);
int gptb200_adamw_step(gptb200_ctx *ctx, float *params, const float *g, float *m, float *v, size_t count, float lr, float beta1,
                       float beta2, float eps, float weight_decay, int step);
int gptb200_scale_and_clip_grad(gptb200_ctx *ctx, float *g, size_t count, float max_norm, int accum_steps);
int gptb200_memory_info(gptb200_ctx *ctx, float *free_mb, float *total_mb);
/* ---- operators of a KV-cached generation step (no counterpart in the reference: its inference loop recomputes the whole
 *      prefix for every token, src/infer/infer.cpp:112-148, "TODO: Add KV Cache" at :120).  The cache of one layer is
 *      [batch][max_len][k (d) | v (d)], the k and v thirds of the reference's packed qkv rows; the position of the new token
 *      lives in device memory (*pos_dev) so that a captured step can be replayed for every position.
 *   embedding_decode:  y[b, :] = wte[tokens[b], :] + wpe[*pos_dev, :]
 *   kv_cache_fill:     cache[b][t] = k | v of qkv[b][t] for t < seq_len (after a forward pass over the prompt)
 *   attention_decode:  stores the new position's k | v (from qkv_new [batch][3 d]) at *pos_dev, then per head
 *                      y[b] = softmax_{t <= *pos_dev}(q . k_t / sqrt(d / heads)) . v_t; head size a power of two in 4 .. 128
 *   advance_position:  *pos_dev += 1 */
int gptb200_embedding_decode(gptb200_ctx *ctx, float *y, const float *wte, const float *wpe, const int *tokens, const int *pos_dev, int batch, int d);
int gptb200_kv_cache_fill(gptb200_ctx *ctx, float *cache, const float *qkv, int batch, int seq_len, int max_len, int d);
int gptb200_attention_decode(gptb200_ctx *ctx, float *y, float *cache, const float *qkv_new, const int *pos_dev, int batch, int max_len, int d,
                             int heads);
int gptb200_advance_position(gptb200_ctx *ctx, int *pos_dev);
/* Gradient scaling, norm clipping and AdamW over one packed buffer of `segments` tensors in two launches: what the reference
 * does with device_scale_and_clip_grad followed by one device_adamw_step per tensor (src/model/gpt.cpp:644-677,
 * cuda/kernels/gradient_clip.cu:35-59, adamw.cu:71-97).  Tensor t covers elements [segment_ends[t-1], segment_ends[t]);
 * segment_decay[t] != 0: weight_decay applies to it.  The gradients are read twice and never rewritten: the factor
 * (1 / accum_steps) * min(1, max_norm / (norm + 1e-6)) is applied on their way into the moment updates.  grad_norm_dev
 * (optional, device memory) receives the norm of the scaled gradients.  At most 32 segments. */
int gptb200_clip_adamw_packed(gptb200_ctx *ctx, float *params, const float *g, float *m, float *v, size_t count, const long long *segment_ends,
                              const unsigned char *segment_decay, int segments, float max_norm, int accum_steps, float lr, float beta1, float beta2,
                              float eps, float weight_decay, int step, float *grad_norm_dev);

/* ---- model driver: one GPT-2 forward / backward / optimiser step issued as the reference's operator
 *      sequence (src/model/gpt.cpp:426-690) over the operators above, with the reference's parameter packing
 *      (src/model/gpt.cpp:46-62) so that its raw fp32 checkpoints load unchanged.
 *      cfg = {max_seq_len, vocab_size, vocab_size_padded, num_layers, num_heads, d_model, d_ffn}.
 *      Token / label arrays are int32 in device memory, [batch x seq].
 *      Errors: every call returns a gptb200_status and nothing aborts.  The first operator that fails inside a call (a CUDA
 *      error, a scratch request beyond the limit) makes that call and every later one return its status, and the operators
 *      behind them become no-ops: destroy the model.  Two cases leave the model usable: gptb200_model_set_size that cannot
 *      get memory (GPTB200_ERR_CUDA) or whose logits tensor would exceed 2^31-1 elements (GPTB200_ERR_TOO_LARGE) changes
 *      nothing, and gptb200_model_loss reports a bounded wait that ran out in any kernel of the step
 *      (GPTB200_ERR_DEVICE_TIMEOUT) and clears it.  A configuration with more than 2^31-1 parameters is refused
 *      (GPTB200_ERR_TOO_LARGE). */
typedef struct gptb200_model gptb200_model;
int gptb200_model_create(gptb200_model **out, const int *cfg, int device, void *cuda_stream, int mode, unsigned long seed, int use_grad);
int gptb200_model_destroy(gptb200_model *m);
gptb200_ctx *gptb200_model_context(gptb200_model *m);
long long gptb200_model_num_params(gptb200_model *m);
float *gptb200_model_weights(gptb200_model *m);   /* device pointer, packed */
float *gptb200_model_grads(gptb200_model *m);     /* device pointer, packed like the weights */
float *gptb200_model_logits(gptb200_model *m);    /* device pointer, [batch*seq x vocab_size_padded], after forward */
int gptb200_model_param_offsets(gptb200_model *m, long long *offsets16);
int gptb200_model_init(gptb200_model *m, float mean, float stddev);
int gptb200_model_load_weights(gptb200_model *m, const float *host, long long count);
int gptb200_model_read(gptb200_model *m, float *host, long long count, int which /* 0 weights, 1 gradients */);
int gptb200_model_load_checkpoint(gptb200_model *m, const char *path);
int gptb200_model_save_checkpoint(gptb200_model *m, const char *path);
int gptb200_model_set_size(gptb200_model *m, int batch, int seq);
int gptb200_model_zero_grad(gptb200_model *m);
int gptb200_model_forward(gptb200_model *m, const int *tokens_dev);
/* layer_done(l, user) is called on the host right after the operators that complete layer l's weight gradients
 * have been enqueued: l = num_layers after the un-embedding and final LayerNorm, l = num_layers-1 .. 0 after each
 * transformer layer, l = -1 after the embedding backward (wte, wpe complete).  May be NULL. */
int gptb200_model_backward(gptb200_model *m, const int *tokens_dev, const int *labels_dev, void (*layer_done)(int, void *), void *user);
/* Data-parallel training: with defer != 0 the backward pass stops before the embedding backward, the one operator that adds to
 * grad_wte / grad_wpe at the very END of the pass (the un-embedding adds to grad_wte at its start).  The caller can then reduce
 * grad_wte over the ranks while the layers still run, gather every rank's rows and tokens afterwards
 * (gptb200_model_embedding_grad: [batch*seq x d_model], valid after the backward pass) and apply them all with
 * gptb200_model_apply_embedding_grad (scale = 1 / ranks): the same sum as reducing after a complete pass, without the
 * largest gradient tensor waiting for the end of it.  layer_done(-1) is not fired in a deferred pass. */
int gptb200_model_defer_embedding_backward(gptb200_model *m, int defer);
float *gptb200_model_embedding_grad(gptb200_model *m);
int gptb200_model_apply_embedding_grad(gptb200_model *m, const float *rows_dev, const int *tokens_dev, int batch, int seq, float scale);
/* on != 0: the un-embedding's logits are turned into their gradient in place at the start of the backward pass
 * (gptb200_softmax_cross_entropy_inplace): no probability tensor and no separate gradient tensor (2 x batch*seq x
 * vocab_size_padded floats less), two trips through HBM less per step.  gptb200_model_logits then holds logits only between
 * forward and backward.  Takes effect at the next gptb200_model_set_size. */
int gptb200_model_set_fused_cross_entropy(gptb200_model *m, int on);
/* on != 0: the FFN's GELU derivative is applied in the epilogue of the down projection's grad_x GEMM
 * (gptb200_linear_backward_input_gelu) instead of by device_activation_backward. */
int gptb200_model_set_fused_gelu_backward(gptb200_model *m, int on);
int gptb200_model_loss(gptb200_model *m, const int *labels_dev, float *loss_out);
/* KV-cached generation (the reference's loop, src/infer/infer.cpp:112-148, recomputes the prefix for every token):
 *   generate_begin  one forward pass over the prompt [batch x prompt_len] (device, int32), keys and values of every layer
 *                   into a cache sized for max_len positions; afterwards gptb200_model_logits holds the prompt's logits
 *                   ([batch*prompt_len x vocab_size_padded]: row b*prompt_len + prompt_len-1 predicts the first new token);
 *   generate_step   one new position: tokens_dev [batch] are the tokens AT that position (sampled from the previous logits);
 *                   logits_dev [batch x vocab_size_padded] receives the logits that predict the next one; every linear layer
 *                   runs with m = batch rows.  The position advances by one; GPTB200_ERR_INVALID_ARG beyond max_len.
 *   generate_position  the position the next generate_step will fill (prompt_len after generate_begin). */
int gptb200_model_generate_begin(gptb200_model *m, const int *prompt_dev, int batch, int prompt_len, int max_len);
int gptb200_model_generate_step(gptb200_model *m, const int *tokens_dev, float *logits_dev);
int gptb200_model_generate_position(gptb200_model *m);
int gptb200_model_clip(gptb200_model *m, float max_norm, int accum_steps);
int gptb200_model_optimizer_step(gptb200_model *m, float lr, float beta1, float beta2, float weight_decay);
/* gptb200_model_clip followed by gptb200_model_optimizer_step in two launches over the packed buffers (see
 * gptb200_clip_adamw_packed): same update, the gradient buffer is left unscaled. */
int gptb200_model_clip_and_optimizer_step(gptb200_model *m, float max_norm, int accum_steps, float lr, float beta1, float beta2, float weight_decay);
/* Self-describing training state (the reference's checkpoint is a raw fp32 parameter image, src/model/gpt.cpp:327-397, and
 * its header is a TODO, src/model/gpt.h:141): a 64-byte header -- magic "GPTB200S", format version, the seven configuration
 * values, the optimiser step, the parameter count, a flag for optimiser state -- followed by the parameters and, when the
 * model holds them, the two AdamW moment buffers, all in the reference's packing.  load checks the header against the
 * model's configuration (GPTB200_ERR_INVALID_ARG on mismatch or a short file) and restores the step counter. */
int gptb200_model_save_state(gptb200_model *m, const char *path);
int gptb200_model_load_state(gptb200_model *m, const char *path);
int gptb200_model_step_count(gptb200_model *m);

/* ---- token loader for data-parallel training: the reference's DataLoader (src/train/data_loader.h, data_loader.cpp:57-160)
 *      with the batch sharded over ranks.  Same file format (flat uint16 token ids) and the same sampling from the C
 *      library's rand() (seed it with srand, as src/train/train.cpp:73 does, identically on every rank): with world = 1 the
 *      batches are the reference's; with world > 1 rank r receives sequences [r * batch, (r + 1) * batch) of the global batch
 *      of world * batch sequences.  Host memory only.  next_batch returns 1 (batch produced), 0 (epoch exhausted) or a
 *      negative status. */
typedef struct gptb200_loader gptb200_loader;
int gptb200_loader_create(gptb200_loader **out, const char *token_file, int seq_len);
int gptb200_loader_destroy(gptb200_loader *ld);
long long gptb200_loader_num_samples(const gptb200_loader *ld);
int gptb200_loader_reset_epoch(gptb200_loader *ld);
int gptb200_loader_next_batch(gptb200_loader *ld, int rank, int world, int batch, int *inputs_host, int *labels_host);

/* ---- no counterpart in the reference: bias-gradient column sums without any allocation.
 *   grad_b[n] += column sums of grad_y[m x n], the same result as the grad_b part of gptb200_linear_backward,
 *   for callers that cannot allocate device memory (the GPU's memory belongs to the host program's own pool, or
 *   the call happens where the runtime forbids allocation).  The partial sums live in a fixed 1 MiB array inside
 *   the library instead of the context's growable scratch buffer; no context is needed.  n <= 8192, otherwise
 *   GPTB200_ERR_TOO_LARGE.  Runs on `cuda_stream`, which must belong to the device that is current at the call (the array
 *   used is that device's copy).  The first call on a device looks up the
 *   array's address; make it before any stream capture.  Calls share the array: calls that overlap on the GPU race. */
int gptb200_bias_grad_noalloc(float *grad_b, const float *grad_y, int m, int n, void *cuda_stream);

#ifdef __cplusplus
}
#endif

#endif /* GPTB200_H */
