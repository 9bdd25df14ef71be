// B200Backend: the reference's operator interface (IGPTBackend) implemented on a B200.
//
// The five linear-path operators go through the extern "C" layer of this library (tcgen05 GEMM kernels,
// include/gptb200.h); a gptb200_ctx takes the place of the cuBLAS handle that the reference's CUDABackend
// owns (src/backend/cuda/cuda_backend.h:40).  The remaining operators are plain kernels (backend_ops.cuh).
// As in the reference (src/backend/cuda/utils/cuda_utils.cuh:21-48) the interface returns void: any error is
// printed with file and line and the process is aborted.  With abort_on_error = false (this library's own model
// driver) the first failing status is kept instead (status()), and every later operator is skipped.
// Everything runs on one stream, in call order.
#pragma once

#include "backend_interface.h"  // this library's copy of the declaration, or the reference's own header

struct gptb200_ctx;

class B200Backend : public IGPTBackend
{
public:
    // `stream` is a cudaStream_t (nullptr = the legacy default stream, as in the reference);
    // `mode`: 0 = 3xTF32 (default), 1 = TF32.
    explicit B200Backend(unsigned long seed = 42, int device = 0, void *stream = nullptr, int mode = 0, bool abort_on_error = true);
    ~B200Backend() override;

    gptb200_ctx *context() const { return ctx_; }
    int status() const { return status_; }      // first failing gptb200_status since construction / clear_status (0 = none)
    void clear_status() { status_ = 0; }

    void device_get_memory_info(float *free_mb, float *total_mb) override;
    void device_malloc(void **ptr, size_t size) override;
    void device_free(void *ptr) override;
    void device_memset(void *ptr, int value, size_t size) override;
    void device_fill_normal(float *ptr, float mean, float stddev, size_t size) override;
    void device_fill_const(float *ptr, float value, size_t size) override;
    void device_memcpy_d2h(void *dst, const void *src, size_t size) override;
    void device_memcpy_h2d(void *dst, const void *src, size_t size) override;
    void device_embedding_forward(float *y, const float *wte, const float *wpe, const int *input_tokens, int batch_size, int seq_len, int hidden_size) override;
    void device_unembedding_forward(float *y, const float *x, const float *wte, int batch_size, int seq_len, int hidden_size, int vocab_size) override;
    void device_embedding_backward(float *grad_wte, float *grad_wpe, const float *grad_y, const int *input_tokens, int batch_size, int seq_len, int hidden_size) override;
    void device_unembedding_backward(float *grad_x, float *grad_wte, const float *grad_y, const float *x, const float *wte, int batch_size, int seq_len, int hidden_size, int vocab_size_padded) override;
    void device_layernorm_residual_fused_forward(float *y, float *means, float *vars, float *x, const float *residual, const float *gamma, const float *beta, int batch_size, int seq_len, int hidden_size) override;
    void device_layernorm_residual_fused_backward(float *grad_x, float *grad_gamma, float *grad_beta, const float *grad_y, const float *grad_residual, const float *x, const float *means, const float *vars, const float *gamma, int batch_size, int seq_len, int hidden_size) override;
    void device_linear_activation_fused_forward(float *y, float *act, const float *x, const float *w, const float *b, bool activation, int batch_size, int seq_len, int input_size, int output_size) override;
    void device_linear_backward(float *grad_x, float *grad_w, float *grad_b, const float *grad_y, const float *x, const float *w, int batch_size, int seq_len, int input_size, int output_size) override;
    void device_activation_backward(float *grad_x, const float *grad_y, const float *x, int batch_size, int seq_len, int output_size) override;
    void device_flash_attention_forward(float *y, float *logsumexp, const float *qkv, int batch_size, int seq_len, int hidden_size, int num_heads) override;
    void device_flash_attention_backward(float *grad_x, float *D_cache, const float *logsumexp, const float *grad_y, const float *y, const float *qkv, int batch_size, int seq_len, int hidden_size, int num_heads) override;
    void device_softmax_forward(float *y, const float *x, int batch_size, int seq_len, int vocab_size, int vocab_size_padded) override;
    void device_cross_entropy_softmax_fused_backward(float *grad_x, const float *y_softmax, const int *tokens_labels, int batch_size, int seq_len, int vocab_size, int vocab_size_padded) override;
    void device_cross_entropy_loss(float *loss, const float *y_softmax, const int *tokens_labels, int batch_size, int seq_len, int vocab_size_padded) override;
    void device_adamw_step(float *params, float *g, float *m, float *v, int size, float lr, float beta1, float beta2, float eps, float weight_decay, int step) override;
    void device_scale_and_clip_grad(float *g, int size, float max_norm, int accum_steps) override;

private:
    gptb200_ctx *ctx_ = nullptr;
    unsigned long seed_ = 42;
    unsigned long long fill_offset_ = 0;  // elements drawn so far by device_fill_normal
    bool abort_on_error_ = true;
    int status_ = 0;
};
