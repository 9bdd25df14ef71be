// B200Backend: see b200_backend.h.  Every method forwards to the extern "C" layer of this library and
// mirrors the reference's error convention (print file:line, abort).
#include <cstdio>
#include <cstdlib>

#include <cuda_runtime.h>

#include "b200_backend.h"
#include "../../include/gptb200.h"

// Two error conventions.  As a drop-in for the reference's backend object (gptb200_backend_create) an error is printed with
// file and line and the process is aborted, as the reference does (src/backend/cuda/utils/cuda_utils.cuh:21-48).  Behind
// this library's own model driver (abort_on_error = false) the first failing status is kept in the object, every later
// operator becomes a no-op, and the gptb200_model_* entry point returns that status to its caller.
#define B200_CHECK(expr)                                                                                     \
    do {                                                                                                     \
        if (status_ != 0) return;                                                                            \
        const int rc_ = (expr);                                                                              \
        if (rc_ != 0) {                                                                                      \
            if (abort_on_error_) {                                                                           \
                printf("B200Backend error: %s:%i:%d = %s (%s)\n", __FILE__, __LINE__, rc_, gptb200_status_string(rc_), \
                       ctx_ ? gptb200_last_error(ctx_) : "");                                               \
                abort();                                                                                     \
            }                                                                                                \
            status_ = rc_;                                                                                   \
            return;                                                                                          \
        }                                                                                                    \
    } while (0)

B200Backend::B200Backend(unsigned long seed, int device, void *stream, int mode, bool abort_on_error) : seed_(seed), abort_on_error_(abort_on_error)
{
    B200_CHECK(gptb200_ctx_create(&ctx_, device, stream, mode));
}

B200Backend::~B200Backend()
{
    if (ctx_) gptb200_ctx_destroy(ctx_);
}

void B200Backend::device_get_memory_info(float *free_mb, float *total_mb) { B200_CHECK(gptb200_memory_info(ctx_, free_mb, total_mb)); }
void B200Backend::device_malloc(void **ptr, size_t size)
{
    if (ptr) *ptr = nullptr;   // a failed (or skipped) allocation leaves a null pointer, never an indeterminate one
    B200_CHECK(gptb200_malloc(ctx_, ptr, size));
}
void B200Backend::device_free(void *ptr)
{
    // memory is released also after an earlier operator failed (teardown of a model that met an error)
    if (status_ != 0) {
        if (ctx_) gptb200_free(ctx_, ptr);
        return;
    }
    B200_CHECK(gptb200_free(ctx_, ptr));
}
void B200Backend::device_memset(void *ptr, int value, size_t size) { B200_CHECK(gptb200_memset(ctx_, ptr, value, size)); }

void B200Backend::device_fill_normal(float *ptr, float mean, float stddev, size_t size)
{
    B200_CHECK(gptb200_fill_normal(ctx_, ptr, mean, stddev, size, seed_, fill_offset_));
    fill_offset_ += size;
}

void B200Backend::device_fill_const(float *ptr, float value, size_t size) { B200_CHECK(gptb200_fill_const(ctx_, ptr, value, size)); }
void B200Backend::device_memcpy_d2h(void *dst, const void *src, size_t size) { B200_CHECK(gptb200_memcpy_d2h(ctx_, dst, src, size)); }
void B200Backend::device_memcpy_h2d(void *dst, const void *src, size_t size) { B200_CHECK(gptb200_memcpy_h2d(ctx_, dst, src, size)); }

void B200Backend::device_embedding_forward(float *y, const float *wte, const float *wpe, const int *input_tokens, int batch_size, int seq_len, int hidden_size)
{
    B200_CHECK(gptb200_embedding_forward(ctx_, y, wte, wpe, input_tokens, batch_size, seq_len, hidden_size));
}

void B200Backend::device_unembedding_forward(float *y, const float *x, const float *wte, int batch_size, int seq_len, int hidden_size, int vocab_size)
{
    B200_CHECK(gptb200_unembed_forward(ctx_, y, x, wte, batch_size * seq_len, hidden_size, vocab_size));
}

void B200Backend::device_embedding_backward(float *grad_wte, float *grad_wpe, const float *grad_y, const int *input_tokens, int batch_size, int seq_len, int hidden_size)
{
    B200_CHECK(gptb200_embedding_backward(ctx_, grad_wte, grad_wpe, grad_y, input_tokens, batch_size, seq_len, hidden_size));
}

void B200Backend::device_unembedding_backward(float *grad_x, float *grad_wte, const float *grad_y, const float *x, const float *wte, int batch_size, int seq_len, int hidden_size, int vocab_size_padded)
{
    B200_CHECK(gptb200_unembed_backward(ctx_, grad_x, grad_wte, grad_y, x, wte, batch_size * seq_len, hidden_size, vocab_size_padded));
}

void B200Backend::device_layernorm_residual_fused_forward(float *y, float *means, float *vars, float *x, const float *residual, const float *gamma, const float *beta, int batch_size, int seq_len, int hidden_size)
{
    B200_CHECK(gptb200_layernorm_forward(ctx_, y, means, vars, x, residual, gamma, beta, batch_size * seq_len, hidden_size));
}

void B200Backend::device_layernorm_residual_fused_backward(float *grad_x, float *grad_gamma, float *grad_beta, const float *grad_y, const float *grad_residual, const float *x, const float *means, const float *vars, const float *gamma, int batch_size, int seq_len, int hidden_size)
{
    B200_CHECK(gptb200_layernorm_backward(ctx_, grad_x, grad_gamma, grad_beta, grad_y, grad_residual, x, means, vars, gamma, batch_size * seq_len, hidden_size));
}

void B200Backend::device_linear_activation_fused_forward(float *y, float *act, const float *x, const float *w, const float *b, bool activation, int batch_size, int seq_len, int input_size, int output_size)
{
    B200_CHECK(gptb200_linear_forward(ctx_, y, act, x, w, b, activation ? 1 : 0, batch_size * seq_len, input_size, output_size));
}

void B200Backend::device_linear_backward(float *grad_x, float *grad_w, float *grad_b, const float *grad_y, const float *x, const float *w, int batch_size, int seq_len, int input_size, int output_size)
{
    B200_CHECK(gptb200_linear_backward(ctx_, grad_x, grad_w, grad_b, grad_y, x, w, batch_size * seq_len, input_size, output_size));
}

void B200Backend::device_activation_backward(float *grad_x, const float *grad_y, const float *x, int batch_size, int seq_len, int output_size)
{
    B200_CHECK(gptb200_gelu_backward(ctx_, grad_x, grad_y, x, batch_size * seq_len, output_size));
}

void B200Backend::device_flash_attention_forward(float *y, float *logsumexp, const float *qkv, int batch_size, int seq_len, int hidden_size, int num_heads)
{
    B200_CHECK(gptb200_attention_forward(ctx_, y, logsumexp, qkv, batch_size, seq_len, hidden_size, num_heads));
}

void B200Backend::device_flash_attention_backward(float *grad_x, float *D_cache, const float *logsumexp, const float *grad_y, const float *y, const float *qkv, int batch_size, int seq_len, int hidden_size, int num_heads)
{
    B200_CHECK(gptb200_attention_backward(ctx_, grad_x, D_cache, logsumexp, grad_y, y, qkv, batch_size, seq_len, hidden_size, num_heads));
}

void B200Backend::device_softmax_forward(float *y, const float *x, int batch_size, int seq_len, int vocab_size, int vocab_size_padded)
{
    B200_CHECK(gptb200_softmax_forward(ctx_, y, x, batch_size * seq_len, vocab_size, vocab_size_padded));
}

void B200Backend::device_cross_entropy_softmax_fused_backward(float *grad_x, const float *y_softmax, const int *tokens_labels, int batch_size, int seq_len, int vocab_size, int vocab_size_padded)
{
    B200_CHECK(gptb200_cross_entropy_softmax_backward(ctx_, grad_x, y_softmax, tokens_labels, batch_size * seq_len, vocab_size, vocab_size_padded));
}

void B200Backend::device_cross_entropy_loss(float *loss, const float *y_softmax, const int *tokens_labels, int batch_size, int seq_len, int vocab_size_padded)
{
    B200_CHECK(gptb200_cross_entropy_loss(ctx_, loss, y_softmax, tokens_labels, batch_size * seq_len, vocab_size_padded));
}

void B200Backend::device_adamw_step(float *params, float *g, float *m, float *v, int size, float lr, float beta1, float beta2, float eps, float weight_decay, int step)
{
    B200_CHECK(gptb200_adamw_step(ctx_, params, g, m, v, static_cast<size_t>(size), lr, beta1, beta2, eps, weight_decay, step));
}

void B200Backend::device_scale_and_clip_grad(float *g, int size, float max_norm, int accum_steps)
{
    B200_CHECK(gptb200_scale_and_clip_grad(ctx_, g, static_cast<size_t>(size), max_norm, accum_steps));
}

// C factory so that a host program (or a test) can obtain the backend object without C++ linkage.
extern "C" IGPTBackend *gptb200_backend_create(unsigned long seed, int device, void *stream, int mode)
{
    return new B200Backend(seed, device, stream, mode);
}

extern "C" void gptb200_backend_destroy(IGPTBackend *be) { delete be; }

extern "C" gptb200_ctx *gptb200_backend_context(IGPTBackend *be) { return static_cast<B200Backend *>(be)->context(); }
