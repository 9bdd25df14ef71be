// Operator interface of the reference model (Filipeak/gpt, src/backend/backend_interface.h:5-238), declared
// here so that this library can be built without the reference tree.  The class name, the virtual-function
// ORDER and every signature are those of the reference: an object of a class derived from this declaration
// is binary-compatible with code compiled against the reference's own header (the drop-in test compiles the
// reference's model driver against B200Backend with the reference's header first on the include path).
//
// All tensors are fp32, row-major, last dimension contiguous, in the backend's own memory space.  Shapes in
// brackets; B = batch_size, T = seq_len, D = hidden_size, Vp = padded vocabulary.
#pragma once

#include <cstddef>

class IGPTBackend
{
public:
    virtual ~IGPTBackend() = default;

    // ---- memory
    virtual void device_get_memory_info(float *free_mb, float *total_mb) = 0;
    virtual void device_malloc(void **ptr, size_t size) = 0;
    virtual void device_free(void *ptr) = 0;
    virtual void device_memset(void *ptr, int value, size_t size) = 0;
    virtual void device_fill_normal(float *ptr, float mean, float stddev, size_t size) = 0;
    virtual void device_fill_const(float *ptr, float value, size_t size) = 0;
    virtual void device_memcpy_d2h(void *dst, const void *src, size_t size) = 0;
    virtual void device_memcpy_h2d(void *dst, const void *src, size_t size) = 0;

    // y[B,T,D] = wte[token] + wpe[position]
    virtual void device_embedding_forward(float *y, const float *wte, const float *wpe, const int *input_tokens, int batch_size, int seq_len, int hidden_size) = 0;

    // y[B,T,Vp] = x[B,T,D] . wte[Vp,D]^T                                      (linear path)
    virtual void device_unembedding_forward(float *y, const float *x, const float *wte, int batch_size, int seq_len, int hidden_size, int vocab_size) = 0;

    // grad_wte[token] += grad_y ; grad_wpe[position] += grad_y
    virtual void device_embedding_backward(float *grad_wte, float *grad_wpe, const float *grad_y, const int *input_tokens, int batch_size, int seq_len, int hidden_size) = 0;

    // grad_x[B,T,D] = grad_y[B,T,Vp] . wte ; grad_wte[Vp,D] += grad_y^T . x     (linear path)
    virtual void device_unembedding_backward(float *grad_x, float *grad_wte, const float *grad_y, const float *x, const float *wte, int batch_size, int seq_len, int hidden_size, int vocab_size_padded) = 0;

    // x += residual (in place, when residual != nullptr); y = LayerNorm(x) * gamma + beta; row statistics kept
    virtual void device_layernorm_residual_fused_forward(float *y, float *means, float *vars, float *x, const float *residual, const float *gamma, const float *beta, int batch_size, int seq_len, int hidden_size) = 0;

    // grad_x = LayerNorm backward (+ grad_residual); grad_gamma, grad_beta accumulate
    virtual void device_layernorm_residual_fused_backward(float *grad_x, float *grad_gamma, float *grad_beta, const float *grad_y, const float *grad_residual, const float *x, const float *means, const float *vars, const float *gamma, int batch_size, int seq_len, int hidden_size) = 0;

    // y[B,T,O] = x[B,T,I] . w[I,O] + b[O]; act = GELU_tanh(y) when activation    (linear path)
    virtual void device_linear_activation_fused_forward(float *y, float *act, const float *x, const float *w, const float *b, bool activation, int batch_size, int seq_len, int input_size, int output_size) = 0;

    // grad_x = grad_y . w^T ; grad_w += x^T . grad_y ; grad_b += column sums      (linear path)
    virtual void device_linear_backward(float *grad_x, float *grad_w, float *grad_b, const float *grad_y, const float *x, const float *w, int batch_size, int seq_len, int input_size, int output_size) = 0;

    // grad_x = grad_y * GELU_tanh'(x)                                             (adjacent to the linear path)
    virtual void device_activation_backward(float *grad_x, const float *grad_y, const float *x, int batch_size, int seq_len, int output_size) = 0;

    // causal multi-head attention on packed qkv[B,T,3D]; logsumexp[B,T,H]
    virtual void device_flash_attention_forward(float *y, float *logsumexp, const float *qkv, int batch_size, int seq_len, int hidden_size, int num_heads) = 0;
    virtual void device_flash_attention_backward(float *grad_x, float *D_cache, const float *logsumexp, const float *grad_y, const float *y, const float *qkv, int batch_size, int seq_len, int hidden_size, int num_heads) = 0;

    // y = softmax over the first vocab_size columns; padding columns become 0
    virtual void device_softmax_forward(float *y, const float *x, int batch_size, int seq_len, int vocab_size, int vocab_size_padded) = 0;

    // grad_x = (softmax - onehot(label)) / (B*T) on the first vocab_size columns
    virtual void device_cross_entropy_softmax_fused_backward(float *grad_x, const float *y_softmax, const int *tokens_labels, int batch_size, int seq_len, int vocab_size, int vocab_size_padded) = 0;

    // loss[1] = mean negative log-likelihood
    virtual void device_cross_entropy_loss(float *loss, const float *y_softmax, const int *tokens_labels, int batch_size, int seq_len, int vocab_size_padded) = 0;

    virtual void device_adamw_step(float *params, float *g, float *m, float *v, int size, float lr, float beta1, float beta2, float eps, float weight_decay, int step) = 0;

    // g /= accum_steps, then global-norm clipping to max_norm
    virtual void device_scale_and_clip_grad(float *g, int size, float max_norm, int accum_steps) = 0;
};
