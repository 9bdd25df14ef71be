// TEST INFRASTRUCTURE -- not part of the product.
//
// C-ABI shim around the UNMODIFIED reference sources (compiled from the reference tree where it lies by
// oracle/Makefile; nothing of the reference is copied into this repository):
//   src/backend/cpu/cpu_backend.cpp   the reference CPU backend (scalar fp32 loops)
//   src/model/gpt.cpp                 the reference model driver (buffer packing, forward/backward op sequence)
// It exports (a) the reference's linear-path operators one by one, (b) the softmax / cross-entropy
// operators that produce the LM-head upstream gradient, and (c) one whole forward+backward of the
// reference GPT class on a given backend: the reference CPU backend, or the same backend with the five
// linear-path operators replaced by the restatement in oracle/linear_oracle.c (which pins the
// restatement against the reference's own gradient test).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unistd.h>

#include "cpu_backend.h"
#include "data_loader.h"
#include "gpt.h"

extern "C" {
void oracle_linear_forward(float *, float *, const float *, const float *, const float *, int, int, int, int);
void oracle_linear_backward(float *, float *, float *, const float *, const float *, const float *, int, int, int);
void oracle_gelu_backward(float *, const float *, const float *, int, int);
void oracle_unembed_forward(float *, const float *, const float *, int, int, int);
void oracle_unembed_backward(float *, float *, const float *, const float *, const float *, int, int, int);
}

namespace {

// Reference CPU backend with the linear-path operators swapped for the restatement.
class RestatedBackend : public CPUBackend
{
public:
    void device_linear_activation_fused_forward(float *y, float *act, const float *x, const float *w, const float *b, bool activation,
                                                int batch_size, int seq_len, int input_size, int output_size) override
    {
        oracle_linear_forward(y, act, x, w, b, activation ? 1 : 0, batch_size * seq_len, input_size, output_size);
    }
    void device_linear_backward(float *grad_x, float *grad_w, float *grad_b, const float *grad_y, const float *x, const float *w,
                                int batch_size, int seq_len, int input_size, int output_size) override
    {
        oracle_linear_backward(grad_x, grad_w, grad_b, grad_y, x, w, batch_size * seq_len, input_size, output_size);
    }
    void device_activation_backward(float *grad_x, const float *grad_y, const float *x, int batch_size, int seq_len, int output_size) override
    {
        oracle_gelu_backward(grad_x, grad_y, x, batch_size * seq_len, output_size);
    }
    void device_unembedding_forward(float *y, const float *x, const float *wte, int batch_size, int seq_len, int hidden_size,
                                    int vocab_size_padded) override
    {
        oracle_unembed_forward(y, x, wte, batch_size * seq_len, hidden_size, vocab_size_padded);
    }
    void device_unembedding_backward(float *grad_x, float *grad_wte, const float *grad_y, const float *x, const float *wte, int batch_size,
                                     int seq_len, int hidden_size, int vocab_size_padded) override
    {
        oracle_unembed_backward(grad_x, grad_wte, grad_y, x, wte, batch_size * seq_len, hidden_size, vocab_size_padded);
    }
};

int run_gpt(IGPTBackend *be, const int *cfg, const float *weights, long long n_weights, const int *inputs, const int *labels, int batch,
            int seq, float *grads_out, float *loss_out, float *logits_out)
{
    gpt_config config;
    config.max_seq_len = cfg[0];
    config.vocab_size = cfg[1];
    config.vocab_size_padded = cfg[2];
    config.num_layers = cfg[3];
    config.num_heads = cfg[4];
    config.d_model = cfg[5];
    config.d_ffn = cfg[6];

    GPT model(be, &config, true);
    if ((long long)model.grad_weights()->buffer_count_ != n_weights) return 2;

    // The reference loads weights from a raw fp32 file (GPT::load_checkpoint, src/model/gpt.cpp:327-361).
    char path[] = "/tmp/gptb200_ref_ckpt_XXXXXX";
    int fd = mkstemp(path);
    if (fd < 0) return 3;
    FILE *fp = fdopen(fd, "wb");
    if (!fp) return 3;
    const size_t wrote = fwrite(weights, sizeof(float), (size_t)n_weights, fp);
    fclose(fp);
    if (wrote != (size_t)n_weights) { unlink(path); return 3; }
    const bool ok = model.load_checkpoint(path);
    unlink(path);
    if (!ok) return 4;

    model.set_size(batch, seq);
    // tokens live in the backend's memory space (src/model/gpt_test.cpp:128-137)
    int *d_inputs = nullptr, *d_labels = nullptr;
    const size_t tok_bytes = (size_t)batch * seq * sizeof(int);
    be->device_malloc((void **)&d_inputs, tok_bytes);
    be->device_malloc((void **)&d_labels, tok_bytes);
    be->device_memcpy_h2d(d_inputs, inputs, tok_bytes);
    be->device_memcpy_h2d(d_labels, labels, tok_bytes);
    // same sequence as src/model/gpt_test.cpp:148-164
    model.zero_grad();
    model.forward(d_inputs);
    model.backward(d_inputs, d_labels);
    const float loss = model.loss(d_labels);
    be->device_free(d_inputs);
    be->device_free(d_labels);
    if (loss_out) *loss_out = loss;
    if (grads_out) be->device_memcpy_d2h(grads_out, model.grad_weights()->buffer_, (size_t)n_weights * sizeof(float));
    if (logits_out)
        be->device_memcpy_d2h(logits_out, model.activations()->logits, (size_t)batch * seq * config.vocab_size_padded * sizeof(float));
    return 0;
}

}  // namespace

extern "C" {

void ref_linear_forward(float *y, float *act, const float *x, const float *w, const float *b, int activation, int m, int k, int n)
{
    CPUBackend be;
    be.device_linear_activation_fused_forward(y, act, x, w, b, activation != 0, 1, m, k, n);
}

void ref_linear_backward(float *grad_x, float *grad_w, float *grad_b, const float *grad_y, const float *x, const float *w, int m, int k,
                         int n)
{
    CPUBackend be;
    be.device_linear_backward(grad_x, grad_w, grad_b, grad_y, x, w, 1, m, k, n);
}

void ref_gelu_backward(float *grad_x, const float *grad_y, const float *x, int m, int n)
{
    CPUBackend be;
    be.device_activation_backward(grad_x, grad_y, x, 1, m, n);
}

void ref_unembed_forward(float *y, const float *x, const float *wte, int m, int d, int vp)
{
    CPUBackend be;
    be.device_unembedding_forward(y, x, wte, 1, m, d, vp);
}

void ref_unembed_backward(float *grad_x, float *grad_wte, const float *grad_y, const float *x, const float *wte, int m, int d, int vp)
{
    CPUBackend be;
    be.device_unembedding_backward(grad_x, grad_wte, grad_y, x, wte, 1, m, d, vp);
}

void ref_softmax_forward(float *y, const float *x, int m, int v, int vp)
{
    CPUBackend be;
    be.device_softmax_forward(y, x, 1, m, v, vp);
}

void ref_cross_entropy_softmax_backward(float *grad_x, const float *probs, const int *labels, int m, int v, int vp)
{
    CPUBackend be;
    be.device_cross_entropy_softmax_fused_backward(grad_x, probs, labels, 1, m, v, vp);
}

// ---- the remaining operators of the reference CPU backend, one by one (for the op-level tests of the plain kernels)
void ref_embedding_forward(float *y, const float *wte, const float *wpe, const int *tokens, int batch, int seq, int d)
{
    CPUBackend be;
    be.device_embedding_forward(y, wte, wpe, tokens, batch, seq, d);
}

void ref_embedding_backward(float *grad_wte, float *grad_wpe, const float *grad_y, const int *tokens, int batch, int seq, int d)
{
    CPUBackend be;
    be.device_embedding_backward(grad_wte, grad_wpe, grad_y, tokens, batch, seq, d);
}

void ref_layernorm_forward(float *y, float *means, float *vars, float *x, const float *residual, const float *gamma, const float *beta, int rows, int d)
{
    CPUBackend be;
    be.device_layernorm_residual_fused_forward(y, means, vars, x, residual, gamma, beta, 1, rows, d);
}

void ref_layernorm_backward(float *grad_x, float *grad_gamma, float *grad_beta, const float *grad_y, const float *grad_residual, const float *x,
                            const float *means, const float *vars, const float *gamma, int rows, int d)
{
    CPUBackend be;
    be.device_layernorm_residual_fused_backward(grad_x, grad_gamma, grad_beta, grad_y, grad_residual, x, means, vars, gamma, 1, rows, d);
}

void ref_attention_forward(float *y, float *logsumexp, const float *qkv, int batch, int seq, int d, int heads)
{
    CPUBackend be;
    be.device_flash_attention_forward(y, logsumexp, qkv, batch, seq, d, heads);
}

void ref_attention_backward(float *grad_qkv, float *d_cache, const float *logsumexp, const float *grad_y, const float *y, const float *qkv, int batch,
                            int seq, int d, int heads)
{
    CPUBackend be;
    be.device_flash_attention_backward(grad_qkv, d_cache, logsumexp, grad_y, y, qkv, batch, seq, d, heads);
}

void ref_cross_entropy_loss(float *loss, const float *probs, const int *labels, int rows, int vp)
{
    CPUBackend be;
    be.device_cross_entropy_loss(loss, probs, labels, 1, rows, vp);
}

// the optimiser-side operators (src/backend/cpu/cpu_backend.cpp:517-556), updating the caller's arrays in place
void ref_adamw_step(float *params, float *g, float *m, float *v, int size, float lr, float beta1, float beta2, float eps, float weight_decay, int step)
{
    CPUBackend be;
    be.device_adamw_step(params, g, m, v, size, lr, beta1, beta2, eps, weight_decay, step);
}

void ref_scale_and_clip_grad(float *g, int size, float max_norm, int accum_steps)
{
    CPUBackend be;
    be.device_scale_and_clip_grad(g, size, max_norm, accum_steps);
}

// The reference's DataLoader (src/train/data_loader.cpp, unmodified) on the CPU backend: srand(seed), then `epochs` epochs of
// up to `max_batches` batches each; every batch's inputs and labels are appended to the output arrays.  Returns the number
// of batches written, < 0 on failure.
int ref_loader_batches(const char *path, int batch, int seq_len, unsigned seed, int epochs, int max_batches, int *inputs_out, int *labels_out)
{
    CPUBackend be;
    DataLoader ld(&be, batch, seq_len);
    if (!ld.load_data(path)) return -1;
    srand(seed);
    const size_t per = (size_t)batch * seq_len;
    int written = 0;
    for (int e = 0; e < epochs; ++e) {
        ld.reset_epoch();
        for (int b = 0; b < max_batches && ld.next_batch(); ++b) {
            be.device_memcpy_d2h(inputs_out + written * per, ld.inputs(), per * sizeof(int));
            be.device_memcpy_d2h(labels_out + written * per, ld.labels(), per * sizeof(int));
            ++written;
        }
    }
    return written;
}

// cfg = {max_seq_len, vocab_size, vocab_size_padded, num_layers, num_heads, d_model, d_ffn}
int ref_gpt_forward_backward(const int *cfg, const float *weights, long long n_weights, const int *inputs, const int *labels, int batch,
                             int seq, int use_restated_ops, float *grads_out, float *loss_out, float *logits_out)
{
    if (use_restated_ops) {
        RestatedBackend be;
        return run_gpt(&be, cfg, weights, n_weights, inputs, labels, batch, seq, grads_out, loss_out, logits_out);
    }
    CPUBackend be;
    return run_gpt(&be, cfg, weights, n_weights, inputs, labels, batch, seq, grads_out, loss_out, logits_out);
}

// The same forward+backward of the reference's GPT class on a backend object supplied by the caller (an
// IGPTBackend* made elsewhere, e.g. by the product library's factory): the drop-in check.
int ref_gpt_forward_backward_on(void *backend, const int *cfg, const float *weights, long long n_weights, const int *inputs,
                                const int *labels, int batch, int seq, float *grads_out, float *loss_out, float *logits_out)
{
    return run_gpt(static_cast<IGPTBackend *>(backend), cfg, weights, n_weights, inputs, labels, batch, seq, grads_out, loss_out, logits_out);
}

}  // extern "C"
