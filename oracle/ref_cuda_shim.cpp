// TEST / MEASUREMENT INFRASTRUCTURE -- not part of the product, never loaded by it.
//
// The reference's own CUDA backend (src/backend/cuda: cuBLAS TF32 sgemm + its bias/GELU, bias-gradient and other
// kernels), compiled UNMODIFIED from the reference tree by oracle/Makefile into oracle/_ref/libref_cuda.so, behind two
// timing entry points.  It is the "same box" comparison: what the reference does on this GPU for the same work.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_runtime.h>

#include "cuda_backend.h"
#include "gpt.h"

extern "C" {

// One FFN fc step through the reference CUDABackend: forward with GELU, then backward (grad_x, grad_w +=, grad_b +=).
// Buffers rotate over `nsets` input sets.  Returns milliseconds per step (CUDA events), < 0 on failure.
float refcuda_ffn_step_ms(int m, int k, int n, int steps, int warmup, int nsets)
{
    CUDABackend be(42);
    IGPTBackend *b = &be;
    std::vector<float *> x(nsets), gy(nsets), y(nsets), act(nsets), gx(nsets);
    float *w, *bias, *gw, *gb;
    for (int i = 0; i < nsets; ++i) {
        b->device_malloc((void **)&x[i], sizeof(float) * m * k);
        b->device_malloc((void **)&gy[i], sizeof(float) * m * n);
        b->device_malloc((void **)&y[i], sizeof(float) * m * n);
        b->device_malloc((void **)&act[i], sizeof(float) * m * n);
        b->device_malloc((void **)&gx[i], sizeof(float) * m * k);
        b->device_fill_normal(x[i], 0.0f, 1.0f, (size_t)m * k);
        b->device_fill_normal(gy[i], 0.0f, 1.0f, (size_t)m * n);
    }
    b->device_malloc((void **)&w, sizeof(float) * k * n);
    b->device_malloc((void **)&bias, sizeof(float) * n);
    b->device_malloc((void **)&gw, sizeof(float) * k * n);
    b->device_malloc((void **)&gb, sizeof(float) * n);
    b->device_fill_normal(w, 0.0f, 0.02f, (size_t)k * n);
    b->device_fill_normal(bias, 0.0f, 0.02f, (size_t)n & ~(size_t)1);  // cuRAND wants an even count
    b->device_memset(gw, 0, sizeof(float) * k * n);
    b->device_memset(gb, 0, sizeof(float) * n);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    float ms = -1.0f;
    for (int it = 0; it < warmup + steps; ++it) {
        if (it == warmup) cudaEventRecord(e0);
        const int s = it % nsets;
        b->device_linear_activation_fused_forward(y[s], act[s], x[s], w, bias, true, 1, m, k, n);
        b->device_linear_backward(gx[s], gw, gb, gy[s], x[s], w, 1, m, k, n);
    }
    cudaEventRecord(e1);
    if (cudaEventSynchronize(e1) == cudaSuccess && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) ms /= steps;
    for (int i = 0; i < nsets; ++i) {
        b->device_free(x[i]); b->device_free(gy[i]); b->device_free(y[i]); b->device_free(act[i]); b->device_free(gx[i]);
    }
    b->device_free(w); b->device_free(bias); b->device_free(gw); b->device_free(gb);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return ms;
}

// One linear layer through the reference CUDABackend, forward and backward timed apart: out2 = {forward ms, backward ms} per
// call (CUDA events; the reference's forward is cublasSgemm + its bias/GELU kernel, its backward two cublasSgemm + its
// bias-gradient kernel, src/backend/cuda/kernels/linear.cu:36-159).  Returns 0, or -1 on failure.
int refcuda_linear_ms(int m, int k, int n, int activation, int steps, int warmup, int nsets, float *out2)
{
    CUDABackend be(42);
    IGPTBackend *b = &be;
    std::vector<float *> x(nsets), gy(nsets), y(nsets), act(nsets), gx(nsets);
    float *w, *bias, *gw, *gb;
    for (int i = 0; i < nsets; ++i) {
        b->device_malloc((void **)&x[i], sizeof(float) * m * k);
        b->device_malloc((void **)&gy[i], sizeof(float) * m * n);
        b->device_malloc((void **)&y[i], sizeof(float) * m * n);
        b->device_malloc((void **)&act[i], sizeof(float) * m * n);
        b->device_malloc((void **)&gx[i], sizeof(float) * m * k);
        b->device_fill_normal(x[i], 0.0f, 1.0f, (size_t)m * k);
        b->device_fill_normal(gy[i], 0.0f, 1.0f, (size_t)m * n);
    }
    b->device_malloc((void **)&w, sizeof(float) * k * n);
    b->device_malloc((void **)&bias, sizeof(float) * n);
    b->device_malloc((void **)&gw, sizeof(float) * k * n);
    b->device_malloc((void **)&gb, sizeof(float) * n);
    b->device_fill_normal(w, 0.0f, 0.02f, (size_t)k * n);
    b->device_fill_normal(bias, 0.0f, 0.02f, (size_t)n & ~(size_t)1);
    b->device_memset(gw, 0, sizeof(float) * k * n);
    b->device_memset(gb, 0, sizeof(float) * n);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    int rc = 0;
    for (int pass = 0; pass < 2 && rc == 0; ++pass) {
        for (int it = 0; it < warmup + steps; ++it) {
            if (it == warmup) cudaEventRecord(e0);
            const int s = it % nsets;
            if (pass == 0)
                b->device_linear_activation_fused_forward(y[s], act[s], x[s], w, bias, activation != 0, 1, m, k, n);
            else
                b->device_linear_backward(gx[s], gw, gb, gy[s], x[s], w, 1, m, k, n);
        }
        cudaEventRecord(e1);
        float ms = -1.0f;
        if (cudaEventSynchronize(e1) != cudaSuccess || cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) rc = -1;
        out2[pass] = ms / steps;
    }
    for (int i = 0; i < nsets; ++i) {
        b->device_free(x[i]); b->device_free(gy[i]); b->device_free(y[i]); b->device_free(act[i]); b->device_free(gx[i]);
    }
    b->device_free(w); b->device_free(bias); b->device_free(gw); b->device_free(gb);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return rc;
}

// The tied un-embedding through the reference CUDABackend (embedding.cu:47-63,140-170): out2 = {forward ms, backward ms}.
int refcuda_unembed_ms(int m, int d, int vp, int steps, int warmup, float *out2)
{
    CUDABackend be(42);
    IGPTBackend *b = &be;
    float *x, *wte, *y, *gy, *gx, *gw;
    b->device_malloc((void **)&x, sizeof(float) * m * d);
    b->device_malloc((void **)&wte, sizeof(float) * (size_t)vp * d);
    b->device_malloc((void **)&y, sizeof(float) * (size_t)m * vp);
    b->device_malloc((void **)&gy, sizeof(float) * (size_t)m * vp);
    b->device_malloc((void **)&gx, sizeof(float) * m * d);
    b->device_malloc((void **)&gw, sizeof(float) * (size_t)vp * d);
    b->device_fill_normal(x, 0.0f, 1.0f, (size_t)m * d);
    b->device_fill_normal(wte, 0.0f, 0.02f, (size_t)vp * d);
    b->device_fill_normal(gy, 0.0f, 1e-4f, (size_t)m * vp);
    b->device_memset(gw, 0, sizeof(float) * (size_t)vp * d);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    int rc = 0;
    for (int pass = 0; pass < 2 && rc == 0; ++pass) {
        for (int it = 0; it < warmup + steps; ++it) {
            if (it == warmup) cudaEventRecord(e0);
            if (pass == 0)
                b->device_unembedding_forward(y, x, wte, 1, m, d, vp);
            else
                b->device_unembedding_backward(gx, gw, gy, x, wte, 1, m, d, vp);
        }
        cudaEventRecord(e1);
        float ms = -1.0f;
        if (cudaEventSynchronize(e1) != cudaSuccess || cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) rc = -1;
        out2[pass] = ms / steps;
    }
    b->device_free(x); b->device_free(wte); b->device_free(y); b->device_free(gy); b->device_free(gx); b->device_free(gw);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return rc;
}

// One training step of the reference's GPT class on its CUDA backend (zero_grad, forward, backward, clip, AdamW), random-init
// weights and uniform random tokens.  cfg = {max_seq_len, vocab_size, vocab_size_padded, num_layers, num_heads, d_model, d_ffn}.
// Returns milliseconds per step (host clock around device-synchronised steps), < 0 on failure.
float refcuda_gpt_step_ms(const int *cfg, int batch, int seq, int steps, int warmup)
{
    gpt_config config{cfg[0], cfg[1], cfg[2], cfg[3], cfg[4], cfg[5], cfg[6]};
    CUDABackend be(42);
    GPT model(&be, &config, true);
    model.init(0.0f, 0.02f);
    model.set_size(batch, seq);
    std::vector<int> toks((size_t)batch * (seq + 1));
    srand(7);
    for (auto &t : toks) t = rand() % config.vocab_size;
    std::vector<int> in((size_t)batch * seq), lbl((size_t)batch * seq);
    for (int b = 0; b < batch; ++b)
        for (int s = 0; s < seq; ++s) {
            in[(size_t)b * seq + s] = toks[(size_t)b * (seq + 1) + s];
            lbl[(size_t)b * seq + s] = toks[(size_t)b * (seq + 1) + s + 1];
        }
    int *d_in, *d_lbl;
    be.device_malloc((void **)&d_in, in.size() * sizeof(int));
    be.device_malloc((void **)&d_lbl, lbl.size() * sizeof(int));
    be.device_memcpy_h2d(d_in, in.data(), in.size() * sizeof(int));
    be.device_memcpy_h2d(d_lbl, lbl.data(), lbl.size() * sizeof(int));
    std::chrono::high_resolution_clock::time_point t0;
    for (int it = 0; it < warmup + steps; ++it) {
        if (it == warmup) {
            cudaDeviceSynchronize();
            t0 = std::chrono::high_resolution_clock::now();
        }
        model.zero_grad();
        model.forward(d_in);
        model.backward(d_in, d_lbl);
        model.unscale_and_clip_grads(1.0f, 1);
        model.optimizer_step(6e-4f, 0.9f, 0.95f, 0.1f);
    }
    if (cudaDeviceSynchronize() != cudaSuccess) return -1.0f;
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::high_resolution_clock::now() - t0).count() / steps;
    be.device_free(d_in);
    be.device_free(d_lbl);
    return (float)ms;
}

}  // extern "C"
