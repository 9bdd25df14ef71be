/*
 * TEST INFRASTRUCTURE -- not part of the product.  Only tests/, __graft_entry__.smoke() and the
 * cpu_baseline / reference legs of bench.py may load this file's library.
 *
 * CPU restatement of the linear-layer operators of Filipeak/gpt's CPU backend
 * (src/backend/cpu/cpu_backend.cpp).  Every output element is computed with the same fp32 operations in
 * the same order as the reference's scalar loops (separate multiply and add, sums in ascending index
 * order), so the results are bit-identical to the reference; only the loop nests are interchanged and
 * threaded over independent output elements, which makes full-size cases finish in seconds.
 * Build with -ffp-contract=off (no FMA contraction) and without -ffast-math.
 *
 * Pinned by tests/test_oracle.py: bit-equality against the unmodified reference functions compiled from
 * the reference tree (oracle/_ref/libref_cpu.so), against op-level golden vectors produced by the
 * reference (tests/golden/ops_*.npz), and, through the reference's own GPT model driver, against the
 * PyTorch gradients of the reference's gradient test (tests/golden/gpt_tiny_*.bin).
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* y[m,o] = sum_i x[m,i] * w[i,o] (i ascending, starting from 0.0f), then + b[o];
 * act = 0.5 y (1 + tanhf(0.79788456 (y + 0.044715 y^3))).
 * Follows CPUBackend::device_linear_activation_fused_forward, cpu_backend.cpp:213-239. */
void oracle_linear_forward(float *y, float *act, const float *x, const float *w, const float *b, int activation, int m, int k, int n)
{
#pragma omp parallel for schedule(static)
    for (int r = 0; r < m; ++r) {
        float *yr = y + (size_t)r * n;
        const float *xr = x + (size_t)r * k;
        for (int o = 0; o < n; ++o) yr[o] = 0.0f;
        for (int i = 0; i < k; ++i) {
            const float xv = xr[i];
            const float *wi = w + (size_t)i * n;
            for (int o = 0; o < n; ++o) yr[o] += xv * wi[o];
        }
        for (int o = 0; o < n; ++o) {
            const float sum = yr[o] + b[o];
            yr[o] = sum;
            if (activation) act[(size_t)r * n + o] = 0.5f * sum * (1.0f + tanhf(0.79788456f * (sum + 0.044715f * sum * sum * sum)));
        }
    }
}

/* grad_x[m,i] = sum_o grad_y[m,o] * w[i,o]   (o ascending, from 0.0f)
 * grad_w[i,o] += x[m,i] * grad_y[m,o]        (tokens m ascending)
 * grad_b[o]   += grad_y[m,o]                 (tokens m ascending)
 * Follows CPUBackend::device_linear_backward, cpu_backend.cpp:241-266. */
void oracle_linear_backward(float *grad_x, float *grad_w, float *grad_b, const float *grad_y, const float *x, const float *w, int m, int k,
                            int n)
{
#pragma omp parallel
    {
#pragma omp for schedule(static) nowait
        for (int r = 0; r < m; ++r) {
            const float *gyr = grad_y + (size_t)r * n;
            float *gxr = grad_x + (size_t)r * k;
            for (int i = 0; i < k; ++i) {
                /* the reference adds grad_y[o] * w[i,o] into grad_x[i] for o = 0..n-1 in turn */
                const float *wi = w + (size_t)i * n;
                float s = 0.0f;
                for (int o = 0; o < n; ++o) s += gyr[o] * wi[o];
                gxr[i] = s;
            }
        }
#pragma omp for schedule(static) nowait
        for (int i = 0; i < k; ++i) {
            float *gwi = grad_w + (size_t)i * n;
            for (int r = 0; r < m; ++r) {
                const float xv = x[(size_t)r * k + i];
                const float *gyr = grad_y + (size_t)r * n;
                for (int o = 0; o < n; ++o) gwi[o] += xv * gyr[o];
            }
        }
#pragma omp for schedule(static)
        for (int o0 = 0; o0 < n; o0 += 64) {
            const int o1 = o0 + 64 < n ? o0 + 64 : n;
            for (int r = 0; r < m; ++r) {
                const float *gyr = grad_y + (size_t)r * n;
                for (int o = o0; o < o1; ++o) grad_b[o] += gyr[o];
            }
        }
    }
}

/* grad_x = grad_y * GELU'(x); constants as in CPUBackend::device_activation_backward, cpu_backend.cpp:268-287. */
void oracle_gelu_backward(float *grad_x, const float *grad_y, const float *x, int m, int n)
{
    const size_t total = (size_t)m * n;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < total; ++i) {
        const float x_val = x[i];
        const float tanh_out = tanhf(0.79788456f * (x_val + 0.044715f * x_val * x_val * x_val));
        const float d = 0.5f * (1.0f + tanh_out) + 0.5f * x_val * (1.0f - tanh_out * tanh_out) * (0.79788456f + 0.107032f * x_val * x_val);
        grad_x[i] = grad_y[i] * d;
    }
}

/* y[m,v] = sum_h x[m,h] * wte[v,h]  (h ascending, from 0.0f).
 * Follows CPUBackend::device_unembedding_forward, cpu_backend.cpp:81-100. */
void oracle_unembed_forward(float *y, const float *x, const float *wte, int m, int d, int vp)
{
#pragma omp parallel for schedule(static) collapse(2)
    for (int r = 0; r < m; ++r) {
        for (int v0 = 0; v0 < vp; v0 += 256) {
            const int v1 = v0 + 256 < vp ? v0 + 256 : vp;
            const float *xr = x + (size_t)r * d;
            for (int v = v0; v < v1; ++v) {
                const float *wv = wte + (size_t)v * d;
                float s = 0.0f;
                for (int h = 0; h < d; ++h) s += xr[h] * wv[h];
                y[(size_t)r * vp + v] = s;
            }
        }
    }
}

/* grad_x[m,h]   = sum_v grad_y[m,v] * wte[v,h]   (v ascending, from 0.0f)
 * grad_wte[v,h] += grad_y[m,v] * x[m,h]           (tokens m ascending)
 * Follows CPUBackend::device_unembedding_backward, cpu_backend.cpp:119-140. */
void oracle_unembed_backward(float *grad_x, float *grad_wte, const float *grad_y, const float *x, const float *wte, int m, int d, int vp)
{
#pragma omp parallel
    {
#pragma omp for schedule(static) nowait
        for (int r = 0; r < m; ++r) {
            float *gxr = grad_x + (size_t)r * d;
            const float *gyr = grad_y + (size_t)r * vp;
            for (int h = 0; h < d; ++h) gxr[h] = 0.0f;
            for (int v = 0; v < vp; ++v) {
                const float g = gyr[v];
                const float *wv = wte + (size_t)v * d;
                for (int h = 0; h < d; ++h) gxr[h] += g * wv[h];
            }
        }
#pragma omp for schedule(static)
        for (int v = 0; v < vp; ++v) {
            float *gwv = grad_wte + (size_t)v * d;
            for (int r = 0; r < m; ++r) {
                const float g = grad_y[(size_t)r * vp + v];
                const float *xr = x + (size_t)r * d;
                for (int h = 0; h < d; ++h) gwv[h] += g * xr[h];
            }
        }
    }
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
