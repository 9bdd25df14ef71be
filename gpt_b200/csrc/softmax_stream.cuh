// Row kernels over the logits [rows, vocab_padded] for rows of 16 K - 51 K floats, as persistent blocks (one per SM) that
// prefetch the NEXT row into shared memory with bulk copies while the current row, held in registers, is reduced and written:
// with one row per block and no prefetch, the load of a row, its two block-wide reductions and its stores run one after the
// other and the kernel reaches half of the DRAM bandwidth.
//   MODE 0: y = softmax(x[:, :v]) (padding columns 0)                                    -- device_softmax_forward (cpu_backend.cpp:439-472)
//   MODE 1: in place, x = (softmax(x) - onehot(label)) / rows, row_loss = -log(p[label] + 1e-8)
//           -- softmax + device_cross_entropy_softmax_fused_backward + the terms of device_cross_entropy_loss (cpu_backend.cpp:439-509)
#pragma once

#include <cfloat>
#include <cstdint>
#include <cuda_runtime.h>

#include "backend_ops.cuh"
#include "ptx_sm100.cuh"

namespace gptb200 {
namespace ops {

constexpr int kRowStreamThreads = 512;
constexpr int kRowStreamVecs = 25;                              // float4 per thread: rows of up to 51 200 floats
constexpr int kRowStreamSmem = kRowStreamThreads * kRowStreamVecs * 16;   // 204 800 bytes of dynamic shared memory (the row buffer)
constexpr long long kRowStreamWaitCycles = 2000000000LL;        // about one second
constexpr int kRowStreamTimeoutCode = 110;                      // status word: a row's bulk copy never completed

template <int MODE>
__global__ void __launch_bounds__(kRowStreamThreads)
softmax_row_stream_kernel(float *__restrict__ y, float *__restrict__ x, float *__restrict__ row_loss, const int *__restrict__ labels, int rows, int v,
                          int vp, int *status)
{
    constexpr int THREADS = kRowStreamThreads, NV = kRowStreamVecs;
    extern __shared__ __align__(128) uint8_t row_buf[];
    __shared__ float red[32];
    __shared__ __align__(8) unsigned long long bar_word;
    const uint32_t bar = ptx::smem_u32(&bar_word), buf = ptx::smem_u32(row_buf);
    const int nvec = vp >> 2;
    const uint32_t row_bytes = static_cast<uint32_t>(vp) * 4u;
    // a row travels as four bulk copies (each a multiple of 16 bytes)
    const uint32_t piece = ((row_bytes / 4u) + 15u) & ~15u;
    auto fetch = [&](size_t r) {
        ptx::mbar_arrive_expect_tx(bar, row_bytes);
        const char *src = reinterpret_cast<const char *>(x + r * vp);
        for (uint32_t off = 0; off < row_bytes; off += piece) ptx::bulk_load_1d(buf + off, src + off, min(piece, row_bytes - off), bar);
    };
    if (threadIdx.x == 0) {
        ptx::mbar_init(bar, 1);
        ptx::fence_mbar_init();
    }
    __syncthreads();
    size_t r = blockIdx.x;
    if (r < static_cast<size_t>(rows) && threadIdx.x == 0) fetch(r);
    uint32_t phase = 0;
    for (; r < static_cast<size_t>(rows); r += gridDim.x, phase ^= 1u) {
        // the row has landed (bounded wait: on expiry the status word says so and the block leaves)
        bool ok = ptx::mbar_try_wait(bar, phase);
        if (!ok) {
            const long long t0 = clock64();
            while (!(ok = ptx::mbar_try_wait(bar, phase)) && clock64() - t0 < kRowStreamWaitCycles) {}
            if (!ok) atomicCAS(status, 0, kRowStreamTimeoutCode);
        }
        if (__syncthreads_or(!ok)) return;
        float4 e[NV];
        float m = -FLT_MAX;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + THREADS * k;
            e[k] = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
            if (c < nvec) {
                const float4 t = ptx::lds128(buf + 16u * c);
                const int i = 4 * c;
                if (i + 3 < v) {
                    e[k] = t;
                } else {   // the last pieces of the row: columns from v on do not take part
                    e[k].x = i < v ? t.x : -FLT_MAX;
                    e[k].y = i + 1 < v ? t.y : -FLT_MAX;
                    e[k].z = i + 2 < v ? t.z : -FLT_MAX;
                }
            }
            m = fmaxf(m, fmaxf(fmaxf(e[k].x, e[k].y), fmaxf(e[k].z, e[k].w)));
        }
        // every thread has its part of the row in registers: the buffer can take the next row while this one is worked on
        __syncthreads();
        const size_t next = r + gridDim.x;
        if (next < static_cast<size_t>(rows) && threadIdx.x == 0) {
            ptx::fence_proxy_async_smem();
            fetch(next);
        }
        m = block_max(m, red);
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            // columns that do not take part hold -FLT_MAX: their difference from the maximum is below every exponent, expf gives 0
            e[k].x = expf(e[k].x - m);
            e[k].y = expf(e[k].y - m);
            e[k].z = expf(e[k].z - m);
            e[k].w = expf(e[k].w - m);
            s += (e[k].x + e[k].y) + (e[k].z + e[k].w);
        }
        s = block_sum(s, red);
        const float rs = 1.0f / s;
        float4 *out = reinterpret_cast<float4 *>((MODE == 0 ? y : x) + r * vp);
        if (MODE == 0) {
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int c = threadIdx.x + THREADS * k;
                if (c < nvec) out[c] = make_float4(e[k].x * rs, e[k].y * rs, e[k].z * rs, e[k].w * rs);   // masked and padding columns: 0
            }
        } else {
            const int label = labels[r];
            const float inv = 1.0f / static_cast<float>(rows), scale = rs * inv;
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int c = threadIdx.x + THREADS * k;
                if (c >= nvec) continue;
                const int i = 4 * c;
                if (i + 3 < v && c != (label >> 2)) {   // neither the label nor the end of the row: p / rows
                    out[c] = make_float4(e[k].x * scale, e[k].y * scale, e[k].z * scale, e[k].w * scale);
                    continue;
                }
                const float p[4] = {e[k].x * rs, e[k].y * rs, e[k].z * rs, e[k].w * rs};
                float g[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (i + j == label) row_loss[r] = -logf(p[j] + 1e-8f);
                    g[j] = i + j < v ? (p[j] - (i + j == label ? 1.0f : 0.0f)) * inv : 0.0f;
                }
                out[c] = make_float4(g[0], g[1], g[2], g[3]);
            }
        }
    }
}

}  // namespace ops
}  // namespace gptb200
