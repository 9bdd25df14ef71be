// Internal definition of the context behind include/gptb200.h, shared by the translation units of
// libgptb200 (never installed, never seen by callers).
#pragma once

#include <cstdarg>
#include <cstdio>
#include <cstdint>
#include <set>
#include <unordered_map>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/gptb200.h"

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A tensor map is a pure function of (base address, extents, box, layout): the context keeps the encoded maps so that a
// repeated call (every layer of every step uses the same few dozen tensors) costs a hash lookup instead of a driver call.
struct TmapKey {
    uintptr_t base;
    long long d0, d1, d2;   // extents (innermost first; d2 = 0 for 2-D maps)
    int box0, box1, kind;   // kind: 0 K-major operand, 1 MN-major operand, 2 output, 3 pre-split operand, 4 / 5 batched (4-D) with either swizzle
    long long b0 = 0, b1 = 0, b2 = 0, b3 = 0;   // batched maps: inner and outer batch counts (d2 = row pitch), inner and outer batch strides
    bool operator==(const TmapKey &o) const
    {
        return base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && box0 == o.box0 && box1 == o.box1 && kind == o.kind && b0 == o.b0 && b1 == o.b1 &&
               b2 == o.b2 && b3 == o.b3;
    }
};
struct TmapKeyHash {
    size_t operator()(const TmapKey &k) const
    {
        uint64_t h = k.base * 0x9E3779B97F4A7C15ull;
        for (uint64_t v : {uint64_t(k.d0), uint64_t(k.d1), uint64_t(k.d2), uint64_t(k.box0) << 32 | uint64_t(k.box1) << 8 | uint64_t(k.kind), uint64_t(k.b0), uint64_t(k.b1),
                           uint64_t(k.b2), uint64_t(k.b3)})
            h = (h ^ v) * 0x100000001B3ull + (h >> 29);
        return size_t(h);
    }
};

struct gptb200_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int mode = GPTB200_MODE_3XTF32;
    int num_sms = 0;
    int max_sms = 0;     // 0 = all; otherwise the GEMM planner uses at most this many SMs (leaves room for a concurrent collective)
    int tile_n = 0;      // 0 = automatic
    int max_splits = 0;  // 0 = automatic
    bool skinny = true;  // weight-streaming kernel for decode-shaped calls (x K-major, no accumulation)
    int skinny_rows = 0; // most rows it takes: 0 = the planner's limit (64)
    int skinny_cluster = 16; // W stored [k][n]: one-launch kernel that splits k over a thread-block cluster of up to this many CTAs
                             // (0 = off; 16 = sixteen for narrow layers only; 32 = sixteen wherever k allows)
    int cluster16 = -1;            // can this device schedule a cluster of 16 CTAs of the decode kernels: -1 = not asked yet
    bool skinny_push = true;       // ... whose CTAs store their sums into the finishing CTA's shared memory (false: the finishing CTA loads them)
    int skinny_cluster_rows = 8;   // ... for calls with at most this many rows
    int skinny_tile_rows = 0;      // that kernel's row tile beyond 32 rows: 0 or 64 = one tile of 64, 32 = row groups of 32
    bool skinny_tile = true;       // beyond that many rows: one-launch register-tiled cluster kernel (false: the k-split kernel)
    int decode_early_launch = 0;     // that kernel is launched with programmatic stream serialization: it prefetches weights while
                                       // its predecessor on the stream still runs (caller's promise: the predecessor does not write them)
    bool skinny_rowwise = true;  // W stored [n][k], no bias: one-launch warp-per-row kernel ...
    int skinny_rowwise_rows = 8;  // ... for calls with at most this many rows (beyond: the register-tiled kernel)
    bool skinny_pipelined = true;  // k-split kernel, 16-row groups, W stored [k][n]: weight loads pipelined through shared memory
    int skinny_fused = 0;  // that kernel adds its partial sums itself (one launch): 1 = always, 0 = with at most two splits, -1 = never
    bool softmax_stream = true;   // long rows of logits: persistent softmax kernels that prefetch the next row (false: one block per row)
    bool attention_tiled = true;  // head size 64: register-tiled attention kernels (false: the one-row-per-thread-group kernels)
    int presplit = 0;        // 3xTF32, CTA pairs: split the operand that many tiles re-read before the launch (0 off, 1 automatic, 2 / 3 force A / B)
    bool fuse_dbias = true;  // grad_w launches of the CTA-pair kernel also produce the bias gradient (false: separate column-sum kernels)
    int pair = 0;        // CTA-pair (cta_group::2) kernel: 1 = always, 0 = heuristic, -1 = never
    int stream_k = 0;    // CTA-pair kernel, ranges cut inside tiles: 1 = always, 0 = heuristic, -1 = never
    long long *d_trace = nullptr;  // clock samples of the CTA-pair kernel (option "trace")
    int *d_status = nullptr;
    unsigned int *d_pair_flags = nullptr;  // per CTA pair, CTA and epilogue warp: number of the launch whose partial tile is complete;
                                           // then the number of completed launches and a CTA counter (both kept by the kernel);
                                           // then the decode kernel's tickets (one per column block, zero between launches)
    float *ws = nullptr;  // scratch: split-K partial tiles, partial rows of column reductions
    size_t ws_bytes = 0;
    float *attn_ws = nullptr;   // scratch of the tensor-core attention: score and score-gradient matrices of all heads
    size_t attn_ws_bytes = 0;
    int exact3x = 2;               // 3xTF32 CTA-pair kernel: correction terms as TF32 products of fp32 low-part tiles instead of one bf16 chain:
                                   // 0 never, 1 always, 2 for launches of at most 6 GFLOP
    int batched_chunk_kb = 1;      // 3xTF32 batched products: k-blocks per accumulator hand-off (0 = as the other launches: 4); 1: the attention
                                   // products then match the fp32 FMA kernels' accuracy (the accumulator's truncating adds are the main error)
    bool batched_exact3x = true;   // 3xTF32 batched products: TF32 correction terms (GemmParams::exact3x)
    int attention_group_mb = 8192; // ... in groups of sequences whose score matrices take at most this many MB of scratch (fewer, larger launches are faster)
    int attention_gemm = 1;     // head size 64: attention as batched tensor-core products + row kernels (0: the fp32 FMA kernels)
    size_t ws_limit = size_t(1) << 30;
    EncodeTiledFn encode = nullptr;
    long long launches = 0;
    std::set<const void *> configured;  // kernels whose dynamic shared-memory limit has been raised
    std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> tmaps;  // encoded tensor maps (emptied when it reaches kTmapCacheMax entries)
    long long tmap_encodes = 0;         // cuTensorMapEncodeTiled calls so far
    char last_error[512] = {0};
};

namespace gptb200 {

constexpr size_t kTmapCacheMax = 4096;

inline int fail(gptb200_ctx *ctx, int code, const char *fmt, ...)
{
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->last_error, sizeof(ctx->last_error), fmt, ap);
        va_end(ap);
    }
    return code;
}

// out[z] = a[z] . b[z] for inner * outer batches in one launch of the CTA-pair kernel (capi.cu).  Operands as stored: K-major
// (rows = free extent, k columns) or MN-major (k rows, free extent as columns); ld = row pitch, stride_inner / stride_outer =
// distance between consecutive inner / outer batches, all in floats.
struct BatchedOperand {
    const float *base;
    bool mn;
    long long ld, stride_inner, stride_outer;
};
// causal: the consumer of a square product reads only columns <= row, so output pieces wholly beyond the diagonal may stay unwritten
int run_gemm_batched(gptb200_ctx *ctx, float *out, long long out_ld, long long out_si, long long out_so, const BatchedOperand &a, const BatchedOperand &b,
                     int M, int N, int K, int inner, int outer, bool causal = false);

// Grows the context's scratch buffer to at least `bytes` (waits for queued work before replacing it).
int ensure_workspace(gptb200_ctx *ctx, size_t bytes);

}  // namespace gptb200

#define CUDA_TRY(ctx, expr)                                                                                          \
    do {                                                                                                             \
        cudaError_t e_ = (expr);                                                                                     \
        if (e_ != cudaSuccess) {                                                                                     \
            cudaGetLastError(); /* reported here: a later, unrelated call must not find it as the runtime's last error */ \
            return gptb200::fail(ctx, GPTB200_ERR_CUDA, "%s:%d %s -> %s", __FILE__, __LINE__, #expr, cudaGetErrorString(e_)); \
        }                                                                                                            \
    } while (0)
