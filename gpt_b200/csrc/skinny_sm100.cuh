// Decode-shaped products (m <= 64 rows): y[m x n] = x[m x k] . W (+ bias, GELU), fp32 FMAs, no TF32 rounding in either mode.
//
// With so few rows the operation is bound by reading the weight matrix once from HBM (4*k*n bytes; activations and outputs
// are negligible) and, for the 2 - 10 MB layers of a small model, by latencies: launch, one DRAM round trip, barriers.  The
// kernels are therefore organised around the weight stream, not around tensor-core tiles, and all but the fallback need one
// launch and no scratch:
//
//   decode_gemm_cluster_kernel   W [k][n], up to 8 rows (16 behind an option): k split over the 8 warps of a CTA and the CTAs
//                                of a thread-block cluster; sums through (distributed) shared memory
//   rowwise_gemv_kernel          W [n][k], up to 8 rows (64 behind an option): a warp per pair of weight rows
//   decode_tile_cluster_kernel   either layout, 9 - 64 rows: register-tiled TM x 128 tile per CTA, cp.async ring, k split over
//                                a cluster
//   skinny_gemm_kernel           the fallback behind the options (described next), + skinny_finish_kernel
//
// skinny_gemm_kernel: every thread owns output columns, keeps one fp32 accumulator per row and column in registers, reads
// its part of the weight matrix exactly once with 16-byte loads and takes the activations from a shared-memory copy
// (broadcast reads).  A CTA covers up to 16 rows; with more rows blockIdx.z selects the group of 16 (the groups of a column
// block run at about the same time, so the weights still come from HBM once and from L2 for the other groups).  The k range
// is split over blockIdx.y so that even a 768-column layer puts several hundred CTAs in flight; partial sums go to scratch
// and are added in a fixed order (split ascending), then bias / GELU are applied.  Who adds them: with `tickets` the CTA that
// finishes a column block last (one atomic ticket per column block, reset by that CTA, so the array stays zero between
// launches and under CUDA-graph replay); without `tickets` the separate skinny_finish_kernel, used beyond two splits, where
// one CTA re-reading all partial sums one dependent load after the other takes longer than a second launch.  Both give the
// same bits.
//
//   W_KN = true : W stored [k][n] (linear layers):   thread = 4 adjacent columns, coalesced 16-byte loads along n
//   W_KN = false: W stored [n][k] (tied un-embedding): thread = 1 column, 16-byte loads along its own row
#pragma once

#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "gemm_sm100.cuh"  // gelu_tanh

namespace gptb200 {

constexpr int kSkinnyThreads = 128;
constexpr int kSkinnyMaxTickets = 1024;  // column blocks per launch that can finish in the kernel itself
constexpr int kSkinnyPipe = 6;      // pipelined variant: bodies of four k-rows in the shared-memory ring (8 KiB each; three CTAs per SM fit)
constexpr int kSkinnyKChunk = 256;  // activations staged per pass: MR * 256 floats of shared memory

template <int MR, bool W_KN>
__global__ void __launch_bounds__(kSkinnyThreads)
skinny_gemm_kernel(float *__restrict__ partial, const float *__restrict__ x, const float *__restrict__ w, int M, int N, int K, int k_per_split,
                   float *__restrict__ y, float *__restrict__ act, const float *__restrict__ bias, unsigned int *__restrict__ tickets, int pipelined)
{
    extern __shared__ __align__(16) float4 w_ring[];   // pipelined: [kSkinnyPipe][4][kSkinnyThreads], thread-private slots
    __shared__ __align__(16) float xs[MR][kSkinnyKChunk];
    __shared__ int is_last;
    constexpr int CPT = W_KN ? 4 : 1;  // columns per thread
    const int col = (blockIdx.x * kSkinnyThreads + threadIdx.x) * CPT;
    const int row0 = blockIdx.z * MR;       // first row of this CTA's group
    const int rows = min(MR, M - row0);     // >= 1
    x += size_t(row0) * K;
    const int k_begin = blockIdx.y * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    const bool col_ok = col < N;  // N is a multiple of 4 on this path
    float acc[MR][CPT];
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
        for (int c = 0; c < CPT; ++c) acc[m][c] = 0.0f;

    for (int k0 = k_begin; k0 < k_end; k0 += kSkinnyKChunk) {
        const int kc = min(kSkinnyKChunk, k_end - k0);  // multiple of 4
        __syncthreads();
        for (int i = threadIdx.x; i < MR * (kSkinnyKChunk / 4); i += kSkinnyThreads) {
            const int m = i / (kSkinnyKChunk / 4), q = i % (kSkinnyKChunk / 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m < rows && 4 * q < kc) v = *reinterpret_cast<const float4 *>(x + size_t(m) * K + k0 + 4 * q);
            *reinterpret_cast<float4 *>(&xs[m][4 * q]) = v;
        }
        __syncthreads();
        if (!col_ok) continue;
        if (W_KN && pipelined) {
            // Weight loads run kSkinnyPipe - 1 bodies (of four k-rows) ahead of the FMAs through cp.async into shared-memory slots
            // that only the issuing thread reads back: no barrier, and 20 loads in flight per thread instead of the eight that
            // registers allow next to 64 accumulators (with 16 rows of x the FMAs of a body take far less than a DRAM round trip).
            const float *wp = w + size_t(k0) * N + col;
            const int bodies = kc >> 2;
            auto issue = [&](int body) {
                if (body < bodies) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(&w_ring[((body % kSkinnyPipe) * 4 + i) * kSkinnyThreads + threadIdx.x]));
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(wp + size_t(body * 4 + i) * N) : "memory");
                    }
                }
                asm volatile("cp.async.commit_group;" ::: "memory");   // one group per body, empty past the end
            };
            for (int b = 0; b < kSkinnyPipe - 1; ++b) issue(b);
            for (int body = 0; body < bodies; ++body) {
                issue(body + kSkinnyPipe - 1);   // into the slot this thread finished reading in the previous iteration
                asm volatile("cp.async.wait_group %0;" ::"n"(kSkinnyPipe - 1) : "memory");
                const float4 *slot = &w_ring[(body % kSkinnyPipe) * 4 * kSkinnyThreads + threadIdx.x];
                const float4 w0 = slot[0], w1 = slot[kSkinnyThreads], w2 = slot[2 * kSkinnyThreads], w3 = slot[3 * kSkinnyThreads];
                const int k = body * 4;
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const float4 xv = *reinterpret_cast<const float4 *>(&xs[m][k]);
                    acc[m][0] += xv.x * w0.x + xv.y * w1.x + xv.z * w2.x + xv.w * w3.x;
                    acc[m][1 % CPT] += xv.x * w0.y + xv.y * w1.y + xv.z * w2.y + xv.w * w3.y;
                    acc[m][2 % CPT] += xv.x * w0.z + xv.y * w1.z + xv.z * w2.z + xv.w * w3.z;
                    acc[m][3 % CPT] += xv.x * w0.w + xv.y * w1.w + xv.z * w2.w + xv.w * w3.w;
                }
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        } else if (W_KN) {
            const float *wp = w + size_t(k0) * N + col;
#pragma unroll 2
            for (int k = 0; k < kc; k += 4) {
                const float4 w0 = __ldcs(reinterpret_cast<const float4 *>(wp + size_t(k) * N));
                const float4 w1 = __ldcs(reinterpret_cast<const float4 *>(wp + size_t(k + 1) * N));
                const float4 w2 = __ldcs(reinterpret_cast<const float4 *>(wp + size_t(k + 2) * N));
                const float4 w3 = __ldcs(reinterpret_cast<const float4 *>(wp + size_t(k + 3) * N));
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const float4 xv = *reinterpret_cast<const float4 *>(&xs[m][k]);
                    acc[m][0] += xv.x * w0.x + xv.y * w1.x + xv.z * w2.x + xv.w * w3.x;
                    acc[m][1] += xv.x * w0.y + xv.y * w1.y + xv.z * w2.y + xv.w * w3.y;
                    acc[m][2] += xv.x * w0.z + xv.y * w1.z + xv.z * w2.z + xv.w * w3.z;
                    acc[m][3] += xv.x * w0.w + xv.y * w1.w + xv.z * w2.w + xv.w * w3.w;
                }
            }
        } else {
            const float *wp = w + size_t(col) * K + k0;
#pragma unroll 4
            for (int k = 0; k < kc; k += 4) {
                const float4 wv = *reinterpret_cast<const float4 *>(wp + k);  // the row's 128-byte line is reused from L1
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const float4 xv = *reinterpret_cast<const float4 *>(&xs[m][k]);
                    acc[m][0] += xv.x * wv.x + xv.y * wv.y + xv.z * wv.z + xv.w * wv.w;
                }
            }
        }
    }
    if (col_ok) {
        float *out = partial + (size_t(blockIdx.y) * M + row0) * N;
#pragma unroll
        for (int m = 0; m < MR; ++m) {
            if (m >= rows) break;
            if (W_KN)
                *reinterpret_cast<float4 *>(out + size_t(m) * N + col) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
            else
                out[size_t(m) * N + col] = acc[m][0];
        }
    }
    if (!tickets) return;  // skinny_finish_kernel follows

    // The last CTA of this column block to get here adds the partial sums of all splits.
    __threadfence();  // this thread's partial sums are visible device-wide before the ticket is taken
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int *ticket = tickets + blockIdx.z * gridDim.x + blockIdx.x;
        const unsigned int t = atomicAdd(ticket, 1u);
        is_last = (t == gridDim.y - 1);
        if (is_last) *ticket = 0;  // every CTA of this launch has taken its ticket: ready for the next launch
    }
    __syncthreads();
    if (!is_last || !col_ok) return;
    __threadfence();
    const int splits = gridDim.y;
    const size_t per_split = size_t(M) * N;
#pragma unroll
    for (int m = 0; m < MR; ++m) {
        if (m >= rows) break;
        const float *p0 = partial + size_t(row0 + m) * N + col;
        float s[CPT];
        if (W_KN) {
            float4 v = __ldcg(reinterpret_cast<const float4 *>(p0));  // L2: other SMs wrote these
            for (int p = 1; p < splits; ++p) {
                const float4 u = __ldcg(reinterpret_cast<const float4 *>(p0 + p * per_split));
                v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
            }
            s[0] = v.x; s[1 % CPT] = v.y; s[2 % CPT] = v.z; s[3 % CPT] = v.w;
        } else {
            float v = __ldcg(p0);
            for (int p = 1; p < splits; ++p) v += __ldcg(p0 + p * per_split);
            s[0] = v;
        }
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            if (bias) s[c] += bias[col + c];
            y[size_t(row0 + m) * N + col + c] = s[c];
            if (act) act[size_t(row0 + m) * N + col + c] = gelu_tanh(s[c]);
        }
    }
}

// Decode-shaped linear layer with W stored [k][n], in ONE launch and without scratch: the k range is split 8 x S ways - over
// the eight warps of a CTA and over the S CTAs of a thread-block cluster (cluster shape (1, S, 1)) - and the partial sums
// meet in shared memory: first the eight warps of a CTA (fixed order), then the S CTAs of the cluster through distributed
// shared memory (rank order; every CTA finishes 1/S of the block's outputs, adds the bias and applies GELU).  A warp reads
// 512 contiguous bytes of a weight row per load; a CTA covers 128 columns.  With K = 768 and S = 8 a warp reads 12 rows, all
// of its loads are in flight at once, and the layer is one dependent DRAM round trip plus two barrier rounds long - the
// k-split kernel above needs a second pass over partial sums in global memory (a second launch, or a serial tail in the
// last CTA) that costs more than the weight stream itself on these few-microsecond layers.
//   grid (ceil(n / 128), S, ceil(m / MR)); x rows beyond the group are clamped (their sums are computed and dropped).
constexpr int kDecodeThreads = 256;

template <int MR>
__global__ void __launch_bounds__(kDecodeThreads)
decode_gemm_cluster_kernel(float *__restrict__ y, float *__restrict__ act, const float *__restrict__ x, const float *__restrict__ w,
                           const float *__restrict__ bias, int M, int N, int K, int early_launch, int push)
{
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int RH = MR < 4 ? MR : 4;                  // rows per in-CTA reduction pass
    constexpr int kBlocks = (MR * 128 + 255) / 256;      // groups of 256 outputs
    __shared__ __align__(16) float red[8][RH][128];      // per warp: partial sums of RH rows x 128 columns
    __shared__ __align__(16) float cta_sum[MR * 128];    // this CTA's sums, read by the whole cluster (pull form)
    __shared__ __align__(16) float recv[(kBlocks + 15) * 256];   // push form: [S ranks][the output groups this CTA finishes]
    // Push form: every CTA stores its sums straight into the shared memory of the CTA that finishes them, ONE cluster barrier
    // later each CTA adds what it received (local reads) and leaves - no remote round trip, no barrier before exit.  Remote
    // shared memory may only be touched once its CTA runs: all CTAs arrive on the cluster barrier first thing and wait for
    // that phase just before the first remote store, by which time it has long completed.
    if (push) cluster.barrier_arrive();
    const int S = gridDim.y;
    const int rank = blockIdx.y;                         // cluster shape (1, S, 1): the rank inside the cluster
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * 128 + lane * 4;
    const bool col_ok = col < N;                         // n is a multiple of 4 on this path
    const int row0 = blockIdx.z * MR;
    const int rows = min(MR, M - row0);
    x += size_t(row0) * K;
    const int ks = (((K + S * 8 - 1) / (S * 8)) + 3) & ~3;     // k-rows per warp, a multiple of 4 (so is k)
    const int k_begin = min(K, (rank * 8 + warp) * ks), k_end = min(K, k_begin + ks);

    float acc[MR][4];
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[m][c] = 0.0f;
    // Weight loads in flight per thread: the loop is one DRAM round trip per unrolled body (measured: 0.85 us per body with
    // eight loads, whatever n), so with few rows of x the registers go to loads: 24 k-rows per body up to two rows of x (a whole warp share of k = 3072 in a cluster of 16), 12 up to eight.
    constexpr int kUnroll = MR <= 2 ? 6 : MR <= 8 ? 3 : 1;
    // Programmatic dependent launch (early_launch): the next kernel on the stream may start as soon as every CTA of this one
    // is running, and this kernel may have started while its predecessor was still running.  Only the weights (and, later,
    // the bias) are read before griddepcontrol.wait, which returns once the predecessor has completed and its writes are
    // visible; x is read and y written after it.  The caller promises that the predecessor does not write w or bias.
    bool waited = !early_launch;
    if (early_launch) asm volatile("griddepcontrol.launch_dependents;");
    if (col_ok) {
        const float *wp = w + col;
        for (int k = k_begin; k < k_end; k += 4 * kUnroll) {
            float4 wv[4 * kUnroll];   // all loads of the body are issued before the first use
#pragma unroll
            for (int i = 0; i < 4 * kUnroll; ++i)
                wv[i] = k + i < k_end ? __ldcs(reinterpret_cast<const float4 *>(wp + size_t(k + i) * N)) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (!waited) {
                asm volatile("griddepcontrol.wait;" ::: "memory");   // the first body's weight loads are already in flight
                waited = true;
            }
#pragma unroll
            for (int g = 0; g < kUnroll; ++g) {
                if (k + 4 * g >= k_end) break;   // warp-uniform
                const float4 w0 = wv[4 * g], w1 = wv[4 * g + 1], w2 = wv[4 * g + 2], w3 = wv[4 * g + 3];
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const float4 xv = __ldg(reinterpret_cast<const float4 *>(x + size_t(min(m, rows - 1)) * K + k + 4 * g));   // warp-uniform
                    acc[m][0] += xv.x * w0.x + xv.y * w1.x + xv.z * w2.x + xv.w * w3.x;
                    acc[m][1] += xv.x * w0.y + xv.y * w1.y + xv.z * w2.y + xv.w * w3.y;
                    acc[m][2] += xv.x * w0.z + xv.y * w1.z + xv.z * w2.z + xv.w * w3.z;
                    acc[m][3] += xv.x * w0.w + xv.y * w1.w + xv.z * w2.w + xv.w * w3.w;
                }
            }
        }
    }
    if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");   // threads without columns or k-rows: before any output
    // the eight warps of this CTA, warp order
#pragma unroll
    for (int h = 0; h < MR; h += RH) {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < RH; ++j)
            *reinterpret_cast<float4 *>(&red[warp][j][lane * 4]) = make_float4(acc[h + j][0], acc[h + j][1], acc[h + j][2], acc[h + j][3]);
        __syncthreads();
        for (int e = threadIdx.x; e < RH * 128; e += kDecodeThreads) {
            const int j = e >> 7, c = e & 127;
            float s = red[0][j][c];
#pragma unroll
            for (int wv = 1; wv < 8; ++wv) s += red[wv][j][c];
            cta_sum[(h + j) * 128 + c] = s;
        }
    }
    if (push) {
        // group g of 256 outputs is finished by rank g % S, which keeps it as its (g / S)-th group
        const int groups = (rows * 128 + 255) >> 8;
        const int per_owner = ((groups + S - 1) / S) * 256;
        __syncthreads();          // cta_sum complete
        cluster.barrier_wait();   // every CTA of the cluster is running
        for (int e = threadIdx.x; e < rows * 128; e += kDecodeThreads) {
            const int g = e >> 8;
            cluster.map_shared_rank(recv, g % S)[rank * per_owner + (g / S) * 256 + (e & 255)] = cta_sum[e];
        }
        cluster.sync();           // all parts have arrived; nothing remote is touched after this
        for (int g = rank; g < groups; g += S) {
            const int e = g * 256 + threadIdx.x;
            const int m = e >> 7, gc = blockIdx.x * 128 + (e & 127);
            if (e >= rows * 128 || gc >= N) continue;
            const float *part = recv + (g / S) * 256 + threadIdx.x;
            float s = 0.0f;
            for (int q = 0; q < S; ++q) s += part[q * per_owner];   // rank order
            if (bias) s += bias[gc];
            y[size_t(row0 + m) * N + gc] = s;
            if (act) act[size_t(row0 + m) * N + gc] = gelu_tanh(s);
        }
        return;
    }
    cluster.sync();
    // pull form: the S CTAs of the cluster, rank order; this CTA finishes every S-th group of 256 outputs
    for (int e = rank * kDecodeThreads + threadIdx.x; e < rows * 128; e += S * kDecodeThreads) {
        const int m = e >> 7, gc = blockIdx.x * 128 + (e & 127);
        if (gc >= N) continue;
        float s = 0.0f;
        for (int q0 = 0; q0 < S; q0 += 8) {   // up to eight remote loads in flight, added in rank order
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = q0 + j < S ? cluster.map_shared_rank(cta_sum, q0 + j)[e] : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (q0 + j < S) s += v[j];
        }
        if (bias) s += bias[gc];
        y[size_t(row0 + m) * N + gc] = s;
        if (act) act[size_t(row0 + m) * N + gc] = gelu_tanh(s);
    }
    cluster.sync();   // no CTA leaves while its sums may still be read
}

// Decode-shaped linear layer with W stored [k][n] and 9 .. 64 rows of x: a register-tiled fp32 GEMM in one launch.  At these
// row counts the fp32 FMAs weigh as much as the weight stream, so every weight element is loaded to shared memory once per
// CTA (cp.async, four-stage ring of 32 k-rows) and used for all rows: a CTA computes a TM x 128 tile (TM = 16, 32 or 64 rows,
// zero-padded), a thread TM/8 rows x 4 columns.  k is split over the S CTAs of a thread-block cluster (cluster shape
// (1, S, 1)); the partial tiles meet through distributed shared memory in rank order, each CTA finishing 1/S of the rows
// (bias, GELU).  No scratch, no second launch; results do not depend on timing.
//   grid (ceil(n / 128), S, ceil(m / TM)); dynamic shared memory kTileStages * (32 * 128 + TM * 32) floats.
constexpr int kTileStages = 4;
constexpr int kTileK = 32;

//   W_NK: W stored [n][k] instead (the tied un-embedding, grad_x): the stage holds w[128 n][32 k] with rows padded to 36 floats
//   (16-byte reads of 32 consecutive rows then touch every bank once) and a thread owns columns lane, lane + 32, + 64, + 96.
constexpr int kTileNkPitch = 36;

template <int TM, bool W_NK>
__global__ void __launch_bounds__(kDecodeThreads)
decode_tile_cluster_kernel(float *__restrict__ y, float *__restrict__ act, const float *__restrict__ x, const float *__restrict__ w,
                           const float *__restrict__ bias, int M, int N, int K, int early_launch)
{
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int RT = TM / 8;                                   // rows per thread
    constexpr int kWFloats = W_NK ? 128 * kTileNkPitch : kTileK * 128;
    constexpr int kStageFloats = kWFloats + TM * kTileK;         // w[32][128] (or w[128][36]) then x[TM][32]
    extern __shared__ __align__(16) float tile_smem[];
    const int S = gridDim.y, rank = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col0 = blockIdx.x * 128;
    {   // row group of this cluster (blockIdx.z)
        const int row0 = blockIdx.z * TM;
        x += size_t(row0) * K;
        y += size_t(row0) * N;
        if (act) act += size_t(row0) * N;
        M = min(TM, M - row0);
    }
    const int k_per_cta = (((K + S - 1) / S) + 3) & ~3;
    const int k_begin = min(K, rank * k_per_cta), k_end = min(K, k_begin + k_per_cta);
    const int chunks = (k_end - k_begin + kTileK - 1) / kTileK;

    auto load_w = [&](int chunk) {   // weights: 32 rows of 32 16-byte pieces
        if (chunk >= chunks) return;
        float *ws = tile_smem + (chunk % kTileStages) * kStageFloats;
        const int k0 = k_begin + chunk * kTileK;
#pragma unroll
        for (int i = 0; i < (kTileK * 32) / kDecodeThreads; ++i) {
            const int c = threadIdx.x + i * kDecodeThreads;
            bool ok;
            const float *src;
            unsigned dst;
            if (W_NK) {   // 128 rows (n) of 8 pieces along k
                const int r = c >> 3, q = c & 7;
                ok = col0 + r < N && k0 + 4 * q < k_end;
                src = ok ? w + size_t(col0 + r) * K + k0 + 4 * q : w;
                dst = static_cast<unsigned>(__cvta_generic_to_shared(ws + r * kTileNkPitch + 4 * q));
            } else {
                const int r = c >> 5, q = c & 31;
                ok = k0 + r < k_end && col0 + 4 * q < N;
                src = ok ? w + size_t(k0 + r) * N + col0 + 4 * q : w;
                dst = static_cast<unsigned>(__cvta_generic_to_shared(ws + r * 128 + 4 * q));
            }
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(ok ? 16 : 0) : "memory");   // out of range: zero fill
        }
    };
    auto load_x = [&](int chunk) {   // x: TM rows of 8 pieces
        if (chunk >= chunks) return;
        float *xs = tile_smem + (chunk % kTileStages) * kStageFloats + kWFloats;
        const int k0 = k_begin + chunk * kTileK;
#pragma unroll
        for (int i = 0; i < (TM * 8 + kDecodeThreads - 1) / kDecodeThreads; ++i) {
            const int c = threadIdx.x + i * kDecodeThreads, r = c >> 3, q = c & 7;
            if (c < TM * 8) {
                const bool ok = r < M && k0 + 4 * q < k_end;
                const float *src = ok ? x + size_t(r) * K + k0 + 4 * q : x;
                const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(xs + r * kTileK + 4 * q));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(ok ? 16 : 0) : "memory");
            }
        }
    };
    auto commit = [] { asm volatile("cp.async.commit_group;" ::: "memory"); };   // one group per chunk, empty past the end

    float acc[RT][4];
#pragma unroll
    for (int j = 0; j < RT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = 0.0f;

    // Early launch: the first stages' weights are requested before the predecessor on the stream is known to have finished,
    // x only after (the first group then holds all of those weights and the first x chunk: still in chunk order).
    for (int sidx = 0; sidx < kTileStages - 1; ++sidx) load_w(sidx);
    if (early_launch) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int sidx = 0; sidx < kTileStages - 1; ++sidx) {
        load_x(sidx);
        commit();
    }
    for (int chunk = 0; chunk < chunks; ++chunk) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kTileStages - 2) : "memory");   // this chunk has landed (own copies)
        __syncthreads();                                                              // ... everyone's; and the slot refilled below is free
        load_w(chunk + kTileStages - 1);
        load_x(chunk + kTileStages - 1);
        commit();
        const float *ws = tile_smem + (chunk % kTileStages) * kStageFloats;
        const float *xs = ws + kWFloats + warp * RT * kTileK;
#pragma unroll
        for (int kk = 0; kk < kTileK; kk += 4) {
            float4 xv[RT];
#pragma unroll
            for (int j = 0; j < RT; ++j) xv[j] = *reinterpret_cast<const float4 *>(xs + j * kTileK + kk);   // warp-uniform: broadcast
            if (W_NK) {
                float4 wc[4];   // four k-values of each of this thread's four columns
#pragma unroll
                for (int c = 0; c < 4; ++c) wc[c] = *reinterpret_cast<const float4 *>(ws + (lane + 32 * c) * kTileNkPitch + kk);
#pragma unroll
                for (int j = 0; j < RT; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[j][c] += xv[j].x * wc[c].x + xv[j].y * wc[c].y + xv[j].z * wc[c].z + xv[j].w * wc[c].w;
                continue;
            }
            const float4 w0 = *reinterpret_cast<const float4 *>(ws + (kk + 0) * 128 + lane * 4);
            const float4 w1 = *reinterpret_cast<const float4 *>(ws + (kk + 1) * 128 + lane * 4);
            const float4 w2 = *reinterpret_cast<const float4 *>(ws + (kk + 2) * 128 + lane * 4);
            const float4 w3 = *reinterpret_cast<const float4 *>(ws + (kk + 3) * 128 + lane * 4);
#pragma unroll
            for (int j = 0; j < RT; ++j) {
                acc[j][0] += xv[j].x * w0.x + xv[j].y * w1.x + xv[j].z * w2.x + xv[j].w * w3.x;
                acc[j][1] += xv[j].x * w0.y + xv[j].y * w1.y + xv[j].z * w2.y + xv[j].w * w3.y;
                acc[j][2] += xv[j].x * w0.z + xv[j].y * w1.z + xv[j].z * w2.z + xv[j].w * w3.z;
                acc[j][3] += xv[j].x * w0.w + xv[j].y * w1.w + xv[j].z * w2.w + xv[j].w * w3.w;
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // the successor may start now (its CTAs hold shared memory while they wait: not before this kernel's main loop is over)
    if (early_launch) asm volatile("griddepcontrol.launch_dependents;");
    __syncthreads();   // all reads of the ring are done: it becomes this CTA's partial tile [TM][128]
#pragma unroll
    for (int j = 0; j < RT; ++j) {
        if (W_NK) {
#pragma unroll
            for (int c = 0; c < 4; ++c) tile_smem[(warp * RT + j) * 128 + lane + 32 * c] = acc[j][c];
        } else {
            *reinterpret_cast<float4 *>(tile_smem + (warp * RT + j) * 128 + lane * 4) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
        }
    }
    cluster.sync();
    // rank order; this CTA finishes every S-th group of 256 four-column pieces
    for (int e = rank * kDecodeThreads + threadIdx.x; e < M * 32; e += S * kDecodeThreads) {
        const int m = e >> 5, gc = col0 + 4 * (e & 31);
        if (gc >= N) continue;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q0 = 0; q0 < S; q0 += 8) {   // up to eight remote loads in flight, added in rank order
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                v[j] = q0 + j < S ? reinterpret_cast<const float4 *>(cluster.map_shared_rank(tile_smem, q0 + j))[e] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (q0 + j < S) { sum.x += v[j].x; sum.y += v[j].y; sum.z += v[j].z; sum.w += v[j].w; }
        }
        if (bias) { sum.x += bias[gc]; sum.y += bias[gc + 1]; sum.z += bias[gc + 2]; sum.w += bias[gc + 3]; }   // bias need not be 16-byte aligned
        *reinterpret_cast<float4 *>(y + size_t(m) * N + gc) = sum;
        if (act) *reinterpret_cast<float4 *>(act + size_t(m) * N + gc) = make_float4(gelu_tanh(sum.x), gelu_tanh(sum.y), gelu_tanh(sum.z), gelu_tanh(sum.w));
    }
    cluster.sync();   // no CTA leaves while its tile may still be read
}

// Decode-shaped product with W stored [n][k] (the tied un-embedding: logits = x . wte^T; also grad_x = grad_y . w^T): one warp
// per pair of weight rows and group of up to MR rows of x (blockIdx.x = group, the fastest-varying index, so that the CTAs
// that read the same weight rows for different groups run at the same time and all but one of them hit L2).  A lane reads 16 contiguous bytes and the warp 512 contiguous bytes of
// a row per load (the k-split kernel above lets every thread walk its own row, 32 rows per load instruction, and reaches
// about half of the HBM bandwidth); x sits in shared memory; the 32 partial sums of a row meet in a butterfly of shuffles
// (fixed order).  One launch, no scratch.  HBM-bound: 4 * n * k bytes.
//   dynamic shared memory: MR * K floats (at most 48 KiB);  grid (groups, any): warps stride over row pairs.
template <int MR>
__global__ void __launch_bounds__(kDecodeThreads)
rowwise_gemv_kernel(float *__restrict__ y, const float *__restrict__ x, const float *__restrict__ w, int M, int N, int K)
{
    extern __shared__ __align__(16) float xs_dyn[];   // [MR][K]
    const int row0 = blockIdx.x * MR;
    x += size_t(row0) * K;
    y += size_t(row0) * N;
    M = min(MR, M - row0);   // rows of this group
    const int kq = K >> 2;
    for (int i = threadIdx.x; i < MR * kq; i += kDecodeThreads) {
        const int m = i / kq, q = i - m * kq;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < M) v = *reinterpret_cast<const float4 *>(x + size_t(m) * K + 4 * q);
        *reinterpret_cast<float4 *>(xs_dyn + size_t(m) * K + 4 * q) = v;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = gridDim.y * (kDecodeThreads / 32);
    constexpr int U = 3;   // loads in flight per lane and row
    for (int n0 = (blockIdx.y * (kDecodeThreads / 32) + warp) * 2; n0 < N; n0 += warps * 2) {
        const float *wa = w + size_t(n0) * K;
        const float *wb = w + size_t(min(n0 + 1, N - 1)) * K;   // odd n: the last row twice, second result dropped
        float acc[2][MR];
#pragma unroll
        for (int m = 0; m < MR; ++m) acc[0][m] = acc[1][m] = 0.0f;
        for (int k0 = lane * 4; k0 < K; k0 += 128 * U) {
            float4 a[U], b[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int k = k0 + 128 * u;
                a[u] = k < K ? __ldcs(reinterpret_cast<const float4 *>(wa + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
                b[u] = k < K ? __ldcs(reinterpret_cast<const float4 *>(wb + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int k = k0 + 128 * u;
                if (k < K) {
#pragma unroll
                    for (int m = 0; m < MR; ++m) {
                        const float4 xv = *reinterpret_cast<const float4 *>(xs_dyn + size_t(m) * K + k);
                        acc[0][m] += xv.x * a[u].x + xv.y * a[u].y + xv.z * a[u].z + xv.w * a[u].w;
                        acc[1][m] += xv.x * b[u].x + xv.y * b[u].y + xv.z * b[u].z + xv.w * b[u].w;
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                float v = acc[r][m];
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                if (lane == ((m * 2 + r) & 31) && m < M && n0 + r < N) y[size_t(m) * N + n0 + r] = v;
            }
    }
}

// y = sum_s partial[s] (s ascending) + bias; act = gelu_tanh(y)
__global__ void skinny_finish_kernel(float *__restrict__ y, float *__restrict__ act, const float *__restrict__ partial,
                                     const float *__restrict__ bias, int M, int N, int splits)
{
    const long long total = 1LL * M * N;
    const long long stride = 1LL * gridDim.x * blockDim.x;
    for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float s = partial[i];
        int p = 1;
        for (; p + 8 <= splits; p += 8) {   // eight loads in flight, added in split order
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = partial[(p + j) * total + i];
#pragma unroll
            for (int j = 0; j < 8; ++j) s += v[j];
        }
        for (; p < splits; ++p) s += partial[p * total + i];
        if (bias) s += bias[i % N];
        y[i] = s;
        if (act) act[i] = gelu_tanh(s);
    }
}

}  // namespace gptb200
