// extern "C" layer of libgptb200: context, operand checks, tensor-map construction, tile / split-K
// selection and kernel launches.  No cuBLAS, no CPU fallback: a call either runs CUDA kernels of this
// library on the context's stream or returns an error code.
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <algorithm>
#include <set>

#include <cuda.h>
#include <cuda_runtime.h>

#include "ctx_internal.h"
#include "gemm_plan.h"
#include "gemm_sm100.cuh"
#include "gemm_sm100_pair.cuh"
#include "skinny_sm100.cuh"
#include "kernels_misc.cuh"

using namespace gptb200;

namespace gptb200 {

int ensure_workspace(gptb200_ctx *ctx, size_t bytes)
{
    if (bytes <= ctx->ws_bytes) return GPTB200_OK;
    if (bytes > ctx->ws_limit) return fail(ctx, GPTB200_ERR_WORKSPACE, "scratch request of %zu bytes exceeds limit %zu", bytes, ctx->ws_limit);
    // Growing the scratch buffer waits for queued work: earlier kernels may still read the old one.
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->ws) CUDA_TRY(ctx, cudaFree(ctx->ws));
    ctx->ws = nullptr;
    ctx->ws_bytes = 0;
    const size_t rounded = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    CUDA_TRY(ctx, cudaMalloc(&ctx->ws, rounded));
    ctx->ws_bytes = rounded;
    return GPTB200_OK;
}

}  // namespace gptb200

namespace {

constexpr int kDbiasTickets = 4096;   // tile columns x 16 that the fused bias gradient can serve (n <= 65536)

// One GEMM operand as stored: `rows` x `cols` fp32, row pitch `cols`.
// K-major operand: rows = free extent (M or N), cols = reduction extent.
// MN-major operand: rows = reduction extent, cols = free extent.
// `mn_major` picks the shared-memory swizzle the tensor core expects for that major-ness: 16-byte chunks
// for K-major tiles, 32-byte chunks for MN-major tiles of 32-bit elements.
int make_tmap(gptb200_ctx *ctx, CUtensorMap *map, const float *base, long long rows, long long cols, int box_cols, int box_rows, bool mn_major)
{
    const TmapKey key{reinterpret_cast<uintptr_t>(base), cols, rows, 0, box_cols, box_rows, mn_major ? 1 : 0};
    const auto hit = ctx->tmaps.find(key);
    if (hit != ctx->tmaps.end()) {
        *map = hit->second;
        return GPTB200_OK;
    }
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * sizeof(float)};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = ctx->encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ctx->tmap_encodes++;
    if (r != CUDA_SUCCESS)
        return fail(ctx, GPTB200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) rows=%lld cols=%lld box=%dx%d", int(r), rows, cols, box_rows, box_cols);
    if (ctx->tmaps.size() >= kTmapCacheMax) ctx->tmaps.clear();
    ctx->tmaps.emplace(key, *map);
    return GPTB200_OK;
}

// Tensor map of an operand's expanded bf16 correction matrix (split_operand_kernel), described in 4-byte words:
//   K-major: [rows][k8 words], box 32 words x 128 rows (like the raw operand);  MN-major: [2 k8 rows][cols / 2 words], box 32 words x 64 rows.
int make_pre_tmap(gptb200_ctx *ctx, CUtensorMap *map, const void *base, long long rows, long long words, int box_rows)
{
    const TmapKey key{reinterpret_cast<uintptr_t>(base), words, rows, 0, 32, box_rows, 3};
    const auto hit = ctx->tmaps.find(key);
    if (hit != ctx->tmaps.end()) {
        *map = hit->second;
        return GPTB200_OK;
    }
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(words), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(words) * 4};
    cuuint32_t box[2] = {32, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = ctx->encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ctx->tmap_encodes++;
    if (r != CUDA_SUCCESS) return fail(ctx, GPTB200_ERR_CUDA, "cuTensorMapEncodeTiled (correction tiles) failed (%d) rows=%lld words=%lld", int(r), rows, words);
    if (ctx->tmaps.size() >= kTmapCacheMax) ctx->tmaps.clear();
    ctx->tmaps.emplace(key, *map);
    return GPTB200_OK;
}

// 4-D tensor map of a batched operand or output: (cols, inner batch, rows, outer batch) with element strides (1, stride_inner,
// ld, stride_outer); box cols x rows of one batch.  swizzle: 0 = 128-byte (K-major operands, outputs), 1 = 128-byte with 32-byte
// atoms (MN-major operands).
int make_batched_tmap(gptb200_ctx *ctx, CUtensorMap *map, const float *base, long long cols, long long rows, long long inner, long long outer,
                      long long ld, long long stride_inner, long long stride_outer, int box_cols, int box_rows, int swizzle)
{
    if (inner == 1) stride_inner = ld;   // the coordinate is always 0: keep the strides in growing order
    if (outer == 1) stride_outer = ld * rows;
    const TmapKey key{reinterpret_cast<uintptr_t>(base), cols, rows, ld, box_cols, box_rows, 4 + swizzle, inner, outer, stride_inner, stride_outer};
    const auto hit = ctx->tmaps.find(key);
    if (hit != ctx->tmaps.end()) {
        *map = hit->second;
        return GPTB200_OK;
    }
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(outer)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(stride_inner) * 4, static_cast<cuuint64_t>(ld) * 4, static_cast<cuuint64_t>(stride_outer) * 4};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(box_cols), 1, static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = ctx->encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   swizzle ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ctx->tmap_encodes++;
    if (r != CUDA_SUCCESS)
        return fail(ctx, GPTB200_ERR_CUDA, "cuTensorMapEncodeTiled (batched) failed (%d) cols=%lld rows=%lld batches=%lldx%lld strides=%lld,%lld,%lld", int(r), cols,
                    rows, inner, outer, stride_inner, ld, stride_outer);
    if (ctx->tmaps.size() >= kTmapCacheMax) ctx->tmaps.clear();
    ctx->tmaps.emplace(key, *map);
    return GPTB200_OK;
}

constexpr double kExact3xFlops = 6.0e9;   // launches up to this size take the TF32 correction terms when "exact3x" is automatic

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct GemmCall {
    int M, N, K;
    const float *a;  // K-major: [M][K]; MN-major: [K][M]
    bool a_mn;
    const float *b;  // K-major: [N][K]; MN-major: [K][N]
    bool b_mn;
    float *out;      // [M][N]
    float *act;      // optional
    const float *bias;
    bool accumulate;  // out += result
    float *dbias = nullptr;  // grad_w form only: dbias[N] += column sums of b, inside the same launch when the CTA-pair kernel runs
    const float *gelu_src = nullptr;  // out = result * gelu_tanh'(gelu_src) element by element, when the CTA-pair kernel runs
};

template <int BN, bool A_MN, bool B_MN, bool X3>
cudaError_t launch_instance(gptb200_ctx *ctx, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to, const CUtensorMap &tact,
                            const GemmParams &p, int grid)
{
    using C = GemmCfg<BN, X3>;
    auto kernel = gemm_tcgen05_kernel<BN, A_MN, B_MN, X3>;
    const void *key = reinterpret_cast<const void *>(kernel);
    if (!ctx->configured.count(key)) {  // the attribute is per device, the context is bound to one device
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return e;
        ctx->configured.insert(key);
    }
    kernel<<<grid, C::kThreads, C::kSmemBytes, ctx->stream>>>(ta, tb, to, tact, p);
    return cudaGetLastError();
}

template <int BN, bool X3>
cudaError_t launch_majors(gptb200_ctx *ctx, bool a_mn, bool b_mn, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to,
                          const CUtensorMap &tact, const GemmParams &p, int grid)
{
    if (!a_mn && b_mn) return launch_instance<BN, false, true, X3>(ctx, ta, tb, to, tact, p, grid);
    if (!a_mn && !b_mn) return launch_instance<BN, false, false, X3>(ctx, ta, tb, to, tact, p, grid);
    if (a_mn && b_mn) return launch_instance<BN, true, true, X3>(ctx, ta, tb, to, tact, p, grid);
    return cudaErrorInvalidValue;  // (MN, K) does not occur on this path
}

template <bool A_MN, bool B_MN, bool X3, bool DB = false>
cudaError_t launch_pair_instance(gptb200_ctx *ctx, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to, const CUtensorMap &tact,
                                 const CUtensorMap &tpre, const GemmParams &p, int grid)
{
    using C = PairCfg<X3>;
    auto kernel = gemm_tcgen05_pair_kernel<A_MN, B_MN, X3, DB>;
    const void *key = reinterpret_cast<const void *>(kernel);
    if (!ctx->configured.count(key)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return e;
        ctx->configured.insert(key);
    }
    kernel<<<grid, C::kThreads, C::kSmemBytes, ctx->stream>>>(ta, tb, to, tact, tpre, p);  // cluster shape (2,1,1) is a kernel attribute
    return cudaGetLastError();
}

template <bool X3>
cudaError_t launch_pair(gptb200_ctx *ctx, bool a_mn, bool b_mn, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to,
                        const CUtensorMap &tact, const CUtensorMap &tpre, const GemmParams &p, int grid)
{
    if (!a_mn && b_mn) return launch_pair_instance<false, true, X3>(ctx, ta, tb, to, tact, tpre, p, grid);
    if (!a_mn && !b_mn) return launch_pair_instance<false, false, X3>(ctx, ta, tb, to, tact, tpre, p, grid);
    if (a_mn && b_mn) {
        if (p.dbias) return launch_pair_instance<true, true, X3, true>(ctx, ta, tb, to, tact, tpre, p, grid);
        return launch_pair_instance<true, true, X3>(ctx, ta, tb, to, tact, tpre, p, grid);
    }
    return cudaErrorInvalidValue;
}

// Output tensor [depth][rows][cols] (depth > 1 only for split-K partial tiles), written in
// [32 rows x box_cols] pieces from swizzled staging tiles (128-byte swizzle for 32 columns, 64-byte swizzle for 16).
int make_out_tmap(gptb200_ctx *ctx, CUtensorMap *map, float *base, long long depth, long long rows, long long cols, int box_cols = 32)
{
    const TmapKey key{reinterpret_cast<uintptr_t>(base), cols, rows, depth, box_cols, 32, 2};
    const auto hit = ctx->tmaps.find(key);
    if (hit != ctx->tmaps.end()) {
        *map = hit->second;
        return GPTB200_OK;
    }
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(depth)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols) * sizeof(float), static_cast<cuuint64_t>(rows) * cols * sizeof(float)};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(box_cols), 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = ctx->encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   box_cols == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ctx->tmap_encodes++;
    if (r != CUDA_SUCCESS)
        return fail(ctx, GPTB200_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed (%d) depth=%lld rows=%lld cols=%lld", int(r), depth, rows, cols);
    if (ctx->tmaps.size() >= kTmapCacheMax) ctx->tmaps.clear();
    ctx->tmaps.emplace(key, *map);
    return GPTB200_OK;
}

template <bool W_KN>
int launch_skinny(gptb200_ctx *ctx, int mr, dim3 grid, float *partial, const GemmCall &c, int k_per_split, unsigned int *tickets)
{
    // 16-row groups of a [k][n] weight: weight loads pipelined through shared memory (see the kernel)
    const bool pipe = W_KN && mr == 16 && ctx->skinny_pipelined;
    const size_t smem = pipe ? size_t(kSkinnyPipe) * 4 * kSkinnyThreads * sizeof(float4) : 0;
    if (pipe) {
        auto kernel = skinny_gemm_kernel<16, W_KN>;
        const void *key = reinterpret_cast<const void *>(kernel);
        if (!ctx->configured.count(key)) {
            CUDA_TRY(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            ctx->configured.insert(key);
        }
    }
    switch (mr) {
        case 1: skinny_gemm_kernel<1, W_KN><<<grid, kSkinnyThreads, 0, ctx->stream>>>(partial, c.a, c.b, c.M, c.N, c.K, k_per_split, c.out, c.act, c.bias, tickets, 0); break;
        case 2: skinny_gemm_kernel<2, W_KN><<<grid, kSkinnyThreads, 0, ctx->stream>>>(partial, c.a, c.b, c.M, c.N, c.K, k_per_split, c.out, c.act, c.bias, tickets, 0); break;
        case 4: skinny_gemm_kernel<4, W_KN><<<grid, kSkinnyThreads, 0, ctx->stream>>>(partial, c.a, c.b, c.M, c.N, c.K, k_per_split, c.out, c.act, c.bias, tickets, 0); break;
        case 8: skinny_gemm_kernel<8, W_KN><<<grid, kSkinnyThreads, 0, ctx->stream>>>(partial, c.a, c.b, c.M, c.N, c.K, k_per_split, c.out, c.act, c.bias, tickets, 0); break;
        default: skinny_gemm_kernel<16, W_KN><<<grid, kSkinnyThreads, smem, ctx->stream>>>(partial, c.a, c.b, c.M, c.N, c.K, k_per_split, c.out, c.act, c.bias, tickets, pipe ? 1 : 0); break;
    }
    ctx->launches++;
    CUDA_TRY(ctx, cudaGetLastError());
    return GPTB200_OK;
}

// Clusters of 16 CTAs are a non-portable size: whether this device (or this slice of it) can schedule one is asked once per
// context, for the most demanding of the decode kernels; if not, clusters stay at eight.
bool cluster16_allowed(gptb200_ctx *ctx)
{
    if (ctx->cluster16 < 0) {
        auto kernel = decode_tile_cluster_kernel<64, false>;
        const size_t smem = size_t(kTileStages) * (kTileK * 128 + 64 * kTileK) * sizeof(float);
        int clusters = 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 16, 1);
        cfg.blockDim = dim3(kDecodeThreads);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 16;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const bool ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) == cudaSuccess &&
                        cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess &&
                        cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters >= 1;
        if (!ok) cudaGetLastError();   // a refused query must not surface as the next launch's error
        ctx->cluster16 = ok ? 1 : 0;
    }
    return ctx->cluster16 == 1;
}

// One-launch cluster kernel for decode-shaped linear layers with W stored [k][n] (see decode_gemm_cluster_kernel).
template <int MR>
int launch_decode_cluster(gptb200_ctx *ctx, const GemmCall &c, int cluster, int groups)
{
    auto kernel = decode_gemm_cluster_kernel<MR>;
    if (cluster > 8) {
        const void *key = reinterpret_cast<const void *>(kernel);
        if (!ctx->configured.count(key)) {
            CUDA_TRY(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
            ctx->configured.insert(key);
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((c.N + 127) / 128, cluster, groups);
    cfg.blockDim = dim3(kDecodeThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = cluster;
    attr[0].val.clusterDim.z = 1;
    // option "decode_early_launch": this kernel may start while the kernel before it on the stream still runs (it reads only
    // w and bias until that kernel has completed) and lets its own successor start early in turn
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->decode_early_launch ? 2 : 1;
    CUDA_TRY(ctx, cudaLaunchKernelEx(&cfg, kernel, c.out, c.act, c.a, c.b, c.bias, c.M, c.N, c.K, ctx->decode_early_launch ? 1 : 0, ctx->skinny_push ? 1 : 0));
    ctx->launches++;
    return GPTB200_OK;
}

// One-launch register-tiled cluster kernel for 9 .. 64 rows with W stored [k][n] (see decode_tile_cluster_kernel).
template <int TM, bool W_NK>
int launch_decode_tile(gptb200_ctx *ctx, const GemmCall &c, int cluster)
{
    auto kernel = decode_tile_cluster_kernel<TM, W_NK>;
    const size_t smem = size_t(kTileStages) * ((W_NK ? 128 * kTileNkPitch : kTileK * 128) + TM * kTileK) * sizeof(float);
    const void *key = reinterpret_cast<const void *>(kernel);
    if (!ctx->configured.count(key)) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        CUDA_TRY(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        ctx->configured.insert(key);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((c.N + 127) / 128, cluster, (c.M + TM - 1) / TM);
    cfg.blockDim = dim3(kDecodeThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = cluster;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // Early launch is measured slower for this kernel (its waiting CTAs hold 74 - 100 KiB of shared memory each; 64 rows: 1.13
    // against 1.04 ms per decode step): option value 2 forces it, 1 applies to the per-warp cluster kernel only.
    const bool early = ctx->decode_early_launch >= 2;
    cfg.numAttrs = early ? 2 : 1;
    CUDA_TRY(ctx, cudaLaunchKernelEx(&cfg, kernel, c.out, c.act, c.a, c.b, c.bias, c.M, c.N, c.K, early ? 1 : 0));
    ctx->launches++;
    return GPTB200_OK;
}

// One-launch warp-per-row kernel for decode-shaped products with W stored [n][k] (see rowwise_gemv_kernel).
template <int MR>
int launch_rowwise(gptb200_ctx *ctx, const GemmCall &c)
{
    const int warps_needed = (c.N + 1) / 2;
    const int groups = (c.M + MR - 1) / MR;
    const int ctas = std::max(1, std::min(std::max(1, ctx->num_sms * 4 / groups), (warps_needed + kDecodeThreads / 32 - 1) / (kDecodeThreads / 32)));
    rowwise_gemv_kernel<MR><<<dim3(groups, ctas), kDecodeThreads, size_t(MR) * c.K * sizeof(float), ctx->stream>>>(c.out, c.a, c.b, c.M, c.N, c.K);
    ctx->launches++;
    CUDA_TRY(ctx, cudaGetLastError());
    return GPTB200_OK;
}

// Decode-shaped forward GEMMs (m <= 64, x K-major): stream the weights once, split k over CTAs; the partial sums are added
// by the last CTA of each column block (one launch) or, when splits * rows is large, by a second small kernel.
// HBM-bound: 4*k*n bytes per call.
int run_skinny(gptb200_ctx *ctx, const GemmCall &c, const GemmPlan &pl)
{
    const bool w_kn = c.b_mn;  // W stored [k][n]
    DecodeOptions o;
    o.cluster = ctx->skinny_cluster; o.cluster_rows = ctx->skinny_cluster_rows;
    o.tile = ctx->skinny_tile; o.tile_rows = ctx->skinny_tile_rows;
    o.rowwise = ctx->skinny_rowwise; o.rowwise_rows = ctx->skinny_rowwise_rows;
    o.cluster16_ok = ctx->skinny_cluster >= 16 ? cluster16_allowed(ctx) : false;
    const DecodePlan d = plan_decode(c.M, c.N, c.K, w_kn, c.bias != nullptr || c.act != nullptr, ctx->num_sms, o);
    if (d.kernel == DECODE_WARP_CLUSTER) {
        switch (d.rows) {
            case 1: return launch_decode_cluster<1>(ctx, c, d.cluster, d.groups);
            case 2: return launch_decode_cluster<2>(ctx, c, d.cluster, d.groups);
            case 4: return launch_decode_cluster<4>(ctx, c, d.cluster, d.groups);
            case 8: return launch_decode_cluster<8>(ctx, c, d.cluster, d.groups);
            default: return launch_decode_cluster<16>(ctx, c, d.cluster, d.groups);
        }
    }
    if (d.kernel == DECODE_TILE_CLUSTER) {
        if (w_kn) {
            if (d.rows == 16) return launch_decode_tile<16, false>(ctx, c, d.cluster);
            if (d.rows == 32) return launch_decode_tile<32, false>(ctx, c, d.cluster);
            return launch_decode_tile<64, false>(ctx, c, d.cluster);
        }
        if (d.rows == 16) return launch_decode_tile<16, true>(ctx, c, d.cluster);
        if (d.rows == 32) return launch_decode_tile<32, true>(ctx, c, d.cluster);
        return launch_decode_tile<64, true>(ctx, c, d.cluster);
    }
    if (d.kernel == DECODE_ROWWISE) {
        switch (d.rows) {
            case 1: return launch_rowwise<1>(ctx, c);
            case 2: return launch_rowwise<2>(ctx, c);
            case 4: return launch_rowwise<4>(ctx, c);
            case 8: return launch_rowwise<8>(ctx, c);
            default: return launch_rowwise<16>(ctx, c);
        }
    }
    const int mr = d.rows, groups = d.groups;   // k-split kernel
    const int rc = ensure_workspace(ctx, pl.workspace_bytes);
    if (rc != GPTB200_OK) return rc;
    const dim3 grid(pl.tiles_n, pl.splits, groups);
    // The last CTA adds the splits one dependent L2 load after the other: measured slower than a second launch beyond a few splits
    // (48 splits: 14 us against 7.6 + launch).
    const bool fused = pl.tiles_n * groups <= kSkinnyMaxTickets &&
                       (ctx->skinny_fused > 0 || (ctx->skinny_fused == 0 && pl.splits <= 2));
    unsigned int *tickets = fused ? ctx->d_pair_flags + size_t(ctx->num_sms) * 8 + 2 : nullptr;   // behind the pair kernel's words
    const int rc2 = w_kn ? launch_skinny<true>(ctx, mr, grid, ctx->ws, c, pl.kb_per_split, tickets)
                         : launch_skinny<false>(ctx, mr, grid, ctx->ws, c, pl.kb_per_split, tickets);
    if (rc2 != GPTB200_OK || fused) return rc2;
    const long long total = 1LL * c.M * c.N;
    skinny_finish_kernel<<<static_cast<int>(std::min<long long>((total + 255) / 256, 1LL * ctx->num_sms * 4)), 256, 0, ctx->stream>>>(
        c.out, c.act, ctx->ws, c.bias, c.M, c.N, pl.splits);
    ctx->launches++;
    CUDA_TRY(ctx, cudaGetLastError());
    return GPTB200_OK;
}

GemmPlanInput plan_input(const gptb200_ctx *ctx, const GemmCall &c)
{
    GemmPlanInput in{};
    in.M = c.M; in.N = c.N; in.K = c.K;
    in.a_mn = c.a_mn; in.b_mn = c.b_mn;
    in.has_epilogue = c.bias != nullptr || c.act != nullptr;
    in.accumulate = c.accumulate;
    in.aligned = aligned16(c.a) && aligned16(c.b) && aligned16(c.out) && (!c.act || aligned16(c.act));
    in.num_sms = ctx->max_sms > 0 ? std::min(ctx->max_sms, ctx->num_sms) : ctx->num_sms;
    in.opt_tile_n = ctx->tile_n; in.opt_max_splits = ctx->max_splits; in.opt_pair = ctx->pair; in.opt_stream_k = ctx->stream_k; in.opt_skinny = ctx->skinny; in.opt_skinny_rows = ctx->skinny_rows;
    in.ws_limit = ctx->ws_limit;
    return in;
}

// *dbias_fused (optional) reports whether c.dbias was computed inside the GEMM launch; if not, the caller runs the
// separate column-sum kernels.
// *gelu_fused (optional): whether c.gelu_src was applied inside the launch (CTA-pair kernel only).
int run_gemm(gptb200_ctx *ctx, const GemmCall &c, bool *dbias_fused = nullptr, bool *gelu_fused = nullptr)
{
    if (dbias_fused) *dbias_fused = false;
    if (gelu_fused) *gelu_fused = false;
    const GemmPlan pl = plan_gemm(plan_input(ctx, c));
    if (pl.kernel == KERNEL_NONE) return GPTB200_OK;
    if (pl.kernel == KERNEL_SKINNY) return run_skinny(ctx, c, pl);
    if (pl.kernel == KERNEL_SIMT) {
        // Plain SIMT kernel for the shapes TMA cannot address.
        const long long a_rs = c.a_mn ? 1 : c.K, a_cs = c.a_mn ? c.M : 1;
        const long long b_rs = c.b_mn ? c.N : 1, b_cs = c.b_mn ? 1 : c.K;
        dim3 block(32, 8);
        dim3 grid(pl.tiles_n, pl.tiles_m);
        simt_gemm_kernel<<<grid, block, 0, ctx->stream>>>(c.M, c.N, c.K, c.a, a_rs, a_cs, c.b, b_rs, b_cs, c.out, c.act, c.bias, c.N,
                                                          c.accumulate ? EPI_ACCUM : EPI_STORE);
        ctx->launches++;
        CUDA_TRY(ctx, cudaGetLastError());
        return GPTB200_OK;
    }

    const bool x3 = ctx->mode == GPTB200_MODE_3XTF32;
    const bool pair = pl.kernel == KERNEL_PAIR;
    const int bn = pl.tile_n;
    const int splits = pl.splits;
    const size_t bytes_per_split = size_t(c.M) * size_t(c.N) * sizeof(float);
    GemmParams p{};
    char *pre_buf = nullptr;   // expanded correction matrix of the operand that is split before the launch (3xTF32, CTA pairs)
    p.M = c.M;
    p.N = c.N;
    p.K = c.K;
    p.tiles_m = pl.tiles_m;
    p.tiles_n = pl.tiles_n;
    p.num_kb = pl.num_kb;
    p.kb_per_split = pl.kb_per_split;
    p.splits = splits;
    p.status = ctx->d_status;

    float *out_base = c.out;
    if (pair && ctx->d_trace) {
        CUDA_TRY(ctx, cudaMemsetAsync(ctx->d_trace, 0, sizeof(long long) * kTraceEvents * kTraceSlots, ctx->stream));
        p.trace = ctx->d_trace;
    }
    if (pair && c.gelu_src && !c.accumulate && aligned16(c.gelu_src)) {
        p.gelu_src = c.gelu_src;
        if (gelu_fused) *gelu_fused = true;
    }
    if (pair) {
        p.sk_total = pl.sk_total;
        p.sk_unit = pl.sk_unit;
        const bool fuse_dbias = c.dbias && c.a_mn && c.b_mn && c.accumulate && ctx->fuse_dbias && pl.tiles_n * 16 <= kDbiasTickets;
        // scratch: [partial tiles of cut ranges][their column sums, 128 per CTA][the tiles' shares of the bias gradient, one row per tile row]
        const size_t cut_dbias_bytes = fuse_dbias && pl.sk_max_share > 1 ? size_t(pl.grid) * PairCfg<false>::kBRows * sizeof(float) : 0;
        const size_t part_bytes = fuse_dbias ? size_t((pl.tiles_m + 1) / 2) * pl.tiles_n * 256 * sizeof(float) : 0;
        if (fuse_dbias || pl.sk_max_share > 1) {
            const int rc = ensure_workspace(ctx, pl.workspace_bytes + cut_dbias_bytes + part_bytes);
            if (rc != GPTB200_OK) return rc;
        }
        if (fuse_dbias) {
            p.dbias = c.dbias;
            p.dbias_src = c.b;
            // TF32 mode is bound by the operand traffic from L2 to the SMs, which the column sums add to: spread them over all tile
            // rows.  3xTF32 has that bandwidth to spare and its epilogue warps drain an accumulator every four k-blocks: fewer,
            // longer batches of loads in the first tile row were measured faster there.
            p.dbias_rows = x3 ? 1 : (pl.tiles_m + 1) / 2;
            p.dbias_part = ctx->ws + (pl.workspace_bytes + cut_dbias_bytes) / sizeof(float);
            p.dbias_tickets = ctx->d_pair_flags + size_t(ctx->num_sms) * 8 + 2 + kSkinnyMaxTickets;
            if (dbias_fused) *dbias_fused = true;
        }
        // 3xTF32: split one operand into its bf16 correction tiles before the launch when many tiles re-read it (a weight matrix
        // is re-read by every row tile, an activation by every column tile): the operand with the larger re-use, provided it is
        // re-read at least three times; its expanded matrix (4 bytes per element) goes behind the other scratch regions.
        const long long tiles_m2 = (pl.tiles_m + 1) / 2;
        if (x3 && ctx->presplit) {
            const long long k8 = (static_cast<long long>(c.K) + 7) & ~7LL;
            const bool a_ok = !c.a_mn || c.M % 8 == 0, b_ok = !c.b_mn || c.N % 8 == 0;
            const long long reuse_a = a_ok ? pl.tiles_n : 0, reuse_b = b_ok ? tiles_m2 : 0;
            int pre = 0;
            if (std::max(reuse_a, reuse_b) >= 3) pre = reuse_b >= reuse_a ? 2 : 1;
            if (ctx->presplit == 2 && a_ok) pre = 1;   // forced choices, for tests
            if (ctx->presplit == 3 && b_ok) pre = 2;
            if (pre) {
                const long long rows = pre == 1 ? c.M : c.N;
                const size_t pre_bytes = size_t(rows) * size_t(k8) * 4;
                const size_t before = (pl.workspace_bytes + cut_dbias_bytes + part_bytes + 255) & ~size_t(255);
                if (before + pre_bytes <= ctx->ws_limit) {
                    const int rc = ensure_workspace(ctx, before + pre_bytes);
                    if (rc != GPTB200_OK) return rc;
                    pre_buf = reinterpret_cast<char *>(ctx->ws) + before;
                    p.pre_operand = pre;
                    if (fuse_dbias) p.dbias_part = ctx->ws + (pl.workspace_bytes + cut_dbias_bytes) / sizeof(float);   // the buffer may have moved
                }
            }
        }
        // 3xTF32 correction terms: as TF32 products of fp32 low-part tiles (error about 2^-22 per term, 12 instructions per k-block)
        // for launches too small to be bound by the tensor pipe or the power limit, where the extra instructions cost a few
        // percent; as one bf16 chain (2^-20, 8 instructions) for the large ones, where they cost 8 %.
        if (x3 && !p.pre_operand && (ctx->exact3x == 1 || (ctx->exact3x == 2 && 2.0 * c.M * c.N * c.K <= kExact3xFlops))) p.exact3x = 1;
        if (pl.sk_max_share > 1) {
            p.sk_slots = ctx->ws;
            p.sk_dbias = ctx->ws + pl.workspace_bytes / sizeof(float);
            p.sk_flags = ctx->d_pair_flags;
            p.sk_state = ctx->d_pair_flags + size_t(ctx->num_sms) * 8;   // two words behind the flags
        }
    }
    if (splits > 1) {
        const int rc = ensure_workspace(ctx, bytes_per_split * splits);
        if (rc != GPTB200_OK) return rc;
        out_base = ctx->ws;
        p.has_act = 0;
        p.bias = nullptr;
        p.epi_mode = EPI_PARTIAL;
    } else {
        p.has_act = c.act ? 1 : 0;
        p.bias = c.bias;
        p.epi_mode = c.accumulate ? EPI_ACCUM : EPI_STORE;
    }

    CUtensorMap ta, tb, to, tact;
    const int out_box_cols = pair ? PairCfg<false>::kStageCols : 32;
    int rc = make_out_tmap(ctx, &to, out_base, splits, c.M, c.N, out_box_cols);
    if (rc != GPTB200_OK) return rc;
    if (p.has_act) {
        rc = make_out_tmap(ctx, &tact, c.act, 1, c.M, c.N, out_box_cols);
        if (rc != GPTB200_OK) return rc;
    } else {
        tact = to;
    }
    if (c.a_mn)
        rc = make_tmap(ctx, &ta, c.a, c.K, c.M, 32, kBK, true);
    else
        rc = make_tmap(ctx, &ta, c.a, c.M, c.K, kBK, kBM, false);
    if (rc != GPTB200_OK) return rc;
    if (c.b_mn)
        rc = make_tmap(ctx, &tb, c.b, c.K, c.N, 32, kBK, true);
    else
        rc = make_tmap(ctx, &tb, c.b, c.N, c.K, kBK, pair ? bn / 2 : bn, false);
    if (rc != GPTB200_OK) return rc;

    CUtensorMap tpre = to;
    if (p.pre_operand) {
        const bool pre_a = p.pre_operand == 1;
        const bool mn = pre_a ? c.a_mn : c.b_mn;
        const float *src = pre_a ? c.a : c.b;
        const long long rows = pre_a ? c.M : c.N;          // free extent of that operand
        const long long k8 = (static_cast<long long>(c.K) + 7) & ~7LL;
        const long long units = mn ? k8 * (rows / 8) : rows * (k8 / 8);
        const int blocks = static_cast<int>(std::min<long long>((units + 255) / 256, 1LL * ctx->num_sms * 16));
        if (mn)
            split_operand_kernel<true><<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<uint4 *>(pre_buf), src, c.K, rows, pre_a ? 0 : 1);
        else
            split_operand_kernel<false><<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<uint4 *>(pre_buf), src, rows, c.K, pre_a ? 0 : 1);
        ctx->launches++;
        CUDA_TRY(ctx, cudaGetLastError());
        rc = mn ? make_pre_tmap(ctx, &tpre, pre_buf, 2 * k8, rows / 2, 64) : make_pre_tmap(ctx, &tpre, pre_buf, rows, k8, 128);
        if (rc != GPTB200_OK) return rc;
    }

    const int grid = pl.grid;
    cudaError_t e;
    if (pair)
        e = x3 ? launch_pair<true>(ctx, c.a_mn, c.b_mn, ta, tb, to, tact, tpre, p, grid) : launch_pair<false>(ctx, c.a_mn, c.b_mn, ta, tb, to, tact, tpre, p, grid);
    else if (bn == 256)
        e = x3 ? launch_majors<256, true>(ctx, c.a_mn, c.b_mn, ta, tb, to, tact, p, grid)
               : launch_majors<256, false>(ctx, c.a_mn, c.b_mn, ta, tb, to, tact, p, grid);
    else
        e = x3 ? launch_majors<128, true>(ctx, c.a_mn, c.b_mn, ta, tb, to, tact, p, grid)
               : launch_majors<128, false>(ctx, c.a_mn, c.b_mn, ta, tb, to, tact, p, grid);
    ctx->launches++;
    CUDA_TRY(ctx, e);

    if (splits > 1) {
        const long long n4 = (1LL * c.M * c.N) >> 2;
        const int blocks = static_cast<int>(std::min<long long>((n4 + 255) / 256, 1LL * ctx->num_sms * 8));
        splitk_reduce_kernel<<<blocks, 256, 0, ctx->stream>>>(c.out, ctx->ws, n4, splits, c.accumulate ? 1 : 0);
        ctx->launches++;
        CUDA_TRY(ctx, cudaGetLastError());
    }
    return GPTB200_OK;
}

int run_bias_grad(gptb200_ctx *ctx, float *gb, const float *gy, int M, int N)
{
    if (M == 0 || N == 0) return GPTB200_OK;
    const int col_groups = (N + 31) / 32;
    int chunks = std::max(1, std::min((ctx->num_sms * 6 + col_groups - 1) / col_groups, (M + 63) / 64));
    chunks = std::min(chunks, 65535);
    const int rows_per_chunk = (M + chunks - 1) / chunks;
    chunks = (M + rows_per_chunk - 1) / rows_per_chunk;
    const int rc = ensure_workspace(ctx, size_t(chunks) * N * sizeof(float));
    if (rc != GPTB200_OK) return rc;
    bias_grad_partial_kernel<<<dim3(col_groups, chunks), dim3(32, 8), 0, ctx->stream>>>(ctx->ws, gy, M, N, rows_per_chunk);
    ctx->launches++;
    CUDA_TRY(ctx, cudaGetLastError());
    bias_grad_final_kernel<<<(N + 127) / 128, 128, 0, ctx->stream>>>(gb, ctx->ws, N, chunks);
    ctx->launches++;
    CUDA_TRY(ctx, cudaGetLastError());
    return GPTB200_OK;
}

// `batches` GEMMs of one shape in one launch of the CTA-pair kernel (whole tiles per pair, store epilogue).
int run_gemm_batched_impl(gptb200_ctx *ctx, float *out, long long out_ld, long long out_si, long long out_so, const BatchedOperand &a,
                          const BatchedOperand &b, int M, int N, int K, int inner, int outer, bool causal)
{
    if (M <= 0 || N <= 0 || K <= 0 || inner <= 0 || outer <= 0) return fail(ctx, GPTB200_ERR_INVALID_ARG, "batched GEMM with an empty dimension");
    if (a.mn && !b.mn) return fail(ctx, GPTB200_ERR_INVALID_ARG, "operand forms (MN-major, K-major) do not occur");
    const bool x3 = ctx->mode == GPTB200_MODE_3XTF32;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K;
    p.tiles_m = (M + kBM - 1) / kBM;
    p.tiles_n = (N + 255) / 256;
    p.num_kb = (K + kBK - 1) / kBK;
    p.kb_per_split = p.num_kb;
    p.splits = 1;
    p.status = ctx->d_status;
    p.epi_mode = EPI_STORE;
    p.batches = inner * outer;
    p.batch_inner = inner;
    if (N <= 128) p.mma_n = (N + 31) / 32 * 32;
    p.exact3x = (x3 && ctx->batched_exact3x) ? 1 : 0;
    p.causal_skip = (causal && M == N) ? 1 : 0;
    if (ctx->d_trace) {   // option "trace": the first CTA pair records its pipeline events
        CUDA_TRY(ctx, cudaMemsetAsync(ctx->d_trace, 0, sizeof(long long) * kTraceEvents * kTraceSlots, ctx->stream));
        p.trace = ctx->d_trace;
    }
    p.chunk_kb = ctx->batched_chunk_kb;
    const long long tiles = 1LL * ((p.tiles_m + 1) / 2) * p.tiles_n * p.batches;
    p.sk_total = tiles * p.num_kb;
    p.sk_unit = p.num_kb;                                   // whole tiles per pair
    const int sms = ctx->max_sms > 0 ? std::min(ctx->max_sms, ctx->num_sms) : ctx->num_sms;   // option "max_sms" bounds these launches too
    const int pairs = static_cast<int>(std::min<long long>(std::max(1, sms / 2), tiles));
    CUtensorMap ta, tb, to;
    int rc = a.mn ? make_batched_tmap(ctx, &ta, a.base, M, K, inner, outer, a.ld, a.stride_inner, a.stride_outer, 32, kBK, 1)
                  : make_batched_tmap(ctx, &ta, a.base, K, M, inner, outer, a.ld, a.stride_inner, a.stride_outer, kBK, kBM, 0);
    if (rc) return rc;
    rc = b.mn ? make_batched_tmap(ctx, &tb, b.base, N, K, inner, outer, b.ld, b.stride_inner, b.stride_outer, 32, kBK, 1)
              : make_batched_tmap(ctx, &tb, b.base, K, N, inner, outer, b.ld, b.stride_inner, b.stride_outer, kBK, N <= 128 ? (N + 31) / 32 * 16 : 128, 0);
    if (rc) return rc;
    rc = make_batched_tmap(ctx, &to, out, N, M, inner, outer, out_ld, out_si, out_so, PairCfg<false>::kStageCols, 32, 0);
    if (rc) return rc;
    const cudaError_t e = x3 ? launch_pair<true>(ctx, a.mn, b.mn, ta, tb, to, to, to, p, 2 * pairs) : launch_pair<false>(ctx, a.mn, b.mn, ta, tb, to, to, to, p, 2 * pairs);
    ctx->launches++;
    CUDA_TRY(ctx, e);
    return GPTB200_OK;
}

int check_dims(gptb200_ctx *ctx, int m, int a, int b)
{
    if (!ctx) return GPTB200_ERR_INVALID_ARG;
    if (m < 0 || a < 0 || b < 0) return fail(ctx, GPTB200_ERR_INVALID_ARG, "negative dimension (%d, %d, %d)", m, a, b);
    // The reference indexes with int (src/backend/common/tensor_utils.h:3-5); keep its m*n < 2^31 limit explicit.
    if (1LL * m * a > 0x7fffffffLL || 1LL * m * b > 0x7fffffffLL || 1LL * a * b > 0x7fffffffLL)
        return fail(ctx, GPTB200_ERR_INVALID_ARG, "tensor with more than 2^31-1 elements (%d, %d, %d)", m, a, b);
    return GPTB200_OK;
}

}  // namespace

namespace gptb200 {
int run_gemm_batched(gptb200_ctx *ctx, float *out, long long out_ld, long long out_si, long long out_so, const BatchedOperand &a, const BatchedOperand &b,
                     int M, int N, int K, int inner, int outer, bool causal)
{
    return run_gemm_batched_impl(ctx, out, out_ld, out_si, out_so, a, b, M, N, K, inner, outer, causal);
}
}  // namespace gptb200

extern "C" {

const char *gptb200_status_string(int status)
{
    switch (status) {
        case GPTB200_OK: return "ok";
        case GPTB200_ERR_INVALID_ARG: return "invalid argument";
        case GPTB200_ERR_CUDA: return "CUDA call failed";
        case GPTB200_ERR_NO_DEVICE: return "no sm_100 device";
        case GPTB200_ERR_DEVICE_TIMEOUT: return "bounded wait inside a kernel ran out";
        case GPTB200_ERR_WORKSPACE: return "scratch request beyond limit";
        case GPTB200_ERR_TOO_LARGE: return "size beyond the entry point's maximum";
        default: return "unknown status";
    }
}

const char *gptb200_last_error(const gptb200_ctx *ctx) { return ctx ? ctx->last_error : "null context"; }

int gptb200_ctx_create(gptb200_ctx **out, int device, void *cuda_stream, int mode)
{
    if (!out) return GPTB200_ERR_INVALID_ARG;
    *out = nullptr;
    if (mode != GPTB200_MODE_3XTF32 && mode != GPTB200_MODE_TF32) return GPTB200_ERR_INVALID_ARG;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return GPTB200_ERR_NO_DEVICE;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return GPTB200_ERR_CUDA;
    if (prop.major != 10) return GPTB200_ERR_NO_DEVICE;
    if (cudaSetDevice(device) != cudaSuccess) return GPTB200_ERR_CUDA;

    gptb200_ctx *ctx = new gptb200_ctx();
    ctx->device = device;
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    ctx->mode = mode;
    ctx->num_sms = prop.multiProcessorCount;

    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
        qres != cudaDriverEntryPointSuccess) {
        delete ctx;
        return GPTB200_ERR_CUDA;
    }
    ctx->encode = reinterpret_cast<EncodeTiledFn>(fn);
    // [pair][CTA][epilogue warp] + launch number, CTA count; then one ticket per column block of the decode kernel; then the
    // tickets of the bias gradient inside the grad_w GEMM (per tile column, CTA and epilogue warp)
    const size_t flag_bytes = (size_t(ctx->num_sms) * 8 + 2 + kSkinnyMaxTickets + kDbiasTickets) * sizeof(unsigned int);
    if (cudaMalloc(&ctx->d_status, sizeof(int)) != cudaSuccess || cudaMemset(ctx->d_status, 0, sizeof(int)) != cudaSuccess ||
        cudaMalloc(&ctx->d_pair_flags, flag_bytes) != cudaSuccess || cudaMemset(ctx->d_pair_flags, 0, flag_bytes) != cudaSuccess) {
        if (ctx->d_status) cudaFree(ctx->d_status);
        delete ctx;
        return GPTB200_ERR_CUDA;
    }
    *out = ctx;
    return GPTB200_OK;
}

int gptb200_ctx_destroy(gptb200_ctx *ctx)
{
    if (!ctx) return GPTB200_ERR_INVALID_ARG;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->attn_ws) cudaFree(ctx->attn_ws);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->d_pair_flags) cudaFree(ctx->d_pair_flags);
    if (ctx->d_trace) cudaFree(ctx->d_trace);
    delete ctx;
    return GPTB200_OK;
}

int gptb200_ctx_set_mode(gptb200_ctx *ctx, int mode)
{
    if (!ctx || (mode != GPTB200_MODE_3XTF32 && mode != GPTB200_MODE_TF32)) return GPTB200_ERR_INVALID_ARG;
    ctx->mode = mode;
    return GPTB200_OK;
}

int gptb200_ctx_get_mode(const gptb200_ctx *ctx) { return ctx ? ctx->mode : -1; }

int gptb200_ctx_set_stream(gptb200_ctx *ctx, void *cuda_stream)
{
    if (!ctx) return GPTB200_ERR_INVALID_ARG;
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    return GPTB200_OK;
}

int gptb200_ctx_set_option(gptb200_ctx *ctx, const char *key, int value)
{
    if (!ctx || !key) return GPTB200_ERR_INVALID_ARG;
    if (!strcmp(key, "tile_n")) {
        if (value != 0 && value != 128 && value != 256) return fail(ctx, GPTB200_ERR_INVALID_ARG, "tile_n must be 0, 128 or 256");
        ctx->tile_n = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "pair")) {
        if (value < -1 || value > 1) return fail(ctx, GPTB200_ERR_INVALID_ARG, "pair must be -1, 0 or 1");
        ctx->pair = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "max_sms")) {
        if (value < 0) return fail(ctx, GPTB200_ERR_INVALID_ARG, "max_sms must be >= 0");
        ctx->max_sms = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "exact3x")) {
        if (value < 0 || value > 2) return fail(ctx, GPTB200_ERR_INVALID_ARG, "exact3x: 0 never, 1 always, 2 automatic");
        ctx->exact3x = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "batched_chunk_kb")) {
        if (value < 0 || value > 4) return fail(ctx, GPTB200_ERR_INVALID_ARG, "batched_chunk_kb: 0 (default) to 4");
        ctx->batched_chunk_kb = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "batched_exact3x")) {
        ctx->batched_exact3x = value != 0;
        return GPTB200_OK;
    }
    if (!strcmp(key, "attention_group_mb")) {
        if (value < 1) return fail(ctx, GPTB200_ERR_INVALID_ARG, "attention_group_mb must be positive");
        ctx->attention_group_mb = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "attention_gemm")) {
        ctx->attention_gemm = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "softmax_stream")) {
        ctx->softmax_stream = value != 0;
        return GPTB200_OK;
    }
    if (!strcmp(key, "attention_tiled")) {
        ctx->attention_tiled = value != 0;
        return GPTB200_OK;
    }
    if (!strcmp(key, "trace")) {
        if (value && !ctx->d_trace) CUDA_TRY(ctx, cudaMalloc(&ctx->d_trace, sizeof(long long) * kTraceEvents * kTraceSlots));
        if (!value && ctx->d_trace) {
            CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            cudaFree(ctx->d_trace);
            ctx->d_trace = nullptr;
        }
        return GPTB200_OK;
    }
    if (!strcmp(key, "stream_k")) {
        if (value < -1 || value > 1) return fail(ctx, GPTB200_ERR_INVALID_ARG, "stream_k must be -1, 0 or 1");
        ctx->stream_k = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny")) {
        ctx->skinny = value != 0;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny_rows")) {
        if (value < 0 || value > kPlanSkinnyMaxRows) return fail(ctx, GPTB200_ERR_INVALID_ARG, "skinny_rows must be in [0, %d]", kPlanSkinnyMaxRows);
        ctx->skinny_rows = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny_push")) {
        ctx->skinny_push = value != 0;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny_tile_rows")) {
        if (value != 0 && value != 32 && value != 64) return fail(ctx, GPTB200_ERR_INVALID_ARG, "skinny_tile_rows must be 0, 32 or 64");
        ctx->skinny_tile_rows = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny_tile")) {
        ctx->skinny_tile = value != 0;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny_pipelined")) {
        ctx->skinny_pipelined = value != 0;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny_rowwise_rows")) {
        if (value < 0 || value > kPlanSkinnyMaxRows) return fail(ctx, GPTB200_ERR_INVALID_ARG, "skinny_rowwise_rows must be in [0, %d]", kPlanSkinnyMaxRows);
        ctx->skinny_rowwise_rows = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny_rowwise")) {
        ctx->skinny_rowwise = value != 0;
        return GPTB200_OK;
    }
    if (!strcmp(key, "decode_early_launch")) {
        if (value < 0 || value > 2) return fail(ctx, GPTB200_ERR_INVALID_ARG, "decode_early_launch must be 0, 1 or 2");
        ctx->decode_early_launch = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny_cluster_rows")) {
        if (value < 0 || value > kPlanSkinnyMaxRows) return fail(ctx, GPTB200_ERR_INVALID_ARG, "skinny_cluster_rows must be in [0, %d]", kPlanSkinnyMaxRows);
        ctx->skinny_cluster_rows = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny_cluster")) {
        if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8 && value != 16 && value != 32)
            return fail(ctx, GPTB200_ERR_INVALID_ARG, "skinny_cluster must be 0, 1, 2, 4, 8, 16 or 32");
        ctx->skinny_cluster = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "skinny_fused")) {
        if (value < -1 || value > 1) return fail(ctx, GPTB200_ERR_INVALID_ARG, "skinny_fused must be -1, 0 or 1");
        ctx->skinny_fused = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "presplit")) {
        if (value < 0 || value > 3) return fail(ctx, GPTB200_ERR_INVALID_ARG, "presplit must be 0, 1, 2 or 3");
        ctx->presplit = value;
        return GPTB200_OK;
    }
    if (!strcmp(key, "fuse_dbias")) {
        ctx->fuse_dbias = value != 0;
        return GPTB200_OK;
    }
    if (!strcmp(key, "max_splits")) {
        if (value < 0 || value > 64) return fail(ctx, GPTB200_ERR_INVALID_ARG, "max_splits must be in [0, 64]");
        ctx->max_splits = value;
        return GPTB200_OK;
    }
    return fail(ctx, GPTB200_ERR_INVALID_ARG, "unknown option '%s'", key);
}

int gptb200_ctx_read_trace(gptb200_ctx *ctx, long long *samples, int capacity)
{
    if (!ctx || !samples || capacity < 0) return GPTB200_ERR_INVALID_ARG;
    if (!ctx->d_trace) return fail(ctx, GPTB200_ERR_INVALID_ARG, "tracing is off (option \"trace\")");
    const int n = std::min(capacity, int(kTraceEvents) * kTraceSlots);
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    CUDA_TRY(ctx, cudaMemcpy(samples, ctx->d_trace, sizeof(long long) * n, cudaMemcpyDeviceToHost));
    return GPTB200_OK;
}

int gptb200_ctx_synchronize(gptb200_ctx *ctx)
{
    if (!ctx) return GPTB200_ERR_INVALID_ARG;
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    int st = 0;
    CUDA_TRY(ctx, cudaMemcpy(&st, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) {
        cudaMemset(ctx->d_status, 0, sizeof(int));
        // a kernel that gave up may have left tickets half counted: they must be zero between launches
        cudaMemset(ctx->d_pair_flags + size_t(ctx->num_sms) * 8 + 2, 0, (kSkinnyMaxTickets + kDbiasTickets) * sizeof(unsigned int));
        return fail(ctx, GPTB200_ERR_DEVICE_TIMEOUT, "device status %d: a bounded wait inside a kernel ran out", st);
    }
    return GPTB200_OK;
}

long long gptb200_ctx_launch_count(const gptb200_ctx *ctx) { return ctx ? ctx->launches : -1; }

long long gptb200_ctx_tensor_map_encodes(const gptb200_ctx *ctx) { return ctx ? ctx->tmap_encodes : -1; }

int gptb200_selftest_wait_timeout(gptb200_ctx *ctx, int limit_us)
{
    if (!ctx || limit_us <= 0 || limit_us > 100000) return GPTB200_ERR_INVALID_ARG;
    int khz = 0;
    CUDA_TRY(ctx, cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device));
    const long long cycles = static_cast<long long>(limit_us) * std::max(khz, 1000) / 1000;
    wait_timeout_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, cycles);
    ctx->launches++;
    CUDA_TRY(ctx, cudaGetLastError());
    return GPTB200_OK;
}

int gptb200_plan_gemm(int num_sms, int m, int n, int k, int a_mn_major, int b_mn_major, int has_epilogue, int accumulate, int *plan8)
{
    if (!plan8 || num_sms <= 0 || m < 0 || n < 0 || k < 0) return GPTB200_ERR_INVALID_ARG;
    GemmPlanInput in{};
    in.M = m; in.N = n; in.K = k;
    in.a_mn = a_mn_major != 0; in.b_mn = b_mn_major != 0;
    in.has_epilogue = has_epilogue != 0; in.accumulate = accumulate != 0; in.aligned = true;
    in.num_sms = num_sms; in.opt_skinny = true; in.ws_limit = size_t(1) << 30;
    const GemmPlan p = plan_gemm(in);
    const long long ws = static_cast<long long>(p.workspace_bytes);
    const int pairs = p.kernel == KERNEL_PAIR ? p.grid / 2 : 1;
    const int kb_each = p.kernel == KERNEL_PAIR ? static_cast<int>((p.sk_total + pairs - 1) / pairs) : p.kb_per_split;
    const int out[8] = {p.kernel, p.tile_n, p.tiles_m, p.tiles_n, p.kernel == KERNEL_PAIR ? p.sk_max_share : p.splits, kb_each, p.grid, static_cast<int>(std::min<long long>(ws >> 10, 0x7fffffff))};
    for (int i = 0; i < 8; ++i) plan8[i] = out[i];
    return GPTB200_OK;
}

int gptb200_plan_decode(int num_sms, int m, int n, int k, int w_kn_major, int has_epilogue, int *plan4)
{
    if (!plan4 || num_sms <= 0 || m <= 0 || n <= 0 || k <= 0) return GPTB200_ERR_INVALID_ARG;
    const DecodePlan d = plan_decode(m, n, k, w_kn_major != 0, has_epilogue != 0, num_sms, DecodeOptions{});
    plan4[0] = d.kernel; plan4[1] = d.rows; plan4[2] = d.groups; plan4[3] = d.cluster;
    return GPTB200_OK;
}

int gptb200_linear_forward(gptb200_ctx *ctx, float *y, float *act, const float *x, const float *w, const float *b, int activation,
                           int m, int k, int n)
{
    int rc = check_dims(ctx, m, k, n);
    if (rc) return rc;
    if (m == 0 || n == 0) return GPTB200_OK;
    // a tensor without elements (k == 0) may come as a null pointer
    if (!y || !b || (activation && !act) || (k > 0 && (!x || !w))) return fail(ctx, GPTB200_ERR_INVALID_ARG, "null tensor pointer");
    GemmCall c{m, n, k, x, false, w, true, y, activation ? act : nullptr, b, false};
    return run_gemm(ctx, c);
}

int gptb200_linear_backward_input(gptb200_ctx *ctx, float *grad_x, const float *grad_y, const float *w, int m, int k, int n)
{
    int rc = check_dims(ctx, m, k, n);
    if (rc) return rc;
    if (1LL * m * k == 0) return GPTB200_OK;
    if (!grad_x || (n > 0 && (!grad_y || !w))) return fail(ctx, GPTB200_ERR_INVALID_ARG, "null tensor pointer");
    if (n == 0) {
        CUDA_TRY(ctx, cudaMemsetAsync(grad_x, 0, size_t(m) * k * sizeof(float), ctx->stream));
        return GPTB200_OK;
    }
    // grad_x[m x k] = grad_y[m x n] . w^T : A = grad_y (K-major), B = w stored [k x n] = [N' x K'] (K-major)
    GemmCall dx{m, k, n, grad_y, false, w, false, grad_x, nullptr, nullptr, false};
    return run_gemm(ctx, dx);
}

int gptb200_linear_backward_input_gelu(gptb200_ctx *ctx, float *grad_x, const float *grad_y, const float *w, const float *pre_act, int m, int k, int n)
{
    int rc = check_dims(ctx, m, k, n);
    if (rc) return rc;
    if (1LL * m * k == 0) return GPTB200_OK;
    if (!grad_x || !pre_act || (n > 0 && (!grad_y || !w))) return fail(ctx, GPTB200_ERR_INVALID_ARG, "null tensor pointer");
    if (n == 0) {
        CUDA_TRY(ctx, cudaMemsetAsync(grad_x, 0, size_t(m) * k * sizeof(float), ctx->stream));
        return GPTB200_OK;
    }
    GemmCall dx{m, k, n, grad_y, false, w, false, grad_x, nullptr, nullptr, false, nullptr, pre_act};
    bool fused = false;
    rc = run_gemm(ctx, dx, nullptr, &fused);
    if (rc || fused) return rc;
    // shapes that do not run the CTA-pair kernel: the derivative as a pass of its own, in place
    return gptb200_gelu_backward(ctx, grad_x, grad_x, pre_act, m, k);
}

int gptb200_linear_backward_weights(gptb200_ctx *ctx, float *grad_w, float *grad_b, const float *grad_y, const float *x, int m, int k, int n)
{
    int rc = check_dims(ctx, m, k, n);
    if (rc) return rc;
    if ((1LL * k * n > 0 && !grad_w) || (n > 0 && !grad_b) || (1LL * m * n > 0 && !grad_y) || (1LL * m * k > 0 && !x))
        return fail(ctx, GPTB200_ERR_INVALID_ARG, "null tensor pointer");
    // grad_w[k x n] += x^T . grad_y : A = x stored [m x k] = [K' x M'] (MN-major), B = grad_y [m x n] = [K' x N'] (MN-major)
    bool dbias_fused = false;
    if (m > 0 && k > 0 && n > 0) {
        GemmCall dw{k, n, m, x, true, grad_y, true, grad_w, nullptr, nullptr, true, grad_b};
        rc = run_gemm(ctx, dw, &dbias_fused);
        if (rc) return rc;
    }
    // shapes that do not run the CTA-pair kernel: the two-stage column-sum kernels
    return dbias_fused ? GPTB200_OK : run_bias_grad(ctx, grad_b, grad_y, m, n);
}

int gptb200_linear_backward(gptb200_ctx *ctx, float *grad_x, float *grad_w, float *grad_b, const float *grad_y, const float *x,
                            const float *w, int m, int k, int n)
{
    int rc = check_dims(ctx, m, k, n);
    if (rc) return rc;
    if ((1LL * m * k > 0 && (!grad_x || !x)) || (1LL * k * n > 0 && (!grad_w || !w)) || (n > 0 && !grad_b) || (1LL * m * n > 0 && !grad_y))
        return fail(ctx, GPTB200_ERR_INVALID_ARG, "null tensor pointer");
    rc = gptb200_linear_backward_input(ctx, grad_x, grad_y, w, m, k, n);
    if (rc) return rc;
    return gptb200_linear_backward_weights(ctx, grad_w, grad_b, grad_y, x, m, k, n);
}

int gptb200_gemm_batched(gptb200_ctx *ctx, float *out, const float *a, const float *b, int m, int n, int k, int a_mn_major, int b_mn_major, int batch_inner,
                         int batch_outer, const long long *a_strides3, const long long *b_strides3, const long long *out_strides3)
{
    if (!ctx) return GPTB200_ERR_INVALID_ARG;
    if (!out || !a || !b || !a_strides3 || !b_strides3 || !out_strides3) return fail(ctx, GPTB200_ERR_INVALID_ARG, "null pointer");
    const BatchedOperand oa{a, a_mn_major != 0, a_strides3[0], a_strides3[1], a_strides3[2]};
    const BatchedOperand ob{b, b_mn_major != 0, b_strides3[0], b_strides3[1], b_strides3[2]};
    return run_gemm_batched_impl(ctx, out, out_strides3[0], out_strides3[1], out_strides3[2], oa, ob, m, n, k, batch_inner, batch_outer, false);
}

int gptb200_gelu_backward(gptb200_ctx *ctx, float *grad_x, const float *grad_y, const float *x, int m, int n)
{
    int rc = check_dims(ctx, m, n, 1);
    if (rc) return rc;
    const long long total = 1LL * m * n;
    if (total == 0) return GPTB200_OK;
    if (!grad_x || !grad_y || !x) return fail(ctx, GPTB200_ERR_INVALID_ARG, "null tensor pointer");
    const int blocks = static_cast<int>(std::min<long long>((total / 4 + 255) / 256 + 1, 1LL * ctx->num_sms * 16));
    gelu_backward_kernel<<<blocks, 256, 0, ctx->stream>>>(grad_x, grad_y, x, total);
    ctx->launches++;
    CUDA_TRY(ctx, cudaGetLastError());
    return GPTB200_OK;
}

int gptb200_unembed_forward(gptb200_ctx *ctx, float *y, const float *x, const float *wte, int m, int d, int vp)
{
    int rc = check_dims(ctx, m, d, vp);
    if (rc) return rc;
    if (m == 0 || vp == 0) return GPTB200_OK;
    if (!y || (d > 0 && (!x || !wte))) return fail(ctx, GPTB200_ERR_INVALID_ARG, "null tensor pointer");
    if (d == 0) {
        CUDA_TRY(ctx, cudaMemsetAsync(y, 0, size_t(m) * vp * sizeof(float), ctx->stream));
        return GPTB200_OK;
    }
    // y[m x vp] = x[m x d] . wte^T : A = x (K-major), B = wte stored [vp x d] = [N' x K'] (K-major)
    GemmCall c{m, vp, d, x, false, wte, false, y, nullptr, nullptr, false};
    return run_gemm(ctx, c);
}

int gptb200_unembed_backward(gptb200_ctx *ctx, float *grad_x, float *grad_wte, const float *grad_y, const float *x, const float *wte,
                             int m, int d, int vp)
{
    int rc = check_dims(ctx, m, d, vp);
    if (rc) return rc;
    if (m == 0 || d == 0) return GPTB200_OK;
    if (!grad_x || !x || (vp > 0 && (!grad_wte || !grad_y || !wte))) return fail(ctx, GPTB200_ERR_INVALID_ARG, "null tensor pointer");
    if (vp == 0) {
        CUDA_TRY(ctx, cudaMemsetAsync(grad_x, 0, size_t(m) * d * sizeof(float), ctx->stream));
        return GPTB200_OK;
    }
    // grad_x[m x d] = grad_y[m x vp] . wte : A = grad_y (K-major), B = wte stored [vp x d] = [K' x N'] (MN-major)
    GemmCall dx{m, d, vp, grad_y, false, wte, true, grad_x, nullptr, nullptr, false};
    rc = run_gemm(ctx, dx);
    if (rc) return rc;
    // grad_wte[vp x d] += grad_y^T . x : A = grad_y stored [m x vp] = [K' x M'] (MN-major), B = x [m x d] = [K' x N'] (MN-major)
    GemmCall dw{vp, d, m, grad_y, true, x, true, grad_wte, nullptr, nullptr, true};
    return run_gemm(ctx, dw);
}

int gptb200_malloc(gptb200_ctx *ctx, void **ptr, size_t bytes)
{
    if (!ctx || !ptr) return GPTB200_ERR_INVALID_ARG;
    CUDA_TRY(ctx, cudaMalloc(ptr, bytes));
    return GPTB200_OK;
}

int gptb200_free(gptb200_ctx *ctx, void *ptr)
{
    if (!ctx) return GPTB200_ERR_INVALID_ARG;
    CUDA_TRY(ctx, cudaFree(ptr));
    return GPTB200_OK;
}

int gptb200_memset(gptb200_ctx *ctx, void *ptr, int value, size_t bytes)
{
    if (!ctx) return GPTB200_ERR_INVALID_ARG;
    CUDA_TRY(ctx, cudaMemsetAsync(ptr, value, bytes, ctx->stream));
    return GPTB200_OK;
}

int gptb200_memcpy_h2d(gptb200_ctx *ctx, void *dst, const void *src, size_t bytes)
{
    if (!ctx) return GPTB200_ERR_INVALID_ARG;
    CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return GPTB200_OK;
}

int gptb200_memcpy_d2h(gptb200_ctx *ctx, void *dst, const void *src, size_t bytes)
{
    if (!ctx) return GPTB200_ERR_INVALID_ARG;
    CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return GPTB200_OK;
}

}  // extern "C"
