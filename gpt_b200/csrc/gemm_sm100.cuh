// Persistent, warp-specialised tcgen05 GEMM for sm_100a:  D[M x N] = A[M x K] * B[K x N], fp32 in HBM,
// TF32 tensor-core math with fp32 accumulation in TMEM.
//
// One kernel covers the six GEMM forms of the linear layers.  Each operand is described by the way it
// is *stored* (row-major, last dimension contiguous):
//   K-major  operand: the reduction index is the contiguous one   (x in y = x.w, grad_y in grad_x = grad_y.w^T, wte in logits = x.wte^T)
//   MN-major operand: the free (M or N) index is the contiguous one (w in y = x.w, both operands of grad_w += x^T.grad_y)
// so no operand is ever transposed in memory: the UMMA shared-memory descriptors express the major-ness.
//
// Roles per CTA (one CTA per SM, static round-robin over work items; warpgroup = 4 warps):
//   warp 0        TMA producer: fills a STAGES-deep ring of 128-byte-swizzled operand tiles
//   warp 1        MMA issuer (one thread): tcgen05.mma kind::tf32 into a double-buffered TMEM accumulator
//   warps 2-3     idle (keep the role groups warpgroup-aligned)
//   warps 4..     epilogue (4 or 8 warps): tcgen05.ld, bias / GELU, swizzled staging tile, TMA store
//                 (or TMA reduce-add for `out +=`); overlaps the next tile's main loop
//   last 4 warps  (3xTF32 only) split each landed tile into its low-order part  lo = a - trunc_tf32(a)
//
// 3xTF32: the tensor core reads only the top 19 bits of an fp32 word, so the raw tile *is* the high
// part; the converter warps write the low parts at the same (swizzled) offsets in a second buffer and the
// MMA thread issues  lo.hi + hi.lo + hi.hi  per k-step.
//
// Accumulator precision: every tcgen05.mma adds into the fp32 accumulator with truncation, which biases
// long sums (measured: relative error grows by about 2^-24 per MMA).  In 3xTF32 mode the MMA thread
// therefore hands the accumulator to the epilogue warps every kChunkKB k-blocks; they add the chunk into
// a running sum kept in registers with round-to-nearest fp32 adds, so the truncation never sees more than
// one chunk.  In plain TF32 mode the operand truncation (2^-11) dominates and a tile is one chunk.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "ptx_sm100.cuh"

namespace gptb200 {

// Device status codes written (first writer wins) to the context's status word.
enum DeviceStatus : int {
    DEV_OK = 0,
    DEV_TIMEOUT_PRODUCER = 101,   // producer gave up waiting for a free stage
    DEV_TIMEOUT_MMA_FULL = 102,   // MMA thread gave up waiting for a landed stage
    DEV_TIMEOUT_MMA_CONV = 103,   // MMA thread gave up waiting for the low-part tiles
    DEV_TIMEOUT_MMA_TMEM = 104,   // MMA thread gave up waiting for a drained accumulator
    DEV_TIMEOUT_EPILOGUE = 105,   // epilogue gave up waiting for a finished accumulator
    DEV_TIMEOUT_CONVERT = 106,    // converter gave up waiting for a landed stage
    DEV_TIMEOUT_DRAIN = 107,      // teardown gave up waiting for outstanding MMAs
    DEV_TIMEOUT_PARTIAL = 109,    // epilogue gave up waiting for another CTA pair's partial tile
    DEV_TIMEOUT_SELFTEST = 108,   // the self-test's wait on a barrier that nothing signals ran out, as intended
};

enum EpilogueMode : int {
    EPI_STORE = 0,    // out = acc (+ bias); optionally act = gelu_tanh(out)
    EPI_ACCUM = 1,    // out += acc
    EPI_PARTIAL = 2,  // workspace[split] = acc   (reduced by splitk_reduce_kernel)
};

struct GemmParams {
    int M, N, K;         // D[M x N] = A[M x K] . B[K x N]
    const float *bias;   // optional [N]
    int has_act;         // second output (GELU of out) through tmap_act
    int tiles_m, tiles_n;
    int splits;          // split-K factor (1 = none)
    int kb_per_split;    // k-blocks (of 32) per split
    int num_kb;          // ceil(K / 32)
    int epi_mode;
    int *status;         // device status word
    // CTA-pair kernel only: the tiles' k-blocks form one line of sk_total = tiles * num_kb entries that is cut into
    // one range per pair, at multiples of sk_unit (1: anywhere, num_kb: whole tiles only).
    long long sk_total;
    int sk_unit;
    float *sk_slots;         // one partial 256 x 256 tile per pair
    unsigned int *sk_flags;  // one word per pair, CTA and epilogue warp: the number of the launch whose partial tile is complete
    unsigned int *sk_state;  // [0] number of completed launches that used the flags, [1] CTAs of this launch that have finished
    long long *trace;        // optional [kTraceEvents][kTraceSlots] clock64 samples of the first k-blocks of CTA 0
    // CTA-pair kernel, batched form (batches > 0): `batches` independent GEMMs of the same shape in one launch, whole tiles per
    // pair.  The three tensor maps are then 4-D -- (innermost, inner batch index, row, outer batch index), the order of growing
    // strides for a head slice of packed rows -- so that an operand may be a strided slice of a larger tensor (one head of the
    // packed qkv rows); batch z = outer * batch_inner + inner.
    // Store epilogue only.
    int batches, batch_inner;
    // batched form with n <= 128: width of the tensor-core instruction (a multiple of 32); each CTA of a pair then supplies mma_n / 2
    // columns of B and only the first mma_n accumulator columns are written.  0 = the full 256.
    int mma_n;
    // 3xTF32, batched form: the correction terms a_lo.b + a.b_lo run as TF32 products of fp32 low-part tiles (relative error about
    // 2^-22 per term) instead of one bf16 chain (2^-20): 12 instead of 8 instructions per k-block.
    int exact3x;
    // Batched form, square products whose consumer only reads columns <= row (causal attention scores): 32-column pieces that lie
    // wholly beyond the diagonal for the 32 rows of an epilogue warp are not written.
    int causal_skip;
    // 3xTF32, batched form: k-blocks per accumulator hand-off (0 = kChunkKB); shorter chunks leave less to the accumulator's truncating adds
    int chunk_kb;
    // CTA-pair kernel, store epilogue: out = acc * gelu_tanh'(gelu_src) element by element (gelu_src [M x N], row pitch N): the
    // GELU derivative of the FFN rides the grad_x GEMM of the layer behind it instead of a pass of its own over HBM.
    const float *gelu_src;
    // CTA-pair kernel, 3xTF32: the bf16 correction tiles of ONE operand (1 = A, 2 = B, 0 = neither) were written to scratch by a
    // pass of their own before the launch (split_operand_kernel) and are fetched by TMA (fifth tensor map) straight into the
    // correction ring; the converter warps then only split the other operand.  Pays when that operand is re-read by many
    // tiles (a weight matrix by every row tile): half of the conversion work leaves the main loop.
    int pre_operand;
    // CTA-pair kernel, grad_w form (both operands MN-major) only: the bias gradient rides this launch.  The tiles of one tile
    // column read the same columns of B (= grad_y [K x N], row pitch N); each of them adds up its share of the k-blocks (epilogue
    // warps, plain loads), the shares are parked in dbias_part and the last tile to finish adds them, in tile order, into dbias[N].
    float *dbias;
    const float *dbias_src;
    float *sk_dbias;         // [pair][CTA][128] column sums of tiles cut by a range boundary (published with the partial tile)
    int dbias_rows;          // tile rows that share the column sums (1: the first tile row does them all)
    float *dbias_part;       // [tile row][tiles_n * 256] the tiles' shares
    unsigned int *dbias_tickets;   // [tile column][CTA][epilogue warp] shares parked so far (reset by the last one)
};

constexpr int kTraceSlots = 128;
enum TraceEvent : int {
    TRACE_LOAD_ISSUE = 0,   // producer: stage free, loads about to be issued
    TRACE_CONV_BEGIN = 1,   // converter (first warp of the group): raw tile landed, low-part buffer free
    TRACE_CONV_END = 2,     // converter: tiles written and published
    TRACE_MMA_FULL = 3,     // MMA thread: raw tile landed
    TRACE_MMA_READY = 4,    // MMA thread: converted tiles of both CTAs ready
    TRACE_MMA_ISSUED = 5,   // MMA thread: MMAs and commits issued
    TRACE_EPI_BEGIN = 6,    // epilogue warp 0 (3xTF32): a tile's sums are complete, output begins (slot = tile number)
    TRACE_EPI_END = 7,      // epilogue warp 0: the tile's output stores are issued
    TRACE_PEER_LOAD_ISSUE = 8,   // the same three events in the second CTA of the pair
    TRACE_PEER_CONV_BEGIN = 9,
    TRACE_PEER_CONV_END = 10,
    kTraceEvents = 11,
};

constexpr int kBM = 128;
constexpr int kBK = 32;                       // 32 fp32 = one 128-byte swizzle row
constexpr int kUmmaK = 8;                     // K per tcgen05.mma kind::tf32
constexpr int kATileBytes = kBM * kBK * 4;    // 16 KiB
constexpr int kBoxBytesMN = kBK * 32 * 4;     // one [32 k-rows x 32 floats] box of an MN-major operand
constexpr int kChunkKB = 4;                   // 3xTF32: k-blocks per accumulator hand-off (K = 128)
constexpr int kStageTileBytes = 32 * 32 * 4;  // one [32 rows x 32 cols] output staging tile
constexpr long long kWaitTimeoutCycles = 2000000000LL;  // about one second

template <int BN, bool X3>
struct GemmCfg {
    static constexpr bool kChunked = X3;
    static constexpr int kEpiWarps = (X3 && BN == 256) ? 8 : 4;   // chunked: 128 running sums per thread
    static constexpr int kColsPerEpiWarp = BN / (kEpiWarps / 4);
    static constexpr int kStageBufsPerWarp = kEpiWarps == 8 ? 1 : 2;
    static constexpr int kStagingBytes = kEpiWarps * kStageBufsPerWarp * kStageTileBytes;  // 32 KiB
    static constexpr int kConvWarps = X3 ? 4 : 0;
    static constexpr int kThreads = (4 + kEpiWarps + kConvWarps) * 32;
    static constexpr int kBTileBytes = BN * kBK * 4;
    static constexpr int kHiBytes = kATileBytes + kBTileBytes;
    static constexpr int kStageBytes = X3 ? 2 * kHiBytes : kHiBytes;
    static constexpr int kStages = X3 ? (BN == 256 ? 2 : 3) : (BN == 256 ? 4 : 6);  // 192 KiB ring
    static constexpr int kBarrierBytes = 8 * (3 * kStages + 5) + 8;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*alignment*/ + 256 /*barriers*/;
    static_assert(kBarrierBytes <= 256, "barrier block overflows its slot");
    static_assert(kSmemBytes <= 232448, "exceeds 227 KiB of shared memory");
    static_assert(!kChunked || kColsPerEpiWarp == 128, "chunked epilogue keeps 128 running sums per thread");
};

__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, int *status, int code,
                                             long long limit_cycles = kWaitTimeoutCycles)
{
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((++spins & 31u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit_cycles) {
                *abort_flag = 1u;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// GELU (tanh form) written as x * sigmoid(2u), u = 0.79788456 (x + 0.044715 x^3):
// identical to 0.5 x (1 + tanh u) and needs one exp2 and one reciprocal (both 1-2 ulp approximations,
// far inside the 1e-5 bound).  exp(-2u) overflows to +inf only for u < -44, where the result is -0.
__device__ __forceinline__ float gelu_tanh(float x)
{
    const float u = 0.79788456f * (x + 0.044715f * x * x * x);
    return __fdividef(x, 1.0f + __expf(-2.0f * u));
}

// d/dx of gelu_tanh(x) = 0.5 x (1 + tanh u), u = 0.79788456 (x + 0.044715 x^3):
//   0.5 (1 + t) + 0.5 x (1 - t^2) * 0.79788456 (1 + 3 * 0.044715 x^2),  t = tanh u = 1 - 2 / (1 + exp(2u))
// (the reference's constants, linear.cu:162-187; exp and division in their fast forms, 1-2 ulp, far inside the 1e-5 bound;
// exp(2u) = +inf for large u gives t = 1 exactly).
__device__ __forceinline__ float gelu_tanh_grad_fast(float x)
{
    const float u = 0.79788456f * (x + 0.044715f * x * x * x);
    const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * (0.79788456f + 0.107032f * x * x);
}

// One epilogue warp's staging state: `kBufs` swizzled [32 x 32] fp32 tiles and the count of TMA stores
// issued so far (only lane 0 issues and waits on bulk groups).
template <int kBufs>
struct StageRing {
    uint32_t base;   // shared-memory address of buffer 0 (1024-byte aligned)
    uint32_t count;
    __device__ __forceinline__ uint32_t acquire(int lane)
    {
        if (lane == 0) {
            if (kBufs == 2)
                ptx::tma_store_wait_read<1>();
            else
                ptx::tma_store_wait_read<0>();
        }
        __syncwarp();
        return base + (count % kBufs) * kStageTileBytes;
    }
};

// Writes this thread's 32 consecutive values (row = lane) into the staging tile with the 128-byte
// swizzle (16-byte chunk index XOR row mod 8) that the output tensor map undoes.
__device__ __forceinline__ void stage_row(uint32_t buf, int lane, const float (&v)[32])
{
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t addr = buf + lane * 128 + ((j ^ (lane & 7)) << 4);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]),
                     "f"(v[4 * j + 3])
                     : "memory");
    }
}

template <int BN, bool A_MN, bool B_MN, bool X3>
__global__ void __launch_bounds__(GemmCfg<BN, X3>::kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_act, const GemmParams p)
{
    using C = GemmCfg<BN, X3>;
    constexpr int STAGES = C::kStages;
    constexpr int kTmemCols = 2 * BN;  // two accumulator buffers (power of two: 256 or 512)
    constexpr int kBoxesA = A_MN ? kBM / 32 : 1;
    constexpr int kBoxesB = B_MN ? BN / 32 : 1;
    constexpr uint32_t kIdesc = ptx::make_idesc_tf32(kBM, BN, A_MN, B_MN);
    constexpr int kFirstEpiWarp = 4;
    constexpr int kFirstConvWarp = 4 + C::kEpiWarps;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

    // [ operand ring | output staging | barriers ]
    const uint32_t staging_base = smem_base + STAGES * C::kStageBytes;
    const uint32_t bar_base = staging_base + C::kStagingBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto conv_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
    auto tmem_full_bar = [&](int b) { return bar_base + 8u * (3 * STAGES + b); };
    auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (3 * STAGES + 2 + b); };
    const uint32_t drain_bar = bar_base + 8u * (3 * STAGES + 4);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + (bar_base - smem_base) + 8 * (3 * STAGES + 5));
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
            ptx::mbar_init(conv_bar(s), 4 * 32);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tmem_full_bar(b), 1);
            ptx::mbar_init(tmem_empty_bar(b), C::kEpiWarps * 32);
        }
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0u;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        ptx::prefetch_tensormap(&tmap_out);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const long long num_items = 1LL * p.tiles_m * p.tiles_n * p.splits;

    auto decode = [&](long long w, int &tm, int &tn, int &kb0, int &kb1, int &split) {
        tm = static_cast<int>(w % p.tiles_m);
        const long long r = w / p.tiles_m;
        tn = static_cast<int>(r % p.tiles_n);
        split = static_cast<int>(r / p.tiles_n);
        kb0 = split * p.kb_per_split;
        kb1 = min(kb0 + p.kb_per_split, p.num_kb);
    };

    if (warp < 4) {
        if (C::kChunked) ptx::reg_dec<56>();
        if (warp == 0) {
            // ------------------------------------------------------------ TMA producer
            uint32_t it = 0;
            bool ok = true;
            for (long long w = blockIdx.x; ok && w < num_items; w += gridDim.x) {
                int tm, tn, kb0, kb1, split;
                decode(w, tm, tn, kb0, kb1, split);
                const int m0 = tm * kBM, n0 = tn * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!bounded_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) {
                        ok = false;
                        break;
                    }
                    if (lane == 0) ptx::mbar_arrive_expect_tx(full_bar(s), C::kHiBytes);
                    __syncwarp();
                    const uint32_t a_dst = smem_base + s * C::kStageBytes;
                    const uint32_t b_dst = a_dst + kATileBytes;
                    const int k0 = kb * kBK;
                    if (lane < kBoxesA) {
                        if (A_MN)
                            ptx::tma_load_2d(a_dst + lane * kBoxBytesMN, &tmap_a, m0 + 32 * lane, k0, full_bar(s));
                        else
                            ptx::tma_load_2d(a_dst, &tmap_a, k0, m0, full_bar(s));
                    } else if (lane < kBoxesA + kBoxesB) {
                        const int j = lane - kBoxesA;
                        if (B_MN)
                            ptx::tma_load_2d(b_dst + j * kBoxBytesMN, &tmap_b, n0 + 32 * j, k0, full_bar(s));
                        else
                            ptx::tma_load_2d(b_dst, &tmap_b, k0, n0, full_bar(s));
                    }
                    __syncwarp();
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------ MMA issuer
            if (lane == 0) {
                uint32_t it = 0;
                uint32_t g = 0;  // accumulator hand-offs so far
                bool ok = true;
                for (long long w = blockIdx.x; ok && w < num_items; w += gridDim.x) {
                    int tm, tn, kb0, kb1, split;
                    decode(w, tm, tn, kb0, kb1, split);
                    int kb = kb0;
                    while (ok && kb < kb1) {
                        const int kend = C::kChunked ? min(kb + kChunkKB, kb1) : kb1;
                        const uint32_t buf = g & 1u;
                        const uint32_t use = (g >> 1) & 1u;
                        if (!bounded_wait(tmem_empty_bar(buf), use ^ 1u, abort_flag, p.status, DEV_TIMEOUT_MMA_TMEM)) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        const uint32_t d_tmem = tmem_base + buf * BN;
                        uint32_t accumulate = 0;
                        for (; kb < kend; ++kb, ++it) {
                            const int s = it % STAGES;
                            const uint32_t ph = (it / STAGES) & 1u;
                            if (!bounded_wait(full_bar(s), ph, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL)) {
                                ok = false;
                                break;
                            }
                            if (X3) {
                                if (!bounded_wait(conv_bar(s), ph, abort_flag, p.status, DEV_TIMEOUT_MMA_CONV)) {
                                    ok = false;
                                    break;
                                }
                            }
                            ptx::tc_fence_after();
                            const uint32_t a_hi = smem_base + s * C::kStageBytes;
                            const uint32_t b_hi = a_hi + kATileBytes;
                            const uint32_t a_lo = a_hi + C::kHiBytes;
                            const uint32_t b_lo = b_hi + C::kHiBytes;
#pragma unroll
                            for (int k = 0; k < kBK / kUmmaK; ++k) {
                                // K-major tile: rows of 128 B (32 k), 16-byte-chunk swizzle over 8-row atoms of 1024 B;
                                //   a k-step (8 floats) is 32 bytes along the row, 8-row groups are 1024 B apart (SBO).
                                // MN-major tile: boxes of [32 k-rows x 32 floats], 32-byte-chunk swizzle over 4-row atoms
                                //   of 512 B; a k-step is 8 rows = 1024 B, 4-row groups are 512 B apart (SBO) and the
                                //   32-float column groups are one 4 KiB box apart (LBO).
                                const uint32_t a_off = A_MN ? k * 1024 : k * 32;
                                const uint32_t b_off = B_MN ? k * 1024 : k * 32;
                                constexpr uint32_t a_lbo = A_MN ? kBoxBytesMN : 16, a_sbo = A_MN ? 512 : 1024;
                                constexpr uint32_t b_lbo = B_MN ? kBoxBytesMN : 16, b_sbo = B_MN ? 512 : 1024;
                                constexpr uint32_t a_lay = A_MN ? ptx::kLayoutSw128Base32B : ptx::kLayoutSw128;
                                constexpr uint32_t b_lay = B_MN ? ptx::kLayoutSw128Base32B : ptx::kLayoutSw128;
                                const uint64_t da_hi = ptx::make_smem_desc(a_hi + a_off, a_lbo, a_sbo, a_lay);
                                const uint64_t db_hi = ptx::make_smem_desc(b_hi + b_off, b_lbo, b_sbo, b_lay);
                                if (X3) {
                                    const uint64_t da_lo = ptx::make_smem_desc(a_lo + a_off, a_lbo, a_sbo, a_lay);
                                    const uint64_t db_lo = ptx::make_smem_desc(b_lo + b_off, b_lbo, b_sbo, b_lay);
                                    ptx::mma_tf32_ss(d_tmem, da_lo, db_hi, kIdesc, accumulate);
                                    ptx::mma_tf32_ss(d_tmem, da_hi, db_lo, kIdesc, 1u);
                                    ptx::mma_tf32_ss(d_tmem, da_hi, db_hi, kIdesc, 1u);
                                } else {
                                    ptx::mma_tf32_ss(d_tmem, da_hi, db_hi, kIdesc, accumulate);
                                }
                                accumulate = 1u;
                            }
                            ptx::mma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
                        }
                        if (ok) {
                            ptx::mma_commit(tmem_full_bar(buf));
                            ++g;
                        }
                    }
                }
                // Do not leave with MMAs still running: they write TMEM that is about to be released.
                ptx::mma_commit(drain_bar);
                bounded_wait(drain_bar, 0u, abort_flag, p.status, DEV_TIMEOUT_DRAIN);
            }
            __syncwarp();
        }
    } else if (warp < kFirstConvWarp) {
        // ------------------------------------------------------------ epilogue
        if (C::kChunked) ptx::reg_inc<C::kEpiWarps == 8 ? 184 : 200>();
        const int e = warp - kFirstEpiWarp;
        const int q = warp & 3;  // TMEM lane quarter this warp may read (warp index mod 4)
        const int col_base = (e >> 2) * C::kColsPerEpiWarp;
        const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
        StageRing<C::kStageBufsPerWarp> ring;
        ring.base = staging_base + e * C::kStageBufsPerWarp * kStageTileBytes;
        ring.count = 0;
        uint32_t g = 0;
        bool ok = true;

        // bias / GELU, staging, TMA store of one [32 rows x 32 cols] piece of the tile
        auto emit = [&](float (&v)[32], int row0, int col0, int split) {
            if (p.bias && p.epi_mode == EPI_STORE) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += (col0 + j < p.N) ? __ldg(p.bias + col0 + j) : 0.0f;
            }
            const bool in_range = row0 < p.M && col0 < p.N;
            {
                const uint32_t buf = ring.acquire(lane);
                stage_row(buf, lane, v);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (in_range) {
                        if (p.epi_mode == EPI_ACCUM)
                            ptx::tma_reduce_add_3d(&tmap_out, col0, row0, 0, buf);
                        else
                            ptx::tma_store_3d(&tmap_out, col0, row0, split, buf);
                    }
                    ptx::tma_store_commit();
                }
                ring.count++;
            }
            if (p.has_act) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
                const uint32_t buf = ring.acquire(lane);
                stage_row(buf, lane, v);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (in_range) ptx::tma_store_3d(&tmap_act, col0, row0, 0, buf);
                    ptx::tma_store_commit();
                }
                ring.count++;
            }
        };

        for (long long w = blockIdx.x; ok && w < num_items; w += gridDim.x) {
            int tm, tn, kb0, kb1, split;
            decode(w, tm, tn, kb0, kb1, split);
            const int row0 = tm * kBM + q * 32;
            const int n0 = tn * BN + col_base;
            if (C::kChunked) {
                float acc[128];
#pragma unroll
                for (int j = 0; j < 128; ++j) acc[j] = 0.0f;
                for (int kb = kb0; ok && kb < kb1; kb += kChunkKB, ++g) {
                    const uint32_t buf = g & 1u;
                    const uint32_t use = (g >> 1) & 1u;
                    if (!bounded_wait(tmem_full_bar(buf), use, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32(tmem_base + lane_base + buf * BN + col_base + c * 32, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[c * 32 + j] += __uint_as_float(v[j]);
                    }
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(tmem_empty_bar(buf));
                }
                if (ok) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = acc[c * 32 + j];
                        emit(v, row0, n0 + c * 32, split);
                    }
                }
            } else {
                const uint32_t buf = g & 1u;
                const uint32_t use = (g >> 1) & 1u;
                ++g;
                if (!bounded_wait(tmem_full_bar(buf), use, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < C::kColsPerEpiWarp / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(tmem_base + lane_base + buf * BN + col_base + c * 32, r);
                    ptx::tmem_ld_wait();
                    if (c == C::kColsPerEpiWarp / 32 - 1) {
                        // every column of this warp's share has been read: release the accumulator early
                        ptx::tc_fence_before();
                        ptx::mbar_arrive(tmem_empty_bar(buf));
                    }
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    emit(v, row0, n0 + c * 32, split);
                }
            }
        }
        // staging memory must outlive the stores that read it
        if (lane == 0) ptx::tma_store_wait_all<0>();
        __syncwarp();
    } else if (X3) {
        // ------------------------------------------------------------ 3xTF32 converter
        ptx::reg_dec<72>();
        const int ctid = threadIdx.x - kFirstConvWarp * 32;
        uint32_t it = 0;
        bool ok = true;
        for (long long w = blockIdx.x; ok && w < num_items; w += gridDim.x) {
            int tm, tn, kb0, kb1, split;
            decode(w, tm, tn, kb0, kb1, split);
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1u;
                if (!bounded_wait(full_bar(s), ph, abort_flag, p.status, DEV_TIMEOUT_CONVERT)) {
                    ok = false;
                    break;
                }
                const float4 *hi = reinterpret_cast<const float4 *>(smem_gen + s * C::kStageBytes);
                float4 *lo = reinterpret_cast<float4 *>(smem_gen + s * C::kStageBytes + C::kHiBytes);
                constexpr int kVec = C::kHiBytes / 16;
#pragma unroll 4
                for (int i = ctid; i < kVec; i += 4 * 32) {
                    const float4 h = hi[i];
                    float4 l;
                    l.x = h.x - __uint_as_float(__float_as_uint(h.x) & 0xFFFFE000u);
                    l.y = h.y - __uint_as_float(__float_as_uint(h.y) & 0xFFFFE000u);
                    l.z = h.z - __uint_as_float(__float_as_uint(h.z) & 0xFFFFE000u);
                    l.w = h.w - __uint_as_float(__float_as_uint(h.w) & 0xFFFFE000u);
                    lo[i] = l;
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(conv_bar(s));
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // A wait ran out somewhere: give copies still in flight time to land before the CTA's
        // shared memory and TMEM are handed to the next CTA.
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Self-test of the bounded wait: one thread waits, with a short limit, on a barrier that nothing will ever signal.
// The wait runs out, the status word receives DEV_TIMEOUT_SELFTEST and the kernel returns normally: exactly the path
// a real kernel takes when an expected signal never comes.
__global__ void wait_timeout_selftest_kernel(int *status, long long limit_cycles)
{
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ uint32_t abort_flag;
    const uint32_t bar = ptx::smem_u32(&bar_storage);
    if (threadIdx.x == 0) {
        ptx::mbar_init(bar, 1);
        abort_flag = 0u;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) bounded_wait(bar, 0u, &abort_flag, status, DEV_TIMEOUT_SELFTEST, limit_cycles);
    __syncthreads();
}

// out[i] (+)= sum_s ws[s][i], fixed order s = 0..splits-1 (deterministic split-K reduction).
__global__ void splitk_reduce_kernel(float *__restrict__ out, const float *__restrict__ ws, long long n4, int splits, int accumulate)
{
    const long long stride = 1LL * gridDim.x * blockDim.x;
    for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 acc = reinterpret_cast<const float4 *>(ws)[i];
        for (int s = 1; s < splits; ++s) {
            const float4 v = reinterpret_cast<const float4 *>(ws)[1LL * s * n4 + i];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        float4 *o = reinterpret_cast<float4 *>(out) + i;
        if (accumulate) {
            const float4 prev = *o;
            acc.x += prev.x; acc.y += prev.y; acc.z += prev.z; acc.w += prev.w;
        }
        *o = acc;
    }
}

}  // namespace gptb200
