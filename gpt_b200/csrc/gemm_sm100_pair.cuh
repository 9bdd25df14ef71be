// CTA-pair form of the tcgen05 GEMM (cta_group::2): two CTAs on neighbouring SMs compute one
// 256 x 256 output tile.  Each CTA loads the 128 rows of A that it owns and HALF of the B tile
// (128 of the 256 output columns); the tensor cores of both SMs read both halves of B.  Compared with the
// one-CTA kernel (gemm_sm100.cuh) an SM receives 32 KiB instead of 48 KiB of operands per k-block for the
// same number of MMAs, and the operand ring is half as wide, so it is deeper (6 stages, 3 in 3xTF32 mode).
//
// Division of work inside the pair (rank 0 = leader):
//   both CTAs   TMA producer (own A rows, own half of B) -> local full[s]
//   both CTAs   3xTF32 converters (own tiles): bf16 correction tiles for a_lo.b + a.b_lo
//   leader      one thread issues every tcgen05.mma.cta_group::2 and the commits
//   both CTAs   epilogue warps drain their own 128 TMEM lanes (the rows they own) and store them
// Cross-CTA signalling (no multicast copy anywhere):
//   TF32:    the peer's TMA loads report their bytes straight to the leader's full[s] (cta_group::2 load form),
//            which the leader arms with the byte count of both CTAs;
//   3xTF32:  loads report to the local full[s]; the converter warps of BOTH CTAs, once the correction tiles are
//            written, arrive on the leader's conv[j] (the peer's with one remote arrive per warp), the only
//            barrier the MMA thread waits on per k-block;
//   leader -> both   "stage s is free" / "accumulator b is full": one tcgen05.commit that signals the barrier at
//            the same offset in both CTAs;
//   peer -> leader   "accumulator b is drained": remote mbarrier.arrive on leader.tmem_empty[b].
// Work distribution: the k-blocks of all tiles form one line (tile after tile) that is cut into one contiguous range
// per CTA pair, so that every pair executes the same number of k-blocks whatever the tile count.  A range may begin
// and end inside a tile.  The pair whose range holds a tile's FIRST k-block owns the tile: it writes the output
// (bias, GELU, accumulate).  A pair whose range begins inside a tile computes that remainder first, stores the raw
// sums in its slot of a scratch buffer and publishes one flag per epilogue warp (release); the owner, which reaches
// the tile at the END of its own range, waits for the flags of the pairs that follow it (acquire, bounded) and
// adds their slots in pair order, so results do not depend on timing.  Pairs that publish never wait, hence the
// scheme cannot deadlock even when not all CTAs are resident at once.
// All waits are bounded exactly as in the one-CTA kernel; both CTAs always reach the closing cluster barrier.
#pragma once

#include <type_traits>

#include "gemm_sm100.cuh"

namespace gptb200 {

#ifndef GPTB200_PAIR_STAGE_COLS
#define GPTB200_PAIR_STAGE_COLS 32
#endif
#ifndef GPTB200_PAIR_STAGING_KIB
#define GPTB200_PAIR_STAGING_KIB 32
#endif
#ifndef GPTB200_PAIR_STAGES_TF32
#define GPTB200_PAIR_STAGES_TF32 6
#endif

// Ring of an epilogue warp's staging tiles (only lane 0 issues stores and waits on their bulk groups).
template <int kBufs, int kPieceBytes>
struct PieceRing {
    uint32_t base;   // shared-memory address of tile 0 (1024-byte aligned)
    uint32_t count;
    __device__ __forceinline__ uint32_t acquire(int lane)
    {
        if (lane == 0) ptx::tma_store_wait_read<kBufs - 1>();   // the store that last read this tile has finished reading
        __syncwarp();
        return base + (count % kBufs) * kPieceBytes;
    }
};

// Writes this thread's COLS consecutive values (row = lane) into a staging tile with the swizzle that the output tensor map
// undoes: rows of 128 bytes with the 16-byte chunk index XOR-ed with (row mod 8), or rows of 64 bytes with the chunk index
// XOR-ed with (row / 2 mod 4).  Either way the eight lanes of a store phase hit all 32 banks.
template <int COLS>
__device__ __forceinline__ void stage_piece(uint32_t buf, int lane, const float *v)
{
#pragma unroll
    for (int j = 0; j < COLS / 4; ++j) {
        const uint32_t addr = COLS == 32 ? buf + lane * 128 + ((j ^ (lane & 7)) << 4) : buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]),
                     "f"(v[4 * j + 3])
                     : "memory");
    }
}

template <bool X3>
struct PairCfg {
    static constexpr int BN = 256;                     // tile columns (both CTAs together)
    static constexpr int kBRows = BN / 2;              // rows of the B tile held by one CTA
    static constexpr bool kChunked = X3;
    static constexpr int kEpiWarps = 8;                // two warps per TMEM lane quarter, 128 columns each
    static constexpr int kColsPerEpiWarp = BN / (kEpiWarps / 4);
    // Output staging: every epilogue warp owns a ring of [32 rows x kStageCols] tiles; a ring of two lets the warp fill one
    // tile while the TMA store of the other is still reading shared memory.
    static constexpr int kStageCols = GPTB200_PAIR_STAGE_COLS;
    static constexpr int kStagePieceBytes = 32 * kStageCols * 4;
    static constexpr int kStagingBytes = (X3 ? 32 : GPTB200_PAIR_STAGING_KIB) * 1024;   // 3xTF32: the operand rings leave 32 KiB
    static constexpr int kStageBufsPerWarp = kStagingBytes / (kEpiWarps * kStagePieceBytes);
    static_assert(kStageCols == 16 || kStageCols == 32, "staging tiles are 16 or 32 columns wide");
    static_assert(kStageBufsPerWarp >= 1 && kStageBufsPerWarp * kEpiWarps * kStagePieceBytes == kStagingBytes, "staging ring does not tile its memory");
    static constexpr int kConvWarps = X3 ? 4 : 0;
    static constexpr int kThreads = (4 + kEpiWarps + kConvWarps) * 32;
    static constexpr int kBTileBytes = kBRows * kBK * 4;             // 16 KiB
    static constexpr int kHiBytes = kATileBytes + kBTileBytes;       // 32 KiB per CTA and stage
    static constexpr int kStageBytes = kHiBytes;       // one stage of the raw-operand ring
    // 3xTF32: raw tiles and low-order tiles have rings of their own (a low-part buffer is only busy from its
    // conversion to the MMAs that read it).  Measured on the FFN shapes: 3 + 3 stages (1246 ns per k-block) beat
    // 4 + 2 (1628 ns): with two low-part buffers the convert -> MMA -> release chain of a buffer becomes the
    // critical path.
    static constexpr int kStages = X3 ? 3 : GPTB200_PAIR_STAGES_TF32;
    static constexpr int kLoStages = X3 ? 3 : 0;
    static constexpr int kNumBarriers = 2 * kStages + 2 * (X3 ? kLoStages : 1) + 5;
    static constexpr int kSmemBytes = (kStages + kLoStages) * kHiBytes + kStagingBytes + 1024 + 256;
    static_assert(8 * kNumBarriers + 8 <= 256, "barrier block overflows its slot");
    static_assert(kSmemBytes <= 232448, "exceeds 227 KiB of shared memory");
};

__device__ __forceinline__ bool bounded_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, int *status, int code)
{
    if (ptx::mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (ptx::mbar_try_wait_cluster(bar, parity)) return true;
        if ((++spins & 31u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitTimeoutCycles) {
                *abort_flag = 1u;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// 3xTF32 on CTA pairs computes a.b as  a_hi.b_hi (tf32 MMAs on the raw fp32 tiles: the tensor core drops the low 13
// mantissa bits)  +  a_lo.b + a.b_lo (bf16 MMAs), with a_lo = a - a_hi.  The converter warps write, per operand tile, a
// bf16 tile with 64 k-positions per 32 k of the raw tile:  A: [a_lo | a]   B: [b | b_lo]  (groups of 8 values of each kind
// alternate), so that ONE bf16 MMA chain over the 64 positions yields both correction terms.  Rounding a_lo, b_lo, a
// and b to bf16 leaves an error of about 1.5e-6 of the result's scale (the products that matter are 2^-11 small).
//
// A tile is converted in 16 warp-sized pieces of 32 units (8 floats each).  Per-lane constants of the addressing:
// source offset and destination offsets (for even and odd pieces) of the lane's unit in piece 0.
//   MN-major raw tile: [32 k-rows x 32 floats] boxes, 32-byte chunks XOR-ed with (k-row & 3).  Piece p holds k-rows
//   4 (p & 7) .. + 3 of the boxes 2 (p >> 3) and 2 (p >> 3) + 1; the eight lanes of a quarter warp take one k-row of the
//   two boxes, the second box's lanes load their two halves in the other order, so that every 16-byte load and store
//   phase covers all 32 banks.  bf16 tile: [8 k-positions x 64 rows] atoms of 1 KiB (16-byte chunks XOR-ed with the
//   k-position), the 8 atoms of a 64-row half one after the other, 8 KiB to the other half.
//   K-major raw tile: 128-byte rows (32 k), 16-byte chunks XOR-ed with (row & 7); piece p holds rows 8 p .. 8 p + 7.  The
//   bf16 tile has the same geometry and swizzle.  Odd rows start with the odd chunk, which is also the logically first.
struct ConvLane {
    uint32_t src, dst_even, dst_odd;
};

template <bool MN>
__device__ __forceinline__ ConvLane conv_lane(int lane, uint32_t tile)
{
    ConvLane c;
    if (MN) {
        const int p32 = lane & 3, bpar = (lane >> 2) & 1, krl = lane >> 3;
        c.src = tile + bpar * kBoxBytesMN + krl * 128 + p32 * 32 + 16 * bpar;
        const int chunk = 4 * bpar + (p32 ^ krl);
        c.dst_even = tile + krl * 128 + ((chunk ^ krl) << 4);
        c.dst_odd = tile + (4 + krl) * 128 + ((chunk ^ (4 + krl)) << 4);
    } else {
        const int r = lane >> 2, q = lane & 3;
        c.src = tile + r * 128 + (2 * q + (r & 1)) * 16;
        c.dst_even = c.src;
        c.dst_odd = c.src;
    }
    return c;
}

template <bool MN>
__device__ __forceinline__ constexpr uint32_t conv_src_offset(int piece)
{
    return MN ? (piece >> 3) * 8192 + (piece & 7) * 512 : piece * 1024;
}

template <bool MN>
__device__ __forceinline__ constexpr uint32_t conv_dst_offset(int piece)
{
    return MN ? (piece >> 3) * 8192 + ((piece & 7) >> 1) * 2048 : piece * 1024;
}

// The arithmetic of one unit: 8 raw floats -> 8 low parts and 8 whole values in bf16, stored as A: [low | whole],
// B: [whole | low] so that one bf16 MMA chain over the doubled k gives a_lo.b + a.b_lo.
template <bool MN, bool IS_B>
__device__ __forceinline__ void convert_store(float4 f1, float4 f2, uint32_t dst, int lane)
{
    if (MN && (lane & 4)) {   // second box of the pair: halves were loaded in the other order
        const float4 t = f1;
        f1 = f2;
        f2 = t;
    }
    const float v[8] = {f1.x, f1.y, f1.z, f1.w, f2.x, f2.y, f2.z, f2.w};
    uint32_t lo[4], whole[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float l0 = v[2 * e] - __uint_as_float(__float_as_uint(v[2 * e]) & 0xFFFFE000u);
        const float l1 = v[2 * e + 1] - __uint_as_float(__float_as_uint(v[2 * e + 1]) & 0xFFFFE000u);
        lo[e] = ptx::pack_bf16x2(l0, l1);
        whole[e] = ptx::pack_bf16x2(v[2 * e], v[2 * e + 1]);
    }
    const uint32_t dst2 = MN ? dst + 1024u : dst ^ 16u;
    if (IS_B) {
        ptx::sts128(dst, whole[0], whole[1], whole[2], whole[3]);
        ptx::sts128(dst2, lo[0], lo[1], lo[2], lo[3]);
    } else {
        ptx::sts128(dst, lo[0], lo[1], lo[2], lo[3]);
        ptx::sts128(dst2, whole[0], whole[1], whole[2], whole[3]);
    }
}

// The pieces first, first + 3, ... (< 16) of one operand tile.  Deliberately a rolled loop: the kernel's code is large
// (the unrolled epilogue above all) and the converter warps were measured to run faster with a compact body than with
// unrolled or load-batched ones.
template <bool MN, bool IS_B>
__device__ __forceinline__ void convert_tile(uint32_t raw, uint32_t cor, const ConvLane &c, int first, int lane)
{
#pragma unroll 1
    for (int p = first; p < 16; p += 3) {
        const uint32_t src = raw + c.src + conv_src_offset<MN>(p);
        const float4 f1 = ptx::lds128(src), f2 = ptx::lds128(src ^ 16u);
        convert_store<MN, IS_B>(f1, f2, cor + ((p & 1) ? c.dst_odd : c.dst_even) + conv_dst_offset<MN>(p), lane);
    }
}

// k-blocks per accumulator hand-off (3xTF32).  While the epilogue warps write the previous tile's output (about 13
// thousand cycles with GELU) they cannot drain the new tile's chunks, and the MMA thread can run only two chunks ahead
// of them; a first chunk of 8 k-blocks removes that stall at tile boundaries (measured: + 1.5 % on the FFN forward GEMM,
// the kernel being power-capped), but the truncation error of the accumulator grows with the square root of the chunk
// length and the whole-model gradient check (GPT-2 124M, 1e-5 per tensor against the CPU model) is left with too little
// margin.  Hence the same length for every chunk.
constexpr int kFirstChunkKB = 4;
__device__ __forceinline__ constexpr int pair_chunk_kb(bool first_of_tile) { return first_of_tile ? kFirstChunkKB : kChunkKB; }

// First k-block (on the line of all tiles' k-blocks) of pair q out of P.
__device__ __forceinline__ long long pair_range_start(const GemmParams &p, long long q, long long P)
{
    const long long units = p.sk_total / p.sk_unit;
    return (q * units / P) * p.sk_unit;
}

// Walk of one pair over the (tile, k-block range) segments of its range.
struct PairWork {
    long long g, g_end;
    int num_kb, tiles_m2;
    __device__ __forceinline__ bool next(int &tm2, int &tn, int &kb0, int &kb1)
    {
        if (g >= g_end) return false;
        const long long tile = g / num_kb;
        kb0 = static_cast<int>(g - tile * num_kb);
        kb1 = static_cast<int>(min(static_cast<long long>(num_kb), kb0 + (g_end - g)));
        tm2 = static_cast<int>(tile % tiles_m2);
        tn = static_cast<int>(tile / tiles_m2);
        g += kb1 - kb0;
        return true;
    }
};

__device__ __forceinline__ void flag_release(unsigned int *flag, unsigned int value)
{
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

__device__ __forceinline__ unsigned int flag_acquire(const unsigned int *flag)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    return v;
}

// One lane polls, the warp learns the outcome.  False: gave up (time limit or abort flag).
__device__ __forceinline__ bool bounded_flag_wait(const unsigned int *flag, unsigned int value, int lane, volatile uint32_t *abort_flag, int *status)
{
    int ok = 1;
    if (lane == 0 && flag_acquire(flag) != value) {
        const long long t0 = clock64();
        uint32_t spins = 0;
        while (flag_acquire(flag) != value) {
            if ((++spins & 15u) == 0) {
                if (*abort_flag) { ok = 0; break; }
                if (clock64() - t0 > kWaitTimeoutCycles) {
                    *abort_flag = 1u;
                    atomicCAS(status, 0, DEV_TIMEOUT_PARTIAL);
                    ok = 0;
                    break;
                }
            }
            __nanosleep(64);
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();   // orders the other lanes' loads of the partial tile behind lane 0's acquire
    return ok != 0;
}

// The correction tiles of one whole operand, written once before a 3xTF32 launch (GemmParams::pre_operand): an expanded bf16
// matrix with 64 k-positions per 32 k in which groups of 8 values alternate -- A: [a_lo | a], B: [b | b_lo] with
// x_lo = x - (x truncated to TF32), the same numbers the converter warps produce in the main loop -- laid out so that a plain
// TMA box load with the 128-byte swizzle lands the tile in the canonical layout of the operand's major-ness:
//   K-major operand [rows][k]:  out[row][16 g + j] (first group), out[row][16 g + 8 + j] (second group), k = 8 g + j; a row has
//                               2 * k8 bf16 (k8 = k rounded up to a multiple of 8), zero beyond k;
//   MN-major operand [k][cols]: out[16 g + j][col] (first group), out[16 g + 8 + j][col] (second group); 2 * k8 rows of `cols`
//                               bf16, zero rows beyond k.
// One thread per 8 consecutive source values that share a k-group (K-major) or per 8 consecutive columns of one k (MN-major).
template <bool MN>
__global__ void split_operand_kernel(uint4 *__restrict__ out, const float *__restrict__ in, long long rows, long long cols, int is_b)
{
    // K-major: in [rows][cols = k];  MN-major: in [rows = k][cols]
    const long long k = MN ? rows : cols, k8 = (k + 7) & ~7LL;
    const long long units = MN ? k8 * (cols / 8) : rows * (k8 / 8);
    for (long long u = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; u < units; u += static_cast<long long>(gridDim.x) * blockDim.x) {
        float v[8];
        long long o_first, o_second;   // uint4 (8 bf16) index of the first and the second group's piece
        if (MN) {
            const long long kk = u / (cols / 8), c8 = u % (cols / 8);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = kk < k ? in[kk * cols + c8 * 8 + e] : 0.0f;
            const long long g = kk >> 3, j = kk & 7;
            o_first = (16 * g + j) * (cols / 8) + c8;
            o_second = (16 * g + 8 + j) * (cols / 8) + c8;
        } else {
            const long long r = u / (k8 / 8), g = u % (k8 / 8);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 8 * g + e < k ? in[r * k + 8 * g + e] : 0.0f;
            o_first = r * (k8 / 4) + 2 * g;
            o_second = o_first + 1;
        }
        uint32_t lo[4], whole[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float l0 = v[2 * e] - __uint_as_float(__float_as_uint(v[2 * e]) & 0xFFFFE000u);
            const float l1 = v[2 * e + 1] - __uint_as_float(__float_as_uint(v[2 * e + 1]) & 0xFFFFE000u);
            lo[e] = ptx::pack_bf16x2(l0, l1);
            whole[e] = ptx::pack_bf16x2(v[2 * e], v[2 * e + 1]);
        }
        const uint4 w4 = make_uint4(whole[0], whole[1], whole[2], whole[3]), l4 = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        out[o_first] = is_b ? w4 : l4;
        out[o_second] = is_b ? l4 : w4;
    }
}

// Bias gradient inside the grad_w GEMM: column sums of B (= grad_y [K x N], row pitch ld) over the k-blocks kb_first,
// kb_first + kb_step, ... < kb_end, for 16 consecutive columns per warp.  A quarter of four lanes covers the 16 columns of one
// row with a 16-byte load each, the eight quarters take eight consecutive rows; `s` carries the lane's running sums of its four
// columns (col .. col + 3) from call to call.  The rows are fetched by the operand loads of the same CTA at about the same time,
// so these loads are served by L2.
template <int UNROLL>
__device__ __forceinline__ void column_sums_16(float4 &s, const float *__restrict__ src, long long ld, int kb_first, int kb_step, int kb_end, int K,
                                               int col, bool col_ok, int lane)
{
    if (kb_first >= kb_end) return;
    const int groups = 4 * ((kb_end - 1 - kb_first) / kb_step + 1);   // groups of eight rows: four per k-block
    const int g = lane >> 2;
    for (int t0 = 0; t0 < groups; t0 += UNROLL) {
        float4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int t = t0 + u;
            const int r = (kb_first + (t >> 2) * kb_step) * kBK + (t & 3) * 8 + g;
            v[u] = (col_ok && t < groups && r < K) ? __ldg(reinterpret_cast<const float4 *>(src + static_cast<long long>(r) * ld + col)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            s.x += v[u].x;
            s.y += v[u].y;
            s.z += v[u].z;
            s.w += v[u].w;
        }
    }
}

// Adds the eight quarters' sums: afterwards every lane holds the total of its four columns (the same bits in all lanes of a
// column group: each butterfly step adds the same two numbers on both sides).
__device__ __forceinline__ void column_sums_finish(float4 &s)
{
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        s.x += __shfl_xor_sync(0xffffffffu, s.x, off);
        s.y += __shfl_xor_sync(0xffffffffu, s.y, off);
        s.z += __shfl_xor_sync(0xffffffffu, s.z, off);
        s.w += __shfl_xor_sync(0xffffffffu, s.w, off);
    }
}

// DB: the bias gradient is computed in this launch (see GemmParams::dbias); instantiated for the grad_w form only.
template <bool A_MN, bool B_MN, bool X3, bool DB = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<X3>::kThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_act,
                         const __grid_constant__ CUtensorMap tmap_pre, const GemmParams p)
{
    using C = PairCfg<X3>;
    constexpr int BN = C::BN;
    constexpr int STAGES = C::kStages;
    constexpr int kTmemCols = 2 * BN;
    constexpr int kBoxesA = A_MN ? kBM / 32 : 1;
    constexpr int kBoxesB = B_MN ? C::kBRows / 32 : 1;
    constexpr uint32_t kIdesc = ptx::make_idesc_tf32(2 * kBM, BN, A_MN, B_MN);  // M = 256 over the pair
    constexpr uint32_t kIdescCorr = ptx::make_idesc_bf16(2 * kBM, BN, A_MN, B_MN);
    constexpr int kFirstEpiWarp = 4;
    constexpr int kFirstConvWarp = 4 + C::kEpiWarps;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

    constexpr int NL = X3 ? C::kLoStages : 1;   // low-part buffers (3xTF32)
    const uint32_t lo_base = smem_base + STAGES * C::kHiBytes;
    const uint32_t staging_base = lo_base + C::kLoStages * C::kHiBytes;
    const uint32_t bar_base = staging_base + C::kStagingBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto conv_bar = [&](int j) { return bar_base + 8u * (2 * STAGES + j); };          // correction tiles of buffer j written, both CTAs (leader only)
    auto lo_empty_bar = [&](int j) { return bar_base + 8u * (2 * STAGES + NL + j); }; // correction buffer j read by its MMAs
    auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 * NL + b); };
    auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 * NL + 2 + b); };  // used in the leader only
    const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 2 * NL + 4);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + (bar_base - smem_base) + 8 * C::kNumBarriers);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();   // 0 = leader
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int j = 0; j < NL; ++j) {
            // leader: one arrival per converter warp (three of each CTA) of the group that owns the buffer, plus the producer's
            // arrival that announces the bytes of a correction tile fetched by TMA (pre_operand)
            ptx::mbar_init(conv_bar(j), (X3 && p.pre_operand) ? 7 : 6);
            ptx::mbar_init(lo_empty_bar(j), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tmem_full_bar(b), 1);
            ptx::mbar_init(tmem_empty_bar(b), 2 * C::kEpiWarps);   // one arrival per epilogue warp of either CTA
        }
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0u;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        ptx::prefetch_tensormap(&tmap_out);
        if (X3 && p.pre_operand) ptx::prefetch_tensormap(&tmap_pre);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();   // the peer's barriers exist before anything is signalled across CTAs
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_m2 = (p.tiles_m + 1) / 2;   // pairs of 128-row tiles
    // narrow batched form: only the first mma_n / 2 columns of this CTA's B tile are loaded, split and read (K-major: that many
    // 128-byte rows, the box of the tensor map has exactly them; MN-major: the 32-column boxes that hold them)
    const uint32_t b_boxes = p.mma_n ? static_cast<uint32_t>((p.mma_n / 2 + 31) / 32) : static_cast<uint32_t>(C::kBRows / 32);
    const uint32_t b_used = !p.mma_n ? static_cast<uint32_t>(C::kBTileBytes) : B_MN ? b_boxes * kBoxBytesMN : static_cast<uint32_t>(p.mma_n / 2) * 128u;
    const long long num_pairs = gridDim.x >> 1;
    const long long pair_id = blockIdx.x >> 1;
    auto trace = [&](int event, uint32_t slot) {
        if (p.trace == nullptr || blockIdx.x > 1 || slot >= kTraceSlots) return;
        if (blockIdx.x == 1) {   // the peer CTA records its producer and converter events only
            if (event > TRACE_CONV_END) return;
            event += TRACE_PEER_LOAD_ISSUE;
        }
        p.trace[event * kTraceSlots + slot] = clock64();
    };
    auto my_work = [&]() {
        PairWork w;
        w.g = pair_range_start(p, pair_id, num_pairs);
        w.g_end = pair_range_start(p, pair_id + 1, num_pairs);
        w.num_kb = p.num_kb;
        w.tiles_m2 = tiles_m2;
        return w;
    };

    // 3xTF32 converters: six warps (warps 2, 3 and the last four) in two groups of three; group g handles the
    // k-blocks with (iteration & 1) == g, so that waking up, converting and signalling one stage overlaps with
    // the other group's stage.
    auto convert_loop = [&](int group, int wgrp) {
        // A stage is 32 warp-sized pieces (32 units of 8 floats): 16 of the A tile, 16 of the B tile.  The three warps of a
        // group take every third piece of A and, starting one warp later, every third piece of B (11, 11 and 10 pieces).
        const int wgrp_b = (wgrp + 2) % 3;
        const ConvLane lane_a = conv_lane<A_MN>(lane, 0u);
        const ConvLane lane_b = conv_lane<B_MN>(lane, kATileBytes);
        uint32_t it = 0;
        bool ok = true;
        PairWork work = my_work();
        int tm2, tn, kb0, kb1;
        while (ok && work.next(tm2, tn, kb0, kb1)) {
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                if (static_cast<int>(it & 1u) != group) continue;
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1u;
                const int j = it % NL;
                const uint32_t lph = (it / NL) & 1u;
                // the low-part buffer must have been read by the MMAs of its previous use, the raw tile must have landed
                if (!bounded_wait_cluster(lo_empty_bar(j), lph ^ 1u, abort_flag, p.status, DEV_TIMEOUT_CONVERT) ||
                    !bounded_wait(full_bar(s), ph, abort_flag, p.status, DEV_TIMEOUT_CONVERT)) {
                    ok = false;
                    break;
                }
                if (wgrp == 0 && lane == 0) trace(TRACE_CONV_BEGIN, it);
                const uint32_t raw = smem_base + s * C::kHiBytes;
                const uint32_t cor = lo_base + j * C::kHiBytes;
                if (p.exact3x) {
                    // low parts as fp32 tiles in the raw tiles' own layout: every 16-byte piece of the stage, a third per warp
#pragma unroll 1
                    for (uint32_t idx = wgrp * 32 + lane; idx < (kATileBytes + b_used) / 16; idx += 96) {
                        const uint32_t off = idx * 16;   // the A tile, then the part of the B tile that the instruction reads
                        float4 v = ptx::lds128(raw + off);
                        v.x -= __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
                        v.y -= __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
                        v.z -= __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
                        v.w -= __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
                        ptx::sts128(cor + off, __float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w));
                    }
                } else {
                    if (p.pre_operand != 1) convert_tile<A_MN, false>(raw, cor, lane_a, wgrp, lane);
                    if (p.pre_operand != 2) convert_tile<B_MN, true>(raw, cor, lane_b, p.pre_operand ? wgrp : wgrp_b, lane);
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (leader)
                        ptx::mbar_arrive(conv_bar(j));
                    else
                        ptx::mbar_arrive_remote(ptx::map_to_cta(conv_bar(j), 0u));
                    if (wgrp == 0) trace(TRACE_CONV_END, it);
                }
            }
        }
    };

    if (warp < 4) {
        if (C::kChunked) ptx::reg_dec<64>();
        if (warp == 0) {
            // ------------------------------------------------------------ TMA producer (both CTAs)
            uint32_t it = 0;
            bool ok = true;
            PairWork work = my_work();
            int tm2, tn, kb0, kb1;
            while (ok && work.next(tm2, tn, kb0, kb1)) {
                const int z = p.batches > 0 ? tn / p.tiles_n : 0;                     // batched form: the tile columns of all batches are numbered through
                if (p.batches > 0) tn -= z * p.tiles_n;
                const int zi = p.batches > 0 ? z % p.batch_inner : 0, zo = p.batches > 0 ? z / p.batch_inner : 0;
                const int m0 = tm2 * 2 * kBM + static_cast<int>(rank) * kBM;          // the rows this CTA owns
                const int n0 = tn * BN + static_cast<int>(rank) * (p.mma_n ? p.mma_n / 2 : C::kBRows);   // the half of B this CTA loads
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!bounded_wait_cluster(empty_bar(s), ph ^ 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) {
                        ok = false;
                        break;
                    }
                    if (lane == 0) trace(TRACE_LOAD_ISSUE, it);
                    // TF32: every load of the pair reports to the leader's barrier, armed by the leader for both CTAs.
                    // 3xTF32: each CTA's loads report to its own barrier (its converter warps wait on it).
                    const uint32_t bar = X3 ? full_bar(s) : ptx::map_to_cta(full_bar(s), 0u);
                    if (lane == 0 && (X3 || leader)) ptx::mbar_arrive_expect_tx(full_bar(s), (X3 ? 1u : 2u) * (kATileBytes + b_used));
                    __syncwarp();
                    const uint32_t a_dst = smem_base + s * C::kHiBytes;
                    const uint32_t b_dst = a_dst + kATileBytes;
                    const int k0 = kb * kBK;
                    if (p.batches > 0) {
                        if (lane < kBoxesA) {
                            if (A_MN)
                                ptx::tma_load_4d_pair(a_dst + lane * kBoxBytesMN, &tmap_a, m0 + 32 * lane, zi, k0, zo, bar);
                            else
                                ptx::tma_load_4d_pair(a_dst, &tmap_a, k0, zi, m0, zo, bar);
                        } else if (lane < kBoxesA + (B_MN ? static_cast<int>(b_boxes) : 1)) {
                            const int j = lane - kBoxesA;
                            if (B_MN)
                                ptx::tma_load_4d_pair(b_dst + j * kBoxBytesMN, &tmap_b, n0 + 32 * j, zi, k0, zo, bar);
                            else
                                ptx::tma_load_4d_pair(b_dst, &tmap_b, k0, zi, n0, zo, bar);
                        }
                    } else if (lane < kBoxesA) {
                        if (A_MN)
                            ptx::tma_load_2d_pair(a_dst + lane * kBoxBytesMN, &tmap_a, m0 + 32 * lane, k0, bar);
                        else
                            ptx::tma_load_2d_pair(a_dst, &tmap_a, k0, m0, bar);
                    } else if (lane < kBoxesA + kBoxesB) {
                        const int j = lane - kBoxesA;
                        if (B_MN)
                            ptx::tma_load_2d_pair(b_dst + j * kBoxBytesMN, &tmap_b, n0 + 32 * j, k0, bar);
                        else
                            ptx::tma_load_2d_pair(b_dst, &tmap_b, k0, n0, bar);
                    }
                    __syncwarp();
                    if (X3 && p.pre_operand) {
                        // The correction tile of the operand that was split before the launch: 16 KiB per CTA from the expanded
                        // bf16 matrix (64 k-positions per 32 k) into correction buffer j, bytes reported to the leader's conv[j].
                        //   K-major:  rows of the operand, 32 four-byte words (64 bf16) per k-block, 128-byte swizzle: one box;
                        //   MN-major: [64 k-positions x 64 rows-of-the-operand] atoms: one box per half of the CTA's 128 rows.
                        const int j = it % NL;
                        const uint32_t lph = (it / NL) & 1u;
                        if (!bounded_wait_cluster(lo_empty_bar(j), lph ^ 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) {
                            ok = false;
                            break;
                        }
                        const bool pre_a = p.pre_operand == 1;
                        const bool pre_mn = pre_a ? A_MN : B_MN;
                        const int r0 = pre_a ? m0 : n0;   // first of this CTA's 128 rows (A) / columns (B)
                        const uint32_t dst = lo_base + j * C::kHiBytes + (pre_a ? 0 : kATileBytes);
                        const uint32_t cbar = ptx::map_to_cta(conv_bar(j), 0u);
                        if (leader && lane == 0) ptx::mbar_arrive_expect_tx(conv_bar(j), 2 * kATileBytes);
                        __syncwarp();
                        if (pre_mn) {
                            if (lane < 2) ptx::tma_load_2d_pair(dst + lane * 8192, &tmap_pre, (r0 + 64 * lane) / 2, 2 * k0, cbar);
                        } else {
                            if (lane == 0) ptx::tma_load_2d_pair(dst, &tmap_pre, k0, r0, cbar);
                        }
                        __syncwarp();
                    }
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------ MMA issuer (leader CTA, one thread)
            if (leader && lane == 0) {
                uint32_t it = 0, g = 0;
                bool ok = true;
                PairWork work = my_work();
                int tm2, tn, kb0, kb1;
                const uint32_t idesc = p.mma_n ? ptx::make_idesc_tf32(2 * kBM, p.mma_n, A_MN, B_MN) : kIdesc;
                const uint32_t idesc_corr = p.mma_n ? ptx::make_idesc_bf16(2 * kBM, p.mma_n, A_MN, B_MN) : kIdescCorr;
                while (ok && work.next(tm2, tn, kb0, kb1)) {
                    int kb = kb0;
                    while (ok && kb < kb1) {
                        const int kend = C::kChunked ? min(kb + (p.chunk_kb ? p.chunk_kb : pair_chunk_kb(kb == kb0)), kb1) : kb1;
                        const uint32_t buf = g & 1u;
                        const uint32_t use = (g >> 1) & 1u;
                        if (!bounded_wait_cluster(tmem_empty_bar(buf), use ^ 1u, abort_flag, p.status, DEV_TIMEOUT_MMA_TMEM)) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        const uint32_t d_tmem = tmem_base + buf * BN;
                        uint32_t accumulate = 0;
                        for (; kb < kend; ++kb, ++it) {
                            const int s = it % STAGES;
                            const uint32_t ph = (it / STAGES) & 1u;
                            // 3xTF32: the converters of both CTAs report to one barrier of the leader; they have seen their raw
                            // tiles land, so that barrier stands for the loads as well
                            if (!X3 && !bounded_wait_cluster(full_bar(s), ph, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL)) { ok = false; break; }
                            trace(TRACE_MMA_FULL, it);
                            const int j = it % NL;
                            const uint32_t lph = (it / NL) & 1u;
                            if (X3 && !bounded_wait_cluster(conv_bar(j), lph, abort_flag, p.status, DEV_TIMEOUT_MMA_CONV)) { ok = false; break; }
                            ptx::tc_fence_after();
                            trace(TRACE_MMA_READY, it);
                            const uint32_t a_hi = smem_base + s * C::kHiBytes;
                            const uint32_t b_hi = a_hi + kATileBytes;
                            const uint32_t a_lo = lo_base + j * C::kHiBytes;
                            const uint32_t b_lo = a_lo + kATileBytes;
                            constexpr uint32_t a_lbo = A_MN ? kBoxBytesMN : 16, a_sbo = A_MN ? 512 : 1024;
                            constexpr uint32_t b_lbo = B_MN ? kBoxBytesMN : 16, b_sbo = B_MN ? 512 : 1024;
                            constexpr uint32_t a_lay = A_MN ? ptx::kLayoutSw128Base32B : ptx::kLayoutSw128;
                            constexpr uint32_t b_lay = B_MN ? ptx::kLayoutSw128Base32B : ptx::kLayoutSw128;
                            if (X3 && p.exact3x) {
                                // correction terms in TF32 as well: a_lo.b + a.b_lo with fp32 low-part tiles laid out like the raw ones
#pragma unroll
                                for (int k = 0; k < kBK / kUmmaK; ++k) {
                                    const uint32_t a_off = A_MN ? k * 1024 : k * 32;
                                    const uint32_t b_off = B_MN ? k * 1024 : k * 32;
                                    const uint64_t da_hi = ptx::make_smem_desc(a_hi + a_off, a_lbo, a_sbo, a_lay);
                                    const uint64_t db_hi = ptx::make_smem_desc(b_hi + b_off, b_lbo, b_sbo, b_lay);
                                    const uint64_t da_lo = ptx::make_smem_desc(a_lo + a_off, a_lbo, a_sbo, a_lay);
                                    const uint64_t db_lo = ptx::make_smem_desc(b_lo + b_off, b_lbo, b_sbo, b_lay);
                                    ptx::mma_tf32_ss_pair(d_tmem, da_lo, db_hi, idesc, accumulate);
                                    ptx::mma_tf32_ss_pair(d_tmem, da_hi, db_lo, idesc, 1u);
                                    accumulate = 1u;
                                }
                            } else if (X3) {
                                // correction terms a_lo.b + a.b_lo: bf16 tiles with 64 k-positions (low parts and whole values
                                // side by side), 16 of them per instruction.  K-major: 128-byte rows, +32 bytes per step;
                                // MN-major: [8 k x 64 m] atoms, 1 KiB per group of 8 k, 8 KiB to the next 64 rows.
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    const uint64_t da = ptx::make_smem_desc(a_lo + (A_MN ? k * 2048 : k * 32), A_MN ? 8192 : 16, 1024, ptx::kLayoutSw128);
                                    const uint64_t db = ptx::make_smem_desc(b_lo + (B_MN ? k * 2048 : k * 32), B_MN ? 8192 : 16, 1024, ptx::kLayoutSw128);
                                    ptx::mma_f16_ss_pair(d_tmem, da, db, idesc_corr, accumulate);
                                    accumulate = 1u;
                                }
                            }
#pragma unroll
                            for (int k = 0; k < kBK / kUmmaK; ++k) {
                                const uint32_t a_off = A_MN ? k * 1024 : k * 32;
                                const uint32_t b_off = B_MN ? k * 1024 : k * 32;
                                const uint64_t da_hi = ptx::make_smem_desc(a_hi + a_off, a_lbo, a_sbo, a_lay);
                                const uint64_t db_hi = ptx::make_smem_desc(b_hi + b_off, b_lbo, b_sbo, b_lay);
                                ptx::mma_tf32_ss_pair(d_tmem, da_hi, db_hi, idesc, accumulate);
                                accumulate = 1u;
                            }
                            // the stage is free in both CTAs once these MMAs have read it
                            ptx::mma_commit_pair_both(empty_bar(s), 3);
                            if (X3) ptx::mma_commit_pair_both(lo_empty_bar(j), 3);
                            trace(TRACE_MMA_ISSUED, it);
                        }
                        if (ok) {
                            ptx::mma_commit_pair_both(tmem_full_bar(buf), 3);
                            ++g;
                        }
                    }
                }
                ptx::mma_commit_pair(drain_bar);
                bounded_wait(drain_bar, 0u, abort_flag, p.status, DEV_TIMEOUT_DRAIN);
            }
            __syncwarp();
        } else if (X3) {
            convert_loop(warp - 2, 0);   // warps 2 and 3: first warp of converter group 0 and 1
        }
    } else if (warp < kFirstConvWarp) {
        // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        if (C::kChunked) ptx::reg_inc<192>();
        const int e = warp - kFirstEpiWarp;
        const int q = warp & 3;
        const int col_base = (e >> 2) * C::kColsPerEpiWarp;
        const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
        PieceRing<C::kStageBufsPerWarp, C::kStagePieceBytes> ring;
        ring.base = staging_base + e * C::kStageBufsPerWarp * C::kStagePieceBytes;
        ring.count = 0;
        uint32_t g = 0, tile_count = 0;
        bool ok = true;
        // This launch's number: kept in device memory and advanced by the launch's last CTA (see the teardown), so that it is
        // right also when the launch is replayed from a CUDA graph with unchanged parameters.  0 never occurs as a number.
        const unsigned int sk_epoch = p.sk_flags ? __ldcg(p.sk_state) + 1u : 0u;
        const uint32_t leader_tmem_empty[2] = {ptx::map_to_cta(tmem_empty_bar(0), 0u), ptx::map_to_cta(tmem_empty_bar(1), 0u)};

        int ezi = 0, ezo = 0;   // batched form: batch coordinates of the tile being written
        // bias_lane: bias[col0 + lane], fetched when the tile was started
        auto emit = [&](float (&v)[32], int row0, int col0, float bias_lane) {
            if (p.mma_n && col0 >= p.mma_n) return;   // narrow batched form: these accumulator columns were not computed
            if (p.causal_skip && col0 > row0 + 31) return;   // nobody reads these
            if (p.bias && p.epi_mode == EPI_STORE) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, bias_lane, j);
            }
            if (p.gelu_src && p.epi_mode == EPI_STORE && row0 + lane < p.M) {
                // this thread's row of the pre-activation, 128 contiguous bytes, a quarter at a time (register budget of the chunked form)
                const float4 *src = reinterpret_cast<const float4 *>(p.gelu_src + static_cast<long long>(row0 + lane) * p.N + col0);
#pragma unroll
                for (int qt = 0; qt < 4; ++qt) {
                    const bool in = col0 + 8 * qt < p.N;      // N is a multiple of 4: a 16-byte piece is inside or outside as a whole
                    const float4 xa = in ? __ldg(src + 2 * qt) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    const float4 xb = (col0 + 8 * qt + 4 < p.N) ? __ldg(src + 2 * qt + 1) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    v[8 * qt] *= gelu_tanh_grad_fast(xa.x);
                    v[8 * qt + 1] *= gelu_tanh_grad_fast(xa.y);
                    v[8 * qt + 2] *= gelu_tanh_grad_fast(xa.z);
                    v[8 * qt + 3] *= gelu_tanh_grad_fast(xa.w);
                    v[8 * qt + 4] *= gelu_tanh_grad_fast(xb.x);
                    v[8 * qt + 5] *= gelu_tanh_grad_fast(xb.y);
                    v[8 * qt + 6] *= gelu_tanh_grad_fast(xb.z);
                    v[8 * qt + 7] *= gelu_tanh_grad_fast(xb.w);
                }
            }
            constexpr int kPieces = 32 / C::kStageCols;
#pragma unroll
            for (int h = 0; h < kPieces; ++h) {
                const uint32_t buf = ring.acquire(lane);
                stage_piece<C::kStageCols>(buf, lane, &v[h * C::kStageCols]);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (row0 < p.M && col0 + h * C::kStageCols < p.N) {
                        if (p.batches > 0)
                            ptx::tma_store_4d(&tmap_out, col0 + h * C::kStageCols, ezi, row0, ezo, buf);
                        else if (p.epi_mode == EPI_ACCUM)
                            ptx::tma_reduce_add_3d(&tmap_out, col0 + h * C::kStageCols, row0, 0, buf);
                        else
                            ptx::tma_store_3d(&tmap_out, col0 + h * C::kStageCols, row0, 0, buf);
                    }
                    ptx::tma_store_commit();
                }
                ring.count++;
            }
            if (p.has_act) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
#pragma unroll
                for (int h = 0; h < kPieces; ++h) {
                    const uint32_t buf = ring.acquire(lane);
                    stage_piece<C::kStageCols>(buf, lane, &v[h * C::kStageCols]);
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (row0 < p.M && col0 + h * C::kStageCols < p.N) ptx::tma_store_3d(&tmap_act, col0 + h * C::kStageCols, row0, 0, buf);
                        ptx::tma_store_commit();
                    }
                    ring.count++;
                }
            }
        };

        PairWork work = my_work();
        int tm2, tn, kb0, kb1;
        while (ok && work.next(tm2, tn, kb0, kb1)) {
            if (p.batches > 0) {
                const int z = tn / p.tiles_n;
                tn -= z * p.tiles_n;
                ezi = z % p.batch_inner;
                ezo = z / p.batch_inner;
            }
            const int row0 = tm2 * 2 * kBM + static_cast<int>(rank) * kBM + q * 32;
            const int n0 = tn * BN + col_base;
            const bool owner = kb0 == 0;              // this pair writes the tile's output
            const bool complete = kb1 == p.num_kb;    // ... and nobody else holds a part of it
            const long long tile_end = (1LL * tn * tiles_m2 + tm2 + 1) * p.num_kb;
            // slot of pair r: [CTA][epilogue warp][128 values][lane]
            auto slot_of = [&](long long r) { return p.sk_slots + ((r * 2 + rank) * C::kEpiWarps + e) * 4096 + lane; };
            auto flag_of = [&](long long r) { return p.sk_flags + (r * 2 + rank) * C::kEpiWarps + e; };
            // bias gradient: the tiles of a tile column read the same columns of B; the first db_rows of them share the column
            // sums, tile (tm2, tn) taking the k-blocks kb = tm2 (mod db_rows); 16 columns per epilogue warp
            // (p.dbias_rows = number of tile rows that share the work: all of them, or only the first)
            const int db_rows = DB ? p.dbias_rows : 1;
            const bool duty = DB && p.dbias != nullptr && tm2 < db_rows;
            const int db_first = kb0 + (tm2 - kb0 % db_rows + db_rows) % db_rows;   // first k-block >= kb0 of this tile's share
            const int bcol = tn * BN + static_cast<int>(rank) * C::kBRows + e * 16 + (lane & 3) * 4;
            float4 bsum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            auto dbias_slot = [&](long long r) { return reinterpret_cast<float4 *>(p.sk_dbias + (r * 2 + rank) * C::kBRows + e * 16) + (lane & 3); };
            auto dbias_add_partner = [&](long long r) {
                if (duty && lane < 4) {
                    const float4 t = __ldcg(dbias_slot(r));
                    bsum.x += t.x; bsum.y += t.y; bsum.z += t.z; bsum.w += t.w;
                }
            };
            // Owner of the tile: bsum is the tile's share.  The shares of the db_rows tiles of this column are parked in scratch;
            // the warp that parks the last one (a ticket per tile column, CTA and epilogue warp, which it also resets) adds them
            // in tile order, so the sum does not depend on who came last, and adds the total into grad_b.
            auto dbias_write = [&]() {
                if (!duty) return;
                if (db_rows > 1) {
                    const long long npad = static_cast<long long>(p.tiles_n) * BN;
                    float *part = p.dbias_part + tn * BN + static_cast<int>(rank) * C::kBRows + e * 16 + (lane & 3) * 4;
                    if (lane < 4) __stcg(reinterpret_cast<float4 *>(part + tm2 * npad), bsum);
                    __threadfence();
                    __syncwarp();
                    int last = 0;
                    if (lane == 0) {
                        unsigned int *ticket = p.dbias_tickets + (tn * 2 + rank) * C::kEpiWarps + e;
                        last = atomicAdd(ticket, 1u) == static_cast<unsigned int>(db_rows - 1);
                        if (last) atomicExch(ticket, 0u);
                        __threadfence();
                    }
                    last = __shfl_sync(0xffffffffu, last, 0);
                    if (!last) return;
                    bsum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (lane < 4) {
                        for (int t = 0; t < db_rows; ++t) {
                            const float4 v = __ldcg(reinterpret_cast<const float4 *>(part + t * npad));
                            bsum.x += v.x; bsum.y += v.y; bsum.z += v.z; bsum.w += v.w;
                        }
                    }
                }
                if (lane < 4 && bcol < p.N) {
                    float *dst = p.dbias + bcol;
                    dst[0] += bsum.x; dst[1] += bsum.y; dst[2] += bsum.z; dst[3] += bsum.w;
                }
            };
            float bias_pre[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (owner && p.bias && p.epi_mode == EPI_STORE) {
#pragma unroll
                for (int c = 0; c < 4; ++c) bias_pre[c] = (n0 + c * 32 + lane < p.N) ? __ldg(p.bias + n0 + c * 32 + lane) : 0.0f;
            }
            if (C::kChunked) {
                float acc[128];
#pragma unroll
                for (int j = 0; j < 128; ++j) acc[j] = 0.0f;
                for (int kb = kb0; ok && kb < kb1; kb += (p.chunk_kb ? p.chunk_kb : pair_chunk_kb(kb == kb0)), ++g) {
                    const uint32_t buf = g & 1u;
                    const uint32_t use = (g >> 1) & 1u;
                    if (!bounded_wait_cluster(tmem_full_bar(buf), use, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE)) {
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
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive_cluster(leader_tmem_empty[buf]);
                    // this tile's share of the k-blocks of the chunk just drained (fetched by the operand loads a moment ago)
                    if (duty) {
                        const int first = kb + (tm2 - kb % db_rows + db_rows) % db_rows;
                        column_sums_16<8>(bsum, p.dbias_src, p.N, first, db_rows, min(kb + pair_chunk_kb(kb == kb0), kb1), p.K, bcol, bcol < p.N, lane);
                    }
                }
                if (duty) column_sums_finish(bsum);
                if (ok && !owner) {
                    float *slot = slot_of(pair_id);
#pragma unroll
                    for (int j = 0; j < 128; ++j) __stcg(slot + j * 32, acc[j]);
                    if (duty && lane < 4) __stcg(dbias_slot(pair_id), bsum);
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) flag_release(flag_of(pair_id), sk_epoch);
                } else if (ok) {
                    if (!complete) {
                        for (long long r = pair_id + 1; ok && r < num_pairs && pair_range_start(p, r, num_pairs) < tile_end; ++r) {
                            ok = bounded_flag_wait(flag_of(r), sk_epoch, lane, abort_flag, p.status);
                            if (!ok) break;
                            const float *slot = slot_of(r);
#pragma unroll
                            for (int j = 0; j < 128; ++j) acc[j] += __ldcg(slot + j * 32);
                            dbias_add_partner(r);
                        }
                    }
                    if (ok) {
                        dbias_write();
                        if (e == 0 && lane == 0) trace(TRACE_EPI_BEGIN, tile_count);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            float v[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = acc[c * 32 + j];
                            emit(v, row0, n0 + c * 32, bias_pre[c]);
                        }
                        if (e == 0 && lane == 0) trace(TRACE_EPI_END, tile_count);
                        ++tile_count;
                    }
                }
            } else {
                const uint32_t buf = g & 1u;
                const uint32_t use = (g >> 1) & 1u;
                ++g;
                // while the tensor cores work on this range: the column sums of its rows of B
                if (duty) {
                    column_sums_16<16>(bsum, p.dbias_src, p.N, db_first, db_rows, kb1, p.K, bcol, bcol < p.N, lane);
                    column_sums_finish(bsum);
                }
                if (!bounded_wait_cluster(tmem_full_bar(buf), use, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                long long r_end = pair_id + 1;   // pairs [pair_id + 1, r_end) hold the rest of this tile
                if (owner && !complete) {
                    while (r_end < num_pairs && pair_range_start(p, r_end, num_pairs) < tile_end) ++r_end;
                    for (long long r = pair_id + 1; ok && r < r_end; ++r) {
                        ok = bounded_flag_wait(flag_of(r), sk_epoch, lane, abort_flag, p.status);
                        if (ok) dbias_add_partner(r);
                    }
                }
                if (ok && owner) dbias_write();
#pragma unroll 1
                for (int c = 0; c < C::kColsPerEpiWarp / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(tmem_base + lane_base + buf * BN + col_base + c * 32, r);
                    ptx::tmem_ld_wait();
                    if (c == C::kColsPerEpiWarp / 32 - 1) {
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive_cluster(leader_tmem_empty[buf]);
                    }
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (!ok) continue;   // the accumulator is still released so that the MMA thread can finish
                    if (!owner) {
                        float *slot = slot_of(pair_id) + c * 32 * 32;
#pragma unroll
                        for (int j = 0; j < 32; ++j) __stcg(slot + j * 32, v[j]);
                    } else {
                        for (long long rr = pair_id + 1; rr < r_end; ++rr) {
                            const float *slot = slot_of(rr) + c * 32 * 32;
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] += __ldcg(slot + j * 32);
                        }
                        emit(v, row0, n0 + c * 32, c == 0 ? bias_pre[0] : c == 1 ? bias_pre[1] : c == 2 ? bias_pre[2] : bias_pre[3]);
                    }
                }
                if (ok && !owner) {
                    if (duty && lane < 4) __stcg(dbias_slot(pair_id), bsum);
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) flag_release(flag_of(pair_id), sk_epoch);
                }
            }
        }
        if (lane == 0) ptx::tma_store_wait_all<0>();
        __syncwarp();
    } else if (X3) {
        // ------------------------------------------------------------ 3xTF32 converters (last four warps)
        ptx::reg_dec<64>();
        const int j = warp - kFirstConvWarp;
        convert_loop(j >> 1, 1 + (j & 1));
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    // Neither CTA may leave while the other can still signal its barriers or read its shared memory.
    ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && p.sk_flags) {
        // the last CTA to get here closes the launch: the next one (same stream, hence after this kernel) sees a new number
        __threadfence();
        if (atomicAdd(p.sk_state + 1, 1u) == gridDim.x - 1) {
            p.sk_state[1] = 0u;
            const unsigned int next = p.sk_state[0] + 1u;
            p.sk_state[0] = next == 0xFFFFFFFFu ? 0u : next;   // the number used is state + 1: skip the wrap to 0
            __threadfence();
        }
    }
}

}  // namespace gptb200
