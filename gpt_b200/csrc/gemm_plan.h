// Host-side planning of one GEMM call: which kernel, which tile, how many split-K parts, how many CTAs and how much
// scratch.  Plain C++ without CUDA so that the same code is used by the launcher (capi.cu) and exercised by CPU
// tests through gptb200_plan_gemm.
#pragma once

#include <algorithm>
#include <cstddef>

namespace gptb200 {

enum GemmKernelKind : int {
    KERNEL_NONE = 0,    // empty output: nothing to launch
    KERNEL_PAIR = 1,    // gemm_tcgen05_pair_kernel: CTA pairs, 256 x 256 tiles
    KERNEL_SINGLE = 2,  // gemm_tcgen05_kernel: one CTA per 128 x tile_n tile
    KERNEL_SKINNY = 3,  // skinny_gemm_kernel: weight streaming for m <= 64 (option: fewer)
    KERNEL_SIMT = 4,    // simt_gemm_kernel: shapes TMA cannot address
};

struct GemmPlanInput {
    int M, N, K;             // D[M x N] = A[M x K] . B[K x N]
    bool a_mn, b_mn;         // operand stored with the free index contiguous
    bool has_epilogue;       // bias and / or GELU output: split-K is not possible
    bool accumulate;         // out += result
    bool aligned;            // base pointers 16-byte aligned
    int num_sms;
    int opt_tile_n;          // 0 automatic, 128, 256
    int opt_max_splits;      // 0 automatic
    int opt_pair;            // 1 always, 0 heuristic, -1 never
    int opt_stream_k;        // CTA-pair kernel: 1 always cut ranges inside tiles, 0 heuristic, -1 whole tiles only
    bool opt_skinny;
    int opt_skinny_rows;     // most rows the weight-streaming kernel takes; 0 = kPlanSkinnyMaxRows
    size_t ws_limit;         // scratch limit in bytes
};

struct GemmPlan {
    int kernel;
    int tile_n;
    int tiles_m, tiles_n;    // 128-row tiles, tile_n-column tiles
    int splits, kb_per_split, num_kb;
    int grid;                // CTAs
    size_t workspace_bytes;  // split-K partial tiles, skinny partial sums, or one partial tile per CTA pair
    // CTA-pair kernel: the k-blocks of all tiles, tile after tile, are cut into `grid / 2` contiguous ranges at multiples
    // of sk_unit k-blocks (num_kb: whole tiles; 1: anywhere, tiles cut by a range boundary are summed through scratch).
    long long sk_total;
    int sk_unit;
    int sk_max_share;        // largest number of pairs that work on one tile
};

constexpr size_t kPairSlotBytes = 256 * 256 * sizeof(float);

constexpr int kPlanBM = 128;
constexpr int kPlanBK = 32;
constexpr int kPlanSkinnyMaxRows = 64;   // beyond this the fp32 FMAs of the weight-streaming kernel cost more than a tensor-core tile

// `units`: number of CTAs (or CTA pairs) that run concurrently
inline int plan_splits(const GemmPlanInput &in, long long tiles, int num_kb, bool allowed, size_t bytes_per_split, int units)
{
    if (!allowed) return 1;
    int cap = in.opt_max_splits > 0 ? in.opt_max_splits : 16;
    cap = std::min(cap, std::max(1, num_kb / 8));  // at least 8 k-blocks per split
    if (bytes_per_split > 0) cap = static_cast<int>(std::min<size_t>(cap, std::max<size_t>(1, (in.ws_limit / 2) / bytes_per_split)));
    if (in.opt_max_splits > 0) return std::max(1, cap);
    int best = 1;
    double best_eff = 0.0;
    for (int s = 1; s <= cap; ++s) {
        const long long items = tiles * s;
        const long long waves = (items + units - 1) / units;
        const double eff = double(items) / double(waves * units);
        if (eff > best_eff + 0.04) {  // take a larger split only for a real gain in SM occupancy
            best_eff = eff;
            best = s;
        }
    }
    return best;
}

// ---- decode-shaped calls (KERNEL_SKINNY): which of the weight-streaming kernels runs, and its launch shape ------------------
enum DecodeKernelKind : int {
    DECODE_KSPLIT = 0,        // skinny_gemm_kernel (+ finish): k split over CTAs, partial sums in scratch
    DECODE_WARP_CLUSTER = 1,  // decode_gemm_cluster_kernel: W [k][n], k split over warps and cluster CTAs
    DECODE_TILE_CLUSTER = 2,  // decode_tile_cluster_kernel: register-tiled, k split over a cluster
    DECODE_ROWWISE = 3,       // rowwise_gemv_kernel: W [n][k], a warp per pair of weight rows
};

struct DecodeOptions {
    int cluster = 16;        // largest cluster: 0 off, 1 .. 8, 16 = sixteen for narrow layers only, 32 = sixteen wherever k allows
    int cluster_rows = 8;    // most rows for the per-warp cluster kernel
    bool tile = true;        // register-tiled kernel beyond that
    int tile_rows = 0;       // its row tile beyond 32 rows: 0 / 64 = one tile of 64, 32 = row groups of 32
    bool rowwise = true;     // W [n][k]: warp-per-row kernel ...
    int rowwise_rows = 8;    // ... up to this many rows
    bool cluster16_ok = true;   // the device can schedule a cluster of 16 CTAs
};

struct DecodePlan {
    int kernel;     // DecodeKernelKind
    int rows;       // rows of x per CTA (per-warp kernel: MR; tiled kernel: TM; row-wise kernel: MR; k-split: MR)
    int groups;     // row groups (blockIdx.z, or blockIdx.x of the row-wise kernel)
    int cluster;    // CTAs per cluster (1 for the kernels without clusters)
};

constexpr int kPlanTileK = 32;   // k-rows per stage of the tiled kernel

// w_kn: W stored [k][n] (linear layers); else [n][k] (un-embedding, grad_x).  has_epilogue: bias and / or GELU output.
inline DecodePlan plan_decode(int M, int N, int K, bool w_kn, bool has_epilogue, int num_sms, const DecodeOptions &o)
{
    DecodePlan d{};
    int mr = 1;
    while (mr < M && mr < 16) mr *= 2;
    d.kernel = DECODE_KSPLIT;
    d.rows = mr;
    d.groups = (M + mr - 1) / mr;
    d.cluster = 1;
    const auto sixteen = [&](long long blocks, bool k_ok) {
        return o.cluster >= 16 && k_ok && (blocks * 16 <= num_sms || o.cluster >= 32) && o.cluster16_ok;
    };
    if (w_kn && o.cluster > 0 && M <= o.cluster_rows) {
        // largest cluster (power of two, at most the option) that leaves every warp at least four k-rows and does not put
        // more than ~four CTAs on each SM; the non-portable size 16 only for layers so narrow that clusters of eight would
        // occupy less than half of the SMs (n = 768: 48 CTAs)
        d.kernel = DECODE_WARP_CLUSTER;
        const long long blocks = 1LL * ((N + 127) / 128) * d.groups;
        while (d.cluster * 2 <= std::min(o.cluster, 8) && K / (d.cluster * 2 * 8) >= 4 && blocks * d.cluster * 2 <= 4LL * num_sms) d.cluster *= 2;
        if (d.cluster == 8 && sixteen(blocks, K / (16 * 8) >= 4)) d.cluster = 16;
        return d;
    }
    if (w_kn && o.tile && o.cluster > 0 && M > o.cluster_rows) {
        // as above, with at least one 32-row chunk of k per CTA.  Beyond 32 rows one 64-row tile: two row groups of 32 were
        // measured slower even where they double the number of busy SMs.
        d.kernel = DECODE_TILE_CLUSTER;
        const long long blocks = (N + 127) / 128;
        while (d.cluster * 2 <= std::min(o.cluster, 8) && K / (d.cluster * 2) >= kPlanTileK && blocks * d.cluster * 2 <= 2LL * num_sms) d.cluster *= 2;
        if (d.cluster == 8 && sixteen(blocks, K / 16 >= kPlanTileK)) d.cluster = 16;
        d.rows = M <= 16 ? 16 : (M <= 32 || o.tile_rows == 32) ? 32 : 64;
        d.groups = (M + d.rows - 1) / d.rows;
        return d;
    }
    if (!w_kn && o.rowwise && !has_epilogue && M <= o.rowwise_rows) {
        // groups of up to 16 rows of x (fewer when they exceed 48 KiB of shared memory); beyond one group the weights are
        // re-read from L2 once per group
        int rows = mr;
        while (rows > 1 && 1LL * rows * K > 12288) rows /= 2;
        if (1LL * rows * K <= 12288 && (rows >= 8 || rows == mr)) {
            d.kernel = DECODE_ROWWISE;
            d.rows = rows;
            d.groups = (M + rows - 1) / rows;
            return d;
        }
    }
    if (!w_kn && o.tile && o.cluster > 0 && !has_epilogue && M > o.rowwise_rows) {
        // W [n][k], more rows than the warp-per-row kernel takes: the tiled kernel; k is split over a cluster only when the
        // column tiles alone leave SMs idle
        d.kernel = DECODE_TILE_CLUSTER;
        const long long blocks = (N + 127) / 128;
        while (d.cluster * 2 <= std::min(o.cluster, 8) && K / (d.cluster * 2) >= 4 * kPlanTileK && blocks * d.cluster * 2 <= 2LL * num_sms) d.cluster *= 2;
        d.rows = M <= 16 ? 16 : M <= 32 ? 32 : 64;
        d.groups = 1;
        return d;
    }
    return d;
}

inline GemmPlan plan_gemm(const GemmPlanInput &in)
{
    GemmPlan p{};
    if (in.M <= 0 || in.N <= 0) return p;
    const bool fours = in.K % 4 == 0 && in.N % 4 == 0;
    // beyond 16 rows only for weight matrices of model size (small ones are launch-bound on any kernel)
    const int skinny_rows = in.opt_skinny_rows > 0 ? std::min(in.opt_skinny_rows, kPlanSkinnyMaxRows) : kPlanSkinnyMaxRows;
    if (in.opt_skinny && in.M <= skinny_rows && (in.M <= 16 || 1LL * in.K * in.N >= 512 * 512) && !in.a_mn && !in.accumulate && in.K >= 32 && fours && in.aligned) {
        p.kernel = KERNEL_SKINNY;
        const int cols_per_block = 128 * (in.b_mn ? 4 : 1);
        p.tiles_n = (in.N + cols_per_block - 1) / cols_per_block;
        p.tiles_m = (in.M + 15) / 16;   // row groups of up to 16 rows (blockIdx.z)
        // Enough CTAs for four per SM (two beyond 16 rows, where registers allow three and the partial sums are no longer
        // small against the weights), each with at least 32 k-rows (16 for up to four rows of x, where the partial sums are
        // tiny: a short weight matrix then still puts ~200 CTAs' loads in flight).
        const int blocks = p.tiles_n * p.tiles_m;
        const int want = in.num_sms * (in.M > 16 ? 2 : 4);
        int splits = std::max(1, std::min((want + blocks - 1) / blocks, in.K / (in.M <= 4 ? 16 : 32)));
        p.kb_per_split = (((in.K + splits - 1) / splits) + 3) & ~3;   // here: k ELEMENTS per split, a multiple of 4
        p.splits = (in.K + p.kb_per_split - 1) / p.kb_per_split;
        p.grid = blocks * p.splits;
        p.workspace_bytes = size_t(p.splits) * in.M * in.N * sizeof(float);
        return p;
    }
    const long long lda = in.a_mn ? in.M : in.K;
    const long long ldb = in.b_mn ? in.N : in.K;
    const bool tma_ok = in.K > 0 && in.aligned && lda % 4 == 0 && ldb % 4 == 0 && in.N % 4 == 0 && !(in.a_mn && !in.b_mn);
    if (!tma_ok) {
        p.kernel = KERNEL_SIMT;
        p.tiles_m = (in.M + 31) / 32;
        p.tiles_n = (in.N + 31) / 32;
        p.splits = 1;
        p.grid = p.tiles_m * p.tiles_n;
        return p;
    }
    // CTA pairs (256 x 256 tiles, cta_group::2): measured faster than one CTA per tile on every GPT-2 124M shape as long
    // as there are enough 256 x 256 work items to occupy most SM pairs; with fewer, 128-wide one-CTA tiles fill the
    // machine better.
    const long long pair_tiles = 1LL * ((in.M + 255) / 256) * ((in.N + 255) / 256);
    const bool split_allowed = !in.has_epilogue;
    const size_t bytes_per_split = size_t(in.M) * size_t(in.N) * sizeof(float);
    p.num_kb = (in.K + kPlanBK - 1) / kPlanBK;
    const int max_pairs = std::max(1, in.num_sms / 2);
    const long long pair_kb = pair_tiles * p.num_kb;
    // pairs that can be given at least eight k-blocks each
    const long long pairs_busy = std::min<long long>(max_pairs, std::max<long long>(pair_tiles, pair_kb / 8));
    bool pair = in.opt_pair > 0 || (in.opt_pair == 0 && in.opt_tile_n == 0 && in.M > kPlanBM && in.N > 128 && pairs_busy * 20 >= 9LL * in.num_sms);
    // Small problems (measured on the GPT-2 layer shapes at 1024 and 2048 rows, both precision modes): cutting tiles between
    // pairs costs a fixed 10 - 20 us per launch (a partner's partial tile is complete only at the end of its range, and the
    // owner's epilogue comes after it), which only a long main loop pays back.
    //   * one wave of 128 x 128 one-CTA tiles with at most 32 k-blocks each beats every CTA-pair plan (qkv forward at 1024 rows
    //     16.5 against 23.1 us in TF32 mode, 28.8 against 45.4 us in 3xTF32 mode);
    //   * when the pairs would outnumber the tiles four to one or more, every tile would be added up from four or more partial
    //     tiles by its one owner: split-K over one-CTA tiles with its parallel reduction kernel is faster (attention projection
    //     grad_w at 2048 rows 24.8 against 37.9 us, FFN-up grad_x at 1024 rows 18.9 against 30.9 us) -- where the epilogue
    //     allows split-K at all.
    const bool automatic = in.opt_pair == 0 && in.opt_tile_n == 0 && in.opt_stream_k == 0 && in.opt_max_splits == 0;
    const long long tiles128 = 1LL * ((in.M + kPlanBM - 1) / kPlanBM) * ((in.N + 127) / 128);
    bool force128 = false;
    if (pair && automatic) {
        const long long kb_each = std::max<long long>(1, pair_kb / pairs_busy);
        if (!in.accumulate && p.num_kb <= 32 && tiles128 <= in.num_sms) {
            pair = false;
            force128 = true;
        } else if (pair_tiles < max_pairs && p.num_kb >= 4 * kb_each && kb_each <= 16 && split_allowed) {
            pair = false;   // (with longer ranges the pair kernel's better main loop wins again: attention projection grad_w at 8192 rows)
        }
    }
    if (pair) {
        p.kernel = KERNEL_PAIR;
        p.tile_n = 256;
        p.tiles_m = (in.M + kPlanBM - 1) / kPlanBM;
        p.tiles_n = (in.N + 255) / 256;
        p.splits = 1;
        p.kb_per_split = p.num_kb;
        p.sk_total = pair_kb;
        const long long whole_pairs = std::min<long long>(max_pairs, pair_tiles);
        const long long rounds = (pair_tiles + whole_pairs - 1) / whole_pairs;
        const double whole_eff = double(pair_tiles) / double(rounds * pairs_busy);   // share of the usable pairs kept busy by whole tiles
        long long pairs;
        // Whole tiles per pair when they keep at least 97 % of the usable pairs busy -- or when the tiles are short (at most 32
        // k-blocks), fit one round and occupy at least half of the pairs: the main loop a cut would save is then shorter than the
        // cut's fixed cost (FFN-up forward at 1024 rows: 22.7 against 28.5 us in TF32 mode, 37.0 against 56.2 us in 3xTF32 mode).
        const bool short_single_round = automatic && pair_tiles <= max_pairs && p.num_kb <= 32 && 2 * pair_tiles >= max_pairs;
        if (in.opt_stream_k < 0 || (in.opt_stream_k == 0 && (whole_eff >= 0.97 || short_single_round))) {
            p.sk_unit = p.num_kb;   // whole tiles, as evenly as they go
            pairs = whole_pairs;
            p.sk_max_share = 1;
        } else {
            p.sk_unit = 1;
            pairs = in.opt_stream_k > 0 ? std::min<long long>(max_pairs, pair_kb) : pairs_busy;
            if (in.opt_stream_k == 0) {
                // Tiles that share an operand lie a fixed distance apart on the line of k-blocks: tiles_m2 * num_kb for the
                // rows of A, num_kb for the columns of B.  If the range length divides that distance (or is a multiple of
                // it), the pairs working on those tiles reach the same k-block of the shared operand at the same time and
                // it is fetched from DRAM once instead of once per tile (measured on the FFN step: 74 pairs x 124.5
                // k-blocks read grad_y three times, 72 x 128 once; + 3 % in spite of four idle SMs).  Up to 7 % of the
                // pairs are given up for that.
                const long long tiles_m2 = (in.M + 255) / 256, tiles_n = (in.N + 255) / 256;
                const long long dist_a = tiles_m2 * p.num_kb, dist_b = p.num_kb;
                double best = 0.0;
                for (long long cand = pairs_busy; cand >= 1 && cand * 100 >= pairs_busy * 93; --cand) {
                    if (pair_kb % cand != 0) continue;
                    const long long len = pair_kb / cand;
                    double score = 0.0;
                    if (tiles_n > 1 && dist_a % len == 0) score += double(in.M) * in.K * double(tiles_n - 1);
                    if (tiles_m2 > 1 && (dist_b % len == 0 || len % dist_b == 0)) score += double(in.K) * in.N * double(tiles_m2 - 1);
                    if (score > best) {
                        best = score;
                        pairs = cand;
                    }
                }
            }
            p.workspace_bytes = size_t(pairs) * kPairSlotBytes;
            p.sk_max_share = 1;
            long long cur_tile = -1;
            int cur = 0;
            for (long long q = 0; q < pairs; ++q) {   // ranges are in tile order: count those that meet the same tile
                const long long g0 = q * pair_kb / pairs, g1 = (q + 1) * pair_kb / pairs;
                if (g0 >= g1) continue;
                const long long t_first = g0 / p.num_kb, t_last = (g1 - 1) / p.num_kb;
                cur = t_first == cur_tile ? cur + 1 : 1;
                cur_tile = t_first;
                p.sk_max_share = std::max(p.sk_max_share, cur);
                if (t_last != t_first) {
                    cur_tile = t_last;
                    cur = 1;
                }
            }
            if (p.sk_max_share == 1) p.workspace_bytes = 0;   // every boundary fell between tiles
        }
        p.grid = 2 * static_cast<int>(pairs);
        return p;
    }
    int bn = in.opt_tile_n;
    if (bn != 128 && bn != 256) {
        const long long tiles256 = 1LL * ((in.M + kPlanBM - 1) / kPlanBM) * ((in.N + 255) / 256);
        bn = (force128 || in.N <= 128 || tiles256 < in.num_sms / 2) ? 128 : 256;
    }
    p.kernel = KERNEL_SINGLE;
    p.tile_n = bn;
    p.tiles_m = (in.M + kPlanBM - 1) / kPlanBM;
    p.tiles_n = (in.N + bn - 1) / bn;
    const long long tiles = 1LL * p.tiles_m * p.tiles_n;
    const int splits = plan_splits(in, tiles, p.num_kb, split_allowed, bytes_per_split, in.num_sms);
    p.kb_per_split = (p.num_kb + splits - 1) / splits;
    p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
    const long long items = tiles * p.splits;
    p.grid = static_cast<int>(std::min<long long>(items, in.num_sms));
    p.workspace_bytes = p.splits > 1 ? bytes_per_split * p.splits : 0;
    return p;
}

}  // namespace gptb200
