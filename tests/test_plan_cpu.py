"""CPU tests of the host-side launch planning (gpt_b200/csrc/gemm_plan.h through gptb200_plan_gemm): no GPU involved."""
import itertools

import pytest

SMS = 148


@pytest.fixture(scope="module")
def plan(built_library):
    import gpt_b200
    return gpt_b200.plan_gemm


def test_gpt2_124m_shapes_use_the_cta_pair_kernel_at_m_8192(plan):
    D, F, V = 768, 3072, 50304
    for k, n in ((D, 3 * D), (D, D), (D, F), (F, D)):
        fwd = plan(SMS, 8192, n, k, False, True, has_epilogue=True)
        assert fwd["kernel"] == "pair" and fwd["grid"] in (144, 146, 148)
        tiles = 32 * ((n + 255) // 256)
        assert fwd["k_per_split"] == -(-tiles * (k // 32) // (fwd["grid"] // 2))   # every pair gets its share of all k-blocks
        dx = plan(SMS, 8192, k, n, False, False)
        assert dx["kernel"] == "pair"
        dw = plan(SMS, k, n, 8192, True, True, accumulate=True)
        assert dw["kernel"] in ("pair", "single")
    assert plan(SMS, 8192, V, D, False, False)["kernel"] == "pair"           # LM head forward
    assert plan(SMS, V, D, 8192, True, True, accumulate=True)["splits"] == 1   # 1179 tiles: whole tiles keep the pairs busy
    fc = plan(SMS, 8192, F, D, False, True, has_epilogue=True)                 # 384 tiles on 74 pairs: 5.19 rounds of whole tiles
    assert fc["splits"] == 2 and fc["scratch_kib"] == fc["grid"] // 2 * 256    # ... so ranges are cut inside tiles
    # 9216 k-blocks: 72 pairs x 128 put the tiles that share rows of x (768 k-blocks apart on the line) in step; 74 x 124.5 do not
    assert fc["grid"] == 144 and fc["k_per_split"] == 128
    dx = plan(SMS, 8192, D, F, False, False)                                   # grad_x: tiles sharing grad_y are 3072 k-blocks apart
    assert dx["grid"] == 144 and dx["k_per_split"] == 128
    dw = plan(SMS, D, F, 8192, True, True, accumulate=True)                    # 36 tiles of 256 k-blocks
    assert dw["kernel"] == "pair" and dw["grid"] == 144 and dw["splits"] == 2


def test_small_problems_avoid_the_fixed_cost_of_cut_ranges(plan):
    """The GPT-2 layer shapes at 1024 and 2048 rows (the per-GPU shards of the data-parallel step): the choices measured
    fastest -- one wave of 128 x 128 one-CTA tiles, split-K instead of tiles added up from four or more partial tiles, whole
    tiles when they are short and fit one round -- and cut ranges where the main loop is long enough to pay for them."""
    D, F = 768, 3072
    # one wave of 128 x 128 tiles, at most 32 k-blocks: qkv forward at 1024 rows (144 tiles), attention projection at 2048 rows (96)
    for m, n in ((1024, 3 * D), (2048, D)):
        p = plan(SMS, m, n, D, False, True, has_epilogue=True)
        assert p["kernel"] == "single" and p["tile_n"] == 128 and p["splits"] == 1
    assert plan(SMS, 2048, D, D, False, False)["kernel"] == "single"           # ... and its grad_x
    # the pairs would outnumber the tiles four to one: split-K over one-CTA tiles
    dx = plan(SMS, 1024, D, F, False, False)                                   # FFN-up grad_x at 1024 rows: 12 pair tiles of 96 k-blocks
    assert dx["kernel"] == "single" and dx["splits"] > 1
    dw = plan(SMS, D, D, 2048, True, True, accumulate=True)                    # attention projection grad_w at 2048 rows: 9 pair tiles
    assert dw["kernel"] == "single" and dw["splits"] > 1
    # ... but not where the epilogue rules split-K out: FFN-down forward keeps the cut ranges
    down = plan(SMS, 1024, D, F, False, True, has_epilogue=True)
    assert down["kernel"] == "pair" and down["splits"] >= 2
    # short tiles that fit one round and occupy more than half of the pairs: whole tiles
    up = plan(SMS, 1024, F, D, False, True, has_epilogue=True)                 # 48 tiles of 24 k-blocks on 74 pairs
    assert up["kernel"] == "pair" and up["splits"] == 1 and up["grid"] == 96 and up["scratch_kib"] == 0
    # long main loops still get equal ranges: FFN-up forward at 2048 rows (96 tiles), grad_w at 1024 rows (36 tiles of 32 k-blocks)
    assert plan(SMS, 2048, F, D, False, True, has_epilogue=True)["splits"] >= 2
    assert plan(SMS, D, F, 1024, True, True, accumulate=True)["kernel"] == "pair"
    assert plan(SMS, D, D, 8192, True, True, accumulate=True)["kernel"] == "pair"   # 9 tiles, but 32 k-blocks per pair: worth cutting


def test_small_and_odd_shapes(plan):
    assert plan(SMS, 64, 96, 32, False, True, True)["kernel"] == "single"      # the reference's test shapes: ragged tiles
    assert plan(SMS, 64, 32, 256, False, True, True)["grid"] == 1
    assert plan(SMS, 8, 3072, 768, False, True, True)["kernel"] == "skinny"    # decode-shaped
    assert plan(SMS, 1, 50304, 768, False, False)["kernel"] == "skinny"
    p64 = plan(SMS, 64, 2304, 768, False, True, True)                          # batch 64: four row groups of 16
    assert p64["kernel"] == "skinny" and p64["tiles_m"] == 4 and p64["grid"] == 4 * p64["tiles_n"] * p64["splits"]
    assert plan(SMS, 65, 2304, 768, False, True, True)["kernel"] != "skinny"
    assert plan(SMS, 16, 768, 768, True, True, False, True)["kernel"] != "skinny"   # weight gradients never stream
    assert plan(SMS, 77, 50, 30, False, True, True)["kernel"] == "simt"        # row pitch not a multiple of 16 bytes
    assert plan(SMS, 5, 9, 7, False, True, True)["kernel"] == "simt"
    assert plan(SMS, 0, 128, 64, False, True, True)["kernel"] == "none"
    assert plan(SMS, 128, 128, 0, False, True, True)["kernel"] == "simt"       # k == 0: y = bias


@pytest.mark.parametrize("sms", [148, 132, 16])
def test_plan_invariants_over_a_sweep(plan, sms):
    dims_m = [1, 17, 128, 129, 256, 1000, 2048, 8192, 32768]
    dims_nk = [32, 96, 128, 260, 768, 2304, 3072, 50304]
    for m, n, k in itertools.product(dims_m, dims_nk, dims_nk):
        if m * n >= 2 ** 31 or m * k >= 2 ** 31:
            continue
        for a_mn, b_mn, epi, acc in ((False, True, True, False), (False, False, False, False), (True, True, False, True)):
            p = plan(sms, m, n, k, a_mn, b_mn, epi, acc)
            assert p["grid"] >= 1
            if p["kernel"] == "pair":
                pairs = p["grid"] // 2
                tiles = ((m + 255) // 256) * ((n + 255) // 256)
                num_kb = (k + 31) // 32
                assert p["grid"] % 2 == 0 and p["grid"] <= sms and p["tile_n"] == 256 and m > 128
                assert pairs * p["k_per_split"] >= tiles * num_kb               # the ranges cover every k-block of every tile
                assert tiles * num_kb >= pairs                                  # and no pair is left without work
                if p["splits"] == 1:
                    assert p["scratch_kib"] == 0
                else:
                    assert p["scratch_kib"] == pairs * 256                      # one 256 x 256 partial tile per pair
                    assert tiles * num_kb // pairs >= 8 or pairs <= tiles       # pairs beyond one per tile get eight k-blocks or more
            if p["kernel"] == "single":
                assert p["grid"] <= sms
                num_kb = (k + 31) // 32
                assert p["splits"] >= 1 and p["k_per_split"] >= 1
                assert p["splits"] * p["k_per_split"] >= num_kb                  # the splits cover all of k
                assert (p["splits"] - 1) * p["k_per_split"] < num_kb             # and none of them is empty
                if epi:
                    assert p["splits"] == 1                                     # bias / GELU epilogues cannot be split
                if p["splits"] > 1:
                    assert p["scratch_kib"] * 1024 >= p["splits"] * m * n * 4 - 1023
                    assert p["scratch_kib"] <= 1 << 20                          # scratch limit of 1 GiB
                    assert p["k_per_split"] >= 8                                # at least eight k-blocks per split
                else:
                    assert p["scratch_kib"] == 0
                assert p["tile_n"] in (128, 256)
            if p["kernel"] == "skinny":
                assert m <= 64 and p["tiles_m"] == (m + 15) // 16 and not acc and p["splits"] * p["k_per_split"] >= k and p["k_per_split"] % 4 == 0


def test_decode_kernel_choice_for_gpt2_124m():
    """Which weight-streaming kernel a decode-shaped call runs (gptb200_plan_decode, default options)."""
    import gpt_b200
    D, F, V = 768, 3072, 50304
    pd = lambda *a, **k: gpt_b200.plan_decode(SMS, *a, **k)
    # batch 1 / 8: per-warp cluster kernel, clusters of 8, and 16 for the 768-wide layers (48 CTAs otherwise)
    for m in (1, 8):
        rows = m
        assert pd(m, 3 * D, D, True, True) == dict(kernel="warp_cluster", rows=rows, groups=1, cluster=8)
        assert pd(m, D, D, True, True) == dict(kernel="warp_cluster", rows=rows, groups=1, cluster=16)
        assert pd(m, F, D, True, True) == dict(kernel="warp_cluster", rows=rows, groups=1, cluster=8)
        assert pd(m, D, F, True, True) == dict(kernel="warp_cluster", rows=rows, groups=1, cluster=16)
        assert pd(m, V, D, False) == dict(kernel="rowwise", rows=rows, groups=1, cluster=1)      # un-embedding
    assert pd(3, D, D, True)["rows"] == 4 and pd(5, D, D, True)["rows"] == 8                     # next power of two
    # 9 .. 64 rows: register-tiled kernel, 16 / 32 / 64-row tiles, k over a cluster
    assert pd(9, 3 * D, D, True, True) == dict(kernel="tile_cluster", rows=16, groups=1, cluster=8)
    assert pd(32, D, F, True, True) == dict(kernel="tile_cluster", rows=32, groups=1, cluster=16)
    assert pd(64, F, D, True, True) == dict(kernel="tile_cluster", rows=64, groups=1, cluster=8)  # 24 column tiles x 8 = 192 CTAs
    assert pd(64, V, D, False) == dict(kernel="tile_cluster", rows=64, groups=1, cluster=1)      # 393 column tiles fill the GPU
    assert pd(40, D, 3 * D, False)["kernel"] == "tile_cluster"                                    # grad_x of the QKV layer
    # k too short to split: one CTA per column tile
    assert pd(2, 132, 36, True)["cluster"] == 1 and pd(12, 260, 36, True)["cluster"] == 1
    # [n][k] weights with bias never take the bias-free kernels
    assert pd(4, D, D, False, True)["kernel"] == "k_split"
    # x too large for the row-wise kernel's shared memory: k-split kernel
    assert pd(8, D, F, False)["kernel"] == "k_split"
    for m, n, k, w_kn in itertools.product((1, 2, 7, 8, 9, 16, 33, 64), (132, 768, 50304), (36, 768, 3072), (True, False)):
        p = pd(m, n, k, w_kn)
        assert p["rows"] * p["groups"] >= m and p["cluster"] in (1, 2, 4, 8, 16)
        if p["kernel"] == "warp_cluster":
            assert k // (p["cluster"] * 8) >= 4 or p["cluster"] == 1
        if p["kernel"] == "tile_cluster":
            assert k // p["cluster"] >= 32 or p["cluster"] == 1
        if p["kernel"] == "rowwise":
            assert p["rows"] * k <= 12288
