"""CPU tests (gloo, world_size 2) of the data-parallel gradient exchange plan: the bucket slices produced by
gpt_b200.data_parallel.GradientBuckets cover every gradient element exactly once, in the order the backward
pass finishes them, and reducing them slice by slice gives the same result as one all-reduce of the buffer."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gpt_b200.data_parallel import GradientBuckets, LAYER_KINDS, per_layer_sizes

TINY = dict(max_seq_len=64, vocab_size=507, vocab_size_padded=512, num_layers=4, num_heads=4, d_model=32, d_ffn=256)
GPT2 = dict(max_seq_len=256, vocab_size=50257, vocab_size_padded=50304, num_layers=12, num_heads=12, d_model=768, d_ffn=3072)
NAMES = ["wte", "wpe", "ln_1_w", "ln_1_b", "qkv_proj_w", "qkv_proj_b", "attn_proj_w", "attn_proj_b", "ln_2_w", "ln_2_b",
         "ffn_up_w", "ffn_up_b", "ffn_down_w", "ffn_down_b", "ln_f_w", "ln_f_b"]


def offsets(cfg):
    """Packing of the reference (src/model/gpt.cpp:46-62): kind-major, all layers of a kind contiguous."""
    L, D = cfg["num_layers"], cfg["d_model"]
    s = per_layer_sizes(cfg)
    sizes = {"wte": cfg["vocab_size_padded"] * D, "wpe": cfg["max_seq_len"] * D, "ln_f_w": D, "ln_f_b": D}
    sizes.update({k: L * s[k] for k in LAYER_KINDS})
    off, o = {}, 0
    for n in NAMES:
        off[n] = o
        o += sizes[n]
    return off, o


@pytest.mark.parametrize("cfg,total", [(TINY, 102592), (GPT2, 123886080)])
@pytest.mark.parametrize("group", [1, 3, 4, 5, 12])
def test_slices_cover_every_element_exactly_once(cfg, total, group):
    off, n = offsets(cfg)
    assert n == total
    b = GradientBuckets(cfg, off, n, group)
    cover = np.zeros(n, np.int8) if n < 10**6 else None
    spans = sorted(b.all_slices())
    pos = 0
    for o, c in spans:          # sorted spans tile [0, n) without gap or overlap
        assert o == pos and c > 0
        pos = o + c
        if cover is not None:
            cover[o:o + c] += 1
    assert pos == n
    if cover is not None:
        assert (cover == 1).all()


def test_a_slice_is_released_only_when_its_layers_are_done():
    off, n = offsets(GPT2)
    b = GradientBuckets(GPT2, off, n, 3)
    s = per_layer_sizes(GPT2)
    done = set()
    for ev in [12] + list(range(11, -2, -1)):
        if 0 <= ev < 12:
            done.add(ev)
        for o, c in b.ready_after(ev):
            for k in LAYER_KINDS:
                if off[k] <= o < off[k] + 12 * s[k]:
                    first = (o - off[k]) // s[k]
                    assert set(range(first, first + c // s[k])) <= done
    assert b.ready_after(12) == [(off["ln_f_w"], 2 * 768)]
    assert b.ready_after(-1) == [(0, off["ln_1_w"])]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    off, n = offsets(TINY)
    b = GradientBuckets(TINY, off, n, 3)
    g = torch.Generator().manual_seed(100 + rank)
    local = torch.randn(n, generator=g)
    whole = local.clone()
    dist.all_reduce(whole)
    whole /= world
    sliced = local.clone()
    calls = 0
    for ev in [4, 3, 2, 1, 0, -1]:      # the order in which the backward pass reports layers
        for o, c in b.ready_after(ev):
            view = sliced[o:o + c]
            dist.all_reduce(view)
            view /= world
            calls += 1
    q.put((rank, bool(torch.equal(whole, sliced)), calls))
    dist.destroy_process_group()


def test_bucketed_allreduce_equals_whole_buffer_allreduce_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in res)
    assert all(calls == 2 + 2 * 12 for _, _, calls in res)   # ln_f, two layer groups x 12 kinds, embeddings
