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


class _FakeModel:
    """Stands in for gpt_b200.Model on the host: its 'gradient' of a batch is the mean over the batch's tokens of a fixed
    pseudo-random vector per token id, written into the packed buffer in the order the real backward pass finishes tensors
    (un-embedding part of wte and the final LayerNorm first, layers from the last to the first, then the embedding part of
    wte - an accumulation into what the un-embedding left there - and wpe), reporting each event through the callback."""

    def __init__(self, cfg):
        self.config = cfg
        self.param_offsets, self.num_params = offsets(cfg)
        self.grads = torch.zeros(self.num_params)

    def _token_grad(self, tokens):
        idx = torch.arange(self.num_params, dtype=torch.float64)
        g = torch.zeros(self.num_params, dtype=torch.float64)
        for t in tokens.flatten().tolist():
            g += torch.sin(idx * 1e-3 * (t + 1)) + 0.01 * t
        return (g / tokens.numel()).float()

    def zero_grad(self):
        self.grads.zero_()

    def forward(self, tokens):
        pass

    def backward(self, tokens, labels, layer_done):
        cfg, off = self.config, self.param_offsets
        L, D = cfg["num_layers"], cfg["d_model"]
        g = self._token_grad(tokens)
        s = per_layer_sizes(cfg)
        n_wte = cfg["vocab_size_padded"] * D
        self.grads[off["wte"]:off["wte"] + n_wte] += 0.25 * g[off["wte"]:off["wte"] + n_wte]      # un-embedding backward
        self.grads[off["ln_f_w"]:off["ln_f_w"] + 2 * D] = g[off["ln_f_w"]:off["ln_f_w"] + 2 * D]
        layer_done(L)
        for l in range(L - 1, -1, -1):
            for k in LAYER_KINDS:
                a = off[k] + l * s[k]
                self.grads[a:a + s[k]] = g[a:a + s[k]]
            layer_done(l)
        self.grads[off["wte"]:off["wte"] + n_wte] += 0.75 * g[off["wte"]:off["wte"] + n_wte]      # embedding backward, at the very end
        a, b = off["wpe"], off["ln_1_w"]
        self.grads[a:b] = g[a:b]
        layer_done(-1)


def _dp_worker(rank, world, port, q):
    from gpt_b200.data_parallel import DataParallelStep
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(7)
    tokens = torch.randint(0, TINY["vocab_size"], (4, 16), generator=g)       # the global batch: four sequences
    model = _FakeModel(TINY)

    def avg(t):
        dist.all_reduce(t)
        t /= world

    dp = DataParallelStep(model, model.grads, world, layers_per_group=3, all_reduce=avg)
    per = tokens.shape[0] // world
    for _ in range(2):                                                        # two steps: zero_grad starts each from zero
        dp.step(tokens[rank * per:(rank + 1) * per], None)
    whole = _FakeModel(TINY)
    whole.zero_grad()
    whole.backward(tokens, None, lambda l: None)                              # single process, whole batch
    err = float((model.grads - whole.grads).abs().max())
    q.put((rank, err, dp.collectives))
    dist.destroy_process_group()


def test_data_parallel_step_gives_the_gradient_of_the_global_batch_gloo():
    """DataParallelStep on two gloo ranks, each with half of the sequences: after the step every rank holds the gradient a single
    process computes on the whole batch - which also requires every bucket to be reduced only after its last write (wte after
    the embedding backward)."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, err, calls in res:
        assert err <= 2e-6
        assert calls == 2 * (2 + 2 * 12)      # per step: ln_f, two layer groups x 12 kinds, embeddings
