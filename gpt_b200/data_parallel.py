"""Data-parallel training step: one process per GPU, the batch (whole sequences) sharded over ranks, weight
gradients summed with NCCL over NVLink / NVSwitch while the rest of the backward pass still runs.

The reference has no multi-GPU path (single process, single stream).  The only place where tokens interact in
the linear path is the reduction over tokens in grad_w / grad_b / grad_wte, so data parallelism needs exactly
one exchange step: an all-reduce of the packed gradient buffer (src/model/gpt.cpp:46-62 packs sixteen tensors
kind-major, every kind holding all layers contiguously).

GradientBuckets turns "layer l is done" events of the backward pass into contiguous slices of that buffer that
are ready to be reduced: layers are grouped (default 3 per group), and when the lowest layer of a group
completes, each of the twelve per-layer kinds contributes one contiguous slice covering the group.  wte, wpe and
the final LayerNorm go last (wte also receives the embedding backward at the very end).  The plan is pure
index arithmetic and is tested on CPU with the gloo backend.

The early form (`early_wte`, the default on GPUs): wte is the largest gradient tensor (154 MB of 494 MB for GPT-2 124M) and
would otherwise be reduced after the whole pass, with nothing left to overlap it.  Its two contributions are the
un-embedding backward at the START of the pass (dense) and the embedding backward at the END (one row per token).  The
backward pass therefore stops before the embedding backward; wte / wpe are reduced together with the final LayerNorm right
after the un-embedding backward; at the end the ranks all-gather the embedding backward's inputs (every rank's rows of the
residual-stream gradient and its tokens: 50 MB in all) and each applies all of them with weight 1 / ranks.
"""
from __future__ import annotations

from typing import Callable

LAYER_KINDS = ["ln_1_w", "ln_1_b", "qkv_proj_w", "qkv_proj_b", "attn_proj_w", "attn_proj_b", "ln_2_w", "ln_2_b",
               "ffn_up_w", "ffn_up_b", "ffn_down_w", "ffn_down_b"]


def per_layer_sizes(cfg: dict) -> dict:
    D, F = cfg["d_model"], cfg["d_ffn"]
    return {"ln_1_w": D, "ln_1_b": D, "qkv_proj_w": D * 3 * D, "qkv_proj_b": 3 * D, "attn_proj_w": D * D, "attn_proj_b": D,
            "ln_2_w": D, "ln_2_b": D, "ffn_up_w": D * F, "ffn_up_b": F, "ffn_down_w": F * D, "ffn_down_b": D}


class GradientBuckets:
    """Maps backward-pass events to (offset, count) slices of the packed gradient buffer that became final."""

    def __init__(self, cfg: dict, param_offsets: dict, num_params: int, layers_per_group: int = 3):
        self.cfg = cfg
        self.off = param_offsets
        self.num_params = num_params
        self.L = cfg["num_layers"]
        self.group = max(1, min(layers_per_group, self.L))
        self.sizes = per_layer_sizes(cfg)

    def ready_after(self, event: int, early_wte: bool = False) -> list[tuple[int, int]]:
        """event: the layer index reported by the backward pass (L, L-1, ..., 0, -1).  early_wte: the embedding backward is
        applied after the reduction (see the module text), so wte / wpe are ready with the final LayerNorm."""
        L, D = self.L, self.cfg["d_model"]
        emb = (self.off["wte"], self.off["ln_1_w"] - self.off["wte"])   # wte and wpe are adjacent at the start of the buffer
        if event == L:      # un-embedding + final LayerNorm done: ln_f_w, ln_f_b are adjacent at the end of the buffer
            return [(self.off["ln_f_w"], 2 * D)] + ([emb] if early_wte else [])
        if event == -1:     # embedding backward done
            return [] if early_wte else [emb]
        if event % self.group != 0:
            return []
        hi = min(event + self.group, L)  # layers [event, hi) are complete
        return [(self.off[k] + event * self.sizes[k], (hi - event) * self.sizes[k]) for k in LAYER_KINDS]

    def all_slices(self) -> list[tuple[int, int]]:
        out = []
        for ev in [self.L] + list(range(self.L - 1, -2, -1)):
            out += self.ready_after(ev)
        return out


class DataParallelStep:
    """Runs zero_grad / forward / backward on the local shard and all-reduces gradients bucket by bucket.

    `model` is a gpt_b200.Model whose context uses `compute_stream`; `grad_tensor` is a torch view of its packed
    gradient buffer.  Collectives are issued on `comm_stream` behind events recorded on the compute stream, so
    they overlap the remaining backward kernels.  Gradients are averaged over ranks: every rank's cross-entropy
    backward divides by its local token count, so the mean over ranks equals the single-GPU gradient of the
    global batch.

    With a host tensor as `grad_tensor` (no CUDA: the gloo tests) the same sequence runs without streams: each bucket is
    reduced synchronously when its layers are reported done.
    """

    def __init__(self, model, grad_tensor, world_size: int, layers_per_group: int = 3, all_reduce: Callable | None = None,
                 comm_sms: int | None = None, early_wte: bool | None = None):
        import torch
        import torch.distributed as dist
        self.torch = torch
        self.dist = dist
        self.model = model
        self.grads = grad_tensor
        self.world = world_size
        self.buckets = GradientBuckets(model.config, model.param_offsets, model.num_params, layers_per_group)
        self.on_gpu = bool(getattr(grad_tensor, "is_cuda", False))
        self.compute_stream = torch.cuda.current_stream() if self.on_gpu else None
        # Collectives are enqueued from this stream.  Which stream NCCL's kernels run on, and its priority, is decided by the
        # process group (ProcessGroupNCCL.Options(is_high_priority_stream=True) at init_process_group), not by this stream's
        # priority; this stream only carries the ordering (event wait before, wait_stream after).
        self.comm_stream = torch.cuda.Stream(priority=-1) if (world_size > 1 and self.on_gpu) else None
        self._all_reduce = all_reduce or (lambda t: dist.all_reduce(t, op=dist.ReduceOp.AVG))
        self.collectives = 0
        # While collectives are in flight the persistent GEMM kernels can leave `comm_sms` SMs free: NCCL's CTAs otherwise wait for
        # a GEMM CTA to finish, and the GEMM's equal k-block ranges assume that all of its CTAs run at once.  That pays when one
        # collective overlaps one GEMM (the FFN micro-step: 0.55 ms per step with all SMs claimed, 0.50 ms with 16 left free at 2
        # GPUs); in the whole training step, where dozens of kernels pass while a bucket is reduced, it does not.
        if comm_sms is None:
            comm_sms = 0   # measured on the training step at 2 and 4 GPUs: ceding 16 or 32 SMs costs more GEMM time than NCCL's waiting CTAs do
        self.comm_sms = comm_sms if world_size > 1 else 0
        self._sms_limited = False
        # early reduction of wte (module text): needs the model driver's hooks and device tensors
        if early_wte is None:
            early_wte = True
        self.early_wte = bool(early_wte and world_size > 1 and self.on_gpu and hasattr(model, "defer_embedding_backward"))
        if self.early_wte:
            model.defer_embedding_backward(True)
        self._gather_rows = self._gather_tokens = None
        self._coalesce = all_reduce is None and hasattr(dist, "_coalescing_manager")

    def _limit_sms(self, on: bool) -> None:
        if not self.on_gpu or self.comm_sms <= 0 or on == self._sms_limited or not hasattr(self.model, "set_option"):
            return
        num_sms = self.torch.cuda.get_device_properties(self.torch.cuda.current_device()).multi_processor_count
        self.model.set_option("max_sms", max(2, num_sms - self.comm_sms) if on else 0)
        self._sms_limited = on

    def _on_layer_done(self, layer: int) -> None:
        slices = self.buckets.ready_after(layer, self.early_wte)
        if not slices or self.world == 1:
            return
        if not self.on_gpu:
            for off, n in slices:
                self._all_reduce(self.grads[off:off + n])
                self.collectives += 1
            return
        self._limit_sms(True)
        ev = self.torch.cuda.Event()
        ev.record(self.compute_stream)
        with self.torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ev)
            self._reduce_slices(slices)

    def _reduce_slices(self, slices) -> None:
        """All slices of one event as ONE NCCL group (one kernel, one host call) where torch offers it."""
        views = [self.grads[off:off + n] for off, n in slices]
        if self._coalesce and len(views) > 1:
            try:
                with self.dist._coalescing_manager(device=self.grads.device, async_ops=False):
                    for v in views:
                        self._all_reduce(v)
                self.collectives += 1
                return
            except Exception:
                self._coalesce = False       # this torch has no such manager: one call per slice from now on
        for v in views:
            self._all_reduce(v)
            self.collectives += 1

    def _apply_embedding_rows(self, tokens) -> None:
        """End of a pass in the early form: gather every rank's embedding-backward inputs, apply them all."""
        torch, m = self.torch, self.model
        B, T = tokens.shape
        D = m.config["d_model"]
        if self._gather_rows is None or self._gather_rows.shape[1] != B * T * D:
            self._gather_rows = torch.empty(self.world, B * T * D, device=tokens.device, dtype=torch.float32)
            self._gather_tokens = torch.empty(self.world, B * T, device=tokens.device, dtype=torch.int32)

        class _Raw:   # the model's gradient of the embedding output, in place
            __cuda_array_interface__ = dict(shape=(B * T * D,), typestr="<f4", data=(m.embedding_grad_ptr, False), version=3, strides=None)
        rows = torch.as_tensor(_Raw(), device=tokens.device)
        ev = torch.cuda.Event()
        ev.record(self.compute_stream)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ev)
            self.dist.all_gather_into_tensor(self._gather_rows.view(-1), rows)
            self.dist.all_gather_into_tensor(self._gather_tokens.view(-1), tokens.reshape(-1).to(torch.int32))
            self.collectives += 2
        self.compute_stream.wait_stream(self.comm_stream)      # also: the reduction of wte / wpe has finished
        for r in range(self.world):
            m.apply_embedding_grad(self._gather_rows[r], self._gather_tokens[r], B, T, 1.0 / self.world)

    def step(self, tokens, labels) -> None:
        m = self.model
        m.zero_grad()
        m.forward(tokens)
        m.backward(tokens, labels, self._on_layer_done)
        self.finish(tokens)

    def finish(self, tokens) -> None:
        """After the backward pass: the compute stream waits for the collectives (and, in the early form, applies the gathered
        embedding-backward rows); afterwards every rank holds the averaged gradients."""
        self._limit_sms(False)
        if self.early_wte:
            self._apply_embedding_rows(tokens)
        elif self.world > 1 and self.on_gpu:
            self.compute_stream.wait_stream(self.comm_stream)
