#!/usr/bin/env python
"""Benchmark of the linear-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--mode 3xtf32|tf32] [--impl ours|reference]

Workload (BASELINE.json configs[1]): one GPT-2 124M FFN fc layer at M = 8192 tokens per GPU --
x [8192 x 768], w [768 x 3072], bias, GELU-tanh -- forward, then backward (grad_x, grad_w +=, grad_b +=) with an
upstream gradient [8192 x 3072].  One step = forward + backward = 6*M*K*N algorithmic flops.  Synthetic
N(0,1) / N(0,0.02) data, seeded.  The step's buffers rotate through 4 sets (about 1.5 GB, larger than the
126 MB L2) so no step finds its inputs in cache.

N > 1 (launched by torch.distributed.run, one rank per GPU): the batch (M) is sharded, every rank runs the same
per-GPU workload (weak scaling) and the weight gradients (grad_w, grad_b) are all-reduced with NCCL inside the
timed region, as in a data-parallel training step.

`value` is timed with CUDA events on the launching stream, inputs resident in HBM, max over ranks.  `e2e` is
the same step through the C ABI starting from pinned HOST buffers: x and the upstream gradient are copied to
the device, and act / grad_x / grad_w / grad_b are copied back, inside the timed region; consecutive steps are
pipelined over a copy-in, a compute and a copy-out stream with two buffer sets.

Beside those headline keys the default line carries sub-records, each a few hundred milliseconds of GPU time:
  shapes         (N = 1) every linear layer of GPT-2 124M at M = 8192 -- QKV, attention projection, FFN up, FFN down, the tied
                 LM head -- and FFN up at M = 1024 and 32768: forward / backward ms, TFLOP/s and fraction of the TF32 peak, in
                 both precision modes;
  reference_gpu  (N = 1) the reference's own CUDA backend (cuBLAS TF32 + its unfused kernels, unmodified sources) on the same
                 shapes and on the training step, run in a child process so that cuBLAS never enters this one;
  decode         (N = 1) the linear layers of a decode step at batch 1 / 8 / 64: GB/s of weight stream and fraction of HBM peak;
  generate       (N = 1) generation of 192 tokens after a 64-token prompt at batch 1 / 8 / 64: tokens/s with the KV cache and
                 in the reference's form (the whole prefix recomputed per token);
  attention      (N = 1) causal attention of one layer at 64 x 256 tokens, forward and backward, in both modes: the batched tensor-core
                 products + row kernels against the fp32 FMA kernels;
  train_step     (every N) the full GPT-2 124M training step at a global batch of 64 x 256 tokens sharded over the ranks
                 (strong scaling): tokens/s, phase times, collectives per step, and dp_parity -- the distance per gradient
                 tensor between the all-reduced N-rank gradients and rank 0 computing the whole batch alone;
  train_step_tf32 (every N) the same step with the linear layers in single-pass TF32 (the precision of the reference's CUDA
                 backend, whose step reference_gpu times) and attention as batched tensor-core products.

--impl reference times the reference's own CPU implementation (unmodified sources, oracle/_ref) of the same
step on the host, on a bounded row sample per step (its cost is exactly linear in M).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_PER_GPU, K_IN, N_OUT = 8192, 768, 3072
FLOPS_PER_STEP = 6.0 * M_PER_GPU * K_IN * N_OUT          # forward + dX + dW, 2*M*K*N each
# DRAM read + write bytes per launch (or per step) from ncu captures of these workloads (dram__bytes_read.sum +
# dram__bytes_write.sum); re-captured whenever the kernel they describe changes.
NCU_DRAM_BYTES = {"ffn_up_forward_M8192_3xtf32": 211.4e6, "ffn_up_forward_M8192_tf32": 206.0e6, "decode_step_batch1": 496.4e6}
METRIC = "linear_layer_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "GPT-2 124M FFN fc (x[8192x768].w[768x3072]+b, GELU-tanh) forward+backward per GPU"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        # TF32 tensor rate is half the bf16 rate; the driver measures bf16 with cuBLAS.
        return dict(tf32_tflops=p["bf16_tflops"] / 2.0, tf32_tflops_sustained=p["bf16_tflops_sustained"] / 2.0, hbm_gbs=p["hbm_gbs"],
                    source="of measured (MEASURED_PEAKS.json bf16 cuBLAS burst / 2: TF32 issues at half the bf16 rate)")
    return dict(tf32_tflops=1590.0 / 2.0, tf32_tflops_sustained=1400.0 / 2.0, hbm_gbs=6650.0,
                source="of fallback (1.59 PFLOP/s bf16 / 2)")


class ClockSampler:
    """Samples nvidia-smi during the timed region (read-only query)."""
    Q = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.path = None
        self.gpu = gpu_index
        exe = shutil.which("nvidia-smi")
        if exe:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen([exe, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(gpu_index)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)

    def stop(self, t_begin: float, t_end: float):
        """Ends the sampling; summary of the samples taken between the two time.time() stamps."""
        out = self.summary(t_begin, t_end)
        self.close()
        return out

    def close(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.proc = None
        if self.path and os.path.exists(self.path):
            os.unlink(self.path)

    def summary(self, t_begin: float, t_end: float):
        """Summary of the samples taken so far between the two time.time() stamps (sampling goes on)."""
        if not self.proc:
            return None
        sm, smax, reasons, n_all = [], 0.0, set(), 0
        for line in open(self.path):
            f = [s.strip() for s in line.split(",")]
            if len(f) < 10:
                continue
            n_all += 1
            try:
                ts = time.mktime(time.strptime(f[0].split(".")[0], "%Y/%m/%d %H:%M:%S")) + float("0." + f[0].split(".")[1])
                clk, cmax = float(f[2]), float(f[3])
            except (ValueError, IndexError):
                continue
            if ts < t_begin - 0.2 or ts > t_end + 0.2:
                continue
            sm.append(clk)
            smax = max(smax, cmax)
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[6:10]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0, samples_total=n_all)
        return dict(sm_mhz=statistics.median(sm), sm_max_mhz=smax, reasons=sorted(reasons), samples=len(sm), samples_total=n_all)


# (name, K, N, GELU output) of the four per-layer linears of GPT-2 124M; the tied LM head is handled apart
LAYER_SHAPES = (("qkv", 768, 2304, False), ("attn_proj", 768, 768, False), ("ffn_up", 768, 3072, True), ("ffn_down", 3072, 768, False))
LM_HEAD = (768, 50304)


def _event_ms(torch, fn, reps, sets, rounds=3):
    """Milliseconds per call of fn(buffer set): CUDA events on the current stream around `reps` back-to-back calls with the
    buffer sets rotating, after three warm-up calls; the best of `rounds` such measurements."""
    for i in range(3):
        fn(sets[i % len(sets)])
    best = float("inf")
    for _ in range(rounds):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            fn(sets[i % len(sets)])
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / reps)
    return best


def shapes_record(torch, dev, sampler, reps=20):
    """Every linear layer of GPT-2 124M at M = 8192 (BASELINE.json configs 1 and 2), plus FFN up at M = 1024 and 32768, in
    both precision modes: forward and backward (grad_x, grad_w +=, grad_b += in two launches) apart.  Buffer sets rotate so
    that each call's operands and outputs exceed the 126 MB L2 wherever the shape allows."""
    import gpt_b200
    peaks = measured_peaks()
    out = {}
    g = torch.Generator(device=dev).manual_seed(11)
    cases = [(name, 8192, k, n, act) for name, k, n, act in LAYER_SHAPES] + [("ffn_up", 1024, 768, 3072, True), ("ffn_up", 32768, 768, 3072, True)]
    for mode_name, mode in (("tf32", gpt_b200.MODE_TF32), ("3xtf32", gpt_b200.MODE_3XTF32)):
        be = gpt_b200.Backend(dev.index, torch.cuda.current_stream().cuda_stream, mode)
        t0 = time.time()
        rec = {}
        for name, M, K, N, act in cases:
            nsets = 2 if M >= 32768 else 4
            sets = [dict(x=torch.randn(M, K, device=dev, generator=g), gy=torch.randn(M, N, device=dev, generator=g), y=torch.empty(M, N, device=dev),
                         a=torch.empty(M, N, device=dev) if act else None, gx=torch.empty(M, K, device=dev)) for _ in range(nsets)]
            w = torch.randn(K, N, device=dev, generator=g) * 0.02
            b = torch.randn(N, device=dev, generator=g) * 0.02
            gw, gb = torch.zeros(K, N, device=dev), torch.zeros(N, device=dev)
            l0 = be.launch_count()
            f_ms = _event_ms(torch, lambda s: be.device_linear_activation_fused_forward(s["y"], s["a"], s["x"], w, b, act, 1, M, K, N), reps, sets)
            l1 = be.launch_count()
            b_ms = _event_ms(torch, lambda s: be.device_linear_backward(s["gx"], gw, gb, s["gy"], s["x"], w, 1, M, K, N), reps, sets)
            l2 = be.launch_count()
            fl = 2.0 * M * K * N
            rec[f"{name}_M{M}"] = dict(m=M, k=K, n=N, gelu=act, forward_ms=f_ms, backward_ms=b_ms, forward_tflops=fl / f_ms / 1e9,
                                       backward_tflops=2 * fl / b_ms / 1e9, forward_frac=fl / f_ms / 1e9 / peaks["tf32_tflops"],
                                       backward_frac=2 * fl / b_ms / 1e9 / peaks["tf32_tflops"],
                                       forward_launches=(l1 - l0) // (3 * reps + 3), backward_launches=(l2 - l1) // (3 * reps + 3))
            del sets, w, b, gw, gb
        # the tied LM head (config 2): logits = x . wte^T; backward = grad_x and grad_wte +=
        D, Vp = LM_HEAD
        M = 8192
        x = torch.randn(M, D, device=dev, generator=g)
        wte = torch.randn(Vp, D, device=dev, generator=g) * 0.02
        logits = torch.empty(M, Vp, device=dev)
        gy = torch.randn(M, Vp, device=dev, generator=g) / M
        gx, gwte = torch.empty(M, D, device=dev), torch.zeros(Vp, D, device=dev)
        f_ms = _event_ms(torch, lambda s: be.device_unembedding_forward(logits, x, wte, 1, M, D, Vp), 5, [None])
        b_ms = _event_ms(torch, lambda s: be.device_unembedding_backward(gx, gwte, gy, x, wte, 1, M, D, Vp), 5, [None])
        fl = 2.0 * M * D * Vp
        rec[f"lm_head_M{M}"] = dict(m=M, k=D, n=Vp, gelu=False, forward_ms=f_ms, backward_ms=b_ms, forward_tflops=fl / f_ms / 1e9,
                                    backward_tflops=2 * fl / b_ms / 1e9, forward_frac=fl / f_ms / 1e9 / peaks["tf32_tflops"],
                                    backward_frac=2 * fl / b_ms / 1e9 / peaks["tf32_tflops"])
        del x, wte, logits, gy, gx, gwte
        be.synchronize()
        clk = sampler.summary(t0, time.time()) if sampler else None
        mhz = (clk or {}).get("sm_mhz")
        if mhz:   # time x median SM clock of this phase: separates clock (power cap) effects from stalls
            for r in rec.values():
                r["forward_sm_cycles"] = r["forward_ms"] * 1e-3 * mhz * 1e6
                r["backward_sm_cycles"] = r["backward_ms"] * 1e-3 * mhz * 1e6
        out[mode_name] = dict(shapes=rec, clocks=clk)
        be.close()
        torch.cuda.empty_cache()
    out["peak_tflops"] = peaks["tf32_tflops"]
    out["note"] = ("frac = 2*M*K*N (forward) or 4*M*K*N (backward: grad_x and grad_w) algorithmic flops / CUDA-event time / peak; "
                   "3xtf32 issues twice that work on the tensor pipe (one TF32 chain and one bf16 chain of the same duration)")
    return out


def reference_gpu_record(steps=10, warmup=3):
    """The reference's own CUDA backend on the same shapes and on the training step, timed in a child process (cuBLAS is
    loaded there, never here)."""
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference_cuda_shapes", "--steps", str(steps), "--warmup", str(warmup)]
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
        line = [l for l in res.stdout.splitlines() if l.startswith("{")]
        return json.loads(line[-1]) if line else dict(unavailable=f"child process printed no record (exit code {res.returncode}): {res.stderr[-200:]}")
    except Exception as e:   # a missing prebuilt library or a timeout must not lose the rest of the line
        return dict(unavailable=f"{type(e).__name__}: {e}")


def run_reference_cuda_shapes(args):
    """--impl reference_cuda_shapes (child process of the default run): the reference's CUDA backend -- cublasSgemm in TF32
    tensor-op mode plus its own bias / GELU and bias-gradient kernels (src/backend/cuda/kernels/linear.cu:36-159,
    embedding.cu:47-63,140-170) -- compiled unmodified into oracle/_ref/libref_cuda.so, on the shapes of `shapes`."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libref_cuda.so")
    if not os.path.exists(path):
        print(json.dumps(dict(impl="reference_cuda", unavailable="the reference's CUDA backend was not prebuilt (oracle/_ref/libref_cuda.so)")))
        return
    lib = ctypes.CDLL(path)
    lib.refcuda_linear_ms.restype = ctypes.c_int
    lib.refcuda_linear_ms.argtypes = [ctypes.c_int] * 7 + [ctypes.POINTER(ctypes.c_float)]
    lib.refcuda_unembed_ms.restype = ctypes.c_int
    lib.refcuda_unembed_ms.argtypes = [ctypes.c_int] * 5 + [ctypes.POINTER(ctypes.c_float)]
    lib.refcuda_gpt_step_ms.restype = ctypes.c_float
    lib.refcuda_gpt_step_ms.argtypes = [ctypes.POINTER(ctypes.c_int)] + [ctypes.c_int] * 4
    peaks = measured_peaks()
    rec = {}
    out2 = (ctypes.c_float * 2)()
    cases = [(name, 8192, k, n, act) for name, k, n, act in LAYER_SHAPES] + [("ffn_up", 1024, 768, 3072, True), ("ffn_up", 32768, 768, 3072, True)]
    for name, M, K, N, act in cases:
        if lib.refcuda_linear_ms(M, K, N, int(act), args.steps, args.warmup, 2 if M >= 32768 else 4, out2) != 0:
            continue
        fl = 2.0 * M * K * N
        rec[f"{name}_M{M}"] = dict(m=M, k=K, n=N, gelu=act, forward_ms=out2[0], backward_ms=out2[1], forward_tflops=fl / out2[0] / 1e9,
                                   backward_tflops=2 * fl / out2[1] / 1e9, forward_frac=fl / out2[0] / 1e9 / peaks["tf32_tflops"],
                                   backward_frac=2 * fl / out2[1] / 1e9 / peaks["tf32_tflops"])
    D, Vp = LM_HEAD
    if lib.refcuda_unembed_ms(8192, D, Vp, max(3, args.steps // 2), args.warmup, out2) == 0:
        fl = 2.0 * 8192 * D * Vp
        rec["lm_head_M8192"] = dict(m=8192, k=D, n=Vp, gelu=False, forward_ms=out2[0], backward_ms=out2[1], forward_tflops=fl / out2[0] / 1e9,
                                    backward_tflops=2 * fl / out2[1] / 1e9, forward_frac=fl / out2[0] / 1e9 / peaks["tf32_tflops"],
                                    backward_frac=2 * fl / out2[1] / 1e9 / peaks["tf32_tflops"])
    cfg = (ctypes.c_int * 7)(256, 50257, 50304, 12, 12, 768, 3072)
    ms = float(lib.refcuda_gpt_step_ms(cfg, 64, 256, 3, 1))
    train = dict(ms_per_step=ms, tokens_per_s=64 * 256 / (ms * 1e-3), global_batch=64, seq_len=256) if ms > 0 else None
    print(json.dumps(dict(impl="reference_cuda", dtype="tf32 (cuBLAS tensor-op math)", shapes=rec, train_step=train,
                          note="the reference's CUDABackend, unmodified sources: cublasSgemm + add_bias/GELU kernel forward, two cublasSgemm "
                               "+ bias-gradient kernel backward; same shapes, same rotation of buffer sets")), flush=True)


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    import gpt_b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        _init_process_group(dist, dev)

    mode = gpt_b200.MODE_TF32 if args.mode == "tf32" else gpt_b200.MODE_3XTF32
    stream = torch.cuda.current_stream()
    be = gpt_b200.Backend(local_rank, stream.cuda_stream, mode)
    if args.max_sms:
        be.set_option("max_sms", args.max_sms)
    for kv in args.ctx_option:
        key, _, value = kv.partition("=")
        be.set_option(key, int(value))
    M, K, N = args.m_per_gpu, K_IN, N_OUT
    flops_per_step = 6.0 * M * K * N
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    NSETS = 4
    sets = []
    for _ in range(NSETS):
        sets.append(dict(x=torch.randn(M, K, device=dev, generator=gen), gy=torch.randn(M, N, device=dev, generator=gen),
                         y=torch.empty(M, N, device=dev), act=torch.empty(M, N, device=dev), gx=torch.empty(M, K, device=dev)))
    w = torch.randn(K, N, device=dev, generator=torch.Generator(device=dev).manual_seed(7)) * 0.02
    b = torch.randn(N, device=dev, generator=torch.Generator(device=dev).manual_seed(8)) * 0.02
    grads = torch.zeros(K * N + N, device=dev)          # weight and bias gradients side by side: one collective per step
    gw, gb = grads[:K * N].view(K, N), grads[K * N:]

    comm = torch.cuda.Stream(priority=-1) if world > 1 else None   # NCCL's CTAs go before pending compute CTAs
    num_sms = torch.cuda.get_device_properties(dev).multi_processor_count
    comm_sms = args.comm_sms if args.comm_sms >= 0 else (16 if world <= 2 else 32)
    sms_beside_nccl = max(2, num_sms - comm_sms) if comm_sms > 0 else 0

    def step(i):
        s = sets[i % NSETS]
        be.device_linear_activation_fused_forward(s["y"], s["act"], s["x"], w, b, True, 1, M, K, N)
        if world == 1:
            be.device_linear_backward(s["gx"], gw, gb, s["gy"], s["x"], w, 1, M, K, N)
            return
        # data parallel: weight gradients first; their all-reduce runs on a second stream while grad_x is computed.  grad_x is
        # launched before the collective is enqueued so that the GPU has work while the host is inside NCCL.
        be.linear_backward_weights(gw, gb, s["gy"], s["x"], M, K, N)
        ready = torch.cuda.Event()
        ready.record(stream)
        be.set_option("max_sms", sms_beside_nccl)                # NCCL's CTAs need SMs of their own next to the persistent GEMM
        be.linear_backward_input(s["gx"], s["gy"], w, M, K, N)
        be.set_option("max_sms", 0)
        with torch.cuda.stream(comm):
            comm.wait_event(ready)
            dist.all_reduce(grads, op=dist.ReduceOp.AVG)   # average: the accumulated gradient keeps its magnitude over many steps
        stream.wait_stream(comm)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for i in range(args.warmup):
        step(i)
    be.synchronize()
    barrier()
    t_begin = time.time()
    launches0 = be.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = be.launch_count() - launches0
    be.synchronize()
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    # ---- per-kernel timing of the dominant kernels (forward GEMM, dX GEMM, dW GEMM), same stream
    peaks = measured_peaks()
    kern = {}
    for name, fn, flops in (
        ("forward_gemm_bias_gelu", lambda s: be.device_linear_activation_fused_forward(s["y"], s["act"], s["x"], w, b, True, 1, M, K, N), 2.0 * M * K * N),
        ("backward_dx_dw_db", lambda s: be.device_linear_backward(s["gx"], gw, gb, s["gy"], s["x"], w, 1, M, K, N), 4.0 * M * K * N),
    ):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 1 if args.profile else max(4, args.steps)
        fn(sets[0])
        e0.record()
        for i in range(reps):
            fn(sets[i % NSETS])
        e1.record()
        torch.cuda.synchronize()
        t_ms = e0.elapsed_time(e1) / reps
        kern[name] = dict(ms=t_ms, tflops=flops / t_ms / 1e9)
    be.synchronize()

    # ---- host time of one call of the C ABI (plan, tensor-map lookup, launch; ctypes included), with the GPU idle at the start
    torch.cuda.synchronize()
    n_host = 0 if args.profile else 200
    t0 = time.perf_counter()
    for i in range(n_host):
        be.linear_backward_input(sets[0]["gx"], sets[0]["gy"], w, 64, K, N)   # a small call: the launch queue never fills up
    host_us = (time.perf_counter() - t0) / max(1, n_host) * 1e6
    torch.cuda.synchronize()

    # ---- end to end from pinned host buffers through the C ABI (rank-local; max over ranks)
    hx = torch.randn(M, K).pin_memory()
    hgy = torch.randn(M, N).pin_memory()
    hact, hgx = torch.empty(M, N).pin_memory(), torch.empty(M, K).pin_memory()
    hgw, hgb = torch.empty(K, N).pin_memory(), torch.empty(N).pin_memory()
    s0 = sets[0]
    h2d = (hx.numel() + hgy.numel()) * 4
    d2h = (hact.numel() + hgx.numel() + hgw.numel() + hgb.numel()) * 4

    # Pipelined over three streams (copy-in, compute, copy-out) and two device buffer sets, the way a host program that
    # wants throughput drives the C ABI: step i's inputs arrive while step i-1 computes and step i-2's results leave, so the
    # two directions of the host link work at the same time.  Every step's copies are inside the timed region.
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    snaps = [(torch.empty_like(gw), torch.empty_like(gb)) for _ in range(2)]
    ev_out = [None, None]

    def e2e_step(i):
        st = sets[i % 2]
        with torch.cuda.stream(s_in):
            if ev_out[i % 2] is not None:
                s_in.wait_event(ev_out[i % 2])         # this set's previous results have left (which implies its compute is done)
            st["x"].copy_(hx, non_blocking=True)
            st["gy"].copy_(hgy, non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(s_in)
        stream.wait_event(ev_in)                       # also orders this step after the copy-out of step i - 2 (same buffers)
        gw_snap, gb_snap = snaps[i % 2]
        be.device_linear_activation_fused_forward(st["y"], st["act"], st["x"], w, b, True, 1, M, K, N)
        be.device_linear_backward(st["gx"], gw, gb, st["gy"], st["x"], w, 1, M, K, N)
        if world > 1:
            dist.all_reduce(grads, op=dist.ReduceOp.AVG)
        gw_snap.copy_(gw, non_blocking=True)           # grad_w / grad_b keep accumulating: the host gets this step's state
        gb_snap.copy_(gb, non_blocking=True)
        ev_comp = torch.cuda.Event()
        ev_comp.record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp)
            hact.copy_(st["act"], non_blocking=True)
            hgx.copy_(st["gx"], non_blocking=True)
            hgw.copy_(gw_snap, non_blocking=True)
            hgb.copy_(gb_snap, non_blocking=True)
            ev_out[i % 2] = torch.cuda.Event()
            ev_out[i % 2].record(s_out)

    e2e_steps = 0 if args.profile else max(4, min(args.steps, 10))
    for i in range(0 if args.profile else 2):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    barrier()                                          # torch.cuda.synchronize(): all three streams have drained
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    be.synchronize()
    # keep the same load running for about a second so that the 50 ms clock samples cover it (not part of any
    # number); the iteration count derives from the rank-reduced step time, so every rank runs the same count
    for i in range(0 if args.profile else int(min(5000, max(10, 1000.0 / (ms / args.steps))))):
        step(i)
    torch.cuda.synchronize()
    clocks = sampler.summary(t_begin, time.time()) if sampler else None
    be.close()

    # ---- sub-records (see the module docstring); the headline keys above are not affected by them
    sub = {}
    if not args.profile and not args.no_subrecords:
        del sets, s0, hx, hgy, hact, hgx, hgw, hgb, snaps, grads, gw, gb
        torch.cuda.empty_cache()
        if world == 1:
            sub["shapes"] = shapes_record(torch, dev, sampler)
            torch.cuda.empty_cache()
            sub["decode"] = decode_record(torch, dev, "3xtf32", (1, 8, 64), 20, 3)
            sub["decode"]["value_gbs"] = {k: v["gbs"] for k, v in sub["decode"]["per_batch"].items()}
            sub["decode"]["frac"] = {k: v["hbm_frac"] for k, v in sub["decode"]["per_batch"].items()}
            torch.cuda.empty_cache()
            sub["generate"] = generate_record(torch, dev, "3xtf32")
            torch.cuda.empty_cache()
            sub["attention"] = {m: attention_record(torch, dev, m, 64, 10, 3) for m in ("3xtf32", "tf32")}
            torch.cuda.empty_cache()
        sub["train_step"] = train_record(torch, dist, world, rank, dev, "3xtf32", 64, 5, 2, sampler, parity=True)
        torch.cuda.empty_cache()
        # the same step with the linear layers in single-pass TF32 -- the precision of the reference's own CUDA backend (cuBLAS
        # TF32 tensor ops), whose step reference_gpu times -- and attention on the tensor cores, the default of that mode
        sub["train_step_tf32"] = train_record(torch, dist, world, rank, dev, "tf32", 64, 5, 2, sampler, parity=False)
        torch.cuda.empty_cache()
        if world == 1 and rank == 0:
            sub["reference_gpu"] = reference_gpu_record()
    if sampler:
        sampler.close()

    if rank == 0:
        ms_per_step = ms / args.steps
        value = flops_per_step * world / (ms_per_step * 1e-3) / 1e12
        x3 = mode == gpt_b200.MODE_3XTF32
        fwd = kern["forward_gemm_bias_gelu"]
        mhz = (clocks or {}).get("sm_mhz")
        if mhz:   # time x median SM clock: separates clock (power cap) effects from stalls
            for kv in kern.values():
                kv["sm_cycles"] = kv["ms"] * 1e-3 * mhz * 1e6
        roof = dict(bound="tensor", achieved=fwd["tflops"], peak=peaks["tf32_tflops"], unit="TFLOP/s", frac=fwd["tflops"] / peaks["tf32_tflops"],
                    traffic=NCU_DRAM_BYTES["ffn_up_forward_M8192_3xtf32" if x3 else "ffn_up_forward_M8192_tf32"] if M == M_PER_GPU else None,
                    traffic_note="dram read+write bytes per launch from an ncu capture of this kernel at this shape; algorithmic 235.9e6",
                    kernel="gemm_tcgen05_pair_kernel<A=K-major, B=MN-major> (forward: x.w + bias, GELU)", peak_source=peaks["source"],
                    issued_tflops=fwd["tflops"] * (2 if x3 else 1),
                    issued_frac=fwd["tflops"] * (2 if x3 else 1) / peaks["tf32_tflops"],
                    note="achieved = 2*M*K*N algorithmic flops per launch / CUDA-event launch time; in 3xTF32 mode the tensor pipe "
                         "executes one TF32 MMA chain plus one bf16 MMA chain of the same duration per algorithmic MMA "
                         "(issued_tflops, in TF32-equivalent work)")
        out = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms_per_step,
                   higher_is_better=True, scaling="weak", vs_baseline=None, dtype="tf32x3 (fp32-accurate split)" if x3 else "tf32",
                   data="synthetic", impl="ours",
                   config=dict(workload=WORKLOAD if M == M_PER_GPU else WORKLOAD.replace("8192", str(M)), m_per_gpu=M, k=K, n=N, mode=args.mode, l2="4 rotating buffer sets (1.5 GB) > 126 MB L2",
                               parallelism=f"dp{world}" if world > 1 else "single", allreduce="grad_w+grad_b (NCCL)" if world > 1 else None),
                   tokens_per_s=M * world / (ms_per_step * 1e-3), kernels=kern, roofline=roof, gpu_launches=int(launches),
                   e2e=None if not e2e_steps else dict(value=flops_per_step * world / (e2e_s / e2e_steps) / 1e12, unit=UNIT,
                                                       h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                                                       ms_per_step=e2e_s / e2e_steps * 1e3, steps=e2e_steps),
                   clocks=clocks, host_us_per_call=host_us, **sub)
        if world == 1 and not args.no_cpu_baseline and not args.profile:
            out["cpu_baseline"] = cpu_reference_sample(rows=args.cpu_rows)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def train_record(torch, dist, world, rank, dev, mode_name="3xtf32", global_batch=64, steps=5, warmup=2, sampler=None, parity=True):
    """One full GPT-2 124M training step (BASELINE.json configs[3]) -- zero_grad, forward, backward with bucketed NCCL
    all-reduce of every weight gradient overlapped with the backward pass, gradient clipping and AdamW -- global batch
    `global_batch` x 256 tokens sharded over the ranks (strong scaling).  Seeded random-init weights (the same on every rank)
    and uniform random token ids.  Returns the record on every rank (timings are the maximum over ranks).

    dp_parity: the gradients that the ranks hold after the all-reduce against rank 0 computing the whole global batch alone,
    per tensor max|a - b| / max|b|: only the order of summation differs."""
    import numpy as np
    import gpt_b200
    from gpt_b200.data_parallel import DataParallelStep
    cfg = gpt_b200.GPT2_124M
    GB, T = global_batch, 256
    assert GB % world == 0
    B = GB // world
    mode = gpt_b200.MODE_TF32 if mode_name == "tf32" else gpt_b200.MODE_3XTF32
    stream = torch.cuda.current_stream()
    model = gpt_b200.Model(cfg, dev.index, stream.cuda_stream, mode, seed=42)
    model.init(0.0, 0.02)           # same seed on every rank: identical replicas
    model.set_fused_cross_entropy(os.environ.get("GPTB200_FUSED_CE", "1") != "0")   # logits -> their gradient in place, no probability tensor
    model.set_fused_gelu_backward(os.environ.get("GPTB200_FUSED_GELU", "1") != "0")  # GELU' in the epilogue of the down projection's grad_x GEMM
    for kv in filter(None, os.environ.get("GPTB200_CTX_OPTIONS", "").split(",")):   # experiments: gptb200_ctx_set_option pairs key=value
        model.set_option(kv.partition("=")[0], int(kv.partition("=")[2]))
    model.set_size(B, T)

    class _Raw:   # torch view of the packed gradient buffer (no copy) for the collectives
        __cuda_array_interface__ = dict(shape=(model.num_params,), typestr="<f4", data=(model.grads_ptr, False), version=3, strides=None)
    grads = torch.as_tensor(_Raw(), device=dev)
    dp = DataParallelStep(model, grads, world, layers_per_group=int(os.environ.get("GPTB200_LAYERS_PER_GROUP", "3")), comm_sms=COMM_SMS if COMM_SMS >= 0 else None,
                          early_wte=os.environ.get("GPTB200_EARLY_WTE", "1") != "0")
    rng = np.random.default_rng(1000)
    all_seqs = rng.integers(0, cfg["vocab_size"], size=(GB, T + 1)).astype(np.int32)
    seqs = all_seqs[rank * B:(rank + 1) * B]
    h_in = torch.from_numpy(np.ascontiguousarray(seqs[:, :T])).pin_memory()
    h_lbl = torch.from_numpy(np.ascontiguousarray(seqs[:, 1:])).pin_memory()
    d_in, d_lbl = h_in.to(dev), h_lbl.to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- dp_parity first, on the untouched initial weights
    dp_parity = None
    if parity and world > 1:
        dp.step(d_in, d_lbl)
        torch.cuda.synchronize()
        g_dp = grads.clone()
        barrier()
        per_tensor = {}
        if rank == 0:
            model.defer_embedding_backward(False)
            model.set_size(GB, T)
            f_in = torch.from_numpy(np.ascontiguousarray(all_seqs[:, :T])).to(dev)
            f_lbl = torch.from_numpy(np.ascontiguousarray(all_seqs[:, 1:])).to(dev)
            model.zero_grad()
            model.forward(f_in)
            model.backward(f_in, f_lbl)
            model.synchronize()
            names = sorted(model.param_offsets, key=model.param_offsets.get)
            offs = [model.param_offsets[n] for n in names] + [model.num_params]
            for i, n in enumerate(names):
                a, b = g_dp[offs[i]:offs[i + 1]], grads[offs[i]:offs[i + 1]]
                per_tensor[n] = float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
            model.set_size(B, T)
            model.defer_embedding_backward(dp.early_wte)
            del f_in, f_lbl
        del g_dp
        barrier()
        if rank == 0:
            dp_parity = dict(max=max(per_tensor.values()), per_tensor=per_tensor,
                             note=f"all-reduced gradients of {world} ranks (per-GPU batch {B}) vs rank 0 alone on the whole batch of {GB}")

    def step(e2e=False):
        if e2e:  # the step as a host program sees it: tokens from pinned host memory in, loss back out
            d_in.copy_(h_in, non_blocking=True)
            d_lbl.copy_(h_lbl, non_blocking=True)
        dp.step(d_in, d_lbl)
        model.clip_and_optimizer_step(1.0, 1, 6e-4, 0.9, 0.95, 0.1)    # clipping and AdamW over the packed buffers: two launches
        return model.loss(d_lbl) if e2e else None

    for _ in range(warmup):
        step()
    model.synchronize()
    barrier()
    t_begin = time.time()
    l0 = model.launch_count()
    c0 = dp.collectives
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    launches = model.launch_count() - l0
    collectives = (dp.collectives - c0) // max(1, steps)
    # where the step's time goes (this rank's view, three steps): the same calls as dp.step with events in between
    phase_names = ("zero_grad+forward", "backward", "wait_for_allreduce", "clip+adamw")
    phases = dict.fromkeys(phase_names, 0.0)
    for _ in range(3):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        ev[0].record()
        model.zero_grad()
        model.forward(d_in)
        ev[1].record()
        model.backward(d_in, d_lbl, dp._on_layer_done)
        ev[2].record()
        dp.finish(d_in)      # wait for the collectives still in flight (+ gather and apply the embedding-backward rows)
        ev[3].record()
        model.clip_and_optimizer_step(1.0, 1, 6e-4, 0.9, 0.95, 0.1)
        ev[4].record()
        torch.cuda.synchronize()
        for i, name in enumerate(phase_names):
            phases[name] += ev[i].elapsed_time(ev[i + 1]) / 3.0
    barrier()
    n_e2e = max(2, min(steps, 5))
    loss = step(True)
    barrier()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        loss = step(True)
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    clocks = sampler.summary(t_begin, time.time()) if sampler else None
    model.synchronize()
    ms_step = ms / steps
    tokens = GB * T
    lin_flops = 3 * 247.1e6 * tokens  # forward + backward of all linear layers: 741.4 MFLOP per token
    rec = dict(tokens_per_s=tokens / (ms_step * 1e-3), ms_per_step=ms_step, global_batch=GB, seq_len=T, per_gpu_batch=B, n_gpus=world,
               mode=mode_name, scaling="strong", steps=steps, warmup=warmup, phases_ms=phases, collectives_per_step=int(collectives),
               gpu_launches_per_step=int(launches // max(1, steps)), linear_path_tflops=lin_flops / (ms_step * 1e-3) / 1e12,
               e2e=dict(value=tokens / (e2e_s / n_e2e), unit="tokens/s", h2d_bytes_per_step=int(2 * B * T * 4), d2h_bytes_per_step=4,
                        ms_per_step=e2e_s / n_e2e * 1e3, loss=loss),
               dp_parity=dp_parity, clocks=clocks, comm_sms=dp.comm_sms, early_wte=dp.early_wte)
    model.close()
    return rec


def run_train(args):
    """--workload train: the training step of train_record as the line's own metric (tokens/s, strong scaling)."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        _init_process_group(dist, dev)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    rec = train_record(torch, dist, world, rank, dev, args.mode, args.global_batch, args.steps, args.warmup, sampler, parity=not args.no_parity)
    if sampler:
        sampler.close()
    if rank == 0:
        peaks = measured_peaks()
        per_gpu = rec["linear_path_tflops"] / world
        out = dict(metric="train_tokens_per_s", value=rec["tokens_per_s"], unit="tokens/s", n_gpus=world, steps=args.steps,
                   warmup=args.warmup, ms_per_step=rec["ms_per_step"], higher_is_better=True, scaling="strong", vs_baseline=None,
                   dtype="tf32x3 (fp32-accurate split)" if args.mode != "tf32" else "tf32", data="synthetic", impl="ours",
                   config=dict(workload="GPT-2 124M full training step (forward, backward, grad all-reduce, clip, AdamW)", global_batch=rec["global_batch"],
                               seq_len=256, per_gpu_batch=rec["per_gpu_batch"], mode=args.mode, parallelism=f"dp{world}",
                               l2="activations and weights (>10 GB per step) exceed the 126 MB L2"),
                   linear_path_tflops=rec["linear_path_tflops"],
                   roofline=dict(bound="tensor", achieved=per_gpu, peak=peaks["tf32_tflops"], unit="TFLOP/s", frac=per_gpu / peaks["tf32_tflops"], traffic=None,
                                 note="linear-path algorithmic flops per GPU over the WHOLE step time (attention, LayerNorm, softmax, "
                                      "optimizer included in the time)", peak_source=peaks["source"]),
                   phases_ms=rec["phases_ms"], gpu_launches=rec["gpu_launches_per_step"] * args.steps, collectives_per_step=rec["collectives_per_step"],
                   dp_parity=rec["dp_parity"], e2e=rec["e2e"], clocks=rec["clocks"])
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


NCCL_MAX_CTAS = int(os.environ.get("GPTB200_NCCL_MAX_CTAS", "0"))   # 0: NCCL's own choice
COMM_SMS = int(os.environ.get("GPTB200_COMM_SMS", "-1"))             # SMs the GEMMs leave to NCCL meanwhile; -1: by world size


def _init_process_group(dist, dev):
    """NCCL process group whose collectives run on a high-priority stream (their CTAs are placed before pending GEMM CTAs) and,
    optionally, with a bound on the CTAs NCCL may use per collective (the gradient all-reduce overlaps the backward pass and
    needs a fraction of the link bandwidth: every SM it does not take stays with the GEMMs)."""
    try:
        from torch.distributed import ProcessGroupNCCL
        opts = ProcessGroupNCCL.Options(is_high_priority_stream=True)
        if NCCL_MAX_CTAS > 0:
            opts.config.max_ctas = NCCL_MAX_CTAS
            opts.config.min_ctas = min(NCCL_MAX_CTAS, 4)
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    except Exception as e:
        print(f"[bench] process group options not applied ({type(e).__name__}: {e})", file=sys.stderr)
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)


def decode_record(torch, dev, mode_name="3xtf32", batches=(1, 8, 64), steps=20, warmup=3, ctx_options=()):
    """The linear layers of one GPT-2 124M decode step (BASELINE.json configs[4]) for each batch size: per layer QKV,
    attention projection, FFN up (GELU), FFN down, then the 50304-wide LM head, with m = batch rows.  HBM-bound: 494.27 MB
    of fp32 weights are read once per step.  GB/s = weight bytes / time (CUDA events around replays of the step captured
    as one CUDA graph, so that the time is the kernels', not the host's launch loop)."""
    import gpt_b200
    cfg = gpt_b200.GPT2_124M
    L, D, F, Vp = cfg["num_layers"], cfg["d_model"], cfg["d_ffn"], cfg["vocab_size_padded"]
    mode = gpt_b200.MODE_TF32 if mode_name == "tf32" else gpt_b200.MODE_3XTF32
    be = gpt_b200.Backend(dev.index, torch.cuda.current_stream().cuda_stream, mode)
    # inference: nothing writes the weights between layers, so each layer may prefetch them while its predecessor still runs
    options = dict(decode_early_launch=1)
    for kv in ctx_options:
        key, _, val = kv.partition("=")
        options[key] = int(val)
    for key, val in options.items():
        be.set_option(key, val)
    g = torch.Generator(device=dev).manual_seed(5)
    W = dict(qkv=[torch.randn(D, 3 * D, device=dev, generator=g) * 0.02 for _ in range(L)],
             proj=[torch.randn(D, D, device=dev, generator=g) * 0.02 for _ in range(L)],
             up=[torch.randn(D, F, device=dev, generator=g) * 0.02 for _ in range(L)],
             down=[torch.randn(F, D, device=dev, generator=g) * 0.02 for _ in range(L)])
    wte = torch.randn(Vp, D, device=dev, generator=g) * 0.02
    bias = dict(qkv=torch.zeros(3 * D, device=dev), proj=torch.zeros(D, device=dev), up=torch.zeros(F, device=dev), down=torch.zeros(D, device=dev))
    weight_bytes = 4.0 * (L * (D * 3 * D + D * D + 2 * D * F) + Vp * D)
    peaks = measured_peaks()
    results = {}
    launches = 0
    for batch in batches:
        x = torch.randn(batch, D, device=dev, generator=g)
        q, a, u, ua, dn, lg = (torch.empty(batch, n, device=dev) for n in (3 * D, D, F, F, D, Vp))

        def step():
            for l in range(L):
                be.device_linear_activation_fused_forward(q, None, x, W["qkv"][l], bias["qkv"], False, 1, batch, D, 3 * D)
                be.device_linear_activation_fused_forward(a, None, x, W["proj"][l], bias["proj"], False, 1, batch, D, D)
                be.device_linear_activation_fused_forward(u, ua, x, W["up"][l], bias["up"], True, 1, batch, D, F)
                be.device_linear_activation_fused_forward(dn, None, ua, W["down"][l], bias["down"], False, 1, batch, F, D)
            be.device_unembedding_forward(lg, x, wte, 1, batch, D, Vp)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            be.set_stream(side.cuda_stream)
            for _ in range(max(warmup, 3)):   # sizes the scratch buffer and sets kernel attributes before capture
                step()
            side.synchronize()
            l0 = be.launch_count()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                step()
            per_step = be.launch_count() - l0
            graph.replay()
            side.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(steps):
                graph.replay()
            e1.record(side)
            side.synchronize()
        torch.cuda.current_stream().wait_stream(side)
        launches += per_step * steps
        ms = e0.elapsed_time(e1) / steps
        results[f"batch{batch}"] = dict(ms_per_step=ms, gbs=weight_bytes / (ms * 1e-3) / 1e9, tokens_per_s=batch / (ms * 1e-3),
                                         hbm_frac=weight_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], launches_per_step=per_step)
    be.set_stream(torch.cuda.current_stream().cuda_stream)
    be.synchronize()
    be.close()
    return dict(per_batch=results, weight_bytes=weight_bytes, peak_gbs=peaks["hbm_gbs"], options=options, gpu_launches=int(launches),
                note="fp32 FMA kernels (no TF32 rounding); algorithmic bytes = the fp32 weights read once per step")


def run_decode(args):
    """--workload decode: see decode_record; the JSON `value` is the batch-8 figure.  The reference has no KV-cached decode
    (src/infer/infer.cpp:121 recomputes the whole prefix), so this measures the GEMM shapes of such a step."""
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    sampler = ClockSampler(0)
    t_begin = time.time()
    rec = decode_record(torch, dev, args.mode, [int(b) for b in args.decode_batches.split(",")], args.steps, args.warmup, args.ctx_option)
    clocks = sampler.stop(t_begin, time.time())
    results = rec["per_batch"]
    r8 = results.get("batch8") or next(iter(results.values()))
    out = dict(metric="decode_linear_weight_stream_gbs", value=r8["gbs"], unit="GB/s", n_gpus=1, steps=args.steps, warmup=args.warmup,
               ms_per_step=r8["ms_per_step"], higher_is_better=True, scaling="weak", vs_baseline=None,
               dtype="f32", data="synthetic", impl="ours",
               config=dict(workload="GPT-2 124M decode step, linear layers only (49 GEMMs with m = batch)", mode=args.mode, options=rec["options"],
                           weight_bytes=rec["weight_bytes"], l2="494 MB of weights per step exceed the 126 MB L2"),
               per_batch=results,
               roofline=dict(bound="hbm", achieved=r8["gbs"], peak=rec["peak_gbs"], unit="GB/s", frac=r8["hbm_frac"], traffic=NCU_DRAM_BYTES["decode_step_batch1"],
                             traffic_note="dram read+write bytes of the 49 kernels of a batch-1 step (ncu); algorithmic 494.27e6",
                             note="algorithmic bytes = fp32 weights read once per step (494.27 MB); batch 8", peak_source="of measured (MEASURED_PEAKS.json copy bandwidth)"),
               gpu_launches=rec["gpu_launches"], clocks=clocks)
    print(json.dumps(out), flush=True)


def generate_record(torch, dev, mode_name="3xtf32", batches=(1, 8, 64), with_prefix_recompute=True):
    """Autoregressive generation with GPT-2 124M random-init weights (BASELINE.json configs[4]): a random-id prompt of 64 tokens
    extended to 256 tokens at temperature 1.0, for each batch size, in two forms:
      kv_cache           one forward pass over the prompt, then one row per sequence per step against cached keys / values
                         (every linear layer runs with m = batch rows); the step is captured once as a CUDA graph (its position
                         lives in device memory) and replayed per token, sampling in between;
      prefix_recompute   the reference's way (src/infer/infer.cpp:112-148, no KV cache): every new token recomputes the whole
                         prefix, m = batch * (64 ... 255) rows.
    Sampling (softmax at temperature 1 + multinomial over the 50257 real tokens) runs on the GPU with torch."""
    import gpt_b200
    cfg = gpt_b200.GPT2_124M
    V, Vp = cfg["vocab_size"], cfg["vocab_size_padded"]
    mode = gpt_b200.MODE_TF32 if mode_name == "tf32" else gpt_b200.MODE_3XTF32
    PROMPT, TOTAL = 64, 256
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    results = {}
    launches = 0
    with torch.cuda.stream(stream):
        model = gpt_b200.Model(cfg, dev.index, stream.cuda_stream, mode, seed=42, use_grad=False)
        model.init(0.0, 0.02)
        model.set_option("decode_early_launch", 1)      # inference: nothing writes the weights between the layers
        for batch in batches:
            torch.manual_seed(batch)
            prompt = torch.randint(0, V, (batch, PROMPT), dtype=torch.int32, device=dev)
            tok = torch.empty(batch, dtype=torch.int32, device=dev)
            logits = torch.empty(batch, Vp, device=dev)

            def sample(lg):
                probs = torch.softmax(lg[:, :V].float(), dim=-1)            # temperature 1.0
                return torch.multinomial(probs, 1).squeeze(1).to(torch.int32)

            def prompt_logits():
                class _Raw:
                    __cuda_array_interface__ = dict(shape=(batch, PROMPT, Vp), typestr="<f4", data=(model.logits_ptr, False), version=3, strides=None)
                return torch.as_tensor(_Raw(), device=dev)[:, PROMPT - 1, :]

            def generate(graph):
                model.generate_begin(prompt, batch, PROMPT, TOTAL)
                tok.copy_(sample(prompt_logits()))
                out = [tok.clone()]
                for _ in range(PROMPT + 1, TOTAL):
                    if graph is not None:
                        graph.replay()
                    else:
                        model.generate_step(tok, logits)
                    tok.copy_(sample(logits))
                    out.append(tok.clone())
                return out

            generate(None)                                   # eager pass: sizes scratch, sets kernel attributes
            stream.synchronize()
            model.generate_begin(prompt, batch, PROMPT, TOTAL)
            tok.copy_(sample(prompt_logits()))
            graph = torch.cuda.CUDAGraph()
            l0 = model.launch_count()
            with torch.cuda.graph(graph, stream=stream):
                model.generate_step(tok, logits)
            per_step = model.launch_count() - l0
            generate(graph)                                  # warm replay pass
            stream.synchronize()
            t0 = time.perf_counter()
            generate(graph)
            stream.synchronize()
            dt = time.perf_counter() - t0
            new_tokens = batch * (TOTAL - PROMPT)
            rec = dict(kv_cache=dict(seconds=dt, tokens_per_s=new_tokens / dt, ms_per_token_step=dt / (TOTAL - PROMPT) * 1e3, launches_per_step=per_step))
            launches += per_step * (TOTAL - PROMPT - 1)
            if with_prefix_recompute:
                seq = torch.zeros(batch, TOTAL, dtype=torch.int32, device=dev)
                seq[:, :PROMPT] = prompt
                model.set_size(batch, TOTAL)

                def recompute():
                    for t in range(PROMPT, TOTAL):
                        model.set_size(batch, t)
                        model.forward(seq[:, :t].contiguous())

                        class _Raw:
                            __cuda_array_interface__ = dict(shape=(batch, t, Vp), typestr="<f4", data=(model.logits_ptr, False), version=3, strides=None)
                        seq[:, t] = sample(torch.as_tensor(_Raw(), device=dev)[:, t - 1, :])

                if batch <= 8:
                    recompute()                              # warm-up pass (the batch-64 form takes seconds: timed cold)
                stream.synchronize()
                l0 = model.launch_count()
                t0 = time.perf_counter()
                recompute()
                stream.synchronize()
                dt2 = time.perf_counter() - t0
                launches += model.launch_count() - l0
                rec["prefix_recompute"] = dict(seconds=dt2, tokens_per_s=new_tokens / dt2, ms_per_token_step=dt2 / (TOTAL - PROMPT) * 1e3)
                rec["kv_cache_speedup"] = dt2 / dt
            results[f"batch{batch}"] = rec
        model.close()
    torch.cuda.current_stream().wait_stream(stream)
    return dict(per_batch=results, prompt_len=PROMPT, total_len=TOTAL, temperature=1.0, mode=mode_name, gpu_launches=int(launches),
                note="tokens/s counts generated tokens; host-side sampling with torch is inside the time")


def attention_record(torch, dev, mode_name="tf32", batch=64, steps=20, warmup=3, ctx_options=()):
    """Causal attention of one GPT-2 124M layer (12 heads of 64, 256 tokens per sequence) through gptb200_attention_forward /
    _backward (the reference's device_flash_attention_forward / _backward, cuda/kernels/attention.cu): microseconds per call as
    batched tensor-core products + row kernels in the given precision mode, and as the fp32 FMA kernels."""
    import gpt_b200
    T, D, H = 256, 768, 12
    be = gpt_b200.Backend(dev.index, torch.cuda.current_stream().cuda_stream, gpt_b200.MODE_TF32 if mode_name == "tf32" else gpt_b200.MODE_3XTF32)
    lib = be.lib
    for kv in ctx_options:
        be.set_option(kv.partition("=")[0], int(kv.partition("=")[2]))
    gen = torch.Generator(device=dev).manual_seed(11)
    qkv = torch.randn(batch, T, 3 * D, device=dev, generator=gen)
    gy = torch.randn(batch, T, D, device=dev, generator=gen)
    y, lse = torch.empty(batch, T, D, device=dev), torch.empty(batch, T, H, device=dev)
    gq, dc = torch.empty(batch, T, 3 * D, device=dev), torch.empty(batch, T, H, device=dev)

    def fwd():
        assert lib.gptb200_attention_forward(be.handle, y.data_ptr(), lse.data_ptr(), qkv.data_ptr(), batch, T, D, H) == 0

    def bwd():
        assert lib.gptb200_attention_backward(be.handle, gq.data_ptr(), dc.data_ptr(), lse.data_ptr(), gy.data_ptr(), y.data_ptr(), qkv.data_ptr(), batch, T, D, H) == 0

    out, launches = {}, 0
    for form, option in (("tensor_core", 1), ("fp32_fma", 0)):
        be.set_option("attention_gemm", option)
        rec = {}
        for name, fn in (("forward", fwd), ("backward", bwd)):
            for _ in range(warmup):
                fn()
            torch.cuda.synchronize()
            l0 = be.launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            launches += be.launch_count() - l0
            rec[name + "_us"] = e0.elapsed_time(e1) / steps * 1e3
            rec[name + "_launches"] = (be.launch_count() - l0) // steps
        out[form] = rec
    be.close()
    # both causal halves of the five products count as algorithmic work: 2 * T * T * 64 flops per product, head and sequence / 2
    flops = {"forward": 2 * 2.0 * T * T * 64 * H * batch / 2, "backward": 5 * 2.0 * T * T * 64 * H * batch / 2}
    for rec in out.values():
        for name in ("forward", "backward"):
            rec[name + "_tflops"] = flops[name] / (rec[name + "_us"] * 1e-6) / 1e12
    return dict(forms=out, batch=batch, seq_len=T, heads=H, head_size=64, mode=mode_name, gpu_launches=int(launches))


def run_attention(args):
    """--workload attention: see attention_record; the JSON `value` is forward + backward of the tensor-core form."""
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    sampler = ClockSampler(0)
    t_begin = time.time()
    rec = attention_record(torch, dev, args.mode, args.global_batch, args.steps, args.warmup, args.ctx_option)
    clocks = sampler.stop(t_begin, time.time())
    tc = rec["forms"]["tensor_core"]
    us = tc["forward_us"] + tc["backward_us"]
    out = dict(metric="attention_layer_us", value=us, unit="us", n_gpus=1, steps=args.steps, warmup=args.warmup, ms_per_step=us * 1e-3,
               higher_is_better=False, scaling="weak", vs_baseline=None, dtype="tf32" if args.mode == "tf32" else "tf32x3 (fp32-accurate split)",
               data="synthetic", impl="ours",
               config=dict(workload="causal attention of one GPT-2 124M layer, forward + backward", batch=rec["batch"], seq_len=rec["seq_len"], heads=rec["heads"],
                           head_size=64, mode=args.mode, l2="qkv, outputs and score matrices of 64 sequences (> 700 MB) exceed the 126 MB L2"),
               forms=rec["forms"], gpu_launches=rec["gpu_launches"], clocks=clocks)
    print(json.dumps(out), flush=True)


def run_generate(args):
    """--workload generate: see generate_record; the JSON `value` is the batch-8 KV-cached figure."""
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    rec = generate_record(torch, dev, args.mode)
    r8 = rec["per_batch"]["batch8"]["kv_cache"]
    out = dict(metric="generate_tokens_per_s", value=r8["tokens_per_s"], unit="tokens/s", n_gpus=1, steps=1, warmup=1,
               ms_per_step=r8["ms_per_token_step"], higher_is_better=True, scaling="weak", vs_baseline=None,
               dtype="f32 (decode-shaped layers use fp32 FMA kernels)", data="synthetic", impl="ours",
               config=dict(workload="GPT-2 124M generation, prompt 64 -> 256 tokens, temperature 1.0, KV cache (the reference recomputes the prefix: see prefix_recompute)",
                           mode=args.mode), per_batch=rec["per_batch"], gpu_launches=rec["gpu_launches"])
    print(json.dumps(out), flush=True)


def cpu_reference_sample(rows: int):
    """The reference CPU backend (unmodified sources behind oracle/_ref, one thread -- it has no threading) on
    `rows` rows of the workload; falls back to the oracle port when the reference library was not prebuilt."""
    import numpy as np
    from oracle.oracle import Oracle, Reference, reference_available
    rng = np.random.default_rng(0)
    K, N = K_IN, N_OUT
    x = rng.standard_normal((rows, K), dtype=np.float32)
    w = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
    b = (0.02 * rng.standard_normal(N)).astype(np.float32)
    gy = rng.standard_normal((rows, N), dtype=np.float32)
    if reference_available():
        impl, kind, cores = Reference(), "reference", 1
    else:
        impl, kind = Oracle(), "port"
        cores = impl.num_threads()
    t0 = time.perf_counter()
    impl.linear_forward(x, w, b, True)
    impl.linear_backward(gy, x, w)
    dt = time.perf_counter() - t0
    flops = 6.0 * rows * K * N
    return dict(value=flops / dt / 1e12, unit=UNIT, cores=cores, kind=kind, host_cores=os.cpu_count(), seconds=dt,
                sample=f"{rows} of {M_PER_GPU} rows of the same step (cost is linear in rows), forward+backward")


def run_reference_cuda(args):
    """--impl reference_cuda (information only, not the contract's reference arm): the reference's own CUDA backend --
    cuBLAS TF32 sgemm plus its separate bias/GELU and bias-gradient kernels -- compiled unmodified into
    oracle/_ref/libref_cuda.so, timed on the same GPU for the same workload."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libref_cuda.so")
    if not os.path.exists(path):
        print(json.dumps(dict(impl="reference_cuda", unavailable="oracle/_ref/libref_cuda.so was not prebuilt")))
        return
    lib = ctypes.CDLL(path)
    lib.refcuda_ffn_step_ms.restype = ctypes.c_float
    lib.refcuda_ffn_step_ms.argtypes = [ctypes.c_int] * 6
    lib.refcuda_gpt_step_ms.restype = ctypes.c_float
    lib.refcuda_gpt_step_ms.argtypes = [ctypes.POINTER(ctypes.c_int)] + [ctypes.c_int] * 4
    if args.workload == "train":
        cfg = (ctypes.c_int * 7)(256, 50257, 50304, 12, 12, 768, 3072)
        ms = float(lib.refcuda_gpt_step_ms(cfg, args.global_batch, 256, args.steps, args.warmup))
        out = dict(metric="train_tokens_per_s", value=args.global_batch * 256 / (ms * 1e-3), unit="tokens/s", n_gpus=1, steps=args.steps,
                   warmup=args.warmup, ms_per_step=ms, higher_is_better=True, dtype="tf32 (cuBLAS)", data="synthetic", impl="reference_cuda",
                   config=dict(workload="GPT-2 124M full training step, reference CUDA backend", global_batch=args.global_batch, seq_len=256))
    else:
        ms = float(lib.refcuda_ffn_step_ms(args.m_per_gpu, K_IN, N_OUT, args.steps, args.warmup, 4))
        out = dict(metric=METRIC, value=6.0 * args.m_per_gpu * K_IN * N_OUT / (ms * 1e-3) / 1e12, unit=UNIT, n_gpus=1, steps=args.steps,
                   warmup=args.warmup, ms_per_step=ms, higher_is_better=True, dtype="tf32 (cuBLAS)", data="synthetic", impl="reference_cuda",
                   config=dict(workload=WORKLOAD + ", reference CUDA backend (cuBLAS + unfused kernels)", m_per_gpu=args.m_per_gpu, k=K_IN, n=N_OUT))
    print(json.dumps(out), flush=True)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = args.ref_rows
    # warm-up and timed steps, each a bounded row sample
    for _ in range(min(args.warmup, 1)):
        cpu_reference_sample(rows)
    t = []
    base = None
    for _ in range(args.steps):
        base = cpu_reference_sample(rows)
        t.append(base["seconds"])
    sec = statistics.mean(t)
    value = 6.0 * rows * K_IN * N_OUT / sec / 1e12
    base["value"] = value
    out = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=args.gpus, steps=args.steps, warmup=min(args.warmup, 1),
               ms_per_step=sec * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
               config=dict(workload=WORKLOAD, m_per_gpu=M_PER_GPU, k=K_IN, n=N_OUT, sample_rows_per_step=rows),
               cpu_baseline=base, e2e=dict(value=value, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--mode", choices=["3xtf32", "tf32"], default="3xtf32")
    ap.add_argument("--impl", choices=["ours", "reference", "reference_cuda", "reference_cuda_shapes"], default="ours")
    ap.add_argument("--cpu-rows", type=int, default=256, help="rows of the workload the cpu_baseline leg runs")
    ap.add_argument("--ref-rows", type=int, default=32, help="rows per step of the --impl reference arm")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", choices=["ffn", "train", "decode", "generate", "attention"], default="ffn",
                    help="ffn: BASELINE configs[1] (default); train: configs[3]; decode: configs[4] (linear layers of a decode step); generate: configs[4] end to end")
    ap.add_argument("--global-batch", type=int, default=64, help="sequences per step over all GPUs (train workload); sequences of the attention workload")
    ap.add_argument("--m-per-gpu", type=int, default=M_PER_GPU, help="tokens per GPU (smaller for profiler captures)")
    ap.add_argument("--max-sms", type=int, default=0, help="SMs the GEMM kernels may occupy (0 = all; experiments)")
    ap.add_argument("--comm-sms", type=int, default=-1,
                    help="SMs left to NCCL while a GEMM overlaps a collective (N > 1); -1: 16 at two GPUs, 32 beyond (measured best)")
    ap.add_argument("--decode-batches", default="1,8,64", help="decode workload: batch sizes (the JSON value is the batch-8 figure)")
    ap.add_argument("--ctx-option", action="append", default=[], metavar="KEY=VALUE",
                    help="gptb200_ctx_set_option before the run (decode workload; experiments)")
    ap.add_argument("--profile", action="store_true", help="only the timed steps: no end-to-end, clock-load or CPU legs, no sub-records")
    ap.add_argument("--no-subrecords", action="store_true", help="leave out the shapes / decode / train_step / reference_gpu sub-records")
    ap.add_argument("--no-parity", action="store_true", help="train workload: skip the N-rank vs one-rank gradient comparison")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference_cuda":
        run_reference_cuda(args)
    elif args.impl == "reference_cuda_shapes":
        run_reference_cuda_shapes(args)
    elif args.workload == "train":
        run_train(args)
    elif args.workload == "decode":
        run_decode(args)
    elif args.workload == "attention":
        run_attention(args)
    elif args.workload == "generate":
        run_generate(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
