"""Whole-model GPU tests: the reference's own model driver (src/model/gpt.cpp, compiled unmodified into
oracle/_ref) runs its forward/backward op sequence on the product library's IGPTBackend object.  This is the
drop-in check: the driver was compiled against the reference's header, the backend object against this
library's copy of the declaration, and the calls go through the virtual table.

Checks, in 3xTF32 mode (the default):
  - the reference's gradient test (src/model/gpt_test.cpp): tiny config, all 16 gradient tensors within 1e-5
    absolute of the PyTorch goldens and of the reference CPU backend;
  - BASELINE config 0: GPT-2 124M, B=4, T=256, seeded weights and uniform random tokens, every gradient tensor
    within 1e-5 (max-normalised) of the CPU model (reference driver + reference CPU backend with the linear
    operators replaced by their bit-identical threaded restatement, so that it finishes in minutes).
TF32 mode: the 2e-3 bound is per operator (tests/test_parity_gpu.py); through a 4-layer model the truncation
errors of successive operators compound, so the whole-model check on the tiny config uses 5e-3 (max-normalised).
"""
import ctypes
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN
from oracle.oracle import split_weights, weight_layout

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib(built_library):
    import torch
    assert torch.cuda.is_available()
    import gpt_b200
    return gpt_b200.load_library()


def _backend(lib, mode):
    ptr = lib.gptb200_backend_create(1234, 0, None, mode)
    assert ptr
    return ptr


def _tiny():
    meta = json.load(open(os.path.join(GOLDEN, "gpt_tiny.json")))
    tokens = np.fromfile(os.path.join(GOLDEN, "gpt_tiny_tokens.bin"), dtype=np.int32)
    weights = np.fromfile(os.path.join(GOLDEN, "gpt_tiny_weights.bin"), dtype=np.float32)
    golden = np.fromfile(os.path.join(GOLDEN, "gpt_tiny_ref_grads.bin"), dtype=np.float32)
    return meta["config"], tokens, weights, golden


def test_reference_gradient_test_on_b200_backend(lib, reference):
    cfg, tokens, weights, golden = _tiny()
    T = cfg["max_seq_len"]
    be = _backend(lib, 0)
    try:
        grads, loss, _ = reference.gpt_forward_backward(cfg, weights, tokens[:T], tokens[1:T + 1], 1, T, backend_ptr=be)
    finally:
        lib.gptb200_backend_destroy(ctypes.c_void_p(be))
    cpu, cpu_loss, _ = reference.gpt_forward_backward(cfg, weights, tokens[:T], tokens[1:T + 1], 1, T)
    assert abs(loss - cpu_loss) < 1e-5 and abs(loss - 6.185424) < 1e-4
    a, g, c = split_weights(cfg, grads), split_weights(cfg, golden), split_weights(cfg, cpu)
    for name in a:  # the repo's criterion, on the true packing, all 16 tensors
        assert np.isfinite(a[name]).all(), name
        assert np.abs(a[name] - g[name]).max() <= 1e-5, (name, "vs PyTorch golden", float(np.abs(a[name] - g[name]).max()))
        assert np.abs(a[name] - c[name]).max() <= 1e-5, (name, "vs reference CPU backend", float(np.abs(a[name] - c[name]).max()))


def test_tiny_model_tf32_mode(lib, reference):
    cfg, tokens, weights, _ = _tiny()
    T = cfg["max_seq_len"]
    be = _backend(lib, 1)
    try:
        grads, loss, _ = reference.gpt_forward_backward(cfg, weights, tokens[:T], tokens[1:T + 1], 1, T, backend_ptr=be)
    finally:
        lib.gptb200_backend_destroy(ctypes.c_void_p(be))
    cpu, cpu_loss, _ = reference.gpt_forward_backward(cfg, weights, tokens[:T], tokens[1:T + 1], 1, T)
    assert abs(loss - cpu_loss) < 2e-3
    a, c = split_weights(cfg, grads), split_weights(cfg, cpu)
    for name in a:
        denom = max(np.abs(c[name]).max(), 1e-30)
        assert np.abs(a[name] - c[name]).max() / denom <= 5e-3, name


GPT2_124M = dict(max_seq_len=256, vocab_size=50257, vocab_size_padded=50304, num_layers=12, num_heads=12, d_model=768, d_ffn=3072)


def gpt2_weights(cfg, seed):
    """Seeded initialisation: N(0, 0.02), residual projections scaled by 1/sqrt(2L), biases 0, LayerNorm gains 1,
    padded vocabulary rows 0 (BASELINE config 0; the reference's init, src/model/gpt.cpp:297-325, plus zeroed padding)."""
    rng = np.random.default_rng(seed)
    parts = []
    for name, shape in weight_layout(cfg):
        n = int(np.prod(shape))
        if name in ("ln_1_w", "ln_2_w", "ln_f_w"):
            w = np.ones(n, np.float32)
        elif name.endswith("_b"):
            w = np.zeros(n, np.float32)
        else:
            w = (0.02 * rng.standard_normal(n, dtype=np.float32)).astype(np.float32)
            if name in ("attn_proj_w", "ffn_down_w"):
                w *= np.float32(1.0 / np.sqrt(2.0 * cfg["num_layers"]))
            if name == "wte":
                w.reshape(shape)[cfg["vocab_size"]:] = 0.0
        parts.append(w)
    return np.concatenate(parts)


def exact_gradients(cfg, weights, inputs, labels, device="cuda"):
    """Loss and all 16 gradient tensors of the model in float64 (torch autograd): the exactly rounded result to the accuracy that
    matters here (1e-5), against which the distance of the GPU result and of the fp32 CPU model can both be measured.  GPT-2 as
    the reference builds it (src/model/gpt.cpp:458-541): learned positions, pre-LayerNorm blocks (eps 1e-5), causal attention
    scaled by 1 / sqrt(head size), tanh GELU, tied un-embedding over the unpadded vocabulary, mean cross-entropy."""
    import torch
    import torch.nn.functional as F
    L, H, D, V = cfg["num_layers"], cfg["num_heads"], cfg["d_model"], cfg["vocab_size"]
    w = {k: torch.tensor(v, dtype=torch.float64, device=device, requires_grad=True) for k, v in split_weights(cfg, weights).items()}
    tok = torch.as_tensor(np.asarray(inputs), device=device).long()
    lbl = torch.as_tensor(np.asarray(labels), device=device).long()
    B, T = tok.shape
    x = w["wte"][tok] + w["wpe"][:T]
    causal = torch.ones(T, T, dtype=torch.bool, device=device).tril()
    for l in range(L):
        h = F.layer_norm(x, (D,), w["ln_1_w"][l], w["ln_1_b"][l], eps=1e-5)
        q, k, v = [t.reshape(B, T, H, D // H).transpose(1, 2) for t in (h @ w["qkv_proj_w"][l] + w["qkv_proj_b"][l]).split(D, dim=-1)]
        att = (q @ k.transpose(-1, -2)) / np.sqrt(D // H)
        att = torch.softmax(att.masked_fill(~causal, float("-inf")), dim=-1)
        x = x + (att @ v).transpose(1, 2).reshape(B, T, D) @ w["attn_proj_w"][l] + w["attn_proj_b"][l]
        h = F.layer_norm(x, (D,), w["ln_2_w"][l], w["ln_2_b"][l], eps=1e-5)
        x = x + F.gelu(h @ w["ffn_up_w"][l] + w["ffn_up_b"][l], approximate="tanh") @ w["ffn_down_w"][l] + w["ffn_down_b"][l]
    x = F.layer_norm(x, (D,), w["ln_f_w"], w["ln_f_b"], eps=1e-5)
    logits = (x @ w["wte"][:V].t()).reshape(B * T, V)
    F.cross_entropy(logits, lbl.reshape(-1)).backward()
    # the reported loss carries the reference's guard against log(0) (cpu_backend.cpp:510); the gradient does not
    p_label = torch.softmax(logits.detach(), dim=-1).gather(1, lbl.reshape(-1, 1))
    loss = -(p_label + 1e-8).log().mean()
    return {k: v.grad.cpu().numpy() for k, v in w.items()}, float(loss)


@pytest.fixture(scope="module")
def config0(reference):
    """BASELINE config 0 (GPT-2 124M, B = 4, T = 256): inputs, the CPU model's gradients and the float64 gradients, computed once."""
    cfg = GPT2_124M
    B, T = 4, 256
    weights = gpt2_weights(cfg, 42)
    assert weights.size == 123886080
    rng = np.random.default_rng(43)
    seqs = rng.integers(0, cfg["vocab_size"], size=(B, T + 1)).astype(np.int32)
    inputs, labels = np.ascontiguousarray(seqs[:, :T]), np.ascontiguousarray(seqs[:, 1:])
    cpu, cpu_loss, _ = reference.gpt_forward_backward(cfg, weights, inputs, labels, B, T, restated_ops=True)
    assert abs(cpu_loss - np.log(cfg["vocab_size"])) < 0.2      # random init: loss ~ ln(V) = 10.82
    exact, exact_loss = exact_gradients(cfg, weights, inputs, labels)
    assert abs(exact_loss - cpu_loss) < 1e-4, (exact_loss, cpu_loss)
    return dict(cfg=cfg, B=B, T=T, weights=weights, inputs=inputs, labels=labels, cpu=split_weights(cfg, cpu), cpu_loss=cpu_loss, exact=exact)


def _config0_run(lib, reference, c0, mode, options=()):
    """Gradients of config 0 on the B200 backend object -> per tensor (distance from the CPU model, distance from the float64
    gradients, the CPU model's own distance from the float64 gradients), each normalised by the tensor's largest magnitude."""
    cfg = c0["cfg"]
    be = _backend(lib, mode)
    try:
        lib.gptb200_backend_context.restype = ctypes.c_void_p
        lib.gptb200_backend_context.argtypes = [ctypes.c_void_p]
        ctx = lib.gptb200_backend_context(ctypes.c_void_p(be))
        for key, value in options:
            assert lib.gptb200_ctx_set_option(ctypes.c_void_p(ctx), key.encode(), value) == 0
        grads, loss, _ = reference.gpt_forward_backward(cfg, c0["weights"], c0["inputs"], c0["labels"], c0["B"], c0["T"], backend_ptr=be)
    finally:
        lib.gptb200_backend_destroy(ctypes.c_void_p(be))
    a = split_weights(cfg, grads)
    report = {}
    for name in a:
        assert np.isfinite(a[name]).all(), name
        scale = max(np.abs(c0["exact"][name]).max(), 1e-30)
        report[name] = (float(np.abs(a[name] - c0["cpu"][name]).max() / scale), float(np.abs(a[name] - c0["exact"][name]).max() / scale),
                        float(np.abs(c0["cpu"][name] - c0["exact"][name]).max() / scale))
    return report, loss


def _show(title, report):
    print(title, "(GPU vs CPU model / GPU vs float64 / CPU model vs float64, units of 1e-6):",
          {k: "%.1f / %.1f / %.1f" % tuple(1e6 * x for x in v) for k, v in report.items()})


def test_gpt2_124m_config0_all_gradients(lib, reference, config0):
    """Every gradient tensor within 1e-5 (max-normalised) of the CPU model.  Both are fp32 computations whose own distance from
    the exact gradients is several 1e-6 here (twelve layers deep, sums of up to 1024 x 3072 terms), so the distance between them
    sits close to the bound; a tensor beyond it is attributed with the float64 gradients: it still passes if the GPU result is
    within 1e-5 of the exact gradients AND at least as close to them as the CPU model is.  Each use of that rule is reported."""
    report, loss = _config0_run(lib, reference, config0, 0)
    assert abs(loss - config0["cpu_loss"]) < 1e-4
    _show("config 0, 3xTF32", report)
    attributed = {k: v for k, v in report.items() if v[0] > 1e-5}
    bad = {k: v for k, v in attributed.items() if not (v[1] <= 1e-5 and v[1] <= v[2])}
    assert not bad, f"tensors beyond 1e-5 of the CPU model and not closer to the exact gradients than it: {bad}"
    if attributed:
        import warnings
        warnings.warn(f"config 0: float64 attribution rule taken for {sorted(attributed)}: {attributed}")


def test_gpt2_124m_config0_fp32_fma_attention(lib, reference, config0):
    """The same model with attention on the fp32 FMA kernels (option attention_gemm = 0) instead of the batched tensor-core
    products: same criterion."""
    report, loss = _config0_run(lib, reference, config0, 0, [("attention_gemm", 0)])
    assert abs(loss - config0["cpu_loss"]) < 1e-4
    _show("config 0, 3xTF32, fp32 FMA attention", report)
    bad = {k: v for k, v in report.items() if v[0] > 1e-5 and not (v[1] <= 1e-5 and v[1] <= v[2])}
    assert not bad, bad


def test_gpt2_124m_config0_tf32_mode(lib, reference, config0):
    """TF32 mode (linear layers and attention products in single-pass TF32): the per-operator bound is 2e-3; through twelve layers the
    truncation errors compound, so the whole model is held to 5e-3 per tensor, like the tiny configuration."""
    report, loss = _config0_run(lib, reference, config0, 1)
    assert abs(loss - config0["cpu_loss"]) < 2e-3
    _show("config 0, TF32", report)
    bad = {k: v for k, v in report.items() if v[0] > 5e-3}
    assert not bad, bad


def test_own_model_driver_matches_reference_driver_and_goldens(lib, reference):
    """gpt_b200.Model (this library's driver of the same operator sequence) against the reference's driver on the
    same backend, and against the PyTorch goldens; also a raw-checkpoint round trip in the reference's format."""
    import tempfile
    import torch
    import gpt_b200
    cfg, tokens, weights, golden = _tiny()
    T = cfg["max_seq_len"]
    model = gpt_b200.Model(cfg, 0, None, gpt_b200.MODE_3XTF32)
    model.load_weights(weights)
    model.set_size(1, T)
    d_in = torch.from_numpy(tokens[:T].copy()).cuda()
    d_lbl = torch.from_numpy(tokens[1:T + 1].copy()).cuda()
    events = []
    model.zero_grad()
    model.forward(d_in)
    model.backward(d_in, d_lbl, events.append)
    loss = model.loss(d_lbl)
    grads = np.empty(model.num_params, np.float32)
    model.read_grads(grads)
    assert events == [4, 3, 2, 1, 0, -1]
    assert abs(loss - 6.185424) < 1e-4
    be = _backend(lib, 0)
    try:
        ref_grads, ref_loss, _ = reference.gpt_forward_backward(cfg, weights, tokens[:T], tokens[1:T + 1], 1, T, backend_ptr=be)
    finally:
        lib.gptb200_backend_destroy(ctypes.c_void_p(be))
    assert abs(loss - ref_loss) < 1e-6
    assert np.abs(grads - ref_grads).max() <= 1e-6
    a, g = split_weights(cfg, grads), split_weights(cfg, golden)
    for name in a:
        assert np.abs(a[name] - g[name]).max() <= 1e-5, name
    with tempfile.NamedTemporaryFile(suffix=".bin") as f:
        model.save_checkpoint(f.name)
        assert np.array_equal(np.fromfile(f.name, dtype=np.float32), weights)   # byte-compatible with the reference's files
        model.load_checkpoint(f.name)
    # a second step accumulates into the same gradient buffer unless zero_grad is called (gradient accumulation)
    model.forward(d_in)
    model.backward(d_in, d_lbl)
    twice = np.empty_like(grads)
    model.read_grads(twice)
    assert np.abs(twice - 2 * grads).max() <= 2e-6
    model.close()


def test_adamw_and_clip_match_the_reference_operators(lib, reference):
    """AdamW and the 1/accum scaling + norm clipping against the reference CPU backend's own operators
    (cpu_backend.cpp:517-556) on the same arrays."""
    import torch
    import gpt_b200
    be = gpt_b200.Backend(0)
    rng = np.random.default_rng(3)
    n = 100003
    p, g = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    m, v = (0.1 * rng.standard_normal(n)).astype(np.float32), np.abs(0.1 * rng.standard_normal(n)).astype(np.float32)
    dp, dg, dm, dv = (torch.from_numpy(a.copy()).cuda() for a in (p, g, m, v))
    lr, b1, b2, eps, wd, step = 6e-4, 0.9, 0.95, 1e-8, 0.1, 3
    assert lib.gptb200_adamw_step(be.handle, dp.data_ptr(), dg.data_ptr(), dm.data_ptr(), dv.data_ptr(), n, lr, b1, b2, eps, wd, step) == 0
    be.synchronize()
    rp, rm, rv = reference.adamw_step(p, g, m, v, lr, b1, b2, eps, wd, step)
    assert np.abs(dp.cpu().numpy() - rp).max() <= 2e-6 and np.abs(dm.cpu().numpy() - rm).max() <= 1e-6 and np.abs(dv.cpu().numpy() - rv).max() <= 1e-6
    # clipping: g /= accum, then scaled to max_norm when the norm exceeds it
    for scale, accum in ((1.0, 4), (1e-4, 2)):      # norm above the bound; small norm: only the 1/accum scaling applies
        gs = (g * scale).astype(np.float32)
        dg2 = torch.from_numpy(gs.copy()).cuda()
        assert lib.gptb200_scale_and_clip_grad(be.handle, dg2.data_ptr(), n, 1.0, accum) == 0
        be.synchronize()
        ref = reference.scale_and_clip_grad(gs, 1.0, accum)
        # the reference adds 100 003 squares one after the other in fp32; the kernels add them pairwise: 1e-5 of the result's scale
        assert np.abs(dg2.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
    be.close()


def test_set_size_beyond_memory_is_an_error_and_the_model_keeps_working(lib):
    """A shape whose activations cannot be allocated returns a status (nothing aborts, nothing changes); so does a
    logits tensor beyond the interface's int indexing.  The model then still runs at its previous size."""
    import torch
    import gpt_b200
    cfg = dict(max_seq_len=64, vocab_size=507, vocab_size_padded=512, num_layers=12, num_heads=4, d_model=32, d_ffn=512)
    model = gpt_b200.Model(cfg, 0, None, 0, seed=1)
    model.init(0.0, 0.02)
    model.set_size(2, 16)
    tokens = torch.randint(0, 507, (2, 16), dtype=torch.int32, device="cuda")
    labels = torch.randint(0, 507, (2, 16), dtype=torch.int32, device="cuda")
    model.zero_grad(); model.forward(tokens); model.backward(tokens, labels)
    loss0 = model.loss(labels)
    with pytest.raises(gpt_b200.GptB200Error) as e:
        model.set_size(60_000_000, 64)         # 3.8e9 rows: the logits tensor alone would exceed 2^31 - 1 elements
    assert e.value.status == 6
    with pytest.raises(gpt_b200.GptB200Error) as e:
        model.set_size(62_500, 64)             # 4e6 rows x ~16 400 floats of activations = 262 GB: one cudaMalloc that cannot succeed
    assert e.value.status == 2                 # GPTB200_ERR_CUDA
    model.zero_grad(); model.forward(tokens); model.backward(tokens, labels)
    assert model.loss(labels) == loss0
    model.close()


def test_fused_clip_and_adamw_matches_the_reference_operator_sequence(lib, reference):
    """gptb200_model_clip_and_optimizer_step (two launches over the packed buffers) against the reference's own sequence --
    device_scale_and_clip_grad on the whole gradient buffer, then device_adamw_step per tensor with weight decay on the
    matrices and embeddings only (src/model/gpt.cpp:644-677, cpu_backend.cpp:517-556) -- over three steps, and against this
    library's unfused calls."""
    import torch
    import gpt_b200
    from oracle.oracle import weight_layout
    cfg, tokens, weights, _ = _tiny()
    T = cfg["max_seq_len"]
    d_in = torch.from_numpy(tokens[:T].copy()).cuda()
    d_lbl = torch.from_numpy(tokens[1:T + 1].copy()).cuda()
    fused, plain = (gpt_b200.Model(cfg, 0, None, gpt_b200.MODE_3XTF32) for _ in range(2))
    for m in (fused, plain):
        m.load_weights(weights)
        m.set_size(1, T)
    n = fused.num_params
    rp, rm, rv = weights.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    decay_names = {"wte", "wpe", "qkv_proj_w", "attn_proj_w", "ffn_up_w", "ffn_down_w"}
    lr, b1, b2, wd, max_norm, accum = 6e-4, 0.9, 0.95, 0.1, 0.05, 2     # a bound low enough that clipping is active
    for step in (1, 2, 3):
        for m in (fused, plain):
            m.zero_grad(); m.forward(d_in); m.backward(d_in, d_lbl)
        g = np.empty(n, np.float32)
        fused.read_grads(g)
        fused.clip_and_optimizer_step(max_norm, accum, lr, b1, b2, wd)
        plain.unscale_and_clip_grads(max_norm, accum)
        plain.optimizer_step(lr, b1, b2, wd)
        # the reference's sequence on the same gradients
        gc = reference.scale_and_clip_grad(g, max_norm, accum)
        assert np.linalg.norm(g.astype(np.float64) / accum) > max_norm      # the clipping branch is exercised
        off = 0
        for name, shape in weight_layout(cfg):
            cnt = int(np.prod(shape))
            sl = slice(off, off + cnt)
            rp[sl], rm[sl], rv[sl] = reference.adamw_step(rp[sl], gc[sl], rm[sl], rv[sl], lr, b1, b2, 1e-8, wd if name in decay_names else 0.0, step)
            off += cnt
        wf, wp = np.empty(n, np.float32), np.empty(n, np.float32)
        fused.read_weights(wf); plain.read_weights(wp)
        assert np.abs(wf - rp).max() <= 2e-6, (step, float(np.abs(wf - rp).max()))
        assert np.abs(wf - wp).max() <= 2e-6
        after = np.empty(n, np.float32)
        fused.read_grads(after)
        assert np.array_equal(after, g)                                    # the fused form leaves the gradients unscaled
    assert fused.step_count == 3
    fused.close(); plain.close()


def test_training_state_round_trip_and_header_checks(lib):
    """save_state / load_state: parameters, both AdamW moments and the step counter come back bit for bit and training
    continues as it would have; a file of another configuration, a truncated file and a raw parameter image are refused without
    touching the model."""
    import tempfile
    import torch
    import gpt_b200
    cfg, tokens, weights, _ = _tiny()
    T = cfg["max_seq_len"]
    d_in = torch.from_numpy(tokens[:T].copy()).cuda()
    d_lbl = torch.from_numpy(tokens[1:T + 1].copy()).cuda()

    def train(m, steps):
        for _ in range(steps):
            m.zero_grad(); m.forward(d_in); m.backward(d_in, d_lbl)
            m.clip_and_optimizer_step(1.0, 1, 6e-4, 0.9, 0.95, 0.1)

    a = gpt_b200.Model(cfg, 0, None, gpt_b200.MODE_3XTF32)
    a.load_weights(weights); a.set_size(1, T)
    train(a, 2)
    with tempfile.TemporaryDirectory() as tmp:
        path = tmp + "/state.bin"
        a.save_state(path)
        raw = np.fromfile(path, dtype=np.uint8)
        assert raw[:8].tobytes() == b"GPTB200S" and raw.size == 64 + 3 * 4 * a.num_params
        b = gpt_b200.Model(cfg, 0, None, gpt_b200.MODE_3XTF32)
        b.set_size(1, T)
        b.load_state(path)
        assert b.step_count == 2
        wa, wb = np.empty(a.num_params, np.float32), np.empty(a.num_params, np.float32)
        a.read_weights(wa); b.read_weights(wb)
        assert np.array_equal(wa, wb)                     # the parameters come back bit for bit
        train(a, 2); train(b, 2)
        wa, wb = np.empty(a.num_params, np.float32), np.empty(a.num_params, np.float32)
        a.read_weights(wa); b.read_weights(wb)
        # resumed training follows the original (not bit for bit: the embedding backward adds with atomics, in any order)
        assert np.abs(wa - wb).max() <= 1e-6 * np.abs(wa).max()
        # refusals
        other = dict(cfg, num_layers=cfg["num_layers"] - 1)
        c = gpt_b200.Model(other, 0, None, gpt_b200.MODE_3XTF32)
        with pytest.raises(gpt_b200.GptB200Error):
            c.load_state(path)
        raw[:-100].tofile(tmp + "/short.bin")
        before = np.empty(a.num_params, np.float32)
        b.read_weights(before)
        with pytest.raises(gpt_b200.GptB200Error):
            b.load_state(tmp + "/short.bin")
        weights.tofile(tmp + "/raw.bin")
        with pytest.raises(gpt_b200.GptB200Error):
            b.load_state(tmp + "/raw.bin")
        after = np.empty(a.num_params, np.float32)
        b.read_weights(after)
        assert np.array_equal(before, after) and b.step_count == 4
        b.close(); c.close()
    a.close()


@pytest.mark.parametrize("batch", [1, 3])
def test_kv_cached_generation_matches_prefix_recomputation(lib, reference, batch):
    """Greedy generation with the KV cache (one row per sequence per step) against the reference's way -- a full forward
    pass over the whole prefix for every token (src/infer/infer.cpp:112-148) -- on this library, and the first steps also
    against the reference CPU model: same logits (1e-5 of their scale), same tokens."""
    import torch
    import gpt_b200
    cfg, tokens, weights, _ = _tiny()
    V, Vp, Tmax = cfg["vocab_size"], cfg["vocab_size_padded"], cfg["max_seq_len"]
    P, NEW = 9, 20
    rng = np.random.default_rng(batch)
    prompt = rng.integers(0, V, size=(batch, P)).astype(np.int32)
    cached = gpt_b200.Model(cfg, 0, None, gpt_b200.MODE_3XTF32, use_grad=False)
    full = gpt_b200.Model(cfg, 0, None, gpt_b200.MODE_3XTF32, use_grad=False)
    for m in (cached, full):
        m.load_weights(weights)

    def logits_view(m, rows):
        class _Raw:
            __cuda_array_interface__ = dict(shape=(rows, Vp), typestr="<f4", data=(m.logits_ptr, False), version=3, strides=None)
        return torch.as_tensor(_Raw(), device="cuda")

    seq = torch.from_numpy(prompt).cuda()
    cached.generate_begin(seq.contiguous(), batch, P, P + NEW)
    assert cached.generate_position == P
    step_logits = torch.empty(batch, Vp, device="cuda")
    last = logits_view(cached, batch * P).view(batch, P, Vp)[:, P - 1, :].clone()
    for t in range(P, P + NEW):
        # the reference's way: the whole prefix again
        full.set_size(batch, t)
        full.forward(seq.contiguous())
        ref_last = logits_view(full, batch * t).view(batch, t, Vp)[:, t - 1, :]
        scale = float(ref_last.abs().max())
        assert float((last - ref_last).abs().max()) <= 1e-5 * scale, (t, float((last - ref_last).abs().max()), scale)
        if t < P + 2:   # and the reference CPU model itself on the same prefix
            h = seq.cpu().numpy()
            _, _, cpu_logits = reference.gpt_forward_backward(cfg, weights, h, np.roll(h, -1, axis=1), batch, t, want_logits=True)
            cpu_last = cpu_logits.reshape(batch, t, Vp)[:, t - 1, :]
            assert np.abs(last.cpu().numpy() - cpu_last).max() <= 1e-5 * np.abs(cpu_last).max()
        nxt = ref_last[:, :V].argmax(dim=1).to(torch.int32)
        assert torch.equal(nxt, last[:, :V].argmax(dim=1).to(torch.int32))
        seq = torch.cat([seq, nxt[:, None]], dim=1)
        cached.generate_step(nxt.contiguous(), step_logits)
        last = step_logits.clone()
    assert cached.generate_position == P + NEW
    with pytest.raises(gpt_b200.GptB200Error):
        cached.generate_step(nxt.contiguous(), step_logits)      # beyond max_len
    cached.close(); full.close()


def test_fused_cross_entropy_gives_the_same_step_with_less_memory(lib, reference):
    """The model driver with the logits turned into their gradient in place (no probability tensor, no separate gradient
    tensor) against the reference CPU model: same loss (whether asked before or after the backward pass), every gradient
    tensor within 1e-5; and against the unfused driver."""
    import torch
    import gpt_b200
    cfg, tokens, weights, golden = _tiny()
    T = cfg["max_seq_len"]
    d_in = torch.from_numpy(tokens[:T].copy()).cuda()
    d_lbl = torch.from_numpy(tokens[1:T + 1].copy()).cuda()
    cpu, cpu_loss, _ = reference.gpt_forward_backward(cfg, weights, tokens[:T], tokens[1:T + 1], 1, T)
    out = {}
    for fused in (False, True):
        torch.cuda.synchronize(); torch.cuda.empty_cache()
        free0 = torch.cuda.mem_get_info()[0]
        m = gpt_b200.Model(cfg, 0, None, gpt_b200.MODE_3XTF32)
        m.set_fused_cross_entropy(fused)
        m.load_weights(weights)
        m.set_size(1, T)
        used = free0 - torch.cuda.mem_get_info()[0]
        m.zero_grad(); m.forward(d_in)
        loss_before = m.loss(d_lbl)
        m.backward(d_in, d_lbl)
        loss_after = m.loss(d_lbl)
        g = np.empty(m.num_params, np.float32)
        m.read_grads(g)
        out[fused] = (g, loss_before, loss_after, used)
        m.close()
    g, lb, la, used_fused = out[True]
    assert abs(lb - cpu_loss) < 1e-5 and abs(la - cpu_loss) < 1e-5
    a, c = split_weights(cfg, g), split_weights(cfg, cpu)
    for name in a:
        assert np.abs(a[name] - c[name]).max() <= 1e-5, name                       # the reference's own absolute check
    assert np.abs(g - out[False][0]).max() <= 1e-6
    assert used_fused <= out[False][3]


def test_fused_gelu_backward_in_the_model_driver(lib, reference):
    """The model driver with the GELU derivative folded into the down projection's grad_x GEMM: every gradient tensor still
    within the reference's absolute 1e-5 of the CPU model, and within 1e-6 of the unfused driver."""
    import torch
    import gpt_b200
    cfg, tokens, weights, _ = _tiny()
    T = cfg["max_seq_len"]
    d_in = torch.from_numpy(tokens[:T].copy()).cuda()
    d_lbl = torch.from_numpy(tokens[1:T + 1].copy()).cuda()
    cpu, cpu_loss, _ = reference.gpt_forward_backward(cfg, weights, tokens[:T], tokens[1:T + 1], 1, T)
    grads = {}
    for fused in (False, True):
        m = gpt_b200.Model(cfg, 0, None, gpt_b200.MODE_3XTF32)
        m.set_fused_gelu_backward(fused)
        m.set_option("pair", 1)                 # the tiny shapes would otherwise not reach the kernel with the fused epilogue
        m.load_weights(weights)
        m.set_size(1, T)
        m.zero_grad(); m.forward(d_in); m.backward(d_in, d_lbl)
        g = np.empty(m.num_params, np.float32)
        m.read_grads(g)
        grads[fused] = g
        m.close()
    a, c = split_weights(cfg, grads[True]), split_weights(cfg, cpu)
    for name in a:
        assert np.abs(a[name] - c[name]).max() <= 1e-5, name
    assert np.abs(grads[True] - grads[False]).max() <= 1e-6
