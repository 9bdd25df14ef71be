"""GPU tests of the plain (non-linear-path) operators against the reference CPU backend, operator by operator:
embedding forward / backward, LayerNorm + residual forward / backward, causal attention forward / backward, softmax,
cross-entropy backward and loss.  Tolerance 1e-5 (max-normalised per tensor); these kernels use fp32 arithmetic only."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

_f = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


@pytest.fixture(scope="module")
def env(built_library, reference):
    import torch
    import gpt_b200
    assert torch.cuda.is_available()
    be = gpt_b200.Backend(0)
    yield torch, be, be.lib, reference.lib
    be.close()


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(name, got, ref, tol=1e-5):
    got = got.cpu().numpy().astype(np.float64) if hasattr(got, "cpu") else np.asarray(got, np.float64)
    assert np.isfinite(got).all(), name
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err <= tol, f"{name}: {err:.3e}"


@pytest.mark.parametrize("batch,seq,d,vp", [(2, 64, 32, 512), (3, 50, 768, 1000)])
def test_embedding(env, batch, seq, d, vp):
    torch, be, lib, ref = env
    rng = np.random.default_rng(1)
    wte, wpe = rng.standard_normal((vp, d), dtype=np.float32), rng.standard_normal((seq, d), dtype=np.float32)
    tok = rng.integers(0, vp - 5, size=(batch, seq)).astype(np.int32)
    y_ref = np.empty((batch, seq, d), np.float32)
    ref.ref_embedding_forward.argtypes = [_f, _f, _f, _i] + [ctypes.c_int] * 3
    ref.ref_embedding_forward(y_ref, wte, wpe, tok, batch, seq, d)
    y, dtok = torch.empty(batch, seq, d, device="cuda"), dev(torch, tok)
    assert lib.gptb200_embedding_forward(be.handle, y.data_ptr(), dev(torch, wte).data_ptr(), dev(torch, wpe).data_ptr(), dtok.data_ptr(), batch, seq, d) == 0
    be.synchronize()
    assert np.array_equal(y.cpu().numpy(), y_ref)       # one add per element: bit-exact
    gy = rng.standard_normal((batch, seq, d), dtype=np.float32)
    gwte0, gwpe0 = rng.standard_normal((vp, d), dtype=np.float32), rng.standard_normal((seq, d), dtype=np.float32)
    gwte_ref, gwpe_ref = gwte0.copy(), gwpe0.copy()
    ref.ref_embedding_backward.argtypes = [_f, _f, _f, _i] + [ctypes.c_int] * 3
    ref.ref_embedding_backward(gwte_ref, gwpe_ref, gy, tok, batch, seq, d)
    gwte, gwpe = dev(torch, gwte0), dev(torch, gwpe0)
    assert lib.gptb200_embedding_backward(be.handle, gwte.data_ptr(), gwpe.data_ptr(), dev(torch, gy).data_ptr(), dtok.data_ptr(), batch, seq, d) == 0
    be.synchronize()
    close("grad_wte", gwte, gwte_ref)
    close("grad_wpe", gwpe, gwpe_ref)


@pytest.mark.parametrize("rows,d,with_residual", [(64, 32, True), (200, 768, True), (33, 100, False), (100, 128, False), (1000, 1024, True),
                                                   (5, 768, True), (4100, 768, False), (64, 1152, True)])
def test_layernorm(env, rows, d, with_residual):
    torch, be, lib, ref = env
    rng = np.random.default_rng(2)
    x0 = rng.standard_normal((rows, d), dtype=np.float32)
    res = rng.standard_normal((rows, d), dtype=np.float32) if with_residual else None
    gamma, beta = rng.standard_normal(d, dtype=np.float32), rng.standard_normal(d, dtype=np.float32)
    x_ref, y_ref, mean_ref, var_ref = x0.copy(), np.empty((rows, d), np.float32), np.empty(rows, np.float32), np.empty(rows, np.float32)
    ref.ref_layernorm_forward.argtypes = [_f, _f, _f, _f, ctypes.c_void_p, _f, _f, ctypes.c_int, ctypes.c_int]
    ref.ref_layernorm_forward(y_ref, mean_ref, var_ref, x_ref, res.ctypes.data if with_residual else None, gamma, beta, rows, d)
    x, y = dev(torch, x0), torch.empty(rows, d, device="cuda")
    mean, var = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    dres = dev(torch, res) if with_residual else None
    dg, db = dev(torch, gamma), dev(torch, beta)
    assert lib.gptb200_layernorm_forward(be.handle, y.data_ptr(), mean.data_ptr(), var.data_ptr(), x.data_ptr(), dres.data_ptr() if with_residual else None,
                                         dg.data_ptr(), db.data_ptr(), rows, d) == 0
    be.synchronize()
    close("y", y, y_ref)
    close("x (in-place residual add)", x, x_ref, 1e-7)
    close("means", mean, mean_ref)
    close("vars", var, var_ref)
    gy = rng.standard_normal((rows, d), dtype=np.float32)
    gres = rng.standard_normal((rows, d), dtype=np.float32) if with_residual else None
    gg0, gb0 = rng.standard_normal(d, dtype=np.float32), rng.standard_normal(d, dtype=np.float32)
    gx_ref, gg_ref, gb_ref = np.empty((rows, d), np.float32), gg0.copy(), gb0.copy()
    ref.ref_layernorm_backward.argtypes = [_f, _f, _f, _f, ctypes.c_void_p, _f, _f, _f, _f, ctypes.c_int, ctypes.c_int]
    ref.ref_layernorm_backward(gx_ref, gg_ref, gb_ref, gy, gres.ctypes.data if with_residual else None, x_ref, mean_ref, var_ref, gamma, rows, d)
    gx, gg, gb = torch.empty(rows, d, device="cuda"), dev(torch, gg0), dev(torch, gb0)
    dgres = dev(torch, gres) if with_residual else None
    assert lib.gptb200_layernorm_backward(be.handle, gx.data_ptr(), gg.data_ptr(), gb.data_ptr(), dev(torch, gy).data_ptr(),
                                          dgres.data_ptr() if with_residual else None, x.data_ptr(), mean.data_ptr(), var.data_ptr(), dg.data_ptr(), rows, d) == 0
    be.synchronize()
    close("grad_x", gx, gx_ref)
    close("grad_gamma", gg, gg_ref)
    close("grad_beta", gb, gb_ref)


# head size 64 has three sets of kernels: batched tensor-core products + row kernels (in either precision mode of the linear
# layers: the products then carry that mode's accuracy), register-tiled fp32 FMA kernels, one row per thread group
@pytest.mark.parametrize("kernels", ["gemm", "gemm-tf32", "gemm-grouped", "tiled", "rows"])
@pytest.mark.parametrize("batch,seq,d,heads", [(1, 64, 32, 4), (2, 100, 128, 2), (2, 256, 768, 12), (1, 37, 64, 4), (3, 130, 192, 3), (1, 1, 64, 1),
                                               (2, 260, 128, 2), (1, 512, 128, 2), (1, 1024, 64, 1), (3, 36, 64, 1), (5, 4, 192, 3), (7, 128, 128, 2)])
def test_attention(env, batch, seq, d, heads, kernels):
    torch, be, lib, ref = env
    if kernels.startswith("gemm") and (d // heads != 64 or seq % 4):
        pytest.skip("the tensor-core form covers head size 64 and sequence lengths that are multiples of 4")
    be.set_option("attention_gemm", 1 if kernels.startswith("gemm") else 0)
    be.set_option("attention_tiled", int(kernels != "rows"))
    be.set_option("attention_group_mb", 1 if kernels == "gemm-grouped" else 8192)   # 1 MB: a few sequences (or one) per group of launches
    tol = 2e-3 if kernels == "gemm-tf32" else 1e-5
    be.set_mode(1 if kernels == "gemm-tf32" else 0)
    try:
        _attention_case(torch, be, lib, ref, batch, seq, d, heads, tol)
    finally:
        be.set_mode(0)
        be.set_option("attention_gemm", 1)
        be.set_option("attention_tiled", 1)
        be.set_option("attention_group_mb", 8192)


def _attention_case(torch, be, lib, ref, batch, seq, d, heads, tol):
    rng = np.random.default_rng(3)
    qkv = rng.standard_normal((batch, seq, 3 * d), dtype=np.float32)
    y_ref, lse_ref = np.empty((batch, seq, d), np.float32), np.empty((batch, seq, heads), np.float32)
    ref.ref_attention_forward.argtypes = [_f, _f, _f] + [ctypes.c_int] * 4
    ref.ref_attention_forward(y_ref, lse_ref, qkv, batch, seq, d, heads)
    dqkv, y, lse = dev(torch, qkv), torch.empty(batch, seq, d, device="cuda"), torch.empty(batch, seq, heads, device="cuda")
    assert lib.gptb200_attention_forward(be.handle, y.data_ptr(), lse.data_ptr(), dqkv.data_ptr(), batch, seq, d, heads) == 0
    be.synchronize()
    close("y", y, y_ref, tol)
    close("logsumexp", lse, lse_ref, tol)
    gy = rng.standard_normal((batch, seq, d), dtype=np.float32)
    gq_ref, dc_ref = np.empty((batch, seq, 3 * d), np.float32), np.empty((batch, seq, heads), np.float32)
    ref.ref_attention_backward.argtypes = [_f, _f, _f, _f, _f, _f] + [ctypes.c_int] * 4
    ref.ref_attention_backward(gq_ref, dc_ref, lse_ref, gy, y_ref, qkv, batch, seq, d, heads)
    gq, dc = torch.empty(batch, seq, 3 * d, device="cuda"), torch.empty(batch, seq, heads, device="cuda")
    assert lib.gptb200_attention_backward(be.handle, gq.data_ptr(), dc.data_ptr(), lse.data_ptr(), dev(torch, gy).data_ptr(), y.data_ptr(), dqkv.data_ptr(),
                                          batch, seq, d, heads) == 0
    be.synchronize()
    close("grad_qkv", gq, gq_ref, tol)
    close("D", dc, dc_ref, tol)


def test_attention_rejects_unsupported_head_size(env):
    torch, be, lib, _ = env
    t = torch.zeros(4 * 3 * 48, device="cuda")
    assert lib.gptb200_attention_forward(be.handle, t.data_ptr(), t.data_ptr(), t.data_ptr(), 1, 4, 48, 2) == 1   # head size 24


@pytest.mark.parametrize("rows,v,vp", [(64, 507, 512), (20, 50257, 50304)])
def test_softmax_and_cross_entropy(env, reference, rows, v, vp):
    torch, be, lib, ref = env
    rng = np.random.default_rng(4)
    logits = (3 * rng.standard_normal((rows, vp))).astype(np.float32)
    labels = rng.integers(0, v, size=rows).astype(np.int32)
    p_ref = reference.softmax_forward(logits, v)
    g_ref = reference.cross_entropy_softmax_backward(p_ref, labels, v)
    loss_ref = np.zeros(1, np.float32)
    ref.ref_cross_entropy_loss.argtypes = [_f, _f, _i, ctypes.c_int, ctypes.c_int]
    ref.ref_cross_entropy_loss(loss_ref, p_ref, labels, rows, vp)
    dl, p, g = dev(torch, logits), torch.full((rows, vp), float("nan"), device="cuda"), torch.zeros(rows, vp, device="cuda")
    dlab, loss = dev(torch, labels), torch.zeros(1, device="cuda")
    assert lib.gptb200_softmax_forward(be.handle, p.data_ptr(), dl.data_ptr(), rows, v, vp) == 0
    assert lib.gptb200_cross_entropy_softmax_backward(be.handle, g.data_ptr(), p.data_ptr(), dlab.data_ptr(), rows, v, vp) == 0
    assert lib.gptb200_cross_entropy_loss(be.handle, loss.data_ptr(), p.data_ptr(), dlab.data_ptr(), rows, vp) == 0
    be.synchronize()
    # The reference adds the row's exponentials one after another in fp32; over 50k columns that sum is itself some 1e-5 off.
    # So the GPU result is held to 1e-5 of the fp64 value, and to the reference within the reference's own distance from fp64.
    z = logits[:, :v].astype(np.float64)
    e64 = np.exp(z - z.max(axis=1, keepdims=True))
    p64 = np.zeros((rows, vp))
    p64[:, :v] = e64 / e64.sum(axis=1, keepdims=True)
    ref_off = np.abs(p_ref - p64).max() / p64.max()
    close("probs vs fp64", p, p64)
    close("probs vs reference", p, p_ref, max(1e-5, 2 * ref_off))
    assert bool((p[:, v:] == 0).all())                  # padding columns are zero
    close("grad_logits", g, g_ref, max(1e-5, 2 * ref_off))
    assert abs(float(loss.item()) - float(loss_ref[0])) <= 1e-5 * abs(float(loss_ref[0]))


@pytest.mark.parametrize("rows,v,vp", [(64, 507, 512), (8, 50257, 50304), (5, 130, 131), (16, 4097, 4100), (1, 3, 4)])
def test_fused_softmax_cross_entropy_in_place(env, reference, rows, v, vp):
    """gptb200_softmax_cross_entropy_inplace against the reference's three operators in sequence (softmax forward,
    cross-entropy backward, loss: cpu_backend.cpp:439-509) on the same logits: same gradient (zero padding columns), same
    loss; and the loss computed straight from untouched logits."""
    torch, be, lib, ref = env
    rng = np.random.default_rng(rows + v)
    logits = (3.0 * rng.standard_normal((rows, vp))).astype(np.float32)
    logits[:, v:] = 7.0                       # padding columns hold something: they must come out as zero
    labels = rng.integers(0, v, size=rows).astype(np.int32)
    probs = reference.softmax_forward(logits, v)
    g_ref = reference.cross_entropy_softmax_backward(probs, labels, v)
    loss_ref = np.zeros(1, np.float32)
    ref.ref_cross_entropy_loss.argtypes = [_f, _f, _i, ctypes.c_int, ctypes.c_int]
    ref.ref_cross_entropy_loss(loss_ref, probs, labels, rows, vp)
    x, lab = dev(torch, logits), dev(torch, labels)
    row_loss, loss = torch.empty(rows, device="cuda"), torch.zeros(1, device="cuda")
    assert lib.gptb200_cross_entropy_loss_from_logits(be.handle, loss.data_ptr(), row_loss.data_ptr(), x.data_ptr(), lab.data_ptr(), rows, v, vp) == 0
    be.synchronize()
    assert abs(float(loss) - float(loss_ref[0])) <= 1e-5 * abs(float(loss_ref[0]))
    assert np.array_equal(x.cpu().numpy(), logits)                                      # untouched
    row_loss.zero_(); loss.zero_()
    assert lib.gptb200_softmax_cross_entropy_inplace(be.handle, x.data_ptr(), row_loss.data_ptr(), lab.data_ptr(), rows, v, vp) == 0
    assert lib.gptb200_row_loss_mean(be.handle, loss.data_ptr(), row_loss.data_ptr(), rows) == 0
    be.synchronize()
    # exact (float64) result: the reference adds the v exponentials one after the other in fp32, which at v = 50257 is itself
    # about 1e-5 from it; a miss against the reference passes only if the GPU is within 1e-5 of the exact result AND at least as
    # close to it as the reference is
    z = logits[:, :v].astype(np.float64)
    p = np.exp(z - z.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    p[np.arange(rows), labels] -= 1.0
    exact = np.zeros((rows, vp))
    exact[:, :v] = p / rows
    got = x.cpu().numpy().astype(np.float64)
    scale = np.abs(exact).max()
    e_ref, e_gpu, e_oracle = np.abs(got - g_ref).max() / scale, np.abs(got - exact).max() / scale, np.abs(g_ref - exact).max() / scale
    assert e_ref <= 1e-5 or (e_gpu <= 1e-5 and e_gpu <= e_oracle), (e_ref, e_gpu, e_oracle)
    assert bool((x[:, v:] == 0).all())
    assert abs(float(loss) - float(loss_ref[0])) <= 1e-5 * abs(float(loss_ref[0]))
