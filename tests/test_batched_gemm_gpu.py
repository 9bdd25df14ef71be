"""Batched products on the CTA-pair tensor-core kernel (gptb200_gemm_batched): every operand form, ragged extents, contiguous
batches and per-head slices of packed qkv rows, against exactly rounded float64 products.

Tolerances as for the linear layers: max|a - b| <= tol * max|ref| per tensor, 1e-5 in 3xTF32 mode, 2e-3 in TF32 mode.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = {0: 1e-5, 1: 2e-3}


@pytest.fixture(scope="module")
def torch():
    import torch as t
    assert t.cuda.is_available(), "GPU tests need a CUDA device"
    return t


@pytest.fixture(scope="module", params=[0, 1], ids=["3xTF32", "TF32"])
def be(request, torch, built_library):
    import gpt_b200
    b = gpt_b200.Backend(0, None, request.param)
    b.mode = request.param
    yield b
    b.close()


def rel_err(a, ref):
    return float((a.double() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)], ids=["K.K", "K.MN", "MN.MN"])
@pytest.mark.parametrize("batches,m,n,k", [(1, 600, 300, 72), (3, 256, 256, 64), (5, 200, 136, 100), (4, 256, 96, 256), (2, 300, 32, 64), (12, 1024, 1024, 64), (2, 1024, 64, 1024), (150, 64, 64, 32)])
def test_contiguous_batches(be, torch, a_mn, b_mn, batches, m, n, k):
    g = torch.Generator(device="cuda").manual_seed(batches * 1000 + m + n + k)
    a = torch.randn(batches, k, m, device="cuda", generator=g) if a_mn else torch.randn(batches, m, k, device="cuda", generator=g)
    b = torch.randn(batches, k, n, device="cuda", generator=g) if b_mn else torch.randn(batches, n, k, device="cuda", generator=g)
    out = torch.full((batches, m, n), float("nan"), device="cuda")
    sa = (m if a_mn else k, a[0].numel(), a[0].numel())
    sb = (n if b_mn else k, b[0].numel(), b[0].numel())
    be.gemm_batched(out, a, b, m, n, k, a_mn, b_mn, 1, batches, sa, sb, (n, m * n, m * n))
    be.synchronize()
    A = a.double().transpose(1, 2) if a_mn else a.double()
    B = b.double() if b_mn else b.double().transpose(1, 2)
    ref = torch.bmm(A, B)
    assert torch.isfinite(out).all()
    e = rel_err(out, ref)
    assert e <= TOL[be.mode], (e, a_mn, b_mn, batches, m, n, k)


@pytest.mark.parametrize("B,T,H", [(2, 256, 12), (3, 200, 4), (1, 1024, 12)])
def test_head_slices_of_packed_rows(be, torch, oracle, B, T, H):
    """The products of causal attention taken straight from the packed [B, T, 3 * D] qkv rows: S = Q . K^T per (sequence, head)
    into [B][T][H][T] scores, then O = S . V back into [B, T, D] rows (no softmax here: the addressing is what is tested)."""
    hd = 64
    D = H * hd
    g = torch.Generator(device="cuda").manual_seed(B * 100 + T + H)
    qkv = torch.randn(B, T, 3 * D, device="cuda", generator=g)
    s = torch.full((B, T, H, T), float("nan"), device="cuda")
    q, k, v = qkv[..., :D], qkv[..., D:2 * D], qkv[..., 2 * D:]
    head = (3 * D, hd, T * 3 * D)                      # row pitch, head stride, sequence stride
    be.gemm_batched(s, q, k, T, T, hd, False, False, H, B, head, head, (H * T, T, T * H * T))
    o = torch.full((B, T, D), float("nan"), device="cuda")
    be.gemm_batched(o, s, v, T, hd, T, False, True, H, B, (H * T, T, T * H * T), head, (D, hd, T * D))
    be.synchronize()
    qh = q.reshape(B, T, H, hd).permute(0, 2, 1, 3).double()
    kh = k.reshape(B, T, H, hd).permute(0, 2, 1, 3).double()
    vh = v.reshape(B, T, H, hd).permute(0, 2, 1, 3).double()
    s_ref = qh @ kh.transpose(-1, -2)                  # [B, H, T, T]
    assert rel_err(s.permute(0, 2, 1, 3), s_ref) <= TOL[be.mode]
    o_ref = (s.permute(0, 2, 1, 3).double() @ vh).permute(0, 2, 1, 3).reshape(B, T, D)
    assert rel_err(o, o_ref) <= TOL[be.mode]
    # the same two products of single heads by the oracle's linear operator (the reference's summation order)
    for b, h in ((0, 0), (B - 1, H - 1)):
        q_bh = np.ascontiguousarray(q[b, :, h * hd:(h + 1) * hd].cpu().numpy())
        k_bh = np.ascontiguousarray(k[b, :, h * hd:(h + 1) * hd].cpu().numpy())
        v_bh = np.ascontiguousarray(v[b, :, h * hd:(h + 1) * hd].cpu().numpy())
        s_or, _ = oracle.linear_forward(q_bh, np.ascontiguousarray(k_bh.T), np.zeros(T, np.float32), False)
        got = s[b, :, h, :].cpu().numpy().astype(np.float64)
        assert np.abs(got - s_or).max() / np.abs(s_or).max() <= TOL[be.mode]
        o_or, _ = oracle.linear_forward(np.ascontiguousarray(s[b, :, h, :].cpu().numpy()), v_bh, np.zeros(hd, np.float32), False)
        got = o[b, :, h * hd:(h + 1) * hd].cpu().numpy().astype(np.float64)
        assert np.abs(got - o_or).max() / np.abs(o_or).max() <= TOL[be.mode]


def test_bad_arguments_are_refused(be, torch):
    import gpt_b200
    x = torch.zeros(4, 64, 64, device="cuda")
    with pytest.raises(gpt_b200.GptB200Error):
        be.gemm_batched(x, x, x, 64, 64, 64, True, False, 1, 4, (64, 4096, 4096), (64, 4096, 4096), (64, 4096, 4096))   # (MN, K) does not occur
    with pytest.raises(gpt_b200.GptB200Error):
        be.gemm_batched(x, x, x, 64, 64, 64, False, False, 1, 4, (66, 4096, 4096), (64, 4096, 4096), (64, 4096, 4096))  # pitch not a multiple of 4 floats
