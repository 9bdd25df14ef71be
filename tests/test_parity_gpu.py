"""GPU parity tests: the CUDA path, called through the C ABI (ctypes), against the CPU oracle.

Tolerances (per tensor, max|a - b| <= tol * max|ref|, the criterion the task states for this path):
  3xTF32 mode (default): 1e-5      TF32 mode: 2e-3
Additionally the reference's own absolute check (|a - b| <= 1e-5 per element, src/model/gpt_test.cpp:37) is
applied where magnitudes are O(1) or below (the reference's test shapes).
"""
import glob
import os

import numpy as np
import pytest

from conftest import GOLDEN

pytestmark = pytest.mark.gpu

TOL = {0: 1e-5, 1: 2e-3}   # gptb200_mode -> relative tolerance
MODE_NAME = {0: "3xTF32", 1: "TF32"}


@pytest.fixture(scope="module")
def torch():
    import torch as t
    assert t.cuda.is_available(), "GPU tests need a CUDA device"
    return t


# (precision mode, kernel choice, k-range cutting): automatic choice in both modes, plus the CTA-pair (cta_group::2) kernel
# and the one-CTA kernel forced, so that every shape below runs through both GEMM kernels; the pair kernel once with whole
# tiles per pair and once with every pair's k-block range cut as finely as possible (tiles summed from several pairs' parts).
# Two more variants force the 3xTF32 pair kernel to take the correction tiles of operand A, or of operand B, from the pass that
# splits an operand before the launch (option "presplit"), whatever the shape; the automatic choice runs in the others.
@pytest.fixture(scope="module", params=[(0, 0, 0, 0), (1, 0, 0, 0), (0, 1, -1, 0), (1, 1, -1, 0), (0, 1, 1, 0), (1, 1, 1, 0), (0, -1, 0, 0),
                                        (0, 1, 1, 2), (0, 1, -1, 3), (0, 1, 0, 1)],
                ids=["3xTF32", "TF32", "3xTF32-pair", "TF32-pair", "3xTF32-pair-cut", "TF32-pair-cut", "3xTF32-single",
                     "3xTF32-pair-cut-splitA", "3xTF32-pair-splitB", "3xTF32-pair-autosplit"])
def be(request, torch, built_library):
    import gpt_b200
    mode, pair, stream_k, presplit = request.param
    b = gpt_b200.Backend(0, None, mode)
    b.set_option("pair", pair)
    b.set_option("stream_k", stream_k)
    b.set_option("presplit", presplit)
    b.mode = mode
    yield b
    b.close()


ATTRIBUTED = []   # every use of check()'s attribution rule in this run (reported at the end of the module)


@pytest.fixture(scope="module", autouse=True)
def _report_attributed():
    yield
    if ATTRIBUTED:
        import warnings
        warnings.warn("the fp64 attribution rule of check() was taken %d time(s): %s" % (
            len(ATTRIBUTED), "; ".join(f"{n} [{m}] oracle {e:.2e} gpu-exact {g:.2e} oracle-exact {o:.2e}" for n, m, e, g, o in ATTRIBUTED)))


def rel_err(a, ref):
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = max(np.abs(ref).max(), 1e-30) if ref.size else 1.0
    return float(np.abs(a - ref).max() / denom) if ref.size else 0.0


def check(name, got, ref, mode, absolute=False, exact=None):
    """`exact` (float64, optional) is the exactly-rounded result.  For reductions tens of thousands of terms
    long the oracle's own sequential fp32 sum is several 1e-6 away from it, so a miss of the 1e-5 bound
    against the oracle is attributed: it still passes if the GPU result is within 1e-5 of the exact result
    AND at least as close to it as the oracle is."""
    assert got.shape == ref.shape, name
    assert np.isfinite(got).all(), f"{name}: non-finite output"
    e = rel_err(got, ref)
    if e > TOL[mode] and exact is not None:
        e_gpu, e_oracle = rel_err(got, exact), rel_err(ref, exact)
        ATTRIBUTED.append((name, MODE_NAME[mode], e, e_gpu, e_oracle))
        print(f"\n[attribution rule taken] {name} [{MODE_NAME[mode]}]: vs oracle {e:.3e} > {TOL[mode]:.0e}; GPU vs exact {e_gpu:.3e}, oracle vs exact {e_oracle:.3e}")
        assert e_gpu <= TOL[mode] and e_gpu <= e_oracle, (
            f"{name} [{MODE_NAME[mode]}]: vs oracle {e:.3e}, GPU vs exact {e_gpu:.3e}, oracle vs exact {e_oracle:.3e}")
    else:
        assert e <= TOL[mode], f"{name} [{MODE_NAME[mode]}]: rel err {e:.3e} > {TOL[mode]:.0e}"
    if absolute and mode == 0:
        assert np.abs(got.astype(np.float64) - ref).max() <= 1e-5, f"{name}: fails the reference's absolute 1e-5 check"


class Dev:
    """Device buffers with canaries on both sides, so an out-of-bounds store shows up as a test failure."""
    PAD = 64

    def __init__(self, torch):
        self.torch = torch
        self.live = []

    def put(self, arr):
        t = self.torch
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        buf = t.full((arr.size + 2 * self.PAD,), 12345.0, dtype=t.float32, device="cuda")
        view = buf[self.PAD:self.PAD + arr.size]
        if arr.size:
            view.copy_(t.from_numpy(arr.reshape(-1)))
        self.live.append(buf)
        return view.view(*arr.shape) if arr.size else view

    def nan(self, *shape):
        return self.put(np.full(shape, np.nan, np.float32))

    def check_canaries(self):
        for buf in self.live:
            assert bool((buf[:self.PAD] == 12345.0).all()) and bool((buf[-self.PAD:] == 12345.0).all()), "canary overwritten"


def run_linear(be, torch, x, w, b, gy, gw0, gb0):
    d = Dev(torch)
    m, k = x.shape
    n = w.shape[1]
    dx, dw, db, dgy = d.put(x), d.put(w), d.put(b), d.put(gy)
    y, act, y2 = d.nan(m, n), d.nan(m, n), d.nan(m, n)
    be.device_linear_activation_fused_forward(y, act, dx, dw, db, True, 1, m, k, n)
    be.device_linear_activation_fused_forward(y2, None, dx, dw, db, False, 1, m, k, n)
    gx, gw, gb = d.nan(m, k), d.put(gw0), d.put(gb0)
    be.device_linear_backward(gx, gw, gb, dgy, dx, dw, 1, m, k, n)
    ggx = d.nan(m, n)
    be.device_activation_backward(ggx, dgy, y, 1, m, n)
    be.synchronize()
    d.check_canaries()
    return {k_: v.cpu().numpy() for k_, v in dict(y=y, act=act, y2=y2, gx=gx, gw=gw, gb=gb, gelu_gx=ggx).items()}


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "ops_linear_*.npz"))), ids=os.path.basename)
def test_linear_ops_against_reference_golden_vectors(be, torch, path):
    g = np.load(path)
    out = run_linear(be, torch, g["x"], g["w"], g["b"], g["gy"], g["gw0"], g["gb0"])
    for name in ("y", "act", "gx", "gw", "gb", "gelu_gx"):
        check(name, out[name], g[name], be.mode, absolute=False)
    assert np.array_equal(out["y"], out["y2"])  # activation flag must not change y


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "ops_unembed_*.npz"))), ids=os.path.basename)
def test_unembed_ops_against_reference_golden_vectors(be, torch, path):
    g = np.load(path)
    d = Dev(torch)
    m, dm = g["x"].shape
    vp = g["wte"].shape[0]
    x, wte, gy = d.put(g["x"]), d.put(g["wte"]), d.put(g["gy"])
    y, gx, gw = d.nan(m, vp), d.nan(m, dm), d.put(g["gwte0"])
    be.device_unembedding_forward(y, x, wte, 1, m, dm, vp)
    be.device_unembedding_backward(gx, gw, gy, x, wte, 1, m, dm, vp)
    be.synchronize()
    d.check_canaries()
    check("logits", y.cpu().numpy(), g["logits"], be.mode)
    check("grad_x", gx.cpu().numpy(), g["gx"], be.mode, absolute=True)
    check("grad_wte", gw.cpu().numpy(), g["gwte"], be.mode)


# (m, k, n): GPT-2 124M layer shapes at a reduced token count, ragged and unaligned shapes, tile-boundary cases
SEEDED_LINEAR = [(256, 768, 2304), (256, 768, 768), (384, 768, 3072), (256, 3072, 768), (1, 768, 3072), (8, 768, 768),
                 (127, 36, 260), (129, 260, 36), (300, 100, 420), (77, 30, 50), (5, 7, 9), (1024, 64, 128),
                 (16, 3072, 768), (3, 768, 2304), (64, 768, 3072)]  # decode-shaped calls: m = batch


@pytest.mark.parametrize("m,k,n", SEEDED_LINEAR, ids=lambda v: str(v))
def test_linear_ops_against_oracle_seeded(be, torch, oracle, m, k, n):
    rng = np.random.default_rng(m * 7919 + k * 31 + n)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = (0.02 * rng.standard_normal((k, n))).astype(np.float32)
    b = (0.02 * rng.standard_normal(n)).astype(np.float32)
    gy = rng.standard_normal((m, n), dtype=np.float32)
    gw0 = rng.standard_normal((k, n), dtype=np.float32)
    gb0 = rng.standard_normal(n, dtype=np.float32)
    out = run_linear(be, torch, x, w, b, gy, gw0, gb0)
    y, act = oracle.linear_forward(x, w, b, True)
    gx, gw, gb = oracle.linear_backward(gy, x, w, gw0, gb0)
    for name, ref in (("y", y), ("act", act), ("gx", gx), ("gw", gw), ("gb", gb), ("gelu_gx", oracle.gelu_backward(gy, out["y"]))):
        check(f"{name} {m}x{k}x{n}", out[name], ref, be.mode)


@pytest.mark.parametrize("m,d,vp,v", [(128, 768, 50304, 50257), (64, 32, 512, 507), (33, 40, 132, 130), (4, 768, 1024, 1000),
                                      (8, 768, 50304, 50257)],
                         ids=lambda v: str(v))
def test_unembed_ops_against_oracle_seeded(be, torch, oracle, m, d, vp, v):
    rng = np.random.default_rng(m + d + vp)
    x = rng.standard_normal((m, d), dtype=np.float32)
    wte = (0.02 * rng.standard_normal((vp, d))).astype(np.float32)
    wte[v:] = 0.0
    logits = oracle.unembed_forward(x, wte)
    # upstream gradient as the model produces it: (softmax - onehot) / m, padding columns zero
    z = logits[:, :v].astype(np.float64)
    p = np.exp(z - z.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    labels = rng.integers(0, v, size=m)
    p[np.arange(m), labels] -= 1.0
    gy = np.zeros((m, vp), np.float32)
    gy[:, :v] = (p / m).astype(np.float32)
    gw0 = (0.01 * rng.standard_normal((vp, d))).astype(np.float32)
    dv = Dev(torch)
    dx, dwte, dgy = dv.put(x), dv.put(wte), dv.put(gy)
    y, gx, gw = dv.nan(m, vp), dv.nan(m, d), dv.put(gw0)
    be.device_unembedding_forward(y, dx, dwte, 1, m, d, vp)
    be.device_unembedding_backward(gx, gw, dgy, dx, dwte, 1, m, d, vp)
    be.synchronize()
    dv.check_canaries()
    rgx, rgw = oracle.unembed_backward(gy, x, wte, gw0)
    check("logits", y.cpu().numpy(), logits, be.mode)
    exact_gx = gy.astype(np.float64) @ wte.astype(np.float64) if vp > 10000 else None  # 50304-term sums
    check("grad_x", gx.cpu().numpy(), rgx, be.mode, exact=exact_gx)
    check("grad_wte", gw.cpu().numpy(), rgw, be.mode)
    assert np.all(y.cpu().numpy()[:, v:] == 0.0)  # zeroed padding rows of wte give exactly zero logits


def test_empty_and_degenerate_shapes(be, torch):
    d = Dev(torch)
    w, b = d.put(np.ones((4, 8), np.float32)), d.put(np.arange(8, dtype=np.float32))
    y = d.nan(3, 8)
    # m == 0: nothing is touched
    be.device_linear_activation_fused_forward(y, None, d.put(np.zeros((0, 4), np.float32)), w, b, False, 1, 0, 4, 8)
    be.synchronize()
    assert bool(torch.isnan(y).all())
    # k == 0: y = b
    be.device_linear_activation_fused_forward(y, None, d.put(np.zeros((3, 0), np.float32)), d.put(np.zeros((0, 8), np.float32)), b, False,
                                              1, 3, 0, 8)
    be.synchronize()
    assert np.array_equal(y.cpu().numpy(), np.tile(np.arange(8, dtype=np.float32), (3, 1)))
    # m == 0 backward: grad_w / grad_b keep their values
    gw, gb = d.put(np.full((4, 8), 2.0, np.float32)), d.put(np.full(8, 3.0, np.float32))
    be.device_linear_backward(d.nan(0, 4), gw, gb, d.put(np.zeros((0, 8), np.float32)), d.put(np.zeros((0, 4), np.float32)), w, 1, 0, 4, 8)
    be.synchronize()
    assert bool((gw == 2.0).all()) and bool((gb == 3.0).all())
    d.check_canaries()


def test_invalid_arguments_return_errors(be, torch):
    import gpt_b200
    d = Dev(torch)
    x = d.put(np.zeros((4, 4), np.float32))
    with pytest.raises(gpt_b200.GptB200Error) as e:
        be.device_linear_activation_fused_forward(None, None, x, x, x, False, 1, 4, 4, 4)
    assert e.value.status == 1
    with pytest.raises(gpt_b200.GptB200Error):
        be.device_linear_activation_fused_forward(x, None, x, x, x, True, 1, 4, 4, 4)  # activation without act buffer
    with pytest.raises(gpt_b200.GptB200Error):
        be.device_linear_activation_fused_forward(x, None, x, x, x, False, 1, -1, 4, 4)
    with pytest.raises(gpt_b200.GptB200Error):
        be.device_unembedding_forward(x, x, x, 1, 70000, 4, 50304)  # m * vp overflows int, as in the reference's indexing


def test_accumulate_semantics_two_micro_batches(be, torch, oracle):
    """grad_w / grad_b accumulate across calls (gradient accumulation, src/train/train.cpp:138-151)."""
    rng = np.random.default_rng(5)
    m, k, n = 192, 64, 160
    w = (0.02 * rng.standard_normal((k, n))).astype(np.float32)
    xs = [rng.standard_normal((m, k), dtype=np.float32) for _ in range(2)]
    gys = [rng.standard_normal((m, n), dtype=np.float32) for _ in range(2)]
    d = Dev(torch)
    gw, gb, dw = d.put(np.zeros((k, n), np.float32)), d.put(np.zeros(n, np.float32)), d.put(w)
    rgw, rgb = np.zeros((k, n), np.float32), np.zeros(n, np.float32)
    for x, gy in zip(xs, gys):
        be.device_linear_backward(d.nan(m, k), gw, gb, d.put(gy), d.put(x), dw, 1, m, k, n)
        _, rgw, rgb = oracle.linear_backward(gy, x, w, rgw, rgb)
    be.synchronize()
    check("grad_w", gw.cpu().numpy(), rgw, be.mode)
    check("grad_b", gb.cpu().numpy(), rgb, be.mode)


def test_backward_halves_equal_the_whole(be, torch):
    """gptb200_linear_backward_weights + gptb200_linear_backward_input give the bits of gptb200_linear_backward."""
    rng = np.random.default_rng(21)
    m, k, n = 700, 96, 260
    d = Dev(torch)
    x, gy, w = d.put(rng.standard_normal((m, k), dtype=np.float32)), d.put(rng.standard_normal((m, n), dtype=np.float32)), d.put(
        (0.02 * rng.standard_normal((k, n))).astype(np.float32))
    gw0, gb0 = rng.standard_normal((k, n), dtype=np.float32), rng.standard_normal(n, dtype=np.float32)
    gx1, gw1, gb1 = d.nan(m, k), d.put(gw0), d.put(gb0)
    be.device_linear_backward(gx1, gw1, gb1, gy, x, w, 1, m, k, n)
    gx2, gw2, gb2 = d.nan(m, k), d.put(gw0), d.put(gb0)
    be.linear_backward_weights(gw2, gb2, gy, x, m, k, n)
    be.linear_backward_input(gx2, gy, w, m, k, n)
    be.synchronize()
    d.check_canaries()
    assert torch.equal(gx1, gx2) and torch.equal(gw1, gw2) and torch.equal(gb1, gb2)


def test_run_to_run_bitwise_repeatability(be, torch):
    """Split-K partial sums are reduced in a fixed order: identical inputs give identical bits."""
    rng = np.random.default_rng(11)
    m, k, n = 4096, 768, 768
    d = Dev(torch)
    x, gy, w = d.put(rng.standard_normal((m, k), dtype=np.float32)), d.put(rng.standard_normal((m, n), dtype=np.float32)), d.put(
        (0.02 * rng.standard_normal((k, n))).astype(np.float32))
    outs = []
    for _ in range(2):
        gx, gw, gb = d.nan(m, k), d.put(np.zeros((k, n), np.float32)), d.put(np.zeros(n, np.float32))
        be.device_linear_backward(gx, gw, gb, gy, x, w, 1, m, k, n)
        be.synchronize()
        outs.append((gx.cpu().numpy(), gw.cpu().numpy(), gb.cpu().numpy()))
    for a, b in zip(*outs):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("mode", [0, 1], ids=["3xTF32", "TF32"])
@pytest.mark.parametrize("m,k,n", [(2048, 768, 3072), (1536, 3072, 768), (1000, 260, 516)], ids=lambda v: str(v))
def test_bias_gradient_rides_the_weight_gradient_launch(torch, built_library, oracle, mode, m, k, n):
    """grad_b comes out of the grad_w GEMM launch (the reference needs a kernel of its own, linear.cu:70-114,146-156): the
    backward call is two launches, grad_b matches the oracle, accumulates, repeats bit for bit, and the separate column-sum
    kernels (option fuse_dbias = 0) give the same values up to summation order.  Whole tiles per pair and cut ranges."""
    import gpt_b200
    rng = np.random.default_rng(m + n)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = (0.02 * rng.standard_normal((k, n))).astype(np.float32)
    gy = rng.standard_normal((m, n), dtype=np.float32)
    gw0, gb0 = rng.standard_normal((k, n), dtype=np.float32), rng.standard_normal(n, dtype=np.float32)
    _, rgw, rgb = oracle.linear_backward(gy, x, w, gw0, gb0)
    for stream_k in (0, 1, -1):
        be = gpt_b200.Backend(0, None, mode)
        be.set_option("pair", 1)
        be.set_option("stream_k", stream_k)
        d = Dev(torch)
        dx, dw, dgy = d.put(x), d.put(w), d.put(gy)
        outs = []
        for rep in range(2):
            gx, gw, gb = d.nan(m, k), d.put(gw0), d.put(gb0)
            l0 = be.launch_count()
            be.device_linear_backward(gx, gw, gb, dgy, dx, dw, 1, m, k, n)
            assert be.launch_count() - l0 == 2, "grad_x GEMM + grad_w GEMM (with the bias gradient inside)"
            be.synchronize()
            outs.append((gw.cpu().numpy(), gb.cpu().numpy()))
        d.check_canaries()
        check(f"grad_b fused stream_k={stream_k}", outs[0][1], rgb, mode)
        check(f"grad_w stream_k={stream_k}", outs[0][0], rgw, mode)
        assert np.array_equal(outs[0][1].view(np.uint32), outs[1][1].view(np.uint32))
        be.set_option("fuse_dbias", 0)
        gx, gw, gb = d.nan(m, k), d.put(gw0), d.put(gb0)
        l0 = be.launch_count()
        be.device_linear_backward(gx, gw, gb, dgy, dx, dw, 1, m, k, n)
        assert be.launch_count() - l0 == 4
        be.synchronize()
        check("grad_b separate kernels", gb.cpu().numpy(), rgb, mode)
        assert np.array_equal(gw.cpu().numpy().view(np.uint32), outs[0][0].view(np.uint32))   # grad_w does not depend on the option
        be.close()


def test_tensor_maps_are_encoded_once_per_tensor(torch, built_library):
    """A repeated call on the same tensors encodes no tensor map (they are kept per address, extents and box)."""
    import gpt_b200
    be = gpt_b200.Backend(0, None, 0)
    t = torch
    m, k, n = 512, 256, 512
    x, w, b = t.randn(m, k, device="cuda"), t.randn(k, n, device="cuda"), t.randn(n, device="cuda")
    y, act = t.empty(m, n, device="cuda"), t.empty(m, n, device="cuda")
    be.device_linear_activation_fused_forward(y, act, x, w, b, True, 1, m, k, n)
    first = be.tensor_map_encodes()
    assert first > 0
    y0 = y.clone()
    for _ in range(3):
        be.device_linear_activation_fused_forward(y, act, x, w, b, True, 1, m, k, n)
    be.synchronize()
    assert be.tensor_map_encodes() == first and t.equal(y, y0)
    x2 = t.randn(m, k, device="cuda")            # another address: new maps for x only
    be.device_linear_activation_fused_forward(y, act, x2, w, b, True, 1, m, k, n)
    be.synchronize()
    assert be.tensor_map_encodes() == first + 1
    ref = x2.double() @ w.double() + b.double()
    assert float((y.double() - ref).abs().max() / ref.abs().max()) <= 1e-5
    be.close()


@pytest.mark.parametrize("m", [8192, 32768])
def test_full_size_ffn_against_oracle_samples(be, torch, oracle, m):
    """BASELINE config 1 at M = 8192 and at its largest M = 32768 (x [M x 768], w [768 x 3072]) against the CPU oracle on
    sampled rows and columns.  The oracle keeps the reference's per-element summation order (k ascending for y, n ascending
    for grad_x, tokens ascending for grad_w / grad_b: cpu_backend.cpp:213-266), so its values for a subset of rows of y /
    grad_x, or a subset of output columns of grad_w / grad_b, are the bits the full-size reference run would give there.
    Plus one size-independent property: exact linearity under a scaling by two."""
    t = torch
    g = t.Generator(device="cuda").manual_seed(1)
    k, n = 768, 3072
    x = t.randn(m, k, device="cuda", generator=g)
    w = t.randn(k, n, device="cuda", generator=g) * 0.02
    b = t.randn(n, device="cuda", generator=g) * 0.02
    zero_b = t.zeros(n, device="cuda")
    y, act, y2, ys = (t.empty(m, n, device="cuda") for _ in range(4))
    be.device_linear_activation_fused_forward(y, act, x, w, b, True, 1, m, k, n)
    # linearity in x: f(2x) - bias == 2 (f(x) - bias) exactly (scaling by 2 is exact in every mode)
    be.device_linear_activation_fused_forward(y2, None, x * 2, w, zero_b, False, 1, m, k, n)
    be.device_linear_activation_fused_forward(ys, None, x, w, zero_b, False, 1, m, k, n)
    be.synchronize()
    assert t.equal(y2, ys * 2)
    del y2, ys
    rows = t.arange(0, m, m // 128 - 3, device="cuda")          # ~130 rows spread over every 128-row tile band
    hx, hw, hb = x.cpu().numpy(), w.cpu().numpy(), b.cpu().numpy()
    hrows = rows.cpu().numpy()
    ry, ract = oracle.linear_forward(hx[hrows], hw, hb, True)
    check(f"y rows M={m}", y[rows].cpu().numpy(), ry, be.mode)
    check(f"act rows M={m}", act[rows].cpu().numpy(), ract, be.mode)
    gy = t.randn(m, n, device="cuda", generator=g)
    gx, gw, gb = t.empty(m, k, device="cuda"), t.zeros(k, n, device="cuda"), t.zeros(n, device="cuda")
    be.device_linear_backward(gx, gw, gb, gy, x, w, 1, m, k, n)
    be.synchronize()
    cols = t.arange(0, n, 97, device="cuda")                     # 32 output columns, every 256-column tile
    hcols = cols.cpu().numpy()
    hgy_cols = gy[:, cols].cpu().numpy()
    _, rgw, rgb = oracle.linear_backward(hgy_cols, hx, hw[:, hcols])
    check(f"grad_w cols M={m}", gw[:, cols].cpu().numpy(), rgw, be.mode)
    check(f"grad_b cols M={m}", gb[cols].cpu().numpy(), rgb, be.mode)
    rgx, _, _ = oracle.linear_backward(gy[rows].cpu().numpy(), hx[hrows], hw)
    check(f"grad_x rows M={m}", gx[rows].cpu().numpy(), rgx, be.mode)
    # grad_b of every column against the column sums (fp64)
    refb = gy.double().sum(0)
    assert float((gb.double() - refb).abs().max() / refb.abs().max()) <= 1e-5


def test_full_size_lm_head_against_oracle_samples(be, torch, oracle):
    """BASELINE config 2 (x [8192 x 768], wte [50304 x 768], 50257 real rows): logits and grad_x (a 50304-term reduction) on
    sampled rows, grad_wte on sampled vocabulary rows, against the CPU oracle (same per-element order as the reference,
    cpu_backend.cpp:81-140); padding rows of wte give zero logits and receive zero gradient."""
    t = torch
    g = t.Generator(device="cuda").manual_seed(2)
    m, d, vp, v = 8192, 768, 50304, 50257
    x = t.randn(m, d, device="cuda", generator=g)
    wte = t.randn(vp, d, device="cuda", generator=g) * 0.02
    wte[v:] = 0.0
    logits = t.empty(m, vp, device="cuda")
    be.device_unembedding_forward(logits, x, wte, 1, m, d, vp)
    be.synchronize()
    rows = t.arange(0, m, 257, device="cuda")
    hrows = rows.cpu().numpy()
    hx, hwte = x.cpu().numpy(), wte.cpu().numpy()
    check("logits rows", logits[rows].cpu().numpy(), oracle.unembed_forward(hx[hrows], hwte), be.mode)
    assert bool((logits[:, v:] == 0).all())
    del logits
    gy = t.randn(m, vp, device="cuda", generator=g) / m
    gy[:, v:] = 0.0                                       # as the cross-entropy backward leaves the padding columns
    gx, gw = t.empty(m, d, device="cuda"), t.zeros(vp, d, device="cuda")
    be.device_unembedding_backward(gx, gw, gy, x, wte, 1, m, d, vp)
    be.synchronize()
    hgy_rows = gy[rows].cpu().numpy()
    rgx, _ = oracle.unembed_backward(hgy_rows, hx[hrows], hwte)
    exact_gx = hgy_rows.astype(np.float64) @ hwte.astype(np.float64)
    check("grad_x rows", gx[rows].cpu().numpy(), rgx, be.mode, exact=exact_gx)
    vrows = t.arange(0, vp, 499, device="cuda")
    hv = vrows.cpu().numpy()
    _, rgw = oracle.unembed_backward(gy[:, vrows].cpu().numpy(), hx, hwte[hv])
    check("grad_wte rows", gw[vrows].cpu().numpy(), rgw, be.mode)
    assert bool((gw[v:] == 0).all())


def test_full_size_lm_head_with_in_place_cross_entropy(torch, built_library, oracle, reference):
    """BASELINE config 2 end to end in the fused form: logits = x . wte^T on the GPU, softmax + cross-entropy backward in place
    (gptb200_softmax_cross_entropy_inplace), then grad_x and grad_wte from that buffer -- at (M, Vp) = (8192, 50304).
    Loss, upstream gradient (sampled rows, against the reference's softmax and cross-entropy operators applied to the
    oracle's logits), grad_x (sampled rows) and grad_wte (sampled vocabulary rows) against the CPU oracle."""
    import ctypes
    import gpt_b200
    t = torch
    g = t.Generator(device="cuda").manual_seed(3)
    m, d, vp, v = 8192, 768, 50304, 50257
    x = t.randn(m, d, device="cuda", generator=g)
    wte = t.randn(vp, d, device="cuda", generator=g) * 0.02
    wte[v:] = 0.0
    labels = t.randint(0, v, (m,), device="cuda", generator=g, dtype=t.int32)
    be = gpt_b200.Backend(0, None, 0)
    buf = t.empty(m, vp, device="cuda")
    be.device_unembedding_forward(buf, x, wte, 1, m, d, vp)
    row_loss, loss = t.empty(m, device="cuda"), t.zeros(1, device="cuda")
    assert be.lib.gptb200_softmax_cross_entropy_inplace(be.handle, buf.data_ptr(), row_loss.data_ptr(), labels.data_ptr(), m, v, vp) == 0
    assert be.lib.gptb200_row_loss_mean(be.handle, loss.data_ptr(), row_loss.data_ptr(), m) == 0
    gx, gw = t.empty(m, d, device="cuda"), t.zeros(vp, d, device="cuda")
    be.device_unembedding_backward(gx, gw, buf, x, wte, 1, m, d, vp)
    be.synchronize()
    hx, hwte, hlab = x.cpu().numpy(), wte.cpu().numpy(), labels.cpu().numpy()
    rows = np.arange(0, m, 257)
    # the reference's operators on the oracle's logits of the sampled rows; its gradient divides by the row count it is given
    ref_logits = oracle.unembed_forward(hx[rows], hwte)
    probs = reference.softmax_forward(ref_logits, v)
    gy_rows = reference.cross_entropy_softmax_backward(probs, hlab[rows], v) * (len(rows) / m)
    check("upstream gradient rows", buf[rows].cpu().numpy(), gy_rows, 0)
    ref_row_loss = -np.log(probs[np.arange(len(rows)), hlab[rows]].astype(np.float64) + 1e-8)
    assert np.abs(row_loss[rows].cpu().numpy() - ref_row_loss).max() <= 1e-5 * np.abs(ref_row_loss).max()
    assert abs(float(loss) - float(row_loss.double().mean())) <= 1e-5 * float(loss)
    assert abs(float(loss) - np.log(v)) < 0.5                    # random logits of small scale: loss near ln(V)
    rgx, _ = oracle.unembed_backward(gy_rows, hx[rows], hwte)
    exact = gy_rows.astype(np.float64) @ hwte.astype(np.float64)
    check("grad_x rows", gx[rows].cpu().numpy(), rgx, 0, exact=exact)
    vrows = np.arange(0, vp, 499)
    hgy_cols = buf[:, t.from_numpy(vrows).cuda()].cpu().numpy()   # the GPU's gradient (checked above) at the sampled vocabulary rows
    _, rgw = oracle.unembed_backward(hgy_cols, hx, hwte[vrows])
    check("grad_wte rows", gw[t.from_numpy(vrows).cuda()].cpu().numpy(), rgw, 0)
    assert bool((gw[v:] == 0).all()) and bool((buf[:, v:] == 0).all())
    be.close()


@pytest.mark.parametrize("m,k,n,w_kn", [(1, 768, 3072, True), (2, 768, 768, True), (8, 3072, 768, True), (16, 768, 2304, True),
                                        (1, 768, 50304, False), (8, 768, 1024, False), (5, 40, 132, False), (2, 3072, 767 * 4, False), (3, 100, 132, False),
                                        (40, 768, 2304, True), (64, 3072, 768, True), (33, 768, 1024, False),
                                        (9, 100, 132, True), (17, 36, 260, True), (61, 3072, 3072, True),
                                        (64, 768, 2048, False), (16, 1024, 512, False), (11, 3072, 768, False)], ids=lambda v: str(v))
def test_decode_kernel_variants_agree(torch, built_library, oracle, m, k, n, w_kn):
    """Decode-shaped calls: the cluster kernels (k split over warps and / or cluster CTAs, summed through distributed shared
    memory; every cluster size) and the k-split kernel (partial sums in scratch, added by the last CTA or by a second kernel: same
    bits both ways, also on repeated calls, since the tickets reset themselves) all match the oracle."""
    import gpt_b200
    rng = np.random.default_rng(m * 131 + k + n)
    x = rng.standard_normal((m, k), dtype=np.float32)
    d = Dev(torch)
    be = gpt_b200.Backend(0, None, 0)
    try:
        if w_kn:
            w = (0.02 * rng.standard_normal((k, n))).astype(np.float32)
            b = (0.02 * rng.standard_normal(n)).astype(np.float32)
            ref = oracle.linear_forward(x, w, b, True)
            dx, dw, db = d.put(x), d.put(w), d.put(b)

            def run():
                y, act = d.nan(m, n), d.nan(m, n)
                be.device_linear_activation_fused_forward(y, act, dx, dw, db, True, 1, m, k, n)
                be.synchronize()
                return y.cpu().numpy(), act.cpu().numpy()
        else:
            w = (0.02 * rng.standard_normal((n, k))).astype(np.float32)
            ref = (oracle.unembed_forward(x, w),)
            dx, dw = d.put(x), d.put(w)

            def run():
                y = d.nan(m, n)
                be.device_unembedding_forward(y, dx, dw, 1, m, k, n)
                be.synchronize()
                return (y.cpu().numpy(),)
        # [k][n] weights: the per-warp cluster kernel at every row count (limit 64) and, beyond eight rows, the register-tiled
        # cluster kernel (limit 8, the default), each at every cluster size
        for cluster, row_limit in (((16, 8), (32, 8), (8, 8), (2, 8), (16, 64), (32, 64), (8, 64), (4, 64), (1, 64)) if w_kn else ()):
            be.set_option("skinny_cluster", cluster)
            be.set_option("skinny_cluster_rows", row_limit)
            be.set_option("skinny_tile_rows", 64 if cluster == 8 else 32 if cluster == 2 else 0)
            be.set_option("skinny_push", 0 if cluster in (4, 32) else 1)
            first, again = run(), run()
            for got, again_, want in zip(first, again, ref):
                check(f"cluster {cluster} rows {row_limit}", got, want, 0)
                assert np.array_equal(got, again_)
        if not w_kn:
            # [n][k] weights: warp-per-row kernel up to eight rows and register-tiled kernel beyond (defaults), then the
            # warp-per-row kernel with row groups at every row count
            for row_limit in (8, 64):
                be.set_option("skinny_rowwise_rows", row_limit)
                first, again = run(), run()
                check(f"rowwise rows {row_limit}", first[0], ref[0], 0)
                assert np.array_equal(first[0], again[0])
            be.set_option("skinny_rowwise", 0)
            be.set_option("skinny_tile", 0)
        be.set_option("skinny_cluster", 0)
        results = []
        for fused in (1, -1, 1, 0):
            be.set_option("skinny_fused", fused)
            results.append(run())
        be.set_option("skinny_pipelined", 0)     # 16-row groups: weight loads straight into registers
        results.append(run())
        d.check_canaries()
        for got, want in zip(results[0], ref):
            check("k-split", got, want, 0)
        for r in results[1:]:
            for a_, b_ in zip(results[0], r):
                assert np.array_equal(a_, b_)
    finally:
        be.close()


def test_bounded_wait_runs_out_and_is_reported(torch, built_library):
    """Failure detection: a wait on a barrier that nothing signals ends after its limit, the kernel returns, the host reads
    the status as GPTB200_ERR_DEVICE_TIMEOUT, and the context keeps working (no trap, no hang, no lost context)."""
    import gpt_b200
    b = gpt_b200.Backend(0)
    assert b.lib.gptb200_selftest_wait_timeout(b.handle, 2000) == 0    # 2 ms limit
    with pytest.raises(gpt_b200.GptB200Error) as e:
        b.synchronize()
    assert e.value.status == 4 and "108" in str(e.value)
    b.synchronize()                                                   # status was cleared
    x = torch.randn(256, 64, device="cuda")
    w = torch.randn(64, 128, device="cuda") * 0.02
    bias = torch.zeros(128, device="cuda")
    y = torch.empty(256, 128, device="cuda")
    b.device_linear_activation_fused_forward(y, None, x, w, bias, False, 1, 256, 64, 128)
    b.synchronize()
    ref = x.double() @ w.double()
    assert float((y.double() - ref).abs().max() / ref.abs().max()) <= 1e-5
    b.close()


def test_kernel_phase_trace_and_cut_ranges_at_full_width(torch, built_library):
    """The CTA-pair kernel with every pair's k-block range cut inside tiles (36 tiles of 64 k-blocks on 74 pairs: most tiles are
    summed from three pairs' parts) gives the same result as with whole tiles, bit for bit on repeated runs; the kernel-phase
    trace of the launch holds increasing clock samples in pipeline order."""
    import gpt_b200
    m, k, n = 1536, 2048, 1536
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(m, k, device="cuda", generator=g)
    w = torch.randn(k, n, device="cuda", generator=g) * 0.02
    bias = torch.randn(n, device="cuda", generator=g)
    ref = x.double() @ w.double() + bias.double()
    out = {}
    for cut in (-1, 1):
        b = gpt_b200.Backend(0)
        b.set_option("pair", 1)
        b.set_option("stream_k", cut)
        b.set_option("trace", 1)
        ys = []
        for _ in range(2):
            y = torch.full((m, n), float("nan"), device="cuda")
            act = torch.full((m, n), float("nan"), device="cuda")
            b.device_linear_activation_fused_forward(y, act, x, w, bias, True, 1, m, k, n)
            b.synchronize()
            ys.append((y, act))
        assert torch.equal(ys[0][0], ys[1][0]) and torch.equal(ys[0][1], ys[1][1])       # no dependence on timing
        assert float((ys[0][0].double() - ref).abs().max() / ref.abs().max()) <= 1e-5
        gelu = torch.nn.functional.gelu(ref, approximate="tanh")
        assert float((ys[0][1].double() - gelu).abs().max() / gelu.abs().max()) <= 1e-5
        tr = np.array(b.read_trace(), dtype=np.int64)
        assert tr.shape == (11, 128)
        kb = 8                                                                             # every pair runs at least 8 k-blocks here
        for event in (0, 1, 2, 4, 5):
            assert (tr[event, :kb] > 0).all(), event
        assert (np.diff(tr[5, :kb]) > 0).all()                                             # k-blocks are issued in order
        assert (tr[0, :kb] < tr[1, :kb]).all() and (tr[1, :kb] < tr[2, :kb]).all()         # load -> conversion begins -> published
        assert (tr[2, :kb] < tr[5, :kb]).all()                                             # ... -> MMAs issued
        b.set_option("trace", 0)
        out[cut] = ys[0][0]
        b.close()
    diff = float((out[1].double() - out[-1].double()).abs().max() / ref.abs().max())
    assert diff <= 4e-6                                                                    # same sums, other grouping of the k range


def test_cut_ranges_replayed_from_a_cuda_graph(torch, built_library):
    """A GEMM whose tiles are summed from several CTA pairs' parts numbers its launches in device memory, so a launch captured
    in a CUDA graph and replayed with unchanged parameters still pairs partial tiles with the right launch."""
    import gpt_b200
    m, k, n = 1024, 4096, 1024
    g = torch.Generator(device="cuda").manual_seed(6)
    w = torch.randn(k, n, device="cuda", generator=g) * 0.02
    bias = torch.zeros(n, device="cuda")
    x = torch.randn(m, k, device="cuda", generator=g)
    y = torch.empty(m, n, device="cuda")
    side = torch.cuda.Stream()
    b = gpt_b200.Backend(0, side.cuda_stream)
    b.set_option("pair", 1)
    b.set_option("stream_k", 1)
    with torch.cuda.stream(side):
        b.device_linear_activation_fused_forward(y, None, x, w, bias, False, 1, m, k, n)    # warm-up: scratch is allocated here
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            b.device_linear_activation_fused_forward(y, None, x, w, bias, False, 1, m, k, n)
    for _ in range(3):
        x.normal_(generator=g)
        y.fill_(float("nan"))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        ref = x.double() @ w.double()
        assert float((y.double() - ref).abs().max() / ref.abs().max()) <= 1e-5
    b.synchronize()
    b.close()


@pytest.mark.parametrize("m", [1, 4, 16])
def test_decode_chain_with_early_launch_matches_plain_launches(torch, built_library, m):
    """Option "decode_early_launch": every decode-shaped layer may start while its predecessor still runs (it prefetches weights
    and reads its input only after the predecessor has completed).  A chain in which each layer reads the previous layer's
    output must give the same bits as with ordinary launches, eagerly and replayed from a CUDA graph."""
    import gpt_b200
    d = 768
    g = torch.Generator(device="cuda").manual_seed(40 + m)
    ws = [torch.randn(d, d, device="cuda", generator=g) * 0.05 for _ in range(8)]
    bs = [torch.randn(d, device="cuda", generator=g) * 0.02 for _ in range(8)]
    x = torch.randn(m, d, device="cuda", generator=g)
    side = torch.cuda.Stream()
    be = gpt_b200.Backend(0, side.cuda_stream)

    def chain(bufs):
        cur = x
        for i, (w, b_) in enumerate(zip(ws, bs)):
            be.device_linear_activation_fused_forward(bufs[2 * i], bufs[2 * i + 1], cur, w, b_, True, 1, m, d, d)
            cur = bufs[2 * i + 1]     # the GELU output feeds the next layer
        return cur

    try:
        with torch.cuda.stream(side):
            plain = [torch.full((m, d), float("nan"), device="cuda") for _ in range(16)]
            chain(plain)
            side.synchronize()
            be.set_option("decode_early_launch", 1)
            for _ in range(3):
                early = [torch.full((m, d), float("nan"), device="cuda") for _ in range(16)]
                side.synchronize()
                chain(early)
                side.synchronize()
                for a, b_ in zip(plain, early):
                    assert torch.equal(a, b_)
            bufs = [torch.empty(m, d, device="cuda") for _ in range(16)]
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                chain(bufs)
        for _ in range(3):
            for t_ in bufs:
                t_.fill_(float("nan"))
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            for a, b_ in zip(plain, bufs):
                assert torch.equal(a, b_)
        ref = x.double()
        for w, b_ in zip(ws, bs):
            ref = torch.nn.functional.gelu(ref @ w.double() + b_.double(), approximate="tanh")
        assert float((plain[-1].double() - ref).abs().max() / ref.abs().max()) <= 3e-5   # eight layers deep
    finally:
        be.synchronize()
        be.close()


@pytest.mark.parametrize("m,k,n", [(2048, 3072, 768), (300, 420, 100), (64, 3072, 768), (129, 260, 36)], ids=lambda v: str(v))
def test_gelu_derivative_rides_the_input_gradient_gemm(be, torch, oracle, m, k, n):
    """gptb200_linear_backward_input_gelu: grad_x = (grad_y . w^T) * gelu'(pre_act) in one call, against the oracle's
    device_linear_backward followed by device_activation_backward (cpu_backend.cpp:241-287) -- through the CTA-pair kernel
    (derivative in the epilogue) and, for the shapes that run another kernel, its two-step form."""
    rng = np.random.default_rng(m + k)
    w = (0.02 * rng.standard_normal((k, n))).astype(np.float32)
    gy = rng.standard_normal((m, n), dtype=np.float32)
    pre = (1.5 * rng.standard_normal((m, k))).astype(np.float32)
    gx_lin, _, _ = oracle.linear_backward(gy, np.zeros((m, k), np.float32), w)
    ref = oracle.gelu_backward(gx_lin, pre)
    d = Dev(torch)
    gx = d.nan(m, k)
    be.linear_backward_input_gelu(gx, d.put(gy), d.put(w), d.put(pre), m, k, n)
    be.synchronize()
    d.check_canaries()
    check(f"grad_x {m}x{k}x{n}", gx.cpu().numpy(), ref, be.mode)
