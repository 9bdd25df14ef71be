"""CPU tests that pin the oracle (oracle/linear_oracle.c):
  - bit-equality with the unmodified reference CPU backend (oracle/_ref) on seeded cases,
  - bit-equality with the committed op-level golden vectors produced by the reference,
  - through the reference's GPT model driver, agreement with the PyTorch gradients of the reference's own
    gradient test (abs 1e-5 per element, src/model/gpt_test.cpp:12,37) on all 16 tensors.
"""
import glob
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN
from oracle.oracle import split_weights


def _eq(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "ops_linear_*.npz"))), ids=os.path.basename)
def test_linear_ops_match_golden_bitwise(oracle, path):
    g = np.load(path)
    y, act = oracle.linear_forward(g["x"], g["w"], g["b"], True)
    assert _eq(y, g["y"]) and _eq(act, g["act"])
    y2, none = oracle.linear_forward(g["x"], g["w"], g["b"], False)
    assert none is None and _eq(y2, g["y"])
    gx, gw, gb = oracle.linear_backward(g["gy"], g["x"], g["w"], g["gw0"], g["gb0"])
    assert _eq(gx, g["gx"]) and _eq(gw, g["gw"]) and _eq(gb, g["gb"])
    assert _eq(oracle.gelu_backward(g["gy"], g["y"]), g["gelu_gx"])


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "ops_unembed_*.npz"))), ids=os.path.basename)
def test_unembed_ops_match_golden_bitwise(oracle, path):
    g = np.load(path)
    assert _eq(oracle.unembed_forward(g["x"], g["wte"]), g["logits"])
    gx, gwte = oracle.unembed_backward(g["gy"], g["x"], g["wte"], g["gwte0"])
    assert _eq(gx, g["gx"]) and _eq(gwte, g["gwte"])


def test_golden_fixtures_present():
    assert len(glob.glob(os.path.join(GOLDEN, "ops_linear_*.npz"))) >= 6
    assert len(glob.glob(os.path.join(GOLDEN, "ops_unembed_*.npz"))) >= 2
    for f in ("gpt_tiny_tokens.bin", "gpt_tiny_weights.bin", "gpt_tiny_ref_grads.bin", "gpt_tiny.json"):
        assert os.path.exists(os.path.join(GOLDEN, f))


@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (3, 5, 7), (64, 32, 96), (130, 100, 260), (17, 768, 64)])
@pytest.mark.parametrize("threads", [1, 5])
def test_restatement_equals_reference_bitwise(oracle, reference, m, k, n, threads):
    oracle.set_num_threads(threads)
    rng = np.random.default_rng(m * 1000 + k * 10 + n)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.05)
    b = rng.standard_normal(n, dtype=np.float32)
    gy = rng.standard_normal((m, n), dtype=np.float32)
    gw0 = rng.standard_normal((k, n), dtype=np.float32)
    gb0 = rng.standard_normal(n, dtype=np.float32)
    for act in (False, True):
        yo, ao = oracle.linear_forward(x, w, b, act)
        yr, ar = reference.linear_forward(x, w, b, act)
        assert _eq(yo, yr)
        if act:
            assert _eq(ao, ar)
    for a, r in zip(oracle.linear_backward(gy, x, w, gw0, gb0), reference.linear_backward(gy, x, w, gw0, gb0)):
        assert _eq(a, r)
    assert _eq(oracle.gelu_backward(gy, yr), reference.gelu_backward(gy, yr))
    # un-embedding with (m, d, vp) = (m, k, n)
    wte = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    assert _eq(oracle.unembed_forward(x, wte), reference.unembed_forward(x, wte))
    gwte0 = rng.standard_normal((n, k), dtype=np.float32)
    for a, r in zip(oracle.unembed_backward(gy, x, wte, gwte0), reference.unembed_backward(gy, x, wte, gwte0)):
        assert _eq(a, r)
    oracle.set_num_threads(0)


def test_empty_inputs(oracle):
    y, act = oracle.linear_forward(np.zeros((0, 4), np.float32), np.ones((4, 3), np.float32), np.ones(3, np.float32), True)
    assert y.shape == (0, 3) and act.shape == (0, 3)
    gx, gw, gb = oracle.linear_backward(np.zeros((0, 3), np.float32), np.zeros((0, 4), np.float32), np.ones((4, 3), np.float32),
                                        np.full((4, 3), 2.0, np.float32), np.full(3, 3.0, np.float32))
    assert gx.shape == (0, 4) and np.all(gw == 2.0) and np.all(gb == 3.0)  # nothing to accumulate


def test_known_answers(oracle):
    # y = x.w + b with integers is exact; GELU(0) = 0, GELU'(0) = 0.5
    x = np.arange(6, dtype=np.float32).reshape(2, 3)
    w = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = np.array([1, -1, 2, -2], np.float32)
    y, _ = oracle.linear_forward(x, w, b, False)
    assert np.array_equal(y, x @ w + b)
    z = np.zeros((2, 4), np.float32)
    _, act = oracle.linear_forward(np.zeros((2, 3), np.float32), w, np.zeros(4, np.float32), True)
    assert np.array_equal(act, z)
    assert np.array_equal(oracle.gelu_backward(np.ones((2, 4), np.float32), z), np.full((2, 4), 0.5, np.float32))
    gx, gw, gb = oracle.linear_backward(np.ones((2, 4), np.float32), x, w)
    assert np.array_equal(gx, np.ones((2, 4), np.float32) @ w.T)
    assert np.array_equal(gw, x.T @ np.ones((2, 4), np.float32)) and np.array_equal(gb, np.full(4, 2.0, np.float32))


def _tiny():
    meta = json.load(open(os.path.join(GOLDEN, "gpt_tiny.json")))
    tokens = np.fromfile(os.path.join(GOLDEN, "gpt_tiny_tokens.bin"), dtype=np.int32)
    weights = np.fromfile(os.path.join(GOLDEN, "gpt_tiny_weights.bin"), dtype=np.float32)
    golden = np.fromfile(os.path.join(GOLDEN, "gpt_tiny_ref_grads.bin"), dtype=np.float32)
    return meta, tokens, weights, golden


def test_tiny_model_restated_ops_match_pytorch_goldens(reference):
    """The reference's gradient test (gpt_test.cpp) with the linear-path ops swapped for the restatement."""
    meta, tokens, weights, golden = _tiny()
    cfg = meta["config"]
    T = cfg["max_seq_len"]
    g_ref, loss_ref, _ = reference.gpt_forward_backward(cfg, weights, tokens[:T], tokens[1:T + 1], 1, T, restated_ops=False)
    g_res, loss_res, _ = reference.gpt_forward_backward(cfg, weights, tokens[:T], tokens[1:T + 1], 1, T, restated_ops=True)
    assert np.array_equal(g_ref.view(np.uint32), g_res.view(np.uint32))  # restatement == reference, whole model
    assert loss_ref == loss_res and abs(loss_ref - 6.185424) < 1e-4       # PyTorch loss printed by tools/prep_grad.py
    a, b = split_weights(cfg, g_res), split_weights(cfg, golden)
    for name in a:  # the repo's check, on the true packing and over all 16 tensors
        assert np.all(np.abs(a[name] - b[name]) <= 1e-5), name
    assert np.abs(g_res - golden).max() < 2e-7
