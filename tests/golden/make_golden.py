"""Regenerates the committed golden fixtures.  Needs the reference tree (environment variable REF) and
oracle/_ref/libref_cpu.so (make -C oracle).  Run from the repository root:

    python tests/golden/make_golden.py

1. gpt_tiny_{tokens,weights,ref_grads}.bin + gpt_tiny.json
   The reference's own gradient-test fixture: tools/prep_grad.py of the reference is executed unmodified
   (seed 1234, config T=64 V=507/512 L=4 H=4 D=32 F=256) and its three output files are moved here.  They hold
   the PyTorch-autograd gradients that src/model/gpt_test.cpp compares both backends against (abs 1e-5).
2. ops_<case>.npz
   Inputs and outputs of the reference CPU backend's five linear-path operators (unmodified sources, through
   oracle/ref_shim.cpp) on small seeded cases, including the ragged shapes of the reference's test config.
"""
import json
import os
import runpy
import shutil
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
REF = os.environ.get("REF")
if not REF or not os.path.isdir(os.path.join(REF, "tools")):
    raise SystemExit("set REF to a checkout of the reference (its tools/ and src/ are used)")
OUT = os.path.join(ROOT, "tests", "golden")

from oracle.oracle import Reference  # noqa: E402

TINY = dict(max_seq_len=64, vocab_size=507, vocab_size_padded=512, num_layers=4, num_heads=4, d_model=32, d_ffn=256)


def tiny_model_fixture():
    tools = os.path.join(REF, "tools")
    cwd = os.getcwd()
    with tempfile.TemporaryDirectory() as tmp:
        os.makedirs(os.path.join(tmp, "data"))
        os.chdir(tmp)
        sys.path.insert(0, tools)
        try:
            runpy.run_path(os.path.join(tools, "prep_grad.py"), run_name="__main__")
        finally:
            sys.path.remove(tools)
            os.chdir(cwd)
        for src, dst in (("gpt_dummy_tokens.bin", "gpt_tiny_tokens.bin"), ("gpt_dummy_weights.bin", "gpt_tiny_weights.bin"),
                         ("gpt_dummy_ref_gradients.bin", "gpt_tiny_ref_grads.bin")):
            shutil.move(os.path.join(tmp, "data", src), os.path.join(OUT, dst))
    ref = Reference()
    tokens = np.fromfile(os.path.join(OUT, "gpt_tiny_tokens.bin"), dtype=np.int32)
    weights = np.fromfile(os.path.join(OUT, "gpt_tiny_weights.bin"), dtype=np.float32)
    golden = np.fromfile(os.path.join(OUT, "gpt_tiny_ref_grads.bin"), dtype=np.float32)
    grads, loss, _ = ref.gpt_forward_backward(TINY, weights, tokens[:-1], tokens[1:], 1, TINY["max_seq_len"])
    meta = dict(config=TINY, seed=1234, reference_cpu_loss=loss, max_abs_diff_cpu_vs_pytorch=float(np.abs(grads - golden).max()),
                max_abs_golden=float(np.abs(golden).max()), n_weights=int(weights.size))
    with open(os.path.join(OUT, "gpt_tiny.json"), "w") as f:
        json.dump(meta, f, indent=1)
    print("tiny model fixture:", meta)


# name -> (m, k, n) for linear cases, (m, d, vp) for un-embedding cases
LINEAR_CASES = {
    "qkv_tiny": (64, 32, 96), "attn_proj_tiny": (64, 32, 32), "ffn_up_tiny": (64, 32, 256), "ffn_down_tiny": (64, 256, 32),
    "ragged": (37, 20, 52), "one_row": (1, 64, 128), "mid": (130, 72, 136),
}
UNEMBED_CASES = {"lm_tiny": (64, 32, 512), "lm_ragged": (19, 24, 132)}


def op_fixtures():
    ref = Reference()
    for idx, (name, (m, k, n)) in enumerate(LINEAR_CASES.items()):
        rng = np.random.default_rng(1000 + idx)
        x = rng.standard_normal((m, k), dtype=np.float32)
        w = (0.02 * rng.standard_normal((k, n))).astype(np.float32)
        b = (0.02 * rng.standard_normal(n)).astype(np.float32)
        gy = rng.standard_normal((m, n), dtype=np.float32)
        gw0 = (0.1 * rng.standard_normal((k, n))).astype(np.float32)   # accumulate-into semantics: non-zero start
        gb0 = (0.1 * rng.standard_normal(n)).astype(np.float32)
        y, act = ref.linear_forward(x, w, b, True)
        y_noact, _ = ref.linear_forward(x, w, b, False)
        assert np.array_equal(y, y_noact)
        gx, gw, gb = ref.linear_backward(gy, x, w, gw0, gb0)
        gelu_gx = ref.gelu_backward(gy, y)
        np.savez_compressed(os.path.join(OUT, f"ops_linear_{name}.npz"), x=x, w=w, b=b, gy=gy, gw0=gw0, gb0=gb0, y=y, act=act, gx=gx, gw=gw,
                            gb=gb, gelu_gx=gelu_gx)
        print("linear", name, (m, k, n))
    for idx, (name, (m, d, vp)) in enumerate(UNEMBED_CASES.items()):
        rng = np.random.default_rng(2000 + idx)
        v = vp - 5
        x = rng.standard_normal((m, d), dtype=np.float32)
        wte = (0.02 * rng.standard_normal((vp, d))).astype(np.float32)
        wte[v:] = 0.0
        labels = rng.integers(0, v, size=m).astype(np.int32)
        gwte0 = (0.1 * rng.standard_normal((vp, d))).astype(np.float32)
        logits = ref.unembed_forward(x, wte)
        probs = ref.softmax_forward(logits, v)
        gy = ref.cross_entropy_softmax_backward(probs, labels, v)
        gx, gwte = ref.unembed_backward(gy, x, wte, gwte0)
        np.savez_compressed(os.path.join(OUT, f"ops_unembed_{name}.npz"), x=x, wte=wte, labels=labels, vocab=np.int32(v), gwte0=gwte0,
                            logits=logits, gy=gy, gx=gx, gwte=gwte)
        print("unembed", name, (m, d, vp))


if __name__ == "__main__":
    tiny_model_fixture()
    op_fixtures()
