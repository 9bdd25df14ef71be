"""The float64 model that the whole-model GPU test uses as its yardstick (tests/test_model_gpu.py: exact_gradients), pinned on CPU:
on the reference's gradient-test configuration it reproduces the PyTorch goldens that the reference's own tools/prep_grad.py wrote
(tests/golden/gpt_tiny_*.bin) and the loss of the reference CPU backend."""
import numpy as np

from oracle.oracle import split_weights


def test_float64_model_reproduces_the_reference_goldens():
    import test_model_gpu as m
    cfg, tokens, weights, golden = m._tiny()
    T = cfg["max_seq_len"]
    grads, loss = m.exact_gradients(cfg, weights, tokens[:T][None], tokens[1:T + 1][None], device="cpu")
    assert abs(loss - 6.185419) < 2e-6                        # the reference CPU backend's loss on these files (its log(p + 1e-8) guard included)
    g = split_weights(cfg, golden)
    assert set(grads) == set(g)
    for name in g:                                           # fp32 goldens against float64: rounding of the goldens only
        assert np.abs(grads[name] - g[name]).max() <= 2e-7, name
