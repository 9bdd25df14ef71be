"""GPU test of gptb200_bias_grad_noalloc, the entry point for callers that cannot allocate device memory (a host
program whose memory pool owns the whole GPU, or a call site where the CUDA runtime forbids allocation).

It is called through the C ABI twice in a row, on different shapes so that the second call finds the first
call's partial sums in the shared static array, and each result is compared with the grad_b that the regular
entry point (gptb200_linear_backward, scratch in the context's growable buffer) produces for the same input and
with the CPU oracle's grad_b, at the tolerance of the other parity tests (1e-5, max-normalised).  A third call uses
the array to its last element (n = 8192) with more rows than fit the per-chunk row count of the small cases, so
that the capped number of row chunks is exercised too.  This file is collected last on purpose."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_no_alloc_bias_grad_matches_linear_backward_twice_in_a_row(built_library, oracle):
    import torch
    import gpt_b200
    assert torch.cuda.is_available()
    lib = gpt_b200.load_library()
    be = gpt_b200.Backend(0)
    rng = np.random.default_rng(99)
    stream = torch.cuda.current_stream().cuda_stream
    for m, k, n in [(1000, 64, 3072), (333, 32, 520), (9000, 8, 8192)]:   # calls in a row: smaller and ragged, then the largest n with capped row chunks
        x = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).cuda()
        w = torch.from_numpy((0.02 * rng.standard_normal((k, n))).astype(np.float32)).cuda()
        gy = torch.from_numpy(rng.standard_normal((m, n), dtype=np.float32)).cuda()
        start = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()   # accumulate-into semantics
        gb_ref, gb_new = start.clone(), start.clone()
        gx, gw = torch.empty(m, k, device="cuda"), torch.zeros(k, n, device="cuda")
        be.device_linear_backward(gx, gw, gb_ref, gy, x, w, 1, m, k, n)
        be.synchronize()
        rc = lib.gptb200_bias_grad_noalloc(gb_new.data_ptr(), gy.data_ptr(), m, n, stream)
        assert rc == 0
        torch.cuda.synchronize()
        ref, new = gb_ref.cpu().numpy().astype(np.float64), gb_new.cpu().numpy().astype(np.float64)
        assert np.isfinite(new).all()
        assert np.abs(new - ref).max() <= 1e-5 * np.abs(ref).max(), (m, n, float(np.abs(new - ref).max()))
        _, _, gb_oracle = oracle.linear_backward(gy.cpu().numpy(), x.cpu().numpy(), w.cpu().numpy(), None, start.cpu().numpy())
        assert np.abs(new - gb_oracle).max() <= 1e-5 * np.abs(gb_oracle).max(), (m, n, float(np.abs(new - gb_oracle).max()))
    # sizes beyond the fixed array are refused, and nothing is launched for empty inputs
    big = torch.zeros(8200, device="cuda")
    assert lib.gptb200_bias_grad_noalloc(big.data_ptr(), big.data_ptr(), 1, 8200, stream) == 6   # GPTB200_ERR_TOO_LARGE
    assert lib.gptb200_bias_grad_noalloc(big.data_ptr(), big.data_ptr(), 0, 16, stream) == 0
    assert lib.gptb200_bias_grad_noalloc(None, big.data_ptr(), 4, 16, stream) == 1
    be.close()
