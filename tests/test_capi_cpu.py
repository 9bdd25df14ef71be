"""CPU checks of the C-ABI library: it builds for sm_100a, loads, exports every symbol include/gptb200.h
declares, and fails loudly (no fallback) when there is no B200 to run on.  No compute calls here."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "gptb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gptb200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_linear_path():
    syms = _declared_symbols()
    for s in ("gptb200_linear_forward", "gptb200_linear_backward", "gptb200_gelu_backward", "gptb200_unembed_forward",
              "gptb200_unembed_backward", "gptb200_ctx_create", "gptb200_ctx_destroy", "gptb200_ctx_set_mode"):
        assert s in syms


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    missing = [s for s in _declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_python_binding_lists_the_same_symbols(built_library):
    import gpt_b200
    assert set(gpt_b200.EXPORTED_SYMBOLS) <= set(_declared_symbols())
    lib = gpt_b200.load_library()
    assert lib.gptb200_status_string(0) == b"ok"
    assert lib.gptb200_status_string(4) == b"bounded wait inside a kernel ran out"


def test_no_device_is_an_error_not_a_fallback(built_library):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import gpt_b200
    with pytest.raises(gpt_b200.GptB200Error) as e:
        gpt_b200.Backend(0)
    assert e.value.status == 3  # GPTB200_ERR_NO_DEVICE


def test_invalid_arguments_are_rejected_without_a_device(built_library):
    import gpt_b200
    lib = gpt_b200.load_library()
    assert lib.gptb200_ctx_create(None, 0, None, 0) == 1            # null out pointer
    ctx = ctypes.c_void_p()
    assert lib.gptb200_ctx_create(ctypes.byref(ctx), 0, None, 7) == 1  # unknown precision mode
    assert lib.gptb200_linear_forward(None, None, None, None, None, None, 0, 1, 1, 1) == 1  # null context


def test_model_entry_points_return_errors_instead_of_aborting(built_library):
    """gptb200_model_create reports a configuration beyond the interface's int element counts, and a missing device, as
    status codes (the C++ backend object behind the model driver does not abort the process)."""
    import torch
    import gpt_b200
    lib = gpt_b200.load_library()
    m = ctypes.c_void_p()
    huge = (ctypes.c_int * 7)(1024, 50257, 50304, 96, 96, 12288, 49152)          # 175 B parameters: more than 2^31 - 1
    assert lib.gptb200_model_create(ctypes.byref(m), huge, 0, None, 0, 42, 1) == 6   # GPTB200_ERR_TOO_LARGE
    bad = (ctypes.c_int * 7)(64, 507, 512, 4, 5, 32, 256)                          # d_model not a multiple of the heads
    assert lib.gptb200_model_create(ctypes.byref(m), bad, 0, None, 0, 42, 1) == 1
    if not torch.cuda.is_available():
        tiny = (ctypes.c_int * 7)(64, 507, 512, 4, 4, 32, 256)
        assert lib.gptb200_model_create(ctypes.byref(m), tiny, 0, None, 0, 42, 1) == 3   # GPTB200_ERR_NO_DEVICE, and we are still alive
        assert not m.value


def test_no_cublas_or_oracle_in_the_product_library(built_library):
    import subprocess
    out = subprocess.run(["ldd", built_library], capture_output=True, text=True).stdout
    assert "cublas" not in out.lower() and "oracle" not in out.lower()
    # the package never imports the oracle
    for dirpath, _, files in os.walk(os.path.join(ROOT, "gpt_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read().lower(), f
