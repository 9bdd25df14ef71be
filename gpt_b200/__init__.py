"""gpt_b200 -- Python binding of libgptb200, the sm_100a replacement for the dense linear-layer path of
Filipeak/gpt (the operators its CUDA backend sends to cuBLAS, src/backend/cuda/kernels/linear.cu and
src/backend/cuda/kernels/embedding.cu:47-63,140-170).

The binding is a ctypes view of include/gptb200.h.  `Backend` mirrors the reference's operator names
(IGPTBackend, src/backend/backend_interface.h) so that a test written against the reference reads the
same here.  Tensors are passed as raw device addresses (ints) or as objects with a `data_ptr()` method
(torch CUDA tensors); nothing is copied or converted on the way.

There is no fallback: if the shared library has not been built, or no sm_100 device is present,
constructing a Backend raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Any

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libgptb200.so")

MODE_3XTF32 = 0
MODE_TF32 = 1

# Every symbol include/gptb200.h declares (checked by the CPU test-suite against the built library).
EXPORTED_SYMBOLS = [
    "gptb200_ctx_create", "gptb200_ctx_destroy", "gptb200_ctx_set_mode", "gptb200_ctx_get_mode",
    "gptb200_ctx_set_stream", "gptb200_ctx_set_option", "gptb200_ctx_synchronize", "gptb200_ctx_launch_count", "gptb200_ctx_tensor_map_encodes", "gptb200_ctx_read_trace",
    "gptb200_status_string", "gptb200_last_error", "gptb200_plan_gemm", "gptb200_plan_decode", "gptb200_selftest_wait_timeout",
    "gptb200_linear_forward", "gptb200_linear_backward", "gptb200_linear_backward_weights", "gptb200_linear_backward_input",
    "gptb200_linear_backward_input_gelu", "gptb200_gemm_batched",
    "gptb200_gelu_backward",
    "gptb200_unembed_forward", "gptb200_unembed_backward",
    "gptb200_malloc", "gptb200_free", "gptb200_memset", "gptb200_memcpy_h2d", "gptb200_memcpy_d2h",
    "gptb200_fill_normal", "gptb200_fill_const", "gptb200_embedding_forward", "gptb200_embedding_backward", "gptb200_embedding_backward_scaled",
    "gptb200_layernorm_forward", "gptb200_layernorm_backward", "gptb200_attention_forward", "gptb200_attention_backward",
    "gptb200_softmax_forward", "gptb200_cross_entropy_softmax_backward", "gptb200_cross_entropy_loss",
    "gptb200_softmax_cross_entropy_inplace", "gptb200_row_loss_mean", "gptb200_cross_entropy_loss_from_logits",
    "gptb200_adamw_step", "gptb200_scale_and_clip_grad", "gptb200_memory_info", "gptb200_clip_adamw_packed",
    "gptb200_embedding_decode", "gptb200_kv_cache_fill", "gptb200_attention_decode", "gptb200_advance_position",
    "gptb200_loader_create", "gptb200_loader_destroy", "gptb200_loader_num_samples", "gptb200_loader_reset_epoch", "gptb200_loader_next_batch",
    "gptb200_bias_grad_noalloc",
]


class GptB200Error(RuntimeError):
    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = status
        super().__init__(f"{what}: status {status}" + (f" ({detail})" if detail else ""))


_lib = None


def load_library(path: str | None = None) -> ctypes.CDLL:
    """dlopen libgptb200.so and declare the argument types of its entry points."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise FileNotFoundError(f"{p} is missing: build it with `python -m gpt_b200.build` (there is no fallback path)")
    lib = ctypes.CDLL(p)
    vp, i, fp = ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p
    sig = {
        "gptb200_ctx_create": (i, [ctypes.POINTER(vp), i, vp, i]),
        "gptb200_ctx_destroy": (i, [vp]),
        "gptb200_ctx_set_mode": (i, [vp, i]),
        "gptb200_ctx_get_mode": (i, [vp]),
        "gptb200_ctx_set_stream": (i, [vp, vp]),
        "gptb200_ctx_set_option": (i, [vp, ctypes.c_char_p, i]),
        "gptb200_ctx_read_trace": (i, [vp, vp, i]),
        "gptb200_ctx_synchronize": (i, [vp]),
        "gptb200_ctx_launch_count": (ctypes.c_longlong, [vp]),
        "gptb200_ctx_tensor_map_encodes": (ctypes.c_longlong, [vp]),
        "gptb200_selftest_wait_timeout": (i, [vp, i]),
        "gptb200_plan_gemm": (i, [i, i, i, i, i, i, i, i, ctypes.POINTER(i)]),
        "gptb200_plan_decode": (i, [i, i, i, i, i, i, ctypes.POINTER(i)]),
        "gptb200_status_string": (ctypes.c_char_p, [i]),
        "gptb200_last_error": (ctypes.c_char_p, [vp]),
        "gptb200_linear_forward": (i, [vp, fp, fp, fp, fp, fp, i, i, i, i]),
        "gptb200_linear_backward": (i, [vp, fp, fp, fp, fp, fp, fp, i, i, i]),
        "gptb200_linear_backward_weights": (i, [vp, fp, fp, fp, fp, i, i, i]),
        "gptb200_linear_backward_input": (i, [vp, fp, fp, fp, i, i, i]),
        "gptb200_linear_backward_input_gelu": (i, [vp, fp, fp, fp, fp, i, i, i]),
        "gptb200_gemm_batched": (i, [vp, fp, fp, fp, i, i, i, i, i, i, i, ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong),
                                     ctypes.POINTER(ctypes.c_longlong)]),
        "gptb200_gelu_backward": (i, [vp, fp, fp, fp, i, i]),
        "gptb200_unembed_forward": (i, [vp, fp, fp, fp, i, i, i]),
        "gptb200_unembed_backward": (i, [vp, fp, fp, fp, fp, fp, i, i, i]),
        "gptb200_malloc": (i, [vp, ctypes.POINTER(vp), ctypes.c_size_t]),
        "gptb200_free": (i, [vp, vp]),
        "gptb200_memset": (i, [vp, vp, i, ctypes.c_size_t]),
        "gptb200_memcpy_h2d": (i, [vp, vp, vp, ctypes.c_size_t]),
        "gptb200_memcpy_d2h": (i, [vp, vp, vp, ctypes.c_size_t]),
    }
    f32, sz, ull = ctypes.c_float, ctypes.c_size_t, ctypes.c_ulonglong
    sig.update({
        "gptb200_fill_normal": (i, [vp, fp, f32, f32, sz, ull, ull]),
        "gptb200_fill_const": (i, [vp, fp, f32, sz]),
        "gptb200_embedding_forward": (i, [vp, fp, fp, fp, fp, i, i, i]),
        "gptb200_embedding_backward": (i, [vp, fp, fp, fp, fp, i, i, i]),
        "gptb200_embedding_backward_scaled": (i, [vp, fp, fp, fp, fp, i, i, i, f32]),
        "gptb200_layernorm_forward": (i, [vp, fp, fp, fp, fp, fp, fp, fp, i, i]),
        "gptb200_layernorm_backward": (i, [vp, fp, fp, fp, fp, fp, fp, fp, fp, fp, i, i]),
        "gptb200_attention_forward": (i, [vp, fp, fp, fp, i, i, i, i]),
        "gptb200_attention_backward": (i, [vp, fp, fp, fp, fp, fp, fp, i, i, i, i]),
        "gptb200_softmax_forward": (i, [vp, fp, fp, i, i, i]),
        "gptb200_cross_entropy_softmax_backward": (i, [vp, fp, fp, fp, i, i, i]),
        "gptb200_cross_entropy_loss": (i, [vp, fp, fp, fp, i, i]),
        "gptb200_softmax_cross_entropy_inplace": (i, [vp, fp, fp, fp, i, i, i]),
        "gptb200_row_loss_mean": (i, [vp, fp, fp, i]),
        "gptb200_cross_entropy_loss_from_logits": (i, [vp, fp, fp, fp, fp, i, i, i]),
        "gptb200_adamw_step": (i, [vp, fp, fp, fp, fp, sz, f32, f32, f32, f32, f32, i]),
        "gptb200_scale_and_clip_grad": (i, [vp, fp, sz, f32, i]),
        "gptb200_memory_info": (i, [vp, ctypes.POINTER(f32), ctypes.POINTER(f32)]),
        "gptb200_clip_adamw_packed": (i, [vp, fp, fp, fp, fp, sz, ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_ubyte), i, f32, i, f32, f32, f32,
                                          f32, f32, i, fp]),
        "gptb200_embedding_decode": (i, [vp, fp, fp, fp, fp, fp, i, i]),
        "gptb200_kv_cache_fill": (i, [vp, fp, fp, i, i, i, i]),
        "gptb200_attention_decode": (i, [vp, fp, fp, fp, fp, i, i, i, i]),
        "gptb200_advance_position": (i, [vp, fp]),
        "gptb200_loader_create": (i, [ctypes.POINTER(vp), ctypes.c_char_p, i]),
        "gptb200_loader_destroy": (i, [vp]),
        "gptb200_loader_num_samples": (ctypes.c_longlong, [vp]),
        "gptb200_loader_reset_epoch": (i, [vp]),
        "gptb200_loader_next_batch": (i, [vp, i, i, i, vp, vp]),
        # C++ object factory: an IGPTBackend* for host programs written against the reference's interface
        "gptb200_bias_grad_noalloc": (i, [fp, fp, i, i, vp]),
        "gptb200_backend_create": (vp, [ctypes.c_ulong, i, vp, i]),
        "gptb200_backend_destroy": (None, [vp]),
        "gptb200_backend_context": (vp, [vp]),
    })
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _lib = lib
    return lib


PLAN_KERNELS = {0: "none", 1: "pair", 2: "single", 3: "skinny", 4: "simt"}


def plan_gemm(num_sms: int, m: int, n: int, k: int, a_mn: bool, b_mn: bool, has_epilogue: bool = False, accumulate: bool = False) -> dict:
    """Launch plan of one GEMM (host logic only, no GPU needed); see gptb200_plan_gemm in include/gptb200.h."""
    lib = load_library()
    out = (ctypes.c_int * 8)()
    rc = lib.gptb200_plan_gemm(num_sms, m, n, k, int(a_mn), int(b_mn), int(has_epilogue), int(accumulate), out)
    if rc != 0:
        raise GptB200Error(rc, "gptb200_plan_gemm")
    keys = ["kernel", "tile_n", "tiles_m", "tiles_n", "splits", "k_per_split", "grid", "scratch_kib"]
    d = dict(zip(keys, list(out)))
    d["kernel"] = PLAN_KERNELS[d["kernel"]]
    return d


DECODE_KERNELS = {0: "k_split", 1: "warp_cluster", 2: "tile_cluster", 3: "rowwise"}


def plan_decode(num_sms: int, m: int, n: int, k: int, w_kn: bool, has_epilogue: bool = False) -> dict:
    """Which decode kernel a call of at most 64 rows runs (host logic only); see gptb200_plan_decode in include/gptb200.h."""
    lib = load_library()
    out = (ctypes.c_int * 4)()
    rc = lib.gptb200_plan_decode(num_sms, m, n, k, int(w_kn), int(has_epilogue), out)
    if rc != 0:
        raise GptB200Error(rc, "gptb200_plan_decode")
    d = dict(zip(["kernel", "rows", "groups", "cluster"], list(out)))
    d["kernel"] = DECODE_KERNELS[d["kernel"]]
    return d


def _ptr(t: Any) -> int | None:
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return int(t.data_ptr())


class Backend:
    """Host-side mirror of the linear-path operators of the reference's IGPTBackend.

    Method names and argument order follow src/backend/backend_interface.h (lines 42-51, 70-82, 120-159);
    `batch_size` and `seq_len` only ever enter as their product, as in the reference.
    """

    def __init__(self, device: int = 0, stream: int | None = None, mode: int = MODE_3XTF32):
        self._lib = load_library()
        self._ctx = ctypes.c_void_p()
        rc = self._lib.gptb200_ctx_create(ctypes.byref(self._ctx), device, ctypes.c_void_p(stream or 0), mode)
        if rc != 0:
            raise GptB200Error(rc, "gptb200_ctx_create", self._lib.gptb200_status_string(rc).decode())

    # ---- context
    def close(self) -> None:
        if self._ctx:
            self._lib.gptb200_ctx_destroy(self._ctx)
            self._ctx = ctypes.c_void_p()

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise GptB200Error(rc, what, self._lib.gptb200_last_error(self._ctx).decode())

    @property
    def handle(self) -> ctypes.c_void_p:
        return self._ctx

    @property
    def lib(self) -> ctypes.CDLL:
        return self._lib

    def set_mode(self, mode: int) -> None:
        self._check(self._lib.gptb200_ctx_set_mode(self._ctx, mode), "gptb200_ctx_set_mode")

    def set_stream(self, stream: int) -> None:
        self._check(self._lib.gptb200_ctx_set_stream(self._ctx, ctypes.c_void_p(stream)), "gptb200_ctx_set_stream")

    def read_trace(self):
        """[11 events][128 k-blocks] SM clock samples of the latest CTA-pair GEMM launch (option "trace" must be on)."""
        buf = (ctypes.c_longlong * (11 * 128))()
        self._check(self._lib.gptb200_ctx_read_trace(self._ctx, buf, 11 * 128), "gptb200_ctx_read_trace")
        return [list(buf[e * 128:(e + 1) * 128]) for e in range(11)]

    def set_option(self, key: str, value: int) -> None:
        self._check(self._lib.gptb200_ctx_set_option(self._ctx, key.encode(), value), "gptb200_ctx_set_option")

    def synchronize(self) -> None:
        self._check(self._lib.gptb200_ctx_synchronize(self._ctx), "gptb200_ctx_synchronize")

    def launch_count(self) -> int:
        return int(self._lib.gptb200_ctx_launch_count(self._ctx))

    def tensor_map_encodes(self) -> int:
        return int(self._lib.gptb200_ctx_tensor_map_encodes(self._ctx))

    # ---- operators (names of the reference interface)
    def device_linear_activation_fused_forward(self, y, act, x, w, b, activation: bool, batch_size: int, seq_len: int,
                                               input_size: int, output_size: int) -> None:
        self._check(self._lib.gptb200_linear_forward(self._ctx, _ptr(y), _ptr(act), _ptr(x), _ptr(w), _ptr(b),
                                                     1 if activation else 0, batch_size * seq_len, input_size, output_size),
                    "gptb200_linear_forward")

    def device_linear_backward(self, grad_x, grad_w, grad_b, grad_y, x, w, batch_size: int, seq_len: int, input_size: int,
                               output_size: int) -> None:
        self._check(self._lib.gptb200_linear_backward(self._ctx, _ptr(grad_x), _ptr(grad_w), _ptr(grad_b), _ptr(grad_y),
                                                      _ptr(x), _ptr(w), batch_size * seq_len, input_size, output_size),
                    "gptb200_linear_backward")

    def linear_backward_weights(self, grad_w, grad_b, grad_y, x, m: int, k: int, n: int) -> None:
        """Weight half of device_linear_backward: grad_w += x^T . grad_y, grad_b += column sums (for data-parallel overlap)."""
        self._check(self._lib.gptb200_linear_backward_weights(self._ctx, _ptr(grad_w), _ptr(grad_b), _ptr(grad_y), _ptr(x), m, k, n),
                    "gptb200_linear_backward_weights")

    def linear_backward_input(self, grad_x, grad_y, w, m: int, k: int, n: int) -> None:
        """Input half of device_linear_backward: grad_x = grad_y . w^T."""
        self._check(self._lib.gptb200_linear_backward_input(self._ctx, _ptr(grad_x), _ptr(grad_y), _ptr(w), m, k, n),
                    "gptb200_linear_backward_input")

    def linear_backward_input_gelu(self, grad_x, grad_y, w, pre_act, m: int, k: int, n: int) -> None:
        """grad_x = (grad_y . w^T) * gelu_tanh'(pre_act): device_linear_backward's input half and device_activation_backward in one."""
        self._check(self._lib.gptb200_linear_backward_input_gelu(self._ctx, _ptr(grad_x), _ptr(grad_y), _ptr(w), _ptr(pre_act), m, k, n),
                    "gptb200_linear_backward_input_gelu")

    def gemm_batched(self, out, a, b, m: int, n: int, k: int, a_mn: bool, b_mn: bool, batch_inner: int, batch_outer: int, a_strides, b_strides,
                     out_strides) -> None:
        """batch_inner * batch_outer products out[z] = a[z] . b[z] in one launch; strides = (row pitch, inner, outer) in floats."""
        arr = lambda s: (ctypes.c_longlong * 3)(*[int(v) for v in s])
        self._check(self._lib.gptb200_gemm_batched(self._ctx, _ptr(out), _ptr(a), _ptr(b), m, n, k, int(a_mn), int(b_mn), batch_inner, batch_outer,
                                                   arr(a_strides), arr(b_strides), arr(out_strides)), "gptb200_gemm_batched")

    def device_activation_backward(self, grad_x, grad_y, x, batch_size: int, seq_len: int, output_size: int) -> None:
        self._check(self._lib.gptb200_gelu_backward(self._ctx, _ptr(grad_x), _ptr(grad_y), _ptr(x), batch_size * seq_len,
                                                    output_size), "gptb200_gelu_backward")

    def device_unembedding_forward(self, y, x, wte, batch_size: int, seq_len: int, hidden_size: int, vocab_size: int) -> None:
        self._check(self._lib.gptb200_unembed_forward(self._ctx, _ptr(y), _ptr(x), _ptr(wte), batch_size * seq_len,
                                                      hidden_size, vocab_size), "gptb200_unembed_forward")

    def device_unembedding_backward(self, grad_x, grad_wte, grad_y, x, wte, batch_size: int, seq_len: int, hidden_size: int,
                                    vocab_size_padded: int) -> None:
        self._check(self._lib.gptb200_unembed_backward(self._ctx, _ptr(grad_x), _ptr(grad_wte), _ptr(grad_y), _ptr(x),
                                                       _ptr(wte), batch_size * seq_len, hidden_size, vocab_size_padded),
                    "gptb200_unembed_backward")

    # ---- memory operators (device_malloc / device_free / device_memset / device_memcpy_*)
    def device_malloc(self, nbytes: int) -> int:
        p = ctypes.c_void_p()
        self._check(self._lib.gptb200_malloc(self._ctx, ctypes.byref(p), nbytes), "gptb200_malloc")
        return int(p.value or 0)

    def device_free(self, ptr: int) -> None:
        self._check(self._lib.gptb200_free(self._ctx, ctypes.c_void_p(ptr)), "gptb200_free")

    def device_memset(self, ptr: int, value: int, nbytes: int) -> None:
        self._check(self._lib.gptb200_memset(self._ctx, ctypes.c_void_p(ptr), value, nbytes), "gptb200_memset")

    def device_memcpy_h2d(self, dst: int, src: int, nbytes: int) -> None:
        self._check(self._lib.gptb200_memcpy_h2d(self._ctx, ctypes.c_void_p(dst), ctypes.c_void_p(src), nbytes),
                    "gptb200_memcpy_h2d")

    def device_memcpy_d2h(self, dst: int, src: int, nbytes: int) -> None:
        self._check(self._lib.gptb200_memcpy_d2h(self._ctx, ctypes.c_void_p(dst), ctypes.c_void_p(src), nbytes),
                    "gptb200_memcpy_d2h")


PARAM_NAMES = ["wte", "wpe", "ln_1_w", "ln_1_b", "qkv_proj_w", "qkv_proj_b", "attn_proj_w", "attn_proj_b", "ln_2_w", "ln_2_b",
               "ffn_up_w", "ffn_up_b", "ffn_down_w", "ffn_down_b", "ln_f_w", "ln_f_b"]
CONFIG_KEYS = ["max_seq_len", "vocab_size", "vocab_size_padded", "num_layers", "num_heads", "d_model", "d_ffn"]
GPT2_124M = dict(max_seq_len=256, vocab_size=50257, vocab_size_padded=50304, num_layers=12, num_heads=12, d_model=768, d_ffn=3072)

_LAYER_DONE = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_void_p)


def _declare_model(lib: ctypes.CDLL) -> None:
    if getattr(lib, "_model_declared", False):
        return
    vp, i, f32, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    sig = {
        "gptb200_model_create": (i, [ctypes.POINTER(vp), ctypes.POINTER(i), i, vp, i, ctypes.c_ulong, i]),
        "gptb200_model_destroy": (i, [vp]),
        "gptb200_model_context": (vp, [vp]),
        "gptb200_model_num_params": (ll, [vp]),
        "gptb200_model_weights": (vp, [vp]),
        "gptb200_model_grads": (vp, [vp]),
        "gptb200_model_logits": (vp, [vp]),
        "gptb200_model_param_offsets": (i, [vp, ctypes.POINTER(ll)]),
        "gptb200_model_init": (i, [vp, f32, f32]),
        "gptb200_model_load_weights": (i, [vp, vp, ll]),
        "gptb200_model_read": (i, [vp, vp, ll, i]),
        "gptb200_model_load_checkpoint": (i, [vp, ctypes.c_char_p]),
        "gptb200_model_save_checkpoint": (i, [vp, ctypes.c_char_p]),
        "gptb200_model_set_size": (i, [vp, i, i]),
        "gptb200_model_zero_grad": (i, [vp]),
        "gptb200_model_forward": (i, [vp, vp]),
        "gptb200_model_backward": (i, [vp, vp, vp, _LAYER_DONE, vp]),
        "gptb200_model_loss": (i, [vp, vp, ctypes.POINTER(f32)]),
        "gptb200_model_clip": (i, [vp, f32, i]),
        "gptb200_model_optimizer_step": (i, [vp, f32, f32, f32, f32]),
        "gptb200_model_clip_and_optimizer_step": (i, [vp, f32, i, f32, f32, f32, f32]),
        "gptb200_model_set_fused_cross_entropy": (i, [vp, i]),
        "gptb200_model_set_fused_gelu_backward": (i, [vp, i]),
        "gptb200_model_generate_begin": (i, [vp, vp, i, i, i]),
        "gptb200_model_generate_step": (i, [vp, vp, vp]),
        "gptb200_model_generate_position": (i, [vp]),
        "gptb200_model_defer_embedding_backward": (i, [vp, i]),
        "gptb200_model_embedding_grad": (vp, [vp]),
        "gptb200_model_apply_embedding_grad": (i, [vp, vp, vp, i, i, f32]),
        "gptb200_model_save_state": (i, [vp, ctypes.c_char_p]),
        "gptb200_model_load_state": (i, [vp, ctypes.c_char_p]),
        "gptb200_model_step_count": (i, [vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    lib._model_declared = True


class Model:
    """Host-side mirror of the reference's GPT class (src/model/gpt.h:135-173) over the B200 backend: same method
    names, same parameter packing, raw-fp32 checkpoints interchangeable with the reference's."""

    def __init__(self, config: dict, device: int = 0, stream: int | None = None, mode: int = MODE_3XTF32, seed: int = 42,
                 use_grad: bool = True):
        self._lib = load_library()
        _declare_model(self._lib)
        self.config = dict(config)
        cfg = (ctypes.c_int * 7)(*[int(config[k]) for k in CONFIG_KEYS])
        self._m = ctypes.c_void_p()
        rc = self._lib.gptb200_model_create(ctypes.byref(self._m), cfg, device, ctypes.c_void_p(stream or 0), mode, seed, int(use_grad))
        if rc != 0:
            raise GptB200Error(rc, "gptb200_model_create", self._lib.gptb200_status_string(rc).decode())
        self.num_params = int(self._lib.gptb200_model_num_params(self._m))
        off = (ctypes.c_longlong * 16)()
        self._check(self._lib.gptb200_model_param_offsets(self._m, off))
        self.param_offsets = dict(zip(PARAM_NAMES, [int(v) for v in off]))
        self._cb_keepalive = None

    def _check(self, rc: int) -> None:
        if rc != 0:
            ctx = self._lib.gptb200_model_context(self._m)
            raise GptB200Error(rc, "gptb200_model", self._lib.gptb200_last_error(ctx).decode() if ctx else "")

    def close(self) -> None:
        if self._m:
            self._lib.gptb200_model_destroy(self._m)
            self._m = ctypes.c_void_p()

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    @property
    def context(self) -> int:
        return int(self._lib.gptb200_model_context(self._m))

    def set_option(self, key: str, value: int) -> None:
        """Tuning option of the model's context (gptb200_ctx_set_option)."""
        self._check(self._lib.gptb200_ctx_set_option(ctypes.c_void_p(self.context), key.encode(), value))

    @property
    def weights_ptr(self) -> int:
        return int(self._lib.gptb200_model_weights(self._m))

    @property
    def grads_ptr(self) -> int:
        return int(self._lib.gptb200_model_grads(self._m))

    @property
    def logits_ptr(self) -> int:
        return int(self._lib.gptb200_model_logits(self._m))

    def launch_count(self) -> int:
        return int(self._lib.gptb200_ctx_launch_count(ctypes.c_void_p(self.context)))

    def synchronize(self) -> None:
        self._check(self._lib.gptb200_ctx_synchronize(ctypes.c_void_p(self.context)))

    def init(self, mean: float = 0.0, stddev: float = 0.02) -> None:
        self._check(self._lib.gptb200_model_init(self._m, mean, stddev))

    def load_weights(self, host_array) -> None:
        """host_array: contiguous float32 numpy array in the reference's checkpoint order."""
        self._check(self._lib.gptb200_model_load_weights(self._m, host_array.ctypes.data, host_array.size))

    def read_weights(self, out) -> None:
        self._check(self._lib.gptb200_model_read(self._m, out.ctypes.data, out.size, 0))

    def read_grads(self, out) -> None:
        self._check(self._lib.gptb200_model_read(self._m, out.ctypes.data, out.size, 1))

    def load_checkpoint(self, filename: str) -> None:
        self._check(self._lib.gptb200_model_load_checkpoint(self._m, filename.encode()))

    def save_checkpoint(self, filename: str) -> None:
        self._check(self._lib.gptb200_model_save_checkpoint(self._m, filename.encode()))

    def set_size(self, batch_size: int, seq_len: int) -> None:
        self._check(self._lib.gptb200_model_set_size(self._m, batch_size, seq_len))

    def zero_grad(self) -> None:
        self._check(self._lib.gptb200_model_zero_grad(self._m))

    def forward(self, input_tokens) -> None:
        self._check(self._lib.gptb200_model_forward(self._m, _ptr(input_tokens)))

    def backward(self, input_tokens, label_tokens, layer_done=None) -> None:
        """layer_done(l): host callback fired when layer l's weight gradients have been enqueued
        (l = num_layers: un-embedding + final LayerNorm; l = -1: embeddings, i.e. everything)."""
        if layer_done is None:
            cb = ctypes.cast(None, _LAYER_DONE)
        else:
            cb = _LAYER_DONE(lambda l, _u: layer_done(l))
        self._cb_keepalive = cb
        self._check(self._lib.gptb200_model_backward(self._m, _ptr(input_tokens), _ptr(label_tokens), cb, None))

    def loss(self, label_tokens) -> float:
        out = ctypes.c_float()
        self._check(self._lib.gptb200_model_loss(self._m, _ptr(label_tokens), ctypes.byref(out)))
        return float(out.value)

    def unscale_and_clip_grads(self, max_norm: float, accum_steps: int) -> None:
        self._check(self._lib.gptb200_model_clip(self._m, max_norm, accum_steps))

    def optimizer_step(self, learning_rate: float, beta1: float, beta2: float, decay: float) -> None:
        self._check(self._lib.gptb200_model_optimizer_step(self._m, learning_rate, beta1, beta2, decay))

    def set_fused_cross_entropy(self, on: bool) -> None:
        """The logits become their gradient in place at the start of the backward pass (no probability / gradient tensors);
        takes effect at the next set_size."""
        self._check(self._lib.gptb200_model_set_fused_cross_entropy(self._m, int(on)))

    def set_fused_gelu_backward(self, on: bool) -> None:
        """The FFN's GELU derivative rides the epilogue of the down projection's grad_x GEMM."""
        self._check(self._lib.gptb200_model_set_fused_gelu_backward(self._m, int(on)))

    def generate_begin(self, prompt_tokens, batch_size: int, prompt_len: int, max_len: int) -> None:
        """Forward pass over the prompt [batch x prompt_len] and the keys / values of every layer into a cache for max_len positions."""
        self._check(self._lib.gptb200_model_generate_begin(self._m, _ptr(prompt_tokens), batch_size, prompt_len, max_len))

    def generate_step(self, tokens, logits_out) -> None:
        """One new position per sequence: tokens [batch] at that position in, logits [batch x vocab_size_padded] for the next one out."""
        self._check(self._lib.gptb200_model_generate_step(self._m, _ptr(tokens), _ptr(logits_out)))

    @property
    def generate_position(self) -> int:
        return int(self._lib.gptb200_model_generate_position(self._m))

    def defer_embedding_backward(self, defer: bool) -> None:
        """Backward passes stop before the embedding backward; see apply_embedding_grad (data-parallel training)."""
        self._check(self._lib.gptb200_model_defer_embedding_backward(self._m, int(defer)))

    @property
    def embedding_grad_ptr(self) -> int:
        """Device address of the gradient of the embedding output, [batch*seq x d_model], valid after a backward pass."""
        return int(self._lib.gptb200_model_embedding_grad(self._m) or 0)

    def apply_embedding_grad(self, rows, tokens, batch_size: int, seq_len: int, scale: float) -> None:
        self._check(self._lib.gptb200_model_apply_embedding_grad(self._m, _ptr(rows), _ptr(tokens), batch_size, seq_len, scale))

    def clip_and_optimizer_step(self, max_norm: float, accum_steps: int, learning_rate: float, beta1: float, beta2: float, decay: float) -> None:
        """unscale_and_clip_grads + optimizer_step in two launches over the packed buffers (the gradients stay unscaled)."""
        self._check(self._lib.gptb200_model_clip_and_optimizer_step(self._m, max_norm, accum_steps, learning_rate, beta1, beta2, decay))

    def save_state(self, filename: str) -> None:
        """Parameters + AdamW moments + step counter behind a header that names the configuration."""
        self._check(self._lib.gptb200_model_save_state(self._m, filename.encode()))

    def load_state(self, filename: str) -> None:
        self._check(self._lib.gptb200_model_load_state(self._m, filename.encode()))

    @property
    def step_count(self) -> int:
        return int(self._lib.gptb200_model_step_count(self._m))


class Loader:
    """Sharded token loader (include/gptb200.h: gptb200_loader_*): the reference's DataLoader (src/train/data_loader.h) with the
    global batch split over ranks.  Seed the C library's rand() alike on every rank before reset_epoch (seed_libc_rand)."""

    def __init__(self, token_file: str, seq_len: int):
        self._lib = load_library()
        self._ld = ctypes.c_void_p()
        self.seq_len = seq_len
        rc = self._lib.gptb200_loader_create(ctypes.byref(self._ld), token_file.encode(), seq_len)
        if rc != 0:
            raise GptB200Error(rc, "gptb200_loader_create", "cannot read the token file, or it holds less than two sequences")

    @staticmethod
    def seed_libc_rand(seed: int) -> None:
        ctypes.CDLL(None).srand(ctypes.c_uint(seed))

    def close(self) -> None:
        if self._ld:
            self._lib.gptb200_loader_destroy(self._ld)
            self._ld = ctypes.c_void_p()

    @property
    def num_samples(self) -> int:
        return int(self._lib.gptb200_loader_num_samples(self._ld))

    def reset_epoch(self) -> None:
        rc = self._lib.gptb200_loader_reset_epoch(self._ld)
        if rc != 0:
            raise GptB200Error(rc, "gptb200_loader_reset_epoch")

    def next_batch(self, rank: int, world: int, batch: int):
        """(inputs, labels) as int32 numpy arrays [batch x seq_len], or None when the epoch is exhausted."""
        import numpy as np
        inputs = np.empty((batch, self.seq_len), np.int32)
        labels = np.empty((batch, self.seq_len), np.int32)
        rc = self._lib.gptb200_loader_next_batch(self._ld, rank, world, batch, inputs.ctypes.data, labels.ctypes.data)
        if rc < 0:
            raise GptB200Error(-rc, "gptb200_loader_next_batch")
        return (inputs, labels) if rc == 1 else None
