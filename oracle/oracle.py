"""TEST INFRASTRUCTURE -- numpy front-end of the CPU oracle (not part of the product).

`Oracle` wraps oracle/liboracle.so, the bit-exact restatement of the reference CPU backend's linear-path
operators (oracle/linear_oracle.c).  `Reference` wraps oracle/_ref/libref_cpu.so, the unmodified reference
sources behind a C shim (oracle/ref_shim.cpp); it exists wherever the library was prebuilt.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference legs may import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_LIB = os.path.join(HERE, "liboracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libref_cpu.so")

_f = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_c = ctypes.c_int


def reference_tree() -> str | None:
    """Path of a checkout of the reference: environment variable REF, else a directory `reference` beside this repository."""
    for cand in (os.environ.get("REF"), os.path.join(HERE, "..", "..", "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src", "backend", "cpu")):
            return os.path.abspath(cand)
    return None


def build(force: bool = False) -> None:
    """Compile the restatement, and the reference shims when a reference tree is found (else prebuilt ones are kept)."""
    if force or not os.path.exists(ORACLE_LIB) or os.path.getmtime(ORACLE_LIB) < os.path.getmtime(os.path.join(HERE, "linear_oracle.c")):
        subprocess.run(["make", "-C", HERE, os.path.join(HERE, "liboracle.so")], check=True, capture_output=True)
    ref = reference_tree()
    subprocess.run(["make", "-C", HERE, "ref"] + ([f"REF={ref}"] if ref else []), check=True, capture_output=True)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class _Ops:
    """The five linear-path operators with numpy in/out; `prefix` selects restatement or reference."""

    def __init__(self, lib: ctypes.CDLL, prefix: str):
        self._fwd = getattr(lib, prefix + "linear_forward")
        self._fwd.argtypes = [_f, ctypes.c_void_p, _f, _f, _f, _c, _c, _c, _c]
        self._bwd = getattr(lib, prefix + "linear_backward")
        self._bwd.argtypes = [_f, _f, _f, _f, _f, _f, _c, _c, _c]
        self._gelu = getattr(lib, prefix + "gelu_backward")
        self._gelu.argtypes = [_f, _f, _f, _c, _c]
        self._uf = getattr(lib, prefix + "unembed_forward")
        self._uf.argtypes = [_f, _f, _f, _c, _c, _c]
        self._ub = getattr(lib, prefix + "unembed_backward")
        self._ub.argtypes = [_f, _f, _f, _f, _f, _c, _c, _c]
        for fn in (self._fwd, self._bwd, self._gelu, self._uf, self._ub):
            fn.restype = None

    def linear_forward(self, x, w, b, activation: bool):
        """Returns (y, act) -- act is None without activation.  x [m,k], w [k,n], b [n]."""
        x, w, b = _f32(x), _f32(w), _f32(b)
        m, k = x.shape
        n = w.shape[1]
        y = np.empty((m, n), np.float32)
        act = np.empty((m, n), np.float32) if activation else None
        self._fwd(y, act.ctypes.data if activation else None, x, w, b, int(activation), m, k, n)
        return y, act

    def linear_backward(self, grad_y, x, w, grad_w=None, grad_b=None):
        """Returns (grad_x, grad_w, grad_b); grad_w / grad_b are accumulated into copies of the given arrays."""
        grad_y, x, w = _f32(grad_y), _f32(x), _f32(w)
        m, k = x.shape
        n = w.shape[1]
        gx = np.empty((m, k), np.float32)
        gw = np.zeros((k, n), np.float32) if grad_w is None else _f32(grad_w).copy()
        gb = np.zeros((n,), np.float32) if grad_b is None else _f32(grad_b).copy()
        self._bwd(gx, gw, gb, grad_y, x, w, m, k, n)
        return gx, gw, gb

    def gelu_backward(self, grad_y, x):
        grad_y, x = _f32(grad_y), _f32(x)
        gx = np.empty_like(x)
        m = x.shape[0] if x.ndim == 2 else 1
        n = x.size // max(m, 1) if x.size else 0
        self._gelu(gx, grad_y, x, m, n)
        return gx

    def unembed_forward(self, x, wte):
        x, wte = _f32(x), _f32(wte)
        m, d = x.shape
        vp = wte.shape[0]
        y = np.empty((m, vp), np.float32)
        self._uf(y, x, wte, m, d, vp)
        return y

    def unembed_backward(self, grad_y, x, wte, grad_wte=None):
        grad_y, x, wte = _f32(grad_y), _f32(x), _f32(wte)
        m, d = x.shape
        vp = wte.shape[0]
        gx = np.empty((m, d), np.float32)
        gw = np.zeros((vp, d), np.float32) if grad_wte is None else _f32(grad_wte).copy()
        self._ub(gx, gw, grad_y, x, wte, m, d, vp)
        return gx, gw


class Oracle(_Ops):
    def __init__(self):
        if not os.path.exists(ORACLE_LIB):
            build()
        self.lib = ctypes.CDLL(ORACLE_LIB)
        super().__init__(self.lib, "oracle_")
        self.lib.oracle_num_threads.restype = _c
        self.lib.oracle_set_num_threads.argtypes = [_c]

    def num_threads(self) -> int:
        return int(self.lib.oracle_num_threads())

    def set_num_threads(self, n: int) -> None:
        self.lib.oracle_set_num_threads(n)


def reference_available() -> bool:
    return os.path.exists(REF_LIB)


class Reference(_Ops):
    """Unmodified reference CPU backend (single-threaded scalar loops) and model driver."""

    def __init__(self):
        if not reference_available():
            raise FileNotFoundError(f"{REF_LIB} has not been built (needs the reference tree at build time)")
        self.lib = ctypes.CDLL(REF_LIB)
        super().__init__(self.lib, "ref_")
        self.lib.ref_softmax_forward.argtypes = [_f, _f, _c, _c, _c]
        self.lib.ref_softmax_forward.restype = None
        self.lib.ref_cross_entropy_softmax_backward.argtypes = [_f, _f, _i, _c, _c, _c]
        self.lib.ref_cross_entropy_softmax_backward.restype = None
        self.lib.ref_gpt_forward_backward.argtypes = [_i, _f, ctypes.c_longlong, _i, _i, _c, _c, _c, _f, _f, ctypes.c_void_p]
        self.lib.ref_gpt_forward_backward.restype = _c
        self.lib.ref_gpt_forward_backward_on.argtypes = [ctypes.c_void_p, _i, _f, ctypes.c_longlong, _i, _i, _c, _c, _f, _f, ctypes.c_void_p]
        self.lib.ref_gpt_forward_backward_on.restype = _c

    def adamw_step(self, params, g, m, v, lr, beta1, beta2, eps, weight_decay, step: int):
        """Returns the updated (params, m, v) of the reference's AdamW operator (cpu_backend.cpp:517-532)."""
        fn = self.lib.ref_adamw_step
        fn.argtypes = [_f, _f, _f, _f, _c] + [ctypes.c_float] * 5 + [_c]
        fn.restype = None
        p, g, m, v = _f32(params).copy(), _f32(g).copy(), _f32(m).copy(), _f32(v).copy()
        fn(p, g, m, v, p.size, lr, beta1, beta2, eps, weight_decay, step)
        return p, m, v

    def scale_and_clip_grad(self, g, max_norm: float, accum_steps: int):
        """Returns the gradient after the reference's 1/accum scaling and norm clipping (cpu_backend.cpp:534-556)."""
        fn = self.lib.ref_scale_and_clip_grad
        fn.argtypes = [_f, _c, ctypes.c_float, _c]
        fn.restype = None
        g = _f32(g).copy()
        fn(g, g.size, max_norm, accum_steps)
        return g

    def loader_batches(self, token_file: str, batch: int, seq_len: int, seed: int, epochs: int, max_batches: int):
        """The reference's own DataLoader (data_loader.cpp, unmodified) after srand(seed): (inputs, labels), each
        [batches x batch x seq_len] int32, `epochs` epochs of at most `max_batches` batches."""
        fn = self.lib.ref_loader_batches
        fn.argtypes = [ctypes.c_char_p, _c, _c, ctypes.c_uint, _c, _c, _i, _i]
        fn.restype = _c
        inputs = np.zeros((epochs * max_batches, batch, seq_len), np.int32)
        labels = np.zeros_like(inputs)
        n = fn(token_file.encode(), batch, seq_len, seed, epochs, max_batches, inputs, labels)
        if n < 0:
            raise RuntimeError("the reference DataLoader could not read " + token_file)
        return inputs[:n], labels[:n]

    def softmax_forward(self, logits, vocab_size: int):
        logits = _f32(logits)
        m, vp = logits.shape
        y = np.empty_like(logits)
        self.lib.ref_softmax_forward(y, logits, m, vocab_size, vp)
        return y

    def cross_entropy_softmax_backward(self, probs, labels, vocab_size: int):
        """(probs - onehot) / m with zero padding columns; the caller's buffer starts at zero as after zero_grad."""
        probs = _f32(probs)
        labels = np.ascontiguousarray(labels, dtype=np.int32)
        m, vp = probs.shape
        g = np.zeros_like(probs)
        self.lib.ref_cross_entropy_softmax_backward(g, probs, labels, m, vocab_size, vp)
        return g

    def gpt_forward_backward(self, cfg: dict, weights, inputs, labels, batch: int, seq: int, restated_ops: bool = False,
                             want_logits: bool = False, backend_ptr: int | None = None):
        """One zero_grad/forward/backward/loss of the reference GPT class.  Returns (grads, loss, logits|None).
        `backend_ptr`: address of an IGPTBackend object to run on instead of the reference CPU backend."""
        c = np.array([cfg[k] for k in ("max_seq_len", "vocab_size", "vocab_size_padded", "num_layers", "num_heads", "d_model", "d_ffn")],
                     dtype=np.int32)
        weights = _f32(weights)
        inputs = np.ascontiguousarray(inputs, dtype=np.int32)
        labels = np.ascontiguousarray(labels, dtype=np.int32)
        grads = np.empty_like(weights)
        loss = np.zeros(1, np.float32)
        logits = np.empty((batch * seq, cfg["vocab_size_padded"]), np.float32) if want_logits else None
        if backend_ptr is not None:
            rc = self.lib.ref_gpt_forward_backward_on(ctypes.c_void_p(backend_ptr), c, weights, weights.size, inputs, labels, batch, seq, grads,
                                                      loss, logits.ctypes.data if want_logits else None)
        else:
            rc = self.lib.ref_gpt_forward_backward(c, weights, weights.size, inputs, labels, batch, seq, int(restated_ops), grads, loss,
                                                   logits.ctypes.data if want_logits else None)
        if rc != 0:
            raise RuntimeError(f"ref_gpt_forward_backward failed with code {rc}")
        return grads, float(loss[0]), logits


# Packing order and shapes of the 16 weight tensors (src/model/gpt.cpp:46-62, tools/gpt_reference.py:20-43).
def weight_layout(cfg: dict):
    L, S, Vp, D, F = cfg["num_layers"], cfg["max_seq_len"], cfg["vocab_size_padded"], cfg["d_model"], cfg["d_ffn"]
    return [
        ("wte", (Vp, D)), ("wpe", (S, D)), ("ln_1_w", (L, D)), ("ln_1_b", (L, D)),
        ("qkv_proj_w", (L, D, 3 * D)), ("qkv_proj_b", (L, 3 * D)), ("attn_proj_w", (L, D, D)), ("attn_proj_b", (L, D)),
        ("ln_2_w", (L, D)), ("ln_2_b", (L, D)), ("ffn_up_w", (L, D, F)), ("ffn_up_b", (L, F)),
        ("ffn_down_w", (L, F, D)), ("ffn_down_b", (L, D)), ("ln_f_w", (D,)), ("ln_f_b", (D,)),
    ]


def split_weights(cfg: dict, flat: np.ndarray) -> dict:
    out, off = {}, 0
    for name, shape in weight_layout(cfg):
        n = int(np.prod(shape))
        out[name] = flat[off:off + n].reshape(shape)
        off += n
    assert off == flat.size, (off, flat.size)
    return out
