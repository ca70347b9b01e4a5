"""ctypes access to the test oracle.  TEST INFRASTRUCTURE ONLY.

Two libraries with the same call surface:

* ``port`` -- ``oracle/libkq_oracle.so``, the C restatement (``kq_oracle.c``).
* ``ref``  -- ``oracle/_ref/libkcref.so``, the reference project's own C++ compiled in place
  from the mounted reference tree (``None`` when it was never built).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(np.int64, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")


class AttnDims(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_heads", "ctx", "head_dim", "kv_stride", "group", "ctx_pad", "k_stride")]


class FaDims(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("H", "T", "D", "group", "tp", "k_row", "k_head", "v_row", "v_head", "N",
                                       "q_tok", "q_head", "m_row", "has_mask", "H_kv")]


class Mat(C.Structure):
    _fields_ = [("blocks", C.c_void_p), ("rows", C.c_int), ("k", C.c_int), ("fmt", C.c_int)]


class Layer(C.Structure):
    _fields_ = [(n, Mat) for n in ("wq", "wk", "wv", "wo", "wg", "wu", "wd")] + [
        ("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("q_norm", C.c_void_p), ("k_norm", C.c_void_p)]


class Model(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden", "inter", "n_layers", "heads", "kv_heads", "head_dim", "vocab",
                                       "max_ctx")] + [
        ("eps", C.c_float), ("rope_base", C.c_float), ("layers", C.POINTER(Layer)), ("out_norm", C.c_void_p),
        ("lm_head", Mat), ("rope_ff", C.c_void_p)]


def _sig(lib, prefix):
    def f(name, res, *args):
        fn = getattr(lib, prefix + name)
        fn.restype, fn.argtypes = res, list(args)
    i, fl = C.c_int, C.c_float
    f("f16_to_f32", fl, C.c_uint16)
    f("f32_to_f16", C.c_uint16, fl)
    f("dequant_row_q4k", None, _u8p, i, _f32p)
    f("dequant_row_q6k", None, _u8p, i, _f32p)
    f("quantize_q8x4", None, _f32p, _i32p, _f32p, i)
    f("quantize_q8k", None, _f32p, _i32p, i)
    f("matvec_q4k_q8", None, _u8p, _i32p, _f32p, _f32p, i, i)
    f("matvec_q6k_q8", None, _u8p, _i32p, _f32p, _f32p, i, i)
    f("matvec_q4k_q8k", None, _u8p, _i32p, _f32p, i, i)
    f("matvec_q6k_q8k", None, _u8p, _i32p, _f32p, i, i)
    f("rms_norm", None, _f32p, _f32p, _f32p, i, i, fl)
    f("add", None, _f32p, _f32p, i)
    f("add_rms_norm", None, _f32p, _f32p, _f32p, _f32p, i, fl)
    f("add_sumsq", None, _f32p, _f32p, _i32p, i)
    f("norm_q8x4", None, _f32p, _f32p, _i32p, i, fl)
    f("rope", None, _f32p, i, i, i, fl)
    f("rope_ff", None, _f32p, _f32p, i, i, i, fl)
    f("rope_ggml", None, _f32p, _f32p, _i32p, _f32p, i, i, i, fl, i)
    f("append_kv", None, _f32p, _f32p, _f32p, _f32p, i, i, i)
    f("attn_scores", None, _f32p, _f32p, _f32p, C.POINTER(AttnDims), fl)
    f("softmax", None, _f32p, i, i, i)
    f("attn_values", None, _f32p, _f32p, _f32p, C.POINTER(AttnDims))
    f("silu_mul", None, _f32p, _f32p, _f32p, i)
    f("silu_mul_q8x4", None, _f32p, _f32p, _i32p, _f32p, i)
    f("mul_rows", None, _f32p, _f32p, _f32p, i, i)
    f("add_sumsq_f", None, _f32p, _f32p, _f32p, _i32p, i, i)
    f("sumsq_part", None, _f32p, _i32p, i, i)
    f("norm_mul_q8", None, _f32p, _f32p, _f32p, _i32p, i, i, fl)
    f("norm_mul_q8k", None, _f32p, _f32p, _f32p, _i32p, _i32p, i, i, fl)
    f("silu_mul_q8f", None, _f32p, _f32p, _f32p, _i32p, i, i)
    f("silu_mul_q8k", None, _f32p, _f32p, _f32p, _i32p, i, i)
    f("matvec_q8w", None, _i8p, _f32p, _f32p, _f32p, i, i)
    f("matvec_q4w", None, _u8p, _f32p, _f32p, _f32p, i, i)
    f("repack_q4x8", None, _u8p, _f32p, _u8p, _f32p, i, i)
    f("matvec_q4x8", None, _u8p, _f32p, _f32p, _f32p, i, i)
    f("repack_q4x8_q8", None, _u8p, _f32p, _i32p, i, i)
    f("matvec_q4x8_q8", None, _i32p, _i32p, _f32p, _f32p, i, i)
    f("repack_f16", None, _u16p, i, i, _i32p)
    f("matmul_f16", None, _u16p, _f32p, _f32p, i, i, i)
    f("set_rows_f16", None, _f32p, _i64p, _u16p, i, i, i, i, i)
    f("flash_attn_f16", None, _f32p, _u16p, _u16p, _u16p, _f32p, C.POINTER(FaDims), fl)


class _Lib:
    """Attribute access strips the library's symbol prefix: ``port.rms_norm(...)``."""

    def __init__(self, path, prefix):
        self.path, self.prefix = path, prefix
        self.lib = C.CDLL(path)
        _sig(self.lib, prefix)

    def __getattr__(self, name):
        return getattr(self.lib, self.prefix + name)


def build(with_ref: bool = True) -> None:
    """Compile the oracle (and, where the reference tree is mounted, oracle/_ref)."""
    subprocess.run(["make", "-C", _HERE, "all" if with_ref else "port"], check=True, stdout=subprocess.DEVNULL)


def _load_port():
    path = os.path.join(_HERE, "libkq_oracle.so")
    if not os.path.exists(path):
        build(with_ref=False)
    lib = _Lib(path, "kqo_")
    i = C.c_int
    lib.lib.kqo_matvec_dequant_f64.restype = None
    lib.lib.kqo_matvec_dequant_f64.argtypes = [_u8p, _f32p, _f32p, i, i, i]
    lib.lib.kqo_decode_token.restype = None
    lib.lib.kqo_decode_token.argtypes = [C.POINTER(Model), _f32p, i, _f32p, _f32p, _i32p]
    lib.lib.kqo_decode_token_ex.restype = None
    lib.lib.kqo_decode_token_ex.argtypes = [C.POINTER(Model), _f32p, i, _f32p, _f32p, _i32p, i]
    lib.lib.kqo_decode_scratch_floats.restype = C.c_long
    lib.lib.kqo_decode_scratch_floats.argtypes = [C.POINTER(Model)]
    lib.lib.kqo_decode_set_trace.restype = None
    lib.lib.kqo_decode_set_trace.argtypes = [C.c_void_p, C.c_long]
    lib.lib.kqo_decode_trace_words.restype = C.c_long
    lib.lib.kqo_decode_set_forced.restype = None
    lib.lib.kqo_decode_set_forced.argtypes = [C.c_void_p, C.c_long]
    lib.lib.kqo_decode_forced_stats.restype = None
    lib.lib.kqo_decode_forced_stats.argtypes = [C.POINTER(C.c_long), C.POINTER(C.c_long), C.POINTER(C.c_int), C.POINTER(C.c_float)]
    lib.lib.kqo_decode_scratch_ints.restype = C.c_long
    lib.lib.kqo_decode_scratch_ints.argtypes = [C.POINTER(Model)]
    return lib


def _load_ref():
    path = os.path.join(_HERE, "_ref", "libkcref.so")
    if not os.path.exists(path):
        return None
    lib = _Lib(path, "kcref_")
    i = C.c_int
    L = lib.lib
    L.kcref_stream_ints.restype, L.kcref_stream_ints.argtypes = C.c_long, [i, i, i]
    L.kcref_repack.restype, L.kcref_repack.argtypes = None, [_u8p, i, i, i, _i32p]
    L.kcref_matvec_stream_q8.restype = None
    L.kcref_matvec_stream_q8.argtypes = [_i32p, _i32p, _f32p, _f32p, i, i, i]
    L.kcref_matvec_stream_q8k.restype = None
    L.kcref_matvec_stream_q8k.argtypes = [_i32p, _i32p, _f32p, i, i, i]
    L.kcref_gguf_open.restype, L.kcref_gguf_open.argtypes = C.c_void_p, [C.c_char_p, i]
    L.kcref_gguf_last_error.restype = C.c_char_p
    L.kcref_gguf_config.restype, L.kcref_gguf_config.argtypes = None, [C.c_void_p, C.POINTER(C.c_int * 8), C.POINTER(C.c_float), C.POINTER(C.c_float)]
    L.kcref_gguf_tensor.restype = i
    L.kcref_gguf_tensor.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint), C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong),
                                    C.POINTER(C.c_longlong * 4), C.POINTER(C.c_ulonglong)]
    L.kcref_gguf_decode.restype, L.kcref_gguf_decode.argtypes = i, [C.c_void_p, i, i, _f32p]
    L.kcref_gguf_close.restype, L.kcref_gguf_close.argtypes = None, [C.c_void_p]
    L.kcref_synthetic_tiny_logits.restype = i
    L.kcref_synthetic_tiny_logits.argtypes = [i, C.c_ulonglong, C.c_ulonglong, i, _f32p, C.POINTER(C.c_double)]
    L.kcref_model_open.restype, L.kcref_model_open.argtypes = C.c_void_p, [C.POINTER(Model)]
    L.kcref_model_decode.restype, L.kcref_model_decode.argtypes = i, [C.c_void_p, _f32p, i, _f32p]
    L.kcref_model_close.restype, L.kcref_model_close.argtypes = None, [C.c_void_p]
    return lib


port = _load_port()
ref = _load_ref()


# ---- numpy conveniences shared by the tests ------------------------------------------------------

def quantize_q8x4(lib, x):
    """x: float32[k] -> (xq int32[k/32*8], xd float32[k/32*2])."""
    x = np.ascontiguousarray(x, np.float32)
    nb = x.size // 32
    xq, xd = np.zeros(nb * 8, np.int32), np.zeros(nb * 2, np.float32)
    lib.quantize_q8x4(x, xq, xd, nb)
    return xq, xd


def quantize_q8k(lib, x):
    x = np.ascontiguousarray(x, np.float32)
    nsb = x.size // 256
    q = np.zeros(nsb * 85, np.int32)
    lib.quantize_q8k(x, q, nsb)
    return q


def dequant(lib, blocks, rows, k, q6):
    out = np.zeros((rows, k), np.float32)
    rb = (k // 256) * (210 if q6 else 144)
    blocks = np.ascontiguousarray(blocks, np.uint8).reshape(rows, rb)
    fn = lib.dequant_row_q6k if q6 else lib.dequant_row_q4k
    for r in range(rows):
        fn(np.ascontiguousarray(blocks[r]), k, out[r])
    return out


def matvec_q8(lib, blocks, x, rows, k, q6):
    """The reference's decode matvec: quantize x per 32, integer dot products."""
    xq, xd = quantize_q8x4(lib, x)
    y = np.zeros(rows, np.float32)
    (lib.matvec_q6k_q8 if q6 else lib.matvec_q4k_q8)(np.ascontiguousarray(blocks, np.uint8).ravel(), xq, xd, y, rows, k)
    return y


def matvec_q8k(lib, blocks, x, rows, k, q6):
    q = quantize_q8k(lib, x)
    y = np.zeros(rows, np.float32)
    (lib.matvec_q6k_q8k if q6 else lib.matvec_q4k_q8k)(np.ascontiguousarray(blocks, np.uint8).ravel(), q, y, rows, k)
    return y


def matvec_dequant_f64(blocks, x, rows, k, q6):
    y = np.zeros(rows, np.float32)
    port.lib.kqo_matvec_dequant_f64(np.ascontiguousarray(blocks, np.uint8).ravel(),
                                    np.ascontiguousarray(x, np.float32), y, rows, k, int(q6))
    return y


class BoundModel:
    """A numpy model (kernelcore_b200.tiny_model.build) bound to the oracle's C structs, with its own
    fp32 KV caches.  Keeps every array alive for the lifetime of the struct."""

    def __init__(self, shape, model):
        self.shape, self.model = shape, model
        self._keep = []
        s = shape
        self.layers = (Layer * s.layers)()
        from kernelcore_b200 import tiny_model as tm
        ms = tm.mat_shapes(s)
        self.k_cache, self.v_cache = [], []
        for l, L in enumerate(model["layers"]):
            for name in tm.MATS:
                rows, k, q6 = ms[name]
                setattr(self.layers[l], name, self._mat(L[name], rows, k, q6))
            self.layers[l].attn_norm = self._ptr(L["attn_norm"])
            self.layers[l].ffn_norm = self._ptr(L["ffn_norm"])
            if s.qk_norm:
                self.layers[l].q_norm = self._ptr(L["q_norm"])
                self.layers[l].k_norm = self._ptr(L["k_norm"])
            kc = np.zeros((s.kv, (s.max_ctx + 7) // 8 * 8), np.float32)
            vc = np.zeros((s.max_ctx, s.kv), np.float32)
            self.k_cache.append(kc)
            self.v_cache.append(vc)
            self.layers[l].k_cache = self._ptr(kc)
            self.layers[l].v_cache = self._ptr(vc)
        self.c = Model()
        for f in ("hidden", "inter", "heads", "kv_heads", "head_dim", "vocab", "max_ctx"):
            setattr(self.c, f, getattr(s, f))
        self.c.n_layers = s.layers
        self.c.eps, self.c.rope_base = s.eps, s.rope_base
        self.c.layers = C.cast(self.layers, C.POINTER(Layer))
        self.c.out_norm = self._ptr(model["out_norm"])
        self.c.lm_head = self._mat(model["lm_head"], s.vocab, s.hidden, True)
        self.c.rope_ff = None

    def _ptr(self, a):
        a = np.ascontiguousarray(a)
        self._keep.append(a)
        return a.ctypes.data

    def _mat(self, blocks, rows, k, q6):
        return Mat(self._ptr(blocks), rows, k, 6 if q6 else 4)

    def embed(self, token: int) -> np.ndarray:
        """Tied embeddings: the token's row of the Q6_K output matrix, dequantised
        (llm/gguf_model.cpp:96-104)."""
        out = np.zeros(self.shape.hidden, np.float32)
        port.dequant_row_q6k(np.ascontiguousarray(self.model["lm_head"][token]), self.shape.hidden, out)
        return out

    def trace_words(self) -> int:
        """int32 words one decode step traces: layer 0's q|k|v input words, then per layer the wo input words,
        the residual stream (hidden floats), the gate|up and down input words, the residual stream again and the
        next q|k|v (after the last layer: lm_head) input words; a vector of k int8 values is k / 4 words."""
        s = self.shape
        return s.layers * ((2 * s.hidden + s.qd + s.inter) // 4 + 2 * s.hidden) + s.hidden // 4

    def trace_layout(self):
        """[(kind, first word, words)] of one step's trace, kind "q8" or "x"."""
        s, out, at = self.shape, [], 0
        def add(kind, n):
            nonlocal at
            out.append((kind, at, n))
            at += n
        add("q8", s.hidden // 4)
        for _ in range(s.layers):
            add("q8", s.qd // 4), add("x", s.hidden), add("q8", s.hidden // 4), add("q8", s.inter // 4), add("x", s.hidden), add("q8", s.hidden // 4)
        return out

    def decode_port(self, x_in, pos, kv_f16=False, trace=None, forced=None):
        """One decode step on the CPU oracle.  kv_f16: K/V rounded to fp16 on entry to the cache; the
        model shape's neox / qk_norm select the Qwen3-style variants.  trace: an int32 array of
        trace_words() that receives the int8 words of every activation vector the step quantizes.
        forced: the words another implementation traced for this step; each vector the step quantizes is
        compared with them and then replaced by them, and so is the residual stream after each addition
        (self.forced_stats = differing int8 values, vectors holding one, largest int8 step, largest residual
        difference relative to its largest magnitude), so every stage runs on the inputs the other
        implementation had."""
        logits = np.zeros(self.shape.vocab, np.float32)
        if forced is not None:
            assert forced.dtype == np.int32 and forced.size == self.trace_words() and forced.flags.c_contiguous
            port.lib.kqo_decode_set_forced(forced.ctypes.data, forced.size)
        if trace is not None:
            assert trace.dtype == np.int32 and trace.size >= self.trace_words() and trace.flags.c_contiguous
            port.lib.kqo_decode_set_trace(trace.ctypes.data, trace.size)
        sf = np.zeros(port.lib.kqo_decode_scratch_floats(C.byref(self.c)), np.float32)
        sq = np.zeros(port.lib.kqo_decode_scratch_ints(C.byref(self.c)), np.int32)
        flags = (1 if kv_f16 else 0) | (2 if self.shape.neox else 0) | (4 if self.shape.qk_norm else 0)
        port.lib.kqo_decode_token_ex(C.byref(self.c), np.ascontiguousarray(x_in, np.float32), pos, logits, sf, sq, flags)
        if trace is not None:
            assert port.lib.kqo_decode_trace_words() == self.trace_words()
            port.lib.kqo_decode_set_trace(None, 0)
        if forced is not None:
            a, b, c, x = C.c_long(), C.c_long(), C.c_int(), C.c_float()
            port.lib.kqo_decode_forced_stats(C.byref(a), C.byref(b), C.byref(c), C.byref(x))
            self.forced_stats = (a.value, b.value, c.value, x.value)
            port.lib.kqo_decode_set_forced(None, 0)
        return logits
