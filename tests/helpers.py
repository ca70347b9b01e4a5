"""Shared test helpers: bit comparisons, the reference's relDiff, and oracle model structs."""
from __future__ import annotations

import ctypes as C

import numpy as np

import oracle


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({4: np.uint32, 2: np.uint16, 8: np.uint64}[a.dtype.itemsize])


def bit_equal(a, b) -> bool:
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and bool((bits(a) == bits(b)).all())


def rel_diff(a, b) -> float:
    """max|a-b| / max|b| -- the reference's relDiff (tests/test_llm_kernels.cpp:54-63)."""
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    if a.shape != b.shape or a.size == 0 or not np.isfinite(a).all():
        return 1e30
    scale = np.abs(b).max()
    m = np.abs(a - b).max()
    return float(m / scale) if scale > 0 else float(m)


def pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class OracleModel:
    """A numpy model (kernelcore_b200.tiny_model.build) bound to the oracle's C structs, with its own
    fp32 KV caches.  Keeps every array alive for the lifetime of the struct."""

    def __init__(self, shape, model):
        self.shape, self.model = shape, model
        self._keep = []
        s = shape
        self.layers = (oracle.Layer * s.layers)()
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
            kc = np.zeros((s.kv, pad8(s.max_ctx)), np.float32)
            vc = np.zeros((s.max_ctx, s.kv), np.float32)
            self.k_cache.append(kc)
            self.v_cache.append(vc)
            self.layers[l].k_cache = self._ptr(kc)
            self.layers[l].v_cache = self._ptr(vc)
        self.c = oracle.Model()
        for f in ("hidden", "inter", "heads", "kv_heads", "head_dim", "vocab", "max_ctx"):
            setattr(self.c, f, getattr(s, f))
        self.c.n_layers = s.layers
        self.c.eps, self.c.rope_base = s.eps, s.rope_base
        self.c.layers = C.cast(self.layers, C.POINTER(oracle.Layer))
        self.c.out_norm = self._ptr(model["out_norm"])
        self.c.lm_head = self._mat(model["lm_head"], s.vocab, s.hidden, True)
        self.c.rope_ff = None

    def _ptr(self, a):
        a = np.ascontiguousarray(a)
        self._keep.append(a)
        return a.ctypes.data

    def _mat(self, blocks, rows, k, q6):
        return oracle.Mat(self._ptr(blocks), rows, k, 6 if q6 else 4)

    def embed(self, token: int) -> np.ndarray:
        """Tied embeddings: the token's row of the Q6_K output matrix, dequantised
        (llm/gguf_model.cpp:96-104)."""
        out = np.zeros(self.shape.hidden, np.float32)
        oracle.port.dequant_row_q6k(np.ascontiguousarray(self.model["lm_head"][token]), self.shape.hidden, out)
        return out

    def decode_port(self, x_in, pos, kv_f16=False):
        """One decode step on the CPU oracle.  kv_f16: K/V rounded to fp16 on entry to the cache; the
        model shape's neox / qk_norm select the Qwen3-style variants."""
        logits = np.zeros(self.shape.vocab, np.float32)
        sf = np.zeros(oracle.port.lib.kqo_decode_scratch_floats(C.byref(self.c)), np.float32)
        sq = np.zeros(oracle.port.lib.kqo_decode_scratch_ints(C.byref(self.c)), np.int32)
        flags = (1 if kv_f16 else 0) | (2 if self.shape.neox else 0) | (4 if self.shape.qk_norm else 0)
        oracle.port.lib.kqo_decode_token_ex(C.byref(self.c), np.ascontiguousarray(x_in, np.float32), pos, logits, sf, sq, flags)
        return logits
