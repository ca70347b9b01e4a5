"""Shared test helpers: bit comparisons, the reference's relDiff, and oracle model structs."""
from __future__ import annotations

import ctypes as C

import numpy as np

import oracle


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({1: np.uint8, 4: np.uint32, 2: np.uint16, 8: np.uint64}[a.dtype.itemsize])


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


def oracle_prefill(shape, model, tokens, q8k=True):
    """The batched prompt pass restated on the CPU oracle, op for op as the reference's batched (ggml) path runs
    it: add + partial sums of squares, RMSNorm * weight + per-256 quantization (add_sumsq_f / sumsq_part /
    norm_mul_q8k), K-quant matvecs on per-256 slots per token, per-head q/k RMSNorm and rope_ggml, fp16 KV rows
    (set_rows_f16), flash_attn_f16 with a causal mask, silu_mul_q8k.  Returns the logits of the last token
    (final RMSNorm + per-32 quantization + Q6_K matvec, the decode tail)."""
    from kernelcore_b200 import tiny_model as tm
    P, s = oracle.port, shape
    n, H, KV, D = len(tokens), s.heads, s.kv_heads, s.head_dim
    qd, kv, nb, nsbh = s.qd, s.kv, s.hidden // 32, s.hidden // 256
    ms = tm.mat_shapes(s)
    ones = np.ones(D // 2, np.float32)
    pos = np.arange(n, dtype=np.int32)
    log2_base = float(np.log2(np.float32(s.rope_base)))

    def mm(blocks, slots, name):
        rows, k, q6 = ms[name]
        out = np.zeros((n, rows), np.float32)
        w = np.ascontiguousarray(blocks, np.uint8).ravel()
        if q8k:
            fn = P.matvec_q6k_q8k if q6 else P.matvec_q4k_q8k
            for c in range(n):
                fn(w, slots[c], out[c], rows, k)
        else:   # per-32 slots [k/32*8 words | k/32 {d, sum} | ...] -- only used to cross-check this function's plumbing
            fn = P.matvec_q6k_q8 if q6 else P.matvec_q4k_q8
            for c in range(n):
                fn(w, slots[c][:k // 4], slots[c][k // 4:k // 4 + k // 16].view(np.float32), out[c], rows, k)
        return out

    def quant_rows(Y, k):
        if q8k:
            sl = np.zeros((n, 85 * (k // 256)), np.int32)
            for c in range(n):
                P.quantize_q8k(Y[c], sl[c], k // 256)
        else:
            sl = np.zeros((n, 11 * (k // 32)), np.int32)
            for c in range(n):
                xq, xd = oracle.quantize_q8x4(P, Y[c])
                sl[c, :k // 4], sl[c, k // 4:k // 4 + k // 16] = xq, xd.view(np.int32)
        return sl

    X = np.zeros((n, s.hidden), np.float32)
    for i, t in enumerate(tokens):
        P.dequant_row_q6k(np.ascontiguousarray(model["lm_head"][t]), s.hidden, X[i])
    T = None
    tp = pad8(n)
    mask = np.full((n, tp), 0xFC00, np.uint16)
    for i in range(n):
        mask[i, :i + 1] = 0
    for L in model["layers"]:
        sq = np.zeros((n, nb * 11), np.int32)
        if T is None:
            P.sumsq_part(X, sq, s.hidden, n)
        else:
            P.add_sumsq_f(X, T, X, sq, s.hidden, n)
        slots, Y = np.zeros((n, 85 * nsbh), np.int32), np.zeros_like(X)
        P.norm_mul_q8k(X, np.ascontiguousarray(L["attn_norm"], np.float32), Y, slots, sq, s.hidden, n, s.eps)
        if not q8k:
            slots = quant_rows(Y, s.hidden)
        q, k, v = mm(L["wq"], slots, "wq"), mm(L["wk"], slots, "wk"), mm(L["wv"], slots, "wv")
        if s.qk_norm:
            qn, kn = np.zeros_like(q), np.zeros_like(k)
            P.rms_norm(q, np.ascontiguousarray(L["q_norm"], np.float32), qn, D, n * H, s.eps)
            P.rms_norm(k, np.ascontiguousarray(L["k_norm"], np.float32), kn, D, n * KV, s.eps)
            q, k = qn, kn
        qr, kr = np.zeros_like(q), np.zeros_like(k)
        P.rope_ggml(q, qr, pos, ones, D, H, n, log2_base, int(s.neox))
        P.rope_ggml(k, kr, pos, ones, D, KV, n, log2_base, int(s.neox))
        kc, vc = np.zeros((n, kv), np.uint16), np.zeros((n, kv), np.uint16)
        idx = np.arange(n, dtype=np.int64)
        P.set_rows_f16(kr, idx, kc, kv // 2, n, kv, kv // 2, n)
        P.set_rows_f16(np.ascontiguousarray(v), idx, vc, kv // 2, n, kv, kv // 2, n)
        d = oracle.FaDims(H, n, D, H // KV, tp, kv // 2, D // 2, kv // 2, D // 2, n, qd, D, tp // 2, 1, KV)
        A = np.zeros((n, qd), np.float32)
        P.flash_attn_f16(qr, kc, vc, mask, A, C.byref(d), float(np.float32(1.0) / np.sqrt(np.float32(D))))
        T = mm(L["wo"], quant_rows(A, qd), "wo")
        sq = np.zeros((n, nb * 11), np.int32)
        P.add_sumsq_f(X, T, X, sq, s.hidden, n)
        slots = np.zeros((n, 85 * nsbh), np.int32)
        P.norm_mul_q8k(X, np.ascontiguousarray(L["ffn_norm"], np.float32), Y, slots, sq, s.hidden, n, s.eps)
        if not q8k:
            slots = quant_rows(Y, s.hidden)
        g, u = mm(L["wg"], slots, "wg"), mm(L["wu"], slots, "wu")
        act, islots = np.zeros_like(g), np.zeros((n, 85 * (s.inter // 256)), np.int32)
        P.silu_mul_q8k(g, u, act, islots, s.inter, n)
        T = mm(L["wd"], islots if q8k else quant_rows(act, s.inter), "wd")
    x = X[n - 1] + T[n - 1]
    y = np.zeros(s.hidden, np.float32)
    P.rms_norm(x, np.ascontiguousarray(model["out_norm"], np.float32), y, s.hidden, 1, s.eps)
    return oracle.matvec_q8(P, model["lm_head"], y, s.vocab, s.hidden, 1)
