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


OracleModel = oracle.BoundModel


def oracle_prefill(shape, model, tokens, q8k=True, tail_q8k=False, tail_ggml=False):
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
    if tail_q8k:   # the batched decode step: add + norm + per-256 quantization of the row, K-quant matvec on the slot
        xr, tr = np.ascontiguousarray(X[n - 1:n]), np.ascontiguousarray(T[n - 1:n])
        sq, slot, yn = np.zeros((1, nb * 11), np.int32), np.zeros((1, 85 * nsbh), np.int32), np.zeros((1, s.hidden), np.float32)
        P.add_sumsq_f(xr, tr, xr, sq, s.hidden, 1)
        P.norm_mul_q8k(xr, np.ascontiguousarray(model["out_norm"], np.float32), yn, slot, sq, s.hidden, 1, s.eps)
        out = np.zeros(s.vocab, np.float32)
        P.matvec_q6k_q8k(np.ascontiguousarray(model["lm_head"], np.uint8).ravel(), slot[0], out, s.vocab, s.hidden)
        return out
    if tail_ggml:  # the ggml graph's last row: ADD + RMS_NORM + MUL fused with per-32 quantization, then the matvec on it
        xr, tr = np.ascontiguousarray(X[n - 1:n]), np.ascontiguousarray(T[n - 1:n])
        slot, yn = np.zeros((1, nb * 11), np.int32), np.zeros((1, s.hidden), np.float32)
        P.add_sumsq_f(xr, tr, xr, slot, s.hidden, 1)
        P.norm_mul_q8(xr, np.ascontiguousarray(model["out_norm"], np.float32), yn, slot, s.hidden, 1, s.eps)
        out = np.zeros(s.vocab, np.float32)
        P.matvec_q6k_q8(np.ascontiguousarray(model["lm_head"], np.uint8).ravel(), slot[0, :nb * 8], slot[0, nb * 8:nb * 10].view(np.float32), out,
                        s.vocab, s.hidden)
        return out
    x = X[n - 1] + T[n - 1]
    y = np.zeros(s.hidden, np.float32)
    P.rms_norm(x, np.ascontiguousarray(model["out_norm"], np.float32), y, s.hidden, 1, s.eps)
    return oracle.matvec_q8(P, model["lm_head"], y, s.vocab, s.hidden, 1)
