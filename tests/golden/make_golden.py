"""Generates tests/golden/*.npz from the reference project's own C++ implementation
(oracle/_ref/libkcref.so, built by `make -C oracle` from the mounted reference tree).

Run from the repository root:  python tests/golden/make_golden.py
Inputs are seeded; every output array in the fixtures was computed by the reference's llm::ref
functions or its decodeToken loop, never by the restatement or by GPU code."""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from helpers import OracleModel, pad8  # noqa: E402
from kernelcore_b200 import synth, tiny_model as tm  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
ref = oracle.ref
assert ref is not None, "build oracle/_ref first (make -C oracle)"


def save(name, **arrays):
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **arrays)
    print(name, {k: v.shape for k, v in arrays.items()})


def kquant():
    out = {}
    for q6 in (0, 1):
        for rows, k in ((8, 256), (40, 768)):  # the reference's own test shapes
            tag = f"{'q6k' if q6 else 'q4k'}_{rows}x{k}"
            w = synth.raw_blocks(rows, k, rows * 31 + k + q6, bool(q6))
            x = np.random.default_rng(61).uniform(-3, 3, k).astype(np.float32)
            xq, xd = oracle.quantize_q8x4(ref, x)
            out[tag + "_w"], out[tag + "_x"] = w, x
            out[tag + "_xq"], out[tag + "_xd"] = xq, xd
            out[tag + "_slot"] = oracle.quantize_q8k(ref, x)
            out[tag + "_deq"] = oracle.dequant(ref, w, rows, k, q6)
            out[tag + "_y_q8"] = oracle.matvec_q8(ref, w, x, rows, k, q6)
            out[tag + "_y_q8k"] = oracle.matvec_q8k(ref, w, x, rows, k, q6)
    save("kquant", **out)


def halfs():
    rng = np.random.default_rng(5)
    specials = np.array([0.0, -0.0, 1.0, -1.0, 65504.0, 65519.0, 65520.0, -70000.0, 5.9604645e-08, 2.9802322e-08,
                         6.0975552e-05, 6.1035156e-05, 1.00048828125, 1.0009765625, 1.00146484375, 3.14159,
                         1e-10, -1e-10, 1e10], np.float32)
    vals = np.concatenate([specials, (rng.standard_normal(4000) * 10 ** rng.uniform(-6, 5, 4000)).astype(np.float32)])
    h = np.array([ref.f32_to_f16(float(v)) for v in vals], np.uint16)
    allh = np.arange(65536, dtype=np.uint16)
    back = np.array([ref.f16_to_f32(int(v)) for v in allh], np.float32)
    save("halfs", f32=vals, f16=h, f16_to_f32_all=back.view(np.uint32))


def glue():
    rng = np.random.default_rng(11)
    out = {}
    n, m = 3072, 8192
    x, t = rng.uniform(-1, 1, n).astype(np.float32), rng.uniform(-1, 1, n).astype(np.float32)
    w = rng.uniform(0.5, 1.5, n).astype(np.float32)
    y = np.zeros(n, np.float32)
    ref.rms_norm(x, w, y, n, 1, 1e-5)
    out.update(norm_x=x, norm_t=t, norm_w=w, rms_norm_y=y.copy())
    rows = rng.uniform(-2, 2, (5, 128)).astype(np.float32)
    wr = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    yr = np.zeros_like(rows)
    ref.rms_norm(rows, wr, yr, 128, 5, 1e-6)
    out.update(rows_x=rows, rows_w=wr, rows_y=yr)
    x2 = x.copy()
    q = np.zeros(11 * n // 32, np.int32)
    ref.add_sumsq(x2, t, q, n // 32)
    ref.norm_q8x4(x2, w, q, n // 32, 1e-5)
    out.update(addnorm_x=x2, addnorm_q=q)
    x3 = x.copy()
    y3 = np.zeros(n, np.float32)
    ref.add_rms_norm(x3, t, w, y3, n, 1e-5)
    out.update(add_rms_norm_y=y3)
    g, u = rng.uniform(-4, 4, m).astype(np.float32), rng.uniform(-2, 2, m).astype(np.float32)
    h = np.zeros(m, np.float32)
    ref.silu_mul(g, u, h, m)
    xq, xd = np.zeros(m // 4, np.int32), np.zeros(m // 16, np.float32)
    ref.silu_mul_q8x4(g, u, xq, xd, m // 32)
    out.update(silu_g=g, silu_u=u, silu_h=h, silu_xq=xq, silu_xd=xd)
    # rope: 3 heads of 64 pairs, positions incl. large ones
    for pos in (0, 1, 517, 4095):
        r = rng.uniform(-1, 1, 3 * 128).astype(np.float32)
        out[f"rope_in_{pos}"] = r.copy()
        a = r.copy()
        ref.rope(a, 64, pos, 3 * 64, float(np.log2(500000.0)))
        out[f"rope_out_{pos}"] = a
        ff = rng.uniform(1, 8, 64).astype(np.float32)
        b = r.copy()
        ref.rope_ff(b, ff, 64, pos, 3 * 64, float(np.log2(500000.0)))
        out[f"ropeff_ff_{pos}"], out[f"ropeff_out_{pos}"] = ff, b
    posv = np.array([0, 3, 77, 1000], np.int32)
    xg = rng.uniform(-1, 1, 4 * 3 * 128).astype(np.float32)
    ones = np.ones(64, np.float32)
    for neox in (0, 1):
        yg = np.zeros_like(xg)
        ref.rope_ggml(xg, yg, posv, ones, 128, 3, 4, float(np.log2(1e6)), neox)
        out[f"ropeggml_y_{neox}"] = yg
    out.update(ropeggml_x=xg, ropeggml_pos=posv)
    # attention: 6 heads / 2 kv heads, head 64, ctx 77 inside a cache of 96
    d = oracle.AttnDims(6, 77, 64, 128, 3, pad8(77), 96)
    qv = rng.uniform(-1, 1, 6 * 64).astype(np.float32)
    kt = rng.uniform(-1, 1, (128, 96)).astype(np.float32)
    vc = rng.uniform(-1, 1, (96, 128)).astype(np.float32)
    sc = np.zeros((6, pad8(77)), np.float32)
    ref.attn_scores(qv, kt, sc, C.byref(d), 0.125)
    p = sc.copy()
    ref.softmax(p, 77, pad8(77), 6)
    o = np.zeros(6 * 64, np.float32)
    ref.attn_values(p, vc, o, C.byref(d))
    out.update(attn_q=qv, attn_kt=kt, attn_v=vc, attn_scores=sc, attn_p=p, attn_out=o)
    # fp16 cache path: set_rows with an out-of-range row, flash attention with and without mask
    src = rng.uniform(-3, 3, (5, 256)).astype(np.float32)
    idx = np.array([2, 0, 9, -1, 40], np.int64)
    dst = np.zeros((12, 256), np.uint16)
    ref.set_rows_f16(src, idx, dst, 128, 5, 256, 128, 12)
    out.update(setrows_src=src, setrows_idx=idx, setrows_dst=dst)
    for tag, (H, Hkv, D, T, N, mask) in {"a": (6, 2, 64, 37, 1, 0), "b": (10, 2, 64, 37, 3, 1), "c": (4, 4, 128, 150, 2, 1)}.items():
        kc = rng.uniform(-1, 1, (T, Hkv * D)).astype(np.float16)
        vcc = rng.uniform(-1, 1, (T, Hkv * D)).astype(np.float16)
        qq = rng.uniform(-1, 1, (N, H, D)).astype(np.float32)
        tp = pad8(T)
        mk = np.zeros((N, tp), np.float16)
        if mask:
            for i in range(N):
                mk[i, T - (N - 1 - i):] = -np.inf  # causal tail
        fd = oracle.FaDims(H, T, D, H // Hkv, tp, Hkv * D // 2, D // 2, Hkv * D // 2, D // 2, N, H * D, D, tp // 2, mask, Hkv)
        fo = np.zeros((N, H, D), np.float32)
        ref.flash_attn_f16(qq, kc.view(np.uint16), vcc.view(np.uint16), mk.view(np.uint16), fo, C.byref(fd), float(D) ** -0.5)
        out.update({f"fa_{tag}_q": qq, f"fa_{tag}_k": kc.view(np.uint16), f"fa_{tag}_v": vcc.view(np.uint16),
                    f"fa_{tag}_mask": mk.view(np.uint16), f"fa_{tag}_out": fo,
                    f"fa_{tag}_dims": np.array([H, Hkv, D, T, N, mask], np.int32)})
    save("glue", **out)


def batched():
    """Column-batched quantizers and per-column matmul results (the matmul kernels are bit-identical per
    column to the matvec mirror, llm/llm_kernels.hpp:255-262)."""
    rng = np.random.default_rng(23)
    out = {}
    rows, k, ncols = 40, 768, 13
    X = rng.uniform(-3, 3, (ncols, k)).astype(np.float32)
    out["X"] = X
    for q6 in (0, 1):
        tag = "q6k" if q6 else "q4k"
        w = synth.raw_blocks(rows, k, 900 + q6, bool(q6))
        out[tag + "_w"] = w
        out[tag + "_Y_q8"] = np.stack([oracle.matvec_q8(ref, w, X[c], rows, k, q6) for c in range(ncols)])
        out[tag + "_Y_q8k"] = np.stack([oracle.matvec_q8k(ref, w, X[c], rows, k, q6) for c in range(ncols)])
    out["slots_q8k"] = np.stack([oracle.quantize_q8k(ref, X[c]) for c in range(ncols)])
    # fused ggml forms on 3 rows of 512
    n, r = 512, 3
    a, b = rng.uniform(-1, 1, (r, n)).astype(np.float32), rng.uniform(-1, 1, (r, n)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, n).astype(np.float32)
    s = np.zeros((r, n), np.float32)
    q = np.zeros(r * 11 * (n // 32), np.int32)
    ref.add_sumsq_f(a, b, s, q, n, r)
    y = np.zeros((r, n), np.float32)
    ref.norm_mul_q8(s, w, y, q, n, r, 1e-5)
    out.update(f_a=a, f_b=b, f_w=w, f_sum=s, f_y=y, f_q=q.copy())
    qk = np.zeros(r * 85 * (n // 256), np.int32)
    sq = np.zeros(r * 11 * (n // 32), np.int32)
    ref.sumsq_part(s, sq, n, r)
    yk = np.zeros((r, n), np.float32)
    ref.norm_mul_q8k(s, w, yk, qk, sq, n, r, 1e-5)
    out.update(f_yk=yk, f_qk=qk)
    g, u = rng.uniform(-4, 4, (r, n)).astype(np.float32), rng.uniform(-2, 2, (r, n)).astype(np.float32)
    ys, qs = np.zeros((r, n), np.float32), np.zeros(r * 11 * (n // 32), np.int32)
    ref.silu_mul_q8f(g, u, ys, qs, n, r)
    ysk, qsk = np.zeros((r, n), np.float32), np.zeros(r * 85 * (n // 256), np.int32)
    ref.silu_mul_q8k(g, u, ysk, qsk, n, r)
    out.update(s_g=g, s_u=u, s_y=ys, s_q=qs, s_yk=ysk, s_qk=qsk)
    save("batched", **out)


def decode():
    """The reference's decodeToken on its C++ backend, tiny model, teacher-forced tokens."""
    shape = tm.tiny()
    model = tm.build(shape, seed=1)
    om = OracleModel(shape, model)
    h = ref.lib.kcref_model_open(C.byref(om.c))
    tokens = [3, 250, 17, 0, 99, 128]
    logits = np.zeros((len(tokens), shape.vocab), np.float32)
    for pos, tok in enumerate(tokens):
        assert ref.lib.kcref_model_decode(h, om.embed(tok), pos, logits[pos]) == 0
    ref.lib.kcref_model_close(h)
    save("decode_tiny", tokens=np.array(tokens, np.int32), logits=logits,
         digest=np.frombuffer(bytes.fromhex(tm.digest(model)), np.uint8))


def synthetic():
    """The reference's buildModels(tinyConfig(w), 42) + allocActs(seed 7) + decodeToken on its C++ backend at position
    17 (its own test's choice, tests/test_llm_kernels.cpp:891-930) and at position 0, for the four synthetic formats."""
    out = {}
    for w, name in enumerate(("q8", "q4", "q4x8", "q4x8q8")):
        for pos in (17, 0):
            logits = np.zeros(1000, np.float32)
            assert ref.lib.kcref_synthetic_tiny_logits(w, 42, 7, pos, logits, None) == 1000
            out[f"{name}_pos{pos}"] = logits
    save("synthetic_tiny", **out)


if __name__ == "__main__":
    synthetic()
    kquant()
    halfs()
    glue()
    batched()
    decode()
