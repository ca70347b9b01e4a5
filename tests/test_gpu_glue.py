"""GPU parity of the normalisation / RoPE / attention / SwiGLU kernels against the golden vectors the
reference produced and against the oracle, through the C ABI."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import bit_equal, pad8, rel_diff
from kernelcore_b200 import lib

pytestmark = pytest.mark.gpu
port = oracle.port


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ints(*v):
    return (C.c_int * len(v))(*v)


def test_rms_norm_and_fused_add_norm_quant(golden):
    g = golden("glue")
    n = 3072
    x, t, w = dev(g["norm_x"]), dev(g["norm_t"]), dev(g["norm_w"])
    y = torch.empty(n, device="cuda")
    lib.call("rms_norm", x, w, y, n, 1, 1e-5)
    assert rel_diff(y.cpu().numpy(), g["rms_norm_y"]) < 1e-6      # tree sum vs sequential sum
    rows = dev(g["rows_x"])
    yr = torch.empty_like(rows)
    lib.call("rms_norm", rows, dev(g["rows_w"]), yr, 128, 5, 1e-6)  # the per-head QK-norm shape
    assert rel_diff(yr.cpu().numpy(), g["rows_y"]) < 1e-6
    x3, y3 = x.clone(), torch.empty(n, device="cuda")
    lib.call("add_rms_norm", x3, t, w, y3, n, 1e-5)
    assert rel_diff(y3.cpu().numpy(), g["add_rms_norm_y"]) < 1e-6
    assert bit_equal(x3.cpu().numpy(), g["addnorm_x"])
    # two-launch and one-launch forms of add + norm + quantize: bit-identical to the reference
    for fused in (False, True):
        x2, q = x.clone(), torch.zeros(11 * n // 32, dtype=torch.int32, device="cuda")
        if fused:
            lib.call("add_norm_q8x4", x2, t, w, q, n // 32, 1e-5)
        else:
            lib.call("add_sumsq", x2, t, q, n // 32)
            lib.call("norm_q8x4", x2, w, q, n // 32, 1e-5)
        assert bit_equal(x2.cpu().numpy(), g["addnorm_x"])
        assert bit_equal(q.cpu().numpy(), g["addnorm_q"])


def test_swiglu(golden):
    g = golden("glue")
    m = 8192
    gg, u = dev(g["silu_g"]), dev(g["silu_u"])
    h = torch.empty(m, device="cuda")
    lib.call("silu_mul", gg, u, h, m)
    assert rel_diff(h.cpu().numpy(), g["silu_h"]) < 1e-6
    xq, xd = torch.zeros(m // 4, dtype=torch.int32, device="cuda"), torch.zeros(m // 16, device="cuda")
    lib.call("silu_mul_q8x4", gg, u, xq, xd, m // 32)
    # exp2 differs by an ulp between libm and the GPU: compare the dequantised activations
    got = xq.cpu().numpy().view(np.int8).reshape(-1, 32) * xd.cpu().numpy()[0::2, None]
    want = g["silu_xq"].view(np.int8).reshape(-1, 32) * g["silu_xd"][0::2, None]
    assert np.abs(got - want).max() <= np.abs(want).max() / 127 * 1.01
    assert (xq.cpu().numpy() == g["silu_xq"]).mean() > 0.99


def test_rope(golden):
    g = golden("glue")
    lb = float(np.log2(500000.0))
    for pos in (0, 1, 517, 4095):
        a = dev(g[f"rope_in_{pos}"])
        lib.call("rope", a, None, 64, pos, 192, lb)
        assert rel_diff(a.cpu().numpy(), g[f"rope_out_{pos}"]) < 1e-3   # the reference's own bound
        b = dev(g[f"rope_in_{pos}"])
        lib.call("rope", b, dev(g[f"ropeff_ff_{pos}"]), 64, pos, 192, lb)
        assert rel_diff(b.cpu().numpy(), g[f"ropeff_out_{pos}"]) < 1e-3
    x, posv = dev(g["ropeggml_x"]), dev(g["ropeggml_pos"])
    for neox in (0, 1):
        y = torch.empty_like(x)
        lib.call("rope_ggml", x, y, posv, None, 128, 3, 4, float(np.log2(1e6)), neox)
        assert rel_diff(y.cpu().numpy(), g[f"ropeggml_y_{neox}"]) < 1e-3


def test_fp32_attention(golden):
    g = golden("glue")
    d = ints(6, 77, 64, 128, 3, pad8(77), 96)
    q, kt, v = dev(g["attn_q"]), dev(g["attn_kt"]), dev(g["attn_v"])
    sc = torch.zeros((6, pad8(77)), device="cuda")
    lib.call("attn_scores", q, kt, sc, d, 0.125)
    assert bit_equal(sc.cpu().numpy()[:, :77], g["attn_scores"][:, :77])
    p = sc.clone()
    lib.call("softmax", p, 77, pad8(77), 6)
    assert rel_diff(p.cpu().numpy()[:, :77], g["attn_p"][:, :77]) < 1e-6
    assert np.allclose(p.cpu().numpy()[:, :77].sum(1), 1.0, atol=1e-5)
    o = torch.empty(384, device="cuda")
    lib.call("attn_values", dev(g["attn_p"]), v, o, d)
    assert bit_equal(o.cpu().numpy(), g["attn_out"])
    # kv_append writes column ctx-1 of the transposed K cache and row ctx-1 of V
    k1, v1 = torch.randn(128, device="cuda"), torch.randn(128, device="cuda")
    kt2, v2 = kt.clone(), v.clone()
    lib.call("kv_append", k1, v1, kt2, v2, d)
    assert torch.equal(kt2[:, 76], k1) and torch.equal(v2[76], v1)
    kt2[:, 76] = kt[:, 76]
    assert torch.equal(kt2, kt)
    bad = ints(6, 77, 64, 128, 4, pad8(77), 96)  # 6 heads not divisible by group 4
    assert lib.call("attn_scores", q, kt, sc, bad, 0.125, raise_on_error=False) == 2


def test_fp16_cache_path(golden):
    g = golden("glue")
    dst = torch.zeros((12, 256), dtype=torch.int16, device="cuda")
    lib.call("set_rows_f16", dev(g["setrows_src"]), dev(g["setrows_idx"]), dst, 128, 5, 256, 128, 12)
    assert (dst.cpu().numpy().view(np.uint16) == g["setrows_dst"]).all()
    h = golden("halfs")
    n = h["f32"].size // 2 * 2
    out = torch.zeros((1, n), dtype=torch.int16, device="cuda")
    lib.call("set_rows_f16", dev(h["f32"][:n]), dev(np.zeros(1, np.int64)), out, n // 2, 1, n, n // 2, 1)
    assert (out.cpu().numpy().view(np.uint16).ravel() == h["f16"][:n]).all()     # incl. 65520, -0, subnormals, ties
    for tag in "abc":
        H, Hkv, D, T, N, mask = (int(v) for v in g[f"fa_{tag}_dims"])
        tp = pad8(T)
        fd = ints(H, T, D, H // Hkv, tp, Hkv * D // 2, D // 2, Hkv * D // 2, D // 2, N, H * D, D, tp // 2, mask, Hkv)
        o = torch.zeros((N, H, D), device="cuda")
        lib.call("flash_attn_f16", dev(g[f"fa_{tag}_q"]), dev(g[f"fa_{tag}_k"].view(np.int16)),
                 dev(g[f"fa_{tag}_v"].view(np.int16)), dev(g[f"fa_{tag}_mask"].view(np.int16)), o, fd, float(D) ** -0.5)
        assert rel_diff(o.cpu().numpy(), g[f"fa_{tag}_out"]) < 2e-6              # tests/test_llm_kernels.cpp:741-794


def test_batched_forms(golden):
    g = golden("batched")
    n, r = 512, 3
    a, b, w = dev(g["f_a"]), dev(g["f_b"]), dev(g["f_w"])
    s = torch.empty((r, n), device="cuda")
    q = torch.zeros(r * 11 * (n // 32), dtype=torch.int32, device="cuda")
    lib.call("add_sumsq_f", a, b, s, q, n, r)
    y = torch.empty((r, n), device="cuda")
    lib.call("norm_mul_q8_f", s, w, y, q, n, r, 1e-5)
    assert bit_equal(s.cpu().numpy(), g["f_sum"]) and bit_equal(y.cpu().numpy(), g["f_y"])
    assert bit_equal(q.cpu().numpy(), g["f_q"])
    sq = torch.zeros(r * 11 * (n // 32), dtype=torch.int32, device="cuda")
    qk = torch.zeros(r * 85 * (n // 256), dtype=torch.int32, device="cuda")
    yk = torch.empty((r, n), device="cuda")
    lib.call("sumsq_part", s, sq, n, r)
    lib.call("norm_mul_q8k_f", s, w, yk, qk, sq, n, r, 1e-5)
    assert bit_equal(yk.cpu().numpy(), g["f_yk"]) and bit_equal(qk.cpu().numpy(), g["f_qk"])
    gg, u = dev(g["s_g"]), dev(g["s_u"])
    ys, qs = torch.empty((r, n), device="cuda"), torch.zeros(r * 11 * (n // 32), dtype=torch.int32, device="cuda")
    lib.call("silu_mul_q8x4f", gg, u, ys, qs, n, r)
    assert rel_diff(ys.cpu().numpy(), g["s_y"]) < 1e-6
    ysk, qsk = torch.empty((r, n), device="cuda"), torch.zeros(r * 85 * (n // 256), dtype=torch.int32, device="cuda")
    lib.call("silu_mul_q8kf", gg, u, ysk, qsk, n, r)
    assert rel_diff(ysk.cpu().numpy(), g["s_yk"]) < 1e-6
    # column-batched quantizers: slots bit-identical to the reference's quantizeQ8K / quantizeQ8x4
    X = g["X"]
    ncols, k = X.shape
    slots = torch.zeros((ncols, 85 * k // 256), dtype=torch.int32, device="cuda")
    lib.call("quantize_cols_k", dev(X), slots, k, ncols)
    assert bit_equal(slots.cpu().numpy(), g["slots_q8k"])
    s32 = torch.zeros((ncols, 11 * k // 32), dtype=torch.int32, device="cuda")
    lib.call("quantize_cols", dev(X), s32, k, ncols)
    for c in range(ncols):
        xq, xd = oracle.quantize_q8x4(port, X[c])
        got = s32[c].cpu().numpy()
        assert bit_equal(got[: k // 4], xq) and bit_equal(got[k // 4: k // 4 + k // 16].view(np.float32), xd)
