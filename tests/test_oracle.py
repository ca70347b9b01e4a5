"""The C restatement (oracle/kq_oracle.c) against the golden vectors the reference's own C++
produced, and -- where oracle/_ref was built -- against the reference library directly."""
import ctypes as C

import numpy as np
import pytest

import oracle
from helpers import OracleModel, bit_equal, pad8, rel_diff
from kernelcore_b200 import synth, tiny_model as tm

port = oracle.port
LIBS = [port] + ([oracle.ref] if oracle.ref is not None else [])


@pytest.mark.parametrize("fmt", ["q4k", "q6k"])
@pytest.mark.parametrize("shape", [(8, 256), (40, 768)])
def test_kquant_against_golden(golden, fmt, shape):
    g = golden("kquant")
    rows, k = shape
    q6 = fmt == "q6k"
    t = f"{fmt}_{rows}x{k}_"
    w, x = g[t + "w"], g[t + "x"]
    xq, xd = oracle.quantize_q8x4(port, x)
    assert bit_equal(xq, g[t + "xq"]) and bit_equal(xd, g[t + "xd"])
    assert bit_equal(oracle.quantize_q8k(port, x), g[t + "slot"])
    assert bit_equal(oracle.dequant(port, w, rows, k, q6), g[t + "deq"])
    assert bit_equal(oracle.matvec_q8(port, w, x, rows, k, q6), g[t + "y_q8"])
    assert bit_equal(oracle.matvec_q8k(port, w, x, rows, k, q6), g[t + "y_q8k"])
    # the reference's own bound between its Q8 product and the float product (test_llm_kernels.cpp:240)
    assert rel_diff(g[t + "y_q8"], oracle.matvec_dequant_f64(w, x, rows, k, q6)) < 3e-2


def test_half_conversions(golden):
    g = golden("halfs")
    got = np.array([port.f32_to_f16(float(v)) for v in g["f32"]], np.uint16)
    assert (got == g["f16"]).all()
    back = np.array([port.f16_to_f32(int(h)) for h in range(65536)], np.float32)
    assert (back.view(np.uint32) == g["f16_to_f32_all"]).all()
    # documented deviations from IEEE: saturation at 65520 and -0 -> +0
    assert port.f32_to_f16(65520.0) == 0x7BFF and port.f32_to_f16(-0.0) == 0


def test_glue_against_golden(golden):
    g = golden("glue")
    n, m = 3072, 8192
    x, t, w = g["norm_x"], g["norm_t"], g["norm_w"]
    y = np.zeros(n, np.float32)
    port.rms_norm(x, w, y, n, 1, 1e-5)
    assert bit_equal(y, g["rms_norm_y"])
    yr = np.zeros((5, 128), np.float32)
    port.rms_norm(g["rows_x"], g["rows_w"], yr, 128, 5, 1e-6)
    assert bit_equal(yr, g["rows_y"])
    x2, q = x.copy(), np.zeros(11 * n // 32, np.int32)
    port.add_sumsq(x2, t, q, n // 32)
    port.norm_q8x4(x2, w, q, n // 32, 1e-5)
    assert bit_equal(x2, g["addnorm_x"]) and bit_equal(q, g["addnorm_q"])
    x3, y3 = x.copy(), np.zeros(n, np.float32)
    port.add_rms_norm(x3, t, w, y3, n, 1e-5)
    assert bit_equal(y3, g["add_rms_norm_y"])
    h = np.zeros(m, np.float32)
    port.silu_mul(g["silu_g"], g["silu_u"], h, m)
    assert rel_diff(h, g["silu_h"]) < 1e-6
    lb = float(np.log2(500000.0))
    for pos in (0, 1, 517, 4095):
        a = g[f"rope_in_{pos}"].copy()
        port.rope(a, 64, pos, 192, lb)
        assert rel_diff(a, g[f"rope_out_{pos}"]) < 1e-6
        b = g[f"rope_in_{pos}"].copy()
        port.rope_ff(b, g[f"ropeff_ff_{pos}"], 64, pos, 192, lb)
        assert rel_diff(b, g[f"ropeff_out_{pos}"]) < 1e-6
    for neox in (0, 1):
        yg = np.zeros_like(g["ropeggml_x"])
        port.rope_ggml(g["ropeggml_x"], yg, g["ropeggml_pos"], np.ones(64, np.float32), 128, 3, 4, float(np.log2(1e6)), neox)
        assert rel_diff(yg, g[f"ropeggml_y_{neox}"]) < 1e-6
    d = oracle.AttnDims(6, 77, 64, 128, 3, pad8(77), 96)
    sc = np.zeros((6, pad8(77)), np.float32)
    port.attn_scores(g["attn_q"], g["attn_kt"], sc, C.byref(d), 0.125)
    assert bit_equal(sc, g["attn_scores"])
    p = sc.copy()
    port.softmax(p, 77, pad8(77), 6)
    assert rel_diff(p[:, :77], g["attn_p"][:, :77]) < 1e-6
    assert np.allclose(p[:, :77].sum(1), 1.0, atol=1e-5)
    o = np.zeros(384, np.float32)
    port.attn_values(np.ascontiguousarray(g["attn_p"]), g["attn_v"], o, C.byref(d))
    assert bit_equal(o, g["attn_out"])
    dst = np.zeros((12, 256), np.uint16)
    port.set_rows_f16(g["setrows_src"], g["setrows_idx"], dst, 128, 5, 256, 128, 12)
    assert (dst == g["setrows_dst"]).all()
    for tag in "abc":
        H, Hkv, D, T, N, mask = (int(v) for v in g[f"fa_{tag}_dims"])
        tp = pad8(T)
        fd = oracle.FaDims(H, T, D, H // Hkv, tp, Hkv * D // 2, D // 2, Hkv * D // 2, D // 2, N, H * D, D, tp // 2, mask, Hkv)
        fo = np.zeros((N, H, D), np.float32)
        port.flash_attn_f16(g[f"fa_{tag}_q"], g[f"fa_{tag}_k"], g[f"fa_{tag}_v"], g[f"fa_{tag}_mask"], fo, C.byref(fd), float(D) ** -0.5)
        assert rel_diff(fo, g[f"fa_{tag}_out"]) < 1e-6


def test_batched_against_golden(golden):
    g = golden("batched")
    X = g["X"]
    rows, k = 40, 768
    for q6, tag in ((0, "q4k"), (1, "q6k")):
        w = g[tag + "_w"]
        for c in range(X.shape[0]):
            assert bit_equal(oracle.matvec_q8(port, w, X[c], rows, k, q6), g[tag + "_Y_q8"][c])
            assert bit_equal(oracle.matvec_q8k(port, w, X[c], rows, k, q6), g[tag + "_Y_q8k"][c])
    for c in range(X.shape[0]):
        assert bit_equal(oracle.quantize_q8k(port, X[c]), g["slots_q8k"][c])
    n, r = 512, 3
    s, q = np.zeros((r, n), np.float32), np.zeros(r * 11 * (n // 32), np.int32)
    port.add_sumsq_f(g["f_a"], g["f_b"], s, q, n, r)
    y = np.zeros((r, n), np.float32)
    port.norm_mul_q8(s, g["f_w"], y, q, n, r, 1e-5)
    assert bit_equal(s, g["f_sum"]) and bit_equal(y, g["f_y"]) and bit_equal(q, g["f_q"])
    qk, sq, yk = np.zeros(r * 85 * (n // 256), np.int32), np.zeros(r * 11 * (n // 32), np.int32), np.zeros((r, n), np.float32)
    port.sumsq_part(s, sq, n, r)
    port.norm_mul_q8k(s, g["f_w"], yk, qk, sq, n, r, 1e-5)
    assert bit_equal(yk, g["f_yk"]) and bit_equal(qk, g["f_qk"])
    ys, qs = np.zeros((r, n), np.float32), np.zeros(r * 11 * (n // 32), np.int32)
    port.silu_mul_q8f(g["s_g"], g["s_u"], ys, qs, n, r)
    assert rel_diff(ys, g["s_y"]) < 1e-6


def test_decode_against_golden(golden):
    g = golden("decode_tiny")
    shape = tm.tiny()
    model = tm.build(shape, seed=1)
    assert bytes.fromhex(tm.digest(model)) == g["digest"].tobytes(), "synthetic model generator drifted"
    om = OracleModel(shape, model)
    for pos, tok in enumerate(g["tokens"]):
        logits = om.decode_port(om.embed(int(tok)), pos)
        assert rel_diff(logits, g["logits"][pos]) < 1e-5
        assert int(logits.argmax()) == int(g["logits"][pos].argmax())


@pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref not built (reference tree not mounted)")
def test_port_equals_reference_library_on_fresh_inputs():
    ref = oracle.ref
    for seed, (rows, k) in enumerate([(8, 256), (16, 1024), (24, 3072), (8, 8192)]):
        for q6 in (0, 1):
            for gen in (synth.kquant_blocks, synth.raw_blocks):
                w = gen(rows, k, 100 + seed, bool(q6))
                x = synth.activations(k, 200 + seed)
                assert bit_equal(oracle.dequant(port, w, rows, k, q6), oracle.dequant(ref, w, rows, k, q6))
                assert bit_equal(oracle.matvec_q8(port, w, x, rows, k, q6), oracle.matvec_q8(ref, w, x, rows, k, q6))
                assert bit_equal(oracle.matvec_q8k(port, w, x, rows, k, q6), oracle.matvec_q8k(ref, w, x, rows, k, q6))
    # quantizer edge cases: all-zero block, exact ties, saturating values
    x = np.zeros(64, np.float32)
    x[32:] = np.array([127, -127, 0.5, -0.5, 1.5, 2.5, -2.5, 63.5] * 4, np.float32)
    for lib in (port, ref):
        xq, xd = oracle.quantize_q8x4(lib, x)
        assert xd[0] == 0 and (xq[:8] == 0).all()
    assert bit_equal(oracle.quantize_q8x4(port, x)[0], oracle.quantize_q8x4(ref, x)[0])


def test_synthetic_formats_port_equals_reference():
    """The reference's 8-bit / 4-bit benchmark formats and fp16 matmul (llm/llm_reference.cpp:10-77, :114-152,
    :740-764): the restatement against the compiled reference, bit for bit, repacks included."""
    rng = np.random.default_rng(21)
    rows, k, nb = 24, 96, 3
    x = rng.standard_normal(k).astype(np.float32)
    scales = rng.uniform(0.01, 0.1, rows * nb).astype(np.float32)
    q8 = rng.integers(-127, 128, rows * k, dtype=np.int8)
    qs = rng.integers(0, 256, rows * k // 2, dtype=np.uint8)
    out = {}
    for name, L in (("port", oracle.port), ("ref", oracle.ref)):
        y8, y4, y48, y48q = (np.zeros(rows, np.float32) for _ in range(4))
        L.matvec_q8w(q8, scales, x, y8, rows, k)
        L.matvec_q4w(qs, scales, x, y4, rows, k)
        qs8, sc8 = np.zeros_like(qs), np.zeros_like(scales)
        L.repack_q4x8(qs, scales, qs8, sc8, rows, k)
        L.matvec_q4x8(qs8, sc8, x, y48, rows, k)
        qw = np.zeros(rows * nb * 5, np.int32)
        L.repack_q4x8_q8(qs, scales, qw, rows, k)
        xq, xd = oracle.quantize_q8x4(L, x)
        L.matvec_q4x8_q8(qw, xq, xd, y48q, rows, k)
        rng = np.random.default_rng(22)      # the same fp16 matrix and X for both libraries
        w16 = rng.integers(0, 0x7C00, rows * k).astype(np.uint16) | (rng.integers(0, 2, rows * k).astype(np.uint16) << 15)
        X = rng.standard_normal((5, k)).astype(np.float32)
        yf = np.zeros((5, rows), np.float32)
        L.matmul_f16(w16, X, yf, rows, k, 5)
        st = np.zeros(rows * k // 2, np.int32)
        L.repack_f16(w16, rows, k, st)
        out[name] = (y8, y4, qs8, sc8, y48, qw, y48q, yf, st)
    for a, b in zip(out["port"], out["ref"]):
        assert bit_equal(a, b)
    # the interleaved forms compute what the row-major form does (different summation order for q4x8)
    assert np.abs(out["port"][4] - out["port"][1]).max() < 1e-4 * np.abs(out["port"][1]).max()
    assert np.abs(out["port"][6] - out["port"][1]).max() < 3e-2 * np.abs(out["port"][1]).max()


def test_batched_pipeline_restatement_agrees_with_the_decode_loop():
    """helpers.oracle_prefill strings the oracle's batched operators together (rope_ggml, set_rows_f16,
    flash_attn_f16 with a causal mask, per-row add + norm).  With per-32 activations it must reproduce the oracle's
    own token-by-token decode loop on an fp16 cache: same arithmetic, different plumbing."""
    from helpers import OracleModel, oracle_prefill
    from kernelcore_b200 import tiny_model as tm
    for shape in (tm.tiny(max_ctx=16), tm.tiny_qwen(max_ctx=16)):
        model = tm.build(shape, seed=8)
        prompt = [int(t) for t in np.random.default_rng(5).integers(0, shape.vocab, 5)]
        om = OracleModel(shape, model)
        for pos, tok in enumerate(prompt):
            want = om.decode_port(om.embed(tok), pos, kv_f16=True)
        assert rel_diff(oracle_prefill(shape, model, prompt, q8k=False), want) < 1e-5
        # per-256 activations: a different quantization of the same model, within the reference's Q8-vs-float bound
        assert rel_diff(oracle_prefill(shape, model, prompt), want) < 5e-2


def test_decode_trace_and_stage_by_stage_mode():
    """The instrumentation the decoder's stage-by-stage test rests on.  A step's trace holds every vector the loop
    quantized and the residual after each addition; replaying the step with its own trace forced changes nothing
    and counts no difference; one int8 step planted in the wo input is counted as exactly that, shows in the next
    residual, and does not reach the logits, because every later vector is replaced as well -- while the same step
    planted without the later replacements (a free-running loop) would."""
    from helpers import OracleModel
    from kernelcore_b200 import tiny_model as tm
    shape = tm.tiny(max_ctx=8)
    model = tm.build(shape, seed=2)
    a, b = OracleModel(shape, model), OracleModel(shape, model)
    layout = a.trace_layout()
    assert sum(n for _, _, n in layout) == a.trace_words() and [k for k, _, _ in layout[:4]] == ["q8", "q8", "x", "q8"]
    trace = np.zeros(a.trace_words(), np.int32)
    for pos, tok in enumerate((3, 200, 17)):
        want = a.decode_port(a.embed(tok), pos, kv_f16=True, trace=trace)
        assert np.any(trace[layout[0][1]:layout[0][1] + layout[0][2]] != 0)
        got = b.decode_port(b.embed(tok), pos, kv_f16=True, forced=trace)
        assert (got == want).all() and b.forced_stats == (0, 0, 0, 0.0)
    planted = trace.copy()
    byte = planted.view(np.int8)
    at = 4 * layout[1][1] + 37                      # a value of the wo input of layer 0
    byte[at] += 1 if byte[at] < 127 else -1
    got = b.decode_port(b.embed(17), 2, kv_f16=True, forced=planted)
    values, vectors, step, residual = b.forced_stats
    assert (values, vectors, step) == (1, 1, 1) and 1e-5 < residual < 1e-2
    assert (got == want).all()
