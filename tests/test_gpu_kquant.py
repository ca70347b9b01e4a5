"""GPU parity of the K-quant path against the oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from helpers import bit_equal, rel_diff
from kernelcore_b200 import kquant, lib, synth

pytestmark = pytest.mark.gpu
port = oracle.port

SHAPES = [(8, 256), (40, 768), (1, 256), (7, 512), (33, 1024), (96, 3072), (24, 8192), (17, 12288)]


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("q6", [False, True])
def test_dequant_bit_exact_and_layout_round_trip(q6, golden):
    g = golden("kquant")
    for rows, k in ((8, 256), (40, 768)):
        t = f"{'q6k' if q6 else 'q4k'}_{rows}x{k}_"
        m = kquant.KMatrix(g[t + "w"], rows, k, q6)
        assert bit_equal(m.dequant().cpu().numpy(), g[t + "deq"])
        assert (m.gguf_bytes().cpu().numpy().reshape(rows, -1) == g[t + "w"]).all()
    for rows, k in SHAPES:
        for gen in (synth.kquant_blocks, synth.raw_blocks):
            w = gen(rows, k, rows + k, q6)
            m = kquant.KMatrix(w, rows, k, q6)
            assert bit_equal(m.dequant().cpu().numpy(), oracle.dequant(port, w, rows, k, q6))
            assert (m.gguf_bytes().cpu().numpy().reshape(rows, -1) == w).all()


def test_quantize_q8x4_bit_exact(golden):
    g = golden("kquant")
    sc = kquant.Q8Scratch(12288)
    for t in ("q4k_8x256_", "q4k_40x768_"):
        xq, xd = kquant.quantize_q8x4(_dev(g[t + "x"]), sc)
        assert bit_equal(xq.cpu().numpy(), g[t + "xq"]) and bit_equal(xd.cpu().numpy(), g[t + "xd"])
    rng = np.random.default_rng(0)
    for k in (32, 256, 3072, 12288):
        x = (rng.standard_normal(k) * 10 ** rng.uniform(-3, 3, k)).astype(np.float32)
        x[: 32] = 0  # an all-zero block: d = 0, id = 0
        if k >= 64:
            x[32:64] = np.array([127, -127, 0.5, -0.5, 1.5, 2.5, -2.5, 63.5] * 4, np.float32)  # exact ties
        xq, xd = kquant.quantize_q8x4(_dev(x), sc)
        wq, wd = oracle.quantize_q8x4(port, x)
        assert bit_equal(xq.cpu().numpy(), wq) and bit_equal(xd.cpu().numpy(), wd)


@pytest.mark.parametrize("q6", [False, True])
def test_matvec_q8_against_golden_and_oracle(q6, golden):
    g = golden("kquant")
    sc = kquant.Q8Scratch(12288)
    for rows, k in ((8, 256), (40, 768)):
        t = f"{'q6k' if q6 else 'q4k'}_{rows}x{k}_"
        m = kquant.KMatrix(g[t + "w"], rows, k, q6)
        y = kquant.matvec(m, _dev(g[t + "x"]), sc).cpu().numpy()
        # the reference's bar between two compilers of the same kernel (app/kquant_vs_cuda.cpp:260-276)
        assert rel_diff(y, g[t + "y_q8"]) < 1e-5
    for rows, k in SHAPES:
        for gen in (synth.kquant_blocks, synth.raw_blocks):
            w = gen(rows, k, 3 * rows + k, q6)
            x = synth.activations(k, rows)
            m = kquant.KMatrix(w, rows, k, q6)
            y = kquant.matvec(m, _dev(x), sc).cpu().numpy()
            assert rel_diff(y, oracle.matvec_q8(port, w, x, rows, k, q6)) < 1e-5, (rows, k, gen.__name__)


@pytest.mark.parametrize("q6", [False, True])
def test_matvec_f32_against_dequant_dot(q6):
    """fp32 activations: within 1e-3 of max|y| of the double-precision dot of the dequantised row
    (in practice ~1e-6: only fp32 accumulation order differs)."""
    for rows, k in SHAPES:
        w = synth.kquant_blocks(rows, k, 5 * rows + k, q6)
        x = synth.activations(k, rows + 1)
        m = kquant.KMatrix(w, rows, k, q6)
        y = kquant.matvec_f32(m, _dev(x)).cpu().numpy()
        assert rel_diff(y, oracle.matvec_dequant_f64(w, x, rows, k, q6)) < 1e-3
        assert rel_diff(y, oracle.matvec_dequant_f64(w, x, rows, k, q6)) < 2e-5


def test_config0_and_lm_head_slice_full_k():
    """Benchmark shapes: the whole 8192x3072 Q4_K matvec and a 16032-row slice (the 8-GPU shard) of
    the 128256x3072 Q6_K lm_head, against the oracle."""
    sc = kquant.Q8Scratch(3072)
    for rows, k, q6 in ((8192, 3072, False), (16032, 3072, True)):
        w = synth.kquant_blocks(rows, k, 0, q6)
        x = synth.activations(k, 1)
        m = kquant.KMatrix(w, rows, k, q6)
        y = kquant.matvec(m, _dev(x), sc).cpu().numpy()
        assert rel_diff(y, oracle.matvec_q8(port, w, x, rows, k, q6)) < 1e-5
        yf = kquant.matvec_f32(m, _dev(x)).cpu().numpy()
        assert rel_diff(yf, oracle.matvec_dequant_f64(w, x, rows, k, q6)) < 1e-3


def test_full_size_linearity_property():
    """Size-independent check at the full lm_head size: the Q8 matvec is linear in the activation
    scale for a fixed set of quantized words, y(2x) == 2 y(x) exactly (powers of two commute with
    every rounding step), and rows of zero-scale blocks give exactly zero."""
    rows, k = 128256, 3072
    w = synth.q6k_blocks(rows, k, 7)
    w.reshape(-1, 210)[: 12 * 5, 208:210] = 0  # first five rows: d = 0
    m = kquant.KMatrix(w, rows, k, True)
    sc = kquant.Q8Scratch(k)
    x = _dev(synth.activations(k, 2))
    y1 = kquant.matvec(m, x, sc).clone()
    y2 = kquant.matvec(m, x * 2, sc).clone()
    assert torch.equal(y1 * 2, y2)
    assert (y1[:5] == 0).all() and torch.isfinite(y1).all()


def test_argument_validation():
    """Bad shapes are refused before any launch (llm/llm_kernels.cpp:264-279 returns InvalidValue)."""
    sc = kquant.Q8Scratch(512)
    xq, xd = sc.views(512)
    y = torch.zeros(8, device="cuda")
    w = torch.zeros(8 * 2 * 144, dtype=torch.uint8, device="cuda")
    assert lib.call("matvec_q4k_q8", w, xq, xd, y, 8, 500, raise_on_error=False) == 2
    assert lib.call("matvec_q4k_q8", w, xq, xd, y, -1, 512, raise_on_error=False) == 2
    assert lib.call("matvec_q4k_q8", None, xq, xd, y, 8, 512, raise_on_error=False) == 2
    assert lib.call("matvec_q4k_q8", w, xq, xd, y, 0, 512, raise_on_error=False) == 0  # empty is fine
    with pytest.raises(lib.KcbError):
        lib.call("matvec_q6k_q8", w, xq, xd, y, 8, 100)
