"""K-quant matmuls (prompt path) against the oracle's per-column mirror, through the C ABI."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import bit_equal, rel_diff
from kernelcore_b200 import kquant, lib, synth

pytestmark = pytest.mark.gpu
port = oracle.port


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def slots_for(X, q8k):
    ncols, k = X.shape
    n = 85 * k // 256 if q8k else 11 * k // 32
    s = torch.zeros((ncols, n), dtype=torch.int32, device="cuda")
    lib.call("quantize_cols_k" if q8k else "quantize_cols", dev(X), s, k, ncols)
    return s


def run(w, X, rows, k, q6, q8k, workspace=False):
    """One pass (kcb_matmul_kq_q8) or, with workspace=True, the route that may contract K in slices
    (kcb_matmul_kq_q8_ws with a caller buffer of kcb_matmul_tc_workspace_bytes)."""
    m = kquant.KMatrix(w, rows, k, q6)
    ncols = X.shape[0]
    y = torch.full((ncols, rows), float("nan"), device="cuda")
    if not workspace:
        lib.call("matmul_kq_q8", m.data, slots_for(X, q8k), y, rows, k, ncols, int(q6), int(q8k))
    else:
        lib.raw.kcb_matmul_tc_workspace_bytes.restype = C.c_size_t
        nbytes = lib.raw.kcb_matmul_tc_workspace_bytes(rows, k, ncols)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
        lib.call("matmul_kq_q8_ws", m.data, slots_for(X, q8k), y, rows, k, ncols, int(q6), int(q8k), ws, C.c_size_t(nbytes))
    return y.cpu().numpy()


@pytest.mark.parametrize("q6", [False, True])
@pytest.mark.parametrize("q8k", [False, True])
def test_golden_columns(golden, q6, q8k):
    """The reference's own matmul test shapes (tests/test_llm_kernels.cpp:277-420): 40 x 768, 13 columns."""
    g = golden("batched")
    tag = "q6k" if q6 else "q4k"
    y = run(g[tag + "_w"], g["X"], 40, 768, q6, q8k)
    assert rel_diff(y, g[tag + ("_Y_q8k" if q8k else "_Y_q8")]) < 1e-5


@pytest.mark.parametrize("q6", [False, True])
@pytest.mark.parametrize("ncols", [16, 17, 33, 64, 65, 128, 130, 300])
def test_tensor_core_q8k_against_the_mirror(ncols, q6):
    """Q4_K / Q6_K x per-256 activations on tcgen05: exact integer contractions and the reference's fp32 order, so
    every output equals llm::ref::matvecQ4KQ8K / matvecQ6KQ8K bit for bit, including ragged column tiles (a last
    tile of 1..64 columns uses one accumulator half only).  raw_blocks draws every byte uniformly, so Q6_K scales reach
    -128 and 127 (the extremes of the plane split) and Q4_K scales and mins 0 and 63."""
    rows, k = 256, 1024
    for gen in (synth.kquant_blocks, synth.raw_blocks):
        w = gen(rows, k, ncols, q6)
        X = np.random.default_rng(ncols).uniform(-3, 3, (ncols, k)).astype(np.float32)
        X[0, :256] = 0  # an all-zero super-block: scale 0
        y = run(w, X, rows, k, q6, True)
        want = np.stack([oracle.matvec_q8k(port, w, X[c], rows, k, int(q6)) for c in range(ncols)])
        assert bit_equal(y, want), (ncols, gen.__name__)
    assert lib.raw.kcb_tc_timeouts() == 0


@pytest.mark.parametrize("q6", [False, True])
@pytest.mark.parametrize("ncols", [17, 130])
def test_one_pass_tiles_are_bit_identical(q6, ncols):
    """150 row tiles: every persistent CTA walks more than one tile (the pipeline runs across tile boundaries); every
    output equals the reference mirror bit for bit, ragged column tiles included, with and without a workspace (this
    shape takes one pass either way)."""
    rows, k = 128 * 150, 1024
    assert lib.raw.kcb_matmul_tc_k_slices(rows, k, ncols) == 1
    w = synth.raw_blocks(rows, k, 5, q6)
    X = np.random.default_rng(5).uniform(-3, 3, (ncols, k)).astype(np.float32)
    want = np.stack([oracle.matvec_q8k(port, w, X[c], rows, k, int(q6)) for c in range(ncols)])
    assert bit_equal(run(w, X, rows, k, q6, True), want)
    assert bit_equal(run(w, X, rows, k, q6, True, workspace=True), want)


def test_ffn_down_shape_splits_k_three_ways():
    """Llama-3.2-3B's FFN-down at a 512-token prompt chunk: Q6_K 3072 x 8192, 96 tiles of 32 super-blocks on 148 SMs.
    Given a workspace the launch contracts it as three K slices (288 units of 11 super-blocks instead of 96 of 32 on
    two thirds of the machine): columns against the oracle to 2e-6, exact doubling under doubled activations.  Without
    a workspace the same call is one pass and bit-identical to the mirror."""
    rows, k, M = 3072, 8192, 512
    assert lib.raw.kcb_matmul_tc_k_slices(rows, k, M) == 3
    w = synth.raw_blocks(rows, k, 11, True)
    X = np.random.default_rng(2).standard_normal((M, k)).astype(np.float32)
    y = run(w, X, rows, k, True, True, workspace=True)
    y1 = run(w, X, rows, k, True, True)
    for c in (0, 255, M - 1):
        want = oracle.matvec_q8k(port, w, X[c], rows, k, 1)
        assert rel_diff(y[c], want) < 2e-6
        assert bit_equal(y1[c], want)
    assert bit_equal(run(w, X * 2, rows, k, True, True, workspace=True), y * 2)
    assert lib.raw.kcb_tc_timeouts() == 0


def test_config2_shape_against_cuda_core_path():
    """The Q4_K benchmark matmul at M = 32, 128, 512 and 2048: 8192 x 3072 Q4_K; spot-check columns against the oracle
    (one pass: bit for bit; M = 128 with a workspace: two K slices, 2e-6) and the linearity property on the rest
    (activations scaled by 2 give exactly doubled outputs)."""
    rows, k = 8192, 3072
    w = synth.q4k_blocks(rows, k, 0)
    for M in (32, 128, 512, 2048):
        X = np.random.default_rng(1).standard_normal((M, k)).astype(np.float32)
        y = run(w, X, rows, k, False, True)
        for c in (0, 17, M - 1):
            assert bit_equal(y[c], oracle.matvec_q8k(port, w, X[c], rows, k, 0))
        assert bit_equal(run(w, X * 2, rows, k, False, True), y * 2)
        if M == 128:
            assert lib.raw.kcb_matmul_tc_k_slices(rows, k, M) == 2
            ys = run(w, X, rows, k, False, True, workspace=True)
            assert 0 < rel_diff(ys, y) < 2e-6 or bit_equal(ys, y)
    assert lib.raw.kcb_tc_timeouts() == 0


@pytest.mark.parametrize("q6", [False, True])
def test_tensor_cores_agree_with_the_cuda_core_matmul(q6):
    """The tensor-core kernels against the CUDA-core dp4a matmul of the same library, which shares no code with them:
    per-256 slots, 40 columns; 264 rows (not a multiple of 128) take the dp4a route, their first 256 the tensor cores.
    Same integers, fp32 sums in a different order: 1e-5."""
    rows, k, ncols = 264, 1024, 40
    w = synth.raw_blocks(rows, k, 21, q6)
    X = np.random.default_rng(21).uniform(-2, 2, (ncols, k)).astype(np.float32)
    y_cc = run(w, X, rows, k, q6, True)
    y_tc = run(np.ascontiguousarray(w[:256]), X, 256, k, q6, True)
    assert rel_diff(y_tc, y_cc[:, :256]) < 1e-5
