"""Edge cases of the hot path: smallest and largest supported shapes, empty batches, all-zero and extreme
activations, rounding boundaries of the 8-bit quantizer, single-position attention."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import bit_equal, pad8, rel_diff
from kernelcore_b200 import kquant, lib, synth

pytestmark = pytest.mark.gpu
port = oracle.port


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("q6", [False, True])
@pytest.mark.parametrize("rows,k", [(8, 256), (8, 32768), (24, 16384), (4736, 256)])
def test_matvec_smallest_and_largest_k(q6, rows, k):
    """k = 256 is one super-block per row, k = 32768 the largest the kernels accept; 4736 rows x 256 puts the
    bulk-copy path on its smallest tiles."""
    w = synth.raw_blocks(rows, k, rows + k, q6)
    x = synth.activations(k, 3)
    y = kquant.matvec(kquant.KMatrix(w, rows, k, q6), dev(x), kquant.Q8Scratch(k)).cpu().numpy()
    assert rel_diff(y, oracle.matvec_q8(port, w, x, rows, k, q6)) < 1e-5
    assert lib.call("matvec_q6k_q8" if q6 else "matvec_q4k_q8", None, None, None, None, 8, 32768 + 256, raise_on_error=False) == 2


def test_quantizer_rounding_boundaries_and_extremes():
    """Values that land exactly on .5 after scaling (round half away from zero, then clamp to +-127), a block of
    zeros (scale 0, inverse 0), negative zero, a tiny block, one huge value: words, scales and sums bit-equal.
    (A block whose largest magnitude is subnormal is left out: there 1 / scale overflows and the reference converts
    inf / NaN to int, which C++ leaves undefined -- x86 and the GPU give different answers, and no activation of a
    model gets there.)"""
    blocks = []
    b = np.zeros(32, np.float32)
    b[0] = 127.0
    b[1:12] = np.arange(11) + 0.5            # exact halves at scale 1
    b[12:23] = -(np.arange(11) + 0.5)
    blocks.append(b)
    blocks.append(np.zeros(32, np.float32))
    z = np.zeros(32, np.float32)
    z[3] = -0.0
    z[7] = 2e-36                              # tiny but normal after the division by 127
    blocks.append(z)
    h = np.full(32, 1.0, np.float32)
    h[5] = 3e38
    blocks.append(h)
    blocks.append(np.full(32, -2.5, np.float32))
    x = np.concatenate(blocks)
    nb = x.size // 32
    xq, xd = torch.zeros(nb * 8, dtype=torch.int32, device="cuda"), torch.zeros(nb * 2, device="cuda")
    lib.call("quantize_q8x4", dev(x), xq, xd, nb)
    wq, wd = oracle.quantize_q8x4(port, x)
    assert bit_equal(xq.cpu().numpy(), wq) and bit_equal(xd.cpu().numpy(), wd)
    # per-256 form on the same values padded to one super-block pair
    xk = np.zeros(512, np.float32)
    xk[:x.size] = x
    slots = torch.zeros((1, 85 * 2), dtype=torch.int32, device="cuda")
    lib.call("quantize_cols_k", dev(xk), slots, 512, 1)
    assert bit_equal(slots.cpu().numpy().ravel(), oracle.quantize_q8k(port, xk))


@pytest.mark.parametrize("q6", [False, True])
def test_zero_activations_and_empty_batches(q6):
    rows, k = 256, 1024
    w = synth.raw_blocks(rows, k, 1, q6)
    m = kquant.KMatrix(w, rows, k, q6)
    y = kquant.matvec(m, torch.zeros(k, device="cuda"), kquant.Q8Scratch(k))
    assert (y == 0).all()                     # scale 0: every product and min term is exactly 0
    slots = torch.zeros((4, 85 * k // 256), dtype=torch.int32, device="cuda")
    out = torch.full((4, rows), 7.0, device="cuda")
    assert lib.call("matmul_kq_q8", m.data, slots, out, rows, k, 0, int(q6), 1, raise_on_error=False) == 2   # ncols <= 0 refused
    assert lib.call("quantize_cols_k", torch.zeros(k, device="cuda"), slots, k, 0, raise_on_error=False) == 0  # empty batch
    assert lib.call("quantize_q8x4", torch.zeros(32, device="cuda"), slots, slots.view(torch.float32), 0, raise_on_error=False) == 0
    assert (out == 7.0).all()
    # one column through the batched entry point (CUDA-core route) equals the per-column mirror
    X = np.random.default_rng(2).standard_normal((1, k)).astype(np.float32)
    lib.call("quantize_cols_k", dev(X), slots, k, 1)
    lib.call("matmul_kq_q8", m.data, slots, out, rows, k, 1, int(q6), 1)
    assert rel_diff(out[0].cpu().numpy(), oracle.matvec_q8k(port, w, X[0], rows, k, int(q6))) < 1e-5


def test_attention_over_a_single_position():
    """T = 1: the softmax weight is exactly 1 and the output is the (fp16-rounded) value row."""
    H, Hkv, D = 4, 2, 64
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, H, D)).astype(np.float32)
    k16 = rng.standard_normal((1, Hkv * D)).astype(np.float16)
    v16 = rng.standard_normal((1, Hkv * D)).astype(np.float16)
    dims = np.array([H, 1, D, H // Hkv, pad8(1), Hkv * D // 2, D // 2, Hkv * D // 2, D // 2, 1, H * D, D, 0, 0, Hkv], np.int32)
    out = torch.zeros(1, H, D, device="cuda")
    lib.call("flash_attn_f16", dev(q), dev(k16.view(np.uint16)), dev(v16.view(np.uint16)), None, out,
             dims.ctypes.data_as(C.c_void_p), C.c_float(0.125))
    want = np.repeat(v16.astype(np.float32).reshape(Hkv, D), H // Hkv, axis=0)
    assert bit_equal(out.cpu().numpy().reshape(H, D), want)


@pytest.mark.parametrize("rows4,rows6,k", [(4096, 1024, 3072), (8, 8, 256), (5120, 1024, 4096), (6144, 3000, 4096), (520, 4000, 1024)])
def test_q4k_and_q6k_matvec_in_one_launch_equal_their_own_launches(rows4, rows6, k):
    """The q|k (Q4_K) and v (Q6_K) projections of a Q4_K_M layer share their input; the pair launch gives what each
    matrix's own launch gives, whether the grid holds every CTA at once or is shared out by bytes: the Q6_K output bit for
    bit, the Q4_K output to 1e-6 of its largest value -- the integer dot products are the same, but the stand-alone Q4_K
    kernels sum a sub-block's 32 products in the integer domain where the pair kernel's lanes hold 16 each and add the
    two halves as floats."""
    w4 = kquant.KMatrix(synth.raw_blocks(rows4, k, 21, False), rows4, k, False)
    w6 = kquant.KMatrix(synth.raw_blocks(rows6, k, 22, True), rows6, k, True)
    nb = k // 32
    xq, xd = torch.zeros(nb * 8, dtype=torch.int32, device="cuda"), torch.zeros(nb * 2, device="cuda")
    lib.call("quantize_q8x4", dev(synth.activations(k, 9)), xq, xd, nb)
    a4, a6 = torch.zeros(rows4, device="cuda"), torch.zeros(rows6, device="cuda")
    lib.call("matvec_q4k_q8", w4.data, xq, xd, a4, rows4, k)
    lib.call("matvec_q6k_q8", w6.data, xq, xd, a6, rows6, k)
    b4, b6 = torch.zeros(rows4, device="cuda"), torch.zeros(rows6, device="cuda")
    lib.call("matvec_q4k_q6k_pair_q8", w4.data, b4, rows4, w6.data, b6, rows6, xq, xd, k)
    assert bit_equal(a6.cpu().numpy(), b6.cpu().numpy())
    a4, b4 = a4.cpu().numpy(), b4.cpu().numpy()
    assert np.abs(a4 - b4).max() <= 1e-6 * np.abs(a4).max()


def test_pair_launch_declines_what_the_bulk_copy_kernel_takes():
    """More than 6144 rows belongs to the bulk-copy kernel, k > 4096 to the staged one: UnsupportedOperation (7) and
    nothing launched; a bad shape is InvalidValue (2)."""
    buf = torch.zeros(1 << 16, device="cuda")
    for rows4, rows6, k, want in ((6152, 1024, 4096, 7), (1024, 6152, 3072, 7), (1024, 1024, 4096 + 256, 7), (1024, 0, 1024, 7),
                                  (1024, 1024, 100, 2)):
        assert lib.call("matvec_q4k_q6k_pair_q8", buf, buf, rows4, buf, buf, rows6, buf, buf, k, raise_on_error=False) == want
