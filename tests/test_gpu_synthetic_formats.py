"""The reference's synthetic 8-bit / 4-bit weight formats and its fp16 matmul on the GPU, bit for bit against the
oracle (itself pinned to the compiled reference in test_oracle.py), through the C ABI and by kernel name."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import bit_equal
from kernelcore_b200 import lib

pytestmark = pytest.mark.gpu
P = oracle.port


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("rows,k", [(8, 32), (40, 96), (1000, 256), (640, 1024)])
def test_matvecs_bit_identical(rows, k):
    rng = np.random.default_rng(rows + k)
    nb = k // 32
    x = rng.standard_normal(k).astype(np.float32)
    scales = rng.uniform(0.01, 0.1, rows * nb).astype(np.float32)
    q8 = rng.integers(-127, 128, rows * k, dtype=np.int8)
    qs = rng.integers(0, 256, rows * k // 2, dtype=np.uint8)
    dx, dsc = dev(x), dev(scales)

    want = np.zeros(rows, np.float32)
    P.matvec_q8w(q8, scales, x, want, rows, k)
    y = torch.full((rows,), float("nan"), device="cuda")
    lib.call("matvec_q8w", dev(q8), dsc, dx, y, rows, k)
    assert bit_equal(y.cpu().numpy(), want)

    P.matvec_q4w(qs, scales, x, want, rows, k)
    y.fill_(float("nan"))
    lib.call("matvec_q4w", dev(qs), dsc, dx, y, rows, k, 0)
    assert bit_equal(y.cpu().numpy(), want)

    qs8, sc8 = np.zeros_like(qs), np.zeros_like(scales)
    P.repack_q4x8(qs, scales, qs8, sc8, rows, k)
    P.matvec_q4x8(qs8, sc8, x, want, rows, k)
    y.fill_(float("nan"))
    lib.call("matvec_q4w", dev(qs8), dev(sc8), dx, y, rows, k, 1)
    assert bit_equal(y.cpu().numpy(), want)

    qw = np.zeros(rows * nb * 5, np.int32)
    P.repack_q4x8_q8(qs, scales, qw, rows, k)
    xq, xd = oracle.quantize_q8x4(P, x)
    P.matvec_q4x8_q8(qw, xq, xd, want, rows, k)
    y.fill_(float("nan"))
    lib.call("matvec_q4x8_q8", dev(qw), dev(xq), dev(xd), y, rows, k)
    assert bit_equal(y.cpu().numpy(), want)
    assert lib.call("matvec_q4w", dev(qs8), dev(sc8), dx, y, rows + 4, k, 1, raise_on_error=False) != 0   # rows % 8


@pytest.mark.parametrize("rows,k,ncols", [(8, 2, 1), (40, 96, 5), (256, 130, 33)])
def test_matmul_f16_bit_identical(rows, k, ncols):
    """Includes fp16 subnormals, both signs and the largest finite values (tests/test_llm_kernels.cpp:710-737 draws
    normal weights; inf / NaN weights are not produced by any model and are left out)."""
    rng = np.random.default_rng(rows)
    w16 = rng.integers(0, 0x7C00, rows * k).astype(np.uint16) | (rng.integers(0, 2, rows * k).astype(np.uint16) << 15)
    w16[:4] = [0x0001, 0x83FF, 0x7BFF, 0x8000]
    X = rng.standard_normal((ncols, k)).astype(np.float32)
    want = np.zeros((ncols, rows), np.float32)
    P.matmul_f16(w16, X, want, rows, k, ncols)
    st = np.zeros(rows * k // 2, np.int32)
    P.repack_f16(w16, rows, k, st)
    y = torch.full((ncols, rows), float("nan"), device="cuda")
    lib.call("matmul_f16", dev(st), dev(X), y, rows, k, ncols)
    assert bit_equal(y.cpu().numpy(), want)


def test_launch_by_name_two_row_form():
    """matvec_q4x8_q8x2 by name with the reference's argument struct (llm/llm_kernels.hpp:62-70): same results as
    matvec_q4x8_q8, rows % 16 enforced (llm/llm_kernels.cpp:236-240)."""
    L = lib.raw

    class Args(C.Structure):
        _fields_ = [("qw", C.c_void_p), ("xq", C.c_void_p), ("xd", C.c_void_p), ("y", C.c_void_p), ("dims", C.c_void_p),
                    ("rows", C.c_int), ("k", C.c_int)]

    assert L.kcb_init() == 0
    try:
        rows, k = 32, 64
        rng = np.random.default_rng(0)
        qs = rng.integers(0, 256, rows * k // 2, dtype=np.uint8)
        scales = rng.uniform(0.01, 0.1, rows * k // 32).astype(np.float32)
        x = rng.standard_normal(k).astype(np.float32)
        qw = np.zeros(rows * (k // 32) * 5, np.int32)
        P.repack_q4x8_q8(qs, scales, qw, rows, k)
        xq, xd = oracle.quantize_q8x4(P, x)
        want = np.zeros(rows, np.float32)
        P.matvec_q4x8_q8(qw, xq, xd, want, rows, k)

        def up(a):
            p = C.c_void_p()
            assert L.kcb_malloc(C.byref(p), C.c_size_t(a.nbytes)) == 0
            assert L.kcb_memcpy(p, a.ctypes.data_as(C.c_void_p), C.c_size_t(a.nbytes), 0) == 0
            return p

        dy = up(np.zeros(rows, np.float32))
        a = Args(up(qw), up(xq), up(xd), dy, up(np.array([rows, k], np.int32)), rows, k)
        assert L.kcb_launch_kernel(b"matvec_q4x8_q8x2", C.byref(a), None) == 0
        got = np.zeros(rows, np.float32)
        assert L.kcb_memcpy(got.ctypes.data_as(C.c_void_p), dy, C.c_size_t(got.nbytes), 1) == 0
        assert bit_equal(got, want)
        a.rows = 24
        assert L.kcb_launch_kernel(b"matvec_q4x8_q8x2", C.byref(a), None) == 2      # InvalidValue: rows % 16
        assert L.kcb_launch_kernel(b"matvec_q4x8_q8", C.byref(a), None) == 0
    finally:
        L.kcb_shutdown()
