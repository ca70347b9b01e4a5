"""The ggml operator layer (include/ggml-kernelcore-ops.h) against the oracle: tensors described the way ggml
describes them (ne / nb / op_params / src), results compared with the reference arithmetic each operator maps to."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import bit_equal, pad8, rel_diff
from kernelcore_b200 import lib, synth

pytestmark = pytest.mark.gpu
P = oracle.port
F32, F16, Q4_K, Q6_K, I32, I64 = 0, 1, 12, 14, 26, 27


class Tensor(C.Structure):
    pass


Tensor._fields_ = [("type", C.c_int), ("ne", C.c_int64 * 4), ("nb", C.c_size_t * 4), ("data", C.c_void_p),
                   ("op_params", C.c_int32 * 16), ("src", C.POINTER(Tensor) * 4)]
_keep = []


def tensor(buf, ttype, ne, nb=None, src=(), params=()):
    """buf: torch CUDA tensor holding the data; ne innermost first, as ggml."""
    t = Tensor()
    t.type = ttype
    ne = list(ne) + [1] * (4 - len(ne))
    item = {F32: 4, F16: 2, I32: 4, I64: 8}.get(ttype, 1)
    if nb is None:
        nb = [item, item * ne[0], item * ne[0] * ne[1], item * ne[0] * ne[1] * ne[2]]
    for i in range(4):
        t.ne[i], t.nb[i] = ne[i], nb[i]
    t.data = buf.data_ptr()
    for i, s in enumerate(src):
        if s is not None:
            t.src[i] = C.pointer(s)
    for i, p in enumerate(params):
        t.op_params[i] = p
    _keep.extend([buf, t, src])
    return t


def f32_bits(v):
    return int(np.float32(v).view(np.int32))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture()
def ctx():
    h = C.c_void_p()
    assert lib.raw.kcb_ggml_ctx_create(None, C.byref(h)) == 0
    assert lib.raw.kcb_ggml_ctx_begin_graph(h) == 0
    yield h
    lib.raw.kcb_ggml_ctx_destroy(h)
    _keep.clear()


def weight(ctx, blocks, ttype, rows, k):
    lib.raw.kcb_ggml_weight_bytes.restype = C.c_size_t
    n = lib.raw.kcb_ggml_weight_bytes(ttype, rows, k)
    buf = torch.zeros(n, dtype=torch.uint8, device="cuda")
    src = np.ascontiguousarray(blocks)
    assert lib.raw.kcb_ggml_set_weight(ctx, C.c_void_p(buf.data_ptr()), src.ctypes.data_as(C.c_void_p), ttype, rows, k) == 0
    return tensor(buf, ttype, [k, rows])


def op(name, ctx, *tensors):
    st = getattr(lib.raw, "kcb_ggml_" + name)(ctx, *[C.byref(t) if isinstance(t, Tensor) else t for t in tensors])
    assert st == 0, (name, st)
    torch.cuda.synchronize()


@pytest.mark.parametrize("q6", [0, 1])
def test_mul_mat_one_column_batch_and_strided(ctx, q6):
    rows, k = 256, 1024
    w = synth.kquant_blocks(rows, k, 3, bool(q6))
    wt = weight(ctx, w, Q6_K if q6 else Q4_K, rows, k)
    X = np.random.default_rng(1).standard_normal((6, k)).astype(np.float32)
    # one column: per-32 activations + matvec
    x1 = tensor(dev(X[0]), F32, [k, 1])
    y1 = torch.zeros(rows, device="cuda")
    op("mul_mat", ctx, tensor(y1, F32, [rows, 1], src=(wt, x1)))
    assert rel_diff(y1.cpu().numpy(), oracle.matvec_q8(P, w, X[0], rows, k, q6)) < 1e-5
    # a contiguous batch: per-256 slots + matmul, bit-identical per column to the reference mirror
    xb = tensor(dev(X), F32, [k, 6])
    yb = torch.zeros(6, rows, device="cuda")
    op("mul_mat", ctx, tensor(yb, F32, [rows, 6], src=(wt, xb)))
    want = np.stack([oracle.matvec_q8k(P, w, X[c], rows, k, q6) for c in range(6)])
    assert rel_diff(yb.cpu().numpy(), want) < 1e-5
    # columns with a stride (a view into a wider tensor): per-32 activations, matmul over the columns
    wide = np.zeros((3, 2 * k), np.float32)
    wide[:, :k] = X[:3]
    xs = tensor(dev(wide), F32, [k, 3], nb=[4, 8 * k, 24 * k, 24 * k])
    ys = torch.zeros(3, rows, device="cuda")
    op("mul_mat", ctx, tensor(ys, F32, [rows, 3], src=(wt, xs)))
    want = np.stack([oracle.matvec_q8(P, w, X[c], rows, k, q6) for c in range(3)])
    assert rel_diff(ys.cpu().numpy(), want) < 1e-5


def test_mul_mat_f16_weights(ctx):
    rows, k, n = 64, 96, 5
    rng = np.random.default_rng(2)
    w16 = rng.integers(0, 0x7C00, rows * k).astype(np.uint16) | (rng.integers(0, 2, rows * k).astype(np.uint16) << 15)
    X = rng.standard_normal((n, k)).astype(np.float32)
    wt = weight(ctx, w16, F16, rows, k)
    y = torch.zeros(n, rows, device="cuda")
    op("mul_mat", ctx, tensor(y, F32, [rows, n], src=(wt, tensor(dev(X), F32, [k, n]))))
    want = np.zeros((n, rows), np.float32)
    P.matmul_f16(w16, X, want, rows, k, n)
    assert bit_equal(y.cpu().numpy(), want)


@pytest.mark.parametrize("rows", [1, 4])
def test_fused_norm_feeds_the_matmul_behind_it(ctx, rows):
    """ADD + RMS_NORM + MUL: floats and the quantized form the following mul_mat picks up without re-quantizing."""
    n, eps = 512, 1e-5
    rng = np.random.default_rng(rows)
    a, b = rng.standard_normal((rows, n)).astype(np.float32), rng.standard_normal((rows, n)).astype(np.float32)
    wn = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    ta, tb = tensor(dev(a), F32, [n, rows]), tensor(dev(b), F32, [n, rows])
    s_buf, y_buf = torch.zeros(rows, n, device="cuda"), torch.zeros(rows, n, device="cuda")
    add = tensor(s_buf, F32, [n, rows], src=(ta, tb))
    norm = tensor(torch.zeros(rows, n, device="cuda"), F32, [n, rows], src=(add,), params=[f32_bits(eps)])
    mul = tensor(y_buf, F32, [n, rows], src=(norm, tensor(dev(wn), F32, [n])))
    op("fused_norm", ctx, add, norm, mul)
    want_sum, sq = np.zeros_like(a), np.zeros((rows, n // 32 * 11), np.int32)
    P.add_sumsq_f(a, b, want_sum, sq, n, rows)
    want_y = np.zeros_like(a)
    if rows > 1:
        slots = np.zeros((rows, 85 * n // 256), np.int32)
        P.norm_mul_q8k(want_sum, wn, want_y, slots, sq, n, rows, eps)
    else:
        P.norm_mul_q8(want_sum, wn, want_y, sq, n, rows, eps)
    assert bit_equal(s_buf.cpu().numpy(), want_sum) and bit_equal(y_buf.cpu().numpy(), want_y)
    mrows = 128
    w = synth.q4k_blocks(mrows, n, 9)
    out = torch.zeros(rows, mrows, device="cuda")
    op("mul_mat", ctx, tensor(out, F32, [mrows, rows], src=(weight(ctx, w, Q4_K, mrows, n), mul)))
    fn = oracle.matvec_q8k if rows > 1 else oracle.matvec_q8
    want = np.stack([fn(P, w, want_y[c], mrows, n, 0) for c in range(rows)])
    assert rel_diff(out.cpu().numpy(), want) < 1e-5


@pytest.mark.parametrize("cols", [1, 3])
def test_swiglu_forms(ctx, cols):
    n = 512
    rng = np.random.default_rng(cols)
    g, u = rng.standard_normal((cols, n)).astype(np.float32), rng.standard_normal((cols, n)).astype(np.float32)
    tg, tu = tensor(dev(g), F32, [n, cols]), tensor(dev(u), F32, [n, cols])
    y = torch.zeros(cols, n, device="cuda")
    op("swiglu", ctx, tensor(y, F32, [n, cols], src=(tg, tu)))
    want = np.zeros_like(g)
    P.silu_mul(g, u, want, n * cols)
    assert rel_diff(y.cpu().numpy(), want) < 1e-6
    y2 = torch.zeros(cols, n, device="cuda")
    act = tensor(y2, F32, [n, cols], src=(tg, tu))
    op("fused_swiglu", ctx, act)
    assert rel_diff(y2.cpu().numpy(), want) < 1e-6
    w = synth.q6k_blocks(128, n, 4)
    out = torch.zeros(cols, 128, device="cuda")
    op("mul_mat", ctx, tensor(out, F32, [128, cols], src=(weight(ctx, w, Q6_K, 128, n), act)))
    fn = oracle.matvec_q8k if cols > 1 else oracle.matvec_q8
    ref = np.stack([fn(P, w, y2.cpu().numpy()[c], 128, n, 1) for c in range(cols)])
    assert rel_diff(out.cpu().numpy(), ref) < 1e-5


@pytest.mark.parametrize("neox", [0, 1])
def test_rope_add_mul_rms_norm(ctx, neox):
    hd, nh, nt = 64, 6, 5
    rng = np.random.default_rng(neox)
    x = rng.standard_normal((nt, nh, hd)).astype(np.float32)
    pos = np.array([0, 1, 7, 300, 4095], np.int32)
    y = torch.zeros(nt, nh, hd, device="cuda")
    params = [0, hd, 2 if neox else 0, 0, 0, f32_bits(500000.0)]
    op("rope", ctx, tensor(y, F32, [hd, nh, nt], src=(tensor(dev(x), F32, [hd, nh, nt]), tensor(dev(pos), I32, [nt])), params=params))
    want = np.zeros_like(x)
    P.rope_ggml(x, want, pos, np.ones(hd // 2, np.float32), hd, nh, nt, float(np.log2(np.float32(500000.0))), neox)
    assert rel_diff(y.cpu().numpy(), want) < 1e-3          # the reference's own bound for rope (tests/test_llm_kernels.cpp:847)
    a, b = x.reshape(nt * nh, hd), rng.standard_normal(hd).astype(np.float32)
    s = torch.zeros(nt * nh, hd, device="cuda")
    ta = tensor(dev(a), F32, [hd, nt * nh])
    op("add", ctx, tensor(s, F32, [hd, nt * nh], src=(ta, ta)))
    assert bit_equal(s.cpu().numpy(), a + a)
    op("mul", ctx, tensor(s, F32, [hd, nt * nh], src=(ta, tensor(dev(b), F32, [hd]))))
    assert bit_equal(s.cpu().numpy(), a * b)
    norm = tensor(torch.zeros(1, device="cuda"), F32, [hd, nt * nh], src=(ta,), params=[f32_bits(1e-6)])
    op("rms_norm", ctx, norm, None, tensor(s, F32, [hd, nt * nh]))
    want = np.zeros_like(a)
    P.rms_norm(a, np.ones(hd, np.float32), want, hd, nt * nh, 1e-6)
    assert rel_diff(s.cpu().numpy(), want) < 1e-6


def test_set_rows_then_flash_attention(ctx):
    """K and V rows written into an fp16 cache by SET_ROWS, then FLASH_ATTN_EXT over the cache with a causal mask."""
    H, Hkv, D, T, N = 6, 2, 64, 21, 3
    rng = np.random.default_rng(5)
    kf, vf = rng.standard_normal((T, Hkv * D)).astype(np.float32), rng.standard_normal((T, Hkv * D)).astype(np.float32)
    q = rng.standard_normal((H, N, D)).astype(np.float32)                 # ggml's [D, N, H]
    idx = np.arange(T, dtype=np.int64)
    kc, vc = torch.zeros(T, Hkv * D, dtype=torch.float16, device="cuda"), torch.zeros(T, Hkv * D, dtype=torch.float16, device="cuda")
    tidx = tensor(dev(idx), I64, [T])
    op("set_rows", ctx, tensor(kc, F16, [Hkv * D, T], src=(tensor(dev(kf), F32, [Hkv * D, T]), tidx)))
    op("set_rows", ctx, tensor(vc, F16, [Hkv * D, T], src=(tensor(dev(vf), F32, [Hkv * D, T]), tidx)))
    want_k, want_v = np.zeros((T, Hkv * D), np.uint16), np.zeros((T, Hkv * D), np.uint16)
    P.set_rows_f16(kf, idx, want_k, Hkv * D // 2, T, Hkv * D, Hkv * D // 2, T)
    P.set_rows_f16(vf, idx, want_v, Hkv * D // 2, T, Hkv * D, Hkv * D // 2, T)
    assert bit_equal(kc.cpu().numpy().view(np.uint16), want_k) and bit_equal(vc.cpu().numpy().view(np.uint16), want_v)
    tp = pad8(T)
    mask = np.full((N, tp), 0xFC00, np.uint16)
    for i in range(N):
        mask[i, :T - N + i + 1] = 0
    # cache viewed as [D, T, Hkv]: row stride Hkv*D halves, head stride D halves
    kt = tensor(kc, F16, [D, T, Hkv], nb=[2, 2 * Hkv * D, 2 * D, 2 * Hkv * D * T])
    vt = tensor(vc, F16, [D, T, Hkv], nb=[2, 2 * Hkv * D, 2 * D, 2 * Hkv * D * T])
    qt = tensor(dev(q), F32, [D, N, H])
    mt = tensor(dev(mask), F16, [tp, N])
    out = torch.zeros(N, H, D, device="cuda")
    scale = float(np.float32(1) / np.sqrt(np.float32(D)))
    op("flash_attn", ctx, tensor(out, F32, [D, H, N], src=(qt, kt, vt, mt), params=[f32_bits(scale)]))
    d = oracle.FaDims(H, T, D, H // Hkv, tp, Hkv * D // 2, D // 2, Hkv * D // 2, D // 2, N, D, N * D, tp // 2, 1, Hkv)
    want = np.zeros((N, H, D), np.float32)
    P.flash_attn_f16(q, want_k, want_v, mask, want, C.byref(d), scale)
    assert rel_diff(out.cpu().numpy(), want) < 2e-6        # tests/test_llm_kernels.cpp:741-794
