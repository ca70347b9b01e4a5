"""The kc runtime on CUDA (through its C layer, kcb_*): lifecycle, memory + range checks, launch by name
with the reference's typed argument structs, streams, events, capture rules and graphs, error model."""
import ctypes as C

import numpy as np
import pytest

from kernelcore_b200 import lib

pytestmark = pytest.mark.gpu
L = lib.raw
L.kcb_last_error_detail.restype = C.c_char_p
H2D, D2H, D2D = 0, 1, 2


class VectorAddArgs(C.Structure):
    _fields_ = [("a", C.c_void_p), ("b", C.c_void_p), ("out", C.c_void_p), ("count", C.c_int)]


class QuantizeArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("xq", C.c_void_p), ("xd", C.c_void_p), ("count", C.c_int)]


class MatvecQ4Q8Args(C.Structure):
    _fields_ = [("qw", C.c_void_p), ("xq", C.c_void_p), ("xd", C.c_void_p), ("y", C.c_void_p), ("dims", C.c_void_p),
                ("rows", C.c_int), ("k", C.c_int)]


def dmalloc(nbytes):
    p = C.c_void_p()
    assert L.kcb_malloc(C.byref(p), C.c_size_t(nbytes)) == 0, L.kcb_last_error_detail()
    return p


def upload(a):
    a = np.ascontiguousarray(a)
    p = dmalloc(a.nbytes)
    assert L.kcb_memcpy(p, a.ctypes.data_as(C.c_void_p), C.c_size_t(a.nbytes), H2D) == 0
    return p


def download(p, shape, dtype):
    out = np.zeros(shape, dtype)
    assert L.kcb_memcpy(out.ctypes.data_as(C.c_void_p), p, C.c_size_t(out.nbytes), D2H) == 0
    return out


@pytest.fixture()
def runtime():
    assert L.kcb_init() == 0
    yield
    assert L.kcb_shutdown() == 0


def test_lifecycle_and_devices():
    n = C.c_int()
    assert L.kcb_shutdown() == 0                                # whatever an earlier test left running
    assert L.kcb_get_device_count(C.byref(n)) == 1            # NotInitialized before kcInit
    assert L.kcb_init() == 0 and L.kcb_init() == 0              # idempotent
    assert L.kcb_get_device_count(C.byref(n)) == 0 and n.value >= 1
    assert L.kcb_set_device(n.value) == 3                      # InvalidDevice
    assert L.kcb_set_device(0) == 0
    name = C.create_string_buffer(128)
    sms, mem = C.c_uint(), C.c_size_t()
    assert L.kcb_get_device_properties(name, C.byref(sms), C.byref(mem), 0) == 0
    assert sms.value > 0 and mem.value > 1 << 30
    assert L.kcb_shutdown() == 0 and L.kcb_shutdown() == 0
    p = C.c_void_p()
    assert L.kcb_malloc(C.byref(p), C.c_size_t(16)) == 1


def test_memory_rules(runtime):
    p = C.c_void_p()
    assert L.kcb_malloc(C.byref(p), C.c_size_t(0)) == 2          # zero bytes: InvalidValue
    a = np.arange(1000, dtype=np.float32)
    d = upload(a)
    assert (download(d, 1000, np.float32) == a).all()
    assert L.kcb_check_range(d, C.c_size_t(4000)) == 0
    assert L.kcb_check_range(d, C.c_size_t(4001)) == 5            # InvalidPointer: past the end
    assert b"exceeds" in L.kcb_last_error_detail()
    interior = C.c_void_p(d.value + 16)
    assert L.kcb_check_range(interior, C.c_size_t(3984)) == 0      # interior pointers are fine for ranges
    assert L.kcb_free(interior) == 5                               # ...but free takes base pointers only
    assert L.kcb_memset(d, 0, C.c_size_t(4000)) == 0
    assert (download(d, 1000, np.float32) == 0).all()
    host = np.zeros(4, np.float32)
    assert L.kcb_memcpy(host.ctypes.data_as(C.c_void_p), C.c_void_p(d.value + 3990), C.c_size_t(16), D2H) == 5
    assert L.kcb_free(d) == 0
    assert L.kcb_free(d) == 5                                      # already freed
    assert L.kcb_check_range(d, C.c_size_t(4)) == 5


def test_launch_by_name_validation_and_sync_result(runtime):
    n = 4096
    a, b = np.random.rand(n).astype(np.float32), np.random.rand(n).astype(np.float32)
    da, db, dout = upload(a), upload(b), dmalloc(n * 4)
    args = VectorAddArgs(da, db, dout, n)
    assert L.kcb_launch_kernel(b"vector_add", C.byref(args), None) == 0   # null stream: synchronous
    assert (download(dout, n, np.float32) == a + b).all()
    assert L.kcb_launch_kernel(b"no_such_kernel", C.byref(args), None) == 9          # KernelNotFound
    bad = VectorAddArgs(da, db, dout, n + 1)
    assert L.kcb_launch_kernel(b"vector_add", C.byref(bad), None) == 5               # range check before launch
    neg = VectorAddArgs(da, db, dout, -1)
    assert L.kcb_launch_kernel(b"vector_add", C.byref(neg), None) == 2
    host_ptr = VectorAddArgs(a.ctypes.data, db, dout, n)                               # a host pointer is not an allocation
    assert L.kcb_launch_kernel(b"vector_add", C.byref(host_ptr), None) == 5


def test_kquant_matvec_by_name_matches_oracle(runtime):
    import oracle
    from helpers import rel_diff
    from kernelcore_b200 import synth
    rows, k = 40, 768
    for q6, name in ((False, b"matvec_q4k_q8"), (True, b"matvec_q6k_q8")):
        w = synth.raw_blocks(rows, k, 5, q6)
        x = synth.activations(k, 6)
        if q6:  # planes, as llm::ref::repackQ6K lays them out
            blk = w.reshape(-1, 210)
            packed = np.concatenate([blk[:, :128].ravel(), blk[:, 128:192].ravel(), blk[:, 192:208].ravel(), blk[:, 208:].ravel()])
        else:
            packed = w.ravel()
        dw, dx = upload(packed), upload(x)
        nb = k // 32
        dxq, dxd, dy, dd = dmalloc(nb * 32), dmalloc(nb * 8), dmalloc(rows * 4), upload(np.array([rows, k], np.int32))
        q = QuantizeArgs(dx, dxq, dxd, nb)
        assert L.kcb_launch_kernel(b"quantize_q8x4", C.byref(q), None) == 0
        m = MatvecQ4Q8Args(dw, dxq, dxd, dy, dd, rows, k)
        assert L.kcb_launch_kernel(name, C.byref(m), None) == 0, L.kcb_last_error_detail()
        y = download(dy, rows, np.float32)
        assert rel_diff(y, oracle.matvec_q8(oracle.port, w, x, rows, k, q6)) < 1e-5
        odd = MatvecQ4Q8Args(dw, dxq, dxd, dy, dd, rows - 1, k)       # rows % 8 != 0 (llm_kernels.cpp:266)
        assert L.kcb_launch_kernel(name, C.byref(odd), None) == 2
        short = MatvecQ4Q8Args(dw, dxq, dxd, dy, dd, rows + 8, k)     # weights too small for the shape
        assert L.kcb_launch_kernel(name, C.byref(short), None) == 5


def test_streams_events_and_capture_rules(runtime):
    s = C.c_void_p()
    assert L.kcb_stream_create(C.byref(s)) == 0
    n = 1 << 20
    a = np.ones(n, np.float32)
    da, dout = upload(a), dmalloc(n * 4)
    e0, e1 = C.c_void_p(), C.c_void_p()
    assert L.kcb_event_create(C.byref(e0)) == 0 and L.kcb_event_create(C.byref(e1)) == 0
    args = VectorAddArgs(da, da, dout, n)
    assert L.kcb_event_record(e0, s) == 0
    for _ in range(10):
        assert L.kcb_launch_kernel(b"vector_add", C.byref(args), s) == 0      # asynchronous on a created stream
    assert L.kcb_event_record(e1, s) == 0
    assert L.kcb_stream_synchronize(s) == 0 and L.kcb_stream_query(s) == 0 and L.kcb_event_query(e1) == 0
    ms = C.c_float()
    assert L.kcb_event_elapsed_ms(e0, e1, C.byref(ms)) == 0 and ms.value > 0
    assert (download(dout, n, np.float32) == 2).all()
    assert L.kcb_stream_synchronize(C.c_void_p(12345)) == 6                     # InvalidResourceHandle

    # capture: launches are validated and recorded, not run; copies / memsets / frees / sync refused
    assert L.kcb_memset(dout, 0, C.c_size_t(n * 4)) == 0
    assert L.kcb_stream_begin_capture(s) == 0
    assert L.kcb_launch_kernel(b"vector_add", C.byref(args), s) == 0
    bad = VectorAddArgs(da, da, dout, n + 1)
    assert L.kcb_launch_kernel(b"vector_add", C.byref(bad), s) == 5             # still validated while recording
    host = np.zeros(n, np.float32)
    assert L.kcb_memcpy(host.ctypes.data_as(C.c_void_p), dout, C.c_size_t(n * 4), D2H) == 7
    assert L.kcb_memset(dout, 0, C.c_size_t(16)) == 7
    assert L.kcb_free(dout) == 7
    assert L.kcb_device_synchronize() == 7
    assert L.kcb_stream_synchronize(s) == 7
    assert L.kcb_stream_concurrent(s, 1) == 0 and L.kcb_stream_concurrent(s, 0) == 0
    g = C.c_void_p()
    assert L.kcb_stream_end_capture(s, C.byref(g)) == 0
    assert (download(dout, n, np.float32) == 0).all()                           # nothing ran during capture
    assert L.kcb_graph_launch(g, None) == 0                                     # null stream: synchronous
    assert (download(dout, n, np.float32) == 2).all()
    assert L.kcb_graph_launch(g, s) == 0 and L.kcb_stream_synchronize(s) == 0   # relaunchable
    assert L.kcb_graph_destroy(g) == 0 and L.kcb_graph_destroy(g) == 6
    assert L.kcb_stream_end_capture(s, C.byref(g)) == 2                          # not capturing
    assert L.kcb_event_destroy(e0) == 0 and L.kcb_event_destroy(e1) == 0
    assert L.kcb_stream_destroy(s) == 0 and L.kcb_stream_destroy(s) == 6


def test_device_reset_frees_everything(runtime):
    d = upload(np.zeros(16, np.float32))
    assert L.kcb_device_reset() == 0
    assert L.kcb_check_range(d, C.c_size_t(4)) == 5
    assert L.kcb_tma_timeouts() == 0


def test_four_launch_flash_attention_by_name(runtime, golden):
    """fa_scores -> fa_max -> fa_exp -> fa_values launched by name with the reference's FaDims structs, against the
    reference's flashAttnF16 output (tests/test_llm_kernels.cpp:741-794, relDiff < 2e-6)."""
    from helpers import pad8, rel_diff
    g = golden("glue")

    class FaDims(C.Structure):
        _fields_ = [(n, C.c_int) for n in ("H", "T", "D", "group", "tp", "k_row", "k_head", "v_row", "v_head", "N", "q_tok",
                                           "q_head", "m_row", "has_mask", "H_kv")]

    class FaScoresArgs(C.Structure):
        _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("mask", C.c_void_p), ("s", C.c_void_p), ("dims", C.c_void_p),
                    ("d", FaDims), ("scale", C.c_float)]

    class FaMaxArgs(C.Structure):
        _fields_ = [("s", C.c_void_p), ("m", C.c_void_p), ("dims", C.c_void_p), ("d", FaDims)]

    class FaValuesArgs(C.Structure):
        _fields_ = [("p", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("dims", C.c_void_p), ("d", FaDims)]

    for tag in "abc":
        H, Hkv, D, T, N, mask = (int(v) for v in g[f"fa_{tag}_dims"])
        tp = pad8(T)
        d = FaDims(H, T, D, H // Hkv, tp, Hkv * D // 2, D // 2, Hkv * D // 2, D // 2, N, H * D, D, tp // 2, mask, Hkv)
        dq, dk, dv = upload(g[f"fa_{tag}_q"]), upload(g[f"fa_{tag}_k"]), upload(g[f"fa_{tag}_v"])
        dm, ddims = upload(g[f"fa_{tag}_mask"]), upload(np.zeros(15, np.int32))
        ds, dmx, dout = dmalloc(H * N * tp * 4), dmalloc(H * N * 4), dmalloc(N * H * D * 4)
        a = FaScoresArgs(dq, dk, dm, ds, ddims, d, float(D) ** -0.5)
        assert L.kcb_launch_kernel(b"fa_scores", C.byref(a), None) == 0, L.kcb_last_error_detail()
        b = FaMaxArgs(ds, dmx, ddims, d)
        assert L.kcb_launch_kernel(b"fa_max", C.byref(b), None) == 0
        assert L.kcb_launch_kernel(b"fa_exp", C.byref(b), None) == 0      # FaExpArgs has the same layout
        c = FaValuesArgs(ds, dv, dout, ddims, d)
        assert L.kcb_launch_kernel(b"fa_values", C.byref(c), None) == 0
        assert rel_diff(download(dout, (N, H, D), np.float32), g[f"fa_{tag}_out"]) < 2e-6
