"""GGUF reader and model loader: a tiny model written as a GGUF file (tests/gguf_writer.py) read back through the
C ABI.  The directory and metadata checks need no GPU; the decode comparison does."""
import ctypes as C

import numpy as np
import pytest

from gguf_writer import write
from kernelcore_b200 import decoder, lib, tiny_model as tm


def open_gguf(path, max_ctx):
    h, d = C.c_void_p(), decoder._Desc()
    st = lib.raw.kcb_gguf_open(str(path).encode(), max_ctx, C.byref(h), C.byref(d))
    lib.raw.kcb_gguf_last_error.restype = C.c_char_p
    return st, h, d


@pytest.mark.parametrize("shape_fn,arch", [(tm.tiny, "llama"), (tm.tiny_qwen, "qwen3")])
def test_directory_metadata_and_tensor_bytes(tmp_path, shape_fn, arch):
    shape = shape_fn(max_ctx=24)
    model = tm.build(shape, seed=4)
    path = tmp_path / "m.gguf"
    write(path, shape, model, arch)
    st, h, d = open_gguf(path, 24)
    assert st == 0, lib.raw.kcb_gguf_last_error()
    for f in ("hidden", "inter", "heads", "kv_heads", "head_dim", "vocab", "max_ctx"):
        assert getattr(d, f) == getattr(shape, f), f
    assert d.n_layers == shape.layers and d.neox == int(shape.neox) and d.qk_norm == int(shape.qk_norm)
    assert abs(d.eps - shape.eps) < 1e-12 and d.rope_base == np.float32(shape.rope_base)
    ms = tm.mat_shapes(shape)
    for l, L in enumerate(model["layers"]):
        for name in tm.MATS:
            m = getattr(d.layers[l], name)
            rows, k, q6 = ms[name]
            assert (m.rows, m.k, m.fmt) == (rows, k, 6 if q6 else 4)
            want = np.ascontiguousarray(L[name], np.uint8).tobytes()
            assert C.string_at(m.blocks, len(want)) == want
        assert C.string_at(d.layers[l].attn_norm, shape.hidden * 4) == np.asarray(L["attn_norm"], np.float32).tobytes()
    assert d.lm_head.rows == shape.vocab and d.lm_head.fmt == 6          # tied: token_embd serves as the output matrix
    lib.raw.kcb_gguf_weight_bytes.restype = C.c_longlong
    assert lib.raw.kcb_gguf_weight_bytes(h) == tm.weight_bytes_per_token(shape)
    lib.raw.kcb_gguf_close(h)


def test_bad_files_are_refused(tmp_path):
    shape = tm.tiny(max_ctx=8)
    model = tm.build(shape, seed=4)
    good = tmp_path / "good.gguf"
    write(good, shape, model)
    raw = good.read_bytes()
    (tmp_path / "magic.gguf").write_bytes(b"GGML" + raw[4:])
    (tmp_path / "short.gguf").write_bytes(raw[:len(raw) // 2])
    (tmp_path / "arch.gguf").write_bytes(raw.replace(b"\x05\x00\x00\x00\x00\x00\x00\x00llama", b"\x05\x00\x00\x00\x00\x00\x00\x00gemma", 1))
    for name, needle in (("magic.gguf", b"not a GGUF"), ("short.gguf", b"past the end"), ("arch.gguf", b"only llama"), ("absent.gguf", b"cannot open")):
        st, h, _ = open_gguf(tmp_path / name, 8)
        assert st == 15 and needle in lib.raw.kcb_gguf_last_error(), (name, lib.raw.kcb_gguf_last_error())
    st, h, _ = open_gguf(good, 8)
    assert st == 0
    lib.raw.kcb_gguf_close(h)


@pytest.mark.gpu
@pytest.mark.parametrize("shape_fn,arch", [(tm.tiny, "llama"), (tm.tiny_qwen, "qwen3")])
def test_decoder_from_file_equals_decoder_from_arrays(tmp_path, shape_fn, arch):
    shape = shape_fn(max_ctx=24)
    model = tm.build(shape, seed=6)
    path = tmp_path / "m.gguf"
    write(path, shape, model, arch)
    st, h, d = open_gguf(path, 24)
    assert st == 0, lib.raw.kcb_gguf_last_error()
    dec = C.c_void_p()
    assert lib.raw.kcb_decoder_create(C.byref(d), C.byref(dec)) == 0
    prompt = np.array([3, 1, 4, 1, 5, 9, 2, 6], np.int32)
    lib.raw.kcb_decoder_set_prompt(dec, prompt.ctypes.data_as(C.c_void_p), 8, 0)
    lib.raw.kcb_decoder_run(dec, 12)
    got, hist = np.zeros(shape.vocab, np.float32), np.zeros(12, np.int32)
    pos = C.c_int()
    assert lib.raw.kcb_decoder_read(dec, got.ctypes.data_as(C.c_void_p), hist.ctypes.data_as(C.c_void_p), 12, C.byref(pos)) == 0
    lib.raw.kcb_decoder_destroy(dec)
    lib.raw.kcb_gguf_close(h)
    with decoder.FastDecoder(shape, model) as ref:
        ref.set_prompt(prompt)
        ref.run(12)
        want, whist, wpos = ref.read(12)
    assert pos.value == wpos == 12 and (hist == whist).all() and (got.view(np.uint32) == want.view(np.uint32)).all()
