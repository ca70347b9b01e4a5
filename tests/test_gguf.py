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


def _patched(raw: bytes, tensor: bytes, field: str, value: int) -> bytes:
    """raw with one field of `tensor`'s directory entry replaced: name, u32 rank, u64 extents, u32 type, u64 offset."""
    at = raw.index(len(tensor).to_bytes(8, "little") + tensor) + 8 + len(tensor)
    rank = int.from_bytes(raw[at:at + 4], "little")
    where = {"ne0": (at + 4, 8), "ne1": (at + 12, 8), "type": (at + 4 + 8 * rank, 4), "offset": (at + 8 + 8 * rank, 8)}[field]
    return raw[:where[0]] + value.to_bytes(where[1], "little") + raw[where[0] + where[1]:]


def test_crafted_directories_cannot_point_outside_the_file(tmp_path):
    """Offsets and extents are 64-bit numbers under the file's control: none of them may wrap a sum or a product into
    something that passes the bounds check (the reader computes sizes in 128 bits and compares by subtraction).  A tensor
    of a type the reader has no block size for stays listed and unreadable, as in the reference (llm/gguf.cpp:126-130),
    and a newer format version is not refused (llm/gguf.cpp:95 refuses only versions below 2)."""
    shape = tm.tiny(max_ctx=8)
    good = tmp_path / "good.gguf"
    write(good, shape, tm.build(shape, seed=4))
    raw = good.read_bytes()
    q = b"blk.0.attn_q.weight"
    cases = {
        "offset_wraps": (_patched(raw, q, "offset", 2**64 - 64), b"past the end"),
        "offset_far": (_patched(raw, q, "offset", 2**62), b"past the end"),
        "rows_huge": (_patched(raw, q, "ne1", 2**62), b"extent out of range"),
        "rows_wrap": (_patched(raw, q, "ne1", 2**39), b"larger than the file"),
        "cols_zero": (_patched(raw, q, "ne0", 0), b"extent out of range"),
        "cols_ragged": (_patched(raw, q, "ne0", shape.hidden + 32), b"whole number of blocks"),
        "type_unknown": (_patched(raw, q, "type", 30), b"matrix type not supported"),       # listed, then refused by the loader
    }
    for name, (data, needle) in cases.items():
        (tmp_path / f"{name}.gguf").write_bytes(data)
        st, h, _ = open_gguf(tmp_path / f"{name}.gguf", 8)
        assert st == 15 and needle in lib.raw.kcb_gguf_last_error(), (name, lib.raw.kcb_gguf_last_error())
    (tmp_path / "v4.gguf").write_bytes(raw[:4] + (4).to_bytes(4, "little") + raw[8:])
    st, h, _ = open_gguf(tmp_path / "v4.gguf", 8)
    assert st == 0, lib.raw.kcb_gguf_last_error()
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
