"""The ggml backend object (kernelcore_b200/csrc/ggml_backend.cpp) driven through ggml's own interface tables by a
C++ program compiled against the ggml stand-in headers (tests/ggml/ggml_backend_test.cpp).

CPU: registry / device / buffer-type properties and the supports_op accept / reject table.  GPU: a tiny Llama-style
model uploaded through set_tensor, the prompt graph llama.cpp would build run by graph_compute, logits against the
oracle's restatement of the batched pipeline, and get_tensor returning the canonical GGUF bytes of staged weights."""
import os
import struct
import subprocess

import numpy as np
import pytest

import oracle
from helpers import oracle_prefill, rel_diff
from kernelcore_b200 import lib, tiny_model as tm

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def driver():
    out_dir = os.path.join(HERE, "ggml", "build")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "ggml_backend_test")
    src = os.path.join(HERE, "ggml", "ggml_backend_test.cpp")
    libdir = os.path.dirname(lib.LIB_PATH)
    subprocess.run(["g++", "-std=c++20", "-O1", "-I" + os.path.join(ROOT, "include", "stub", "ggml"), "-I" + os.path.join(ROOT, "include"), src,
                    "-o", exe, "-L" + libdir, "-lkernelcore_b200", "-Wl,-rpath," + libdir], check=True)
    return exe


def test_exports_and_support_rules(driver):
    """No device needed: the three exported functions exist, the registry / device / buffer types answer as llama.cpp
    expects, and supports_op accepts and rejects what the reference's rules do."""
    for sym in ("ggml_backend_kernelcore_init", "ggml_backend_is_kc", "ggml_backend_kernelcore_reg"):
        assert hasattr(lib.raw, sym)
    r = subprocess.run([driver, "rules"], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stdout + r.stderr


def _pad16(b: bytes) -> bytes:
    return b + b"\0" * (-len(b) % 16)


@pytest.mark.gpu
@pytest.mark.parametrize("n_tokens,bound", [(3, 1e-5), (8, 1e-5), (21, 3e-2)])
def test_prompt_graph_through_graph_compute(driver, tmp_path, n_tokens, bound):
    """ADD + RMS_NORM + MUL fusion, shared quantized inputs of q/k/v and gate/up, rope, SET_ROWS + FLASH_ATTN_EXT over the
    fp16 cache, SwiGLU with quantized output, the one-column tail: logits of the last prompt token against the oracle's
    batched pipeline (same bounds as the decoder's prompt pass: 1e-5 on lengths where no re-quantized activation lands
    on a rounding boundary, 3e-2 always), twice over the same graph."""
    s = tm.tiny(max_ctx=32)
    model = tm.build(s, seed=8)
    tokens = [int(t) for t in np.random.default_rng(n_tokens).integers(0, s.vocab, n_tokens)]
    X = np.zeros((n_tokens, s.hidden), np.float32)
    for i, t in enumerate(tokens):
        oracle.port.dequant_row_q6k(np.ascontiguousarray(model["lm_head"][t]), s.hidden, X[i])
    hdr = struct.pack("9i2f5i", s.hidden, s.inter, s.layers, s.heads, s.kv_heads, s.head_dim, s.vocab, n_tokens, int(s.neox), s.eps, s.rope_base,
                      0, 0, 0, 0, 0)
    blob = [hdr, _pad16(X.tobytes())]
    for L in model["layers"]:
        for name in tm.MATS:
            blob.append(_pad16(np.ascontiguousarray(L[name]).tobytes()))
        blob += [_pad16(L["attn_norm"].tobytes()), _pad16(L["ffn_norm"].tobytes())]
    blob += [_pad16(model["out_norm"].tobytes()), _pad16(np.ascontiguousarray(model["lm_head"]).tobytes())]
    mpath, opath = tmp_path / "model.bin", tmp_path / "out.bin"
    mpath.write_bytes(b"".join(blob))
    r = subprocess.run([driver, "graph", str(mpath), str(opath)], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.startswith("ok"), r.stdout + r.stderr
    out = opath.read_bytes()
    logits = np.frombuffer(out[:s.vocab * 4], np.float32)
    want = oracle_prefill(s, model, tokens, tail_ggml=True)
    assert rel_diff(logits, want) < bound
    assert int(logits.argmax()) == int(want.argmax())
    # get_tensor of staged weights: the canonical GGUF bytes that went in (Q4_K stored as is, Q6_K back from its planes)
    wq, wv = np.ascontiguousarray(model["layers"][0]["wq"]).tobytes(), np.ascontiguousarray(model["layers"][0]["wv"]).tobytes()
    rest = out[s.vocab * 4:]
    assert rest[:len(wq)] == wq and rest[len(wq):len(wq) + len(wv)] == wv
