"""Writes a kernelcore_b200.tiny_model model as a GGUF v3 file the way llama.cpp lays one out (header, metadata
pairs, tensor directory, 32-byte aligned tensor data), so the GGUF reader can be tested without a downloaded model."""
import struct

import numpy as np

from kernelcore_b200 import tiny_model as tm

F32, Q4_K, Q6_K = 0, 12, 14
U32, F32V, STR, ARR = 4, 6, 8, 9


def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def _kv(key, vtype, payload):
    return _s(key.encode()) + struct.pack("<I", vtype) + payload


def write(path, shape: tm.Shape, model: dict, arch="llama", tokens=("<s>", "Ġhello", "Ċ")):
    ms = tm.mat_shapes(shape)
    names = {"wq": "attn_q", "wk": "attn_k", "wv": "attn_v", "wo": "attn_output", "wg": "ffn_gate", "wu": "ffn_up", "wd": "ffn_down"}
    tensors = [("token_embd.weight", Q6_K, [shape.hidden, shape.vocab], np.ascontiguousarray(model["lm_head"], np.uint8).tobytes())]
    for l, L in enumerate(model["layers"]):
        for key, gname in names.items():
            rows, k, q6 = ms[key]
            tensors.append((f"blk.{l}.{gname}.weight", Q6_K if q6 else Q4_K, [k, rows], np.ascontiguousarray(L[key], np.uint8).tobytes()))
        tensors.append((f"blk.{l}.attn_norm.weight", F32, [shape.hidden], np.asarray(L["attn_norm"], np.float32).tobytes()))
        tensors.append((f"blk.{l}.ffn_norm.weight", F32, [shape.hidden], np.asarray(L["ffn_norm"], np.float32).tobytes()))
        if shape.qk_norm:
            tensors.append((f"blk.{l}.attn_q_norm.weight", F32, [shape.head_dim], np.asarray(L["q_norm"], np.float32).tobytes()))
            tensors.append((f"blk.{l}.attn_k_norm.weight", F32, [shape.head_dim], np.asarray(L["k_norm"], np.float32).tobytes()))
    tensors.append(("output_norm.weight", F32, [shape.hidden], np.asarray(model["out_norm"], np.float32).tobytes()))

    u32 = lambda v: struct.pack("<I", v)
    kvs = [
        _kv("general.architecture", STR, _s(arch.encode())),
        _kv("general.name", STR, _s(shape.name.encode())),
        _kv(f"{arch}.embedding_length", U32, u32(shape.hidden)),
        _kv(f"{arch}.feed_forward_length", U32, u32(shape.inter)),
        _kv(f"{arch}.block_count", U32, u32(shape.layers)),
        _kv(f"{arch}.attention.head_count", U32, u32(shape.heads)),
        _kv(f"{arch}.attention.head_count_kv", U32, u32(shape.kv_heads)),
        _kv(f"{arch}.attention.key_length", U32, u32(shape.head_dim)),
        _kv(f"{arch}.attention.layer_norm_rms_epsilon", F32V, struct.pack("<f", shape.eps)),
        _kv(f"{arch}.rope.freq_base", F32V, struct.pack("<f", shape.rope_base)),
        _kv("tokenizer.ggml.tokens", ARR, struct.pack("<IQ", STR, len(tokens)) + b"".join(_s(t.encode()) for t in tokens)),
    ]
    directory, offset = b"", 0
    for name, ttype, ne, data in tensors:
        directory += _s(name.encode()) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne) + struct.pack("<IQ", ttype, offset)
        offset += (len(data) + 31) // 32 * 32
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kvs)) + b"".join(kvs) + directory
    with open(path, "wb") as f:
        f.write(head + b"\0" * (-len(head) % 32))
        for _, _, _, data in tensors:
            f.write(data + b"\0" * (-len(data) % 32))
