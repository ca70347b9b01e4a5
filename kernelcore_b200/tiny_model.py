"""Seeded random-init decoder models in the Q4_K_M mix (Q4_K for q, k, o, gate, up; Q6_K for
v, down and the tied output/embedding matrix), as host numpy arrays of GGUF blocks."""
from __future__ import annotations

import dataclasses
import hashlib

import numpy as np

from . import synth


@dataclasses.dataclass
class Shape:
    name: str
    hidden: int
    inter: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    max_ctx: int
    eps: float = 1e-5
    rope_base: float = 500000.0
    neox: bool = False       # NEOX pairing (i, i + head_dim/2) instead of adjacent pairs
    qk_norm: bool = False    # per-head RMSNorm on q and k before RoPE (Qwen3)

    @property
    def kv(self):
        return self.kv_heads * self.head_dim

    @property
    def qd(self):
        return self.heads * self.head_dim


def tiny(max_ctx: int = 40) -> Shape:
    """Small shapes for correctness checks: the reference's tinyConfig (llm/llm_model.cpp:51-57)
    with the FFN width and vocabulary moved to multiples of 256 / 8 that K-quants need."""
    return Shape("tiny", 256, 512, 2, 4, 2, 64, 256, max_ctx)


def tiny_qwen(max_ctx: int = 40) -> Shape:
    """Tiny shapes with the Qwen3 features: NEOX RoPE pairing, per-head q/k RMSNorm, head_dim 128, group 4."""
    return Shape("tiny-qwen", 256, 512, 2, 4, 1, 128, 256, max_ctx, eps=1e-6, rope_base=1e6, neox=True, qk_norm=True)


def reference_tiny() -> Shape:
    """The reference's tinyConfig (llm/llm_model.cpp:51-57) exactly: the shape of its synthetic-format models."""
    return Shape("tiny", 256, 640, 2, 4, 2, 64, 1000, 40)


def llama32_3b(max_ctx: int) -> Shape:
    return Shape("llama-3.2-3b-arch", 3072, 8192, 28, 24, 8, 128, 128256, max_ctx)


def qwen3_8b(max_ctx: int) -> Shape:
    return Shape("qwen3-8b-arch", 4096, 12288, 36, 32, 8, 128, 151936, max_ctx, eps=1e-6, rope_base=1e6, neox=True,
                 qk_norm=True)


MATS = ("wq", "wk", "wv", "wo", "wg", "wu", "wd")


def mat_shapes(s: Shape):
    """name -> (rows, k, is_q6k)."""
    return {"wq": (s.qd, s.hidden, False), "wk": (s.kv, s.hidden, False), "wv": (s.kv, s.hidden, True),
            "wo": (s.hidden, s.qd, False), "wg": (s.inter, s.hidden, False), "wu": (s.inter, s.hidden, False),
            "wd": (s.hidden, s.inter, True)}


def weight_bytes_per_token(s: Shape) -> int:
    per = sum(r * (k // 256) * synth.block_bytes(q6) for r, k, q6 in mat_shapes(s).values())
    return per * s.layers + s.vocab * (s.hidden // 256) * synth.Q6K_BLOCK


def _scaled(gen_rows, k, seed, q6, spread):
    """Blocks whose dequantised rows give y = W x of about unit variance for unit-variance x."""
    w = synth.kquant_blocks(gen_rows, k, seed, q6)
    n = gen_rows * (k // 256)
    rng = np.random.default_rng(seed + 7919)
    blk = w.reshape(n, -1)
    if q6:   # weights ~ d * sc * q, sc in [-32,31], q in [-32,31]: std ~ d * 18.5 * 18.5
        d = (1.0 + spread * rng.uniform(-1, 1, n)) / (342.0 * np.sqrt(k))
        blk[:, 208:210] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    else:    # weights ~ d*sc*q - dmin*m with dmin = 7.5 d: zero mean, std ~ 258 d
        d = (1.0 + spread * rng.uniform(-1, 1, n)) / (258.0 * np.sqrt(k))
        blk[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
        blk[:, 2:4] = (d * 7.5).astype(np.float16).view(np.uint8).reshape(-1, 2)
    return blk.reshape(gen_rows, -1)


def build(s: Shape, seed: int):
    """Returns {"layers": [{"wq": uint8[rows, row_bytes], ..., "attn_norm": f32[hidden], "ffn_norm": ...}],
    "out_norm": f32[hidden], "lm_head": uint8[vocab, row_bytes] (Q6_K)}, deterministic in seed."""
    rng = np.random.default_rng(seed)
    layers = []
    for l in range(s.layers):
        L = {}
        for i, (name, (rows, k, q6)) in enumerate(mat_shapes(s).items()):
            L[name] = _scaled(rows, k, seed * 1000 + l * 16 + i, q6, 0.1)
        L["attn_norm"] = (1.0 + 0.1 * rng.uniform(-1, 1, s.hidden)).astype(np.float32)
        L["ffn_norm"] = (1.0 + 0.1 * rng.uniform(-1, 1, s.hidden)).astype(np.float32)
        if s.qk_norm:
            L["q_norm"] = (1.0 + 0.1 * rng.uniform(-1, 1, s.head_dim)).astype(np.float32)
            L["k_norm"] = (1.0 + 0.1 * rng.uniform(-1, 1, s.head_dim)).astype(np.float32)
        layers.append(L)
    out_norm = (1.0 + 0.1 * rng.uniform(-1, 1, s.hidden)).astype(np.float32)
    lm_head = _scaled(s.vocab, s.hidden, seed * 1000 + 999, True, 0.1)
    return {"layers": layers, "out_norm": out_norm, "lm_head": lm_head}


def digest(model) -> str:
    """sha256 over every weight byte, to detect generator drift against committed goldens."""
    h = hashlib.sha256()
    for L in model["layers"]:
        for name in sorted(L):
            h.update(np.ascontiguousarray(L[name]).tobytes())
    h.update(model["out_norm"].tobytes())
    h.update(np.ascontiguousarray(model["lm_head"]).tobytes())
    return h.hexdigest()
