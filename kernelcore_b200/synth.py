"""Seeded synthetic GGUF K-quant data with the value distributions the benchmark
configurations name.  Pure numpy; shared by the tests and the benchmark drivers."""
from __future__ import annotations

import numpy as np

Q4K_BLOCK = 144  # fp16 d, fp16 dmin, 12 B packed 6-bit scales/mins, 128 B nibbles
Q6K_BLOCK = 210  # 128 B low nibbles, 64 B high 2-bit pairs, 16 int8 scales, fp16 d


def block_bytes(q6: bool) -> int:
    return Q6K_BLOCK if q6 else Q4K_BLOCK


def _f16_bytes(values: np.ndarray) -> np.ndarray:
    return values.astype(np.float16).view(np.uint8).reshape(-1, 2)


def q4k_blocks(rows: int, k: int, seed: int) -> np.ndarray:
    """rows x (k/256) Q4_K super-blocks as uint8[rows, k/256*144].

    d = fp16(|N(0,1)| * 0.01), dmin = fp16(|N(0,1)| * 0.005); the twelve scale bytes are
    uniform random, which makes every unpacked 6-bit scale and min uniform in [0, 63]; the 128
    quant bytes are uniform random nibbles."""
    assert k % 256 == 0
    rng = np.random.default_rng(seed)
    n = rows * (k // 256)
    blk = rng.integers(0, 256, size=(n, Q4K_BLOCK), dtype=np.uint8)
    blk[:, 0:2] = _f16_bytes(np.abs(rng.standard_normal(n)) * 0.01)
    blk[:, 2:4] = _f16_bytes(np.abs(rng.standard_normal(n)) * 0.005)
    return blk.reshape(rows, -1)


def q6k_blocks(rows: int, k: int, seed: int) -> np.ndarray:
    """rows x (k/256) Q6_K super-blocks as uint8[rows, k/256*210].

    ql and qh uniform random, sixteen int8 sub-block scales uniform in [-32, 31],
    d = fp16(|N(0,1)| * 0.002)."""
    assert k % 256 == 0
    rng = np.random.default_rng(seed)
    n = rows * (k // 256)
    blk = rng.integers(0, 256, size=(n, Q6K_BLOCK), dtype=np.uint8)
    blk[:, 192:208] = rng.integers(-32, 32, size=(n, 16), dtype=np.int8).view(np.uint8)
    blk[:, 208:210] = _f16_bytes(np.abs(rng.standard_normal(n)) * 0.002)
    return blk.reshape(rows, -1)


def kquant_blocks(rows: int, k: int, seed: int, q6: bool) -> np.ndarray:
    return q6k_blocks(rows, k, seed) if q6 else q4k_blocks(rows, k, seed)


def raw_blocks(rows: int, k: int, seed: int, q6: bool) -> np.ndarray:
    """Every byte random except the fp16 scales, which are positive in [2^-9, 2^-6)
    (bit patterns 0x1800 + r % 0x0C00) -- the distribution of the reference's own K-quant
    test (tests/test_llm_kernels.cpp:208-221).  Exercises all 8 bits of the Q6_K scales."""
    rng = np.random.default_rng(seed)
    bb = block_bytes(q6)
    n = rows * (k // 256)
    blk = rng.integers(0, 256, size=(n, bb), dtype=np.uint8)

    def half(col):
        h = (0x1800 + rng.integers(0, 0x0C00, size=n)).astype(np.uint16)
        blk[:, col] = (h & 0xFF).astype(np.uint8)
        blk[:, col + 1] = (h >> 8).astype(np.uint8)

    if q6:
        half(208)
    else:
        half(0)
        half(2)
    return blk.reshape(rows, -1)


def activations(k: int, seed: int, scale: float = 1.0) -> np.ndarray:
    return (np.random.default_rng(seed).standard_normal(k) * scale).astype(np.float32)
