"""Device-resident K-quant matrices and the decode matvec, over the C ABI."""
from __future__ import annotations

import numpy as np
import torch

from . import lib


class KMatrix:
    """A Q4_K or Q6_K weight matrix in device memory in the layout the kernels stream:
    Q4_K as GGUF blocks, Q6_K as planes.  Built from canonical GGUF block bytes."""

    def __init__(self, blocks, rows: int, k: int, q6: bool, device="cuda"):
        assert k % 256 == 0
        self.rows, self.k, self.q6 = rows, k, bool(q6)
        nbytes = lib.raw.kcb_kquant_bytes(rows, k, int(q6))
        if isinstance(blocks, np.ndarray):
            blocks = torch.from_numpy(np.ascontiguousarray(blocks).reshape(-1))
        assert blocks.dtype == torch.uint8 and blocks.numel() == nbytes, (blocks.numel(), nbytes)
        src = blocks.to(device, non_blocking=False).contiguous()
        if self.q6:
            self.data = torch.empty_like(src)
            lib.call("q6k_to_planes", src, self.data, rows, k)
        else:
            self.data = src

    @property
    def nbytes(self) -> int:
        return self.data.numel()

    def gguf_bytes(self) -> torch.Tensor:
        """Canonical GGUF block bytes (device uint8)."""
        if not self.q6:
            return self.data
        out = torch.empty_like(self.data)
        lib.call("q6k_from_planes", self.data, out, self.rows, self.k)
        return out

    def dequant(self) -> torch.Tensor:
        out = torch.empty((self.rows, self.k), dtype=torch.float32, device=self.data.device)
        lib.call("dequant_q6k" if self.q6 else "dequant_q4k", self.data, out, self.rows, self.k)
        return out


class Q8Scratch:
    """The reference's 8-bit activation scratch for vectors up to max_k values: one int buffer
    [nb*8 words | nb*2 floats {scale, sum} | nb floats] (llm/llm_kernels.hpp:82-85)."""

    def __init__(self, max_k: int, device="cuda"):
        self.max_k = max_k
        self.buf = torch.zeros(11 * (max_k // 32), dtype=torch.int32, device=device)

    def views(self, k: int):
        nb = k // 32
        return self.buf[: nb * 8], self.buf[nb * 8: nb * 10].view(torch.float32)


def quantize_q8x4(x: torch.Tensor, scratch: Q8Scratch):
    k = x.numel()
    xq, xd = scratch.views(k)
    lib.call("quantize_q8x4", x, xq, xd, k // 32)
    return xq, xd


def matvec_q8(w: KMatrix, xq: torch.Tensor, xd: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    lib.call("matvec_q6k_q8" if w.q6 else "matvec_q4k_q8", w.data, xq, xd, y, w.rows, w.k)
    return y


def matvec(w: KMatrix, x: torch.Tensor, scratch: Q8Scratch, y: torch.Tensor | None = None) -> torch.Tensor:
    """The reference's Backend::matvec for K-quant weights (llm/llm_model.cpp:385-397): quantize x
    per 32 into the scratch, then the integer-dot matvec."""
    if y is None:
        y = torch.empty(w.rows, dtype=torch.float32, device=x.device)
    xq, xd = quantize_q8x4(x, scratch)
    return matvec_q8(w, xq, xd, y)


def matvec_f32(w: KMatrix, x: torch.Tensor, y: torch.Tensor | None = None) -> torch.Tensor:
    if y is None:
        y = torch.empty(w.rows, dtype=torch.float32, device=x.device)
    lib.call("matvec_q6k_f32" if w.q6 else "matvec_q4k_f32", w.data, x, y, w.rows, w.k)
    return y
