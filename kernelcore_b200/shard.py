"""Row sharding of K-quant matrices across ranks (one rank per GPU) and the peer-pointer arithmetic of the
fused all-gather.  Pure host logic, shared by the benchmark and the tests."""
from __future__ import annotations


def row_range(rows: int, rank: int, world: int) -> tuple[int, int]:
    """[r0, r1) owned by `rank`: equal contiguous shares; every share a multiple of 8 rows (the kernels' row
    granularity, and the reference's chunk rule llm/llm_kernels.cpp:281-288)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank / world")
    if rows % (8 * world):
        raise ValueError(f"{rows} rows do not split into {world} shares of whole 8-row groups")
    per = rows // world
    return rank * per, (rank + 1) * per


def gather_targets(buffer_ptrs, rank: int, r0: int, itemsize: int = 4):
    """(own pointer, [peer pointers]) of this rank's slice inside every rank's full-length output buffer."""
    off = r0 * itemsize
    return buffer_ptrs[rank] + off, [p + off for i, p in enumerate(buffer_ptrs) if i != rank]
