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


def head_shares(heads: int, kv_heads: int, rank: int, world: int) -> tuple[range, range]:
    """Query heads and kv heads of `rank`: contiguous, whole query groups stay with their kv head."""
    if kv_heads % world or heads % kv_heads:
        raise ValueError(f"{kv_heads} kv heads do not split over {world} ranks")
    hq, hk = heads // world, kv_heads // world
    return range(rank * hq, (rank + 1) * hq), range(rank * hk, (rank + 1) * hk)


def k_window(first_channel: int, channels: int) -> tuple[int, int, int]:
    """(first super-block, super-blocks, first Q8 block inside the window) of the whole 256-weight super-blocks
    that cover input channels [first_channel, first_channel + channels) of a K-split matrix.  A share that is
    not a multiple of 256 (Llama-3.2-3B attention output at 8 ranks: 384 channels) reads the straddled
    super-block on both neighbours; the channels a rank does not own enter as zero Q8 blocks."""
    if first_channel % 32 or channels % 32 or channels <= 0:
        raise ValueError("shares are whole 32-channel Q8 blocks")
    sb0 = first_channel // 256
    nsb = (first_channel + channels + 255) // 256 - sb0
    return sb0, nsb, (first_channel - sb0 * 256) // 32


def k_slice_blocks(blocks, rows: int, k: int, block_bytes: int, sb0: int, nsb: int):
    """Columns [sb0*256, (sb0+nsb)*256) of every row of a row-major GGUF block array (numpy uint8)."""
    return blocks.reshape(rows, k // 256, block_bytes)[:, sb0:sb0 + nsb].reshape(-1).copy()
