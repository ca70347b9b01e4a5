"""Row-sharded matvec across 2 ranks on CPU (gloo): each rank runs the oracle on its shard, the shards are
all-gathered, and the result equals the unsharded oracle bit for bit -- the host-side contract of the
multi-GPU benchmark path (shard ranges, gather offsets), without a GPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, k, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    from kernelcore_b200 import shard, synth
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w = synth.q6k_blocks(rows, k, 3)          # every rank regenerates the same seeded matrix
    x = synth.activations(k, 4)
    r0, r1 = shard.row_range(rows, rank, world)
    y_local = torch.from_numpy(oracle.matvec_q8(oracle.port, w[r0:r1], x, r1 - r0, k, 1))
    y_full = torch.empty(rows, dtype=torch.float32)
    dist.all_gather_into_tensor(y_full, y_local)
    want = oracle.matvec_q8(oracle.port, w, x, rows, k, 1)
    ok = bool((y_full.numpy().view(np.uint32) == want.view(np.uint32)).all())
    own, peers = shard.gather_targets([1000, 5000], rank, r0)
    ok = ok and own == [1000, 5000][rank] + 4 * r0 and peers == [[5000, 1000][rank] + 4 * r0]
    out[rank] = ok
    dist.destroy_process_group()


def test_two_rank_row_sharding_matches_unsharded():
    world, rows, k = 2, 64, 512
    with mp.Manager() as man:
        out = man.dict()
        mp.spawn(_worker, args=(world, _free_port(), rows, k, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_row_range_rules():
    sys.path.insert(0, ROOT)
    from kernelcore_b200 import shard
    assert [shard.row_range(128256, r, 8) for r in (0, 7)] == [(0, 16032), (112224, 128256)]
    with pytest.raises(ValueError):
        shard.row_range(100, 0, 8)
    with pytest.raises(ValueError):
        shard.row_range(128, 2, 2)


def _ksplit_worker(rank, world, port, rows, k, q6, out):
    """K-split of one matrix (the attention-output / FFN-down split of tensor-parallel decode): every rank runs
    the oracle on its window of whole super-blocks with the channels it does not own zeroed, the partial vectors
    are gathered and added in rank order on every rank."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    from kernelcore_b200 import shard, synth
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w = synth.q6k_blocks(rows, k, 5) if q6 else synth.q4k_blocks(rows, k, 5)
    x = synth.activations(k, 6)
    share = k // world
    sb0, nsb, first = shard.k_window(rank * share, share)
    win = shard.k_slice_blocks(w, rows, k, 210 if q6 else 144, sb0, nsb)
    xw = np.zeros(nsb * 256, np.float32)
    xw[first * 32:first * 32 + share] = x[rank * share:(rank + 1) * share]
    part = torch.from_numpy(oracle.matvec_q8(oracle.port, win, xw, rows, nsb * 256, q6))
    parts = [torch.empty(rows, dtype=torch.float32) for _ in range(world)]
    dist.all_gather(parts, part)
    total = parts[0].clone()
    for p in parts[1:]:
        total += p
    want = oracle.matvec_q8(oracle.port, w, x, rows, k, q6)
    err = float(np.abs(total.numpy() - want).max() / np.abs(want).max())
    out[rank] = (err, total.numpy().tobytes())
    dist.destroy_process_group()


@pytest.mark.parametrize("q6", [0, 1])
def test_two_rank_k_split_with_straddled_super_block(q6):
    world, rows, k = 2, 40, 768          # shares of 384 channels: 1.5 super-blocks each, block 1 read by both
    with mp.Manager() as man:
        out = man.dict()
        mp.spawn(_ksplit_worker, args=(world, _free_port(), rows, k, q6, out), nprocs=world, join=True)
        res = dict(out)
    assert res[0][0] < 2e-6 and res[1][0] < 2e-6       # same products, only the order of fp32 additions differs
    assert res[0][1] == res[1][1]                      # every rank holds the same bits


def test_head_shares_and_k_windows():
    sys.path.insert(0, ROOT)
    from kernelcore_b200 import shard
    q, kv = shard.head_shares(24, 8, 5, 8)
    assert list(q) == [15, 16, 17] and list(kv) == [5]
    assert shard.k_window(5 * 384, 384) == (7, 2, 4)    # channels 1920..2303: super-blocks 7-8, from Q8 block 4
    assert shard.k_window(2 * 1024, 1024) == (8, 4, 0)
    with pytest.raises(ValueError):
        shard.head_shares(24, 8, 0, 3)
    with pytest.raises(ValueError):
        shard.k_window(100, 384)
