"""The row-sharded lm_head matvec with its all-gather fused in (kcb_matvec_q6k_f32x_sharded, world 2) on two GPUs
against the oracle: each rank multiplies its half of the rows and stores the results into both ranks' logits through
peer mappings; after the kernel's own step barrier every rank holds the full vector.  Skipped on a single-GPU box."""
import ctypes as C
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

ROWS, K, STEPS = 16032 * 2, 3072, 5


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    from kernelcore_b200 import kquant, lib, shard, synth
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    r0, r1 = shard.row_range(ROWS, rank, world)
    blocks = synth.q6k_blocks(ROWS, K, 3)                         # the same matrix on every rank; each keeps its rows
    mine = kquant.KMatrix(blocks[r0:r1], r1 - r0, K, True)
    y = symm_mem.empty(ROWS, dtype=torch.float32, device=dev)
    flags = symm_mem.empty(64, dtype=torch.int32, device=dev)
    flags.zero_()
    hy = symm_mem.rendezvous(y, dist.group.WORLD.group_name)
    hf = symm_mem.rendezvous(flags, dist.group.WORLD.group_name)
    own, peers = shard.gather_targets(list(hy.buffer_ptrs), rank, r0)
    peer_tab = (C.c_void_p * len(peers))(*peers)
    flag_tab = (C.c_void_p * world)(*list(hf.buffer_ptrs))
    counters = torch.zeros(2, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    dist.barrier()
    got = []
    for step in range(STEPS):                                     # a new x every step: a stale gather would show
        x = torch.from_numpy(synth.activations(K, 50 + step)).to(dev)
        y.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()                                            # nobody's rows land before the peer's fill
        lib.call("matvec_q6k_f32x_sharded", mine.data, x, C.c_void_p(own), peer_tab, len(peers), flag_tab, counters, rank, world,
                 r1 - r0, K, None, None)
        torch.cuda.synchronize()
        got.append(y.cpu().numpy().copy())                        # after the kernel's barrier: the whole vector, on this rank
        dist.barrier()
    out[rank] = (np.stack(got), int(lib.raw.kcb_peer_timeouts()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gather_against_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    sys.path.insert(0, ROOT)
    import oracle
    from helpers import rel_diff
    from kernelcore_b200 import synth
    with mp.Manager() as man:
        out = man.dict()
        mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
        res = dict(out)
    assert res[0][1] == 0 and res[1][1] == 0                      # no wait gave up
    assert np.array_equal(res[0][0], res[1][0])                   # both ranks hold the same bits
    blocks = synth.q6k_blocks(ROWS, K, 3)
    for step in range(STEPS):
        want = oracle.matvec_q8(oracle.port, blocks, synth.activations(K, 50 + step), ROWS, K, 1)
        assert rel_diff(res[0][0][step], want) < 1e-5, step
