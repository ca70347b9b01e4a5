"""Tensor-parallel graph decoder on 2 GPUs (one process per GPU) against the single-GPU decoder.

Skipped on a single-GPU box.  The ranks shard heads, FFN rows and vocabulary rows; the partial hidden vectors of
the K-split attention-output / FFN-down matvecs are summed inside the following norm kernel out of both ranks'
memories.  Only the order of those fp32 additions differs from one GPU, so logits agree to the bound the
single-GPU decoder test states for Q8 re-quantization (3e-2 of max|logit| at every position), and the ranks agree
with each other exactly."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

STEPS, PROMPT = 24, 16


def _shape(which=0):
    from kernelcore_b200 import tiny_model as tm
    if which == 0:   # FFN share 384 = 1.5 super-blocks (a straddled K window), 8 query / 2 kv heads of 64
        return tm.Shape("tp-tiny", 512, 768, 2, 8, 2, 64, 512, 48)
    if which == 1:   # attention-output share 384 channels as well (12 heads of 64 over 2 ranks): both K windows straddle a super-block
        return tm.Shape("tp-straddle", 768, 768, 2, 12, 4, 64, 512, 48)
    # every share a whole number of super-blocks (256 attention channels, 512 FFN rows per rank): the batched prompt pass runs too
    return tm.Shape("tp-aligned", 512, 1024, 2, 8, 2, 64, 512, 48)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, which, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    from kernelcore_b200 import decoder, lib, tiny_model as tm
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    shape = _shape(which)
    model = tm.build(shape, seed=11)
    area = symm_mem.empty(decoder.FastDecoder.tp_shared_bytes(shape), dtype=torch.uint8, device=dev)
    area.zero_()
    handle = symm_mem.rendezvous(area, dist.group.WORLD.group_name)
    torch.cuda.synchronize()
    dist.barrier()
    prompt = [int(t) for t in np.random.default_rng(2).integers(0, shape.vocab, PROMPT)]
    with decoder.FastDecoder(shape, model, tp=(rank, world, list(handle.buffer_ptrs))) as dec:
        dec.set_prompt(prompt)
        dist.barrier()
        per_step = []
        for _ in range(STEPS):
            dec.run(1)
            logits, _, _ = dec.read(0)
            r0, r1 = dec.local_rows()
            per_step.append(logits[r0:r1].copy())
        _, hist, pos = dec.read(STEPS)
        # the batched prompt pass under tensor parallelism, then two more steps through the graph on top of its cache
        dist.barrier()
        batched = None
        try:
            dec.prefill(prompt)
            logits, _, ppos = dec.read(0)
            r0, r1 = dec.local_rows()
            first = logits[r0:r1].copy()
            dec.run(2)
            _, hist2, ppos2 = dec.read(PROMPT + 2)
            # a batch of three sequences in lockstep: prompts, then four steps
            seqs = [[int(t) for t in np.random.default_rng(30 + i).integers(0, shape.vocab, 8)] for i in range(3)]
            dec.batch_begin(3)
            for i, sq in enumerate(seqs):
                dec.batch_prefill(i, sq)
            first_rows = [dec.batch_read(i)[0][:r1 - r0].copy() for i in range(3)]
            dec.batch_run(4)
            hists = [dec.batch_read(i, 12)[1].copy() for i in range(3)]
            batched = (first, (ppos, ppos2), hist2.copy(), np.stack(first_rows), np.stack(hists))
        except lib.KcbError as e:      # shares that straddle a super-block: refused on every rank alike, before any launch
            batched = str(e)
        out[rank] = (np.stack(per_step), hist.copy(), pos, decoder.FastDecoder.tp_timeouts(), batched)
        dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("which", [0, 1, 2])
def test_two_rank_decoder_matches_single_gpu(which):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    sys.path.insert(0, ROOT)
    from helpers import rel_diff
    from kernelcore_b200 import decoder, tiny_model as tm
    world = 2
    with mp.Manager() as man:
        out = man.dict()
        mp.spawn(_worker, args=(world, _free_port(), which, out), nprocs=world, join=True)
        res = dict(out)
    assert res[0][3] == 0 and res[1][3] == 0                      # no wait gave up
    assert res[0][2] == res[1][2] == STEPS
    assert np.array_equal(res[0][1], res[1][1])                   # both ranks picked the same tokens
    tp_logits = np.concatenate([res[0][0], res[1][0]], axis=1)   # [steps][vocab]
    shape = _shape(which)
    model = tm.build(shape, seed=11)
    prompt = [int(t) for t in np.random.default_rng(2).integers(0, shape.vocab, PROMPT)]
    # one GPU, forced to the tokens the two-rank run consumed, so every step sees the same inputs
    consumed = prompt + [int(t) for t in res[0][1][PROMPT - 1:STEPS - 1]]
    with decoder.FastDecoder(shape, model) as dec:
        dec.set_prompt(consumed[:STEPS])
        errs = []
        for s in range(STEPS):
            dec.run(1)
            logits, _, _ = dec.read(0)
            errs.append(rel_diff(tp_logits[s], logits))
    assert max(errs) < 3e-2, errs
    assert errs[0] < 1e-4, errs
    # the batched prompt pass under tensor parallelism
    if which != 2:
        assert isinstance(res[0][4], str) and "super-blocks" in res[0][4] and isinstance(res[1][4], str)
        return
    (f0, pos0, h0, b0, bh0), (f1, pos1, h1, b1, bh1) = res[0][4], res[1][4]
    assert pos0 == pos1 == (PROMPT, PROMPT + 2)
    assert np.array_equal(h0, h1)                                 # the ranks went on with the same tokens
    with decoder.FastDecoder(shape, model) as dec:
        dec.prefill(prompt)
        assert rel_diff(np.concatenate([f0, f1]), dec.read(0)[0]) < 3e-2
    assert res[0][3] == 0 and res[1][3] == 0
    # the batch of sequences: ranks picked the same tokens for every sequence; logits after the prompts match one GPU
    assert np.array_equal(bh0, bh1) and (bh0[:, 8:12] >= 0).all() and (bh0[:, 8:12] < shape.vocab).all()
    seqs = [[int(t) for t in np.random.default_rng(30 + i).integers(0, shape.vocab, 8)] for i in range(3)]
    with decoder.FastDecoder(shape, model) as dec:
        dec.batch_begin(3)
        for i, sq in enumerate(seqs):
            dec.batch_prefill(i, sq)
        for i in range(3):
            assert rel_diff(np.concatenate([b0[i], b1[i]]), dec.batch_read(i)[0]) < 3e-2, i
