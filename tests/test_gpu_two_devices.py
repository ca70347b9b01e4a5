"""Two GPUs driven from ONE process: the per-device bookkeeping of the launchers (one cudaFuncSetAttribute per kernel and
device for the launches that need more than 48 KB of shared memory, the cached occupancy answers, the allocation-free
entry's per-device scratch address).  Every kernel family that carries such state runs on device 1 first and then on
device 0, and both results are checked against the oracle.  Skipped on a single-GPU box."""
import numpy as np
import pytest
import torch

import oracle
from helpers import rel_diff
from kernelcore_b200 import kquant, lib, synth

pytestmark = pytest.mark.gpu


def _run_on(device):
    torch.cuda.set_device(device)
    dev = torch.device("cuda", device)
    out = {}
    # the bulk-copy streaming matvec (226 KB of dynamic shared memory), Q6_K and Q4_K, above the 64 MB route limit
    for q6, rows, k in ((True, 84000, 1024), (False, 124000, 1024)):
        w = synth.kquant_blocks(rows, k, 3, q6)
        x = synth.activations(k, 4)
        m = kquant.KMatrix(w, rows, k, q6)
        assert m.data.device == dev
        y = kquant.matvec(m, torch.from_numpy(x).to(dev), kquant.Q8Scratch(k)).cpu().numpy()
        out[f"stream_q{6 if q6 else 4}"] = rel_diff(y, oracle.matvec_q8(oracle.port, w, x, rows, k, q6))
    # the decode matvec kernel (224 KB ring) through the plain entry point
    rows, k = 4096, 3072
    w = synth.kquant_blocks(rows, k, 5, False)
    x = synth.activations(k, 6)
    y = kquant.matvec(kquant.KMatrix(w, rows, k, False), torch.from_numpy(x).to(dev), kquant.Q8Scratch(k)).cpu().numpy()
    out["decode_matvec"] = rel_diff(y, oracle.matvec_q8(oracle.port, w, x, rows, k, False))
    # the tensor-core matmul (tensor maps, > 48 KB of shared memory), bit for bit
    rows, k, ncols = 256, 1024, 128
    w = synth.kquant_blocks(rows, k, 7, False)
    X = np.random.default_rng(8).standard_normal((ncols, k)).astype(np.float32)
    m = kquant.KMatrix(w, rows, k, False)
    slots = torch.zeros((ncols, 85 * k // 256), dtype=torch.int32, device=dev)
    Y = torch.empty((ncols, rows), device=dev)
    lib.call("quantize_cols_k", torch.from_numpy(X).to(dev), slots, k, ncols)
    lib.call("matmul_kq_q8", m.data, slots, Y, rows, k, ncols, 0, 1)
    Y = Y.cpu().numpy()
    out["matmul_bits"] = all((Y[c].view(np.uint32) == oracle.matvec_q8k(oracle.port, w, X[c], rows, k, 0).view(np.uint32)).all() for c in (0, 77, 127))
    # the allocation-free entry point: its scratch address is per device
    rows, k = 512, 1024
    w = synth.kquant_blocks(rows, k, 9, False)
    x = synth.activations(k, 10)
    m = kquant.KMatrix(w, rows, k, False)
    y = torch.empty(rows, device=dev)
    lib.call("matvec_q4k_f32x_static", m.data, torch.from_numpy(x).to(dev), y, rows, k)
    out["static"] = rel_diff(y.cpu().numpy(), oracle.matvec_q8(oracle.port, w, x, rows, k, False))
    torch.cuda.synchronize(dev)
    return out


def test_every_stateful_launcher_on_both_devices_of_one_process():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    try:
        for device in (1, 0, 1):
            got = _run_on(device)
            assert got.pop("matmul_bits"), device
            assert all(v < 1e-5 for v in got.values()), (device, got)
        assert lib.raw.kcb_tma_timeouts() == 0 and lib.raw.kcb_tc_timeouts() == 0
    finally:
        torch.cuda.set_device(0)
