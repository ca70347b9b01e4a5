"""The single-launch fp32-x matvec (in-kernel Q8 quantization) against the two-launch path and the oracle."""
import numpy as np
import pytest
import torch

import oracle
from helpers import rel_diff
from kernelcore_b200 import kquant, lib, synth

pytestmark = pytest.mark.gpu


def test_single_launch_matvec_equals_two_launch_path():
    for rows, k in ((16032, 3072), (8192, 1024), (4736, 4096)):
        w = synth.q6k_blocks(rows, k, rows)
        m = kquant.KMatrix(w, rows, k, True)
        x = torch.from_numpy(synth.activations(k, 9)).cuda()
        want = kquant.matvec(m, x, kquant.Q8Scratch(k)).clone()
        got = torch.full((rows,), float("nan"), device="cuda")
        lib.call("matvec_q6k_f32x_sharded", m.data, x, got, None, 0, None, None, 0, 1, rows, k, None, None)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert rel_diff(got.cpu().numpy(), oracle.matvec_q8(oracle.port, w, x.cpu().numpy(), rows, k, 1)) < 1e-5
    assert lib.raw.kcb_tma_timeouts() == 0


def test_host_buffer_pipe_equals_device_path():
    """kcb_host_matvec_*: pinned host x in, host y out, two slots in flight; every result equals the device-side call."""
    import ctypes as C
    rows, k = 16032, 3072
    mats = [kquant.KMatrix(synth.q6k_blocks(rows, k, s), rows, k, True) for s in (1, 2, 3)]
    xs = [torch.from_numpy(synth.activations(k, 20 + i)).pin_memory() for i in range(7)]
    ys = [torch.full((rows,), float("nan")).pin_memory() for _ in range(7)]
    pipe = C.c_void_p()
    assert lib.raw.kcb_host_matvec_create(rows, k, C.byref(pipe)) == 0
    for i in range(7):
        assert lib.raw.kcb_host_matvec_submit(pipe, C.c_void_p(mats[i % 3].data.data_ptr()), C.c_void_p(xs[i].data_ptr()), C.c_void_p(ys[i].data_ptr())) == 0
    assert lib.raw.kcb_host_matvec_sync(pipe) == 0
    for i in range(7):
        want = torch.empty(rows, device="cuda")
        lib.call("matvec_q6k_f32x_sharded", mats[i % 3].data, xs[i].cuda(), want, None, 0, None, None, 0, 1, rows, k, None, None)
        torch.cuda.synchronize()
        assert torch.equal(ys[i], want.cpu()), i
    assert lib.raw.kcb_host_matvec_create(rows + 1, k, C.byref(C.c_void_p())) == 2      # rows % 8
    lib.raw.kcb_host_matvec_destroy(pipe)
