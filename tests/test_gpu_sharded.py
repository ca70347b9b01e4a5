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
