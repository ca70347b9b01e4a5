"""The allocation-free Q4_K matvec (kcb_matvec_q4k_f32x_static) against the ordinary two-call path.

Collected last on purpose (file name), so a stop-at-first-failure run has already exercised everything else.
The entry point keeps its activation scratch in a device array inside the library for callers that cannot
allocate at call time; here it must give the same y as kcb_quantize_q8x4 + kcb_matvec_q4k_q8 with a caller
scratch, on two calls in a row that reuse the shared array with different inputs and sizes."""
import numpy as np
import pytest
import torch

import oracle
from helpers import rel_diff
from kernelcore_b200 import kquant, lib, synth

pytestmark = pytest.mark.gpu


def test_static_scratch_matvec_matches_two_call_path_twice():
    max_k = lib.raw.kcb_static_scratch_max_k()
    assert max_k == 16384
    # two consecutive calls: a large k first, then a smaller one that leaves stale words in the shared array
    for call, (rows, k) in enumerate([(8192, 3072), (2048, 1024)]):
        w = kquant.KMatrix(synth.q4k_blocks(rows, k, 40 + call), rows, k, False)
        x = torch.from_numpy(synth.activations(k, 50 + call)).cuda()
        want = kquant.matvec(w, x, kquant.Q8Scratch(k)).clone()
        got = torch.full((rows,), float("nan"), device="cuda")
        lib.call("matvec_q4k_f32x_static", w.data, x, got, rows, k)
        torch.cuda.synchronize()
        assert rel_diff(got.cpu().numpy(), want.cpu().numpy()) < 1e-5
        assert torch.equal(got, want)  # same kernels on the same words: in fact identical
        # and against the CPU oracle's Q8 arithmetic on the same blocks and activations (the bar of the other matvec tests)
        ref = oracle.matvec_q8(oracle.port, synth.q4k_blocks(rows, k, 40 + call), x.cpu().numpy(), rows, k, 0)
        assert rel_diff(got.cpu().numpy(), ref) < 1e-5
        if call == 0:
            # the first call on a device also loads the module and looks up the array's address; from the second call on
            # the entry point must leave the device's free memory untouched
            free_before = torch.cuda.mem_get_info()[0]
        else:
            assert torch.cuda.mem_get_info()[0] == free_before
    # sizes beyond the built-in scratch are refused up front, nothing is launched
    y = torch.zeros(8, device="cuda")
    big = torch.zeros(max_k + 256, device="cuda")
    wbig = torch.zeros(8 * (max_k + 256) // 256 * 144, dtype=torch.uint8, device="cuda")
    assert lib.call("matvec_q4k_f32x_static", wbig, big, y, 8, max_k + 256, raise_on_error=False) == 2
    assert lib.call("matvec_q4k_f32x_static", wbig, big, y, 8, 100, raise_on_error=False) == 2
