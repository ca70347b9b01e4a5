"""Failure paths that really run: a cross-GPU wait that nothing answers, and the runtime's sticky fault state.

No kernel faults, traps or is left waiting here.  The waits are the library's own bounded polls with the limit turned
down (the default is about a second per wait); what stands in for the absent peer is a zeroed flag array in this
GPU's own memory.  The runtime's fault is an error code planted on the host.  The reference's counterparts, which
kill worker threads and inject traps, are tests/test_fault.cpp:17-137."""
import ctypes as C
import time

import numpy as np
import pytest
import torch

from kernelcore_b200 import decoder, lib, tiny_model as tm

pytestmark = pytest.mark.gpu
L = lib.raw
L.kcb_last_error_detail.restype = C.c_char_p
KERNEL_FAULT, CONTEXT_POISONED = 12, 13
CUDA_ERROR_LAUNCH_FAILURE = 719


def _flag_table(*arrays):
    table = (C.c_void_p * len(arrays))(*[a.data_ptr() for a in arrays])
    return C.cast(table, C.POINTER(C.c_void_p))


def test_step_barrier_gives_up_on_an_absent_peer_and_then_fails_fast():
    mine, peers = torch.zeros(2, dtype=torch.int32, device="cuda"), torch.zeros(2, dtype=torch.int32, device="cuda")
    flags = _flag_table(mine, peers)          # rank 0 = this GPU; "rank 1" never runs
    assert L.kcb_peer_reset() == 0 and L.kcb_peer_set_poll_limit(2000) == 0
    try:
        before = L.kcb_peer_timeouts()
        assert L.kcb_peer_barrier(flags, 0, 2, 1, None) == 0
        torch.cuda.synchronize()                                 # the kernel returned by itself
        assert L.kcb_peer_timeouts() == before + 1
        assert peers.tolist() == [1, 0] and mine.tolist() == [1, 0]     # it announced itself to both, heard from nobody
        # the group is now marked broken: the next barrier polls once, even with a long limit
        assert L.kcb_peer_set_poll_limit(1 << 30) == 0
        t0 = time.perf_counter()
        assert L.kcb_peer_barrier(flags, 0, 2, 2, None) == 0
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 0.5
        assert L.kcb_peer_timeouts() == before + 2
        # the host deals with it (here: the peer's flag arrives) and clears the mark; barriers work again
        mine[1] = 3
        assert L.kcb_peer_reset() == 0 and L.kcb_peer_set_poll_limit(2000) == 0
        assert L.kcb_peer_barrier(flags, 0, 2, 3, None) == 0
        torch.cuda.synchronize()
        assert L.kcb_peer_timeouts() == 0
        # and the context is intact: ordinary work runs
        assert float((torch.ones(1024, device="cuda") * 2).sum()) == 2048.0
    finally:
        L.kcb_peer_reset()
        L.kcb_peer_set_poll_limit(0)


def test_tensor_parallel_exchange_gives_up_on_an_absent_rank():
    """Rank 0 of a two-rank decoder whose rank 1 does not exist: each exchange of the step (two per layer and the pick)
    waits for a partial sum that never comes.  The first wait runs out its (shortened) limit, the rest poll once; the
    step ends, the expiry is counted, the handle closes cleanly and a single-GPU decoder works afterwards."""
    shape = tm.Shape("tp-tiny", 512, 768, 2, 8, 2, 64, 512, 48)
    model = tm.build(shape, seed=11)
    nbytes = decoder.FastDecoder.tp_shared_bytes(shape)
    areas = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    assert L.kcb_decoder_tp_reset() == 0 and L.kcb_decoder_tp_set_poll_limit(2000) == 0
    try:
        with decoder.FastDecoder(shape, model, tp=(0, 2, [a.data_ptr() for a in areas])) as d:
            assert decoder.FastDecoder.tp_timeouts() == 0        # creation exchanges with nobody
            d.set_prompt([1, 2, 3])
            t0 = time.perf_counter()
            d.run(1)
            d.sync()
            assert time.perf_counter() - t0 < 2.0
            assert decoder.FastDecoder.tp_timeouts() >= 1
            _, _, pos = d.read(want_logits=False)
            assert pos == 1                                      # the step ran to its end
        assert L.kcb_decoder_tp_reset() == 0
        assert decoder.FastDecoder.tp_timeouts() == 0
        small = tm.tiny(max_ctx=8)
        with decoder.FastDecoder(small, tm.build(small, seed=1)) as d:
            d.set_prompt([5])
            d.run(1)
            assert np.isfinite(d.read()[0]).all()
    finally:
        L.kcb_decoder_tp_reset()
        L.kcb_decoder_tp_set_poll_limit(0)


def test_fault_poisons_the_context_until_device_reset():
    """kc runtime error model: a device-side failure surfaces as KernelFault from the call that observes it, every later
    call on the device answers ContextPoisoned, kcGetLastFault describes it, kcDeviceReset clears the state and work
    resumes.  The failure is a CUDA error code planted on the host (kcb_test_inject_device_error); no kernel fails."""
    assert L.kcb_init() == 0
    try:
        p = C.c_void_p()
        assert L.kcb_malloc(C.byref(p), C.c_size_t(4096)) == 0
        assert L.kcb_memset(p, 0, C.c_size_t(4096)) == 0
        assert L.kcb_test_inject_device_error(CUDA_ERROR_LAUNCH_FAILURE) == 0
        assert L.kcb_device_synchronize() == KERNEL_FAULT
        assert b"cudaErrorLaunchFailure" in L.kcb_last_error_detail()
        fault = (C.c_uint8 * 512)()
        assert L.kcb_get_last_fault(fault) == 0
        assert int.from_bytes(bytes(fault[:4]), "little") == CUDA_ERROR_LAUNCH_FAILURE      # kc::FaultInfo::code
        q = C.c_void_p()
        for status in (L.kcb_device_synchronize(), L.kcb_malloc(C.byref(q), C.c_size_t(64)), L.kcb_memset(p, 0, C.c_size_t(64))):
            assert status == CONTEXT_POISONED
        assert b"kcDeviceReset" in L.kcb_last_error_detail()
        assert L.kcb_device_reset() == 0
        assert L.kcb_check_range(p, C.c_size_t(4)) == 5          # the reset released the old allocation
        host = np.arange(256, dtype=np.float32)
        assert L.kcb_malloc(C.byref(p), C.c_size_t(host.nbytes)) == 0
        assert L.kcb_memcpy(p, host.ctypes.data_as(C.c_void_p), C.c_size_t(host.nbytes), 0) == 0
        back = np.zeros_like(host)
        assert L.kcb_memcpy(back.ctypes.data_as(C.c_void_p), p, C.c_size_t(host.nbytes), 1) == 0
        assert (back == host).all() and L.kcb_device_synchronize() == 0
    finally:
        L.kcb_device_reset()
        assert L.kcb_shutdown() == 0
