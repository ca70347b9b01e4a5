"""Decode loop parity (Mode L): llm::decodeToken on the CUDA backend against the logits the reference's
own decodeToken + C++ backend produced (golden) and against the oracle restatement."""
import ctypes as C

import numpy as np
import pytest

from helpers import OracleModel, rel_diff
from kernelcore_b200 import decoder, tiny_model as tm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("graphs", [0, 1])
def test_tiny_model_against_reference_logits(golden, graphs):
    g = golden("decode_tiny")
    shape = tm.tiny()
    model = tm.build(shape, seed=1)
    with decoder.Model(shape, model, graphs=graphs) as m:
        for pos, tok in enumerate(g["tokens"]):
            logits, arg = m.decode(int(tok), pos)
            # the reference's bar for its kernels against its C++ backend (tests/test_llm_kernels.cpp:925-928)
            assert rel_diff(logits, g["logits"][pos]) < 1e-4
            assert arg == int(g["logits"][pos].argmax())


def test_greedy_generation_matches_oracle():
    """Free-running greedy decode: same tokens as the CPU oracle for 12 steps, and bad positions refused."""
    shape = tm.tiny(max_ctx=24)
    model = tm.build(shape, seed=3)
    om = OracleModel(shape, model)
    with decoder.Model(shape, model, graphs=1) as m:
        tok_gpu = tok_cpu = 7
        for pos in range(12):
            lg, arg = m.decode(tok_gpu, pos)
            lc = om.decode_port(om.embed(tok_cpu), pos)
            assert rel_diff(lg, lc) < 1e-4
            tok_gpu, tok_cpu = arg, int(lc.argmax())
            assert tok_gpu == tok_cpu
        with pytest.raises(RuntimeError):
            m.decode(1, shape.max_ctx)          # position outside the KV cache
