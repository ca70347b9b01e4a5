"""ctypes binding of libkernelcore_b200.so (the C ABI in include/kernelcore_b200.h).

There is no fallback: if the shared library is missing or a call fails, an exception is raised."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkernelcore_b200.so")


class KcbError(RuntimeError):
    def __init__(self, what: str, status: int, text: str):
        super().__init__(f"{what}: status {status} ({text})")
        self.status = status


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C kernelcore_b200/csrc` (or __graft_entry__.build()); "
            "there is no CPU or PyTorch fallback for these kernels")
    return C.CDLL(LIB_PATH)


_lib = _load()
_lib.kcb_error_string.restype = C.c_char_p
_lib.kcb_error_string.argtypes = [C.c_int]
_lib.kcb_build_arch.restype = C.c_char_p
_lib.kcb_kquant_bytes.restype = C.c_size_t
_lib.kcb_kquant_bytes.argtypes = [C.c_int, C.c_int, C.c_int]

raw = _lib  # direct access for tests that check symbols / error codes


def check(status: int, what: str) -> None:
    if status != 0:
        raise KcbError(what, status, _lib.kcb_error_string(status).decode())


def _p(t):
    """Device pointer of a torch tensor (or None / int passthrough)."""
    if t is None:
        return None
    if isinstance(t, int):
        return C.c_void_p(t)
    return C.c_void_p(t.data_ptr())


def _stream(stream=None):
    import torch
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


def call(name: str, *args, stream=None, raise_on_error=True) -> int:
    """Calls kcb_<name>(*args, stream).  Tensors are passed by device pointer, ints as C ints,
    floats as C floats."""
    fn = getattr(_lib, "kcb_" + name)
    conv = []
    for a in args:
        if a is None or hasattr(a, "data_ptr"):
            conv.append(_p(a))
        elif isinstance(a, float):
            conv.append(C.c_float(a))
        elif isinstance(a, int):
            conv.append(C.c_int(a))
        else:
            conv.append(a)
    fn.restype = C.c_int
    status = fn(*conv, _stream(stream))
    if raise_on_error:
        check(status, "kcb_" + name)
    return status
