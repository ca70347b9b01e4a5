"""No GPU needed: the C-ABI library loads and exports every symbol include/kernelcore_b200.h declares,
refuses to run without a device, and the host-side headers hold the reference's numeric contracts."""
import ctypes as C
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = "".join(open(os.path.join(ROOT, "include", h)).read() for h in ("kernelcore_b200.h", "ggml-kernelcore-ops.h"))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kcb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from kernelcore_b200 import lib
    names = declared_symbols()
    assert len(names) > 60
    missing = [n for n in names if not hasattr(lib.raw, n)]
    assert not missing, missing
    assert lib.raw.kcb_build_arch() == b"sm_100a"
    assert lib.raw.kcb_kquant_bytes(8192, 3072, 0) == 14155776      # BASELINE config 0 weight bytes
    assert lib.raw.kcb_kquant_bytes(128256, 3072, 1) == 323205120   # config 1
    assert lib.raw.kcb_error_string(2) == b"invalid value"


def test_error_codes_match_reference_numbering():
    text = open(os.path.join(ROOT, "include", "kernelcore", "api.hpp")).read()
    body = re.search(r"enum class Error : int \{(.*?)\};", text, re.S).group(1)
    body = re.sub(r"//[^\n]*", "", body)
    names = [n.strip().split("=")[0].strip() for n in body.split(",") if n.strip()]
    assert names == ["Success", "NotInitialized", "InvalidValue", "InvalidDevice", "OutOfMemory", "InvalidPointer",
                     "InvalidResourceHandle", "UnsupportedOperation", "InvalidKernelImage", "KernelNotFound",
                     "DynamicCodeBlocked", "LaunchFailure", "KernelFault", "ContextPoisoned", "NotReady", "InternalError"]


def test_headers_compile_as_plain_cxx(tmp_path):
    """The public headers must compile with a host compiler alone (no CUDA), like the reference's."""
    src = tmp_path / "t.cpp"
    src.write_text('#include <kernelcore/api.hpp>\n#include <llm_kernels.hpp>\n#include <llm_model.hpp>\n#include <kernelcore_b200.h>\n#include <ggml-kernelcore-ops.h>\n'
                   'static_assert(sizeof(llm::MatvecQ4Q8Args) == 48, "");\nstatic_assert(sizeof(llm::AttnDims) == 28, "");\n'
                   'static_assert(llm::scratchInts(96) == 1056 && llm::scratchKInts(12) == 1020, "");\nint main() { return 0; }\n')
    inc = os.path.join(ROOT, "include")
    r = subprocess.run(["g++", "-std=c++20", "-fsyntax-only", f"-I{inc}", f"-I{inc}/llm", str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_runtime_refuses_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from kernelcore_b200 import lib
    assert lib.raw.kcb_init() == 3            # InvalidDevice: there is no CPU fallback
    p = C.c_void_p()
    assert lib.raw.kcb_malloc(C.byref(p), C.c_size_t(16)) == 1   # NotInitialized
    lib.raw.kcb_last_error_detail.restype = C.c_char_p
    assert b"kcInit" in lib.raw.kcb_last_error_detail()
