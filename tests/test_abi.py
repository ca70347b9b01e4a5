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
    assert lib.raw.kcb_kquant_bytes(8192, 3072, 0) == 14155776      # weight bytes of the Q4_K 8192 x 3072 benchmark matrix
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


def test_every_kernel_name_of_the_reference_is_registered():
    """The names llm::registerKernels puts in the reference's table (llm/llm_kernels.cpp:1016-1062) plus the runtime's
    built-in vector_add: each must resolve here (launching needs a GPU; the table does not)."""
    import ctypes as C

    from kernelcore_b200 import lib
    lib.raw.kcb_kernel_name.restype = C.c_char_p
    have = {lib.raw.kcb_kernel_name(i).decode() for i in range(lib.raw.kcb_kernel_count())}
    reference = """matvec_q8 matvec_q4 matvec_q4x8 quantize_q8x4 matvec_q4x8_q8 matvec_q4x8_q8x2 matvec_q4k_q8 matvec_q6k_q8
        matmul_q4k_q8x4 matmul_q6k_q8x4 matmul_q4k_q8x8 matmul_q6k_q8x8 quantize_cols quantize_cols_k matmul_q4k_q8kx4
        matmul_q6k_q8kx4 matmul_q4k_q8kx8 matmul_q6k_q8kx8 rope_ff mul_rows rope_ggml add_sumsq_f sumsq_part norm_mul_q8_f
        silu_mul_q8x4f norm_mul_q8k_f silu_mul_q8kf add_rms_norm silu_mul_q8x4 add_sumsq norm_q8x4 rms_norm rope kv_append
        attn_scores softmax attn_values silu_mul matmul_f16 set_rows_f16 fa_scores fa_max fa_exp fa_values vector_add""".split()
    assert len(reference) == 45
    assert not [n for n in reference if n not in have]
    assert lib.raw.kcb_kernel_name(-1) is None and lib.raw.kcb_kernel_name(10 ** 6) is None


def test_tensor_core_k_slices_follow_the_wave_model():
    """The number of K slices of a tensor-core matmul given a workspace is pure host arithmetic (units per persistent
    CTA x (super-blocks per unit + 1), plus the adding kernel): pinned here on the shapes the GPU tests and the benchmark
    rely on, because one pass means bit identity with the reference's mirror and more slices mean ~1e-6."""
    import ctypes as C
    from kernelcore_b200 import lib
    ks = lib.raw.kcb_matmul_tc_k_slices
    ws = lib.raw.kcb_matmul_tc_workspace_bytes
    ws.restype = C.c_size_t
    assert ks(8192, 3072, 512) == 1 and ks(8192, 3072, 2048) == 1      # the Q4_K 8192 x 3072 benchmark matmul: 256 / 1024 tiles
    assert ks(8192, 3072, 128) == 2 and ks(8192, 3072, 32) == 2        # 64 tiles
    assert ks(3072, 8192, 512) == 3                                    # Llama-3.2-3B FFN-down: 96 tiles of 32 super-blocks
    assert ks(3072, 3072, 512) == 1 and ks(4096, 3072, 512) == 1      # wo, q|k: a split would gain < 10 %
    assert ks(1024, 3072, 512) == 4                                    # v: 32 tiles
    assert ks(16384, 3072, 512) == 1                                   # gate|up
    assert ks(128 * 150, 1024, 128) == 1 and ks(128 * 150, 1024, 64) == 1 and ks(128 * 150, 1024, 16) == 1
    assert ks(4096, 12288, 512) == 1                                   # Qwen3-8B FFN-down: 128 tiles fill 86 % of the SMs
    assert ks(3072, 8192, 32) == 6                                     # 24 tiles x 32 super-blocks
    assert ks(100, 1024, 16) == 0 and ks(128, 768, 16) == 0            # not tensor-core shapes
    assert ws(8192, 3072, 512) == 0 and ws(3072, 8192, 512) == 3 * 512 * 3072 * 4 and ws(100, 1024, 16) == 0


def test_misaligned_pointers_are_refused_before_any_launch():
    """The kernels read weights, quantized activations and fp32 vectors 16 bytes at a time, and bulk copies need 16-byte
    aligned addresses; the reference's range check accepts any interior pointer.  So the launchers check alignment on
    the host and answer InvalidPointer (5) instead of letting a kernel fault.  Nothing here launches: every call is
    refused first (which is why it runs without a GPU), and the pointers are never dereferenced."""
    import ctypes as C
    from kernelcore_b200 import lib
    L = lib.raw
    good, odd4, odd1 = C.c_void_p(0x7000_0000_1000), C.c_void_p(0x7000_0000_1004), C.c_void_p(0x7000_0000_1001)
    INVALID_POINTER, INVALID_VALUE = 5, 2
    f = C.c_float
    cases = [
        (L.kcb_matvec_q4k_q8, (odd4, good, good, good, 64, 1024, None)),          # weights need 16
        (L.kcb_matvec_q4k_q8, (good, odd4, good, good, 64, 1024, None)),          # Q8 words need 16
        (L.kcb_matvec_q4k_q8, (good, good, odd4, good, 64, 1024, None)),          # Q8 scales need 16
        (L.kcb_matvec_q4k_q8, (good, good, good, odd1, 64, 1024, None)),          # outputs need 4
        (L.kcb_matvec_q6k_q8, (odd4, good, good, good, 64, 1024, None)),
        (L.kcb_quantize_q8x4, (odd1, good, good, 32, None)),                      # scalar loads and stores: 4
        (L.kcb_quantize_q8x4, (good, odd1, good, 32, None)),
        (L.kcb_quantize_cols_k, (odd1, good, 1024, 4, None)),
        (L.kcb_matmul_kq_q8, (odd4, good, good, 128, 1024, 16, 0, 1, None)),
        (L.kcb_matmul_kq_q8, (good, odd4, good, 128, 1024, 16, 0, 1, None)),
        (L.kcb_matmul_kq_q8, (good, good, odd1, 128, 1024, 16, 0, 1, None)),
        (L.kcb_rms_norm, (odd1, good, good, 256, 1, f(1e-5), None)),
        (L.kcb_add_rms_norm, (good, odd1, good, good, 256, f(1e-5), None)),
        (L.kcb_rope, (odd1, None, 32, 0, 64, f(19.0), None)),
        (L.kcb_matvec_q4k_f32x_static, (good, good, good, 64, 1024 + 1, None)),  # (k not a multiple of 256: InvalidValue)
    ]
    for fn, args in cases[:-1]:
        assert fn(*args) == INVALID_POINTER, (fn.__name__, args)
    assert cases[-1][0](*cases[-1][1]) == INVALID_VALUE
    # null pointers and bad shapes stay InvalidValue, also checked before anything is launched
    assert L.kcb_matvec_q4k_q8(None, good, good, good, 64, 1024, None) == INVALID_VALUE
    assert L.kcb_matvec_q4k_q8(good, good, good, good, 64, 1000, None) == INVALID_VALUE
