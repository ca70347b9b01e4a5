// extern "C" surface declared in include/kernelcore_b200.h: thin forwarding onto the launchers.
#include "../../include/kernelcore_b200.h"

#include "common.cuh"
#include "ops.h"

using namespace kcb;

static cudaStream_t st(void* s) { return static_cast<cudaStream_t>(s); }

extern "C" {

int kcb_abi_version(void) { return 1; }
const char* kcb_build_arch(void) { return "sm_100a"; }

const char* kcb_error_string(int e) {
    switch (e) {
    case KCB_SUCCESS: return "success";
    case KCB_NOT_INITIALIZED: return "runtime not initialized";
    case KCB_INVALID_VALUE: return "invalid value";
    case KCB_INVALID_DEVICE: return "invalid device";
    case KCB_OUT_OF_MEMORY: return "out of memory";
    case KCB_INVALID_POINTER: return "invalid pointer";
    case KCB_INVALID_RESOURCE_HANDLE: return "invalid resource handle";
    case KCB_UNSUPPORTED_OPERATION: return "unsupported operation";
    case KCB_INVALID_KERNEL_IMAGE: return "invalid kernel image";
    case KCB_KERNEL_NOT_FOUND: return "kernel not found";
    case KCB_DYNAMIC_CODE_BLOCKED: return "dynamic code blocked";
    case KCB_LAUNCH_FAILURE: return "launch failure";
    case KCB_KERNEL_FAULT: return "kernel fault";
    case KCB_CONTEXT_POISONED: return "context poisoned";
    case KCB_NOT_READY: return "not ready";
    case KCB_INTERNAL_ERROR: return "internal error";
    }
    return "unknown error";
}

unsigned kcb_tma_timeouts(void) { return tma_timeouts(); }

size_t kcb_kquant_bytes(int rows, int k, int q6) {
    if (rows < 0 || k < 0 || k % 256) return 0;
    return static_cast<size_t>(rows) * (k / 256) * (q6 ? kQ6KBlock : kQ4KBlock);
}
int kcb_q6k_to_planes(const void* src, void* dst, int rows, int k, void* s) { return q6k_convert(src, dst, rows, k, 1, st(s)); }
int kcb_q6k_from_planes(const void* src, void* dst, int rows, int k, void* s) { return q6k_convert(src, dst, rows, k, 0, st(s)); }
int kcb_dequant_q4k(const void* w, float* out, int rows, int k, void* s) { return dequant_q4k(w, out, rows, k, st(s)); }
int kcb_dequant_q6k(const void* w, float* out, int rows, int k, void* s) { return dequant_q6k(w, out, rows, k, st(s)); }

int kcb_quantize_q8x4(const float* x, int32_t* xq, float* xd, int count, void* s) { return quantize_q8x4(x, xq, xd, count, st(s)); }
int kcb_quantize_cols(const float* x, int32_t* q, int k, int ncols, void* s) { return quantize_cols(x, q, k, ncols, st(s)); }
int kcb_quantize_cols_k(const float* x, int32_t* q, int k, int ncols, void* s) { return quantize_cols_k(x, q, k, ncols, st(s)); }

int kcb_matvec_q4k_q8(const void* w, const int32_t* xq, const float* xd, float* y, int rows, int k, void* s) {
    return matvec_q4k_q8(w, xq, xd, y, rows, k, st(s));
}
int kcb_matvec_q6k_q8(const void* w, const int32_t* xq, const float* xd, float* y, int rows, int k, void* s) {
    return matvec_q6k_q8(w, xq, xd, y, rows, k, st(s));
}
int kcb_matvec_q4k_f32(const void* w, const float* x, float* y, int rows, int k, void* s) { return matvec_q4k_f32(w, x, y, rows, k, st(s)); }
int kcb_matvec_q6k_f32(const void* w, const float* x, float* y, int rows, int k, void* s) { return matvec_q6k_f32(w, x, y, rows, k, st(s)); }

}  // extern "C"
