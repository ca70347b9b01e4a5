// extern "C" surface declared in include/kernelcore_b200.h: thin forwarding onto the launchers.
#include "../../include/kernelcore_b200.h"

#include "common.cuh"
#include "dispatch.h"
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
int kcb_matvec_q4k_q6k_pair_q8(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, const int32_t* xq, const float* xd,
                               int k, void* s) {
    return matvec_q4k_q6k_pair_q8(w4, y4, rows4, w6, y6, rows6, xq, xd, k, st(s));
}
int kcb_matvec_q4k_f32(const void* w, const float* x, float* y, int rows, int k, void* s) { return matvec_q4k_f32(w, x, y, rows, k, st(s)); }
int kcb_matvec_q6k_f32(const void* w, const float* x, float* y, int rows, int k, void* s) { return matvec_q6k_f32(w, x, y, rows, k, st(s)); }


int kcb_rms_norm(const float* x, const float* w, float* y, int n, int rows, float eps, void* s) { return rms_norm(x, w, y, n, rows, eps, st(s)); }
int kcb_add_rms_norm(float* x, const float* t, const float* w, float* y, int n, float eps, void* s) { return add_rms_norm(x, t, w, y, n, eps, st(s)); }
int kcb_add_sumsq(float* x, const float* t, int32_t* q, int nb, void* s) {
    if (!t) return KCB_INVALID_VALUE;
    return add_norm_q8(x, t, x, nullptr, nullptr, q, nullptr, nb * 32, 1, 0.f, 1, 0, st(s));
}
int kcb_norm_q8x4(const float* x, const float* w, int32_t* q, int nb, float eps, void* s) {
    return add_norm_q8(x, nullptr, nullptr, w, nullptr, q, nullptr, nb * 32, 1, eps, 2, 0, st(s));
}
int kcb_add_norm_q8x4(float* x, const float* t, const float* w, int32_t* q, int nb, float eps, void* s) {
    if (!t) return KCB_INVALID_VALUE;
    return add_norm_q8(x, t, x, w, nullptr, q, nullptr, nb * 32, 1, eps, 3, 0, st(s));
}
int kcb_add_sumsq_f(const float* a, const float* b, float* out, int32_t* q, int n, int rows, void* s) {
    if (!b || !out || n % 256) return KCB_INVALID_VALUE;
    return add_norm_q8(a, b, out, nullptr, nullptr, q, nullptr, n, rows, 0.f, 1, 0, st(s));
}
int kcb_sumsq_part(const float* x, int32_t* q, int n, int rows, void* s) {
    if (n % 256) return KCB_INVALID_VALUE;
    return add_norm_q8(x, nullptr, nullptr, nullptr, nullptr, q, nullptr, n, rows, 0.f, 1, 0, st(s));
}
int kcb_norm_mul_q8_f(const float* x, const float* w, float* y, int32_t* q, int n, int rows, float eps, void* s) {
    if (!y || n % 256) return KCB_INVALID_VALUE;
    return add_norm_q8(x, nullptr, nullptr, w, y, q, nullptr, n, rows, eps, 2, 0, st(s));
}
int kcb_norm_mul_q8k_f(const float* x, const float* w, float* y, int32_t* q, const int32_t* sq, int n, int rows, float eps, void* s) {
    if (!y) return KCB_INVALID_VALUE;
    return add_norm_q8(x, nullptr, nullptr, w, y, q, const_cast<int32_t*>(sq), n, rows, eps, 2, 1, st(s));
}
int kcb_silu_mul(const float* g, const float* u, float* out, int count, void* s) {
    return count < 0 ? KCB_INVALID_VALUE : silu_mul(g, u, out, static_cast<size_t>(count), st(s));
}
int kcb_silu_mul_q8x4(const float* g, const float* u, int32_t* xq, float* xd, int count, void* s) {
    if (count < 0) return KCB_INVALID_VALUE;
    if (count == 0) return KCB_SUCCESS;
    return silu_mul_q8(g, u, nullptr, nullptr, xq, xd, count * 32, 1, st(s));
}
int kcb_silu_mul_q8x4f(const float* g, const float* u, float* y, int32_t* q, int n, int cols, void* s) {
    if (!y || n % 256) return KCB_INVALID_VALUE;
    return silu_mul_q8(g, u, y, q, nullptr, nullptr, n, cols, st(s));
}
int kcb_silu_mul_q8kf(const float* g, const float* u, float* y, int32_t* q, int n, int cols, void* s) {
    if (!y || n <= 0 || n % 256 || cols < 0) return KCB_INVALID_VALUE;
    const int e = silu_mul(g, u, y, static_cast<size_t>(n) * cols, st(s));
    return e != KCB_SUCCESS ? e : quantize_cols_k(y, q, n, cols, st(s));
}
int kcb_mul_rows(const float* x, const float* w, float* y, int n, int count, void* s) {
    return count < 0 ? KCB_INVALID_VALUE : mul_rows(x, w, y, n, static_cast<size_t>(count), st(s));
}
int kcb_vector_add(const float* a, const float* b, float* out, int count, void* s) {
    return count < 0 ? KCB_INVALID_VALUE : vector_add(a, b, out, static_cast<size_t>(count), st(s));
}
int kcb_rope(float* x, const float* ff, int pairs, int pos, int count, float lb, void* s) { return rope(x, ff, pairs, pos, count, lb, st(s)); }
int kcb_rope_ggml(const float* x, float* y, const int32_t* pos, const float* ff, int head_dim, int n_head, int n_tokens, float lb,
                  int neox, void* s) {
    return rope_ggml(x, y, pos, ff, head_dim, n_head, n_tokens, lb, neox, st(s));
}

// AttnDims sanity, as the reference's adapters check it (llm/llm_kernels.cpp:92-103).
static bool attn_ok(const int* d) {
    if (!d) return false;
    const int n_heads = d[0], ctx = d[1], head_dim = d[2], kv_stride = d[3], group = d[4], ctx_pad = d[5], k_stride = d[6];
    if (n_heads <= 0 || ctx <= 0 || head_dim <= 0 || group <= 0 || n_heads % group) return false;
    if (static_cast<long long>(n_heads / group) * head_dim > kv_stride) return false;
    return !(head_dim % 8 || ctx_pad % 8 || ctx_pad < ctx || k_stride < ctx);
}
int kcb_kv_append(const float* k, const float* v, float* kt, float* vc, const int* d, void* s) {
    if (!attn_ok(d)) return KCB_INVALID_VALUE;
    return kv_append(k, v, kt, vc, d[3], d[6], d[1] - 1, st(s));
}
int kcb_attn_scores(const float* q, const float* kt, float* scores, const int* d, float scale, void* s) {
    if (!attn_ok(d)) return KCB_INVALID_VALUE;
    return attn_scores(q, kt, scores, d[0], d[1], d[2], d[4], d[5], d[6], scale, st(s));
}
int kcb_softmax(float* x, int n, int stride, int rows, void* s) { return softmax(x, n, stride, rows, st(s)); }
int kcb_attn_values(const float* p, const float* v, float* out, const int* d, void* s) {
    if (!attn_ok(d)) return KCB_INVALID_VALUE;
    return attn_values(p, v, out, d[0], d[1], d[2], d[3], d[4], d[5], st(s));
}
int kcb_set_rows_f16(const float* src, const int64_t* idx, void* dst, int pairs, int rows, int src_row, int dst_row, int dst_rows,
                     void* s) {
    return set_rows_f16(src, reinterpret_cast<const long long*>(idx), dst, pairs, rows, src_row, dst_row, dst_rows, st(s));
}
int kcb_flash_attn_f16(const float* q, const void* k, const void* v, const void* mask, float* out, const int* dims, float scale,
                       void* s) {
    return flash_attn_f16(q, k, v, mask, out, dims, scale, st(s));
}

int kcb_matmul_kq_q8(const void* w, const int32_t* xq, float* y, int rows, int k, int ncols, int q6, int q8k, void* s) {
    return matmul_kq_q8(w, xq, y, rows, k, ncols, q6, q8k, st(s));
}
int kcb_matmul_kq_q8_ws(const void* w, const int32_t* xq, float* y, int rows, int k, int ncols, int q6, int q8k, void* workspace,
                        size_t workspace_bytes, void* s) {
    return matmul_kq_q8(w, xq, y, rows, k, ncols, q6, q8k, st(s), workspace, workspace_bytes);
}
size_t kcb_matmul_tc_workspace_bytes(int rows, int k, int ncols) { return matmul_tc_workspace_bytes(rows, k, ncols); }
unsigned kcb_tc_timeouts(void) { return tc_pipe_timeouts(); }
int kcb_matmul_tc_k_slices(int rows, int k, int ncols) { return matmul_tc_pipe_k_slices(rows, k, ncols); }
int kcb_kernel_count(void) { return kernel_count(); }
const char* kcb_kernel_name(int i) { return kernel_name(i); }
int kcb_matvec_q8w(const int8_t* q, const float* scales, const float* x, float* y, int rows, int k, void* s) {
    return matvec_q8w(q, scales, x, y, rows, k, st(s));
}
int kcb_matvec_q4w(const uint8_t* qs, const float* scales, const float* x, float* y, int rows, int k, int interleaved, void* s) {
    return matvec_q4w(qs, scales, x, y, rows, k, interleaved, st(s));
}
int kcb_matvec_q4x8_q8(const int32_t* qw, const int32_t* xq, const float* xd, float* y, int rows, int k, void* s) {
    return matvec_q4x8_q8(qw, xq, xd, y, rows, k, st(s));
}
int kcb_matmul_f16(const int32_t* qw, const float* x, float* y, int rows, int k, int ncols, void* s) {
    return matmul_f16(qw, x, y, rows, k, ncols, st(s));
}
int kcb_matvec_q6k_q8_gather(const void* w, const int32_t* xq, const float* xd, float* y_local, float* const* y_peers, int npeers,
                             int rows, int k, void* s) {
    return matvec_q6k_q8_gather(w, xq, xd, y_local, y_peers, npeers, rows, k, st(s));
}
int kcb_peer_barrier(unsigned* const* flags, int rank, int world, unsigned epoch, void* s) { return peer_barrier(flags, rank, world, epoch, nullptr, st(s)); }
int kcb_matvec_q6k_f32x_sharded(const void* w, const float* x, float* y_local, float* const* y_peers, int npeers,
                                unsigned* const* flags, unsigned* counters, int rank, int world, int rows, int k, void* ev_before,
                                void* ev_after, void* s) {
    if (ev_before && cudaEventRecord(static_cast<cudaEvent_t>(ev_before), st(s)) != cudaSuccess) return KCB_INVALID_RESOURCE_HANDLE;
    const int e = matvec_q6k_f32x_sharded(w, x, y_local, y_peers, npeers, flags, counters, counters ? counters + 1 : nullptr, rank, world,
                                          rows, k, st(s));
    if (e != KCB_SUCCESS) return e;
    if (ev_after && cudaEventRecord(static_cast<cudaEvent_t>(ev_after), st(s)) != cudaSuccess) return KCB_INVALID_RESOURCE_HANDLE;
    return KCB_SUCCESS;
}

unsigned kcb_peer_timeouts(void) { return peer_timeouts() + tma_timeouts(); }
int kcb_peer_set_poll_limit(unsigned polls) { return peer_set_poll_limit(polls); }
int kcb_peer_reset(void) { return peer_reset(); }

}  // extern "C"
