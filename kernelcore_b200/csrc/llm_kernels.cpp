// Typed adapters: one per kernel name of the reference's table (llm/llm_kernels.cpp:1017-1062).
// Each checks the shape rules the reference's adapter checks, range-checks every buffer against the
// live allocations of the current device (the reference's LaunchContext::checkDeviceRange; this replaces
// compute-sanitizer-style protection with host-side checks before anything is launched) and then
// enqueues the CUDA implementation.  The reference's adapters also read the device-side `dims` arrays on
// the host, which only works because its device memory is host memory; here `dims` is range-checked and
// otherwise unused.

#include "common.cuh"
#include "dispatch.h"
#include "ops.h"

#include <llm_kernels.hpp>

#include <cstring>
#include <limits>

namespace kcb {
namespace {

using namespace llm;

#define TRY(expr)                                  \
    do {                                           \
        if (const int e_ = (expr); e_ != KCB_SUCCESS) return e_; \
    } while (0)

constexpr long long kMaxIndex = std::numeric_limits<int32_t>::max();
bool fits(long long a, long long b = 1) { return a >= 0 && b >= 0 && (b == 0 || a <= kMaxIndex / b); }
size_t f32(long long n) { return static_cast<size_t>(n) * sizeof(float); }
size_t i32(long long n) { return static_cast<size_t>(n) * sizeof(int); }

bool attn_shape_ok(const AttnDims& d) {  // llm/llm_kernels.cpp:92-103
    if (d.n_heads <= 0 || d.ctx <= 0 || d.head_dim <= 0 || d.group <= 0 || d.n_heads % d.group) return false;
    if (!fits(d.n_heads, d.ctx) || !fits(d.n_heads, d.head_dim) || !fits(d.ctx, d.kv_stride)) return false;
    if (static_cast<long long>(d.n_heads / d.group) * d.head_dim > d.kv_stride) return false;
    if (d.head_dim % 8 || d.ctx_pad % 8 || d.ctx_pad < d.ctx || d.k_stride < d.ctx) return false;
    return fits(d.n_heads, d.ctx_pad) && fits(d.kv_stride, d.k_stride);
}

int k_vector_add(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const kc::kernels::VectorAddArgs*>(p);
    if (a.count < 0) return KCB_INVALID_VALUE;
    TRY(rc.check(a.a, f32(a.count), "a"));
    TRY(rc.check(a.b, f32(a.count), "b"));
    TRY(rc.check(a.out, f32(a.count), "out"));
    return vector_add(a.a, a.b, a.out, a.count, s);
}

int k_quantize(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const QuantizeArgs*>(p);
    if (a.count < 0 || !fits(a.count, 32)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.x, f32(static_cast<long long>(a.count) * 32), "x"));
    TRY(rc.check(a.xq, i32(static_cast<long long>(a.count) * 8), "xq"));
    TRY(rc.check(a.xd, f32(static_cast<long long>(a.count) * 2), "xd"));
    return quantize_q8x4(a.x, a.xq, a.xd, a.count, s);
}

template <bool kQ6>
int k_matvec_kq(const void* p, const RangeChecker& rc, cudaStream_t s) {  // llm/llm_kernels.cpp:264-279
    const auto& a = *static_cast<const MatvecQ4Q8Args*>(p);
    if (a.rows < 0 || a.rows % 8 || a.k <= 0 || a.k % 256 || !fits(a.rows, a.k)) return KCB_INVALID_VALUE;
    const long long nb = a.k / 32, nsb = a.k / 256;
    TRY(rc.check(a.qw, static_cast<size_t>(a.rows) * nsb * (kQ6 ? kQ6KBlock : kQ4KBlock), "qw"));
    TRY(rc.check(a.xq, i32(nb * 8), "xq"));
    TRY(rc.check(a.xd, f32(nb * 2), "xd"));
    TRY(rc.check(a.y, f32(a.rows), "y"));
    TRY(rc.check(a.dims, 2 * sizeof(int), "dims"));
    return kQ6 ? matvec_q6k_q8(a.qw, a.xq, a.xd, a.y, a.rows, a.k, s) : matvec_q4k_q8(a.qw, a.xq, a.xd, a.y, a.rows, a.k, s);
}

template <bool kQ6, bool kQ8K>
int k_matmul_kq(const void* p, const RangeChecker& rc, cudaStream_t s) {  // llm/llm_kernels.cpp:294-313
    const auto& a = *static_cast<const MatmulKQ8Args*>(p);
    if (a.rows <= 0 || a.rows % 8 || a.k <= 0 || a.k % 256 || a.ncols <= 0 || a.row_block <= 0 || !fits(a.rows, a.k))
        return KCB_INVALID_VALUE;
    const long long nb = a.k / 32, nsb = a.k / 256;
    const int slot = kQ8K ? scratchKInts(static_cast<int>(nsb)) : scratchInts(static_cast<int>(nb));
    if (!fits(slot, a.ncols) || !fits(a.rows, a.ncols)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.qw, static_cast<size_t>(a.rows) * nsb * (kQ6 ? kQ6KBlock : kQ4KBlock), "qw"));
    TRY(rc.check(a.xq, i32(static_cast<long long>(slot) * a.ncols), "xq"));
    TRY(rc.check(a.y, f32(static_cast<long long>(a.rows) * a.ncols), "y"));
    TRY(rc.check(a.dims, 4 * sizeof(int), "dims"));
    return matmul_kq_q8(a.qw, a.xq, a.y, a.rows, a.k, a.ncols, kQ6, kQ8K, s);
}

template <bool kQ8K>
int k_quantize_cols(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const QuantizeColsArgs*>(p);
    const int blk = kQ8K ? 256 : 32;
    if (a.k <= 0 || a.k % blk || a.ncols < 0 || !fits(a.k, a.ncols)) return KCB_INVALID_VALUE;
    const int slot = kQ8K ? scratchKInts(a.k / 256) : scratchInts(a.k / 32);
    if (!fits(slot, a.ncols)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.x, f32(static_cast<long long>(a.k) * a.ncols), "x"));
    TRY(rc.check(a.q, i32(static_cast<long long>(slot) * a.ncols), "q"));
    TRY(rc.check(a.dims, 2 * sizeof(int), "dims"));
    return kQ8K ? quantize_cols_k(a.x, a.q, a.k, a.ncols, s) : quantize_cols(a.x, a.q, a.k, a.ncols, s);
}

int k_rms_norm(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const RmsNormArgs*>(p);
    if (a.n <= 0 || a.rows < 0 || !fits(a.n, a.rows)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.x, f32(static_cast<long long>(a.n) * a.rows), "x"));
    TRY(rc.check(a.w, f32(a.n), "w"));
    TRY(rc.check(a.y, f32(static_cast<long long>(a.n) * a.rows), "y"));
    return rms_norm(a.x, a.w, a.y, a.n, a.rows, a.eps, s);
}
int k_add_rms_norm(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const AddRmsNormArgs*>(p);
    if (a.n <= 0) return KCB_INVALID_VALUE;
    TRY(rc.check(a.x, f32(a.n), "x"));
    TRY(rc.check(a.t, f32(a.n), "t"));
    TRY(rc.check(a.w, f32(a.n), "w"));
    TRY(rc.check(a.y, f32(a.n), "y"));
    return add_rms_norm(a.x, a.t, a.w, a.y, a.n, a.eps, s);
}
int k_add_sumsq(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const AddSumsqArgs*>(p);
    if (a.nb <= 0 || !fits(a.nb, 32)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.x, f32(static_cast<long long>(a.nb) * 32), "x"));
    TRY(rc.check(a.t, f32(static_cast<long long>(a.nb) * 32), "t"));
    TRY(rc.check(a.q, i32(scratchInts(a.nb)), "q"));
    return add_norm_q8(a.x, a.t, a.x, nullptr, nullptr, a.q, nullptr, a.nb * 32, 1, 0.f, 1, 0, s);
}
int k_norm_q8x4(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const NormQ8Args*>(p);
    if (a.nb <= 0 || !fits(a.nb, 32)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.x, f32(static_cast<long long>(a.nb) * 32), "x"));
    TRY(rc.check(a.w, f32(static_cast<long long>(a.nb) * 32), "w"));
    TRY(rc.check(a.q, i32(scratchInts(a.nb)), "q"));
    return add_norm_q8(a.x, nullptr, nullptr, a.w, nullptr, a.q, nullptr, a.nb * 32, 1, a.eps, 2, 0, s);
}
int k_add_sumsq_f(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const AddSumsqFArgs*>(p);
    if (a.n <= 0 || a.n % 256 || a.rows < 0 || !fits(a.n, a.rows)) return KCB_INVALID_VALUE;
    const long long e = static_cast<long long>(a.n) * a.rows;
    TRY(rc.check(a.a, f32(e), "a"));
    TRY(rc.check(a.b, f32(e), "b"));
    TRY(rc.check(a.out, f32(e), "out"));
    TRY(rc.check(a.q, i32(static_cast<long long>(scratchInts(a.n / 32)) * a.rows), "q"));
    TRY(rc.check(a.dims, 3 * sizeof(int), "dims"));
    return add_norm_q8(a.a, a.b, a.out, nullptr, nullptr, a.q, nullptr, a.n, a.rows, 0.f, 1, 0, s);
}
int k_sumsq_part(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const SumsqPartArgs*>(p);
    if (a.n <= 0 || a.n % 256 || a.rows < 0 || !fits(a.n, a.rows)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.x, f32(static_cast<long long>(a.n) * a.rows), "x"));
    TRY(rc.check(a.q, i32(static_cast<long long>(scratchInts(a.n / 32)) * a.rows), "q"));
    TRY(rc.check(a.dims, 3 * sizeof(int), "dims"));
    return add_norm_q8(a.x, nullptr, nullptr, nullptr, nullptr, a.q, nullptr, a.n, a.rows, 0.f, 1, 0, s);
}
template <bool kQ8K>
int k_norm_mul(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const NormMulQ8Args*>(p);
    if (a.n <= 0 || a.n % 256 || a.rows < 0 || !fits(a.n, a.rows)) return KCB_INVALID_VALUE;
    const long long e = static_cast<long long>(a.n) * a.rows;
    TRY(rc.check(a.x, f32(e), "x"));
    TRY(rc.check(a.w, f32(a.n), "w"));
    TRY(rc.check(a.y, f32(e), "y"));
    if (!kQ8K) {
        TRY(rc.check(a.q, i32(static_cast<long long>(scratchInts(a.n / 32)) * a.rows), "q"));
        TRY(rc.check(a.dims, 3 * sizeof(int), "dims"));
        return add_norm_q8(a.x, nullptr, nullptr, a.w, a.y, a.q, nullptr, a.n, a.rows, a.eps, 2, 0, s);
    }
    // q: rows per-256 slots, then rows per-32 slots holding the partial sums (llm/llm_kernels.hpp:212-216)
    const long long kslots = static_cast<long long>(scratchKInts(a.n / 256)) * a.rows;
    TRY(rc.check(a.q, i32(kslots + static_cast<long long>(scratchInts(a.n / 32)) * a.rows), "q"));
    TRY(rc.check(a.dims, 4 * sizeof(int), "dims"));
    return add_norm_q8(a.x, nullptr, nullptr, a.w, a.y, a.q, a.q + kslots, a.n, a.rows, a.eps, 2, 1, s);
}
int k_silu_mul(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const SiluMulArgs*>(p);
    if (a.count < 0) return KCB_INVALID_VALUE;
    TRY(rc.check(a.g, f32(a.count), "g"));
    TRY(rc.check(a.u, f32(a.count), "u"));
    TRY(rc.check(a.out, f32(a.count), "out"));
    return silu_mul(a.g, a.u, a.out, a.count, s);
}
int k_silu_mul_q8x4(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const SiluMulQ8Args*>(p);
    if (a.count < 0 || !fits(a.count, 32)) return KCB_INVALID_VALUE;
    if (a.count == 0) return KCB_SUCCESS;
    const long long n = static_cast<long long>(a.count) * 32;
    TRY(rc.check(a.g, f32(n), "g"));
    TRY(rc.check(a.u, f32(n), "u"));
    TRY(rc.check(a.xq, i32(static_cast<long long>(a.count) * 8), "xq"));
    TRY(rc.check(a.xd, f32(static_cast<long long>(a.count) * 2), "xd"));
    return silu_mul_q8(a.g, a.u, nullptr, nullptr, a.xq, a.xd, static_cast<int>(n), 1, s);
}
template <bool kQ8K>
int k_silu_mul_f(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const SiluMulQ8FArgs*>(p);
    if (a.n <= 0 || a.n % 256 || a.cols < 0 || !fits(a.n, a.cols)) return KCB_INVALID_VALUE;
    const long long e = static_cast<long long>(a.n) * a.cols;
    const int slot = kQ8K ? scratchKInts(a.n / 256) : scratchInts(a.n / 32);
    TRY(rc.check(a.g, f32(e), "g"));
    TRY(rc.check(a.u, f32(e), "u"));
    TRY(rc.check(a.y, f32(e), "y"));
    TRY(rc.check(a.q, i32(static_cast<long long>(slot) * a.cols), "q"));
    TRY(rc.check(a.dims, 2 * sizeof(int), "dims"));
    if (!kQ8K) return silu_mul_q8(a.g, a.u, a.y, a.q, nullptr, nullptr, a.n, a.cols, s);
    TRY(silu_mul(a.g, a.u, a.y, static_cast<size_t>(e), s));
    return quantize_cols_k(a.y, a.q, a.n, a.cols, s);
}
int k_mul_rows(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const MulRowsArgs*>(p);
    if (a.n <= 0 || a.n % 8 || a.count < 0) return KCB_INVALID_VALUE;
    TRY(rc.check(a.x, f32(a.count), "x"));
    TRY(rc.check(a.w, f32(a.n), "w"));
    TRY(rc.check(a.y, f32(a.count), "y"));
    return mul_rows(a.x, a.w, a.y, a.n, a.count, s);
}
int k_rope(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const RopeArgs*>(p);
    if (a.pairs_per_head <= 0 || a.count < 0 || a.pos < 0 || !fits(a.count, 2)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.x, f32(static_cast<long long>(a.count) * 2), "x"));
    return rope(a.x, nullptr, a.pairs_per_head, a.pos, a.count, a.log2_base, s);
}
int k_rope_ff(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const RopeFFArgs*>(p);
    if (a.pairs_per_head <= 0 || a.count < 0 || a.pos < 0 || !fits(a.count, 2)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.x, f32(static_cast<long long>(a.count) * 2), "x"));
    TRY(rc.check(a.ff, f32(a.pairs_per_head), "ff"));
    return rope(a.x, a.ff, a.pairs_per_head, a.pos, a.count, a.log2_base, s);
}
int k_rope_ggml(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const RopeGgmlArgs*>(p);
    if (a.head_dim <= 0 || a.head_dim % 16 || a.n_head <= 0 || a.n_tokens <= 0 || !fits(static_cast<long long>(a.head_dim) * a.n_head, a.n_tokens))
        return KCB_INVALID_VALUE;
    const long long e = static_cast<long long>(a.head_dim) * a.n_head * a.n_tokens;
    TRY(rc.check(a.x, f32(e), "x"));
    TRY(rc.check(a.y, f32(e), "y"));
    TRY(rc.check(a.pos, i32(a.n_tokens), "pos"));
    TRY(rc.check(a.ff, f32(a.head_dim / 2), "ff"));
    TRY(rc.check(a.dims, (a.neox ? 5 : 3) * sizeof(int), "dims"));
    return rope_ggml(a.x, a.y, a.pos, a.ff, a.head_dim, a.n_head, a.n_tokens, a.log2_base, a.neox ? 1 : 0, s);
}
int k_kv_append(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const KvAppendArgs*>(p);
    if (!attn_shape_ok(a.d)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.k, f32(a.d.kv_stride), "k"));
    TRY(rc.check(a.v, f32(a.d.kv_stride), "v"));
    TRY(rc.check(a.kt, f32(static_cast<long long>(a.d.kv_stride) * a.d.k_stride), "kt"));
    TRY(rc.check(a.vc, f32(static_cast<long long>(a.d.ctx) * a.d.kv_stride), "vc"));
    TRY(rc.check(a.dims, 7 * sizeof(int), "dims"));
    return kv_append(a.k, a.v, a.kt, a.vc, a.d.kv_stride, a.d.k_stride, a.d.ctx - 1, s);
}
int k_attn_scores(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const AttnScoresArgs*>(p);
    if (!attn_shape_ok(a.d)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.q, f32(static_cast<long long>(a.d.n_heads) * a.d.head_dim), "q"));
    TRY(rc.check(a.k, f32(static_cast<long long>(a.d.kv_stride) * a.d.k_stride), "k"));
    TRY(rc.check(a.scores, f32(static_cast<long long>(a.d.n_heads) * a.d.ctx_pad), "scores"));
    TRY(rc.check(a.dims, 7 * sizeof(int), "dims"));
    return attn_scores(a.q, a.k, a.scores, a.d.n_heads, a.d.ctx, a.d.head_dim, a.d.group, a.d.ctx_pad, a.d.k_stride, a.scale, s);
}
int k_softmax(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const SoftmaxArgs*>(p);
    if (a.n <= 0 || a.stride < a.n || a.rows < 0 || !fits(a.stride, a.rows)) return KCB_INVALID_VALUE;
    if (a.rows == 0) return KCB_SUCCESS;
    TRY(rc.check(a.x, f32(static_cast<long long>(a.rows - 1) * a.stride + a.n), "x"));
    return softmax(a.x, a.n, a.stride, a.rows, s);
}
int k_attn_values(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const AttnValuesArgs*>(p);
    if (!attn_shape_ok(a.d)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.p, f32(static_cast<long long>(a.d.n_heads) * a.d.ctx_pad), "p"));
    TRY(rc.check(a.v, f32(static_cast<long long>(a.d.ctx) * a.d.kv_stride), "v"));
    TRY(rc.check(a.out, f32(static_cast<long long>(a.d.n_heads) * a.d.head_dim), "out"));
    TRY(rc.check(a.dims, 7 * sizeof(int), "dims"));
    return attn_values(a.p, a.v, a.out, a.d.n_heads, a.d.ctx, a.d.head_dim, a.d.kv_stride, a.d.group, a.d.ctx_pad, s);
}
int k_set_rows_f16(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const SetRowsF16Args*>(p);
    if (a.pairs <= 0 || a.pairs % 8 || a.rows < 0 || a.dst_rows < 0 || a.src_row < 2 * a.pairs || a.dst_row < a.pairs) return KCB_INVALID_VALUE;
    if (a.rows == 0) return KCB_SUCCESS;
    TRY(rc.check(a.src, f32(static_cast<long long>(a.rows - 1) * a.src_row + 2 * a.pairs), "src"));
    TRY(rc.check(a.idx, static_cast<size_t>(a.rows) * 8, "idx"));
    if (a.dst_rows) TRY(rc.check(a.dst, i32(static_cast<long long>(a.dst_rows - 1) * a.dst_row + a.pairs), "dst"));
    TRY(rc.check(a.dims, 5 * sizeof(int), "dims"));
    return set_rows_f16(a.src, reinterpret_cast<const long long*>(a.idx), a.dst, a.pairs, a.rows, a.src_row, a.dst_row, a.dst_rows, s);
}
bool fa_shape_ok(const FaDims& d) {
    return d.H > 0 && d.T > 0 && d.D > 0 && d.D % 8 == 0 && d.group > 0 && d.H % d.group == 0 && d.N > 0 && d.tp >= d.T && d.tp % 8 == 0 &&
           d.H_kv == d.H / d.group;
}
int fa_check_kv(const FaDims& d, const int* k, const int* v, const RangeChecker& rc) {
    if (k) TRY(rc.check(k, i32(static_cast<long long>(d.T - 1) * d.k_row + static_cast<long long>(d.H_kv - 1) * d.k_head + d.D / 2), "k"));
    if (v) TRY(rc.check(v, i32(static_cast<long long>(d.T - 1) * d.v_row + static_cast<long long>(d.H_kv - 1) * d.v_head + d.D / 2), "v"));
    return KCB_SUCCESS;
}
int k_flash_attn_f16(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const FlashAttnF16Args*>(p);
    if (!fa_shape_ok(a.d)) return KCB_INVALID_VALUE;
    const FaDims& d = a.d;
    TRY(rc.check(a.q, f32(static_cast<long long>(d.N - 1) * d.q_tok + static_cast<long long>(d.H - 1) * d.q_head + d.D), "q"));
    TRY(fa_check_kv(d, a.k, a.v, rc));
    if (d.has_mask) TRY(rc.check(a.mask, i32(static_cast<long long>(d.N - 1) * d.m_row + (d.T + 1) / 2), "mask"));
    TRY(rc.check(a.out, f32(static_cast<long long>(d.N) * d.H * d.D), "out"));
    int dims[kFaDims];
    faDimsInts(d, dims);
    return flash_attn_f16(a.q, a.k, a.v, a.mask, a.out, dims, a.scale, s);
}
// fa_scores / fa_max / fa_exp / fa_values: score rows s[H*N][tp], maxima m[H*N] (llm/llm_kernels.hpp:339-366)
int k_fa_scores(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const FaScoresArgs*>(p);
    if (!fa_shape_ok(a.d)) return KCB_INVALID_VALUE;
    const FaDims& d = a.d;
    TRY(rc.check(a.q, f32(static_cast<long long>(d.N - 1) * d.q_tok + static_cast<long long>(d.H - 1) * d.q_head + d.D), "q"));
    TRY(fa_check_kv(d, a.k, nullptr, rc));
    if (d.has_mask) TRY(rc.check(a.mask, i32(static_cast<long long>(d.N - 1) * d.m_row + (d.T + 1) / 2), "mask"));
    TRY(rc.check(a.s, f32(static_cast<long long>(d.H) * d.N * d.tp), "s"));
    TRY(rc.check(a.dims, kFaDims * sizeof(int), "dims"));
    int dims[kFaDims];
    faDimsInts(d, dims);
    return fa_stage(0, a.q, a.k, nullptr, a.mask, a.s, nullptr, nullptr, dims, a.scale, s);
}
int k_fa_max(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const FaMaxArgs*>(p);
    if (!fa_shape_ok(a.d)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.s, f32(static_cast<long long>(a.d.H) * a.d.N * a.d.tp), "s"));
    TRY(rc.check(a.m, f32(static_cast<long long>(a.d.H) * a.d.N), "m"));
    TRY(rc.check(a.dims, kFaDims * sizeof(int), "dims"));
    int dims[kFaDims];
    faDimsInts(a.d, dims);
    return fa_stage(1, nullptr, nullptr, nullptr, nullptr, const_cast<float*>(a.s), a.m, nullptr, dims, 0.f, s);
}
int k_fa_exp(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const FaExpArgs*>(p);
    if (!fa_shape_ok(a.d)) return KCB_INVALID_VALUE;
    TRY(rc.check(a.s, f32(static_cast<long long>(a.d.H) * a.d.N * a.d.tp), "s"));
    TRY(rc.check(a.m, f32(static_cast<long long>(a.d.H) * a.d.N), "m"));
    TRY(rc.check(a.dims, kFaDims * sizeof(int), "dims"));
    int dims[kFaDims];
    faDimsInts(a.d, dims);
    return fa_stage(2, nullptr, nullptr, nullptr, nullptr, a.s, const_cast<float*>(a.m), nullptr, dims, 0.f, s);
}
int k_fa_values(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const FaValuesArgs*>(p);
    if (!fa_shape_ok(a.d)) return KCB_INVALID_VALUE;
    const FaDims& d = a.d;
    TRY(rc.check(a.p, f32(static_cast<long long>(d.H) * d.N * d.tp), "p"));
    TRY(fa_check_kv(d, nullptr, a.v, rc));
    TRY(rc.check(a.out, f32(static_cast<long long>(d.N) * d.H * d.D), "out"));
    TRY(rc.check(a.dims, kFaDims * sizeof(int), "dims"));
    int dims[kFaDims];
    faDimsInts(d, dims);
    return fa_stage(3, nullptr, nullptr, a.v, nullptr, const_cast<float*>(a.p), nullptr, a.out, dims, 0.f, s);
}
// The synthetic weight formats (llm/llm_kernels.cpp:110-262 of the reference validate the same extents).
int k_matvec_q8w(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const MatvecQ8Args*>(p);
    if (a.rows < 0 || a.k <= 0 || a.k % 32 || !fits(a.rows, a.k)) return KCB_INVALID_VALUE;
    const long long nb = a.k / 32;
    TRY(rc.check(a.q, static_cast<size_t>(a.rows) * a.k, "q"));
    TRY(rc.check(a.scales, f32(a.rows * nb), "scales"));
    TRY(rc.check(a.x, f32(a.k), "x"));
    TRY(rc.check(a.y, f32(a.rows), "y"));
    TRY(rc.check(a.dims, 2 * sizeof(int), "dims"));
    return matvec_q8w(a.q, a.scales, a.x, a.y, a.rows, a.k, s);
}
template <bool kInterleaved>
int k_matvec_q4w(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const MatvecQ4Args*>(p);
    if (a.rows < 0 || (kInterleaved && a.rows % 8) || a.k <= 0 || a.k % 32 || !fits(a.rows, a.k)) return KCB_INVALID_VALUE;
    const long long nb = a.k / 32;
    TRY(rc.check(a.qs, static_cast<size_t>(a.rows) * (a.k / 2), "qs"));
    TRY(rc.check(a.scales, f32(a.rows * nb), "scales"));
    TRY(rc.check(a.x, f32(a.k), "x"));
    TRY(rc.check(a.y, f32(a.rows), "y"));
    TRY(rc.check(a.dims, 2 * sizeof(int), "dims"));
    return matvec_q4w(a.qs, a.scales, a.x, a.y, a.rows, a.k, kInterleaved, s);
}
template <int kRowMult>  // matvec_q4x8_q8x2 is the same arithmetic with rows % 16 == 0
int k_matvec_q4x8_q8(const void* p, const RangeChecker& rc, cudaStream_t s) {
    const auto& a = *static_cast<const MatvecQ4Q8Args*>(p);
    if (a.rows < 0 || a.rows % kRowMult || a.k <= 0 || a.k % 32 || !fits(a.rows, a.k)) return KCB_INVALID_VALUE;
    const long long nb = a.k / 32;
    TRY(rc.check(a.qw, static_cast<size_t>(a.rows) * a.k * 5 / 8, "qw"));
    TRY(rc.check(a.xq, i32(nb * 8), "xq"));
    TRY(rc.check(a.xd, f32(nb * 2), "xd"));
    TRY(rc.check(a.y, f32(a.rows), "y"));
    TRY(rc.check(a.dims, 2 * sizeof(int), "dims"));
    return matvec_q4x8_q8(a.qw, a.xq, a.xd, a.y, a.rows, a.k, s);
}
int k_matmul_f16(const void* p, const RangeChecker& rc, cudaStream_t s) {  // llm/llm_kernels.cpp:835-850
    const auto& a = *static_cast<const MatmulF16Args*>(p);
    if (a.rows <= 0 || a.rows % 8 || a.k <= 0 || a.k % 2 || a.ncols <= 0 || !fits(a.rows, a.k) || !fits(a.k, a.ncols) || !fits(a.rows, a.ncols))
        return KCB_INVALID_VALUE;
    TRY(rc.check(a.qw, i32(static_cast<long long>(a.rows) * (a.k / 2)), "qw"));
    TRY(rc.check(a.x, f32(static_cast<long long>(a.k) * a.ncols), "x"));
    TRY(rc.check(a.y, f32(static_cast<long long>(a.rows) * a.ncols), "y"));
    TRY(rc.check(a.dims, 3 * sizeof(int), "dims"));
    return matmul_f16(a.qw, a.x, a.y, a.rows, a.k, a.ncols, s);
}

const KernelDesc kTable[] = {
    {"vector_add", &k_vector_add},
    {"quantize_q8x4", &k_quantize},
    {"matvec_q4k_q8", &k_matvec_kq<false>},
    {"matvec_q6k_q8", &k_matvec_kq<true>},
    {"matmul_q4k_q8x4", &k_matmul_kq<false, false>},
    {"matmul_q4k_q8x8", &k_matmul_kq<false, false>},
    {"matmul_q6k_q8x4", &k_matmul_kq<true, false>},
    {"matmul_q6k_q8x8", &k_matmul_kq<true, false>},
    {"matmul_q4k_q8kx4", &k_matmul_kq<false, true>},
    {"matmul_q4k_q8kx8", &k_matmul_kq<false, true>},
    {"matmul_q6k_q8kx4", &k_matmul_kq<true, true>},
    {"matmul_q6k_q8kx8", &k_matmul_kq<true, true>},
    {"quantize_cols", &k_quantize_cols<false>},
    {"quantize_cols_k", &k_quantize_cols<true>},
    {"rms_norm", &k_rms_norm},
    {"add_rms_norm", &k_add_rms_norm},
    {"add_sumsq", &k_add_sumsq},
    {"norm_q8x4", &k_norm_q8x4},
    {"add_sumsq_f", &k_add_sumsq_f},
    {"sumsq_part", &k_sumsq_part},
    {"norm_mul_q8_f", &k_norm_mul<false>},
    {"norm_mul_q8k_f", &k_norm_mul<true>},
    {"silu_mul", &k_silu_mul},
    {"silu_mul_q8x4", &k_silu_mul_q8x4},
    {"silu_mul_q8x4f", &k_silu_mul_f<false>},
    {"silu_mul_q8kf", &k_silu_mul_f<true>},
    {"mul_rows", &k_mul_rows},
    {"rope", &k_rope},
    {"rope_ff", &k_rope_ff},
    {"rope_ggml", &k_rope_ggml},
    {"kv_append", &k_kv_append},
    {"attn_scores", &k_attn_scores},
    {"softmax", &k_softmax},
    {"attn_values", &k_attn_values},
    {"set_rows_f16", &k_set_rows_f16},
    {"flash_attn_f16", &k_flash_attn_f16},
    {"fa_scores", &k_fa_scores},
    {"fa_max", &k_fa_max},
    {"fa_exp", &k_fa_exp},
    {"fa_values", &k_fa_values},
    {"matvec_q8", &k_matvec_q8w},
    {"matvec_q4", &k_matvec_q4w<false>},
    {"matvec_q4x8", &k_matvec_q4w<true>},
    {"matvec_q4x8_q8", &k_matvec_q4x8_q8<8>},
    {"matvec_q4x8_q8x2", &k_matvec_q4x8_q8<16>},
    {"matmul_f16", &k_matmul_f16},

};
constexpr int kCount = sizeof(kTable) / sizeof(kTable[0]);

}  // namespace

const KernelDesc* find_kernel(const char* name) {
    for (const KernelDesc& k : kTable)
        if (std::strcmp(k.name, name) == 0) return &k;
    return nullptr;
}
int kernel_count() { return kCount; }
const char* kernel_name(int i) { return i >= 0 && i < kCount ? kTable[i].name : nullptr; }

}  // namespace kcb

kc::Error llm::registerKernels() noexcept {
    int n = 0;
    return kcGetDeviceCount(&n);  // Success once kcInit has run; the built-in table needs no registration
}
