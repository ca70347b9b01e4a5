// Normalisation, RoPE, attention, SwiGLU and KV-cache kernels around the quantized matvecs, sm_100a.
//
// Each kernel replaces one (or a short run) of the reference's one-thread-per-output kernels under
// kernels/llm/ and keeps its arithmetic: the same separately rounded fp32 operations (explicit _rn
// intrinsics where the compiler would otherwise fuse a multiply-add), the same exp2-based softmax and
// SiLU, the same sin/cos argument quirk.  Where the reference sums sequentially and the sum is short
// (attention dot products, per-32 partial sums of squares) the order is kept and results are
// bit-identical; block-wide reductions (plain RMSNorm, softmax denominators) use a tree and agree to
// fp32 rounding.

#include "common.cuh"
#include "ops.h"

namespace kcb {
namespace {

__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : -INFINITY;
    return warp_max(t);
}

__device__ __forceinline__ float swiglu(float g, float u) {  // g / (1 + 2^(-g log2 e)) * u
    const float e = exp2f(__fmul_rn(-g, 1.44269504f));
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, e)), u);
}

// ---- RMSNorm ------------------------------------------------------------------------------------
// kernels/llm/rms_norm.cu:2-11 (one thread per row there).  One CTA per row; optional residual add
// first (kernels/llm/add_rms_norm.cu:4-17): x += t in place, then y = x * r * w.
__global__ void rms_norm_kernel(float* x, const float* __restrict__ t, const float* __restrict__ w, float* y, int n,
                                float eps) {
    __shared__ float red[32];
    float* xr = x + static_cast<size_t>(blockIdx.x) * n;
    float* yr = y + static_cast<size_t>(blockIdx.x) * n;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        float v = xr[j];
        if (t) {
            v = __fadd_rn(v, t[j]);
            xr[j] = v;
        }
        ss += v * v;
    }
    const float r = rinv_rms(block_sum(ss, red), n, eps);
    for (int j = threadIdx.x; j < n; j += blockDim.x) yr[j] = __fmul_rn(__fmul_rn(xr[j], r), w[j]);
}

// ---- residual add + RMSNorm + Q8 quantize ---------------------------------------------------------
// kernels/llm/add_sumsq.cu:6-19 and norm_q8x4.cu:6-45 (ggml forms add_sumsq_f.cu, sumsq_part.cu,
// norm_mul_q8_f.cu, norm_mul_q8k_f.cu).  Phase A: one thread per block of 32 adds t (if given) and sums
// the 32 squares in index order -- the reference's order, so the partial sums and everything derived
// from them are bit-identical.  Phase B: every thread adds the nb partial sums in block order,
// y = x * r * w, then one warp per block quantizes.  `phases` bit 0 = A, bit 1 = B; one CTA per row.
// out: where x + t goes (== x for the in-place form); y: optional fp32 copy of the normalised row;
// q: scratch slot(s); kq: != 0 -> per-256 slots (85 * n / 256 ints per row) in q, partial sums in sq.
__global__ void add_norm_q8_kernel(const float* __restrict__ a, const float* __restrict__ t, float* out,
                                   const float* __restrict__ w, float* y, int* q, int* sq, int n, float eps,
                                   int phases, int kq) {
    extern __shared__ float sh[];  // n floats (normalised row) + nb partial sums
    const int nb = n / 32, row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float* part = sh + n;
    int* slot = (kq ? sq : q) + static_cast<size_t>(row) * nb * 11;
    float* ss = reinterpret_cast<float*>(slot + nb * 10);
    const float* ar = a + static_cast<size_t>(row) * n;
    float* orow = out ? out + static_cast<size_t>(row) * n : nullptr;
    if (phases & 1) {
        // a warp per block of 32: coalesced add and store, then one lane adds the 32 squares in index order
        // out of shared memory (the reference's order; the other 31 lanes have nothing to add to it)
        for (int b = warp; b < nb; b += nw) {
            float v = ar[b * 32 + lane];
            if (t) v = __fadd_rn(v, t[static_cast<size_t>(row) * n + b * 32 + lane]);
            if (orow) orow[b * 32 + lane] = v;
            sh[b * 32 + lane] = v;
            __syncwarp();
            if (lane == 0) {
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float x = sh[b * 32 + i];
                    s = __fadd_rn(s, __fmul_rn(x, x));
                }
                ss[b] = s;
                part[b] = s;
            }
        }
    } else {
        for (int b = threadIdx.x; b < nb; b += blockDim.x) part[b] = ss[b];
    }
    if (!(phases & 2)) return;
    __syncthreads();
    float tot = 0.0f;
    for (int b = 0; b < nb; ++b) tot = __fadd_rn(tot, part[b]);
    const float r = rinv_rms(tot, n, eps);
    const float* xr = (phases & 1) && orow ? orow : ar;
    float* yr = y ? y + static_cast<size_t>(row) * n : nullptr;
    if (!kq) {
        int* xq = q + static_cast<size_t>(row) * nb * 11;
        float* xd = reinterpret_cast<float*>(xq + nb * 8);
        for (int b = warp; b < nb; b += nw) {
            const float h = __fmul_rn(__fmul_rn(xr[b * 32 + lane], r), w[b * 32 + lane]);
            if (yr) yr[b * 32 + lane] = h;
            quantize_block_warp(h, xq, xd, b, lane);
        }
        return;
    }
    // per-256 slots: normalise into shared memory (and y), then one warp per super-block
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const float h = __fmul_rn(__fmul_rn(xr[j], r), w[j]);
        sh[j] = h;
        if (yr) yr[j] = h;
    }
    __syncthreads();
    const int nsb = n / 256;
    int* ks = q + static_cast<size_t>(row) * nsb * 85;
    for (int s = warp; s < nsb; s += nw) {
        float v[8], am = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = sh[s * 256 + lane * 8 + i];
            am = fmaxf(am, fabsf(v[i]));
        }
        am = warp_max(am);
        const float d = __fdiv_rn(am, 127.0f);
        const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        unsigned w0 = 0, w1 = 0;
        int s8 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float tt = __fmul_rn(v[i], id);
            int qi = tt >= 0.0f ? __float2int_rz(__fadd_rn(tt, 0.5f)) : __float2int_rz(__fsub_rn(tt, 0.5f));
            qi = max(-127, min(127, qi));
            s8 += qi;
            if (i < 4) w0 |= (static_cast<unsigned>(qi) & 255u) << (8 * i);
            else w1 |= (static_cast<unsigned>(qi) & 255u) << (8 * (i - 4));
        }
        ks[s * 64 + lane * 2] = static_cast<int>(w0);
        ks[s * 64 + lane * 2 + 1] = static_cast<int>(w1);
        const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
        const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
        if ((lane & 1) == 0) ks[nsb * 65 + s * 16 + (lane >> 1)] = s16;
        if (lane == 0) reinterpret_cast<float*>(ks)[nsb * 64 + s] = d;
        unsigned pw[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int bsum = __shfl_sync(0xffffffffu, s32, 4 * i);
            pw[i / 4] |= (static_cast<unsigned>(bsum >> 6) & 255u) << (8 * (i % 4));
            pw[2 + i / 4] |= static_cast<unsigned>(bsum & 63) << (8 * (i % 4));
        }
        if (lane < 4) ks[nsb * 81 + s * 4 + lane] = static_cast<int>(lane == 0 ? pw[0] : lane == 1 ? pw[1] : lane == 2 ? pw[2] : pw[3]);
    }
}

// The same operation for the graph decoder, where latency matters more than summation order: one CTA,
// the sum of squares by groups of 128 (add_norm_q8_cta; the same arithmetic runs as the tail of the matvec
// launches of the decoder).  x += t (t may be null), Q8 blocks of norm(x) * w into (xq, xd).
__global__ void __launch_bounds__(1024) add_norm_q8_fast_kernel(float* x, const float* t, const float* __restrict__ w,
                                                                 int* xq, float* xd, int n, float eps) {
    __shared__ float gsum[11264 / 128];
    add_norm_q8_cta<3>(x, t, w, xq, xd, n, eps, gsum);
}
// n % 32 == 0 but not a multiple of 128: values staged in shared memory, tree reduction, the last blocks one by one.
__global__ void __launch_bounds__(1024) add_norm_q8_odd_kernel(float* x, const float* t, const float* __restrict__ w,
                                                                int* xq, float* xd, int n, float eps) {
    extern __shared__ __align__(16) float sh[];  // n floats
    __shared__ float red[32];
    float ss = 0.0f;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        float v = x[j];
        if (t) {
            v = __fadd_rn(v, t[j]);
            x[j] = v;
        }
        sh[j] = v;
        ss += v * v;
    }
    const float r = rinv_rms(block_sum(ss, red), n, eps);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b = warp; b < n / 32; b += nw)
        quantize_block_warp(__fmul_rn(__fmul_rn(sh[b * 32 + lane], r), w[b * 32 + lane]), xq, xd, b, lane);
}

// Two-stage greedy pick over the logits: per-CTA (value, index) candidates, first index wins ties.
__global__ void argmax_partial_kernel(const float* __restrict__ logits, int vocab, float* cand_v, int* cand_i) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        const float v = logits[i];
        if (v > best) best = v, idx = i;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
    }
    if (lane == 0) bv[warp] = best, bi[warp] = idx;
    __syncthreads();
    if (warp == 0) {
        best = lane < nw ? bv[lane] : -INFINITY;
        idx = lane < nw ? bi[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
        }
        if (lane == 0) cand_v[blockIdx.x] = best, cand_i[blockIdx.x] = idx;
    }
}

// ---- SwiGLU (+ quantize) ----------------------------------------------------------------------------
// kernels/llm/silu_mul.cu:2-9, silu_mul_q8x4.cu:5-41, silu_mul_q8x4f.cu:18-60, silu_mul_q8kf.cu:16-75.
__global__ void silu_mul_kernel(const float* __restrict__ g, const float* __restrict__ u, float* out, size_t count) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) out[i] = swiglu(g[i], u[i]);
}
// One warp per block of 32; column c's slot is q + c * 11 * nb ints (or the flat xq/xd pair).
// May be launched with a programmatic dependency on the kernel that writes g and u (the decode step does): results of
// that kernel from griddepcontrol.wait on, and g / u through plain loads (no read-only path for data that changes while
// this kernel is resident).
__global__ void silu_mul_q8_kernel(const float* g, const float* u, float* y, int* q, int nb, int cols, int* xq_flat, float* xd_flat) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (wid >= static_cast<long long>(nb) * cols) return;
    const int c = static_cast<int>(wid / nb), b = static_cast<int>(wid % nb);
    const size_t o = static_cast<size_t>(c) * nb * 32 + b * 32 + lane;
    const float h = swiglu(g[o], u[o]);
    if (y) y[o] = h;
    int* xq = xq_flat ? xq_flat : q + static_cast<size_t>(c) * nb * 11;
    float* xd = xd_flat ? xd_flat : reinterpret_cast<float*>(xq + nb * 8);
    quantize_block_warp(h, xq, xd, b, lane);
}
__global__ void mul_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, float* y, int n, size_t count) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) y[i] = __fmul_rn(x[i], w[i % n]);
}
__global__ void vector_add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* out, size_t count) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) out[i] = __fadd_rn(a[i], b[i]);
}

// ---- RoPE ---------------------------------------------------------------------------------------------
// kernels/llm/rope.cu:4-17, rope_ff.cu:5-19, rope_ggml.cu:21-44.  theta = pos * 2^(-i/pairs * log2 base)
// [/ ff_i]; the angle goes through (theta * 1/(2 pi)) * 2 pi in fp32 as the reference's mirror does.
__device__ __forceinline__ void rotate(float theta, float x0, float x1, float* o0, float* o1) {
    const float ang = __fmul_rn(__fmul_rn(theta, 0.159154943f), 6.28318548f);
    float s, c;
    sincosf(ang, &s, &c);
    *o0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    *o1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}
__device__ __forceinline__ float rope_theta(int pos, int i, int pairs, float log2_base, const float* ff) {
    const float e = __fmul_rn(__fdiv_rn(-static_cast<float>(i), static_cast<float>(pairs)), log2_base);
    float th = __fmul_rn(static_cast<float>(pos), exp2f(e));
    if (ff) th = __fdiv_rn(th, ff[i]);
    return th;
}
__global__ void rope_kernel(float* x, const float* __restrict__ ff, int pairs, int pos, int count, float log2_base) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= count) return;
    const float th = rope_theta(pos, idx % pairs, pairs, log2_base, ff);
    rotate(th, x[2 * idx], x[2 * idx + 1], &x[2 * idx], &x[2 * idx + 1]);
}
__global__ void rope_ggml_kernel(const float* __restrict__ x, float* y, const int* __restrict__ pos,
                                 const float* __restrict__ ff, int head_dim, int n_head, int n_tokens, float log2_base,
                                 int neox) {
    const int pairs = head_dim / 2;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pairs * n_head * n_tokens) return;
    const int t = idx / (pairs * n_head), i = idx % pairs, head = idx / pairs;
    const float th = rope_theta(pos[t], i, pairs, log2_base, ff);
    const int a = neox ? head * head_dim + i : 2 * idx, b = neox ? a + pairs : a + 1;
    rotate(th, x[a], x[b], &y[a], &y[b]);
}

// ---- fp32 KV cache and attention in the decode loop's layouts ----------------------------------------
// kernels/llm/kv_append.cu:4-14, attn_scores.cu:18-38, softmax.cu:3-18, attn_values.cu:15-32.
// K is cached transposed, kt[kv_stride][k_stride]; V as vc[ctx][kv_stride]; scores p[n_heads][ctx_pad].
__global__ void kv_append_kernel(const float* __restrict__ k, const float* __restrict__ v, float* kt, float* vc, int n,
                                 int k_stride, int pos) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    kt[static_cast<size_t>(j) * k_stride + pos] = k[j];
    vc[static_cast<size_t>(pos) * n + j] = v[j];
}
// One thread per (head, position): the head_dim products are added in index order (bit-identical to the
// reference); consecutive threads read consecutive positions of the transposed cache.
__global__ void attn_scores_kernel(const float* __restrict__ q, const float* __restrict__ kt, float* scores, int n_heads,
                                   int ctx, int head_dim, int group, int ctx_pad, int k_stride, float scale) {
    extern __shared__ float qs[];  // this head's query
    const int h = blockIdx.y;
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) qs[i] = q[h * head_dim + i];
    __syncthreads();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= ctx) return;
    const float* kb = kt + static_cast<size_t>(h / group) * head_dim * k_stride + t;
    float s = 0.0f;
#pragma unroll 8
    for (int i = 0; i < head_dim; ++i) s = __fadd_rn(s, __fmul_rn(qs[i], kb[static_cast<size_t>(i) * k_stride]));
    scores[static_cast<size_t>(h) * ctx_pad + t] = __fmul_rn(s, scale);
}
__global__ void softmax_kernel(float* x, int n, int stride) {
    __shared__ float red[32];
    float* xr = x + static_cast<size_t>(blockIdx.x) * stride;
    float m = -INFINITY;
    for (int j = threadIdx.x; j < n; j += blockDim.x) m = fmaxf(m, xr[j]);
    m = block_max(m, red);
    float sum = 0.0f;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const float e = exp2f(__fmul_rn(__fsub_rn(xr[j], m), 1.44269504f));
        xr[j] = e;
        sum += e;
    }
    const float inv = __fdiv_rn(1.0f, block_sum(sum, red));
    for (int j = threadIdx.x; j < n; j += blockDim.x) xr[j] = __fmul_rn(xr[j], inv);
}
// One thread per (head, channel), positions added in order (bit-identical); threads of a warp read
// consecutive channels of one V row.
__global__ void attn_values_kernel(const float* __restrict__ p, const float* __restrict__ v, float* out, int n_heads,
                                   int ctx, int head_dim, int kv_stride, int group, int ctx_pad) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_heads * head_dim) return;
    const int h = idx / head_dim, i = idx % head_dim;
    const float* pr = p + static_cast<size_t>(h) * ctx_pad;
    const float* vp = v + static_cast<size_t>(h / group) * head_dim + i;
    float s = 0.0f;
#pragma unroll 4
    for (int t = 0; t < ctx; ++t) s = __fadd_rn(s, __fmul_rn(pr[t], vp[static_cast<size_t>(t) * kv_stride]));
    out[idx] = s;
}

// ---- fp16 KV cache: SET_ROWS and attention ---------------------------------------------------------------
// kernels/llm/set_rows_f16.cu:67-83.  Round to nearest even; 65520 and above (and NaN) give 0x7bff with
// the sign of "x < 0"; an input of -0 gives +0 (negative values that round to zero keep their sign bit).
__global__ void set_rows_f16_kernel(const float* __restrict__ src, const long long* __restrict__ idx, unsigned* dst,
                                    int pairs, int rows, int src_row, int dst_row, int dst_rows) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<long long>(pairs) * rows) return;
    const int r = static_cast<int>(i / pairs), j = static_cast<int>(i % pairs);
    const int row = static_cast<int>(idx[r]);  // the low 32 bits, as the reference reads them
    if (static_cast<unsigned>(row) >= static_cast<unsigned>(dst_rows)) return;
    const float2 v = *reinterpret_cast<const float2*>(src + static_cast<size_t>(r) * src_row + 2 * j);
    dst[static_cast<size_t>(row) * dst_row + j] = f32_to_f16_bits(v.x) | (f32_to_f16_bits(v.y) << 16);
}

// kernels/llm/fa_scores.cu:41-99, fa_max.cu:14-25, fa_exp.cu:15-24, fa_values.cu:36-95 in one kernel.
// One CTA per (query i, head h).  Scores for all T positions live in shared memory; a warp scores one
// position at a time (lanes across the head dimension), then exp2-softmax, then one thread per output
// channel walks V.  out[i][h][d] = sum_t p_t V[t][h/group][d] / sum_t p_t.  Strides in 32-bit words.
struct FaParams {
    int H, T, D, group, tp, k_row, k_head, v_row, v_head, N, q_tok, q_head, m_row, has_mask, H_kv;
};
__global__ void flash_attn_f16_kernel(const float* __restrict__ q, const unsigned* __restrict__ k,
                                      const unsigned* __restrict__ v, const unsigned* __restrict__ mask, float* out,
                                      FaParams d, float scale) {
    extern __shared__ float sh[];  // T scores + D query values
    __shared__ float red[32];
    float* s = sh;
    float* qs = sh + d.T;
    const int i = blockIdx.x / d.H, h = blockIdx.x % d.H, kvh = h / d.group;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* qh = q + static_cast<size_t>(i) * d.q_tok + static_cast<size_t>(h) * d.q_head;
    for (int j = threadIdx.x; j < d.D; j += blockDim.x) qs[j] = qh[j];
    __syncthreads();
    const unsigned short* mrow = reinterpret_cast<const unsigned short*>(mask) + static_cast<size_t>(i) * d.m_row * 2;
    float mx = -INFINITY;
    for (int t = warp; t < d.T; t += nw) {
        const unsigned* kr = k + static_cast<size_t>(t) * d.k_row + static_cast<size_t>(kvh) * d.k_head;
        float a = 0.0f;
        for (int w = lane; w < d.D / 2; w += 32) {
            const unsigned kw = kr[w];
            a += qs[2 * w] * half_bits_to_float(kw & 0xFFFFu) + qs[2 * w + 1] * half_bits_to_float(kw >> 16);
        }
        a = warp_sum(a);
        const float mv = d.has_mask ? half_bits_to_float(mrow[t]) : 0.0f;
        const float sc = __fadd_rn(__fmul_rn(a, scale), mv);
        if (lane == 0) s[t] = sc;
        mx = fmaxf(mx, sc);
    }
    mx = block_max(mx, red);
    float sum = 0.0f;
    for (int t = threadIdx.x; t < d.T; t += blockDim.x) {
        const float e = exp2f(__fmul_rn(__fsub_rn(s[t], mx), 1.44269504f));
        s[t] = e;
        sum += e;
    }
    sum = block_sum(sum, red);
    for (int dd = threadIdx.x; dd < d.D; dd += blockDim.x) {
        const unsigned short* vp = reinterpret_cast<const unsigned short*>(v) + static_cast<size_t>(kvh) * d.v_head * 2 + dd;
        float a = 0.0f;
        for (int t = 0; t < d.T; ++t) a += s[t] * half_bits_to_float(vp[static_cast<size_t>(t) * d.v_row * 2]);
        out[(static_cast<size_t>(i) * d.H + h) * d.D + dd] = __fdiv_rn(a, sum);
    }
}

// The four-launch form of the same attention, kept because the reference's graph code launches them by name
// (kernels/llm/fa_scores.cu:41-99, fa_max.cu:14-25, fa_exp.cu:15-24, fa_values.cu:36-95): scores with mask, row
// maxima, in-place exp2, and the weighted V sum divided by the row sum.  Sequential sums in the reference's order.
__global__ void fa_scores_kernel(const float* __restrict__ q, const unsigned* __restrict__ k, const unsigned short* __restrict__ mask,
                                 float* s, FaParams d, float scale) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(d.H) * d.N * d.T) return;
    const int t = static_cast<int>(idx % d.T), i = static_cast<int>((idx / d.T) % d.N), h = static_cast<int>(idx / (static_cast<long long>(d.T) * d.N));
    const unsigned* kr = k + static_cast<size_t>(t) * d.k_row + static_cast<size_t>(h / d.group) * d.k_head;
    const float* qh = q + static_cast<size_t>(i) * d.q_tok + static_cast<size_t>(h) * d.q_head;
    float a = 0.0f;
    for (int j = 0; j < d.D / 2; ++j) {
        const unsigned w = kr[j];
        a = __fadd_rn(a, __fadd_rn(__fmul_rn(qh[2 * j], half_bits_to_float(w & 0xFFFFu)), __fmul_rn(qh[2 * j + 1], half_bits_to_float(w >> 16))));
    }
    const float mv = d.has_mask ? half_bits_to_float(mask[static_cast<size_t>(i) * d.m_row * 2 + t]) : 0.0f;
    s[(static_cast<size_t>(h) * d.N + i) * d.tp + t] = __fadd_rn(__fmul_rn(a, scale), mv);
}
__global__ void fa_max_kernel(const float* __restrict__ s, float* m, FaParams d) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= d.H * d.N) return;
    const float* sr = s + static_cast<size_t>(row) * d.tp;
    float mx = sr[0];
    for (int t = 1; t < d.T; ++t) mx = fmaxf(mx, sr[t]);
    m[row] = mx;
}
__global__ void fa_exp_kernel(float* s, const float* __restrict__ m, FaParams d) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(d.H) * d.N * d.T) return;
    const int t = static_cast<int>(idx % d.T);
    const long long row = idx / d.T;
    float* p = s + row * d.tp + t;
    *p = exp2f(__fmul_rn(__fsub_rn(*p, m[row]), 1.44269504f));
}
__global__ void fa_values_kernel(const float* __restrict__ p, const unsigned* __restrict__ v, float* out, FaParams d) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(d.N) * d.H * d.D) return;
    const int dd = static_cast<int>(idx % d.D), h = static_cast<int>((idx / d.D) % d.H), i = static_cast<int>(idx / (static_cast<long long>(d.D) * d.H));
    const float* pr = p + (static_cast<size_t>(h) * d.N + i) * d.tp;
    const unsigned short* vp = reinterpret_cast<const unsigned short*>(v) + static_cast<size_t>(h / d.group) * d.v_head * 2 + dd;
    float a = 0.0f, sum = 0.0f;
    for (int t = 0; t < d.T; ++t) {
        const float w = pr[t];
        a = __fadd_rn(a, __fmul_rn(w, half_bits_to_float(vp[static_cast<size_t>(t) * d.v_row * 2])));
        sum = __fadd_rn(sum, w);
    }
    out[idx] = __fdiv_rn(a, sum);
}

inline unsigned blocks_for(size_t n, int per) { return static_cast<unsigned>((n + per - 1) / per); }

}  // namespace

// True if any of the (possibly null) pointers is not 4-byte aligned: the glue kernels read and write 32-bit words.
template <class... P>
inline bool any_misaligned4(P... p) {
    return (... || misaligned(p, 4));
}

int rms_norm(const float* x, const float* w, float* y, int n, int rows, float eps, cudaStream_t s) {
    if (n <= 0 || rows < 0 || !x || !w || !y) return KCB_INVALID_VALUE;
    if (any_misaligned4(x, w, y)) return KCB_INVALID_POINTER;
    if (rows == 0) return KCB_SUCCESS;
    rms_norm_kernel<<<rows, n >= 1024 ? 256 : 64, 0, s>>>(const_cast<float*>(x), nullptr, w, y, n, eps);
    return launch_status();
}
int add_rms_norm(float* x, const float* t, const float* w, float* y, int n, float eps, cudaStream_t s) {
    if (n <= 0 || !x || !t || !w || !y) return KCB_INVALID_VALUE;
    if (any_misaligned4(x, t, w, y)) return KCB_INVALID_POINTER;
    rms_norm_kernel<<<1, 1024, 0, s>>>(x, t, w, y, n, eps);
    return launch_status();
}
// phases: 1 = add + partial sums, 2 = norm + quantize, 3 = both in one launch.
int add_norm_q8(const float* a, const float* t, float* out, const float* w, float* y, int* q, int* sq, int n, int rows,
                float eps, int phases, int kq, cudaStream_t s) {
    if (n <= 0 || n % (kq ? 256 : 32) || rows < 0 || !a || !q || (kq && !sq) || ((phases & 2) && !w)) return KCB_INVALID_VALUE;
    if (any_misaligned4(a, t, out, w, y, q, sq)) return KCB_INVALID_POINTER;
    if (rows == 0) return KCB_SUCCESS;
    const size_t smem = (static_cast<size_t>(n) + n / 32) * sizeof(float);
    if (smem > 48 * 1024) return KCB_INVALID_VALUE;
    add_norm_q8_kernel<<<rows, n >= 2048 ? 1024 : 256, smem, s>>>(a, t, out, w, y, q, sq, n, eps, phases, kq);
    return launch_status();
}
int add_norm_q8_fast(float* x, const float* t, const float* w, int* xq, float* xd, int n, float eps, cudaStream_t s) {
    if (n <= 0 || n % 32 || n > 11264 || !x || !w || !xq || !xd) return KCB_INVALID_VALUE;
    if (any_misaligned4(x, t, w, xq, xd)) return KCB_INVALID_POINTER;
    if (n % 128 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(t) | reinterpret_cast<uintptr_t>(w)) & 15) == 0)
        add_norm_q8_fast_kernel<<<1, 1024, 0, s>>>(x, t, w, xq, xd, n, eps);
    else
        add_norm_q8_odd_kernel<<<1, 1024, static_cast<size_t>(n) * sizeof(float), s>>>(x, t, w, xq, xd, n, eps);
    return launch_status();
}
int argmax_partial(const float* logits, int vocab, float* cand_v, int* cand_i, int ncand, cudaStream_t s) {
    if (vocab <= 0 || ncand <= 0 || !logits || !cand_v || !cand_i) return KCB_INVALID_VALUE;
    if (any_misaligned4(logits, cand_v, cand_i)) return KCB_INVALID_POINTER;
    argmax_partial_kernel<<<ncand, 256, 0, s>>>(logits, vocab, cand_v, cand_i);
    return launch_status();
}
int silu_mul(const float* g, const float* u, float* out, size_t count, cudaStream_t s) {
    if (!g || !u || !out) return KCB_INVALID_VALUE;
    if (any_misaligned4(g, u, out)) return KCB_INVALID_POINTER;
    if (count == 0) return KCB_SUCCESS;
    silu_mul_kernel<<<blocks_for(count, 256), 256, 0, s>>>(g, u, out, count);
    return launch_status();
}
int silu_mul_q8(const float* g, const float* u, float* y, int* q, int* xq, float* xd, int n, int cols, cudaStream_t s, bool pdl) {
    if (n <= 0 || n % 32 || cols < 0 || !g || !u || (!q && !(xq && xd))) return KCB_INVALID_VALUE;
    if (any_misaligned4(g, u, y, q, xq, xd)) return KCB_INVALID_POINTER;
    if (cols == 0) return KCB_SUCCESS;
    const size_t warps = static_cast<size_t>(n / 32) * cols;
    if (!pdl) {
        silu_mul_q8_kernel<<<blocks_for(warps, 8), 256, 0, s>>>(g, u, y, q, n / 32, cols, xq, xd);
        return launch_status();
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks_for(warps, 8)), cfg.blockDim = dim3(256), cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, silu_mul_q8_kernel, g, u, y, q, n / 32, cols, xq, xd) == cudaSuccess ? KCB_SUCCESS : KCB_LAUNCH_FAILURE;
}
int mul_rows(const float* x, const float* w, float* y, int n, size_t count, cudaStream_t s) {
    if (n <= 0 || !x || !w || !y) return KCB_INVALID_VALUE;
    if (any_misaligned4(x, w, y)) return KCB_INVALID_POINTER;
    if (count == 0) return KCB_SUCCESS;
    mul_rows_kernel<<<blocks_for(count, 256), 256, 0, s>>>(x, w, y, n, count);
    return launch_status();
}
int vector_add(const float* a, const float* b, float* out, size_t count, cudaStream_t s) {
    if (!a || !b || !out) return KCB_INVALID_VALUE;
    if (any_misaligned4(a, b, out)) return KCB_INVALID_POINTER;
    if (count == 0) return KCB_SUCCESS;
    vector_add_kernel<<<blocks_for(count, 256), 256, 0, s>>>(a, b, out, count);
    return launch_status();
}
int rope(float* x, const float* ff, int pairs, int pos, int count, float log2_base, cudaStream_t s) {
    if (pairs <= 0 || count < 0 || pos < 0 || !x) return KCB_INVALID_VALUE;
    if (any_misaligned4(x, ff)) return KCB_INVALID_POINTER;
    if (count == 0) return KCB_SUCCESS;
    rope_kernel<<<blocks_for(count, 128), 128, 0, s>>>(x, ff, pairs, pos, count, log2_base);
    return launch_status();
}
int rope_ggml(const float* x, float* y, const int* pos, const float* ff, int head_dim, int n_head, int n_tokens,
              float log2_base, int neox, cudaStream_t s) {
    if (head_dim <= 0 || head_dim % 2 || n_head < 0 || n_tokens < 0 || !x || !y || !pos) return KCB_INVALID_VALUE;
    if (any_misaligned4(x, y, pos, ff)) return KCB_INVALID_POINTER;
    const size_t count = static_cast<size_t>(head_dim / 2) * n_head * n_tokens;
    if (count == 0) return KCB_SUCCESS;
    rope_ggml_kernel<<<blocks_for(count, 128), 128, 0, s>>>(x, y, pos, ff, head_dim, n_head, n_tokens, log2_base, neox);
    return launch_status();
}
int kv_append(const float* k, const float* v, float* kt, float* vc, int n, int k_stride, int pos, cudaStream_t s) {
    if (n <= 0 || pos < 0 || pos >= k_stride || !k || !v || !kt || !vc) return KCB_INVALID_VALUE;
    if (any_misaligned4(k, v, kt, vc)) return KCB_INVALID_POINTER;
    kv_append_kernel<<<blocks_for(n, 128), 128, 0, s>>>(k, v, kt, vc, n, k_stride, pos);
    return launch_status();
}
int attn_scores(const float* q, const float* kt, float* scores, int n_heads, int ctx, int head_dim, int group,
                int ctx_pad, int k_stride, float scale, cudaStream_t s) {
    if (n_heads <= 0 || ctx <= 0 || head_dim <= 0 || group <= 0 || !q || !kt || !scores) return KCB_INVALID_VALUE;
    if (any_misaligned4(q, kt, scores)) return KCB_INVALID_POINTER;
    const dim3 grid(blocks_for(ctx, 128), n_heads);
    attn_scores_kernel<<<grid, 128, head_dim * sizeof(float), s>>>(q, kt, scores, n_heads, ctx, head_dim, group, ctx_pad, k_stride, scale);
    return launch_status();
}
int softmax(float* x, int n, int stride, int rows, cudaStream_t s) {
    if (n <= 0 || stride < n || rows < 0 || !x) return KCB_INVALID_VALUE;
    if (any_misaligned4(x)) return KCB_INVALID_POINTER;
    if (rows == 0) return KCB_SUCCESS;
    softmax_kernel<<<rows, n >= 1024 ? 256 : 64, 0, s>>>(x, n, stride);
    return launch_status();
}
int attn_values(const float* p, const float* v, float* out, int n_heads, int ctx, int head_dim, int kv_stride, int group,
                int ctx_pad, cudaStream_t s) {
    if (n_heads <= 0 || ctx <= 0 || head_dim <= 0 || group <= 0 || !p || !v || !out) return KCB_INVALID_VALUE;
    if (any_misaligned4(p, v, out)) return KCB_INVALID_POINTER;
    attn_values_kernel<<<blocks_for(static_cast<size_t>(n_heads) * head_dim, 64), 64, 0, s>>>(p, v, out, n_heads, ctx, head_dim, kv_stride, group, ctx_pad);
    return launch_status();
}
int set_rows_f16(const float* src, const long long* idx, void* dst, int pairs, int rows, int src_row, int dst_row,
                 int dst_rows, cudaStream_t s) {
    if (pairs <= 0 || rows < 0 || dst_rows < 0 || !src || !idx || !dst) return KCB_INVALID_VALUE;
    if (misaligned(src, 8) || (src_row & 1) || misaligned(idx, 8) || misaligned(dst, 4)) return KCB_INVALID_POINTER;  // float pairs in, half pairs out
    if (rows == 0) return KCB_SUCCESS;
    set_rows_f16_kernel<<<blocks_for(static_cast<size_t>(pairs) * rows, 256), 256, 0, s>>>(src, idx, static_cast<unsigned*>(dst), pairs, rows, src_row, dst_row, dst_rows);
    return launch_status();
}
int flash_attn_f16(const float* q, const void* k, const void* v, const void* mask, float* out, const int* dims15,
                   float scale, cudaStream_t s) {
    if (!q || !k || !v || !out || !dims15) return KCB_INVALID_VALUE;
    if (any_misaligned4(q, k, v, mask, out)) return KCB_INVALID_POINTER;
    FaParams d;
    int* f = reinterpret_cast<int*>(&d);
    for (int i = 0; i < 15; ++i) f[i] = dims15[i];
    if (d.H <= 0 || d.T <= 0 || d.D <= 0 || d.D % 2 || d.group <= 0 || d.N <= 0 || (d.has_mask && !mask)) return KCB_INVALID_VALUE;
    const size_t smem = (static_cast<size_t>(d.T) + d.D) * sizeof(float);
    if (smem > 200 * 1024) return KCB_UNSUPPORTED_OPERATION;
    if (smem > 48 * 1024) {
        static PerDeviceFlag raised;
        if (!raise_dynamic_smem(flash_attn_f16_kernel, 200 * 1024, raised)) return KCB_LAUNCH_FAILURE;
    }
    flash_attn_f16_kernel<<<d.N * d.H, 256, smem, s>>>(q, static_cast<const unsigned*>(k), static_cast<const unsigned*>(v),
                                                         static_cast<const unsigned*>(mask), out, d, scale);
    return launch_status();
}

// which: 0 fa_scores, 1 fa_max, 2 fa_exp, 3 fa_values.  Pointers not used by a stage may be null.
int fa_stage(int which, const float* q, const void* k, const void* v, const void* mask, float* s_buf, float* m_buf, float* out,
             const int* dims15, float scale, cudaStream_t s) {
    if (!dims15) return KCB_INVALID_VALUE;
    FaParams d;
    int* f = reinterpret_cast<int*>(&d);
    for (int i = 0; i < 15; ++i) f[i] = dims15[i];
    if (d.H <= 0 || d.T <= 0 || d.D <= 0 || d.D % 2 || d.group <= 0 || d.N <= 0 || d.tp < d.T) return KCB_INVALID_VALUE;
    const size_t cells = static_cast<size_t>(d.H) * d.N * d.T;
    switch (which) {
    case 0:
        if (!q || !k || !s_buf || (d.has_mask && !mask)) return KCB_INVALID_VALUE;
        fa_scores_kernel<<<blocks_for(cells, 256), 256, 0, s>>>(q, static_cast<const unsigned*>(k), static_cast<const unsigned short*>(mask), s_buf, d, scale);
        break;
    case 1:
        if (!s_buf || !m_buf) return KCB_INVALID_VALUE;
        fa_max_kernel<<<blocks_for(static_cast<size_t>(d.H) * d.N, 64), 64, 0, s>>>(s_buf, m_buf, d);
        break;
    case 2:
        if (!s_buf || !m_buf) return KCB_INVALID_VALUE;
        fa_exp_kernel<<<blocks_for(cells, 256), 256, 0, s>>>(s_buf, m_buf, d);
        break;
    case 3:
        if (!s_buf || !v || !out) return KCB_INVALID_VALUE;
        fa_values_kernel<<<blocks_for(static_cast<size_t>(d.N) * d.H * d.D, 128), 128, 0, s>>>(s_buf, static_cast<const unsigned*>(v), out, d);
        break;
    default: return KCB_INVALID_VALUE;
    }
    return launch_status();
}

}  // namespace kcb
