// Dequant-fused K-quant matvec for decode, y[rows] = W[rows][k] . x[k], sm_100a.
//
// Replaces the reference's one-thread-per-row kernels kernels/llm/matvec_q4k_q8.cu:33-88 and
// kernels/llm/matvec_q6k_q8.cu:33-105.  Same arithmetic contract -- weights are never expanded in
// memory, activations are the Q8 blocks of 32 that quantize_q8x4 writes, all dot products are exact
// 8-bit integer dot products -- but laid out for a GPU:
//
//   * W stays in its GGUF super-block bytes (4.5 bits/weight Q4_K, 6.5625 Q6_K).  Q4_K blocks are
//     used as they are (144 B, 16-byte aligned).  Q6_K blocks (210 B, only 2-byte aligned) are split
//     once at load time into four planes of identical total size: ql[rows][nsb][128],
//     qh[rows][nsb][64], sc[rows][nsb][16], d[rows][nsb] -- every plane 16-byte aligned per block.
//   * one warp owns RPW rows; every lane streams 16 B of quants per row per step with a 128-bit
//     no-allocate load, so a warp request covers whole contiguous 512 B runs of the row;
//   * the activation words, their scales and (Q6_K) their half-block sums are staged once per CTA in
//     shared memory and reused by every row the CTA touches;
//   * lanes combine through one shuffle tree per row.
//
// Integer partial sums are exact; the fp32 scale products are summed in a different order from the
// reference's single-thread loop, so y agrees with it to fp32 rounding (tests bound it at 1e-5 of
// max|y|, the reference's own cross-compiler bar), not bit for bit.

#include "common.cuh"
#include "ops.h"

#include <algorithm>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

namespace kcb {
namespace {

constexpr unsigned kLo4 = 0x0F0F0F0Fu;
constexpr unsigned kHi2 = 0x30303030u;
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ int sbyte_of(unsigned w, int i) { return static_cast<int>(w << (24 - 8 * i)) >> 24; }

// ---- shared staging of the Q8 activation scratch ------------------------------------------------
// xw: packed int8 words as quantize_q8x4 wrote them; dx[b] = {d_b, d_b * sum_b}; s16[2b+h] = sum of
// the h-th 16 values of block b (Q6_K only).
template <bool kQ6>
__device__ __forceinline__ void stage_q8(const int* __restrict__ xq, const float* __restrict__ xd, int nsb, int* xw,
                                         float2* dx, int* s16) {
    const int nwords = nsb * 64, nb = nsb * 8;
    for (int i = threadIdx.x; i < nwords; i += kThreads) xw[i] = xq[i];
    for (int i = threadIdx.x; i < nb; i += kThreads) {
        const float d = xd[2 * i], s = xd[2 * i + 1];
        dx[i] = make_float2(d, __fmul_rn(d, s));
    }
    if (kQ6) {
        for (int i = threadIdx.x; i < nb * 2; i += kThreads) {
            int s = 0;
#pragma unroll
            for (int w = 0; w < 4; ++w) s = __dp4a(0x01010101, xq[i * 4 + w], s);
            s16[i] = s;
        }
    }
    __syncthreads();
}

// ---- Q4_K ---------------------------------------------------------------------------------------
// Lane (g, c8): super-block sb = 4*it + g, 16-byte chunk c8 of its 128 quant bytes.  Chunk c8 holds
// the low nibbles of sub-block 2j (weights 16h..16h+15) and the high nibbles of sub-block 2j+1, with
// j = c8 >> 1, h = c8 & 1.
struct Q4Regs {
    uint4 hd, q;
};

template <int RPW>
__global__ void __launch_bounds__(kThreads) matvec_q4k_q8_kernel(const uint8_t* __restrict__ w,
                                                                  const int* __restrict__ xq,
                                                                  const float* __restrict__ xd, float* __restrict__ y,
                                                                  int rows, int nsb) {
    extern __shared__ __align__(16) int sm[];
    int* xw = sm;
    float2* dx = reinterpret_cast<float2*>(sm + nsb * 64);
    stage_q8<false>(xq, xd, nsb, xw, dx, nullptr);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 3, c8 = lane & 7, j = c8 >> 1, h = c8 & 1;
    const size_t row_bytes = static_cast<size_t>(nsb) * kQ4KBlock;
    const int stride = gridDim.x * kWarps * RPW;

    for (int row0 = (blockIdx.x * kWarps + warp) * RPW; row0 < rows; row0 += stride) {
        float acc[RPW];
        Q4Regs nxt[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            acc[r] = 0.0f;
            if (row0 + r < rows && g < nsb) {
                const uint8_t* blk = w + (row0 + r) * row_bytes + static_cast<size_t>(g) * kQ4KBlock;
                nxt[r].hd = ldg_stream(blk);
                nxt[r].q = ldg_stream(blk + 16 + 16 * c8);
            }
        }
        for (int sb = g; sb < nsb; sb += 4) {
            Q4Regs cur[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) cur[r] = nxt[r];
            if (sb + 4 < nsb) {
#pragma unroll
                for (int r = 0; r < RPW; ++r)
                    if (row0 + r < rows) {
                        const uint8_t* blk = w + (row0 + r) * row_bytes + static_cast<size_t>(sb + 4) * kQ4KBlock;
                        nxt[r].hd = ldg_stream(blk);
                        nxt[r].q = ldg_stream(blk + 16 + 16 * c8);
                    }
            }
            const int b = sb * 8 + 2 * j;
            const uint4 xa = *reinterpret_cast<const uint4*>(xw + b * 8 + 4 * h);
            const uint4 xb = *reinterpret_cast<const uint4*>(xw + b * 8 + 8 + 4 * h);
            const float4 dd = *reinterpret_cast<const float4*>(dx + b);  // {d_b, d_b*sum_b, d_b+1, d_b+1*sum_b+1}
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                if (row0 + r >= rows) continue;
                const uint4 q = cur[r].q, hd = cur[r].hd;
                int da = 0, db = 0;
                da = __dp4a(static_cast<int>(q.x & kLo4), static_cast<int>(xa.x), da);
                da = __dp4a(static_cast<int>(q.y & kLo4), static_cast<int>(xa.y), da);
                da = __dp4a(static_cast<int>(q.z & kLo4), static_cast<int>(xa.z), da);
                da = __dp4a(static_cast<int>(q.w & kLo4), static_cast<int>(xa.w), da);
                db = __dp4a(static_cast<int>((q.x >> 4) & kLo4), static_cast<int>(xb.x), db);
                db = __dp4a(static_cast<int>((q.y >> 4) & kLo4), static_cast<int>(xb.y), db);
                db = __dp4a(static_cast<int>((q.z >> 4) & kLo4), static_cast<int>(xb.z), db);
                db = __dp4a(static_cast<int>((q.w >> 4) & kLo4), static_cast<int>(xb.w), db);
                // 6-bit scales/mins of sub-blocks 2j, 2j+1 out of the 12 packed bytes (words hd.y..hd.w)
                unsigned scw, mw;
                if (j < 2) {
                    scw = hd.y & 0x3F3F3F3Fu;
                    mw = hd.z & 0x3F3F3F3Fu;
                } else {
                    scw = (hd.w & kLo4) | ((hd.y >> 2) & kHi2);
                    mw = ((hd.w >> 4) & kLo4) | ((hd.z >> 2) & kHi2);
                }
                const int sh = 16 * (j & 1);
                const int sca = (scw >> sh) & 255, scb = (scw >> (sh + 8)) & 255;
                const float d = half_bits_to_float(hd.x & 0xFFFFu), dmin = half_bits_to_float(hd.x >> 16);
                float t = static_cast<float>(sca * da) * dd.x + static_cast<float>(scb * db) * dd.z;
                float part = d * t;
                if (h == 0) {  // the min term belongs to the whole sub-block: one lane of the pair adds it
                    const int ma = (mw >> sh) & 255, mb = (mw >> (sh + 8)) & 255;
                    part -= dmin * (static_cast<float>(ma) * dd.y + static_cast<float>(mb) * dd.w);
                }
                acc[r] += part;
            }
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const float s = warp_sum(acc[r]);
            if (lane == 0 && row0 + r < rows) y[row0 + r] = s;
        }
    }
}

// ---- Q6_K (planes) ------------------------------------------------------------------------------
// Lane (g, r8): super-block sb = 4*it + g; r8 = 4n + 2a + h picks the 16-byte chunk r8 of the block's
// 128 ql bytes: low nibbles are weights 16h..16h+15 of 32-block t = a of half n, high nibbles the same
// positions of block t = a + 2; both take their two high bits from qh bytes [32n + 16h, +16), shifted by
// 2t.  Each 16 weights share one int8 scale (index 8n + 2t + h).
struct Q6Regs {
    uint4 ql, qh;
    uint2 sc;
    unsigned d;
};

template <int RPW>
__global__ void __launch_bounds__(kThreads) matvec_q6k_q8_kernel(const uint8_t* __restrict__ w,
                                                                  const int* __restrict__ xq,
                                                                  const float* __restrict__ xd, float* __restrict__ y,
                                                                  int rows, int nsb, int rows_total) {
    extern __shared__ __align__(16) int sm[];
    int* xw = sm;
    float2* dx = reinterpret_cast<float2*>(sm + nsb * 64);
    int* s16 = sm + nsb * 64 + nsb * 16;
    stage_q8<true>(xq, xd, nsb, xw, dx, s16);

    const size_t nblk = static_cast<size_t>(rows_total) * nsb;
    const uint8_t* ql = w;
    const uint8_t* qh = w + nblk * 128;
    const uint8_t* sc = w + nblk * 192;
    const unsigned short* dp = reinterpret_cast<const unsigned short*>(w + nblk * 208);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 3, r8 = lane & 7, n = r8 >> 2, a = (r8 >> 1) & 1, h = r8 & 1;
    const int shl = 4 - 2 * a, shr = 2 * a, sci = 2 * a + h;
    const int stride = gridDim.x * kWarps * RPW;

    auto load = [&](Q6Regs& t, int row, int sb) {
        const size_t blk = static_cast<size_t>(row) * nsb + sb;
        t.ql = ldg_stream(ql + blk * 128 + 16 * r8);
        t.qh = ldg_stream(qh + blk * 64 + 32 * n + 16 * h);
        t.sc = __ldg(reinterpret_cast<const uint2*>(sc + blk * 16 + 8 * n));
        t.d = __ldg(dp + blk);
    };

    for (int row0 = (blockIdx.x * kWarps + warp) * RPW; row0 < rows; row0 += stride) {
        float acc[RPW];
        Q6Regs nxt[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            acc[r] = 0.0f;
            if (row0 + r < rows && g < nsb) load(nxt[r], row0 + r, g);
        }
        for (int sb = g; sb < nsb; sb += 4) {
            Q6Regs cur[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) cur[r] = nxt[r];
            if (sb + 4 < nsb) {
#pragma unroll
                for (int r = 0; r < RPW; ++r)
                    if (row0 + r < rows) load(nxt[r], row0 + r, sb + 4);
            }
            const int b = sb * 8 + 4 * n + a;  // 32-block of the low nibbles; the high nibbles' is b + 2
            const uint4 xa = *reinterpret_cast<const uint4*>(xw + b * 8 + 4 * h);
            const uint4 xb = *reinterpret_cast<const uint4*>(xw + (b + 2) * 8 + 4 * h);
            const float dxa = dx[b].x, dxb = dx[b + 2].x;
            const int sa = 32 * s16[2 * b + h], sb2 = 32 * s16[2 * (b + 2) + h];
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                if (row0 + r >= rows) continue;
                const uint4 l = cur[r].ql, hq = cur[r].qh;
                int dl = 0, dh = 0;
                dl = __dp4a(static_cast<int>((l.x & kLo4) | ((hq.x << shl) & kHi2)), static_cast<int>(xa.x), dl);
                dl = __dp4a(static_cast<int>((l.y & kLo4) | ((hq.y << shl) & kHi2)), static_cast<int>(xa.y), dl);
                dl = __dp4a(static_cast<int>((l.z & kLo4) | ((hq.z << shl) & kHi2)), static_cast<int>(xa.z), dl);
                dl = __dp4a(static_cast<int>((l.w & kLo4) | ((hq.w << shl) & kHi2)), static_cast<int>(xa.w), dl);
                dh = __dp4a(static_cast<int>(((l.x >> 4) & kLo4) | ((hq.x >> shr) & kHi2)), static_cast<int>(xb.x), dh);
                dh = __dp4a(static_cast<int>(((l.y >> 4) & kLo4) | ((hq.y >> shr) & kHi2)), static_cast<int>(xb.y), dh);
                dh = __dp4a(static_cast<int>(((l.z >> 4) & kLo4) | ((hq.z >> shr) & kHi2)), static_cast<int>(xb.z), dh);
                dh = __dp4a(static_cast<int>(((l.w >> 4) & kLo4) | ((hq.w >> shr) & kHi2)), static_cast<int>(xb.w), dh);
                const int tl = sbyte_of(cur[r].sc.x, sci) * (dl - sa);   // the -32 offset through the x sums
                const int th = sbyte_of(cur[r].sc.y, sci) * (dh - sb2);
                const float d = half_bits_to_float(cur[r].d);
                acc[r] += d * (static_cast<float>(tl) * dxa + static_cast<float>(th) * dxb);
            }
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const float s = warp_sum(acc[r]);
            if (lane == 0 && row0 + r < rows) y[row0 + r] = s;
        }
    }
}

// ---- fp32 activations: exact dequantised weight times x, fp32 accumulate --------------------------
// Same lane mapping; the weight is rebuilt exactly as the reference's dequantisers do
// (llm/llm_reference.cpp:342-383: separately rounded products) and multiplied with fp32 x from shared
// memory.  Slower than the integer path (one FMA per weight); it exists for callers that hold fp32
// activations and want the float product rather than the Q8 one.
__global__ void __launch_bounds__(kThreads) matvec_q4k_f32_kernel(const uint8_t* __restrict__ w,
                                                                   const float* __restrict__ x, float* __restrict__ y,
                                                                   int rows, int nsb) {
    extern __shared__ __align__(16) int sm[];
    float* xs = reinterpret_cast<float*>(sm);
    for (int i = threadIdx.x; i < nsb * 256; i += kThreads) xs[i] = x[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 3, c8 = lane & 7, j = c8 >> 1, h = c8 & 1;
    const size_t row_bytes = static_cast<size_t>(nsb) * kQ4KBlock;
    for (int row = blockIdx.x * kWarps + warp; row < rows; row += gridDim.x * kWarps) {
        float acc = 0.0f;
        for (int sb = g; sb < nsb; sb += 4) {
            const uint8_t* blk = w + row * row_bytes + static_cast<size_t>(sb) * kQ4KBlock;
            const uint4 hd = ldg_stream(blk);
            const uint4 q = ldg_stream(blk + 16 + 16 * c8);
            unsigned scw, mw;
            if (j < 2) {
                scw = hd.y & 0x3F3F3F3Fu;
                mw = hd.z & 0x3F3F3F3Fu;
            } else {
                scw = (hd.w & kLo4) | ((hd.y >> 2) & kHi2);
                mw = ((hd.w >> 4) & kLo4) | ((hd.z >> 2) & kHi2);
            }
            const int sh = 16 * (j & 1);
            const float d = half_bits_to_float(hd.x & 0xFFFFu), dmin = half_bits_to_float(hd.x >> 16);
            const float dl = __fmul_rn(d, static_cast<float>((scw >> sh) & 255));
            const float dh = __fmul_rn(d, static_cast<float>((scw >> (sh + 8)) & 255));
            const float ml = __fmul_rn(dmin, static_cast<float>((mw >> sh) & 255));
            const float mh = __fmul_rn(dmin, static_cast<float>((mw >> (sh + 8)) & 255));
            const float* xl = xs + sb * 256 + 64 * j + 16 * h;
            const unsigned qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int bq = 0; bq < 4; ++bq) {
                    const unsigned byte = (qw[i] >> (8 * bq)) & 255u;
                    const float wl = __fsub_rn(__fmul_rn(dl, static_cast<float>(byte & 15u)), ml);
                    const float wh = __fsub_rn(__fmul_rn(dh, static_cast<float>(byte >> 4)), mh);
                    acc = fmaf(wl, xl[4 * i + bq], acc);
                    acc = fmaf(wh, xl[32 + 4 * i + bq], acc);
                }
        }
        acc = warp_sum(acc);
        if (lane == 0) y[row] = acc;
    }
}

__global__ void __launch_bounds__(kThreads) matvec_q6k_f32_kernel(const uint8_t* __restrict__ w,
                                                                   const float* __restrict__ x, float* __restrict__ y,
                                                                   int rows, int nsb, int rows_total) {
    extern __shared__ __align__(16) int sm[];
    float* xs = reinterpret_cast<float*>(sm);
    for (int i = threadIdx.x; i < nsb * 256; i += kThreads) xs[i] = x[i];
    __syncthreads();
    const size_t nblk = static_cast<size_t>(rows_total) * nsb;
    const uint8_t* ql = w;
    const uint8_t* qh = w + nblk * 128;
    const uint8_t* sc = w + nblk * 192;
    const unsigned short* dp = reinterpret_cast<const unsigned short*>(w + nblk * 208);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 3, r8 = lane & 7, n = r8 >> 2, a = (r8 >> 1) & 1, h = r8 & 1;
    for (int row = blockIdx.x * kWarps + warp; row < rows; row += gridDim.x * kWarps) {
        float acc = 0.0f;
        for (int sb = g; sb < nsb; sb += 4) {
            const size_t blk = static_cast<size_t>(row) * nsb + sb;
            const uint4 l = ldg_stream(ql + blk * 128 + 16 * r8);
            const uint4 hq = ldg_stream(qh + blk * 64 + 32 * n + 16 * h);
            const uint2 s8 = __ldg(reinterpret_cast<const uint2*>(sc + blk * 16 + 8 * n));
            const float d = half_bits_to_float(__ldg(dp + blk));
            // d * float(sc) first, then * float(q): the reference's left-to-right product
            const float dsl = __fmul_rn(d, static_cast<float>(sbyte_of(s8.x, 2 * a + h)));
            const float dsh = __fmul_rn(d, static_cast<float>(sbyte_of(s8.y, 2 * a + h)));
            const float* xl = xs + sb * 256 + 128 * n + 32 * a + 16 * h;
            const unsigned lw[4] = {l.x, l.y, l.z, l.w}, hw[4] = {hq.x, hq.y, hq.z, hq.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int bq = 0; bq < 4; ++bq) {
                    const unsigned lb = (lw[i] >> (8 * bq)) & 255u, hb = (hw[i] >> (8 * bq)) & 255u;
                    const int q1 = static_cast<int>((lb & 15u) | (((hb >> (2 * a)) & 3u) << 4)) - 32;
                    const int q2 = static_cast<int>((lb >> 4) | (((hb >> (2 * a + 4)) & 3u) << 4)) - 32;
                    acc = fmaf(__fmul_rn(dsl, static_cast<float>(q1)), xl[4 * i + bq], acc);
                    acc = fmaf(__fmul_rn(dsh, static_cast<float>(q2)), xl[64 + 4 * i + bq], acc);
                }
        }
        acc = warp_sum(acc);
        if (lane == 0) y[row] = acc;
    }
}

// ---- bit-exact dequantisation to fp32 ------------------------------------------------------------
// One thread per 16-byte quant chunk (32 weights); products rounded separately, as the reference.
__global__ void dequant_q4k_kernel(const uint8_t* __restrict__ w, float* __restrict__ out, size_t nblk) {
    const size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= nblk * 8) return;
    const size_t blk = t >> 3;
    const int c8 = static_cast<int>(t & 7), j = c8 >> 1, h = c8 & 1;
    const uint8_t* p = w + blk * kQ4KBlock;
    const uint4 hd = *reinterpret_cast<const uint4*>(p);
    const uint4 q = *reinterpret_cast<const uint4*>(p + 16 + 16 * c8);
    unsigned scw, mw;
    if (j < 2) {
        scw = hd.y & 0x3F3F3F3Fu;
        mw = hd.z & 0x3F3F3F3Fu;
    } else {
        scw = (hd.w & kLo4) | ((hd.y >> 2) & kHi2);
        mw = ((hd.w >> 4) & kLo4) | ((hd.z >> 2) & kHi2);
    }
    const int sh = 16 * (j & 1);
    const float d = half_bits_to_float(hd.x & 0xFFFFu), dmin = half_bits_to_float(hd.x >> 16);
    const float dl = __fmul_rn(d, static_cast<float>((scw >> sh) & 255));
    const float dh = __fmul_rn(d, static_cast<float>((scw >> (sh + 8)) & 255));
    const float ml = __fmul_rn(dmin, static_cast<float>((mw >> sh) & 255));
    const float mh = __fmul_rn(dmin, static_cast<float>((mw >> (sh + 8)) & 255));
    float* o = out + blk * 256 + 64 * j + 16 * h;
    const unsigned qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int bq = 0; bq < 4; ++bq) {
            const unsigned byte = (qw[i] >> (8 * bq)) & 255u;
            o[4 * i + bq] = __fsub_rn(__fmul_rn(dl, static_cast<float>(byte & 15u)), ml);
            o[32 + 4 * i + bq] = __fsub_rn(__fmul_rn(dh, static_cast<float>(byte >> 4)), mh);
        }
}

__global__ void dequant_q6k_kernel(const uint8_t* __restrict__ w, float* __restrict__ out, size_t nblk) {
    const size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= nblk * 8) return;
    const size_t blk = t >> 3;
    const int r8 = static_cast<int>(t & 7), n = r8 >> 2, a = (r8 >> 1) & 1, h = r8 & 1;
    const uint4 l = *reinterpret_cast<const uint4*>(w + blk * 128 + 16 * r8);
    const uint4 hq = *reinterpret_cast<const uint4*>(w + nblk * 128 + blk * 64 + 32 * n + 16 * h);
    const uint2 s8 = *reinterpret_cast<const uint2*>(w + nblk * 192 + blk * 16 + 8 * n);
    const float d = half_bits_to_float(*reinterpret_cast<const unsigned short*>(w + nblk * 208 + blk * 2));
    const float dsl = __fmul_rn(d, static_cast<float>(sbyte_of(s8.x, 2 * a + h)));
    const float dsh = __fmul_rn(d, static_cast<float>(sbyte_of(s8.y, 2 * a + h)));
    float* o = out + blk * 256 + 128 * n + 32 * a + 16 * h;
    const unsigned lw[4] = {l.x, l.y, l.z, l.w}, hw[4] = {hq.x, hq.y, hq.z, hq.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int bq = 0; bq < 4; ++bq) {
            const unsigned lb = (lw[i] >> (8 * bq)) & 255u, hb = (hw[i] >> (8 * bq)) & 255u;
            const int q1 = static_cast<int>((lb & 15u) | (((hb >> (2 * a)) & 3u) << 4)) - 32;
            const int q2 = static_cast<int>((lb >> 4) | (((hb >> (2 * a + 4)) & 3u) << 4)) - 32;
            o[4 * i + bq] = __fmul_rn(dsl, static_cast<float>(q1));
            o[64 + 4 * i + bq] = __fmul_rn(dsh, static_cast<float>(q2));
        }
}

// ---- Q6_K: GGUF blocks <-> planes ----------------------------------------------------------------
// One thread per 2 bytes of a block (105 threads' worth); load-time only.
__global__ void q6k_planes_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, size_t nblk, int to_planes) {
    const size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= nblk * 105) return;
    const size_t blk = t / 105;
    const int o = static_cast<int>(t % 105) * 2;  // byte offset inside the 210-byte block
    size_t plane;
    if (o < 128) plane = blk * 128 + o;
    else if (o < 192) plane = nblk * 128 + blk * 64 + (o - 128);
    else if (o < 208) plane = nblk * 192 + blk * 16 + (o - 192);
    else plane = nblk * 208 + blk * 2;
    const size_t gg = blk * kQ6KBlock + o;
    if (to_planes) *reinterpret_cast<unsigned short*>(dst + plane) = *reinterpret_cast<const unsigned short*>(src + gg);
    else *reinterpret_cast<unsigned short*>(dst + gg) = *reinterpret_cast<const unsigned short*>(src + plane);
}

// ---- register-resident activations (k <= 4096) -----------------------------------------------------
// A lane's k-positions are fixed by its lane id, so for ITERS = ceil(nsb / 4) <= 4 the lane keeps its
// whole slice of the Q8 activations (words, scales, half-block sums) in registers for the life of the
// kernel: the row loop then holds nothing but the weight loads, the unpack and the dot products.  All
// loads of a row are issued before its arithmetic, and (PF) the next row's loads before this row's
// arithmetic, so every warp keeps 4-8 KB in flight.
template <int ITERS, bool PF>
__device__ __forceinline__ void matvec_q4k_q8_reg_body(const uint8_t* __restrict__ w, const int* __restrict__ xq,
                                                         const float* __restrict__ xd, float* __restrict__ y, int rows, int nsb,
                                                         int cta, int nctas) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 3, c8 = lane & 7, j = c8 >> 1, h = c8 & 1;
    const int sh = 16 * (j & 1);

    uint4 xa[ITERS], xb[ITERS];
    float4 dd[ITERS];  // {d_b, d_b * sum_b, d_b+1, d_b+1 * sum_b+1}; the min part is zero on h == 1 lanes
    bool ok[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int sb = 4 * it + g;
        ok[it] = sb < nsb;
        xa[it] = xb[it] = make_uint4(0, 0, 0, 0);
        dd[it] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ok[it]) {
            const int b = sb * 8 + 2 * j;
            xa[it] = __ldg(reinterpret_cast<const uint4*>(xq + b * 8 + 4 * h));
            xb[it] = __ldg(reinterpret_cast<const uint4*>(xq + b * 8 + 8 + 4 * h));
            const float4 t = __ldg(reinterpret_cast<const float4*>(xd + 2 * b));  // {d_b, sum_b, d_b+1, sum_b+1}
            dd[it] = make_float4(t.x, h == 0 ? __fmul_rn(t.x, t.y) : 0.f, t.z, h == 0 ? __fmul_rn(t.z, t.w) : 0.f);
        }
    }

    const size_t row_bytes = static_cast<size_t>(nsb) * kQ4KBlock;
    const int nwarps = nctas * kWarps;
    const uint8_t* lane_base = w + static_cast<size_t>(g) * kQ4KBlock;

    auto load = [&](Q4Regs (&t)[ITERS], int row) {
        const uint8_t* p = lane_base + row * row_bytes;
#pragma unroll
        for (int it = 0; it < ITERS; ++it)
            if (ok[it]) {
                t[it].hd = ldg_stream(p + it * 4 * kQ4KBlock);
                t[it].q = ldg_stream(p + it * 4 * kQ4KBlock + 16 + 16 * c8);
            }
    };
    auto compute = [&](const Q4Regs (&t)[ITERS]) {
        float acc = 0.0f;
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            if (!ok[it]) continue;
            const uint4 q = t[it].q, hd = t[it].hd;
            int da = 0, db = 0;
            da = __dp4a(static_cast<int>(q.x & kLo4), static_cast<int>(xa[it].x), da);
            da = __dp4a(static_cast<int>(q.y & kLo4), static_cast<int>(xa[it].y), da);
            da = __dp4a(static_cast<int>(q.z & kLo4), static_cast<int>(xa[it].z), da);
            da = __dp4a(static_cast<int>(q.w & kLo4), static_cast<int>(xa[it].w), da);
            db = __dp4a(static_cast<int>((q.x >> 4) & kLo4), static_cast<int>(xb[it].x), db);
            db = __dp4a(static_cast<int>((q.y >> 4) & kLo4), static_cast<int>(xb[it].y), db);
            db = __dp4a(static_cast<int>((q.z >> 4) & kLo4), static_cast<int>(xb[it].z), db);
            db = __dp4a(static_cast<int>((q.w >> 4) & kLo4), static_cast<int>(xb[it].w), db);
            unsigned scw, mw;
            if (j < 2) {
                scw = hd.y & 0x3F3F3F3Fu;
                mw = hd.z & 0x3F3F3F3Fu;
            } else {
                scw = (hd.w & kLo4) | ((hd.y >> 2) & kHi2);
                mw = ((hd.w >> 4) & kLo4) | ((hd.z >> 2) & kHi2);
            }
            const int sca = (scw >> sh) & 255, scb = (scw >> (sh + 8)) & 255;
            const int ma = (mw >> sh) & 255, mb = (mw >> (sh + 8)) & 255;
            const float d = half_bits_to_float(hd.x & 0xFFFFu), dmin = half_bits_to_float(hd.x >> 16);
            const float t1 = static_cast<float>(sca * da) * dd[it].x + static_cast<float>(scb * db) * dd[it].z;
            const float t2 = static_cast<float>(ma) * dd[it].y + static_cast<float>(mb) * dd[it].w;
            acc += d * t1 - dmin * t2;
        }
        return acc;
    };

    int row = cta * kWarps + warp;
    if (row >= rows) return;
    Q4Regs cur[ITERS];
    load(cur, row);
    for (; row < rows; row += nwarps) {
        float acc;
        if (PF) {
            Q4Regs nxt[ITERS];
            const int rn = row + nwarps;
            if (rn < rows) load(nxt, rn);
            acc = compute(cur);
#pragma unroll
            for (int it = 0; it < ITERS; ++it) cur[it] = nxt[it];
        } else {
            acc = compute(cur);
            if (row + nwarps < rows) load(cur, row + nwarps);
        }
        acc = warp_sum(acc);
        if (lane == 0) y[row] = acc;
    }
}
template <int ITERS, bool PF>
__global__ void __launch_bounds__(kThreads) matvec_q4k_q8_reg_kernel(const uint8_t* __restrict__ w,
                                                                      const int* __restrict__ xq,
                                                                      const float* __restrict__ xd,
                                                                      float* __restrict__ y, int rows, int nsb) {
    matvec_q4k_q8_reg_body<ITERS, PF>(w, xq, xd, y, rows, nsb, blockIdx.x, gridDim.x);
}

template <int ITERS, bool PF>
__device__ __forceinline__ void matvec_q6k_q8_reg_body(const uint8_t* __restrict__ w, const int* __restrict__ xq,
                                                         const float* __restrict__ xd, float* __restrict__ y, int rows, int nsb,
                                                         int cta, int nctas) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 3, r8 = lane & 7, n = r8 >> 2, a = (r8 >> 1) & 1, h = r8 & 1;
    const int shl = 4 - 2 * a, shr = 2 * a;
    // byte (2a + h) of a scale word, sign-extended, in one permute: selector nibbles {i, i|8, i|8, i|8}
    const unsigned sel = static_cast<unsigned>(2 * a + h) * 0x1111u | 0x8880u;

    uint4 xa[ITERS], xb[ITERS];
    float dxa[ITERS], dxb[ITERS];
    int sa[ITERS], sb2[ITERS];
    bool ok[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int sb = 4 * it + g;
        ok[it] = sb < nsb;
        xa[it] = xb[it] = make_uint4(0, 0, 0, 0);
        dxa[it] = dxb[it] = 0.f;
        sa[it] = sb2[it] = 0;
        if (ok[it]) {
            const int b = sb * 8 + 4 * n + a;
            xa[it] = __ldg(reinterpret_cast<const uint4*>(xq + b * 8 + 4 * h));
            xb[it] = __ldg(reinterpret_cast<const uint4*>(xq + (b + 2) * 8 + 4 * h));
            dxa[it] = __ldg(xd + 2 * b);
            dxb[it] = __ldg(xd + 2 * (b + 2));
            int s0 = 0, s1 = 0;
            s0 = __dp4a(0x01010101, static_cast<int>(xa[it].x), s0);
            s0 = __dp4a(0x01010101, static_cast<int>(xa[it].y), s0);
            s0 = __dp4a(0x01010101, static_cast<int>(xa[it].z), s0);
            s0 = __dp4a(0x01010101, static_cast<int>(xa[it].w), s0);
            s1 = __dp4a(0x01010101, static_cast<int>(xb[it].x), s1);
            s1 = __dp4a(0x01010101, static_cast<int>(xb[it].y), s1);
            s1 = __dp4a(0x01010101, static_cast<int>(xb[it].z), s1);
            s1 = __dp4a(0x01010101, static_cast<int>(xb[it].w), s1);
            sa[it] = 32 * s0;  // the -32 weight offset, applied through the activation sums
            sb2[it] = 32 * s1;
        }
    }

    const size_t nblk = static_cast<size_t>(rows) * nsb;
    const uint8_t* ql = w + static_cast<size_t>(g) * 128 + 16 * r8;
    const uint8_t* qh = w + nblk * 128 + static_cast<size_t>(g) * 64 + 32 * n + 16 * h;
    const uint8_t* sc = w + nblk * 192 + static_cast<size_t>(g) * 16 + 8 * n;
    const uint8_t* dp = w + nblk * 208 + static_cast<size_t>(g) * 2;
    const int nwarps = nctas * kWarps;

    auto load = [&](Q6Regs (&t)[ITERS], int row) {
        const size_t blk = static_cast<size_t>(row) * nsb;
#pragma unroll
        for (int it = 0; it < ITERS; ++it)
            if (ok[it]) {
                t[it].ql = ldg_stream(ql + (blk + 4 * it) * 128);
                t[it].qh = ldg_stream(qh + (blk + 4 * it) * 64);
                t[it].sc = __ldg(reinterpret_cast<const uint2*>(sc + (blk + 4 * it) * 16));
                t[it].d = __ldg(reinterpret_cast<const unsigned short*>(dp + (blk + 4 * it) * 2));
            }
    };
    auto compute = [&](const Q6Regs (&t)[ITERS]) {
        float acc = 0.0f;
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            if (!ok[it]) continue;
            const uint4 l = t[it].ql, hq = t[it].qh;
            int dl = 0, dh = 0;
            dl = __dp4a(static_cast<int>((l.x & kLo4) | ((hq.x << shl) & kHi2)), static_cast<int>(xa[it].x), dl);
            dl = __dp4a(static_cast<int>((l.y & kLo4) | ((hq.y << shl) & kHi2)), static_cast<int>(xa[it].y), dl);
            dl = __dp4a(static_cast<int>((l.z & kLo4) | ((hq.z << shl) & kHi2)), static_cast<int>(xa[it].z), dl);
            dl = __dp4a(static_cast<int>((l.w & kLo4) | ((hq.w << shl) & kHi2)), static_cast<int>(xa[it].w), dl);
            dh = __dp4a(static_cast<int>(((l.x >> 4) & kLo4) | ((hq.x >> shr) & kHi2)), static_cast<int>(xb[it].x), dh);
            dh = __dp4a(static_cast<int>(((l.y >> 4) & kLo4) | ((hq.y >> shr) & kHi2)), static_cast<int>(xb[it].y), dh);
            dh = __dp4a(static_cast<int>(((l.z >> 4) & kLo4) | ((hq.z >> shr) & kHi2)), static_cast<int>(xb[it].z), dh);
            dh = __dp4a(static_cast<int>(((l.w >> 4) & kLo4) | ((hq.w >> shr) & kHi2)), static_cast<int>(xb[it].w), dh);
            const int tl = prmt_sbyte(t[it].sc.x, sel) * (dl - sa[it]);
            const int th = prmt_sbyte(t[it].sc.y, sel) * (dh - sb2[it]);
            acc += half_bits_to_float(t[it].d) * (static_cast<float>(tl) * dxa[it] + static_cast<float>(th) * dxb[it]);
        }
        return acc;
    };

    int row = cta * kWarps + warp;
    if (row >= rows) return;
    Q6Regs cur[ITERS];
    load(cur, row);
    for (; row < rows; row += nwarps) {
        float acc;
        if (PF) {
            Q6Regs nxt[ITERS];
            const int rn = row + nwarps;
            if (rn < rows) load(nxt, rn);
            acc = compute(cur);
#pragma unroll
            for (int it = 0; it < ITERS; ++it) cur[it] = nxt[it];
        } else {
            acc = compute(cur);
            if (row + nwarps < rows) load(cur, row + nwarps);
        }
        acc = warp_sum(acc);
        if (lane == 0) y[row] = acc;
    }
}
template <int ITERS, bool PF>
__global__ void __launch_bounds__(kThreads) matvec_q6k_q8_reg_kernel(const uint8_t* __restrict__ w,
                                                                      const int* __restrict__ xq,
                                                                      const float* __restrict__ xd,
                                                                      float* __restrict__ y, int rows, int nsb) {
    matvec_q6k_q8_reg_body<ITERS, PF>(w, xq, xd, y, rows, nsb, blockIdx.x, gridDim.x);
}

// Two matrices on the same activations in one launch: CTAs [0, ctas4) run the Q4_K body on (w4, y4), the rest the
// Q6_K body on (w6, y6) -- the decoder's q|k and v projections in the Q4_K_M mix, which differ in format and
// would otherwise be two dependent launches.  Each half computes exactly what its own launch would.
template <int ITERS>
__global__ void __launch_bounds__(kThreads) matvec_q4k_q6k_pair_kernel(const uint8_t* __restrict__ w4, float* __restrict__ y4, int rows4,
                                                                       const uint8_t* __restrict__ w6, float* __restrict__ y6, int rows6,
                                                                       const int* __restrict__ xq, const float* __restrict__ xd, int nsb,
                                                                       int ctas4) {
    if (static_cast<int>(blockIdx.x) < ctas4)
        matvec_q4k_q8_reg_body<ITERS, true>(w4, xq, xd, y4, rows4, nsb, blockIdx.x, ctas4);
    else
        matvec_q6k_q8_reg_body<ITERS, true>(w6, xq, xd, y6, rows6, nsb, blockIdx.x - ctas4, gridDim.x - ctas4);
}

// ---- bulk-copy (TMA) pipelined kernels: the roofline path for large matrices --------------------------
// One persistent CTA per SM.  Tiles of TR consecutive rows are brought into a ring of shared-memory
// stages by cp.async.bulk (one copy per tile for Q4_K, one per plane for Q6_K), each stage completing
// on its own mbarrier; warp w of the CTA consumes row w of the tile straight out of shared memory with
// the same lane mapping as above and the activation slice held in registers.  With 4-5 stages of 28-40
// KB the SM keeps > 100 KB of weight bytes in flight no matter how the warps are scheduled, which is
// what HBM3e needs; the register-only kernels above top out near 65 % of the roofline.
// Stage reuse is ordered by one __syncthreads per tile: after it, thread 0 refills the stage just
// consumed.  Every mbarrier wait is bounded; on expiry the CTA records it in g_tma_timeouts and leaves.
__device__ unsigned g_tma_timeouts = 0;
// Cross-GPU waits (the step barrier below and the one fused into the sharded matvec) give up after g_peer_poll_limit
// polls (about a second by default), count the expiry and mark the group broken: later barriers still announce
// themselves but poll once, so a rank whose peer is gone returns at once instead of waiting out every step.
// peer_reset() clears both after the host has dealt with the failure.
__device__ unsigned g_peer_timeouts = 0;
__device__ unsigned g_peer_broken = 0;
__device__ unsigned g_peer_poll_limit = 1u << 22;

// Other ranks' gather buffers (already offset to this rank's first row), for the fused all-gather epilogue.
struct PeerOut {
    float* y[7] = {};
    int n = 0;
    // optional step barrier run by the last CTA to finish (world > 1): flags[i] = rank i's counters
    unsigned* flags[8] = {};
    unsigned* epoch_counter = nullptr;  // local device word, incremented once per launch
    unsigned* done_counter = nullptr;   // local device word, CTAs finished in this launch
    int rank = 0, world = 1;
};
constexpr unsigned kHi4 = 0xF0F0F0F0u;
// dot product of four unsigned bytes with four signed bytes, accumulated (the plain intrinsic takes both as signed)
__device__ __forceinline__ unsigned dp4a_u8s8(unsigned a, unsigned b, unsigned c) {
    unsigned d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
constexpr int kProlBytes = 5120;  // shared-memory room for an in-kernel Q8 copy of x (k <= 4096)

constexpr int kTmaMaxStages = 8;

template <bool kQ6, int ITERS, int TR, int RPW>
// The launch carries a programmatic dependency on the kernel before it in the stream: the first weight tiles are
// requested before griddepcontrol.wait (weights never depend on a preceding kernel), everything that reads the
// activations or writes results comes after it.  The activation pointers are therefore plain (no const __restrict__, no
// __ldg): the read-only data path is only defined for data that does not change while the kernel is resident, and under
// a programmatic dependency the kernel is resident while its predecessor may still be writing them.
__global__ void __launch_bounds__(TR / RPW * 32, 1) matvec_kq_q8_tma_kernel(const uint8_t* __restrict__ w, const int* xq, const float* xd, float* y,
                                                                             int rows, int nsb, int stages, PeerOut peers, const float* xf32) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float ytile[2][TR];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint8_t* buf = smem + 128 + kProlBytes;
    constexpr int kBlk = kQ6 ? kQ6KBlock : kQ4KBlock;
    constexpr int NW = TR / RPW;  // warps per CTA; warp w owns tile rows w, w + NW, ...
    const uint32_t stage_bytes = static_cast<uint32_t>(TR) * nsb * kBlk;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 3, c8 = lane & 7;
    const int ntiles = (rows + TR - 1) / TR;
    const int my_tiles = blockIdx.x < ntiles ? (ntiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const size_t nblk = static_cast<size_t>(rows) * nsb;

    auto issue = [&](int i) {  // thread 0 only
        const int s = i % stages;
        const int r0 = (blockIdx.x + i * gridDim.x) * TR;
        const int nr = min(TR, rows - r0);
        uint8_t* dst = buf + static_cast<size_t>(s) * stage_bytes;
        const size_t b0 = static_cast<size_t>(r0) * nsb;
        const uint32_t nb = static_cast<uint32_t>(nr) * nsb;
        mbar_expect_tx(&full[s], nb * kBlk);
        if (kQ6) {
            bulk_g2s(dst, w + b0 * 128, nb * 128, &full[s]);
            bulk_g2s(dst + TR * nsb * 128, w + nblk * 128 + b0 * 64, nb * 64, &full[s]);
            bulk_g2s(dst + TR * nsb * 192, w + nblk * 192 + b0 * 16, nb * 16, &full[s]);
            bulk_g2s(dst + TR * nsb * 208, w + nblk * 208 + b0 * 2, nb * 2, &full[s]);
        } else {
            bulk_g2s(dst, w + b0 * kQ4KBlock, nb * kQ4KBlock, &full[s]);
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
        mbar_init_fence();
        for (int i = 0; i < stages && i < my_tiles; ++i) issue(i);  // weights first: they depend on no preceding kernel
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next kernel may queue up behind this one
    asm volatile("griddepcontrol.wait;" ::: "memory");               // the preceding kernel's results from here on
    __syncthreads();                                                 // (the barriers are initialised for every thread)
    // fp32 activations (quantized below): groups of four blocks (128 values), group gi = warp + i * NW, one 16-byte
    // load per lane; their latency overlaps the weight tiles already in flight
    constexpr int kMaxPerWarp = (16 * 2 + NW - 1) / NW;  // nsb <= 16: at most 32 groups
    float4 xv[kMaxPerWarp];
    if (xf32) {
#pragma unroll
        for (int i = 0; i < kMaxPerWarp; ++i) {
            const int gi = warp + i * NW;
            xv[i] = gi < nsb * 2 ? *(reinterpret_cast<const float4*>(xf32) + gi * 32 + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }

    // fp32 activations: every CTA quantizes x itself (quantize_q8x4's arithmetic, one warp per block of 32) while
    // its first weight tiles are in flight; saves a launch and the scratch round trip.
    if (xf32) {
        int* sxq = reinterpret_cast<int*>(smem + 128);
        float* sxd = reinterpret_cast<float*>(sxq + nsb * 64);
#pragma unroll
        for (int i = 0; i < kMaxPerWarp; ++i) {
            const int gi = warp + i * NW;
            if (gi < nsb * 2) quantize_4blocks_warp(xv[i], sxq, sxd, gi * 4, lane);
        }
        __syncthreads();
        xq = sxq;
        xd = sxd;
    }

    // ---- this lane's slice of the activations, in registers ----
    // Q6_K: eight lanes per super-block (g = which of four super-blocks of a step, c8 = which 16 bytes of the low-nibble
    // plane), each warp takes its RPW rows one after the other.
    // Q4_K: FOUR lanes per super-block -- lane j4 owns the whole 32-byte chunk of sub-blocks 2 j4 and 2 j4 + 1 -- and the
    // two half-warps take the warp's two rows at the same time.  The 16-byte header of a block (d, dmin, twelve bytes of
    // 6-bit scales and mins) is then unpacked by four lanes per block instead of eight, per 64 weights instead of 32:
    // the kernel is bound by its integer instruction stream, not by memory, and this is a third of it.
    static_assert(kQ6 || RPW == 2, "the Q4_K lane mapping takes two rows per warp");
    uint4 xa[ITERS], xb[ITERS];
    uint4 xa1[kQ6 ? 1 : ITERS], xb1[kQ6 ? 1 : ITERS];  // Q4_K: the second 16 values of each of the two blocks
    float4 dd[ITERS];
    int sa[ITERS], sb2[ITERS];
    bool ok[ITERS];
    // Q4_K lane roles
    const int hw = lane >> 4, g4 = (lane >> 2) & 3, j = lane & 3, sh = 16 * (j & 1);
    // Q6_K lane roles
    const int h = c8 & 1;
    const int n = c8 >> 2, a = (c8 >> 1) & 1;
    const int shl = 4 - 2 * a, shr = 2 * a;
    const unsigned sel = static_cast<unsigned>(2 * a + h) * 0x1111u | 0x8880u;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int sb = 4 * it + (kQ6 ? g : g4);
        ok[it] = sb < nsb;
        xa[it] = xb[it] = make_uint4(0, 0, 0, 0);
        if (!kQ6) xa1[it] = xb1[it] = make_uint4(0, 0, 0, 0);
        dd[it] = make_float4(0.f, 0.f, 0.f, 0.f);
        sa[it] = sb2[it] = 0;
        if (!ok[it]) continue;
        if (kQ6) {
            const int b = sb * 8 + 4 * n + a;
            xa[it] = *reinterpret_cast<const uint4*>(xq + b * 8 + 4 * h);
            xb[it] = *reinterpret_cast<const uint4*>(xq + (b + 2) * 8 + 4 * h);
            dd[it].x = xd[2 * b];
            dd[it].z = xd[2 * (b + 2)];
            int s0 = 0, s1 = 0;
            s0 = __dp4a(0x01010101, static_cast<int>(xa[it].x), s0);
            s0 = __dp4a(0x01010101, static_cast<int>(xa[it].y), s0);
            s0 = __dp4a(0x01010101, static_cast<int>(xa[it].z), s0);
            s0 = __dp4a(0x01010101, static_cast<int>(xa[it].w), s0);
            s1 = __dp4a(0x01010101, static_cast<int>(xb[it].x), s1);
            s1 = __dp4a(0x01010101, static_cast<int>(xb[it].y), s1);
            s1 = __dp4a(0x01010101, static_cast<int>(xb[it].z), s1);
            s1 = __dp4a(0x01010101, static_cast<int>(xb[it].w), s1);
            sa[it] = 32 * s0;
            sb2[it] = 32 * s1;
        } else {
            const int b = sb * 8 + 2 * j;
            xa[it] = *reinterpret_cast<const uint4*>(xq + b * 8);
            xa1[it] = *reinterpret_cast<const uint4*>(xq + b * 8 + 4);
            xb[it] = *reinterpret_cast<const uint4*>(xq + b * 8 + 8);
            xb1[it] = *reinterpret_cast<const uint4*>(xq + b * 8 + 12);
            const float4 t = *reinterpret_cast<const float4*>(xd + 2 * b);
            dd[it] = make_float4(t.x, __fmul_rn(t.x, t.y), t.z, __fmul_rn(t.z, t.w));
        }
    }

    // one (row, super-block step) of work out of shared memory
    auto q6_step = [&](const uint8_t* st, int rl, int it) -> float {
        const size_t blk = static_cast<size_t>(rl) * nsb + g + 4 * it;
        const uint4 l = *reinterpret_cast<const uint4*>(st + blk * 128 + 16 * c8);
        const uint4 hq = *reinterpret_cast<const uint4*>(st + TR * nsb * 128 + blk * 64 + 32 * n + 16 * h);
        const uint2 sc = *reinterpret_cast<const uint2*>(st + TR * nsb * 192 + blk * 16 + 8 * n);
        const unsigned dq = *reinterpret_cast<const unsigned short*>(st + TR * nsb * 208 + blk * 2);
        int dl0 = 0, dl1 = 0, dh0 = 0, dh1 = 0;
        dl0 = __dp4a(static_cast<int>((l.x & kLo4) | ((hq.x << shl) & kHi2)), static_cast<int>(xa[it].x), dl0);
        dl1 = __dp4a(static_cast<int>((l.y & kLo4) | ((hq.y << shl) & kHi2)), static_cast<int>(xa[it].y), dl1);
        dl0 = __dp4a(static_cast<int>((l.z & kLo4) | ((hq.z << shl) & kHi2)), static_cast<int>(xa[it].z), dl0);
        dl1 = __dp4a(static_cast<int>((l.w & kLo4) | ((hq.w << shl) & kHi2)), static_cast<int>(xa[it].w), dl1);
        dh0 = __dp4a(static_cast<int>(((l.x >> 4) & kLo4) | ((hq.x >> shr) & kHi2)), static_cast<int>(xb[it].x), dh0);
        dh1 = __dp4a(static_cast<int>(((l.y >> 4) & kLo4) | ((hq.y >> shr) & kHi2)), static_cast<int>(xb[it].y), dh1);
        dh0 = __dp4a(static_cast<int>(((l.z >> 4) & kLo4) | ((hq.z >> shr) & kHi2)), static_cast<int>(xb[it].z), dh0);
        dh1 = __dp4a(static_cast<int>(((l.w >> 4) & kLo4) | ((hq.w >> shr) & kHi2)), static_cast<int>(xb[it].w), dh1);
        const int tl = prmt_sbyte(sc.x, sel) * (dl0 + dl1 - sa[it]);
        const int th = prmt_sbyte(sc.y, sel) * (dh0 + dh1 - sb2[it]);
        return half_bits_to_float(dq) * (static_cast<float>(tl) * dd[it].x + static_cast<float>(th) * dd[it].z);
    };
    // Q4_K: the lane's 64 weights of one block (sub-blocks 2 j and 2 j + 1: low and high nibbles of 32 bytes).  The high
    // nibbles stay in place (bytes 16 q): their dot product is an exact multiple of 16 and shifts back once.
    auto q4_step = [&](const uint8_t* st, int rl, int it) -> float {
        const uint8_t* pb = st + (static_cast<size_t>(rl) * nsb + g4 + 4 * it) * kQ4KBlock;
        const uint4 hd = *reinterpret_cast<const uint4*>(pb);
        const uint4 q0 = *reinterpret_cast<const uint4*>(pb + 16 + 32 * j);
        const uint4 q1 = *reinterpret_cast<const uint4*>(pb + 32 + 32 * j);
        int da0 = 0, da1 = 0, da2 = 0, da3 = 0;  // four short chains each
        unsigned db0 = 0, db1 = 0, db2 = 0, db3 = 0;
        da0 = __dp4a(static_cast<int>(q0.x & kLo4), static_cast<int>(xa[it].x), da0);
        da1 = __dp4a(static_cast<int>(q0.y & kLo4), static_cast<int>(xa[it].y), da1);
        da2 = __dp4a(static_cast<int>(q0.z & kLo4), static_cast<int>(xa[it].z), da2);
        da3 = __dp4a(static_cast<int>(q0.w & kLo4), static_cast<int>(xa[it].w), da3);
        db0 = dp4a_u8s8(q0.x & kHi4, xb[it].x, db0);
        db1 = dp4a_u8s8(q0.y & kHi4, xb[it].y, db1);
        db2 = dp4a_u8s8(q0.z & kHi4, xb[it].z, db2);
        db3 = dp4a_u8s8(q0.w & kHi4, xb[it].w, db3);
        da0 = __dp4a(static_cast<int>(q1.x & kLo4), static_cast<int>(xa1[it].x), da0);
        da1 = __dp4a(static_cast<int>(q1.y & kLo4), static_cast<int>(xa1[it].y), da1);
        da2 = __dp4a(static_cast<int>(q1.z & kLo4), static_cast<int>(xa1[it].z), da2);
        da3 = __dp4a(static_cast<int>(q1.w & kLo4), static_cast<int>(xa1[it].w), da3);
        db0 = dp4a_u8s8(q1.x & kHi4, xb1[it].x, db0);
        db1 = dp4a_u8s8(q1.y & kHi4, xb1[it].y, db1);
        db2 = dp4a_u8s8(q1.z & kHi4, xb1[it].z, db2);
        db3 = dp4a_u8s8(q1.w & kHi4, xb1[it].w, db3);
        da0 += da2, da1 += da3;
        db0 += db2, db1 += db3;
        const int db = static_cast<int>(db0 + db1) >> 4;
        unsigned scw, mw;
        if (j < 2) {
            scw = hd.y & 0x3F3F3F3Fu;
            mw = hd.z & 0x3F3F3F3Fu;
        } else {
            scw = (hd.w & kLo4) | ((hd.y >> 2) & kHi2);
            mw = ((hd.w >> 4) & kLo4) | ((hd.z >> 2) & kHi2);
        }
        const int sca = (scw >> sh) & 255, scb = (scw >> (sh + 8)) & 255;
        const int ma = (mw >> sh) & 255, mb = (mw >> (sh + 8)) & 255;
        const float d = half_bits_to_float(hd.x & 0xFFFFu), dmin = half_bits_to_float(hd.x >> 16);
        const float t1 = static_cast<float>(sca * (da0 + da1)) * dd[it].x + static_cast<float>(scb * db) * dd[it].z;
        const float t2 = static_cast<float>(ma) * dd[it].y + static_cast<float>(mb) * dd[it].w;
        return d * t1 - dmin * t2;
    };

    for (int i = 0; i < my_tiles; ++i) {
        const int s = i % stages;
        const uint32_t parity = static_cast<uint32_t>(i / stages) & 1u;
        if (!mbar_wait_bounded(&full[s], parity)) {
            if (lane == 0) atomicAdd(&g_tma_timeouts, 1u);
            for (int t = 0; t < 1000; ++t) __nanosleep(1000);  // bounded grace for copies still in flight
            // data never arrived: leave without touching y.  The CTA still counts as finished (once, by thread 0) so
            // that the last-CTA detection of this and every later launch stays right; it announces without waiting.
            if (threadIdx.x == 0 && peers.world > 1 && atomicAdd(peers.done_counter, 1u) == gridDim.x - 1) {
                atomicExch(peers.done_counter, 0u);
                const unsigned e = atomicAdd(peers.epoch_counter, 1u) + 1u;
                __threadfence_system();
                for (int r = 0; r < peers.world; ++r)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[r] + peers.rank), "r"(e) : "memory");
            }
            return;
        }
        const int row0 = (blockIdx.x + i * gridDim.x) * TR;
        const uint8_t* st = buf + static_cast<size_t>(s) * stage_bytes;
        if constexpr (kQ6) {
            float acc[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) acc[r] = 0.0f;
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                if (!ok[it]) continue;
#pragma unroll
                for (int r = 0; r < RPW; ++r) {
                    const int rl = warp + r * NW;
                    if (row0 + rl < rows) acc[r] += q6_step(st, rl, it);
                }
            }
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                const float v = warp_sum(acc[r]);
                const int row = row0 + warp + r * NW;
                if (lane == 0 && row < rows) {
                    y[row] = v;
                    ytile[i & 1][warp + r * NW] = v;
                }
            }
        } else {  // half-warp hw on tile row warp + hw * NW
            const int rl = warp + hw * NW;
            float acc = 0.0f;
            if (row0 + rl < rows) {
#pragma unroll
                for (int it = 0; it < ITERS; ++it)
                    if (ok[it]) acc += q4_step(st, rl, it);
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);  // within the half-warp
            if ((lane & 15) == 0 && row0 + rl < rows) {
                y[row0 + rl] = acc;
                ytile[i & 1][rl] = acc;
            }
        }
        __syncthreads();  // every warp is done with stage s
        if (threadIdx.x == 0 && i + stages < my_tiles) issue(i + stages);
        // fused all-gather: warp p stores the tile's TR results to rank p's gather buffer as one coalesced line (an
        // NVLink transaction per tile and peer instead of one per row).  ytile is double-buffered: tile i + 2 writes
        // this buffer only after the barrier of tile i + 1, which these warps reach after their stores.
        if (warp < peers.n && lane < TR && row0 + lane < rows) peers.y[warp][row0 + lane] = ytile[i & 1][lane];
    }
    // Step barrier across GPUs, run once per launch by whichever CTA finishes last: release this launch's epoch
    // into every rank's flag array, then wait (bounded) until every rank's epoch has arrived here.
    if (peers.world > 1) {
        __shared__ unsigned s_epoch;  // 0: another CTA finishes last
        // The last tile's peer stores are made by warps 0 .. peers.n - 1 after the loop's final barrier: this barrier
        // orders them before thread 0, whose system-scope fence is then cumulative over them -- a peer that sees the
        // new epoch sees every row of this CTA.
        if (threadIdx.x == 32) s_epoch = 0;  // thread 0 may have left on a timeout (it has then done the accounting)
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();  // this CTA's peer stores before its arrival
            unsigned e = 0;
            if (atomicAdd(peers.done_counter, 1u) == gridDim.x - 1) {
                atomicExch(peers.done_counter, 0u);
                e = atomicAdd(peers.epoch_counter, 1u) + 1u;  // epochs start at 1
            }
            s_epoch = e;
        }
        __syncthreads();
        const unsigned epoch = s_epoch;
        if (epoch != 0 && threadIdx.x < static_cast<unsigned>(peers.world)) {  // one thread per rank: announce and wait in parallel
            const int r = threadIdx.x;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[r] + peers.rank), "r"(epoch) : "memory");
            bool arrived = false;
            const unsigned limit = *reinterpret_cast<volatile unsigned*>(&g_peer_broken) ? 1u : *reinterpret_cast<volatile unsigned*>(&g_peer_poll_limit);
            for (unsigned it = 0; it < limit && !arrived; ++it) {
                unsigned v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(peers.flags[peers.rank] + r) : "memory");
                arrived = static_cast<int>(v - epoch) >= 0;
                if (!arrived) __nanosleep(64);
            }
            if (!arrived) {
                atomicAdd(&g_peer_timeouts, 1u);
                atomicExch(&g_peer_broken, 1u);
            }
        }
    }
}

template <bool kQ6, int ITERS, int TR, int RPW>
int launch_tma_cfg(const uint8_t* wb, const int* xq, const float* xd, float* y, int rows, int nsb, cudaStream_t s, const PeerOut& peers,
                   const float* xf32) {
    auto kern = matvec_kq_q8_tma_kernel<kQ6, ITERS, TR, RPW>;
    const size_t stage_bytes = static_cast<size_t>(TR) * nsb * (kQ6 ? kQ6KBlock : kQ4KBlock);
    int stages = static_cast<int>((226 * 1024 - 128 - kProlBytes) / stage_bytes);  // 227 KB of shared memory per CTA on sm_100
    if (stages > kTmaMaxStages) stages = kTmaMaxStages;
    if (stages < 2) return KCB_UNSUPPORTED_OPERATION;
    const size_t smem = 128 + kProlBytes + stages * stage_bytes;
    static PerDeviceFlag raised;  // per instantiation and device
    if (!raise_dynamic_smem(kern, 226 * 1024, raised)) return KCB_LAUNCH_FAILURE;
    const int ntiles = (rows + TR - 1) / TR;
    const int grid = ntiles < kSmCount ? ntiles : kSmCount;
    static const bool pdl = !(getenv("KCB_MATVEC_PDL") && atoi(getenv("KCB_MATVEC_PDL")) == 0);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid), cfg.blockDim = dim3(TR / RPW * 32), cfg.dynamicSmemBytes = smem, cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, wb, xq, xd, y, rows, nsb, stages, peers, xf32) == cudaSuccess ? KCB_SUCCESS : KCB_LAUNCH_FAILURE;
}

template <bool kQ6, int ITERS>
int launch_tma(const uint8_t* wb, const int* xq, const float* xd, float* y, int rows, int nsb, cudaStream_t s, const PeerOut& peers,
               const float* xf32) {
    // Measured on B200 (lm_head 128256 x 3072 Q6_K): 16 warps x 2 interleaved rows 94 % of the copy
    // roofline; 32 warps x 1 row 87 %; 16 warps x 1 row 82 %; 8 warps x 2 rows 71 %.
    return launch_tma_cfg<kQ6, ITERS, 32, 2>(wb, xq, xd, y, rows, nsb, s, peers, xf32);
}

template <bool kQ6>
int launch_tma_iters(const uint8_t* wb, const int* xq, const float* xd, float* y, int rows, int nsb, cudaStream_t s,
                     const PeerOut& peers = PeerOut{}, const float* xf32 = nullptr) {
    switch ((nsb + 3) / 4) {
    case 1: return launch_tma<kQ6, 1>(wb, xq, xd, y, rows, nsb, s, peers, xf32);
    case 2: return launch_tma<kQ6, 2>(wb, xq, xd, y, rows, nsb, s, peers, xf32);
    case 3: return launch_tma<kQ6, 3>(wb, xq, xd, y, rows, nsb, s, peers, xf32);
    case 4: return launch_tma<kQ6, 4>(wb, xq, xd, y, rows, nsb, s, peers, xf32);
    }
    return KCB_UNSUPPORTED_OPERATION;
}

// The pipelined path needs whole 8-row groups (16-byte aligned d plane tiles) and enough tiles to give
// every SM work.
bool use_tma(int rows, int nsb) { return rows % 8 == 0 && nsb <= 16 && rows >= 32 * kSmCount; }

// Resident CTAs per SM of a kernel: asked of the driver once per (kernel, shared-memory size, device), then cached.
template <class Kern>
int ctas_per_sm(Kern kern, size_t smem) {
    static std::mutex m;
    static std::map<std::tuple<const void*, size_t, int>, int> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    const auto key = std::make_tuple(reinterpret_cast<const void*>(kern), smem, dev);
    std::lock_guard<std::mutex> lock(m);
    const auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThreads, smem) != cudaSuccess || n < 1) n = 1;
    cache[key] = n;
    return n;
}

template <class Kern>
int grid_for(Kern kern, int rows, int rows_per_cta, size_t smem = 0) {
    const int need = (rows + rows_per_cta - 1) / rows_per_cta;
    const int cap = kSmCount * ctas_per_sm(kern, smem);
    return need < cap ? need : cap;
}

int grid_for_rows(int rows, int rpw) {
    const int need = (rows + kWarps * rpw - 1) / (kWarps * rpw);
    const int cap = kSmCount * 6;  // 6 CTAs of 8 warps per SM keep 48 warps streaming
    return need < 1 ? 1 : (need < cap ? need : cap);
}

bool shape_ok(int rows, int k) { return rows >= 0 && k > 0 && k % 256 == 0 && k <= 32768; }

}  // namespace

// ---- row-sharded matvec fused with its all-gather, and the cross-GPU step barrier --------------------
// One rank per GPU.  Rank r owns rows [r0, r0 + rows) of the matrix; its kernel writes every result both into
// its own full-length y and, with plain stores through NVLink peer mappings, into every other rank's y at the
// same offset -- the transfer rides on the matvec's own stores instead of a separate collective.
// peer_barrier then makes the step visible: each rank releases `epoch` into its slot of every peer's flag
// array and waits (bounded) until all its own slots reach `epoch`.

struct PeerFlags {
    unsigned* f[8] = {};
};

__global__ void peer_barrier_kernel(PeerFlags flags, int rank, int world, unsigned epoch, unsigned* epoch_counter) {
    __shared__ unsigned next;
    if (epoch_counter) {  // device-side step counter: the same launch can be replayed (CUDA graphs, one call per step)
        if (threadIdx.x == 0) next = atomicAdd(epoch_counter, 1u) + 1u;
        __syncthreads();
        epoch = next;
    }
    const int r = threadIdx.x;
    if (r >= world) return;
    __threadfence_system();  // order this GPU's earlier peer stores before the flag
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.f[r] + rank), "r"(epoch) : "memory");
    const unsigned* mine = flags.f[rank] + r;
    const unsigned limit = *reinterpret_cast<volatile unsigned*>(&g_peer_broken) ? 1u : *reinterpret_cast<volatile unsigned*>(&g_peer_poll_limit);
    for (unsigned i = 0; i < limit; ++i) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (static_cast<int>(v - epoch) >= 0) return;
        __nanosleep(64);
    }
    atomicAdd(&g_peer_timeouts, 1u);  // a peer never arrived: report and leave, nothing spins forever
    atomicExch(&g_peer_broken, 1u);
}

unsigned peer_timeouts() {
    unsigned v = 0;
    cudaMemcpyFromSymbol(&v, g_peer_timeouts, sizeof v);
    return v;
}
int peer_set_poll_limit(unsigned polls) {
    if (polls == 0) polls = 1u << 22;
    return cudaMemcpyToSymbol(g_peer_poll_limit, &polls, sizeof polls) == cudaSuccess ? KCB_SUCCESS : KCB_INTERNAL_ERROR;
}
int peer_reset() {
    const unsigned zero = 0;
    const bool ok = cudaMemcpyToSymbol(g_peer_timeouts, &zero, sizeof zero) == cudaSuccess && cudaMemcpyToSymbol(g_peer_broken, &zero, sizeof zero) == cudaSuccess;
    return ok ? KCB_SUCCESS : KCB_INTERNAL_ERROR;
}

int peer_barrier(unsigned* const* flags, int rank, int world, unsigned epoch, unsigned* epoch_counter, cudaStream_t s) {
    if (!flags || world < 1 || world > 8 || rank < 0 || rank >= world) return KCB_INVALID_VALUE;
    PeerFlags pf;
    for (int i = 0; i < world; ++i) {
        if (!flags[i]) return KCB_INVALID_VALUE;
        pf.f[i] = flags[i];
    }
    peer_barrier_kernel<<<1, 32, 0, s>>>(pf, rank, world, epoch, epoch_counter);
    return launch_status();
}

int matvec_q6k_q8_gather(const void* w, const int* xq, const float* xd, float* y_local, float* const* y_peers, int npeers, int rows,
                         int k, cudaStream_t s) {
    if (!shape_ok(rows, k) || !w || !xq || !xd || !y_local || npeers < 0 || npeers > 7 || (npeers && !y_peers)) return KCB_INVALID_VALUE;
    if (misaligned(w, 16) || misaligned(xq, 16) || misaligned(xd, 16) || misaligned(y_local, 4)) return KCB_INVALID_POINTER;
    if (rows == 0) return KCB_SUCCESS;
    const int nsb = k / 256;
    if (!(rows % 8 == 0 && nsb <= 16)) return KCB_UNSUPPORTED_OPERATION;
    PeerOut po;
    po.n = npeers;
    for (int i = 0; i < npeers; ++i) {
        if (!y_peers[i]) return KCB_INVALID_VALUE;
        po.y[i] = y_peers[i];
    }
    return launch_tma_iters<true>(static_cast<const uint8_t*>(w), xq, xd, y_local, rows, nsb, s, po);
}

// Row shard of a Q6_K matrix times fp32 x in ONE launch: in-kernel activation quantization, matvec, stores into
// the other ranks' outputs and the cross-GPU step barrier (world > 1).
int matvec_q6k_f32x_sharded(const void* w, const float* x, float* y_local, float* const* y_peers, int npeers, unsigned* const* flags,
                            unsigned* epoch_counter, unsigned* done_counter, int rank, int world, int rows, int k, cudaStream_t s) {
    if (!shape_ok(rows, k) || !w || !x || !y_local || npeers < 0 || npeers > 7 || (npeers && !y_peers) || world < 1 || world > 8 ||
        false)
        return KCB_INVALID_VALUE;
    if (misaligned(w, 16) || misaligned(x, 16) || misaligned(y_local, 4)) return KCB_INVALID_POINTER;  // x is read with 16-byte loads
    if (rows == 0) return KCB_SUCCESS;
    const int nsb = k / 256;
    if (!(rows % 8 == 0 && nsb <= 16)) return KCB_UNSUPPORTED_OPERATION;
    PeerOut po;
    po.n = npeers;
    for (int i = 0; i < npeers; ++i) po.y[i] = y_peers[i];
    if (world > 1) {
        if (!flags || !epoch_counter || !done_counter || rank < 0 || rank >= world) return KCB_INVALID_VALUE;
        for (int i = 0; i < world; ++i) po.flags[i] = flags[i];
        po.epoch_counter = epoch_counter, po.done_counter = done_counter, po.rank = rank, po.world = world;
    }
    return launch_tma_iters<true>(static_cast<const uint8_t*>(w), nullptr, nullptr, y_local, rows, nsb, s, po, x);
}

unsigned tma_timeouts() {
    unsigned v = 0;
    cudaMemcpyFromSymbol(&v, g_tma_timeouts, sizeof v);
    return v;
}

#define KCB_LAUNCH_REG(KERN, ITERS_)                                                                         \
    do {                                                                                                     \
        auto kern = KERN<ITERS_, true>;                                                                      \
        kern<<<grid_for(kern, rows, kWarps), kThreads, 0, s>>>(wb, xq, xd, y, rows, nsb);                    \
    } while (0)

// Matrices of up to 64 MB take the decode step's matvec kernel (decode_matvec.cu) with a programmatic dependency on the
// kernel before them in the stream: its weight tiles are requested before it waits for that kernel, and a run of
// such launches overlaps each one's ramp with its predecessor's tail (8192 x 3072 Q4_K: 5.7 us against 6.8 us per
// launch, 3072 x 8192 Q6_K: 7.2 against 9.3).  Larger matrices stream longer than a launch and stay on the kernels
// below.  KCB_MATVEC_DMV=0 switches the route off, =1 keeps it without the programmatic dependency.
static int dmv_mode(int rows, int k, bool q6) {
    static const int mode = getenv("KCB_MATVEC_DMV") ? atoi(getenv("KCB_MATVEC_DMV")) : 2;
    const size_t bytes = static_cast<size_t>(rows) * (k / 256) * (q6 ? kQ6KBlock : kQ4KBlock);
    if (!mode || bytes > (static_cast<size_t>(64) << 20) || !decode_matvec_shape_ok(q6 ? 0 : rows, q6 ? rows : 0, k)) return 0;
    return mode;
}

int matvec_q4k_q8(const void* w, const int* xq, const float* xd, float* y, int rows, int k, cudaStream_t s) {
    if (!shape_ok(rows, k) || !w || !xq || !xd || !y) return KCB_INVALID_VALUE;
    if (misaligned(w, 16) || misaligned(xq, 16) || misaligned(xd, 16) || misaligned(y, 4)) return KCB_INVALID_POINTER;
    if (rows == 0) return KCB_SUCCESS;
    const int nsb = k / 256, iters = (nsb + 3) / 4;
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    if (const int mode = dmv_mode(rows, k, false); mode) return decode_matvec_q8(w, y, rows, nullptr, nullptr, 0, k, xq, xd, mode == 2, s);
    if (use_tma(rows, nsb)) return launch_tma_iters<false>(wb, xq, xd, y, rows, nsb, s);
    if (iters <= 4) {
        switch (iters) {
        case 1: KCB_LAUNCH_REG(matvec_q4k_q8_reg_kernel, 1); break;
        case 2: KCB_LAUNCH_REG(matvec_q4k_q8_reg_kernel, 2); break;
        case 3: KCB_LAUNCH_REG(matvec_q4k_q8_reg_kernel, 3); break;
        default: KCB_LAUNCH_REG(matvec_q4k_q8_reg_kernel, 4); break;
        }
        return launch_status();
    }
    const size_t smem = static_cast<size_t>(nsb) * (64 * 4 + 8 * 8);
    if (rows >= kSmCount * 6 * kWarps * 2)
        matvec_q4k_q8_kernel<2><<<grid_for_rows(rows, 2), kThreads, smem, s>>>(wb, xq, xd, y, rows, nsb);
    else
        matvec_q4k_q8_kernel<1><<<grid_for_rows(rows, 1), kThreads, smem, s>>>(wb, xq, xd, y, rows, nsb);
    return launch_status();
}

int matvec_q6k_q8(const void* w, const int* xq, const float* xd, float* y, int rows, int k, cudaStream_t s) {
    if (!shape_ok(rows, k) || !w || !xq || !xd || !y) return KCB_INVALID_VALUE;
    if (misaligned(w, 16) || misaligned(xq, 16) || misaligned(xd, 16) || misaligned(y, 4)) return KCB_INVALID_POINTER;
    if (rows == 0) return KCB_SUCCESS;
    const int nsb = k / 256, iters = (nsb + 3) / 4;
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    if (const int mode = dmv_mode(rows, k, true); mode) return decode_matvec_q8(nullptr, nullptr, 0, w, y, rows, k, xq, xd, mode == 2, s);
    if (use_tma(rows, nsb)) return launch_tma_iters<true>(wb, xq, xd, y, rows, nsb, s);
    if (iters <= 4) {
        switch (iters) {
        case 1: KCB_LAUNCH_REG(matvec_q6k_q8_reg_kernel, 1); break;
        case 2: KCB_LAUNCH_REG(matvec_q6k_q8_reg_kernel, 2); break;
        case 3: KCB_LAUNCH_REG(matvec_q6k_q8_reg_kernel, 3); break;
        default: KCB_LAUNCH_REG(matvec_q6k_q8_reg_kernel, 4); break;
        }
        return launch_status();
    }
    const size_t smem = static_cast<size_t>(nsb) * (64 * 4 + 8 * 8 + 16 * 4);
    if (rows >= kSmCount * 6 * kWarps * 2)
        matvec_q6k_q8_kernel<2><<<grid_for_rows(rows, 2), kThreads, smem, s>>>(wb, xq, xd, y, rows, nsb, rows);
    else
        matvec_q6k_q8_kernel<1><<<grid_for_rows(rows, 1), kThreads, smem, s>>>(wb, xq, xd, y, rows, nsb, rows);
    return launch_status();
}

// q|k-style pair: a Q4_K matrix and a Q6_K matrix (planes) on the same Q8 activations in one launch.  Only for the
// register-resident kernels (k <= 4096) and matrices of at most 6144 rows; otherwise KCB_UNSUPPORTED_OPERATION and
// the caller launches them one after the other.
int matvec_q4k_q6k_pair_q8(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, const int* xq, const float* xd, int k,
                           cudaStream_t s) {
    if (!shape_ok(rows4, k) || !shape_ok(rows6, k) || !w4 || !w6 || !y4 || !y6 || !xq || !xd) return KCB_INVALID_VALUE;
    if (misaligned(w4, 16) || misaligned(w6, 16) || misaligned(xq, 16) || misaligned(xd, 16) || misaligned(y4, 4) || misaligned(y6, 4))
        return KCB_INVALID_POINTER;
    const int nsb = k / 256, iters = (nsb + 3) / 4;
    // up to kPairMaxRows the launch saved is worth more than the bulk-copy kernel's better streaming (measured on a
    // 5120 x 4096 + 1024 x 4096 pair: +3.5 % tokens/s on the whole decode step)
    constexpr int kPairMaxRows = 6144;
    if (rows4 == 0 || rows6 == 0 || iters > 4 || rows4 > kPairMaxRows || rows6 > kPairMaxRows) return KCB_UNSUPPORTED_OPERATION;
    const uint8_t* b4 = static_cast<const uint8_t*>(w4);
    const uint8_t* b6 = static_cast<const uint8_t*>(w6);
    const int need4 = (rows4 + kWarps - 1) / kWarps, need6 = (rows6 + kWarps - 1) / kWarps;
#define KCB_LAUNCH_PAIR(ITERS_)                                                                                            \
    do {                                                                                                                   \
        auto kern = matvec_q4k_q6k_pair_kernel<ITERS_>;                                                                    \
        const int cap = kSmCount * ctas_per_sm(kern, 0);                                                                   \
        int c4 = need4, c6 = need6;                                                                                        \
        if (c4 + c6 > cap) { /* resident CTAs shared in proportion to the bytes each half streams */                      \
            const double f4 = static_cast<double>(rows4) * kQ4KBlock, f6 = static_cast<double>(rows6) * kQ6KBlock;         \
            c4 = std::max(1, std::min(need4, static_cast<int>(cap * f4 / (f4 + f6))));                                     \
            c6 = std::max(1, std::min(need6, cap - c4));                                                                   \
        }                                                                                                                  \
        kern<<<c4 + c6, kThreads, 0, s>>>(b4, y4, rows4, b6, y6, rows6, xq, xd, nsb, c4);                                  \
    } while (0)
    switch (iters) {
    case 1: KCB_LAUNCH_PAIR(1); break;
    case 2: KCB_LAUNCH_PAIR(2); break;
    case 3: KCB_LAUNCH_PAIR(3); break;
    default: KCB_LAUNCH_PAIR(4); break;
    }
#undef KCB_LAUNCH_PAIR
    return launch_status();
}

int matvec_q4k_f32(const void* w, const float* x, float* y, int rows, int k, cudaStream_t s) {
    if (!shape_ok(rows, k) || k > 12288 || !w || !x || !y) return KCB_INVALID_VALUE;
    if (misaligned(w, 16) || misaligned(x, 4) || misaligned(y, 4)) return KCB_INVALID_POINTER;
    if (rows == 0) return KCB_SUCCESS;
    matvec_q4k_f32_kernel<<<grid_for_rows(rows, 1), kThreads, static_cast<size_t>(k) * 4, s>>>(static_cast<const uint8_t*>(w), x, y, rows, k / 256);
    return launch_status();
}

int matvec_q6k_f32(const void* w, const float* x, float* y, int rows, int k, cudaStream_t s) {
    if (!shape_ok(rows, k) || k > 12288 || !w || !x || !y) return KCB_INVALID_VALUE;
    if (misaligned(w, 16) || misaligned(x, 4) || misaligned(y, 4)) return KCB_INVALID_POINTER;
    if (rows == 0) return KCB_SUCCESS;
    matvec_q6k_f32_kernel<<<grid_for_rows(rows, 1), kThreads, static_cast<size_t>(k) * 4, s>>>(static_cast<const uint8_t*>(w), x, y, rows, k / 256, rows);
    return launch_status();
}

int dequant_q4k(const void* w, float* out, int rows, int k, cudaStream_t s) {
    if (!shape_ok(rows, k) || !w || !out) return KCB_INVALID_VALUE;
    if (misaligned(w, 16) || misaligned(out, 4)) return KCB_INVALID_POINTER;
    const size_t nblk = static_cast<size_t>(rows) * (k / 256);
    if (nblk == 0) return KCB_SUCCESS;
    dequant_q4k_kernel<<<static_cast<unsigned>((nblk * 8 + 255) / 256), 256, 0, s>>>(static_cast<const uint8_t*>(w), out, nblk);
    return launch_status();
}

int dequant_q6k(const void* w, float* out, int rows, int k, cudaStream_t s) {
    if (!shape_ok(rows, k) || !w || !out) return KCB_INVALID_VALUE;
    if (misaligned(w, 16) || misaligned(out, 4)) return KCB_INVALID_POINTER;
    const size_t nblk = static_cast<size_t>(rows) * (k / 256);
    if (nblk == 0) return KCB_SUCCESS;
    dequant_q6k_kernel<<<static_cast<unsigned>((nblk * 8 + 255) / 256), 256, 0, s>>>(static_cast<const uint8_t*>(w), out, nblk);
    return launch_status();
}

int q6k_convert(const void* src, void* dst, int rows, int k, int to_planes, cudaStream_t s) {
    if (!shape_ok(rows, k) || !src || !dst) return KCB_INVALID_VALUE;
    if (misaligned(src, 2) || misaligned(dst, 2)) return KCB_INVALID_POINTER;  // moved two bytes at a time
    const size_t nblk = static_cast<size_t>(rows) * (k / 256);
    if (nblk == 0) return KCB_SUCCESS;
    q6k_planes_kernel<<<static_cast<unsigned>((nblk * 105 + 255) / 256), 256, 0, s>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), nblk, to_planes);
    return launch_status();
}

}  // namespace kcb
