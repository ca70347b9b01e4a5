// Matvecs of the single-sequence decode step with their producers folded in.
//
// A decode step of the reference (llm/llm_model.cpp:287-360) alternates small vector kernels (residual add + RMSNorm +
// quantize, SwiGLU + quantize, the merge of the attention partials + quantize) with the K-quant matvecs that consume
// their output (kernels/llm/matvec_q4k_q8.cu, matvec_q6k_q8.cu).  On a B200 every one of those launches is shorter than
// its own ramp, so here the vector kernel becomes the PROLOGUE of the matvec that reads it: every CTA recomputes the
// few-KB activation vector out of L2 straight into shared memory (same arithmetic, bit for bit, as the stand-alone
// kernels) and then streams its rows of the matrix.  Three more things make the chain of launches cheap:
//   * weights do not depend on the step's data, so each CTA requests its first weight tiles (bulk copies into a
//     shared-memory ring) BEFORE it waits for the preceding kernel (programmatic dependent launch): the matrix is
//     already arriving while the previous kernel drains;
//   * each kernel releases its dependents as soon as its own prologue is done;
//   * rows are dealt in tiles to one persistent CTA of 16 warps per SM with a ring of up to six tiles in 224 KB of shared
//     memory; wide matrices split a row's super-blocks over two (k <= 8192) or four (k <= 16384) warps so that a lane's
//     activation slice still fits in registers.  (Two CTAs of 8 warps and 110 KB per SM, so that the next kernel's CTAs sit beside this
//     one's and its weights arrive while this one computes, measured slower: 7.4 against 5.7 us on an 8192 x 3072
//     Q4_K matrix, 638 against 687 tokens/s on the Llama-3.2-3B-shape decode step in the same run.)
// (Having each CTA also ask the L2 for its share of the NEXT launch's matrix -- cp.async.bulk.prefetch.L2, right after its
// own first tiles or behind its own last one -- measured slower both ways: 816 and 798 against 840 tokens/s on the
// Llama-3.2-3B-shape step; the prefetches queue with the tiles the CTAs are waiting for.)
// The per-row arithmetic is that of the bulk-copy matvec in kquant_matvec.cu (integer dot products, the reference's
// fp32 scale products, one shuffle tree per row; Q4_K on four lanes per super-block where a CTA has three or more tiles,
// on eight where the launch is latency bound).  A q|k|v product can carry a tail that rotates the q and k pairs of each
// finished tile and appends k and v to the fp16 cache (DecodeRopeTail, ops.h); a gate|up product can carry one that turns
// each pair of gate / up tiles into a quantized block of SwiGLU values (DecodeSwigluTail): unlike the SwiGLU PROLOGUE of
// the down projection, which every CTA repeats for the whole vector, the tail computes each value once.  Every mbarrier
// wait is bounded; on expiry the CTA counts the event and leaves.

#include "common.cuh"
#include "ops.h"

#include <algorithm>
#include <cstdlib>

namespace kcb {
namespace {

constexpr unsigned kLo4 = 0x0F0F0F0Fu;
constexpr unsigned kHi4 = 0xF0F0F0F0u;
constexpr unsigned kHi2 = 0x30303030u;
// dot product of four unsigned bytes with four signed bytes, accumulated (the plain intrinsic takes both as signed)
__device__ __forceinline__ unsigned dp4a_u8s8(unsigned a, unsigned b, unsigned c) {
    unsigned d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
constexpr int kWarps = 16, kThreads = 32 * kWarps;
constexpr int kMaxStages = 6;
constexpr int kSmemBudget = 224 * 1024;  // per CTA: one CTA per SM
constexpr int kBarBytes = 128;

__device__ unsigned g_dmv_timeouts = 0;


struct DmvMat {
    const uint8_t* w = nullptr;  // Q4_K blocks or Q6_K planes of `rows` rows
    float* y = nullptr;
    int rows = 0;
    int row_off = 0;             // with a rotation tail: where this matrix's rows stand in q heads | k heads | v heads
};

// ---- prologues: the activation vector as Q8 blocks of 32 in shared memory ------------------------------------------
// Whatever the preceding kernels of the step produce is read with ordinary loads through pointers that are NOT declared
// const __restrict__: under a programmatic dependency this kernel is already running while its predecessor writes, and
// the read-only data path (ld.global.nc, which the compiler also picks for const __restrict__ pointers) is only defined
// for data that does not change during the kernel's lifetime.  Weights and norm vectors may use it.
// x_out = x_in + t (t may be null), then blocks of RMSNorm(x_out) * w.  The arithmetic of add_norm_q8_cta (common.cuh):
// sums of squares per 128 values by a warp butterfly, group sums added 32 apart in order, so the result does not depend
// on the CTA's size.  Only the CTA with `store` set writes x_out (all compute the same values).
template <int MAXIT>
__device__ __forceinline__ void pro_add_norm(const float* x_in, const float* t, float* x_out, bool store, const float* __restrict__ w, int* xq,
                                             float* xd, int n, float eps, float* gsum) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int groups = n / 128;
    float4 v[MAXIT], ww[MAXIT];
#pragma unroll
    for (int i = 0; i < MAXIT; ++i) {
        const int gi = warp + i * kWarps;
        v[i] = ww[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (gi < groups) {
            ww[i] = __ldg(reinterpret_cast<const float4*>(w + gi * 128) + lane);
            float4 a = *(reinterpret_cast<const float4*>(x_in + gi * 128) + lane);
            if (t) {
                const float4 b = *(reinterpret_cast<const float4*>(t + gi * 128) + lane);
                a = make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
            }
            if (store) *(reinterpret_cast<float4*>(x_out + gi * 128) + lane) = a;
            v[i] = a;
            const float p = __fadd_rn(__fadd_rn(__fmul_rn(a.x, a.x), __fmul_rn(a.y, a.y)), __fadd_rn(__fmul_rn(a.z, a.z), __fmul_rn(a.w, a.w)));
            const float s = warp_sum(p);
            if (lane == 0) gsum[gi] = s;
        }
    }
    __syncthreads();
    float tot = 0.0f;
    for (int g = lane; g < groups; g += 32) tot = __fadd_rn(tot, gsum[g]);
    const float r = rinv_rms(warp_sum(tot), n, eps);
#pragma unroll
    for (int i = 0; i < MAXIT; ++i) {
        const int gi = warp + i * kWarps;
        if (gi < groups)
            quantize_4blocks_warp(make_float4(__fmul_rn(__fmul_rn(v[i].x, r), ww[i].x), __fmul_rn(__fmul_rn(v[i].y, r), ww[i].y),
                                              __fmul_rn(__fmul_rn(v[i].z, r), ww[i].z), __fmul_rn(__fmul_rn(v[i].w, r), ww[i].w)),
                                  xq, xd, gi * 4, lane);
    }
}

// SwiGLU g / (1 + 2^(-g log2 e)) * u quantized per 32 (kernels/llm/silu_mul_q8x4.cu): one warp per block of 32, all of
// a lane's inputs requested before the first is used (one round trip to L2, not one per block).  n <= 32 * kWarps * MAXB.
template <int MAXB>
__device__ __forceinline__ void pro_swiglu(const float* g, const float* u, int* xq, float* xd, int n) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nb = n / 32;
    float gv[MAXB], uv[MAXB];
#pragma unroll
    for (int i = 0; i < MAXB; ++i) {
        const int b = warp + i * kWarps;
        gv[i] = b < nb ? g[b * 32 + lane] : 0.0f;  // (plain loads: see the note on the read-only path above)
        uv[i] = b < nb ? u[b * 32 + lane] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < MAXB; ++i) {
        const int b = warp + i * kWarps;
        if (b < nb) {
            const float e = exp2f(__fmul_rn(-gv[i], 1.44269504f));
            quantize_block_warp(__fmul_rn(__fdiv_rn(gv[i], __fadd_rn(1.0f, e)), uv[i]), xq, xd, b, lane);
        }
    }
}

// Merge of the split-KV attention partials {acc[hd], max, sum} per head and split, normalised and quantized per 32
// channels: one warp per block of 32 channels, weights 2^((max_s - max) log2 e) and sums in split order.
__device__ __forceinline__ void pro_combine(const float* part, int* xq, float* xd, int heads, int hd, int nsplit) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int b = warp; b < heads * hd / 32; b += kWarps) {
        const int h = b * 32 / hd, d = (b * 32) % hd + lane;
        const float* ph = part + static_cast<size_t>(h) * nsplit * (hd + 2);
        float ll = 0.0f, aa = 0.0f;
        if (nsplit <= 32) {
            float pv[32];
#pragma unroll
            for (int s = 0; s < 32; ++s) pv[s] = s < nsplit ? ph[s * (hd + 2) + d] : 0.0f;
            const float pm = lane < nsplit ? ph[lane * (hd + 2) + hd] : -INFINITY;
            const float pl = lane < nsplit ? ph[lane * (hd + 2) + hd + 1] : 0.0f;
            const float mm = warp_max(pm);
            const float wl = pm == -INFINITY ? 0.0f : exp2f((pm - mm) * 1.44269504f);
#pragma unroll
            for (int s = 0; s < 32; ++s) {
                const float wgt = __shfl_sync(0xffffffffu, wl, s), ls = __shfl_sync(0xffffffffu, pl, s);
                if (s < nsplit) {
                    ll = __fmaf_rn(ls, wgt, ll);
                    aa = __fmaf_rn(pv[s], wgt, aa);
                }
            }
        } else {
            float mm = -INFINITY;
            for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, ph[s * (hd + 2) + hd]);
            for (int s = 0; s < nsplit; ++s) {
                const float pm = ph[s * (hd + 2) + hd];
                const float wgt = pm == -INFINITY ? 0.0f : exp2f((pm - mm) * 1.44269504f);
                ll = __fmaf_rn(ph[s * (hd + 2) + hd + 1], wgt, ll);
                aa = __fmaf_rn(ph[s * (hd + 2) + d], wgt, aa);
            }
        }
        quantize_block_warp(__fdiv_rn(aa, ll), xq, xd, b, lane);
    }
}

// Which tiles a CTA takes.  Plain: tiles cta, cta + nctas, ... of the matrix.  With a SwiGLU tail (sw_inter != 0): PAIRS
// cta, cta + nctas, ... -- even steps the pair's tile of gate rows, odd steps the tile of the same up rows.
__device__ __forceinline__ int dmv_my_tiles(int rows, int tr, int cta, int nctas, int sw_inter) {
    if (sw_inter) {
        const int np = sw_inter / tr;
        return cta < np ? 2 * ((np - 1 - cta) / nctas + 1) : 0;
    }
    const int nt = (rows + tr - 1) / tr;
    return cta < nt ? (nt - 1 - cta) / nctas + 1 : 0;
}
__device__ __forceinline__ int dmv_tile_row0(int i, int tr, int cta, int nctas, int sw_inter) {
    return sw_inter ? (i & 1) * sw_inter + (cta + (i >> 1) * nctas) * tr : (cta + i * nctas) * tr;
}

// ---- the matvec body --------------------------------------------------------------------------------------------------
// CTA `cta` of `nctas` takes tiles cta, cta + nctas, ... of TR rows.  KSPLIT warps share a row: warp w works on tile
// row (w % (kWarps / KSPLIT)) [+ multiples of that], super-blocks [ks * nsb / KSPLIT, (ks + 1) * nsb / KSPLIT) with
// ks = w / (kWarps / KSPLIT).  ITERS = ceil(nsb / KSPLIT / 4).
template <bool kQ6, int ITERS, int TR, int KSPLIT, bool kLanes4>
__device__ __forceinline__ void dmv_body(const DmvMat m, int nsb, const int* sxq, const float* sxd, uint64_t* full, uint8_t* buf, int stages, int cta,
                                         int nctas, float (*ytile)[TR * KSPLIT], const DecodeRopeTail& tail, const DecodeSwigluTail& sw) {
    constexpr int kBlk = kQ6 ? kQ6KBlock : kQ4KBlock;
    constexpr int NR = kWarps / KSPLIT;  // rows worked on at once (Q4_K: twice that, see below)
    constexpr int RPW = TR / NR;         // rows per warp and tile
    static_assert(TR % NR == 0 && RPW >= 1, "tile rows must be a multiple of the rows worked on at once");
    // Q4_K: four lanes per super-block (lane j owns the 32-byte chunk of sub-blocks 2 j and 2 j + 1) and the two
    // half-warps on two of the warp's rows at the same time, as in the streaming kernel (kquant_matvec.cu): the block
    // header is unpacked once per 64 weights.
    // With an odd number of rows per warp (16-row tiles on 16 warps) the half-warps share ONE row instead and split its
    // super-blocks, eight per step.
    // kLanes4 false keeps eight lanes per super-block for Q4_K as well (half a chunk each, rows one after the other): more
    // independent work per lane, which is what counts when a CTA has a tile or two and the launch is latency bound.
    constexpr bool kEight = kQ6 || !kLanes4;  // eight lanes per super-block
    constexpr bool kPair = !kEight && RPW % 2 == 0;
    constexpr int NIT = (kEight || kPair) ? ITERS : (ITERS + 1) / 2;  // steps of a lane over a row's super-blocks
    const int rows = m.rows;
    const uint32_t stage_bytes = static_cast<uint32_t>(TR) * nsb * kBlk;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 3, c8 = lane & 7;
    const int wr = warp % NR, ks = warp / NR;
    const int nsb_w = nsb / KSPLIT, sb_base = ks * nsb_w;
    const int sw_inter = (KSPLIT == 1 && TR == 32) ? sw.inter : 0;  // SwiGLU tail: whole Q8 blocks need 32-row tiles
    const int my_tiles = dmv_my_tiles(rows, TR, cta, nctas, sw_inter);
    const size_t nblk = static_cast<size_t>(rows) * nsb;
    const bool with_tail = KSPLIT == 1 && tail.hd != 0;  // results go through ytile and the rotation / cache tail
    const bool to_tile = with_tail || sw_inter != 0;     // results go to ytile only (a tail consumes them)

    auto issue = [&](int i) {  // thread 0 only; the kernel has already requested tiles 0 .. stages - 1
        const int s = i % stages;
        const int r0 = dmv_tile_row0(i, TR, cta, nctas, sw_inter);
        const int nr = min(TR, rows - r0);
        uint8_t* dst = buf + static_cast<size_t>(s) * stage_bytes;
        const size_t b0 = static_cast<size_t>(r0) * nsb;
        const uint32_t nb = static_cast<uint32_t>(nr) * nsb;
        mbar_expect_tx(&full[s], nb * kBlk);
        if (kQ6) {
            bulk_g2s(dst, m.w + b0 * 128, nb * 128, &full[s]);
            bulk_g2s(dst + TR * nsb * 128, m.w + nblk * 128 + b0 * 64, nb * 64, &full[s]);
            bulk_g2s(dst + TR * nsb * 192, m.w + nblk * 192 + b0 * 16, nb * 16, &full[s]);
            bulk_g2s(dst + TR * nsb * 208, m.w + nblk * 208 + b0 * 2, nb * 2, &full[s]);
        } else {
            bulk_g2s(dst, m.w + b0 * kQ4KBlock, nb * kQ4KBlock, &full[s]);
        }
    };
    // ---- this lane's slice of the activations, in registers ----
    uint4 xa[ITERS], xb[ITERS];
    uint4 xa1[kEight ? 1 : ITERS], xb1[kEight ? 1 : ITERS];  // four lanes: the second 16 values of each of the lane's two blocks
    float4 dd[ITERS];
    int sa[ITERS], sb2[ITERS];
    bool ok[ITERS];
    const int hw = lane >> 4, g4 = (lane >> 2) & 3;                  // Q4_K lane roles, four lanes per super-block
    const int j = kEight ? c8 >> 1 : lane & 3, sh = 16 * (j & 1);   // (eight lanes: chunk j, half h of it)
    const int h = c8 & 1, n = c8 >> 2, a = (c8 >> 1) & 1;                              // Q6_K lane roles
    const int shl = 4 - 2 * a, shr = 2 * a;
    const unsigned sel = static_cast<unsigned>(2 * a + h) * 0x1111u | 0x8880u;
    const auto q4_sb = [&](int it) { return kPair ? 4 * it + g4 : 8 * it + 4 * hw + g4; };  // the lane's super-block at step it
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int sbl = kEight ? 4 * it + g : q4_sb(it);
        ok[it] = sbl < nsb_w;
        xa[it] = xb[it] = make_uint4(0, 0, 0, 0);
        if (!kEight) xa1[it] = xb1[it] = make_uint4(0, 0, 0, 0);
        dd[it] = make_float4(0.f, 0.f, 0.f, 0.f);
        sa[it] = sb2[it] = 0;
        if (!ok[it]) continue;
        const int sb = sb_base + sbl;
        if (kQ6) {
            const int b = sb * 8 + 4 * n + a;
            xa[it] = *reinterpret_cast<const uint4*>(sxq + b * 8 + 4 * h);
            xb[it] = *reinterpret_cast<const uint4*>(sxq + (b + 2) * 8 + 4 * h);
            dd[it].x = sxd[2 * b];
            dd[it].z = sxd[2 * (b + 2)];
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
        } else {
            const int b = sb * 8 + 2 * j;
            const float4 t = *reinterpret_cast<const float4*>(sxd + 2 * b);
            if (kEight) {
                xa[it] = *reinterpret_cast<const uint4*>(sxq + b * 8 + 4 * h);
                xb[it] = *reinterpret_cast<const uint4*>(sxq + b * 8 + 8 + 4 * h);
                dd[it] = make_float4(t.x, h == 0 ? __fmul_rn(t.x, t.y) : 0.f, t.z, h == 0 ? __fmul_rn(t.z, t.w) : 0.f);
            } else {
                xa[it] = *reinterpret_cast<const uint4*>(sxq + b * 8);
                xa1[it] = *reinterpret_cast<const uint4*>(sxq + b * 8 + 4);
                xb[it] = *reinterpret_cast<const uint4*>(sxq + b * 8 + 8);
                xb1[it] = *reinterpret_cast<const uint4*>(sxq + b * 8 + 12);
                dd[it] = make_float4(t.x, __fmul_rn(t.x, t.y), t.z, __fmul_rn(t.z, t.w));
            }
        }
    }

    auto q6_step = [&](const uint8_t* st, int rl, int it) -> float {
        const size_t blk = static_cast<size_t>(rl) * nsb + sb_base + g + 4 * it;
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
    // eight lanes per super-block: the lane's 32 weights of one block (half a chunk)
    auto q4_step8 = [&](const uint8_t* st, int rl, int it) -> float {
        const uint8_t* pb = st + (static_cast<size_t>(rl) * nsb + sb_base + g + 4 * it) * kQ4KBlock;
        const uint4 hd = *reinterpret_cast<const uint4*>(pb);
        const uint4 q = *reinterpret_cast<const uint4*>(pb + 16 + 16 * c8);
        int da0 = 0, da1 = 0, db0 = 0, db1 = 0;
        da0 = __dp4a(static_cast<int>(q.x & kLo4), static_cast<int>(xa[it].x), da0);
        da1 = __dp4a(static_cast<int>(q.y & kLo4), static_cast<int>(xa[it].y), da1);
        da0 = __dp4a(static_cast<int>(q.z & kLo4), static_cast<int>(xa[it].z), da0);
        da1 = __dp4a(static_cast<int>(q.w & kLo4), static_cast<int>(xa[it].w), da1);
        db0 = __dp4a(static_cast<int>((q.x >> 4) & kLo4), static_cast<int>(xb[it].x), db0);
        db1 = __dp4a(static_cast<int>((q.y >> 4) & kLo4), static_cast<int>(xb[it].y), db1);
        db0 = __dp4a(static_cast<int>((q.z >> 4) & kLo4), static_cast<int>(xb[it].z), db0);
        db1 = __dp4a(static_cast<int>((q.w >> 4) & kLo4), static_cast<int>(xb[it].w), db1);
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
        const float t1 = static_cast<float>(sca * (da0 + da1)) * dd[it].x + static_cast<float>(scb * (db0 + db1)) * dd[it].z;
        const float t2 = static_cast<float>(ma) * dd[it].y + static_cast<float>(mb) * dd[it].w;
        return d * t1 - dmin * t2;
    };
    // four lanes: the lane's 64 weights of one block; the high nibbles stay in place (bytes 16 q) and their dot product, an exact
    // multiple of 16, shifts back once
    auto q4_step = [&](const uint8_t* st, int rl, int it) -> float {
        const uint8_t* pb = st + (static_cast<size_t>(rl) * nsb + sb_base + q4_sb(it)) * kQ4KBlock;
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
            if (lane == 0) atomicAdd(&g_dmv_timeouts, 1u);
            for (int t = 0; t < 1000; ++t) __nanosleep(1000);  // bounded grace for copies still in flight
            return;  // data never arrived: leave without touching y
        }
        const int row0 = dmv_tile_row0(i, TR, cta, nctas, sw_inter);
        const uint8_t* st = buf + static_cast<size_t>(s) * stage_bytes;
        if constexpr (kEight) {
            float acc[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) acc[r] = 0.0f;
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                if (!ok[it]) continue;
#pragma unroll
                for (int r = 0; r < RPW; ++r) {
                    const int rl = wr + r * NR;
                    if (row0 + rl < rows) acc[r] += kQ6 ? q6_step(st, rl, it) : q4_step8(st, rl, it);
                }
            }
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                const float v = warp_sum(acc[r]);
                const int rl = wr + r * NR;
                if (KSPLIT == 1 && !to_tile) {
                    if (lane == 0 && row0 + rl < rows) m.y[row0 + rl] = v;
                } else if (lane == 0) {
                    ytile[i & 3][ks * TR + rl] = v;  // four buffers: tile i + 4 writes this one only after the barriers of tiles i + 1 .. i + 3
                }
            }
        } else if constexpr (!kPair) {  // both half-warps on row wr + r NR, eight super-blocks per step
            float acc[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) acc[r] = 0.0f;
#pragma unroll
            for (int it = 0; it < NIT; ++it) {
                if (!ok[it]) continue;
#pragma unroll
                for (int r = 0; r < RPW; ++r) {
                    const int rl = wr + r * NR;
                    if (row0 + rl < rows) acc[r] += q4_step(st, rl, it);
                }
            }
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                const float v = warp_sum(acc[r]);
                const int rl = wr + r * NR;
                if (KSPLIT == 1 && !to_tile) {
                    if (lane == 0 && row0 + rl < rows) m.y[row0 + rl] = v;
                } else if (lane == 0) {
                    ytile[i & 3][ks * TR + rl] = v;
                }
            }
        } else {  // half-warp hw on rows wr + (2 p + hw) NR
            float acc[RPW / 2];
#pragma unroll
            for (int p = 0; p < RPW / 2; ++p) acc[p] = 0.0f;
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                if (!ok[it]) continue;
#pragma unroll
                for (int p = 0; p < RPW / 2; ++p) {
                    const int rl = wr + (2 * p + hw) * NR;
                    if (row0 + rl < rows) acc[p] += q4_step(st, rl, it);
                }
            }
#pragma unroll
            for (int p = 0; p < RPW / 2; ++p) {
                float v = acc[p];
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);  // within the half-warp
                const int rl = wr + (2 * p + hw) * NR;
                if ((lane & 15) != 0) continue;
                if (KSPLIT == 1 && !to_tile) {
                    if (row0 + rl < rows) m.y[row0 + rl] = v;
                } else {
                    ytile[i & 3][ks * TR + rl] = v;
                }
            }
        }
        __syncthreads();  // every warp is done with stage s (and the K shares of the tile's rows are in ytile)
        if (threadIdx.x == 0 && i + stages < my_tiles) issue(i + stages);
        if (KSPLIT == 1 && with_tail && threadIdx.x < TR / 2) {
            // the tile's rows sit in ytile: rotate the q and k pairs, append k and v to the cache (see DecodeRopeTail)
            const int r = row0 + 2 * static_cast<int>(threadIdx.x);
            if (r < rows) {
                const float x0 = ytile[i & 3][2 * threadIdx.x], x1 = ytile[i & 3][2 * threadIdx.x + 1];
                const int L = m.row_off + r, qd = tail.heads * tail.hd, kvd = tail.kv_heads * tail.hd;
                const int pos = min(*tail.pos_p, tail.max_ctx - 1);
                if (L >= qd + kvd) {  // v: cast and append
                    unsigned short* dst = tail.vc + static_cast<size_t>(pos) * kvd + (L - qd - kvd);
                    dst[0] = static_cast<unsigned short>(f32_to_f16_bits(x0));
                    dst[1] = static_cast<unsigned short>(f32_to_f16_bits(x1));
                } else {
                    float y0, y1;
                    rope_pair(x0, x1, (L % tail.hd) / 2, tail.hd / 2, pos, tail.log2_base, tail.ff, y0, y1);
                    if (L < qd) {
                        m.y[r] = y0;
                        m.y[r + 1] = y1;
                    } else {
                        unsigned short* dst = tail.kc + static_cast<size_t>(pos) * kvd + (L - qd);
                        dst[0] = static_cast<unsigned short>(f32_to_f16_bits(y0));
                        dst[1] = static_cast<unsigned short>(f32_to_f16_bits(y1));
                    }
                }
            }
        }
        if (sw_inter != 0 && (i & 1) && warp == 0) {
            // the pair is complete: gate rows in the buffer of tile i - 1, up rows in this tile's (see DecodeSwigluTail)
            const float gv = ytile[(i - 1) & 3][lane], uv = ytile[i & 3][lane];
            const float e = exp2f(__fmul_rn(-gv, 1.44269504f));
            quantize_block_warp(__fmul_rn(__fdiv_rn(gv, __fadd_rn(1.0f, e)), uv), sw.xq, sw.xd, cta + (i >> 1) * nctas, lane);
        }
        if (KSPLIT > 1 && threadIdx.x < TR && row0 + static_cast<int>(threadIdx.x) < rows) {
            float v = ytile[i & 3][threadIdx.x];
#pragma unroll
            for (int q = 1; q < KSPLIT; ++q) v = __fadd_rn(v, ytile[i & 3][q * TR + threadIdx.x]);  // shares added in K order
            m.y[row0 + threadIdx.x] = v;
        }
    }
}

struct DmvPro {
    // PRO 0: Q8 blocks given
    const int* xq = nullptr;
    const float* xd = nullptr;
    // PRO 1: x_out = x_in + t (t may be null), RMSNorm * wn
    const float* x_in = nullptr;
    const float* t = nullptr;
    float* x_out = nullptr;
    const float* wn = nullptr;
    float eps = 0.0f;
    // PRO 2: SwiGLU of g, u
    const float* g = nullptr;
    const float* u = nullptr;
    // PRO != 0: where one CTA leaves the int8 words the prologue produced (test instrumentation; null = nowhere)
    int* trace = nullptr;
    // PRO 3: merge of attention partials
    const float* part = nullptr;
    int heads = 0, hd = 0, nsplit = 0;
    // optional tail of a q|k|v product (hd == 0: none)
    DecodeRopeTail tail;
    // optional tail of a gate|up product (inter == 0: none)
    DecodeSwigluTail sw;
};

// One launch: matrix m4 (Q4_K) on CTAs [0, c4) and, when c6 > 0, matrix m6 (Q6_K planes) on CTAs [c4, c4 + c6), both on
// the same activations.  kQ6First: a single Q6_K matrix (m6 only, c4 == 0).
template <int ITERS, int TR, int KSPLIT, int PRO, bool kHas4, bool kHas6, bool kLanes4 = false>
__global__ void __launch_bounds__(kThreads, 1) dmv_kernel(const DmvMat m4, const DmvMat m6, int c4, int nsb, const DmvPro pro, int stages4, int stages6) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float ytile[4][TR * KSPLIT];
    __shared__ float gsum[64];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    int* sxq = reinterpret_cast<int*>(smem + kBarBytes);
    float* sxd = reinterpret_cast<float*>(sxq + nsb * 64);
    uint8_t* buf = smem + kBarBytes + ((nsb * 320 + 127) / 128) * 128;
    const bool is4 = kHas4 && (!kHas6 || static_cast<int>(blockIdx.x) < c4);
    const int cta = is4 ? blockIdx.x : blockIdx.x - c4;
    const int nctas = is4 ? (kHas6 ? c4 : gridDim.x) : gridDim.x - c4;
    const int stages = is4 ? stages4 : stages6;

    // weights first: they do not depend on anything the preceding kernels write
    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) mbar_init(&full[s], 1);
        mbar_init_fence();
        const DmvMat& m = is4 ? m4 : m6;
        const int blkb = is4 ? kQ4KBlock : kQ6KBlock;
        const int sw_inter = (KSPLIT == 1 && TR == 32) ? pro.sw.inter : 0;
        const int my_tiles = dmv_my_tiles(m.rows, TR, cta, nctas, sw_inter);
        const uint32_t stage_bytes = static_cast<uint32_t>(TR) * nsb * blkb;
        const size_t nblk = static_cast<size_t>(m.rows) * nsb;
        for (int i = 0; i < stages && i < my_tiles; ++i) {
            const int r0 = dmv_tile_row0(i, TR, cta, nctas, sw_inter);
            const int nr = min(TR, m.rows - r0);
            uint8_t* dst = buf + static_cast<size_t>(i) * stage_bytes;
            const size_t b0 = static_cast<size_t>(r0) * nsb;
            const uint32_t nb = static_cast<uint32_t>(nr) * nsb;
            mbar_expect_tx(&full[i], nb * blkb);
            if (!is4) {
                bulk_g2s(dst, m.w + b0 * 128, nb * 128, &full[i]);
                bulk_g2s(dst + TR * nsb * 128, m.w + nblk * 128 + b0 * 64, nb * 64, &full[i]);
                bulk_g2s(dst + TR * nsb * 192, m.w + nblk * 192 + b0 * 16, nb * 16, &full[i]);
                bulk_g2s(dst + TR * nsb * 208, m.w + nblk * 208 + b0 * 2, nb * 2, &full[i]);
            } else {
                bulk_g2s(dst, m.w + b0 * kQ4KBlock, nb * kQ4KBlock, &full[i]);
            }
        }
    }
    // from here on the preceding kernels' results are complete and visible (a no-op without a programmatic dependency)
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (PRO == 0) {
        for (int i = threadIdx.x; i < nsb * 64; i += kThreads) sxq[i] = pro.xq[i];
        for (int i = threadIdx.x; i < nsb * 16; i += kThreads) sxd[i] = pro.xd[i];
    } else if (PRO == 1) {
        pro_add_norm<4>(pro.x_in, pro.t, pro.x_out, blockIdx.x == 0, pro.wn, sxq, sxd, nsb * 256, pro.eps, gsum);
    } else if (PRO == 2) {
        pro_swiglu<(KSPLIT > 2 ? 32 : 16)>(pro.g, pro.u, sxq, sxd, nsb * 256);  // n <= 8192, 16384 with four warps per row
    } else {
        pro_combine(pro.part, sxq, sxd, pro.heads, pro.hd, pro.nsplit);
    }
    __syncthreads();
    if (PRO != 0 && pro.trace && blockIdx.x == 0)
        for (int i = threadIdx.x; i < nsb * 64; i += kThreads) pro.trace[i] = sxq[i];
    // this kernel's inputs are consumed: the next kernel may come up and request its weights
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (is4) {
        if constexpr (kHas4) dmv_body<false, ITERS, TR, KSPLIT, kLanes4>(m4, nsb, sxq, sxd, full, buf, stages, cta, nctas, ytile, pro.tail, pro.sw);
    } else {
        if constexpr (kHas6) dmv_body<true, ITERS, TR, KSPLIT, false>(m6, nsb, sxq, sxd, full, buf, stages, cta, nctas, ytile, pro.tail, pro.sw);
    }
}

template <class Kern>
int launch_dmv(Kern kern, int grid, size_t smem, bool pdl, cudaStream_t s, const DmvMat& m4, const DmvMat& m6, int c4, int nsb, const DmvPro& pro, int st4,
               int st6, PerDeviceFlag& raised) {
    if (!raise_dynamic_smem(kern, kSmemBudget, raised)) return KCB_LAUNCH_FAILURE;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = smem, cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, m4, m6, c4, nsb, pro, st4, st6) == cudaSuccess ? KCB_SUCCESS : KCB_LAUNCH_FAILURE;
}

int stages_for(int tiles_per_cta, size_t stage_bytes, size_t fixed) {
    int st = static_cast<int>((kSmemBudget - fixed) / stage_bytes);
    st = std::min(st, kMaxStages);
    return std::min(st, std::max(tiles_per_cta, 1));
}

// CTAs for the two matrices of a launch: the SMs shared in proportion to the bytes each streams.
void share_ctas(int t4, int t6, int rows4, int rows6, int& c4, int& c6) {
    c4 = c6 = 0;
    if (t4 && t6) {
        const double f4 = static_cast<double>(rows4) * kQ4KBlock, f6 = static_cast<double>(rows6) * kQ6KBlock;
        c4 = std::max(1, std::min(t4, static_cast<int>(kSmCount * f4 / (f4 + f6))));
        c6 = std::max(1, std::min(t6, kSmCount - c4));
    } else if (t4) {
        c4 = std::min(t4, kSmCount);
    } else {
        c6 = std::min(t6, kSmCount);
    }
}

// k <= 4096: TR-row tiles, one warp per TR / 8 rows, ITERS = ceil(nsb / 4).
template <int PRO, int TR>
int dmv_launch_narrow(const DmvMat& m4, const DmvMat& m6, int nsb, const DmvPro& pro, bool pdl, cudaStream_t s) {
    const size_t fixed = kBarBytes + static_cast<size_t>((nsb * 320 + 127) / 128) * 128;
    const bool has4 = m4.rows > 0, has6 = m6.rows > 0;
    const int t4 = (m4.rows + TR - 1) / TR, t6 = (m6.rows + TR - 1) / TR;
    int c4, c6;
    share_ctas(t4, t6, m4.rows, m6.rows, c4, c6);
    // SwiGLU tail (one matrix, 32-row tiles): the unit of work is a pair of tiles
    const int sw_pairs = (TR == 32 && pro.sw.inter) ? pro.sw.inter / TR : 0;
    if (sw_pairs) (has4 ? c4 : c6) = std::min(sw_pairs, kSmCount);
    const int per4 = !has4 ? 0 : sw_pairs ? 2 * ((sw_pairs + c4 - 1) / c4) : (t4 + c4 - 1) / c4;  // tiles of the busiest CTA
    const int per6 = !has6 ? 0 : sw_pairs ? 2 * ((sw_pairs + c6 - 1) / c6) : (t6 + c6 - 1) / c6;
    const int st4 = has4 ? stages_for(per4, static_cast<size_t>(TR) * nsb * kQ4KBlock, fixed) : 1;
    const int st6 = has6 ? stages_for(per6, static_cast<size_t>(TR) * nsb * kQ6KBlock, fixed) : 1;
    if (st4 < 1 || st6 < 1) return KCB_UNSUPPORTED_OPERATION;
    const size_t smem = fixed + std::max(has4 ? static_cast<size_t>(st4) * TR * nsb * kQ4KBlock : 0, has6 ? static_cast<size_t>(st6) * TR * nsb * kQ6KBlock : 0);
    // Q4_K with three or more tiles per CTA is bound by its instruction stream: four lanes per super-block; with fewer the
    // launch is latency bound and eight lanes (more independent work per lane) are faster (8192 x 3072: 5.6 against 5.9 us)
    const bool lanes4 = has4 && per4 >= 3;
#define KCB_DMV(ITERS_, H4, H6)                                                                                                            \
    do {                                                                                                                                   \
        static PerDeviceFlag raised, raised4;                                                                                              \
        if (H4 && lanes4)                                                                                                                  \
            return launch_dmv(dmv_kernel<ITERS_, TR, 1, PRO, H4, H6, H4>, c4 + c6, smem, pdl, s, m4, m6, c4, nsb, pro, st4, st6, raised4); \
        return launch_dmv(dmv_kernel<ITERS_, TR, 1, PRO, H4, H6, false>, c4 + c6, smem, pdl, s, m4, m6, c4, nsb, pro, st4, st6, raised);   \
    } while (0)
#define KCB_DMV_IT(H4, H6)          \
    switch ((nsb + 3) / 4) {        \
    case 1: KCB_DMV(1, H4, H6);     \
    case 2: KCB_DMV(2, H4, H6);     \
    case 3: KCB_DMV(3, H4, H6);     \
    default: KCB_DMV(4, H4, H6);    \
    }
    if (has4 && has6) { KCB_DMV_IT(true, true) }
    if (has4) { KCB_DMV_IT(true, false) }
    KCB_DMV_IT(false, true)
#undef KCB_DMV_IT
#undef KCB_DMV
}

// Row-times of a launch with TR-row tiles: rounds of the busiest CTA x rows per tile.
int row_times(int rows4, int rows6, int tr) {
    const int t4 = (rows4 + tr - 1) / tr, t6 = (rows6 + tr - 1) / tr;
    int c4, c6;
    share_ctas(t4, t6, rows4, rows6, c4, c6);
    const int r4 = t4 ? (t4 + c4 - 1) / c4 : 0, r6 = t6 ? (t6 + c6 - 1) / c6 : 0;
    return std::max(r4, r6) * tr;
}

// k in (8192, 16384], a multiple of 1024: 8-row tiles, four warps per row (at most 16 super-blocks each).
template <int PRO>
int dmv_launch_quad(const DmvMat& m4, const DmvMat& m6, int nsb, const DmvPro& pro, bool pdl, cudaStream_t s) {
    if (nsb > 64 || nsb % 4 || PRO == 1 || PRO == 3) return KCB_UNSUPPORTED_OPERATION;  // (no norm / merge prologue is that wide)
    constexpr int TR = 8;
    const bool has4 = m4.rows > 0;
    const size_t fixed = kBarBytes + static_cast<size_t>((nsb * 320 + 127) / 128) * 128;
    const int rows = has4 ? m4.rows : m6.rows;
    const int tiles = (rows + TR - 1) / TR, c = std::min(tiles, kSmCount);
    const size_t stage_bytes = static_cast<size_t>(TR) * nsb * (has4 ? kQ4KBlock : kQ6KBlock);
    const int st = stages_for((tiles + c - 1) / c, stage_bytes, fixed);
    if (st < 1) return KCB_UNSUPPORTED_OPERATION;
    const size_t smem = fixed + static_cast<size_t>(st) * stage_bytes;
    static PerDeviceFlag raised[4];
    const bool three = nsb <= 48;  // super-blocks per warp <= 12: three rounds of four
    if constexpr (PRO == 0 || PRO == 2) {
        if (has4) return three ? launch_dmv(dmv_kernel<3, TR, 4, PRO, true, false>, c, smem, pdl, s, m4, m6, c, nsb, pro, st, 1, raised[0])
                               : launch_dmv(dmv_kernel<4, TR, 4, PRO, true, false>, c, smem, pdl, s, m4, m6, c, nsb, pro, st, 1, raised[1]);
        return three ? launch_dmv(dmv_kernel<3, TR, 4, PRO, false, true>, c, smem, pdl, s, m4, m6, 0, nsb, pro, 1, st, raised[2])
                     : launch_dmv(dmv_kernel<4, TR, 4, PRO, false, true>, c, smem, pdl, s, m4, m6, 0, nsb, pro, 1, st, raised[3]);
    }
    return KCB_UNSUPPORTED_OPERATION;
}

template <int PRO>
int dmv_dispatch(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, int k, const DmvPro& pro, bool pdl, cudaStream_t s) {
    const int nsb = k / 256;
    DmvMat m4{static_cast<const uint8_t*>(w4), y4, rows4}, m6{static_cast<const uint8_t*>(w6), y6, rows6};
    m6.row_off = rows4;  // (read by the rotation tail only)
    if (pro.tail.hd != 0 && nsb > 16) return KCB_INVALID_VALUE;
    if (pro.sw.inter) return nsb <= 16 ? dmv_launch_narrow<PRO, 32>(m4, m6, nsb, pro, pdl, s) : KCB_INVALID_VALUE;
    if (nsb <= 16) {
        // 16-row tiles only where they balance the SMs clearly better (few tiles per CTA), else 32-row tiles, two rows per
        // warp: a row of twelve super-blocks on a half-warp is three full steps, on a whole warp two with a quarter of the
        // lanes idle in the second, and the 32-row tile has half the per-tile waits.  Measured per 27 KB of Q4_K, 0.65
        // against 0.85 us; 16384 x 3072 (7 rounds of 16 rows or 4 of 32): 9.6 against 10.2 us, the Llama-3.2-3B-shape
        // step 855 against 840 tokens/s.  KCB_DMV_TR16_BIAS sets the factor (1 = by rounds x rows alone).
        static const float bias = getenv("KCB_DMV_TR16_BIAS") ? static_cast<float>(atof(getenv("KCB_DMV_TR16_BIAS"))) : 1.15f;
        return row_times(rows4, rows6, 16) * bias < row_times(rows4, rows6, 32) ? dmv_launch_narrow<PRO, 16>(m4, m6, nsb, pro, pdl, s)
                                                                                 : dmv_launch_narrow<PRO, 32>(m4, m6, nsb, pro, pdl, s);
    }
    // k up to 8192: 8-row tiles, two warps per row (16 super-blocks each at most); up to 16384: four warps per row
    const bool has4 = rows4 > 0;
    if (rows4 > 0 && rows6 > 0) return KCB_UNSUPPORTED_OPERATION;
    if (nsb > 32) return dmv_launch_quad<PRO>(m4, m6, nsb, pro, pdl, s);
    if (nsb % 2) return KCB_UNSUPPORTED_OPERATION;
    constexpr int TR = 8;
    const size_t fixed = kBarBytes + static_cast<size_t>((nsb * 320 + 127) / 128) * 128;
    const int rows = has4 ? rows4 : rows6;
    const int tiles = (rows + TR - 1) / TR, c = std::min(tiles, kSmCount);
    const size_t stage_bytes = static_cast<size_t>(TR) * nsb * (has4 ? kQ4KBlock : kQ6KBlock);
    const int st = stages_for((tiles + c - 1) / c, stage_bytes, fixed);
    if (st < 1) return KCB_UNSUPPORTED_OPERATION;
    const size_t smem = fixed + static_cast<size_t>(st) * stage_bytes;
    static PerDeviceFlag raised4, raised6;
    if (has4) return launch_dmv(dmv_kernel<4, TR, 2, PRO, true, false>, c, smem, pdl, s, m4, m6, c, nsb, pro, st, 1, raised4);
    return launch_dmv(dmv_kernel<4, TR, 2, PRO, false, true>, c, smem, pdl, s, m4, m6, 0, nsb, pro, 1, st, raised6);
}

}  // namespace

unsigned decode_matvec_timeouts() {
    unsigned v = 0;
    cudaMemcpyFromSymbol(&v, g_dmv_timeouts, sizeof v);
    return v;
}

bool decode_matvec_shape_ok(int rows4, int rows6, int k) {
    if (k <= 0 || k % 256 || rows4 < 0 || rows6 < 0 || rows4 % 8 || rows6 % 8 || rows4 + rows6 == 0) return false;
    // (rows % 8 and an even number of super-blocks keep every Q6_K plane of a 4- or 8-row tile 16-byte aligned)
    const int nsb = k / 256;
    if (nsb <= 16) return true;
    if (rows4 && rows6) return false;
    return nsb <= 32 ? nsb % 2 == 0 : (nsb <= 64 && nsb % 4 == 0);  // (k > 8192: given Q8 blocks or the SwiGLU prologue only)
}

// y4 = W4 a, y6 = W6 a (either may be absent: rows 0) with the activation vector a produced by the prologue:
//   Q8 blocks given | x_out = x_in + t, RMSNorm(x_out) * wn | SwiGLU(g, u) | merge of attention partials.
// pdl: launch with a programmatic dependency on the preceding kernel of the stream.
int decode_matvec_q8(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, int k, const int* xq, const float* xd, bool pdl,
                     cudaStream_t s) {
    if (!decode_matvec_shape_ok(rows4, rows6, k) || !xq || !xd) return KCB_INVALID_VALUE;
    DmvPro p;
    p.xq = xq, p.xd = xd;
    return dmv_dispatch<0>(w4, y4, rows4, w6, y6, rows6, k, p, pdl, s);
}
int decode_matvec_norm(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, int k, const float* x_in, const float* t, float* x_out,
                       const float* wn, float eps, bool pdl, cudaStream_t s, int* trace, const DecodeRopeTail* tail, const DecodeSwigluTail* swiglu) {
    if (!decode_matvec_shape_ok(rows4, rows6, k) || k % 128 || k > 8192 || !x_in || !x_out || !wn) return KCB_INVALID_VALUE;
    if (misaligned(x_in, 16) || misaligned(t, 16) || misaligned(x_out, 16) || misaligned(wn, 16)) return KCB_INVALID_POINTER;
    DmvPro p;
    p.x_in = x_in, p.t = t, p.x_out = x_out, p.wn = wn, p.eps = eps, p.trace = trace;
    if (tail) {  // q heads | k heads | v heads over the rows of the Q4_K matrix and then the Q6_K one, whole heads each
        const int all = (tail->heads + 2 * tail->kv_heads) * tail->hd;
        if (k > 4096 || tail->hd <= 0 || tail->hd % 2 || rows4 + rows6 != all || rows4 % tail->hd || !tail->pos_p || !tail->kc || !tail->vc)
            return KCB_INVALID_VALUE;
        p.tail = *tail;
    }
    if (swiglu && swiglu->inter) {  // one matrix of gate rows then up rows, whole 32-row tiles each
        if (tail || k > 4096 || (rows4 && rows6) || swiglu->inter % 32 || rows4 + rows6 != 2 * swiglu->inter || !swiglu->xq || !swiglu->xd)
            return KCB_INVALID_VALUE;
        if (misaligned(swiglu->xq, 16) || misaligned(swiglu->xd, 8)) return KCB_INVALID_POINTER;
        p.sw = *swiglu;
    }
    return dmv_dispatch<1>(w4, y4, rows4, w6, y6, rows6, k, p, pdl, s);
}
int decode_matvec_swiglu(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, int k, const float* g, const float* u, bool pdl,
                         cudaStream_t s, int* trace) {
    if (!decode_matvec_shape_ok(rows4, rows6, k) || !g || !u) return KCB_INVALID_VALUE;
    DmvPro p;
    p.g = g, p.u = u, p.trace = trace;
    return dmv_dispatch<2>(w4, y4, rows4, w6, y6, rows6, k, p, pdl, s);
}
int decode_matvec_combine(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, int k, const float* part, int heads, int hd,
                          int nsplit, bool pdl, cudaStream_t s) {
    if (!decode_matvec_shape_ok(rows4, rows6, k) || !part || heads * hd != k || hd % 32 || nsplit < 1) return KCB_INVALID_VALUE;
    DmvPro p;
    p.part = part, p.heads = heads, p.hd = hd, p.nsplit = nsplit;
    return dmv_dispatch<3>(w4, y4, rows4, w6, y6, rows6, k, p, pdl, s);
}

}  // namespace kcb
