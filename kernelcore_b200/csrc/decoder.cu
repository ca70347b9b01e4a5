// Graph-replayed decoder: one CUDA graph per model, captured once and replayed for every token.
//
// The reference's decode loop (llm/llm_model.cpp:287-360) re-records ~450 launches per token because its
// kernels take the position by value.  Here every position-dependent kernel reads the position (and the
// input token) from device memory, the last kernel of a step picks the next token (greedy argmax) and
// advances the position, so the host only replays the same graph: no per-token capture, no host
// round trip between tokens.  Same arithmetic as the Backend path -- Q8 activations per 32, integer-dot
// matvecs, RMSNorm / RoPE / SwiGLU formulas of kernels/llm/*.cu -- with two deliberate layout changes:
// q|k and gate|up are stored as one matrix each when their formats agree (as the reference's fused
// Layer::wqkv / wgu, llm/llm_model.hpp:100-113), and the KV cache is fp16 rows [ctx][kv_heads*head_dim]
// (the ggml backend's cache, kernels/llm/set_rows_f16.cu, fa_*.cu) attended by a split-KV kernel with an
// online exp2 softmax.

#include "../../include/kernelcore_b200.h"

#include "common.cuh"
#include "ops.h"

#include <cooperative_groups.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

// Prompt attention: tokens per CTA and positions a lane group takes per step.  Measured on Qwen3-8B shapes, 4096-token
// prompt (tokens/s of the whole pass): 8 x 2: 7984, 4 x 2: 8628, 4 x 4: 8490, 2 x 4: 8670; the per-token kernel: 7152.
#ifndef KCB_PROMPT_TB
#define KCB_PROMPT_TB 4
#endif
#ifndef KCB_PROMPT_PS
#define KCB_PROMPT_PS 2
#endif
namespace kcb {
namespace {
namespace cg = cooperative_groups;

__device__ __forceinline__ int sbyte_of(unsigned w, int i) { return static_cast<int>(w << (24 - 8 * i)) >> 24; }

// x[hidden] = dequantised row `token` of a Q6_K (planes) or Q4_K matrix: the tied-embedding lookup
// (llm/gguf_model.cpp:96-104), bit-exact with llm::ref::dequantRowQ6K / Q4K.
__device__ __forceinline__ void embed_row(const uint8_t* __restrict__ w, size_t nblk, int nsb, int q6, int token, int t, float* __restrict__ x);

__global__ void embed_kernel(const uint8_t* __restrict__ w, size_t nblk, int nsb, int q6, int vocab,
                             const int* __restrict__ token_p, const int* __restrict__ forced, const int* __restrict__ n_forced,
                             const int* __restrict__ pos_p, int* token_used, float* __restrict__ x) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nsb * 8) return;
    const int pos = *pos_p;
    int token = pos < *n_forced ? forced[pos] : *token_p;
    token = min(max(token, 0), vocab - 1);
    if (t == 0) *token_used = token;
    embed_row(w, nblk, nsb, q6, token, t, x);
}
// Prompt form: row blockIdx.y of x is the embedding of tokens[blockIdx.y].
__global__ void embed_rows_kernel(const uint8_t* __restrict__ w, size_t nblk, int nsb, int q6, int vocab,
                                  const int* __restrict__ tokens, float* __restrict__ x) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nsb * 8) return;
    const int token = min(max(tokens[blockIdx.y], 0), vocab - 1);
    embed_row(w, nblk, nsb, q6, token, t, x + static_cast<size_t>(blockIdx.y) * nsb * 256);
}
__device__ __forceinline__ void embed_row(const uint8_t* __restrict__ w, size_t nblk, int nsb, int q6, int token, int t, float* __restrict__ x) {
    const size_t blk = static_cast<size_t>(token) * nsb + (t >> 3);
    const int c8 = t & 7;
    float* out = x + (t >> 3) * 256;
    if (q6) {
        const int n = c8 >> 2, a = (c8 >> 1) & 1, h = c8 & 1;
        const uint4 l = *reinterpret_cast<const uint4*>(w + blk * 128 + 16 * c8);
        const uint4 hq = *reinterpret_cast<const uint4*>(w + nblk * 128 + blk * 64 + 32 * n + 16 * h);
        const uint2 s8 = *reinterpret_cast<const uint2*>(w + nblk * 192 + blk * 16 + 8 * n);
        const float d = half_bits_to_float(*reinterpret_cast<const unsigned short*>(w + nblk * 208 + blk * 2));
        const float dsl = __fmul_rn(d, static_cast<float>(sbyte_of(s8.x, 2 * a + h)));
        const float dsh = __fmul_rn(d, static_cast<float>(sbyte_of(s8.y, 2 * a + h)));
        float* o = out + 128 * n + 32 * a + 16 * h;
        const unsigned lw[4] = {l.x, l.y, l.z, l.w}, hw[4] = {hq.x, hq.y, hq.z, hq.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const unsigned lb = (lw[i] >> (8 * b)) & 255u, hb = (hw[i] >> (8 * b)) & 255u;
                const int q1 = static_cast<int>((lb & 15u) | (((hb >> (2 * a)) & 3u) << 4)) - 32;
                const int q2 = static_cast<int>((lb >> 4) | (((hb >> (2 * a + 4)) & 3u) << 4)) - 32;
                o[4 * i + b] = __fmul_rn(dsl, static_cast<float>(q1));
                o[64 + 4 * i + b] = __fmul_rn(dsh, static_cast<float>(q2));
            }
    } else {
        const int j = c8 >> 1, h = c8 & 1;
        const uint8_t* p = w + blk * kQ4KBlock;
        const uint4 hd = *reinterpret_cast<const uint4*>(p);
        const uint4 q = *reinterpret_cast<const uint4*>(p + 16 + 16 * c8);
        unsigned scw, mw;
        if (j < 2) {
            scw = hd.y & 0x3F3F3F3Fu;
            mw = hd.z & 0x3F3F3F3Fu;
        } else {
            scw = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
            mw = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
        }
        const int sh = 16 * (j & 1);
        const float d = half_bits_to_float(hd.x & 0xFFFFu), dmin = half_bits_to_float(hd.x >> 16);
        const float dl = __fmul_rn(d, static_cast<float>((scw >> sh) & 255)), dh = __fmul_rn(d, static_cast<float>((scw >> (sh + 8)) & 255));
        const float ml = __fmul_rn(dmin, static_cast<float>((mw >> sh) & 255)), mh = __fmul_rn(dmin, static_cast<float>((mw >> (sh + 8)) & 255));
        float* o = out + 64 * j + 16 * h;
        const unsigned qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const unsigned byte = (qw[i] >> (8 * b)) & 255u;
                o[4 * i + b] = __fsub_rn(__fmul_rn(dl, static_cast<float>(byte & 15u)), ml);
                o[32 + 4 * i + b] = __fsub_rn(__fmul_rn(dh, static_cast<float>(byte >> 4)), mh);
            }
    }
}

// RoPE of q and k (+ optional per-head RMSNorm first) at the device-side position, K and V appended to the
// fp16 cache rows of that position.  One warp per head: q heads, then k heads, then v heads.
// kernels/llm/rope.cu:4-17 / rope_ff.cu / rope_ggml.cu:21-44 for the rotation, set_rows_f16.cu for the cast.
// Token blockIdx.y (decode: one) sits at position *pos_p + pos0 + blockIdx.y; its q|k heads are row blockIdx.y of
// qk (row stride qk_stride floats), its v heads row blockIdx.y of v.
__global__ void rope_kv_f16_kernel(float* qk, float* v, int qk_stride, int v_stride, const int* pos_p, int pos0,
                                   unsigned short* kc, unsigned short* vc, const float* __restrict__ ff,
                                   const float* __restrict__ qn, const float* __restrict__ kn, int heads, int kv_heads, int hd,
                                   float log2_base, int neox, float eps, int max_ctx, int seq_rows = 0) {
    // programmatic dependent launch (a no-op for ordinary launches): results of the preceding kernel from here on,
    // and the next kernel may come up and fetch what does not depend on this one
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (w >= heads + 2 * kv_heads) return;
    const int tok = blockIdx.y;
    // seq_rows != 0: a batch of independent sequences, token `tok` belongs to sequence `tok`, whose cache starts
    // seq_rows rows further on; all sequences stand at the same position
    const int pos = min((pos_p ? *pos_p : 0) + pos0 + (seq_rows ? 0 : tok), max_ctx - 1);
    const int kvdim = kv_heads * hd;
    kc += static_cast<size_t>(tok) * seq_rows * kvdim;
    vc += static_cast<size_t>(tok) * seq_rows * kvdim;
    float* base = w < heads + kv_heads ? qk + static_cast<size_t>(tok) * qk_stride + static_cast<size_t>(w) * hd
                                       : v + static_cast<size_t>(tok) * v_stride + static_cast<size_t>(w - heads - kv_heads) * hd;
    if (w >= heads + kv_heads) {  // v head: cast and store
        unsigned short* dst = vc + static_cast<size_t>(pos) * kvdim + static_cast<size_t>(w - heads - kv_heads) * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = static_cast<unsigned short>(f32_to_f16_bits(base[i]));
        return;
    }
    const float* wn = w < heads ? qn : kn;
    float r = 1.0f;
    if (wn) {
        float ss = 0.0f;
        for (int i = lane; i < hd; i += 32) ss += base[i] * base[i];
        ss = warp_sum(ss);
        r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(hd)), eps)));
    }
    const int pairs = hd / 2;
    unsigned short* kdst = w >= heads ? kc + static_cast<size_t>(pos) * kvdim + static_cast<size_t>(w - heads) * hd : nullptr;
    for (int p = lane; p < pairs; p += 32) {
        const int a = neox ? p : 2 * p, b = neox ? p + pairs : 2 * p + 1;
        float x0 = base[a], x1 = base[b];
        if (wn) {
            x0 = __fmul_rn(__fmul_rn(x0, r), wn[a]);
            x1 = __fmul_rn(__fmul_rn(x1, r), wn[b]);
        }
        float y0, y1;
        rope_pair(x0, x1, p, pairs, pos, log2_base, ff, y0, y1);
        if (kdst) {
            kdst[a] = static_cast<unsigned short>(f32_to_f16_bits(y0));
            kdst[b] = static_cast<unsigned short>(f32_to_f16_bits(y1));
        } else {
            base[a] = y0;
            base[b] = y1;
        }
    }
}

// Split-KV decode attention over the fp16 cache.  CTA (kvh, sp) covers positions [sp*chunk, (sp+1)*chunk) of
// kv head kvh for the G query heads that share it.  A warp scores four positions per step (8 lanes per
// position, HD/8 channels per lane), keeps an online exp2 softmax (running max m, sum l, weighted V sum)
// per lane group, and the CTA merges its groups into one partial {m, l, acc[HD]} per query head.
// Same quantities as kernels/llm/fa_scores.cu ... fa_values.cu: s = scale * q.k, p = 2^((s - max) log2 e),
// out = sum p v / sum p.
// Prompt form: blockIdx.z = token, whose query row is qkv + token * q_stride and whose position is
// *pos_p + pos0 + token (causal: it attends to the cache rows up to its own); with `direct` set (nsplit == 1)
// the normalised output goes straight to direct[token][heads * HD].
template <int HD, int G>
// (qkv, the cache and the position are written by preceding kernels of the same step, which may still be running when
// this one starts under a programmatic dependency: no const __restrict__, i.e. no read-only data path, on them)
__global__ void __launch_bounds__(128) attn_partial_kernel(const float* qkv, const unsigned short* kc, const unsigned short* vc, const int* pos_p,
                                                            float* part, int heads, int kv_heads, int nsplit,
                                                            float scale, int max_ctx, int q_stride, int pos0, float* __restrict__ direct,
                                                            int seq_rows = 0) {
    constexpr int DPL = HD / 8;  // channels per lane
    constexpr int NW = 4;
    extern __shared__ float sm[];  // [NW*4][G][HD + 2]
    asm volatile("griddepcontrol.wait;" ::: "memory");  // (see rope_kv_f16_kernel)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // blockIdx.x counts groups of G query heads; G == heads / kv_heads: one CTA per kv head, G == 1: one per query head
    const int h0 = blockIdx.x * G, kvh = h0 / (heads / kv_heads), sp = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, grp = lane >> 3, l8 = lane & 7;
    const int tok = blockIdx.z;
    const int ctx = min((pos_p ? *pos_p : 0) + pos0 + (seq_rows ? 0 : tok), max_ctx - 1) + 1;
    kc += static_cast<size_t>(tok) * seq_rows * kv_heads * HD;  // batch of sequences: this token's own cache
    vc += static_cast<size_t>(tok) * seq_rows * kv_heads * HD;
    part += static_cast<size_t>(tok) * heads * nsplit * (HD + 2);
    const int chunk = (ctx + nsplit - 1) / nsplit;
    const int t0 = sp * chunk, t1 = min(ctx, t0 + chunk);
    const int kvdim = kv_heads * HD;
    qkv += static_cast<size_t>(tok) * q_stride;

    float q[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < DPL; ++i) q[g][i] = qkv[static_cast<size_t>(h0 + g) * HD + l8 * DPL + i];
    float m[G], l[G], acc[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] = 0.0f;
    }
    // K/V rows are fetched one step ahead: the 16-byte loads of step i+1 are in flight while step i is scored
    constexpr int NV = DPL / 8;  // 16-byte loads per lane and row
    uint4 kn[NV], vn[NV];
    auto fetch = [&](int t) {
        if (t < t1) {
            const unsigned short* kr = kc + static_cast<size_t>(t) * kvdim + kvh * HD + l8 * DPL;
            const unsigned short* vr = vc + static_cast<size_t>(t) * kvdim + kvh * HD + l8 * DPL;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                kn[i] = *reinterpret_cast<const uint4*>(kr + 8 * i);
                vn[i] = *reinterpret_cast<const uint4*>(vr + 8 * i);
            }
        } else {
#pragma unroll
            for (int i = 0; i < NV; ++i) kn[i] = vn[i] = make_uint4(0u, 0u, 0u, 0u);
        }
    };
    fetch(t0 + warp * 4 + grp);
    for (int tb = t0 + warp * 4; tb < t1; tb += NW * 4) {  // warp-uniform trip count: every lane takes part in the shuffles
        const int t = tb + grp;
        const bool live = t < t1;
        float kf[DPL], vf[DPL];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const unsigned ku[4] = {kn[i].x, kn[i].y, kn[i].z, kn[i].w}, vu[4] = {vn[i].x, vn[i].y, vn[i].z, vn[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                kf[8 * i + 2 * j] = half_bits_to_float(ku[j] & 0xFFFFu);
                kf[8 * i + 2 * j + 1] = half_bits_to_float(ku[j] >> 16);
                vf[8 * i + 2 * j] = half_bits_to_float(vu[j] & 0xFFFFu);
                vf[8 * i + 2 * j + 1] = half_bits_to_float(vu[j] >> 16);
            }
        }
        fetch(t + NW * 4);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) s += q[g][i] * kf[i];
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (live) {
                s *= scale;
                const float mn = fmaxf(m[g], s);
                const float corr = exp2f((m[g] - mn) * 1.44269504f);
                const float p = exp2f((s - mn) * 1.44269504f);
                l[g] = l[g] * corr + p;
#pragma unroll
                for (int i = 0; i < DPL; ++i) acc[g][i] = acc[g][i] * corr + p * vf[i];
                m[g] = mn;
            }
        }
    }
    // lane groups -> shared memory
    float* mine = sm + static_cast<size_t>(warp * 4 + grp) * G * (HD + 2);
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) mine[g * (HD + 2) + l8 * DPL + i] = acc[g][i];
        if (l8 == 0) {
            mine[g * (HD + 2) + HD] = m[g];
            mine[g * (HD + 2) + HD + 1] = l[g];
        }
    }
    __syncthreads();
    for (int o = threadIdx.x; o < G * HD; o += blockDim.x) {
        const int g = o / HD, d = o % HD;
        float mm = -INFINITY;
        for (int pi = 0; pi < NW * 4; ++pi) mm = fmaxf(mm, sm[static_cast<size_t>(pi) * G * (HD + 2) + g * (HD + 2) + HD]);
        float ll = 0.0f, aa = 0.0f;
        for (int pi = 0; pi < NW * 4; ++pi) {
            const float* pp = sm + static_cast<size_t>(pi) * G * (HD + 2) + g * (HD + 2);
            const float wgt = pp[HD] == -INFINITY ? 0.0f : exp2f((pp[HD] - mm) * 1.44269504f);
            ll += pp[HD + 1] * wgt;
            aa += pp[d] * wgt;
        }
        if (direct) {
            direct[static_cast<size_t>(tok) * heads * HD + static_cast<size_t>(h0 + g) * HD + d] = __fdiv_rn(aa, ll);
            continue;
        }
        float* dst = part + (static_cast<size_t>(h0 + g) * nsplit + sp) * (HD + 2);
        dst[d] = aa;
        if (d == 0) {
            dst[HD] = mm;
            dst[HD + 1] = ll;
        }
    }
}

// One block of 32 attention outputs (a warp, one value per lane): the floats to attn and their quantize_q8x4 form -- words,
// scale and sum -- to the Q8 scratch the wo matvec reads.
__device__ __forceinline__ void attn_store_block_q8(float v, int b, int lane, float* attn, int* xq, float* xd) {
    attn[b * 32 + lane] = v;
    // quantize_q8x4 of this block
    const float amax = warp_max(fabsf(v));
    const float dq = __fdiv_rn(amax, 127.0f);
    const float id = dq > 0.0f ? __fdiv_rn(1.0f, dq) : 0.0f;
    const float t = __fmul_rn(v, id);
    int qi = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
    qi = max(-127, min(127, qi));
    const int sum = warp_sum_i(qi);
    unsigned word = (static_cast<unsigned>(qi) & 255u) << (8 * (lane & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if ((lane & 3) == 0) xq[b * 8 + (lane >> 2)] = static_cast<int>(word);
    if (lane == 0) {
        xd[b * 2] = dq;
        xd[b * 2 + 1] = static_cast<float>(sum);
    }
}

// Decode attention with the merge inside the launch: the kAttnCluster CTAs of a thread-block cluster split the positions
// of one kv head (CTA `rank` takes [rank * chunk, (rank + 1) * chunk), eight warps, one position per lane group and step,
// same online exp2 softmax as attn_partial_kernel), each leaves its partial {acc[G][HD], max, sum} in its own shared
// memory, and after one cluster barrier the warps of the cluster merge the partials through distributed shared memory --
// block b of 32 channels by warp b / kAttnCluster of CTA b % kAttnCluster, in split order with the arithmetic of
// attn_combine_q8_kernel -- and write attn and its Q8 form.  Against the two launches it replaces: no trip of the partials
// through L2, no second launch.  The position and the K / V rows of earlier steps do not depend on the kernel before
// (only the newest row and q do), so they are requested before griddepcontrol.wait.
constexpr int kAttnCluster = 8;
template <int HD, int G>
__global__ void __launch_bounds__(256) attn_decode_cluster_kernel(const float* qkv, const unsigned short* kc, const unsigned short* vc, const int* pos_p,
                                                                  float* attn, int* xq, float* xd, int heads, int kv_heads, float scale, int max_ctx) {
    constexpr int DPL = HD / 8, NW = 8, NV = DPL / 8, PW = HD + 2;
    extern __shared__ float sm[];              // [NW * 4][G][PW] lane-group partials, [G][PW] this CTA's partial, [G][32] weights
    float* cta_part = sm + NW * 4 * G * PW;
    cg::cluster_group cluster = cg::this_cluster();
    const int sp = static_cast<int>(cluster.block_rank());
    const int kvh = blockIdx.x / kAttnCluster, h0 = kvh * G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, grp = lane >> 3, l8 = lane & 7;
    // (*pos_p changes only in the step's last kernel, which is not launched with a programmatic dependency)
    const int ctx = min(*pos_p, max_ctx - 1) + 1;
    const int chunk = (ctx + kAttnCluster - 1) / kAttnCluster;
    const int t0 = sp * chunk, t1 = min(ctx, t0 + chunk);
    const int kvdim = kv_heads * HD;
    uint4 kn[NV], vn[NV];
    auto fetch = [&](int t, int limit) {
        if (t < limit) {
            const unsigned short* kr = kc + static_cast<size_t>(t) * kvdim + kvh * HD + l8 * DPL;
            const unsigned short* vr = vc + static_cast<size_t>(t) * kvdim + kvh * HD + l8 * DPL;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                kn[i] = *reinterpret_cast<const uint4*>(kr + 8 * i);
                vn[i] = *reinterpret_cast<const uint4*>(vr + 8 * i);
            }
        } else {
#pragma unroll
            for (int i = 0; i < NV; ++i) kn[i] = vn[i] = make_uint4(0u, 0u, 0u, 0u);
        }
    };
    const int first = t0 + warp * 4 + grp;
    fetch(first, min(t1, ctx - 1));  // rows of earlier steps: complete long before this step began
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (first == ctx - 1) fetch(first, t1);  // the row this step appended
    float q[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < DPL; ++i) q[g][i] = qkv[static_cast<size_t>(h0 + g) * HD + l8 * DPL + i];
    float m[G], l[G], acc[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] = 0.0f;
    }
    for (int tb = t0 + warp * 4; tb < t1; tb += NW * 4) {  // warp-uniform trip count
        const int t = tb + grp;
        const bool live = t < t1;
        float kf[DPL], vf[DPL];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const unsigned ku[4] = {kn[i].x, kn[i].y, kn[i].z, kn[i].w}, vu[4] = {vn[i].x, vn[i].y, vn[i].z, vn[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                kf[8 * i + 2 * j] = half_bits_to_float(ku[j] & 0xFFFFu);
                kf[8 * i + 2 * j + 1] = half_bits_to_float(ku[j] >> 16);
                vf[8 * i + 2 * j] = half_bits_to_float(vu[j] & 0xFFFFu);
                vf[8 * i + 2 * j + 1] = half_bits_to_float(vu[j] >> 16);
            }
        }
        fetch(t + NW * 4, t1);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) s += q[g][i] * kf[i];
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (live) {
                s *= scale;
                const float mn = fmaxf(m[g], s);
                const float corr = exp2f((m[g] - mn) * 1.44269504f);
                const float p = exp2f((s - mn) * 1.44269504f);
                l[g] = l[g] * corr + p;
#pragma unroll
                for (int i = 0; i < DPL; ++i) acc[g][i] = acc[g][i] * corr + p * vf[i];
                m[g] = mn;
            }
        }
    }
    // lane groups -> shared memory -> one partial per CTA
    float* mine = sm + static_cast<size_t>(warp * 4 + grp) * G * PW;
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) mine[g * PW + l8 * DPL + i] = acc[g][i];
        if (l8 == 0) {
            mine[g * PW + HD] = m[g];
            mine[g * PW + HD + 1] = l[g];
        }
    }
    __syncthreads();
    // warp g: the CTA-wide max of head g, every lane group's weight (lane = lane group) and the weighted sum of the sums,
    // once per head instead of once per output channel; then a channel is 32 multiply-adds in lane-group order
    static_assert(NW * 4 == 32 && G <= NW, "one lane per lane group, one warp per head of the group");
    float* wsm = cta_part + G * PW;  // [G][32]
    if (warp < G) {
        const float* pp = sm + lane * G * PW + warp * PW;
        const float pm = pp[HD], pl = pp[HD + 1];
        const float mm = warp_max(pm);
        const float wgt = pm == -INFINITY ? 0.0f : exp2f((pm - mm) * 1.44269504f);
        wsm[warp * 32 + lane] = wgt;
        float ll = 0.0f;
#pragma unroll
        for (int pi = 0; pi < 32; ++pi) ll = __fmaf_rn(__shfl_sync(0xffffffffu, pl, pi), __shfl_sync(0xffffffffu, wgt, pi), ll);
        if (lane == 0) {
            cta_part[warp * PW + HD] = mm;
            cta_part[warp * PW + HD + 1] = ll;
        }
    }
    __syncthreads();
    for (int o = threadIdx.x; o < G * HD; o += blockDim.x) {
        const int g = o / HD, d = o % HD;
        float aa = 0.0f;
#pragma unroll 8
        for (int pi = 0; pi < 32; ++pi) aa = __fmaf_rn(sm[pi * G * PW + g * PW + d], wsm[g * 32 + pi], aa);
        cta_part[g * PW + d] = aa;
    }
    cluster.sync();  // every CTA's partial is in place (a hardware barrier over the co-scheduled cluster: nothing to poll)
    const int bl = warp * kAttnCluster + sp;  // this warp's block of 32 channels among the G * HD / 32 of the kv head
    if (bl < G * HD / 32) {
        const int g = bl * 32 / HD, d = (bl * 32) % HD + lane;
        float pv[kAttnCluster];
#pragma unroll
        for (int s = 0; s < kAttnCluster; ++s) pv[s] = cluster.map_shared_rank(cta_part, s)[g * PW + d];
        const float* mine_ml = cluster.map_shared_rank(cta_part, lane % kAttnCluster) + g * PW + HD;
        const float pm = lane < kAttnCluster ? mine_ml[0] : -INFINITY;
        const float pl = lane < kAttnCluster ? mine_ml[1] : 0.0f;
        const float mm = warp_max(pm);
        const float wl = pm == -INFINITY ? 0.0f : exp2f((pm - mm) * 1.44269504f);
        float ll = 0.0f, aa = 0.0f;
#pragma unroll
        for (int s = 0; s < kAttnCluster; ++s) {
            const float wgt = __shfl_sync(0xffffffffu, wl, s), ls = __shfl_sync(0xffffffffu, pl, s);
            ll = __fmaf_rn(ls, wgt, ll);
            aa = __fmaf_rn(pv[s], wgt, aa);
        }
        attn_store_block_q8(__fdiv_rn(aa, ll), (h0 * HD) / 32 + bl, lane, attn, xq, xd);
    }
    cluster.sync();  // nobody leaves while its shared memory is still being read
}

// Causal attention of a prompt chunk over the fp16 cache, blocked over tokens: CTA (kv head, block of TB consecutive
// tokens) brings the K and V rows of its kv head into shared memory 32 positions at a time (cp.async, double buffered)
// and every one of its TB * G warps -- one per (token, query head of the group) -- scores them from there: a K / V row
// is read from L2 once per TB * G (token, head) pairs instead of once each.  A lane group (eight lanes) takes PS
// positions per step and updates its online exp2 softmax once for all of them, which shortens the chain of dependent
// exponentials and rescalings that bounds a warp; the four lane groups merge by shuffles at the end and the normalised
// output goes straight to out[token][heads * HD].  Token t of the chunk sits at position pos0 + t and attends to cache
// rows 0 .. pos0 + t.
template <int HD, int G, int TB, int PS>
__global__ void __launch_bounds__(TB * G * 32) attn_prompt_kernel(const float* q, const unsigned short* kc, const unsigned short* vc, float* out, int heads,
                                                                  int kv_heads, int n_tok, float scale, int q_stride, int pos0) {
    constexpr int DPL = HD / 8, NV = DPL / 8, kTile = 32, kThreads = TB * G * 32;
    constexpr int kRowWords = HD / 2;                        // 32-bit words of an fp16 row
    extern __shared__ __align__(16) unsigned tile[];         // [2][K | V][kTile][kRowWords]
    const int kvh = blockIdx.x, tok0 = blockIdx.y * TB;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, grp = lane >> 3, l8 = lane & 7;
    const int ti = warp / G, g = warp % G;
    const int tok = tok0 + ti, h = kvh * G + g;
    const bool live_warp = tok < n_tok;
    const int my_last = pos0 + tok;                           // last position this token attends to
    const int blk_last = pos0 + min(tok0 + TB, n_tok) - 1;    // ... and the block's
    const int n_tiles = blk_last / kTile + 1;
    const int kvdim = kv_heads * HD;

    // lane l8 of a group holds channels c(i) = (i / 8) * (HD / NV) + l8 * 8 + i % 8: its 16-byte loads of a row are then
    // next to its neighbours' (no shared-memory bank conflicts)
    const auto chan = [&](int i) { return (i / 8) * (HD / NV) + l8 * 8 + (i % 8); };
    float qv[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) qv[i] = live_warp ? q[static_cast<size_t>(tok) * q_stride + static_cast<size_t>(h) * HD + chan(i)] : 0.0f;
    float m = -INFINITY, l = 0.0f, acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;

    auto load_tile = [&](int t, int buf) {  // rows t * 32 .. of K and V, 16 bytes per thread and step
        constexpr int kChunks = 2 * kTile * kRowWords / 4;  // 16-byte pieces of one tile (K and V)
        for (int c = threadIdx.x; c < kChunks; c += kThreads) {
            const int which = c / (kTile * kRowWords / 4), r = (c / (kRowWords / 4)) % kTile, w4 = c % (kRowWords / 4);
            const int pos = min(t * kTile + r, blk_last);     // (rows past the block's last position are never scored)
            const unsigned short* src = (which ? vc : kc) + static_cast<size_t>(pos) * kvdim + kvh * HD + w4 * 8;
            unsigned* dst = tile + ((static_cast<size_t>(buf) * 2 + which) * kTile + r) * kRowWords + w4 * 4;
            const unsigned sa = static_cast<unsigned>(__cvta_generic_to_shared(dst));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // one row of the tile as this lane's DPL floats
    const auto row = [&](const unsigned* base, int r, float* f) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const uint4 u = *reinterpret_cast<const uint4*>(base + static_cast<size_t>(r) * kRowWords + i * (kRowWords / NV) + l8 * 4);
            const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[8 * i + 2 * j] = half_bits_to_float(w[j] & 0xFFFFu);
                f[8 * i + 2 * j + 1] = half_bits_to_float(w[j] >> 16);
            }
        }
    };
    load_tile(0, 0);
    for (int t = 0; t < n_tiles; ++t) {
        if (t + 1 < n_tiles) {
            load_tile(t + 1, (t + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // tile t has landed for every thread
        const unsigned* kt = tile + (static_cast<size_t>(t & 1) * 2) * kTile * kRowWords;
        const unsigned* vt = kt + kTile * kRowWords;
        if (live_warp) {
#pragma unroll
            for (int s = 0; s < kTile / (4 * PS); ++s) {  // positions 4 PS s + 4 u + grp of the tile, u < PS
                if (t * kTile + 4 * PS * s > my_last) break;   // warp-uniform: the whole step lies beyond this token
                float sc[PS], f[PS][DPL];
                bool live[PS];
#pragma unroll
                for (int u = 0; u < PS; ++u) {
                    const int r = 4 * PS * s + 4 * u + grp;
                    live[u] = t * kTile + r <= my_last;
                    row(kt, r, f[u]);
                    sc[u] = 0.0f;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) sc[u] += qv[i] * f[u][i];
                }
#pragma unroll
                for (int o = 1; o <= 4; o <<= 1)
#pragma unroll
                    for (int u = 0; u < PS; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
                if (live[0]) {  // (a later position of the step is live only if the first is)
                    float mn = m;
#pragma unroll
                    for (int u = 0; u < PS; ++u) {
                        sc[u] = live[u] ? sc[u] * scale : -INFINITY;
                        mn = fmaxf(mn, sc[u]);
                    }
                    const float corr = exp2f((m - mn) * 1.44269504f);
                    float psum = 0.0f;
#pragma unroll
                    for (int u = 0; u < PS; ++u) {
                        sc[u] = exp2f((sc[u] - mn) * 1.44269504f);  // exp2(-inf) = 0
                        psum += sc[u];
                        row(vt, 4 * PS * s + 4 * u + grp, f[u]);
                    }
                    l = l * corr + psum;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) {
                        float a = 0.0f;
#pragma unroll
                        for (int u = 0; u < PS; ++u) a += sc[u] * f[u][i];
                        acc[i] = acc[i] * corr + a;
                    }
                    m = mn;
                }
            }
        }
        __syncthreads();  // everyone is done with buffer t & 1 before tile t + 2 overwrites it
    }
    if (!live_warp) return;
    // the warp's four lane groups -> one result (groups 1..3 may have seen nothing: weight 0)
#pragma unroll
    for (int o = 8; o <= 16; o <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m, o), lo = __shfl_xor_sync(0xffffffffu, l, o);
        const float mm = fmaxf(m, mo);
        const float wa = m == -INFINITY ? 0.0f : exp2f((m - mm) * 1.44269504f);
        const float wb = mo == -INFINITY ? 0.0f : exp2f((mo - mm) * 1.44269504f);
        l = l * wa + lo * wb;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] = acc[i] * wa + __shfl_xor_sync(0xffffffffu, acc[i], o) * wb;
        m = mm;
    }
    if (grp == 0) {
        float* dst = out + static_cast<size_t>(tok) * heads * HD + static_cast<size_t>(h) * HD;
#pragma unroll
        for (int i = 0; i < DPL; ++i) dst[chan(i)] = __fdiv_rn(acc[i], l);
    }
}

// Merges the nsplit partials of every head, normalises, and writes attn[heads*HD] together with its Q8
// quantization (the wo matvec's input): one warp per block of 32 output channels.
__global__ void attn_combine_q8_kernel(const float* part, float* attn, int* xq, float* xd, int heads,
                                       int hd, int nsplit) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // (see rope_kv_f16_kernel)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;  // block of 32 channels
    if (b >= heads * hd / 32) return;
    const int h = b * 32 / hd, d = (b * 32) % hd + lane;
    const float* ph = part + static_cast<size_t>(h) * nsplit * (hd + 2);
    float ll = 0.0f, aa = 0.0f;
    if (nsplit <= 32) {
        // one round trip: lane s asks for split s's {max, sum}, every lane for its channel of all splits; the weights
        // are computed once per split and handed round by shuffles; the sums run in split order as in the loop below
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
    attn_store_block_q8(__fdiv_rn(aa, ll), b, lane, attn, xq, xd);
}

// Batched form of the merge: token blockIdx.y, normalised floats to out[token][heads * hd] (quantized per 256 afterwards).
__global__ void attn_combine_rows_kernel(const float* __restrict__ part, float* __restrict__ out, int heads, int hd, int nsplit) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= heads * hd) return;
    const int h = i / hd, d = i % hd, tok = blockIdx.y;
    const float* ph = part + (static_cast<size_t>(tok) * heads + h) * nsplit * (hd + 2);
    float mm = -INFINITY;
    for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, ph[s * (hd + 2) + hd]);
    float ll = 0.0f, aa = 0.0f;
    for (int s = 0; s < nsplit; ++s) {
        const float pm = ph[s * (hd + 2) + hd];
        const float wgt = pm == -INFINITY ? 0.0f : exp2f((pm - mm) * 1.44269504f);
        ll += ph[s * (hd + 2) + hd + 1] * wgt;
        aa += ph[s * (hd + 2) + d] * wgt;
    }
    out[static_cast<size_t>(tok) * heads * hd + i] = __fdiv_rn(aa, ll);
}

// Greedy pick of every sequence of a batch: one CTA per row of logits, first maximum; the pick becomes the sequence's
// next token and goes into its history at the common position.
// With out_v / out_i given, the row's (maximum, index) go there instead -- one rank's candidates under tensor parallelism.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float* __restrict__ logits, int vocab, int* tok, int* history,
                                                           const int* __restrict__ pos_p, int max_ctx, float* out_v = nullptr, int* out_i = nullptr) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = logits + static_cast<size_t>(blockIdx.x) * vocab;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > best) best = v, idx = i;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
    }
    if (lane == 0) bv[warp] = best, bi[warp] = idx;
    __syncthreads();
    if (warp == 0) {
        best = bv[lane], idx = bi[lane];  // 32 warps
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
        }
        if (lane == 0 && out_v) {
            out_v[blockIdx.x] = best;
            out_i[blockIdx.x] = idx;
        } else if (lane == 0) {
            const int pos = *pos_p;
            tok[blockIdx.x] = idx;
            if (pos < max_ctx) history[static_cast<size_t>(blockIdx.x) * max_ctx + pos] = idx;
        }
    }
}
__global__ void advance_pos_kernel(int* pos_p) { *pos_p += 1; }

// Greedy pick (first maximum, as a sequential scan would), token history, position advance.
__global__ void argmax_advance_kernel(const float* __restrict__ cand_v, const int* __restrict__ cand_i, int ncand, int* token,
                                      int* history, int* pos_p, int max_ctx) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < ncand; i += blockDim.x) {
        const float v = cand_v[i];
        const int ci = cand_i[i];
        if (v > best || (v == best && ci < idx)) best = v, idx = ci;
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) bv[warp] = best, bi[warp] = idx;
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? bv[lane] : -INFINITY;
        idx = lane < nw ? bi[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
        }
        if (lane == 0) {
            const int pos = *pos_p;
            *token = idx;
            if (pos < max_ctx) history[pos] = idx;
            *pos_p = pos + 1;
        }
    }
}

// ---- tensor parallelism: exchange points of a decode step -------------------------------------------------
// Heads and FFN rows are sharded over `world` ranks (one process per GPU); the attention-output and FFN-down
// matrices are split along K, so each rank holds a partial hidden vector at those two points of a layer
// (the all-reduce boundaries of Megatron-style sharding).  The exchange is fused into the kernel that consumes
// the sum: it announces this rank's arrival in every rank's flag array, waits (bounded) for all ranks, reads
// every rank's partial straight out of that rank's memory with ordinary loads over NVLink, and adds them in
// rank order -- every rank computes the same bits, so the replicated residual stream never diverges.
// Partials are double-buffered by exchange parity: a rank can be at most one exchange ahead of a peer that is
// still reading.  Waits give up after a fixed number of polls, count the event and mark the group dead so
// later waits return at once; nothing spins forever.
struct TpCtx {
    float* partial[8] = {};   // rank r: [2][hidden] floats
    unsigned* flags[8] = {};  // rank r: flags[src] = last exchange number src announced to r
    float* cand_v[8] = {};    // rank r's argmax candidates
    int* cand_i[8] = {};
    float* rows[8] = {};      // rank r: [2][kTpRowsChunk][hidden] floats, the K-split partial products of a prompt chunk
    unsigned* epoch = nullptr;  // this rank's exchange counter (local memory)
    int rank = 0, world = 1;
};
__device__ unsigned g_tp_timeouts = 0;
__device__ unsigned g_tp_dead = 0;
__device__ unsigned g_tp_poll_limit = 1u << 22;  // polls of one wait before it gives up (about a second)

__device__ __forceinline__ float ld_peer_f32(const float* p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_peer_f32x4(const float* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_peer_s32(const int* p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Every thread of a single-CTA kernel calls this; on return all ranks have entered the same exchange and their
// earlier kernels' writes are visible to this CTA's sys-scope loads.
__device__ void tp_arrive_and_wait(const TpCtx& c) {
    __shared__ unsigned e_sh;
    if (threadIdx.x == 0) e_sh = atomicAdd(c.epoch, 1u) + 1u;
    __syncthreads();
    const unsigned e = e_sh;
    if (threadIdx.x < static_cast<unsigned>(c.world)) {
        const int r = threadIdx.x;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(c.flags[r] + c.rank), "r"(e) : "memory");
        const unsigned limit = *reinterpret_cast<volatile unsigned*>(&g_tp_dead) ? 1u : *reinterpret_cast<volatile unsigned*>(&g_tp_poll_limit);
        bool arrived = false;
        for (unsigned i = 0; i < limit; ++i) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(c.flags[c.rank] + r) : "memory");
            if (static_cast<int>(v - e) >= 0) {
                arrived = true;
                break;
            }
            if (i > 64) __nanosleep(64);
        }
        if (!arrived) {
            atomicAdd(&g_tp_timeouts, 1u);
            atomicExch(&g_tp_dead, 1u);
        }
    }
    __syncthreads();
}

// x += sum over ranks of partial (rank order); then RMSNorm(x) * w quantized to Q8 blocks, as
// add_norm_q8_fast_kernel does for one GPU.
__global__ void __launch_bounds__(1024) tp_add_norm_q8_kernel(float* x, TpCtx c, int parity, const float* __restrict__ w, int* xq,
                                                               float* xd, int n, float eps) {
    extern __shared__ __align__(16) float sh[];  // n floats
    __shared__ float red[32];
    tp_arrive_and_wait(c);
    float ss = 0.0f;
    for (int j = 4 * threadIdx.x; j < n; j += 4 * blockDim.x) {  // n is a multiple of 256
        // all ranks' loads are issued before the first use: one NVLink round trip, not `world` of them
        float4 p[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (r < c.world) p[r] = ld_peer_f32x4(c.partial[r] + static_cast<size_t>(parity) * n + j);
        float4 t = p[0];
#pragma unroll
        for (int r = 1; r < 8; ++r)
            if (r < c.world) t.x = __fadd_rn(t.x, p[r].x), t.y = __fadd_rn(t.y, p[r].y), t.z = __fadd_rn(t.z, p[r].z), t.w = __fadd_rn(t.w, p[r].w);
        float4 v = *reinterpret_cast<const float4*>(x + j);
        v.x = __fadd_rn(v.x, t.x), v.y = __fadd_rn(v.y, t.y), v.z = __fadd_rn(v.z, t.z), v.w = __fadd_rn(v.w, t.w);
        *reinterpret_cast<float4*>(x + j) = v;
        *reinterpret_cast<float4*>(sh + j) = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float r = rinv_rms(block_sum(ss, red), n, eps);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int gi = warp; gi < n / 128; gi += nw) {  // four blocks of 32 per warp and step (n is a multiple of 256)
        const float4 v = *reinterpret_cast<const float4*>(sh + gi * 128 + 4 * lane);
        const float4 ww = *reinterpret_cast<const float4*>(w + gi * 128 + 4 * lane);
        quantize_4blocks_warp(make_float4(__fmul_rn(__fmul_rn(v.x, r), ww.x), __fmul_rn(__fmul_rn(v.y, r), ww.y),
                                          __fmul_rn(__fmul_rn(v.z, r), ww.z), __fmul_rn(__fmul_rn(v.w, r), ww.w)),
                              xq, xd, gi * 4, lane);
    }
}

// Greedy pick over every rank's candidates (rank r's indices are local to its vocab/world rows), first index
// wins ties; token history and position advance -- identical on every rank.
__global__ void tp_argmax_advance_kernel(TpCtx c, int ncand, int rows_per_rank, int* token, int* history, int* pos_p, int max_ctx) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    tp_arrive_and_wait(c);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < ncand * c.world; i += blockDim.x) {
        const int r = i / ncand, k = i - r * ncand;
        const float v = ld_peer_f32(c.cand_v[r] + k);
        const int ci = ld_peer_s32(c.cand_i[r] + k);
        const int gi = ci == 0x7fffffff ? ci : ci + r * rows_per_rank;
        if (v > best || (v == best && gi < idx)) best = v, idx = gi;
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) bv[warp] = best, bi[warp] = idx;
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? bv[lane] : -INFINITY;
        idx = lane < nw ? bi[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
        }
        if (lane == 0) {
            const int pos = *pos_p;
            *token = idx;
            if (pos < max_ctx) history[pos] = idx;
            *pos_p = pos + 1;
        }
    }
}

// The batched prompt pass under tensor parallelism: the barrier of an exchange as a launch of its own, then the sum of
// every rank's partial rows (rank order, so all ranks compute the same bits) as a grid over the whole chunk.
__global__ void tp_barrier_kernel(TpCtx c) { tp_arrive_and_wait(c); }
__global__ void tp_sum_rows_kernel(TpCtx c, size_t offset, float* out, size_t count4) {
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count4; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float4 p[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (r < c.world) p[r] = ld_peer_f32x4(c.rows[r] + offset + 4 * i);
        float4 t = p[0];
#pragma unroll
        for (int r = 1; r < 8; ++r)
            if (r < c.world) t.x = __fadd_rn(t.x, p[r].x), t.y = __fadd_rn(t.y, p[r].y), t.z = __fadd_rn(t.z, p[r].z), t.w = __fadd_rn(t.w, p[r].w);
        *reinterpret_cast<float4*>(out + 4 * i) = t;
    }
}

// Greedy pick of every sequence of a batch under tensor parallelism: rank r left (maximum, local index) of its vocabulary
// rows for sequence b at rows[r] + offset + b and + cap + b; the first maximum in global index order wins, on every rank alike.
__global__ void tp_pick_rows_kernel(TpCtx c, size_t offset, int cap, int n_seq, int rows_per_rank, int* tok, int* history, const int* pos_p, int max_ctx) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_seq) return;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int r = 0; r < c.world; ++r) {
        const float v = ld_peer_f32(c.rows[r] + offset + b);
        const int i = ld_peer_s32(reinterpret_cast<const int*>(c.rows[r] + offset + cap) + b);
        if (v > best) best = v, idx = i + r * rows_per_rank;
    }
    const int pos = *pos_p;
    tok[b] = idx;
    if (pos < max_ctx) history[static_cast<size_t>(b) * max_ctx + pos] = idx;
}

constexpr int kCand = 296;
constexpr size_t kTpFlagBytes = 256;
constexpr int kTpRowsChunk = 512;  // tokens per chunk of the batched prompt pass
inline size_t tp_vector_bytes(int hidden) {  // flags, the decode step's two partial vectors, the pick's candidates
    const size_t b = kTpFlagBytes + static_cast<size_t>(2) * hidden * 4 + static_cast<size_t>(kCand) * 8;
    return (b + 255) / 256 * 256;
}
inline size_t tp_shared_bytes(int hidden) { return tp_vector_bytes(hidden) + static_cast<size_t>(2) * kTpRowsChunk * hidden * 4; }

struct DMat {
    uint8_t* data = nullptr;
    int rows = 0, k = 0;
    bool q6 = false;
};
struct DLayer {
    std::vector<DMat> qkv, gu;  // merged where formats agree: {q|k, v} and {gate|up} for the Q4_K_M mix
    DMat wo, wd;
    float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    unsigned short *kc = nullptr, *vc = nullptr;
};

#define CU(x)                                                            \
    do {                                                                 \
        if ((x) != cudaSuccess) {                                        \
            err_ = std::string(#x) + ": " + cudaGetErrorString(cudaGetLastError()); \
            return KCB_INTERNAL_ERROR;                                   \
        }                                                                \
    } while (0)

class Decoder {
public:
    ~Decoder() {
        if (exec_) cudaGraphExecDestroy(exec_);
        if (graph_) cudaGraphDestroy(graph_);
        if (stream_) cudaStreamDestroy(stream_);
        for (void* p : owned_) cudaFree(p);
    }
    std::string err_;

    // rank / world / shared: tensor-parallel placement.  world == 1 ignores `shared`; otherwise shared[r] is rank r's
    // exchange area (tp_shared_bytes, zero-filled before any rank is created) as mapped into this process.
    int init(const kcb_model_desc& d, int rank = 0, int world = 1, void* const* shared = nullptr) {
        max_ctx = d.max_ctx, eps = d.eps, log2_base = std::log2(d.rope_base), neox = d.neox, qk_norm = d.qk_norm;
        hidden = d.hidden, hd = d.head_dim;
        if (d.hidden % 256 || d.inter % 256 || (d.heads * hd) % 256 || d.heads % d.kv_heads || (hd != 64 && hd != 128) || max_ctx < 1) {
            err_ = "unsupported model shape (hidden, inter, heads*head_dim multiples of 256; head_dim 64 or 128)";
            return KCB_INVALID_VALUE;
        }
        if (world < 1 || world > 8 || rank < 0 || rank >= world || (world > 1 && !shared) || d.kv_heads % world || d.inter % (32 * world) ||
            d.vocab % (8 * world)) {
            err_ = "unsupported sharding (1..8 ranks; kv heads, FFN rows / 32 and vocabulary rows / 8 must divide by the rank count)";
            return KCB_INVALID_VALUE;
        }
        // local shares: heads and kv heads, FFN rows, vocabulary rows
        heads = d.heads / world, kv_heads = d.kv_heads / world, inter = d.inter / world, vocab = d.vocab / world;
        vocab_total = d.vocab;
        tp.rank = rank, tp.world = world;
        const int group = heads / kv_heads;
        if (group != 1 && group != 2 && group != 3 && group != 4 && group != 8) {
            err_ = "unsupported query-group size";
            return KCB_INVALID_VALUE;
        }
        CU(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
        // K windows of the attention-output and FFN-down matrices: whole super-blocks covering this rank's
        // channels; activations outside the share stay zero Q8 blocks (d = 0, q = 0), which add exactly 0.
        const int qd = heads * hd;
        wo_win = k_window(rank * qd, qd);
        wd_win = k_window(rank * inter, inter);
        for (int l = 0; l < d.n_layers; ++l) {
            const kcb_layer& s = d.layers[l];
            DLayer L;
            const kcb_mat qkv_parts[3] = {row_slice(s.wq, static_cast<long long>(rank) * qd, qd),
                                          row_slice(s.wk, static_cast<long long>(rank) * kv_heads * hd, kv_heads * hd),
                                          row_slice(s.wv, static_cast<long long>(rank) * kv_heads * hd, kv_heads * hd)};
            const kcb_mat gu_parts[2] = {row_slice(s.wg, static_cast<long long>(rank) * inter, inter),
                                         row_slice(s.wu, static_cast<long long>(rank) * inter, inter)};
            if (s.wq.rows != d.heads * hd || s.wk.rows != d.kv_heads * hd || s.wv.rows != d.kv_heads * hd || s.wg.rows != d.inter ||
                s.wu.rows != d.inter || s.wo.k != d.heads * hd || s.wd.k != d.inter || s.wo.rows != hidden || s.wd.rows != hidden) {
                err_ = "layer matrix shapes do not match the model dimensions";
                return KCB_INVALID_VALUE;
            }
            if (const int e = merged(L.qkv, qkv_parts, 3); e) return e;
            if (const int e = merged(L.gu, gu_parts, 2); e) return e;
            if (const int e = upload_k(L.wo, s.wo, wo_win.sb0, wo_win.nsb); e) return e;
            if (const int e = upload_k(L.wd, s.wd, wd_win.sb0, wd_win.nsb); e) return e;
            if (const int e = up(L.attn_norm, s.attn_norm, hidden); e) return e;
            if (const int e = up(L.ffn_norm, s.ffn_norm, hidden); e) return e;
            if (qk_norm) {
                if (const int e = up(L.q_norm, s.q_norm, hd); e) return e;
                if (const int e = up(L.k_norm, s.k_norm, hd); e) return e;
            }
            const size_t cache = static_cast<size_t>(max_ctx) * kv_heads * hd * 2;
            if (const int e = dev(reinterpret_cast<void**>(&L.kc), cache); e) return e;
            if (const int e = dev(reinterpret_cast<void**>(&L.vc), cache); e) return e;
            layers.push_back(L);
        }
        if (d.lm_head.rows != d.vocab || d.lm_head.k != hidden) {
            err_ = "lm_head shape does not match the model dimensions";
            return KCB_INVALID_VALUE;
        }
        // The tied embedding needs any row of the full matrix; the logits matvec only this rank's rows.
        if (world > 1) {
            const long long counted = weight_bytes;
            if (const int e = merged_one(embed_w, d.lm_head); e) return e;
            weight_bytes = counted;  // one row per token is read from it
            const kcb_mat mine = row_slice(d.lm_head, static_cast<long long>(rank) * vocab, vocab);
            if (const int e = merged_one(lm_head, mine); e) return e;
        } else {
            if (const int e = merged_one(lm_head, d.lm_head); e) return e;
            embed_w = lm_head;
        }
        if (const int e = up(out_norm, d.out_norm, hidden); e) return e;
        if (d.rope_ff)
            if (const int e = up(rope_ff, d.rope_ff, hd / 2); e) return e;
        const int kv = kv_heads * hd;
        const int maxk = hidden;
        nsplit = std::max(1, std::min(32, (2 * kSmCount + kv_heads - 1) / kv_heads));
        nsplit = std::min(nsplit, std::max(1, max_ctx / 64));
        if (const int e = dev(reinterpret_cast<void**>(&x), hidden * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&x2), hidden * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&t), hidden * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&qkv), (qd + 2 * kv) * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&attn), qd * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&gu), 2 * inter * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&logits), static_cast<size_t>(vocab_total) * 4); e) return e;
        CU(cudaMemsetAsync(logits, 0, static_cast<size_t>(vocab_total) * 4, stream_));
        if (const int e = dev(reinterpret_cast<void**>(&xq), static_cast<size_t>(11) * (maxk / 32) * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&xq_wo), static_cast<size_t>(11) * (wo_win.nsb * 8) * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&xq_wd), static_cast<size_t>(11) * (wd_win.nsb * 8) * 4); e) return e;
        CU(cudaMemsetAsync(xq_wo, 0, static_cast<size_t>(11) * (wo_win.nsb * 8) * 4, stream_));
        CU(cudaMemsetAsync(xq_wd, 0, static_cast<size_t>(11) * (wd_win.nsb * 8) * 4, stream_));
        if (world > 1) {
            for (int r = 0; r < world; ++r) {
                if (!shared[r]) {
                    err_ = "missing exchange area of a rank";
                    return KCB_INVALID_VALUE;
                }
                uint8_t* b = static_cast<uint8_t*>(shared[r]);
                tp.flags[r] = reinterpret_cast<unsigned*>(b);
                tp.partial[r] = reinterpret_cast<float*>(b + kTpFlagBytes);
                tp.cand_v[r] = tp.partial[r] + 2 * hidden;
                tp.cand_i[r] = reinterpret_cast<int*>(tp.cand_v[r] + kCand);
                tp.rows[r] = reinterpret_cast<float*>(b + tp_vector_bytes(hidden));
            }
            if (const int e = dev(reinterpret_cast<void**>(&tp.epoch), 64); e) return e;
            CU(cudaMemsetAsync(tp.epoch, 0, 64, stream_));
        }
        if (const int e = dev(reinterpret_cast<void**>(&part), static_cast<size_t>(heads) * nsplit * (hd + 2) * 4); e) return e;
        if (world > 1) {
            cand_v = tp.cand_v[rank], cand_i = tp.cand_i[rank];
        } else {
            if (const int e = dev(reinterpret_cast<void**>(&cand_v), kCand * 4); e) return e;
            if (const int e = dev(reinterpret_cast<void**>(&cand_i), kCand * 4); e) return e;
        }
        if (const int e = dev(reinterpret_cast<void**>(&state), 64); e) return e;  // {pos, token, n_forced, token_used}
        if (const int e = dev(reinterpret_cast<void**>(&forced), static_cast<size_t>(max_ctx) * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&history), static_cast<size_t>(max_ctx) * 4); e) return e;
        CU(cudaMemsetAsync(state, 0, 64, stream_));
        CU(cudaMemsetAsync(history, 0, static_cast<size_t>(max_ctx) * 4, stream_));
        // warm every kernel once outside capture (lazy module loading, one-time attribute calls), then capture
        // (the warm-up step exchanges with nobody: ranks are created at different times and only meet at the first replay)
        if (const int e = record(false); e) return e;
        CU(cudaStreamSynchronize(stream_));
        CU(cudaMemsetAsync(state, 0, 64, stream_));
        return capture();
    }
    // Captures one decode step into the graph that run() replays.
    int capture() {
        if (exec_) cudaGraphExecDestroy(exec_), exec_ = nullptr;
        if (graph_) cudaGraphDestroy(graph_), graph_ = nullptr;
        CU(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeRelaxed));
        const int e = record(true);
        cudaGraph_t g = nullptr;
        const cudaError_t ce = cudaStreamEndCapture(stream_, &g);
        if (e) {
            if (g) cudaGraphDestroy(g);
            return e;
        }
        if (ce != cudaSuccess || !g) {
            err_ = "stream capture failed";
            return KCB_INTERNAL_ERROR;
        }
        graph_ = g;
        CU(cudaGraphInstantiate(&exec_, graph_, 0));
        size_t n = 0;
        cudaGraphGetNodes(graph_, nullptr, &n);
        launches_per_token = static_cast<int>(n);
        CU(cudaStreamSynchronize(stream_));
        return KCB_SUCCESS;
    }

    // Test instrumentation: from now on every step also leaves, in a device buffer, the int8 words of each activation
    // vector it quantizes and the residual stream (hidden floats) after each of a layer's two additions, in the order
    // the step runs: layer 0's q|k|v input words, then per layer the wo input words, the residual, the gate|up and down
    // input words, the residual, the next q|k|v (after the last layer: lm_head) input words.  A test can then check
    // every stage against the CPU restatement on the same inputs and count the int8 values that rounded the other way.
    // Re-captures the step graph.
    int enable_trace() {
        if (tp.world != 1) return KCB_UNSUPPORTED_OPERATION;
        if (trace_) return KCB_SUCCESS;
        trace_words_ = 0;
        for (const DLayer& L : layers) trace_words_ += (2 * hidden + L.wo.k + L.wd.k) / 4 + 2 * hidden;
        trace_words_ += hidden / 4;
        if (const int e = dev(reinterpret_cast<void**>(&trace_), trace_words_ * 4); e) return e;
        CU(cudaMemsetAsync(trace_, 0, trace_words_ * 4, stream_));
        CU(cudaStreamSynchronize(stream_));
        return capture();
    }
    int read_trace(int* host, size_t n_words) {
        if (!trace_ || !host || n_words > trace_words_) return KCB_INVALID_VALUE;
        CU(cudaStreamSynchronize(stream_));
        CU(cudaMemcpy(host, trace_, n_words * 4, cudaMemcpyDeviceToHost));
        return KCB_SUCCESS;
    }
    size_t trace_words() const { return trace_words_; }
    int set_prompt(const int* tokens, int n, int start_pos) {
        if (n < 0 || start_pos < 0 || start_pos + n > max_ctx || (n && !tokens)) return KCB_INVALID_VALUE;
        std::vector<int> f(static_cast<size_t>(max_ctx), 0);
        for (int i = 0; i < n; ++i) f[static_cast<size_t>(start_pos + i)] = tokens[i];
        const int st[4] = {start_pos, 0, start_pos + n, 0};
        CU(cudaMemcpyAsync(forced, f.data(), f.size() * 4, cudaMemcpyHostToDevice, stream_));
        CU(cudaMemcpyAsync(state, st, sizeof st, cudaMemcpyHostToDevice, stream_));
        CU(cudaStreamSynchronize(stream_));
        return KCB_SUCCESS;
    }
    int run(int steps) {
        for (int i = 0; i < steps; ++i) CU(cudaGraphLaunch(exec_, stream_));
        return KCB_SUCCESS;
    }
    // Batched prompt pass: the n tokens go through every layer together, in chunks of at most kPrefillChunk, with the
    // arithmetic of the reference's batched (ggml) path -- per-256 activation slots (llm/llm_kernels.hpp:86-89),
    // tensor-core K-quant matmuls, add + RMSNorm + quantize per row (kernels/llm/add_sumsq_f.cu, norm_mul_q8k_f.cu),
    // causal attention over the fp16 cache -- and leave the decoder where n single steps would: KV rows
    // [start_pos, start_pos + n) filled, logits and greedy pick of the last token, position start_pos + n.
    // seq >= 0: the prompt of sequence `seq` of a batch (batch_begin): its own cache, first pick into the batch's token list.
    int prefill(const int* tokens, int n, int start_pos, int seq = -1) {
        if (tp.world != 1 && (wo_win.first_block != 0 || wd_win.first_block != 0 || layers.front().wo.k != heads * hd || layers.front().wd.k != inter)) {
            err_ = "batched prompt pass under tensor parallelism needs every rank's share of the attention output and of the FFN to be whole "
                   "256-channel super-blocks; feed the prompt through kcb_decoder_set_prompt + kcb_decoder_run";
            return KCB_UNSUPPORTED_OPERATION;
        }
        if (n < 1 || start_pos < 0 || start_pos + n > max_ctx || !tokens || seq >= batch_) return KCB_INVALID_VALUE;
        if (const int e = prefill_buffers(std::min(n, kPrefillChunk)); e) return e;
        const size_t seq_off = seq >= 0 ? static_cast<size_t>(seq) * max_ctx * kv_heads * hd : 0;
        std::vector<int> f(static_cast<size_t>(max_ctx), 0);
        for (int i = 0; i < n; ++i) f[static_cast<size_t>(start_pos + i)] = tokens[i];
        CU(cudaMemcpyAsync(forced, f.data(), f.size() * 4, cudaMemcpyHostToDevice, stream_));
        CU(cudaStreamSynchronize(stream_));  // f goes out of scope
        const int qd = heads * hd, kv = kv_heads * hd, nsbh = hidden / 256;
        for (int c0 = 0; c0 < n; c0 += kPrefillChunk) {
            const int m = std::min(kPrefillChunk, n - c0), p0 = start_pos + c0;
            const size_t nblk = static_cast<size_t>(embed_w.rows) * nsbh;
            embed_rows_kernel<<<dim3((nsbh * 8 + 127) / 128, m), 128, 0, stream_>>>(embed_w.data, nblk, nsbh, embed_w.q6, vocab_total, forced + p0, pX);
            if (const int e = launch_status(); e) return e;
            for (size_t l = 0; l < layers.size(); ++l) {
                const DLayer& L = layers[l];
                // X (+= T of the previous layer), normalise, quantize
                if (const int e = add_norm_q8(pX, l ? pT : nullptr, pX, L.attn_norm, nullptr, pSlots, pSq, hidden, m, eps, 3, 1, stream_); e) return e;
                // q|k and v rows of every token: token-major outputs (the reference's column-major Y)
                const bool fused_qkv = L.qkv.size() == 1;  // {q|k|v} when the three formats agree, else {q|k, v}
                if (!(fused_qkv || (L.qkv.size() == 2 && L.qkv[0].rows == qd + kv)) || (L.gu.size() == 1 && L.gu[0].q6)) {
                    err_ = "batched prompt pass supports q and k in one format (v either) and Q4_K gate/up, or split gate/up";
                    return KCB_UNSUPPORTED_OPERATION;
                }
                float* outs[2] = {pQK, pV};
                int which = 0;
                for (const DMat& w : L.qkv)
                    if (const int e = matmul_kq_q8(w.data, pSlots, outs[which++], w.rows, w.k, m, w.q6, 1, stream_, pWs, kWsBytes); e) return e;
                const int qk_stride = fused_qkv ? qd + 2 * kv : qd + kv;
                float* vrows = fused_qkv ? pQK + qd + kv : pV;
                const int v_stride = fused_qkv ? qk_stride : kv;
                unsigned short* kc = seq >= 0 ? kcB[l] + seq_off : L.kc;
                unsigned short* vc = seq >= 0 ? vcB[l] + seq_off : L.vc;
                rope_kv_f16_kernel<<<dim3((heads + 2 * kv_heads + 3) / 4, m), 128, 0, stream_>>>(pQK, vrows, qk_stride, v_stride, nullptr, p0, kc, vc,
                                                                                                  rope_ff, L.q_norm, L.k_norm, heads, kv_heads, hd,
                                                                                                  log2_base, neox, eps, max_ctx);
                if (const int e = launch_status(); e) return e;
                if (const int e = hd == 128 ? attention<128>(L, pQK, qk_stride, m, p0, pA, kc, vc) : attention<64>(L, pQK, qk_stride, m, p0, pA, kc, vc); e)
                    return e;
                if (const int e = quantize_cols_k(pA, pSlots, qd, m, stream_); e) return e;
                if (const int e = matmul_kq_q8(L.wo.data, pSlots, rows_out(), L.wo.rows, L.wo.k, m, L.wo.q6, 1, stream_, pWs, kWsBytes); e) return e;
                if (const int e = sum_rows(m); e) return e;
                if (const int e = add_norm_q8(pX, pT, pX, L.ffn_norm, nullptr, pSlots, pSq, hidden, m, eps, 3, 1, stream_); e) return e;
                // gate and up separately so that each is a contiguous [m][inter] matrix for SwiGLU
                float* go = pG;
                for (const DMat& w : L.gu) {
                    const size_t row_bytes = static_cast<size_t>(w.k / 256) * kQ4KBlock;
                    if (w.rows == 2 * inter && !w.q6) {
                        if (const int e = matmul_kq_q8(w.data, pSlots, pG, inter, w.k, m, 0, 1, stream_, pWs, kWsBytes); e) return e;
                        if (const int e = matmul_kq_q8(w.data + row_bytes * inter, pSlots, pU, inter, w.k, m, 0, 1, stream_, pWs, kWsBytes); e) return e;
                    } else {
                        if (const int e = matmul_kq_q8(w.data, pSlots, go, w.rows, w.k, m, w.q6, 1, stream_, pWs, kWsBytes); e) return e;
                        go = pU;
                    }
                }
                if (const int e = silu_mul(pG, pU, pG, static_cast<size_t>(m) * inter, stream_); e) return e;
                if (const int e = quantize_cols_k(pG, pSlots, inter, m, stream_); e) return e;
                if (const int e = matmul_kq_q8(L.wd.data, pSlots, rows_out(), L.wd.rows, L.wd.k, m, L.wd.q6, 1, stream_, pWs, kWsBytes); e) return e;
                if (const int e = sum_rows(m); e) return e;
            }
            if (c0 + m < n) continue;
            // last token: residual add, final norm, logits, greedy pick, position
            const int st[4] = {start_pos + n - 1, 0, 0, 0};
            int* pos_word = seq >= 0 ? seq_pos + seq : state;  // position word the pick advances
            int* tok_word = seq >= 0 ? tokB + seq : state + 1;
            int* hist = seq >= 0 ? historyB + static_cast<size_t>(seq) * max_ctx : history;
            float* lg = seq >= 0 ? logitsB + static_cast<size_t>(seq) * vocab : logits + static_cast<size_t>(tp.rank) * vocab;
            if (seq >= 0) CU(cudaMemcpyAsync(pos_word, st, 4, cudaMemcpyHostToDevice, stream_));
            else CU(cudaMemcpyAsync(state, st, sizeof st, cudaMemcpyHostToDevice, stream_));
            float* xl = pX + static_cast<size_t>(m - 1) * hidden;
            if (const int e = add_norm_q8_fast(xl, pT + static_cast<size_t>(m - 1) * hidden, out_norm, xq, xd_of(xq, hidden), hidden, eps, stream_); e) return e;
            if (const int e = mv(lm_head, xq, lg); e) return e;
            if (const int e = argmax_partial(lg, vocab, cand_v, cand_i, kCand, stream_); e) return e;
            if (tp.world == 1) argmax_advance_kernel<<<1, 256, 0, stream_>>>(cand_v, cand_i, kCand, tok_word, hist, pos_word, max_ctx);
            else tp_argmax_advance_kernel<<<1, 256, 0, stream_>>>(tp, kCand, vocab, tok_word, hist, pos_word, max_ctx);
            if (const int e = launch_status(); e) return e;
        }
        CU(cudaStreamSynchronize(stream_));
        return KCB_SUCCESS;
    }
    // Where a K-split matmul of the prompt pass writes its [m][hidden] product: the chunk scratch on one GPU, this rank's
    // half of its exchange area (by exchange parity) under tensor parallelism.
    float* rows_out() { return tp.world == 1 ? pT : tp.rows[tp.rank] + rows_parity_ * static_cast<size_t>(kPrefillChunk) * hidden; }
    // Under tensor parallelism: all ranks meet, then pT = the sum of every rank's partial rows.  The parity alternates so
    // that a rank one exchange ahead writes the half its peers are not reading.
    int sum_rows(int m) {
        if (tp.world == 1) return KCB_SUCCESS;
        tp_barrier_kernel<<<1, 32, 0, stream_>>>(tp);
        if (const int e = launch_status(); e) return e;
        const size_t count4 = static_cast<size_t>(m) * hidden / 4;
        const int grid = static_cast<int>(std::min<size_t>((count4 + 255) / 256, static_cast<size_t>(4) * kSmCount));
        tp_sum_rows_kernel<<<grid, 256, 0, stream_>>>(tp, rows_parity_ * static_cast<size_t>(kPrefillChunk) * hidden, pT, count4);
        rows_parity_ ^= 1;
        return launch_status();
    }
    // ---- a batch of independent sequences decoded in lockstep (every sequence at the same position) ----------------
    // One step feeds one token per sequence through every layer together: the weights are read once per step for the whole
    // batch (per-256 activation slots + the tensor-core matmuls from 16 sequences up), each sequence attends to its own
    // fp16 cache.  The arithmetic per sequence is that of the batched prompt pass with one row.
    int batch_begin(int n_seq) {
        if (tp.world != 1 && (wo_win.first_block != 0 || wd_win.first_block != 0 || layers.front().wo.k != heads * hd || layers.front().wd.k != inter)) {
            err_ = "batched decoding under tensor parallelism needs every rank's share of the attention output and of the FFN to be whole "
                   "256-channel super-blocks";
            return KCB_UNSUPPORTED_OPERATION;
        }
        if (n_seq < 1 || n_seq > kPrefillChunk || batch_ != 0) return KCB_INVALID_VALUE;
        if (const int e = prefill_buffers(std::max(n_seq, 128)); e) return e;
        const size_t cache = static_cast<size_t>(n_seq) * max_ctx * kv_heads * hd * 2;
        for (size_t l = 0; l < layers.size(); ++l) {
            unsigned short *k = nullptr, *v = nullptr;
            if (const int e = dev(reinterpret_cast<void**>(&k), cache); e) return e;
            if (const int e = dev(reinterpret_cast<void**>(&v), cache); e) return e;
            kcB.push_back(k), vcB.push_back(v);
        }
        if (const int e = dev(reinterpret_cast<void**>(&tokB), static_cast<size_t>(n_seq) * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&seq_pos), static_cast<size_t>(n_seq) * 4 + 64); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&historyB), static_cast<size_t>(n_seq) * max_ctx * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&logitsB), static_cast<size_t>(n_seq) * vocab * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&partB), static_cast<size_t>(n_seq) * heads * nsplit * (hd + 2) * 4); e) return e;
        CU(cudaMemsetAsync(historyB, 0, static_cast<size_t>(n_seq) * max_ctx * 4, stream_));
        CU(cudaMemsetAsync(tokB, 0, static_cast<size_t>(n_seq) * 4, stream_));
        bpos = seq_pos + n_seq;  // the batch's common position word
        batch_ = n_seq, batch_pos_ = -1;
        CU(cudaStreamSynchronize(stream_));
        return KCB_SUCCESS;
    }
    int batch_prefill(int seq, const int* tokens, int n) {
        if (seq < 0 || seq >= batch_ || (batch_pos_ >= 0 && n != batch_pos_)) {
            err_ = "every sequence of a batch takes a prompt of the same length";
            return KCB_INVALID_VALUE;
        }
        if (const int e = prefill(tokens, n, 0, seq); e) return e;
        batch_pos_ = n;
        CU(cudaMemcpyAsync(bpos, &batch_pos_, 4, cudaMemcpyHostToDevice, stream_));
        CU(cudaStreamSynchronize(stream_));
        return KCB_SUCCESS;
    }
    int batch_step() {
        const int B = batch_, qd = heads * hd, kv = kv_heads * hd, nsbh = hidden / 256;
        const size_t nblk = static_cast<size_t>(embed_w.rows) * nsbh;
        embed_rows_kernel<<<dim3((nsbh * 8 + 127) / 128, B), 128, 0, stream_>>>(embed_w.data, nblk, nsbh, embed_w.q6, vocab_total, tokB, pX);
        if (const int e = launch_status(); e) return e;
        for (size_t l = 0; l < layers.size(); ++l) {
            const DLayer& L = layers[l];
            if (const int e = add_norm_q8(pX, l ? pT : nullptr, pX, L.attn_norm, nullptr, pSlots, pSq, hidden, B, eps, 3, 1, stream_); e) return e;
            const bool fused_qkv = L.qkv.size() == 1;
            if (!(fused_qkv || (L.qkv.size() == 2 && L.qkv[0].rows == qd + kv)) || (L.gu.size() == 1 && L.gu[0].q6)) {
                err_ = "batched decoding supports q and k in one format (v either) and Q4_K gate/up, or split gate/up";
                return KCB_UNSUPPORTED_OPERATION;
            }
            float* outs[2] = {pQK, pV};
            int which = 0;
            for (const DMat& w : L.qkv)
                if (const int e = matmul_kq_q8(w.data, pSlots, outs[which++], w.rows, w.k, B, w.q6, 1, stream_, pWs, kWsBytes); e) return e;
            const int qk_stride = fused_qkv ? qd + 2 * kv : qd + kv;
            float* vrows = fused_qkv ? pQK + qd + kv : pV;
            const int v_stride = fused_qkv ? qk_stride : kv;
            rope_kv_f16_kernel<<<dim3((heads + 2 * kv_heads + 3) / 4, B), 128, 0, stream_>>>(pQK, vrows, qk_stride, v_stride, bpos, 0, kcB[l], vcB[l],
                                                                                              rope_ff, L.q_norm, L.k_norm, heads, kv_heads, hd,
                                                                                              log2_base, neox, eps, max_ctx, max_ctx);
            if (const int e = launch_status(); e) return e;
            if (const int e = hd == 128 ? attention<128>(L, pQK, qk_stride, B, 0, nullptr, kcB[l], vcB[l], bpos, max_ctx, partB)
                                        : attention<64>(L, pQK, qk_stride, B, 0, nullptr, kcB[l], vcB[l], bpos, max_ctx, partB);
                e)
                return e;
            attn_combine_rows_kernel<<<dim3((qd + 127) / 128, B), 128, 0, stream_>>>(partB, pA, heads, hd, nsplit);
            if (const int e = launch_status(); e) return e;
            if (const int e = quantize_cols_k(pA, pSlots, qd, B, stream_); e) return e;
            if (const int e = matmul_kq_q8(L.wo.data, pSlots, rows_out(), L.wo.rows, L.wo.k, B, L.wo.q6, 1, stream_, pWs, kWsBytes); e) return e;
            if (const int e = sum_rows(B); e) return e;
            if (const int e = add_norm_q8(pX, pT, pX, L.ffn_norm, nullptr, pSlots, pSq, hidden, B, eps, 3, 1, stream_); e) return e;
            float* go = pG;
            for (const DMat& w : L.gu) {
                const size_t row_bytes = static_cast<size_t>(w.k / 256) * kQ4KBlock;
                if (w.rows == 2 * inter && !w.q6) {
                    if (const int e = matmul_kq_q8(w.data, pSlots, pG, inter, w.k, B, 0, 1, stream_, pWs, kWsBytes); e) return e;
                    if (const int e = matmul_kq_q8(w.data + row_bytes * inter, pSlots, pU, inter, w.k, B, 0, 1, stream_, pWs, kWsBytes); e) return e;
                } else {
                    if (const int e = matmul_kq_q8(w.data, pSlots, go, w.rows, w.k, B, w.q6, 1, stream_, pWs, kWsBytes); e) return e;
                    go = pU;
                }
            }
            if (const int e = silu_mul(pG, pU, pG, static_cast<size_t>(B) * inter, stream_); e) return e;
            if (const int e = quantize_cols_k(pG, pSlots, inter, B, stream_); e) return e;
            if (const int e = matmul_kq_q8(L.wd.data, pSlots, rows_out(), L.wd.rows, L.wd.k, B, L.wd.q6, 1, stream_, pWs, kWsBytes); e) return e;
            if (const int e = sum_rows(B); e) return e;
        }
        if (const int e = add_norm_q8(pX, pT, pX, out_norm, nullptr, pSlots, pSq, hidden, B, eps, 3, 1, stream_); e) return e;
        if (const int e = matmul_kq_q8(lm_head.data, pSlots, logitsB, lm_head.rows, lm_head.k, B, lm_head.q6, 1, stream_, pWs, kWsBytes); e) return e;
        if (tp.world == 1) {
            argmax_rows_kernel<<<B, 1024, 0, stream_>>>(logitsB, vocab, tokB, historyB, bpos, max_ctx);
        } else {  // every rank's (maximum, index) per sequence through the exchange area, then the same pick on every rank
            float* mine = rows_out();
            argmax_rows_kernel<<<B, 1024, 0, stream_>>>(logitsB, vocab, nullptr, nullptr, bpos, max_ctx, mine, reinterpret_cast<int*>(mine + kPrefillChunk));
            if (const int e = launch_status(); e) return e;
            tp_barrier_kernel<<<1, 32, 0, stream_>>>(tp);
            if (const int e = launch_status(); e) return e;
            tp_pick_rows_kernel<<<(B + 127) / 128, 128, 0, stream_>>>(tp, rows_parity_ * static_cast<size_t>(kPrefillChunk) * hidden, kPrefillChunk, B, vocab, tokB,
                                                                      historyB, bpos, max_ctx);
            rows_parity_ ^= 1;
        }
        advance_pos_kernel<<<1, 1, 0, stream_>>>(bpos);
        return launch_status();
    }
    int batch_run(int steps) {
        if (batch_ == 0 || batch_pos_ < 0 || steps < 0 || batch_pos_ + steps > max_ctx) return KCB_INVALID_VALUE;
        for (int i = 0; i < steps; ++i)
            if (const int e = batch_step(); e) return e;
        batch_pos_ += steps;
        return KCB_SUCCESS;
    }
    int batch_read(int seq, float* logits_host, int* history_host, int n_hist, int* pos_host) {
        if (seq < 0 || seq >= batch_) return KCB_INVALID_VALUE;
        CU(cudaStreamSynchronize(stream_));
        if (logits_host) CU(cudaMemcpy(logits_host, logitsB + static_cast<size_t>(seq) * vocab, static_cast<size_t>(vocab) * 4, cudaMemcpyDeviceToHost));
        if (history_host && n_hist > 0)
            CU(cudaMemcpy(history_host, historyB + static_cast<size_t>(seq) * max_ctx, static_cast<size_t>(std::min(n_hist, max_ctx)) * 4, cudaMemcpyDeviceToHost));
        if (pos_host) *pos_host = batch_pos_;
        return KCB_SUCCESS;
    }
    int sync() {
        CU(cudaStreamSynchronize(stream_));
        return KCB_SUCCESS;
    }
    int read(float* logits_host, int* history_host, int n_hist, int* pos_host) {
        CU(cudaStreamSynchronize(stream_));
        if (logits_host) CU(cudaMemcpy(logits_host, logits, static_cast<size_t>(vocab_total) * 4, cudaMemcpyDeviceToHost));
        if (history_host && n_hist > 0) CU(cudaMemcpy(history_host, history, static_cast<size_t>(std::min(n_hist, max_ctx)) * 4, cudaMemcpyDeviceToHost));
        if (pos_host) CU(cudaMemcpy(pos_host, state, 4, cudaMemcpyDeviceToHost));
        return KCB_SUCCESS;
    }
    cudaStream_t stream() const { return stream_; }
    int launches_per_token = 0;
    long long weight_bytes = 0;

private:
    static constexpr int kPrefillChunk = kTpRowsChunk;
    // Scratch of the batched prompt pass for chunks of up to m tokens, allocated on first use.
    int prefill_buffers(int m) {
        if (m <= prefill_cap_) return KCB_SUCCESS;
        const int cap = std::min(kPrefillChunk, std::max(m, 128));
        const int qd = heads * hd, kv = kv_heads * hd;
        const int maxk = std::max(std::max(hidden, inter), qd);
        const size_t M = static_cast<size_t>(cap);
        if (const int e = dev(reinterpret_cast<void**>(&pX), M * hidden * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&pT), M * hidden * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&pQK), M * (qd + 2 * kv) * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&pV), M * kv * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&pA), M * qd * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&pG), M * inter * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&pU), M * inter * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&pSlots), M * 85 * (maxk / 256) * 4); e) return e;
        if (const int e = dev(reinterpret_cast<void**>(&pSq), M * 11 * (hidden / 32) * 4); e) return e;
        if (!pWs)  // K slices of the tensor-core matmuls (the launches keep them within this size)
            if (const int e = dev(&pWs, kWsBytes); e) return e;
        prefill_cap_ = cap;
        return KCB_SUCCESS;
    }
    int dev(void** p, size_t bytes) {
        CU(cudaMalloc(p, bytes));
        owned_.push_back(*p);
        return KCB_SUCCESS;
    }
    int up(float*& dst, const float* src, int n) {
        if (!src) {
            err_ = "missing norm / frequency vector";
            return KCB_INVALID_VALUE;
        }
        if (const int e = dev(reinterpret_cast<void**>(&dst), static_cast<size_t>(n) * 4); e) return e;
        // on the decoder's own stream: a blocking copy from pageable memory may return before the DMA lands, and
        // this (non-blocking) stream would not wait for it
        CU(cudaMemcpyAsync(dst, src, static_cast<size_t>(n) * 4, cudaMemcpyHostToDevice, stream_));
        CU(cudaStreamSynchronize(stream_));
        return KCB_SUCCESS;
    }
    // Uploads GGUF blocks of one or more row-concatenated matrices of the same format and k.
    int upload(DMat& m, const kcb_mat* parts, int nparts) {
        m.k = parts[0].k, m.q6 = parts[0].fmt == 6, m.rows = 0;
        for (int i = 0; i < nparts; ++i) m.rows += parts[i].rows;
        if (m.k % 256 || m.rows % 8) {
            err_ = "matrix shape not supported (rows % 8, k % 256)";
            return KCB_INVALID_VALUE;
        }
        const size_t bytes = kcb_kquant_bytes(m.rows, m.k, m.q6);
        weight_bytes += static_cast<long long>(bytes);
        if (const int e = dev(reinterpret_cast<void**>(&m.data), bytes); e) return e;
        uint8_t* staging = m.data;
        void* tmp = nullptr;
        if (m.q6) {
            CU(cudaMalloc(&tmp, bytes));
            staging = static_cast<uint8_t*>(tmp);
        }
        size_t off = 0;
        for (int i = 0; i < nparts; ++i) {
            const kcb_mat& p = parts[i];
            const size_t b = kcb_kquant_bytes(p.rows, p.k, m.q6);
            if (cudaMemcpyAsync(staging + off, p.blocks, b, cudaMemcpyHostToDevice, stream_) != cudaSuccess ||
                cudaStreamSynchronize(stream_) != cudaSuccess) {
                if (tmp) cudaFree(tmp);
                err_ = "weight upload failed";
                return KCB_INTERNAL_ERROR;
            }
            off += b;
        }
        if (m.q6) {
            const int e = q6k_convert(staging, m.data, m.rows, m.k, 1, stream_);
            cudaStreamSynchronize(stream_);
            cudaFree(tmp);
            if (e) return e;
        }
        return KCB_SUCCESS;
    }
    int merged_one(DMat& m, const kcb_mat& p) { return upload(m, &p, 1); }
    static kcb_mat row_slice(const kcb_mat& m, long long r0, int n) {
        kcb_mat s = m;
        s.blocks = static_cast<const uint8_t*>(m.blocks) + static_cast<size_t>(r0) * (m.k / 256) * (m.fmt == 6 ? kQ6KBlock : kQ4KBlock);
        s.rows = n;
        return s;
    }
    struct KWindow {
        int sb0 = 0, nsb = 0, first_block = 0;  // super-blocks [sb0, sb0 + nsb); the share starts at Q8 block first_block of the window
    };
    static KWindow k_window(int ch0, int n) {
        KWindow w;
        w.sb0 = ch0 / 256;
        w.nsb = (ch0 + n + 255) / 256 - w.sb0;
        w.first_block = (ch0 - w.sb0 * 256) / 32;
        return w;
    }
    // Uploads columns [sb0*256, (sb0+nsb)*256) of every row of one matrix.
    int upload_k(DMat& m, const kcb_mat& p, int sb0, int nsb) {
        m.k = nsb * 256, m.q6 = p.fmt == 6, m.rows = p.rows;
        if (p.k % 256 || m.rows % 8 || sb0 < 0 || nsb < 1 || (sb0 + nsb) * 256 > p.k) {
            err_ = "matrix shape not supported (rows % 8, k % 256)";
            return KCB_INVALID_VALUE;
        }
        const size_t blk = m.q6 ? kQ6KBlock : kQ4KBlock;
        const size_t bytes = kcb_kquant_bytes(m.rows, m.k, m.q6);
        weight_bytes += static_cast<long long>(bytes);
        if (const int e = dev(reinterpret_cast<void**>(&m.data), bytes); e) return e;
        uint8_t* staging = m.data;
        void* tmp = nullptr;
        if (m.q6) {
            CU(cudaMalloc(&tmp, bytes));
            staging = static_cast<uint8_t*>(tmp);
        }
        cudaError_t ce = cudaMemcpy2DAsync(staging, nsb * blk, static_cast<const uint8_t*>(p.blocks) + sb0 * blk, (p.k / 256) * blk, nsb * blk,
                                           m.rows, cudaMemcpyHostToDevice, stream_);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(stream_);
        if (ce != cudaSuccess) {
            if (tmp) cudaFree(tmp);
            err_ = "weight upload failed";
            return KCB_INTERNAL_ERROR;
        }
        if (m.q6) {
            const int e = q6k_convert(staging, m.data, m.rows, m.k, 1, stream_);
            cudaStreamSynchronize(stream_);
            cudaFree(tmp);
            if (e) return e;
        }
        return KCB_SUCCESS;
    }
    int merged(std::vector<DMat>& out, const kcb_mat* parts, int n) {
        int i = 0;
        while (i < n) {
            int j = i + 1;
            while (j < n && parts[j].fmt == parts[i].fmt && parts[j].k == parts[i].k) ++j;
            DMat m;
            if (const int e = upload(m, parts + i, j - i); e) return e;
            out.push_back(m);
            i = j;
        }
        return KCB_SUCCESS;
    }
    // Q8 scratch of a k-channel vector: words, then {d, sum} pairs (llm/llm_kernels.hpp:82-85).
    static float* xd_of(int* q, int k) { return reinterpret_cast<float*>(q + (k / 32) * 8); }
    int mv(const DMat& m, int* in, float* y) {
        return m.q6 ? matvec_q6k_q8(m.data, in, xd_of(in, m.k), y, m.rows, m.k, stream_) : matvec_q4k_q8(m.data, in, xd_of(in, m.k), y, m.rows, m.k, stream_);
    }
    // x += (sum over ranks of) t, then norm + quantize into xq; `exchange` false keeps the sum local (warm-up).
    int add_norm(float* t_local, const float* w, bool exchange) {
        if (tp.world == 1) return add_norm_q8_fast(x, t_local, w, xq, xd_of(xq, hidden), hidden, eps, stream_);
        TpCtx c = tp;
        if (!exchange) {  // a group of one: this rank's own areas in slot 0
            c.world = 1, c.rank = 0;
            c.partial[0] = tp.partial[tp.rank], c.flags[0] = tp.flags[tp.rank] + tp.rank;
        }
        tp_add_norm_q8_kernel<<<1, 1024, static_cast<size_t>(hidden) * sizeof(float), stream_>>>(x, c, xchg_ & 1, w, xq, xd_of(xq, hidden), hidden, eps);
        ++xchg_;
        return launch_status();
    }
    float* partial_out() { return tp.world == 1 ? t : tp.partial[tp.rank] + static_cast<size_t>(xchg_ & 1) * hidden; }
    // Decode: one token at the device-side position, nsplit partials.  Prompt (direct != nullptr): n_tok query rows
    // of stride q_stride at host-known positions pos0.., one CTA per (kv head, token), normalised output.
    // Batch of sequences (seq_rows != 0): n_tok query rows, token i reads the cache of sequence i (kc, vc given, seq_rows
    // rows apart) up to the common device-side position *pos_dev, nsplit partials per token into part_buf.
    template <int HD>
    int attention(const DLayer& L, const float* q = nullptr, int q_stride = 0, int n_tok = 1, int pos0 = 0, float* direct = nullptr,
                  const unsigned short* kc = nullptr, const unsigned short* vc = nullptr, const int* pos_dev = nullptr, int seq_rows = 0,
                  float* part_buf = nullptr) {
        // one CTA per kv head and its group of query heads; the prompt pass (many tokens, no split) takes one CTA per
        // query head instead: a quarter of the registers, so four times the warps hide the cache-read latency
        if (direct && seq_rows == 0 && !pos_dev && prompt_blocked_) {
            if (!q) q = qkv;
            if (!kc) kc = L.kc, vc = L.vc;
            const int G = heads / kv_heads;
            constexpr int TB = KCB_PROMPT_TB, PS = KCB_PROMPT_PS;
            const dim3 grid(kv_heads, (n_tok + TB - 1) / TB);
            const size_t smem = static_cast<size_t>(2) * 2 * 32 * (HD / 2) * 4;  // two buffers of K | V, 32 fp16 rows each
            const float scale = 1.0f / std::sqrt(static_cast<float>(HD));
#define KCB_PROMPT(G_)                                                                                                                       \
    do {                                                                                                                                     \
        static PerDeviceFlag raised;                                                                                                         \
        if (!raise_dynamic_smem(attn_prompt_kernel<HD, G_, TB, PS>, smem, raised)) return KCB_LAUNCH_FAILURE;                                \
        attn_prompt_kernel<HD, G_, TB, PS><<<grid, TB * G_ * 32, smem, stream_>>>(q, kc, vc, direct, heads, kv_heads, n_tok, scale, q_stride, pos0); \
        return launch_status();                                                                                                              \
    } while (0)
            switch (G) {
            case 1: KCB_PROMPT(1);
            case 2: KCB_PROMPT(2);
            case 3: KCB_PROMPT(3);
            case 4: KCB_PROMPT(4);
            default: break;  // larger groups: the per-token kernel below
            }
#undef KCB_PROMPT
        }
        const int group = direct ? 1 : heads / kv_heads;
        const int ns = direct ? 1 : nsplit;
        const dim3 grid(heads / group, ns, n_tok);
        const size_t smem = static_cast<size_t>(16) * group * (HD + 2) * 4;
        const float scale = 1.0f / std::sqrt(static_cast<float>(HD));
        const int* pos_p = pos_dev ? pos_dev : (direct ? nullptr : state);
        if (!q) q = qkv;
        if (!kc) kc = L.kc, vc = L.vc;
        float* pb = part_buf ? part_buf : part;
#define KCB_ATTN(G_)                                                                                                        \
    attn_partial_kernel<HD, G_><<<grid, 128, smem, stream_>>>(q, kc, vc, pos_p, pb, heads, kv_heads, ns, scale, max_ctx, q_stride, pos0, direct, seq_rows)
        switch (group) {
        case 1: KCB_ATTN(1); break;
        case 2: KCB_ATTN(2); break;
        case 3: KCB_ATTN(3); break;
        case 4: KCB_ATTN(4); break;
        default: KCB_ATTN(8); break;
        }
#undef KCB_ATTN
        return launch_status();
    }
    // The step with the small vector kernels folded into the matvecs that read them (decode_matvec.cu): per layer
    //   [add + norm + quantize | q|k (+ v) | rope + cache append]  attention + merge + quantize (one cluster launch)  wo
    //   [add + norm + quantize | gate|up]  SwiGLU + quantize  down      (SwiGLU a prologue of down up to 4096 values)
    // chained by programmatic dependent launches, so each kernel's weights are requested while its predecessor still runs.
    // Single GPU; matrices whose shapes the fused kernels do not take keep the step on the unfused path (record()).
    // where the next traced vector of k int8 values goes (nullptr when tracing is off)
    int* trace_slot(int k) {
        if (!trace_) return nullptr;
        int* p = trace_ + trace_off_;
        trace_off_ += static_cast<size_t>(k / 4);
        return p;
    }
    int trace_copy(const int* words, int k) {
        if (int* p = trace_slot(k)) CU(cudaMemcpyAsync(p, words, static_cast<size_t>(k / 4) * 4, cudaMemcpyDeviceToDevice, stream_));
        return KCB_SUCCESS;
    }
    // the residual stream (hidden floats) into the trace
    int trace_residual(const float* xs) {
        if (int* p = trace_slot(4 * hidden)) CU(cudaMemcpyAsync(p, xs, static_cast<size_t>(hidden) * 4, cudaMemcpyDeviceToDevice, stream_));
        return KCB_SUCCESS;
    }
    bool fused_ok() const {
        if (tp.world != 1 || hidden % 128 || hidden > 4096) return false;
        if (const char* e = getenv("KCB_DECODE_FUSED"); e && atoi(e) == 0) return false;
        const auto one_or_pair = [](const std::vector<DMat>& v) {
            return v.size() == 1 || (v.size() == 2 && !v[0].q6 && v[1].q6 && v[0].k == v[1].k);
        };
        for (const DLayer& L : layers) {
            if (!one_or_pair(L.qkv) || !one_or_pair(L.gu)) return false;
            if (!decode_matvec_shape_ok(L.wo.q6 ? 0 : L.wo.rows, L.wo.q6 ? L.wo.rows : 0, L.wo.k)) return false;
            if (!decode_matvec_shape_ok(L.wd.q6 ? 0 : L.wd.rows, L.wd.q6 ? L.wd.rows : 0, L.wd.k)) return false;
        }
        return true;
    }
    struct Pair {
        const void* w4 = nullptr;
        float* y4 = nullptr;
        int rows4 = 0;
        const void* w6 = nullptr;
        float* y6 = nullptr;
        int rows6 = 0;
    };
    static Pair pair_of(const std::vector<DMat>& v, float* y) {
        Pair p;
        for (const DMat& m : v) {
            if (m.q6) p.w6 = m.data, p.y6 = y, p.rows6 = m.rows;
            else p.w4 = m.data, p.y4 = y, p.rows4 = m.rows;
            y += m.rows;
        }
        return p;
    }
    static Pair pair_of(const DMat& m, float* y) { return pair_of(std::vector<DMat>{m}, y); }
    template <class Kern, class... Args>
    int launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, bool pdl, Args... args) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream_;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr, cfg.numAttrs = pdl ? 1 : 0;
        return cudaLaunchKernelEx(&cfg, kern, args...) == cudaSuccess ? KCB_SUCCESS : KCB_LAUNCH_FAILURE;
    }
    // Decode attention and merge in one cluster launch: group sizes up to 4 (register budget of 256 threads) and contexts
    // up to 4096 (a cluster of eight CTAs takes 256 positions per step; beyond that the 32-way split of the two-launch
    // form wins back more than the launch it costs).
    bool attn_in_cluster() const {
        const int group = heads / kv_heads;
        return attn_cluster_ && group <= 4 && group * kv_heads == heads && max_ctx <= 4096;
    }
    // (xq_out / xd_out: where the quantized output goes; default the wo scratch from its first block)
    template <int HD, int G>
    int attention_cluster_launch(const DLayer& L, bool pdl, int* xq_out, float* xd_out) {
        constexpr size_t smem = (static_cast<size_t>(33) * G * (HD + 2) + G * 32) * 4;
        static PerDeviceFlag raised;
        if (!raise_dynamic_smem(attn_decode_cluster_kernel<HD, G>, static_cast<int>(smem), raised)) return KCB_LAUNCH_FAILURE;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(kv_heads * kAttnCluster), cfg.blockDim = dim3(256), cfg.dynamicSmemBytes = smem, cfg.stream = stream_;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = kAttnCluster, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr, cfg.numAttrs = pdl ? 2 : 1;
        const float scale = 1.0f / std::sqrt(static_cast<float>(HD));
        const float* q = qkv;
        const unsigned short *kc = L.kc, *vc = L.vc;
        const int* pos_p = state;
        if (!xq_out) xq_out = xq_wo, xd_out = xd_of(xq_wo, L.wo.k);
        return cudaLaunchKernelEx(&cfg, attn_decode_cluster_kernel<HD, G>, q, kc, vc, pos_p, attn, xq_out, xd_out, heads, kv_heads, scale, max_ctx) ==
                       cudaSuccess
                   ? KCB_SUCCESS
                   : KCB_LAUNCH_FAILURE;
    }
    template <int HD>
    int attention_cluster(const DLayer& L, bool pdl, int* xq_out = nullptr, float* xd_out = nullptr) {
        switch (heads / kv_heads) {
        case 1: return attention_cluster_launch<HD, 1>(L, pdl, xq_out, xd_out);
        case 2: return attention_cluster_launch<HD, 2>(L, pdl, xq_out, xd_out);
        case 3: return attention_cluster_launch<HD, 3>(L, pdl, xq_out, xd_out);
        default: return attention_cluster_launch<HD, 4>(L, pdl, xq_out, xd_out);
        }
    }
    template <int HD>
    int attention_pdl(const DLayer& L, bool pdl) {
        const int group = heads / kv_heads;
        const dim3 grid(heads / group, nsplit, 1);
        const size_t smem = static_cast<size_t>(16) * group * (HD + 2) * 4;
        const float scale = 1.0f / std::sqrt(static_cast<float>(HD));
        const float* q = qkv;
        const unsigned short *kc = L.kc, *vc = L.vc;
        const int* pos_p = state;
        float* direct = nullptr;
#define KCB_ATTN(G_) return launch_pdl(attn_partial_kernel<HD, G_>, grid, dim3(128), smem, pdl, q, kc, vc, pos_p, part, heads, kv_heads, nsplit, scale, max_ctx, 0, 0, direct, 0)
        switch (group) {
        case 1: KCB_ATTN(1);
        case 2: KCB_ATTN(2);
        case 3: KCB_ATTN(3);
        case 4: KCB_ATTN(4);
        default: KCB_ATTN(8);
        }
#undef KCB_ATTN
    }
    // Which producers stay launches of their own.  Measured on Qwen3-8B shapes (tokens/s): nothing folded in 402; q|k|v and
    // wo only 429; the 57 MB gate|up with its norm as well 448-455; the 41 MB down projection with its 12288-wide SwiGLU as
    // well 365-380.  On Llama-3.2-3B shapes (SwiGLU a launch of its own): norms folded into q|k|v and gate|up 782, into
    // q|k|v only 726, into neither 666; the lm_head's norm stays a launch (723 against 720 when that was the only change).
    // The SwiGLU prologue costs per value (an exponential and a division in every CTA) and delays the matvec behind it,
    // where the stand-alone kernel spreads the values over many CTAs and overlaps the matvec's weight requests: folded in
    // up to swiglu_limit_ values only (4096; KCB_DECODE_SWIGLU_MAX) -- on Llama-3.2-3B shapes the 8192-wide one folded
    // into the down projection gave 718 tokens/s, as a launch of its own 781 (801 once that launch carried a programmatic
    // dependency as well).  The norm prologue is a few thousand multiply-adds: folded in for every matrix
    // the decode matvec kernel takes at all (norm_limit_, 64 MB; KCB_DECODE_FUSE_MB), beyond which the streaming kernel
    // with its deeper ring is the better matvec anyway.
    bool streams_long(const DMat& m) const { return m.k > swiglu_limit_ || kcb_kquant_bytes(m.rows, m.k, m.q6) > fuse_limit_; }
    // cur (+= add) -> RMSNorm * w -> Q8 -> y = [W...] a, for one matrix or a Q4_K / Q6_K pair on the same input.
    // Fused: one launch, the new residual stream lands in `other` and the two pointers swap.  Streaming: in place.
    // tail (q|k|v only): rotation and cache append inside the fused launch; *tail_done tells whether that happened.
    int norm_then_matvecs(const std::vector<DMat>& mats, float* y, float*& cur, float*& other, const float* add, const float* w, bool pdl,
                          const DecodeRopeTail* tail = nullptr, bool* tail_done = nullptr, const DecodeSwigluTail* swiglu = nullptr) {
        if (tail_done) *tail_done = false;
        size_t bytes = 0;
        for (const DMat& m : mats) bytes += kcb_kquant_bytes(m.rows, m.k, m.q6);
        int* xs = add ? trace_slot(4 * hidden) : nullptr;
        if (bytes > fuse_limit_) {
            if (const int e = add_norm_q8_fast(cur, add, w, xq, xd_of(xq, hidden), hidden, eps, stream_); e) return e;
            if (xs) CU(cudaMemcpyAsync(xs, cur, static_cast<size_t>(hidden) * 4, cudaMemcpyDeviceToDevice, stream_));
            if (const int e = trace_copy(xq, hidden); e) return e;
            for (const DMat& m : mats) {
                if (const int e = mv(m, xq, y); e) return e;
                y += m.rows;
            }
            return KCB_SUCCESS;
        }
        const Pair p = pair_of(mats, y);
        const bool use_tail = tail && p.rows4 % tail->hd == 0;  // (whole heads in the Q4_K matrix)
        const bool use_swiglu = swiglu && mats.size() == 1 && hidden <= 4096 && swiglu->inter % 32 == 0;
        if (const int e = decode_matvec_norm(p.w4, p.y4, p.rows4, p.w6, p.y6, p.rows6, hidden, cur, add, other, w, eps, pdl, stream_, trace_slot(hidden),
                                             use_tail ? tail : nullptr, use_swiglu ? swiglu : nullptr);
            e)
            return e;
        if (tail_done) *tail_done = use_tail || use_swiglu;
        std::swap(cur, other);
        if (xs) CU(cudaMemcpyAsync(xs, cur, static_cast<size_t>(hidden) * 4, cudaMemcpyDeviceToDevice, stream_));
        return KCB_SUCCESS;
    }
    int record_fused() {
        const int qd = heads * hd;
        int *pos_p = state, *tok_p = state + 1, *nforced_p = state + 2, *used_p = state + 3;
        const bool pdl = !(getenv("KCB_DECODE_PDL") && atoi(getenv("KCB_DECODE_PDL")) == 0);
        trace_off_ = 0;
        const size_t nblk = static_cast<size_t>(embed_w.rows) * (hidden / 256);
        embed_kernel<<<(hidden / 256 * 8 + 127) / 128, 128, 0, stream_>>>(embed_w.data, nblk, hidden / 256, embed_w.q6, vocab_total, tok_p, forced,
                                                                          nforced_p, pos_p, used_p, x);
        if (const int e = launch_status(); e) return e;
        float *cur = x, *other = x2;  // the residual stream ping-pongs: every CTA of a norm prologue reads cur, one writes other
        const float* add = nullptr;   // what the next norm prologue adds to the residual stream first
        for (size_t l = 0; l < layers.size(); ++l) {
            const DLayer& L = layers[l];
            // adjacent-pair RoPE without per-head norms: rotation and cache append ride on the q|k|v launch's finished tiles
            DecodeRopeTail tail;
            tail.pos_p = pos_p, tail.kc = L.kc, tail.vc = L.vc, tail.ff = rope_ff, tail.heads = heads, tail.kv_heads = kv_heads, tail.hd = hd;
            tail.max_ctx = max_ctx, tail.log2_base = log2_base;
            const bool can_tail = rope_tail_ && !neox && !L.q_norm && !L.k_norm && hd % 2 == 0;
            bool rotated = false;
            if (const int e = norm_then_matvecs(L.qkv, qkv, cur, other, add, L.attn_norm, pdl, can_tail ? &tail : nullptr, &rotated); e) return e;
            if (!rotated) {
                float* vrows = qkv + qd + kv_heads * hd;
                const float *ff = rope_ff, *qn = L.q_norm, *kn = L.k_norm;
                if (const int e = launch_pdl(rope_kv_f16_kernel, dim3((heads + 2 * kv_heads + 3) / 4), dim3(128), 0, pdl, qkv, vrows, 0, 0,
                                             const_cast<const int*>(pos_p), 0, L.kc, L.vc, ff, qn, kn, heads, kv_heads, hd, log2_base, neox, eps, max_ctx, 0);
                    e)
                    return e;
            }
            if (attn_in_cluster()) {  // partials merged through the cluster's shared memory
                if (const int e = hd == 128 ? attention_cluster<128>(L, pdl) : attention_cluster<64>(L, pdl); e) return e;
            } else {
                if (const int e = hd == 128 ? attention_pdl<128>(L, pdl) : attention_pdl<64>(L, pdl); e) return e;
                // the merge of the partials is a launch of its own here: a block of 32 channels per warp over 24 CTAs is one
                // round trip to L2.  Every CTA of the wo launch redoing all 96 blocks as a prologue took six; the last CTA
                // of each kv head merging behind a fence and a counter gave 737 tokens/s where this form gave 772.
                if (const int e = launch_pdl(attn_combine_q8_kernel, dim3((qd / 32 + 3) / 4), dim3(128), 0, pdl, const_cast<const float*>(part), attn, xq_wo,
                                             xd_of(xq_wo, L.wo.k), heads, hd, nsplit);
                    e)
                    return e;
            }
            if (const int e = trace_copy(xq_wo, L.wo.k); e) return e;
            const Pair o = pair_of(L.wo, t);
            if (const int e = decode_matvec_q8(o.w4, o.y4, o.rows4, o.w6, o.y6, o.rows6, L.wo.k, xq_wo, xd_of(xq_wo, L.wo.k), pdl, stream_); e) return e;
            // SwiGLU: a tail of the gate|up launch where that takes one (every value computed once, no launch), else a
            // prologue of the down projection (small vectors) or a launch of its own
            DecodeSwigluTail sw;
            sw.inter = inter, sw.xq = xq_wd, sw.xd = xd_of(xq_wd, L.wd.k);
            const bool want_sw = swiglu_tail_ && streams_long(L.wd);
            bool swiglu_done = false;
            if (const int e = norm_then_matvecs(L.gu, gu, cur, other, t, L.ffn_norm, pdl, nullptr, &swiglu_done, want_sw ? &sw : nullptr); e) return e;
            if (swiglu_done) {
                if (const int e = trace_copy(xq_wd, L.wd.k); e) return e;
                if (const int e = mv(L.wd, xq_wd, t); e) return e;
            } else if (streams_long(L.wd)) {  // SwiGLU + quantize as its own launch, then the streaming matvec
                if (const int e = silu_mul_q8(gu, gu + inter, nullptr, nullptr, xq_wd, xd_of(xq_wd, L.wd.k), inter, 1, stream_, pdl); e) return e;
                if (const int e = trace_copy(xq_wd, L.wd.k); e) return e;
                if (const int e = mv(L.wd, xq_wd, t); e) return e;
            } else {
                const Pair dn = pair_of(L.wd, t);
                if (const int e = decode_matvec_swiglu(dn.w4, dn.y4, dn.rows4, dn.w6, dn.y6, dn.rows6, L.wd.k, gu, gu + inter, pdl, stream_, trace_slot(L.wd.k)); e)
                    return e;
            }
            add = t;
        }
        if (const int e = norm_then_matvecs(std::vector<DMat>{lm_head}, logits, cur, other, add, out_norm, pdl); e) return e;
        if (const int e = argmax_partial(logits, vocab, cand_v, cand_i, kCand, stream_); e) return e;
        argmax_advance_kernel<<<1, 256, 0, stream_>>>(cand_v, cand_i, kCand, tok_p, history, pos_p, max_ctx);
        return launch_status();
    }

    // Enqueues one decode step on stream_.
    int record(bool exchange) {
        if (fused_ok()) return record_fused();
        const int qd = heads * hd;
        int *pos_p = state, *tok_p = state + 1, *nforced_p = state + 2, *used_p = state + 3;
        xchg_ = 0;
        trace_off_ = 0;
        const size_t nblk = static_cast<size_t>(embed_w.rows) * (hidden / 256);
        embed_kernel<<<(hidden / 256 * 8 + 127) / 128, 128, 0, stream_>>>(embed_w.data, nblk, hidden / 256, embed_w.q6, vocab_total, tok_p, forced,
                                                                          nforced_p, pos_p, used_p, x);
        if (const int e = launch_status(); e) return e;
        if (const int e = add_norm_q8_fast(x, nullptr, layers[0].attn_norm, xq, xd_of(xq, hidden), hidden, eps, stream_); e) return e;
        if (const int e = trace_copy(xq, hidden); e) return e;
        for (size_t l = 0; l < layers.size(); ++l) {
            const DLayer& L = layers[l];
            float* y = qkv;
            // Q4_K_M mix: q|k in Q4_K and v in Q6_K take one launch where both fit the register-resident kernels
            int paired = KCB_UNSUPPORTED_OPERATION;
            if (L.qkv.size() == 2 && !L.qkv[0].q6 && L.qkv[1].q6 && L.qkv[0].k == L.qkv[1].k)
                paired = matvec_q4k_q6k_pair_q8(L.qkv[0].data, y, L.qkv[0].rows, L.qkv[1].data, y + L.qkv[0].rows, L.qkv[1].rows, xq,
                                                xd_of(xq, hidden), L.qkv[0].k, stream_);
            if (paired != KCB_SUCCESS && paired != KCB_UNSUPPORTED_OPERATION) return paired;
            if (paired == KCB_UNSUPPORTED_OPERATION)
                for (const DMat& m : L.qkv) {
                    if (const int e = mv(m, xq, y); e) return e;
                    y += m.rows;
                }
            rope_kv_f16_kernel<<<(heads + 2 * kv_heads + 3) / 4, 128, 0, stream_>>>(qkv, qkv + qd + kv_heads * hd, 0, 0, pos_p, 0, L.kc, L.vc, rope_ff,
                                                                                     L.q_norm, L.k_norm, heads, kv_heads, hd, log2_base, neox, eps, max_ctx);
            if (const int e = launch_status(); e) return e;
            int* xq_attn = xq_wo + wo_win.first_block * 8;  // (tensor parallel: this rank's heads are a window of wo's input)
            float* xd_attn = xd_of(xq_wo, L.wo.k) + wo_win.first_block * 2;
            if (attn_in_cluster()) {
                if (const int e = hd == 128 ? attention_cluster<128>(L, false, xq_attn, xd_attn) : attention_cluster<64>(L, false, xq_attn, xd_attn); e) return e;
            } else {
                if (const int e = hd == 128 ? attention<128>(L) : attention<64>(L); e) return e;
                attn_combine_q8_kernel<<<(qd / 32 + 3) / 4, 128, 0, stream_>>>(part, attn, xq_attn, xd_attn, heads, hd, nsplit);
                if (const int e = launch_status(); e) return e;
            }
            if (const int e = trace_copy(xq_wo, L.wo.k); e) return e;
            float* po = partial_out();
            if (const int e = mv(L.wo, xq_wo, po); e) return e;
            if (const int e = add_norm(po, L.ffn_norm, exchange); e) return e;
            if (const int e = trace_residual(x); e) return e;
            if (const int e = trace_copy(xq, hidden); e) return e;
            y = gu;
            for (const DMat& m : L.gu) {
                if (const int e = mv(m, xq, y); e) return e;
                y += m.rows;
            }
            if (const int e = silu_mul_q8(gu, gu + inter, nullptr, nullptr, xq_wd + wd_win.first_block * 8, xd_of(xq_wd, L.wd.k) + wd_win.first_block * 2,
                                          inter, 1, stream_);
                e)
                return e;
            if (const int e = trace_copy(xq_wd, L.wd.k); e) return e;
            po = partial_out();
            if (const int e = mv(L.wd, xq_wd, po); e) return e;
            const float* next = l + 1 < layers.size() ? layers[l + 1].attn_norm : out_norm;
            if (const int e = add_norm(po, next, exchange); e) return e;
            if (const int e = trace_residual(x); e) return e;
            if (const int e = trace_copy(xq, hidden); e) return e;
        }
        float* my_logits = logits + static_cast<size_t>(tp.rank) * vocab;
        if (const int e = mv(lm_head, xq, my_logits); e) return e;
        if (const int e = argmax_partial(my_logits, vocab, cand_v, cand_i, kCand, stream_); e) return e;
        if (tp.world == 1) {
            argmax_advance_kernel<<<1, 256, 0, stream_>>>(cand_v, cand_i, kCand, tok_p, history, pos_p, max_ctx);
        } else {
            TpCtx c = tp;
            if (!exchange) {
                c.world = 1, c.rank = 0;
                c.cand_v[0] = cand_v, c.cand_i[0] = cand_i, c.flags[0] = tp.flags[tp.rank] + tp.rank;
            }
            tp_argmax_advance_kernel<<<1, 256, 0, stream_>>>(c, kCand, exchange ? vocab : 0, tok_p, history, pos_p, max_ctx);
        }
        return launch_status();
    }

    // heads, kv_heads, inter and vocab are this rank's shares
    int hidden = 0, inter = 0, heads = 0, kv_heads = 0, hd = 0, vocab = 0, vocab_total = 0, max_ctx = 0, neox = 0, qk_norm = 0, nsplit = 1;
    TpCtx tp;
    float *pX = nullptr, *pT = nullptr, *pQK = nullptr, *pV = nullptr, *pA = nullptr, *pG = nullptr, *pU = nullptr;
    int *pSlots = nullptr, *pSq = nullptr, prefill_cap_ = 0;
    void* pWs = nullptr;
    static constexpr size_t kWsBytes = 64u << 20;
    // batch of sequences
    int batch_ = 0, batch_pos_ = -1;
    std::vector<unsigned short*> kcB, vcB;
    int *tokB = nullptr, *seq_pos = nullptr, *bpos = nullptr, *historyB = nullptr;
    float *logitsB = nullptr, *partB = nullptr;
    KWindow wo_win, wd_win;
    int xchg_ = 0;  // exchanges recorded so far in the current step (parity picks the partial buffer)
    float eps = 1e-5f, log2_base = 0.f;
    std::vector<DLayer> layers;
    DMat lm_head, embed_w;
    float *out_norm = nullptr, *rope_ff = nullptr;
    float *x = nullptr, *x2 = nullptr, *t = nullptr, *qkv = nullptr, *attn = nullptr, *gu = nullptr, *logits = nullptr, *part = nullptr;
    float* cand_v = nullptr;
    int* cand_i = nullptr;
    int *xq = nullptr, *xq_wo = nullptr, *xq_wd = nullptr, *state = nullptr, *forced = nullptr, *history = nullptr;
    cudaStream_t stream_ = nullptr;
    bool prompt_blocked_ = !(getenv("KCB_PROMPT_ATTN_BLOCKED") && atoi(getenv("KCB_PROMPT_ATTN_BLOCKED")) == 0);
    bool rope_tail_ = !(getenv("KCB_DECODE_ROPE_TAIL") && atoi(getenv("KCB_DECODE_ROPE_TAIL")) == 0);
    bool attn_cluster_ = !(getenv("KCB_DECODE_ATTN_CLUSTER") && atoi(getenv("KCB_DECODE_ATTN_CLUSTER")) == 0);
    bool swiglu_tail_ = !(getenv("KCB_DECODE_SWIGLU_TAIL") && atoi(getenv("KCB_DECODE_SWIGLU_TAIL")) == 0);
    size_t fuse_limit_ = (getenv("KCB_DECODE_FUSE_MB") ? static_cast<size_t>(atoi(getenv("KCB_DECODE_FUSE_MB"))) : 64) << 20;
    int swiglu_limit_ = getenv("KCB_DECODE_SWIGLU_MAX") ? atoi(getenv("KCB_DECODE_SWIGLU_MAX")) : 4096;
    size_t rows_parity_ = 0;  // which half of the exchange area's row buffers the next K-split matmul of a prompt chunk writes
    int* trace_ = nullptr;
    size_t trace_words_ = 0, trace_off_ = 0;
    cudaGraph_t graph_ = nullptr;
    cudaGraphExec_t exec_ = nullptr;
    std::vector<void*> owned_;
};

thread_local std::string tl_err;

}  // namespace
}  // namespace kcb

using kcb::Decoder;

extern "C" {

int kcb_decoder_create(const kcb_model_desc* desc, void** out) {
    if (!desc || !out || !desc->layers || desc->n_layers <= 0) return kcb::KCB_INVALID_VALUE;
    *out = nullptr;
    auto* d = new Decoder;
    const int e = d->init(*desc);
    if (e != kcb::KCB_SUCCESS) {
        kcb::tl_err = d->err_;
        delete d;
        return e;
    }
    *out = d;
    return kcb::KCB_SUCCESS;
}
size_t kcb_decoder_tp_shared_bytes(const kcb_model_desc* desc) { return desc && desc->hidden > 0 ? kcb::tp_shared_bytes(desc->hidden) : 0; }
int kcb_decoder_create_tp(const kcb_model_desc* desc, int rank, int world, void* const* shared, void** out) {
    if (!desc || !out || !desc->layers || desc->n_layers <= 0) return kcb::KCB_INVALID_VALUE;
    *out = nullptr;
    auto* d = new Decoder;
    const int e = d->init(*desc, rank, world, shared);
    if (e != kcb::KCB_SUCCESS) {
        kcb::tl_err = d->err_;
        delete d;
        return e;
    }
    *out = d;
    return kcb::KCB_SUCCESS;
}
unsigned kcb_decoder_tp_timeouts(void) {
    unsigned v = 0;
    cudaMemcpyFromSymbol(&v, kcb::g_tp_timeouts, sizeof v);
    return v;
}
int kcb_decoder_tp_set_poll_limit(unsigned polls) {
    if (polls == 0) polls = 1u << 22;
    return cudaMemcpyToSymbol(kcb::g_tp_poll_limit, &polls, sizeof polls) == cudaSuccess ? kcb::KCB_SUCCESS : kcb::KCB_INTERNAL_ERROR;
}
int kcb_decoder_tp_reset(void) {
    const unsigned zero = 0;
    const bool ok = cudaMemcpyToSymbol(kcb::g_tp_timeouts, &zero, sizeof zero) == cudaSuccess && cudaMemcpyToSymbol(kcb::g_tp_dead, &zero, sizeof zero) == cudaSuccess;
    return ok ? kcb::KCB_SUCCESS : kcb::KCB_INTERNAL_ERROR;
}
int kcb_decoder_set_prompt(void* h, const int* tokens, int n, int start_pos) {
    return h ? static_cast<Decoder*>(h)->set_prompt(tokens, n, start_pos) : kcb::KCB_INVALID_VALUE;
}
int kcb_decoder_prefill(void* h, const int* tokens, int n, int start_pos) {
    if (!h) return kcb::KCB_INVALID_VALUE;
    auto* d = static_cast<Decoder*>(h);
    const int e = d->prefill(tokens, n, start_pos);
    if (e != kcb::KCB_SUCCESS) kcb::tl_err = d->err_;
    return e;
}
#define KCB_DEC_CALL(expr)                                   \
    if (!h) return kcb::KCB_INVALID_VALUE;                   \
    auto* d = static_cast<Decoder*>(h);                      \
    const int e = (expr);                                    \
    if (e != kcb::KCB_SUCCESS) kcb::tl_err = d->err_;        \
    return e
int kcb_decoder_batch_begin(void* h, int n_seq) { KCB_DEC_CALL(d->batch_begin(n_seq)); }
int kcb_decoder_batch_prefill(void* h, int seq, const int* tokens, int n) { KCB_DEC_CALL(d->batch_prefill(seq, tokens, n)); }
int kcb_decoder_batch_run(void* h, int steps) { KCB_DEC_CALL(d->batch_run(steps)); }
int kcb_decoder_batch_read(void* h, int seq, float* logits_host, int* history_host, int n_history, int* pos_host) {
    KCB_DEC_CALL(d->batch_read(seq, logits_host, history_host, n_history, pos_host));
}
#undef KCB_DEC_CALL
int kcb_decoder_run(void* h, int steps) { return h && steps >= 0 ? static_cast<Decoder*>(h)->run(steps) : kcb::KCB_INVALID_VALUE; }
int kcb_decoder_sync(void* h) { return h ? static_cast<Decoder*>(h)->sync() : kcb::KCB_INVALID_VALUE; }
int kcb_decoder_read(void* h, float* logits_host, int* history_host, int n_history, int* pos_host) {
    return h ? static_cast<Decoder*>(h)->read(logits_host, history_host, n_history, pos_host) : kcb::KCB_INVALID_VALUE;
}
int kcb_decoder_info(void* h, int* launches_per_token, long long* weight_bytes) {
    if (!h) return kcb::KCB_INVALID_VALUE;
    if (launches_per_token) *launches_per_token = static_cast<Decoder*>(h)->launches_per_token;
    if (weight_bytes) *weight_bytes = static_cast<Decoder*>(h)->weight_bytes;
    return kcb::KCB_SUCCESS;
}
int kcb_decoder_enable_trace(void* h, size_t* words_per_step) {
    if (!h) return kcb::KCB_INVALID_VALUE;
    auto* d = static_cast<Decoder*>(h);
    const int e = d->enable_trace();
    if (e != kcb::KCB_SUCCESS) kcb::tl_err = d->err_;
    else if (words_per_step) *words_per_step = d->trace_words();
    return e;
}
int kcb_decoder_read_trace(void* h, int* words_host, size_t n_words) {
    return h ? static_cast<Decoder*>(h)->read_trace(words_host, n_words) : kcb::KCB_INVALID_VALUE;
}
void* kcb_decoder_stream(void* h) { return h ? static_cast<Decoder*>(h)->stream() : nullptr; }
int kcb_decoder_destroy(void* h) {
    delete static_cast<Decoder*>(h);
    return kcb::KCB_SUCCESS;
}
const char* kcb_decoder_last_error(void) { return kcb::tl_err.c_str(); }

}  // extern "C"
