// Activation quantizers, sm_100a.  Integer outputs are bit-identical to the reference's
// kernels/llm/quantize_q8x4.cu:8-41, quantize_cols.cu:16-53 and quantize_cols_k.cu:20-74: every
// fp32 step uses an explicitly rounded intrinsic so the compiler cannot fuse x*id + 0.5 into an FMA.

#include "common.cuh"
#include "ops.h"

namespace kcb {
namespace {

__device__ __forceinline__ int round_clamp(float v, float id) {
    const float t = __fmul_rn(v, id);
    int q = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
    return max(-127, min(127, q));
}

// One warp per block of 32 values.  Slot layout per column (llm/llm_kernels.hpp:82-85):
// [nb*8 words | nb x {d, float(sum q)} | nb partial sums of squares (untouched here)].
__global__ void quantize_q8x4_kernel(const float* __restrict__ x, int* __restrict__ q, int nb, int ncols, int k,
                                     int slot_ints, int* __restrict__ xq_flat, float* __restrict__ xd_flat) {
    const int lane = threadIdx.x & 31;
    const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (wid >= static_cast<long long>(nb) * ncols) return;
    const int c = static_cast<int>(wid / nb), b = static_cast<int>(wid % nb);
    const float v = x[static_cast<size_t>(c) * k + b * 32 + lane];
    const float amax = warp_max(fabsf(v));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    const int qi = round_clamp(v, id);
    const int sum = warp_sum_i(qi);
    unsigned word = (static_cast<unsigned>(qi) & 255u) << (8 * (lane & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    int* xq = xq_flat ? xq_flat : q + static_cast<size_t>(c) * slot_ints;
    float* xd = xd_flat ? xd_flat : reinterpret_cast<float*>(xq + nb * 8);
    if ((lane & 3) == 0) xq[b * 8 + (lane >> 2)] = static_cast<int>(word);
    if (lane == 0) {
        xd[b * 2] = d;
        xd[b * 2 + 1] = static_cast<float>(sum);
    }
}

// One warp per super-block of 256 values: lane L owns values [8L, 8L+8).  Slot layout per column
// (llm/llm_kernels.hpp:86-89): [nsb*64 words | nsb f32 d | nsb*16 sums of 16 | nsb*4 words holding the
// sums of 32 as bytes: B>>6 of blocks 0-3, 4-7, then B&63 likewise].
__global__ void quantize_q8k_kernel(const float* __restrict__ x, int* __restrict__ q, int nsb, int ncols, int k) {
    const int lane = threadIdx.x & 31;
    const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (wid >= static_cast<long long>(nsb) * ncols) return;
    const int c = static_cast<int>(wid / nsb), s = static_cast<int>(wid % nsb);
    const float4* xp = reinterpret_cast<const float4*>(x + static_cast<size_t>(c) * k + s * 256 + lane * 8);
    const float4 a = xp[0], b = xp[1];
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float am = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(v[i]));
    am = warp_max(am);
    const float d = __fdiv_rn(am, 127.0f);
    const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    unsigned w0 = 0, w1 = 0;
    int s8 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int q0 = round_clamp(v[i], id), q1 = round_clamp(v[4 + i], id);
        s8 += q0 + q1;
        w0 |= (static_cast<unsigned>(q0) & 255u) << (8 * i);
        w1 |= (static_cast<unsigned>(q1) & 255u) << (8 * i);
    }
    int* slot = q + static_cast<size_t>(c) * nsb * 85;
    slot[s * 64 + lane * 2] = static_cast<int>(w0);
    slot[s * 64 + lane * 2 + 1] = static_cast<int>(w1);
    const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
    const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
    if ((lane & 1) == 0) slot[nsb * 65 + s * 16 + (lane >> 1)] = s16;
    if (lane == 0) reinterpret_cast<float*>(slot)[nsb * 64 + s] = d;
    unsigned pw[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int bsum = __shfl_sync(0xffffffffu, s32, 4 * i);
        pw[i / 4] |= (static_cast<unsigned>(bsum >> 6) & 255u) << (8 * (i % 4));
        pw[2 + i / 4] |= static_cast<unsigned>(bsum & 63) << (8 * (i % 4));
    }
    if (lane < 4) slot[nsb * 81 + s * 4 + lane] = static_cast<int>(lane == 0 ? pw[0] : lane == 1 ? pw[1] : lane == 2 ? pw[2] : pw[3]);
}

}  // namespace

int quantize_q8x4(const float* x, int* xq, float* xd, int count, cudaStream_t s) {
    if (count < 0 || !x || !xq || !xd) return KCB_INVALID_VALUE;
    if (misaligned(x, 4) || misaligned(xq, 4) || misaligned(xd, 4)) return KCB_INVALID_POINTER;
    if (count == 0) return KCB_SUCCESS;
    quantize_q8x4_kernel<<<(count + 7) / 8, 256, 0, s>>>(x, nullptr, count, 1, count * 32, 0, xq, xd);
    return launch_status();
}

int quantize_cols(const float* x, int* q, int k, int ncols, cudaStream_t s) {
    if (k <= 0 || k % 32 || ncols < 0 || !x || !q) return KCB_INVALID_VALUE;
    if (misaligned(x, 4) || misaligned(q, 4)) return KCB_INVALID_POINTER;
    if (ncols == 0) return KCB_SUCCESS;
    const int nb = k / 32;
    const long long warps = static_cast<long long>(nb) * ncols;
    quantize_q8x4_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, s>>>(x, q, nb, ncols, k, nb * 11, nullptr, nullptr);
    return launch_status();
}

int quantize_cols_k(const float* x, int* q, int k, int ncols, cudaStream_t s) {
    if (k <= 0 || k % 256 || ncols < 0 || !x || !q) return KCB_INVALID_VALUE;
    if (misaligned(x, 16) || misaligned(q, 4)) return KCB_INVALID_POINTER;  // x is read with 16-byte loads
    if (ncols == 0) return KCB_SUCCESS;
    const long long warps = static_cast<long long>(k / 256) * ncols;
    quantize_q8k_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, s>>>(x, q, k / 256, ncols, k);
    return launch_status();
}

}  // namespace kcb
