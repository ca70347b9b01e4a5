// Shared device helpers for the sm_100a kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace kcb {

// Status codes returned across the C ABI: the integer values of the reference's kc::Error
// (include/kernelcore/error.hpp:8-25 of the reference project).
enum : int {
    KCB_SUCCESS = 0,
    KCB_NOT_INITIALIZED = 1,
    KCB_INVALID_VALUE = 2,
    KCB_INVALID_DEVICE = 3,
    KCB_OUT_OF_MEMORY = 4,
    KCB_INVALID_POINTER = 5,
    KCB_INVALID_RESOURCE_HANDLE = 6,
    KCB_UNSUPPORTED_OPERATION = 7,
    KCB_INVALID_KERNEL_IMAGE = 8,
    KCB_KERNEL_NOT_FOUND = 9,
    KCB_DYNAMIC_CODE_BLOCKED = 10,
    KCB_LAUNCH_FAILURE = 11,
    KCB_KERNEL_FAULT = 12,
    KCB_CONTEXT_POISONED = 13,
    KCB_NOT_READY = 14,
    KCB_INTERNAL_ERROR = 15,
};

constexpr int kQ4KBlock = 144;  // bytes per 256 weights
constexpr int kQ6KBlock = 210;
constexpr int kSmCount = 148;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 128-bit streaming load: weights are read exactly once, keep them out of L1.
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float half_bits_to_float(unsigned h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}

// fp32 -> fp16 bits as the reference's SET_ROWS kernel converts (kernels/llm/set_rows_f16.cu:20-62): round to
// nearest even; 65520 and above (and NaN) give 0x7bff with the sign of "x < 0"; an input of -0 gives +0.
__device__ __forceinline__ unsigned f32_to_f16_bits(float x) {
    const unsigned sign = x < 0.0f ? 0x8000u : 0u;
    const float a = fabsf(x);
    if (!(a < 65520.0f)) return sign | 0x7bffu;
    return sign | (static_cast<unsigned>(__half_as_ushort(__float2half_rn(a))) & 0x7fffu);
}

// Rotation of one RoPE pair (x0, x1) = elements of pair index p (of `pairs` per head) at position pos: the arithmetic of
// kernels/llm/rope.cu:4-17 / rope_ff.cu of the reference, separately rounded.  ff: optional frequency factors.
__device__ __forceinline__ void rope_pair(float x0, float x1, int p, int pairs, int pos, float log2_base, const float* ff, float& y0, float& y1) {
    const float e = __fmul_rn(__fdiv_rn(-static_cast<float>(p), static_cast<float>(pairs)), log2_base);
    float th = __fmul_rn(static_cast<float>(pos), exp2f(e));
    if (ff) th = __fdiv_rn(th, ff[p]);
    const float ang = __fmul_rn(__fmul_rn(th, 0.159154943f), 6.28318548f);
    float s, c;
    sincosf(ang, &s, &c);
    y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    y1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

// Quantizes the 32 values held one per lane into Q8 block `b` of (xq, xd) -- quantize_q8x4's block.
__device__ __forceinline__ void quantize_block_warp(float v, int* xq, float* xd, int b, int lane) {
    const float amax = warp_max(fabsf(v));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    const float t = __fmul_rn(v, id);
    int q = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
    q = max(-127, min(127, q));
    const int sum = warp_sum_i(q);
    unsigned word = (static_cast<unsigned>(q) & 255u) << (8 * (lane & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if ((lane & 3) == 0) xq[b * 8 + (lane >> 2)] = static_cast<int>(word);
    if (lane == 0) {
        xd[b * 2] = d;
        xd[b * 2 + 1] = static_cast<float>(sum);
    }
}

// Four Q8 blocks per warp at once: lane l holds values 4*(l & 7) .. +3 of block b4 + (l >> 3) (so a warp covers 128
// consecutive values with one 16-byte load per lane).  Same arithmetic as quantize_block_warp -- the maximum, the
// scale, each rounding and the integer sum do not depend on how the 32 values are spread over lanes -- with three
// shuffle steps per reduction instead of five and no shuffles to pack the words.
__device__ __forceinline__ void quantize_4blocks_warp(float4 v, int* xq, float* xd, int b4, int lane) {
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    const float e[4] = {v.x, v.y, v.z, v.w};
    unsigned word = 0;
    int sum = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float t = __fmul_rn(e[i], id);
        int q = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
        q = max(-127, min(127, q));
        sum += q;
        word |= (static_cast<unsigned>(q) & 255u) << (8 * i);
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    const int b = b4 + (lane >> 3);
    xq[b * 8 + (lane & 7)] = static_cast<int>(word);
    if ((lane & 7) == 0) {
        xd[b * 2] = d;
        xd[b * 2 + 1] = static_cast<float>(sum);
    }
}

// ---- block-wide sum and the RMSNorm factor ---------------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* red) {  // red: >= 32 floats of shared memory
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.0f;
    return warp_sum(t);
}
__device__ __forceinline__ float rinv_rms(float sumsq, int n, float eps) {  // 1 / sqrt(ss / n + eps)
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, static_cast<float>(n)), eps)));
}

// Residual add + RMSNorm + Q8 blocks by one whole CTA: x += t (t may be null), then blocks of norm(x) * w into
// (xq, xd).  n % 128 == 0 and n <= 128 * MAXIT * warps of the CTA; x, t and w 16-byte aligned; gsum holds n / 128
// floats of shared memory.  The sum of squares is taken per 128 values (a warp's butterfly over four products per
// lane) and the group sums are added 32 apart in order, so the result does not depend on the CTA's size.
template <int MAXIT>
__device__ __forceinline__ void add_norm_q8_cta(float* x, const float* t, const float* __restrict__ w, int* xq, float* xd, int n,
                                                float eps, float* gsum) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int groups = n / 128;
    float4 v[MAXIT], ww[MAXIT];
#pragma unroll
    for (int i = 0; i < MAXIT; ++i) {
        const int gi = warp + i * nw;
        v[i] = ww[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (gi < groups) {
            ww[i] = __ldg(reinterpret_cast<const float4*>(w + gi * 128) + lane);  // needed last, asked for first
            float4* px = reinterpret_cast<float4*>(x + gi * 128) + lane;
            float4 a = *px;
            if (t) {
                const float4 b = *(reinterpret_cast<const float4*>(t + gi * 128) + lane);
                a = make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
                *px = a;
            }
            v[i] = a;
            const float p = __fadd_rn(__fadd_rn(__fmul_rn(a.x, a.x), __fmul_rn(a.y, a.y)), __fadd_rn(__fmul_rn(a.z, a.z), __fmul_rn(a.w, a.w)));
            const float s = warp_sum(p);
            if (lane == 0) gsum[gi] = s;
        }
    }
    __syncthreads();
    float tot = 0.0f;  // every warp takes the same total, so no second barrier
    for (int g = lane; g < groups; g += 32) tot = __fadd_rn(tot, gsum[g]);
    const float r = rinv_rms(warp_sum(tot), n, eps);
#pragma unroll
    for (int i = 0; i < MAXIT; ++i) {
        const int gi = warp + i * nw;
        if (gi < groups) {
            quantize_4blocks_warp(make_float4(__fmul_rn(__fmul_rn(v[i].x, r), ww[i].x), __fmul_rn(__fmul_rn(v[i].y, r), ww[i].y),
                                              __fmul_rn(__fmul_rn(v[i].z, r), ww[i].z), __fmul_rn(__fmul_rn(v[i].w, r), ww[i].w)),
                                  xq, xd, gi * 4, lane);
        }
    }
}

// ---- mbarrier + bulk-copy (TMA) primitives ---------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kMbarSpinLimit polls so a lost copy can never hang the GPU.
constexpr int kMbarSpinLimit = 1 << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < kMbarSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Plain (non-multicast) bulk copy global -> this CTA's shared memory; completion counted on `bar`.
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// byte i of w, sign-extended, in one PRMT: `sel` = i * 0x1111 | 0x8880 (msb of a nibble = replicate sign)
__device__ __forceinline__ int prmt_sbyte(unsigned w, unsigned sel) {
    int r;
    asm("prmt.b32 %0, %1, 0, %2;" : "=r"(r) : "r"(w), "r"(sel));
    return r;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is a setting of one device, and a process may drive several
// (kcSetDevice selects one per thread): the "already raised" flag is kept per device, not per process.
constexpr int kMaxDevices = 64;
struct PerDeviceFlag {
    std::atomic<bool> set[kMaxDevices] = {};
};
template <class Kern>
inline bool raise_dynamic_smem(Kern kern, int bytes, PerDeviceFlag& f) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return false;
    if (f.set[dev].load(std::memory_order_acquire)) return true;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
    f.set[dev].store(true, std::memory_order_release);
    return true;
}

// Host-side alignment test made by the launchers before anything is enqueued: the kernels read weights and Q8
// scratch with 16-byte loads and bulk copies, so a pointer that is valid for the reference (any interior address)
// but misaligned gets KCB_INVALID_POINTER here instead of a device-side misaligned-address fault.
inline bool misaligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; }

// Launch-error to status code; never synchronises.
inline int launch_status() { return cudaGetLastError() == cudaSuccess ? KCB_SUCCESS : KCB_LAUNCH_FAILURE; }

}  // namespace kcb
