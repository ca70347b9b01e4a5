// Q4_K / Q6_K x Q8_K-activation matmuls on the 5th-generation tensor cores (tcgen05, int8 -> int32, TMEM).
//
// Replaces the reference's kernels/llm/matmul_q4k_q8kx4.cu:41 / matmul_q4k_q8kx8.cu:41-239 (prompt
// processing; one thread per (row, 4 or 8 columns) with dp4a there).  Y[c*rows + r] = sum over super-blocks
//     (d * dx_c) * float(is) - (dmin * dx_c) * float(im),
//     is = sum_j sc_j * dot32(q_j, x_j),   im = sum_j m_j * B_j         (llm/llm_reference.cpp:529-562)
// with q 4-bit weights, sc/m 6-bit sub-block scales/mins, x int8 activations with one scale dx per 256 and
// B_j the activation sums per 32.  Both integer sums are exact GEMMs once the scale is folded into the weight:
//   * w' = sc_j * q is at most 945, so it is split as w' = 32 a + b with a, b < 32: two int8 planes, two
//     accumulators, is = 32 Da + Db, each a K = 256 contraction per super-block on the tensor core;
//   * the min term is a K = 8 contraction of the mins with the activation sums; the reference already stores
//     the sums as two bytes (B >> 6, B & 63), so im = 64 Dh + Dl with two more accumulators.
// One CTA owns a 128-row x TN-column output tile (TN = 128, or 32 for narrow batches): per super-block it unpacks
// the weight planes into shared memory (no-swizzle K-major core-matrix layout), copies the activation bytes, one
// thread issues 18 tcgen05.mma (M 128, N TN, K 32) into four TMEM accumulators, and all 8 warps read them back with
// tcgen05.ld and apply the two fp32 scale products in the reference's order -- so every output is bit-identical to
// the reference's per-column mirror.  Accumulators across super-blocks stay in registers (TN / 2 per thread).
// Every wait on the MMA-completion mbarrier is bounded; on expiry the CTA records it, frees its TMEM and leaves.

#include "common.cuh"
#include "ops.h"

#include <algorithm>
#include <map>
#include <mutex>

namespace kcb {
namespace {

constexpr int TM = 128;  // rows per tile; the column tile TN (128 or 32) is a template parameter of the kernels
constexpr int kSlab = 128 * 32;  // one K-step (32 bytes of K) of a 128-row operand
constexpr int kThreads = 256;

// shared-memory map (bytes)
constexpr int kOffAa = 0;                   // 8 slabs: plane a (w' >> 5)
constexpr int kOffAb = kOffAa + 8 * kSlab;  // 8 slabs: plane b (w' & 31)
constexpr int kOffAm = kOffAb + 8 * kSlab;  // 1 slab: mins in K bytes 0..7
constexpr int kOffBx = kOffAm + kSlab;      // 8 slabs: activation bytes
constexpr int kOffBh = kOffBx + 8 * kSlab;  // 1 slab: activation sums >> 6
constexpr int kOffBl = kOffBh + kSlab;      // 1 slab: activation sums & 63
constexpr int kOffDx = kOffBl + kSlab;      // 128 floats: activation scale of each column for this super-block
constexpr int kOffBar = kOffDx + 512;       // mbarrier, TMEM base
constexpr int kSmemBytes = kOffBar + 64;

__device__ unsigned g_tc_timeouts = 0;

// K-major, no swizzle: 8-row x 16-byte core matrices; the two 16-byte K chunks of a K-step are 128 B apart
// (leading byte offset), consecutive 8-row groups 256 B apart (stride byte offset); version 1 descriptor.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(128 >> 4) << 16) |
           (static_cast<uint64_t>(256 >> 4) << 32) | (static_cast<uint64_t>(1) << 46);
}
// int32 accumulate, signed 8-bit A and B, both K-major, N = 128, M = 128.
template <int TN>
constexpr uint32_t kIdescFor = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(TN >> 3) << 17) | (static_cast<uint32_t>(TM >> 4) << 24);

template <int TN>
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    constexpr uint32_t kIdesc = kIdescFor<TN>;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr));
}

// tcgen05.ld is asynchronous: its destination registers hold the data only after tcgen05.wait::ld.  The wait is an asm
// statement without register operands, so nothing would stop the compiler from scheduling arithmetic on those
// registers ahead of it; passing them through this empty asm (volatile asm statements keep their order) ties
// every later use to a point after the wait.
__device__ __forceinline__ void after_tmem_wait(int (&v)[16]) {
    asm volatile("" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]),
                      "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])::"memory");
}

// Packed fp32 pairs (sm_100 f32x2 arithmetic): each lane of a pair is rounded exactly as the scalar _rn operation.
// Only the multiplies of the epilogues are packed: ptxas contracts mul.rn.f32x2 followed by sub / add.rn.f32x2 into
// one fused operation (a single rounding, measured: 58 % of the results change in the last bits, -fmad=false
// notwithstanding), which would break bit-identity with the reference, so subtraction and accumulation stay scalar
// _rn intrinsics.
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// Two 16-bit lanes at a time: (four 4-bit values in bytes) * sc, split into (>> 5) and (& 31) byte planes.
__device__ __forceinline__ void scale_split(unsigned nib4, unsigned sc, unsigned& a, unsigned& b) {
    const unsigned pe = (nib4 & 0x00FF00FFu) * sc, po = ((nib4 >> 8) & 0x00FF00FFu) * sc;
    a = ((pe >> 5) & 0x00FF00FFu) | (((po >> 5) & 0x00FF00FFu) << 8);
    b = (pe & 0x001F001Fu) | ((po & 0x001F001Fu) << 8);
}

template <int TN>
__global__ void __launch_bounds__(kThreads, TN == 128 ? 1 : 2) matmul_q4k_q8k_tc_kernel(const uint8_t* __restrict__ w, const int* __restrict__ xq,
                                                                         float* __restrict__ y, int rows, int nsb, int ncols, int sb_per_split, float* __restrict__ partial) {
    extern __shared__ __align__(1024) uint8_t sm[];
    uint64_t* bar = reinterpret_cast<uint64_t*>(sm + kOffBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kOffBar + 16);
    float* dxs = reinterpret_cast<float*>(sm + kOffDx);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r_tile = blockIdx.x * TM, c_tile = blockIdx.y * TN;
    const int slot_ints = nsb * 85;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(4 * TN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init_fence();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    // epilogue role: TMEM lane (= tile row) 32 * (warp & 3) + lane, columns [TN/2 * (warp >> 2), + TN/2)
    const int erow = 32 * (warp & 3) + lane, ecol0 = (TN / 2) * (warp >> 2);
    float acc[TN / 2];
#pragma unroll
    for (int i = 0; i < TN / 2; ++i) acc[i] = 0.0f;
    // unpack role: tile row tid / 2, quant chunks 2 * (tid & 1) and + 1 (sub-blocks 4 * hsel .. + 3)
    const int urow = tid >> 1, hsel = tid & 1;
    const uint8_t* urow_blocks = w + static_cast<size_t>(r_tile + urow) * nsb * kQ4KBlock;
    const uint8_t* erow_blocks = w + static_cast<size_t>(r_tile + erow) * nsb * kQ4KBlock;
    const uint32_t ubase = (urow >> 3) * 256 + (urow & 7) * 16;

    bool failed = false;
    // split K (partial != nullptr): this CTA contracts super-blocks [sb0, sb1) and leaves its sum in slice blockIdx.z
    const int sb0 = blockIdx.z * sb_per_split, sb1 = min(nsb, sb0 + sb_per_split);
    for (int sb = sb0; sb < sb1 && !failed; ++sb) {
        // ---- weight planes ----
        {
            const uint8_t* blk = urow_blocks + static_cast<size_t>(sb) * kQ4KBlock;
            const uint4 hd = __ldg(reinterpret_cast<const uint4*>(blk));
            const unsigned sclo = hd.y & 0x3F3F3F3Fu, schi = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
            const unsigned scw = hsel ? schi : sclo;  // scales of sub-blocks 4*hsel .. 4*hsel+3
            uint4 qv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) qv[i] = ldg_stream(blk + 16 + 64 * hsel + 16 * i);
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {  // quant chunk 2*hsel + jj -> K-steps s_lo (low nibbles), s_lo + 1 (high)
                const int s_lo = 4 * hsel + 2 * jj;
                const unsigned sc_l = (scw >> (16 * jj)) & 255u, sc_h = (scw >> (16 * jj + 8)) & 255u;
                const unsigned qw[8] = {qv[2 * jj].x, qv[2 * jj].y, qv[2 * jj].z, qv[2 * jj].w,
                                        qv[2 * jj + 1].x, qv[2 * jj + 1].y, qv[2 * jj + 1].z, qv[2 * jj + 1].w};
                unsigned al[8], bl[8], ah[8], bh[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    scale_split(qw[i] & 0x0F0F0F0Fu, sc_l, al[i], bl[i]);
                    scale_split((qw[i] >> 4) & 0x0F0F0F0Fu, sc_h, ah[i], bh[i]);
                }
                uint8_t* pa = sm + kOffAa + s_lo * kSlab + ubase;
                uint8_t* pb = sm + kOffAb + s_lo * kSlab + ubase;
                *reinterpret_cast<uint4*>(pa) = make_uint4(al[0], al[1], al[2], al[3]);
                *reinterpret_cast<uint4*>(pa + 128) = make_uint4(al[4], al[5], al[6], al[7]);
                *reinterpret_cast<uint4*>(pb) = make_uint4(bl[0], bl[1], bl[2], bl[3]);
                *reinterpret_cast<uint4*>(pb + 128) = make_uint4(bl[4], bl[5], bl[6], bl[7]);
                *reinterpret_cast<uint4*>(pa + kSlab) = make_uint4(ah[0], ah[1], ah[2], ah[3]);
                *reinterpret_cast<uint4*>(pa + kSlab + 128) = make_uint4(ah[4], ah[5], ah[6], ah[7]);
                *reinterpret_cast<uint4*>(pb + kSlab) = make_uint4(bh[0], bh[1], bh[2], bh[3]);
                *reinterpret_cast<uint4*>(pb + kSlab + 128) = make_uint4(bh[4], bh[5], bh[6], bh[7]);
            }
            if (hsel == 0) {  // mins of the 8 sub-blocks as K bytes 0..7, zeros behind
                const unsigned mlo = hd.z & 0x3F3F3F3Fu, mhi = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
                *reinterpret_cast<uint4*>(sm + kOffAm + ubase) = make_uint4(mlo, mhi, 0u, 0u);
                *reinterpret_cast<uint4*>(sm + kOffAm + ubase + 128) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        // ---- activation bytes, sums and scales of this super-block ----
#pragma unroll
        for (int it = 0; it < TN * 16 / kThreads; ++it) {
            // part = 2 * K-step + 16-byte half.  Lanes: 8 neighbouring columns x 4 neighbouring parts, so a warp's
            // global reads are 64-byte runs and its shared-memory stores collide 4 ways instead of 16
            const int i = tid + kThreads * it;
            const int col = (i & 7) + 8 * (i >> 7), part = ((i >> 3) & 3) + 4 * ((i >> 5) & 3);
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (c_tile + col < ncols) v = __ldg(reinterpret_cast<const uint4*>(xq + static_cast<size_t>(c_tile + col) * slot_ints + sb * 64 + part * 4));
            *reinterpret_cast<uint4*>(sm + kOffBx + (part >> 1) * kSlab + (col >> 3) * 256 + (part & 1) * 128 + (col & 7) * 16) = v;
        }
        if (tid < TN) {
            const int col = tid;
            uint4 pw = make_uint4(0u, 0u, 0u, 0u);
            float dx = 0.0f;
            if (c_tile + col < ncols) {
                const int* slot = xq + static_cast<size_t>(c_tile + col) * slot_ints;
                pw = __ldg(reinterpret_cast<const uint4*>(slot + nsb * 81 + sb * 4));
                dx = __int_as_float(__ldg(slot + nsb * 64 + sb));
            }
            const uint32_t o = (col >> 3) * 256 + (col & 7) * 16;
            *reinterpret_cast<uint4*>(sm + kOffBh + o) = make_uint4(pw.x, pw.y, 0u, 0u);
            *reinterpret_cast<uint4*>(sm + kOffBh + o + 128) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(sm + kOffBl + o) = make_uint4(pw.z, pw.w, 0u, 0u);
            *reinterpret_cast<uint4*>(sm + kOffBl + o + 128) = make_uint4(0u, 0u, 0u, 0u);
            dxs[col] = dx;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
        __syncthreads();
        // ---- 18 MMAs by one thread, completion on the mbarrier ----
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t base = smem_u32(sm);
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const uint64_t bd = smem_desc(base + kOffBx + s * kSlab);
                mma_i8<TN>(tmem + 0, smem_desc(base + kOffAa + s * kSlab), bd, s > 0);
                mma_i8<TN>(tmem + TN, smem_desc(base + kOffAb + s * kSlab), bd, s > 0);
            }
            const uint64_t md = smem_desc(base + kOffAm);
            mma_i8<TN>(tmem + 2 * TN, md, smem_desc(base + kOffBh), 0);
            mma_i8<TN>(tmem + 3 * TN, md, smem_desc(base + kOffBl), 0);
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
        }
        // ---- epilogue: read the four accumulators, apply the reference's two scale products ----
        const bool ok = mbar_wait_bounded(bar, static_cast<uint32_t>(sb - sb0) & 1u);
        if (__syncthreads_or(!ok)) {
            failed = true;
            break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned hdw = __ldg(reinterpret_cast<const unsigned*>(erow_blocks + static_cast<size_t>(sb) * kQ4KBlock));
        const float d = half_bits_to_float(hdw & 0xFFFFu), dmin = half_bits_to_float(hdw >> 16);
        const f32x2 d2 = pack2(d, d), dmin2 = pack2(dmin, dmin);
        const uint32_t trow = tmem + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + ecol0;
#pragma unroll
        for (int ch = 0; ch < TN / 32; ++ch) {
            int va[16], vb[16], vh[16], vl[16];
            tmem_ld16(trow + 16 * ch, va);
            tmem_ld16(trow + TN + 16 * ch, vb);
            tmem_ld16(trow + 2 * TN + 16 * ch, vh);
            tmem_ld16(trow + 3 * TN + 16 * ch, vl);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            after_tmem_wait(va), after_tmem_wait(vb), after_tmem_wait(vh), after_tmem_wait(vl);
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                const float2 dxp = *reinterpret_cast<const float2*>(dxs + ecol0 + 16 * ch + i);
                const f32x2 dx2 = pack2(dxp.x, dxp.y);
                const f32x2 is2 = pack2(static_cast<float>(32 * va[i] + vb[i]), static_cast<float>(32 * va[i + 1] + vb[i + 1]));
                const f32x2 im2 = pack2(static_cast<float>(64 * vh[i] + vl[i]), static_cast<float>(64 * vh[i + 1] + vl[i + 1]));
                float t1a, t1b, t2a, t2b;
                unpack2(mul2(mul2(d2, dx2), is2), t1a, t1b);
                unpack2(mul2(mul2(dmin2, dx2), im2), t2a, t2b);
                acc[16 * ch + i] = __fadd_rn(acc[16 * ch + i], __fsub_rn(t1a, t2a));
                acc[16 * ch + i + 1] = __fadd_rn(acc[16 * ch + i + 1], __fsub_rn(t1b, t2b));
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();  // TMEM and the operand slabs are free for the next super-block
    }
    float* out = partial ? partial + static_cast<size_t>(blockIdx.z) * ncols * rows : y;
    if (failed) {
        if (tid == 0) atomicAdd(&g_tc_timeouts, 1u);
    } else {
#pragma unroll
        for (int i = 0; i < TN / 2; ++i) {
            const int c = c_tile + ecol0 + i;
            if (c < ncols) out[static_cast<size_t>(c) * rows + r_tile + erow] = acc[i];
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(4 * TN) : "memory");
}

// ---- Q6_K --------------------------------------------------------------------------------------------------
// llm::ref::matvecQ6KQ8K (llm/llm_reference.cpp:564-596): per super-block
//     acc += (d * dx_c) * float(is),   is = sum over 16-weight groups g of sc_g * (dot16(q_g, x_g) - 32 * B_g)
// with q the raw 6-bit weights (0..63), sc the int8 group scale and B_g the activation sum of the group.  The
// -32 offset folds into the weight: is = sum_k w'_k x_k with w' = sc * (q - 32), |w'| <= 4096.  w' is split as
// w' = 64 a + b with a = w' >> 6 (arithmetic, -64..64) and b = w' & 63: two int8 planes, two accumulators,
// is = 64 Da + Db -- the same integer, so every output is bit-identical to the reference's per-column mirror.
// Weights are read from the device layout of Q6_K (four planes: ql | qh | scales | d).

// q4: four 6-bit weights in bytes, scb = sc + 128 (0..255), crep = (8192 - 32 sc) in both 16-bit lanes.
// Per 16-bit lane u = q * scb - 128 q + crep = sc * (q - 32) + 8192, in 4128..12288: never negative, no borrow
// between lanes.  (u >> 6) - 128 == w' >> 6 and subtracting 128 from a byte is flipping its top bit.
__device__ __forceinline__ void scale_split_q6(unsigned q4, unsigned scb, unsigned crep, unsigned& a, unsigned& b) {
    const unsigned qe = q4 & 0x00FF00FFu, qo = (q4 >> 8) & 0x00FF00FFu;
    const unsigned ue = qe * scb + crep - (qe << 7), uo = qo * scb + crep - (qo << 7);
    a = (((ue >> 6) & 0x00FF00FFu) | (((uo >> 6) & 0x00FF00FFu) << 8)) ^ 0x80808080u;
    b = (ue & 0x003F003Fu) | ((uo & 0x003F003Fu) << 8);
}

template <int TN>
__global__ void __launch_bounds__(kThreads, TN == 128 ? 1 : 2) matmul_q6k_q8k_tc_kernel(const uint8_t* __restrict__ w, const int* __restrict__ xq,
                                                                         float* __restrict__ y, int rows, int nsb, int ncols, int sb_per_split, float* __restrict__ partial) {
    extern __shared__ __align__(1024) uint8_t sm[];
    uint64_t* bar = reinterpret_cast<uint64_t*>(sm + kOffBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kOffBar + 16);
    float* dxs = reinterpret_cast<float*>(sm + kOffDx);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r_tile = blockIdx.x * TM, c_tile = blockIdx.y * TN;
    const int slot_ints = nsb * 85;
    const size_t nblk = static_cast<size_t>(rows) * nsb;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * TN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init_fence();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    const int erow = 32 * (warp & 3) + lane, ecol0 = (TN / 2) * (warp >> 2);
    float acc[TN / 2];
#pragma unroll
    for (int i = 0; i < TN / 2; ++i) acc[i] = 0.0f;
    // unpack role: tile row tid / 2, half n = tid & 1 of the super-block (weights 128 n .. 128 n + 127, K-steps 4n .. 4n+3)
    const int urow = tid >> 1, n = tid & 1;
    const size_t ublk0 = static_cast<size_t>(r_tile + urow) * nsb, eblk0 = static_cast<size_t>(r_tile + erow) * nsb;
    const uint32_t ubase = (urow >> 3) * 256 + (urow & 7) * 16;

    bool failed = false;
    // split K (partial != nullptr): this CTA contracts super-blocks [sb0, sb1) and leaves its sum in slice blockIdx.z
    const int sb0 = blockIdx.z * sb_per_split, sb1 = min(nsb, sb0 + sb_per_split);
    for (int sb = sb0; sb < sb1 && !failed; ++sb) {
        {
            const size_t blk = ublk0 + sb;
            uint4 lq[4], hq[2];
#pragma unroll
            for (int i = 0; i < 4; ++i) lq[i] = ldg_stream(w + blk * 128 + 64 * n + 16 * i);
#pragma unroll
            for (int i = 0; i < 2; ++i) hq[i] = ldg_stream(w + nblk * 128 + blk * 64 + 32 * n + 16 * i);
            const uint2 scw = __ldg(reinterpret_cast<const uint2*>(w + nblk * 192 + blk * 16 + 8 * n));
#pragma unroll
            for (int t = 0; t < 4; ++t) {      // K-step 4n + t: weights 128n + 32t .. +31
#pragma unroll
                for (int c = 0; c < 2; ++c) {  // 16 weights sharing scale 2t + c
                    const int si = 2 * t + c;
                    const int sc = static_cast<int>(((si < 4 ? scw.x : scw.y) << (24 - 8 * (si & 3)))) >> 24;
                    const unsigned scb = static_cast<unsigned>(sc + 128);
                    const unsigned c16 = static_cast<unsigned>(8192 - 32 * sc), crep = c16 | (c16 << 16);
                    const uint4 lv = lq[2 * (t & 1) + c], hv = hq[c];
                    const unsigned lw[4] = {lv.x, lv.y, lv.z, lv.w}, hw[4] = {hv.x, hv.y, hv.z, hv.w};
                    unsigned a[4], b[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const unsigned nib = (t >= 2 ? lw[i] >> 4 : lw[i]) & 0x0F0F0F0Fu;
                        const unsigned q4 = nib | (((hw[i] >> (2 * t)) & 0x03030303u) << 4);
                        scale_split_q6(q4, scb, crep, a[i], b[i]);
                    }
                    const int s = 4 * n + t;
                    *reinterpret_cast<uint4*>(sm + kOffAa + s * kSlab + ubase + 128 * c) = make_uint4(a[0], a[1], a[2], a[3]);
                    *reinterpret_cast<uint4*>(sm + kOffAb + s * kSlab + ubase + 128 * c) = make_uint4(b[0], b[1], b[2], b[3]);
                }
            }
        }
#pragma unroll
        for (int it = 0; it < TN * 16 / kThreads; ++it) {
            const int i = tid + kThreads * it;  // lane mapping as in the Q4_K kernel
            const int col = (i & 7) + 8 * (i >> 7), part = ((i >> 3) & 3) + 4 * ((i >> 5) & 3);
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (c_tile + col < ncols) v = __ldg(reinterpret_cast<const uint4*>(xq + static_cast<size_t>(c_tile + col) * slot_ints + sb * 64 + part * 4));
            *reinterpret_cast<uint4*>(sm + kOffBx + (part >> 1) * kSlab + (col >> 3) * 256 + (part & 1) * 128 + (col & 7) * 16) = v;
        }
        if (tid < TN) {
            float dx = 0.0f;
            if (c_tile + tid < ncols) dx = __int_as_float(__ldg(xq + static_cast<size_t>(c_tile + tid) * slot_ints + nsb * 64 + sb));
            dxs[tid] = dx;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t base = smem_u32(sm);
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const uint64_t bd = smem_desc(base + kOffBx + s * kSlab);
                mma_i8<TN>(tmem + 0, smem_desc(base + kOffAa + s * kSlab), bd, s > 0);
                mma_i8<TN>(tmem + TN, smem_desc(base + kOffAb + s * kSlab), bd, s > 0);
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
        }
        const bool ok = mbar_wait_bounded(bar, static_cast<uint32_t>(sb - sb0) & 1u);
        if (__syncthreads_or(!ok)) {
            failed = true;
            break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float d = half_bits_to_float(__ldg(reinterpret_cast<const unsigned short*>(w + nblk * 208 + (eblk0 + sb) * 2)));
        const f32x2 d2 = pack2(d, d);
        const uint32_t trow = tmem + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + ecol0;
#pragma unroll
        for (int ch = 0; ch < TN / 32; ++ch) {
            int va[16], vb[16];
            tmem_ld16(trow + 16 * ch, va);
            tmem_ld16(trow + TN + 16 * ch, vb);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            after_tmem_wait(va), after_tmem_wait(vb);
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                const float2 dxp = *reinterpret_cast<const float2*>(dxs + ecol0 + 16 * ch + i);
                const f32x2 is2 = pack2(static_cast<float>(64 * va[i] + vb[i]), static_cast<float>(64 * va[i + 1] + vb[i + 1]));
                float ta, tb;
                unpack2(mul2(mul2(d2, pack2(dxp.x, dxp.y)), is2), ta, tb);
                acc[16 * ch + i] = __fadd_rn(acc[16 * ch + i], ta);
                acc[16 * ch + i + 1] = __fadd_rn(acc[16 * ch + i + 1], tb);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
    }
    float* out = partial ? partial + static_cast<size_t>(blockIdx.z) * ncols * rows : y;
    if (failed) {
        if (tid == 0) atomicAdd(&g_tc_timeouts, 1u);
    } else {
#pragma unroll
        for (int i = 0; i < TN / 2; ++i) {
            const int c = c_tile + ecol0 + i;
            if (c < ncols) out[static_cast<size_t>(c) * rows + r_tile + erow] = acc[i];
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * TN) : "memory");
}

}  // namespace

namespace {
// Up to 64 columns (a batch of sequences decoding in lockstep) take 32-column tiles: a quarter of the epilogue and
// copy work per super-block, a quarter of the TMEM, so two CTAs share an SM and one's unpacking overlaps the other's
// MMAs; wider batches take 128-column tiles, which unpack each weight tile once per 128 columns.
// y[i] = ((p_0[i] + p_1[i]) + p_2[i]) + ...: the K slices of a split contraction, added in slice order.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, float* __restrict__ y, size_t n, int splits) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float a = partial[i];
    for (int z = 1; z < splits; ++z) a = __fadd_rn(a, partial[static_cast<size_t>(z) * n + i]);
    y[i] = a;
}

// Scratch for the K slices, one buffer per stream (calls on different streams may overlap), grown on demand and
// kept for the life of the process.
float* splitk_scratch(cudaStream_t s, size_t floats) {
    static std::mutex m;
    static std::map<cudaStream_t, std::pair<float*, size_t>> bufs;
    std::lock_guard<std::mutex> lock(m);
    auto& b = bufs[s];
    if (b.second < floats) {
        if (b.first) {
            cudaStreamSynchronize(s);
            cudaFree(b.first);
        }
        b = {nullptr, 0};
        void* p = nullptr;
        if (cudaMalloc(&p, floats * sizeof(float)) != cudaSuccess) return nullptr;
        b = {static_cast<float*>(p), floats};
    }
    return b.first;
}

// Super-blocks per K slice of a launch (nsb: one pass).  Few tiles leave SMs without one (or the last wave mostly
// empty) and every CTA with a long serial chain over the super-blocks: split K where a wave model says it pays.  A
// launch of `c` CTAs runs in ceil(c / slots) waves, a CTA costs its super-blocks plus ~1.5 super-block times of set-up
// and store, and the second kernel that adds the slices (in slice order: deterministic, but the fp32 sum is
// associated differently from the one-pass result, so outputs agree with the reference's mirror to ~1e-6 instead of
// bit for bit) costs about as much again.  The split must win by 10 %, contract at least two super-blocks per CTA
// and keep the slices within 64 MB.
int super_blocks_per_slice(int rows, int nsb, int ncols, int tn) {
    if (nsb < 4) return nsb;
    const int tiles = (rows / TM) * ((ncols + tn - 1) / tn);
    const int slots = kSmCount * (tn == 32 ? 2 : 1);  // CTAs the machine holds at once
    const auto cost = [&](int n_splits) {
        const int p = (nsb + n_splits - 1) / n_splits;
        const int waves = (tiles * n_splits + slots - 1) / slots;
        return waves * (2 * p + 3) + (n_splits > 1 ? 3 : 0);  // in half super-block times
    };
    int best = 1, best_cost = cost(1);
    for (int c = 2; c <= nsb / 2; ++c) {
        if ((nsb + c - 1) / c * (c - 1) >= nsb) continue;  // the last slice would be empty
        if (static_cast<size_t>(c) * ncols * rows * sizeof(float) > (64u << 20)) break;
        if (cost(c) < best_cost) best = c, best_cost = cost(c);
    }
    return best > 1 && 10 * best_cost <= 9 * cost(1) ? (nsb + best - 1) / best : nsb;
}
constexpr int tile_columns(int ncols) { return ncols <= 64 ? 32 : 128; }

template <bool kQ6, int TN>
int launch_tc_tn(const uint8_t* w, const int* xq, float* y, int rows, int nsb, int ncols, cudaStream_t s) {
    auto kern = kQ6 ? matmul_q6k_q8k_tc_kernel<TN> : matmul_q4k_q8k_tc_kernel<TN>;
    static bool attr_set = false;  // per instantiation
    if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) return KCB_LAUNCH_FAILURE;
        attr_set = true;
    }
    // K slices only outside stream capture, where the scratch can be allocated
    int per = nsb;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) per = super_blocks_per_slice(rows, nsb, ncols, TN);
    const int splits = (nsb + per - 1) / per;
    float* partial = nullptr;
    if (splits > 1) {
        partial = splitk_scratch(s, static_cast<size_t>(splits) * ncols * rows);
        if (!partial) return KCB_OUT_OF_MEMORY;
    } else {
        per = nsb;
    }
    const dim3 grid(rows / TM, (ncols + TN - 1) / TN, splits);
    kern<<<grid, kThreads, kSmemBytes, s>>>(w, xq, y, rows, nsb, ncols, per, partial);
    if (const int e = launch_status(); e != KCB_SUCCESS || splits == 1) return e;
    const size_t n = static_cast<size_t>(ncols) * rows;
    splitk_reduce_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(partial, y, n, splits);
    return launch_status();
}
template <bool kQ6>
int launch_tc(const uint8_t* w, const int* xq, float* y, int rows, int nsb, int ncols, cudaStream_t s) {
    return tile_columns(ncols) == 32 ? launch_tc_tn<kQ6, 32>(w, xq, y, rows, nsb, ncols, s) : launch_tc_tn<kQ6, 128>(w, xq, y, rows, nsb, ncols, s);
}
}  // namespace

// K slices a tensor-core launch of this shape takes outside stream capture (1: one pass, outputs bit-identical to the
// reference's mirror); 0 for shapes the tensor-core path does not take.
int matmul_tc_k_slices(int rows, int k, int ncols) {
    if (rows <= 0 || rows % TM || k <= 0 || k % 1024 || ncols <= 0) return 0;
    const int nsb = k / 256, per = super_blocks_per_slice(rows, nsb, ncols, tile_columns(ncols));
    return (nsb + per - 1) / per;
}

unsigned tc_timeouts() {
    unsigned v = 0;
    cudaMemcpyFromSymbol(&v, g_tc_timeouts, sizeof v);
    return v;
}

// Tensor-core path for Q4_K weights and per-256 activation slots; rows must be a multiple of 128.
int matmul_q4k_q8k_tc(const void* w, const int* xq, float* y, int rows, int k, int ncols, cudaStream_t s) {
    // k % 1024: a column's slot is 85 * k / 256 ints and is read with 16-byte loads
    if (rows <= 0 || rows % TM || k <= 0 || k % 1024 || ncols <= 0 || !w || !xq || !y) return KCB_INVALID_VALUE;
    return launch_tc<false>(static_cast<const uint8_t*>(w), xq, y, rows, k / 256, ncols, s);
}

// Tensor-core path for Q6_K weights (device planes) and per-256 activation slots; rows a multiple of 128.
int matmul_q6k_q8k_tc(const void* w, const int* xq, float* y, int rows, int k, int ncols, cudaStream_t s) {
    // k % 1024: a column's slot is 85 * k / 256 ints and is read with 16-byte loads
    if (rows <= 0 || rows % TM || k <= 0 || k % 1024 || ncols <= 0 || !w || !xq || !y) return KCB_INVALID_VALUE;
    return launch_tc<true>(static_cast<const uint8_t*>(w), xq, y, rows, k / 256, ncols, s);
}

}  // namespace kcb
