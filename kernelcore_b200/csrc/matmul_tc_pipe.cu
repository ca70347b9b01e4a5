// Pipelined Q4_K / Q6_K x Q8_K-activation matmuls on the 5th-generation tensor cores (tcgen05, int8 -> int32, TMEM):
// the prompt-phase contraction, warp-specialised so that weight unpacking, tensor-core work and the fp32 epilogue of
// neighbouring super-blocks overlap.
//
// Replaces the reference's kernels/llm/matmul_q4k_q8kx8.cu:41-239 / matmul_q6k_q8kx8.cu (one thread per row and 8
// columns, dp4a).  Arithmetic contract (llm/llm_reference.cpp:529-596), per output and super-block:
//     Q4_K:  acc += (d * dx) * float(is) - (dmin * dx) * float(im),  is = sum_j sc_j * dot32(q_j, x_j), im = sum_j m_j * B_j
//     Q6_K:  acc += (d * dx) * float(is),                             is = sum_g sc_g * (dot16(q_g, x_g) - 32 * B_g)
// The integers are exact GEMMs once the sub-block scale is folded into the weight:
//   * Q4_K: sc = 8 s1 + s0 with s1, s0 < 8, so sc * q = 8 (s1 q) + (s0 q) with both products <= 105: two int8 planes
//     made by ONE 32-bit multiply per four weights each (bytes never carry), is = 8 Da + Db.  The mins are a K = 8
//     contraction with the activation sums, which the reference stores as two bytes (B >> 6, B & 63): im = 64 Dh + Dl.
//   * Q6_K: w' = sc * (q - 32) = 64 a + b (a = w' >> 6, b = w' & 63), is = 64 Da + Db.
// The epilogue applies the reference's fp32 products in its order, so one-pass outputs are bit-identical to the
// reference's per-column mirror.
//
// One persistent CTA per SM walks a static list of (128-row x 128-column tile, super-block range) units:
//   * producer warps: one weight row (Q6_K: half a row) per thread; the next super-block's bytes are requested before
//     this one is unpacked; planes go to shared memory in the no-swizzle K-major core-matrix layout (conflict-free
//     512-byte stores per warp).  Producer thread 0 also issues the bulk tensor copies (TMA, no multicast) of the
//     activation bytes (128-byte-swizzled K-major tiles), the activation sums and the activation scales;
//   * one thread issues the MMAs: the 128 columns are two halves of 64 with their own TMEM accumulators, so the
//     epilogue of one half runs while the tensor core works on the other and on the next super-block;
//   * eight epilogue warps read TMEM (tcgen05.ld), combine the planes and accumulate in registers.
// Operand slabs are double-buffered (full / empty mbarriers), accumulators are handed over with tmem_full / tmem_empty
// mbarriers.  Every wait is bounded: on expiry the CTA raises a flag that the other roles poll, waits a bounded grace
// period for copies in flight, counts the event, frees its TMEM and returns.

#include "common.cuh"
#include "ops.h"

#include <cuda.h>  // CUtensorMap and its enums; the encoder itself is looked up through the runtime (no libcuda link)

#include <algorithm>
#include <mutex>

namespace kcb {
namespace {

constexpr int TM = 128, TN = 128, HN = 64;  // tile rows, tile columns, columns per accumulator half
constexpr int kEpiWarps = 8;
constexpr int kChunk = TM * 16;   // one 16-byte K chunk of a 128-row operand: [row][16 B]
constexpr int kAtom = 128 * 128;  // 128 rows x 128 K bytes in the 128-byte-swizzle layout
constexpr int kDxSlots = 4;

template <bool kQ6>
struct Cfg {
    static constexpr int kProdWarps = kQ6 ? 8 : 4;
    static constexpr int kProducers = 32 * kProdWarps;
    static constexpr int kThreads = 32 * (kEpiWarps + 1) + kProducers;
    static constexpr int kAccs = kQ6 ? 2 : 4;          // TMEM accumulators per half
    static constexpr int kHalfCols = kAccs * HN;        // TMEM columns of one half
    static constexpr int kTmemCols = 2 * kHalfCols;     // 512 (Q4_K) / 256 (Q6_K)
    // one operand stage
    static constexpr int kOffAa = 0;                    // plane a: 8 K-steps x 2 chunks
    static constexpr int kOffAb = 16 * kChunk;          // plane b
    static constexpr int kOffAm = 32 * kChunk;          // Q4_K: mins in K bytes 0..7 | mins in K bytes 8..15
    static constexpr int kOffBx = kOffAm + (kQ6 ? 0 : 2 * kChunk);  // two swizzled atoms (1024-byte aligned)
    static constexpr int kOffBs = kOffBx + 2 * kAtom;   // Q4_K: activation sums, one chunk
    static constexpr int kStage = kOffBs + (kQ6 ? 0 : kChunk);
    // behind the two stages
    static constexpr int kOffZero = 2 * kStage;         // Q4_K: a chunk of zeros (second K chunk of the min MMAs)
    static constexpr int kOffDx = kOffZero + (kQ6 ? 0 : kChunk);  // ring of kDxSlots chunks: [column][4 floats]
    static constexpr int kOffBar = kOffDx + kDxSlots * kChunk;
    static constexpr int kSmem = kOffBar + 256 + 1024;  // + room to align the base to 1024 bytes
    static_assert(kOffBx % 1024 == 0 && kStage % 1024 == 0, "swizzled atoms need 1024-byte alignment");
};

__device__ unsigned g_tcp_timeouts = 0;

// ---- descriptors and tcgen05 wrappers --------------------------------------------------------------------------
// K-major, no swizzle: core matrices of 8 rows x 16 bytes; `lbo` = distance between the two 16-byte K chunks of a
// K = 32 step, `sbo` = distance between 8-row groups.
__device__ __forceinline__ uint64_t desc_nosw(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo >> 4) << 16) | (static_cast<uint64_t>(sbo >> 4) << 32) |
           (static_cast<uint64_t>(1) << 46);
}
// K-major, 128-byte swizzle (what a tensor copy with the 128-byte swizzle writes): rows of 128 K bytes, 8-row groups
// 1024 bytes apart; a K = 32 step inside the row is addressed by adding 32 bytes to the start address.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) |
           (static_cast<uint64_t>(2) << 61);
}
// int32 accumulate, signed 8-bit A and B, both K-major, M = 128, N = 64.
constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(HN >> 3) << 17) | (static_cast<uint32_t>(TM >> 4) << 24);

__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr));
}
// tcgen05.ld is asynchronous: the registers hold the data only after tcgen05.wait::ld, an asm statement without register
// operands.  Passing the registers through this empty volatile asm ties every later use to a point behind the wait.
__device__ __forceinline__ void after_tmem_wait(int (&v)[8]) {
    asm volatile("" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7])::"memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Tiled 2-D tensor copy global -> this CTA's shared memory (no multicast); completion counted on `bar`.
__device__ __forceinline__ void tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
// Bounded wait that also gives up when another role of the CTA has raised the failure flag.
__device__ __forceinline__ bool wait_or_fail(uint64_t* bar, uint32_t parity, volatile int* fail) {
    for (int i = 0; i < kMbarSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255) == 255 && *fail) return false;
    }
    *fail = 1;
    return false;
}

// Packed fp32 pairs: each lane of a pair is rounded exactly as the scalar _rn operation.  Only multiplies are packed;
// ptxas would contract a packed multiply followed by a packed add / subtract into one fused operation (a single
// rounding), which would break bit identity with the reference, so those stay scalar _rn intrinsics.
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

// ---- weight blocks in registers and their unpacking ------------------------------------------------------------
struct Q4Blk {
    uint4 hd, q[8];
};
__device__ __forceinline__ void load_blk(Q4Blk& b, const uint8_t* w, size_t /*nblk*/, size_t blk, int /*n*/) {
    const uint4* p = reinterpret_cast<const uint4*>(w + blk * kQ4KBlock);
    b.hd = __ldg(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) b.q[i] = __ldg(p + 1 + i);
}
// One row of one super-block: planes a = (sc >> 3) * q and b = (sc & 7) * q for the eight K-steps (sub-blocks), the mins
// as K bytes 0..7 of one chunk and 8..15 of the other.
template <class C>
__device__ __forceinline__ void unpack_blk(const Q4Blk& b, uint8_t* stage, int row, int /*n*/) {
    const unsigned sclo = b.hd.y & 0x3F3F3F3Fu, schi = (b.hd.w & 0x0F0F0F0Fu) | ((b.hd.y >> 2) & 0x30303030u);
    const unsigned mlo = b.hd.z & 0x3F3F3F3Fu, mhi = ((b.hd.w >> 4) & 0x0F0F0F0Fu) | ((b.hd.z >> 2) & 0x30303030u);
    uint8_t* pa = stage + C::kOffAa + row * 16;
    uint8_t* pb = stage + C::kOffAb + row * 16;
#pragma unroll
    for (int g = 0; g < 4; ++g) {  // 32 quant bytes: low nibbles = sub-block 2g, high nibbles = sub-block 2g + 1
        const unsigned scw = (g < 2 ? sclo : schi) >> (16 * (g & 1));
        const unsigned sl = scw & 255u, sh = (scw >> 8) & 255u;
        const unsigned sl1 = sl >> 3, sl0 = sl & 7u, sh1 = sh >> 3, sh0 = sh & 7u;
#pragma unroll
        for (int c = 0; c < 2; ++c) {  // 16 bytes = K chunk c of both sub-blocks
            const uint4 v = b.q[2 * g + c];
            const unsigned lx = v.x & 0x0F0F0F0Fu, ly = v.y & 0x0F0F0F0Fu, lz = v.z & 0x0F0F0F0Fu, lw = v.w & 0x0F0F0F0Fu;
            const unsigned hx = (v.x >> 4) & 0x0F0F0F0Fu, hy = (v.y >> 4) & 0x0F0F0F0Fu, hz = (v.z >> 4) & 0x0F0F0F0Fu, hw = (v.w >> 4) & 0x0F0F0F0Fu;
            const int klo = (2 * (2 * g) + c) * kChunk, khi = (2 * (2 * g + 1) + c) * kChunk;
            *reinterpret_cast<uint4*>(pa + klo) = make_uint4(lx * sl1, ly * sl1, lz * sl1, lw * sl1);
            *reinterpret_cast<uint4*>(pb + klo) = make_uint4(lx * sl0, ly * sl0, lz * sl0, lw * sl0);
            *reinterpret_cast<uint4*>(pa + khi) = make_uint4(hx * sh1, hy * sh1, hz * sh1, hw * sh1);
            *reinterpret_cast<uint4*>(pb + khi) = make_uint4(hx * sh0, hy * sh0, hz * sh0, hw * sh0);
        }
    }
    *reinterpret_cast<uint4*>(stage + C::kOffAm + row * 16) = make_uint4(mlo, mhi, 0u, 0u);
    *reinterpret_cast<uint4*>(stage + C::kOffAm + kChunk + row * 16) = make_uint4(0u, 0u, mlo, mhi);
}

struct Q6Blk {
    uint4 lq[4], hq[2];
    uint2 sc;
};
// Half n of a block (weights 128 n .. 128 n + 127) out of the device planes ql | qh | scales | d.
__device__ __forceinline__ void load_blk(Q6Blk& b, const uint8_t* w, size_t nblk, size_t blk, int n) {
#pragma unroll
    for (int i = 0; i < 4; ++i) b.lq[i] = __ldg(reinterpret_cast<const uint4*>(w + blk * 128 + 64 * n + 16 * i));
#pragma unroll
    for (int i = 0; i < 2; ++i) b.hq[i] = __ldg(reinterpret_cast<const uint4*>(w + nblk * 128 + blk * 64 + 32 * n + 16 * i));
    b.sc = __ldg(reinterpret_cast<const uint2*>(w + nblk * 192 + blk * 16 + 8 * n));
}
// q4: four 6-bit weights in bytes, scb = sc + 128 (0..255), crep = (8192 - 32 sc) in both 16-bit lanes.
// Per 16-bit lane u = q * scb - 128 q + crep = sc * (q - 32) + 8192, in 4128..12288: never negative, no borrow
// between lanes.  (u >> 6) - 128 == w' >> 6 and subtracting 128 from a byte is flipping its top bit.
__device__ __forceinline__ void scale_split_q6(unsigned q4, unsigned scb, unsigned crep, unsigned& a, unsigned& b) {
    const unsigned qe = q4 & 0x00FF00FFu, qo = (q4 >> 8) & 0x00FF00FFu;
    const unsigned ue = qe * scb + crep - (qe << 7), uo = qo * scb + crep - (qo << 7);
    a = (((ue >> 6) & 0x00FF00FFu) | (((uo >> 6) & 0x00FF00FFu) << 8)) ^ 0x80808080u;
    b = (ue & 0x003F003Fu) | ((uo & 0x003F003Fu) << 8);
}
template <class C>
__device__ __forceinline__ void unpack_blk(const Q6Blk& blk, uint8_t* stage, int row, int n) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {      // K-step 4n + t: weights 128n + 32t .. +31
#pragma unroll
        for (int c = 0; c < 2; ++c) {  // 16 weights sharing scale 2t + c
            const int si = 2 * t + c;
            const int sc = static_cast<int>(((si < 4 ? blk.sc.x : blk.sc.y) << (24 - 8 * (si & 3)))) >> 24;
            const unsigned scb = static_cast<unsigned>(sc + 128);
            const unsigned c16 = static_cast<unsigned>(8192 - 32 * sc), crep = c16 | (c16 << 16);
            const uint4 lv = blk.lq[2 * (t & 1) + c], hv = blk.hq[c];
            const unsigned lw[4] = {lv.x, lv.y, lv.z, lv.w}, hw[4] = {hv.x, hv.y, hv.z, hv.w};
            unsigned a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const unsigned nib = (t >= 2 ? lw[i] >> 4 : lw[i]) & 0x0F0F0F0Fu;
                const unsigned q4 = nib | (((hw[i] >> (2 * t)) & 0x03030303u) << 4);
                scale_split_q6(q4, scb, crep, a[i], b[i]);
            }
            const int ko = (2 * (4 * n + t) + c) * kChunk + row * 16;
            *reinterpret_cast<uint4*>(stage + C::kOffAa + ko) = make_uint4(a[0], a[1], a[2], a[3]);
            *reinterpret_cast<uint4*>(stage + C::kOffAb + ko) = make_uint4(b[0], b[1], b[2], b[3]);
        }
    }
}

// ---- the kernel ------------------------------------------------------------------------------------------------
// Units: u -> (row tile, column tile, K slice); CTA b takes units b, b + gridDim.x, ...; a unit contracts super-blocks
// [z * per, min(nsb, (z + 1) * per)) and stores into y (one slice) or into slice z of `partial`.
template <bool kQ6>
__global__ void __launch_bounds__(Cfg<kQ6>::kThreads, 1)
    matmul_kq_q8k_pipe_kernel(const uint8_t* __restrict__ w, const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_s,
                              float* __restrict__ y, int rows, int nsb, int ncols, int per, int n_rt, int n_ct, int units,
                              float* __restrict__ partial) {
    using C = Cfg<kQ6>;
    using Blk = typename std::conditional<kQ6, Q6Blk, Q4Blk>::type;
    extern __shared__ uint8_t sm_raw[];
    uint8_t* sm = sm_raw + ((1024u - (smem_u32(sm_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + C::kOffBar);
    uint64_t* full = bars;            // [2] operands of a stage written (producers + tensor copies)
    uint64_t* empty = bars + 2;       // [2] the MMAs reading a stage have completed
    uint64_t* tfull = bars + 4;       // [2] accumulators of a half complete
    uint64_t* tempty = bars + 6;      // [2] accumulators of a half read back
    uint64_t* dxfull = bars + 8;      // [kDxSlots] activation scales of an item landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* fail = reinterpret_cast<volatile int*>(bars + 13);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t nblk = static_cast<size_t>(rows) * nsb;

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&full[s], C::kProducers + 1);
            mbar_init(&empty[s], 1);
            mbar_init(&tfull[s], 1);
            mbar_init(&tempty[s], kEpiWarps);
        }
        for (int s = 0; s < kDxSlots; ++s) mbar_init(&dxfull[s], 1);
        *fail = 0;
        mbar_init_fence();
    }
    if (!kQ6)  // zeros behind the min operands, written once
        for (int i = tid; i < kChunk / 16; i += C::kThreads) *reinterpret_cast<uint4*>(sm + C::kOffZero + i * 16) = make_uint4(0u, 0u, 0u, 0u);
    if (warp == kEpiWarps) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    auto unit_of = [&](int u, int& rt, int& ct, int& sb0, int& sb1) {
        rt = u % n_rt;
        const int r = u / n_rt;
        ct = r % n_ct;
        sb0 = (r / n_ct) * per;
        sb1 = min(nsb, sb0 + per);
    };

    if (warp < kEpiWarps) {
        // ================= epilogue: TMEM lanes 32 * (warp & 3) .. + 31, columns 32 * (warp >> 2) .. + 31 of each half
        const int erow = 32 * (warp & 3) + lane, cs = warp >> 2;
        const uint32_t tlane = tmem + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + 32 * cs;
        int it = 0, use[2] = {0, 0};  // items so far; uses of each accumulator half (a ragged last column tile skips half 1)
        bool ok = true;
        for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
            int rt, ct, sb0, sb1;
            unit_of(u, rt, ct, sb0, sb1);
            const int c_tile = ct * TN, nh = ncols - c_tile > HN ? 2 : 1;
            const size_t eblk = static_cast<size_t>(rt * TM + erow) * nsb;
            float acc[2 * 32];
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
            for (int sb = sb0; sb < sb1 && ok; ++sb, ++it) {
                float d, dmin = 0.0f;
                if (kQ6) {
                    d = half_bits_to_float(__ldg(reinterpret_cast<const unsigned short*>(w + nblk * 208 + (eblk + sb) * 2)));
                } else {
                    const unsigned hdw = __ldg(reinterpret_cast<const unsigned*>(w + (eblk + sb) * kQ4KBlock));
                    d = half_bits_to_float(hdw & 0xFFFFu), dmin = half_bits_to_float(hdw >> 16);
                }
                const f32x2 d2 = pack2(d, d), dmin2 = pack2(dmin, dmin);
                const int slot = it & (kDxSlots - 1);
                ok = wait_or_fail(&dxfull[slot], static_cast<uint32_t>(it / kDxSlots) & 1u, fail);
                if (!ok) break;
                const float* dxs = reinterpret_cast<const float*>(sm + C::kOffDx + slot * kChunk) + (sb & 3);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h >= nh) break;
                    ok = wait_or_fail(&tfull[h], static_cast<uint32_t>(use[h]++) & 1u, fail);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t t0 = tlane + h * C::kHalfCols;
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {  // 8 columns at a time
                        const int col0 = HN * h + 32 * cs + 8 * ch;
                        if (c_tile + col0 >= ncols) continue;
                        int va[8], vb[8];
                        tmem_ld8(t0 + 8 * ch, va);
                        tmem_ld8(t0 + HN + 8 * ch, vb);
                        if (kQ6) {
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            after_tmem_wait(va), after_tmem_wait(vb);
#pragma unroll
                            for (int i = 0; i < 8; i += 2) {
                                const f32x2 dx2 = pack2(dxs[(col0 + i) * 4], dxs[(col0 + i + 1) * 4]);
                                const f32x2 is2 = pack2(static_cast<float>(64 * va[i] + vb[i]), static_cast<float>(64 * va[i + 1] + vb[i + 1]));
                                float ta, tb;
                                unpack2(mul2(mul2(d2, dx2), is2), ta, tb);
                                acc[32 * h + 8 * ch + i] = __fadd_rn(acc[32 * h + 8 * ch + i], ta);
                                acc[32 * h + 8 * ch + i + 1] = __fadd_rn(acc[32 * h + 8 * ch + i + 1], tb);
                            }
                        } else {
                            int vh[8], vl[8];
                            tmem_ld8(t0 + 2 * HN + 8 * ch, vh);
                            tmem_ld8(t0 + 3 * HN + 8 * ch, vl);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            after_tmem_wait(va), after_tmem_wait(vb), after_tmem_wait(vh), after_tmem_wait(vl);
#pragma unroll
                            for (int i = 0; i < 8; i += 2) {
                                const f32x2 dx2 = pack2(dxs[(col0 + i) * 4], dxs[(col0 + i + 1) * 4]);
                                const f32x2 is2 = pack2(static_cast<float>(8 * va[i] + vb[i]), static_cast<float>(8 * va[i + 1] + vb[i + 1]));
                                const f32x2 im2 = pack2(static_cast<float>(64 * vh[i] + vl[i]), static_cast<float>(64 * vh[i + 1] + vl[i + 1]));
                                float t1a, t1b, t2a, t2b;
                                unpack2(mul2(mul2(d2, dx2), is2), t1a, t1b);
                                unpack2(mul2(mul2(dmin2, dx2), im2), t2a, t2b);
                                acc[32 * h + 8 * ch + i] = __fadd_rn(acc[32 * h + 8 * ch + i], __fsub_rn(t1a, t2a));
                                acc[32 * h + 8 * ch + i + 1] = __fadd_rn(acc[32 * h + 8 * ch + i + 1], __fsub_rn(t1b, t2b));
                            }
                        }
                    }
                    // this warp's share of the half has been read: hand the accumulators back
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tempty[h]);
                }
            }
            if (ok) {
                float* out = (partial ? partial + static_cast<size_t>(sb0 / per) * ncols * rows : y) + rt * TM + erow;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int c = c_tile + HN * h + 32 * cs + j;
                        if (c < ncols) out[static_cast<size_t>(c) * rows] = acc[32 * h + j];
                    }
            }
        }
    } else if (warp == kEpiWarps) {
        // ================= MMA issue: one thread
        if (lane == 0) {
            int it = 0, use[2] = {0, 0};
            bool ok = true;
            const uint32_t base = smem_u32(sm);
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
                int rt, ct, sb0, sb1;
                unit_of(u, rt, ct, sb0, sb1);
                const int nh = ncols - ct * TN > HN ? 2 : 1;
                for (int sb = sb0; sb < sb1 && ok; ++sb, ++it) {
                    const int s = it & 1;
                    const uint32_t ph = static_cast<uint32_t>(it >> 1) & 1u;
                    ok = wait_or_fail(&full[s], ph, fail);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st = base + s * C::kStage;
                    for (int h = 0; h < nh && ok; ++h) {
                        ok = wait_or_fail(&tempty[h], (static_cast<uint32_t>(use[h]++) & 1u) ^ 1u, fail);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t td = tmem + h * C::kHalfCols;
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {
                            const uint64_t bd = desc_sw128(st + C::kOffBx + (ks >> 2) * kAtom + h * (HN * 128) + (ks & 3) * 32);
                            mma_i8(td, desc_nosw(st + C::kOffAa + 2 * ks * kChunk, kChunk, 128), bd, ks > 0);
                            mma_i8(td + HN, desc_nosw(st + C::kOffAb + 2 * ks * kChunk, kChunk, 128), bd, ks > 0);
                        }
                        if (!kQ6) {
                            const uint32_t zero = base + C::kOffZero;
                            const uint32_t am = st + C::kOffAm, bs = st + C::kOffBs + h * (HN * 16);
                            const uint64_t sd = desc_nosw(bs, zero - bs, 128);
                            mma_i8(td + 2 * HN, desc_nosw(am, zero - am, 128), sd, 0);
                            mma_i8(td + 3 * HN, desc_nosw(am + kChunk, zero - (am + kChunk), 128), sd, 0);
                        }
                        mma_commit(&tfull[h]);
                    }
                    mma_commit(&empty[s]);
                }
            }
        }
    } else {
        // ================= producers: weight planes (all) and the tensor copies of the activations (thread 0)
        const int p = tid - 32 * (kEpiWarps + 1);
        const int row = p & (TM - 1), n = p >> 7;
        int it = 0;
        bool ok = true;
        Blk cur, nxt;
        {
            int rt, ct, sb0, sb1;
            if (static_cast<int>(blockIdx.x) < units) {
                unit_of(blockIdx.x, rt, ct, sb0, sb1);
                load_blk(cur, w, nblk, static_cast<size_t>(rt * TM + row) * nsb + sb0, n);
            }
        }
        for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
            int rt, ct, sb0, sb1;
            unit_of(u, rt, ct, sb0, sb1);
            for (int sb = sb0; sb < sb1 && ok; ++sb, ++it) {
                // next item's weights: requested now, unpacked one round later
                {
                    int nrt = rt, nsb_next = sb + 1;
                    bool have = nsb_next < sb1;
                    if (!have && u + static_cast<int>(gridDim.x) < units) {
                        int nct, nsb1;
                        unit_of(u + gridDim.x, nrt, nct, nsb_next, nsb1);
                        have = true;
                    }
                    if (have) load_blk(nxt, w, nblk, static_cast<size_t>(nrt * TM + row) * nsb + nsb_next, n);
                }
                const int s = it & 1;
                ok = wait_or_fail(&empty[s], (static_cast<uint32_t>(it >> 1) & 1u) ^ 1u, fail);
                if (!ok) break;
                uint8_t* st = sm + s * C::kStage;
                if (p == 0) {
                    const int c_tile = ct * TN;
                    mbar_expect_tx(&full[s], 2 * kAtom + (kQ6 ? 0 : kChunk));
                    tma_2d(st + C::kOffBx, &map_x, sb * 256, c_tile, &full[s]);
                    tma_2d(st + C::kOffBx + kAtom, &map_x, sb * 256 + 128, c_tile, &full[s]);
                    if (!kQ6) tma_2d(st + C::kOffBs, &map_s, nsb * 324 + sb * 16, c_tile, &full[s]);
                    const int slot = it & (kDxSlots - 1);
                    mbar_expect_tx(&dxfull[slot], kChunk);
                    tma_2d(sm + C::kOffDx + slot * kChunk, &map_s, nsb * 256 + (sb >> 2) * 16, c_tile, &dxfull[slot]);
                }
                unpack_blk<C>(cur, st, row, n);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core
                mbar_arrive(&full[s]);
                cur = nxt;
            }
        }
    }

    // ---- common exit -------------------------------------------------------------------------------------------------
    if (*fail)
        for (int t = 0; t < 1000; ++t) __nanosleep(1000);  // bounded grace for copies and MMAs still in flight
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && *fail) atomicAdd(&g_tcp_timeouts, 1u);
    if (warp == kEpiWarps) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
    }
}

// y[i] = ((p_0[i] + p_1[i]) + p_2[i]) + ...: the K slices of a split contraction, added in slice order.
__global__ void splitk_sum_kernel(const float* __restrict__ partial, float* __restrict__ y, size_t n, int splits) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float a = partial[i];
    for (int z = 1; z < splits; ++z) a = __fadd_rn(a, partial[static_cast<size_t>(z) * n + i]);
    y[i] = a;
}

// ---- host side ---------------------------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encoder() {
    static EncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}
// The activation slots as a 2-D byte tensor [ncols][slot_bytes]; boxes of 128 columns x `box_bytes`.
bool slots_map(CUtensorMap* m, const int* xq, int nsb, int ncols, int box_bytes, bool swizzle) {
    const EncodeTiled enc = encoder();
    if (!enc) return false;
    const cuuint64_t slot_bytes = static_cast<cuuint64_t>(nsb) * 85 * 4;
    const cuuint64_t dims[2] = {slot_bytes, static_cast<cuuint64_t>(ncols)};
    const cuuint64_t strides[1] = {slot_bytes};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), 128u};
    const cuuint32_t estr[2] = {1u, 1u};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int*>(xq), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// K slices of a launch.  A persistent CTA runs its units back to back, a unit of p super-blocks costing about p + 1
// super-block times (pipeline fill), and the second kernel that adds the slices about two more.  Splitting must win by
// 10 %, keep at least two super-blocks per slice and the slices within 64 MB.
int super_blocks_per_slice_pipe(int rows, int nsb, int ncols) {
    if (nsb < 4) return nsb;
    const int tiles = (rows / TM) * ((ncols + TN - 1) / TN);
    const auto cost = [&](int c) {
        const int p = (nsb + c - 1) / c;
        return (tiles * c + kSmCount - 1) / kSmCount * (p + 1) + (c > 1 ? 2 : 0);
    };
    int best = 1, best_cost = cost(1);
    for (int c = 2; c <= nsb / 2; ++c) {
        if ((nsb + c - 1) / c * (c - 1) >= nsb) continue;  // the last slice would be empty
        if (static_cast<size_t>(c) * ncols * rows * sizeof(float) > (64u << 20)) break;
        if (cost(c) < best_cost) best = c, best_cost = cost(c);
    }
    return best > 1 && 10 * best_cost <= 9 * cost(1) ? (nsb + best - 1) / best : nsb;
}

template <bool kQ6>
int launch_pipe(const uint8_t* w, const int* xq, float* y, int rows, int nsb, int ncols, float* workspace, size_t workspace_bytes, cudaStream_t s) {
    using C = Cfg<kQ6>;
    auto kern = matmul_kq_q8k_pipe_kernel<kQ6>;
    static PerDeviceFlag raised;
    if (!raise_dynamic_smem(kern, C::kSmem, raised)) return KCB_LAUNCH_FAILURE;
    CUtensorMap map_x, map_s;
    if (!slots_map(&map_x, xq, nsb, ncols, 128, true) || !slots_map(&map_s, xq, nsb, ncols, 16, false)) return KCB_INTERNAL_ERROR;
    // K slices only when the caller's workspace holds them: the same route inside and outside stream capture
    int per = super_blocks_per_slice_pipe(rows, nsb, ncols);
    int splits = (nsb + per - 1) / per;
    if (splits > 1 && (!workspace || workspace_bytes < static_cast<size_t>(splits) * ncols * rows * sizeof(float))) per = nsb, splits = 1;
    const int n_rt = rows / TM, n_ct = (ncols + TN - 1) / TN, units = n_rt * n_ct * splits;
    const int grid = std::min(units, kSmCount);
    kern<<<grid, C::kThreads, C::kSmem, s>>>(w, map_x, map_s, y, rows, nsb, ncols, per, n_rt, n_ct, units, splits > 1 ? workspace : nullptr);
    if (const int e = launch_status(); e != KCB_SUCCESS || splits == 1) return e;
    const size_t n = static_cast<size_t>(ncols) * rows;
    splitk_sum_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(workspace, y, n, splits);
    return launch_status();
}

}  // namespace

unsigned tc_pipe_timeouts() {
    unsigned v = 0;
    cudaMemcpyFromSymbol(&v, g_tcp_timeouts, sizeof v);
    return v;
}

// K slices the pipelined launch of this shape takes when given a workspace of matmul_tc_workspace_bytes (1: one pass).
int matmul_tc_pipe_k_slices(int rows, int k, int ncols) {
    if (rows <= 0 || rows % TM || k <= 0 || k % 1024 || ncols <= 0) return 0;
    const int nsb = k / 256, per = super_blocks_per_slice_pipe(rows, nsb, ncols);
    return (nsb + per - 1) / per;
}
size_t matmul_tc_workspace_bytes(int rows, int k, int ncols) {
    const int c = matmul_tc_pipe_k_slices(rows, k, ncols);
    return c > 1 ? static_cast<size_t>(c) * ncols * rows * sizeof(float) : 0;
}

// Tensor-core path for K-quant weights and per-256 activation slots; rows a multiple of 128, k of 1024 (a column's slot
// is 85 * k / 256 ints and must be a multiple of 16 bytes for the tensor copies).  `workspace` (device memory, may be
// null) lets the launch split K across CTAs when that pays; without it the launch is one pass.
int matmul_kq_q8k_tc_pipe(const void* w, const int* xq, float* y, int rows, int k, int ncols, int q6, void* workspace, size_t workspace_bytes,
                          cudaStream_t s) {
    if (rows <= 0 || rows % TM || k <= 0 || k % 1024 || ncols <= 0 || !w || !xq || !y) return KCB_INVALID_VALUE;
    if (misaligned(w, 16) || misaligned(xq, 16) || misaligned(y, 4) || misaligned(workspace, 4)) return KCB_INVALID_POINTER;
    return q6 ? launch_pipe<true>(static_cast<const uint8_t*>(w), xq, y, rows, k / 256, ncols, static_cast<float*>(workspace), workspace_bytes, s)
              : launch_pipe<false>(static_cast<const uint8_t*>(w), xq, y, rows, k / 256, ncols, static_cast<float*>(workspace), workspace_bytes, s);
}

}  // namespace kcb
