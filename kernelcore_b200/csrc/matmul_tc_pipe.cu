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
// Orientation: the ACTIVATIONS are the M operand (128 columns of the batch = 128 TMEM lanes) and the weight planes the
// N operand: one MMA of N = 128 covers plane a and plane b of 64 weight rows, so the activation slab is read from
// shared memory once for both planes, and an epilogue thread (= one activation column) finds Da and Db of a weight
// row side by side in its own lane.  The 128 weight rows of a tile are two halves of 64 with their own TMEM
// accumulators: the epilogue of one half runs while the tensor core works on the other and on the next super-block.
//
// One persistent CTA per SM walks a static list of (128-row x 128-column tile, super-block range) units:
//   * producer warps: one weight row (Q6_K: half a row) per thread; the next super-block's bytes are requested before
//     this one is unpacked; planes go to shared memory in the no-swizzle K-major core-matrix layout (conflict-free
//     512-byte stores per warp), the row's fp16 scales as floats into a small ring.  Producer thread 0 also issues
//     the bulk tensor copies (TMA, no multicast) of the activation bytes (128-byte-swizzled K-major tiles) and the
//     activation sums;
//   * one thread issues the MMAs (18 per super-block for Q4_K, 16 for Q6_K);
//   * eight epilogue warps read TMEM (tcgen05.ld, the next four rows requested while these four are combined) and
//     accumulate in registers; a thread's activation scale is a scalar per super-block.
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

constexpr int TM = 128, TN = 128, HR = 64;  // weight rows per tile, activation columns per tile, weight rows per accumulator half
constexpr int kEpiWarps = 8;
constexpr int kChunk = 128 * 16;  // one 16-byte K chunk of a 128-row operand: [row][16 B]
constexpr int kAtom = 128 * 128;  // 128 rows x 128 K bytes in the 128-byte-swizzle layout
constexpr int kRing = 4;          // slots of the per-row scale ring

template <bool kQ6>
struct Cfg {
    static constexpr int kProdWarps = kQ6 ? 8 : 4;
    static constexpr int kProducers = 32 * kProdWarps;
    // warps: 8 epilogue (two warpgroups) | kProdWarps producers (whole warpgroups) | one warpgroup holding the MMA
    // warp and three idle warps, which exists to hand its registers to the epilogue warpgroups (setmaxnreg below)
    static constexpr int kMmaWarp = kEpiWarps + kProdWarps;
    static constexpr int kThreads = 32 * (kMmaWarp + 4);
    static constexpr int kRegsLaunch = kQ6 ? 96 : 128;   // what kThreads allows: 65536 / 640, 65536 / 512
    static constexpr int kRegsEpi = kQ6 ? 120 : 168;     // epilogue warps after the hand-over
    static constexpr int kRegsMma = 40;                   // the MMA warpgroup keeps this much
    static_assert(8 * 32 * (kRegsEpi - kRegsLaunch) <= 4 * 32 * (kRegsLaunch - kRegsMma), "the epilogue takes what the MMA warpgroup gives up");
    static constexpr int kHalfCols = kQ6 ? 128 : 256;   // TMEM columns of one half: Da | Db (| Dh | Dl), 64 each
    static constexpr int kTmemCols = 2 * kHalfCols;      // 512 (Q4_K) / 256 (Q6_K)
    // one operand stage
    static constexpr int kOffW = 0;                      // [half][K-step][chunk][plane a rows 0..63 | plane b rows 0..63][16 B]
    static constexpr int kOffWm = 32 * kChunk;           // Q4_K: [half][mins in K bytes 0..7 (64 rows) | mins in K bytes 8..15 (64 rows)]
    static constexpr int kOffX = kOffWm + (kQ6 ? 0 : 2 * kChunk);  // two swizzled atoms (1024-byte aligned)
    static constexpr int kOffXs = kOffX + 2 * kAtom;     // Q4_K: activation sums, one chunk
    static constexpr int kStage = kOffXs + (kQ6 ? 0 : kChunk);
    // behind the two stages
    static constexpr int kOffZero = 2 * kStage;          // Q4_K: a chunk of zeros (second K chunk of the min MMAs)
    static constexpr int kOffDd = kOffZero + (kQ6 ? 0 : kChunk);  // ring: per row pair {d, d', dmin, dmin'} (Q6_K: {d, d'})
    static constexpr int kDdSlot = kQ6 ? 512 : 1024;
    static constexpr int kOffBar = kOffDd + kRing * kDdSlot;
    static constexpr int kSmem = kOffBar + 256 + 1024;   // + room to align the base to 1024 bytes
    static_assert(kOffX % 1024 == 0 && kStage % 1024 == 0, "swizzled atoms need 1024-byte alignment");
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
// int32 accumulate, signed 8-bit A and B, both K-major, M = 128, N = 128.
constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(128 >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);

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

__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 pack2i(int a, int b) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a), "r"(b));
    return r;
}
// Exact int32 -> fp32 without the conversion unit (which issues at a sixteenth of the fp32 rate and was what the
// epilogue waited for).  For |v| < 2^22 the bit pattern 0x4B400000 + v is the float 1.5 * 2^23 + v, so subtracting
// 1.5 * 2^23 gives float(v) exactly; with the exponent raised by s (0x4B400000 + (s << 23)) the same pattern is
// 1.5 * 2^(23 + s) + 2^s v.  A value F a + b with |a|, |b| < 2^22 and F = 2^s is therefore converted as
// (2^s a exactly) + (b exactly) in ONE fp32 addition, which rounds the exact integer once, to nearest even -- the
// result of converting the integer F a + b itself, for every input.
template <int S>
__device__ __forceinline__ f32x2 planes_to_float2(int a0, int a1, int b0, int b1) {
    constexpr int kMagicA = 0x4B400000 + (S << 23), kMagicB = 0x4B400000;
    const float ca = -__int_as_float(kMagicA), cb = -12582912.0f;
    const f32x2 fa = add2(pack2i(a0 + kMagicA, a1 + kMagicA), pack2(ca, ca));
    const f32x2 fb = add2(pack2i(b0 + kMagicB, b1 + kMagicB), pack2(cb, cb));
    return add2(fa, fb);
}
// |v| < 2^22 (the min sums: at most 8 * 63 * 4064).
__device__ __forceinline__ f32x2 small_to_float2(int v0, int v1) {
    return add2(pack2i(v0 + 0x4B400000, v1 + 0x4B400000), pack2(-12582912.0f, -12582912.0f));
}

// ---- weight blocks in registers and their unpacking ------------------------------------------------------------
// `wb` points at the half's weight operand: [K-step][chunk][128 rows: plane a of the half's 64 weight rows, then plane
// b][16 B]; `lr` is the row's index inside the half.
struct Q4Blk {
    uint4 hd, q[8];
};
__device__ __forceinline__ void load_blk(Q4Blk& b, const uint8_t* w, size_t /*nblk*/, size_t blk, int /*n*/) {
    const uint4* p = reinterpret_cast<const uint4*>(w + blk * kQ4KBlock);
    b.hd = __ldg(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) b.q[i] = __ldg(p + 1 + i);
}
// One row of one super-block: planes a = (sc >> 3) * q and b = (sc & 7) * q for the eight K-steps (sub-blocks); the mins
// as K bytes 0..7 (rows 0..63 of the min operand) and as K bytes 8..15 (rows 64..127); d and dmin into `dd`.
__device__ __forceinline__ void unpack_blk(const Q4Blk& b, uint8_t* wb, uint8_t* wm, float* dd, int lr, int /*n*/) {
    const unsigned sclo = b.hd.y & 0x3F3F3F3Fu, schi = (b.hd.w & 0x0F0F0F0Fu) | ((b.hd.y >> 2) & 0x30303030u);
    const unsigned mlo = b.hd.z & 0x3F3F3F3Fu, mhi = ((b.hd.w >> 4) & 0x0F0F0F0Fu) | ((b.hd.z >> 2) & 0x30303030u);
    uint8_t* pa = wb + lr * 16;
    uint8_t* pb = pa + HR * 16;
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
    *reinterpret_cast<uint4*>(wm + lr * 16) = make_uint4(mlo, mhi, 0u, 0u);
    *reinterpret_cast<uint4*>(wm + (HR + lr) * 16) = make_uint4(0u, 0u, mlo, mhi);
    // {d_r, d_r+1, dmin_r, dmin_r+1} per row pair: the epilogue reads a pair's scales as two packed operands
    dd[(lr >> 1) * 4 + (lr & 1)] = half_bits_to_float(b.hd.x & 0xFFFFu);
    dd[(lr >> 1) * 4 + 2 + (lr & 1)] = half_bits_to_float(b.hd.x >> 16);
}

struct Q6Blk {
    uint4 lq[4], hq[2];
    uint2 sc;
    unsigned d;
};
// Half n of a block (weights 128 n .. 128 n + 127) out of the device planes ql | qh | scales | d.
__device__ __forceinline__ void load_blk(Q6Blk& b, const uint8_t* w, size_t nblk, size_t blk, int n) {
#pragma unroll
    for (int i = 0; i < 4; ++i) b.lq[i] = __ldg(reinterpret_cast<const uint4*>(w + blk * 128 + 64 * n + 16 * i));
#pragma unroll
    for (int i = 0; i < 2; ++i) b.hq[i] = __ldg(reinterpret_cast<const uint4*>(w + nblk * 128 + blk * 64 + 32 * n + 16 * i));
    b.sc = __ldg(reinterpret_cast<const uint2*>(w + nblk * 192 + blk * 16 + 8 * n));
    b.d = __ldg(reinterpret_cast<const unsigned short*>(w + nblk * 208 + blk * 2));
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
__device__ __forceinline__ void unpack_blk(const Q6Blk& blk, uint8_t* wb, uint8_t* /*wm*/, float* dd, int lr, int n) {
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
            uint8_t* pa = wb + (2 * (4 * n + t) + c) * kChunk + lr * 16;
            *reinterpret_cast<uint4*>(pa) = make_uint4(a[0], a[1], a[2], a[3]);
            *reinterpret_cast<uint4*>(pa + HR * 16) = make_uint4(b[0], b[1], b[2], b[3]);
        }
    }
    if (n == 0) dd[lr] = half_bits_to_float(blk.d);
}

// ---- the kernel ------------------------------------------------------------------------------------------------
// Units: u -> (row tile, column tile, K slice); CTA b takes units b, b + gridDim.x, ...; a unit contracts super-blocks
// [z * per, min(nsb, (z + 1) * per)) and stores into y (one slice) or into slice z of `partial`.
template <bool kQ6>
__global__ void __launch_bounds__(Cfg<kQ6>::kThreads, 1)
    matmul_kq_q8k_pipe_kernel(const uint8_t* __restrict__ w, const int* __restrict__ xq, const __grid_constant__ CUtensorMap map_x,
                              const __grid_constant__ CUtensorMap map_s, float* __restrict__ y, int rows, int nsb, int ncols, int per, int n_rt,
                              int n_ct, int units, float* __restrict__ partial) {
    using C = Cfg<kQ6>;
    using Blk = typename std::conditional<kQ6, Q6Blk, Q4Blk>::type;
    extern __shared__ uint8_t sm_raw[];
    uint8_t* sm = sm_raw + ((1024u - (smem_u32(sm_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + C::kOffBar);
    uint64_t* full = bars;        // [2] operands of a stage written (producers + tensor copies)
    uint64_t* empty = bars + 2;   // [2] the MMAs reading a stage have completed
    uint64_t* tfull = bars + 4;   // [2] accumulators of a half complete
    uint64_t* tempty = bars + 6;  // [2] accumulators of a half read back
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* fail = reinterpret_cast<volatile int*>(bars + 9);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t nblk = static_cast<size_t>(rows) * nsb;
    const int slot_ints = nsb * 85;

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&full[s], C::kProdWarps + 1);  // one arrival per producer warp + the tensor copies' expect_tx
            mbar_init(&empty[s], 1);
            mbar_init(&tfull[s], 1);
            mbar_init(&tempty[s], kEpiWarps);
        }
        *fail = 0;
        mbar_init_fence();
    }
    if (!kQ6)  // zeros behind the min operands, written once
        for (int i = tid; i < kChunk / 16; i += C::kThreads) *reinterpret_cast<uint4*>(sm + C::kOffZero + i * 16) = make_uint4(0u, 0u, 0u, 0u);
    if (warp == C::kMmaWarp) {
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
        // ================= epilogue: activation column 32 * (warp & 3) + lane of the tile (its TMEM lane), weight rows
        // 32 * (warp >> 2) .. + 31 of each half
        // The CTA's registers are shared out at launch by thread count (128 / 96 per thread); the MMA warpgroup needs few
        // and releases the rest, which these two warpgroups pick up: their 64 accumulators plus the rows in flight need
        // the room to keep several rows' dependency chains interleaved.  The request waits until the release has happened.
        if (kQ6) asm volatile("setmaxnreg.inc.sync.aligned.u32 120;");
        else asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
        const int ecol = 32 * (warp & 3) + lane, rs = warp >> 2;
        const uint32_t tlane = tmem + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + 32 * rs;
        int it = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
            int rt, ct, sb0, sb1;
            unit_of(u, rt, ct, sb0, sb1);
            const int col = ct * TN + ecol;
            const bool warp_live = ct * TN + 32 * (warp & 3) < ncols;  // a ragged last column tile leaves whole warps idle
            const int* slot = xq + static_cast<size_t>(min(col, ncols - 1)) * slot_ints + nsb * 64;  // this column's scales
            float acc[2 * 32];
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
            float dx_next = __int_as_float(__ldg(slot + sb0));
            for (int sb = sb0; sb < sb1 && ok; ++sb, ++it) {
                const float dx = dx_next;
                if (sb + 1 < sb1) dx_next = __int_as_float(__ldg(slot + sb + 1));
                const f32x2 dx2 = pack2(dx, dx);
                const uint8_t* ddslot = sm + C::kOffDd + (it & (kRing - 1)) * C::kDdSlot;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    ok = wait_or_fail(&tfull[h], static_cast<uint32_t>(it) & 1u, fail);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (warp_live) {
                        const uint32_t t0 = tlane + h * C::kHalfCols;
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {  // eight weight rows at a time
                            const int lr0 = 32 * rs + 8 * ch;  // first of them inside the half
                            int va[8], vb[8], vh[8], vl[8];
                            tmem_ld8(t0 + 8 * ch, va);
                            tmem_ld8(t0 + HR + 8 * ch, vb);
                            if (!kQ6) {
                                tmem_ld8(t0 + 2 * HR + 8 * ch, vh);
                                tmem_ld8(t0 + 3 * HR + 8 * ch, vl);
                            }
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            after_tmem_wait(va), after_tmem_wait(vb);
                            if (!kQ6) after_tmem_wait(vh), after_tmem_wait(vl);
#pragma unroll
                            for (int pr = 0; pr < 4; ++pr) {
                                const int rp = (HR * h + lr0) / 2 + pr;  // row pair inside the tile
                                float* a0 = &acc[32 * h + 8 * ch + 2 * pr];
                                if (kQ6) {
                                    const f32x2 d2 = *reinterpret_cast<const f32x2*>(ddslot + rp * 8);
                                    const f32x2 is2 = planes_to_float2<6>(va[2 * pr], va[2 * pr + 1], vb[2 * pr], vb[2 * pr + 1]);
                                    float ta, tb;
                                    unpack2(mul2(mul2(d2, dx2), is2), ta, tb);
                                    a0[0] = __fadd_rn(a0[0], ta);
                                    a0[1] = __fadd_rn(a0[1], tb);
                                } else {
                                    const ulonglong2 dq = *reinterpret_cast<const ulonglong2*>(ddslot + rp * 16);  // {d, d'}, {dmin, dmin'}
                                    const f32x2 is2 = planes_to_float2<3>(va[2 * pr], va[2 * pr + 1], vb[2 * pr], vb[2 * pr + 1]);
                                    const f32x2 im2 = small_to_float2(64 * vh[2 * pr] + vl[2 * pr], 64 * vh[2 * pr + 1] + vl[2 * pr + 1]);
                                    float t1a, t1b, t2a, t2b;
                                    unpack2(mul2(mul2(dq.x, dx2), is2), t1a, t1b);
                                    unpack2(mul2(mul2(dq.y, dx2), im2), t2a, t2b);
                                    a0[0] = __fadd_rn(a0[0], __fsub_rn(t1a, t2a));
                                    a0[1] = __fadd_rn(a0[1], __fsub_rn(t1b, t2b));
                                }
                            }
                        }
                    }
                    // this warp's share of the half has been read: hand the accumulators back
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tempty[h]);
                }
            }
            if (ok && col < ncols) {  // 2 x 32 consecutive rows of column `col`
                float* out = (partial ? partial + static_cast<size_t>(sb0 / per) * ncols * rows : y) + static_cast<size_t>(col) * rows + rt * TM + 32 * rs;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<float4*>(out + HR * h + j) = make_float4(acc[32 * h + j], acc[32 * h + j + 1], acc[32 * h + j + 2], acc[32 * h + j + 3]);
            }
        }
    } else if (warp >= C::kMmaWarp) {
        // ================= MMA issue: one thread of this warpgroup (the other three warps only release registers)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == C::kMmaWarp && lane == 0) {
            int it = 0;
            bool ok = true;
            const uint32_t base = smem_u32(sm);
            const uint32_t zero = base + C::kOffZero;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
                int rt, ct, sb0, sb1;
                unit_of(u, rt, ct, sb0, sb1);
                for (int sb = sb0; sb < sb1 && ok; ++sb, ++it) {
                    const int s = it & 1;
                    ok = wait_or_fail(&full[s], static_cast<uint32_t>(it >> 1) & 1u, fail);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st = base + s * C::kStage;
                    for (int h = 0; h < 2 && ok; ++h) {
                        ok = wait_or_fail(&tempty[h], (static_cast<uint32_t>(it) & 1u) ^ 1u, fail);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t td = tmem + h * C::kHalfCols;
                        const uint32_t wb = st + C::kOffW + h * (16 * kChunk);
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks)  // M = 128 activation columns, N = plane a | plane b of 64 weight rows
                            mma_i8(td, desc_sw128(st + C::kOffX + (ks >> 2) * kAtom + (ks & 3) * 32), desc_nosw(wb + 2 * ks * kChunk, kChunk, 128), ks > 0);
                        if (!kQ6) {  // N = Dh | Dl: the sums chunk against the mins in K bytes 0..7 / 8..15
                            const uint32_t xs = st + C::kOffXs, wm = st + C::kOffWm + h * kChunk;
                            mma_i8(td + 2 * HR, desc_nosw(xs, zero - xs, 128), desc_nosw(wm, zero - wm, 128), 0);
                        }
                        mma_commit(&tfull[h]);
                    }
                    mma_commit(&empty[s]);
                }
            }
        }
    } else {
        // ================= producers: weight planes and row scales (all), tensor copies of the activations (thread 0)
        const int p = tid - 32 * kEpiWarps;
        const int row = p & (TM - 1), n = p >> 7, half = row >> 6, lr = row & (HR - 1);
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
                    tma_2d(st + C::kOffX, &map_x, sb * 256, c_tile, &full[s]);
                    tma_2d(st + C::kOffX + kAtom, &map_x, sb * 256 + 128, c_tile, &full[s]);
                    if (!kQ6) tma_2d(st + C::kOffXs, &map_s, nsb * 324 + sb * 16, c_tile, &full[s]);
                }
                // The scale ring slot of item `it` was last read by the epilogue of item it - 4, which finished before
                // the MMAs of item it - 2 could start (they waited for the accumulators of item it - 3 to be read back),
                // and this thread has just seen those MMAs complete.
                float* dd = reinterpret_cast<float*>(sm + C::kOffDd + (it & (kRing - 1)) * C::kDdSlot) + half * (C::kDdSlot / 8);
                unpack_blk(cur, st + C::kOffW + half * (16 * kChunk), st + C::kOffWm + half * kChunk, dd, lr, n);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core
                __syncwarp();  // every lane's stores and fence before the warp's one arrival
                if (lane == 0) mbar_arrive(&full[s]);
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
    if (warp == C::kMmaWarp) {
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
    kern<<<grid, C::kThreads, C::kSmem, s>>>(w, xq, map_x, map_s, y, rows, nsb, ncols, per, n_rt, n_ct, units, splits > 1 ? workspace : nullptr);
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
    if (misaligned(w, 16) || misaligned(xq, 16) || misaligned(y, 16) || misaligned(workspace, 16)) return KCB_INVALID_POINTER;  // y is stored four rows at a time
    return q6 ? launch_pipe<true>(static_cast<const uint8_t*>(w), xq, y, rows, k / 256, ncols, static_cast<float*>(workspace), workspace_bytes, s)
              : launch_pipe<false>(static_cast<const uint8_t*>(w), xq, y, rows, k / 256, ncols, static_cast<float*>(workspace), workspace_bytes, s);
}

}  // namespace kcb
