// K-quant matmul on CUDA cores, Y[c * rows + r] = sum_j W[r][j] X[c][j], for small column counts and as
// the exact-arithmetic companion of the tensor-core path.
//
// Replaces the reference's kernels/llm/matmul_q4k_q8x4.cu:40, matmul_q4k_q8x8.cu:40-228,
// matmul_q6k_q8x4/x8.cu:35 (activations quantized per 32) and matmul_q4k_q8kx4/x8.cu:41-239,
// matmul_q6k_q8kx4/x8.cu:41 (per 256).  One warp owns one weight row: each lane unpacks its 16 bytes
// of quants once per super-block step and reuses the unpacked words for every column of the CTA's
// column tile, whose activation slots sit in shared memory.  Integer dot products are exact; the fp32
// scale products are summed across lanes in tree order, so a column agrees with the reference's
// per-column mirror (llm/llm_reference.cpp:413-489, :529-596) to fp32 rounding.

#include "common.cuh"
#include "ops.h"

#include <cstdlib>

namespace kcb {
namespace {

constexpr unsigned kLo4 = 0x0F0F0F0Fu;
constexpr unsigned kHi2 = 0x30303030u;
constexpr int kThreads = 256, kWarps = 8, kMaxCols = 8;

// Shared layout per staged column: [nsb*64 words][nb float2 {d, d*sum} (per-32) | nsb floats d + nb ints B (per-256)]
// plus, for Q6_K, [2*nb ints: sums of 16].
template <bool kQ6, bool kQ8K>
__global__ void __launch_bounds__(kThreads) matmul_kq_kernel(const uint8_t* __restrict__ w, const int* __restrict__ xq,
                                                              float* __restrict__ y, int rows, int nsb, int ncols,
                                                              int slot_ints, int nc_tile) {
    extern __shared__ __align__(16) int sm[];
    const int nb = nsb * 8;
    const int col_ints = nsb * 64 + nb * 2 + (kQ6 ? nb * 2 : 0);
    const int c0 = blockIdx.y * nc_tile;
    const int nc = min(nc_tile, ncols - c0);
    for (int c = 0; c < nc; ++c) {
        const int* slot = xq + static_cast<size_t>(c0 + c) * slot_ints;
        int* dst = sm + c * col_ints;
        for (int i = threadIdx.x; i < nsb * 64; i += kThreads) dst[i] = slot[i];
        float2* dx = reinterpret_cast<float2*>(dst + nsb * 64);
        if (kQ8K) {
            const float* xd = reinterpret_cast<const float*>(slot + nsb * 64);
            const int* bs = slot + nsb * 65;
            for (int i = threadIdx.x; i < nb; i += kThreads)  // {d of the super-block, sum of the 32-block}
                dx[i] = make_float2(xd[i >> 3], __int_as_float(bs[2 * i] + bs[2 * i + 1]));
            if (kQ6) {
                int* s16 = dst + nsb * 64 + nb * 2;
                for (int i = threadIdx.x; i < nb * 2; i += kThreads) s16[i] = bs[i];
            }
        } else {
            const float* xd = reinterpret_cast<const float*>(slot + nb * 8);
            for (int i = threadIdx.x; i < nb; i += kThreads) dx[i] = make_float2(xd[2 * i], __fmul_rn(xd[2 * i], xd[2 * i + 1]));
            if (kQ6) {
                int* s16 = dst + nsb * 64 + nb * 2;
                for (int i = threadIdx.x; i < nb * 2; i += kThreads) {
                    int s = 0;
#pragma unroll
                    for (int q = 0; q < 4; ++q) s = __dp4a(0x01010101, slot[i * 4 + q], s);
                    s16[i] = s;
                }
            }
        }
    }
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * kWarps + warp;
    if (row >= rows) return;
    const int g = lane >> 3, c8 = lane & 7;
    float acc[kMaxCols];
#pragma unroll
    for (int c = 0; c < kMaxCols; ++c) acc[c] = 0.0f;

    if (!kQ6) {
        const int j = c8 >> 1, h = c8 & 1, sh = 16 * (j & 1);
        const uint8_t* rp = w + static_cast<size_t>(row) * nsb * kQ4KBlock;
        for (int sb = g; sb < nsb; sb += 4) {
            const uint4 hd = ldg_stream(rp + static_cast<size_t>(sb) * kQ4KBlock);
            const uint4 q = ldg_stream(rp + static_cast<size_t>(sb) * kQ4KBlock + 16 + 16 * c8);
            const unsigned lo[4] = {q.x & kLo4, q.y & kLo4, q.z & kLo4, q.w & kLo4};
            const unsigned hi[4] = {(q.x >> 4) & kLo4, (q.y >> 4) & kLo4, (q.z >> 4) & kLo4, (q.w >> 4) & kLo4};
            unsigned scw, mw;
            if (j < 2) {
                scw = hd.y & 0x3F3F3F3Fu;
                mw = hd.z & 0x3F3F3F3Fu;
            } else {
                scw = (hd.w & kLo4) | ((hd.y >> 2) & kHi2);
                mw = ((hd.w >> 4) & kLo4) | ((hd.z >> 2) & kHi2);
            }
            const int sca = (scw >> sh) & 255, scb = (scw >> (sh + 8)) & 255;
            const float fma_ = static_cast<float>((mw >> sh) & 255), fmb = static_cast<float>((mw >> (sh + 8)) & 255);
            const float d = half_bits_to_float(hd.x & 0xFFFFu), dmin = half_bits_to_float(hd.x >> 16);
            const int b = sb * 8 + 2 * j;
#pragma unroll
            for (int c = 0; c < kMaxCols; ++c) {
                if (c >= nc) break;
                const int* col = sm + c * col_ints;
                const uint4 xa = *reinterpret_cast<const uint4*>(col + b * 8 + 4 * h);
                const uint4 xb = *reinterpret_cast<const uint4*>(col + b * 8 + 8 + 4 * h);
                const float4 dd = *reinterpret_cast<const float4*>(col + nsb * 64 + 2 * b);
                int da = 0, db = 0;
                da = __dp4a(static_cast<int>(lo[0]), static_cast<int>(xa.x), da);
                da = __dp4a(static_cast<int>(lo[1]), static_cast<int>(xa.y), da);
                da = __dp4a(static_cast<int>(lo[2]), static_cast<int>(xa.z), da);
                da = __dp4a(static_cast<int>(lo[3]), static_cast<int>(xa.w), da);
                db = __dp4a(static_cast<int>(hi[0]), static_cast<int>(xb.x), db);
                db = __dp4a(static_cast<int>(hi[1]), static_cast<int>(xb.y), db);
                db = __dp4a(static_cast<int>(hi[2]), static_cast<int>(xb.z), db);
                db = __dp4a(static_cast<int>(hi[3]), static_cast<int>(xb.w), db);
                if (kQ8K) {  // dd = {d_s, B_2j (int bits), d_s, B_2j+1 (int bits)}
                    const int is = sca * da + scb * db;
                    float part = (d * dd.x) * static_cast<float>(is);
                    if (h == 0) part -= (dmin * dd.x) * (fma_ * static_cast<float>(__float_as_int(dd.y)) + fmb * static_cast<float>(__float_as_int(dd.w)));
                    acc[c] += part;
                } else {
                    float part = d * (static_cast<float>(sca * da) * dd.x + static_cast<float>(scb * db) * dd.z);
                    if (h == 0) part -= dmin * (fma_ * dd.y + fmb * dd.w);
                    acc[c] += part;
                }
            }
        }
    } else {
        const int n = c8 >> 2, a = (c8 >> 1) & 1, h = c8 & 1;
        const int shl = 4 - 2 * a, shr = 2 * a;
        const unsigned sel = static_cast<unsigned>(2 * a + h) * 0x1111u | 0x8880u;
        const size_t nblk = static_cast<size_t>(rows) * nsb;
        for (int sb = g; sb < nsb; sb += 4) {
            const size_t blk = static_cast<size_t>(row) * nsb + sb;
            const uint4 l = ldg_stream(w + blk * 128 + 16 * c8);
            const uint4 hq = ldg_stream(w + nblk * 128 + blk * 64 + 32 * n + 16 * h);
            const uint2 sc = __ldg(reinterpret_cast<const uint2*>(w + nblk * 192 + blk * 16 + 8 * n));
            const float d = half_bits_to_float(__ldg(reinterpret_cast<const unsigned short*>(w + nblk * 208 + blk * 2)));
            const unsigned lo[4] = {(l.x & kLo4) | ((hq.x << shl) & kHi2), (l.y & kLo4) | ((hq.y << shl) & kHi2),
                                    (l.z & kLo4) | ((hq.z << shl) & kHi2), (l.w & kLo4) | ((hq.w << shl) & kHi2)};
            const unsigned hi[4] = {((l.x >> 4) & kLo4) | ((hq.x >> shr) & kHi2), ((l.y >> 4) & kLo4) | ((hq.y >> shr) & kHi2),
                                    ((l.z >> 4) & kLo4) | ((hq.z >> shr) & kHi2), ((l.w >> 4) & kLo4) | ((hq.w >> shr) & kHi2)};
            const int scl = prmt_sbyte(sc.x, sel), sch = prmt_sbyte(sc.y, sel);
            const int b = sb * 8 + 4 * n + a;
#pragma unroll
            for (int c = 0; c < kMaxCols; ++c) {
                if (c >= nc) break;
                const int* col = sm + c * col_ints;
                const uint4 xa = *reinterpret_cast<const uint4*>(col + b * 8 + 4 * h);
                const uint4 xb = *reinterpret_cast<const uint4*>(col + (b + 2) * 8 + 4 * h);
                const float dxa = __int_as_float(col[nsb * 64 + 2 * b]), dxb = __int_as_float(col[nsb * 64 + 2 * (b + 2)]);
                const int* s16 = col + nsb * 64 + nb * 2;
                int dl = 0, dh = 0;
                dl = __dp4a(static_cast<int>(lo[0]), static_cast<int>(xa.x), dl);
                dl = __dp4a(static_cast<int>(lo[1]), static_cast<int>(xa.y), dl);
                dl = __dp4a(static_cast<int>(lo[2]), static_cast<int>(xa.z), dl);
                dl = __dp4a(static_cast<int>(lo[3]), static_cast<int>(xa.w), dl);
                dh = __dp4a(static_cast<int>(hi[0]), static_cast<int>(xb.x), dh);
                dh = __dp4a(static_cast<int>(hi[1]), static_cast<int>(xb.y), dh);
                dh = __dp4a(static_cast<int>(hi[2]), static_cast<int>(xb.z), dh);
                dh = __dp4a(static_cast<int>(hi[3]), static_cast<int>(xb.w), dh);
                const int tl = scl * (dl - 32 * s16[2 * b + h]);
                const int th = sch * (dh - 32 * s16[2 * (b + 2) + h]);
                if (kQ8K) acc[c] += (d * dxa) * static_cast<float>(tl + th);  // one activation scale per super-block
                else acc[c] += d * (static_cast<float>(tl) * dxa + static_cast<float>(th) * dxb);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < kMaxCols; ++c) {
        if (c >= nc) break;
        const float v = warp_sum(acc[c]);
        if (lane == 0) y[static_cast<size_t>(c0 + c) * rows + row] = v;
    }
}

}  // namespace

// q6: Q6_K planes, else Q4_K blocks.  q8k: slots of 85*k/256 ints (per-256 scales), else 11*k/32.
// workspace (device memory, may be null): room for the K slices of a tensor-core launch (matmul_tc_workspace_bytes);
// without it every launch is one pass.
int matmul_kq_q8(const void* w, const int* xq, float* y, int rows, int k, int ncols, int q6, int q8k, cudaStream_t s, void* workspace,
                 size_t workspace_bytes) {
    if (rows <= 0 || k <= 0 || k % 256 || k > 32768 || ncols <= 0 || !w || !xq || !y) return KCB_INVALID_VALUE;
    if (misaligned(w, 16) || misaligned(xq, 16) || misaligned(y, 4)) return KCB_INVALID_POINTER;
    // Per-256 activation slots and whole 128-row tiles go to the tensor cores (bit-identical results);
    // KCB_MATMUL_TC=0 keeps everything on the CUDA-core kernel below (comparison measurements).
    static const bool tc = [] {
        const char* e = getenv("KCB_MATMUL_TC");
        return !e || atoi(e) != 0;
    }();
    // (the activation slots of 85 * nsb ints are read in 16-byte pieces: nsb % 4 == 0)
    if (tc && q8k && rows % 128 == 0 && ncols >= 16 && (k / 256) % 4 == 0)
        return matmul_kq_q8k_tc_pipe(w, xq, y, rows, k, ncols, q6, workspace, workspace_bytes, s);
    const int nsb = k / 256, nb = nsb * 8;
    const int slot_ints = q8k ? nsb * 85 : nb * 11;
    const size_t col_bytes = static_cast<size_t>(nsb * 64 + nb * 2 + (q6 ? nb * 2 : 0)) * 4;
    int nc_tile = static_cast<int>((44 * 1024) / col_bytes);
    if (nc_tile > kMaxCols) nc_tile = kMaxCols;
    if (nc_tile < 1) return KCB_INVALID_VALUE;
    const dim3 grid((rows + kWarps - 1) / kWarps, (ncols + nc_tile - 1) / nc_tile);
    const size_t smem = col_bytes * nc_tile;
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    if (q6 && q8k) matmul_kq_kernel<true, true><<<grid, kThreads, smem, s>>>(wb, xq, y, rows, nsb, ncols, slot_ints, nc_tile);
    else if (q6) matmul_kq_kernel<true, false><<<grid, kThreads, smem, s>>>(wb, xq, y, rows, nsb, ncols, slot_ints, nc_tile);
    else if (q8k) matmul_kq_kernel<false, true><<<grid, kThreads, smem, s>>>(wb, xq, y, rows, nsb, ncols, slot_ints, nc_tile);
    else matmul_kq_kernel<false, false><<<grid, kThreads, smem, s>>>(wb, xq, y, rows, nsb, ncols, slot_ints, nc_tile);
    return launch_status();
}

}  // namespace kcb
