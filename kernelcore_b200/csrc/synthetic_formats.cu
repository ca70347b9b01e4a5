// The reference's synthetic weight formats and its fp16 matmul, sm_100a.
//
// matvec_q8 / matvec_q4 / matvec_q4x8 / matvec_q4x8_q8 (kernels/llm/matvec_q8.cu, matvec_q4.cu, matvec_q4x8.cu,
// matvec_q4x8_q8.cu, matvec_q4x8_q8x2.cu) carry the random-weight models of the reference's own benchmark and
// tiny-model test (llm/llm_model.cpp:175-254); matmul_f16 (kernels/llm/matmul_f16.cu:40-80) serves fp16 weight
// tensors.  None of them is on the GGUF decode path, so they are written for parity, not bandwidth: one thread
// per output, the reference's order of separately rounded fp32 operations, results bit-identical to
// llm::ref::matvecQ8 / matvecQ4 / matvecQ4x8 / matvecQ4x8Q8 / matmulF16 (llm/llm_reference.cpp:10-77, :114-135,
// :756-764).  The 8-row interleaved layouts make neighbouring threads read neighbouring bytes or words.

#include "common.cuh"
#include "ops.h"

namespace kcb {
namespace {

__global__ void matvec_q8w_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales, const float* __restrict__ x,
                                  float* __restrict__ y, int rows, int k) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const int nb = k / 32;
    float acc = 0.0f;
    for (int b = 0; b < nb; ++b) {
        float s = 0.0f;
        const int8_t* qb = q + static_cast<size_t>(row) * k + static_cast<size_t>(b) * 32;
        for (int j = 0; j < 32; ++j) s = __fadd_rn(s, __fmul_rn(static_cast<float>(qb[j]), x[b * 32 + j]));
        acc = __fadd_rn(acc, __fmul_rn(s, scales[static_cast<size_t>(row) * nb + b]));
    }
    y[row] = acc;
}

__global__ void matvec_q4w_kernel(const uint8_t* __restrict__ qs, const float* __restrict__ scales, const float* __restrict__ x,
                                  float* __restrict__ y, int rows, int k) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const int nb = k / 32;
    float acc = 0.0f;
    for (int b = 0; b < nb; ++b) {
        float s = 0.0f;
        const uint8_t* qb = qs + static_cast<size_t>(row) * (k / 2) + static_cast<size_t>(b) * 16;
        for (int j = 0; j < 16; ++j) {
            const int v = qb[j];
            s = __fadd_rn(s, __fmul_rn(static_cast<float>((v & 15) - 8), x[b * 32 + j]));
            s = __fadd_rn(s, __fmul_rn(static_cast<float>((v >> 4) - 8), x[b * 32 + j + 16]));
        }
        acc = __fadd_rn(acc, __fmul_rn(s, scales[static_cast<size_t>(row) * nb + b]));
    }
    y[row] = acc;
}

__global__ void matvec_q4x8_kernel(const uint8_t* __restrict__ qs8, const float* __restrict__ scales8, const float* __restrict__ x,
                                   float* __restrict__ y, int rows, int k) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const int nb = k / 32, g = row / 8, l = row % 8;
    float acc = 0.0f;
    for (int b = 0; b < nb; ++b) {
        const size_t blk = static_cast<size_t>(g) * nb + b;
        const uint8_t* qb = qs8 + blk * 128 + l;
        const float* xb = x + b * 32;
        float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
        for (int j = 0; j < 16; j += 2) {
            const int v0 = qb[j * 8], v1 = qb[j * 8 + 8];
            s0 = __fadd_rn(s0, __fmul_rn(static_cast<float>((v0 & 15) - 8), xb[j]));
            s1 = __fadd_rn(s1, __fmul_rn(static_cast<float>((v0 >> 4) - 8), xb[j + 16]));
            s2 = __fadd_rn(s2, __fmul_rn(static_cast<float>((v1 & 15) - 8), xb[j + 1]));
            s3 = __fadd_rn(s3, __fmul_rn(static_cast<float>((v1 >> 4) - 8), xb[j + 17]));
        }
        acc = __fadd_rn(acc, __fmul_rn(__fadd_rn(__fadd_rn(s0, s2), __fadd_rn(s1, s3)), scales8[blk * 8 + l]));
    }
    y[row] = acc;
}

__global__ void matvec_q4x8_q8_kernel(const int* __restrict__ qw, const int* __restrict__ xq, const float* __restrict__ xd,
                                      float* __restrict__ y, int rows, int k) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const int nb = k / 32, g = row / 8, l = row % 8;
    float acc = 0.0f;
    for (int b = 0; b < nb; ++b) {
        const int* blk = qw + (static_cast<size_t>(g) * nb + b) * 40;
        int lo = 0, hi = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int q = blk[w * 8 + l];
            lo = __dp4a(q & 0x0F0F0F0F, xq[b * 8 + w], lo);
            hi = __dp4a((q >> 4) & 0x0F0F0F0F, xq[b * 8 + 4 + w], hi);
        }
        const float sc = __int_as_float(blk[32 + l]);
        const int dot = lo + hi - 8 * static_cast<int>(xd[b * 2 + 1]);
        acc = __fadd_rn(acc, __fmul_rn(static_cast<float>(dot), __fmul_rn(sc, xd[b * 2])));
    }
    y[row] = acc;
}

// qw: fp16 pairs as 32-bit words, 8 rows interleaved (llm::ref::repackF16); one thread per (row, column).
__global__ void matmul_f16_kernel(const int* __restrict__ qw, const float* __restrict__ x, float* __restrict__ y, int rows, int k,
                                  int ncols) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(rows) * ncols) return;
    const int c = static_cast<int>(idx / rows), row = static_cast<int>(idx % rows);
    const int kw = k / 2;
    const int* wp = qw + static_cast<size_t>(row / 8) * kw * 8 + row % 8;
    const float* xc = x + static_cast<size_t>(c) * k;
    float a = 0.0f;
    for (int w = 0; w < kw; ++w) {
        const unsigned q = static_cast<unsigned>(wp[static_cast<size_t>(w) * 8]);
        a = __fadd_rn(a, __fadd_rn(__fmul_rn(half_bits_to_float(q & 0xFFFFu), xc[2 * w]), __fmul_rn(half_bits_to_float(q >> 16), xc[2 * w + 1])));
    }
    y[static_cast<size_t>(c) * rows + row] = a;
}

inline unsigned grid_for(long long n, int per) { return static_cast<unsigned>((n + per - 1) / per); }
bool shape_ok(int rows, int k, int row_mult) { return rows >= 0 && rows % row_mult == 0 && k > 0 && k % 32 == 0; }

}  // namespace

int matvec_q8w(const int8_t* q, const float* scales, const float* x, float* y, int rows, int k, cudaStream_t s) {
    if (!shape_ok(rows, k, 1) || !q || !scales || !x || !y) return KCB_INVALID_VALUE;
    if (rows == 0) return KCB_SUCCESS;
    matvec_q8w_kernel<<<grid_for(rows, 64), 64, 0, s>>>(q, scales, x, y, rows, k);
    return launch_status();
}
int matvec_q4w(const uint8_t* qs, const float* scales, const float* x, float* y, int rows, int k, int interleaved, cudaStream_t s) {
    if (!shape_ok(rows, k, interleaved ? 8 : 1) || !qs || !scales || !x || !y) return KCB_INVALID_VALUE;
    if (rows == 0) return KCB_SUCCESS;
    if (interleaved) matvec_q4x8_kernel<<<grid_for(rows, 64), 64, 0, s>>>(qs, scales, x, y, rows, k);
    else matvec_q4w_kernel<<<grid_for(rows, 64), 64, 0, s>>>(qs, scales, x, y, rows, k);
    return launch_status();
}
int matvec_q4x8_q8(const int* qw, const int* xq, const float* xd, float* y, int rows, int k, cudaStream_t s) {
    if (!shape_ok(rows, k, 8) || !qw || !xq || !xd || !y) return KCB_INVALID_VALUE;
    if (rows == 0) return KCB_SUCCESS;
    matvec_q4x8_q8_kernel<<<grid_for(rows, 64), 64, 0, s>>>(qw, xq, xd, y, rows, k);
    return launch_status();
}
int matmul_f16(const int* qw, const float* x, float* y, int rows, int k, int ncols, cudaStream_t s) {
    if (rows <= 0 || rows % 8 || k <= 0 || k % 2 || ncols <= 0 || !qw || !x || !y) return KCB_INVALID_VALUE;
    matmul_f16_kernel<<<grid_for(static_cast<long long>(rows) * ncols, 128), 128, 0, s>>>(qw, x, y, rows, k, ncols);
    return launch_status();
}

}  // namespace kcb
