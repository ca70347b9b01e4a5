// Internal C++ launchers behind the C ABI.  Every function enqueues work on `s` and returns a
// status code (common.cuh); none synchronises or allocates.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace kcb {

// kquant_matvec.cu
int matvec_q4k_q8(const void* w, const int* xq, const float* xd, float* y, int rows, int k, cudaStream_t s);
int matvec_q6k_q8(const void* w, const int* xq, const float* xd, float* y, int rows, int k, cudaStream_t s);
int matvec_q4k_f32(const void* w, const float* x, float* y, int rows, int k, cudaStream_t s);
int matvec_q6k_f32(const void* w, const float* x, float* y, int rows, int k, cudaStream_t s);
int dequant_q4k(const void* w, float* out, int rows, int k, cudaStream_t s);
int dequant_q6k(const void* w, float* out, int rows, int k, cudaStream_t s);
unsigned tma_timeouts();  // bounded mbarrier waits that expired since load (synchronous read)
int q6k_convert(const void* src, void* dst, int rows, int k, int to_planes, cudaStream_t s);

// quantize.cu
int quantize_q8x4(const float* x, int* xq, float* xd, int count, cudaStream_t s);
int quantize_cols(const float* x, int* q, int k, int ncols, cudaStream_t s);
int quantize_cols_k(const float* x, int* q, int k, int ncols, cudaStream_t s);

}  // namespace kcb
