/*
 * kernelcore_b200.h -- C ABI of the B200 implementation of Kernelcore's quantized-LLM hot path.
 *
 * Plain pointers and sizes only.  Every pointer named "device" is CUDA device memory of the current
 * device; `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  Every
 * function returns an int status whose values are the reference's kc::Error codes
 * (include/kernelcore/error.hpp:8-25 of the reference): 0 = Success, 2 = InvalidValue,
 * 5 = InvalidPointer, 7 = UnsupportedOperation, 11 = LaunchFailure, ...  Op entry points only enqueue
 * work; they never synchronise and never allocate.
 *
 * Each declaration cites the reference interface it stands in for (path inside the reference project).
 */
#ifndef KERNELCORE_B200_H
#define KERNELCORE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- library ------------------------------------------------------------------------------- */
/* ABI revision and build arch string ("sm_100a"). */
int         kcb_abi_version(void);
const char* kcb_build_arch(void);
/* Text for a status code: kcGetErrorString, include/kernelcore/api.hpp:80. */
const char* kcb_error_string(int status);

/* Number of bounded device-side waits (mbarrier polls of the bulk-copy pipelines) that gave up since
 * the library was loaded; 0 in a healthy process.  Synchronous.  No counterpart in the reference: its
 * fault reporting is kcGetLastFault (include/kernelcore/api.hpp:79). */
unsigned kcb_tma_timeouts(void);

/* ---- weight layouts -------------------------------------------------------------------------
 * Q4_K matrices live on the device as canonical GGUF super-blocks, row-major: rows*(k/256) blocks
 * of 144 bytes.  Q6_K matrices live as four planes (ql | qh | scales | d) of the same total size,
 * rows*(k/256)*210 bytes; kcb_q6k_to_planes / kcb_q6k_from_planes convert from / to canonical GGUF
 * blocks on the device.  These replace the host-side 8-row interleaving of
 * llm::ref::repackQ4K / repackQ6K (llm/llm_reference.cpp:385-411) that the reference's loaders run
 * (llm/gguf_model.cpp:29-49, integrations/llama.cpp/.../ggml-kernelcore.cpp:175-190); the inverse
 * serves get_tensor (ggml-kernelcore.cpp:192-206). */
size_t kcb_kquant_bytes(int rows, int k, int q6);
int    kcb_q6k_to_planes(const void* gguf_blocks_dev, void* planes_dev, int rows, int k, void* stream);
int    kcb_q6k_from_planes(const void* planes_dev, void* gguf_blocks_dev, int rows, int k, void* stream);

/* Bit-exact dequantisation to fp32 [rows][k]: llm::ref::dequantRowQ4K / dequantRowQ6K
 * (llm/llm_reference.cpp:342-383), used for embedding rows (llm/gguf_model.cpp:96-104). */
int kcb_dequant_q4k(const void* w_dev, float* out_dev, int rows, int k, void* stream);
int kcb_dequant_q6k(const void* planes_dev, float* out_dev, int rows, int k, void* stream);

/* ---- activation quantizers ------------------------------------------------------------------- */
/* kernel "quantize_q8x4", llm::QuantizeArgs (llm/llm_kernels.hpp:51-57; kernels/llm/quantize_q8x4.cu:8-41):
 * count blocks of 32 floats -> xq[count*8] packed int8 words, xd[count*2] = {scale, sum of q}. */
int kcb_quantize_q8x4(const float* x_dev, int32_t* xq_dev, float* xd_dev, int count, void* stream);
/* kernels "quantize_cols" / "quantize_cols_k", llm::QuantizeColsArgs (llm/llm_kernels.hpp:273-283):
 * ncols columns of k floats -> slots of 11*k/32 ints (per-32 scales) or 85*k/256 ints (per-256). */
int kcb_quantize_cols(const float* x_dev, int32_t* q_dev, int k, int ncols, void* stream);
int kcb_quantize_cols_k(const float* x_dev, int32_t* q_dev, int k, int ncols, void* stream);

/* ---- decode matvec ---------------------------------------------------------------------------- */
/* kernels "matvec_q4k_q8" / "matvec_q6k_q8", llm::MatvecQ4Q8Args (llm/llm_kernels.hpp:59-70;
 * kernels/llm/matvec_q4k_q8.cu:33-88, matvec_q6k_q8.cu:33-105): y[rows] = W x with x given as the
 * Q8 blocks quantize_q8x4 wrote.  k % 256 == 0, k <= 32768. */
int kcb_matvec_q4k_q8(const void* w_dev, const int32_t* xq_dev, const float* xd_dev, float* y_dev, int rows, int k,
                      void* stream);
int kcb_matvec_q6k_q8(const void* planes_dev, const int32_t* xq_dev, const float* xd_dev, float* y_dev, int rows,
                      int k, void* stream);
/* The same product on fp32 activations: y = dequant(W) x with fp32 accumulation, the quantity the
 * reference's tests call "dequantized floats" (tests/test_llm_kernels.cpp:228-236).  k <= 12288. */
int kcb_matvec_q4k_f32(const void* w_dev, const float* x_dev, float* y_dev, int rows, int k, void* stream);
int kcb_matvec_q6k_f32(const void* planes_dev, const float* x_dev, float* y_dev, int rows, int k, void* stream);

#ifdef __cplusplus
}
#endif
#endif
