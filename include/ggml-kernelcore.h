/*
 * ggml-kernelcore.h -- the ggml backend's three exported entry points, as the reference declares them
 * (integrations/llama.cpp/ggml/include/ggml-kernelcore.h:16-18 of the reference project): llama.cpp's backend registry
 * calls ggml_backend_kernelcore_reg, its scheduler creates backends with ggml_backend_kernelcore_init.
 *
 * Here the backend runs the K-quant matrix products, RMSNorm, RoPE, SwiGLU, the fp16 KV-cache writes and attention as
 * CUDA kernels on a B200 (kernelcore_b200/csrc/ggml_backend.cpp over the operator layer in ggml-kernelcore-ops.h).
 * It compiles against llama.cpp's ggml headers; where no llama.cpp tree is present, include/stub/ggml holds a
 * stand-in with the members the backend touches.
 */
#pragma once

#include "ggml.h"
#include "ggml-backend.h"

#ifdef __cplusplus
extern "C" {
#endif

GGML_BACKEND_API ggml_backend_t ggml_backend_kernelcore_init(void);
GGML_BACKEND_API bool ggml_backend_is_kc(ggml_backend_t backend);
GGML_BACKEND_API ggml_backend_reg_t ggml_backend_kernelcore_reg(void);

#ifdef __cplusplus
}
#endif
