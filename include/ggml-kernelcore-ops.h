/*
 * ggml-kernelcore-ops.h -- the operator layer of the reference's llama.cpp backend on CUDA.
 *
 * The reference's ggml backend (integrations/llama.cpp/ggml/src/ggml-kernelcore/ggml-kernelcore.cpp) is two
 * things: glue to ggml's backend registry, buffers and graph walk (:706-1054; needs a llama.cpp source tree),
 * and, under it, one function per graph operator that reads ggml tensors and launches kernels (:471-697).
 * This header is the second part.  Each entry point replaces the reference function cited beside it, takes the
 * same tensors, and applies the same rules (which activations are quantized per 32 and which per 256 values,
 * which quantized inputs are shared between matmuls, how strides map to kernel arguments).
 *
 * Tensors are passed as kcb_tensor: the fields of ggml_tensor the operators read, with the same meaning
 * (type values are ggml's enum; ne = elements per dimension, nb = strides in bytes; data = device pointer;
 * op_params / src as in ggml).  A backend's graph_compute fills one from each ggml_tensor (or casts, if it
 * keeps the fields layout-compatible) and calls the operator.
 *
 * Weight tensors hold the device layout: Q4_K as GGUF blocks, Q6_K as four planes (kcb_q6k_to_planes), fp16
 * weights as llm::ref::repackF16 words; kcb_ggml_set_weight converts on upload (the reference repacks in its
 * set_tensor, ggml-kernelcore.cpp:180-200).
 */
#ifndef GGML_KERNELCORE_OPS_H
#define GGML_KERNELCORE_OPS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { KCB_TYPE_F32 = 0, KCB_TYPE_F16 = 1, KCB_TYPE_Q4_K = 12, KCB_TYPE_Q6_K = 14, KCB_TYPE_I32 = 26, KCB_TYPE_I64 = 27 };
enum { KCB_ROPE_TYPE_NEOX = 2 };

typedef struct kcb_tensor {
    int type;
    int64_t ne[4];
    size_t nb[4];
    void* data;
    int32_t op_params[16];
    const struct kcb_tensor* src[4];
} kcb_tensor;

/* One context per backend instance: the stream the operators launch on, the scratch that holds quantized
 * activations, and the list of inputs already quantized in the current graph (ggml-kernelcore.cpp:330-398). */
int kcb_ggml_ctx_create(void* stream, void** ctx);
/* Start of a graph: forget which inputs are quantized, reuse the scratch from its beginning.  Waits for the
 * stream first, since earlier launches may still read the scratch. */
int kcb_ggml_ctx_begin_graph(void* ctx);
/* Waits for everything launched through this context (a synchronous graph_compute ends with it). */
int kcb_ggml_ctx_sync(void* ctx);
int kcb_ggml_ctx_destroy(void* ctx);

/* Bytes a weight tensor of this type occupies on the device, and the upload + layout conversion. */
size_t kcb_ggml_weight_bytes(int type, int rows, int k);
int kcb_ggml_set_weight(void* ctx, void* dst_dev, const void* src_host, int type, int rows, int k);

/* All return 0 or a kc::Error code.  The reference function each one replaces: */
int kcb_ggml_mul_mat(void* ctx, const kcb_tensor* dst);                 /* mul_mat_impl   :562-603 */
int kcb_ggml_fused_norm(void* ctx, const kcb_tensor* add, const kcb_tensor* norm, const kcb_tensor* mul); /* :502-522 */
int kcb_ggml_rms_norm(void* ctx, const kcb_tensor* norm, const float* weight_dev, const kcb_tensor* out); /* :612-620 */
int kcb_ggml_mul(void* ctx, const kcb_tensor* dst);                     /* mul            :626-633 */
int kcb_ggml_add(void* ctx, const kcb_tensor* dst);                     /* add            :635-640 */
int kcb_ggml_rope(void* ctx, const kcb_tensor* dst);                    /* rope           :642-653 */
int kcb_ggml_swiglu(void* ctx, const kcb_tensor* dst);                  /* swiglu         :655-659 */
int kcb_ggml_fused_swiglu(void* ctx, const kcb_tensor* dst);            /* fused_swiglu   :525-534 */
int kcb_ggml_set_rows(void* ctx, const kcb_tensor* dst);                /* set_rows       :664-674 */
int kcb_ggml_flash_attn(void* ctx, const kcb_tensor* dst);              /* flash_attn     :677-711 */

#ifdef __cplusplus
}
#endif
#endif
