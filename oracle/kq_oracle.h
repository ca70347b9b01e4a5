/*
 * kq_oracle.h -- CPU restatement of Kernelcore's quantized-LLM arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker the GPU kernels are
 * compared against; nothing on the product path may link, import or call it.
 *
 * Every function restates one function of the reference's plain C++ mirror
 * (llm/llm_reference.cpp) in C, with the same loop order and the same
 * separately rounded fp32 operations (build with -ffp-contract=off).  One
 * deliberate difference: K-quant weights are read from canonical GGUF
 * super-blocks (144 B Q4_K, 210 B Q6_K, row-major) instead of the reference's
 * 8-row interleaved word stream (llm_reference.cpp:385-411).  The stream is a
 * pure byte shuffle of those blocks with fp16 d/dmin widened to fp32, so the
 * arithmetic on either layout is identical.
 *
 * Parity is pinned: tests compare every function here with the reference's
 * own llm::ref implementation (compiled from the reference sources into
 * oracle/_ref by oracle/Makefile) and with committed golden vectors that the
 * reference produced.
 */
#ifndef KQ_ORACLE_H
#define KQ_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Attention shape, field for field llm::AttnDims (llm/llm_kernels.hpp:14-23). */
typedef struct {
    int n_heads, ctx, head_dim, kv_stride, group, ctx_pad, k_stride;
} kqo_attn_dims;

/* Flash-attention shape, field for field llm::FaDims (llm/llm_kernels.hpp:316-332). */
typedef struct {
    int H, T, D, group, tp, k_row, k_head, v_row, v_head, N, q_tok, q_head, m_row, has_mask, H_kv;
} kqo_fa_dims;

/* fp16 <-> fp32 (llm_reference.cpp:284-309, :730-739). */
float    kqo_f16_to_f32(uint16_t h);
uint16_t kqo_f32_to_f16(float x);

/* GGUF K-quant rows -> fp32 (llm_reference.cpp:342-359, :361-383). */
void kqo_dequant_row_q4k(const uint8_t* src, int k, float* out);
void kqo_dequant_row_q6k(const uint8_t* src, int k, float* out);

/* Activation quantizers (llm_reference.cpp:79-104, :491-527). */
void kqo_quantize_q8x4(const float* x, int32_t* xq, float* xd, int count);
void kqo_quantize_q8k(const float* x, int32_t* q, int nsb);

/* y = W x on Q8 activations; w = rows * (k/256) GGUF blocks, row-major
 * (llm_reference.cpp:413-445, :447-489, :529-562, :564-596). */
void kqo_matvec_q4k_q8(const uint8_t* w, const int32_t* xq, const float* xd, float* y, int rows, int k);
void kqo_matvec_q6k_q8(const uint8_t* w, const int32_t* xq, const float* xd, float* y, int rows, int k);
void kqo_matvec_q4k_q8k(const uint8_t* w, const int32_t* xq, float* y, int rows, int k);
void kqo_matvec_q6k_q8k(const uint8_t* w, const int32_t* xq, float* y, int rows, int k);

/* y = W x with fp32 x: double-precision dot of the dequantised row, rounded to
 * fp32 once (tests/test_llm_kernels.cpp:228-236).  q6 != 0 selects Q6_K. */
void kqo_matvec_dequant_f64(const uint8_t* w, const float* x, float* y, int rows, int k, int q6);

/* Glue (llm_reference.cpp:153-280, :598-727). */
void kqo_rms_norm(const float* x, const float* w, float* y, int n, int rows, float eps);
void kqo_add(float* x, const float* t, int n);
void kqo_add_rms_norm(float* x, const float* t, const float* w, float* y, int n, float eps);
void kqo_add_sumsq(float* x, const float* t, int32_t* q, int nb);
void kqo_norm_q8x4(const float* x, const float* w, int32_t* q, int nb, float eps);
void kqo_rope(float* x, int pairs_per_head, int pos, int count, float log2_base);
void kqo_rope_ff(float* x, const float* ff, int pairs_per_head, int pos, int count, float log2_base);
void kqo_rope_ggml(const float* x, float* y, const int32_t* pos, const float* ff, int head_dim, int n_head,
                   int n_tokens, float log2_base, int neox);
void kqo_append_kv(const float* k, const float* v, float* kt, float* vc, int n, int k_stride, int pos);
void kqo_attn_scores(const float* q, const float* kt, float* scores, const kqo_attn_dims* d, float scale);
void kqo_softmax(float* x, int n, int stride, int rows);
void kqo_attn_values(const float* p, const float* v, float* out, const kqo_attn_dims* d);
void kqo_silu_mul(const float* g, const float* u, float* out, int count);
void kqo_silu_mul_q8x4(const float* g, const float* u, int32_t* xq, float* xd, int count);
void kqo_mul_rows(const float* x, const float* w, float* y, int n, int count);
void kqo_add_sumsq_f(const float* a, const float* b, float* out, int32_t* q, int n, int rows);
void kqo_sumsq_part(const float* x, int32_t* q, int n, int rows);
void kqo_norm_mul_q8(const float* x, const float* w, float* y, int32_t* q, int n, int rows, float eps);
void kqo_norm_mul_q8k(const float* x, const float* w, float* y, int32_t* q, const int32_t* sq, int n, int rows,
                      float eps);
void kqo_silu_mul_q8f(const float* g, const float* u, float* y, int32_t* q, int n, int cols);
void kqo_silu_mul_q8k(const float* g, const float* u, float* y, int32_t* q, int n, int cols);

/* fp16 KV-cache path (llm_reference.cpp:765-798). */
void kqo_set_rows_f16(const float* src, const int64_t* idx, uint16_t* dst, int pairs, int rows, int src_row,
                      int dst_row, int dst_rows);
void kqo_flash_attn_f16(const float* q, const uint16_t* k, const uint16_t* v, const uint16_t* mask, float* out,
                        const kqo_fa_dims* d, float scale);

/* The reference's synthetic 8-bit / 4-bit benchmark formats and fp16 weights (llm_reference.cpp:10-77, :114-152,
 * :740-764).  The *x8 layouts interleave 8 rows; kqo_repack_* build them from the row-major form. */
void kqo_matvec_q8w(const int8_t* q, const float* scales, const float* x, float* y, int rows, int k);
void kqo_matvec_q4w(const uint8_t* qs, const float* scales, const float* x, float* y, int rows, int k);
void kqo_repack_q4x8(const uint8_t* qs, const float* scales, uint8_t* qs8, float* scales8, int rows, int k);
void kqo_matvec_q4x8(const uint8_t* qs8, const float* scales8, const float* x, float* y, int rows, int k);
void kqo_repack_q4x8_q8(const uint8_t* qs, const float* scales, int32_t* qw, int rows, int k);
void kqo_matvec_q4x8_q8(const int32_t* qw, const int32_t* xq, const float* xd, float* y, int rows, int k);
void kqo_repack_f16(const uint16_t* w, int rows, int k, int32_t* out);
void kqo_matmul_f16(const uint16_t* w, const float* x, float* y, int rows, int k, int ncols);

/* One matrix of a decode model: GGUF blocks, row-major.  fmt: 4 = Q4_K, 6 = Q6_K. */
typedef struct {
    const uint8_t* blocks;
    int rows, k, fmt;
} kqo_mat;

/* One transformer layer in the reference's split form (llm/llm_model.hpp:100-113 with
 * qkv_parts / gu_parts as llm/gguf_model.cpp:72-91 fills them). */
typedef struct {
    kqo_mat wq, wk, wv, wo, wg, wu, wd;
    const float* attn_norm;
    const float* ffn_norm;
    float* k_cache; /* transposed fp32 [kv_stride][k_stride] */
    float* v_cache; /* fp32 [max_ctx][kv_stride] */
    const float* q_norm; /* [head_dim], only read with flag 4 of kqo_decode_token_ex */
    const float* k_norm;
} kqo_layer;

typedef struct {
    int hidden, inter, n_layers, heads, kv_heads, head_dim, vocab, max_ctx;
    float eps, rope_base;
    const kqo_layer* layers;
    const float* out_norm;
    kqo_mat lm_head;
    const float* rope_ff; /* may be NULL */
} kqo_model;

/* One decode step (llm/llm_model.cpp:287-360 on the single-thread C++ backend
 * :505-564): x_in = embedding row (hidden floats); writes vocab logits.
 * scratch_f: at least hidden*3 + (heads*head_dim + 2*kv) + heads*ctx_pad(max_ctx)
 *            + heads*head_dim + 3*inter floats; scratch_q: 11*max(hidden,inter,heads*head_dim)/32 ints. */
void kqo_decode_token(const kqo_model* m, const float* x_in, int pos, float* logits, float* scratch_f,
                      int32_t* scratch_q);
/* flags: 1 = fp16-rounded KV cache, 2 = NEOX RoPE, 4 = per-head q/k RMSNorm; 0 = kqo_decode_token. */
void kqo_decode_token_ex(const kqo_model* m, const float* x_in, int pos, float* logits, float* scratch_f,
                         int32_t* scratch_q, int flags);
/* Test instrumentation: from now on every decode step writes to buf the int8 words of each activation vector it
 * quantizes and the residual stream (hidden floats, as bit patterns) after each of a layer's two additions, in the order
 * the step runs: layer 0's q|k|v words, then per layer wo words, residual, gate|up words, down words, residual, the next
 * q|k|v words (after the last layer: the lm_head's).  NULL switches it off.
 * kqo_decode_trace_words() = words the last step produced (more than cap_words: the tail was dropped). */
void kqo_decode_set_trace(int32_t* buf, long cap_words);
long kqo_decode_trace_words(void);
/* Test instrumentation: the trace another implementation made of the same step.  Each vector the loop quantizes, and
 * the residual stream after each addition, is compared with it (kqo_decode_forced_stats: differing int8 values, vectors
 * holding one, largest int8 step, largest residual difference relative to the residual's largest magnitude; reset by
 * every step) and then replaced by it, so each stage is checked on the inputs the other implementation had. */
void kqo_decode_set_forced(const int32_t* words, long n_words);
void kqo_decode_forced_stats(long* values, long* vectors, int* max_step, float* residual_rel);
long kqo_decode_scratch_floats(const kqo_model* m);
long kqo_decode_scratch_ints(const kqo_model* m);

#ifdef __cplusplus
}
#endif
#endif
