// llm_kernels.hpp -- typed argument structs of the LLM kernels, launched by name through
// kcLaunchKernel(name, &args, stream).
//
// Field-for-field the structs of the reference's llm/llm_kernels.hpp:14-366 (callers build them
// positionally), with these differences in meaning on the GPU:
//   * every pointer is CUDA device memory from kcMalloc;
//   * the `dims` members (device int arrays the reference's CPU kernels read their sizes from) are
//     range-checked but never read: sizes travel by value in the struct;
//   * K-quant weight pointers (`qw`) hold the device layout written by llm::ref::repackQ4K / repackQ6K
//     of llm_reference.hpp in this tree: GGUF Q4_K blocks as they are, Q6_K split into planes.
#pragma once

#include <kernelcore/api.hpp>

#include <cstdint>

namespace llm {

inline int padTo8(int n) { return (n + 7) / 8 * 8; }

// Attention shape.  K cache transposed kt[kv_stride][k_stride]; V cache v[ctx][kv_stride]; scores
// p[n_heads][ctx_pad].  As device int[7] in this field order.
struct AttnDims {
    int n_heads = 0, ctx = 0, head_dim = 0, kv_stride = 0, group = 0, ctx_pad = 0, k_stride = 0;
};

// Legacy synthetic formats (kernels matvec_q8, matvec_q4, matvec_q4x8).
struct MatvecQ8Args { const int8_t* q; const float* scales; const float* x; float* y; const int* dims; int rows; int k; };
struct MatvecQ4Args { const uint8_t* qs; const float* scales; const float* x; float* y; const int* dims; int rows; int k; };

// quantize_q8x4: count blocks of 32 floats -> xq[count][8] words, xd[count][2] = {scale, sum of q}.
struct QuantizeArgs { const float* x; int* xq; float* xd; int count; };

// matvec_q4k_q8 / matvec_q6k_q8 (and the legacy matvec_q4x8_q8): y = W x on Q8 activations.
struct MatvecQ4Q8Args { const int* qw; const int* xq; const float* xd; float* y; const int* dims; int rows; int k; };

// add_rms_norm: x += t; y = norm(x) * w, one row.
struct AddRmsNormArgs { float* x; const float* t; const float* w; float* y; int n; float eps; };

// Q8 activation scratch for nb blocks of 32: [nb*8 words | nb*2 floats {scale, sum} | nb floats].
constexpr int scratchInts(int nb) { return nb * 11; }
inline float* scratchScales(int* q, int nb) { return reinterpret_cast<float*>(q + nb * 8); }
// Per-256 scratch, per column: [nsb*64 words | nsb scales | nsb*16 sums of 16 | nsb*4 words of sums of 32].
constexpr int scratchKInts(int nsb) { return nsb * 85; }

struct AddSumsqArgs { float* x; const float* t; int* q; int nb; };                       // add_sumsq
struct NormQ8Args { const float* x; const float* w; int* q; int nb; float eps; };        // norm_q8x4
struct SiluMulQ8Args { const float* g; const float* u; int* xq; float* xd; int count; };  // silu_mul_q8x4
struct RmsNormArgs { const float* x; const float* w; float* y; int n; int rows; float eps; };
struct RopeArgs { float* x; int pairs_per_head; int pos; int count; float log2_base; };
struct RopeFFArgs { float* x; const float* ff; int pairs_per_head; int pos; int count; float log2_base; };
struct MulRowsArgs { const float* x; const float* w; float* y; int n; int count; };
struct RopeGgmlArgs {
    const float* x; float* y; const int* pos; const float* ff; const int* dims;
    int head_dim; int n_head; int n_tokens; float log2_base; bool neox = false;
};
struct AddSumsqFArgs { const float* a; const float* b; float* out; int* q; const int* dims; int n; int rows; };
struct SumsqPartArgs { const float* x; int* q; const int* dims; int n; int rows; };
struct NormMulQ8Args { const float* x; const float* w; float* y; int* q; const int* dims; int n; int rows; float eps; };
struct SiluMulQ8FArgs { const float* g; const float* u; float* y; int* q; const int* dims; int n; int cols; };
struct AttnScoresArgs { const float* q; const float* k; float* scores; const int* dims; AttnDims d; float scale; };
struct SoftmaxArgs { float* x; int n; int stride; int rows; };
struct KvAppendArgs { const float* k; const float* v; float* kt; float* vc; const int* dims; AttnDims d; };
struct AttnValuesArgs { const float* p; const float* v; float* out; const int* dims; AttnDims d; };
struct SiluMulArgs { const float* g; const float* u; float* out; int count; };

// matmul_q4k_q8x4/x8, matmul_q6k_q8x4/x8 (per-32 slots) and matmul_*_q8kx4/x8 (per-256 slots):
// Y[c * rows + r] for ncols activation columns.  row_block is a CPU tiling hint and is ignored.
struct MatmulKQ8Args { const int* qw; const int* xq; float* y; const int* dims; int rows; int k; int ncols; int row_block = 8; };
// quantize_cols / quantize_cols_k: ncols columns of k floats into per-column slots.
struct QuantizeColsArgs { const float* x; int* q; const int* dims; int k; int ncols; };
struct MatmulF16Args { const int* qw; const float* x; float* y; const int* dims; int rows; int k; int ncols; };
struct SetRowsF16Args { const float* src; const int* idx; int* dst; const int* dims; int pairs; int rows; int src_row; int dst_row; int dst_rows; };

// FLASH_ATTN_EXT over an fp16 KV cache; strides of K, V and the mask in 32-bit words, of Q in floats.
struct FaDims {
    int H = 0, T = 0, D = 0, group = 0, tp = 0, k_row = 0, k_head = 0, v_row = 0, v_head = 0, N = 0, q_tok = 0, q_head = 0,
        m_row = 0, has_mask = 0, H_kv = 0;
};
constexpr int kFaDims = 15;
inline void faDimsInts(const FaDims& d, int* out) {
    const int v[kFaDims] = {d.H, d.T, d.D, d.group, d.tp, d.k_row, d.k_head, d.v_row, d.v_head, d.N, d.q_tok, d.q_head,
                            d.m_row, d.has_mask, d.H_kv};
    for (int i = 0; i < kFaDims; ++i) out[i] = v[i];
}
struct FaScoresArgs { const float* q; const int* k; const int* mask; float* s; const int* dims; FaDims d; float scale; };
struct FaMaxArgs { const float* s; float* m; const int* dims; FaDims d; };
struct FaExpArgs { float* s; const float* m; const int* dims; FaDims d; };
struct FaValuesArgs { const float* p; const int* v; float* out; const int* dims; FaDims d; };

// One-launch attention over the fp16 cache (kernel "flash_attn_f16"): what the four fa_* launches
// compute together.  Not in the reference's table; the ggml layer uses it.
struct FlashAttnF16Args { const float* q; const int* k; const int* v; const int* mask; float* out; FaDims d; float scale; };

// Makes the kernel names above launchable.  The built-in table needs no registration here, so this only
// checks that the runtime is initialised; kept because callers invoke it after kcInit.
kc::Error registerKernels() noexcept;

}  // namespace llm
