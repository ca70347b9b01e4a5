// Internal C++ launchers behind the C ABI.  Every function that takes a stream enqueues work on it and returns a
// status code (common.cuh) without synchronising or allocating; the first launch of a kernel that needs more than 48 KB
// of shared memory makes one cudaFuncSetAttribute call per device, and every launch of a tensor-core matmul
// encodes its two tensor maps on the host.  The few functions without a stream (the *_timeouts readers, the poll-limit
// and reset calls) are synchronous copies from or to a device variable.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace kcb {

// kquant_matvec.cu
int matvec_q4k_q8(const void* w, const int* xq, const float* xd, float* y, int rows, int k, cudaStream_t s);
int matvec_q6k_q8(const void* w, const int* xq, const float* xd, float* y, int rows, int k, cudaStream_t s);
// Both products in one launch (k <= 4096 and at most 6144 rows each, else KCB_UNSUPPORTED_OPERATION).
int matvec_q4k_q6k_pair_q8(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, const int* xq, const float* xd, int k,
                           cudaStream_t s);
int matvec_q4k_f32(const void* w, const float* x, float* y, int rows, int k, cudaStream_t s);
int matvec_q6k_f32(const void* w, const float* x, float* y, int rows, int k, cudaStream_t s);
int dequant_q4k(const void* w, float* out, int rows, int k, cudaStream_t s);
int dequant_q6k(const void* w, float* out, int rows, int k, cudaStream_t s);
unsigned tma_timeouts();
int matvec_q6k_f32x_sharded(const void* w, const float* x, float* y_local, float* const* y_peers, int npeers, unsigned* const* flags,
                            unsigned* epoch_counter, unsigned* done_counter, int rank, int world, int rows, int k, cudaStream_t s);
unsigned peer_timeouts();
int peer_set_poll_limit(unsigned polls);  // 0 = the default; synchronous
int peer_reset();                         // clears the expiry count and the "group broken" mark; synchronous
int peer_barrier(unsigned* const* flags, int rank, int world, unsigned epoch, unsigned* epoch_counter, cudaStream_t s);
int matvec_q6k_q8_gather(const void* w, const int* xq, const float* xd, float* y_local, float* const* y_peers, int npeers, int rows,
                         int k, cudaStream_t s);  // bounded mbarrier waits that expired since load (synchronous read)
int q6k_convert(const void* src, void* dst, int rows, int k, int to_planes, cudaStream_t s);

// quantize.cu
int quantize_q8x4(const float* x, int* xq, float* xd, int count, cudaStream_t s);
int quantize_cols(const float* x, int* q, int k, int ncols, cudaStream_t s);
int quantize_cols_k(const float* x, int* q, int k, int ncols, cudaStream_t s);


// matmul_kq.cu
int matmul_kq_q8(const void* w, const int* xq, float* y, int rows, int k, int ncols, int q6, int q8k, cudaStream_t s, void* workspace = nullptr,
                 size_t workspace_bytes = 0);

// matmul_tc_pipe.cu: the warp-specialised tensor-core kernels.  `workspace` (device, may be null) allows K slices.
int matmul_kq_q8k_tc_pipe(const void* w, const int* xq, float* y, int rows, int k, int ncols, int q6, void* workspace, size_t workspace_bytes,
                          cudaStream_t s);
int matmul_tc_pipe_k_slices(int rows, int k, int ncols);
size_t matmul_tc_workspace_bytes(int rows, int k, int ncols);
unsigned tc_pipe_timeouts();

// decode_matvec.cu: the decode step's matvecs with their producers as prologues (see the file header).
// trace != nullptr: the k / 4 int8 words the prologue produced are also written there (by one CTA; test instrumentation).
// Optional tail of decode_matvec_norm for a layer's q|k|v product (k <= 4096, adjacent-pair RoPE, no per-head norm): every
// finished tile rotates its q and k pairs at the device-side position (the arithmetic of rope_kv_f16_kernel), leaves q
// rotated in y and appends k and v as fp16 to the cache rows of that position, so the step needs no rotation launch.
// Output rows are taken in the order q heads | k heads | v heads (the Q4_K matrix first, then the Q6_K one).
struct DecodeRopeTail {
    const int* pos_p = nullptr;      // device-side position
    unsigned short* kc = nullptr;    // fp16 caches [max_ctx][kv_heads * hd]
    unsigned short* vc = nullptr;
    const float* ff = nullptr;       // optional frequency factors [hd / 2]
    int heads = 0, kv_heads = 0, hd = 0, max_ctx = 0;
    float log2_base = 0.0f;
};
// Optional tail of decode_matvec_norm for a gate|up product (one matrix of 2 * inter rows: gate rows, then up rows;
// k <= 4096, inter a multiple of 32): a CTA takes the 32-row tile of gate rows and the tile of the same up rows one after
// the other, and one warp turns the pair into 32 values of SwiGLU(gate) * up and their quantize_q8x4 block (the arithmetic
// of silu_mul_q8), written to xq / xd -- the down projection's input -- so that the step needs no SwiGLU launch.  The
// gate and up products themselves are not stored.
struct DecodeSwigluTail {
    int inter = 0;  // 0: none
    int* xq = nullptr;
    float* xd = nullptr;
};
bool decode_matvec_shape_ok(int rows4, int rows6, int k);
int decode_matvec_q8(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, int k, const int* xq, const float* xd, bool pdl,
                     cudaStream_t s);
int decode_matvec_norm(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, int k, const float* x_in, const float* t, float* x_out,
                       const float* wn, float eps, bool pdl, cudaStream_t s, int* trace = nullptr, const DecodeRopeTail* tail = nullptr,
                       const DecodeSwigluTail* swiglu = nullptr);
int decode_matvec_swiglu(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, int k, const float* g, const float* u, bool pdl,
                         cudaStream_t s, int* trace = nullptr);
int decode_matvec_combine(const void* w4, float* y4, int rows4, const void* w6, float* y6, int rows6, int k, const float* part, int heads, int hd,
                          int nsplit, bool pdl, cudaStream_t s);
unsigned decode_matvec_timeouts();

// glue.cu
int rms_norm(const float* x, const float* w, float* y, int n, int rows, float eps, cudaStream_t s);
int add_rms_norm(float* x, const float* t, const float* w, float* y, int n, float eps, cudaStream_t s);
int add_norm_q8(const float* a, const float* t, float* out, const float* w, float* y, int* q, int* sq, int n, int rows,
                float eps, int phases, int kq, cudaStream_t s);
int add_norm_q8_fast(float* x, const float* t, const float* w, int* xq, float* xd, int n, float eps, cudaStream_t s);
int argmax_partial(const float* logits, int vocab, float* cand_v, int* cand_i, int ncand, cudaStream_t s);
int silu_mul(const float* g, const float* u, float* out, size_t count, cudaStream_t s);
// (pdl: launch with a programmatic dependency on the kernel before it in the stream)
int silu_mul_q8(const float* g, const float* u, float* y, int* q, int* xq, float* xd, int n, int cols, cudaStream_t s, bool pdl = false);
int mul_rows(const float* x, const float* w, float* y, int n, size_t count, cudaStream_t s);
int vector_add(const float* a, const float* b, float* out, size_t count, cudaStream_t s);
int rope(float* x, const float* ff, int pairs, int pos, int count, float log2_base, cudaStream_t s);
int rope_ggml(const float* x, float* y, const int* pos, const float* ff, int head_dim, int n_head, int n_tokens,
              float log2_base, int neox, cudaStream_t s);
int kv_append(const float* k, const float* v, float* kt, float* vc, int n, int k_stride, int pos, cudaStream_t s);
int attn_scores(const float* q, const float* kt, float* scores, int n_heads, int ctx, int head_dim, int group,
                int ctx_pad, int k_stride, float scale, cudaStream_t s);
int softmax(float* x, int n, int stride, int rows, cudaStream_t s);
int attn_values(const float* p, const float* v, float* out, int n_heads, int ctx, int head_dim, int kv_stride, int group,
                int ctx_pad, cudaStream_t s);
int set_rows_f16(const float* src, const long long* idx, void* dst, int pairs, int rows, int src_row, int dst_row,
                 int dst_rows, cudaStream_t s);
int flash_attn_f16(const float* q, const void* k, const void* v, const void* mask, float* out, const int* dims15,
                   float scale, cudaStream_t s);

int fa_stage(int which, const float* q, const void* k, const void* v, const void* mask, float* s_buf, float* m_buf, float* out,
             const int* dims15, float scale, cudaStream_t s);

// synthetic_formats.cu
int matvec_q8w(const int8_t* q, const float* scales, const float* x, float* y, int rows, int k, cudaStream_t s);
int matvec_q4w(const uint8_t* qs, const float* scales, const float* x, float* y, int rows, int k, int interleaved, cudaStream_t s);
int matvec_q4x8_q8(const int* qw, const int* xq, const float* xd, float* y, int rows, int k, cudaStream_t s);
int matmul_f16(const int* qw, const float* x, float* y, int rows, int k, int ncols, cudaStream_t s);

}  // namespace kcb
