// llm_model.hpp -- the decoder model, its memory placement, the Backend interface and the decode step.
//
// Mirrors the reference's llm/llm_model.hpp:23-209 (Config, Allocator, Mat, Layer, Model, Acts,
// Profiler, Backend, decodeToken, makeKcBackend) so code written against it compiles here.  Differences:
//   * Weights::Q4K / Q6K / Gguf matrices hold this build's device layouts (llm_reference.hpp);
//   * makeKcBackend returns a backend whose launches are CUDA kernels (through kcLaunchKernel);
//   * there is no makeCppBackend: the product has no CPU execution path (the CPU oracle is test code);
//   * Config gains `neox` and `qk_norm` (Qwen3-style RoPE pairing and per-head q/k RMSNorm), Layer the
//     two per-head norm vectors, Backend a batched rmsNormRows with a default that throws.
#pragma once

#include "llm_kernels.hpp"

#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace llm {

enum class Weights { Q8, Q4, Q4X8, Q4X8Q8, Q4K, Q6K, Gguf };
inline bool quantizedActs(Weights w) { return w == Weights::Q4X8Q8 || w == Weights::Q4K || w == Weights::Q6K || w == Weights::Gguf; }

struct Config {
    std::string name;
    int     hidden = 0, inter = 0, layers = 0, heads = 0, kv_heads = 0, head_dim = 0, vocab = 0;
    int     max_ctx = 0;  // KV cache capacity
    float   eps = 1e-5f;
    float   rope_base = 500000.0f;
    Weights weights = Weights::Q4;
    int64_t file_weight_bytes = 0;
    bool    neox = false;     // RoPE pairs (i, i + head_dim / 2) instead of (2i, 2i + 1)
    bool    qk_norm = false;  // per-head RMSNorm of q and k before RoPE

    int      kvStride() const { return kv_heads * head_dim; }
    int      group() const { return heads / kv_heads; }
    int      kStride() const { return padTo8(max_ctx); }
    AttnDims attnDims(int ctx) const { return {heads, ctx, head_dim, kvStride(), group(), padTo8(ctx), kStride()}; }
    int64_t  weightParams() const;
    int64_t  weightBytes() const;
};

Config llama32_3b(int max_ctx, Weights w);
Config llama32_1b(int max_ctx, Weights w);
Config qwen3_8b(int max_ctx, Weights w);
Config tinyConfig(Weights w);
const char* weightsName(Weights w);

class Allocator {
public:
    virtual ~Allocator() = default;
    virtual void* alloc(size_t bytes) = 0;
    virtual void  upload(void* dst, const void* src, size_t bytes) = 0;
    virtual void  download(void* dst, const void* src, size_t bytes) = 0;
};

class HostAllocator final : public Allocator {  // plain host memory (staging, tests)
public:
    ~HostAllocator() override;
    void* alloc(size_t bytes) override;
    void  upload(void* dst, const void* src, size_t bytes) override;
    void  download(void* dst, const void* src, size_t bytes) override;

private:
    std::vector<void*> blocks_;
};

class KcAllocator final : public Allocator {  // kcMalloc / kcMemcpy: device memory of the current GPU
public:
    ~KcAllocator() override;
    void* alloc(size_t bytes) override;
    void  upload(void* dst, const void* src, size_t bytes) override;
    void  download(void* dst, const void* src, size_t bytes) override;

private:
    std::vector<void*> blocks_;
};

struct Mat {
    int          rows = 0, k = 0;
    Weights      format = Weights::Q8;
    const void*  q = nullptr;     // device weight data in the format's layout
    const float* s = nullptr;     // legacy formats: separate scales
    const int*   dims = nullptr;  // device int[2] {rows, k}
};

struct Layer {
    Mat          wqkv, wo, wgu, wd;
    const float* attn_norm = nullptr;
    const float* ffn_norm = nullptr;
    float*       k_cache = nullptr;  // transposed [kv_stride][kStride()]
    float*       v_cache = nullptr;  // [max_ctx][kv_stride]
    std::vector<Mat> qkv_parts, gu_parts;  // q, k, v and gate, up as separate matrices (mixed formats)
    const float* q_norm = nullptr;  // [head_dim], with Config::qk_norm
    const float* k_norm = nullptr;
};

struct Model {
    Config             cfg;
    std::vector<Layer> layers;
    const float*       out_norm = nullptr;
    Mat                lm_head;
    int*               attn_dims = nullptr;  // device int[7], rewritten per token
    const float*       rope_ff = nullptr;
    std::function<void(int token, float* out)> embed;  // host floats of one token's embedding
};

struct Acts {
    float *x0 = nullptr, *x = nullptr, *xn = nullptr, *scores = nullptr, *attn = nullptr;
    float *q = nullptr, *k = nullptr, *v = nullptr;
    float *t = nullptr, *h = nullptr, *logits = nullptr;
    float *g = nullptr, *u = nullptr;
    int*   xq = nullptr;
};

Acts allocActs(const Config& cfg, Allocator& alloc, uint64_t seed);

// A K-quant model from canonical GGUF block bytes on the host (what a GGUF file holds): packs and uploads
// every matrix through `alloc`, allocates the KV caches, and sets `embed` to the tied-embedding lookup
// (one row of the output matrix, dequantised).  The reference's loader is llm/gguf_model.cpp:51-106.
struct HostMat { const uint8_t* blocks; int rows; int k; bool q6; };
struct HostLayer { HostMat wq, wk, wv, wo, wg, wu, wd; const float* attn_norm; const float* ffn_norm; const float* q_norm; const float* k_norm; };
struct HostModel { Config cfg; std::vector<HostLayer> layers; const float* out_norm; HostMat lm_head; const float* rope_ff; };
Model uploadModel(const HostModel& host, Allocator& alloc);

enum class Op : int { MatvecAttn, MatvecFfn, MatvecLmHead, RmsNorm, Rope, Attention, SiluMul, Add, Count };
constexpr int kOpCount = static_cast<int>(Op::Count);
const char* opName(Op op);

class Profiler {
public:
    virtual ~Profiler() = default;
    virtual void begin(Op op) = 0;
    virtual void end(Op op) = 0;
};

class Backend {
public:
    virtual ~Backend() = default;
    virtual void setScratch(int* q) = 0;
    virtual void setContext(int ctx) = 0;
    virtual void matvec(const Mat& w, const float* x, float* y) = 0;
    virtual void rmsNorm(const float* x, const float* w, float* y) = 0;
    virtual void addRmsNorm(float* x, const float* t, const float* w, float* y) = 0;
    virtual void siluMulQuant(const float* g, const float* u, int n) = 0;
    virtual void matvecQuantized(const Mat& w, float* y) = 0;
    virtual void addRmsNormQuant(float* x, const float* t, const float* w) = 0;
    virtual void rope(float* x, int heads, int pos) = 0;
    virtual void appendKv(const float* k, const float* v, float* kt, float* vc, int pos) = 0;
    virtual void attnScores(const float* q, const float* k, float* scores) = 0;
    virtual void softmax(float* scores) = 0;
    virtual void attnValues(const float* p, const float* v, float* out) = 0;
    virtual void siluMul(const float* g, const float* u, float* out, int n) = 0;
    virtual void add(float* x, const float* t, int n) = 0;
    virtual void copy(float* dst, const float* src, int n) = 0;
    virtual void upload(float* dst, const float* host, int n) = 0;
    virtual void finish() = 0;
    virtual void beginToken(bool profiling) { (void)profiling; }
    virtual void endToken() {}
    // In-place RMSNorm of `rows` rows of n values with one weight vector (per-head q/k norm).
    virtual void rmsNormRows(float* x, const float* w, int n, int rows);
};

// One decode step at position `pos`: embedding (token >= 0 with Model::embed, else Acts::x0), every
// layer with K/V appended at pos and attention over pos + 1 positions, final norm, lm_head -> a.logits.
void decodeToken(Backend& b, const Model& m, const Acts& a, int pos, Profiler* prof = nullptr, int token = -1);

// Launches through kcLaunchKernel on the current device.  `workers` and `two_rows` are CPU scheduling
// knobs of the reference and are ignored; graphs: record each token into one CUDA graph.
std::unique_ptr<Backend> makeKcBackend(const Model& m, unsigned workers, bool graphs = true, bool two_rows = false);

}  // namespace llm
