// The decoder model as the host sees it: its shape (Config), where its memory lives (Allocator), its weights and
// caches (Mat, Layer, Model), its activations (Acts), the operations a decode step is made of (Backend) and the
// step itself (decodeToken).
//
// Type, member and function names are those of the reference's llm/llm_model.hpp:23-209, so programs written
// against that header compile against this one.  What differs:
//   - Weights::Q4K / Q6K / Gguf matrices hold this build's device layouts (see llm_reference.hpp);
//   - makeKcBackend() gives a backend whose every operation is a CUDA kernel on the kc runtime's default stream;
//   - makeCppBackend() does not exist: nothing here computes on the CPU;
//   - Config::neox and Config::qk_norm, Layer::q_norm / k_norm and Backend::rmsNormRows() are additions for
//     Qwen3-style models (RoPE pairs half a head apart, RMSNorm of every q and k head before the rotation).
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "llm_kernels.hpp"

namespace llm {

// ---- weight formats -------------------------------------------------------------------------------------------
enum class Weights { Q8, Q4, Q4X8, Q4X8Q8, Q4K, Q6K, Gguf };

const char* weightsName(Weights w);

// Formats whose matvec consumes 8-bit activation blocks rather than floats.
inline bool quantizedActs(Weights w) {
    switch (w) {
    case Weights::Q4X8Q8:
    case Weights::Q4K:
    case Weights::Q6K:
    case Weights::Gguf: return true;
    default: return false;
    }
}

// ---- model shape ----------------------------------------------------------------------------------------------
struct Config {
    std::string name;
    int hidden = 0;
    int inter = 0;  // FFN width
    int layers = 0;
    int heads = 0;
    int kv_heads = 0;
    int head_dim = 0;
    int vocab = 0;
    int max_ctx = 0;  // positions the KV cache holds
    float eps = 1e-5f;
    float rope_base = 500000.0f;
    Weights weights = Weights::Q4;
    int64_t file_weight_bytes = 0;  // as stored in the model file, when loaded from one
    bool neox = false;              // RoPE rotates (i, i + head_dim / 2) instead of (2i, 2i + 1)
    bool qk_norm = false;           // RMSNorm over each q and k head before RoPE

    int group() const { return heads / kv_heads; }        // query heads per kv head
    int kvStride() const { return kv_heads * head_dim; }  // floats per cached position
    int kStride() const { return padTo8(max_ctx); }       // row length of the transposed K cache
    AttnDims attnDims(int ctx) const { return {heads, ctx, head_dim, kvStride(), group(), padTo8(ctx), kStride()}; }
    int64_t weightParams() const;
    int64_t weightBytes() const;
};

// Shapes of the models the benchmarks name, and a small one for tests.
Config tinyConfig(Weights w);
Config llama32_1b(int max_ctx, Weights w);
Config llama32_3b(int max_ctx, Weights w);
Config qwen3_8b(int max_ctx, Weights w);

// ---- memory placement -----------------------------------------------------------------------------------------
// Where a model's buffers live.  Blocks stay allocated until the allocator is destroyed.
class Allocator {
public:
    virtual ~Allocator() = default;
    virtual void* alloc(size_t bytes) = 0;
    virtual void upload(void* dst, const void* src, size_t bytes) = 0;    // host -> allocator's memory
    virtual void download(void* dst, const void* src, size_t bytes) = 0;  // and back
};

namespace detail {
// The blocks an allocator has handed out, each with the function that gives it back; released newest first.
class BlockLedger {
public:
    using Release = void (*)(void*);
    explicit BlockLedger(Release release) : release_(release) {}
    BlockLedger(const BlockLedger&) = delete;
    BlockLedger& operator=(const BlockLedger&) = delete;
    ~BlockLedger();
    void* keep(void* block);

private:
    Release release_;
    std::vector<void*> held_;
};
}  // namespace detail

// Ordinary host memory: staging buffers and tests.
class HostAllocator final : public Allocator {
public:
    HostAllocator();
    void* alloc(size_t bytes) override;
    void upload(void* dst, const void* src, size_t bytes) override;
    void download(void* dst, const void* src, size_t bytes) override;

private:
    detail::BlockLedger ledger_;
};

// Memory of the current GPU, through kcMalloc and kcMemcpy.
class KcAllocator final : public Allocator {
public:
    KcAllocator();
    void* alloc(size_t bytes) override;
    void upload(void* dst, const void* src, size_t bytes) override;
    void download(void* dst, const void* src, size_t bytes) override;

private:
    detail::BlockLedger ledger_;
};

// ---- weights, caches, activations -----------------------------------------------------------------------------
struct Mat {
    int rows = 0;
    int k = 0;
    Weights format = Weights::Q8;
    const void* q = nullptr;    // weight data on the device, laid out as `format` says
    const float* s = nullptr;   // scales, for the formats that keep them apart
    const int* dims = nullptr;  // {rows, k} as two ints on the device
};

struct Layer {
    Mat wqkv, wo, wgu, wd;
    const float* attn_norm = nullptr;
    const float* ffn_norm = nullptr;
    float* k_cache = nullptr;  // transposed: [kvStride()][kStride()]
    float* v_cache = nullptr;  // [max_ctx][kvStride()]
    // q, k, v and gate, up one by one, for files that mix formats inside a layer
    std::vector<Mat> qkv_parts, gu_parts;
    const float* q_norm = nullptr;  // head_dim weights each; only with Config::qk_norm
    const float* k_norm = nullptr;
};

struct Model {
    Config cfg;
    std::vector<Layer> layers;
    const float* out_norm = nullptr;
    Mat lm_head;
    int* attn_dims = nullptr;       // seven ints on the device, rewritten for every token
    const float* rope_ff = nullptr;  // optional RoPE frequency factors
    // writes the embedding row of `token` to `out` (host floats)
    std::function<void(int token, float* out)> embed;
};

struct Acts {
    float* x0 = nullptr;  // input embedding when decodeToken() is given no token
    float* x = nullptr;   // residual stream
    float* xn = nullptr;
    float* scores = nullptr;
    float* attn = nullptr;
    float* q = nullptr;
    float* k = nullptr;
    float* v = nullptr;
    float* t = nullptr;
    float* h = nullptr;
    float* logits = nullptr;
    float* g = nullptr;
    float* u = nullptr;
    int* xq = nullptr;  // quantized-activation scratch
};

Acts allocActs(const Config& cfg, Allocator& alloc, uint64_t seed);

// A model of random weights in one of the synthetic formats (Q8, Q4, Q4X8, Q4X8Q8), the same in every allocator of
// `allocs` and, for a given seed, the same values the reference's buildModels draws (llm/llm_model.cpp:217-254): fused
// q|k|v and gate|up matrices, norm weights near one, KV caches pre-filled with uniform values so that a step at any
// position attends over defined data.  One Model per allocator is appended to `out` (which is cleared first).
void buildModels(const Config& cfg, uint64_t seed, const std::vector<Allocator*>& allocs, std::vector<Model>& out);

// A K-quant model described by pointers to canonical GGUF block bytes on the host.  uploadModel() converts each
// matrix to its device layout and uploads it through `alloc`, allocates the KV caches and makes Model::embed look
// rows up in the (tied) output matrix.  The reference builds the same thing in llm/gguf_model.cpp:51-106.
struct HostMat {
    const uint8_t* blocks;
    int rows;
    int k;
    bool q6;
};
struct HostLayer {
    HostMat wq, wk, wv, wo, wg, wu, wd;
    const float* attn_norm;
    const float* ffn_norm;
    const float* q_norm;
    const float* k_norm;
};
struct HostModel {
    Config cfg;
    std::vector<HostLayer> layers;
    const float* out_norm;
    HostMat lm_head;
    const float* rope_ff;
};
Model uploadModel(const HostModel& host, Allocator& alloc);

// ---- profiling hooks ------------------------------------------------------------------------------------------
enum class Op : int { MatvecAttn, MatvecFfn, MatvecLmHead, RmsNorm, Rope, Attention, SiluMul, Add, Count };
constexpr int kOpCount = static_cast<int>(Op::Count);
const char* opName(Op op);

class Profiler {
public:
    virtual ~Profiler() = default;
    virtual void begin(Op op) = 0;
    virtual void end(Op op) = 0;
};

// ---- the operations of a decode step --------------------------------------------------------------------------
class Backend {
public:
    virtual ~Backend() = default;

    // per-token set-up
    virtual void setScratch(int* q) = 0;
    virtual void setContext(int ctx) = 0;
    virtual void beginToken(bool profiling) { (void)profiling; }
    virtual void endToken() {}
    virtual void finish() = 0;

    // matrix times vector, on floats or on the quantized scratch
    virtual void matvec(const Mat& w, const float* x, float* y) = 0;
    virtual void matvecQuantized(const Mat& w, float* y) = 0;

    // normalisation, residual, SwiGLU (the *Quant forms leave their result quantized in the scratch)
    virtual void rmsNorm(const float* x, const float* w, float* y) = 0;
    virtual void addRmsNorm(float* x, const float* t, const float* w, float* y) = 0;
    virtual void addRmsNormQuant(float* x, const float* t, const float* w) = 0;
    virtual void rmsNormRows(float* x, const float* w, int n, int rows);  // in place, one weight vector for all rows
    virtual void siluMul(const float* g, const float* u, float* out, int n) = 0;
    virtual void siluMulQuant(const float* g, const float* u, int n) = 0;
    virtual void add(float* x, const float* t, int n) = 0;

    // attention
    virtual void rope(float* x, int heads, int pos) = 0;
    virtual void appendKv(const float* k, const float* v, float* kt, float* vc, int pos) = 0;
    virtual void attnScores(const float* q, const float* k, float* scores) = 0;
    virtual void softmax(float* scores) = 0;
    virtual void attnValues(const float* p, const float* v, float* out) = 0;

    // data movement
    virtual void copy(float* dst, const float* src, int n) = 0;
    virtual void upload(float* dst, const float* host, int n) = 0;
};

// One decode step at position `pos`.  The input is the embedding of `token` (through Model::embed) or, for a negative
// token, whatever Acts::x0 holds.  Every layer appends its K/V at `pos` and attends over pos + 1 positions; the final
// norm and the LM head leave the logits in Acts::logits.
void decodeToken(Backend& b, const Model& m, const Acts& a, int pos, Profiler* prof = nullptr, int token = -1);

// The CUDA backend of the current device: every operation is enqueued on the kc runtime's default stream, the
// residual add, RMSNorm and quantization of addRmsNormQuant as one launch.  With `graphs` each token is recorded into
// one CUDA graph.  `workers` and `two_rows` schedule CPU threads in the reference and mean nothing here.
std::unique_ptr<Backend> makeKcBackend(const Model& m, unsigned workers, bool graphs = true, bool two_rows = false);

}  // namespace llm
