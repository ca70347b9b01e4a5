// Model shapes the benchmarks name, and the names of weight formats and profiler categories
// (interfaces: llm/llm_model.hpp:23-62 and :146-150 of the reference).
#include <llm_model.hpp>

#include <array>

namespace llm {

namespace {

struct Dims {
    const char* name;
    int hidden, inter, layers, heads, kv_heads, head_dim, vocab;
};

Config configOf(const Dims& d, int max_ctx, Weights w) {
    Config c;
    c.name = d.name;
    c.hidden = d.hidden;
    c.inter = d.inter;
    c.layers = d.layers;
    c.heads = d.heads;
    c.kv_heads = d.kv_heads;
    c.head_dim = d.head_dim;
    c.vocab = d.vocab;
    c.max_ctx = max_ctx;
    c.weights = w;
    return c;
}

constexpr Dims kTiny{"tiny", 256, 640, 2, 4, 2, 64, 1000};
constexpr Dims kLlama1B{"Llama 3.2 1B shapes", 2048, 8192, 16, 32, 8, 64, 128256};
constexpr Dims kLlama3B{"Llama 3.2 3B shapes", 3072, 8192, 28, 24, 8, 128, 128256};
constexpr Dims kQwen8B{"Qwen3 8B shapes", 4096, 12288, 36, 32, 8, 128, 151936};

}  // namespace

Config tinyConfig(Weights w) { return configOf(kTiny, 40, w); }
Config llama32_1b(int max_ctx, Weights w) { return configOf(kLlama1B, max_ctx, w); }
Config llama32_3b(int max_ctx, Weights w) { return configOf(kLlama3B, max_ctx, w); }
Config qwen3_8b(int max_ctx, Weights w) {
    Config c = configOf(kQwen8B, max_ctx, w);
    c.eps = 1e-6f;
    c.rope_base = 1e6f;
    c.neox = true;
    c.qk_norm = true;
    return c;
}

// Weights of the decoder stack and the output matrix; embeddings are tied to the latter.
int64_t Config::weightParams() const {
    const int64_t h = hidden, q = int64_t(heads) * head_dim, kv = kvStride(), f = inter;
    const int64_t attention = h * (q + 2 * kv) + q * h;
    const int64_t ffn = 3 * f * h;
    return layers * (attention + ffn) + int64_t(vocab) * h;
}

int64_t Config::weightBytes() const {
    const int64_t n = weightParams();
    switch (weights) {
    case Weights::Gguf: return file_weight_bytes;
    case Weights::Q4K: return n / 256 * 144;
    case Weights::Q6K: return n / 256 * 210;
    case Weights::Q8: return n + n / 32 * int64_t(sizeof(float));  // a byte per weight, a float scale per 32
    default: return n / 2 + n / 32 * int64_t(sizeof(float));        // a nibble per weight, a float scale per 32
    }
}

const char* weightsName(Weights w) {
    static constexpr std::array<const char*, 7> text = {"Q8",   "Q4",   "Q4 x8", "Q4 x8 with 8-bit activations",
                                                        "Q4_K", "Q6_K", "GGUF K-quants (Q4_K / Q6_K) with 8-bit activations"};
    const size_t i = static_cast<size_t>(w);
    return i < text.size() ? text[i] : "?";
}

const char* opName(Op op) {
    switch (op) {
    case Op::MatvecAttn: return "matvec attention (q,k,v,o)";
    case Op::MatvecFfn: return "matvec FFN (gate,up,down)";
    case Op::MatvecLmHead: return "matvec lm_head";
    case Op::RmsNorm: return "rms_norm (first layer)";
    case Op::Rope: return "rope + KV append";
    case Op::Attention: return "attention (scores,softmax,values)";
    case Op::SiluMul: return "silu_mul (+ quantize)";
    case Op::Add: return "residual add + rms_norm";
    case Op::Count: break;
    }
    return "?";
}

}  // namespace llm
