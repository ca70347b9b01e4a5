// Decoder model plumbing on the host: configurations, allocators, weight packing and upload, the
// per-token decode step and the Backend that turns each step into named kernel launches.
//
// Follows the interfaces of the reference's llm/llm_model.cpp (decodeToken :287-360, KcBackend :366-503,
// allocators :99-131, allocActs :257-283) and llm/gguf_model.cpp:29-106 (model assembly with separate
// q/k/v and gate/up matrices and tied embeddings).  Everything a Backend method launches is a CUDA
// kernel; failures surface as std::runtime_error carrying the kc error text, as in the reference.

#include <llm_model.hpp>
#include <llm_reference.hpp>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

namespace llm {

// ---- weight packing ---------------------------------------------------------------------------------
namespace ref {

void repackQ4K(const uint8_t* src, int rows, int k, int* qw) { std::memcpy(qw, src, packedBytes(rows, k, false)); }

void repackQ6K(const uint8_t* src, int rows, int k, int* qw) {
    const size_t nblk = size_t(rows) * size_t(k / 256);
    uint8_t* out = reinterpret_cast<uint8_t*>(qw);
    uint8_t *ql = out, *qh = out + nblk * 128, *sc = out + nblk * 192, *d = out + nblk * 208;
    for (size_t b = 0; b < nblk; ++b) {
        const uint8_t* blk = src + b * 210;
        std::memcpy(ql + b * 128, blk, 128);
        std::memcpy(qh + b * 64, blk + 128, 64);
        std::memcpy(sc + b * 16, blk + 192, 16);
        std::memcpy(d + b * 2, blk + 208, 2);
    }
}

void unpackQ6K(const int* qw, int rows, int k, uint8_t* dst) {
    const size_t nblk = size_t(rows) * size_t(k / 256);
    const uint8_t* in = reinterpret_cast<const uint8_t*>(qw);
    const uint8_t *ql = in, *qh = in + nblk * 128, *sc = in + nblk * 192, *d = in + nblk * 208;
    for (size_t b = 0; b < nblk; ++b) {
        uint8_t* blk = dst + b * 210;
        std::memcpy(blk, ql + b * 128, 128);
        std::memcpy(blk + 128, qh + b * 64, 64);
        std::memcpy(blk + 192, sc + b * 16, 16);
        std::memcpy(blk + 208, d + b * 2, 2);
    }
}

}  // namespace ref

// ---- configurations ---------------------------------------------------------------------------------
int64_t Config::weightParams() const {
    const int64_t qd = int64_t(heads) * head_dim, kv = kvStride();
    return (qd * hidden + 2 * kv * hidden + int64_t(hidden) * qd + 3 * int64_t(inter) * hidden) * layers + int64_t(vocab) * hidden;
}

int64_t Config::weightBytes() const {
    if (weights == Weights::Gguf) return file_weight_bytes;
    const int64_t p = weightParams();
    if (weights == Weights::Q4K) return p / 256 * 144;
    if (weights == Weights::Q6K) return p / 256 * 210;
    return (weights == Weights::Q8 ? p : p / 2) + p / 32 * int64_t(sizeof(float));
}

namespace {
Config shape(const char* name, int hidden, int inter, int layers, int heads, int kv_heads, int head_dim, int vocab, int max_ctx,
             Weights w) {
    Config c;
    c.name = name;
    c.hidden = hidden, c.inter = inter, c.layers = layers, c.heads = heads, c.kv_heads = kv_heads, c.head_dim = head_dim;
    c.vocab = vocab, c.max_ctx = max_ctx, c.weights = w;
    return c;
}
}  // namespace

Config llama32_3b(int max_ctx, Weights w) { return shape("Llama 3.2 3B shapes", 3072, 8192, 28, 24, 8, 128, 128256, max_ctx, w); }
Config llama32_1b(int max_ctx, Weights w) { return shape("Llama 3.2 1B shapes", 2048, 8192, 16, 32, 8, 64, 128256, max_ctx, w); }
Config qwen3_8b(int max_ctx, Weights w) {
    Config c = shape("Qwen3 8B shapes", 4096, 12288, 36, 32, 8, 128, 151936, max_ctx, w);
    c.eps = 1e-6f, c.rope_base = 1e6f, c.neox = true, c.qk_norm = true;
    return c;
}
Config tinyConfig(Weights w) { return shape("tiny", 256, 640, 2, 4, 2, 64, 1000, 40, w); }

const char* weightsName(Weights w) {
    switch (w) {
    case Weights::Q8: return "Q8";
    case Weights::Q4: return "Q4";
    case Weights::Q4X8: return "Q4 x8";
    case Weights::Q4X8Q8: return "Q4 x8 with 8-bit activations";
    case Weights::Q4K: return "Q4_K";
    case Weights::Q6K: return "Q6_K";
    case Weights::Gguf: return "GGUF K-quants (Q4_K / Q6_K) with 8-bit activations";
    }
    return "?";
}

const char* opName(Op op) {
    static const char* names[kOpCount] = {"matvec attention (q,k,v,o)", "matvec FFN (gate,up,down)", "matvec lm_head",
                                          "rms_norm (first layer)",     "rope + KV append",          "attention (scores,softmax,values)",
                                          "silu_mul (+ quantize)",      "residual add + rms_norm"};
    const int i = static_cast<int>(op);
    return i >= 0 && i < kOpCount ? names[i] : "?";
}

// ---- allocators -------------------------------------------------------------------------------------
namespace {
[[noreturn]] void kcFail(const char* what, kc::Error e) {
    throw std::runtime_error(std::string(what) + ": " + kcGetErrorString(e) + " (" + kcGetLastErrorDetail() + ")");
}
void kcCheck(kc::Error e, const char* what) {
    if (e != kc::Error::Success) kcFail(what, e);
}
}  // namespace

HostAllocator::~HostAllocator() {
    for (void* p : blocks_) std::free(p);
}
void* HostAllocator::alloc(size_t bytes) {
    void* p = std::aligned_alloc(64, (std::max<size_t>(bytes, 1) + 63) / 64 * 64);
    if (!p) throw std::runtime_error("host allocation failed");
    blocks_.push_back(p);
    return p;
}
void HostAllocator::upload(void* dst, const void* src, size_t bytes) { std::memcpy(dst, src, bytes); }
void HostAllocator::download(void* dst, const void* src, size_t bytes) { std::memcpy(dst, src, bytes); }

KcAllocator::~KcAllocator() {
    for (void* p : blocks_) kcFree(p);
}
void* KcAllocator::alloc(size_t bytes) {
    void* p = nullptr;
    kcCheck(kcMalloc(&p, std::max<size_t>(bytes, 1)), "kcMalloc");
    blocks_.push_back(p);
    return p;
}
void KcAllocator::upload(void* dst, const void* src, size_t bytes) {
    kcCheck(kcMemcpy(dst, src, bytes, kc::CopyKind::HostToDevice), "kcMemcpy H2D");
}
void KcAllocator::download(void* dst, const void* src, size_t bytes) {
    kcCheck(kcMemcpy(dst, src, bytes, kc::CopyKind::DeviceToHost), "kcMemcpy D2H");
}

// ---- activations and model upload -------------------------------------------------------------------
namespace {
template <class T>
T* uploaded(Allocator& alloc, const T* host, size_t n) {
    void* p = alloc.alloc(n * sizeof(T));
    alloc.upload(p, host, n * sizeof(T));
    return static_cast<T*>(p);
}
float* zeros(Allocator& alloc, size_t n) {
    const std::vector<float> z(n, 0.0f);
    return uploaded(alloc, z.data(), n);
}
struct XorShift {  // the reference's generator for the fixed start vector (llm/llm_model.cpp:138-148)
    uint64_t s;
    float uniform() {
        s ^= s << 13, s ^= s >> 7, s ^= s << 17;
        return static_cast<float>(s >> 40) * (2.0f / 16777216.0f) - 1.0f;
    }
};
Mat uploadMat(const HostMat& h, Allocator& alloc, int64_t* bytes) {
    if (h.rows % 8 || h.k % 256) throw std::runtime_error("matrix shape not supported (rows % 8, k % 256)");
    const size_t n = ref::packedBytes(h.rows, h.k, h.q6);
    std::vector<int> packed((n + 3) / 4);
    if (h.q6) ref::repackQ6K(h.blocks, h.rows, h.k, packed.data());
    else ref::repackQ4K(h.blocks, h.rows, h.k, packed.data());
    *bytes += int64_t(n);
    const int dims[2] = {h.rows, h.k};
    return Mat{h.rows, h.k, h.q6 ? Weights::Q6K : Weights::Q4K, uploaded(alloc, reinterpret_cast<const uint8_t*>(packed.data()), n),
               nullptr, uploaded(alloc, dims, 2)};
}
}  // namespace

Acts allocActs(const Config& c, Allocator& alloc, uint64_t seed) {
    Acts a;
    XorShift rng{seed | 1};
    std::vector<float> x0(size_t(c.hidden));
    for (float& f : x0) f = rng.uniform();
    a.x0 = uploaded(alloc, x0.data(), x0.size());
    a.x = zeros(alloc, size_t(c.hidden));
    a.xn = zeros(alloc, size_t(c.hidden));
    const int qd = c.heads * c.head_dim;
    a.q = zeros(alloc, size_t(qd + 2 * c.kvStride()));
    a.k = a.q + qd;
    a.v = a.k + c.kvStride();
    a.scores = zeros(alloc, size_t(c.heads) * padTo8(c.max_ctx));
    a.attn = zeros(alloc, size_t(qd));
    a.t = zeros(alloc, size_t(c.hidden));
    a.g = zeros(alloc, size_t(2 * c.inter));
    a.u = a.g + c.inter;
    a.h = zeros(alloc, size_t(c.inter));
    a.logits = zeros(alloc, size_t(c.vocab));
    const int maxk = std::max({c.hidden, c.inter, qd});
    a.xq = reinterpret_cast<int*>(zeros(alloc, size_t(scratchInts(maxk / 32))));
    return a;
}

Model uploadModel(const HostModel& host, Allocator& alloc) {
    const Config& c = host.cfg;
    if (c.head_dim % 8 || c.hidden % 256 || c.inter % 256 || c.heads % c.kv_heads || c.max_ctx < 1)
        throw std::runtime_error("model shapes not supported");
    Model m;
    m.cfg = c;
    m.cfg.weights = Weights::Gguf;
    int64_t bytes = 0;
    for (const HostLayer& h : host.layers) {
        Layer L;
        L.qkv_parts = {uploadMat(h.wq, alloc, &bytes), uploadMat(h.wk, alloc, &bytes), uploadMat(h.wv, alloc, &bytes)};
        L.wo = uploadMat(h.wo, alloc, &bytes);
        L.gu_parts = {uploadMat(h.wg, alloc, &bytes), uploadMat(h.wu, alloc, &bytes)};
        L.wd = uploadMat(h.wd, alloc, &bytes);
        L.attn_norm = uploaded(alloc, h.attn_norm, size_t(c.hidden));
        L.ffn_norm = uploaded(alloc, h.ffn_norm, size_t(c.hidden));
        if (c.qk_norm) {
            L.q_norm = uploaded(alloc, h.q_norm, size_t(c.head_dim));
            L.k_norm = uploaded(alloc, h.k_norm, size_t(c.head_dim));
        }
        L.k_cache = zeros(alloc, size_t(c.kStride()) * c.kvStride());
        L.v_cache = zeros(alloc, size_t(c.max_ctx) * c.kvStride());
        m.layers.push_back(std::move(L));
    }
    m.out_norm = uploaded(alloc, host.out_norm, size_t(c.hidden));
    m.lm_head = uploadMat(host.lm_head, alloc, &bytes);
    if (host.rope_ff) m.rope_ff = uploaded(alloc, host.rope_ff, size_t(c.head_dim / 2));
    const AttnDims d = c.attnDims(c.max_ctx);
    const int dims[7] = {d.n_heads, d.ctx, d.head_dim, d.kv_stride, d.group, d.ctx_pad, d.k_stride};
    m.attn_dims = uploaded(alloc, dims, 7);
    m.cfg.file_weight_bytes = bytes;

    // Tied embeddings: a token's embedding is its row of the output matrix, dequantised.  The row's
    // GGUF bytes are read from the caller's host copy and expanded on the host with the format's own
    // formula -- a table lookup, not a compute path -- exactly where the reference does it
    // (llm/gguf_model.cpp:96-104).
    const HostMat e = host.lm_head;
    const int hidden = c.hidden;
    m.embed = [e, hidden](int token, float* out) {
        if (token < 0 || token >= e.rows) throw std::out_of_range("token id outside the vocabulary");
        const int nsb = hidden / 256;
        auto half = [](const uint8_t* p) {
            const uint32_t h = uint32_t(p[0]) | uint32_t(p[1]) << 8, sign = (h & 0x8000u) << 16, ex = (h >> 10) & 31u, man = h & 1023u;
            uint32_t bits;
            if (ex == 0) {
                if (!man) bits = sign;
                else {
                    uint32_t mm = man;
                    int sh = 0;
                    while (!(mm & 0x400u)) mm <<= 1, ++sh;
                    bits = sign | uint32_t(113 - sh) << 23 | (mm & 1023u) << 13;
                }
            } else bits = sign | (ex == 31 ? 0x7F800000u : (ex + 112u) << 23) | man << 13;
            float f;
            std::memcpy(&f, &bits, 4);
            return f;
        };
        for (int s = 0; s < nsb; ++s) {
            float* y = out + s * 256;
            if (e.q6) {
                const uint8_t* b = e.blocks + (size_t(token) * nsb + s) * 210;
                const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
                const float d = half(b + 208);
                for (int i = 0; i < 256; ++i) {
                    const int n = i >> 7, t = (i >> 5) & 3, l = i & 31;
                    const int lo = t & 1 ? b[64 * n + l + 32] : b[64 * n + l];
                    const int nib = t >> 1 ? lo >> 4 : lo & 15;
                    const int q = (nib | (((b[128 + 32 * n + l] >> (2 * t)) & 3) << 4)) - 32;
                    y[i] = d * float(sc[8 * n + l / 16 + 2 * t]) * float(q);
                }
            } else {
                const uint8_t* b = e.blocks + (size_t(token) * nsb + s) * 144;
                const float d = half(b), dmin = half(b + 2);
                const uint8_t* p = b + 4;
                for (int j = 0; j < 8; ++j) {
                    const int sc = j < 4 ? p[j] & 63 : (p[j + 4] & 15) | ((p[j - 4] >> 6) << 4);
                    const int mn = j < 4 ? p[j + 4] & 63 : (p[j + 4] >> 4) | ((p[j] >> 6) << 4);
                    const float dl = d * float(sc), ml = dmin * float(mn);
                    for (int l = 0; l < 32; ++l) {
                        const int byte = b[16 + 32 * (j >> 1) + l];
                        y[32 * j + l] = dl * float(j & 1 ? byte >> 4 : byte & 15) - ml;
                    }
                }
            }
        }
    };
    return m;
}

// ---- decode step ----------------------------------------------------------------------------------------
void Backend::rmsNormRows(float*, const float*, int, int) { throw std::logic_error("this backend has no per-head RMSNorm"); }

void decodeToken(Backend& b, const Model& m, const Acts& a, int pos, Profiler* prof, int token) {
    const Config& c = m.cfg;
    if (pos < 0 || pos >= c.max_ctx) throw std::out_of_range("decode position outside the KV cache");
    struct Scope {  // brackets one op category for the optional profiler
        Profiler* p;
        Op o;
        Scope(Profiler* p_, Op o_) : p(p_), o(o_) {
            if (p) p->begin(o);
        }
        ~Scope() {
            if (p) p->end(o);
        }
    };
    b.setScratch(a.xq);
    b.setContext(pos + 1);
    if (token >= 0 && m.embed) {
        std::vector<float> e(size_t(c.hidden));
        m.embed(token, e.data());
        b.upload(a.x, e.data(), c.hidden);
    } else {
        b.copy(a.x, a.x0, c.hidden);
    }
    b.beginToken(prof != nullptr);
    const bool q8 = quantizedActs(c.weights);
    // One fused matrix, or several writing consecutive slices of y from one input; x == nullptr means the
    // input already sits quantized in the scratch.
    auto project = [&b](const Mat& fused, const std::vector<Mat>& parts, const float* x, float* y) {
        if (parts.empty()) {
            if (x) b.matvec(fused, x, y);
            else b.matvecQuantized(fused, y);
            return;
        }
        for (const Mat& part : parts) {
            if (x) b.matvec(part, x, y), x = nullptr;
            else b.matvecQuantized(part, y);
            y += part.rows;
        }
    };
    {
        Scope s(prof, Op::RmsNorm);
        b.rmsNorm(a.x, m.layers.front().attn_norm, a.xn);
    }
    const int n_layers = int(m.layers.size());
    for (int l = 0; l < n_layers; ++l) {
        const Layer& L = m.layers[size_t(l)];
        {
            Scope s(prof, Op::MatvecAttn);  // after layer 0 the preceding norm already quantized the input
            project(L.wqkv, L.qkv_parts, q8 && l > 0 ? nullptr : a.xn, a.q);
        }
        {
            Scope s(prof, Op::Rope);
            if (c.qk_norm) {
                b.rmsNormRows(a.q, L.q_norm, c.head_dim, c.heads);
                b.rmsNormRows(a.k, L.k_norm, c.head_dim, c.kv_heads);
            }
            b.rope(a.q, c.heads + c.kv_heads, pos);  // q and k are adjacent
            b.appendKv(a.k, a.v, L.k_cache, L.v_cache, pos);
        }
        {
            Scope s(prof, Op::Attention);
            b.attnScores(a.q, L.k_cache, a.scores);
            b.softmax(a.scores);
            b.attnValues(a.scores, L.v_cache, a.attn);
        }
        {
            Scope s(prof, Op::MatvecAttn);
            b.matvec(L.wo, a.attn, a.t);
        }
        const float* next_norm = l + 1 < n_layers ? m.layers[size_t(l) + 1].attn_norm : m.out_norm;
        if (q8) {
            {
                Scope s(prof, Op::Add);
                b.addRmsNormQuant(a.x, a.t, L.ffn_norm);
            }
            {
                Scope s(prof, Op::MatvecFfn);
                project(L.wgu, L.gu_parts, nullptr, a.g);
            }
            {
                Scope s(prof, Op::SiluMul);
                b.siluMulQuant(a.g, a.u, c.inter);
            }
            {
                Scope s(prof, Op::MatvecFfn);
                b.matvecQuantized(L.wd, a.t);
            }
            Scope s(prof, Op::Add);
            b.addRmsNormQuant(a.x, a.t, next_norm);
        } else {
            {
                Scope s(prof, Op::Add);
                b.addRmsNorm(a.x, a.t, L.ffn_norm, a.xn);
            }
            {
                Scope s(prof, Op::MatvecFfn);
                b.matvec(L.wgu, a.xn, a.g);
            }
            {
                Scope s(prof, Op::SiluMul);
                b.siluMul(a.g, a.u, a.h, c.inter);
            }
            {
                Scope s(prof, Op::MatvecFfn);
                b.matvec(L.wd, a.h, a.t);
            }
            Scope s(prof, Op::Add);
            b.addRmsNorm(a.x, a.t, next_norm, a.xn);
        }
    }
    {
        Scope s(prof, Op::MatvecLmHead);
        if (q8) b.matvecQuantized(m.lm_head, a.logits);
        else b.matvec(m.lm_head, a.xn, a.logits);
    }
    b.endToken();
}

// ---- the kc* backend --------------------------------------------------------------------------------------
namespace {

class KcBackend final : public Backend {
public:
    KcBackend(const Model& m, bool graphs) : m_(m), graphs_(graphs), ctx_(m.cfg.max_ctx) {}
    ~KcBackend() override {
        dropCapture();
        if (pos_dev_) kcFree(pos_dev_);
        if (ones_dev_) kcFree(ones_dev_);
    }

    void setScratch(int* q) override { xq_ = q; }
    void setContext(int ctx) override {
        ctx_ = ctx;
        const AttnDims d = m_.cfg.attnDims(ctx);
        const int dims[7] = {d.n_heads, d.ctx, d.head_dim, d.kv_stride, d.group, d.ctx_pad, d.k_stride};
        kcCheck(kcMemcpy(m_.attn_dims, dims, sizeof dims, kc::CopyKind::HostToDevice), "kcMemcpy dims");
        if (m_.cfg.neox) {  // the NEOX rope kernel reads the position from device memory
            if (!pos_dev_) {
                kcCheck(kcMalloc(reinterpret_cast<void**>(&pos_dev_), sizeof(int)), "kcMalloc pos");
                const std::vector<float> ones(size_t(m_.cfg.head_dim / 2), 1.0f);
                kcCheck(kcMalloc(reinterpret_cast<void**>(&ones_dev_), ones.size() * sizeof(float)), "kcMalloc ones");
                kcCheck(kcMemcpy(ones_dev_, ones.data(), ones.size() * sizeof(float), kc::CopyKind::HostToDevice), "kcMemcpy ones");
            }
            const int pos = ctx - 1;
            kcCheck(kcMemcpy(pos_dev_, &pos, sizeof pos, kc::CopyKind::HostToDevice), "kcMemcpy pos");
        }
    }
    void matvec(const Mat& w, const float* x, float* y) override {
        if (!quantizedActs(w.format)) throw std::runtime_error("only K-quant matrices are supported by this build");
        const QuantizeArgs qa{x, xq_, scratchScales(xq_, w.k / 32), w.k / 32};
        launch("quantize_q8x4", &qa);
        matvecQuantized(w, y);
    }
    void matvecQuantized(const Mat& w, float* y) override {
        const MatvecQ4Q8Args a{static_cast<const int*>(w.q), xq_, scratchScales(xq_, w.k / 32), y, w.dims, w.rows, w.k};
        if (w.format == Weights::Q4K) launch("matvec_q4k_q8", &a);
        else if (w.format == Weights::Q6K) launch("matvec_q6k_q8", &a);
        else throw std::runtime_error("only K-quant matrices are supported by this build");
    }
    void rmsNorm(const float* x, const float* w, float* y) override {
        const RmsNormArgs a{x, w, y, m_.cfg.hidden, 1, m_.cfg.eps};
        launch("rms_norm", &a);
    }
    void rmsNormRows(float* x, const float* w, int n, int rows) override {
        const RmsNormArgs a{x, w, x, n, rows, m_.cfg.eps};
        launch("rms_norm", &a);
    }
    void addRmsNorm(float* x, const float* t, const float* w, float* y) override {
        const AddRmsNormArgs a{x, t, w, y, m_.cfg.hidden, m_.cfg.eps};
        launch("add_rms_norm", &a);
    }
    void siluMulQuant(const float* g, const float* u, int n) override {
        const SiluMulQ8Args a{g, u, xq_, scratchScales(xq_, n / 32), n / 32};
        launch("silu_mul_q8x4", &a);
    }
    void addRmsNormQuant(float* x, const float* t, const float* w) override {
        const int nb = m_.cfg.hidden / 32;
        const AddSumsqArgs s{x, t, xq_, nb};
        launch("add_sumsq", &s);
        const NormQ8Args n{x, w, xq_, nb, m_.cfg.eps};
        launch("norm_q8x4", &n);
    }
    void rope(float* x, int heads, int pos) override {
        const int pairs = m_.cfg.head_dim / 2;
        const float lb = std::log2(m_.cfg.rope_base);
        if (m_.cfg.neox) {  // (i, i + head_dim/2) pairs: the ggml-style kernel, in place, one token
            if (pos != ctx_ - 1) throw std::logic_error("rope: position must be the last of the context");
            const RopeGgmlArgs a{x, x, pos_dev_, m_.rope_ff ? m_.rope_ff : ones_dev_, m_.attn_dims, m_.cfg.head_dim, heads, 1, lb, true};
            launch("rope_ggml", &a);
            return;
        }
        if (m_.rope_ff) {
            const RopeFFArgs a{x, m_.rope_ff, pairs, pos, heads * pairs, lb};
            launch("rope_ff", &a);
        } else {
            const RopeArgs a{x, pairs, pos, heads * pairs, lb};
            launch("rope", &a);
        }
    }
    void appendKv(const float* k, const float* v, float* kt, float* vc, int pos) override {
        if (pos != ctx_ - 1) throw std::logic_error("appendKv: position must be the last of the context");
        const KvAppendArgs a{k, v, kt, vc, m_.attn_dims, m_.cfg.attnDims(ctx_)};
        launch("kv_append", &a);
    }
    void attnScores(const float* q, const float* k, float* scores) override {
        const AttnScoresArgs a{q, k, scores, m_.attn_dims, m_.cfg.attnDims(ctx_), 1.0f / std::sqrt(float(m_.cfg.head_dim))};
        launch("attn_scores", &a);
    }
    void softmax(float* scores) override {
        const SoftmaxArgs a{scores, ctx_, padTo8(ctx_), m_.cfg.heads};
        launch("softmax", &a);
    }
    void attnValues(const float* p, const float* v, float* out) override {
        const AttnValuesArgs a{p, v, out, m_.attn_dims, m_.cfg.attnDims(ctx_)};
        launch("attn_values", &a);
    }
    void siluMul(const float* g, const float* u, float* out, int n) override {
        const SiluMulArgs a{g, u, out, n};
        launch("silu_mul", &a);
    }
    void add(float* x, const float* t, int n) override {
        const kc::kernels::VectorAddArgs a{x, t, x, n};
        launch("vector_add", &a);
    }
    void copy(float* dst, const float* src, int n) override {
        kcCheck(kcMemcpy(dst, src, size_t(n) * sizeof(float), kc::CopyKind::DeviceToDevice), "kcMemcpy");
    }
    void upload(float* dst, const float* host, int n) override {
        kcCheck(kcMemcpy(dst, host, size_t(n) * sizeof(float), kc::CopyKind::HostToDevice), "kcMemcpy");
    }
    void finish() override { kcCheck(kcDeviceSynchronize(), "kcDeviceSynchronize"); }
    void beginToken(bool profiling) override {
        dropCapture();  // an earlier token may have thrown between begin and end
        if (!graphs_ || profiling) return;
        kcCheck(kcStreamBeginCapture(nullptr), "kcStreamBeginCapture");
        capturing_ = true;
    }
    void endToken() override {
        if (!capturing_) return;
        capturing_ = false;
        kcGraph_t g = nullptr;
        kcCheck(kcStreamEndCapture(nullptr, &g), "kcStreamEndCapture");
        const kc::Error e = kcGraphLaunch(g, nullptr);  // synchronous: the logits are ready afterwards
        const std::string why = e == kc::Error::Success ? "" : std::string("kcGraphLaunch: ") + kcGetErrorString(e) + " (" + kcGetLastErrorDetail() + ")";
        kcGraphDestroy(g);
        if (e != kc::Error::Success) throw std::runtime_error(why);
    }

private:
    void dropCapture() noexcept {
        if (!capturing_) return;
        capturing_ = false;
        kcGraph_t g = nullptr;
        if (kcStreamEndCapture(nullptr, &g) == kc::Error::Success) kcGraphDestroy(g);
    }
    void launch(const char* name, const void* args) {
        const kc::Error e = kcLaunchKernel(name, args);
        if (e != kc::Error::Success) kcFail(name, e);
    }

    const Model& m_;
    bool graphs_;
    bool capturing_ = false;
    int ctx_;
    int* xq_ = nullptr;
    int* pos_dev_ = nullptr;
    float* ones_dev_ = nullptr;
};

}  // namespace

std::unique_ptr<Backend> makeKcBackend(const Model& m, unsigned, bool graphs, bool) { return std::make_unique<KcBackend>(m, graphs); }

}  // namespace llm
