// One decode step over any llm::Backend.
//
// The order of Backend calls, and which profiler category each falls in, is the reference's (llm/llm_model.cpp:287-360),
// because third-party backends and profilers are written against it: first norm; per layer q|k|v, [head norms,] rope,
// KV append, scores, softmax, values, output projection, add + norm, gate|up, SwiGLU, down, add + norm; then the LM
// head.  With quantized activations the norm and SwiGLU calls leave their result in the scratch and the matvec that
// follows reads it from there.
#include <llm_model.hpp>

#include <stdexcept>
#include <vector>

namespace llm {

void Backend::rmsNormRows(float*, const float*, int, int) { throw std::logic_error("this backend has no per-head RMSNorm"); }

namespace {

class TokenStep {
public:
    TokenStep(Backend& backend, const Model& model, const Acts& acts, int pos, Profiler* profiler)
        : b_(backend), m_(model), a_(acts), c_(model.cfg), pos_(pos), prof_(profiler), scratch_(quantizedActs(model.cfg.weights)) {}

    void run() {
        enter(Op::RmsNorm);
        b_.rmsNorm(a_.x, m_.layers.front().attn_norm, a_.xn);
        for (size_t l = 0; l < m_.layers.size(); ++l) {
            const Layer& layer = m_.layers[l];
            const bool last = l + 1 == m_.layers.size();
            attention(layer, /*input_in_scratch=*/scratch_ && l > 0);
            feedForward(layer, last ? m_.out_norm : m_.layers[l + 1].attn_norm);
        }
        enter(Op::MatvecLmHead);
        if (scratch_) b_.matvecQuantized(m_.lm_head, a_.logits);
        else b_.matvec(m_.lm_head, a_.xn, a_.logits);
        leave();
    }

private:
    // Profiler brackets: entering a category closes the one that is open.
    void enter(Op op) {
        if (!prof_) return;
        leave();
        prof_->begin(op);
        open_ = op;
    }
    void leave() {
        if (prof_ && open_ != Op::Count) prof_->end(open_);
        open_ = Op::Count;
    }

    // y = W x for a matrix kept whole or as parts whose outputs are consecutive slices of y.  x == nullptr: the input
    // is already quantized in the scratch; otherwise the first matvec quantizes it there for the others.
    void product(const Mat& whole, const std::vector<Mat>& parts, const float* x, float* y) {
        const Mat* first = parts.empty() ? &whole : parts.data();
        const size_t count = parts.empty() ? 1 : parts.size();
        for (size_t i = 0; i < count; ++i) {
            if (x != nullptr && i == 0) b_.matvec(first[i], x, y);
            else b_.matvecQuantized(first[i], y);
            y += first[i].rows;
        }
    }

    void attention(const Layer& L, bool input_in_scratch) {
        enter(Op::MatvecAttn);
        product(L.wqkv, L.qkv_parts, input_in_scratch ? nullptr : a_.xn, a_.q);
        enter(Op::Rope);
        if (c_.qk_norm) {
            b_.rmsNormRows(a_.q, L.q_norm, c_.head_dim, c_.heads);
            b_.rmsNormRows(a_.k, L.k_norm, c_.head_dim, c_.kv_heads);
        }
        b_.rope(a_.q, c_.heads + c_.kv_heads, pos_);  // k follows q in memory
        b_.appendKv(a_.k, a_.v, L.k_cache, L.v_cache, pos_);
        enter(Op::Attention);
        b_.attnScores(a_.q, L.k_cache, a_.scores);
        b_.softmax(a_.scores);
        b_.attnValues(a_.scores, L.v_cache, a_.attn);
        enter(Op::MatvecAttn);
        b_.matvec(L.wo, a_.attn, a_.t);
    }

    void feedForward(const Layer& L, const float* next_norm) {
        enter(Op::Add);
        if (scratch_) b_.addRmsNormQuant(a_.x, a_.t, L.ffn_norm);
        else b_.addRmsNorm(a_.x, a_.t, L.ffn_norm, a_.xn);
        enter(Op::MatvecFfn);
        if (scratch_) product(L.wgu, L.gu_parts, nullptr, a_.g);
        else b_.matvec(L.wgu, a_.xn, a_.g);
        enter(Op::SiluMul);
        if (scratch_) b_.siluMulQuant(a_.g, a_.u, c_.inter);
        else b_.siluMul(a_.g, a_.u, a_.h, c_.inter);
        enter(Op::MatvecFfn);
        if (scratch_) b_.matvecQuantized(L.wd, a_.t);
        else b_.matvec(L.wd, a_.h, a_.t);
        enter(Op::Add);
        if (scratch_) b_.addRmsNormQuant(a_.x, a_.t, next_norm);
        else b_.addRmsNorm(a_.x, a_.t, next_norm, a_.xn);
    }

    Backend& b_;
    const Model& m_;
    const Acts& a_;
    const Config& c_;
    const int pos_;
    Profiler* const prof_;
    const bool scratch_;  // activations travel between calls as 8-bit blocks in Acts::xq
    Op open_ = Op::Count;
};

}  // namespace

void decodeToken(Backend& b, const Model& m, const Acts& a, int pos, Profiler* prof, int token) {
    if (pos < 0 || pos >= m.cfg.max_ctx) throw std::out_of_range("decode position outside the KV cache");
    if (m.layers.empty()) throw std::invalid_argument("model has no layers");
    b.setScratch(a.xq);
    b.setContext(pos + 1);
    if (token >= 0 && m.embed) {
        std::vector<float> row(size_t(m.cfg.hidden));
        m.embed(token, row.data());
        b.upload(a.x, row.data(), m.cfg.hidden);
    } else {
        b.copy(a.x, a.x0, m.cfg.hidden);
    }
    b.beginToken(prof != nullptr);
    TokenStep(b, m, a, pos, prof).run();
    b.endToken();
}

}  // namespace llm
