// ref_shim.cpp -- C entry points onto the reference project's OWN implementation.
//
// TEST INFRASTRUCTURE ONLY.  oracle/Makefile compiles this file together with the
// reference's llm/llm_reference.cpp and llm/llm_model.cpp, in place from the mounted
// reference tree, into oracle/_ref/libkcref.so.  No reference source is copied: this file
// only declares C wrappers that forward to llm::ref::* and llm::decodeToken.  The library is
// used to (1) validate the C restatement in kq_oracle.c, (2) generate the golden vectors
// under tests/golden, (3) time the reference's CPU path as the benchmark's CPU baseline.
//
// Weights cross this boundary as canonical GGUF blocks; the wrappers run the reference's
// repackQ4K / repackQ6K to obtain the 8-row interleaved stream its matvecs consume.

#include "kq_oracle.h"  // struct layouts only (kqo_attn_dims, kqo_fa_dims, kqo_model)

#include "llm_model.hpp"
#include "gguf_model.hpp"
#include "llm_reference.hpp"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <vector>

// ---- the handful of kc* symbols llm_model.cpp links against ---------------------------------
// Only HostAllocator + CppBackend are exercised here; the Kernelcore-runtime classes in that file
// still need their externals resolved.  Memory is host memory, launches are refused.
kc::Error kcMalloc(void** p, size_t n) noexcept {
    *p = std::malloc(n);
    return *p ? kc::Error::Success : kc::Error::OutOfMemory;
}
kc::Error kcFree(void* p) noexcept {
    std::free(p);
    return kc::Error::Success;
}
kc::Error kcMemcpy(void* d, const void* s, size_t n, kc::CopyKind) noexcept {
    std::memcpy(d, s, n);
    return kc::Error::Success;
}
kc::Error kcLaunchKernel(const char*, const void*, kcStream_t) noexcept { return kc::Error::UnsupportedOperation; }
kc::Error kcLaunchKernelChunked(const char*, const void*, unsigned, int64_t, kcStream_t) noexcept {
    return kc::Error::UnsupportedOperation;
}
kc::Error kcStreamBeginCapture(kcStream_t) noexcept { return kc::Error::UnsupportedOperation; }
kc::Error kcStreamEndCapture(kcStream_t, kcGraph_t*) noexcept { return kc::Error::UnsupportedOperation; }
kc::Error kcGraphLaunch(kcGraph_t, kcStream_t) noexcept { return kc::Error::UnsupportedOperation; }
kc::Error kcGraphDestroy(kcGraph_t) noexcept { return kc::Error::Success; }
kc::Error kcDeviceSynchronize() noexcept { return kc::Error::Success; }
const char* kcGetErrorString(kc::Error) noexcept { return "kc stub"; }
const char* kcGetLastErrorDetail() noexcept { return ""; }

namespace {

llm::AttnDims attn(const kqo_attn_dims* d) {
    return {d->n_heads, d->ctx, d->head_dim, d->kv_stride, d->group, d->ctx_pad, d->k_stride};
}
llm::FaDims fa(const kqo_fa_dims* d) {
    llm::FaDims f;
    f.H = d->H, f.T = d->T, f.D = d->D, f.group = d->group, f.tp = d->tp, f.k_row = d->k_row, f.k_head = d->k_head;
    f.v_row = d->v_row, f.v_head = d->v_head, f.N = d->N, f.q_tok = d->q_tok, f.q_head = d->q_head;
    f.m_row = d->m_row, f.has_mask = d->has_mask, f.H_kv = d->H_kv;
    return f;
}
std::vector<int> stream(const uint8_t* w, int rows, int k, int q6) {
    std::vector<int> qw(size_t(rows) * (k / 256) * (q6 ? 53 : 37));
    if (q6) llm::ref::repackQ6K(w, rows, k, qw.data());
    else llm::ref::repackQ4K(w, rows, k, qw.data());
    return qw;
}

struct OpenModel {
    llm::HostAllocator alloc;
    llm::Model model;
    llm::Acts acts;
    std::unique_ptr<llm::Backend> backend;
    std::vector<float> x_in;
};

llm::Mat mat(OpenModel& om, const kqo_mat& w) {
    const std::vector<int> qw = stream(w.blocks, w.rows, w.k, w.fmt == 6);
    void* q = om.alloc.alloc(qw.size() * sizeof(int));
    std::memcpy(q, qw.data(), qw.size() * sizeof(int));
    int* dims = static_cast<int*>(om.alloc.alloc(2 * sizeof(int)));
    dims[0] = w.rows, dims[1] = w.k;
    return llm::Mat{w.rows, w.k, w.fmt == 6 ? llm::Weights::Q6K : llm::Weights::Q4K, q, nullptr, dims};
}

} // namespace

extern "C" {

float kcref_f16_to_f32(uint16_t h) { return llm::ref::f16ToF32(h); }
uint16_t kcref_f32_to_f16(float x) { return llm::ref::f32ToF16(x); }
void kcref_dequant_row_q4k(const uint8_t* s, int k, float* o) { llm::ref::dequantRowQ4K(s, k, o); }
void kcref_dequant_row_q6k(const uint8_t* s, int k, float* o) { llm::ref::dequantRowQ6K(s, k, o); }
void kcref_quantize_q8x4(const float* x, int32_t* xq, float* xd, int n) { llm::ref::quantizeQ8x4(x, xq, xd, n); }
void kcref_quantize_q8k(const float* x, int32_t* q, int nsb) { llm::ref::quantizeQ8K(x, q, nsb); }

// The reference's own weight stream, for timing its matvec without the repack.
long kcref_stream_ints(int rows, int k, int q6) { return long(rows) * (k / 256) * (q6 ? 53 : 37); }
void kcref_repack(const uint8_t* w, int rows, int k, int q6, int32_t* qw) {
    if (q6) llm::ref::repackQ6K(w, rows, k, qw);
    else llm::ref::repackQ4K(w, rows, k, qw);
}
void kcref_matvec_stream_q8(const int32_t* qw, const int32_t* xq, const float* xd, float* y, int rows, int k, int q6) {
    if (q6) llm::ref::matvecQ6KQ8(qw, xq, xd, y, rows, k);
    else llm::ref::matvecQ4KQ8(qw, xq, xd, y, rows, k);
}
void kcref_matvec_stream_q8k(const int32_t* qw, const int32_t* xq, float* y, int rows, int k, int q6) {
    if (q6) llm::ref::matvecQ6KQ8K(qw, xq, y, rows, k);
    else llm::ref::matvecQ4KQ8K(qw, xq, y, rows, k);
}

void kcref_matvec_q8w(const int8_t* q, const float* scales, const float* x, float* y, int rows, int k) {
    llm::ref::matvecQ8(q, scales, x, y, rows, k);
}
void kcref_matvec_q4w(const uint8_t* qs, const float* scales, const float* x, float* y, int rows, int k) {
    llm::ref::matvecQ4(qs, scales, x, y, rows, k);
}
void kcref_repack_q4x8(const uint8_t* qs, const float* scales, uint8_t* qs8, float* scales8, int rows, int k) {
    llm::ref::repackQ4x8(qs, scales, qs8, scales8, rows, k);
}
void kcref_matvec_q4x8(const uint8_t* qs8, const float* scales8, const float* x, float* y, int rows, int k) {
    llm::ref::matvecQ4x8(qs8, scales8, x, y, rows, k);
}
void kcref_repack_q4x8_q8(const uint8_t* qs, const float* scales, int32_t* qw, int rows, int k) {
    llm::ref::repackQ4x8Q8(qs, scales, qw, rows, k);
}
void kcref_matvec_q4x8_q8(const int32_t* qw, const int32_t* xq, const float* xd, float* y, int rows, int k) {
    llm::ref::matvecQ4x8Q8(qw, xq, xd, y, rows, k);
}
void kcref_repack_f16(const uint16_t* w, int rows, int k, int32_t* out) { llm::ref::repackF16(w, rows, k, out); }
void kcref_matmul_f16(const uint16_t* w, const float* x, float* y, int rows, int k, int ncols) {
    llm::ref::matmulF16(w, x, y, rows, k, ncols);
}
void kcref_matvec_q4k_q8(const uint8_t* w, const int32_t* xq, const float* xd, float* y, int rows, int k) {
    llm::ref::matvecQ4KQ8(stream(w, rows, k, 0).data(), xq, xd, y, rows, k);
}
void kcref_matvec_q6k_q8(const uint8_t* w, const int32_t* xq, const float* xd, float* y, int rows, int k) {
    llm::ref::matvecQ6KQ8(stream(w, rows, k, 1).data(), xq, xd, y, rows, k);
}
void kcref_matvec_q4k_q8k(const uint8_t* w, const int32_t* xq, float* y, int rows, int k) {
    llm::ref::matvecQ4KQ8K(stream(w, rows, k, 0).data(), xq, y, rows, k);
}
void kcref_matvec_q6k_q8k(const uint8_t* w, const int32_t* xq, float* y, int rows, int k) {
    llm::ref::matvecQ6KQ8K(stream(w, rows, k, 1).data(), xq, y, rows, k);
}

void kcref_rms_norm(const float* x, const float* w, float* y, int n, int rows, float eps) {
    llm::ref::rmsNorm(x, w, y, n, rows, eps);
}
void kcref_add(float* x, const float* t, int n) { llm::ref::add(x, t, n); }
void kcref_add_rms_norm(float* x, const float* t, const float* w, float* y, int n, float eps) {
    llm::ref::addRmsNorm(x, t, w, y, n, eps);
}
void kcref_add_sumsq(float* x, const float* t, int32_t* q, int nb) { llm::ref::addSumsq(x, t, q, nb); }
void kcref_norm_q8x4(const float* x, const float* w, int32_t* q, int nb, float eps) {
    llm::ref::normQ8x4(x, w, q, nb, eps);
}
void kcref_rope(float* x, int pairs, int pos, int count, float lb) { llm::ref::rope(x, pairs, pos, count, lb); }
void kcref_rope_ff(float* x, const float* ff, int pairs, int pos, int count, float lb) {
    llm::ref::ropeFF(x, ff, pairs, pos, count, lb);
}
void kcref_rope_ggml(const float* x, float* y, const int32_t* pos, const float* ff, int head_dim, int n_head,
                     int n_tokens, float lb, int neox) {
    llm::ref::ropeGgml(x, y, pos, ff, head_dim, n_head, n_tokens, lb, neox != 0);
}
void kcref_append_kv(const float* k, const float* v, float* kt, float* vc, int n, int k_stride, int pos) {
    llm::ref::appendKv(k, v, kt, vc, n, k_stride, pos);
}
void kcref_attn_scores(const float* q, const float* kt, float* s, const kqo_attn_dims* d, float scale) {
    llm::ref::attnScores(q, kt, s, attn(d), scale);
}
void kcref_softmax(float* x, int n, int stride, int rows) { llm::ref::softmax(x, n, stride, rows); }
void kcref_attn_values(const float* p, const float* v, float* out, const kqo_attn_dims* d) {
    llm::ref::attnValues(p, v, out, attn(d));
}
void kcref_silu_mul(const float* g, const float* u, float* out, int n) { llm::ref::siluMul(g, u, out, n); }
void kcref_silu_mul_q8x4(const float* g, const float* u, int32_t* xq, float* xd, int n) {
    llm::ref::siluMulQ8x4(g, u, xq, xd, n);
}
void kcref_mul_rows(const float* x, const float* w, float* y, int n, int count) { llm::ref::mulRows(x, w, y, n, count); }
void kcref_add_sumsq_f(const float* a, const float* b, float* out, int32_t* q, int n, int rows) {
    llm::ref::addSumsqF(a, b, out, q, n, rows);
}
void kcref_sumsq_part(const float* x, int32_t* q, int n, int rows) { llm::ref::sumsqPart(x, q, n, rows); }
void kcref_norm_mul_q8(const float* x, const float* w, float* y, int32_t* q, int n, int rows, float eps) {
    llm::ref::normMulQ8(x, w, y, q, n, rows, eps);
}
void kcref_norm_mul_q8k(const float* x, const float* w, float* y, int32_t* q, const int32_t* sq, int n, int rows,
                        float eps) {
    llm::ref::normMulQ8K(x, w, y, q, sq, n, rows, eps);
}
void kcref_silu_mul_q8f(const float* g, const float* u, float* y, int32_t* q, int n, int cols) {
    llm::ref::siluMulQ8F(g, u, y, q, n, cols);
}
void kcref_silu_mul_q8k(const float* g, const float* u, float* y, int32_t* q, int n, int cols) {
    llm::ref::siluMulQ8K(g, u, y, q, n, cols);
}
void kcref_set_rows_f16(const float* src, const int64_t* idx, uint16_t* dst, int pairs, int rows, int src_row,
                        int dst_row, int dst_rows) {
    llm::ref::setRowsF16(src, idx, dst, pairs, rows, src_row, dst_row, dst_rows);
}
void kcref_flash_attn_f16(const float* q, const uint16_t* k, const uint16_t* v, const uint16_t* mask, float* out,
                          const kqo_fa_dims* d, float scale) {
    llm::ref::flashAttnF16(q, k, v, mask, out, fa(d), scale);
}

// ---- the reference's decode loop on its single-thread C++ backend ----------------------------
void* kcref_model_open(const kqo_model* m) {
    auto om = std::make_unique<OpenModel>();
    llm::Config c;
    c.name = "oracle";
    c.hidden = m->hidden, c.inter = m->inter, c.layers = m->n_layers, c.heads = m->heads, c.kv_heads = m->kv_heads;
    c.head_dim = m->head_dim, c.vocab = m->vocab, c.max_ctx = m->max_ctx, c.eps = m->eps, c.rope_base = m->rope_base;
    c.weights = llm::Weights::Gguf;
    om->model.cfg = c;
    for (int l = 0; l < m->n_layers; ++l) {
        const kqo_layer& s = m->layers[l];
        llm::Layer L;
        L.qkv_parts = {mat(*om, s.wq), mat(*om, s.wk), mat(*om, s.wv)};
        L.wo = mat(*om, s.wo);
        L.gu_parts = {mat(*om, s.wg), mat(*om, s.wu)};
        L.wd = mat(*om, s.wd);
        L.attn_norm = s.attn_norm, L.ffn_norm = s.ffn_norm;
        L.k_cache = s.k_cache, L.v_cache = s.v_cache;
        om->model.layers.push_back(std::move(L));
    }
    om->model.out_norm = m->out_norm;
    om->model.lm_head = mat(*om, m->lm_head);
    om->model.rope_ff = m->rope_ff;
    om->x_in.resize(size_t(m->hidden));
    OpenModel* raw = om.get();
    om->model.embed = [raw](int, float* out) { std::memcpy(out, raw->x_in.data(), raw->x_in.size() * sizeof(float)); };
    om->acts = llm::allocActs(c, om->alloc, 1);
    om->backend = llm::makeCppBackend(om->model);
    return om.release();
}
int kcref_model_decode(void* h, const float* x_in, int pos, float* logits) {
    auto* om = static_cast<OpenModel*>(h);
    try {
        std::memcpy(om->x_in.data(), x_in, om->x_in.size() * sizeof(float));
        llm::decodeToken(*om->backend, om->model, om->acts, pos, nullptr, 0);
        std::memcpy(logits, om->acts.logits, size_t(om->model.cfg.vocab) * sizeof(float));
    } catch (...) {
        return 1;
    }
    return 0;
}
void kcref_model_close(void* h) { delete static_cast<OpenModel*>(h); }

// ---- the reference's own GGUF reader and loader (llm/gguf.cpp, llm/gguf_model.cpp) -------------------------------
// kcref_gguf_open reads a file with the reference's reader and loads it with llm::loadGguf onto its single-thread C++
// backend: the counterpart of kcb_gguf_open + kcb_model_create, for files this project's tests write.  A reader and a
// writer by the same author could share a misreading of the format; the reference's reader does not.
struct OpenGguf {
    std::unique_ptr<llm::gguf::File> file;
    llm::HostAllocator alloc;
    llm::Model model;
    llm::Acts acts;
    std::unique_ptr<llm::Backend> backend;
    std::string error;
};
static thread_local std::string g_gguf_error;
const char* kcref_gguf_last_error() { return g_gguf_error.c_str(); }
void* kcref_gguf_open(const char* path, int max_ctx) {
    auto g = std::make_unique<OpenGguf>();
    try {
        g->file = std::make_unique<llm::gguf::File>(path);
        g->model = llm::loadGguf(*g->file, max_ctx, g->alloc);
        g->acts = llm::allocActs(g->model.cfg, g->alloc, 1);
        g->backend = llm::makeCppBackend(g->model);
    } catch (const std::exception& e) {
        g_gguf_error = e.what();
        return nullptr;
    }
    return g.release();
}
// dims: hidden, inter, layers, heads, kv_heads, head_dim, vocab, max_ctx; eps and rope_base as floats.
void kcref_gguf_config(void* h, int* dims, float* eps, float* rope_base) {
    const llm::Config& c = static_cast<OpenGguf*>(h)->model.cfg;
    const int v[8] = {c.hidden, c.inter, c.layers, c.heads, c.kv_heads, c.head_dim, c.vocab, c.max_ctx};
    std::memcpy(dims, v, sizeof v);
    *eps = c.eps, *rope_base = c.rope_base;
}
// One directory entry as the reference's reader sees it; returns 0 when the tensor is absent.
int kcref_gguf_tensor(void* h, const char* name, unsigned* type, unsigned long long* offset, unsigned long long* bytes, long long* ne4,
                      unsigned long long* byte_sum) {
    const llm::gguf::Tensor* t = static_cast<OpenGguf*>(h)->file->find(name);
    if (!t) return 0;
    *type = t->type, *offset = t->offset, *bytes = t->bytes;
    for (int d = 0; d < 4; ++d) ne4[d] = d < int(t->ne.size()) ? t->ne[size_t(d)] : 1;
    unsigned long long sum = 0;
    for (size_t i = 0; i < t->bytes; ++i) sum += static_cast<unsigned long long>(t->data[i]) * (i % 251 + 1);
    *byte_sum = sum;
    return 1;
}
int kcref_gguf_decode(void* h, int token, int pos, float* logits) {
    auto* g = static_cast<OpenGguf*>(h);
    try {
        llm::decodeToken(*g->backend, g->model, g->acts, pos, nullptr, token);
        std::memcpy(logits, g->acts.logits, size_t(g->model.cfg.vocab) * sizeof(float));
    } catch (const std::exception& e) {
        g_gguf_error = e.what();
        return 1;
    }
    return 0;
}
void kcref_gguf_close(void* h) { delete static_cast<OpenGguf*>(h); }

// The reference's synthetic tiny model (llm::tinyConfig + llm::buildModels, weights 0 = Q8, 1 = Q4, 2 = Q4X8,
// 3 = Q4X8Q8) on its single-thread C++ backend: one decodeToken from the start vector of allocActs at `pos`, as its
// own test tiny_decode_token_kc_vs_cpp does (tests/test_llm_kernels.cpp:891-930).  Returns the vocabulary size, or
// -1 on an exception.  A checksum over the first matrix's bytes and scales is written to *weight_sum when not null.
int kcref_synthetic_tiny_logits(int weights, unsigned long long model_seed, unsigned long long start_seed, int pos, float* logits,
                                double* weight_sum) {
    try {
        const llm::Config cfg = llm::tinyConfig(static_cast<llm::Weights>(weights));
        llm::HostAllocator alloc;
        std::vector<llm::Model> models;
        llm::buildModels(cfg, model_seed, {&alloc}, models);
        const llm::Acts acts = llm::allocActs(cfg, alloc, start_seed);
        auto backend = llm::makeCppBackend(models[0]);
        llm::decodeToken(*backend, models[0], acts, pos);
        if (logits) std::memcpy(logits, acts.logits, size_t(cfg.vocab) * sizeof(float));
        if (weight_sum) {
            const llm::Mat& w = models[0].layers[0].wqkv;
            double sum = 0.0;
            const size_t bytes = size_t(w.rows) * size_t(w.k) / (weights == 0 ? 1 : 2) + (weights == 3 ? size_t(w.rows) * size_t(w.k) / 8 : 0);
            const uint8_t* q = static_cast<const uint8_t*>(w.q);
            for (size_t i = 0; i < bytes; ++i) sum += double(q[i]) * double(i % 251 + 1);
            *weight_sum = sum;
        }
        return cfg.vocab;
    } catch (...) {
        return -1;
    }
}

} // extern "C"
