// Where a model's bytes live: the two allocators, the device layouts of K-quant matrices, the activation buffers
// of a decode step and the upload of a model described by GGUF blocks on the host.
//
// Interfaces: llm/llm_model.hpp:64-98 (allocators), :139-144 (allocActs) and llm/gguf_model.cpp:29-106 (a model
// assembled from separate q/k/v and gate/up matrices with tied embeddings) of the reference.  Errors leave as
// std::runtime_error with the kc runtime's text, as the reference's do.
#include <llm_model.hpp>
#include <llm_reference.hpp>

#include "llm_host.hpp"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

namespace llm {

// ---- errors ---------------------------------------------------------------------------------------------------
namespace host {

void require(kc::Error status, std::string_view doing) {
    if (status == kc::Error::Success) return;
    std::string text(doing);
    text += ": ";
    text += kcGetErrorString(status);
    if (const char* detail = kcGetLastErrorDetail(); detail && *detail) {
        text += " (";
        text += detail;
        text += ")";
    }
    throw std::runtime_error(text);
}

}  // namespace host

// ---- allocators -----------------------------------------------------------------------------------------------
namespace detail {

BlockLedger::~BlockLedger() {
    while (!held_.empty()) {
        release_(held_.back());
        held_.pop_back();
    }
}

void* BlockLedger::keep(void* block) {
    held_.push_back(block);
    return block;
}

}  // namespace detail

namespace {
constexpr size_t kHostAlign = 64;
void releaseDevice(void* p) { kcFree(p); }
size_t atLeastOne(size_t bytes) { return bytes ? bytes : 1; }
}  // namespace

HostAllocator::HostAllocator() : ledger_(&std::free) {}

void* HostAllocator::alloc(size_t bytes) {
    const size_t rounded = (atLeastOne(bytes) + kHostAlign - 1) & ~(kHostAlign - 1);  // aligned_alloc wants a multiple
    if (void* p = std::aligned_alloc(kHostAlign, rounded)) return ledger_.keep(p);
    throw std::runtime_error("host allocation failed");
}
void HostAllocator::upload(void* dst, const void* src, size_t bytes) { std::memcpy(dst, src, bytes); }
void HostAllocator::download(void* dst, const void* src, size_t bytes) { std::memcpy(dst, src, bytes); }

KcAllocator::KcAllocator() : ledger_(&releaseDevice) {}

void* KcAllocator::alloc(size_t bytes) {
    void* p = nullptr;
    host::require(kcMalloc(&p, atLeastOne(bytes)), "kcMalloc");
    return ledger_.keep(p);
}
void KcAllocator::upload(void* dst, const void* src, size_t bytes) {
    host::require(kcMemcpy(dst, src, bytes, kc::CopyKind::HostToDevice), "kcMemcpy H2D");
}
void KcAllocator::download(void* dst, const void* src, size_t bytes) {
    host::require(kcMemcpy(dst, src, bytes, kc::CopyKind::DeviceToHost), "kcMemcpy D2H");
}

// ---- device layouts of K-quant matrices -----------------------------------------------------------------------
namespace ref {

namespace {
// A Q6_K block is ql[128] qh[64] scales[16] d[2]; on the device each of the four fields is a plane of its own over
// all blocks of the matrix, so that a warp's loads of one field are contiguous.
struct Q6Field {
    size_t in_block, bytes;
};
constexpr Q6Field kQ6Fields[4] = {{0, 128}, {128, 64}, {192, 16}, {208, 2}};
constexpr size_t kQ6Block = 210;

template <bool kToPlanes>
void q6Shuffle(const uint8_t* src, uint8_t* dst, size_t blocks) {
    size_t plane = 0;
    for (const Q6Field& f : kQ6Fields) {
        for (size_t b = 0; b < blocks; ++b) {
            const size_t in_planes = plane + b * f.bytes, in_blocks = b * kQ6Block + f.in_block;
            if (kToPlanes) std::memcpy(dst + in_planes, src + in_blocks, f.bytes);
            else std::memcpy(dst + in_blocks, src + in_planes, f.bytes);
        }
        plane += blocks * f.bytes;
    }
}
}  // namespace

void repackQ4K(const uint8_t* src, int rows, int k, int* qw) { std::memcpy(qw, src, packedBytes(rows, k, false)); }
void repackQ6K(const uint8_t* src, int rows, int k, int* qw) {
    q6Shuffle<true>(src, reinterpret_cast<uint8_t*>(qw), size_t(rows) * size_t(k / 256));
}
void unpackQ6K(const int* qw, int rows, int k, uint8_t* dst) {
    q6Shuffle<false>(reinterpret_cast<const uint8_t*>(qw), dst, size_t(rows) * size_t(k / 256));
}

}  // namespace ref

// ---- activations ----------------------------------------------------------------------------------------------
uint64_t host::SeedStream::word() {
    state_ ^= state_ << 13;
    state_ ^= state_ >> 7;
    state_ ^= state_ << 17;
    return state_;
}
float host::SeedStream::unit() { return static_cast<float>(word() >> 40) * (2.0f / 16777216.0f) - 1.0f; }

// One block holds every activation buffer, each starting on a 256-byte boundary; it is staged on the host (zeros,
// and the start vector drawn from `seed` in x0) and uploaded in one copy.
Acts allocActs(const Config& c, Allocator& alloc, uint64_t seed) {
    const size_t hidden = size_t(c.hidden), qd = size_t(c.heads) * size_t(c.head_dim), kv = size_t(c.kvStride());
    const size_t widest = std::max({hidden, size_t(c.inter), qd});
    struct Slice {
        float* Acts::*field;
        size_t floats;
    };
    const Slice slices[] = {
        {&Acts::x0, hidden},
        {&Acts::x, hidden},
        {&Acts::xn, hidden},
        {&Acts::q, qd + 2 * kv},  // q | k | v in one buffer: one rope launch covers q and k
        {&Acts::scores, size_t(c.heads) * size_t(padTo8(c.max_ctx))},
        {&Acts::attn, qd},
        {&Acts::t, hidden},
        {&Acts::g, 2 * size_t(c.inter)},  // gate | up
        {&Acts::h, size_t(c.inter)},
        {&Acts::logits, size_t(c.vocab)},
    };
    constexpr size_t kGrain = 64;  // floats: 256 bytes
    const auto padded = [](size_t n) { return (n + kGrain - 1) / kGrain * kGrain; };
    size_t total = padded(size_t(scratchInts(int(widest / 32))));
    for (const Slice& s : slices) total += padded(s.floats);

    std::vector<float> staged(total, 0.0f);
    host::SeedStream draw(seed | 1);
    for (size_t i = 0; i < hidden; ++i) staged[i] = draw.unit();  // x0 is the first slice

    float* base = static_cast<float*>(alloc.alloc(total * sizeof(float)));
    alloc.upload(base, staged.data(), total * sizeof(float));
    Acts a;
    size_t at = 0;
    for (const Slice& s : slices) {
        a.*s.field = base + at;
        at += padded(s.floats);
    }
    a.k = a.q + qd;
    a.v = a.k + kv;
    a.u = a.g + c.inter;
    a.xq = reinterpret_cast<int*>(base + at);
    return a;
}

// ---- a model from GGUF blocks on the host ---------------------------------------------------------------------
namespace {

class Uploader {
public:
    explicit Uploader(Allocator& alloc) : alloc_(alloc) {}

    template <class T>
    T* copyOf(const T* src, size_t n) {
        T* dst = static_cast<T*>(alloc_.alloc(n * sizeof(T)));
        alloc_.upload(dst, src, n * sizeof(T));
        return dst;
    }
    float* zeroed(size_t n) {
        zeros_.assign(n, 0.0f);
        return copyOf(zeros_.data(), n);
    }
    Mat matrix(const HostMat& h) {
        if (h.rows % 8 != 0 || h.k % 256 != 0) throw std::runtime_error("matrix shape not supported (rows % 8, k % 256)");
        const size_t bytes = ref::packedBytes(h.rows, h.k, h.q6);
        packed_.resize((bytes + sizeof(int) - 1) / sizeof(int));
        (h.q6 ? ref::repackQ6K : ref::repackQ4K)(h.blocks, h.rows, h.k, packed_.data());
        weight_bytes_ += int64_t(bytes);
        Mat m;
        m.rows = h.rows;
        m.k = h.k;
        m.format = h.q6 ? Weights::Q6K : Weights::Q4K;
        m.q = copyOf(reinterpret_cast<const uint8_t*>(packed_.data()), bytes);
        const int dims[2] = {h.rows, h.k};
        m.dims = copyOf(dims, 2);
        return m;
    }
    int64_t weightBytes() const { return weight_bytes_; }

private:
    Allocator& alloc_;
    std::vector<float> zeros_;
    std::vector<int> packed_;
    int64_t weight_bytes_ = 0;
};

void checkShapes(const Config& c) {
    const bool ok = c.head_dim % 8 == 0 && c.hidden % 256 == 0 && c.inter % 256 == 0 && c.kv_heads > 0 && c.heads % c.kv_heads == 0 && c.max_ctx >= 1;
    if (!ok) throw std::runtime_error("model shapes not supported");
}

}  // namespace

Model uploadModel(const HostModel& host, Allocator& alloc) {
    const Config& c = host.cfg;
    checkShapes(c);
    Uploader up(alloc);
    Model m;
    m.cfg = c;
    m.cfg.weights = Weights::Gguf;
    m.layers.reserve(host.layers.size());
    const size_t hidden = size_t(c.hidden), cache_row = size_t(c.kvStride());
    for (const HostLayer& h : host.layers) {
        Layer& L = m.layers.emplace_back();
        for (const HostMat* part : {&h.wq, &h.wk, &h.wv}) L.qkv_parts.push_back(up.matrix(*part));
        L.wo = up.matrix(h.wo);
        for (const HostMat* part : {&h.wg, &h.wu}) L.gu_parts.push_back(up.matrix(*part));
        L.wd = up.matrix(h.wd);
        L.attn_norm = up.copyOf(h.attn_norm, hidden);
        L.ffn_norm = up.copyOf(h.ffn_norm, hidden);
        if (c.qk_norm) {
            L.q_norm = up.copyOf(h.q_norm, size_t(c.head_dim));
            L.k_norm = up.copyOf(h.k_norm, size_t(c.head_dim));
        }
        L.k_cache = up.zeroed(cache_row * size_t(c.kStride()));
        L.v_cache = up.zeroed(cache_row * size_t(c.max_ctx));
    }
    m.out_norm = up.copyOf(host.out_norm, hidden);
    m.lm_head = up.matrix(host.lm_head);
    if (host.rope_ff) m.rope_ff = up.copyOf(host.rope_ff, size_t(c.head_dim / 2));
    const std::array<int, 7> dims = host::attnDimsInts(c.attnDims(c.max_ctx));
    m.attn_dims = up.copyOf(dims.data(), dims.size());
    m.cfg.file_weight_bytes = up.weightBytes();

    // Tied embeddings: a token's embedding is its row of the output matrix, expanded on the host from the caller's
    // own copy of the GGUF blocks -- a table lookup, where the reference does it too (llm/gguf_model.cpp:96-104).
    m.embed = [table = host.lm_head, width = c.hidden](int token, float* out) {
        if (token < 0 || token >= table.rows) throw std::out_of_range("token id outside the vocabulary");
        host::expandRow(table.blocks, table.q6, token, width, out);
    };
    return m;
}

}  // namespace llm
