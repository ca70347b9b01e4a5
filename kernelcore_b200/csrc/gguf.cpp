// GGUF reader and model loader (llm/gguf.cpp, llm/gguf_model.cpp of the reference) on POSIX.
//
// File layout (GGUF v2 / v3, little endian): "GGUF", u32 version, u64 tensor count, u64 metadata count; metadata
// pairs {string key, u32 type, value}; tensor infos {string name, u32 n_dims, u64 dims[n], u32 type, u64 offset};
// padding to general.alignment (default 32); tensor data.  Strings are {u64 length, bytes}.  The file is mapped
// read-only and tensors point into the mapping.

#include "../../include/kernelcore_b200.h"
#include "../../include/llm/gguf_model.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <memory>
#include <stdexcept>

namespace llm::gguf {

const char* typeName(uint32_t t) {
    switch (t) {
    case 0: return "F32";
    case 1: return "F16";
    case 2: return "Q4_0";
    case 8: return "Q8_0";
    case 12: return "Q4_K";
    case 13: return "Q5_K";
    case 14: return "Q6_K";
    default: return "?";
    }
}

bool blockInfo(uint32_t t, size_t* block_bytes, size_t* block_values) {
    size_t b = 0, v = 0;
    switch (t) {
    case 0: b = 4, v = 1; break;
    case 1: b = 2, v = 1; break;
    case 2: b = 18, v = 32; break;
    case 8: b = 34, v = 32; break;
    case 12: b = 144, v = 256; break;
    case 13: b = 176, v = 256; break;
    case 14: b = 210, v = 256; break;
    default: return false;
    }
    if (block_bytes) *block_bytes = b;
    if (block_values) *block_values = v;
    return true;
}

namespace {

struct Cursor {
    const uint8_t* p;
    const uint8_t* end;
    template <class T>
    T take() {
        if (static_cast<size_t>(end - p) < sizeof(T)) throw std::runtime_error("GGUF file truncated");
        T v;
        std::memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = take<uint64_t>();
        if (n > static_cast<uint64_t>(end - p)) throw std::runtime_error("GGUF string runs past the end of the file");
        std::string s(reinterpret_cast<const char*>(p), static_cast<size_t>(n));
        p += n;
        return s;
    }
};

double scalar(Cursor& c, uint32_t type) {
    switch (type) {
    case 0: return c.take<uint8_t>();
    case 1: return c.take<int8_t>();
    case 2: return c.take<uint16_t>();
    case 3: return c.take<int16_t>();
    case 4: return c.take<uint32_t>();
    case 5: return c.take<int32_t>();
    case 6: return c.take<float>();
    case 7: return c.take<uint8_t>() ? 1.0 : 0.0;
    case 10: return static_cast<double>(c.take<uint64_t>());
    case 11: return static_cast<double>(c.take<int64_t>());
    case 12: return c.take<double>();
    default: throw std::runtime_error("GGUF metadata type not supported: " + std::to_string(type));
    }
}

Value value(Cursor& c, uint32_t type) {
    Value v;
    if (type == 8) {
        v.str = c.str();
    } else if (type == 9) {
        const uint32_t item = c.take<uint32_t>();
        const uint64_t n = c.take<uint64_t>();
        if (item == 9) throw std::runtime_error("nested GGUF arrays are not supported");
        for (uint64_t i = 0; i < n; ++i) {
            if (item == 8) v.strs.push_back(c.str());
            else v.nums.push_back(scalar(c, item));
        }
    } else {
        v.num = scalar(c, type);
    }
    return v;
}

}  // namespace

File::File(const std::string& path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error("cannot open " + path);
    struct stat st;
    if (::fstat(fd_, &st) != 0 || st.st_size < 24) {
        ::close(fd_);
        throw std::runtime_error("not a GGUF file: " + path);
    }
    size_ = static_cast<size_t>(st.st_size);
    void* m = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (m == MAP_FAILED) {
        ::close(fd_);
        throw std::runtime_error("cannot map " + path);
    }
    base_ = static_cast<const uint8_t*>(m);
    try {
        Cursor c{base_, base_ + size_};
        if (std::memcmp(c.p, "GGUF", 4) != 0) throw std::runtime_error("not a GGUF file: " + path);
        c.p += 4;
        const uint32_t version = c.take<uint32_t>();
        if (version < 2) throw std::runtime_error("GGUF version not supported: " + std::to_string(version));  // (as llm/gguf.cpp:95)
        const uint64_t n_tensors = c.take<uint64_t>(), n_meta = c.take<uint64_t>();
        for (uint64_t i = 0; i < n_meta; ++i) {
            std::string key = c.str();
            const uint32_t type = c.take<uint32_t>();
            meta_[key] = value(c, type);
        }
        std::vector<Tensor> order;
        for (uint64_t i = 0; i < n_tensors; ++i) {
            Tensor t;
            t.name = c.str();
            const uint32_t nd = c.take<uint32_t>();
            if (nd == 0 || nd > 4) throw std::runtime_error("tensor rank not supported: " + t.name);
            for (uint32_t d = 0; d < nd; ++d) {
                const uint64_t n = c.take<uint64_t>();
                if (n == 0 || n > (uint64_t(1) << 40)) throw std::runtime_error("tensor extent out of range: " + t.name);
                t.ne.push_back(static_cast<int64_t>(n));
            }
            t.type = c.take<uint32_t>();
            t.offset = c.take<uint64_t>();
            // A type this reader has no block size for (BF16, Q5_0, Q3_K, ...) stays in the list with bytes = 0 and no
            // data pointer, as the reference lists it (llm/gguf.cpp:126-130): the file opens, the tensor cannot be read.
            size_t bb = 0, bv = 0;
            t.bytes = 0;
            if (blockInfo(t.type, &bb, &bv)) {
                if (t.ne[0] % static_cast<int64_t>(bv)) throw std::runtime_error("row length is not a whole number of blocks: " + t.name);
                unsigned __int128 bytes = static_cast<unsigned __int128>(t.ne[0] / static_cast<int64_t>(bv)) * bb;
                for (uint32_t d = 1; d < nd; ++d) {
                    bytes *= static_cast<uint64_t>(t.ne[d]);
                    if (bytes > size_) throw std::runtime_error("tensor is larger than the file: " + t.name);
                }
                if (bytes > size_) throw std::runtime_error("tensor is larger than the file: " + t.name);
                t.bytes = static_cast<size_t>(bytes);
            }
            order.push_back(std::move(t));
        }
        const auto al = meta_.find("general.alignment");
        const double want = al != meta_.end() ? al->second.num : 32.0;
        if (!(want >= 1.0 && want <= 65536.0)) throw std::runtime_error("general.alignment out of range");
        const size_t align = static_cast<size_t>(want);
        if (align & (align - 1)) throw std::runtime_error("general.alignment is not a power of two");
        const size_t header = static_cast<size_t>(c.p - base_);
        const size_t data0 = (header + align - 1) / align * align;
        if (data0 > size_ && !order.empty()) throw std::runtime_error("the file ends inside its header");
        for (Tensor& t : order) {
            if (t.bytes != 0) {  // (written so that no sum of file-controlled numbers can wrap)
                const size_t room = data0 <= size_ ? size_ - data0 : 0;
                if (t.offset > room || t.bytes > room - t.offset) throw std::runtime_error("tensor data runs past the end of the file: " + t.name);
                t.data = base_ + data0 + t.offset;
            }
            tensors_[t.name] = t;
        }
    } catch (...) {
        ::munmap(const_cast<uint8_t*>(base_), size_);
        ::close(fd_);
        throw;
    }
}

File::~File() {
    if (base_) ::munmap(const_cast<uint8_t*>(base_), size_);
    if (fd_ >= 0) ::close(fd_);
}

const Tensor* File::find(const std::string& name) const {
    const auto it = tensors_.find(name);
    return it == tensors_.end() ? nullptr : &it->second;
}
const Tensor& File::tensor(const std::string& name) const {
    const Tensor* t = find(name);
    if (!t) throw std::runtime_error("tensor missing: " + name);
    return *t;
}
double File::num(const std::string& key) const {
    const auto it = meta_.find(key);
    if (it == meta_.end()) throw std::runtime_error("metadata missing: " + key);
    return it->second.num;
}
double File::num(const std::string& key, double fallback) const {
    const auto it = meta_.find(key);
    return it == meta_.end() ? fallback : it->second.num;
}
std::string File::str(const std::string& key) const {
    const auto it = meta_.find(key);
    if (it == meta_.end()) throw std::runtime_error("metadata missing: " + key);
    return it->second.str;
}

}  // namespace llm::gguf

namespace llm {
namespace {

using gguf::Tensor;

const float* floats(const Tensor& t, int64_t n) {
    if (t.type != 0 || t.cols() * t.rows() != n) throw std::runtime_error("expected an f32 tensor of " + std::to_string(n) + " values: " + t.name);
    if (reinterpret_cast<uintptr_t>(t.data) % 4) throw std::runtime_error("misaligned f32 tensor: " + t.name);
    return reinterpret_cast<const float*>(t.data);
}

HostMat matrix(const Tensor& t, int rows, int k, int64_t* file_bytes) {
    if (t.rows() != rows || t.cols() != k) throw std::runtime_error("unexpected matrix shape: " + t.name);
    if (rows % 8 || k % 256) throw std::runtime_error("matrix shape not supported: " + t.name);
    if (t.type != static_cast<uint32_t>(gguf::Type::Q4_K) && t.type != static_cast<uint32_t>(gguf::Type::Q6_K))
        throw std::runtime_error(std::string("matrix type not supported: ") + t.name + " " + gguf::typeName(t.type));
    *file_bytes += static_cast<int64_t>(t.bytes);
    return HostMat{t.data, rows, k, t.type == static_cast<uint32_t>(gguf::Type::Q6_K)};
}

}  // namespace

HostModel hostModel(const gguf::File& f, int max_ctx) {
    const std::string arch = f.str("general.architecture");
    if (arch != "llama" && arch != "qwen3") throw std::runtime_error("only llama- and qwen3-architecture GGUF files");
    HostModel h;
    Config& c = h.cfg;
    const auto it = f.meta().find("general.name");
    c.name = it == f.meta().end() ? arch : it->second.str;
    c.hidden = static_cast<int>(f.num(arch + ".embedding_length"));
    c.inter = static_cast<int>(f.num(arch + ".feed_forward_length"));
    c.layers = static_cast<int>(f.num(arch + ".block_count"));
    c.heads = static_cast<int>(f.num(arch + ".attention.head_count"));
    c.kv_heads = static_cast<int>(f.num(arch + ".attention.head_count_kv", c.heads));
    c.head_dim = static_cast<int>(f.num(arch + ".attention.key_length", c.heads ? c.hidden / c.heads : 0));
    c.eps = static_cast<float>(f.num(arch + ".attention.layer_norm_rms_epsilon", 1e-5));
    c.rope_base = static_cast<float>(f.num(arch + ".rope.freq_base", 10000.0));
    c.neox = arch == "qwen3";  // llama.cpp rotates Qwen pairs (i, i + head_dim / 2)
    const Tensor& emb = f.tensor("token_embd.weight");
    c.vocab = static_cast<int>(emb.rows());
    c.max_ctx = max_ctx;
    c.weights = Weights::Gguf;
    if (c.layers <= 0 || c.heads <= 0 || c.kv_heads <= 0 || c.head_dim % 8 || c.hidden % 256 || c.inter % 256 || max_ctx <= 0)
        throw std::runtime_error("model shapes not supported");
    c.qk_norm = f.find("blk.0.attn_q_norm.weight") != nullptr;
    const int qd = c.heads * c.head_dim, kv = c.kv_heads * c.head_dim;
    int64_t bytes = 0;
    for (int l = 0; l < c.layers; ++l) {
        const std::string p = "blk." + std::to_string(l) + ".";
        HostLayer L{};
        L.wq = matrix(f.tensor(p + "attn_q.weight"), qd, c.hidden, &bytes);
        L.wk = matrix(f.tensor(p + "attn_k.weight"), kv, c.hidden, &bytes);
        L.wv = matrix(f.tensor(p + "attn_v.weight"), kv, c.hidden, &bytes);
        L.wo = matrix(f.tensor(p + "attn_output.weight"), c.hidden, qd, &bytes);
        L.wg = matrix(f.tensor(p + "ffn_gate.weight"), c.inter, c.hidden, &bytes);
        L.wu = matrix(f.tensor(p + "ffn_up.weight"), c.inter, c.hidden, &bytes);
        L.wd = matrix(f.tensor(p + "ffn_down.weight"), c.hidden, c.inter, &bytes);
        L.attn_norm = floats(f.tensor(p + "attn_norm.weight"), c.hidden);
        L.ffn_norm = floats(f.tensor(p + "ffn_norm.weight"), c.hidden);
        if (c.qk_norm) {
            L.q_norm = floats(f.tensor(p + "attn_q_norm.weight"), c.head_dim);
            L.k_norm = floats(f.tensor(p + "attn_k_norm.weight"), c.head_dim);
        }
        h.layers.push_back(L);
    }
    h.out_norm = floats(f.tensor("output_norm.weight"), c.hidden);
    const Tensor* out = f.find("output.weight");
    h.lm_head = matrix(out ? *out : emb, c.vocab, c.hidden, &bytes);  // tied embeddings when there is no output.weight
    const Tensor* rf = f.find("rope_freqs.weight");
    h.rope_ff = rf ? floats(*rf, c.head_dim / 2) : nullptr;
    c.file_weight_bytes = bytes;
    return h;
}

Model loadGguf(const gguf::File& f, int max_ctx, Allocator& alloc) { return uploadModel(hostModel(f, max_ctx), alloc); }

std::vector<std::string> ggufVocab(const gguf::File& f) {
    const auto it = f.meta().find("tokenizer.ggml.tokens");
    return it == f.meta().end() ? std::vector<std::string>{} : it->second.strs;
}

// GPT-2 byte-level BPE writes every byte as a printable code point: the printable Latin-1 bytes as themselves, the
// rest as U+0100 + n in order of appearance.  Undo that; pieces that are not in that alphabet (special tokens) stay.
std::string tokenText(const std::vector<std::string>& vocab, int id) {
    if (id < 0 || id >= static_cast<int>(vocab.size())) return "<" + std::to_string(id) + ">";
    static const std::map<uint32_t, uint8_t> back = [] {
        std::map<uint32_t, uint8_t> m;
        int n = 0;
        for (int b = 0; b < 256; ++b) {
            const bool printable = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
            m[printable ? static_cast<uint32_t>(b) : 256u + static_cast<uint32_t>(n++)] = static_cast<uint8_t>(b);
        }
        return m;
    }();
    const std::string& piece = vocab[static_cast<size_t>(id)];
    std::string out;
    for (size_t i = 0; i < piece.size();) {
        const uint8_t c0 = static_cast<uint8_t>(piece[i]);
        uint32_t cp = c0;
        size_t len = 1;
        if (c0 >= 0xC0 && c0 < 0xE0 && i + 1 < piece.size()) cp = ((c0 & 0x1Fu) << 6) | (static_cast<uint8_t>(piece[i + 1]) & 0x3Fu), len = 2;
        else if (c0 >= 0xE0) return piece;  // outside the byte alphabet: a special token, keep as written
        const auto it = back.find(cp);
        if (it == back.end()) return piece;
        out.push_back(static_cast<char>(it->second));
        i += len;
    }
    return out;
}

}  // namespace llm

// ---- C view ----------------------------------------------------------------------------------------------------
namespace {
// status codes of the C ABI (kc::Error values, include/kernelcore/api.hpp); this file is plain host code
constexpr int kSuccess = 0, kInvalidValue = 2, kInternalError = 15;
struct OpenGguf {
    std::unique_ptr<llm::gguf::File> file;
    llm::HostModel host;
    std::vector<kcb_layer> layers;
};
thread_local std::string tl_gguf_err;
kcb_mat c_mat(const llm::HostMat& m) { return kcb_mat{m.blocks, m.rows, m.k, m.q6 ? 6 : 4}; }
}  // namespace

extern "C" {

int kcb_gguf_open(const char* path, int max_ctx, void** out, kcb_model_desc* desc) {
    if (!path || !out || !desc) return kInvalidValue;
    *out = nullptr;
    try {
        auto g = std::make_unique<OpenGguf>();
        g->file = std::make_unique<llm::gguf::File>(path);
        g->host = llm::hostModel(*g->file, max_ctx);
        const llm::Config& c = g->host.cfg;
        for (const llm::HostLayer& L : g->host.layers)
            g->layers.push_back(kcb_layer{c_mat(L.wq), c_mat(L.wk), c_mat(L.wv), c_mat(L.wo), c_mat(L.wg), c_mat(L.wu), c_mat(L.wd), L.attn_norm,
                                          L.ffn_norm, L.q_norm, L.k_norm});
        std::memset(desc, 0, sizeof *desc);
        desc->hidden = c.hidden, desc->inter = c.inter, desc->n_layers = c.layers, desc->heads = c.heads, desc->kv_heads = c.kv_heads;
        desc->head_dim = c.head_dim, desc->vocab = c.vocab, desc->max_ctx = c.max_ctx, desc->eps = c.eps, desc->rope_base = c.rope_base;
        desc->neox = c.neox, desc->qk_norm = c.qk_norm;
        desc->layers = g->layers.data(), desc->out_norm = g->host.out_norm, desc->lm_head = c_mat(g->host.lm_head), desc->rope_ff = g->host.rope_ff;
        *out = g.release();
    } catch (const std::exception& e) {
        tl_gguf_err = e.what();
        return kInternalError;
    }
    return kSuccess;
}
long long kcb_gguf_weight_bytes(void* h) { return h ? static_cast<OpenGguf*>(h)->host.cfg.file_weight_bytes : 0; }
int kcb_gguf_close(void* h) {
    delete static_cast<OpenGguf*>(h);
    return kSuccess;
}
const char* kcb_gguf_last_error(void) { return tl_gguf_err.c_str(); }

}  // extern "C"
