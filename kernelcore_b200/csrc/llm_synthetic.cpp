// llm::buildModels: random-weight models in the synthetic formats (Q8, Q4, Q4X8, Q4X8Q8).
//
// The values are the reference's for the same seed (llm/llm_model.cpp:175-254), because its benchmark and its tiny-model
// test compare logits across builds.  What fixes them is the order in which the seed stream is consumed, which this
// file keeps: per matrix the quantized bytes (eight per stream word, low byte first; Q8 never -128) and then one scale
// per 32 weights around 1 / sqrt(var * k) +- 10 % -- var being the variance of the stored integers, so that y = W x has
// about unit variance; per layer q|k|v, wo, gate|up, down, the two norm weight vectors (1 +- 0.1) and the K and V
// caches (uniform in [-1, 1), so a step at any position attends over defined data); last the output norm and lm_head.
#include <llm_model.hpp>

#include "llm_host.hpp"

#include <cmath>
#include <cstring>
#include <stdexcept>

namespace llm {
namespace {

// One host buffer copied into every allocator; element i of the result lives in allocator i.
template <class T>
std::vector<T*> replicate(const std::vector<Allocator*>& allocs, const T* data, size_t count) {
    std::vector<T*> copies;
    copies.reserve(allocs.size());
    for (Allocator* a : allocs) {
        T* p = static_cast<T*>(a->alloc(count * sizeof(T)));
        a->upload(p, data, count * sizeof(T));
        copies.push_back(p);
    }
    return copies;
}
template <class T>
std::vector<T*> replicate(const std::vector<Allocator*>& allocs, const std::vector<T>& v) {
    return replicate(allocs, v.data(), v.size());
}

class Synthesizer {
public:
    Synthesizer(uint64_t seed, const std::vector<Allocator*>& allocs) : draw_(seed | 1), allocs_(allocs) {}

    std::vector<float*> vector(size_t n, float center, float spread) {
        std::vector<float> v(n);
        for (float& f : v) f = draw_.around(center, spread);
        return replicate(allocs_, v);
    }

    // One matrix per allocator, all with the same values.
    std::vector<Mat> matrix(int rows, int k, Weights format) {
        const bool bytes_per_weight = format == Weights::Q8;
        const bool by_eight = format == Weights::Q4X8 || format == Weights::Q4X8Q8;
        if (by_eight && rows % 8 != 0) throw std::invalid_argument(std::string(weightsName(format)) + " needs a multiple of 8 rows");
        const size_t weights = size_t(rows) * size_t(k);

        std::vector<uint8_t> q(bytes_per_weight ? weights : weights / 2);
        for (size_t at = 0; at < q.size(); at += 8) {
            uint64_t bits = draw_.word();
            for (size_t j = at; j < std::min(at + 8, q.size()); ++j, bits >>= 8) q[j] = uint8_t(bits);
        }
        float variance = 21.25f;  // nibble - 8, uniform over -8..7
        if (bytes_per_weight) {
            for (uint8_t& b : q) b = b == 0x80 ? 0x81 : b;  // int8 uniform over -127..127
            variance = 127.0f * 127.0f / 3.0f;
        }
        const float base = 1.0f / std::sqrt(variance * static_cast<float>(k));
        std::vector<float> scales(weights / 32);
        const float spread = 0.1f * base;
        for (float& s : scales) s = draw_.around(base, spread);

        const int dims[2] = {rows, k};
        const std::vector<int*> dims_dev = replicate(allocs_, dims, 2);
        std::vector<const void*> q_dev;
        std::vector<float*> s_dev(allocs_.size(), nullptr);
        if (format == Weights::Q4X8Q8) {
            for (int* p : replicate(allocs_, wordsByEight(q, scales, rows, k))) q_dev.push_back(p);
        } else {
            if (format == Weights::Q4X8) bytesByEight(q, scales, rows, k);
            for (uint8_t* p : replicate(allocs_, q)) q_dev.push_back(p);
            s_dev = replicate(allocs_, scales);
        }
        std::vector<Mat> out(allocs_.size());
        for (size_t i = 0; i < out.size(); ++i) {
            out[i].rows = rows, out[i].k = k, out[i].format = format;
            out[i].q = q_dev[i], out[i].s = s_dev[i], out[i].dims = dims_dev[i];
        }
        return out;
    }

private:
    // The 8-row interleaved layouts.  Rows are taken in groups of eight; block b (32 weights, 16 bytes) of the eight rows
    // of group g is stored together as "group block" g * (k / 32) + b.
    //   Q4X8:   16 x 8 bytes, byte j of row l at [j * 8 + l]; the eight scales of a group block side by side.
    //   Q4X8Q8: 40 ints: word w (bytes 4w..4w+3) of row l at [w * 8 + l], then the eight scales as bit patterns.
    static void bytesByEight(std::vector<uint8_t>& q, std::vector<float>& scales, int rows, int k) {
        const size_t nb = size_t(k / 32);
        std::vector<uint8_t> q8(q.size());
        std::vector<float> s8(scales.size());
        for (size_t row = 0; row < size_t(rows); ++row)
            for (size_t b = 0; b < nb; ++b) {
                const size_t group_block = row / 8 * nb + b, lane = row % 8;
                const uint8_t* src = q.data() + (row * nb + b) * 16;
                for (size_t j = 0; j < 16; ++j) q8[group_block * 128 + j * 8 + lane] = src[j];
                s8[group_block * 8 + lane] = scales[row * nb + b];
            }
        q.swap(q8);
        scales.swap(s8);
    }
    static std::vector<int> wordsByEight(const std::vector<uint8_t>& q, const std::vector<float>& scales, int rows, int k) {
        const size_t nb = size_t(k / 32);
        std::vector<int> out(size_t(rows) * nb * 5);
        for (size_t row = 0; row < size_t(rows); ++row)
            for (size_t b = 0; b < nb; ++b) {
                int* group_block = out.data() + (row / 8 * nb + b) * 40;
                const size_t lane = row % 8;
                for (size_t w = 0; w < 4; ++w) std::memcpy(group_block + w * 8 + lane, q.data() + (row * nb + b) * 16 + 4 * w, 4);
                std::memcpy(group_block + 32 + lane, &scales[row * nb + b], 4);
            }
        return out;
    }

    host::SeedStream draw_;
    const std::vector<Allocator*>& allocs_;
};

void checkSynthetic(const Config& c) {
    const int qd = c.heads * c.head_dim;
    const bool ok = c.hidden % 32 == 0 && c.inter % 32 == 0 && qd % 32 == 0 && c.head_dim % 8 == 0 && c.kv_heads > 0 && c.heads % c.kv_heads == 0 &&
                    c.max_ctx >= 1 && c.layers >= 1;
    if (!ok) throw std::invalid_argument("model shapes must be multiples of 32 with heads divisible by kv_heads");
    switch (c.weights) {
    case Weights::Q8:
    case Weights::Q4:
    case Weights::Q4X8:
    case Weights::Q4X8Q8: return;
    default: throw std::invalid_argument("buildModels makes the synthetic formats only (Q8, Q4, Q4X8, Q4X8Q8)");
    }
}

}  // namespace

void buildModels(const Config& c, uint64_t seed, const std::vector<Allocator*>& allocs, std::vector<Model>& out) {
    checkSynthetic(c);
    out.assign(allocs.size(), Model{});
    for (Model& m : out) {
        m.cfg = c;
        m.layers.resize(size_t(c.layers));
    }
    Synthesizer make(seed, allocs);
    const int qd = c.heads * c.head_dim, kv = c.kvStride();
    const size_t hidden = size_t(c.hidden);
    // `field` of layer `l` of every model <- the copy in that model's allocator
    const auto place = [&out](int l, auto Layer::*field, const auto& copies) {
        for (size_t i = 0; i < out.size(); ++i) out[i].layers[size_t(l)].*field = copies[i];
    };
    for (int l = 0; l < c.layers; ++l) {  // the order of these draws is part of the format (see the file header)
        place(l, &Layer::wqkv, make.matrix(qd + 2 * kv, c.hidden, c.weights));
        place(l, &Layer::wo, make.matrix(c.hidden, qd, c.weights));
        place(l, &Layer::wgu, make.matrix(2 * c.inter, c.hidden, c.weights));
        place(l, &Layer::wd, make.matrix(c.hidden, c.inter, c.weights));
        place(l, &Layer::attn_norm, make.vector(hidden, 1.0f, 0.1f));
        place(l, &Layer::ffn_norm, make.vector(hidden, 1.0f, 0.1f));
        place(l, &Layer::k_cache, make.vector(size_t(c.kStride()) * size_t(kv), 0.0f, 1.0f));
        place(l, &Layer::v_cache, make.vector(size_t(c.max_ctx) * size_t(kv), 0.0f, 1.0f));
    }
    const std::vector<float*> out_norm = make.vector(hidden, 1.0f, 0.1f);
    const std::vector<Mat> head = make.matrix(c.vocab, c.hidden, c.weights);
    const std::array<int, 7> dims = host::attnDimsInts(c.attnDims(c.max_ctx));
    const std::vector<int*> dims_dev = replicate(allocs, dims.data(), dims.size());
    for (size_t i = 0; i < out.size(); ++i) {
        out[i].out_norm = out_norm[i];
        out[i].lm_head = head[i];
        out[i].attn_dims = dims_dev[i];
    }
}

}  // namespace llm
