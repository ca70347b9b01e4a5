// Helpers shared by the host-side files of the llm:: layer (not installed; the public headers are include/llm/*.hpp).
#pragma once

#include <llm_model.hpp>

#include <array>
#include <cstdint>
#include <string_view>

namespace llm::host {

// Throws std::runtime_error("<doing>: <error text> (<detail>)") unless status is Success.
void require(kc::Error status, std::string_view doing);

// The xorshift64 stream (13, 7, 17) the reference seeds its synthetic data from (llm/llm_model.cpp:138-147): the
// start vector of allocActs and the weights of buildModels are drawn from it, so equal seeds give equal bits.
class SeedStream {
public:
    explicit SeedStream(uint64_t seed) : state_(seed) {}
    uint64_t word();
    float unit();  // [-1, 1): the top 24 bits of a word
    float around(float center, float spread) { return center + spread * unit(); }

private:
    uint64_t state_;
};

// AttnDims in the order the attention kernels read it from device memory.
inline std::array<int, 7> attnDimsInts(const AttnDims& d) { return {d.n_heads, d.ctx, d.head_dim, d.kv_stride, d.group, d.ctx_pad, d.k_stride}; }

// Row `row` of a K-quant matrix (canonical GGUF blocks, `width` values per row) as floats, with the formats' own
// formulas: Q4_K d * sc * q - dmin * m, Q6_K d * sc * (q - 32).
void expandRow(const uint8_t* blocks, bool q6, int row, int width, float* out);

}  // namespace llm::host
