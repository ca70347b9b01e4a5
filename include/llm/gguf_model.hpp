#pragma once

// Loads a Llama- or Qwen3-architecture GGUF model (Q4_K / Q6_K matrices, f32 norms) for the decode loop.
// Interface of the reference's llm/gguf_model.hpp:1-24; hostModel() is the step before the upload, for callers that
// feed the graph decoder (kcb_decoder_create) instead of llm::decodeToken.

#include "gguf.hpp"
#include "llm_model.hpp"

#include <string>
#include <vector>

namespace llm {

// Matrices and norm vectors as pointers into the mapped file; the file must outlive the result.
HostModel hostModel(const gguf::File& f, int max_ctx);
// The file must outlive the model (token embeddings are read from it on demand).
Model loadGguf(const gguf::File& f, int max_ctx, Allocator& alloc);

// Token text: GPT-2 byte-level BPE pieces mapped back to bytes (special tokens as written).
std::vector<std::string> ggufVocab(const gguf::File& f);
std::string              tokenText(const std::vector<std::string>& vocab, int id);

}  // namespace llm
