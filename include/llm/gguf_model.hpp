// From a mapped GGUF file to a model the decode paths can run.
//
// Llama- and Qwen3-architecture files are understood: Q4_K / Q6_K weight matrices, f32 norm vectors, optional
// RoPE frequency factors, optional per-head q/k norms.  loadGguf(), ggufVocab() and tokenText() carry the names and
// signatures of the reference's llm/gguf_model.hpp, so its callers build unchanged; hostModel() is the extra step in
// between for callers that feed the graph decoder (kcb_decoder_create) rather than llm::decodeToken.
#pragma once

#include <string>
#include <vector>

#include "gguf.hpp"
#include "llm_model.hpp"

namespace llm {

// Describes the model without moving a byte: every matrix and vector of the result points into `file`'s mapping.
// Throws std::runtime_error for an architecture, a tensor type or a shape this project does not run.
HostModel hostModel(const gguf::File& file, int max_ctx);

// hostModel() followed by uploadModel(): weights go to the device through `alloc`.  Token embeddings stay in the
// file and are read per token, so `file` has to live as long as the returned model.
Model loadGguf(const gguf::File& file, int max_ctx, Allocator& alloc);

// The tokenizer's pieces in id order (empty when the file carries none), and one piece turned back into the bytes
// it stands for: GPT-2 byte-level BPE maps every byte to a printable code point, special tokens stay as written.
std::vector<std::string> ggufVocab(const gguf::File& file);
std::string tokenText(const std::vector<std::string>& vocab, int id);

}  // namespace llm
