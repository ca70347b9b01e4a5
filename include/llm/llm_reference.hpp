// llm_reference.hpp -- host-side weight packing for the CUDA kernels.
//
// The reference's llm/llm_reference.hpp is its CPU mirror of every kernel (the test oracle) plus the
// repack functions its loaders call.  This build keeps only what the product path needs on the host --
// the packers, under the reference's names and signatures -- because there is no CPU execution path
// here; the oracle lives outside the product, under oracle/.
#pragma once

#include <cstddef>
#include <cstdint>

namespace llm::ref {

// GGUF Q4_K blocks -> the device layout of matvec_q4k_q8 / matmul_q4k_*: the blocks themselves, copied
// (rows * k / 256 * 36 ints).  The reference's repackQ4K (llm/llm_reference.cpp:385-398) builds an 8-row
// interleaved stream of 37 ints per block instead, so a buffer sized for the reference always suffices.
void repackQ4K(const uint8_t* src, int rows, int k, int* qw);
// GGUF Q6_K blocks -> four planes ql | qh | scales | d (rows * k / 256 * 210 bytes, i.e. 52.5 ints per
// block against the reference's 53, llm/llm_reference.cpp:400-411).
void repackQ6K(const uint8_t* src, int rows, int k, int* qw);
// The inverse of repackQ6K (canonical GGUF bytes back, for get_tensor).
void unpackQ6K(const int* qw, int rows, int k, uint8_t* dst);

inline size_t packedBytes(int rows, int k, bool q6) { return size_t(rows) * size_t(k / 256) * (q6 ? 210 : 144); }

}  // namespace llm::ref
