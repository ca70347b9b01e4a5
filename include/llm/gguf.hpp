// GGUF model files (llama.cpp / Ollama), read-only.
//
// A File maps the whole file with POSIX mmap and indexes two things: the key/value metadata and the tensor
// directory.  Tensor::data points straight into the mapping, so a tensor's bytes are never copied on the host and a
// File has to outlive everything that was handed one of its pointers.
//
// The names below (namespace, Type, Tensor, Value, File and its accessors) are the ones the reference's reader
// declares in llm/gguf.hpp, so code written against that header (app/llm_real.cpp) compiles against this one.
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace llm::gguf {

// ggml's numeric tensor-type codes, as far as Llama-family files use them.
enum class Type : uint32_t {
    F32 = 0,
    F16 = 1,
    Q4_0 = 2,
    Q8_0 = 8,
    Q4_K = 12,  // 144 bytes per 256 values
    Q5_K = 13,
    Q6_K = 14,  // 210 bytes per 256 values
};

// Printable name of a type code ("Q4_K", "F32", ... or "?" for codes outside the enum).
const char* typeName(uint32_t type_code);

// Block geometry of a type code: bytes per block and values per block.  False for codes this reader cannot size.
bool blockInfo(uint32_t type_code, size_t* block_bytes, size_t* block_values);

// One entry of the tensor directory.
struct Tensor {
    std::string name;
    // Extents, fastest-varying first: ne[0] values are contiguous (a row), ne[1] counts rows, and so on.
    std::vector<int64_t> ne;
    uint32_t type = 0;              // a Type code
    uint64_t offset = 0;            // where the tensor starts, counted from the beginning of the data section
    const uint8_t* data = nullptr;  // the same place inside the mapping
    size_t bytes = 0;               // size in the file

    int64_t cols() const { return ne.empty() ? 0 : ne[0]; }
    int64_t rows() const { return ne.size() < 2 ? 1 : ne[1]; }
};

// One metadata value.  Scalars of any integer, float or bool type land in `num`, strings in `str`; an array fills
// `nums` or `strs` depending on its element type.
struct Value {
    std::string str;
    double num = 0;
    std::vector<std::string> strs;
    std::vector<double> nums;
};

class File {
public:
    // Maps and indexes `path`; std::runtime_error for a missing file, a bad magic, an unsupported version or a
    // directory entry that points outside the file.
    explicit File(const std::string& path);
    ~File();
    File(const File&) = delete;
    File& operator=(const File&) = delete;

    // Tensor directory.
    const std::map<std::string, Tensor>& tensors() const { return tensors_; }
    const Tensor* find(const std::string& name) const;    // nullptr when absent
    const Tensor& tensor(const std::string& name) const;  // std::runtime_error when absent

    // Metadata.
    const std::map<std::string, Value>& meta() const { return meta_; }
    double num(const std::string& key) const;  // std::runtime_error when absent
    double num(const std::string& key, double fallback) const;
    std::string str(const std::string& key) const;  // std::runtime_error when absent

private:
    std::map<std::string, Tensor> tensors_;
    std::map<std::string, Value> meta_;
    const uint8_t* base_ = nullptr;  // start of the mapping
    size_t size_ = 0;                // its length
    int fd_ = -1;
};

}  // namespace llm::gguf
