// A bounds-checked GGUF v2/v3 reader over a memory-mapped file.
//
// It accepts and rejects the same files as the reference's parser
// (crates/bobcat-gguf/src/lib.rs:316-344, :517-751): magic and version, metadata entries with
// every value type, duplicate keys and tensor names, 1 to 4 dimensions, whole quantisation blocks
// per row, aligned offsets, data inside the file.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "common.h"

namespace bc {

// Tensor types this library reads; ids are ggml's (crates/bobcat-gguf/src/lib.rs:126-152).
enum TensorType : uint32_t { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q8_0 = 8, T_Q4K = 12, T_Q5K = 13, T_Q6K = 14, T_BF16 = 30 };

// Elements and bytes of one block (lib.rs:156-166). Returns false for unknown ids.
bool type_block(uint32_t type, uint64_t* elements, uint64_t* bytes);
uint64_t type_row_bytes(uint32_t type, uint64_t n_cols);

struct GgufTensor {
    std::string name;
    uint32_t type = 0;
    std::vector<uint64_t> shape;  // innermost first
    uint64_t offset = 0;          // byte offset inside the file
    uint64_t n_bytes = 0;
};

struct GgufValue {
    uint32_t type = 0;        // GGUF value type id
    uint64_t scalar_bits = 0; // fixed-size values, little-endian bits
    uint64_t start = 0, len = 0;  // strings: byte range; arrays: payload range
    uint32_t element = 0;     // arrays: element type
    uint64_t count = 0;       // arrays: element count
};

class Gguf {
  public:
    Gguf() = default;
    ~Gguf();
    Gguf(const Gguf&) = delete;
    Gguf& operator=(const Gguf&) = delete;

    // Map and parse `path`. BC_ERR_IO when the file cannot be opened, BC_ERR_GGUF when malformed.
    bc_status open(const char* path);
    // Parse bytes the caller owns (for tests of malformed input). The bytes must outlive this.
    bc_status parse(const uint8_t* bytes, size_t len);

    const uint8_t* bytes() const { return bytes_; }
    size_t size() const { return size_; }

    bool u32(const std::string& key, uint32_t* out) const;
    bool f32(const std::string& key, float* out) const;
    bool string(const std::string& key, std::string* out) const;
    bool array_len(const std::string& key, uint64_t* out) const;
    bool array_u32(const std::string& key, uint64_t index, uint32_t* out) const;
    const GgufTensor* tensor(const std::string& name) const;
    const uint8_t* data(const GgufTensor& t) const { return bytes_ + t.offset; }

  private:
    const uint8_t* bytes_ = nullptr;
    size_t size_ = 0;
    void* mapping_ = nullptr;
    size_t mapping_len_ = 0;
    std::map<std::string, GgufValue> metadata_;
    std::map<std::string, GgufTensor> tensors_;
};

}  // namespace bc
