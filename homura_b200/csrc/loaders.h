// Host-side checkpoint readers: config.json, safetensors, GGUF.
// Mirrors what Homura's loaders accept on the decode path:
//   TransformerConfig       src/hf/config.rs:11-73
//   load_safetensors_bf16   src/hf/safetensors.rs:31-96
//   GgufFile                src/gguf.rs:345-450, 508-582
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/homura_b200.h"

namespace hm {

// Read-only memory map of a file.
class MappedFile {
   public:
    MappedFile() = default;
    ~MappedFile();
    MappedFile(const MappedFile&) = delete;
    MappedFile& operator=(const MappedFile&) = delete;
    bool open(const std::string& path, std::string* err);
    const uint8_t* data() const { return data_; }
    size_t size() const { return size_; }

   private:
    uint8_t* data_ = nullptr;
    size_t size_ = 0;
};

struct TensorView {
    std::string name;
    int dtype = -1;               // hm_dtype
    std::vector<int64_t> shape;   // outermost first
    const uint8_t* data = nullptr;
    size_t nbytes = 0;
};

// ---- minimal JSON (objects, arrays, strings, numbers, true/false/null) -----------------
struct Json {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;
    const Json* get(const std::string& key) const;
};
bool json_parse(const char* text, size_t len, Json* out, std::string* err);

// config.json -> hm_config (defaults: eps 1e-6, theta 1e4, max_pos 2048, src/hf/config.rs:39-47).
bool parse_config_json(const std::string& path, hm_config* cfg, std::string* err);

// safetensors: 8-byte LE header length + JSON header + data.  Views point into `file`.
bool parse_safetensors(const MappedFile& file, std::vector<TensorView>* out, std::string* err);

// GGUF v2/v3.
struct GgufValue {
    enum Kind { None, UInt, Int, Float, Bool, Str, Arr } kind = None;
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0.0;
    bool b = false;
    std::string s;
    uint64_t arr_len = 0;  // arrays are skipped; only their length is kept (vocab fallback)
    bool as_u64(uint64_t* out) const;
    bool as_f32(float* out) const;
};
struct GgufFile {
    uint32_t version = 0;
    std::map<std::string, GgufValue> metadata;
    std::vector<TensorView> tensors;  // dtype = hm_dtype or -1 when the ggml type is unsupported
    std::vector<uint32_t> ggml_types;
    const TensorView* find(const std::string& name) const;
};
bool parse_gguf(const MappedFile& file, GgufFile* out, std::string* err);
// <arch>.* keys -> hm_config (src/gguf.rs:508-582).
bool gguf_config(const GgufFile& g, hm_config* cfg, std::string* err);

// ggml type table (src/gguf.rs:112-164): elements per block, bytes per block; 0 if unknown.
void ggml_type_geometry(uint32_t ggml_type, int* block_elems, int* block_bytes);

// f64-built RoPE table (src/hf/precompute.rs:10-40).
void build_rope_table(int head_dim, int max_pos, double theta, std::vector<float>* cos_out, std::vector<float>* sin_out);

}  // namespace hm
