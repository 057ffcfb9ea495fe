// Host-side checkpoint readers.  See loaders.h for the reference anchors.
#include "loaders.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdlib>
#include <cstring>

namespace hm {

// ---- MappedFile ---------------------------------------------------------------------------
MappedFile::~MappedFile() {
    if (data_) munmap(data_, size_);
}

bool MappedFile::open(const std::string& path, std::string* err) {
    int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) {
        *err = "cannot open " + path + ": " + std::strerror(errno);
        return false;
    }
    struct stat st;
    if (fstat(fd, &st) != 0) {
        *err = "cannot stat " + path;
        ::close(fd);
        return false;
    }
    size_ = (size_t)st.st_size;
    if (size_ == 0) {
        *err = path + " is empty";
        ::close(fd);
        return false;
    }
    void* p = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) {
        *err = "mmap failed for " + path;
        data_ = nullptr;
        return false;
    }
    data_ = static_cast<uint8_t*>(p);
    return true;
}

// ---- JSON ---------------------------------------------------------------------------------
namespace {
struct JsonParser {
    const char* p;
    const char* end;
    std::string err;

    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool fail(const char* m) {
        if (err.empty()) err = m;
        return false;
    }
    bool parse_string(std::string* out) {
        if (p >= end || *p != '"') return fail("expected string");
        ++p;
        out->clear();
        while (p < end && *p != '"') {
            if (*p == '\\') {
                ++p;
                if (p >= end) return fail("bad escape");
                switch (*p) {
                    case 'n': out->push_back('\n'); break;
                    case 't': out->push_back('\t'); break;
                    case 'r': out->push_back('\r'); break;
                    case 'b': out->push_back('\b'); break;
                    case 'f': out->push_back('\f'); break;
                    case 'u': {
                        if (end - p < 5) return fail("bad \\u escape");
                        unsigned code = (unsigned)std::strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16);
                        p += 4;
                        if (code < 0x80) {
                            out->push_back((char)code);
                        } else if (code < 0x800) {
                            out->push_back((char)(0xC0 | (code >> 6)));
                            out->push_back((char)(0x80 | (code & 0x3F)));
                        } else {
                            out->push_back((char)(0xE0 | (code >> 12)));
                            out->push_back((char)(0x80 | ((code >> 6) & 0x3F)));
                            out->push_back((char)(0x80 | (code & 0x3F)));
                        }
                        break;
                    }
                    default: out->push_back(*p);
                }
                ++p;
            } else {
                out->push_back(*p++);
            }
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }
    bool parse_value(Json* v, int depth) {
        if (depth > 64) return fail("json too deep");
        ws();
        if (p >= end) return fail("unexpected end of json");
        if (*p == '{') {
            v->kind = Json::Obj;
            ++p;
            ws();
            if (p < end && *p == '}') {
                ++p;
                return true;
            }
            while (true) {
                ws();
                std::string key;
                if (!parse_string(&key)) return false;
                ws();
                if (p >= end || *p != ':') return fail("expected ':'");
                ++p;
                Json child;
                if (!parse_value(&child, depth + 1)) return false;
                v->obj.emplace_back(std::move(key), std::move(child));
                ws();
                if (p < end && *p == ',') {
                    ++p;
                    continue;
                }
                if (p < end && *p == '}') {
                    ++p;
                    return true;
                }
                return fail("expected ',' or '}'");
            }
        }
        if (*p == '[') {
            v->kind = Json::Arr;
            ++p;
            ws();
            if (p < end && *p == ']') {
                ++p;
                return true;
            }
            while (true) {
                Json child;
                if (!parse_value(&child, depth + 1)) return false;
                v->arr.push_back(std::move(child));
                ws();
                if (p < end && *p == ',') {
                    ++p;
                    continue;
                }
                if (p < end && *p == ']') {
                    ++p;
                    return true;
                }
                return fail("expected ',' or ']'");
            }
        }
        if (*p == '"') {
            v->kind = Json::Str;
            return parse_string(&v->str);
        }
        if (end - p >= 4 && !std::strncmp(p, "true", 4)) {
            v->kind = Json::Bool;
            v->b = true;
            p += 4;
            return true;
        }
        if (end - p >= 5 && !std::strncmp(p, "false", 5)) {
            v->kind = Json::Bool;
            v->b = false;
            p += 5;
            return true;
        }
        if (end - p >= 4 && !std::strncmp(p, "null", 4)) {
            v->kind = Json::Null;
            p += 4;
            return true;
        }
        // number
        const char* s = p;
        while (p < end && (std::strchr("+-0123456789.eE", *p) != nullptr)) ++p;
        if (s == p) return fail("unexpected character in json");
        v->kind = Json::Num;
        v->num = std::strtod(std::string(s, p).c_str(), nullptr);
        return true;
    }
};
}  // namespace

const Json* Json::get(const std::string& key) const {
    if (kind != Obj) return nullptr;
    for (auto& kv : obj)
        if (kv.first == key) return &kv.second;
    return nullptr;
}

bool json_parse(const char* text, size_t len, Json* out, std::string* err) {
    JsonParser ps{text, text + len, {}};
    if (!ps.parse_value(out, 0)) {
        *err = "json: " + ps.err;
        return false;
    }
    return true;
}

// ---- config.json ----------------------------------------------------------------------------
bool parse_config_json(const std::string& path, hm_config* cfg, std::string* err) {
    MappedFile f;
    if (!f.open(path, err)) return false;
    Json j;
    if (!json_parse(reinterpret_cast<const char*>(f.data()), f.size(), &j, err)) return false;
    if (j.kind != Json::Obj) {
        *err = "config.json: top level is not an object";
        return false;
    }
    auto need = [&](const char* k, int32_t* dst) {
        const Json* v = j.get(k);
        if (!v || v->kind != Json::Num) {
            *err = std::string("config.json: missing field `") + k + "`";
            return false;
        }
        *dst = (int32_t)v->num;
        return true;
    };
    std::memset(cfg, 0, sizeof(*cfg));
    if (!need("hidden_size", &cfg->hidden_size) || !need("intermediate_size", &cfg->intermediate_size) ||
        !need("num_attention_heads", &cfg->num_attention_heads) || !need("num_hidden_layers", &cfg->num_hidden_layers) ||
        !need("vocab_size", &cfg->vocab_size))
        return false;
    auto num = [&](const char* k) -> const Json* {
        const Json* v = j.get(k);
        return (v && v->kind == Json::Num) ? v : nullptr;
    };
    cfg->num_key_value_heads = num("num_key_value_heads") ? (int32_t)num("num_key_value_heads")->num : cfg->num_attention_heads;
    cfg->rms_norm_eps = num("rms_norm_eps") ? num("rms_norm_eps")->num : 1e-6;
    cfg->rope_theta = num("rope_theta") ? num("rope_theta")->num : 10000.0;
    cfg->max_position_embeddings = num("max_position_embeddings") ? (int32_t)num("max_position_embeddings")->num : 2048;
    const Json* tie = j.get("tie_word_embeddings");
    cfg->tie_word_embeddings = (tie && tie->kind == Json::Bool && tie->b) ? 1 : 0;
    cfg->head_dim = num("head_dim") ? (int32_t)num("head_dim")->num : (cfg->num_attention_heads > 0 ? cfg->hidden_size / cfg->num_attention_heads : 0);
    cfg->eos_token_id = num("eos_token_id") ? (uint32_t)num("eos_token_id")->num : UINT32_MAX;
    cfg->bos_token_id = num("bos_token_id") ? (uint32_t)num("bos_token_id")->num : UINT32_MAX;
    if (cfg->hidden_size <= 0 || cfg->num_attention_heads <= 0 || cfg->num_hidden_layers <= 0 || cfg->vocab_size <= 0 ||
        cfg->num_key_value_heads <= 0 || cfg->intermediate_size <= 0) {
        *err = "config.json: non-positive dimension";
        return false;
    }
    return true;
}

// ---- safetensors ----------------------------------------------------------------------------
bool parse_safetensors(const MappedFile& file, std::vector<TensorView>* out, std::string* err) {
    if (file.size() < 8) {
        *err = "safetensors file too small (< 8 bytes)";
        return false;
    }
    uint64_t hlen;
    std::memcpy(&hlen, file.data(), 8);
    if (hlen > file.size() - 8) {
        *err = "safetensors header length " + std::to_string(hlen) + " exceeds file size " + std::to_string(file.size());
        return false;
    }
    Json j;
    if (!json_parse(reinterpret_cast<const char*>(file.data() + 8), (size_t)hlen, &j, err)) return false;
    if (j.kind != Json::Obj) {
        *err = "safetensors header is not an object";
        return false;
    }
    const size_t base = 8 + (size_t)hlen;
    for (auto& kv : j.obj) {
        if (kv.first == "__metadata__") continue;
        const Json* dt = kv.second.get("dtype");
        const Json* sh = kv.second.get("shape");
        const Json* off = kv.second.get("data_offsets");
        if (!dt || dt->kind != Json::Str || !sh || sh->kind != Json::Arr || !off || off->kind != Json::Arr || off->arr.size() != 2) {
            *err = "safetensors: malformed entry for " + kv.first;
            return false;
        }
        TensorView t;
        t.name = kv.first;
        size_t esz = 0;
        if (dt->str == "BF16") { t.dtype = HM_BF16; esz = 2; }
        else if (dt->str == "F16") { t.dtype = HM_F16; esz = 2; }
        else if (dt->str == "F32") { t.dtype = HM_F32; esz = 4; }
        else if (dt->str == "I64") { t.dtype = HM_I64; esz = 8; }
        else if (dt->str == "I32") { t.dtype = HM_I32; esz = 4; }
        else {
            *err = "unsupported safetensors dtype: " + dt->str;
            return false;
        }
        size_t n = 1;
        for (auto& d : sh->arr) {
            t.shape.push_back((int64_t)d.num);
            n *= (size_t)d.num;
        }
        const size_t b = (size_t)off->arr[0].num, e = (size_t)off->arr[1].num;
        if (e < b || base + e > file.size() || e - b != n * esz) {
            *err = "safetensors: data_offsets out of range for " + kv.first;
            return false;
        }
        t.data = file.data() + base + b;
        t.nbytes = e - b;
        out->push_back(std::move(t));
    }
    return true;
}

// ---- GGUF -------------------------------------------------------------------------------------
void ggml_type_geometry(uint32_t t, int* be, int* bb) {
    switch (t) {
        case 0: *be = 1; *bb = 4; break;     // F32
        case 1: *be = 1; *bb = 2; break;     // F16
        case 2: *be = 32; *bb = 18; break;   // Q4_0
        case 3: *be = 32; *bb = 20; break;   // Q4_1
        case 6: *be = 32; *bb = 22; break;   // Q5_0
        case 7: *be = 32; *bb = 24; break;   // Q5_1
        case 8: *be = 32; *bb = 34; break;   // Q8_0
        case 9: *be = 32; *bb = 40; break;   // Q8_1
        case 10: *be = 256; *bb = 84; break;   // Q2_K
        case 11: *be = 256; *bb = 110; break;  // Q3_K
        case 12: *be = 256; *bb = 144; break;  // Q4_K
        case 13: *be = 256; *bb = 176; break;  // Q5_K
        case 14: *be = 256; *bb = 210; break;  // Q6_K
        case 15: *be = 256; *bb = 292; break;  // Q8_K
        case 24: *be = 1; *bb = 1; break;    // I8
        case 25: *be = 1; *bb = 2; break;    // I16
        case 26: *be = 1; *bb = 4; break;    // I32
        case 27: *be = 1; *bb = 8; break;    // I64
        case 28: *be = 1; *bb = 8; break;    // F64
        case 30: *be = 1; *bb = 2; break;    // BF16
        default: *be = 0; *bb = 0;
    }
}

bool GgufValue::as_u64(uint64_t* out) const {
    if (kind == UInt) { *out = u; return true; }
    if (kind == Int) { *out = (uint64_t)i; return true; }
    return false;
}
bool GgufValue::as_f32(float* out) const {
    if (kind == Float) { *out = (float)f; return true; }
    return false;
}

const TensorView* GgufFile::find(const std::string& name) const {
    for (auto& t : tensors)
        if (t.name == name) return &t;
    return nullptr;
}

namespace {
struct Cursor {
    const uint8_t* p;
    size_t size, pos = 0;
    bool ok = true;
    template <typename T>
    T rd() {
        T v{};
        if (pos + sizeof(T) > size) {
            ok = false;
            return v;
        }
        std::memcpy(&v, p + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str() {
        uint64_t n = rd<uint64_t>();
        if (!ok || n > size - pos) {
            ok = false;
            return {};
        }
        std::string s(reinterpret_cast<const char*>(p + pos), (size_t)n);
        pos += (size_t)n;
        return s;
    }
};

bool read_value(Cursor& c, uint32_t type, GgufValue* v, int depth) {
    switch (type) {
        case 0: v->kind = GgufValue::UInt; v->u = c.rd<uint8_t>(); break;
        case 1: v->kind = GgufValue::Int; v->i = c.rd<int8_t>(); break;
        case 2: v->kind = GgufValue::UInt; v->u = c.rd<uint16_t>(); break;
        case 3: v->kind = GgufValue::Int; v->i = c.rd<int16_t>(); break;
        case 4: v->kind = GgufValue::UInt; v->u = c.rd<uint32_t>(); break;
        case 5: v->kind = GgufValue::Int; v->i = c.rd<int32_t>(); break;
        case 6: v->kind = GgufValue::Float; v->f = c.rd<float>(); break;
        case 7: v->kind = GgufValue::Bool; v->b = c.rd<uint8_t>() != 0; break;
        case 8: v->kind = GgufValue::Str; v->s = c.str(); break;
        case 10: v->kind = GgufValue::UInt; v->u = c.rd<uint64_t>(); break;
        case 11: v->kind = GgufValue::Int; v->i = c.rd<int64_t>(); break;
        case 12: v->kind = GgufValue::Float; v->f = c.rd<double>(); break;
        case 9: {
            if (depth > 4) return false;
            const uint32_t et = c.rd<uint32_t>();
            const uint64_t n = c.rd<uint64_t>();
            v->kind = GgufValue::Arr;
            v->arr_len = n;
            for (uint64_t i = 0; i < n && c.ok; ++i) {
                GgufValue tmp;
                if (!read_value(c, et, &tmp, depth + 1)) return false;
            }
            break;
        }
        default: return false;
    }
    return c.ok;
}
}  // namespace

bool parse_gguf(const MappedFile& file, GgufFile* out, std::string* err) {
    if (file.size() < 16) {
        *err = "GGUF file too small";
        return false;
    }
    Cursor c{file.data(), file.size()};
    const uint32_t magic = c.rd<uint32_t>();
    if (magic != 0x46554747u) {
        *err = "invalid GGUF magic";
        return false;
    }
    out->version = c.rd<uint32_t>();
    if (out->version < 2 || out->version > 3) {
        *err = "unsupported GGUF version: " + std::to_string(out->version) + " (expected 2 or 3)";
        return false;
    }
    const uint64_t nt = out->version >= 3 ? c.rd<uint64_t>() : c.rd<uint32_t>();
    const uint64_t nkv = out->version >= 3 ? c.rd<uint64_t>() : c.rd<uint32_t>();
    for (uint64_t i = 0; i < nkv && c.ok; ++i) {
        std::string key = c.str();
        const uint32_t type = c.rd<uint32_t>();
        GgufValue v;
        if (!read_value(c, type, &v, 0)) {
            *err = "GGUF: bad metadata value for key " + key;
            return false;
        }
        out->metadata[key] = std::move(v);
    }
    if (!c.ok) {
        *err = "GGUF: truncated metadata";
        return false;
    }
    size_t alignment = 32;
    auto it = out->metadata.find("general.alignment");
    uint64_t a64;
    if (it != out->metadata.end() && it->second.as_u64(&a64) && a64 > 0) alignment = (size_t)a64;
    std::vector<uint64_t> offsets;
    for (uint64_t i = 0; i < nt && c.ok; ++i) {
        TensorView t;
        t.name = c.str();
        const uint32_t nd = c.rd<uint32_t>();
        if (nd > 8) {
            *err = "GGUF: tensor rank too large for " + t.name;
            return false;
        }
        std::vector<int64_t> dims(nd);
        for (uint32_t d = 0; d < nd; ++d) dims[d] = (int64_t)c.rd<uint64_t>();
        t.shape.assign(dims.rbegin(), dims.rend());  // innermost-first on disk (src/gguf.rs:412-417)
        const uint32_t gt = c.rd<uint32_t>();
        offsets.push_back(c.rd<uint64_t>());
        int be, bb;
        ggml_type_geometry(gt, &be, &bb);
        if (be == 0) {
            *err = "unknown GGML type code " + std::to_string(gt) + " for tensor '" + t.name + "'";
            return false;
        }
        switch (gt) {
            case 0: t.dtype = HM_F32; break;
            case 1: t.dtype = HM_F16; break;
            case 30: t.dtype = HM_BF16; break;
            case 8: t.dtype = HM_Q8_0; break;
            case 2: t.dtype = HM_Q4_0; break;
            case 12: t.dtype = HM_Q4_K; break;
            case 14: t.dtype = HM_Q6_K; break;
            default: t.dtype = -1;
        }
        size_t n = 1;
        for (auto d : t.shape) n *= (size_t)d;
        if (n % be != 0) {
            *err = "GGUF: element count of " + t.name + " is not a multiple of its block size";
            return false;
        }
        t.nbytes = n / be * bb;
        out->tensors.push_back(std::move(t));
        out->ggml_types.push_back(gt);
    }
    if (!c.ok) {
        *err = "GGUF: truncated tensor table";
        return false;
    }
    const size_t data0 = (c.pos + alignment - 1) / alignment * alignment;
    for (size_t i = 0; i < out->tensors.size(); ++i) {
        TensorView& t = out->tensors[i];
        if (data0 + offsets[i] + t.nbytes > file.size()) {
            *err = "GGUF: tensor data of " + t.name + " runs past the end of the file";
            return false;
        }
        t.data = file.data() + data0 + offsets[i];
    }
    return true;
}

bool gguf_config(const GgufFile& g, hm_config* cfg, std::string* err) {
    auto it = g.metadata.find("general.architecture");
    if (it == g.metadata.end() || it->second.kind != GgufValue::Str) {
        *err = "missing general.architecture metadata";
        return false;
    }
    const std::string arch = it->second.s;
    auto get_u64 = [&](const std::string& key, uint64_t* out) {
        auto f = g.metadata.find(arch + "." + key);
        return f != g.metadata.end() && f->second.as_u64(out);
    };
    auto get_f32 = [&](const std::string& key, float* out) {
        auto f = g.metadata.find(arch + "." + key);
        return f != g.metadata.end() && f->second.as_f32(out);
    };
    std::memset(cfg, 0, sizeof(*cfg));
    uint64_t v;
    auto need = [&](const char* key, int32_t* dst) {
        if (!get_u64(key, &v)) {
            *err = std::string("missing or invalid metadata: ") + arch + "." + key;
            return false;
        }
        *dst = (int32_t)v;
        return true;
    };
    if (!need("embedding_length", &cfg->hidden_size) || !need("feed_forward_length", &cfg->intermediate_size) ||
        !need("attention.head_count", &cfg->num_attention_heads) || !need("block_count", &cfg->num_hidden_layers))
        return false;
    cfg->num_key_value_heads = get_u64("attention.head_count_kv", &v) ? (int32_t)v : cfg->num_attention_heads;
    if (get_u64("vocab_size", &v)) {
        cfg->vocab_size = (int32_t)v;
    } else {
        auto tk = g.metadata.find("tokenizer.ggml.tokens");
        if (tk != g.metadata.end() && tk->second.kind == GgufValue::Arr) {
            cfg->vocab_size = (int32_t)tk->second.arr_len;
        } else {
            *err = "cannot determine vocab_size";
            return false;
        }
    }
    float f;
    cfg->rms_norm_eps = get_f32("attention.layer_norm_rms_epsilon", &f) ? (double)f : 1e-6;
    cfg->rope_theta = get_f32("rope.freq_base", &f) ? (double)f : 10000.0;
    cfg->max_position_embeddings = get_u64("context_length", &v) ? (int32_t)v : 2048;
    cfg->tie_word_embeddings = g.find("output.weight") ? 0 : 1;
    cfg->head_dim = get_u64("attention.key_length", &v) ? (int32_t)v : cfg->hidden_size / cfg->num_attention_heads;
    auto tok = [&](const char* key) -> uint32_t {
        auto t = g.metadata.find(key);
        uint64_t x;
        return (t != g.metadata.end() && t->second.as_u64(&x)) ? (uint32_t)x : UINT32_MAX;
    };
    cfg->eos_token_id = tok("tokenizer.ggml.eos_token_id");
    cfg->bos_token_id = tok("tokenizer.ggml.bos_token_id");
    return true;
}

void build_rope_table(int head_dim, int max_pos, double theta, std::vector<float>* cos_out, std::vector<float>* sin_out) {
    const int half = head_dim / 2;
    cos_out->assign((size_t)max_pos * head_dim, 0.f);
    sin_out->assign((size_t)max_pos * head_dim, 0.f);
    for (int pos = 0; pos < max_pos; ++pos) {
        for (int i = 0; i < half; ++i) {
            const double freq = 1.0 / std::pow(theta, 2.0 * (double)i / (double)head_dim);
            const double angle = (double)pos * freq;
            const float c = (float)std::cos(angle), s = (float)std::sin(angle);
            (*cos_out)[(size_t)pos * head_dim + i] = c;
            (*cos_out)[(size_t)pos * head_dim + half + i] = c;
            (*sin_out)[(size_t)pos * head_dim + i] = s;
            (*sin_out)[(size_t)pos * head_dim + half + i] = s;
        }
    }
}

}  // namespace hm
