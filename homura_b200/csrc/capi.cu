// extern "C" surface declared in include/homura_b200.h.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "engine.h"
#include "gemm_tc.h"
#include "kquant.h"
#include "sampler.h"
#include "loaders.h"

using namespace hm;

struct hm_engine {
    Engine* impl = nullptr;
};

namespace {
thread_local std::string g_err;

int gfail(int code, const std::string& msg) {
    g_err = msg;
    return code;
}

// ---- host/device pointer staging for the standalone kernel entry points -------------------
bool is_device_ptr(const void* p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

// Keeps temporaries of one call; inputs are copied in on construction, outputs copied back
// by finish().
class Staging {
   public:
    explicit Staging(cudaStream_t st) : st_(st) {}
    ~Staging() {
        for (void* p : owned_) cudaFree(p);
    }
    template <typename T>
    const T* in(const T* p, size_t count) {
        if (!p || is_device_ptr(p)) return p;
        void* d = nullptr;
        if (!ok(cudaMalloc(&d, std::max<size_t>(count * sizeof(T), 16)))) return nullptr;
        owned_.push_back(d);
        ok(cudaMemcpyAsync(d, p, count * sizeof(T), cudaMemcpyHostToDevice, st_));
        return static_cast<const T*>(d);
    }
    template <typename T>
    T* out(T* p, size_t count, bool copy_in = false) {
        if (!p || is_device_ptr(p)) return p;
        void* d = nullptr;
        if (!ok(cudaMalloc(&d, std::max<size_t>(count * sizeof(T), 16)))) return nullptr;
        owned_.push_back(d);
        if (copy_in) ok(cudaMemcpyAsync(d, p, count * sizeof(T), cudaMemcpyHostToDevice, st_));
        outs_.push_back({p, d, count * sizeof(T)});
        return static_cast<T*>(d);
    }
    void* scratch(size_t bytes, bool zero) {
        void* d = nullptr;
        if (!ok(cudaMalloc(&d, std::max<size_t>(bytes, 16)))) return nullptr;
        owned_.push_back(d);
        if (zero) ok(cudaMemsetAsync(d, 0, bytes, st_));
        return d;
    }
    bool staged() const { return !owned_.empty(); }
    bool ok(cudaError_t e) {
        if (e != cudaSuccess && err_ == cudaSuccess) err_ = e;
        return e == cudaSuccess;
    }
    // copies outputs back and synchronises when anything was staged or scratch was used
    int finish(cudaError_t launch_err) {
        ok(launch_err);
        if (err_ == cudaSuccess)
            for (auto& o : outs_) ok(cudaMemcpyAsync(o.host, o.dev, o.bytes, cudaMemcpyDeviceToHost, st_));
        if (!owned_.empty()) ok(cudaStreamSynchronize(st_));
        if (err_ != cudaSuccess) return gfail(HM_ERR_CUDA, std::string("CUDA error: ") + cudaGetErrorString(err_));
        return HM_OK;
    }

   private:
    struct Out {
        void* host;
        void* dev;
        size_t bytes;
    };
    cudaStream_t st_;
    std::vector<void*> owned_;
    std::vector<Out> outs_;
    cudaError_t err_ = cudaSuccess;
};

// Split-K scratch of the standalone entry points: one growing buffer per device plus a ticket
// array that the kernels leave zeroed.  Calls on one device are therefore not re-entrant.
struct DeviceScratch {
    float* partial = nullptr;
    size_t partial_floats = 0;
    unsigned int* tickets = nullptr;  // kMaxTickets entries
    int* wait_err = nullptr;          // raised by a kernel whose bounded wait ran out
};
constexpr size_t kMaxTickets = 1 << 16;
std::mutex g_scratch_mu;
std::map<int, DeviceScratch> g_scratch;

cudaError_t get_scratch(size_t partial_floats, size_t ntickets, float** partial, unsigned int** tickets) {
    if (ntickets > kMaxTickets) return cudaErrorInvalidValue;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    DeviceScratch& s = g_scratch[dev];
    if (!s.tickets) {
        e = cudaMalloc(&s.tickets, kMaxTickets * sizeof(unsigned int));
        if (e != cudaSuccess) return e;
        e = cudaMemset(s.tickets, 0, kMaxTickets * sizeof(unsigned int));
        if (e != cudaSuccess) return e;
    }
    if (partial_floats > s.partial_floats) {
        e = cudaDeviceSynchronize();  // nothing may still be using the old buffer
        if (e != cudaSuccess) return e;
        if (s.partial) cudaFree(s.partial);
        s.partial = nullptr;
        s.partial_floats = 0;
        e = cudaMalloc(&s.partial, partial_floats * sizeof(float));
        if (e != cudaSuccess) return e;
        s.partial_floats = partial_floats;
    }
    *partial = s.partial;
    *tickets = s.tickets;
    return cudaSuccess;
}

// Device word that kernels with bounded waits raise; allocated once per device.
cudaError_t get_wait_err(int** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    DeviceScratch& s = g_scratch[dev];
    if (!s.wait_err) {
        e = cudaMalloc(&s.wait_err, sizeof(int));
        if (e != cudaSuccess) return e;
        e = cudaMemset(s.wait_err, 0, sizeof(int));
        if (e != cudaSuccess) return e;
    }
    *out = s.wait_err;
    return cudaSuccess;
}

// After a synchronisation: reads and clears the word; true when a wait had run out.
bool take_wait_err() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    int* p = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_scratch_mu);
        auto it = g_scratch.find(dev);
        if (it == g_scratch.end() || !it->second.wait_err) return false;
        p = it->second.wait_err;
    }
    int h = 0;
    if (cudaMemcpy(&h, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return false;
    if (h) cudaMemset(p, 0, sizeof(int));
    return h != 0;
}

int sm_count_of_current_device() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

bool have_device() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return n > 0;
}

#define NEED_DEVICE()                                                                             \
    do {                                                                                          \
        if (!have_device()) return gfail(HM_ERR_CUDA, "no CUDA device available (no CPU fallback)"); \
    } while (0)

}  // namespace

namespace hm {
int set_global_error(int code, const char* msg) { return gfail(code, msg ? msg : ""); }

// sample_token, src/generate.rs:698-801.  Candidates are ordered by descending probability
// with a stable sort (the reference uses sort_unstable_by, so ties may order differently).
uint32_t host_sample_token(const float* logits_in, int n, const hm_sampling& cfg, const uint32_t* generated, int ngen, uint64_t* rng) {
    std::vector<float> logits(logits_in, logits_in + n);
    if (cfg.repetition_penalty != 1.0f) {
        for (int i = 0; i < ngen; ++i) {
            const size_t idx = generated[i];
            if (idx < (size_t)n) {
                if (logits[idx] > 0.0f) logits[idx] /= cfg.repetition_penalty;
                else logits[idx] *= cfg.repetition_penalty;
            }
        }
    }
    if (cfg.frequency_penalty != 0.0f || cfg.presence_penalty != 0.0f) {
        std::map<size_t, size_t> counts;
        for (int i = 0; i < ngen; ++i) counts[generated[i]] += 1;
        for (auto& kv : counts) {
            if (kv.first < (size_t)n) {
                logits[kv.first] -= cfg.frequency_penalty * (float)kv.second;
                logits[kv.first] -= cfg.presence_penalty;
            }
        }
    }
    if (cfg.temperature <= 0.0f) {
        int best = 0;
        for (int i = 1; i < n; ++i)
            if (!(logits[best] > logits[i])) best = i;  // max_by keeps the last maximum
        return (uint32_t)best;
    }
    const float inv_temp = 1.0f / cfg.temperature;
    for (auto& l : logits) l *= inv_temp;
    float mx = -INFINITY;
    for (float l : logits) mx = std::max(mx, l);
    std::vector<float> probs(n);
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) {
        probs[i] = std::exp(logits[i] - mx);
        sum += probs[i];
    }
    for (auto& p : probs) p /= sum;
    if (cfg.min_p > 0.0f) {
        float maxp = 0.0f;
        for (float p : probs) maxp = std::max(maxp, p);
        const float thr = cfg.min_p * maxp;
        for (auto& p : probs)
            if (p < thr) p = 0.0f;
    }
    std::vector<std::pair<int, float>> idx(n);
    for (int i = 0; i < n; ++i) idx[i] = {i, probs[i]};
    std::stable_sort(idx.begin(), idx.end(), [](const std::pair<int, float>& a, const std::pair<int, float>& b) { return a.second > b.second; });
    if (cfg.top_k > 0 && cfg.top_k < n) idx.resize(cfg.top_k);
    float cumulative = 0.0f;
    size_t cutoff = idx.size();
    for (size_t i = 0; i < idx.size(); ++i) {
        cumulative += idx[i].second;
        if (cumulative >= cfg.top_p) {
            cutoff = i + 1;
            break;
        }
    }
    float total = 0.0f;
    for (size_t i = 0; i < cutoff; ++i) total += idx[i].second;
    uint64_t s = *rng;  // xorshift64 (13, 7, 17), src/generate.rs:634-641
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    *rng = s;
    const float r = ((float)(s >> 40) / (float)(1ull << 24)) * total;
    float accum = 0.0f;
    for (size_t i = 0; i < cutoff; ++i) {
        accum += idx[i].second;
        if (accum >= r) return (uint32_t)idx[i].first;
    }
    return cutoff ? (uint32_t)idx[cutoff - 1].first : 0u;
}
}  // namespace hm

extern "C" {

const char* hm_version(void) { return "homura_b200 0.1 (sm_100a)"; }

int hm_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

const char* hm_last_error_global(void) { return g_err.c_str(); }

int hm_engine_create(const hm_config* cfg, int device, hm_engine** out) {
    if (!cfg || !out) return gfail(HM_ERR_INVALID, "hm_engine_create: null argument");
    Engine* e = nullptr;
    std::string err;
    int rc = Engine::create(*cfg, device, &e, &err);
    if (rc) return gfail(rc, err);
    *out = new hm_engine{e};
    return HM_OK;
}

void hm_engine_destroy(hm_engine* e) {
    if (!e) return;
    delete e->impl;
    delete e;
}

const char* hm_last_error(hm_engine* e) { return e ? e->impl->err.c_str() : g_err.c_str(); }

int hm_load_tensor(hm_engine* e, const char* name, int dtype, const int64_t* shape, int ndim, const void* host_data, size_t nbytes) {
    if (!e) return gfail(HM_ERR_INVALID, "null engine");
    return e->impl->load_tensor(name, dtype, shape, ndim, host_data, nbytes);
}

int hm_finalize_weights(hm_engine* e) {
    if (!e) return gfail(HM_ERR_INVALID, "null engine");
    return e->impl->finalize();
}

int hm_get_config(hm_engine* e, hm_config* out) {
    if (!e || !out) return gfail(HM_ERR_INVALID, "null argument");
    *out = e->impl->config();
    return HM_OK;
}

int hm_weight_bytes(hm_engine* e, uint64_t* out) {
    if (!e || !out) return gfail(HM_ERR_INVALID, "null argument");
    *out = e->impl->weight_bytes();
    return HM_OK;
}

// Vectors (norm weights, biases) first: whether a model has QK-norm is inferred from its tensors, and the layout of
// a quantised QKV projection (rotation in its epilogue or not) is fixed when its first part is loaded.
static int load_views(Engine* eng, const std::vector<TensorView>& views, std::string* err) {
    for (int pass = 0; pass < 2; ++pass) {
        for (const TensorView& t : views) {
            if (t.dtype < 0) {
                *err = "unsupported GGML type for tensor '" + t.name + "'";
                return HM_ERR_UNSUPPORTED;
            }
            if (t.name.find("rotary_emb.inv_freq") != std::string::npos) continue;
            if ((t.shape.size() == 1) != (pass == 0)) continue;
            int rc = eng->load_tensor(t.name.c_str(), t.dtype, t.shape.data(), (int)t.shape.size(), t.data, t.nbytes);
            if (rc) {
                *err = eng->err;
                return rc;
            }
        }
    }
    return HM_OK;
}

// model.safetensors, else the shards named by model.safetensors.index.json in file-name order, each once
// (src/hf/model.rs:86-127).
static int safetensors_files(const std::string& dir, std::vector<std::string>* files, std::string* err) {
    MappedFile probe;
    std::string e2;
    if (probe.open(dir + "/model.safetensors", &e2)) {
        files->push_back(dir + "/model.safetensors");
        return HM_OK;
    }
    MappedFile idx;
    if (!idx.open(dir + "/model.safetensors.index.json", &e2)) {
        *err = "no model.safetensors or model.safetensors.index.json found in " + dir;
        return HM_ERR_IO;
    }
    Json j;
    if (!json_parse((const char*)idx.data(), idx.size(), &j, err)) return HM_ERR_IO;
    const Json* wm = j.get("weight_map");
    if (!wm || wm->kind != Json::Obj) {
        *err = "model.safetensors.index.json missing weight_map";
        return HM_ERR_IO;
    }
    for (auto& kv : wm->obj)
        if (kv.second.kind == Json::Str) files->push_back(dir + "/" + kv.second.str);
    std::sort(files->begin(), files->end());
    files->erase(std::unique(files->begin(), files->end()), files->end());
    if (files->empty()) {
        *err = "model.safetensors.index.json names no shard";
        return HM_ERR_IO;
    }
    return HM_OK;
}

int hm_model_load(const char* model_dir, int weight_dtype, int device, hm_engine** out) {
    if (!model_dir || !out) return gfail(HM_ERR_INVALID, "hm_model_load: null argument");
    // HM_F32 is HfModel::load's default (src/hf/model.rs:37-39): the reference widens the file's weights to f32 and
    // multiplies f32 x f32.  For a bf16 checkpoint the widened values are the bf16 values, so keeping them as bf16
    // gives the same products; files whose projections really are f32 / f16 are refused when their first
    // projection tensor is loaded (an f32-weight streaming kernel is not built).
    if (weight_dtype != HM_BF16 && weight_dtype != HM_F32)
        return gfail(HM_ERR_UNSUPPORTED, "hm_model_load: weight_dtype must be HM_BF16 or HM_F32 (Homura's --dtype bf16 / f32)");
    const std::string dir(model_dir);
    hm_config cfg;
    std::string err;
    if (!parse_config_json(dir + "/config.json", &cfg, &err)) return gfail(HM_ERR_IO, err);
    NEED_DEVICE();
    std::vector<std::string> files;
    {
        const int frc = safetensors_files(dir, &files, &err);
        if (frc) return gfail(frc, err);
    }
    Engine* eng = nullptr;
    int rc = Engine::create(cfg, device, &eng, &err);
    if (rc) return gfail(rc, err);
    for (auto& f : files) {
        MappedFile mf;
        if (!mf.open(f, &err)) {
            delete eng;
            return gfail(HM_ERR_IO, err);
        }
        std::vector<TensorView> views;
        if (!parse_safetensors(mf, &views, &err)) {
            delete eng;
            return gfail(HM_ERR_IO, err);
        }
        rc = load_views(eng, views, &err);
        if (rc) {
            delete eng;
            return gfail(rc, err);
        }
    }
    rc = eng->finalize();
    if (rc) {
        err = eng->err;
        delete eng;
        return gfail(rc, err);
    }
    *out = new hm_engine{eng};
    return HM_OK;
}

int hm_model_load_gguf(const char* gguf_path, int device, hm_engine** out) {
    if (!gguf_path || !out) return gfail(HM_ERR_INVALID, "hm_model_load_gguf: null argument");
    MappedFile mf;
    std::string err;
    if (!mf.open(gguf_path, &err)) return gfail(HM_ERR_IO, err);
    GgufFile g;
    if (!parse_gguf(mf, &g, &err)) return gfail(HM_ERR_IO, err);
    hm_config cfg;
    if (!gguf_config(g, &cfg, &err)) return gfail(HM_ERR_IO, err);
    NEED_DEVICE();
    Engine* eng = nullptr;
    int rc = Engine::create(cfg, device, &eng, &err);
    if (rc) return gfail(rc, err);
    rc = load_views(eng, g.tensors, &err);
    if (!rc) {
        rc = eng->finalize();
        if (rc) err = eng->err;
    }
    if (rc) {
        delete eng;
        return gfail(rc, err);
    }
    *out = new hm_engine{eng};
    return HM_OK;
}

static uint64_t fnv1a(const uint8_t* p, size_t n) {
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < n; ++i) {
        h ^= p[i];
        h *= 1099511628211ull;
    }
    return h;
}

static void json_escape(const std::string& in, std::string* out) {
    for (char ch : in) {
        if (ch == '"' || ch == '\\') out->push_back('\\');
        out->push_back(ch);
    }
}

int hm_checkpoint_info(const char* path, char* buf, size_t cap, size_t* needed) {
    if (!path) return gfail(HM_ERR_INVALID, "hm_checkpoint_info: null path");
    const std::string p(path);
    std::string err, fmt;
    hm_config cfg;
    std::vector<TensorView> views;
    MappedFile mf;
    std::vector<std::unique_ptr<MappedFile>> shards;  // the views point into these
    GgufFile g;
    const bool is_gguf = p.size() > 5 && p.compare(p.size() - 5, 5, ".gguf") == 0;
    if (is_gguf) {
        fmt = "gguf";
        if (!mf.open(p, &err)) return gfail(HM_ERR_IO, err);
        if (!parse_gguf(mf, &g, &err)) return gfail(HM_ERR_IO, err);
        if (!gguf_config(g, &cfg, &err)) return gfail(HM_ERR_IO, err);
        views = g.tensors;
    } else {
        fmt = "safetensors";
        if (!parse_config_json(p + "/config.json", &cfg, &err)) return gfail(HM_ERR_IO, err);
        std::vector<std::string> files;
        const int frc = safetensors_files(p, &files, &err);
        if (frc) return gfail(frc, err);
        for (size_t i = 0; i < files.size(); ++i) {
            std::vector<TensorView> part;
            shards.emplace_back(new MappedFile());
            if (!shards[i]->open(files[i], &err)) return gfail(HM_ERR_IO, err);
            if (!parse_safetensors(*shards[i], &part, &err)) return gfail(HM_ERR_IO, err);
            views.insert(views.end(), part.begin(), part.end());
        }
    }
    static const char* dn[] = {"F32", "BF16", "F16", "Q8_0", "Q4_0", "I64", "I32", "U8", "Q4_K", "Q6_K"};
    std::string o = "{\"format\":\"" + fmt + "\",\"config\":{";
    char tmp[512];
    std::snprintf(tmp, sizeof(tmp),
                  "\"hidden_size\":%d,\"intermediate_size\":%d,\"num_attention_heads\":%d,\"num_hidden_layers\":%d,\"num_key_value_heads\":%d,"
                  "\"vocab_size\":%d,\"max_position_embeddings\":%d,\"head_dim\":%d,\"tie_word_embeddings\":%s,\"rms_norm_eps\":%.17g,\"rope_theta\":%.17g,"
                  "\"eos_token_id\":%lld,\"bos_token_id\":%lld",
                  cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.vocab_size,
                  cfg.max_position_embeddings, cfg.head_dim, cfg.tie_word_embeddings ? "true" : "false", cfg.rms_norm_eps, cfg.rope_theta,
                  cfg.eos_token_id == UINT32_MAX ? -1ll : (long long)cfg.eos_token_id, cfg.bos_token_id == UINT32_MAX ? -1ll : (long long)cfg.bos_token_id);
    o += tmp;
    o += "},\"tensors\":[";
    bool first = true;
    for (const TensorView& t : views) {
        if (!first) o += ",";
        first = false;
        o += "{\"name\":\"";
        json_escape(t.name, &o);
        o += "\",\"dtype\":\"";
        o += (t.dtype >= 0 && t.dtype < 10) ? dn[t.dtype] : "UNSUPPORTED";
        o += "\",\"shape\":[";
        for (size_t i = 0; i < t.shape.size(); ++i) {
            if (i) o += ",";
            o += std::to_string(t.shape[i]);
        }
        std::snprintf(tmp, sizeof(tmp), "],\"nbytes\":%zu,\"fnv1a\":\"%016llx\"}", t.nbytes, (unsigned long long)fnv1a(t.data, t.nbytes));
        o += tmp;
    }
    o += "]}";
    if (needed) *needed = o.size() + 1;
    if (!buf || cap < o.size() + 1) return gfail(HM_ERR_INVALID, "hm_checkpoint_info: buffer too small");
    std::memcpy(buf, o.c_str(), o.size() + 1);
    return HM_OK;
}

int hm_kv_alloc(hm_engine* e, int batch, int max_seq_len, int page_tokens, int kv_dtype) { return e ? e->impl->kv_alloc(batch, max_seq_len, page_tokens, kv_dtype) : gfail(HM_ERR_INVALID, "null engine"); }
int hm_kv_free(hm_engine* e) { return e ? e->impl->kv_free() : gfail(HM_ERR_INVALID, "null engine"); }
int hm_kv_reset(hm_engine* e, int seq) { return e ? e->impl->kv_reset(seq) : gfail(HM_ERR_INVALID, "null engine"); }
int hm_kv_len(hm_engine* e, int seq, int* out) { return e ? e->impl->kv_len(seq, out) : gfail(HM_ERR_INVALID, "null engine"); }
int hm_kv_append(hm_engine* e, int seq, int layer, const float* k_rows, const float* v_rows, int n_new, int advance) {
    return e ? e->impl->kv_append(seq, layer, k_rows, v_rows, n_new, advance) : gfail(HM_ERR_INVALID, "null engine");
}
int hm_kv_view(hm_engine* e, int seq, int layer, float* k_out, float* v_out) { return e ? e->impl->kv_view(seq, layer, k_out, v_out) : gfail(HM_ERR_INVALID, "null engine"); }

int hm_prefill(hm_engine* e, int seq, const int64_t* ids, int n, float* logits_or_null, uint32_t* first_token) {
    return e ? e->impl->prefill(seq, ids, n, logits_or_null, first_token) : gfail(HM_ERR_INVALID, "null engine");
}
int hm_decode_step(hm_engine* e, const uint32_t* tokens, float* logits_or_null, uint32_t* next_tokens) {
    return e ? e->impl->decode_step(tokens, logits_or_null, next_tokens) : gfail(HM_ERR_INVALID, "null engine");
}
int hm_generate(hm_engine* e, int seq, const int64_t* prompt, int n_prompt, int max_new_tokens, const hm_sampling* sampling, uint32_t* out_ids, int* n_out) {
    return e ? e->impl->generate(seq, prompt, n_prompt, max_new_tokens, sampling, out_ids, n_out) : gfail(HM_ERR_INVALID, "null engine");
}
int hm_decode_greedy_n(hm_engine* e, const uint32_t* first_tokens, int steps, uint32_t* out_ids) {
    return e ? e->impl->decode_greedy_n(first_tokens, steps, out_ids) : gfail(HM_ERR_INVALID, "null engine");
}
int hm_sample_token(const float* logits, int n, const hm_sampling* cfg, const uint32_t* generated, int n_generated, uint64_t* rng_state, uint32_t* out) {
    if (!logits || n < 1 || !cfg || !rng_state || !out || (n_generated > 0 && !generated)) return gfail(HM_ERR_INVALID, "hm_sample_token: bad arguments");
    *out = host_sample_token(logits, n, *cfg, generated, n_generated, rng_state);
    return HM_OK;
}
int hm_sample_token_device(const float* logits, int n, const hm_sampling* cfg, const uint32_t* generated, int n_generated, uint64_t* rng_state, uint32_t* out) {
    if (!logits || n < 1 || !cfg || !rng_state || !out || n_generated < 0 || (n_generated > 0 && !generated)) return gfail(HM_ERR_INVALID, "hm_sample_token_device: bad arguments");
    NEED_DEVICE();
    Staging sg(nullptr);
    SamplerArgs a{};
    a.logits = sg.in(logits, (size_t)n);
    a.ld_logits = n;
    a.n = n;
    a.cfg = *cfg;
    a.generated = n_generated ? sg.in(generated, (size_t)n_generated) : nullptr;
    a.n_generated = n_generated;
    a.rng = (unsigned long long*)sg.scratch(8, false);
    a.scaled = (float*)sg.scratch((size_t)n * 4, false);
    a.count = (int*)sg.scratch((size_t)n * 4, true);
    a.next_tok = (uint32_t*)sg.scratch(4, false);
    a.overflow = (int*)sg.scratch(4, true);
    if (!a.logits || !a.rng || !a.scaled || !a.count || !a.next_tok || !a.overflow || (n_generated && !a.generated)) return sg.finish(cudaErrorMemoryAllocation);
    sg.ok(cudaMemcpyAsync(a.rng, rng_state, 8, cudaMemcpyHostToDevice, nullptr));
    cudaError_t ce = launch_sample(a, 1, nullptr);
    int over = 0;
    uint64_t rng_after = *rng_state;
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(&rng_after, a.rng, 8, cudaMemcpyDeviceToHost, nullptr);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(out, a.next_tok, 4, cudaMemcpyDeviceToHost, nullptr);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(&over, a.overflow, 4, cudaMemcpyDeviceToHost, nullptr);
    const int rc = sg.finish(ce);
    if (rc != HM_OK) return rc;
    if (over && cfg->temperature > 0.f) {
        // the top-p prefix reaches beyond the candidates the kernel gathers (top-k disabled or above 1024 on a
        // nearly flat row): the kernel left token and RNG untouched and the host sampler finishes the token
        std::vector<float> lh;
        std::vector<uint32_t> gh;
        const float* lp = logits;
        const uint32_t* gp = generated;
        if (is_device_ptr(logits)) {
            lh.resize(n);
            if (cudaMemcpy(lh.data(), logits, (size_t)n * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return gfail(HM_ERR_CUDA, "hm_sample_token_device: logits read-back failed");
            lp = lh.data();
        }
        if (n_generated && is_device_ptr(generated)) {
            gh.resize(n_generated);
            if (cudaMemcpy(gh.data(), generated, (size_t)n_generated * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return gfail(HM_ERR_CUDA, "hm_sample_token_device: history read-back failed");
            gp = gh.data();
        }
        *out = host_sample_token(lp, n, *cfg, gp, n_generated, rng_state);
        return HM_OK;
    }
    *rng_state = rng_after;
    return HM_OK;
}
int hm_decode_step_sampled(hm_engine* e, const uint32_t* tokens, const hm_sampling* sampling, uint64_t* rng_state, float* logits_or_null, uint32_t* next_tokens) {
    return e ? e->impl->decode_step_sampled(tokens, sampling, rng_state, logits_or_null, next_tokens) : gfail(HM_ERR_INVALID, "null engine");
}
int hm_time_decode(hm_engine* e, int warmup, int steps, float* ms_total) { return e ? e->impl->time_decode(warmup, steps, ms_total) : gfail(HM_ERR_INVALID, "null engine"); }
int hm_profile_decode(hm_engine* e, int steps, hm_kernel_stat* out, int cap, int* n_out) {
    return e ? e->impl->profile_decode(steps, out, cap, n_out) : gfail(HM_ERR_INVALID, "null engine");
}
int hm_selftest_expire_wait(hm_engine* e) { return e ? e->impl->selftest_expire_wait() : gfail(HM_ERR_INVALID, "null engine"); }
void* hm_engine_stream(hm_engine* e) { return e ? (void*)e->impl->stream() : nullptr; }
int hm_launches_per_step(hm_engine* e, int* out) {
    if (!e || !out) return gfail(HM_ERR_INVALID, "null argument");
    *out = e->impl->launches_per_step();
    return HM_OK;
}

// ---- standalone kernels ---------------------------------------------------------------------

int hm_pack_bf16_slabs(const void* w_kn, int K, int N, void* dst, void* stream) {
    if (!w_kn || !dst || K < 1 || N < 1) return gfail(HM_ERR_INVALID, "hm_pack_bf16_slabs: bad arguments");
    NEED_DEVICE();
    cudaStream_t st = (cudaStream_t)stream;
    Staging sg(st);
    const size_t dst_elems = (size_t)((N + SLAB - 1) / SLAB) * K * SLAB;
    const uint16_t* src = sg.in((const uint16_t*)w_kn, (size_t)K * N);
    uint16_t* d = sg.out((uint16_t*)dst, dst_elems);
    if (!src || !d) return sg.finish(cudaErrorMemoryAllocation);
    return sg.finish(launch_pack_slabs_from_kn(src, K, N, d, st));
}

int hm_gemv_bf16(const float* x, const void* w_bf16, int layout, int M, int K, int N, float* y, void* stream) {
    if (!x || !w_bf16 || !y || M < 1 || M > 16 || K < 1 || N < 1) return gfail(HM_ERR_INVALID, "hm_gemv_bf16: bad arguments (1 <= M <= 16)");
    if (layout == HM_LAYOUT_KN && N % 8 != 0) return gfail(HM_ERR_UNSUPPORTED, "hm_gemv_bf16: row-major [K,N] needs N to be a multiple of 8 (128-bit loads)");
    if (layout != HM_LAYOUT_KN && layout != HM_LAYOUT_SLAB128) return gfail(HM_ERR_INVALID, "hm_gemv_bf16: unknown layout");
    NEED_DEVICE();
    cudaStream_t st = (cudaStream_t)stream;
    Staging sg(st);
    const int nslabs = (N + SLAB - 1) / SLAB;
    const size_t w_elems = layout == HM_LAYOUT_KN ? (size_t)K * N : (size_t)nslabs * K * SLAB;
    const int Mcap = (M + MAX_M - 1) / MAX_M * MAX_M;
    // rows are processed in groups of up to 8; pad the activation rows so padded lanes read zeros
    const float* xd;
    const int tail = M % MAX_M;
    if (is_device_ptr(x) && (tail == 0 || tail == 1 || tail == 2 || tail == 4)) {
        xd = x;  // every row group has exactly the row count its kernel variant reads
    } else {
        float* xp = (float*)sg.scratch((size_t)Mcap * K * 4, true);
        if (!xp) return sg.finish(cudaErrorMemoryAllocation);
        sg.ok(cudaMemcpyAsync(xp, x, (size_t)M * K * 4, cudaMemcpyDefault, st));
        xd = xp;
    }
    const uint16_t* wd = sg.in((const uint16_t*)w_bf16, w_elems);
    float* yd = sg.out(y, (size_t)M * N);
    if (!wd || !yd) return sg.finish(cudaErrorMemoryAllocation);
    const int sms = sm_count_of_current_device();
    cudaError_t ce = cudaSuccess;
    for (int m0 = 0; m0 < M && ce == cudaSuccess; m0 += MAX_M) {
        const int mv = std::min(MAX_M, M - m0);
        const int mp = mv <= 1 ? 1 : mv <= 2 ? 2 : mv <= 4 ? 4 : 8;
        GemvArgs a{};
        a.W = wd;
        if (layout == HM_LAYOUT_KN) {
            a.slab_stride = SLAB * 2;
            a.row_stride = (long long)N * 2;
        } else {
            a.slab_stride = (long long)K * SLAB * 2;
            a.row_stride = SLAB * 2;
        }
        a.K = K;
        a.N = N;
        a.m_valid = mv;
        // same split policy as the engine: K shared by the CTAs of a cluster, reduced through
        // distributed shared memory; global partials + tickets when clusters are switched off
        const char* ncl = std::getenv("HM_NO_CLUSTER");  // read per call so a host can switch paths at run time
        const bool no_cluster = ncl && ncl[0] == '1';
        const int max_cl = gemv_max_cluster();
        if (!no_cluster) {
            gemv_pick_cluster(K, N, mp, sms, max_cl, &a.ksplit, &a.rows_per_split);
            a.cluster = a.ksplit > 1 && a.ksplit <= max_cl ? a.ksplit : 0;
        }
        if (no_cluster || (a.ksplit > 1 && a.cluster == 0)) {
            a.cluster = 0;
            gemv_pick_split(K, N, mp, sms, &a.ksplit, &a.rows_per_split);
        }
        a.x = xd + (size_t)m0 * K;
        a.ldx = K;
        a.pro = PRO_PLAIN;
        a.epi = EPI_STORE;
        a.y = yd + (size_t)m0 * N;
        a.ldy = N;
        const size_t pf = a.cluster ? 0 : gemv_partial_floats(N, a.ksplit, mp);
        if (pf) {
            ce = get_scratch(pf, (size_t)nslabs, &a.partial, &a.tickets);
            if (ce != cudaSuccess) break;
        }
        ce = get_wait_err(&a.err_flag);  // raised by the bounded waits of the staged / cluster variants
        if (ce != cudaSuccess) break;
        ce = launch_gemv_bf16(a, mp, st, false);
    }
    const bool synced = sg.staged();
    const int rc = sg.finish(ce);
    if (rc != HM_OK) return rc;
    // with device pointers only the call stays asynchronous; hm_dev_sync reports a wait that ran out
    if (synced && take_wait_err()) return gfail(HM_ERR_TIMEOUT, "hm_gemv_bf16: a bounded device-side wait ran out");
    return HM_OK;
}

int hm_gemm_bf16_tc(const float* x, const void* w_tc, int M, int K, int N, int ksplit, float* y, void* stream) {
    if (!x || !w_tc || !y || M < 1 || M > 64 || K < 1 || N < 1 || ksplit < 0 || ksplit > 16) return gfail(HM_ERR_INVALID, "hm_gemm_bf16_tc: bad arguments (1 <= M <= 64, 0 <= ksplit <= 16)");
    NEED_DEVICE();
    cudaStream_t st = (cudaStream_t)stream;
    Staging sg(st);
    const float* xd = sg.in(x, (size_t)M * K);
    const uint16_t* wd = sg.in((const uint16_t*)w_tc, tc_packed_elems(K, N));
    float* yd = sg.out(y, (size_t)M * N);
    if (!xd || !wd || !yd) return sg.finish(cudaErrorMemoryAllocation);
    int* err = nullptr;
    if (!sg.ok(get_wait_err(&err))) return sg.finish(cudaSuccess);
    TcArgs a{};
    a.W = wd;
    a.K = K;
    a.Kp = tc_padded_k(K);
    a.N = N;
    a.M = M;
    a.ksplit = ksplit ? ksplit : tc_pick_split(K, N, sm_count_of_current_device());
    a.epi = EPI_STORE;
    a.y = yd;
    a.ldy = N;
    a.err_flag = err;
    // packed activations live in the per-device scratch (grown on demand, shared by calls on this device)
    float* xp = nullptr;
    unsigned int* unused = nullptr;
    if (!sg.ok(get_scratch((tc_xpack_bytes(M, K) + 3) / 4, 1, &xp, &unused))) return sg.finish(cudaSuccess);
    a.xp = (const unsigned char*)xp;
    cudaError_t ce = launch_tc_pack_x(xd, K, M, K, nullptr, 0.f, xp, st, false);
    if (ce == cudaSuccess) ce = launch_gemm_tc(a, st, false);
    const bool synced = sg.staged();
    const int rc = sg.finish(ce);
    if (rc != HM_OK) return rc;
    // with device pointers only the call stays asynchronous; hm_dev_sync reports a wait that ran out
    if (synced && take_wait_err()) return gfail(HM_ERR_TIMEOUT, "hm_gemm_bf16_tc: a bounded device-side wait ran out");
    return HM_OK;
}

size_t hm_tc_packed_elems(int K, int N) { return (K < 1 || N < 1) ? 0 : tc_packed_elems(K, N); }

int hm_pack_bf16_tc(const void* w_kn, int K, int N, void* dst, void* stream) {
    if (!w_kn || !dst || K < 1 || N < 1) return gfail(HM_ERR_INVALID, "hm_pack_bf16_tc: bad arguments");
    NEED_DEVICE();
    cudaStream_t st = (cudaStream_t)stream;
    Staging sg(st);
    const uint16_t* sd = sg.in((const uint16_t*)w_kn, (size_t)K * N);
    const size_t n = tc_packed_elems(K, N);
    uint16_t* dd = sg.out((uint16_t*)dst, n);
    if (!sd || !dd) return sg.finish(cudaErrorMemoryAllocation);
    cudaError_t ce = cudaMemsetAsync(dd, 0, n * 2, st);
    if (ce == cudaSuccess) ce = launch_pack_tc(sd, N, K, true, dd, 0, -1, st);
    return sg.finish(ce);
}

int hm_gemv_quant(const float* x, const void* blocks, int dtype, int M, int K, int N, float* y, void* stream) {
    if (!x || !blocks || !y || M < 1 || M > 8 || K < 32 || N < 1) return gfail(HM_ERR_INVALID, "hm_gemv_quant: bad arguments (1 <= M <= 8)");
    const bool kq = dtype == HM_Q4_K || dtype == HM_Q6_K;
    if (dtype != HM_Q8_0 && dtype != HM_Q4_0 && !kq) return gfail(HM_ERR_UNSUPPORTED, "hm_gemv_quant: dtype must be HM_Q8_0, HM_Q4_0, HM_Q4_K or HM_Q6_K");
    if (K % (kq ? 256 : 32) != 0) return gfail(HM_ERR_INVALID, "hm_gemv_quant: K must be a multiple of the block size (32, or 256 for the K-quants)");
    NEED_DEVICE();
    cudaStream_t st = (cudaStream_t)stream;
    Staging sg(st);
    const int mp = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
    float* xp = (float*)sg.scratch((size_t)mp * K * 4, true);
    float* yd = sg.out(y, (size_t)M * N);
    if (!xp || !yd) return sg.finish(cudaErrorMemoryAllocation);
    sg.ok(cudaMemcpyAsync(xp, x, (size_t)M * K * 4, cudaMemcpyDefault, st));
    if (kq) {
        const size_t nsb = (size_t)N * (K / 256);
        const uint8_t* bd = sg.in((const uint8_t*)blocks, nsb * (dtype == HM_Q4_K ? 144 : 210));
        uint8_t* data = (uint8_t*)sg.scratch(kquant_data_bytes(K, N), true);
        uint8_t* types = (uint8_t*)sg.scratch(kquant_tiles(N), true);
        if (!bd || !data || !types) return sg.finish(cudaErrorMemoryAllocation);
        cudaError_t ce = launch_kquant_split(bd, N, K, dtype == HM_Q6_K, 0, -1, data, types, st);
        if (ce == cudaSuccess) {
            KQuantArgs a{};
            a.data = data;
            a.tile_type = types;
            a.K = K;
            a.N = N;
            a.m_valid = M;
            a.act_quant = 1;
            a.x = xp;
            a.ldx = K;
            a.pro = PRO_PLAIN;
            a.epi = EPI_STORE;
            a.y = yd;
            a.ldy = N;
            ce = launch_gemv_kquant(a, mp, sm_count_of_current_device(), st, false);
        }
        return sg.finish(ce);
    }
    const int q4 = dtype == HM_Q4_0;
    const size_t nb = (size_t)N * (K / 32);
    const uint8_t* bd = sg.in((const uint8_t*)blocks, nb * (q4 ? 18 : 34));
    uint16_t* scales = (uint16_t*)sg.scratch(quant_scale_elems(K, N) * 2, true);
    uint8_t* codes = (uint8_t*)sg.scratch(quant_code_bytes(K, N, q4), true);
    if (!bd || !scales || !codes) return sg.finish(cudaErrorMemoryAllocation);
    cudaError_t ce = launch_split_blocks(bd, N, K, q4, 0, -1, scales, codes, st);
    if (ce == cudaSuccess) {
        QuantArgs a{};
        ce = get_wait_err(&a.err_flag);
        a.scales = scales;
        a.codes = codes;
        a.q4 = q4;
        a.K = K;
        a.N = N;
        a.m_valid = M;
        a.x = xp;
        a.ldx = K;
        a.pro = PRO_PLAIN;
        a.epi = EPI_STORE;
        a.y = yd;
        a.ldy = N;
        if (ce == cudaSuccess) ce = launch_gemv_quant(a, mp, sm_count_of_current_device(), st, false);
    }
    const int rc = sg.finish(ce);  // the scratch copies above always stage, so this call synchronised
    if (rc != HM_OK) return rc;
    if (take_wait_err()) return gfail(HM_ERR_TIMEOUT, "hm_gemv_quant: a bounded device-side wait ran out");
    return HM_OK;
}

int hm_dequant(const void* blocks, int dtype, size_t n_blocks, float* out, void* stream) {
    if (!blocks || !out) return gfail(HM_ERR_INVALID, "hm_dequant: null argument");
    const bool kq = dtype == HM_Q4_K || dtype == HM_Q6_K;
    if (dtype != HM_Q8_0 && dtype != HM_Q4_0 && !kq) return gfail(HM_ERR_UNSUPPORTED, "hm_dequant: dtype must be HM_Q8_0, HM_Q4_0, HM_Q4_K or HM_Q6_K");
    if (n_blocks == 0) return HM_OK;
    NEED_DEVICE();
    cudaStream_t st = (cudaStream_t)stream;
    Staging sg(st);
    if (kq) {
        const uint8_t* bd = sg.in((const uint8_t*)blocks, n_blocks * (dtype == HM_Q4_K ? 144 : 210));
        float* od = sg.out(out, n_blocks * 256);
        if (!bd || !od) return sg.finish(cudaErrorMemoryAllocation);
        return sg.finish(launch_dequant_k(bd, n_blocks, dtype == HM_Q6_K, od, st));
    }
    const int q4 = dtype == HM_Q4_0;
    const uint8_t* bd = sg.in((const uint8_t*)blocks, n_blocks * (q4 ? 18 : 34));
    float* od = sg.out(out, n_blocks * 32);
    if (!bd || !od) return sg.finish(cudaErrorMemoryAllocation);
    return sg.finish(launch_dequant(bd, n_blocks, q4, od, st));
}

int hm_rms_norm(const float* x, const float* w, float eps, int rows, int n, float* out, void* stream) {
    if (!x || !w || !out || rows < 0 || n < 1) return gfail(HM_ERR_INVALID, "hm_rms_norm: bad arguments");
    if (rows == 0) return HM_OK;
    NEED_DEVICE();
    cudaStream_t st = (cudaStream_t)stream;
    Staging sg(st);
    const float* xd = sg.in(x, (size_t)rows * n);
    const float* wd = sg.in(w, (size_t)n);
    float* od = sg.out(out, (size_t)rows * n);
    if (!xd || !wd || !od) return sg.finish(cudaErrorMemoryAllocation);
    return sg.finish(launch_rms_norm(xd, wd, eps, rows, n, od, st));
}

int hm_qknorm_rope(float* x, int rows, int heads, int hd, const float* norm_w, float eps, const float* cos_rows, const float* sin_rows, void* stream) {
    if (!x || !cos_rows || !sin_rows || rows < 0 || heads < 1) return gfail(HM_ERR_INVALID, "hm_qknorm_rope: bad arguments");
    if (hd != 64 && hd != 128) return gfail(HM_ERR_UNSUPPORTED, "hm_qknorm_rope: head_dim must be 64 or 128");
    if (rows == 0) return HM_OK;
    NEED_DEVICE();
    cudaStream_t st = (cudaStream_t)stream;
    Staging sg(st);
    float* xd = sg.out(x, (size_t)rows * heads * hd, true);
    const float* nd = sg.in(norm_w, (size_t)hd);
    const float* cd = sg.in(cos_rows, (size_t)rows * hd);
    const float* sd = sg.in(sin_rows, (size_t)rows * hd);
    if (!xd || !cd || !sd) return sg.finish(cudaErrorMemoryAllocation);
    return sg.finish(launch_qknorm_rope(xd, rows, heads, hd, nd, eps, cd, sd, st));
}

int hm_attn_decode_paged(const float* q, const void* k_pages, const void* v_pages, int kv_dtype, const int32_t* page_table, const int32_t* kv_len, int B, int heads, int kv_heads, int hd,
                         int page_tokens, int max_pages, float* out, void* stream) {
    if (!q || !k_pages || !v_pages || !page_table || !kv_len || !out || B < 1 || heads < 1 || kv_heads < 1 || max_pages < 1)
        return gfail(HM_ERR_INVALID, "hm_attn_decode_paged: bad arguments");
    if (page_tokens != 16) return gfail(HM_ERR_UNSUPPORTED, "hm_attn_decode_paged: page size must be 16 tokens");
    if (hd != 64 && hd != 128) return gfail(HM_ERR_UNSUPPORTED, "hm_attn_decode_paged: head_dim must be 64 or 128");
    if (heads % kv_heads != 0 || heads / kv_heads > 8) return gfail(HM_ERR_UNSUPPORTED, "hm_attn_decode_paged: heads / kv_heads must be an integer <= 8");
    if (kv_dtype != HM_F32 && kv_dtype != HM_BF16) return gfail(HM_ERR_UNSUPPORTED, "hm_attn_decode_paged: cache dtype must be f32 or bf16");
    NEED_DEVICE();
    if (!is_device_ptr(k_pages) || !is_device_ptr(v_pages)) return gfail(HM_ERR_INVALID, "hm_attn_decode_paged: the page pools must live in device memory");
    cudaStream_t st = (cudaStream_t)stream;
    Staging sg(st);
    // A host kv_len is validated and sizes the split; a device kv_len is trusted (reading it back would
    // serialise the stream) and the split is sized for max_pages.
    int longest = max_pages * page_tokens;
    if (!is_device_ptr(kv_len)) {
        longest = 0;
        for (int b = 0; b < B; ++b) {
            if (kv_len[b] < 1 || kv_len[b] > max_pages * page_tokens) return gfail(HM_ERR_INVALID, "hm_attn_decode_paged: kv_len must be in [1, max_pages*page_tokens]");
            longest = std::max(longest, kv_len[b]);
        }
    }
    AttnArgs a{};
    a.q = sg.in(q, (size_t)B * heads * hd);
    a.k_pool = k_pages;
    a.v_pool = v_pages;
    a.page_table = sg.in(page_table, (size_t)B * max_pages);
    a.kv_len = sg.in(kv_len, (size_t)B);
    a.max_pages = max_pages;
    a.page_tokens = page_tokens;
    a.heads = heads;
    a.kv_heads = kv_heads;
    a.hd = hd;
    a.nsplit = attn_pick_nsplit(B, kv_heads, (longest + page_tokens - 1) / page_tokens, sm_count_of_current_device(), kv_dtype == HM_BF16);
    a.scale = (float)(1.0 / std::sqrt((double)hd));
    a.stream_pages = 1;
    if (!sg.ok(get_wait_err(&a.err_flag))) return sg.finish(cudaSuccess);
    a.out = sg.out(out, (size_t)B * heads * hd);
    if (a.nsplit > 1) {
        const size_t acc_f = (size_t)B * heads * a.nsplit * hd, ml_f = (size_t)B * heads * a.nsplit * 2;
        float* base = nullptr;
        cudaError_t se = get_scratch(acc_f + ml_f, (size_t)B * kv_heads, &base, &a.tickets);
        if (se != cudaSuccess) return sg.finish(se);
        a.part_acc = base;
        a.part_ml = base + acc_f;
    }
    if (!a.q || !a.page_table || !a.kv_len || !a.out) return sg.finish(cudaErrorMemoryAllocation);
    const cudaError_t le = launch_attn_decode(a, B, kv_dtype == HM_BF16, st, false);
    const bool synced = sg.staged();
    const int rc = sg.finish(le);
    if (rc != HM_OK) return rc;
    if (synced && take_wait_err()) return gfail(HM_ERR_TIMEOUT, "hm_attn_decode_paged: a bounded device-side wait ran out");
    return HM_OK;
}

int hm_argmax(const float* logits, int rows, int n, uint32_t* out, void* stream) {
    if (!logits || !out || rows < 0 || n < 1) return gfail(HM_ERR_INVALID, "hm_argmax: bad arguments");
    if (rows == 0) return HM_OK;
    NEED_DEVICE();
    cudaStream_t st = (cudaStream_t)stream;
    Staging sg(st);
    const float* ld = sg.in(logits, (size_t)rows * n);
    uint32_t* od = sg.out(out, (size_t)rows);
    if (!ld || !od) return sg.finish(cudaErrorMemoryAllocation);
    return sg.finish(launch_argmax_rows(ld, rows, n, od, st));
}

int hm_dev_alloc(size_t nbytes, void** out) {
    if (!out) return gfail(HM_ERR_INVALID, "null argument");
    NEED_DEVICE();
    cudaError_t e = cudaMalloc(out, nbytes);
    if (e != cudaSuccess) return gfail(HM_ERR_CUDA, std::string("cudaMalloc: ") + cudaGetErrorString(e));
    return HM_OK;
}
int hm_dev_free(void* p) {
    if (p && cudaFree(p) != cudaSuccess) return gfail(HM_ERR_CUDA, "cudaFree failed");
    return HM_OK;
}
int hm_dev_copy(void* dst, const void* src, size_t nbytes) {
    NEED_DEVICE();
    cudaError_t e = cudaMemcpy(dst, src, nbytes, cudaMemcpyDefault);
    if (e != cudaSuccess) return gfail(HM_ERR_CUDA, std::string("cudaMemcpy: ") + cudaGetErrorString(e));
    return HM_OK;
}
int hm_dev_set(int device) {
    NEED_DEVICE();
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return gfail(HM_ERR_INVALID, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    return HM_OK;
}
int hm_dev_mem_info(size_t* free_bytes, size_t* total_bytes) {
    if (!free_bytes || !total_bytes) return gfail(HM_ERR_INVALID, "null argument");
    NEED_DEVICE();
    cudaError_t e = cudaMemGetInfo(free_bytes, total_bytes);
    if (e != cudaSuccess) return gfail(HM_ERR_CUDA, std::string("cudaMemGetInfo: ") + cudaGetErrorString(e));
    return HM_OK;
}
int hm_dev_sync(void) {
    NEED_DEVICE();
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return gfail(HM_ERR_CUDA, std::string("cudaDeviceSynchronize: ") + cudaGetErrorString(e));
    if (take_wait_err()) return gfail(HM_ERR_TIMEOUT, "hm_dev_sync: a bounded device-side wait ran out in an earlier kernel");
    return HM_OK;
}

}  // extern "C"
