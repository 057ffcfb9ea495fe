// Engine implementation.  See engine.h.
#include "engine.h"
#include "gemm_tc.h"
#include "kquant.h"
#include "sampler.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstdio>
#include <cstring>

#include "loaders.h"

namespace hm {

#define HM_CUDA(call)                                      \
    do {                                                   \
        cudaError_t _e = (call);                           \
        if (_e != cudaSuccess) return cuda_fail(_e, #call); \
    } while (0)

size_t LinearW::bytes() const {
    if (kind == HM_BF16) return (size_t)((N + SLAB - 1) / SLAB) * K * SLAB * 2;
    if (kind == HM_Q8_0) return (size_t)N * (K / 32) * 34;
    if (kind == HM_Q4_0) return (size_t)N * (K / 32) * 18;
    if (kind == HM_Q4_K) return kq_bytes;
    return 0;
}

int Engine::fail(int code, const std::string& msg) {
    err = msg;
    return code;
}
int Engine::cuda_fail(cudaError_t e, const char* what) {
    err = std::string("CUDA error: ") + cudaGetErrorString(e) + " in " + what;
    return HM_ERR_CUDA;
}
bool Engine::set_device() { return cudaSetDevice(device_) == cudaSuccess; }

int Engine::create(const hm_config& cfg, int device, Engine** out, std::string* err) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        *err = "no CUDA device available (this engine has no CPU fallback)";
        return HM_ERR_CUDA;
    }
    if (device < 0 || device >= ndev) {
        *err = "device index out of range";
        return HM_ERR_INVALID;
    }
    if (cfg.hidden_size <= 0 || cfg.num_attention_heads <= 0 || cfg.num_hidden_layers <= 0 || cfg.vocab_size <= 0 || cfg.intermediate_size <= 0) {
        *err = "config has a non-positive dimension";
        return HM_ERR_INVALID;
    }
    Engine* e = new Engine();
    e->cfg_ = cfg;
    e->device_ = device;
    e->H_ = cfg.hidden_size;
    e->I_ = cfg.intermediate_size;
    e->heads_ = cfg.num_attention_heads;
    e->kvh_ = cfg.num_key_value_heads > 0 ? cfg.num_key_value_heads : cfg.num_attention_heads;
    e->hd_ = cfg.head_dim > 0 ? cfg.head_dim : cfg.hidden_size / cfg.num_attention_heads;
    e->cfg_.num_key_value_heads = e->kvh_;
    e->cfg_.head_dim = e->hd_;
    e->qdim_ = e->heads_ * e->hd_;
    e->kvdim_ = e->kvh_ * e->hd_;
    e->L_ = cfg.num_hidden_layers;
    e->V_ = cfg.vocab_size;
    e->cfg_.has_qkv_bias = 0;
    e->cfg_.has_qk_norm = 0;
    e->cfg_.weight_dtype = -1;
    auto bad = [&](const char* m) {
        *err = m;
        delete e;
        return HM_ERR_UNSUPPORTED;
    };
    if (e->hd_ != 64 && e->hd_ != 128) return bad("head_dim must be 64 or 128");
    if (e->heads_ % e->kvh_ != 0 || e->heads_ / e->kvh_ > 8) return bad("heads / kv_heads must be an integer <= 8");
    if (e->H_ % 32 != 0 || e->I_ % 64 != 0) return bad("hidden_size must be a multiple of 32 and intermediate_size of 64");
    if (cudaSetDevice(device) != cudaSuccess) return bad("cudaSetDevice failed");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) e->sm_count_ = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&e->stream_, cudaStreamNonBlocking) != cudaSuccess) return bad("cudaStreamCreate failed");
    e->layers_.resize(e->L_);
    const char* nopdl = std::getenv("HM_NO_PDL");
    e->pdl_ = !(nopdl && nopdl[0] == '1');
    const char* nocl = std::getenv("HM_NO_CLUSTER");
    e->use_clusters_ = !(nocl && nocl[0] == '1');
    e->max_cluster_ = gemv_max_cluster();
    const char* notc = std::getenv("HM_NO_TC");
    e->use_tc_ = !(notc && notc[0] == '1');
    *out = e;
    return HM_OK;
}

Engine::~Engine() {
    if (!set_device()) return;
    if (stream_) cudaStreamSynchronize(stream_);
    drop_host_logits_graph();
    if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
    if (graph_) cudaGraphDestroy(graph_);
    auto fr = [](void* p) {
        if (p) cudaFree(p);
    };
    fr(embed_); fr(final_norm_); fr(rope_cos_); fr(rope_sin_);
    for (auto& l : layers_) {
        fr(l.in_ln); fr(l.post_ln); fr(l.qkv_bias); fr(l.q_norm); fr(l.k_norm);
        for (LinearW* w : {&l.qkv, &l.o, &l.gu, &l.down}) { fr(w->slabs); fr(w->tc); fr(w->scales); fr(w->codes); fr(w->kq_data); fr(w->kq_tile_type); }
    }
    fr(lm_head_.slabs); fr(lm_head_.tc); fr(lm_head_.scales); fr(lm_head_.codes); fr(lm_head_.kq_data); fr(lm_head_.kq_tile_type);
    fr(xpack_); fr(xpack_attn_); fr(xpack_act_); fr(xpack_h_); fr(xpack_h2_); fr(ss_h_); fr(ss_h2_); fr(h_); fr(q_); fr(attn_); fr(act_); fr(qkv_raw_); fr(gu_raw_); fr(logits_); fr(amax_val_); fr(amax_idx_);
    fr(partial_); fr(tickets_); fr(att_acc_); fr(att_ml_); fr(att_tickets_); fr(err_flag_); fr(fin_ticket_);
    for (void* p : k_pool_) fr(p);
    for (void* p : v_pool_) fr(p);
    fr(qrows_img_); fr(qrows_bs_); fr(kqrows_codes_); fr(kqrows_actd_);
    fr(gemv_trace_); fr(smp_scaled_); fr(smp_count_); fr(smp_rng_); fr(smp_gen_start_); fr(smp_overflow_);
    fr(page_table_); fr(pos_dev_); fr(tokens_dev_); fr(next_dev_); fr(hist_dev_); fr(pf_tokens_); fr(pf_pos_); fr(pf_seq_);
    if (pin_u32_) cudaFreeHost(pin_u32_);
    if (pin_logits_) cudaFreeHost(pin_logits_);
    if (stream_) cudaStreamDestroy(stream_);
}

// ---- weight loading -----------------------------------------------------------------------

int Engine::stage(const void* host, size_t nbytes, void** dev) {
    HM_CUDA(cudaMalloc(dev, nbytes));
    cudaError_t e = cudaMemcpyAsync(*dev, host, nbytes, cudaMemcpyHostToDevice, stream_);
    if (e != cudaSuccess) {
        cudaFree(*dev);
        return cuda_fail(e, "cudaMemcpyAsync(H2D weights)");
    }
    return HM_OK;
}

// One part (n_part outputs starting at n_off) of a possibly fused projection with N_total
// outputs.  bf16 [out,in] goes to the slab layout; GGUF blocks [out, in/32] are split into
// scale and code arrays (rows of the parts are simply concatenated).
// rope_part: 1 = q or k rows, 2 = v rows of the fused QKV projection (0: any other projection)
int Engine::load_linear(LinearW& L, int K, int N_total, int n_off, int n_part, int interleave_which, int dtype, const void* host, size_t nbytes, int rope_part) {
    const bool kq = dtype == HM_Q4_K || dtype == HM_Q6_K;
    if (dtype != HM_BF16 && dtype != HM_Q8_0 && dtype != HM_Q4_0 && !kq)
        return fail(HM_ERR_UNSUPPORTED, "projection weights must be stored as bf16, Q8_0, Q4_0, Q4_K or Q6_K: this checkpoint holds f32 / f16 projections, and the f32-weight streaming kernel they need is not built");
    // Q4_K and Q6_K mix freely (per 32-row tile), as the Q4_K_M files of the Hub do; they are one family here
    const int family = kq ? (int)HM_Q4_K : dtype;
    if (L.kind >= 0 && L.kind != family) return fail(HM_ERR_UNSUPPORTED, "parts of a fused projection have different dtypes");
    if (cfg_.weight_dtype >= 0 && cfg_.weight_dtype != family && &L != &lm_head_)
        return fail(HM_ERR_UNSUPPORTED, "projection weights of one model must share a dtype family");
    if (&L != &lm_head_) cfg_.weight_dtype = family;
    const bool q = dtype != HM_BF16;
    if (q && K % 32 != 0) return fail(HM_ERR_INVALID, "quantised projection: in_features must be a multiple of 32");
    if (kq && K % 256 != 0) return fail(HM_ERR_INVALID, "K-quant projection: in_features must be a multiple of 256");
    if (kq && interleave_which < 0 && (n_off % 32 != 0 || (n_part % 32 != 0 && n_off + n_part != N_total)))
        return fail(HM_ERR_UNSUPPORTED, "K-quant parts of a fused projection must start and end on multiples of 32 rows");
    const size_t expect = kq ? (size_t)n_part * (K / 256) * (dtype == HM_Q4_K ? 144 : 210) : q ? (size_t)n_part * (K / 32) * (dtype == HM_Q8_0 ? 34 : 18) : (size_t)n_part * K * 2;
    if (nbytes != expect) return fail(HM_ERR_INVALID, "tensor byte size does not match its shape");
    L.K = K;
    L.N = N_total;
    L.kind = family;
    void* tmp = nullptr;
    int rc = stage(host, nbytes, &tmp);
    if (rc) return rc;
    cudaError_t ce = cudaSuccess;
    if (!q) {
        if (!L.slabs) {
            const size_t bytes = (size_t)((N_total + SLAB - 1) / SLAB) * K * SLAB * 2;
            ce = cudaMalloc(&L.slabs, bytes);
            if (ce == cudaSuccess) ce = cudaMemsetAsync(L.slabs, 0, bytes, stream_);
        }
        if (ce == cudaSuccess) ce = launch_pack_slabs_from_nk((const uint16_t*)tmp, n_part, K, L.slabs, n_off, interleave_which, stream_);
        if (use_tc_ && ce == cudaSuccess) {
            // second copy for passes over more than 8 rows (same 64 + 64 gate/up interleave per 128 features)
            if (!L.tc) {
                const size_t bytes = tc_packed_elems(K, N_total) * 2;
                ce = cudaMalloc(&L.tc, bytes);
                if (ce == cudaSuccess) ce = cudaMemsetAsync(L.tc, 0, bytes, stream_);
            }
            if (ce == cudaSuccess) ce = launch_pack_tc((const uint16_t*)tmp, n_part, K, false, L.tc, n_off, interleave_which, stream_);
        }
    }
    // the QKV projection of a quantised model rotates in its own epilogue when a rotation pair can share a 32-row tile
    // and there is no QK-norm (which needs a whole head in one CTA); all three parts must then agree
    const bool rope_rows = q && rope_part != 0 && !cfg_.has_qk_norm && (hd_ / 2) % 16 == 0 && qdim_ % 32 == 0 && kvdim_ % 32 == 0;
    if (q && rope_part != 0) {
        if (L.loaded_parts > 0 && L.rope_rows != rope_rows) {
            cudaFree(tmp);
            return fail(HM_ERR_STATE, "q, k and v projections of a layer disagree on their row layout");
        }
        L.rope_rows = rope_rows;
    }
    const int rope_hd = rope_rows && rope_part == 1 ? hd_ : 0;
    if (!q) {
    } else if (kq) {
        if (!L.kq_data) {
            ce = cudaMalloc(&L.kq_data, kquant_data_bytes(K, N_total));
            if (ce == cudaSuccess) ce = cudaMalloc(&L.kq_tile_type, kquant_tiles(N_total));
            if (ce == cudaSuccess) ce = cudaMemsetAsync(L.kq_data, 0, kquant_data_bytes(K, N_total), stream_);
            if (ce == cudaSuccess) ce = cudaMemsetAsync(L.kq_tile_type, 0, kquant_tiles(N_total), stream_);
        }
        // gate and up share a tile (16 + 16 rows): they must be of one type for the tile's decode
        if (interleave_which >= 0 && L.loaded_parts > 0 && L.kq_part_type != dtype) {
            cudaFree(tmp);
            return fail(HM_ERR_UNSUPPORTED, "gate and up projections of a layer must share one K-quant type");
        }
        L.kq_part_type = dtype;
        if (dtype == HM_Q6_K) L.kq_has_q6 = true;
        if (ce == cudaSuccess) ce = launch_kquant_split((const uint8_t*)tmp, n_part, K, dtype == HM_Q6_K, n_off, interleave_which, L.kq_data, L.kq_tile_type, stream_, rope_hd);
        L.kq_bytes += nbytes;
        quant_ = true;
    } else {
        const int q4 = dtype == HM_Q4_0;
        if (!L.scales) {
            ce = cudaMalloc(&L.scales, quant_scale_elems(K, N_total) * 2);
            if (ce == cudaSuccess) ce = cudaMalloc(&L.codes, quant_code_bytes(K, N_total, q4));
            if (ce == cudaSuccess) ce = cudaMemsetAsync(L.scales, 0, quant_scale_elems(K, N_total) * 2, stream_);
            if (ce == cudaSuccess) ce = cudaMemsetAsync(L.codes, 0, quant_code_bytes(K, N_total, q4), stream_);
        }
        if (ce == cudaSuccess) ce = launch_split_blocks((const uint8_t*)tmp, n_part, K, q4, n_off, interleave_which, L.scales, L.codes, stream_, rope_hd);
        quant_ = true;
    }
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(stream_);
    cudaFree(tmp);
    if (ce != cudaSuccess) return cuda_fail(ce, "load_linear");
    L.loaded_parts++;
    return HM_OK;
}

int Engine::load_vec_f32(float** dst, size_t n_total, size_t off, int dtype, const void* host, size_t n, size_t nbytes) {
    size_t esz = dtype == HM_F32 ? 4 : (dtype == HM_BF16 || dtype == HM_F16) ? 2 : 0;
    if (!esz) return fail(HM_ERR_UNSUPPORTED, "norm / bias tensors must be f32, bf16 or f16");
    if (nbytes != n * esz || off + n > n_total) return fail(HM_ERR_INVALID, "tensor byte size does not match its shape");
    if (!*dst) {
        HM_CUDA(cudaMalloc(dst, n_total * 4));
        HM_CUDA(cudaMemsetAsync(*dst, 0, n_total * 4, stream_));
    }
    void* tmp = nullptr;
    int rc = stage(host, nbytes, &tmp);
    if (rc) return rc;
    cudaError_t ce = launch_convert_to_f32(tmp, dtype, n, *dst + off, stream_);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(stream_);
    cudaFree(tmp);
    if (ce != cudaSuccess) return cuda_fail(ce, "load_vec_f32");
    return HM_OK;
}

static bool parse_layer_name(const std::string& name, const char* prefix, int* layer, std::string* rest) {
    const size_t pl = std::strlen(prefix);
    if (name.compare(0, pl, prefix) != 0) return false;
    const size_t dot = name.find('.', pl);
    if (dot == std::string::npos) return false;
    *layer = std::atoi(name.substr(pl, dot - pl).c_str());
    *rest = name.substr(dot + 1);
    return true;
}

// Names and rules of load_transformer_weights (src/hf/weights.rs:267-417) and of the GGUF
// variant (src/gguf.rs:589-708).
int Engine::load_tensor(const char* cname, int dtype, const int64_t* shape, int ndim, const void* host, size_t nbytes) {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (finalized_) return fail(HM_ERR_STATE, "weights already finalised");
    if (!cname || !shape || !host || ndim < 1 || ndim > 2) return fail(HM_ERR_INVALID, "load_tensor: bad arguments");
    const std::string name(cname);
    size_t n = 1;
    for (int i = 0; i < ndim; ++i) {
        if (shape[i] <= 0) return fail(HM_ERR_INVALID, "load_tensor: non-positive dimension in " + name);
        n *= (size_t)shape[i];
    }
    auto shape2 = [&](int64_t a, int64_t b) { return ndim == 2 && shape[0] == a && shape[1] == b; };
    auto shape1 = [&](int64_t a) { return ndim == 1 && shape[0] == a; };
    auto bad_shape = [&]() { return fail(HM_ERR_INVALID, "unexpected shape for tensor " + name); };

    if (name == "model.embed_tokens.weight" || name == "token_embd.weight") {
        if (!shape2(V_, H_)) return bad_shape();
        if (embed_) return fail(HM_ERR_STATE, "embedding loaded twice");
        // Gather table: kept as bf16 rows when the file is bf16 (widening a bf16 row to f32 on
        // the fly equals Homura's up-front conversion, src/hf/weights.rs:284-292), else f32.
        if (dtype == HM_BF16) {
            if (nbytes != n * 2) return bad_shape();
            int rc = stage(host, nbytes, &embed_);
            if (rc) return rc;
            HM_CUDA(cudaStreamSynchronize(stream_));
            embed_dtype_ = HM_BF16;
        } else if (dtype == HM_F32 || dtype == HM_F16) {
            float* t = nullptr;
            int rc = load_vec_f32(&t, n, 0, dtype, host, n, nbytes);
            if (rc) return rc;
            embed_ = t;
            embed_dtype_ = HM_F32;
        } else if (dtype == HM_Q8_0 || dtype == HM_Q4_0) {
            if (nbytes != n / 32 * (dtype == HM_Q8_0 ? 34u : 18u)) return bad_shape();
            void* tmp = nullptr;
            int rc = stage(host, nbytes, &tmp);
            if (rc) return rc;
            cudaError_t ce = cudaMalloc(&embed_, n * 4);
            if (ce == cudaSuccess) ce = launch_dequant((const uint8_t*)tmp, n / 32, dtype == HM_Q4_0, (float*)embed_, stream_);
            if (ce == cudaSuccess) ce = cudaStreamSynchronize(stream_);
            cudaFree(tmp);
            if (ce != cudaSuccess) return cuda_fail(ce, "embedding dequant");
            embed_dtype_ = HM_F32;
        } else if (dtype == HM_Q4_K || dtype == HM_Q6_K) {
            if (n % 256 != 0 || nbytes != n / 256 * (dtype == HM_Q4_K ? 144u : 210u)) return bad_shape();
            void* tmp = nullptr;
            int rc = stage(host, nbytes, &tmp);
            if (rc) return rc;
            cudaError_t ce = cudaMalloc(&embed_, n * 4);
            if (ce == cudaSuccess) ce = launch_dequant_k((const uint8_t*)tmp, n / 256, dtype == HM_Q6_K, (float*)embed_, stream_);
            if (ce == cudaSuccess) ce = cudaStreamSynchronize(stream_);
            cudaFree(tmp);
            if (ce != cudaSuccess) return cuda_fail(ce, "embedding dequant");
            embed_dtype_ = HM_F32;
        } else {
            return fail(HM_ERR_UNSUPPORTED, "unsupported embedding dtype");
        }
        // Tied LM head = the embedding, transposed (src/hf/weights.rs:101-113).
        if (cfg_.tie_word_embeddings) {
            if (dtype == HM_F32 || dtype == HM_F16)
                return fail(HM_ERR_UNSUPPORTED, "tied LM head from an f32/f16 embedding is outside this engine's path (bf16 or quantised only)");
            return load_linear(lm_head_, H_, V_, 0, V_, -1, dtype, host, nbytes);
        }
        return HM_OK;
    }
    if (name == "model.norm.weight" || name == "output_norm.weight") {
        if (!shape1(H_)) return bad_shape();
        return load_vec_f32(&final_norm_, H_, 0, dtype, host, n, nbytes);
    }
    if (name == "lm_head.weight" || name == "output.weight") {
        if (!shape2(V_, H_)) return bad_shape();
        if (cfg_.tie_word_embeddings) return HM_OK;  // ignored, as in src/hf/weights.rs:383-387
        return load_linear(lm_head_, H_, V_, 0, V_, -1, dtype, host, nbytes);
    }
    int li = -1;
    std::string rest;
    const bool hf = parse_layer_name(name, "model.layers.", &li, &rest);
    const bool gg = !hf && parse_layer_name(name, "blk.", &li, &rest);
    if (!hf && !gg) return fail(HM_ERR_INVALID, "unknown tensor name: " + name);
    if (li < 0 || li >= L_) return fail(HM_ERR_INVALID, "layer index out of range in " + name);
    LayerW& Lw = layers_[li];
    auto is = [&](const char* a, const char* b) { return rest == (hf ? a : b); };
    const int QKV = qdim_ + 2 * kvdim_;
    if (is("input_layernorm.weight", "attn_norm.weight")) return shape1(H_) ? load_vec_f32(&Lw.in_ln, H_, 0, dtype, host, n, nbytes) : bad_shape();
    if (is("post_attention_layernorm.weight", "ffn_norm.weight")) return shape1(H_) ? load_vec_f32(&Lw.post_ln, H_, 0, dtype, host, n, nbytes) : bad_shape();
    if (is("self_attn.q_proj.weight", "attn_q.weight")) return shape2(qdim_, H_) ? load_linear(Lw.qkv, H_, QKV, 0, qdim_, -1, dtype, host, nbytes, 1) : bad_shape();
    if (is("self_attn.k_proj.weight", "attn_k.weight")) return shape2(kvdim_, H_) ? load_linear(Lw.qkv, H_, QKV, qdim_, kvdim_, -1, dtype, host, nbytes, 1) : bad_shape();
    if (is("self_attn.v_proj.weight", "attn_v.weight")) return shape2(kvdim_, H_) ? load_linear(Lw.qkv, H_, QKV, qdim_ + kvdim_, kvdim_, -1, dtype, host, nbytes, 2) : bad_shape();
    if (is("self_attn.o_proj.weight", "attn_output.weight")) return shape2(H_, qdim_) ? load_linear(Lw.o, qdim_, H_, 0, H_, -1, dtype, host, nbytes) : bad_shape();
    if (is("mlp.gate_proj.weight", "ffn_gate.weight")) return shape2(I_, H_) ? load_linear(Lw.gu, H_, 2 * I_, 0, I_, 0, dtype, host, nbytes) : bad_shape();
    if (is("mlp.up_proj.weight", "ffn_up.weight")) return shape2(I_, H_) ? load_linear(Lw.gu, H_, 2 * I_, I_, I_, 1, dtype, host, nbytes) : bad_shape();
    if (is("mlp.down_proj.weight", "ffn_down.weight")) return shape2(H_, I_) ? load_linear(Lw.down, I_, H_, 0, H_, -1, dtype, host, nbytes) : bad_shape();
    if (is("self_attn.q_proj.bias", "attn_q.bias")) {
        cfg_.has_qkv_bias = 1;
        return shape1(qdim_) ? load_vec_f32(&Lw.qkv_bias, QKV, 0, dtype, host, n, nbytes) : bad_shape();
    }
    if (is("self_attn.k_proj.bias", "attn_k.bias")) return shape1(kvdim_) ? load_vec_f32(&Lw.qkv_bias, QKV, qdim_, dtype, host, n, nbytes) : bad_shape();
    if (is("self_attn.v_proj.bias", "attn_v.bias")) return shape1(kvdim_) ? load_vec_f32(&Lw.qkv_bias, QKV, qdim_ + kvdim_, dtype, host, n, nbytes) : bad_shape();
    if (is("self_attn.q_norm.weight", "attn_q_norm.weight")) {
        // a quantised QKV projection stored for rotation in its own epilogue cannot take a QK-norm afterwards
        for (const LayerW& l : layers_)
            if (l.qkv.rope_rows) return fail(HM_ERR_STATE, "QK-norm weights must be loaded before the quantised q / k / v projections (hm_model_load does so)");
        cfg_.has_qk_norm = 1;
        return shape1(hd_) ? load_vec_f32(&Lw.q_norm, hd_, 0, dtype, host, n, nbytes) : bad_shape();
    }
    if (is("self_attn.k_norm.weight", "attn_k_norm.weight")) return shape1(hd_) ? load_vec_f32(&Lw.k_norm, hd_, 0, dtype, host, n, nbytes) : bad_shape();
    return fail(HM_ERR_INVALID, "unknown tensor name: " + name);
}

int Engine::finalize() {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (finalized_) return HM_OK;
    if (!embed_) return fail(HM_ERR_STATE, "missing weight: model.embed_tokens.weight");
    if (!final_norm_) return fail(HM_ERR_STATE, "missing weight: model.norm.weight");
    if (lm_head_.kind < 0) return fail(HM_ERR_STATE, "missing weight: lm_head.weight");
    for (int i = 0; i < L_; ++i) {
        const LayerW& l = layers_[i];
        const std::string p = "missing weight in layer " + std::to_string(i) + ": ";
        if (!l.in_ln) return fail(HM_ERR_STATE, p + "input_layernorm");
        if (!l.post_ln) return fail(HM_ERR_STATE, p + "post_attention_layernorm");
        if (l.qkv.loaded_parts != 3) return fail(HM_ERR_STATE, p + "q/k/v projection");
        if (l.o.loaded_parts != 1) return fail(HM_ERR_STATE, p + "o projection");
        if (l.gu.loaded_parts != 2) return fail(HM_ERR_STATE, p + "gate/up projection");
        if (l.down.loaded_parts != 1) return fail(HM_ERR_STATE, p + "down projection");
        if (cfg_.has_qk_norm && (!l.q_norm || !l.k_norm)) return fail(HM_ERR_STATE, p + "q_norm/k_norm");
    }
    std::vector<float> c, s;
    build_rope_table(hd_, cfg_.max_position_embeddings, cfg_.rope_theta, &c, &s);
    HM_CUDA(cudaMalloc(&rope_cos_, c.size() * 4));
    HM_CUDA(cudaMalloc(&rope_sin_, s.size() * 4));
    HM_CUDA(cudaMemcpy(rope_cos_, c.data(), c.size() * 4, cudaMemcpyHostToDevice));
    HM_CUDA(cudaMemcpy(rope_sin_, s.data(), s.size() * 4, cudaMemcpyHostToDevice));
    HM_CUDA(cudaMalloc(&err_flag_, 4));
    HM_CUDA(cudaMemset(err_flag_, 0, 4));
    HM_CUDA(cudaMalloc(&fin_ticket_, 4));
    HM_CUDA(cudaMemset(fin_ticket_, 0, 4));
    finalized_ = true;
    return HM_OK;
}

uint64_t Engine::weight_bytes() const {
    uint64_t b = lm_head_.bytes();
    for (auto& l : layers_) b += l.qkv.bytes() + l.o.bytes() + l.gu.bytes() + l.down.bytes();
    return b;
}

// ---- scratch ---------------------------------------------------------------------------------

int Engine::ensure_scratch(int rows) {
    const bool tall = use_tc_ && !quant_;  // prefill chunks of TC_ROWS rows on the tensor-core GEMM
    if (tall || quant_) rows = std::max(rows, TC_ROWS);
    const int cap = (rows + MAX_M - 1) / MAX_M * MAX_M;
    if (cap <= scratch_rows_) return HM_OK;
    auto re = [&](auto** p, size_t count) -> cudaError_t {
        if (*p) cudaFree(*p);
        *p = nullptr;
        cudaError_t e = cudaMalloc((void**)p, count * sizeof(**p));
        if (e == cudaSuccess) e = cudaMemset(*p, 0, count * sizeof(**p));
        return e;
    };
    const int nslabs_v = (V_ + SLAB - 1) / SLAB;
    HM_CUDA(re(&h_, (size_t)cap * H_));
    HM_CUDA(re(&q_, (size_t)cap * qdim_));
    HM_CUDA(re(&attn_, (size_t)cap * qdim_));
    HM_CUDA(re(&act_, (size_t)cap * I_));
    HM_CUDA(re(&logits_, (size_t)cap * V_));
    HM_CUDA(re(&amax_val_, (size_t)cap * nslabs_v));
    HM_CUDA(re(&amax_idx_, (size_t)cap * nslabs_v));
    if (!tall && use_tc_ && lm_head_.kind == HM_BF16 && lm_head_.tc) {
        // a GGUF model whose LM head is the bf16 embedding: passes over more than 8 rows run that one projection on the tensor cores
        xpack_bytes_ = tc_xpack_bytes(TC_ROWS, H_);
        HM_CUDA(re(&xpack_, xpack_bytes_));
    }
    if (quant_) {
        // digit planes / Q8_K codes of up to 64 rows of the widest projection input (launch_gemm_quant, launch_gemm_q4k)
        qrows_k_ = std::max(std::max(H_, qdim_), I_);
        if (qrows_k_ % 256 == 0) {
            HM_CUDA(re(&kqrows_codes_, kquant_rows_code_bytes(qrows_k_)));
            HM_CUDA(re(&kqrows_actd_, kquant_rows_scale_floats(qrows_k_)));
        }
        HM_CUDA(re(&qrows_img_, quant_rows_image_words(qrows_k_)));
        HM_CUDA(re(&qrows_bs_, quant_rows_scale_floats(qrows_k_)));
    }
    if (quant_ || tall) {
        HM_CUDA(re(&qkv_raw_, (size_t)cap * (qdim_ + 2 * kvdim_)));
        HM_CUDA(re(&gu_raw_, (size_t)cap * 2 * I_));
        if (tall) {
            xpack_bytes_ = tc_xpack_bytes(TC_ROWS, std::max(std::max(H_, qdim_), I_));
            HM_CUDA(re(&xpack_, xpack_bytes_));
            HM_CUDA(re(&xpack_attn_, tc_xpack_bytes(TC_ROWS, qdim_)));
            HM_CUDA(re(&xpack_act_, tc_xpack_bytes(TC_ROWS, I_)));
            HM_CUDA(re(&xpack_h_, tc_xpack_bytes(TC_ROWS, H_)));
            HM_CUDA(re(&xpack_h2_, tc_xpack_bytes(TC_ROWS, H_)));
            HM_CUDA(re(&ss_h_, (size_t)((H_ + 127) / 128) * TC_ROWS));
            HM_CUDA(re(&ss_h2_, (size_t)((H_ + 127) / 128) * TC_ROWS));
        }
    }
    // split-K scratch sized for the worst projection at M = 8
    size_t pf = 0;
    int max_slabs = nslabs_v;
    auto acc = [&](const LinearW& w) {
        if (w.kind != HM_BF16) return;
        for (int M : {1, 2, 4, 8}) {
            int ks, rps;
            gemv_pick_split(w.K, w.N, M, sm_count_, &ks, &rps);
            pf = std::max(pf, gemv_partial_floats(w.N, ks, M));
        }
        max_slabs = std::max(max_slabs, (w.N + SLAB - 1) / SLAB);
    };
    for (auto& l : layers_) { acc(l.qkv); acc(l.o); acc(l.gu); acc(l.down); }
    acc(lm_head_);
    partial_floats_ = std::max<size_t>(pf, 1);
    HM_CUDA(re(&partial_, partial_floats_));
    HM_CUDA(re(&tickets_, (size_t)max_slabs));
    scratch_rows_ = cap;
    return HM_OK;
}

// ---- KV cache --------------------------------------------------------------------------------

int Engine::kv_alloc(int batch, int max_seq_len, int page_tokens, int kv_dtype) {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (!finalized_) return fail(HM_ERR_STATE, "kv_alloc before weights are finalised");
    if (batch_ > 0) return fail(HM_ERR_STATE, "KV cache already allocated");
    if (batch < 1 || max_seq_len < 1) return fail(HM_ERR_INVALID, "kv_alloc: batch and max_seq_len must be positive");
    if (page_tokens != 16) return fail(HM_ERR_UNSUPPORTED, "kv_alloc: page size must be 16 tokens");
    if (kv_dtype != HM_F32 && kv_dtype != HM_BF16) return fail(HM_ERR_UNSUPPORTED, "kv_alloc: cache dtype must be f32 or bf16");
    if (max_seq_len > cfg_.max_position_embeddings) return fail(HM_ERR_INVALID, "kv_alloc: max_seq_len exceeds max_position_embeddings (RoPE table)");
    kv_bf16_ = kv_dtype == HM_BF16;
    page_tokens_ = page_tokens;
    max_pages_ = (max_seq_len + page_tokens - 1) / page_tokens;
    const size_t n_pages = (size_t)batch * max_pages_;
    const size_t page_elems = (size_t)kvh_ * page_tokens * hd_;
    const size_t pool_bytes = n_pages * page_elems * (kv_bf16_ ? 2 : 4);
    k_pool_.assign(L_, nullptr);
    v_pool_.assign(L_, nullptr);
    for (int l = 0; l < L_; ++l) {
        HM_CUDA(cudaMalloc(&k_pool_[l], pool_bytes));
        HM_CUDA(cudaMalloc(&v_pool_[l], pool_bytes));
        HM_CUDA(cudaMemset(k_pool_[l], 0, pool_bytes));
        HM_CUDA(cudaMemset(v_pool_[l], 0, pool_bytes));
    }
    // Every sequence owns max_pages pages; the mapping is a fixed pseudo-random permutation of
    // the pool so that consecutive logical pages are not physically adjacent.
    std::vector<int32_t> perm(n_pages);
    for (size_t i = 0; i < n_pages; ++i) perm[i] = (int32_t)i;
    uint64_t st = 0x9E3779B97F4A7C15ull;
    for (size_t i = n_pages; i > 1; --i) {
        st ^= st << 13; st ^= st >> 7; st ^= st << 17;
        std::swap(perm[i - 1], perm[st % i]);
    }
    HM_CUDA(cudaMalloc(&page_table_, n_pages * 4));
    HM_CUDA(cudaMemcpy(page_table_, perm.data(), n_pages * 4, cudaMemcpyHostToDevice));
    HM_CUDA(cudaMalloc(&pos_dev_, batch * 4));
    HM_CUDA(cudaMemset(pos_dev_, 0, batch * 4));
    HM_CUDA(cudaMalloc(&tokens_dev_, batch * 4));
    HM_CUDA(cudaMemset(tokens_dev_, 0, batch * 4));
    HM_CUDA(cudaMalloc(&next_dev_, batch * 4));
    HM_CUDA(cudaMemset(next_dev_, 0, batch * 4));
    HM_CUDA(cudaMalloc(&hist_dev_, (size_t)batch * (max_seq_len + 1) * 4));
    HM_CUDA(cudaMemset(hist_dev_, 0, (size_t)batch * (max_seq_len + 1) * 4));
    HM_CUDA(cudaMalloc(&pf_tokens_, (size_t)max_seq_len * 4));
    HM_CUDA(cudaMalloc(&pf_pos_, (size_t)max_seq_len * 4));
    HM_CUDA(cudaMalloc(&pf_seq_, (size_t)max_seq_len * 4));
    pin_u32_cap_ = std::max<size_t>((size_t)3 * max_seq_len, (size_t)batch * (max_seq_len + 6)) + 16;  // the last word receives the device error word
    HM_CUDA(cudaMallocHost(&pin_u32_, pin_u32_cap_ * 4));
    pin_u32_[pin_u32_cap_ - 1] = 0;
    HM_CUDA(cudaMalloc(&smp_rng_, (size_t)batch * 8));
    HM_CUDA(cudaMemset(smp_rng_, 0, (size_t)batch * 8));
    HM_CUDA(cudaMalloc(&smp_gen_start_, (size_t)batch * 4));
    HM_CUDA(cudaMemset(smp_gen_start_, 0, (size_t)batch * 4));
    HM_CUDA(cudaMalloc(&smp_overflow_, (size_t)batch * 4));
    HM_CUDA(cudaMemset(smp_overflow_, 0, (size_t)batch * 4));
    len_.assign(batch, 0);
    gen_start_.assign(batch, 0);
    batch_ = batch;
    max_seq_ = max_seq_len;
    int rc = ensure_scratch(std::max(batch, MAX_M));
    if (rc) return rc;
    // attention split scratch
    // sized for the decode step (one row per sequence)
    // up to 1024 tokens of capacity the splits of a (row, KV head) are one cluster of at most 16 CTAs, one page
    // per split while the context allows (a page is about 0.65 us of dependent instructions, so pages of a
    // split cost more than the wider merge); longer caches need more CTAs than a cluster holds and merge
    // through global scratch + ticket
    // ... and only while the (row, KV head) pairs alone do not fill the GPU: with half an SM's worth of pairs or more
    // the launch is a throughput problem (64 sequences stream 39 MB of pages per layer), which the cost model
    // of attn_pick_nsplit answers with few splits of many pages each, i.e. the bulk-copy ring kernel
    att_cluster_ = use_clusters_ && max_pages_ <= 64 && (long)batch * kvh_ < sm_count_ / 2;
    att_nsplit_ = att_cluster_ ? attn_pick_cluster(max_pages_, std::min(max_cluster_, 16)) : attn_pick_nsplit(batch, kvh_, max_pages_, sm_count_, kv_bf16_);
    HM_CUDA(cudaMalloc(&att_acc_, (size_t)scratch_rows_ * heads_ * att_nsplit_ * hd_ * 4));
    HM_CUDA(cudaMalloc(&att_ml_, (size_t)scratch_rows_ * heads_ * att_nsplit_ * 2 * 4));
    HM_CUDA(cudaMalloc(&att_tickets_, (size_t)scratch_rows_ * kvh_ * 4));
    HM_CUDA(cudaMemset(att_tickets_, 0, (size_t)scratch_rows_ * kvh_ * 4));
#ifdef HM_PHASE_TRACE
    if (const char* gt = std::getenv("HM_GEMV_TRACE")) {
        if (gt[0] == '1' && !gemv_trace_) {
            HM_CUDA(cudaMalloc(&gemv_trace_, 512 * 16 * sizeof(unsigned long long)));
            HM_CUDA(cudaMemset(gemv_trace_, 0, 512 * 16 * sizeof(unsigned long long)));
        }
    }
#endif
    return capture_decode_graph();
}

// Releases the KV cache and everything sized by it (decode graph, token history, staging, sampler state), so
// that kv_alloc may be called again with another batch, length or page dtype.  Weights stay resident.
int Engine::kv_free() {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (batch_ == 0) return HM_OK;
    HM_CUDA(cudaStreamSynchronize(stream_));
    drop_host_logits_graph();
    if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
    if (graph_) cudaGraphDestroy(graph_);
    graph_exec_ = nullptr;
    graph_ = nullptr;
    auto fr = [](auto*& p) {
        if (p) cudaFree(p);
        p = nullptr;
    };
    for (void*& p : k_pool_) fr(p);
    for (void*& p : v_pool_) fr(p);
    k_pool_.clear();
    v_pool_.clear();
    fr(page_table_); fr(pos_dev_); fr(tokens_dev_); fr(next_dev_); fr(hist_dev_); fr(pf_tokens_); fr(pf_pos_); fr(pf_seq_);
    fr(att_acc_); fr(att_ml_); fr(att_tickets_);
    fr(smp_scaled_); fr(smp_count_); fr(smp_rng_); fr(smp_gen_start_); fr(smp_overflow_);
    if (pin_u32_) cudaFreeHost(pin_u32_);
    pin_u32_ = nullptr;
    pin_u32_cap_ = 0;
    len_.clear();
    gen_start_.clear();
    batch_ = 0;
    max_seq_ = 0;
    launches_per_step_ = 0;
    return HM_OK;
}

int Engine::launch_step() {
    HM_CUDA(cudaGraphLaunch(graph_exec_, stream_));
    return HM_OK;
}

int Engine::kv_reset(int seq) {
    if (batch_ == 0) return HM_OK;  // reset before first use is a no-op (src/hf/model.rs:232-237)
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (seq >= batch_) return fail(HM_ERR_INVALID, "kv_reset: sequence index out of range");
    HM_CUDA(cudaStreamSynchronize(stream_));
    if (seq < 0) {
        std::fill(len_.begin(), len_.end(), 0);
        HM_CUDA(cudaMemset(pos_dev_, 0, batch_ * 4));
    } else {
        len_[seq] = 0;
        HM_CUDA(cudaMemset(pos_dev_ + seq, 0, 4));
    }
    return HM_OK;
}

int Engine::kv_len(int seq, int* out) {
    if (!out) return fail(HM_ERR_INVALID, "kv_len: null output");
    if (batch_ == 0) {
        *out = 0;
        return HM_OK;
    }
    if (seq < 0 || seq >= batch_) return fail(HM_ERR_INVALID, "kv_len: sequence index out of range");
    *out = len_[seq];
    return HM_OK;
}

int Engine::kv_append(int seq, int layer, const float* k_rows, const float* v_rows, int n_new, int advance) {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (batch_ == 0) return fail(HM_ERR_STATE, "kv_append before kv_alloc");
    if (seq < 0 || seq >= batch_ || layer < 0 || layer >= L_ || n_new < 0) return fail(HM_ERR_INVALID, "kv_append: index out of range");
    if (len_[seq] + n_new > max_seq_)
        return fail(HM_ERR_KV_FULL, "KV cache full (" + std::to_string(len_[seq]) + " + " + std::to_string(n_new) + " > " + std::to_string(max_seq_) + ")");
    if (n_new > 0 && (k_rows || v_rows)) {
        const size_t bytes = (size_t)kvh_ * n_new * hd_ * 4;
        float *dk = nullptr, *dv = nullptr;
        if (k_rows) {
            HM_CUDA(cudaMalloc(&dk, bytes));
            HM_CUDA(cudaMemcpyAsync(dk, k_rows, bytes, cudaMemcpyHostToDevice, stream_));
        }
        if (v_rows) {
            HM_CUDA(cudaMalloc(&dv, bytes));
            HM_CUDA(cudaMemcpyAsync(dv, v_rows, bytes, cudaMemcpyHostToDevice, stream_));
        }
        KvDesc kv{k_pool_[layer], v_pool_[layer], page_table_, max_pages_, page_tokens_, kvh_, hd_, kv_bf16_ ? 1 : 0};
        cudaError_t ce = launch_kv_write_rows(kv, seq, len_[seq], dk, dv, n_new, stream_);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(stream_);
        if (dk) cudaFree(dk);
        if (dv) cudaFree(dv);
        if (ce != cudaSuccess) return cuda_fail(ce, "kv_append");
    }
    if (advance) {
        len_[seq] += n_new;
        HM_CUDA(cudaMemcpy(pos_dev_ + seq, &len_[seq], 4, cudaMemcpyHostToDevice));
    }
    return HM_OK;
}

int Engine::kv_view(int seq, int layer, float* k_out, float* v_out) {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (batch_ == 0) return fail(HM_ERR_STATE, "kv_view before kv_alloc");
    if (seq < 0 || seq >= batch_ || layer < 0 || layer >= L_ || !k_out || !v_out) return fail(HM_ERR_INVALID, "kv_view: bad arguments");
    const int len = len_[seq];
    if (len == 0) return HM_OK;
    const size_t bytes = (size_t)kvh_ * len * hd_ * 4;
    float *dk = nullptr, *dv = nullptr;
    HM_CUDA(cudaMalloc(&dk, bytes));
    HM_CUDA(cudaMalloc(&dv, bytes));
    KvDesc kv{k_pool_[layer], v_pool_[layer], page_table_, max_pages_, page_tokens_, kvh_, hd_, kv_bf16_ ? 1 : 0};
    cudaError_t ce = launch_kv_read_rows(kv, seq, len, dk, dv, stream_);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(k_out, dk, bytes, cudaMemcpyDeviceToHost, stream_);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(v_out, dv, bytes, cudaMemcpyDeviceToHost, stream_);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(stream_);
    cudaFree(dk);
    cudaFree(dv);
    if (ce != cudaSuccess) return cuda_fail(ce, "kv_view");
    return HM_OK;
}

// ---- the pass ----------------------------------------------------------------------------------

enum ProfClass { PC_EMBED = 0, PC_QKV, PC_ATTN, PC_O, PC_GATE_UP, PC_DOWN, PC_LM_HEAD, PC_SAMPLE, PC_COUNT };
static const char* kProfNames[PC_COUNT] = {"embed", "qkv_rope_kvwrite", "attention", "o_proj_residual", "gate_up_swiglu", "down_residual", "lm_head", "argmax"};

void Engine::prof_mark(int) {}

static int pad_m(int m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : 8; }

// Projection over up to TC_ROWS rows per launch on the tensor cores (gemm_tc.cu): one kernel packs
// the activations (folding an RMSNorm when norm_w is given), the GEMM applies bias and residual on store.
int Engine::enqueue_linear_tc(const LinearW& L, int M, const float* x, int ldx, const float* norm_w, int epi, float* y, int ldy, const float* bias, const float* resid, int layer, const int32_t* row_pos,
                              const int32_t* row_seq, int* launches, const unsigned char* prepacked, unsigned char* pack_out, const TcFuse* fuse) {
    if (!L.tc) return fail(HM_ERR_STATE, "tensor-core weight copy missing");
    for (int m0 = 0; m0 < M; m0 += TC_ROWS) {
        const int mc = std::min(TC_ROWS, M - m0);
        if (tc_xpack_bytes(mc, L.K) > xpack_bytes_) return fail(HM_ERR_STATE, "activation pack scratch too small");
        cudaError_t ce = cudaSuccess;
        if (!prepacked) {  // the producer did not write the tile image itself
            unsigned long long* ptr = nullptr;
#ifdef HM_PHASE_TRACE
            if (gemv_trace_ && *launches < 512) ptr = gemv_trace_ + (size_t)*launches * 16;
#endif
            ce = launch_tc_pack_x(x + (size_t)m0 * ldx, ldx, mc, L.K, norm_w, (float)cfg_.rms_norm_eps, xpack_, stream_, pdl_, ptr);
            if (ce != cudaSuccess) return cuda_fail(ce, "activation pack launch");
            ++*launches;
        }
        TcArgs a{};
        a.W = L.tc;
        a.K = L.K;
        a.Kp = tc_padded_k(L.K);
        a.N = L.N;
        a.M = mc;
        a.ksplit = tc_pick_split(L.K, L.N, sm_count_);
        a.xp = prepacked ? prepacked : xpack_;
        a.xp_out = pack_out;
        a.xp_mpad = tc_mpad(mc);
        if (fuse) {
            a.ss_in = fuse->ss_in;
            a.ss_parts = fuse->ss_parts;
            a.xp_next = fuse->xp_next;
            a.next_norm_w = fuse->next_norm_w;
            a.ss_out = fuse->ss_out;
        }
        a.epi = epi;
        a.bias = bias;
        a.resid = resid ? resid + (size_t)m0 * ldy : nullptr;
        a.y = y + (size_t)m0 * ldy;
        a.ldy = ldy;
        a.q_dim = qdim_;
        a.kv_dim = kvdim_;
        a.hd = hd_;
        a.has_qk_norm = cfg_.has_qk_norm;
        a.eps = (float)cfg_.rms_norm_eps;
        if (layer >= 0) {
            a.q_norm_w = layers_[layer].q_norm;
            a.k_norm_w = layers_[layer].k_norm;
            a.kv = KvDesc{k_pool_[layer], v_pool_[layer], page_table_, max_pages_, page_tokens_, kvh_, hd_, kv_bf16_ ? 1 : 0};
        }
        a.rope_cos = rope_cos_;
        a.rope_sin = rope_sin_;
        a.row_pos = row_pos ? row_pos + m0 : nullptr;
        a.row_seq = row_seq ? row_seq + m0 : nullptr;
        a.seq_base = m0;
        if (epi == EPI_LOGITS) {
            const int nblocks = (L.N + SLAB - 1) / SLAB;
            a.amax_val = amax_val_ + (size_t)m0 * nblocks;
            a.amax_idx = amax_idx_ + (size_t)m0 * nblocks;
        }
        a.err_flag = err_flag_;
#ifdef HM_PHASE_TRACE
        if (gemv_trace_ && *launches < 512) a.trace = gemv_trace_ + (size_t)*launches * 16;
#endif
        ce = launch_gemm_tc(a, stream_, pdl_);
        if (ce != cudaSuccess) return cuda_fail(ce, "tensor-core projection launch");
        ++*launches;
    }
    return HM_OK;
}

RopeEpi Engine::rope_epi(int layer, const int32_t* row_pos, const int32_t* row_seq, int m0) const {
    RopeEpi r{};
    r.q_dim = qdim_;
    r.kv_dim = kvdim_;
    r.hd = hd_;
    r.rope_cos = rope_cos_;
    r.rope_sin = rope_sin_;
    r.row_pos = row_pos + m0;
    r.row_seq = row_seq ? row_seq + m0 : nullptr;
    r.seq_base = m0;
    r.kv = KvDesc{k_pool_[layer], v_pool_[layer], page_table_, max_pages_, page_tokens_, kvh_, hd_, kv_bf16_ ? 1 : 0};
    return r;
}

int Engine::enqueue_linear(const LinearW& L, int M, const float* x, int ldx, int pro, const float* norm_w, int epi, float* y, int ldy, const float* bias, const float* resid, int layer,
                           const int32_t* row_pos, const int32_t* row_seq, float* amax_val, int32_t* amax_idx, int* launches, const ArgmaxFold* fold) {
    // Q8_0 / Q4_0 projections over more than eight rows (prefill chunks, larger batches): the rows become digit planes once
    // and 64-row launches multiply them, instead of every CTA of an 8-row launch packing its own
    if ((L.kind == HM_Q8_0 || L.kind == HM_Q4_0) && M > MAX_M && qrows_img_ && L.K <= qrows_k_ && (epi == EPI_STORE || epi == EPI_SWIGLU || epi == EPI_QKV_ROPE)) {
        QuantArgs probe{};
        probe.x = x;
        probe.ldx = ldx;
        probe.K = L.K;
        probe.norm_w = pro == PRO_RMSNORM ? norm_w : nullptr;
        probe.codes = L.codes;
        probe.scales = L.scales;
        if (quant_rows_supported(probe)) {
            for (int m0 = 0; m0 < M; m0 += TC_ROWS) {
                QuantArgs a{};
                a.err_flag = err_flag_;
                a.scales = L.scales;
                a.codes = L.codes;
                a.q4 = L.kind == HM_Q4_0;
                a.K = L.K;
                a.N = L.N;
                a.m_valid = std::min(TC_ROWS, M - m0);
                a.x = x + (size_t)m0 * ldx;
                a.ldx = ldx;
                a.pro = pro;
                a.norm_w = norm_w;
                a.eps = (float)cfg_.rms_norm_eps;
                a.epi = epi;
                a.y = y + (size_t)m0 * ldy;
                a.ldy = ldy;
                a.bias = bias;
                a.resid = resid ? resid + (size_t)m0 * ldy : nullptr;
                if (epi == EPI_QKV_ROPE) {
                    if (!L.rope_rows || layer < 0) return fail(HM_ERR_STATE, "projection rows are not in rotation-pair order");
                    a.rope = rope_epi(layer, row_pos, row_seq, m0);
                }
                const cudaError_t ce = launch_gemm_quant(a, qrows_img_, qrows_bs_, sm_count_, stream_, pdl_, launches);
                if (ce != cudaSuccess) return cuda_fail(ce, "quantised projection over a row block");
            }
            pf_ptr_ = nullptr;
            pf_bytes_ = 0;
            return HM_OK;
        }
    }
    // K-quant projections (quantised activations) over more than eight rows: the rows are quantised to Q8_K once
    // and 64-row launches multiply the codes on the integer tensor-core path
    if (L.kind == HM_Q4_K && &L != &lm_head_ && M > MAX_M && kqrows_codes_ && L.K <= qrows_k_ && L.K % 256 == 0 &&
        (epi == EPI_STORE || epi == EPI_SWIGLU || epi == EPI_QKV_ROPE)) {
        KQuantArgs probe{};
        probe.x = x;
        probe.ldx = ldx;
        probe.K = L.K;
        probe.norm_w = pro == PRO_RMSNORM ? norm_w : nullptr;
        probe.data = L.kq_data;
        if (kquant_rows_supported(probe)) {
            for (int m0 = 0; m0 < M; m0 += TC_ROWS) {
                KQuantArgs a{};
                a.err_flag = err_flag_;
                a.data = L.kq_data;
                a.tile_type = L.kq_tile_type;
                a.K = L.K;
                a.N = L.N;
                a.m_valid = std::min(TC_ROWS, M - m0);
                a.act_quant = 1;
                a.has_q6 = L.kq_has_q6 ? 1 : 0;
                a.x = x + (size_t)m0 * ldx;
                a.ldx = ldx;
                a.pro = pro;
                a.norm_w = norm_w;
                a.eps = (float)cfg_.rms_norm_eps;
                a.epi = epi;
                a.y = y + (size_t)m0 * ldy;
                a.ldy = ldy;
                a.bias = bias;
                a.resid = resid ? resid + (size_t)m0 * ldy : nullptr;
                if (epi == EPI_QKV_ROPE) {
                    if (!L.rope_rows || layer < 0) return fail(HM_ERR_STATE, "projection rows are not in rotation-pair order");
                    a.rope = rope_epi(layer, row_pos, row_seq, m0);
                }
                const cudaError_t ce = launch_gemm_q4k(a, kqrows_codes_, kqrows_actd_, sm_count_, stream_, pdl_, launches);
                if (ce != cudaSuccess) return cuda_fail(ce, "Q4_K projection over a row block");
            }
            pf_ptr_ = nullptr;
            pf_bytes_ = 0;
            return HM_OK;
        }
    }
    for (int m0 = 0; m0 < M; m0 += MAX_M) {
        const int mv = std::min(MAX_M, M - m0), mp = pad_m(mv);
        cudaError_t ce;
        if (L.kind == HM_BF16) {
            GemvArgs a{};
            a.W = L.slabs;
            a.err_flag = err_flag_;
#ifdef HM_PHASE_TRACE
            if (gemv_trace_ && *launches < 512) a.trace = gemv_trace_ + (size_t)*launches * 16;
#endif
            if (m0 == 0) {
                a.pf_ptr = pf_ptr_;
                a.pf_bytes = pf_bytes_;
            }
            a.slab_stride = (long long)L.K * SLAB * 2;
            a.row_stride = SLAB * 2;
            a.K = L.K;
            a.N = L.N;
            a.m_valid = mv;
            if (use_clusters_) {
                gemv_pick_cluster(L.K, L.N, mp, sm_count_, max_cluster_, &a.ksplit, &a.rows_per_split);
                a.cluster = a.ksplit > 1 && a.ksplit <= max_cluster_ ? a.ksplit : 0;
            }
            if (!use_clusters_ || (a.ksplit > 1 && a.cluster == 0)) {
                a.cluster = 0;
                gemv_pick_split(L.K, L.N, mp, sm_count_, &a.ksplit, &a.rows_per_split);
            }
            a.x = x + (size_t)m0 * ldx;
            a.ldx = ldx;
            a.pro = pro;
            a.norm_w = norm_w;
            a.eps = (float)cfg_.rms_norm_eps;
            a.epi = epi;
            a.y = y + (size_t)m0 * ldy;
            a.ldy = ldy;
            a.bias = bias;
            a.resid = resid ? resid + (size_t)m0 * ldy : nullptr;
            a.q_dim = qdim_;
            a.kv_dim = kvdim_;
            a.hd = hd_;
            a.has_qk_norm = cfg_.has_qk_norm;
            if (layer >= 0) {
                a.q_norm_w = layers_[layer].q_norm;
                a.k_norm_w = layers_[layer].k_norm;
                a.kv = KvDesc{k_pool_[layer], v_pool_[layer], page_table_, max_pages_, page_tokens_, kvh_, hd_, kv_bf16_ ? 1 : 0};
            }
            a.rope_cos = rope_cos_;
            a.rope_sin = rope_sin_;
            a.row_pos = row_pos ? row_pos + m0 : nullptr;
            a.row_seq = row_seq ? row_seq + m0 : nullptr;
            a.seq_base = m0;
            const int nslabs = (L.N + SLAB - 1) / SLAB;
            a.amax_val = amax_val ? amax_val + (size_t)m0 * nslabs : nullptr;
            a.amax_idx = amax_idx ? amax_idx + (size_t)m0 * nslabs : nullptr;
            a.partial = partial_;
            a.tickets = tickets_;
            if (fold) {
                a.fin_ticket = fin_ticket_;
                a.next_tok = fold->next_tok + m0;
                a.feed_tok = fold->feed_tok ? fold->feed_tok + m0 : nullptr;
                a.pos = fold->pos ? fold->pos + m0 : nullptr;
                a.hist = fold->hist ? fold->hist + (size_t)m0 * fold->hist_stride : nullptr;
                a.hist_stride = fold->hist_stride;
            }
            if (a.cluster == 0 && gemv_partial_floats(L.N, a.ksplit, mp) > partial_floats_) return fail(HM_ERR_STATE, "split-K scratch too small");
            ce = launch_gemv_bf16(a, mp, stream_, pdl_);
        } else if (L.kind == HM_Q4_K) {
            KQuantArgs a{};
            a.data = L.kq_data;
            a.tile_type = L.kq_tile_type;
            a.K = L.K;
            a.N = L.N;
            a.m_valid = mv;
            // layer projections quantise the activation row to Q8_K; the LM head runs f32 x dequantised weights
            a.act_quant = &L != &lm_head_;
            a.x = x + (size_t)m0 * ldx;
            a.ldx = ldx;
            a.pro = pro;
            a.norm_w = norm_w;
            a.eps = (float)cfg_.rms_norm_eps;
            a.epi = epi;
            a.y = y + (size_t)m0 * ldy;
            a.ldy = ldy;
            a.bias = bias;
            a.resid = resid ? resid + (size_t)m0 * ldy : nullptr;
            if (epi == EPI_QKV_ROPE) {
                if (!L.rope_rows || layer < 0) return fail(HM_ERR_STATE, "projection rows are not in rotation-pair order");
                a.rope = rope_epi(layer, row_pos, row_seq, m0);
            }
            ce = launch_gemv_kquant(a, mp, sm_count_, stream_, pdl_);
        } else {
            QuantArgs a{};
            a.err_flag = err_flag_;
#ifdef HM_PHASE_TRACE
            if (gemv_trace_ && *launches < 512) a.trace = gemv_trace_ + (size_t)*launches * 16;
#endif
            a.scales = L.scales;
            a.codes = L.codes;
            a.q4 = L.kind == HM_Q4_0;
            a.K = L.K;
            a.N = L.N;
            a.m_valid = mv;
            a.x = x + (size_t)m0 * ldx;
            a.ldx = ldx;
            a.pro = pro;
            a.norm_w = norm_w;
            a.eps = (float)cfg_.rms_norm_eps;
            a.epi = epi;
            a.y = y + (size_t)m0 * ldy;
            a.ldy = ldy;
            a.bias = bias;
            a.resid = resid ? resid + (size_t)m0 * ldy : nullptr;
            if (epi == EPI_QKV_ROPE) {
                if (!L.rope_rows || layer < 0) return fail(HM_ERR_STATE, "projection rows are not in rotation-pair order");
                a.rope = rope_epi(layer, row_pos, row_seq, m0);
            }
            ce = launch_gemv_quant(a, mp, sm_count_, stream_, pdl_);
        }
        if (ce != cudaSuccess) return cuda_fail(ce, "projection launch");
        ++*launches;
    }
    pf_ptr_ = nullptr;
    pf_bytes_ = 0;
    return HM_OK;
}

int Engine::enqueue_pass(int M, const uint32_t* tokens_dev, const int32_t* row_pos, const int32_t* row_seq, int lm_row0, int lm_rows, bool advance, uint32_t* next_dev, uint32_t* feed_dev,
                         int32_t* pos_dev, uint32_t* hist_dev, int* launches) {
    (void)advance;
    cudaError_t ce = cudaSuccess;
    auto want = [&](int cls) { return only_class_ < 0 || only_class_ == cls; };
    if (want(PC_EMBED)) {
        ce = launch_embed_gather(embed_, embed_dtype_ == HM_BF16 ? 1 : 0, tokens_dev, M, H_, V_, h_, err_flag_, stream_, pdl_);
        if (ce != cudaSuccess) return cuda_fail(ce, "embed_gather");
        ++*launches;
    }
    const int QKV = qdim_ + 2 * kvdim_;
    const float eps = (float)cfg_.rms_norm_eps;
    // more than 8 rows of a bf16 model: tensor-core projections with the epilogues as kernels of their own
    const bool tall = use_tc_ && !quant_ && M > MAX_M;
    // Weight prefetch, decode passes of bf16 models: every kernel asks the L2 for the weights of the
    // kernel two launches ahead, so HBM keeps streaming while the short dependent kernels run.
    const bool pf = use_prefetch_ && !quant_ && !tall && only_class_ < 0;
    auto prefetch = [&](const LinearW* w, size_t off = 0, size_t cap = ~(size_t)0) {
        pf_ptr_ = nullptr;
        pf_bytes_ = 0;
        if (!pf || !w || !w->slabs || off >= w->bytes()) return;
        pf_ptr_ = (const char*)w->slabs + off;
        pf_bytes_ = std::min(cap, w->bytes() - off);
    };
    constexpr size_t LM_PF = 24u << 20;  // the LM head does not fit the L2: only its first 2 x 24 MB are fetched early
    int rc;
    // passes of 9..64 rows: the attention output and the SwiGLU output go straight into the packed
    // activation tiles of the next tensor-core GEMM (no packing launch in between) ...
    const bool direct_pack = tall && M <= TC_ROWS && qdim_ % 64 == 0 && I_ % 64 == 0;
    // ... and so does the hidden state after the O and down projections, whose RMSNorm is split between the
    // producer's epilogue (weight multiply, sums of squares) and the consumer's (row factor)
    const bool fused = direct_pack && H_ % 128 == 0;
    for (int l = 0; l < L_; ++l) {
        const LayerW& w = layers_[l];
        KvDesc kv{k_pool_[l], v_pool_[l], page_table_, max_pages_, page_tokens_, kvh_, hd_, kv_bf16_ ? 1 : 0};
        if (!want(PC_QKV)) {
        } else if (tall && fused && l > 0) {
            // the previous layer's down projection left (hidden * input_layernorm weight) packed, with the rows' sums of squares
            TcFuse f;
            f.ss_in = ss_h_;
            f.ss_parts = H_ / 128;
            rc = enqueue_linear_tc(w.qkv, M, h_, H_, nullptr, EPI_QKV_ROPE, q_, qdim_, w.qkv_bias, nullptr, l, row_pos, row_seq, launches, xpack_h_, nullptr, &f);
            if (rc) return rc;
        } else if (tall) {
            rc = enqueue_linear_tc(w.qkv, M, h_, H_, w.in_ln, EPI_QKV_ROPE, q_, qdim_, w.qkv_bias, nullptr, l, row_pos, row_seq, launches);
            if (rc) return rc;
        } else if (w.qkv.kind == HM_BF16 || w.qkv.rope_rows) {
            prefetch(&w.o);
            rc = enqueue_linear(w.qkv, M, h_, H_, PRO_RMSNORM, w.in_ln, EPI_QKV_ROPE, q_, qdim_, w.qkv_bias, nullptr, l, row_pos, row_seq, nullptr, nullptr, launches);
            if (rc) return rc;
        } else {
            rc = enqueue_linear(w.qkv, M, h_, H_, PRO_RMSNORM, w.in_ln, EPI_STORE, qkv_raw_, QKV, w.qkv_bias, nullptr, l, row_pos, row_seq, nullptr, nullptr, launches);
            if (rc) return rc;
            ce = launch_post_qkv(qkv_raw_, M, heads_, kvh_, hd_, cfg_.has_qk_norm, w.q_norm, w.k_norm, (float)cfg_.rms_norm_eps, rope_cos_, rope_sin_, row_pos, row_seq, kv, q_, stream_, pdl_);
            if (ce != cudaSuccess) return cuda_fail(ce, "post_qkv");
            ++*launches;
        }
        AttnArgs at{};
        at.q = q_;
        at.k_pool = k_pool_[l];
        at.v_pool = v_pool_[l];
        at.page_table = page_table_;
        at.row_seq = row_seq;
        at.row_pos = row_pos;
        at.kv_len = nullptr;
        at.max_pages = max_pages_;
        at.page_tokens = page_tokens_;
        at.heads = heads_;
        at.kv_heads = kvh_;
        at.hd = hd_;
        // fewer splits when the rows alone fill the SMs: about two CTAs per SM on the cluster path (caches
        // of up to 1024 tokens), the kernel's cost model on the long-context path
        at.nsplit = std::min(att_nsplit_, att_cluster_ ? std::max(1, (2 * sm_count_ + M * kvh_ - 1) / (M * kvh_)) : attn_pick_nsplit(M, kvh_, max_pages_, sm_count_, kv_bf16_));
        at.cluster = att_cluster_ ? 1 : 0;
        at.stream_pages = 1;
        if (direct_pack) {
            at.xp_out = xpack_attn_;
            at.xp_mpad = tc_mpad(M);
        }
#ifdef HM_PHASE_TRACE
        if (gemv_trace_ && *launches < 512) at.trace = gemv_trace_ + (size_t)*launches * 16;
#endif
        // decode passes: one row per sequence (prefill chunks write several positions of one sequence); launches of at most two
        // CTAs per SM are latency-bound and keep all their pages resident, larger ones keep their shared memory small
        at.early_pages = row_seq == nullptr ? ((long)M * kvh_ * at.nsplit <= 2L * sm_count_ ? 2 : 1) : 0;
        at.err_flag = err_flag_;
        at.scale = (float)(1.0 / std::sqrt((double)hd_));  // src/hf/emitter.rs:719
        at.out = attn_;
        at.part_acc = att_acc_;
        at.part_ml = att_ml_;
        at.tickets = att_tickets_;
        if (pf) {
            at.pf_ptr = w.gu.slabs;
            at.pf_bytes = w.gu.bytes();
        }
        if (want(PC_ATTN)) {
            ce = launch_attn_decode(at, M, kv_bf16_, stream_, pdl_);
            if (ce != cudaSuccess) return cuda_fail(ce, "attention launch");
            ++*launches;
        }
        if (want(PC_O) && tall) {
            TcFuse f;
            if (fused) {
                f.xp_next = xpack_h2_;
                f.next_norm_w = w.post_ln;
                f.ss_out = ss_h2_;
            }
            rc = enqueue_linear_tc(w.o, M, attn_, qdim_, nullptr, EPI_STORE, h_, H_, nullptr, h_, l, row_pos, row_seq, launches, direct_pack ? xpack_attn_ : nullptr, nullptr, fused ? &f : nullptr);
            if (rc) return rc;
        } else if (want(PC_O)) {
            prefetch(&w.down);
            rc = enqueue_linear(w.o, M, attn_, qdim_, PRO_PLAIN, nullptr, EPI_STORE, h_, H_, nullptr, h_, l, row_pos, row_seq, nullptr, nullptr, launches);
            if (rc) return rc;
        }
        if (!want(PC_GATE_UP)) {
        } else if (tall && fused) {
            TcFuse f;
            f.ss_in = ss_h2_;
            f.ss_parts = H_ / 128;
            rc = enqueue_linear_tc(w.gu, M, h_, H_, nullptr, EPI_SWIGLU, act_, I_, nullptr, nullptr, l, row_pos, row_seq, launches, xpack_h2_, xpack_act_, &f);
            if (rc) return rc;
        } else if (tall) {
            rc = enqueue_linear_tc(w.gu, M, h_, H_, w.post_ln, EPI_SWIGLU, act_, I_, nullptr, nullptr, l, row_pos, row_seq, launches, nullptr, direct_pack ? xpack_act_ : nullptr);
            if (rc) return rc;
        } else if (w.gu.kind == HM_BF16) {
            if (l + 1 < L_) prefetch(&layers_[l + 1].qkv);
            else if (lm_rows > 0) prefetch(&lm_head_, 0, LM_PF);
            rc = enqueue_linear(w.gu, M, h_, H_, PRO_RMSNORM, w.post_ln, EPI_SWIGLU, act_, I_, nullptr, nullptr, l, row_pos, row_seq, nullptr, nullptr, launches);
            if (rc) return rc;
        } else {
            // gate and up rows sit interleaved 16 + 16 in every 32-row tile: SwiGLU in the epilogue
            rc = enqueue_linear(w.gu, M, h_, H_, PRO_RMSNORM, w.post_ln, EPI_SWIGLU, act_, I_, nullptr, nullptr, l, row_pos, row_seq, nullptr, nullptr, launches);
            if (rc) return rc;
        }
        if (want(PC_DOWN) && tall) {
            TcFuse f;
            if (fused) {  // for the next layer's QKV projection, or for the LM head after the last layer
                f.xp_next = xpack_h_;
                f.next_norm_w = l + 1 < L_ ? layers_[l + 1].in_ln : final_norm_;
                f.ss_out = ss_h_;
            }
            rc = enqueue_linear_tc(w.down, M, act_, I_, nullptr, EPI_STORE, h_, H_, nullptr, h_, l, row_pos, row_seq, launches, direct_pack ? xpack_act_ : nullptr, nullptr, fused ? &f : nullptr);
            if (rc) return rc;
        } else if (want(PC_DOWN)) {
            if (l + 1 == L_ && lm_rows > 0) prefetch(&lm_head_, LM_PF, LM_PF);
            rc = enqueue_linear(w.down, M, act_, I_, PRO_PLAIN, nullptr, EPI_STORE, h_, H_, nullptr, h_, l, row_pos, row_seq, nullptr, nullptr, launches);
            if (rc) return rc;
        }
    }
    if (lm_rows > 0) {
        const int nslabs = (V_ + SLAB - 1) / SLAB;
        const float* x = h_ + (size_t)lm_row0 * H_;
        const bool lm_tall = use_tc_ && lm_head_.kind == HM_BF16 && lm_head_.tc && lm_rows > MAX_M;
        const bool slab_argmax = lm_head_.kind == HM_BF16;  // per-block argmax partials from the projection's epilogue
        const bool fold_argmax = slab_argmax && !lm_tall;    // the streaming kernel's last epilogue also produces the greedy token
        lm_folds_argmax_ = fold_argmax;
        if (want(PC_LM_HEAD) && lm_tall && fused && lm_row0 == 0 && lm_rows == M) {
            TcFuse f;
            f.ss_in = ss_h_;
            f.ss_parts = H_ / 128;
            rc = enqueue_linear_tc(lm_head_, lm_rows, x, H_, nullptr, EPI_LOGITS, logits_, V_, nullptr, nullptr, -1, nullptr, nullptr, launches, xpack_h_, nullptr, &f);
            if (rc) return rc;
        } else if (want(PC_LM_HEAD) && lm_tall) {
            rc = enqueue_linear_tc(lm_head_, lm_rows, x, H_, final_norm_, EPI_LOGITS, logits_, V_, nullptr, nullptr, -1, nullptr, nullptr, launches);
            if (rc) return rc;
        } else if (want(PC_LM_HEAD)) {
            const ArgmaxFold fold{next_dev, feed_dev, pos_dev, hist_dev, max_seq_ + 1};
            float* lm_dst = (lm_out_ && fold_argmax) ? lm_out_ : logits_;
            rc = slab_argmax ? enqueue_linear(lm_head_, lm_rows, x, H_, PRO_RMSNORM, final_norm_, EPI_LOGITS, lm_dst, V_, nullptr, nullptr, -1, nullptr, nullptr, amax_val_, amax_idx_, launches, &fold)
                             : enqueue_linear(lm_head_, lm_rows, x, H_, PRO_RMSNORM, final_norm_, EPI_STORE, logits_, V_, nullptr, nullptr, -1, nullptr, nullptr, nullptr, nullptr, launches);
            if (rc) return rc;
        }
        if (want(PC_SAMPLE) && !fold_argmax) {
            ce = slab_argmax ? launch_argmax_finish(amax_val_, amax_idx_, nslabs, lm_rows, next_dev, feed_dev, pos_dev, hist_dev, max_seq_ + 1, stream_, pdl_)
                             : launch_argmax_finish(logits_, nullptr, V_, lm_rows, next_dev, feed_dev, pos_dev, hist_dev, max_seq_ + 1, stream_, pdl_);
            if (ce != cudaSuccess) return cuda_fail(ce, "argmax_finish");
            ++*launches;
        }
    }
    return HM_OK;
}

int Engine::capture_decode_graph() {
    int launches = 0;
    HM_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_pass(batch_, tokens_dev_, pos_dev_, nullptr, 0, batch_, true, next_dev_, tokens_dev_, pos_dev_, hist_dev_, &launches);
    cudaGraph_t g = nullptr;
    cudaError_t ce = cudaStreamEndCapture(stream_, &g);
    if (rc) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaStreamEndCapture");
    graph_ = g;
    HM_CUDA(cudaGraphInstantiate(&graph_exec_, graph_, 0));
    launches_per_step_ = launches;
    return HM_OK;
}

// The device error word (raised by a token id out of range, or by a bounded device-side wait that ran out)
// travels back with the results of every pass: queue_error_copy() before the pass's synchronisation,
// check_device_error() after it.
int Engine::queue_error_copy() {
    HM_CUDA(cudaMemcpyAsync(pin_u32_ + pin_u32_cap_ - 1, err_flag_, 4, cudaMemcpyDeviceToHost, stream_));
    return HM_OK;
}

int Engine::check_device_error() {
    const uint32_t flag = pin_u32_[pin_u32_cap_ - 1];
    if (flag) {
        pin_u32_[pin_u32_cap_ - 1] = 0;
        cudaMemsetAsync(err_flag_, 0, 4, stream_);
        cudaStreamSynchronize(stream_);
        if (flag == 2) return fail(HM_ERR_TIMEOUT, "a bounded device-side wait ran out in a kernel of this pass; its results are not valid");
        return fail(HM_ERR_INVALID, "token id out of range (>= vocab_size)");
    }
    return HM_OK;
}

// Queues the bounded-wait probe on the engine's stream with the engine's error word: the next pass
// (prefill, decode step, ...) finds the word raised and reports HM_ERR_TIMEOUT; the one after is clean.
int Engine::selftest_expire_wait() {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (batch_ == 0) return fail(HM_ERR_STATE, "selftest_expire_wait before kv_alloc");
    // any 16 aligned device bytes serve as the source of the probe's real copy
    HM_CUDA(launch_bounded_wait_probe(rope_cos_, err_flag_, 20000ull, nullptr, stream_));
    return HM_OK;
}

// ---- GenerativeModel ---------------------------------------------------------------------------

// Where a device-to-host copy of logits lands.  Into pageable memory the driver stages such a copy piece by piece (about 80 us for
// one 608 KB row); into pinned memory it is one DMA.  A pageable destination therefore receives its rows through a pinned buffer of
// the engine (one DMA, then a host copy after the stream synchronisation); a pinned or registered destination is written directly.
bool Engine::alloc_pin_logits(size_t bytes) {
    bytes = std::max(bytes, (size_t)std::max(batch_, 1) * V_ * 4);
    if (pin_logits_bytes_ >= bytes) return true;
    drop_host_logits_graph();  // it stores into the buffer that is about to be replaced
    if (pin_logits_) cudaFreeHost(pin_logits_);
    pin_logits_ = pin_logits_dev_ = nullptr;
    pin_logits_bytes_ = 0;
    void* dev = nullptr;
    if (cudaHostAlloc(&pin_logits_, bytes, cudaHostAllocMapped) != cudaSuccess || cudaHostGetDevicePointer(&dev, pin_logits_, 0) != cudaSuccess) {
        cudaGetLastError();
        if (pin_logits_) cudaFreeHost(pin_logits_);
        pin_logits_ = nullptr;
        return false;
    }
    pin_logits_dev_ = static_cast<float*>(dev);
    pin_logits_bytes_ = bytes;
    return true;
}

float* Engine::logits_landing(float* user, size_t bytes) {
    cudaPointerAttributes at{};
    if (cudaPointerGetAttributes(&at, user) == cudaSuccess && at.type != cudaMemoryTypeUnregistered) return user;
    cudaGetLastError();
    return alloc_pin_logits(bytes) ? pin_logits_ : user;
}

void Engine::drop_host_logits_graph() {
    if (graph_exec_host_) cudaGraphExecDestroy(graph_exec_host_);
    if (graph_host_) cudaGraphDestroy(graph_host_);
    graph_exec_host_ = nullptr;
    graph_host_ = nullptr;
    host_graph_tried_ = false;
}

// A second decode graph for callers that take the logits of every step (the reference trait's decode_step returns them).  Its LM
// head stores the rows straight into the mapped pinned buffer: posted writes over PCIe that overlap the launch's weight stream, so
// no device-to-host copy follows the step (that copy costs more than the LM head itself for a 608 KB row).  Built only where the
// LM-head launch also produces the greedy token, so that nothing on the device reads the logits of such a step afterwards.
int Engine::ensure_host_logits_graph() {
    if (graph_exec_host_ || host_graph_tried_) return HM_OK;
    host_graph_tried_ = true;
    if (lm_head_.kind != HM_BF16 || batch_ > MAX_M || !graph_exec_) return HM_OK;
    if (!alloc_pin_logits((size_t)batch_ * V_ * 4)) return HM_OK;
    host_graph_tried_ = true;  // alloc_pin_logits may have cleared it
    HM_CUDA(cudaStreamSynchronize(stream_));
    int launches = 0;
    HM_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
    lm_out_ = pin_logits_dev_;
    int rc = enqueue_pass(batch_, tokens_dev_, pos_dev_, nullptr, 0, batch_, true, next_dev_, tokens_dev_, pos_dev_, hist_dev_, &launches);
    const bool folded = lm_folds_argmax_;
    lm_out_ = nullptr;
    cudaGraph_t g = nullptr;
    cudaError_t ce = cudaStreamEndCapture(stream_, &g);
    if (rc || ce != cudaSuccess || !folded) {
        if (g) cudaGraphDestroy(g);
        cudaGetLastError();
        return rc ? rc : (ce != cudaSuccess ? cuda_fail(ce, "cudaStreamEndCapture") : HM_OK);
    }
    graph_host_ = g;
    HM_CUDA(cudaGraphInstantiate(&graph_exec_host_, graph_host_, 0));
    return HM_OK;
}

int Engine::prefill(int seq, const int64_t* ids, int n, float* logits, uint32_t* first_token) {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (batch_ == 0) return fail(HM_ERR_STATE, "prefill before kv_alloc");
    if (seq < 0 || seq >= batch_ || !ids || n < 1) return fail(HM_ERR_INVALID, "prefill: bad arguments");
    const int len0 = len_[seq];
    if (len0 + n > max_seq_) return fail(HM_ERR_KV_FULL, "KV cache full (" + std::to_string(len0) + " + " + std::to_string(n) + " > " + std::to_string(max_seq_) + ")");
    for (int i = 0; i < n; ++i)
        if (ids[i] < 0 || ids[i] >= V_) return fail(HM_ERR_INVALID, "prefill: token id out of range");
    HM_CUDA(cudaStreamSynchronize(stream_));
    uint32_t* st = pin_u32_;
    for (int i = 0; i < n; ++i) {
        st[i] = (uint32_t)ids[i];
        st[n + i] = (uint32_t)(len0 + i);
        st[2 * n + i] = (uint32_t)seq;
    }
    HM_CUDA(cudaMemcpyAsync(pf_tokens_, st, (size_t)n * 4, cudaMemcpyHostToDevice, stream_));
    HM_CUDA(cudaMemcpyAsync(pf_pos_, st + n, (size_t)n * 4, cudaMemcpyHostToDevice, stream_));
    HM_CUDA(cudaMemcpyAsync(pf_seq_, st + 2 * n, (size_t)n * 4, cudaMemcpyHostToDevice, stream_));
    // pos_dev[seq] = len0+n-1; the argmax finish of the last chunk advances it to len0+n
    st[3 * n] = (uint32_t)(len0 + n - 1);
    HM_CUDA(cudaMemcpyAsync(pos_dev_ + seq, st + 3 * n, 4, cudaMemcpyHostToDevice, stream_));
    st[3 * n + 2] = (uint32_t)(len0 + n);
    HM_CUDA(cudaMemcpyAsync(smp_gen_start_ + seq, st + 3 * n + 2, 4, cudaMemcpyHostToDevice, stream_));
    int launches = 0;
    // GGUF models run a chunk's projections as 8-row groups of the quantised kernels, launched back to back: the groups after
    // the first find the projection's weights in the L2, and attention, embedding and LM head run once per chunk
    const int chunk = (use_tc_ || quant_) ? TC_ROWS : MAX_M;
    for (int c0 = 0; c0 < n; c0 += chunk) {
        const int mc = std::min(chunk, n - c0);
        const bool last = c0 + mc >= n;
        int rc = enqueue_pass(mc, pf_tokens_ + c0, pf_pos_ + c0, pf_seq_ + c0, mc - 1, last ? 1 : 0, false, next_dev_ + seq, tokens_dev_ + seq, pos_dev_ + seq, hist_dev_ + (size_t)seq * (max_seq_ + 1),
                              &launches);
        if (rc) return rc;
    }
    uint32_t* tok_pin = st + 3 * n + 1;
    HM_CUDA(cudaMemcpyAsync(tok_pin, next_dev_ + seq, 4, cudaMemcpyDeviceToHost, stream_));
    float* land = logits ? logits_landing(logits, (size_t)V_ * 4) : nullptr;
    if (logits) HM_CUDA(cudaMemcpyAsync(land, logits_, (size_t)V_ * 4, cudaMemcpyDeviceToHost, stream_));
    if (int qrc = queue_error_copy()) return qrc;
    HM_CUDA(cudaStreamSynchronize(stream_));
    int rc = check_device_error();
    if (rc) return rc;
    if (logits && land != logits) std::memcpy(logits, land, (size_t)V_ * 4);
    if (first_token) *first_token = *tok_pin;
    len_[seq] = len0 + n;
    gen_start_[seq] = len0 + n;  // what follows this prompt is "generated" for the penalties (src/generate.rs:150-152)
    return HM_OK;
}

int Engine::decode_step(const uint32_t* tokens, float* logits, uint32_t* next_tokens) {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (batch_ == 0) return fail(HM_ERR_STATE, "decode_step before kv_alloc");
    if (!tokens) return fail(HM_ERR_INVALID, "decode_step: null tokens");
    for (int b = 0; b < batch_; ++b) {
        if (len_[b] + 1 > max_seq_) return fail(HM_ERR_KV_FULL, "KV cache full (" + std::to_string(len_[b]) + " + 1 > " + std::to_string(max_seq_) + ")");
        if (tokens[b] >= (uint32_t)V_) return fail(HM_ERR_INVALID, "decode_step: token id out of range");
    }
    std::memcpy(pin_u32_, tokens, (size_t)batch_ * 4);
    HM_CUDA(cudaMemcpyAsync(tokens_dev_, pin_u32_, (size_t)batch_ * 4, cudaMemcpyHostToDevice, stream_));
    float* land = nullptr;
    if (logits) {
        int grc = ensure_host_logits_graph();
        if (grc) return grc;
        land = graph_exec_host_ ? pin_logits_ : logits_landing(logits, (size_t)batch_ * V_ * 4);
    }
    if (logits && graph_exec_host_) {
        HM_CUDA(cudaGraphLaunch(graph_exec_host_, stream_));  // the LM head writes the rows into pin_logits_ itself
    } else {
        int lrc = launch_step();
        if (lrc) return lrc;
    }
    HM_CUDA(cudaMemcpyAsync(pin_u32_ + batch_, next_dev_, (size_t)batch_ * 4, cudaMemcpyDeviceToHost, stream_));
    if (logits && !graph_exec_host_) HM_CUDA(cudaMemcpyAsync(land, logits_, (size_t)batch_ * V_ * 4, cudaMemcpyDeviceToHost, stream_));
    if (int qrc = queue_error_copy()) return qrc;
    HM_CUDA(cudaStreamSynchronize(stream_));
    {
        int erc = check_device_error();
        if (erc) return erc;
    }
    if (logits && land != logits) std::memcpy(logits, land, (size_t)batch_ * V_ * 4);
    if (next_tokens) std::memcpy(next_tokens, pin_u32_ + batch_, (size_t)batch_ * 4);
    for (int b = 0; b < batch_; ++b) len_[b] += 1;
    return HM_OK;
}

int Engine::decode_greedy_n(const uint32_t* first_tokens, int steps, uint32_t* out_ids) {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (batch_ == 0) return fail(HM_ERR_STATE, "decode_greedy_n before kv_alloc");
    if (steps < 0 || (steps > 0 && !out_ids)) return fail(HM_ERR_INVALID, "decode_greedy_n: bad arguments");
    for (int b = 0; b < batch_; ++b)
        if (len_[b] + steps > max_seq_) return fail(HM_ERR_KV_FULL, "KV cache full (" + std::to_string(len_[b]) + " + " + std::to_string(steps) + " > " + std::to_string(max_seq_) + ")");
    if (first_tokens) {
        for (int b = 0; b < batch_; ++b)
            if (first_tokens[b] >= (uint32_t)V_) return fail(HM_ERR_INVALID, "decode_greedy_n: token id out of range");
        std::memcpy(pin_u32_, first_tokens, (size_t)batch_ * 4);
        HM_CUDA(cudaMemcpyAsync(tokens_dev_, pin_u32_, (size_t)batch_ * 4, cudaMemcpyHostToDevice, stream_));
    }
    for (int s = 0; s < steps; ++s) {
        int lrc = launch_step();
        if (lrc) return lrc;
    }
    // history rows: token at position p of sequence b is hist[b][p]; the new ones are len+1 .. len+steps
    for (int b = 0; b < batch_; ++b)
        HM_CUDA(cudaMemcpyAsync(pin_u32_ + batch_ + (size_t)b * steps, hist_dev_ + (size_t)b * (max_seq_ + 1) + len_[b] + 1, (size_t)steps * 4, cudaMemcpyDeviceToHost, stream_));
    if (int qrc = queue_error_copy()) return qrc;
    HM_CUDA(cudaStreamSynchronize(stream_));
    {
        int erc = check_device_error();
        if (erc) return erc;
    }
    if (steps > 0) std::memcpy(out_ids, pin_u32_ + batch_, (size_t)batch_ * steps * 4);
    for (int b = 0; b < batch_; ++b) len_[b] += steps;
    return HM_OK;
}

int Engine::time_decode(int warmup, int steps, float* ms_total) {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (batch_ == 0) return fail(HM_ERR_STATE, "time_decode before kv_alloc");
    if (warmup < 0 || steps < 1 || !ms_total) return fail(HM_ERR_INVALID, "time_decode: bad arguments");
    for (int b = 0; b < batch_; ++b)
        if (len_[b] + warmup + steps > max_seq_) return fail(HM_ERR_KV_FULL, "KV cache full: not enough room for the timed steps");
    cudaEvent_t e0, e1;
    HM_CUDA(cudaEventCreate(&e0));
    HM_CUDA(cudaEventCreate(&e1));
    for (int s = 0; s < warmup; ++s) {
        int lrc = launch_step();
        if (lrc) return lrc;
    }
    HM_CUDA(cudaStreamSynchronize(stream_));
    HM_CUDA(cudaEventRecord(e0, stream_));
    for (int s = 0; s < steps; ++s) {
        int lrc = launch_step();
        if (lrc) return lrc;
    }
    HM_CUDA(cudaEventRecord(e1, stream_));
    if (int qrc = queue_error_copy()) return qrc;
    HM_CUDA(cudaStreamSynchronize(stream_));
    HM_CUDA(cudaEventElapsedTime(ms_total, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    {
        int erc = check_device_error();
        if (erc) return erc;
    }
#ifdef HM_PHASE_TRACE
    if (gemv_trace_ && std::getenv("HM_TRACE_DUMP")) {
        // raw stamps of the last step, one line per launch of the pass: for offline reading
        std::vector<unsigned long long> t(512 * 16);
        HM_CUDA(cudaMemcpy(t.data(), gemv_trace_, t.size() * 8, cudaMemcpyDeviceToHost));
        if (FILE* f = std::fopen(std::getenv("HM_TRACE_DUMP"), "w")) {
            for (int l = 0; l < 512; ++l) {
                std::fprintf(f, "%d", l);
                for (int i = 0; i < 16; ++i) std::fprintf(f, " %llu", t[(size_t)l * 16 + i]);
                std::fprintf(f, "\n");
            }
            std::fclose(f);
        }
    } else if (gemv_trace_) {
        // HM_GEMV_TRACE=1: %globaltimer stamps of CTA 0 of every projection launch of the last step:
        // resident -> predecessor done -> activations staged -> weights multiplied -> partials published ->
        // split-K reduced -> stored.  Averaged per launch position within a layer.
        std::vector<unsigned long long> t(512 * 16);
        HM_CUDA(cudaMemcpy(t.data(), gemv_trace_, t.size() * 8, cudaMemcpyDeviceToHost));
        // launch indices of the projections in a decode pass: 1 + l*5 + {0: qkv, 2: o, 3: gate_up, 4: down}, then 1 + 5L: LM head
        const char* names[5] = {"qkv", "attn", "o", "gate_up", "down"};
        for (int c = 0; c < 5; ++c) {
            double d[6] = {0, 0, 0, 0, 0, 0}, gap = 0;
            int n = 0;
            for (int l = 0; l < L_; ++l) {
                const unsigned long long* r = t.data() + (size_t)(1 + l * 5 + c) * 16;
                bool whole = true;
                for (int i = 0; i < 7; ++i) whole = whole && r[i] != 0;
                if (!whole) continue;
                for (int i = 0; i < 6; ++i) d[i] += (double)(r[i + 1] - r[i]);
                // time from the previous launch's last store (as CTA 0 saw it) to this one seeing its predecessor done
                const int prev = c == 0 ? (l == 0 ? -1 : 1 + (l - 1) * 5 + 4) : 1 + l * 5 + c - 1;
                if (prev >= 0 && t[(size_t)prev * 16 + 6]) gap += (double)(r[1] - t[(size_t)prev * 16 + 6]);
                ++n;
            }
            if (n && c == 1) {
                double late = 0;
                int nl = 0;
                for (int l = 0; l < L_; ++l) {
                    const unsigned long long* r = t.data() + (size_t)(1 + l * 5 + c) * 16;
                    if (r[1] && r[7] > r[1]) { late += (double)(r[7] - r[1]); ++nl; }
                }
                double ph[4] = {0, 0, 0, 0};
                int np = 0;
                for (int l = 0; l < L_; ++l) {
                    const unsigned long long* r = t.data() + (size_t)(1 + l * 5 + c) * 16;
                    if (!r[5] || !r[10] || !r[11] || !r[12] || !r[6]) continue;
                    ph[0] += (double)(r[10] - r[5]); ph[1] += (double)(r[11] - r[10]); ph[2] += (double)(r[12] - r[11]); ph[3] += (double)(r[6] - r[12]);
                    ++np;
                }
                if (np) std::fprintf(stderr, "[hm gemv trace] attn     rank-0 merge: scales %.2f | sums %.2f | divide+store %.2f | return %.2f us\n", ph[0] / np / 1e3, ph[1] / np / 1e3, ph[2] / np / 1e3, ph[3] / np / 1e3);
                if (nl) std::fprintf(stderr, "[hm gemv trace] attn     split holding the new token: pages done %.2f us after dep seen (mean of %d)\n", late / nl / 1e3, nl);
            }
            if (n) {
                // slots 8, 9: latest CTA of the launch to become resident / to finish (atomic maxima over all CTAs)
                double lr = 0, lf = 0;
                int nn = 0;
                for (int l = 0; l < L_; ++l) {
                    const unsigned long long* r = t.data() + (size_t)(1 + l * 5 + c) * 16;
                    if (!r[1] || !r[6] || !r[8] || !r[9]) continue;
                    lr += (double)r[8] - (double)r[1];
                    lf += (double)r[9] - (double)r[6];
                    ++nn;
                }
                if (nn) std::fprintf(stderr, "[hm gemv trace] %-8s last CTA resident %+.2f us relative to CTA 0 seeing its dependency; last CTA finished %+.2f us after CTA 0\n", names[c], lr / nn / 1e3, lf / nn / 1e3);
            }
            if (n)
                std::fprintf(stderr, "[hm gemv trace] %-8s resident->dep %.2f | stage inputs %.2f | multiply %.2f | publish+cluster barrier %.2f | reduce %.2f | epilogue %.2f | prev store -> dep seen %.2f us (mean of %d)\n", names[c],
                             d[0] / n / 1e3, d[1] / n / 1e3, d[2] / n / 1e3, d[3] / n / 1e3, d[4] / n / 1e3, d[5] / n / 1e3, gap / n / 1e3, n);
        }
    }
#endif
    for (int b = 0; b < batch_; ++b) len_[b] += warmup + steps;
    return HM_OK;
}

// Per class: a CUDA graph holding only that class's launches of one decode step (the real
// arguments, programmatic edges included) is replayed `steps` times between two events on the
// engine's stream.  The argmax class advances the device position, so it runs last and the
// sequences do move forward by `steps` tokens.
int Engine::profile_decode(int steps, hm_kernel_stat* out, int cap, int* n_out) {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (batch_ == 0) return fail(HM_ERR_STATE, "profile_decode before kv_alloc");
    if (steps < 1 || !out || !n_out || cap < PC_COUNT) return fail(HM_ERR_INVALID, "profile_decode: bad arguments (cap >= 8)");
    for (int b = 0; b < batch_; ++b)
        if (len_[b] + steps > max_seq_) return fail(HM_ERR_KV_FULL, "KV cache full: not enough room for the profiled steps");
    HM_CUDA(cudaStreamSynchronize(stream_));
    double kv_tokens = 0.0;
    for (int b = 0; b < batch_; ++b) kv_tokens += len_[b] + 1;
    cudaEvent_t e0, e1;
    HM_CUDA(cudaEventCreate(&e0));
    HM_CUDA(cudaEventCreate(&e1));
    float ms[PC_COUNT] = {0};
    int count[PC_COUNT] = {0};
    int rc = HM_OK;
    for (int c = 0; c < PC_COUNT && rc == HM_OK; ++c) {
        int launches = 0;
        only_class_ = c;
        cudaError_t ce = cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal);
        if (ce == cudaSuccess) rc = enqueue_pass(batch_, tokens_dev_, pos_dev_, nullptr, 0, batch_, true, next_dev_, tokens_dev_, pos_dev_, hist_dev_, &launches);
        only_class_ = -1;
        cudaGraph_t g = nullptr;
        cudaError_t ce2 = cudaStreamEndCapture(stream_, &g);
        if (ce != cudaSuccess || ce2 != cudaSuccess || rc != HM_OK) {
            if (g) cudaGraphDestroy(g);
            if (rc == HM_OK) rc = cuda_fail(ce != cudaSuccess ? ce : ce2, "profile capture");
            break;
        }
        count[c] = launches;
        if (launches > 0) {
            cudaGraphExec_t ge = nullptr;
            ce = cudaGraphInstantiate(&ge, g, 0);
            if (ce == cudaSuccess) {
                const bool moves_pos = c == PC_SAMPLE || (c == PC_LM_HEAD && lm_folds_argmax_);
                for (int w = 0; w < 2 && !moves_pos; ++w) cudaGraphLaunch(ge, stream_);  // warm-up (not for the class that moves the position)
                cudaEventRecord(e0, stream_);
                for (int s = 0; s < steps; ++s) cudaGraphLaunch(ge, stream_);
                cudaEventRecord(e1, stream_);
                ce = cudaStreamSynchronize(stream_);
                if (ce == cudaSuccess) cudaEventElapsedTime(&ms[c], e0, e1);
                cudaGraphExecDestroy(ge);
            }
            if (ce != cudaSuccess) rc = cuda_fail(ce, "profile replay");
        }
        cudaGraphDestroy(g);
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc) return rc;
    for (int b = 0; b < batch_; ++b) len_[b] += steps;
    uint64_t bytes[PC_COUNT] = {0};
    bytes[PC_EMBED] = (uint64_t)batch_ * H_ * (embed_dtype_ == HM_BF16 ? 2 : 4);
    for (auto& l : layers_) {
        bytes[PC_QKV] += l.qkv.bytes();
        bytes[PC_O] += l.o.bytes();
        bytes[PC_GATE_UP] += l.gu.bytes();
        bytes[PC_DOWN] += l.down.bytes();
    }
    bytes[PC_LM_HEAD] = lm_head_.bytes();
    bytes[PC_ATTN] = (uint64_t)(kv_tokens * L_ * 2.0 * kvh_ * hd_ * (kv_bf16_ ? 2 : 4));
    for (int c = 0; c < PC_COUNT; ++c) {
        std::memset(&out[c], 0, sizeof(out[c]));
        std::strncpy(out[c].name, kProfNames[c], sizeof(out[c].name) - 1);
        out[c].launches_per_step = count[c];
        out[c].ms_per_step = ms[c] / steps;
        out[c].bytes_per_step = bytes[c];
    }
    *n_out = PC_COUNT;
    return HM_OK;
}

// sample_token on the host (defined in capi.cu)
uint32_t host_sample_token(const float* logits, int n, const hm_sampling& cfg, const uint32_t* generated, int ngen, uint64_t* rng);

int Engine::ensure_sampler_scratch() {
    if (smp_scaled_) return HM_OK;
    HM_CUDA(cudaMalloc(&smp_scaled_, (size_t)batch_ * V_ * 4));
    HM_CUDA(cudaMalloc(&smp_count_, (size_t)batch_ * V_ * 4));
    HM_CUDA(cudaMemset(smp_count_, 0, (size_t)batch_ * V_ * 4));
    return HM_OK;
}

// The sampler kernel over the engine's own state: logits of the last pass, token history by position
// (generated tokens = positions from the end of the sequence's last prefill on), one RNG word per sequence.
SamplerArgs Engine::sampler_args(const hm_sampling& s) const {
    SamplerArgs sa{};
    sa.logits = logits_;
    sa.ld_logits = V_;
    sa.n = V_;
    sa.cfg = s;
    sa.hist = hist_dev_;
    sa.hist_stride = max_seq_ + 1;
    sa.gen_start = smp_gen_start_;
    sa.pos = pos_dev_;
    sa.rng = smp_rng_;
    sa.scaled = smp_scaled_;
    sa.count = smp_count_;
    sa.next_tok = next_dev_;
    sa.feed_tok = tokens_dev_;
    sa.overflow = smp_overflow_;
    return sa;
}

// decode_step + sample_token for every sequence (src/hf/model.rs:359-371 followed by src/generate.rs:698-801):
// the fed tokens enter the history (the penalties look at them), the decode graph runs, the sampler kernel
// picks one token per sequence with that sequence's RNG word.  Rows the kernel hands back (top-k disabled
// or above SAMPLER_MAX_K on a nearly flat distribution) are finished by the host sampler on their logits.
int Engine::decode_step_sampled(const uint32_t* tokens, const hm_sampling* sp, uint64_t* rng_state, float* logits, uint32_t* next_tokens) {
    if (!set_device()) return fail(HM_ERR_CUDA, "cudaSetDevice failed");
    if (batch_ == 0) return fail(HM_ERR_STATE, "decode_step_sampled before kv_alloc");
    if (!tokens || !sp || !rng_state) return fail(HM_ERR_INVALID, "decode_step_sampled: null argument");
    const hm_sampling s = *sp;
    const bool pure_greedy = !(s.temperature > 0.f) && s.repetition_penalty == 1.0f && s.frequency_penalty == 0.f && s.presence_penalty == 0.f;
    if (pure_greedy) return decode_step(tokens, logits, next_tokens);
    for (int b = 0; b < batch_; ++b) {
        if (len_[b] + 1 > max_seq_) return fail(HM_ERR_KV_FULL, "KV cache full (" + std::to_string(len_[b]) + " + 1 > " + std::to_string(max_seq_) + ")");
        if (tokens[b] >= (uint32_t)V_) return fail(HM_ERR_INVALID, "decode_step_sampled: token id out of range");
    }
    int rc = ensure_sampler_scratch();
    if (rc) return rc;
    // staging: [0, B) tokens in, [B, 2B) tokens out, [2B, 3B) overflow words, then B RNG words (8-byte aligned)
    uint32_t* pin = pin_u32_;
    const size_t B = (size_t)batch_;
    uint64_t* pin_rng = reinterpret_cast<uint64_t*>(pin + ((3 * B + 1) & ~(size_t)1));
    std::memcpy(pin, tokens, B * 4);
    std::memcpy(pin_rng, rng_state, B * 8);
    HM_CUDA(cudaMemcpyAsync(tokens_dev_, pin, B * 4, cudaMemcpyHostToDevice, stream_));
    HM_CUDA(cudaMemcpyAsync(smp_rng_, pin_rng, B * 8, cudaMemcpyHostToDevice, stream_));
    HM_CUDA(launch_hist_set(tokens_dev_, pos_dev_, hist_dev_, max_seq_ + 1, batch_, stream_));
    rc = launch_step();
    if (rc) return rc;
    const SamplerArgs sa = sampler_args(s);
    HM_CUDA(launch_sample(sa, batch_, stream_));
    HM_CUDA(cudaMemcpyAsync(pin + B, next_dev_, B * 4, cudaMemcpyDeviceToHost, stream_));
    HM_CUDA(cudaMemcpyAsync(pin + 2 * B, smp_overflow_, B * 4, cudaMemcpyDeviceToHost, stream_));
    HM_CUDA(cudaMemcpyAsync(pin_rng, smp_rng_, B * 8, cudaMemcpyDeviceToHost, stream_));
    float* land = logits ? logits_landing(logits, B * V_ * 4) : nullptr;
    if (logits) HM_CUDA(cudaMemcpyAsync(land, logits_, B * V_ * 4, cudaMemcpyDeviceToHost, stream_));
    rc = queue_error_copy();
    if (rc) return rc;
    HM_CUDA(cudaStreamSynchronize(stream_));
    rc = check_device_error();
    if (rc) return rc;
    if (logits && land != logits) std::memcpy(logits, land, B * V_ * 4);
    std::memcpy(rng_state, pin_rng, B * 8);
    std::vector<float> row;
    std::vector<uint32_t> gen;
    for (int b = 0; b < batch_; ++b) {
        uint32_t tok = pin[B + b];
        if (s.temperature > 0.f && pin[2 * B + b]) {
            row.resize(V_);
            const int ngen = std::max(0, len_[b] + 1 - gen_start_[b]);
            gen.resize(ngen);
            HM_CUDA(cudaMemcpy(row.data(), logits_ + (size_t)b * V_, (size_t)V_ * 4, cudaMemcpyDeviceToHost));
            if (ngen) HM_CUDA(cudaMemcpy(gen.data(), hist_dev_ + (size_t)b * (max_seq_ + 1) + gen_start_[b], (size_t)ngen * 4, cudaMemcpyDeviceToHost));
            tok = host_sample_token(row.data(), V_, s, gen.data(), ngen, &rng_state[b]);
            HM_CUDA(cudaMemcpy(tokens_dev_ + b, &tok, 4, cudaMemcpyHostToDevice));
            HM_CUDA(cudaMemcpy(hist_dev_ + (size_t)b * (max_seq_ + 1) + len_[b] + 1, &tok, 4, cudaMemcpyHostToDevice));
        }
        if (next_tokens) next_tokens[b] = tok;
    }
    for (int b = 0; b < batch_; ++b) len_[b] += 1;
    return HM_OK;
}

// generate_streaming_core (src/generate.rs:100-315) without the text side.
int Engine::generate(int seq, const int64_t* prompt, int n_prompt, int max_new, const hm_sampling* sp, uint32_t* out_ids, int* n_out) {
    if (!n_out || !out_ids) return fail(HM_ERR_INVALID, "generate: null output");
    *n_out = 0;
    if (n_prompt == 0 || max_new == 0) return HM_OK;  // src/generate.rs:111-113
    if (batch_ != 1) return fail(HM_ERR_UNSUPPORTED, "generate drives a single sequence: allocate the cache with batch = 1");
    hm_sampling s{};
    if (sp) s = *sp; else { s.temperature = 0.f; s.repetition_penalty = 1.f; s.top_p = 1.f; }
    const bool device_greedy = s.temperature <= 0.f && s.repetition_penalty == 1.0f && s.frequency_penalty == 0.f && s.presence_penalty == 0.f;
    const uint32_t eos = cfg_.eos_token_id;
    uint32_t first = 0;
    int rc = prefill(seq, prompt, n_prompt, nullptr, &first);
    if (rc) return rc;
    if (first == eos) return HM_OK;  // "EOS after prefill", src/generate.rs:159-162
    std::vector<uint32_t> gen;
    gen.push_back(first);
    int real_pos = len_[seq];
    if (device_greedy) {
        // Greedy tokens never leave the device between steps; EOS is looked for in blocks.
        uint32_t cur = first;
        bool stop = false;
        std::vector<uint32_t> blk(32);
        while (!stop && (int)gen.size() < max_new && real_pos < max_seq_) {
            const int want = std::min({32, max_new - (int)gen.size(), max_seq_ - real_pos});
            rc = decode_greedy_n(&cur, want, blk.data());
            if (rc) return rc;
            for (int i = 0; i < want; ++i) {
                if (blk[i] == eos) {
                    // tokens after EOS were speculative: roll the cache length back
                    len_[seq] = real_pos + i + 1;
                    HM_CUDA(cudaMemcpy(pos_dev_ + seq, &len_[seq], 4, cudaMemcpyHostToDevice));
                    stop = true;
                    break;
                }
                gen.push_back(blk[i]);
            }
            real_pos = len_[seq];
            cur = gen.back();
        }
    } else {
        uint64_t rng;
        if (s.seed_set) rng = s.seed | 1ull;
        else {
            struct timespec ts;
            clock_gettime(CLOCK_REALTIME, &ts);
            rng = ((uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec) | 1ull;
        }
        const char* hs = std::getenv("HM_HOST_SAMPLER");  // test knob: every token through the host sampler
        if (!(hs && hs[0] == '1')) {
            // Sampled tokens never leave the device between steps: every step replays the decode graph
            // (which also leaves the plain argmax in the feed slot) and then the sampler kernel
            // replaces it; EOS is looked for in blocks, as on the greedy path.  Settings for which the
            // kernel may have to hand a token to the host sampler (top-k disabled or above
            // SAMPLER_MAX_K) synchronise after every token instead.
            rc = ensure_sampler_scratch();
            if (rc) return rc;
            const bool exact = !(s.temperature > 0.f) || (s.top_k >= 1 && s.top_k <= SAMPLER_MAX_K) || V_ <= SAMPLER_MAX_K;
            HM_CUDA(cudaMemcpyAsync(smp_rng_ + seq, &rng, 8, cudaMemcpyHostToDevice, stream_));
            HM_CUDA(cudaMemcpyAsync(tokens_dev_ + seq, &first, 4, cudaMemcpyHostToDevice, stream_));
            SamplerArgs sa = sampler_args(s);
            bool stop = false;
            std::vector<uint32_t> blk(32);
            std::vector<float> logits;
            while (!stop && (int)gen.size() < max_new && real_pos < max_seq_) {
                const int want = exact ? std::min({32, max_new - (int)gen.size(), max_seq_ - real_pos}) : 1;
                for (int i = 0; i < want; ++i) {
                    rc = launch_step();
                    if (rc) return rc;
                    const cudaError_t ce = launch_sample(sa, batch_, stream_);
                    if (ce != cudaSuccess) return cuda_fail(ce, "sampler launch");
                }
                // the sampled tokens of the block are the history entries after the last known position
                HM_CUDA(cudaMemcpyAsync(blk.data(), hist_dev_ + (size_t)seq * (max_seq_ + 1) + real_pos + 1, (size_t)want * 4, cudaMemcpyDeviceToHost, stream_));
                int over = 0;
                if (!exact) HM_CUDA(cudaMemcpyAsync(&over, smp_overflow_ + seq, 4, cudaMemcpyDeviceToHost, stream_));
                rc = queue_error_copy();
                if (rc) return rc;
                HM_CUDA(cudaStreamSynchronize(stream_));
                rc = check_device_error();
                if (rc) return rc;
                len_[seq] = real_pos + want;
                if (over) {
                    // the top-p prefix reaches beyond the candidates the kernel gathers: this token comes from the
                    // host sampler on the step's logits, with the RNG word the kernel left untouched
                    logits.resize(V_);
                    HM_CUDA(cudaMemcpy(logits.data(), logits_ + (size_t)seq * V_, (size_t)V_ * 4, cudaMemcpyDeviceToHost));
                    HM_CUDA(cudaMemcpy(&rng, smp_rng_ + seq, 8, cudaMemcpyDeviceToHost));
                    blk[0] = host_sample_token(logits.data(), V_, s, gen.data(), (int)gen.size(), &rng);
                    HM_CUDA(cudaMemcpy(smp_rng_ + seq, &rng, 8, cudaMemcpyHostToDevice));
                    HM_CUDA(cudaMemcpy(tokens_dev_ + seq, &blk[0], 4, cudaMemcpyHostToDevice));
                    HM_CUDA(cudaMemcpy(hist_dev_ + (size_t)seq * (max_seq_ + 1) + real_pos + 1, &blk[0], 4, cudaMemcpyHostToDevice));
                }
                for (int i = 0; i < want; ++i) {
                    if (blk[i] == eos) {
                        len_[seq] = real_pos + i + 1;  // tokens after EOS were speculative: roll the cache length back
                        HM_CUDA(cudaMemcpy(pos_dev_ + seq, &len_[seq], 4, cudaMemcpyHostToDevice));
                        stop = true;
                        break;
                    }
                    gen.push_back(blk[i]);
                }
                real_pos = len_[seq];
            }
        } else {
            std::vector<float> logits(V_);
            uint32_t cur = first;
            for (int step = 1; step < max_new; ++step) {
                if (real_pos >= max_seq_) break;
                rc = decode_step(&cur, logits.data(), nullptr);
                if (rc) return rc;
                cur = host_sample_token(logits.data(), V_, s, gen.data(), (int)gen.size(), &rng);
                real_pos += 1;
                if (cur == eos) break;
                gen.push_back(cur);
            }
        }
    }
    std::memcpy(out_ids, gen.data(), gen.size() * 4);
    *n_out = (int)gen.size();
    return HM_OK;
}

}  // namespace hm
