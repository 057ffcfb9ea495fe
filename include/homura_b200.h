/*
 * homura_b200.h -- C ABI of the B200 decode engine that stands behind Homura's generation
 * interface for decoder-only RoPE transformers (Qwen2 / Qwen3 / Llama configs).
 *
 * Every entry point is what a Rust `extern "C"` block in Homura would bind in place of the
 * CPU path cited next to it (file:line in the Homura repository).  Conventions:
 *   - every call returns an int status (HM_OK == 0); nothing throws or aborts across the ABI;
 *   - the engine owns all device memory; host buffers passed in stay caller-owned;
 *   - one engine per GPU; calls on one engine are not re-entrant (Homura serialises them on
 *     a Mutex, src/hf/model.rs:24,205); different engines may be driven from different threads;
 *   - data pointers of the model-level calls are HOST pointers; the standalone kernel entry
 *     points accept host OR device pointers (detected with cudaPointerGetAttributes): host
 *     buffers are staged through device memory inside the call;
 *   - there is no CPU fallback: without a CUDA device calls return HM_ERR_CUDA.
 */
#ifndef HOMURA_B200_H
#define HOMURA_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define HM_API __attribute__((visibility("default")))
#else
#define HM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hm_engine hm_engine;

enum hm_status {
    HM_OK = 0,
    HM_ERR_INVALID = 1,     /* bad argument / shape / token id */
    HM_ERR_CUDA = 2,        /* CUDA runtime error or no device */
    HM_ERR_KV_FULL = 3,     /* "KV cache full" -- a panic in src/runtime.rs:523-529 */
    HM_ERR_IO = 4,          /* file missing / truncated / malformed */
    HM_ERR_UNSUPPORTED = 5, /* dtype or shape outside the supported path */
    HM_ERR_TIMEOUT = 6,     /* a bounded device-side wait ran out */
    HM_ERR_STATE = 7        /* call order (e.g. decode before kv_alloc) */
};

/* DType subset on this path: src/dtype.rs:8-26 (+ Q4_0, which Homura has no DType for). */
enum hm_dtype { HM_F32 = 0, HM_BF16 = 1, HM_F16 = 2, HM_Q8_0 = 3, HM_Q4_0 = 4, HM_I64 = 5, HM_I32 = 6, HM_U8 = 7, HM_Q4_K = 8, HM_Q6_K = 9 };

/* Weight layouts accepted by the standalone projection kernels. */
enum hm_layout {
    HM_LAYOUT_KN = 0,      /* row-major [K, N]: Homura's matmul layout after load (src/hf/weights.rs:304-381) */
    HM_LAYOUT_SLAB128 = 1  /* [ceil(N/128)][K][128]: the engine's streaming layout (see hm_pack_bf16_slabs) */
};

/* Mirror of TransformerConfig, src/hf/config.rs:11-38.  num_key_value_heads / head_dim are
 * the resolved values (kv_heads(), head_dim()); eos/bos are UINT32_MAX when absent. */
typedef struct hm_config {
    int32_t hidden_size;
    int32_t intermediate_size;
    int32_t num_attention_heads;
    int32_t num_hidden_layers;
    int32_t num_key_value_heads;
    int32_t vocab_size;
    int32_t max_position_embeddings;
    int32_t head_dim;
    int32_t tie_word_embeddings;
    int32_t has_qkv_bias; /* inferred from tensor names, src/hf/weights.rs:272-274 */
    int32_t has_qk_norm;
    int32_t weight_dtype; /* hm_dtype of the projection weights */
    uint32_t eos_token_id;
    uint32_t bos_token_id;
    double rms_norm_eps;
    double rope_theta;
} hm_config;

/* Mirror of SamplingConfig, src/generate.rs:648-683 (stop_sequences are text-level and stay
 * with the caller).  seed_set == 0 means "seed from system time" (src/generate.rs:619-625). */
typedef struct hm_sampling {
    float temperature;
    int32_t top_k;
    float top_p;
    float min_p;
    float repetition_penalty;
    float frequency_penalty;
    float presence_penalty;
    int32_t seed_set;
    uint64_t seed;
} hm_sampling;

/* ---- library ------------------------------------------------------------------------ */
HM_API const char* hm_version(void);
/* Number of visible CUDA devices (0 when there is no driver/GPU). */
HM_API int hm_device_count(void);
/* Message of the last failing call made on this thread when no engine handle exists yet. */
HM_API const char* hm_last_error_global(void);

/* ---- model lifecycle ---------------------------------------------------------------- */
/* HfModel::load_with_dtype, src/hf/model.rs:79-145: config.json + model.safetensors (or the
 * sharded index) from `model_dir`.  weight_dtype HM_BF16 keeps bf16 projections; HM_F32 (what
 * HfModel::load asks for, src/hf/model.rs:37-39) is accepted for checkpoints stored in bf16, where
 * widening to f32 changes no value; a checkpoint whose projections are stored as f32 / f16 is
 * HM_ERR_UNSUPPORTED (no f32-weight kernel). */
HM_API int hm_model_load(const char* model_dir, int weight_dtype, int device, hm_engine** out);
/* HfModel::load_gguf, src/hf/model.rs:46-75: config from `<arch>.*` metadata, blk.N.* tensors. */
HM_API int hm_model_load_gguf(const char* gguf_path, int device, hm_engine** out);
/* Build from tensors handed over one by one (what a caller that already parsed a checkpoint
 * does): load_transformer_weights, src/hf/weights.rs:267-417 / src/gguf.rs:589-708.  Whether the model has
 * QK-norm is inferred from its tensors and decides how quantised q / k / v projections are stored: hand over the
 * q_norm / k_norm weights before those projections (HM_ERR_STATE otherwise; hm_model_load* do so). */
HM_API int hm_engine_create(const hm_config* cfg, int device, hm_engine** out);
HM_API int hm_load_tensor(hm_engine* e, const char* name, int dtype, const int64_t* shape, int ndim, const void* host_data, size_t nbytes);
HM_API int hm_finalize_weights(hm_engine* e);
HM_API void hm_engine_destroy(hm_engine* e);
HM_API const char* hm_last_error(hm_engine* e);
/* HfModel::config, src/hf/model.rs:246-249 */
HM_API int hm_get_config(hm_engine* e, hm_config* out);
/* Bytes of projection + LM-head weights one decode step streams (the roofline numerator). */
HM_API int hm_weight_bytes(hm_engine* e, uint64_t* out);

/* Host-only: parses a checkpoint the way the loaders above do and writes a JSON description
 * into buf -- {"format", "config": {...}, "tensors": [{"name","dtype","shape","nbytes","fnv1a"}]}.
 * `path` is a model directory (config.json + model.safetensors) or a .gguf file.  Needs no GPU
 * (the counterpart of `homura info`, src/main.rs:99-157).  Returns HM_ERR_INVALID when buf is
 * too small (the needed size is stored in *needed when non-NULL). */
HM_API int hm_checkpoint_info(const char* path, char* buf, size_t cap, size_t* needed);

/* ---- persistent KV cache ------------------------------------------------------------ */
/* KvCache::new, src/runtime.rs:396-418 (allocated lazily by run_kv, src/runtime.rs:1592-1645):
 * `batch` independent sequences of up to max_seq_len tokens in pages of page_tokens (16);
 * kv_dtype HM_F32 (Homura's cache dtype) or HM_BF16. */
HM_API int hm_kv_alloc(hm_engine* e, int batch, int max_seq_len, int page_tokens, int kv_dtype);
/* Drops the cache (weights stay resident) so that hm_kv_alloc can be called again with another batch,
 * length or dtype: what init_kv_cache does when called on a model that already has a cache,
 * src/runtime.rs:1898-1938. */
HM_API int hm_kv_free(hm_engine* e);
/* reset_kv_cache, src/hf/model.rs:232-237; seq < 0 resets every sequence. */
HM_API int hm_kv_reset(hm_engine* e, int seq);
/* kv_cache_len, src/hf/model.rs:240-243 */
HM_API int hm_kv_len(hm_engine* e, int seq, int* out);
/* KvCache::append_key/append_value + advance_by, src/runtime.rs:521-570,625-634: rows are
 * f32 [kv_heads, n_new, head_dim]; advance != 0 moves the sequence length forward. */
HM_API int hm_kv_append(hm_engine* e, int seq, int layer, const float* k_rows, const float* v_rows, int n_new, int advance);
/* KvCache::view, src/runtime.rs:463-507: contiguous f32 [kv_heads, len, head_dim] copies. */
HM_API int hm_kv_view(hm_engine* e, int seq, int layer, float* k_out, float* v_out);

/* ---- generation (trait GenerativeModel, src/generate.rs:19-30) ---------------------- */
/* HfGenerationContext::prefill, src/hf/model.rs:314-357: runs n prompt ids of sequence `seq`
 * (extending its cache if it already holds tokens), returns argmax at the last position and,
 * when logits_or_null != NULL, the V logits of that position. */
HM_API int hm_prefill(hm_engine* e, int seq, const int64_t* ids, int n, float* logits_or_null, uint32_t* first_token);
/* HfGenerationContext::decode_step, src/hf/model.rs:359-371, for all `batch` sequences at once:
 * tokens[batch] in; greedy next tokens out (argmax, ties to the highest index,
 * src/generate.rs:457-468); logits_or_null is [batch, vocab] f32 when wanted (any host memory: pageable
 * destinations are filled through a pinned buffer of the engine). */
HM_API int hm_decode_step(hm_engine* e, const uint32_t* tokens, float* logits_or_null, uint32_t* next_tokens);
/* The same step followed by sample_token (src/generate.rs:698-801) for every sequence, with the sampler
 * options of SamplingConfig (src/generate.rs:648-667): what the reference's loop does per token
 * (decode_step, then sample_token, src/generate.rs:187-230), for `batch` sequences in one call.  The fed
 * tokens enter each sequence's history; the penalties look at the tokens since that sequence's last
 * hm_prefill.  rng_state[batch] holds one xorshift64 word per sequence (seed | 1, src/generate.rs:626-632),
 * advanced by one draw when temperature > 0.  temperature <= 0 is the reference's greedy mode: penalties,
 * then argmax.  Runs on the device for every setting; rows whose top-p prefix reaches beyond the 1024
 * largest candidates (possible only with top_k disabled or above 1024) are finished by the host sampler
 * on that row's logits inside the call. */
HM_API int hm_decode_step_sampled(hm_engine* e, const uint32_t* tokens, const hm_sampling* sampling, uint64_t* rng_state, float* logits_or_null, uint32_t* next_tokens);
/* generate_streaming_core, src/generate.rs:100-315, on sequence `seq`: prefill + up to
 * max_new_tokens-1 decode steps, sampling per `sampling` (tokens stay on the device between steps for
 * every setting, the reference CLI's `--temperature 0` with its default repetition penalty included);
 * stops at EOS or at max_seq_len.  out_ids receives the generated ids, *n_out their count. */
HM_API int hm_generate(hm_engine* e, int seq, const int64_t* prompt, int n_prompt, int max_new_tokens, const hm_sampling* sampling, uint32_t* out_ids, int* n_out);
/* Greedy decode of `steps` tokens for every sequence with the token fed back on the device
 * (no host round trip between steps); out_ids is [batch, steps].  Used by the throughput bench. */
HM_API int hm_decode_greedy_n(hm_engine* e, const uint32_t* first_tokens, int steps, uint32_t* out_ids);
/* sample_token, src/generate.rs:698-801, on host logits (state is the xorshift64 word). */
HM_API int hm_sample_token(const float* logits, int n, const hm_sampling* cfg, const uint32_t* generated, int n_generated, uint64_t* rng_state, uint32_t* out);
/* The same sampler as one GPU kernel (what hm_generate and hm_decode_step_sampled use): logits may be a
 * host or a device pointer.  Penalties, candidate order and the xorshift64 draw are exact; probabilities
 * can differ from the host path in their last bits (tree sum, device expf), so in rare cases the draw
 * falls on the other side of a boundary.  temperature <= 0: penalties, then argmax (ties to the highest
 * index).  With top_k disabled or above 1024 a row whose top-p prefix does not end inside the 1024 largest
 * candidates is finished by the host sampler inside the call. */
HM_API int hm_sample_token_device(const float* logits, int n, const hm_sampling* cfg, const uint32_t* generated, int n_generated, uint64_t* rng_state, uint32_t* out);

/* ---- timing on the engine's stream (CUDA events) ------------------------------------ */
/* Runs `steps` greedy decode steps after `warmup` untimed ones and reports the device time
 * of the timed steps in milliseconds. */
HM_API int hm_time_decode(hm_engine* e, int warmup, int steps, float* ms_total);
/* Per-kernel-class timing of the decode step, the counterpart of HOMURA_PROFILE=1
 * (src/runtime.rs:1351-1353,1849-1873; classes as in scripts/profile.py:339-369): for every
 * class a CUDA graph with only that class's launches of one decode step is replayed `steps`
 * times between two CUDA events on the engine's stream; reports, per class, launches and mean
 * device time per step plus the algorithmic bytes the class moves per step.  The sequences
 * advance by `steps` tokens. */
typedef struct hm_kernel_stat {
    char name[32];
    int32_t launches_per_step;
    float ms_per_step;
    uint64_t bytes_per_step;
} hm_kernel_stat;
HM_API int hm_profile_decode(hm_engine* e, int steps, hm_kernel_stat* out, int cap, int* n_out);
/* Failure-path self-test (no counterpart in the reference, whose CPU kernels never wait on hardware): queues
 * a one-CTA kernel on the engine's stream whose mbarrier is armed for bytes that nobody sends; its bounded
 * wait gives up after 20000 polls and raises the engine's device error word.  The NEXT pass on this engine
 * (hm_prefill, hm_decode_step, ...) therefore returns HM_ERR_TIMEOUT, and the call after that is clean
 * again -- which is how a host learns that every device-side wait of this library is bounded and how the
 * status surfaces.  Nothing faults or hangs; the context stays usable. */
HM_API int hm_selftest_expire_wait(hm_engine* e);
/* The engine's stream as a cudaStream_t, for callers that record their own events. */
HM_API void* hm_engine_stream(hm_engine* e);
/* Number of kernel launches one decode step of this engine issues. */
HM_API int hm_launches_per_step(hm_engine* e, int* out);

/* ---- standalone kernels (the per-kernel sweeps) ------------------------------------- */
/* y[M,N] = x[M,K] @ W, bf16 weights, f32 activations and accumulation: the mixed matmul of
 * src/graph_builder/emit_linalg.rs:1928-2008,2224-2307.  M <= 16.  stream may be NULL. */
HM_API int hm_gemv_bf16(const float* x, const void* w_bf16, int layout, int M, int K, int N, float* y, void* stream);
/* The same projection for callers that must not allocate.  It has no counterpart in the
 * reference (whose kernels run on the CPU and never needed device scratch); it exists so that a
 * host with a "kernels only touch memory their caller owns" rule can keep that rule on the GPU.
 * It calls no cudaMalloc / cudaFree and
 * no allocating library routine: the split-K scratch is a fixed array inside the library
 * (4 MiB of partial sums + 4096 slab tickets, held by every GPU that loads the library until
 * the process exits), so it is meant for hosts whose token path may not reach an allocator --
 * a plan runner that hands kernels nothing but pre-owned memory, or a serving loop that cannot
 * absorb the device-wide synchronisation an allocation may cause.
 *   - x, w_bf16 and y must be DEVICE pointers; M must be 1, 2, 4, 8 or 16;
 *   - shapes whose split-K scratch would exceed the built-in array (or N > 524288) are rejected
 *     with HM_ERR_UNSUPPORTED -- use hm_gemv_bf16 for those;
 *   - the first call on each device resolves the array's device address; make that call
 *     before starting any stream capture;
 *   - every call on a device shares the one array: calls that may overlap on the GPU (different
 *     streams, different threads) race on it -- issue them on one stream or serialise them. */
HM_API int hm_gemv_bf16_noalloc(const float* x, const void* w_bf16, int layout, int M, int K, int N, float* y, void* stream);
/* Re-layout row-major [K,N] bf16 into HM_LAYOUT_SLAB128 (dst holds ceil(N/128)*K*128 elements). */
HM_API int hm_pack_bf16_slabs(const void* w_kn, int K, int N, void* dst, void* stream);
/* The same mixed matmul for 1 <= M <= 64 rows on the 5th-generation tensor cores (tcgen05 with the
 * accumulator in tensor memory).  w_tc is the weight packed by hm_pack_bf16_tc.  f32 activations are
 * split into three bf16 terms inside the kernel, so results agree with the f32 x bf16 product of
 * emit_linalg.rs:1928-2008 to f32 rounding (accumulation order differs from the CPU loop).
 * ksplit = CTAs per 128-feature block sharing K through a thread-block cluster: 0 = choose, else 1..16. */
HM_API int hm_gemm_bf16_tc(const float* x, const void* w_tc, int M, int K, int N, int ksplit, float* y, void* stream);
/* Elements (bf16) of the packed tensor-core weight for a [K,N] matrix: both dims padded to tiles. */
HM_API size_t hm_tc_packed_elems(int K, int N);
/* Re-layout bf16 weights, row-major [K,N] (layout HM_LAYOUT_KN) into the tensor-core tile layout:
 * [ceil(N/128)][ceil(K/64)][128][64], K-major, 128-byte swizzled (the shared-memory image of a tile). */
HM_API int hm_pack_bf16_tc(const void* w_kn, int K, int N, void* dst, void* stream);
/* Q8_0 / Q4_0 dequant-matmul on GGUF blocks [N, K/32] (src/graph_builder/emit_quant.rs:30-142;
 * Q4_0 has no counterpart in Homura, see src/gguf.rs:94-109,141), and the K-quants HM_Q4_K / HM_Q6_K
 * on super-blocks [N, K/256] of 144 / 210 bytes with Homura's semantics for them: the activation row
 * is quantised to Q8_K and the dot products run in integers (emit_quant.rs:165-567, 569-816).  M <= 8. */
HM_API int hm_gemv_quant(const float* x, const void* blocks, int dtype, int M, int K, int N, float* y, void* stream);
/* CPU-visible dequantisation of GGUF blocks on the GPU (dequant_q8_0 / dequant_q4_k / dequant_q6_k,
 * src/gguf.rs:817-917); n_blocks counts 32-value blocks, or 256-value super-blocks for the K-quants. */
HM_API int hm_dequant(const void* blocks, int dtype, size_t n_blocks, float* out, void* stream);
/* RMSNorm, src/graph_builder/emit_linalg.rs:7-26: rows x n. */
HM_API int hm_rms_norm(const float* x, const float* w, float eps, int rows, int n, float* out, void* stream);
/* bias + per-head QK RMSNorm + RoPE half rotation of the QKV epilogue
 * (src/hf/emitter.rs:604-649): x [rows, heads, hd] in place; norm_w may be NULL. */
HM_API int hm_qknorm_rope(float* x, int rows, int heads, int hd, const float* norm_w, float eps, const float* cos_rows, const float* sin_rows, void* stream);
/* GQA decode attention over a paged cache (src/hf/emitter.rs:683-737, floordiv head map of
 * src/graph_builder/emit_linalg.rs:93-245): q [B, heads, hd] f32; k_pages and v_pages are blocks
 * [n_pages, kv_heads] of one [page_tokens, hd] tile each, of kv_dtype, stored the way the engine's
 * KV-write epilogues lay them out: K chunk-major in chunks of 4 elements, [hd/4][page_tokens][4] (element
 * (t, d) at ((d/4)*page_tokens + t)*4 + d%4); V as rows [page_tokens][hd] on f32 pages and chunk-major in
 * chunks of 8 on bf16 pages, [hd/8][page_tokens][8] (element (t, d) at ((d/8)*page_tokens + t)*8 + d%8);
 * page_table [B, max_pages] int32;
 * kv_len [B] int32; out [B, heads*hd] f32.  A host kv_len is range-checked; a kv_len in device
 * memory is trusted (entries must lie in [1, max_pages*page_tokens]) and the call stays asynchronous
 * when every pointer is a device pointer. */
HM_API int hm_attn_decode_paged(const float* q, const void* k_pages, const void* v_pages, int kv_dtype, const int32_t* page_table, const int32_t* kv_len, int B, int heads, int kv_heads, int hd, int page_tokens, int max_pages, float* out, void* stream);
/* argmax with ties to the highest index (src/generate.rs:457-468): logits [rows, n]. */
HM_API int hm_argmax(const float* logits, int rows, int n, uint32_t* out, void* stream);

/* ---- device memory helpers for HBM-resident measurements ---------------------------- */
HM_API int hm_dev_alloc(size_t nbytes, void** out);
HM_API int hm_dev_free(void* p);
HM_API int hm_dev_copy(void* dst, const void* src, size_t nbytes); /* any direction, synchronous */
HM_API int hm_dev_sync(void);
HM_API int hm_dev_set(int device);                               /* device the helpers above (and the standalone kernels) use on this thread */
HM_API int hm_dev_mem_info(size_t* free_bytes, size_t* total_bytes); /* cudaMemGetInfo of the current device */

#ifdef __cplusplus
}
#endif
#endif /* HOMURA_B200_H */
