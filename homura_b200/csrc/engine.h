// Device-resident decode engine: weights, paged KV cache, the decode step as a CUDA graph.
//
// Takes the place of HfModel + ExecutionPlan::run_kv on the decode path
// (src/hf/model.rs:37-267, src/runtime.rs:1580-1892): instead of routing host Buffers
// between ~5 compiled kernels per layer, the step is a fixed chain of fused kernels whose
// activations never leave HBM, captured once and replayed per token.
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "../../include/homura_b200.h"
#include "common.cuh"
#include "sampler.h"

namespace hm {

struct LinearW {
    int K = 0, N = 0;        // N = output count of the (possibly fused) projection
    int kind = -1;           // HM_BF16 (slab layout) | HM_Q8_0 | HM_Q4_0 (split scales + codes)
    uint16_t* slabs = nullptr;
    uint16_t* tc = nullptr;  // second copy in the tensor-core tile layout (gemm_tc.h), used for passes over more than 8 rows
    uint16_t* scales = nullptr;
    uint8_t* codes = nullptr;
    uint8_t* kq_data = nullptr;       // K-quants (kind HM_Q4_K stands for the family): tiled super-blocks, kquant.h
    uint8_t* kq_tile_type = nullptr;  // per 32-row tile: 1 = Q4_K, 2 = Q6_K
    size_t kq_bytes = 0;              // GGUF bytes loaded into it (what a step streams)
    int kq_part_type = -1;            // type of the part loaded last (gate and up must agree: they share tiles)
    bool kq_has_q6 = false;           // some tile is Q6_K: passes over more than 8 rows keep the 8-row launches (the row-block kernel is Q4_K only)
    int loaded_parts = 0;
    bool rope_rows = false;  // quantised fused QKV: q and k rows stored in rotation-pair tiles (rope_tile_row), the projection's epilogue rotates
    size_t bytes() const;
};

struct LayerW {
    float* in_ln = nullptr;
    float* post_ln = nullptr;
    float* qkv_bias = nullptr;  // fused [q_dim + 2 kv_dim]
    float* q_norm = nullptr;
    float* k_norm = nullptr;
    LinearW qkv, o, gu, down;
};

// final argmax folded into the LM-head launch (see GemvArgs::fin_ticket)
struct ArgmaxFold {
    uint32_t *next_tok, *feed_tok;
    int32_t* pos;
    uint32_t* hist;
    int hist_stride;
};

class Engine {
   public:
    static int create(const hm_config& cfg, int device, Engine** out, std::string* err);
    ~Engine();

    int load_tensor(const char* name, int dtype, const int64_t* shape, int ndim, const void* host, size_t nbytes);
    int finalize();

    int kv_alloc(int batch, int max_seq_len, int page_tokens, int kv_dtype);
    int kv_free();
    int kv_reset(int seq);
    int kv_len(int seq, int* out);
    int kv_append(int seq, int layer, const float* k_rows, const float* v_rows, int n_new, int advance);
    int kv_view(int seq, int layer, float* k_out, float* v_out);

    int prefill(int seq, const int64_t* ids, int n, float* logits, uint32_t* first_token);
    int decode_step(const uint32_t* tokens, float* logits, uint32_t* next_tokens);
    int decode_step_sampled(const uint32_t* tokens, const hm_sampling* s, uint64_t* rng_state, float* logits, uint32_t* next_tokens);
    int decode_greedy_n(const uint32_t* first_tokens, int steps, uint32_t* out_ids);
    int generate(int seq, const int64_t* prompt, int n_prompt, int max_new, const hm_sampling* s, uint32_t* out_ids, int* n_out);
    int time_decode(int warmup, int steps, float* ms_total);
    int profile_decode(int steps, hm_kernel_stat* out, int cap, int* n_out);
    int selftest_expire_wait();

    const hm_config& config() const { return cfg_; }
    uint64_t weight_bytes() const;
    cudaStream_t stream() const { return stream_; }
    int launches_per_step() const { return launches_per_step_; }
    std::string err;

   private:
    Engine() = default;
    int fail(int code, const std::string& msg);
    int cuda_fail(cudaError_t e, const char* what);
    bool set_device();
    int stage(const void* host, size_t nbytes, void** dev);  // temp device copy of a host tensor
    int load_linear(LinearW& L, int K, int N_total, int n_off, int n_part, int interleave_which, int dtype, const void* host, size_t nbytes, int rope_part = 0);
    int load_vec_f32(float** dst, size_t n_total, size_t off, int dtype, const void* host, size_t n, size_t nbytes);
    int ensure_scratch(int rows);
    RopeEpi rope_epi(int layer, const int32_t* row_pos, const int32_t* row_seq, int m0) const;
    // Enqueue one pass over M rows (decode: one row per sequence; prefill: a chunk of one
    // sequence).  lm_row0/lm_rows select the rows that go through the LM head.
    int enqueue_pass(int M, const uint32_t* tokens_dev, const int32_t* row_pos, const int32_t* row_seq, int lm_row0, int lm_rows, bool advance, uint32_t* next_dev, uint32_t* feed_dev, int32_t* pos_dev, uint32_t* hist_dev, int* launches);
    int enqueue_linear(const LinearW& L, int M, const float* x, int ldx, int pro, const float* norm_w, int epi, float* y, int ldy, const float* bias, const float* resid, int layer, const int32_t* row_pos, const int32_t* row_seq, float* amax_val, int32_t* amax_idx, int* launches, const struct ArgmaxFold* fold = nullptr);
    // RMSNorm handed from one tensor-core GEMM to the next without a packing launch (see TcArgs)
    struct TcFuse {
        const float* ss_in = nullptr;   // consumer: partial sums of squares of the rows of `prepacked`
        int ss_parts = 0;
        unsigned char* xp_next = nullptr;  // producer: activation image of the next GEMM, scaled by next_norm_w
        const float* next_norm_w = nullptr;
        float* ss_out = nullptr;
    };
    int enqueue_linear_tc(const LinearW& L, int M, const float* x, int ldx, const float* norm_w, int epi, float* y, int ldy, const float* bias, const float* resid, int layer, const int32_t* row_pos, const int32_t* row_seq, int* launches,
                          const unsigned char* prepacked = nullptr, unsigned char* pack_out = nullptr, const TcFuse* fuse = nullptr);
    int capture_decode_graph();
    int ensure_host_logits_graph();
    int ensure_sampler_scratch();
    SamplerArgs sampler_args(const hm_sampling& s) const;
    int launch_step();        // replay the captured decode graph
    int queue_error_copy();    // device error word -> pinned host word, on the engine's stream
    int check_device_error();  // after the synchronisation that follows queue_error_copy()
    void prof_mark(int cls);

    hm_config cfg_{};
    int device_ = 0, sm_count_ = 148;
    int H_ = 0, I_ = 0, heads_ = 0, kvh_ = 0, hd_ = 0, qdim_ = 0, kvdim_ = 0, L_ = 0, V_ = 0;
    bool finalized_ = false, quant_ = false, pdl_ = true;
    bool use_clusters_ = true;  // split reductions through thread-block clusters / DSMEM (HM_NO_CLUSTER=1: global scratch + tickets)
    int max_cluster_ = 8;
    bool use_prefetch_ = true;  // decode kernels pull the weights of the kernel two launches ahead into the L2
    const void* pf_ptr_ = nullptr;  // prefetch target handed to the next projection launch
    unsigned long long pf_bytes_ = 0;
    bool use_tc_ = true;  // bf16 models: passes over more than 8 rows run the tcgen05 GEMM (HM_NO_TC=1: 8-row groups of the streaming kernel)
    cudaStream_t stream_ = nullptr;

    // weights
    void* embed_ = nullptr;  // [V,H] bf16 (embed_dtype_ == HM_BF16) or f32
    int embed_dtype_ = -1;
    float* final_norm_ = nullptr;
    std::vector<LayerW> layers_;
    LinearW lm_head_;
    float *rope_cos_ = nullptr, *rope_sin_ = nullptr;

    // activations / scratch for up to scratch_rows_ rows
    int scratch_rows_ = 0;
    float *h_ = nullptr, *q_ = nullptr, *attn_ = nullptr, *act_ = nullptr, *qkv_raw_ = nullptr, *gu_raw_ = nullptr, *logits_ = nullptr;
    unsigned char* xpack_ = nullptr;  // packed activations of one tensor-core projection (gemm_tc.h)
    unsigned char *xpack_attn_ = nullptr, *xpack_act_ = nullptr;  // written directly by the attention kernel / the SwiGLU epilogue
    unsigned char *xpack_h_ = nullptr, *xpack_h2_ = nullptr;      // written by the down / O epilogues: (hidden * next norm weight) for the next QKV or LM head / gate-up GEMM
    float *ss_h_ = nullptr, *ss_h2_ = nullptr;                    // [H/128][64] partial sums of squares of those rows
    uint32_t* qrows_img_ = nullptr;  // Q8_0 / Q4_0 models: digit planes of the up to 64 rows a projection launch multiplies (launch_gemm_quant)
    float* qrows_bs_ = nullptr;      // their block scales
    int qrows_k_ = 0;                // widest projection input the two buffers hold
    int8_t* kqrows_codes_ = nullptr;  // K-quant models: Q8_K codes of the up to 64 rows a projection launch multiplies (launch_gemm_q4k)
    float* kqrows_actd_ = nullptr;    // their block scales
    size_t xpack_bytes_ = 0;
    float* amax_val_ = nullptr;
    int32_t* amax_idx_ = nullptr;
    float* partial_ = nullptr;
    size_t partial_floats_ = 0;
    unsigned int* tickets_ = nullptr;
    float *att_acc_ = nullptr, *att_ml_ = nullptr;
    unsigned int* att_tickets_ = nullptr;
    int att_nsplit_ = 1;
    bool att_cluster_ = true;
    int* err_flag_ = nullptr;
    unsigned int* fin_ticket_ = nullptr;  // ticket of the LM head's folded argmax

    // KV cache
    int batch_ = 0, max_seq_ = 0, page_tokens_ = 16, max_pages_ = 0;
    bool kv_bf16_ = false;
    std::vector<void*> k_pool_, v_pool_;
    int32_t* page_table_ = nullptr;
    int32_t* pos_dev_ = nullptr;      // [batch] current length = position of the next token
    uint32_t* tokens_dev_ = nullptr;  // [batch] input token of the next decode step
    uint32_t* next_dev_ = nullptr;    // [batch] argmax of the last step
    uint32_t* hist_dev_ = nullptr;    // [batch][max_seq+1] token history by position
    std::vector<int> len_;            // host mirror of pos_dev_
    // prefill staging (device), capacity max_seq_
    uint32_t* pf_tokens_ = nullptr;
    int32_t *pf_pos_ = nullptr, *pf_seq_ = nullptr;
    // pinned host staging
    uint32_t* pin_u32_ = nullptr;
    size_t pin_u32_cap_ = 0;
    float* pin_logits_ = nullptr;      // mapped pinned buffer: landing place of logits on their way to pageable memory
    float* pin_logits_dev_ = nullptr;  // the same buffer as the device addresses it
    size_t pin_logits_bytes_ = 0;
    bool alloc_pin_logits(size_t bytes);
    float* logits_landing(float* user, size_t bytes);
    // decode graph whose LM head stores the logits straight into pin_logits_ (see ensure_host_logits_graph)
    cudaGraph_t graph_host_ = nullptr;
    cudaGraphExec_t graph_exec_host_ = nullptr;
    bool host_graph_tried_ = false;
    float* lm_out_ = nullptr;  // LM-head destination override while that graph is being captured
    void drop_host_logits_graph();

    cudaGraph_t graph_ = nullptr;
    cudaGraphExec_t graph_exec_ = nullptr;
    int launches_per_step_ = 0;

    int only_class_ = -1;
    bool lm_folds_argmax_ = false;  // the LM-head launch of the last enqueued pass also did the final argmax
    unsigned long long* gemv_trace_ = nullptr;  // builds with -DHM_PHASE_TRACE and HM_GEMV_TRACE=1: [512][16] timestamps, one row per launch of a pass

    // device-side sampler scratch (sampler.cu), allocated on first sampled generation
    float* smp_scaled_ = nullptr;
    int* smp_count_ = nullptr;
    unsigned long long* smp_rng_ = nullptr;
    int32_t* smp_gen_start_ = nullptr;
    int* smp_overflow_ = nullptr;
    std::vector<int> gen_start_;  // host mirror of smp_gen_start_
};

}  // namespace hm
