// Argument block of the persistent decode kernel (decode_persistent.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hm {

constexpr int G_MAX_MK = 8;
// attention scratch in shared memory: raw q/k/v, rotated q, new k, new v, K tile, V tile, probabilities
constexpr int MK_ATT_FLOATS = (G_MAX_MK + 2) * 128 + G_MAX_MK * 128 + 128 + 128 + 16 * (128 + 4) + 16 * 128 + 8 * 16;

// One value handed from CTA to CTA together with the generation (step number) that makes it valid.
struct alignas(8) LL {
    float v;
    uint32_t gen;
};

struct MkLayer {
    const uint16_t *wqkv, *wo, *wgu, *wdown;  // 128-column slab layout
    const float *in_ln, *post_ln, *qkv_bias, *q_norm, *k_norm;
    void *k_pool, *v_pool;
};

struct MkArgs {
    int H, I, heads, kvh, hd, qdim, kvdim, L, V;
    float eps, scale;
    int has_qk_norm, kv_bf16, embed_bf16;
    // phase geometry: slabs, K-splits S and rows per split R
    int slabs_qkv, slabs_h, slabs_gu, slabs_v;
    int S1, R1, S3, R3, S4, R4, S5, R5;
    int att_cap;              // page chunks per KV head (capacity of the attention partial arrays)
    int barriers_per_launch;  // 5 * L + 1
    const MkLayer* layers;    // device array [L]
    const void* embed;
    const uint16_t* wlm;
    const float* final_norm;
    const float *rope_cos, *rope_sin;
    const int32_t* page_table;  // sequence 0
    // sequence state (device)
    const uint32_t* token;
    int32_t* pos;
    uint32_t *next_tok, *feed_tok, *hist;
    // exchange buffers: per layer `layer_stride` entries, sub-arrays at the o_* offsets
    LL* ll;
    size_t layer_stride;
    size_t o_hcur, o_hmid, o_pqkv, o_ssin, o_attml, o_attacc, o_po, o_pgu, o_sspost, o_pdown;
    LL *amax_v, *amax_i;  // [grid] argmax candidates (index stored as int bits)
    float* logits;
    unsigned int* launch_idx;  // step counter: generation = launch_idx + 1
    int* err_flag;
    unsigned long long* trace;  // optional [barriers_per_launch + 1] globaltimer stamps of CTA 0 (HM_MK_TRACE=1)
};

size_t mk_smem_bytes();
int mk_threads();
int mk_xs_max();
cudaError_t mk_prepare(int* max_ctas_per_sm);
cudaError_t launch_decode_persistent(const MkArgs& a, int nb, cudaStream_t st);

}  // namespace hm
