// Argument block and launchers of the K-quant (Q4_K / Q6_K) projections (kquant.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hm {

constexpr int KQ_SLOT_BYTES = 13 * 512 + 64;  // one (32-row tile, 256-value super-block) slot: Q6_K size, Q4_K uses the first 9 * 512

struct KQuantArgs {
    const unsigned char* data;     // [tiles][K/256][KQ_SLOT_BYTES] (launch_kquant_split)
    const unsigned char* tile_type;  // [tiles]: 1 = Q4_K, 2 = Q6_K, 0 = no rows
    int K, N, m_valid;
    int ksplit, kb_per_split;  // filled in by launch_gemv_kquant
    int act_quant;             // 1: Q8_K activation codes + integer dot (layer projections); 0: f32 activations (LM head)
    const float* x;
    int ldx;
    int pro;  // PRO_PLAIN / PRO_RMSNORM (f64 sum of squares)
    const float* norm_w;
    float eps;
    int epi;  // EPI_STORE, EPI_SWIGLU (gate / up rows interleaved 16 + 16 per tile) or EPI_QKV_ROPE (q and k rows in rotation-pair tiles)
    float* y;
    int ldy;
    const float* bias;
    const float* resid;
    RopeEpi rope;  // EPI_QKV_ROPE
    int* err_flag;            // launch_gemm_q4k: raised to 2 when the bounded wait for the staged slots runs out
    const int8_t* codes_in;   // launch_gemm_q4k: Q8_K codes of the rows [K/256][64][256], written by its packing launch
    const float* actd_in;     // and their block scales [K/256][64]
    int has_q6;               // launch_gemm_q4k: the projection holds Q6_K tiles (slots are staged whole)
    int stage_bytes;          // filled in by launch_gemm_q4k
    int alias_slots;          // filled in by launch_gemm_q4k: rank 0's split-K receive slots reuse the staged slots (one more cluster barrier)
};

size_t kquant_data_bytes(int K, int N);
size_t kquant_tiles(int N);
// GGUF super-blocks of n_rows output rows (q6 = 0: Q4_K, 144 B; 1: Q6_K, 210 B) -> tiled array; rows land at n_off + n,
// or interleaved 16 + 16 per tile when interleave_which is 0 (gate) or 1 (up).  data must start zeroed.
// rope_hd > 0: q or k rows of a fused QKV projection, stored in rotation-pair tiles (rope_tile_row).
cudaError_t launch_kquant_split(const uint8_t* blocks, int n_rows, int K, int q6, int n_off, int interleave_which, uint8_t* data, uint8_t* tile_type, cudaStream_t st, int rope_hd = 0);
cudaError_t launch_dequant_k(const uint8_t* blocks, size_t nblocks, int q6, float* out, cudaStream_t st);
cudaError_t launch_gemv_kquant(const KQuantArgs& a, int M, int sm_count, cudaStream_t st, bool pdl);
// K-quant projection (Q4_K and Q6_K tiles, quantised activations) over up to 64 rows (a.m_valid): a launch that quantises the rows to
// Q8_K (codes / act_d: kquant_rows_code_bytes / kquant_rows_scale_floats of the projection's K) and the multiply.
size_t kquant_rows_code_bytes(int K);
size_t kquant_rows_scale_floats(int K);
bool kquant_rows_supported(const KQuantArgs& a);
cudaError_t launch_gemm_q4k(const KQuantArgs& a, int8_t* codes, float* act_d, int sm_count, cudaStream_t st, bool pdl, int* launches);

}  // namespace hm
