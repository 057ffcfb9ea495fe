// Argument block and launchers of the tensor-core skinny GEMM (gemm_tc.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace hm {

constexpr int TC_ROWS = 64;  // activation rows one launch covers

struct TcArgs {
    const uint16_t* W;  // swizzled K-major tiles [n-block][k-block][128][64] bf16 (launch_pack_tc)
    int K, Kp, N;       // contraction length, K rounded up to 64, output features
    int M;              // activation rows, 1..64
    int ksplit;         // CTAs per cluster sharing one n-block (1 = no split, at most 16)
    const unsigned char* xp;  // activations packed by launch_tc_pack_x (tc_xpack_bytes(M, K) bytes)
    int mpad, nstage, tmem_cols;  // filled in by launch_gemm_tc
    int epi;                 // EPI_STORE (bias, residual), EPI_SWIGLU, EPI_LOGITS or EPI_QKV_ROPE: as in GemvArgs
    const float* bias;       // optional [N]
    const float* resid;      // optional [M][ldy], added as resid + y
    float* y;                // [M][ldy]
    int ldy;
    unsigned char* xp_out;   // EPI_SWIGLU only, optional: write the result as packed activations for the next GEMM instead of y
    int xp_mpad;
    // RMSNorm across two GEMMs without a packing launch in between.  Producer side (EPI_STORE): besides y, the
    // epilogue writes (y * next_norm_w) as the packed activations of the next GEMM and, per 128-feature block,
    // every row's sum of y^2.  Consumer side: the accumulators are scaled by 1 / sqrt(sum of the row's partial
    // sums / K + eps) before the epilogue, i.e. y = inv_rms * (W . (x * w)) instead of W . ((x * inv_rms) * w).
    unsigned char* xp_next;      // producer: activation image of the next GEMM (rows padded to xp_mpad)
    const float* next_norm_w;    // producer: [N] norm weights of the next GEMM's RMSNorm
    float* ss_out;               // producer: [ceil(N/128)][64] partial sums of squares
    const float* ss_in;          // consumer: [ss_parts][64] partial sums of squares of the activation rows, or NULL
    int ss_parts;
    // EPI_QKV_ROPE
    int q_dim, kv_dim, hd, has_qk_norm;
    float eps;
    const float *q_norm_w, *k_norm_w, *rope_cos, *rope_sin;
    const int32_t *row_pos, *row_seq;
    int seq_base;  // row m is sequence seq_base + m when row_seq is null (a 64-row chunk of a larger batch)
    KvDesc kv;
    // EPI_LOGITS: per-row argmax of every 128-feature block
    float* amax_val;
    int32_t* amax_idx;
    int* err_flag;  // set to 2 when a bounded wait ran out
    unsigned long long* trace;  // builds with -DHM_PHASE_TRACE: 16 %globaltimer stamps of CTA 0 of this launch
};

size_t tc_xpack_bytes(int M, int K);  // bytes of the packed activations of M rows
size_t tc_packed_elems(int K, int N);  // bf16 elements of the packed weight (both dims padded)
int tc_padded_k(int K);
int tc_mpad(int M);  // rows padded to 16 / 32 / 64
int tc_pick_split(int K, int N, int sm_count);  // cluster size that fills the SMs once
// f32 rows -> three bf16 terms per element in the tile layout the GEMM copies in bulk; folds an
// RMSNorm (weight norm_w, epsilon eps) when norm_w is not NULL.
cudaError_t launch_tc_pack_x(const float* x, int ldx, int M, int K, const float* norm_w, float eps, void* xp, cudaStream_t st, bool pdl, unsigned long long* trace = nullptr);
cudaError_t launch_gemm_tc(const TcArgs& a, cudaStream_t st, bool pdl);
// src is [N][K] (src_is_kn = false) or [K][N]; rows land at n_off + n, or interleaved 64/64 per
// 128-row block when interleave_which is 0 (gate) or 1 (up).
cudaError_t launch_pack_tc(const uint16_t* src, int N, int K, bool src_is_kn, uint16_t* dst, int n_off, int interleave_which, cudaStream_t st);

}  // namespace hm
