// GGUF K-quant projections: Q4_K and Q6_K super-blocks of 256 weights.
//
// Semantics follow Homura's kernels for these formats (src/graph_builder/emit_quant.rs:165-567 for
// Q4_K, 569-816 for Q6_K, themselves modelled on ggml's vec_dot_q4_K_q8_K / q6_K_q8_K): the f32
// activation row is quantised per 256-value block to Q8_K (scale amax/127, codes roundeven(x*127/amax),
// sums of every 16 codes), the dot products run in integers, and each block contributes
//   Q4_K:  (d*act_d) * sum_sb sc[sb]*isum[sb]  -  (dmin*act_d) * sum_g mn[g/2]*bsums[g]
//   Q6_K:  (d*act_d) * sum_sb sc[sb]*isum[sb]
// in f32.  The LM head and the embedding are NOT run that way by the reference: it widens them to
// f32 (src/gguf.rs:725-812, 833-917) and multiplies f32 x f32, which the ACTQ = false variant of the
// kernel mirrors (f32 activations against weights dequantised in registers).
//
// Layout: as for Q8_0 / Q4_0 (quant.cu) the blocks are re-laid at load in tiles of 32 output rows so
// that a warp's lanes, one output row each, read 512 contiguous bytes per load:
//   tile t, super-block kb:  [piece p][32 rows][16 B], then (Q6_K) the 32 f16 super-block scales
//   Q4_K pieces: 0 = {d, dmin, 12 packed scale bytes}, 1..8 = the 128 nibble bytes
//   Q6_K pieces: 0..7 = ql, 8..11 = qh, 12 = the 16 i8 sub-block scales
// Every (tile, super-block) slot has the Q6_K size, so a projection fused from parts of both types
// (attn_q / attn_k in Q4_K with attn_v in Q6_K, as Q4_K_M files have it) stays one array with one
// type byte per tile.  dp4a does the integer dot products.
#include <algorithm>

#include "common.cuh"
#include "launch_attrs.h"
#include "kquant.h"

namespace hm {
namespace {

constexpr int KT = 256;  // threads

__device__ __forceinline__ void q4k_scales(const uint32_t hdr[4], int sc[8], int mn[8]) {
    // bytes 4..15 of the block header = hdr[1..3]; get_scale_min_k4 (src/gguf.rs:848-864)
    uint8_t sr[12];
#pragma unroll
    for (int i = 0; i < 12; ++i) sr[i] = (uint8_t)(hdr[1 + (i >> 2)] >> (8 * (i & 3)));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        sc[i] = sr[i] & 0x3F;
        mn[i] = sr[4 + i] & 0x3F;
        sc[4 + i] = (sr[8 + i] & 0x0F) | ((sr[i] >> 6) << 4);
        mn[4 + i] = (sr[8 + i] >> 4) | ((sr[4 + i] >> 6) << 4);
    }
}

// ---- bit-exact dequantisation (src/gguf.rs:833-917) -----------------------------------------
__global__ void dequant_k_kernel(const uint8_t* __restrict__ blocks, size_t nblocks, int q6, float* __restrict__ out) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nblocks * 256; i += (size_t)gridDim.x * blockDim.x) {
        const size_t b = i >> 8;
        const int e = (int)(i & 255);
        if (q6) {
            const uint8_t* blk = blocks + b * 210;
            const float d = f16_bits_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
            const int chunk = e >> 7, r = e & 127, group = r >> 5, l = r & 31;
            const uint8_t qlb = blk[chunk * 64 + (group & 1) * 32 + l];
            const int lo = group >= 2 ? (qlb >> 4) : (qlb & 0x0F);
            const int hi = (blk[128 + chunk * 32 + l] >> (group * 2)) & 3;
            const int q = (lo | (hi << 4)) - 32;
            const float sc = (float)(int8_t)blk[192 + (e >> 4)];
            out[i] = __fmul_rn(__fmul_rn(d, sc), (float)q);
        } else {
            const uint8_t* blk = blocks + b * 144;
            const float d = f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            const float dmin = f16_bits_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
            const uint8_t* sr = blk + 4;
            const int sb = e >> 5, l = e & 31;
            int sc, mn;
            if (sb < 4) {
                sc = sr[sb] & 0x3F;
                mn = sr[4 + sb] & 0x3F;
            } else {
                sc = (sr[4 + sb] & 0x0F) | ((sr[sb - 4] >> 6) << 4);
                mn = (sr[4 + sb] >> 4) | ((sr[sb] >> 6) << 4);
            }
            const uint8_t qb = blk[16 + (sb >> 1) * 32 + l];
            const int nib = (sb & 1) ? (qb >> 4) : (qb & 0x0F);
            out[i] = __fsub_rn(__fmul_rn((float)nib, __fmul_rn(d, (float)sc)), __fmul_rn(dmin, (float)mn));
        }
    }
}

// ---- re-layout of GGUF blocks [rows][K/256] into the tiled array ------------------------------
__global__ void kq_split_kernel(const uint8_t* __restrict__ blocks, size_t nblocks, int nb, int q6, int n_off, int interleave_which, int rope_hd, uint8_t* __restrict__ data, uint8_t* __restrict__ tile_type) {
    const int bsz = q6 ? 210 : 144;
    for (size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x; b < nblocks; b += (size_t)gridDim.x * blockDim.x) {
        const uint8_t* s = blocks + b * bsz;
        const int nl = (int)(b / nb), kb = (int)(b % nb);
        const int n = rope_hd > 0 ? rope_tile_row(nl, n_off, rope_hd) : interleave_which >= 0 ? (nl >> 4) * 32 + interleave_which * 16 + (nl & 15) : n_off + nl;
        const int tile = n >> 5, r = n & 31;
        uint8_t* dst = data + ((size_t)tile * nb + kb) * KQ_SLOT_BYTES;
        const int pieces = q6 ? 13 : 9;
        for (int p = 0; p < pieces; ++p)
            for (int j = 0; j < 16; ++j) dst[(p * 32 + r) * 16 + j] = s[p * 16 + j];
        if (q6) {
            dst[13 * 512 + r * 2 + 0] = s[208];
            dst[13 * 512 + r * 2 + 1] = s[209];
        } else {
            // piece 9 (unused by the format's 9 pieces): the eight sub-block scales and minima as bytes, for the row-block kernel
            const uint8_t* sr = s + 4;
            for (int i = 0; i < 4; ++i) {
                dst[(9 * 32 + r) * 16 + i] = sr[i] & 0x3F;
                dst[(9 * 32 + r) * 16 + 8 + i] = sr[4 + i] & 0x3F;
                dst[(9 * 32 + r) * 16 + 4 + i] = (uint8_t)((sr[8 + i] & 0x0F) | ((sr[i] >> 6) << 4));
                dst[(9 * 32 + r) * 16 + 12 + i] = (uint8_t)((sr[8 + i] >> 4) | ((sr[4 + i] >> 6) << 4));
            }
        }
        if (kb == 0) tile_type[tile] = (uint8_t)(q6 ? 2 : 1);
    }
}

__device__ __forceinline__ float u8_f32(uint32_t w, int b) { return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u + b)) - 8388608.0f; }

// One super-block of one output row (this lane) against M activation rows.
// ACTQ: integer dot products against the Q8_K codes in shared memory; else f32 against xs.
template <int M, bool ACTQ>
__device__ __forceinline__ void kq_block_q4k(const uint4 (&pc)[13], const int8_t* __restrict__ q8, const float* __restrict__ act_d, const int32_t* __restrict__ bsums, const float* __restrict__ xs,
                                             const float* __restrict__ xsum16, int kspan, int nbspan, int kbl, float (&acc)[M]) {
    const uint32_t hdr[4] = {pc[0].x, pc[0].y, pc[0].z, pc[0].w};
    const float d = f16_bits_to_f32((uint16_t)(hdr[0] & 0xFFFF)), dmin = f16_bits_to_f32((uint16_t)(hdr[0] >> 16));
    int sc[8], mn[8];
    q4k_scales(hdr, sc, mn);
#pragma unroll
    for (int m = 0; m < M; ++m) {
        if (ACTQ) {
            const int* a32 = reinterpret_cast<const int*>(q8 + (size_t)m * kspan + kbl * 256);
            int scale_accum = 0;
#pragma unroll
            for (int pair = 0; pair < 4; ++pair) {
                int lo_sum = 0, hi_sum = 0;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint4 v = pc[1 + pair * 2 + h];
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        lo_sum = __dp4a((int)(w[i] & 0x0F0F0F0Fu), a32[(pair * 64 + h * 16) / 4 + i], lo_sum);
                        hi_sum = __dp4a((int)((w[i] >> 4) & 0x0F0F0F0Fu), a32[(pair * 64 + 32 + h * 16) / 4 + i], hi_sum);
                    }
                }
                scale_accum += sc[2 * pair] * lo_sum + sc[2 * pair + 1] * hi_sum;
            }
            const int32_t* bs = bsums + ((size_t)m * nbspan + kbl) * 16;
            int min_accum = 0;
#pragma unroll
            for (int g = 0; g < 16; ++g) min_accum += mn[g >> 1] * bs[g];
            const float ad = act_d[m * nbspan + kbl];
            const float kb_val = __fsub_rn(__fmul_rn(__fmul_rn(d, ad), (float)scale_accum), __fmul_rn(__fmul_rn(dmin, ad), (float)min_accum));
            acc[m] = __fadd_rn(acc[m], kb_val);
        } else {
            // f32 activations: sum over sub-blocks of (d*sc) * sum(nib * x) - (dmin*mn) * sum(x)
            const float* xb = xs + (size_t)m * kspan + kbl * 256;
            const float* xs16 = xsum16 + ((size_t)m * nbspan + kbl) * 16;
            float v = 0.f;
#pragma unroll
            for (int pair = 0; pair < 4; ++pair) {
                float lo_p = 0.f, hi_p = 0.f;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint4 q = pc[1 + pair * 2 + h];
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t lo = w[i] & 0x0F0F0F0Fu, hi = (w[i] >> 4) & 0x0F0F0F0Fu;
                        const float4 xl = *reinterpret_cast<const float4*>(xb + pair * 64 + h * 16 + i * 4);
                        const float4 xh = *reinterpret_cast<const float4*>(xb + pair * 64 + 32 + h * 16 + i * 4);
                        lo_p = fmaf(u8_f32(lo, 0), xl.x, lo_p);
                        lo_p = fmaf(u8_f32(lo, 1), xl.y, lo_p);
                        lo_p = fmaf(u8_f32(lo, 2), xl.z, lo_p);
                        lo_p = fmaf(u8_f32(lo, 3), xl.w, lo_p);
                        hi_p = fmaf(u8_f32(hi, 0), xh.x, hi_p);
                        hi_p = fmaf(u8_f32(hi, 1), xh.y, hi_p);
                        hi_p = fmaf(u8_f32(hi, 2), xh.z, hi_p);
                        hi_p = fmaf(u8_f32(hi, 3), xh.w, hi_p);
                    }
                }
                const float sx_lo = xs16[pair * 4 + 0] + xs16[pair * 4 + 1], sx_hi = xs16[pair * 4 + 2] + xs16[pair * 4 + 3];
                v = fmaf(d * (float)sc[2 * pair], lo_p, v);
                v = fmaf(-(dmin * (float)mn[2 * pair]), sx_lo, v);
                v = fmaf(d * (float)sc[2 * pair + 1], hi_p, v);
                v = fmaf(-(dmin * (float)mn[2 * pair + 1]), sx_hi, v);
            }
            acc[m] += v;
        }
    }
}

template <int M, bool ACTQ>
__device__ __forceinline__ void kq_block_q6k(const uint4 (&pc)[13], uint16_t dbits, const int8_t* __restrict__ q8, const float* __restrict__ act_d, const int32_t* __restrict__ bsums,
                                             const float* __restrict__ xs, const float* __restrict__ xsum16, int kspan, int nbspan, int kbl, float (&acc)[M]) {
    const float d = f16_bits_to_f32(dbits);
    const uint32_t scw[4] = {pc[12].x, pc[12].y, pc[12].z, pc[12].w};
#pragma unroll
    for (int m = 0; m < M; ++m) {
        int scale_accum = 0;
        float v = 0.f;
#pragma unroll
        for (int sb = 0; sb < 16; ++sb) {
            const int chunk = sb >> 3, group = (sb & 7) >> 1, parity = sb & 1;
            const uint4 ql = pc[chunk * 4 + (group & 1) * 2 + parity];
            const uint4 qh = pc[8 + chunk * 2 + parity];
            const uint32_t lw[4] = {ql.x, ql.y, ql.z, ql.w}, hw[4] = {qh.x, qh.y, qh.z, qh.w};
            const int s = (int)(int8_t)(scw[sb >> 2] >> (8 * (sb & 3)));
            if (ACTQ) {
                const int* a32 = reinterpret_cast<const int*>(q8 + (size_t)m * kspan + kbl * 256 + sb * 16);
                int isum = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t lo = group >= 2 ? (lw[i] >> 4) & 0x0F0F0F0Fu : lw[i] & 0x0F0F0F0Fu;
                    const uint32_t hi = (hw[i] >> (2 * group)) & 0x03030303u;
                    isum = __dp4a((int)(lo | (hi << 4)), a32[i], isum);  // codes 0..63; the -32 goes through the group sum
                }
                isum -= 32 * bsums[((size_t)m * nbspan + kbl) * 16 + sb];
                scale_accum += s * isum;
            } else {
                const float* xb = xs + (size_t)m * kspan + kbl * 256 + sb * 16;
                float p = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t lo = group >= 2 ? (lw[i] >> 4) & 0x0F0F0F0Fu : lw[i] & 0x0F0F0F0Fu;
                    const uint32_t hi = (hw[i] >> (2 * group)) & 0x03030303u;
                    const uint32_t q = lo | (hi << 4);
                    const float4 x4 = *reinterpret_cast<const float4*>(xb + i * 4);
                    p = fmaf(u8_f32(q, 0), x4.x, p);
                    p = fmaf(u8_f32(q, 1), x4.y, p);
                    p = fmaf(u8_f32(q, 2), x4.z, p);
                    p = fmaf(u8_f32(q, 3), x4.w, p);
                }
                p = fmaf(-32.0f, xsum16[((size_t)m * nbspan + kbl) * 16 + sb], p);
                v = fmaf(d * (float)s, p, v);
            }
        }
        if (ACTQ) acc[m] = __fadd_rn(acc[m], __fmul_rn(__fmul_rn(d, act_d[m * nbspan + kbl]), (float)scale_accum));
        else acc[m] += v;
    }
}

template <int M, bool ACTQ, bool CL>
__global__ void __launch_bounds__(KT) gemv_kquant_kernel(const KQuantArgs a) {
    extern __shared__ __align__(16) unsigned char ksm[];
    const int nbspan = a.kb_per_split, kspan = nbspan * 256;
    // shared memory: [activations: int8 codes or f32][per-block scales][per-16 sums][8 warps x M x 32 partials]
    int8_t* q8 = reinterpret_cast<int8_t*>(ksm);
    float* xs = reinterpret_cast<float*>(ksm);
    unsigned char* p = ksm + (size_t)M * kspan * (ACTQ ? 1 : 4);
    float* act_d = reinterpret_cast<float*>(p);
    p += sizeof(float) * (size_t)M * nbspan;
    int32_t* bsums = reinterpret_cast<int32_t*>(p);  // int32 group sums (ACTQ) or f32 sums of 16 activations
    float* xsum16 = reinterpret_cast<float*>(p);
    p += 4 * (size_t)M * nbspan * 16;
    float* red = reinterpret_cast<float*>(p);
    __shared__ double s_wsum[8][MAX_M];
    __shared__ float s_inv[MAX_M];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = a.K / 256;
    const int tile = blockIdx.x / a.ksplit, split = blockIdx.x - tile * a.ksplit;
    const int kb0 = split * nbspan, kb1 = min(nb, kb0 + nbspan);
    const int nkb = max(0, kb1 - kb0);
    const int ttype = a.tile_type[tile];  // 1 = Q4_K, 2 = Q6_K, 0 = unused tile
    const unsigned char* tbase = a.data + ((size_t)tile * nb + kb0) * KQ_SLOT_BYTES;
    const int npieces = ttype == 2 ? 13 : 9;

    pdl_launch_dependents();
    // weights never depend on the previous kernel: ask the L2 for this CTA's super-blocks before the dependency wait
    // (a Q4_K tile fills 9 of its slot's 13 pieces and no scale words: only the bytes that will be read are asked for)
    if (ttype != 0) {
        const unsigned used = ttype == 2 ? (unsigned)KQ_SLOT_BYTES : 9u * 512u;
        for (int kbl = tid; kbl < nkb; kbl += KT) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(tbase + (size_t)kbl * KQ_SLOT_BYTES), "r"(used) : "memory");
    }
    pdl_wait();

    // ---- prologue: activations of this CTA's K range (RMSNorm with an f64 sum of squares on request,
    //      emitter_quant.rs:713-791), then Q8_K quantisation per 256 values ----
    float inv[M];
#pragma unroll
    for (int m = 0; m < M; ++m) inv[m] = 1.0f;
    // One-round-trip prologue (quantised activations behind an RMSNorm, up to four 256-value blocks per warp): every
    // block of every row is read once, 8 values per lane, and stays in registers while the sums of squares meet in
    // shared memory; the blocks of this CTA's K range are then normalised and quantised from the registers, in the
    // reference's operation order ((x * inv) * w, emitter_quant.rs:713-791, then Q8_K as emit_quant.rs:409-460).
    // (Quantising x * w and applying inv to the finished dot would save the barrier as well, and Q8_K codes are
    // invariant under a positive row factor in exact arithmetic; but a product that rounds the other way moves a
    // code that sits exactly on .5, which the quantised embeddings and bf16 norm weights of the test models produce
    // often enough to leave the tolerance.)
    // Plain rows (O and down projections) take the same path over the blocks of this CTA's K range only.
    constexpr int IT = M == 1 ? 4 : 8;  // a single row keeps its register count (three CTAs per SM)
    const bool normed = a.pro == PRO_RMSNORM;
    const int nbi = normed ? nb : nkb, kbi0 = normed ? 0 : kb0;  // blocks visited per row, and the first of them
    const bool one_pass = ACTQ && (a.ldx & 3) == 0 && M * nbi <= 8 * IT && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 &&
                          (!normed || (reinterpret_cast<uintptr_t>(a.norm_w) & 15) == 0);
    if (one_pass) {
        float4 xa[IT][2];
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int item = warp + 8 * it;
            xa[it][0] = xa[it][1] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (item < M * nbi) {
                const int m = item / nbi, kb = kbi0 + item - m * nbi;
                const float* xr = a.x + (size_t)m * a.ldx + (size_t)kb * 256 + lane * 8;
                xa[it][0] = ld_cg_f32x4(xr);
                xa[it][1] = ld_cg_f32x4(xr + 4);
            }
        }
        if (normed) {
            double ss[M];
#pragma unroll
            for (int m = 0; m < M; ++m) ss[m] = 0.0;
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const int item = warp + 8 * it;
                if (item < M * nbi) {
                    const int m = item / nbi;
                    const float xv[8] = {xa[it][0].x, xa[it][0].y, xa[it][0].z, xa[it][0].w, xa[it][1].x, xa[it][1].y, xa[it][1].z, xa[it][1].w};
                    double sq = 0.0;
#pragma unroll
                    for (int i = 0; i < 8; ++i) sq += (double)xv[i] * (double)xv[i];
#pragma unroll
                    for (int mm = 0; mm < M; ++mm)
                        if (mm == m) ss[mm] += sq;
                }
            }
#pragma unroll
            for (int m = 0; m < M; ++m) {
                double t = ss[m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                if (lane == 0) s_wsum[warp][m] = t;
            }
            __syncthreads();
            if (tid < M) {
                double t = 0.0;
                for (int wv = 0; wv < 8; ++wv) t += s_wsum[wv][tid];
                const float mean = (float)(t * (1.0 / (double)a.K));
                s_inv[tid] = 1.0f / sqrtf(mean + a.eps);
            }
            __syncthreads();
        }
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int item = warp + 8 * it;
            if (item >= M * nbi) continue;
            const int m = item / nbi, kb = kbi0 + item - m * nbi;
            if (kb < kb0 || kb >= kb1) continue;  // warp-uniform
            const int kbl = kb - kb0;
            const float xv[8] = {xa[it][0].x, xa[it][0].y, xa[it][0].z, xa[it][0].w, xa[it][1].x, xa[it][1].y, xa[it][1].z, xa[it][1].w};
            float v[8];
            if (normed) {
                const float4 w0 = __ldg(reinterpret_cast<const float4*>(a.norm_w + (size_t)kb * 256 + lane * 8));
                const float4 w1 = __ldg(reinterpret_cast<const float4*>(a.norm_w + (size_t)kb * 256 + lane * 8 + 4));
                const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                const float rinv = s_inv[m];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = (xv[i] * rinv) * wv[i];
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = xv[i];
            }
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float iscale = amax == 0.f ? 0.f : __fdiv_rn(127.0f, amax);
            int sum = 0;
            uint32_t packed[2] = {0u, 0u};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float r = rintf(__fmul_rn(v[i], iscale));
                r = fminf(r, 127.0f);
                r = fmaxf(r, -127.0f);
                const int q = (int)r;
                sum += q;
                packed[i >> 2] |= ((uint32_t)(q & 0xFF)) << (8 * (i & 3));
            }
            *reinterpret_cast<uint2*>(q8 + (size_t)m * kspan + kbl * 256 + lane * 8) = make_uint2(packed[0], packed[1]);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);  // groups of 16 codes = two lanes
            if ((lane & 1) == 0) bsums[((size_t)m * nbspan + kbl) * 16 + (lane >> 1)] = sum;
            if (lane == 0) act_d[m * nbspan + kbl] = __fdiv_rn(amax, 127.0f);
        }
    } else if (a.pro == PRO_RMSNORM) {
        constexpr int XV = 8;  // rows of up to 8192 elements: every 16-byte piece requested before the first use
        const bool vec_row = (a.K & 3) == 0 && a.K <= XV * 4 * KT && (a.ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            double s = 0.0;
            const float* xr = a.x + (size_t)m * a.ldx;
            if (vec_row) {
                float4 xv[XV];
#pragma unroll
                for (int i = 0; i < XV; ++i) {
                    const int idx = tid + i * KT;
                    xv[i] = idx < (a.K >> 2) ? ld_cg_f32x4(xr + 4 * (size_t)idx) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int i = 0; i < XV; ++i) {
                    s += (double)xv[i].x * (double)xv[i].x;
                    s += (double)xv[i].y * (double)xv[i].y;
                    s += (double)xv[i].z * (double)xv[i].z;
                    s += (double)xv[i].w * (double)xv[i].w;
                }
            } else
            for (int k = tid; k < a.K; k += KT) {
                const double v = (double)xr[k];
                s += v * v;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) s_wsum[warp][m] = s;
        }
        __syncthreads();
        if (tid < M) {
            double s = 0.0;
            for (int wv = 0; wv < 8; ++wv) s += s_wsum[wv][tid];
            const float mean = (float)(s * (1.0 / (double)a.K));
            s_inv[tid] = 1.0f / sqrtf(mean + a.eps);
        }
        __syncthreads();
#pragma unroll
        for (int m = 0; m < M; ++m) inv[m] = s_inv[m];
    }
    // a warp takes whole 256-value blocks: lane holds 8 consecutive values
    for (int item = warp; item < (one_pass ? 0 : M * nkb); item += 8) {
        const int m = item / nkb, kbl = item - m * nkb;
        const float* xr = a.x + (size_t)m * a.ldx + (size_t)(kb0 + kbl) * 256 + lane * 8;
        float v[8];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float x = xr[i];
            if (a.pro == PRO_RMSNORM) x = (x * inv[m]) * a.norm_w[(kb0 + kbl) * 256 + lane * 8 + i];
            v[i] = x;
            amax = fmaxf(amax, fabsf(x));
        }
        if (ACTQ) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float iscale = amax == 0.f ? 0.f : __fdiv_rn(127.0f, amax);
            int sum = 0;
            uint32_t packed[2] = {0u, 0u};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float r = rintf(__fmul_rn(v[i], iscale));
                r = fminf(r, 127.0f);
                r = fmaxf(r, -127.0f);
                const int q = (int)r;
                sum += q;
                packed[i >> 2] |= ((uint32_t)(q & 0xFF)) << (8 * (i & 3));
            }
            *reinterpret_cast<uint2*>(q8 + (size_t)m * kspan + kbl * 256 + lane * 8) = make_uint2(packed[0], packed[1]);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);  // groups of 16 codes = two lanes
            if ((lane & 1) == 0) bsums[((size_t)m * nbspan + kbl) * 16 + (lane >> 1)] = sum;
            if (lane == 0) act_d[m * nbspan + kbl] = __fdiv_rn(amax, 127.0f);
        } else {
            float* dst = xs + (size_t)m * kspan + kbl * 256 + lane * 8;
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
            float s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            if ((lane & 1) == 0) xsum16[((size_t)m * nbspan + kbl) * 16 + (lane >> 1)] = s;
        }
    }
    __syncthreads();

    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    if (ttype != 0) {
        for (int kbl = warp; kbl < nkb; kbl += 8) {
            const unsigned char* slot = tbase + (size_t)kbl * KQ_SLOT_BYTES;
            uint4 pc[13];
#pragma unroll
            for (int q = 0; q < 13; ++q) pc[q] = q < npieces ? ld_stream_u4(reinterpret_cast<const uint4*>(slot) + q * 32 + lane) : make_uint4(0, 0, 0, 0);
            if (ttype == 2) {
                const uint16_t dbits = *reinterpret_cast<const uint16_t*>(slot + 13 * 512 + lane * 2);
                kq_block_q6k<M, ACTQ>(pc, dbits, q8, act_d, bsums, xs, xsum16, kspan, nbspan, kbl, acc);
            } else {
                kq_block_q4k<M, ACTQ>(pc, q8, act_d, bsums, xs, xsum16, kspan, nbspan, kbl, acc);
            }
        }
    }

    // ---- sum the 8 warps (fixed order), then the cluster ranks (fixed order) ----
#pragma unroll
    for (int m = 0; m < M; ++m) red[(warp * M + m) * 32 + lane] = acc[m];
    __syncthreads();
    float v = 0.f;
    if (tid < M * 32) {
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w * M * 32 + tid];
    }
    __syncthreads();
    if (tid < M * 32) red[tid] = v;
    bool writer = true;
    if (CL) {
        // every rank pushes its partial into rank 0's shared memory, arrives at the cluster barrier and is
        // done; rank 0 waits once and adds the slots in rank order from its own memory
        float* slots = red + 8 * M * 32;  // [ksplit][M][32]
        if (tid < M * 32) {
            if (split == 0) slots[tid] = v;
            else st_dsmem_f32(dsmem_addr(slots + split * (M * 32) + tid, 0u), v);
        }
        cluster_arrive_release();
        if (split != 0) return;
        cluster_wait_acquire();
        if (tid < M * 32) {
            v = slots[tid];
            for (int r = 1; r < a.ksplit; ++r) v += slots[r * (M * 32) + tid];
        }
    }
    if (a.epi == EPI_SWIGLU) {
        if (writer && tid < M * 32) red[tid] = v;
        __syncthreads();
        if (writer && tid < M * 32 && (tid & 31) < 16) {
            const int m = tid >> 5, j = tile * 16 + (tid & 31);
            if (m < a.m_valid && j < a.N / 2) {
                const float g = red[tid], u = red[tid + 16];
                a.y[(size_t)m * a.ldy + j] = (g / (1.0f + expf(-g))) * u;
            }
        }
    } else if (a.epi == EPI_QKV_ROPE) {
        if (writer && tid < M * 32) red[tid] = v;
        __syncthreads();
        if (writer && tid < M * 32) rope_tile_epilogue(a.rope, red, v, tid, tile, a.m_valid, a.N, a.bias, a.y, a.ldy);
    } else if (writer && tid < M * 32) {
        const int m = tid >> 5, n = tile * 32 + (tid & 31);
        if (m < a.m_valid && n < a.N) {
            if (a.bias) v += a.bias[n];
            if (a.resid) v = a.resid[(size_t)m * a.ldy + n] + v;
            a.y[(size_t)m * a.ldy + n] = v;
        }
    }
}

template <int M, bool ACTQ, bool CL>
cudaError_t launch_k3(const KQuantArgs& a, cudaStream_t st, bool pdl) {
    const size_t nbs = (size_t)a.kb_per_split;
    const size_t smem = (size_t)M * nbs * 256 * (ACTQ ? 1 : 4) + 4 * (size_t)M * nbs + 4 * (size_t)M * nbs * 16 + 4 * (size_t)8 * M * 32 + (CL ? 4 * (size_t)a.ksplit * M * 32 : 0);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    {
        cudaError_t e = ensure_dyn_smem(gemv_kquant_kernel<M, ACTQ, CL>, smem);
        if (e != cudaSuccess) return e;
    }
    const int tiles = (a.N + 31) / 32;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * a.ksplit));
    cfg.blockDim = dim3(KT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    int n = 0;
    if (pdl) {
        at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (CL) {
        at[n].id = cudaLaunchAttributeClusterDimension;
        at[n].val.clusterDim.x = (unsigned)a.ksplit;
        at[n].val.clusterDim.y = 1;
        at[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = at;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, gemv_kquant_kernel<M, ACTQ, CL>, a);
}

template <int M>
cudaError_t launch_km(const KQuantArgs& a_in, int sm_count, cudaStream_t st, bool pdl) {
    KQuantArgs a = a_in;
    const int nb = a.K / 256, tiles = (a.N + 31) / 32;
    // K split over a cluster: enough CTAs for about two per SM, at most 8 ranks, at least one
    // super-block per CTA, and activations of at most ~48 KB
    int ks = (2 * sm_count + tiles - 1) / tiles;
    ks = std::min(ks, std::min(8, nb));
    const int max_kb = std::max(1, (a.act_quant ? 49152 : 12288) / (M * 256));
    while (ks < std::min(8, nb) && (nb + ks - 1) / ks > max_kb) ++ks;
    ks = std::max(ks, 1);
    a.kb_per_split = (nb + ks - 1) / ks;
    a.ksplit = (nb + a.kb_per_split - 1) / a.kb_per_split;
    if (a.act_quant) return a.ksplit > 1 ? launch_k3<M, true, true>(a, st, pdl) : launch_k3<M, true, false>(a, st, pdl);
    return a.ksplit > 1 ? launch_k3<M, false, true>(a, st, pdl) : launch_k3<M, false, false>(a, st, pdl);
}

}  // namespace

size_t kquant_data_bytes(int K, int N) { return (size_t)((N + 31) / 32) * (K / 256) * KQ_SLOT_BYTES; }
size_t kquant_tiles(int N) { return (size_t)(N + 31) / 32; }

cudaError_t launch_kquant_split(const uint8_t* blocks, int n_rows, int K, int q6, int n_off, int interleave_which, uint8_t* data, uint8_t* tile_type, cudaStream_t st, int rope_hd) {
    if (rope_hd > 0 && ((rope_hd >> 1) % 16 != 0 || n_rows % rope_hd != 0 || n_off % 32 != 0 || interleave_which >= 0)) return cudaErrorInvalidValue;
    const size_t nblocks = (size_t)n_rows * (K / 256);
    size_t g = (nblocks + 127) / 128;
    g = std::min<size_t>(std::max<size_t>(g, 1), 148 * 32);
    kq_split_kernel<<<(unsigned)g, 128, 0, st>>>(blocks, nblocks, K / 256, q6, n_off, interleave_which, rope_hd, data, tile_type);
    return cudaGetLastError();
}

cudaError_t launch_dequant_k(const uint8_t* blocks, size_t nblocks, int q6, float* out, cudaStream_t st) {
    size_t g = (nblocks * 256 + 255) / 256;
    g = std::min<size_t>(std::max<size_t>(g, 1), 148 * 32);
    dequant_k_kernel<<<(unsigned)g, 256, 0, st>>>(blocks, nblocks, q6, out);
    return cudaGetLastError();
}

cudaError_t launch_gemv_kquant(const KQuantArgs& a, int M, int sm_count, cudaStream_t st, bool pdl) {
    if (a.K % 256 != 0) return cudaErrorInvalidValue;
    switch (M) {
        case 1: return launch_km<1>(a, sm_count, st, pdl);
        case 2: return launch_km<2>(a, sm_count, st, pdl);
        case 4: return launch_km<4>(a, sm_count, st, pdl);
        case 8: return launch_km<8>(a, sm_count, st, pdl);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace hm
