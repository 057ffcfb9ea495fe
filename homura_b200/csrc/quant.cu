// GGUF block-quantised projections: Q8_0 (Homura's emit_dequant_matmul_q8_0,
// src/graph_builder/emit_quant.rs:30-142) and Q4_0 (no counterpart in Homura, which maps the
// type to no DType, src/gguf.rs:94-109; defined here from the public ggml block format:
// f16 scale d, 16 bytes, byte i = element i (low nibble) | element i+16 (high nibble),
// value = (nibble - 8) * d).
//
// The codes are small integers, so the block dot products run on the integer tensor-core path
// (mma.sync m16n8k32, s8 x s8 -> s32, exact) without converting a single weight.  The f32
// activations stay f32 in effect: every 32-element block of a row is rewritten once per CTA as
// block floating point, one power-of-two scale and a signed 28-bit integer per element, cut into
// four 7-bit digit planes.  The planes are the columns of the MMA's B operand, so one MMA gives,
// for 16 output rows, the four integer dots  sum_k code_k * digit_t(x_k); they recombine exactly
// in integers two by two and then in f32 as  d_row * 2^s * (I_01 * 2^14 + I_23).  The rounding
// left is 2^-27 of a block's largest activation plus the f32 rounding of each block's partial
// dot, i.e. that of an f32 FMA chain.  Q4_0's "- 8" is a correction by the digit sums of the block.
//
// GGUF stores blocks [N, K/32] of 34 (Q8_0) or 18 (Q4_0) bytes, which no 128-bit load can
// address.  At load the blocks are re-laid in tiles of 32 output rows (same bits, new order),
// in MMA fragment order: lane = 4 * g + q holds rows g, g + 8, g + 16, g + 24 of the tile and
// the k-values 4q..4q+3 and 16+4q..16+4q+3 of the block:
//   scales f16 [N/32][K/32][g 0..7][4 rows]
//   codes Q8_0 [N/32][K/32][row group 0..1][lane][16 B]   (row, k 4q..), (row + 8, k 4q..), (row, k 16+4q..), (row + 8, k 16+4q..)
//   codes Q4_0 [N/32][K/32][lane][16 B]                   bytes 4q..4q+3 of rows g, g + 8, g + 16, g + 24
// so that every lane reads its A fragments with one or two 16-byte loads and its four scales
// with one 8-byte load.  A CTA's 8 warps take the k-blocks of its K range round-robin and are
// summed through shared memory in warp order; K may further be split over the CTAs of a
// thread-block cluster, summed in rank order through distributed shared memory.
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"
#include "launch_attrs.h"
#include "mbarrier.cuh"

namespace hm {


namespace {

constexpr int QT = 256;

// blocks: rows [0, n_part) of a projection part, stored at rows n_off.. of the tiled arrays.
// interleave_which 0 / 1: gate / up rows of a fused SwiGLU projection, 16 + 16 per 32-row tile.
// rope_hd > 0: rows of a head in tiles of 16 first-half dimensions + their 16 rotation partners.
__global__ void split_blocks_kernel(const uint8_t* __restrict__ blocks, size_t nblocks, int nb, int q4, int n_off, int interleave_which, int rope_hd, uint16_t* __restrict__ scales, uint8_t* __restrict__ codes) {
    const int bsz = q4 ? 18 : 34;
    for (size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x; b < nblocks; b += (size_t)gridDim.x * blockDim.x) {
        const uint8_t* s = blocks + b * bsz;
        const int nl = (int)(b / nb), kb = (int)(b % nb);
        int n = interleave_which >= 0 ? (nl >> 4) * 32 + interleave_which * 16 + (nl & 15) : n_off + nl;
        if (rope_hd > 0) n = rope_tile_row(nl, n_off, rope_hd);
        const size_t tk = (size_t)(n >> 5) * nb + kb;
        const int r = n & 31, g = r & 7, r8 = r >> 3;  // row = g + 8 * r8
        scales[tk * 32 + g * 4 + r8] = (uint16_t)(s[0] | (s[1] << 8));
        if (q4) {
            // byte j of the row: lane 4g + (j >> 2), word r8, byte j & 3
            for (int j = 0; j < 16; ++j) codes[(tk * 32 + g * 4 + (j >> 2)) * 16 + r8 * 4 + (j & 3)] = s[2 + j];
        } else {
            // element j of the row: row group r8 >> 1, lane 4g + ((j & 15) >> 2), word (r8 & 1) + 2 * (j >> 4), byte j & 3
            for (int j = 0; j < 32; ++j) codes[((tk * 2 + (r8 >> 1)) * 32 + g * 4 + ((j & 15) >> 2)) * 16 + ((r8 & 1) + 2 * (j >> 4)) * 4 + (j & 3)] = s[2 + j];
        }
    }
}

// Bit-exact unpack: out = f32(code) * f32(f16 scale)  (dequant_q8_0, src/gguf.rs:817-831).
__global__ void dequant_kernel(const uint8_t* __restrict__ blocks, size_t nblocks, int q4, float* __restrict__ out) {
    const int bsz = q4 ? 18 : 34;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nblocks * 32; i += (size_t)gridDim.x * blockDim.x) {
        const size_t b = i / 32;
        const int j = (int)(i % 32);
        const uint8_t* s = blocks + b * bsz;
        const float d = f16_bits_to_f32((uint16_t)(s[0] | (s[1] << 8)));
        float q;
        if (q4) {
            const uint8_t byte = s[2 + (j & 15)];
            q = (float)((int)(j < 16 ? (byte & 0x0F) : (byte >> 4)) - 8);
        } else {
            q = (float)(int8_t)s[2 + j];
        }
        out[i] = q * d;
    }
}

constexpr int QU = 4;  // k-blocks a warp keeps in flight

// D = A * B with a zero accumulator
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Shared-memory image of the activations, per k-block and per pair of rows (one MMA's eight B columns = two rows x
// four digit planes):  img [kb][pair][half of the block][column][4 B = k 4q..4q+3]  (lane 4 * column + q reads word
// `lane` of each half) and bs [kb][pair][2], the rows' block scales 2^s.  A single row (M = 1) keeps four columns;
// the lanes of the other four read the same words and their results are dropped.
template <int M>
struct Img {
    static constexpr int NG = (M + 1) / 2;
    static constexpr int HALF = M == 1 ? 16 : 32;  // words per half block
    static constexpr int WORDS = 2 * HALF;          // per (k-block, row pair)
};

// One 16-byte piece (elements 4 * sub .. 4 * sub + 3 of a 32-element block, the block's eight pieces held by eight
// consecutive lanes) becomes four digit words.  The block's elements are q = rint(x * 2^(29 - e)) with e the exponent
// of the block's largest magnitude (|q| <= 2^30), and q = ((b3 * 256 + b2) * 256 + b1) * 256 + b0 with every b in
// -128..127: adding 0x808080 and flipping those three bits again turns the bytes of q into exactly these digits.
// Blocks below 2^-96 count as zero; a block holding an infinity or a NaN gets a NaN scale.  Every lane of the warp
// must call this (shuffles); only lanes with `store` write.
template <int M>
__device__ __forceinline__ void emit_digits(float4 v, bool store, int slot, int m, int sub, uint32_t* __restrict__ img, float* __restrict__ bs) {
    float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    // fmaxf drops a NaN operand: carry the "not finite" bit of every element beside the maximum
    unsigned nonfinite = ((__float_as_uint(v.x) & 0x7F800000u) == 0x7F800000u) | ((__float_as_uint(v.y) & 0x7F800000u) == 0x7F800000u) |
                         ((__float_as_uint(v.z) & 0x7F800000u) == 0x7F800000u) | ((__float_as_uint(v.w) & 0x7F800000u) == 0x7F800000u);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        nonfinite |= __shfl_xor_sync(0xffffffffu, nonfinite, o);
    }
    const int e = (int)((__float_as_uint(mx) >> 23) & 255u);
    const bool live = e >= 31 && !nonfinite;
    const float mult = live ? __uint_as_float((uint32_t)(283 - e) << 23) : 0.f;
    const float scale = nonfinite ? __uint_as_float(0x7FC00000u) : (live ? __uint_as_float((uint32_t)(e - 29) << 23) : 0.f);
    uint32_t d[4];
    const float xv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) d[j] = ((uint32_t)__float2int_rn(xv[j] * mult) + 0x00808080u) ^ 0x00808080u;
    // 4 x 4 byte transpose: word t = digit t of the four elements
    const uint32_t t01 = __byte_perm(d[0], d[1], 0x5140), t23 = __byte_perm(d[2], d[3], 0x5140);
    const uint32_t u01 = __byte_perm(d[0], d[1], 0x7362), u23 = __byte_perm(d[2], d[3], 0x7362);
    if (store) {
        uint32_t* dst = img + (size_t)slot * Img<M>::WORDS + (sub >> 2) * Img<M>::HALF + (m & 1) * 16 + (sub & 3);
        dst[0] = __byte_perm(t01, t23, 0x5410);
        dst[4] = __byte_perm(t01, t23, 0x7632);
        dst[8] = __byte_perm(u01, u23, 0x5410);
        dst[12] = __byte_perm(u01, u23, 0x7632);
        if (sub == 0) bs[slot * 2 + (m & 1)] = scale;
    }
}

// rows staged as f32 [M][kspan] -> digit image (the path for rows that the register path below cannot take)
template <int M>
__device__ __forceinline__ void build_digit_image(const float* __restrict__ xs, int kspan, int nkb, uint32_t* __restrict__ img, float* __restrict__ bs, int tid) {
    const int sub = tid & 7, total = nkb * M;
    for (int base = 0; base < total; base += QT / 8) {
        const int it = base + (tid >> 3);
        const bool valid = it < total;
        const int kb = it / M, m = it - kb * M;
        const float4 v = valid ? *reinterpret_cast<const float4*>(xs + (size_t)m * kspan + kb * 32 + sub * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        emit_digits<M>(v, valid, kb * Img<M>::NG + (m >> 1), m, sub, img, bs);
    }
}

// One k-block of a 32-row tile against NG row pairs.  Lane 4g + q ends up with, for the tile rows g, g + 8, g + 16,
// g + 24 and activation row 2 * pair + (q >> 1), the partial over the digit planes 2 * (q & 1) and 2 * (q & 1) + 1;
// the caller weights the two halves by 1 and 2^16 and adds them.
template <int M, bool Q4>
__device__ __forceinline__ void q_block(const uint4 (&c)[2], uint2 sc, const uint32_t* __restrict__ img, const float* __restrict__ bs, int lane, float (&acc)[Img<M>::NG][4]) {
    constexpr int NG = Img<M>::NG;
    uint32_t a[2][4];
    if (Q4) {
        // word r8: bytes 4q..4q+3 of row g + 8 * r8; low nibbles = elements 4q.., high nibbles = elements 16 + 4q..
        const uint32_t w[4] = {c[0].x, c[0].y, c[0].z, c[0].w};
#pragma unroll
        for (int rg = 0; rg < 2; ++rg) {
            a[rg][0] = w[2 * rg] & 0x0F0F0F0Fu;
            a[rg][1] = w[2 * rg + 1] & 0x0F0F0F0Fu;
            a[rg][2] = (w[2 * rg] >> 4) & 0x0F0F0F0Fu;
            a[rg][3] = (w[2 * rg + 1] >> 4) & 0x0F0F0F0Fu;
        }
    } else {
#pragma unroll
        for (int rg = 0; rg < 2; ++rg) {
            a[rg][0] = c[rg].x;
            a[rg][1] = c[rg].y;
            a[rg][2] = c[rg].z;
            a[rg][3] = c[rg].w;
        }
    }
    const float2 d01 = __half22float2(*reinterpret_cast<const __half2*>(&sc.x)), d23 = __half22float2(*reinterpret_cast<const __half2*>(&sc.y));
    const float d[4] = {d01.x, d01.y, d23.x, d23.y};
    const int li = M == 1 ? (lane & 15) : lane;
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        const uint32_t b0 = img[ng * Img<M>::WORDS + li], b1 = img[ng * Img<M>::WORDS + Img<M>::HALF + li];
        const float bsv = bs[ng * 2 + ((lane >> 1) & 1)];
        int off = 0;
        if (Q4) {
            // the nibbles enter as 0..15: take 8 x the digit sums of the block off again (an all-ones A gives them in every row)
            int cs[4];
            mma_s8(cs, 0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u, b0, b1);
            off = (cs[1] * 256 + cs[0]) * 8;
        }
#pragma unroll
        for (int rg = 0; rg < 2; ++rg) {
            int cc[4];
            mma_s8(cc, a[rg][0], a[rg][1], a[rg][2], a[rg][3], b0, b1);
            const int i0 = cc[1] * 256 + cc[0] - off, i1 = cc[3] * 256 + cc[2] - off;
            acc[ng][2 * rg] = fmaf(d[2 * rg] * bsv, (float)i0, acc[ng][2 * rg]);
            acc[ng][2 * rg + 1] = fmaf(d[2 * rg + 1] * bsv, (float)i1, acc[ng][2 * rg + 1]);
        }
    }
}

// ST: the CTA's whole slice of codes and scales (two contiguous byte ranges of the tiled arrays) is pulled into
// shared memory by two bulk copies issued BEFORE the dependency wait, so that in the decode chain the weights'
// HBM latency overlaps the launch before this one and the multiply runs out of shared memory.
template <int M, bool Q4, bool CL, bool ST>
__global__ void __launch_bounds__(QT, (M == 1 && ST) ? 3 : 1) gemv_quant_kernel(const QuantArgs a) {
    extern __shared__ __align__(128) float qsm[];
    // A staged slice may leave its last eight k-blocks (one per warp) in global memory: 8.5 KB less per CTA is what lets
    // three CTAs of the Q8_0 gate/up projection share an SM, i.e. the whole launch be resident at once.
    const int tail = ST ? a.reg_tail : 0;
    const int kbs_st = a.kb_per_split - 8 * tail;  // staged k-blocks (capacity)
    const int kspan = a.kb_per_split * 32;  // activations this CTA needs
    constexpr int CHB = (Q4 ? 1 : 2) * 512;  // code bytes of one k-block of a 32-row tile
    // staged weights first (bulk copies want 16-byte aligned destinations): codes, then scales
    const unsigned char* codes_s = reinterpret_cast<const unsigned char*>(qsm);
    const uint16_t* scales_s = reinterpret_cast<const uint16_t*>(codes_s + (size_t)kbs_st * CHB);
    constexpr int NG = Img<M>::NG;  // pairs of activation rows = MMAs per block and row group
    constexpr int IW = Img<M>::WORDS;
    float* xs = ST ? qsm + ((size_t)kbs_st * (CHB + 64)) / 4 : qsm;  // [M][kspan] f32, only when the rows cannot go from registers to digits
    uint32_t* img = reinterpret_cast<uint32_t*>(xs + (a.from_regs ? 0 : M * kspan));  // [kb][NG][IW]
    float* bsc = reinterpret_cast<float*>(img + (size_t)a.kb_per_split * NG * IW);     // [kb][NG][2]
    float* red = bsc + a.kb_per_split * NG * 2;                                        // [8 warps][M][32], then vals [M][32] at red[0..]
    constexpr int NCHUNK = 4;           // the slice arrives in up to four pieces, each on its own barrier, so that the
    __shared__ uint64_t s_wbar[NCHUNK];  // multiply of a CTA that started late overlaps the rest of its copies
    __shared__ volatile int s_abort;
    __shared__ double s_wsum[8][MAX_M];
    __shared__ float s_inv[MAX_M];
    __shared__ float s_post[MAX_M];  // RMSNorm factor still to be applied to the finished dot (1 when the rows were scaled before the digits)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = a.K / 32;
    const int tile = blockIdx.x / a.ksplit, split = blockIdx.x - tile * a.ksplit;
    const int kb0 = split * a.kb_per_split, kb1 = min(nb, kb0 + a.kb_per_split);
    const int nkb = max(0, kb1 - kb0);
    constexpr int CH = Q4 ? 1 : 2;
    const uint4* cbase = reinterpret_cast<const uint4*>(a.codes) + ((size_t)tile * nb + kb0) * (CH * 32) + lane;
    const uint2* sbase = reinterpret_cast<const uint2*>(a.scales + ((size_t)tile * nb + kb0) * 32) + (lane >> 2);  // the lane's four rows

    HM_TRACE(const bool tr = a.trace != nullptr && blockIdx.x == 0 && tid == 0;)
    HM_TRACE(if (tr) a.trace[0] = global_timer();)
    HM_TRACE(if (a.trace && tid == 0) atomicMax(a.trace + 8, global_timer());)
    pdl_launch_dependents();

    // weights never depend on a previous kernel: the whole slice into shared memory (ST), or the first batch of
    // streaming loads into registers, before the dependency wait
    uint4 c[QU][2];
    uint2 sc[QU];
    const int nkb_s = nkb - 8 * tail;  // staged k-blocks of this CTA (the launcher asks for a tail only on unsplit K of at least 16 blocks)
    const int ck = max(8, ((nkb_s + NCHUNK - 1) / NCHUNK + 7) / 8 * 8);  // k-blocks per piece: a multiple of the 8 warps
    if (ST) {
        if (tid == 0) {
            for (int ch = 0; ch < NCHUNK; ++ch) mb_init(&s_wbar[ch], 1);
            s_abort = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            const unsigned char* csrc = reinterpret_cast<const unsigned char*>(a.codes) + ((size_t)tile * nb + kb0) * CHB;
            for (int ch = 0; ch < NCHUNK; ++ch) {
                const int k_lo = min(nkb_s, ch * ck), k_hi = min(nkb_s, k_lo + ck);
                if (k_hi <= k_lo) break;
                const uint32_t cbytes = (uint32_t)(k_hi - k_lo) * CHB, sbytes = ch == 0 ? (uint32_t)nkb_s * 64u : 0u;
                mb_expect_tx(&s_wbar[ch], cbytes + sbytes);
                if (sbytes) bulk_copy(const_cast<uint16_t*>(scales_s), a.scales + ((size_t)tile * nb + kb0) * 32, sbytes, &s_wbar[0]);
                bulk_copy(const_cast<unsigned char*>(codes_s) + (size_t)k_lo * CHB, csrc + (size_t)k_lo * CHB, cbytes, &s_wbar[ch]);
            }
        }
    } else {
#pragma unroll
        for (int u = 0; u < QU; ++u) {
            const int kb = warp + 8 * u;
            const bool ok = kb < nkb;
#pragma unroll
            for (int h = 0; h < CH; ++h) c[u][h] = ok ? ld_stream_u4(cbase + ((size_t)kb * CH + h) * 32) : make_uint4(0, 0, 0, 0);
            sc[u] = ok ? __ldg(sbase + (size_t)kb * 8) : make_uint2(0u, 0u);
        }
    }

    // RMSNorm weights of the whole row (they do not depend on the previous kernel either): up to XV 16-byte pieces
    // per thread, requested before the dependency wait
    constexpr int XV = 8;  // rows of up to 8192 elements take the one-round-trip path below
    const bool vec_row = a.from_regs && a.pro == PRO_RMSNORM;
    const int k4 = a.K >> 2;
    float4 nwv[XV];
    if (vec_row) {
#pragma unroll
        for (int i = 0; i < XV; ++i) {
            const int idx = tid + i * QT;
            nwv[i] = idx < k4 ? __ldg(reinterpret_cast<const float4*>(a.norm_w) + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }

    pdl_wait();
    HM_TRACE(if (tr) a.trace[1] = global_timer();)

    // ---- prologue: this CTA's K range of every activation row becomes the digit image ----
    if (tid < M) s_post[tid] = 1.0f;
    if (vec_row) {
        // One L2 round trip per row: every piece of the row is requested before the first use.  The pieces in this
        // CTA's K range go from the registers to digits at once, as x * norm_weight; the RMSNorm factor is a scalar of
        // the row and multiplies the finished dot instead (s_post), so that nothing waits for the sum of squares, which
        // runs in f64 as the reference's GGUF path does (emitter_quant.rs:713-791) and is only reduced after the multiply.
        const int lo = kb0 * 32, hi = lo + nkb * 32;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float4* xr4 = reinterpret_cast<const float4*>(a.x + (size_t)m * a.ldx);
            float4 xv[XV];
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                const int idx = tid + i * QT;
                xv[i] = idx < k4 ? ld_cg_f32x4(reinterpret_cast<const float*>(xr4 + idx)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                if (i * QT >= k4) break;  // uniform: the row ends before this round of pieces
                const int el = (tid + i * QT) * 4;
                const bool in = el >= lo && el < hi;
                if (!__any_sync(0xffffffffu, in)) continue;
                const float4 v = make_float4(xv[i].x * nwv[i].x, xv[i].y * nwv[i].y, xv[i].z * nwv[i].z, xv[i].w * nwv[i].w);
                emit_digits<M>(v, in, ((el - lo) >> 5) * NG + (m >> 1), m, tid & 7, img, bsc);
            }
            double ssq = 0.0;
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                if (i * QT >= k4) break;
                ssq += (double)xv[i].x * (double)xv[i].x;
                ssq += (double)xv[i].y * (double)xv[i].y;
                ssq += (double)xv[i].z * (double)xv[i].z;
                ssq += (double)xv[i].w * (double)xv[i].w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
            if (lane == 0) s_wsum[warp][m] = ssq;
        }
    } else if (a.from_regs) {
        // plain rows: this CTA's range, 16 bytes per lane, all rows requested before the first use
        const int n4 = nkb * 8;
        for (int p0 = 0; p0 < n4; p0 += QT) {
            const int p = p0 + tid;
            const bool in = p < n4;
            float4 xv[M];
#pragma unroll
            for (int m = 0; m < M; ++m) xv[m] = in ? ld_cg_f32x4(a.x + (size_t)m * a.ldx + kb0 * 32 + 4 * (size_t)p) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (!__any_sync(0xffffffffu, in)) continue;
#pragma unroll
            for (int m = 0; m < M; ++m) emit_digits<M>(xv[m], in, (p >> 3) * NG + (m >> 1), m, tid & 7, img, bsc);
        }
    } else {
        if (a.pro == PRO_RMSNORM) {
            // sum of squares in f64 over the whole row (emitter_quant.rs:713-791)
#pragma unroll
            for (int m = 0; m < M; ++m) {
                double ssq = 0.0;
                const float* xr = a.x + (size_t)m * a.ldx;
                for (int k = tid; k < a.K; k += QT) {
                    const double v = (double)xr[k];
                    ssq += v * v;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
                if (lane == 0) s_wsum[warp][m] = ssq;
            }
            __syncthreads();
            if (tid < M) {
                double t = 0.0;
                for (int wv = 0; wv < 8; ++wv) t += s_wsum[wv][tid];
                const float mean = (float)(t * (1.0 / (double)a.K));
                s_inv[tid] = 1.0f / sqrtf(mean + a.eps);
            }
            __syncthreads();
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float inv = s_inv[m];
                const float* xr = a.x + (size_t)m * a.ldx + kb0 * 32;
                for (int k = tid; k < nkb * 32; k += QT) xs[m * kspan + k] = (xr[k] * inv) * a.norm_w[kb0 * 32 + k];
            }
        } else {
            stage_rows<QT, M>(a.x + kb0 * 32, a.ldx, xs, kspan, nkb * 32, tid);
        }
        __syncthreads();
        build_digit_image<M>(xs, kspan, nkb, img, bsc, tid);
    }
    __syncthreads();
    HM_TRACE(if (tr) a.trace[2] = global_timer();)

    float acc[NG][4];
#pragma unroll
    for (int ng = 0; ng < NG; ++ng)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[ng][i] = 0.f;
    if (ST) {
        // every thread waits (bounded) for the two bulk copies, then the warp's k-blocks come from shared memory:
        // lane = output row, 16-byte reads of consecutive lanes are consecutive (no bank conflicts)
        int waited = -1;
        bool ok = true;
        // the warp's unstaged block, requested now and multiplied last
        const int kbt = nkb_s + ((warp - nkb_s) & 7);
        uint4 tc[2];
        uint2 tsc = make_uint2(0u, 0u);
        if (tail) {
#pragma unroll
            for (int h = 0; h < CH; ++h) tc[h] = ld_stream_u4(cbase + ((size_t)kbt * CH + h) * 32);
            tsc = __ldg(sbase + (size_t)kbt * 8);
        }
        for (int kb = warp; kb < nkb_s && ok; kb += 8) {
            while (kb >= (waited + 1) * ck && ok) {  // the piece that holds this k-block
                ++waited;
                ok = __all_sync(0xffffffffu, mb_wait(&s_wbar[waited], 0, a.err_flag, &s_abort));
                HM_TRACE(if (tr && waited == 0) a.trace[10] = global_timer();)  // first piece of the staged weights has landed
            }
            if (!ok) break;
            uint4 cc[2];
#pragma unroll
            for (int h = 0; h < CH; ++h) cc[h] = *reinterpret_cast<const uint4*>(codes_s + ((size_t)(kb * CH + h) * 32 + lane) * 16);
            q_block<M, Q4>(cc, *reinterpret_cast<const uint2*>(scales_s + kb * 32 + (lane >> 2) * 4), img + (size_t)kb * NG * IW, bsc + kb * NG * 2, lane, acc);
        }
        if (tail && ok) q_block<M, Q4>(tc, tsc, img + (size_t)kbt * NG * IW, bsc + kbt * NG * 2, lane, acc);
    } else
    for (int base = warp; base < nkb; base += 8 * QU) {
        // issue the next batch, then consume the current one
        uint4 cn[QU][2];
        uint2 sn[QU];
#pragma unroll
        for (int u = 0; u < QU; ++u) {
            const int kb = base + 8 * (QU + u);
            const bool ok = kb < nkb;
#pragma unroll
            for (int h = 0; h < CH; ++h) cn[u][h] = ok ? ld_stream_u4(cbase + ((size_t)kb * CH + h) * 32) : make_uint4(0, 0, 0, 0);
            sn[u] = ok ? __ldg(sbase + (size_t)kb * 8) : make_uint2(0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < QU; ++u) {
            const int kb = base + 8 * u;
            if (kb < nkb) q_block<M, Q4>(c[u], sc[u], img + (size_t)kb * NG * IW, bsc + kb * NG * 2, lane, acc);
        }
#pragma unroll
        for (int u = 0; u < QU; ++u) {
            c[u][0] = cn[u][0];
            if (!Q4) c[u][1] = cn[u][1];
            sc[u] = sn[u];
        }
    }

    // ---- sum the 8 warps (fixed order), then the cluster ranks (fixed order) ----
    HM_TRACE(if (tr) a.trace[3] = global_timer();)
    // the lane pair (q even, q odd) holds the two halves of a dot: planes 0,1 weigh 1, planes 2,3 weigh 2^16
    {
        const int q = lane & 3, g = lane >> 2;
        const float wgt = (q & 1) ? 65536.0f : 1.0f;
#pragma unroll
        for (int ng = 0; ng < NG; ++ng) {
            const int m = 2 * ng + (q >> 1);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float mine = acc[ng][i] * wgt;
                const float sum = mine + __shfl_xor_sync(0xffffffffu, mine, 1);  // a + b == b + a: both lanes hold the same bits
                if ((q & 1) == 0 && m < M) red[(warp * M + m) * 32 + 8 * i + g] = sum;
            }
        }
    }
    __syncthreads();
    float v = 0.f;
    if (tid < M * 32) {
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w * M * 32 + tid];
    }
    if (vec_row && tid >= QT - M) {
        // the rows' RMSNorm factors, by threads that have no part in the sum above
        const int m = tid - (QT - M);
        double t = 0.0;
        for (int wv = 0; wv < 8; ++wv) t += s_wsum[wv][m];
        const float mean = (float)(t * (1.0 / (double)a.K));
        s_post[m] = 1.0f / sqrtf(mean + a.eps);
    }
    __syncthreads();
    if (tid < M * 32) red[tid] = v;  // vals [M][32]
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
        if (split != 0) {
            HM_TRACE(if (a.trace && tid == 0) atomicMax(a.trace + 9, global_timer());)
            return;
        }
        cluster_wait_acquire();
        HM_TRACE(if (tr) a.trace[4] = global_timer();)
        if (tid < M * 32) {
            v = slots[tid];
            for (int r = 1; r < a.ksplit; ++r) v += slots[r * (M * 32) + tid];
        }
    }
    if (tid < M * 32) v *= s_post[tid >> 5];
    HM_TRACE(if (tr) a.trace[5] = global_timer();)
    if (a.epi == EPI_SWIGLU) {
        // tile = 16 gate rows followed by the 16 matching up rows
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
        // a q or k tile holds 16 dimensions of a head's first half and, 16 rows further, their rotation partners
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
    HM_TRACE(if (tr) a.trace[6] = global_timer();)
    HM_TRACE(if (a.trace && tid == 0) atomicMax(a.trace + 9, global_timer());)
}

constexpr size_t QUANT_STAGE_MAX = 96 * 1024;  // largest weight slice staged in shared memory (two CTAs per SM stay resident)

template <int M, bool Q4, bool CL, bool ST>
cudaError_t launch_q4(const QuantArgs& a, size_t smem, cudaStream_t st, bool pdl);

template <int M, bool Q4, bool CL>
cudaError_t launch_q3(const QuantArgs& a_in, int sm_count, cudaStream_t st, bool pdl) {
    QuantArgs a = a_in;
    // rows go from registers straight to digits when 16-byte loads can address them (RMSNorm: whole rows of up to 8192 elements)
    a.from_regs = (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (a.ldx & 3) == 0 &&
                  (a.pro != PRO_RMSNORM || ((reinterpret_cast<uintptr_t>(a.norm_w) & 15) == 0 && (a.K & 3) == 0 && a.K <= 8 * 4 * QT));
    size_t smem = sizeof(float) * ((a.from_regs ? 0 : (size_t)M * a.kb_per_split * 32) + (size_t)a.kb_per_split * Img<M>::NG * (Img<M>::WORDS + 2) + 8 * M * 32 + (CL ? (size_t)a.ksplit * M * 32 : 0));
    constexpr size_t BLK = (Q4 ? 1 : 2) * 512 + 64;  // staged bytes per k-block
    size_t slice = (size_t)a.kb_per_split * BLK;
    const bool aligned = ((reinterpret_cast<uintptr_t>(a.codes) | reinterpret_cast<uintptr_t>(a.scales)) & 15) == 0;
#ifndef HM_QUANT_NO_STAGE
    if (aligned && slice <= QUANT_STAGE_MAX && smem + slice <= 110 * 1024) {
        // CTAs an SM holds: three by registers (M = 1), fewer by shared memory (1 KB per CTA is the system's)
        const auto per_sm = [](size_t bytes) { return (int)std::min<size_t>(M == 1 ? 3 : 2, (227 * 1024) / (bytes + 1024 + 1024)); };
        const long ctas = (long)((a.N + 31) / 32) * a.ksplit;
        if (a.ksplit == 1 && a.kb_per_split >= 16 && ctas > (long)per_sm(smem + slice) * sm_count && per_sm(smem + slice - 8 * BLK) > per_sm(smem + slice)) {
            a.reg_tail = 1;  // one more CTA per SM: the Q8_0 gate/up launch becomes resident at once, the LM head runs fewer waves
            slice -= 8 * BLK;
        }
        return launch_q4<M, Q4, CL, true>(a, smem + slice, st, pdl);
    }
#endif
    (void)slice;
    (void)aligned;
    return launch_q4<M, Q4, CL, false>(a, smem, st, pdl);
}

template <int M, bool Q4, bool CL, bool ST>
cudaError_t launch_q4(const QuantArgs& a, size_t smem, cudaStream_t st, bool pdl) {
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    {
        cudaError_t e = ensure_dyn_smem(gemv_quant_kernel<M, Q4, CL, ST>, smem);
        if (e != cudaSuccess) return e;
    }
    const int tiles = (a.N + 31) / 32;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * a.ksplit));
    cfg.blockDim = dim3(QT);
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
    return cudaLaunchKernelEx(&cfg, gemv_quant_kernel<M, Q4, CL, ST>, a);
}

template <int M>
cudaError_t launch_qm(const QuantArgs& a_in, int sm_count, cudaStream_t st, bool pdl) {
    QuantArgs a = a_in;
    const int nb = a.K / 32, tiles = (a.N + 31) / 32;
    // K split: enough CTAs for two per SM, at most 8 per cluster, at least one k-block per warp, and
    // an activation slice of at most 48 KB
    int ks = (2 * sm_count + tiles - 1) / tiles;  // measured: one or three and more CTAs per SM are slower on every format
    if (ks > 8) ks = 8;
    while (ks > 1 && nb / ks < 8) --ks;
    const int max_kb = std::max(1, (12288 / M) / 32);
    while (ks < 8 && (nb + ks - 1) / ks > max_kb) ++ks;
    if (ks < 1) ks = 1;
    a.kb_per_split = (nb + ks - 1) / ks;
    a.ksplit = (nb + a.kb_per_split - 1) / a.kb_per_split;
    if (a.q4) return a.ksplit > 1 ? launch_q3<M, true, true>(a, sm_count, st, pdl) : launch_q3<M, true, false>(a, sm_count, st, pdl);
    return a.ksplit > 1 ? launch_q3<M, false, true>(a, sm_count, st, pdl) : launch_q3<M, false, false>(a, sm_count, st, pdl);
}


// ---- passes over 9..64 rows (prefill chunks, batches of more than eight sequences) -------------------------------
// The 1..8-row kernel lets every CTA rewrite the activation rows as digit planes for itself; with tens of rows that
// prologue outweighs the multiply.  Here one small launch rewrites the rows once (into global memory, which is the
// L2 for the launch that follows), and the multiply's eight warps own eight rows each: every warp walks all k-blocks
// of the CTA's range, the tile's codes staged in shared memory once and read by all of them, so a weight byte that
// crosses the SM's load path serves 64 rows instead of 8 and no sum across warps is needed.
constexpr int GR = 64;                 // rows per launch
constexpr int GPAIRS = GR / 2;         // row pairs per k-block in the image
constexpr int GW = Img<2>::WORDS;      // 64 words per (k-block, pair)

__global__ void __launch_bounds__(QT) quant_pack_rows_kernel(const float* __restrict__ x, int ldx, int M, int K, const float* __restrict__ norm_w, float eps,
                                                             uint32_t* __restrict__ img, float* __restrict__ bs) {
    __shared__ double s_w[8];
    __shared__ float s_inv;
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool row_ok = m < M;  // rows up to GR are written (as zeros) so that the multiply never reads stale planes
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)m * ldx);
    const int k4 = K >> 2;
    float inv = 1.0f;
    if (norm_w) {
        // sum of squares in f64 (emitter_quant.rs:713-791), then (x * inv) * w as the reference orders it
        double ssq = 0.0;
        if (row_ok)
            for (int p = tid; p < k4; p += QT) {
                const float4 v = ld_cg_f32x4(reinterpret_cast<const float*>(xr + p));
                ssq += (double)v.x * (double)v.x + (double)v.y * (double)v.y;
                ssq += (double)v.z * (double)v.z + (double)v.w * (double)v.w;
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        if (lane == 0) s_w[warp] = ssq;
        __syncthreads();
        if (tid == 0) {
            double t = 0.0;
            for (int w = 0; w < 8; ++w) t += s_w[w];
            s_inv = 1.0f / sqrtf((float)(t * (1.0 / (double)K)) + eps);
        }
        __syncthreads();
        inv = s_inv;
    }
    for (int p0 = 0; p0 < k4; p0 += QT) {
        const int p = p0 + tid;
        const bool in = p < k4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in && row_ok) {
            v = ld_cg_f32x4(reinterpret_cast<const float*>(xr + p));
            if (norm_w) {
                const float4 w = __ldg(reinterpret_cast<const float4*>(norm_w) + p);
                v = make_float4((v.x * inv) * w.x, (v.y * inv) * w.y, (v.z * inv) * w.z, (v.w * inv) * w.w);
            }
        }
        if (!__any_sync(0xffffffffu, in)) continue;
        emit_digits<2>(v, in, (p >> 3) * GPAIRS + (m >> 1), m, tid & 7, img, bs);
    }
}

// per-warp ring of B fragments: 16-byte asynchronous copies, four k-blocks ahead
constexpr int GB_STAGES = 4;
constexpr int GB_WORDS = 4 * GW + 8;  // a warp's four row pairs of one k-block (1 KB) + their eight block scales
__device__ __forceinline__ void cp_async16(void* dst_shared, const void* src_global) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(dst_shared)), "l"(src_global) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <bool Q4, bool CL>
__global__ void __launch_bounds__(QT) gemm_quant_kernel(const QuantArgs a) {
    extern __shared__ __align__(128) float gsm[];
    constexpr int CHB = (Q4 ? 1 : 2) * 512;
    constexpr int CH = Q4 ? 1 : 2;
    const unsigned char* codes_s = reinterpret_cast<const unsigned char*>(gsm);
    const uint16_t* scales_s = reinterpret_cast<const uint16_t*>(codes_s + (size_t)a.kb_per_split * CHB);
    // cluster: rank 0's receive slots [ksplit][GR][32] follow the ring, or (alias_slots: when that is what lets two CTAs share
    // an SM) take the place of the staged slice once every rank is done with its own, at the price of a cluster barrier
    const size_t slice_b = (size_t)a.kb_per_split * (CHB + 64), slots_b = CL ? sizeof(float) * GR * 32 * (size_t)a.ksplit : (size_t)0;
    const bool alias = CL && a.alias_slots;
    const size_t head = alias && slots_b > slice_b ? slots_b : slice_b;
    float* vals = gsm + head / 4;                                      // [GR][32] sums of this tile
    uint32_t* bring = reinterpret_cast<uint32_t*>(vals + GR * 32);    // [8 warps][GB_STAGES][GB_WORDS]
    float* slots = alias ? gsm : reinterpret_cast<float*>(bring + 8 * GB_STAGES * GB_WORDS);
    constexpr int NCHUNK = 4;
    __shared__ uint64_t s_wbar[NCHUNK];
    __shared__ volatile int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = a.K / 32;
    const int tile = blockIdx.x / a.ksplit, split = blockIdx.x - tile * a.ksplit;
    const int kb0 = split * a.kb_per_split, kb1 = min(nb, kb0 + a.kb_per_split);
    const int nkb = max(0, kb1 - kb0);
    pdl_launch_dependents();
    // the tile's codes and scales do not depend on the launch in front: staged before the dependency wait, in pieces
    const int ck = max(8, ((nkb + NCHUNK - 1) / NCHUNK + 7) / 8 * 8);
    if (tid == 0) {
        for (int ch = 0; ch < NCHUNK; ++ch) mb_init(&s_wbar[ch], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const unsigned char* csrc = reinterpret_cast<const unsigned char*>(a.codes) + ((size_t)tile * nb + kb0) * CHB;
        for (int ch = 0; ch < NCHUNK; ++ch) {
            const int k_lo = min(nkb, ch * ck), k_hi = min(nkb, k_lo + ck);
            if (k_hi <= k_lo) break;
            const uint32_t cbytes = (uint32_t)(k_hi - k_lo) * CHB, sbytes = ch == 0 ? (uint32_t)nkb * 64u : 0u;
            mb_expect_tx(&s_wbar[ch], cbytes + sbytes);
            if (sbytes) bulk_copy(const_cast<uint16_t*>(scales_s), a.scales + ((size_t)tile * nb + kb0) * 32, sbytes, &s_wbar[0]);
            bulk_copy(const_cast<unsigned char*>(codes_s) + (size_t)k_lo * CHB, csrc + (size_t)k_lo * CHB, cbytes, &s_wbar[ch]);
        }
    }
    pdl_wait();
    __syncthreads();  // barrier words initialised before anybody polls them

    // this warp's eight rows: pairs 4 * warp .. 4 * warp + 3 of every k-block, 1 KB of planes + 32 B of scales, fetched by
    // asynchronous copies into the warp's own ring, GB_STAGES k-blocks ahead of the multiply
    const uint32_t* imgw = a.img_in + ((size_t)kb0 * GPAIRS + 4 * warp) * GW;
    const float* bsw = a.bs_in + ((size_t)kb0 * GPAIRS + 4 * warp) * 2;
    uint32_t* myring = bring + (size_t)warp * GB_STAGES * GB_WORDS;
    float acc[4][4];
#pragma unroll
    for (int ng = 0; ng < 4; ++ng)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[ng][i] = 0.f;
    auto issue = [&](int kb) {
        if (kb < nkb) {
            const uint32_t* src = imgw + (size_t)kb * GPAIRS * GW;
            uint32_t* dst = myring + (kb % GB_STAGES) * GB_WORDS;
            cp_async16(dst + lane * 4, src + lane * 4);
            cp_async16(dst + 128 + lane * 4, src + 128 + lane * 4);
            if (lane < 2) cp_async16(dst + 4 * GW + lane * 4, bsw + (size_t)kb * GPAIRS * 2 + lane * 4);
        }
        cp_async_commit();  // (an empty group past the end keeps the count per k-block uniform)
    };
#pragma unroll
    for (int s0 = 0; s0 < GB_STAGES; ++s0) issue(s0);
    int waited = -1;
    bool ok = true;
    for (int kb = 0; kb < nkb && ok; ++kb) {
        cp_async_wait<GB_STAGES - 1>();
        __syncwarp();
        uint32_t b0[4], b1[4];
        float bsv[4];
        {
            const uint32_t* stg = myring + (kb % GB_STAGES) * GB_WORDS;
#pragma unroll
            for (int ng = 0; ng < 4; ++ng) {
                b0[ng] = stg[ng * GW + lane];
                b1[ng] = stg[ng * GW + 32 + lane];
                bsv[ng] = __uint_as_float(stg[4 * GW + ng * 2 + ((lane >> 1) & 1)]);
            }
        }
        __syncwarp();
        issue(kb + GB_STAGES);
        while (kb >= (waited + 1) * ck && ok) {
            ++waited;
            ok = __all_sync(0xffffffffu, mb_wait(&s_wbar[waited], 0, a.err_flag, &s_abort));
        }
        if (!ok) break;
        uint4 c[2];
#pragma unroll
        for (int h = 0; h < CH; ++h) c[h] = *reinterpret_cast<const uint4*>(codes_s + ((size_t)(kb * CH + h) * 32 + lane) * 16);
        const uint2 sc = *reinterpret_cast<const uint2*>(scales_s + kb * 32 + (lane >> 2) * 4);
        uint32_t av[2][4];
        if (Q4) {
            const uint32_t w[4] = {c[0].x, c[0].y, c[0].z, c[0].w};
#pragma unroll
            for (int rg = 0; rg < 2; ++rg) {
                av[rg][0] = w[2 * rg] & 0x0F0F0F0Fu;
                av[rg][1] = w[2 * rg + 1] & 0x0F0F0F0Fu;
                av[rg][2] = (w[2 * rg] >> 4) & 0x0F0F0F0Fu;
                av[rg][3] = (w[2 * rg + 1] >> 4) & 0x0F0F0F0Fu;
            }
        } else {
#pragma unroll
            for (int rg = 0; rg < 2; ++rg) {
                av[rg][0] = c[rg].x;
                av[rg][1] = c[rg].y;
                av[rg][2] = c[rg].z;
                av[rg][3] = c[rg].w;
            }
        }
        const float2 d01 = __half22float2(*reinterpret_cast<const __half2*>(&sc.x)), d23 = __half22float2(*reinterpret_cast<const __half2*>(&sc.y));
        const float d[4] = {d01.x, d01.y, d23.x, d23.y};
#pragma unroll
        for (int ng = 0; ng < 4; ++ng) {
            int off = 0;
            if (Q4) {
                int cs[4];
                mma_s8(cs, 0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u, b0[ng], b1[ng]);
                off = (cs[1] * 256 + cs[0]) * 8;
            }
#pragma unroll
            for (int rg = 0; rg < 2; ++rg) {
                int cc[4];
                mma_s8(cc, av[rg][0], av[rg][1], av[rg][2], av[rg][3], b0[ng], b1[ng]);
                const int i0 = cc[1] * 256 + cc[0] - off, i1 = cc[3] * 256 + cc[2] - off;
                acc[ng][2 * rg] = fmaf(d[2 * rg] * bsv[ng], (float)i0, acc[ng][2 * rg]);
                acc[ng][2 * rg + 1] = fmaf(d[2 * rg + 1] * bsv[ng], (float)i1, acc[ng][2 * rg + 1]);
            }
        }
    }
    // the lane pair (q even, q odd) holds the two halves of a dot: planes 0,1 weigh 1, planes 2,3 weigh 2^16
    {
        const int q = lane & 3, g = lane >> 2;
        const float wgt = (q & 1) ? 65536.0f : 1.0f;
#pragma unroll
        for (int ng = 0; ng < 4; ++ng) {
            const int m = 8 * warp + 2 * ng + (q >> 1);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float mine = acc[ng][i] * wgt;
                const float sum = mine + __shfl_xor_sync(0xffffffffu, mine, 1);
                if ((q & 1) == 0) vals[m * 32 + 8 * i + g] = sum;
            }
        }
    }
    __syncthreads();
    if (CL) {
        // every rank pushes its sums into rank 0's slots and is done; rank 0 adds them in rank order
        if (alias) cluster_sync_all();  // nobody reads staged codes any more: the slots may overwrite them
        for (int t = tid; t < GR * 32; t += QT) {
            if (split == 0) slots[t] = vals[t];
            else st_dsmem_f32(dsmem_addr(slots + (size_t)split * (GR * 32) + t, 0u), vals[t]);
        }
        cluster_arrive_release();
        if (split != 0) return;
        cluster_wait_acquire();
        for (int t = tid; t < GR * 32; t += QT) {
            float v = slots[t];
            for (int r = 1; r < a.ksplit; ++r) v += slots[(size_t)r * (GR * 32) + t];
            vals[t] = v;
        }
        __syncthreads();
    }
    for (int t = tid; t < GR * 32; t += QT) {
        const int m = t >> 5, p = t & 31;
        float v = vals[t];
        if (a.epi == EPI_SWIGLU) {
            const int j = tile * 16 + p;
            if (p < 16 && m < a.m_valid && j < a.N / 2) {
                const float g = v, u = vals[t + 16];
                a.y[(size_t)m * a.ldy + j] = (g / (1.0f + expf(-g))) * u;
            }
        } else if (a.epi == EPI_QKV_ROPE) {
            rope_tile_epilogue(a.rope, vals, v, t, tile, a.m_valid, a.N, a.bias, a.y, a.ldy);
        } else {
            const int n = tile * 32 + p;
            if (m < a.m_valid && n < a.N) {
                if (a.bias) v += a.bias[n];
                if (a.resid) v = a.resid[(size_t)m * a.ldy + n] + v;
                a.y[(size_t)m * a.ldy + n] = v;
            }
        }
    }
}

template <bool Q4, bool CL>
cudaError_t launch_gq2(const QuantArgs& a, size_t smem, cudaStream_t st, bool pdl) {
    cudaError_t e = ensure_dyn_smem(gemm_quant_kernel<Q4, CL>, smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(((a.N + 31) / 32) * a.ksplit));
    cfg.blockDim = dim3(QT);
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
    return cudaLaunchKernelEx(&cfg, gemm_quant_kernel<Q4, CL>, a);
}

}  // namespace

size_t quant_scale_elems(int K, int N) { return (size_t)((N + 31) / 32) * (K / 32) * 32; }
size_t quant_code_bytes(int K, int N, int q4) { return quant_scale_elems(K, N) * (q4 ? 16 : 32); }

cudaError_t launch_split_blocks(const uint8_t* blocks, int n_rows, int K, int q4, int n_off, int interleave_which, uint16_t* scales, uint8_t* codes, cudaStream_t st, int rope_hd) {
    if (rope_hd > 0 && ((rope_hd >> 1) % 16 != 0 || n_rows % rope_hd != 0 || n_off % 32 != 0 || interleave_which >= 0)) return cudaErrorInvalidValue;
    const size_t nblocks = (size_t)n_rows * (K / 32);
    size_t g = (nblocks + 255) / 256;
    if (g > 148 * 32) g = 148 * 32;
    if (g < 1) g = 1;
    split_blocks_kernel<<<(unsigned)g, 256, 0, st>>>(blocks, nblocks, K / 32, q4, n_off, interleave_which, rope_hd, scales, codes);
    return cudaGetLastError();
}

cudaError_t launch_dequant(const uint8_t* blocks, size_t nblocks, int q4, float* out, cudaStream_t st) {
    size_t g = (nblocks * 32 + 255) / 256;
    if (g > 148 * 32) g = 148 * 32;
    if (g < 1) g = 1;
    dequant_kernel<<<(unsigned)g, 256, 0, st>>>(blocks, nblocks, q4, out);
    return cudaGetLastError();
}

cudaError_t launch_gemv_quant(const QuantArgs& a, int M, int sm_count, cudaStream_t st, bool pdl) {
    switch (M) {
        case 1: return launch_qm<1>(a, sm_count, st, pdl);
        case 2: return launch_qm<2>(a, sm_count, st, pdl);
        case 4: return launch_qm<4>(a, sm_count, st, pdl);
        case 8: return launch_qm<8>(a, sm_count, st, pdl);
        default: return cudaErrorInvalidValue;
    }
}

size_t quant_rows_image_words(int K) { return (size_t)(K / 32) * GPAIRS * GW; }
size_t quant_rows_scale_floats(int K) { return (size_t)(K / 32) * GPAIRS * 2; }
bool quant_rows_supported(const QuantArgs& a) {
    return (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (a.ldx & 3) == 0 && (a.K & 31) == 0 && (!a.norm_w || (reinterpret_cast<uintptr_t>(a.norm_w) & 15) == 0) &&
           ((reinterpret_cast<uintptr_t>(a.codes) | reinterpret_cast<uintptr_t>(a.scales)) & 15) == 0;
}

// Up to 64 rows: one launch that writes the rows' digit planes (img, bs: quant_rows_image_words / quant_rows_scale_floats of
// the projection's K), one that multiplies.  a.m_valid = rows; a.pro / a.norm_w as for launch_gemv_quant.
cudaError_t launch_gemm_quant(const QuantArgs& a_in, uint32_t* img, float* bs, int sm_count, cudaStream_t st, bool pdl, int* launches) {
    QuantArgs a = a_in;
    if (a.m_valid < 1 || a.m_valid > GR || !quant_rows_supported(a)) return cudaErrorInvalidValue;
    cudaError_t e;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(GR);
        cfg.blockDim = dim3(QT);
        cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = pdl ? 1 : 0;
        e = cudaLaunchKernelEx(&cfg, quant_pack_rows_kernel, a.x, a.ldx, a.m_valid, a.K, a.pro == PRO_RMSNORM ? a.norm_w : (const float*)nullptr, a.eps, img, bs);
    }
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
    a.img_in = img;
    a.bs_in = bs;
    const int nb = a.K / 32, tiles = (a.N + 31) / 32;
    const size_t BLK = (a.q4 ? 1 : 2) * 512 + 64;
    // K split: about one CTA per SM, at most 8 per cluster, a staged slice of at most 96 KB
    int ks = (sm_count + tiles - 1) / tiles;
    if (ks > 8) ks = 8;
    while (ks > 1 && nb / ks < 8) --ks;
    while (ks < 8 && (size_t)((nb + ks - 1) / ks) * BLK > QUANT_STAGE_MAX) ++ks;
    if (ks < 1) ks = 1;
    a.kb_per_split = (nb + ks - 1) / ks;
    a.ksplit = (nb + a.kb_per_split - 1) / a.kb_per_split;
    if ((size_t)a.kb_per_split * BLK > QUANT_STAGE_MAX + 32 * 1024) return cudaErrorInvalidValue;  // K beyond what eight ranks can stage
    const size_t slice_b = (size_t)a.kb_per_split * BLK, slots_b = a.ksplit > 1 ? sizeof(float) * GR * 32 * (size_t)a.ksplit : (size_t)0;
    const size_t rest_b = sizeof(float) * GR * 32 + sizeof(uint32_t) * 8 * GB_STAGES * GB_WORDS;
    size_t smem = slice_b + slots_b + rest_b;
    const size_t two_per_sm = 112 * 1024;  // 2 x (this + 1 KB) fits the SM's 227 KB
    if (slots_b && smem > two_per_sm && std::max(slice_b, slots_b) + rest_b <= two_per_sm) {
        a.alias_slots = 1;  // measured: worth the extra cluster barrier only where it doubles the CTAs per SM
        smem = std::max(slice_b, slots_b) + rest_b;
    }
    if (a.q4) e = a.ksplit > 1 ? launch_gq2<true, true>(a, smem, st, pdl) : launch_gq2<true, false>(a, smem, st, pdl);
    else e = a.ksplit > 1 ? launch_gq2<false, true>(a, smem, st, pdl) : launch_gq2<false, false>(a, smem, st, pdl);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace hm
