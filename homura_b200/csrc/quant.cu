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
        if (rope_hd > 0) {
            const int head = nl / rope_hd, d = nl - head * rope_hd, half = rope_hd >> 1;
            const int hi = d >= half ? 1 : 0, dd = d - hi * half;
            n = n_off + head * rope_hd + (dd >> 4) * 32 + hi * 16 + (dd & 15);
        }
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

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared-memory image of the activations, per k-block and per pair of rows (one MMA's eight B columns = two rows x
// four digit planes):  img [kb][pair][half of the block][column][4 B = k 4q..4q+3]  (lane 4 * column + q reads word
// `lane` of each half), bs [kb][pair][2] the rows' block scales 2^s, cs [kb][pair][4] eight times the digit sums of
// the column pairs (Q4_0's offset; combined like the dots: 128 * even plane + odd plane).
constexpr int IMG_WORDS = 64;  // per (k-block, row pair)

// A block's elements become q = rint(x * 2^(26 - e)) with e the exponent of the block's largest magnitude (|q| <= 2^27),
// then q = ((d0 * 128 + d1) * 128 + d2) * 128 + d3 with d1..d3 in 0..127 and d0 in -64..64.  Blocks below 2^-100 count
// as zero; a block holding an infinity or a NaN gets a NaN scale.
template <int M>
__device__ __forceinline__ void build_digit_image(const float* __restrict__ xs, int kspan, int nkb, uint32_t* __restrict__ img, float* __restrict__ bs, int* __restrict__ cs, int tid) {
    constexpr int NG = (M + 1) / 2;
    const int sub = tid & 7, total = nkb * M;
    for (int base = 0; base < total; base += QT / 8) {
        const int it = base + (tid >> 3);
        const bool valid = it < total;
        const int kb = it / M, m = it - kb * M;
        const float4 v = valid ? *reinterpret_cast<const float4*>(xs + (size_t)m * kspan + kb * 32 + sub * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
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
        const bool live = e >= 27 && !nonfinite;
        const float mult = live ? __uint_as_float((uint32_t)(280 - e) << 23) : 0.f;
        const float scale = nonfinite ? __uint_as_float(0x7FC00000u) : (live ? __uint_as_float((uint32_t)(e - 26) << 23) : 0.f);
        const float xv[4] = {v.x, v.y, v.z, v.w};
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        int s01 = 0, s23 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int q = nonfinite ? 0 : __float2int_rn(xv[j] * mult);
            const int d3 = q & 127;
            q >>= 7;
            const int d2 = q & 127;
            q >>= 7;
            const int d1 = q & 127;
            const int d0 = q >> 7;
            w[0] |= (uint32_t)(d0 & 255) << (8 * j);
            w[1] |= (uint32_t)d1 << (8 * j);
            w[2] |= (uint32_t)d2 << (8 * j);
            w[3] |= (uint32_t)d3 << (8 * j);
            s01 += d0 * 128 + d1;
            s23 += d2 * 128 + d3;
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            s01 += __shfl_xor_sync(0xffffffffu, s01, o);
            s23 += __shfl_xor_sync(0xffffffffu, s23, o);
        }
        if (valid) {
            const int slot = kb * NG + (m >> 1);
            uint32_t* dst = img + (size_t)slot * IMG_WORDS + (sub >> 2) * 32 + (m & 1) * 16 + (sub & 3);
#pragma unroll
            for (int t = 0; t < 4; ++t) dst[t * 4] = w[t];
            if (M == 1) {  // the pair's second row does not exist
#pragma unroll
                for (int t = 0; t < 4; ++t) dst[16 + t * 4] = 0u;
            }
            if (sub == 0) {
                bs[slot * 2 + (m & 1)] = scale;
                cs[slot * 4 + (m & 1) * 2] = 8 * s01;
                cs[slot * 4 + (m & 1) * 2 + 1] = 8 * s23;
                if (M == 1) {
                    bs[slot * 2 + 1] = 0.f;
                    cs[slot * 4 + 2] = 0;
                    cs[slot * 4 + 3] = 0;
                }
            }
        }
    }
}

// One k-block of a 32-row tile against NG row pairs.  Lane 4g + q ends up with, for the tile rows g, g + 8, g + 16,
// g + 24 and activation row 2 * pair + (q >> 1), the partial over the digit planes 2 * (q & 1) and 2 * (q & 1) + 1;
// the caller weights the two halves by 2^14 and 1 and adds them.
template <int NG, bool Q4>
__device__ __forceinline__ void q_block(const uint4 (&c)[2], uint2 sc, const uint32_t* __restrict__ img, const float* __restrict__ bs, const int* __restrict__ cs, int lane, float (&acc)[NG][4]) {
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
    const int q = lane & 3;
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        const uint32_t b0 = img[ng * IMG_WORDS + lane], b1 = img[ng * IMG_WORDS + 32 + lane];
        const float bsv = bs[ng * 2 + (q >> 1)];
        const int off = Q4 ? cs[ng * 4 + q] : 0;
#pragma unroll
        for (int rg = 0; rg < 2; ++rg) {
            int cc[4] = {0, 0, 0, 0};
            mma_s8(cc, a[rg][0], a[rg][1], a[rg][2], a[rg][3], b0, b1);
            const int i0 = cc[0] * 128 + cc[1] - off, i1 = cc[2] * 128 + cc[3] - off;
            acc[ng][2 * rg] = fmaf(d[2 * rg] * bsv, (float)i0, acc[ng][2 * rg]);
            acc[ng][2 * rg + 1] = fmaf(d[2 * rg + 1] * bsv, (float)i1, acc[ng][2 * rg + 1]);
        }
    }
}

// ST: the CTA's whole slice of codes and scales (two contiguous byte ranges of the tiled arrays) is pulled into
// shared memory by two bulk copies issued BEFORE the dependency wait, so that in the decode chain the weights'
// HBM latency overlaps the launch before this one and the multiply runs out of shared memory.
template <int M, bool Q4, bool CL, bool ST>
__global__ void __launch_bounds__(QT) gemv_quant_kernel(const QuantArgs a) {
    extern __shared__ __align__(128) float qsm[];
    const int kspan = a.kb_per_split * 32;  // activations this CTA needs
    constexpr int CHB = (Q4 ? 1 : 2) * 512;  // code bytes of one k-block of a 32-row tile
    // staged weights first (bulk copies want 16-byte aligned destinations): codes, then scales
    const unsigned char* codes_s = reinterpret_cast<const unsigned char*>(qsm);
    const uint16_t* scales_s = reinterpret_cast<const uint16_t*>(codes_s + (size_t)a.kb_per_split * CHB);
    constexpr int NG = (M + 1) / 2;  // pairs of activation rows = MMAs per block and row group
    float* xs = ST ? qsm + ((size_t)a.kb_per_split * (CHB + 64)) / 4 : qsm;  // [M][kspan] f32, read once by the digit pass
    uint32_t* img = reinterpret_cast<uint32_t*>(xs + M * kspan);                  // [kb][NG][IMG_WORDS]
    float* bsc = reinterpret_cast<float*>(img + (size_t)a.kb_per_split * NG * IMG_WORDS);  // [kb][NG][2]
    int* csum = reinterpret_cast<int*>(bsc + a.kb_per_split * NG * 2);            // [kb][NG][4]
    float* red = reinterpret_cast<float*>(csum + a.kb_per_split * NG * 4);        // [8 warps][M][32], then vals [M][32] at red[0..]
    constexpr int NCHUNK = 4;           // the slice arrives in up to four pieces, each on its own barrier, so that the
    __shared__ uint64_t s_wbar[NCHUNK];  // multiply of a CTA that started late overlaps the rest of its copies
    __shared__ volatile int s_abort;
    __shared__ double s_wsum[8][MAX_M];
    __shared__ float s_inv[MAX_M];
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
    const int ck = max(8, ((nkb + NCHUNK - 1) / NCHUNK + 7) / 8 * 8);  // k-blocks per piece: a multiple of the 8 warps
    if (ST) {
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
    const bool vec_row = a.pro == PRO_RMSNORM && (a.K & 3) == 0 && a.K <= XV * 4 * QT && (a.ldx & 3) == 0 &&
                         ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.norm_w)) & 15) == 0;
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

    // ---- prologue: this CTA's K range of every activation row into shared memory ----
    if (vec_row) {
        // one L2 round trip per row: every piece of the row is requested before the first use, the sum of squares
        // runs in f64 as the reference's GGUF path does (emitter_quant.rs:713-791), and the pieces that fall into
        // this CTA's K range go to shared memory straight from the registers
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
            double s = 0.0;
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                s += (double)xv[i].x * (double)xv[i].x;
                s += (double)xv[i].y * (double)xv[i].y;
                s += (double)xv[i].z * (double)xv[i].z;
                s += (double)xv[i].w * (double)xv[i].w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) s_wsum[warp][m] = s;
            __syncthreads();
            if (tid == 0) {
                double t = 0.0;
                for (int wv = 0; wv < 8; ++wv) t += s_wsum[wv][m];
                const float mean = (float)(t * (1.0 / (double)a.K));
                s_inv[m] = 1.0f / sqrtf(mean + a.eps);
            }
            __syncthreads();
            const float inv = s_inv[m];
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                const int e = (tid + i * QT) * 4;
                if (e >= lo && e < hi)
                    *reinterpret_cast<float4*>(xs + m * kspan + (e - lo)) =
                        make_float4((xv[i].x * inv) * nwv[i].x, (xv[i].y * inv) * nwv[i].y, (xv[i].z * inv) * nwv[i].z, (xv[i].w * inv) * nwv[i].w);
            }
        }
    } else if (a.pro == PRO_RMSNORM) {
        // sum of squares in f64 over the whole row (emitter_quant.rs:713-791)
#pragma unroll
        for (int m = 0; m < M; ++m) {
            double s = 0.0;
            const float* xr = a.x + (size_t)m * a.ldx;
            for (int k = tid; k < a.K; k += QT) {
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
        for (int m = 0; m < M; ++m) {
            const float inv = s_inv[m];
            const float* xr = a.x + (size_t)m * a.ldx + kb0 * 32;
            for (int k = tid; k < nkb * 32; k += QT) xs[m * kspan + k] = (xr[k] * inv) * a.norm_w[kb0 * 32 + k];
        }
    } else {
        // the loads of all rows are issued before the first store (one L2 round trip per 1024 elements of a row)
        stage_rows<QT, M>(a.x + kb0 * 32, a.ldx, xs, kspan, nkb * 32, tid);
    }
    __syncthreads();
    HM_TRACE(if (tr) a.trace[7] = global_timer();)
    build_digit_image<M>(xs, kspan, nkb, img, bsc, csum, tid);
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
        for (int kb = warp; kb < nkb && ok; kb += 8) {
            const int ch = kb / ck;
            while (waited < ch && ok) {
                ++waited;
                ok = __all_sync(0xffffffffu, mb_wait(&s_wbar[waited], 0, a.err_flag, &s_abort));
                HM_TRACE(if (tr && waited == 0) a.trace[10] = global_timer();)  // first piece of the staged weights has landed
            }
            if (!ok) break;
            uint4 cc[2];
#pragma unroll
            for (int h = 0; h < CH; ++h) cc[h] = *reinterpret_cast<const uint4*>(codes_s + ((size_t)(kb * CH + h) * 32 + lane) * 16);
            q_block<NG, Q4>(cc, *reinterpret_cast<const uint2*>(scales_s + kb * 32 + (lane >> 2) * 4), img + (size_t)kb * NG * IMG_WORDS, bsc + kb * NG * 2, csum + kb * NG * 4, lane, acc);
        }
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
            if (kb < nkb) q_block<NG, Q4>(c[u], sc[u], img + (size_t)kb * NG * IMG_WORDS, bsc + kb * NG * 2, csum + kb * NG * 4, lane, acc);
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
    // the lane pair (q even, q odd) holds the two halves of a dot: planes 0,1 weigh 2^14, planes 2,3 weigh 1
    {
        const int q = lane & 3, g = lane >> 2;
        const float wgt = (q & 1) ? 1.0f : 16384.0f;
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
        // bias, half rotation (src/hf/emitter.rs:560-640; same operation order as the separate kernel of the K-quant plan) and the
        // KV-page write: a q or k tile holds 16 dimensions of a head's first half and, 16 rows further, their partners
        if (writer && tid < M * 32) red[tid] = v;
        __syncthreads();
        const int m = tid >> 5, p = tid & 31, n0 = tile * 32;
        if (writer && tid < M * 32 && m < a.m_valid && n0 < a.N) {
            const int pos = a.row_pos[m];
            const int seq = a.row_seq ? a.row_seq[m] : a.seq_base + m;
            const bool is_q = n0 < a.q_dim, is_k = !is_q && n0 < a.q_dim + a.kv_dim;
            const int part_off = is_q ? 0 : (is_k ? a.q_dim : a.q_dim + a.kv_dim);
            const int head = (n0 - part_off) / a.hd;
            int d;
            float val;
            if (is_q || is_k) {
                const int half = a.hd >> 1, hi = p >> 4;
                d = (((n0 - part_off) - head * a.hd) >> 5) * 16 + (p & 15) + hi * half;
                const int dp = hi ? d - half : d + half, base = part_off + head * a.hd;
                val = v;
                float oth = red[tid ^ 16];
                if (a.bias) {
                    val += a.bias[base + d];
                    oth += a.bias[base + dp];
                }
                oth = hi ? oth : -oth;
                val = fmaf(oth, a.rope_sin[(size_t)pos * a.hd + d], val * a.rope_cos[(size_t)pos * a.hd + d]);
            } else {
                d = (n0 - part_off) - head * a.hd + p;
                val = a.bias ? v + a.bias[n0 + p] : v;
            }
            if (is_q) {
                a.y[(size_t)m * a.ldy + head * a.hd + d] = val;
            } else {
                const int page = a.kv.page_table[(size_t)seq * a.kv.max_pages + pos / a.kv.page_tokens];
                const size_t off = ((size_t)page * a.kv.kv_heads + head) * a.kv.page_tokens * a.hd +
                                   (is_k ? k_tile_off(pos % a.kv.page_tokens, d) : v_tile_off(pos % a.kv.page_tokens, d, a.hd, a.kv.bf16));
                void* pool = is_k ? a.kv.k_pool : a.kv.v_pool;
                if (a.kv.bf16) reinterpret_cast<uint16_t*>(pool)[off] = f32_to_bf16_rne(val);
                else reinterpret_cast<float*>(pool)[off] = val;
            }
        }
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
cudaError_t launch_q3(const QuantArgs& a, cudaStream_t st, bool pdl) {
    constexpr int NG = (M + 1) / 2;
    size_t smem = sizeof(float) * ((size_t)M * a.kb_per_split * 32 + (size_t)a.kb_per_split * NG * (IMG_WORDS + 6) + 8 * M * 32 + (CL ? (size_t)a.ksplit * M * 32 : 0));
    const size_t slice = (size_t)a.kb_per_split * ((Q4 ? 1 : 2) * 512 + 64);
    const bool aligned = ((reinterpret_cast<uintptr_t>(a.codes) | reinterpret_cast<uintptr_t>(a.scales)) & 15) == 0;
#ifndef HM_QUANT_NO_STAGE
    if (aligned && slice <= QUANT_STAGE_MAX && smem + slice <= 110 * 1024) return launch_q4<M, Q4, CL, true>(a, smem + slice, st, pdl);
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
    if (a.q4) return a.ksplit > 1 ? launch_q3<M, true, true>(a, st, pdl) : launch_q3<M, true, false>(a, st, pdl);
    return a.ksplit > 1 ? launch_q3<M, false, true>(a, st, pdl) : launch_q3<M, false, false>(a, st, pdl);
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

}  // namespace hm
