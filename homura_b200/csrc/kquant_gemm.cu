// Q4_K projections over 9..64 activation rows (prefill chunks, batches of more than eight sequences) on the integer
// tensor-core path.  The reference's K-quant matmul is integer arithmetic by definition (Q8_K activation codes against
// the 4-bit weight codes, src/graph_builder/emit_quant.rs:165-816), so nothing is approximated: one launch quantises
// the rows to Q8_K once (the reference's operation order, (x * inv) * w, then emit_quant.rs:409-460), and the multiply
// feeds the codes to mma.sync.m16n8k32 (s8 x s8 -> s32) as they are: A = 16 output rows x the 32 weight codes of a
// sub-block, B = the 32 activation codes of 8 rows.  A warp owns 8 activation rows and walks every super-block of the
// CTA's K range; the 32-row tile's slot (header, 128 B of nibbles and the unpacked sub-block scales per row) is staged
// in shared memory once for all eight warps.  Per sub-block one more MMA with the sub-block's minimum replicated in A
// accumulates sum(min * code), so the per-(row, row) work outside the MMAs is four integer multiply-adds per sub-block
// and one float expression per super-block, the same expression as the 1..8-row kernel evaluates.
// Q6_K tiles (a Q4_K_M file keeps attn_v and ffn_down in Q6_K) have sixteen sub-blocks of 16 weights with signed 8-bit scales:
// their codes are put together from the low nibbles and the 2-bit planes, shifted to -32..31 per byte, and go through
// mma.sync.m16n8k16; no minima.
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"
#include "kquant.h"
#include "launch_attrs.h"
#include "mbarrier.cuh"

namespace hm {
namespace {

constexpr int KT = 256;
constexpr int GR = 64;                     // activation rows per launch
constexpr int Q4_STAGED = 10 * 512;        // pieces 0..9 of a slot: header, nibbles, unpacked scales / minima
constexpr int Q6_STAGED = KQ_SLOT_BYTES;   // the whole slot: 8 ql + 4 qh + 1 scale piece, then the rows' f16 super-block scales
constexpr int ROWB = 272;                  // a row's 256 codes in the ring, padded so that the eight rows of a B fragment hit 32 banks
constexpr int RING_STAGE = 8 * ROWB;       // a warp's eight rows of one super-block
constexpr int RING_STAGES = 2;

__device__ __forceinline__ void mma_s8_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_s8_acc(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
// four 6-bit codes (low nibbles | 2-bit plane << 4), each minus 32, as signed bytes
__device__ __forceinline__ uint32_t q6_codes(uint32_t lw, uint32_t hw, int group) {
    const uint32_t lo = (group >= 2 ? (lw >> 4) : lw) & 0x0F0F0F0Fu, hi = (hw >> (2 * group)) & 0x03030303u;
    const uint32_t c = lo | (hi << 4);                      // 0..63 per byte
    return ((c | 0x80808080u) - 0x20202020u) ^ 0x80808080u;  // per-byte c - 32 (no borrow crosses a byte)
}
__device__ __forceinline__ void cp_async16(void* dst_shared, const void* src_global) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(dst_shared)), "l"(src_global) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// rows -> Q8_K: codes [K/256][GR][256] int8, act_d [K/256][GR]; rows past M are written as zeros
__global__ void __launch_bounds__(KT) kquant_pack_rows_kernel(const float* __restrict__ x, int ldx, int M, int K, const float* __restrict__ norm_w, float eps, int8_t* __restrict__ codes, float* __restrict__ act_d) {
    __shared__ double s_w[8];
    __shared__ float s_inv;
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool row_ok = m < M;
    const float* xr = x + (size_t)m * ldx;
    const int nb = K / 256;
    float inv = 1.0f;
    if (norm_w) {
        double ssq = 0.0;
        if (row_ok)
            for (int p = tid; p < (K >> 2); p += KT) {
                const float4 v = ld_cg_f32x4(xr + 4 * (size_t)p);
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
    for (int kb = warp; kb < nb; kb += 8) {
        float v[8];
        if (row_ok) {
            const float4 x0 = ld_cg_f32x4(xr + (size_t)kb * 256 + lane * 8), x1 = ld_cg_f32x4(xr + (size_t)kb * 256 + lane * 8 + 4);
            const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            if (norm_w) {
                const float4 w0 = __ldg(reinterpret_cast<const float4*>(norm_w + (size_t)kb * 256 + lane * 8)), w1 = __ldg(reinterpret_cast<const float4*>(norm_w + (size_t)kb * 256 + lane * 8 + 4));
                const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = (xv[i] * inv) * wv[i];
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = xv[i];
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float iscale = amax == 0.f ? 0.f : __fdiv_rn(127.0f, amax);
        uint32_t packed[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float r = rintf(__fmul_rn(v[i], iscale));
            r = fminf(r, 127.0f);
            r = fmaxf(r, -127.0f);
            packed[i >> 2] |= ((uint32_t)((int)r & 0xFF)) << (8 * (i & 3));
        }
        *reinterpret_cast<uint2*>(codes + ((size_t)kb * GR + m) * 256 + lane * 8) = make_uint2(packed[0], packed[1]);
        if (lane == 0) act_d[(size_t)kb * GR + m] = __fdiv_rn(amax, 127.0f);
    }
}

template <bool CL>
__global__ void __launch_bounds__(KT) gemm_q4k_kernel(const KQuantArgs a) {
    extern __shared__ __align__(128) unsigned char ksm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int nb = a.K / 256;
    const int tile = blockIdx.x / a.ksplit, split = blockIdx.x - tile * a.ksplit;
    const int kb0 = split * a.kb_per_split, kb1 = min(nb, kb0 + a.kb_per_split);
    const int nkb = max(0, kb1 - kb0);
    const int ttype = a.tile_type[tile];                                               // 1 = Q4_K, 2 = Q6_K (0: no rows)
    const int staged = ttype == 2 ? Q6_STAGED : Q4_STAGED;                             // bytes of a slot this tile needs
    unsigned char* slice = ksm;                                                        // [kb_per_split][staged]
    // cluster: rank 0's receive slots [ksplit][GR][32] follow the ring, or (alias_slots: when that is what lets two CTAs share
    // an SM) take the place of the staged slots once every rank is done with its own, at the price of a cluster barrier
    const size_t slice_b = (size_t)a.kb_per_split * a.stage_bytes, slots_b = CL ? sizeof(float) * GR * 32 * (size_t)a.ksplit : (size_t)0;
    const bool alias = CL && a.alias_slots;
    float* vals = reinterpret_cast<float*>(ksm + (alias && slots_b > slice_b ? slots_b : slice_b));  // [GR][32]
    unsigned char* ring = reinterpret_cast<unsigned char*>(vals + GR * 32);            // [8 warps][RING_STAGES][RING_STAGE]
    float* slots = alias ? reinterpret_cast<float*>(ksm) : reinterpret_cast<float*>(ring + 8 * RING_STAGES * RING_STAGE);
    constexpr int NCHUNK = 4;
    __shared__ uint64_t s_wbar[NCHUNK];
    __shared__ volatile int s_abort;
    const unsigned char* tbase = a.data + ((size_t)tile * nb + kb0) * KQ_SLOT_BYTES;
    pdl_launch_dependents();
    // the tile's slots do not depend on the launch in front: staged before the dependency wait, in up to four pieces
    const int ck = max(1, (nkb + NCHUNK - 1) / NCHUNK);
    if (tid == 0) {
        for (int ch = 0; ch < NCHUNK; ++ch) mb_init(&s_wbar[ch], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int ch = 0; ch < NCHUNK; ++ch) {
            const int k_lo = min(nkb, ch * ck), k_hi = min(nkb, k_lo + ck);
            if (k_hi <= k_lo) break;
            mb_expect_tx(&s_wbar[ch], (uint32_t)(k_hi - k_lo) * staged);
            for (int kbl = k_lo; kbl < k_hi; ++kbl) bulk_copy(slice + (size_t)kbl * staged, tbase + (size_t)kbl * KQ_SLOT_BYTES, staged, &s_wbar[ch]);
        }
    }
    pdl_wait();
    __syncthreads();

    // this warp's eight activation rows: 2 KB of codes per super-block through a two-stage ring of asynchronous copies
    const int8_t* cw = a.codes_in + ((size_t)kb0 * GR + 8 * warp) * 256;
    const float* adw = a.actd_in + (size_t)kb0 * GR + 8 * warp + 2 * q;
    unsigned char* myring = ring + (size_t)warp * RING_STAGES * RING_STAGE;
    auto issue = [&](int kbl) {
        if (kbl < nkb) {
            const int8_t* src = cw + (size_t)kbl * GR * 256;
            unsigned char* dst = myring + (kbl % RING_STAGES) * RING_STAGE;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int seg = lane + 32 * i;  // 128 segments of 16 B: row = seg / 16, piece = seg % 16
                cp_async16(dst + (seg >> 4) * ROWB + (seg & 15) * 16, src + seg * 16);
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s0 = 0; s0 < RING_STAGES; ++s0) issue(s0);
    float acc[2][2][2];  // [row group][row g / g + 8][activation row 2q / 2q + 1]
#pragma unroll
    for (int i = 0; i < 8; ++i) (&acc[0][0][0])[i] = 0.f;
    int waited = -1;
    bool ok = true;
    for (int kbl = 0; kbl < nkb && ok; ++kbl) {
        const float ad0 = __ldg(adw + (size_t)kbl * GR), ad1 = __ldg(adw + (size_t)kbl * GR + 1);
        cp_async_wait<RING_STAGES - 1>();
        __syncwarp();
        while (kbl >= (waited + 1) * ck && ok) {
            ++waited;
            ok = __all_sync(0xffffffffu, mb_wait(&s_wbar[waited], 0, a.err_flag, &s_abort));
        }
        if (!ok) break;
        const unsigned char* slot = slice + (size_t)kbl * staged;
        const unsigned char* brow = myring + (kbl % RING_STAGES) * RING_STAGE + g * ROWB + 4 * q;
        if (ttype == 2) {
#pragma unroll
            for (int rg = 0; rg < 2; ++rg) {
                const int rA = 16 * rg + g, rB = rA + 8;
                const uint4 scA = *reinterpret_cast<const uint4*>(slot + (12 * 32 + rA) * 16), scB = *reinterpret_cast<const uint4*>(slot + (12 * 32 + rB) * 16);
                const uint32_t sAw[4] = {scA.x, scA.y, scA.z, scA.w}, sBw[4] = {scB.x, scB.y, scB.z, scB.w};
                int sacc[2][2] = {{0, 0}, {0, 0}};
#pragma unroll
                for (int sb = 0; sb < 16; ++sb) {
                    const int chunk = sb >> 3, group = (sb & 7) >> 1, parity = sb & 1;
                    const int pl = chunk * 4 + (group & 1) * 2 + parity, ph = 8 + chunk * 2 + parity;
                    const uint32_t a0 = q6_codes(*reinterpret_cast<const uint32_t*>(slot + (pl * 32 + rA) * 16 + 4 * q), *reinterpret_cast<const uint32_t*>(slot + (ph * 32 + rA) * 16 + 4 * q), group);
                    const uint32_t a1 = q6_codes(*reinterpret_cast<const uint32_t*>(slot + (pl * 32 + rB) * 16 + 4 * q), *reinterpret_cast<const uint32_t*>(slot + (ph * 32 + rB) * 16 + 4 * q), group);
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + sb * 16);
                    int cc[4];
                    mma_s8_k16(cc, a0, a1, b0);
                    const int sA = (int)(int8_t)(sAw[sb >> 2] >> (8 * (sb & 3))), sB = (int)(int8_t)(sBw[sb >> 2] >> (8 * (sb & 3)));
                    sacc[0][0] += sA * cc[0];
                    sacc[0][1] += sA * cc[1];
                    sacc[1][0] += sB * cc[2];
                    sacc[1][1] += sB * cc[3];
                }
                const float dA = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(slot + 13 * 512 + rA * 2)));
                const float dB = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(slot + 13 * 512 + rB * 2)));
                acc[rg][0][0] = __fadd_rn(acc[rg][0][0], __fmul_rn(__fmul_rn(dA, ad0), (float)sacc[0][0]));
                acc[rg][0][1] = __fadd_rn(acc[rg][0][1], __fmul_rn(__fmul_rn(dA, ad1), (float)sacc[0][1]));
                acc[rg][1][0] = __fadd_rn(acc[rg][1][0], __fmul_rn(__fmul_rn(dB, ad0), (float)sacc[1][0]));
                acc[rg][1][1] = __fadd_rn(acc[rg][1][1], __fmul_rn(__fmul_rn(dB, ad1), (float)sacc[1][1]));
            }
        } else
#pragma unroll
        for (int rg = 0; rg < 2; ++rg) {
            const int rA = 16 * rg + g, rB = rA + 8;
            const uint32_t hA = *reinterpret_cast<const uint32_t*>(slot + rA * 16), hB = *reinterpret_cast<const uint32_t*>(slot + rB * 16);
            const uint4 sA = *reinterpret_cast<const uint4*>(slot + 9 * 512 + rA * 16), sB = *reinterpret_cast<const uint4*>(slot + 9 * 512 + rB * 16);
            int sacc[2][2] = {{0, 0}, {0, 0}};
            int cmin[4] = {0, 0, 0, 0};
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const uint32_t w00 = *reinterpret_cast<const uint32_t*>(slot + ((1 + 2 * p) * 32 + rA) * 16 + 4 * q);
                const uint32_t w01 = *reinterpret_cast<const uint32_t*>(slot + ((1 + 2 * p) * 32 + rB) * 16 + 4 * q);
                const uint32_t w10 = *reinterpret_cast<const uint32_t*>(slot + ((2 + 2 * p) * 32 + rA) * 16 + 4 * q);
                const uint32_t w11 = *reinterpret_cast<const uint32_t*>(slot + ((2 + 2 * p) * 32 + rB) * 16 + 4 * q);
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {
                    const int s = 2 * p + hi;  // sub-block: low nibbles of the pair's 32 bytes, then high nibbles
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + s * 32), b1 = *reinterpret_cast<const uint32_t*>(brow + s * 32 + 16);
                    const uint32_t a0 = (hi ? (w00 >> 4) : w00) & 0x0F0F0F0Fu, a1 = (hi ? (w01 >> 4) : w01) & 0x0F0F0F0Fu;
                    const uint32_t a2 = (hi ? (w10 >> 4) : w10) & 0x0F0F0F0Fu, a3 = (hi ? (w11 >> 4) : w11) & 0x0F0F0F0Fu;
                    int cc[4];
                    mma_s8_zero(cc, a0, a1, a2, a3, b0, b1);
                    const int scA = (int)(((s < 4 ? sA.x : sA.y) >> (8 * (s & 3))) & 0xFFu), scB = (int)(((s < 4 ? sB.x : sB.y) >> (8 * (s & 3))) & 0xFFu);
                    sacc[0][0] += scA * cc[0];
                    sacc[0][1] += scA * cc[1];
                    sacc[1][0] += scB * cc[2];
                    sacc[1][1] += scB * cc[3];
                    const uint32_t mA = (((s < 4 ? sA.z : sA.w) >> (8 * (s & 3))) & 0xFFu) * 0x01010101u, mB = (((s < 4 ? sB.z : sB.w) >> (8 * (s & 3))) & 0xFFu) * 0x01010101u;
                    mma_s8_acc(cmin, mA, mB, mA, mB, b0, b1);
                }
            }
            const float dA = __half2float(__ushort_as_half((unsigned short)(hA & 0xFFFFu))), mnA = __half2float(__ushort_as_half((unsigned short)(hA >> 16)));
            const float dB = __half2float(__ushort_as_half((unsigned short)(hB & 0xFFFFu))), mnB = __half2float(__ushort_as_half((unsigned short)(hB >> 16)));
            // the 1..8-row kernel's expression, per super-block
            acc[rg][0][0] = __fadd_rn(acc[rg][0][0], __fsub_rn(__fmul_rn(__fmul_rn(dA, ad0), (float)sacc[0][0]), __fmul_rn(__fmul_rn(mnA, ad0), (float)cmin[0])));
            acc[rg][0][1] = __fadd_rn(acc[rg][0][1], __fsub_rn(__fmul_rn(__fmul_rn(dA, ad1), (float)sacc[0][1]), __fmul_rn(__fmul_rn(mnA, ad1), (float)cmin[1])));
            acc[rg][1][0] = __fadd_rn(acc[rg][1][0], __fsub_rn(__fmul_rn(__fmul_rn(dB, ad0), (float)sacc[1][0]), __fmul_rn(__fmul_rn(mnB, ad0), (float)cmin[2])));
            acc[rg][1][1] = __fadd_rn(acc[rg][1][1], __fsub_rn(__fmul_rn(__fmul_rn(dB, ad1), (float)sacc[1][1]), __fmul_rn(__fmul_rn(mnB, ad1), (float)cmin[3])));
        }
        __syncwarp();
        issue(kbl + RING_STAGES);
    }
#pragma unroll
    for (int rg = 0; rg < 2; ++rg)
#pragma unroll
        for (int rs = 0; rs < 2; ++rs)
#pragma unroll
            for (int c = 0; c < 2; ++c) vals[(8 * warp + 2 * q + c) * 32 + 16 * rg + 8 * rs + g] = acc[rg][rs][c];
    __syncthreads();
    if (CL) {
        if (alias) cluster_sync_all();  // nobody reads staged slots any more: the receive slots may overwrite them
        for (int t = tid; t < GR * 32; t += KT) {
            if (split == 0) slots[t] = vals[t];
            else st_dsmem_f32(dsmem_addr(slots + (size_t)split * (GR * 32) + t, 0u), vals[t]);
        }
        cluster_arrive_release();
        if (split != 0) return;
        cluster_wait_acquire();
        for (int t = tid; t < GR * 32; t += KT) {
            float v = slots[t];
            for (int r = 1; r < a.ksplit; ++r) v += slots[(size_t)r * (GR * 32) + t];
            vals[t] = v;
        }
        __syncthreads();
    }
    for (int t = tid; t < GR * 32; t += KT) {
        const int m = t >> 5, p = t & 31;
        float v = vals[t];
        if (a.epi == EPI_SWIGLU) {
            const int j = tile * 16 + p;
            if (p < 16 && m < a.m_valid && j < a.N / 2) {
                const float gt = v, u = vals[t + 16];
                a.y[(size_t)m * a.ldy + j] = (gt / (1.0f + expf(-gt))) * u;
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

template <bool CL>
cudaError_t launch_gk(const KQuantArgs& a, size_t smem, cudaStream_t st, bool pdl) {
    cudaError_t e = ensure_dyn_smem(gemm_q4k_kernel<CL>, smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(((a.N + 31) / 32) * a.ksplit));
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
    return cudaLaunchKernelEx(&cfg, gemm_q4k_kernel<CL>, a);
}

}  // namespace

size_t kquant_rows_code_bytes(int K) { return (size_t)(K / 256) * GR * 256; }
size_t kquant_rows_scale_floats(int K) { return (size_t)(K / 256) * GR; }
bool kquant_rows_supported(const KQuantArgs& a) {
    return (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (a.ldx & 3) == 0 && (a.K & 255) == 0 && (!a.norm_w || (reinterpret_cast<uintptr_t>(a.norm_w) & 15) == 0) &&
           (reinterpret_cast<uintptr_t>(a.data) & 15) == 0;
}

cudaError_t launch_gemm_q4k(const KQuantArgs& a_in, int8_t* codes, float* act_d, int sm_count, cudaStream_t st, bool pdl, int* launches) {
    KQuantArgs a = a_in;
    if (a.m_valid < 1 || a.m_valid > GR || !kquant_rows_supported(a)) return cudaErrorInvalidValue;
    cudaError_t e;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(GR);
        cfg.blockDim = dim3(KT);
        cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = pdl ? 1 : 0;
        e = cudaLaunchKernelEx(&cfg, kquant_pack_rows_kernel, a.x, a.ldx, a.m_valid, a.K, a.pro == PRO_RMSNORM ? a.norm_w : (const float*)nullptr, a.eps, codes, act_d);
    }
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
    a.codes_in = codes;
    a.actd_in = act_d;
    const int nb = a.K / 256, tiles = (a.N + 31) / 32;
    // K split: about one CTA per SM, at most 8 per cluster, a staged slice of at most 96 KB
    int ks = (sm_count + tiles - 1) / tiles;
    ks = std::min(ks, std::min(8, nb));
    a.stage_bytes = a.has_q6 ? Q6_STAGED : Q4_STAGED;
    while (ks < 8 && ks < nb && (size_t)((nb + ks - 1) / ks) * a.stage_bytes > 96 * 1024) ++ks;
    ks = std::max(ks, 1);
    a.kb_per_split = (nb + ks - 1) / ks;
    a.ksplit = (nb + a.kb_per_split - 1) / a.kb_per_split;
    if ((size_t)a.kb_per_split * a.stage_bytes > 128 * 1024) return cudaErrorInvalidValue;
    const size_t slice_b = (size_t)a.kb_per_split * a.stage_bytes, slots_b = a.ksplit > 1 ? sizeof(float) * GR * 32 * (size_t)a.ksplit : (size_t)0;
    const size_t rest_b = sizeof(float) * GR * 32 + (size_t)8 * RING_STAGES * RING_STAGE;
    size_t smem = slice_b + slots_b + rest_b;
    const size_t two_per_sm = 112 * 1024;  // 2 x (this + 1 KB) fits the SM's 227 KB
    if (slots_b && smem > two_per_sm && std::max(slice_b, slots_b) + rest_b <= two_per_sm) {
        a.alias_slots = 1;
        smem = std::max(slice_b, slots_b) + rest_b;
    }
    e = a.ksplit > 1 ? launch_gk<true>(a, smem, st, pdl) : launch_gk<false>(a, smem, st, pdl);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace hm
