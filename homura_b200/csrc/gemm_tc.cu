// Skinny tensor-core GEMM for 9..64 activation rows: y[M,N] = x[M,K] @ W with bf16 weights, f32
// activations and f32 accumulation -- Homura's mixed matmul (src/graph_builder/emit_linalg.rs:
// 1928-2008, 2224-2307) where the contraction is dense enough for the 5th-generation tensor cores
// (batched decode, prefill chunks).
//
// Shape of the problem on a B200: the weights are streamed once from HBM (still the bound:
// 64 rows give 64 flop/B against a ridge of ~210), so the kernel is built like the streaming
// GEMV, with tcgen05 doing the math:
//   * "swap AB": the 128 output features of a CTA are the MMA's M, the <= 64 activation rows are
//     its N, so one tcgen05.mma (M=128, N=64*T, K=16) consumes a 128x16 weight tile.
//   * weights live in HBM as the exact shared-memory image of their tiles: [n-block][k-block]
//     [128 rows][64 k] bf16, K-major, with the 128-byte swizzle already applied, so one 16 KB
//     cp.async.bulk per stage lands them where the UMMA descriptor expects (no tensor map, no
//     multicast).
//   * activations stay f32 in the model (the reference multiplies f32 x bf16).  To keep that
//     precision on bf16 tensor cores each activation is split into T = 3 bf16 terms
//     (x = hi + mid + lo exactly to 2^-24 relative), stacked along the MMA's N; the epilogue adds
//     the three 64-column groups of the accumulator.  The tensor pipe has the headroom.
//   * accumulator in TMEM (128 lanes x 256 columns), read back with tcgen05.ld by four warps.
//   * K can be split across the CTAs of a thread-block cluster; the split accumulators are
//     reduce-scattered by activation row through distributed shared memory, so every CTA ends up
//     with complete 128-column rows for its share of the rows and runs the epilogue on them.
// Roles: warp 0 = bulk-copy producer, warp 1 = TMEM owner + MMA issuer, warps 2-5 = activation
// staging (f32 -> 3 x bf16, swizzled) and epilogue.  Every mbarrier wait is bounded.
#include <cstdlib>

#include "common.cuh"
#include "gemm_tc.h"
#include "launch_attrs.h"
#include "mbarrier.cuh"

namespace hm {
namespace {

constexpr int TC_THREADS = 192;
constexpr int BM = 128;  // output features per CTA (MMA M)
constexpr int BK = 64;   // k per stage (128 B of bf16)
constexpr int MR = 64;   // activation rows (MMA N = MR * terms)
constexpr int TERMS = 3;
constexpr int W_TILE = BM * BK * 2;          // 16 KB
constexpr int NSTG = 8;  // barrier slots; stages in use depend on the row padding

// Shared-memory matrix descriptor, K-major operand with 128-byte swizzle: rows of 128 B, groups of
// 8 rows 1024 B apart (stride byte offset), descriptor version 1, layout type SWIZZLE_128B (2).
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);  // start address
    d |= (uint64_t)1 << 16;                      // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset
    d |= (uint64_t)1 << 46;                      // version
    d |= (uint64_t)2 << 61;                      // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D f32, A/B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}

struct TcShared {
    uint64_t full[NSTG], empty[NSTG], acc_full;
    uint64_t rbar;  // split-K: counts the bytes of the other ranks' partial rows arriving in this CTA's receive slots
    uint32_t tmem_base;
    volatile int abort_flag;
    float inv[MR];  // per activation row: the RMSNorm factor applied to the accumulators (ss_in given)
    int pos[MR], page[MR];  // QKV epilogue: position and KV page of every row's token, fetched while the MMAs run
};

// ---- activation packing: f32 rows -> three bf16 terms in the shared-memory image of the B tiles ----
// out: [k-block][term][mpad][64] bf16, rows of 128 B, 16-byte chunks XOR-swizzled by (row & 7) where
// row = term * mpad + m.  One block per padded row; an RMSNorm is folded in when norm_w is given
// (x' = (x * inv_rms) * w, src/graph_builder/emit_linalg.rs:7-26).
__global__ void __launch_bounds__(256) tc_pack_x_kernel(const float* __restrict__ x, int ldx, int M, int mpad, int K, int Kp, const float* __restrict__ norm_w, float eps, unsigned char* __restrict__ out, unsigned long long* trace) {
    HM_TRACE(const bool tr = trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0;)
    HM_TRACE(if (tr) trace[0] = global_timer();)
    pdl_launch_dependents();
    pdl_wait();
    HM_TRACE(if (tr) trace[2] = global_timer();)
    const int m = blockIdx.x, tid = threadIdx.x;
    const bool row_ok = m < M;
    const float* xr = x + (size_t)m * ldx;
    __shared__ float sw[8];
    __shared__ float s_inv;
    float inv = 1.0f;
    if (norm_w) {
        float s = 0.f;
        if (row_ok)
            for (int i = tid; i < K; i += 256) s = fmaf(xr[i], xr[i], s);
        s = warp_sum(s);
        if ((tid & 31) == 0) sw[tid >> 5] = s;
        __syncthreads();
        if (tid == 0) {
            float t = 0.f;
            for (int i = 0; i < 8; ++i) t += sw[i];
            s_inv = 1.0f / sqrtf(t / (float)K + eps);
        }
        __syncthreads();
        inv = s_inv;
    }
    const size_t tile_bytes = (size_t)TERMS * mpad * 128;
    for (int c = tid; c < Kp / 8; c += 256) {  // one 16-byte chunk (8 k) per term per iteration
        const int k0 = c * 8, kb = k0 / BK, chunk = (k0 % BK) >> 3;
        uint32_t term[TERMS][4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            uint16_t h[2], md[2], l[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int k = k0 + 2 * e + u;
                float v = (row_ok && k < K) ? xr[k] : 0.f;
                if (norm_w && k < K) v = (v * inv) * __ldg(norm_w + k);
                h[u] = f32_to_bf16_rne(v);
                const float r1 = v - bf16_bits_to_f32(h[u]);
                md[u] = f32_to_bf16_rne(r1);
                l[u] = f32_to_bf16_rne(r1 - bf16_bits_to_f32(md[u]));
            }
            term[0][e] = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
            term[1][e] = (uint32_t)md[0] | ((uint32_t)md[1] << 16);
            term[2][e] = (uint32_t)l[0] | ((uint32_t)l[1] << 16);
        }
#pragma unroll
        for (int t = 0; t < TERMS; ++t) {
            const int row = t * mpad + m;
            const size_t off = (size_t)kb * tile_bytes + (size_t)row * 128 + (size_t)((chunk ^ (row & 7)) << 4);
            *reinterpret_cast<uint4*>(out + off) = make_uint4(term[t][0], term[t][1], term[t][2], term[t][3]);
        }
    }
    HM_TRACE(if (trace && threadIdx.x == 0) atomicMax(trace + 12, global_timer());)
}

// ---- epilogues on rows [m_lo, m_hi) of the f32 tile [m][128] (output features n0 .. n0+127) ----
// The same four epilogues as the streaming projection kernel (gemv_bf16.cu), for up to 64 rows.
__device__ __forceinline__ bool tc_better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i > bi); }

__device__ void tc_epilogue(const TcArgs& a, float* tile, int m_lo, int m_hi, int nblk, int tid, const int* s_pos, const int* s_page) {
    const int n0 = nblk * BM, rows = m_hi - m_lo;
    const int lane = tid & 31, warp = tid >> 5;
    constexpr int NW = TC_THREADS / 32;
    if (a.epi == EPI_STORE) {
        const bool vec = (a.ldy & 3) == 0 && ((reinterpret_cast<uintptr_t>(a.y) | reinterpret_cast<uintptr_t>(a.resid) | reinterpret_cast<uintptr_t>(a.bias)) & 15) == 0 && n0 + BM <= a.N;
        if (vec) {
            // eight consecutive features per thread (one 16-byte chunk of the next GEMM's activation image); the 16
            // threads of a row are half a warp, which is where the row's sum of squares is reduced
            const int items = rows * (BM / 8);
            for (int base = 0; base < items; base += TC_THREADS) {
                const int idx = base + tid;
                const bool ok = idx < items;
                const int m = m_lo + (ok ? idx : 0) / (BM / 8), c = ((ok ? idx : 0) % (BM / 8)) * 8;
                float v[8];
                {
                    const float4 t0 = *reinterpret_cast<const float4*>(tile + m * BM + c), t1 = *reinterpret_cast<const float4*>(tile + m * BM + c + 4);
                    v[0] = t0.x; v[1] = t0.y; v[2] = t0.z; v[3] = t0.w; v[4] = t1.x; v[5] = t1.y; v[6] = t1.z; v[7] = t1.w;
                }
                if (ok && a.resid) {
                    const float4 r0 = ld_cg_f32x4(a.resid + (size_t)m * a.ldy + n0 + c), r1 = ld_cg_f32x4(a.resid + (size_t)m * a.ldy + n0 + c + 4);
                    float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
                    if (a.bias) { b0 = __ldg(reinterpret_cast<const float4*>(a.bias + n0 + c)); b1 = __ldg(reinterpret_cast<const float4*>(a.bias + n0 + c + 4)); }
                    v[0] = r0.x + (v[0] + b0.x); v[1] = r0.y + (v[1] + b0.y); v[2] = r0.z + (v[2] + b0.z); v[3] = r0.w + (v[3] + b0.w);
                    v[4] = r1.x + (v[4] + b1.x); v[5] = r1.y + (v[5] + b1.y); v[6] = r1.z + (v[6] + b1.z); v[7] = r1.w + (v[7] + b1.w);
                } else if (ok && a.bias) {
                    const float4 b0 = __ldg(reinterpret_cast<const float4*>(a.bias + n0 + c)), b1 = __ldg(reinterpret_cast<const float4*>(a.bias + n0 + c + 4));
                    v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w; v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
                }
                if (ok) {
                    *reinterpret_cast<float4*>(a.y + (size_t)m * a.ldy + n0 + c) = make_float4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<float4*>(a.y + (size_t)m * a.ldy + n0 + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
                }
                if (a.xp_next) {
                    float ss = 0.f;
                    if (ok) {
                        const float4 w0 = __ldg(reinterpret_cast<const float4*>(a.next_norm_w + n0 + c)), w1 = __ldg(reinterpret_cast<const float4*>(a.next_norm_w + n0 + c + 4));
#pragma unroll
                        for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
                        const float xs[8] = {v[0] * w0.x, v[1] * w0.y, v[2] * w0.z, v[3] * w0.w, v[4] * w1.x, v[5] * w1.y, v[6] * w1.z, v[7] * w1.w};
                        tc_xpack_store8(a.xp_next, a.xp_mpad, m, n0 + c, xs);
                    }
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (ok && (idx & 15) == 0) a.ss_out[nblk * MR + m] = ss;
                }
            }
        } else {
            for (int idx = tid; idx < rows * BM; idx += TC_THREADS) {
                const int m = m_lo + idx / BM, c = idx % BM, n = n0 + c;
                if (n < a.N) {
                    float v = tile[m * BM + c];
                    if (a.bias) v += __ldg(a.bias + n);
                    if (a.resid) v = a.resid[(size_t)m * a.ldy + n] + v;
                    a.y[(size_t)m * a.ldy + n] = v;
                }
            }
        }
    } else if (a.epi == EPI_SWIGLU) {
        // block = 64 gate features followed by the 64 matching up features (src/hf/emitter.rs SwiGLU)
        if (a.xp_out && nblk * 64 + 64 <= a.N / 2) {
            // eight consecutive outputs per thread, written as one 16-byte chunk per bf16 term of the next GEMM's activation image
            for (int idx = tid; idx < rows * 8; idx += TC_THREADS) {
                const int m = m_lo + idx / 8, c = (idx % 8) * 8;
                float act[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float g = tile[m * BM + c + e], u = tile[m * BM + 64 + c + e];
                    act[e] = (g / (1.0f + expf(-g))) * u;
                }
                tc_xpack_store8(a.xp_out, a.xp_mpad, m, nblk * 64 + c, act);
            }
        } else {
            for (int idx = tid; idx < rows * 64; idx += TC_THREADS) {
                const int m = m_lo + idx / 64, c = idx % 64, j = nblk * 64 + c;
                if (j < a.N / 2) {
                    const float g = tile[m * BM + c], u = tile[m * BM + 64 + c];
                    const float act = (g / (1.0f + expf(-g))) * u;
                    if (a.xp_out) tc_xpack_store(a.xp_out, a.xp_mpad, m, j, act);
                    else a.y[(size_t)m * a.ldy + j] = act;
                }
            }
        }
    } else if (a.epi == EPI_LOGITS) {
        for (int idx = tid; idx < rows * BM; idx += TC_THREADS) {
            const int m = m_lo + idx / BM, c = idx % BM, n = n0 + c;
            if (n < a.N) a.y[(size_t)m * a.ldy + n] = tile[m * BM + c];
        }
        const int nblocks = (a.N + BM - 1) / BM;
        for (int m = m_lo + warp; m < m_hi; m += NW) {  // per-row argmax of this block, ties to the higher index
            float bv = -INFINITY;
            int bi = -1;
#pragma unroll
            for (int i = 0; i < BM / 32; ++i) {
                const int c = lane + i * 32, n = n0 + c;
                if (n < a.N) {
                    const float v = tile[m * BM + c];
                    if (bi < 0 || tc_better(v, n, bv, bi)) { bv = v; bi = n; }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi >= 0 && (bi < 0 || tc_better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
            }
            if (lane == 0) {
                a.amax_val[(size_t)m * nblocks + nblk] = bv;
                a.amax_idx[(size_t)m * nblocks + nblk] = bi;
            }
        }
    } else {  // EPI_QKV_ROPE: bias, per-head QK RMSNorm, RoPE half rotation, K/V page write (src/hf/emitter.rs:604-649)
        const int hd = a.hd, half = hd >> 1, hps = BM / hd;
        if (a.bias) {
            for (int idx = tid; idx < rows * BM; idx += TC_THREADS) {
                const int m = m_lo + idx / BM, c = idx % BM;
                if (n0 + c < a.N) tile[m * BM + c] += __ldg(a.bias + n0 + c);
            }
            __syncthreads();
        }
        if (a.has_qk_norm) {
            for (int p = warp; p < rows * hps; p += NW) {
                const int m = m_lo + p / hps, hh = p % hps;
                const int nh = n0 + hh * hd;
                if (nh >= a.q_dim + a.kv_dim || nh >= a.N) continue;  // V heads are not normalised
                float* v = tile + m * BM + hh * hd;
                float s = 0.f;
                for (int d = lane; d < hd; d += 32) s = fmaf(v[d], v[d], s);
                s = warp_sum(s);
                const float inv = 1.0f / sqrtf(s / (float)hd + a.eps);
                const float* nw = (nh < a.q_dim) ? a.q_norm_w : a.k_norm_w;
                for (int d = lane; d < hd; d += 32) v[d] = (v[d] * inv) * __ldg(nw + d);
            }
            __syncthreads();
        }
        // Rotation and stores, four dims of the first half of a head and their partners in the second half per
        // thread: one 16-byte read of the cos and sin rows serves both (the two halves of a row are equal,
        // src/hf/precompute.rs:10-40), and Q / K / V leave as 16-byte (f32) or 8-byte (bf16 page) stores.  The
        // K tile is chunk-major, so four consecutive dims of one token are contiguous there as well.
        const int ipr = BM / 8, iph = hd / 8;
        for (int idx = tid; idx < rows * ipr; idx += TC_THREADS) {
            const int m = m_lo + idx / ipr, it = idx % ipr;
            const int hh = it / iph, d0 = (it % iph) * 4;
            const int nh = n0 + hh * hd;
            if (nh >= a.N) continue;
            const float4 lo = *reinterpret_cast<const float4*>(tile + m * BM + hh * hd + d0);
            const float4 hi = *reinterpret_cast<const float4*>(tile + m * BM + hh * hd + half + d0);
            float4 olo = lo, ohi = hi;
            const int pos = s_pos[m];
            if (nh < a.q_dim + a.kv_dim) {
                const float4 cs = __ldg(reinterpret_cast<const float4*>(a.rope_cos + (size_t)pos * hd + d0));
                const float4 sn = __ldg(reinterpret_cast<const float4*>(a.rope_sin + (size_t)pos * hd + d0));
                olo = make_float4(fmaf(-hi.x, sn.x, lo.x * cs.x), fmaf(-hi.y, sn.y, lo.y * cs.y), fmaf(-hi.z, sn.z, lo.z * cs.z), fmaf(-hi.w, sn.w, lo.w * cs.w));
                ohi = make_float4(fmaf(lo.x, sn.x, hi.x * cs.x), fmaf(lo.y, sn.y, hi.y * cs.y), fmaf(lo.z, sn.z, hi.z * cs.z), fmaf(lo.w, sn.w, hi.w * cs.w));
            }
            if (nh < a.q_dim) {
                float* q = a.y + (size_t)m * a.ldy + nh;
                *reinterpret_cast<float4*>(q + d0) = olo;
                *reinterpret_cast<float4*>(q + half + d0) = ohi;
            } else {
                const bool is_k = nh < a.q_dim + a.kv_dim;
                const int kvh = (nh - a.q_dim - (is_k ? 0 : a.kv_dim)) / hd;
                const int tok = pos % a.kv.page_tokens;
                const size_t base = ((size_t)s_page[m] * a.kv.kv_heads + kvh) * a.kv.page_tokens * hd;
                const size_t o0 = base + (is_k ? k_tile_off(tok, d0) : v_tile_off(tok, d0, hd, a.kv.bf16));
                const size_t o1 = base + (is_k ? k_tile_off(tok, half + d0) : v_tile_off(tok, half + d0, hd, a.kv.bf16));
                void* pool = is_k ? a.kv.k_pool : a.kv.v_pool;
                if (a.kv.bf16) {
                    uint16_t* pp = reinterpret_cast<uint16_t*>(pool);
                    *reinterpret_cast<uint2*>(pp + o0) = make_uint2((uint32_t)f32_to_bf16_rne(olo.x) | ((uint32_t)f32_to_bf16_rne(olo.y) << 16), (uint32_t)f32_to_bf16_rne(olo.z) | ((uint32_t)f32_to_bf16_rne(olo.w) << 16));
                    *reinterpret_cast<uint2*>(pp + o1) = make_uint2((uint32_t)f32_to_bf16_rne(ohi.x) | ((uint32_t)f32_to_bf16_rne(ohi.y) << 16), (uint32_t)f32_to_bf16_rne(ohi.z) | ((uint32_t)f32_to_bf16_rne(ohi.w) << 16));
                } else {
                    float* pp = reinterpret_cast<float*>(pool);
                    *reinterpret_cast<float4*>(pp + o0) = olo;
                    *reinterpret_cast<float4*>(pp + o1) = ohi;
                }
            }
        }
    }
}

// ---- the GEMM: warp 0 = bulk-copy producer, warp 1 = TMEM owner + MMA issuer, warps 2-5 = epilogue ----
template <bool CL>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const TcArgs a) {
    extern __shared__ __align__(1024) unsigned char dsm[];
    __shared__ TcShared sh;
    unsigned char* stage0 = dsm + ((1024u - (s32(dsm) & 1023u)) & 1023u);  // swizzle atoms need 1024-byte alignment
    const int mpad = a.mpad;
    const uint32_t x_tile = (uint32_t)(TERMS * mpad * 128);
    const uint32_t stage_bytes = W_TILE + x_tile;  // multiple of 1024 for mpad in {16, 32, 64}
    // [mpad][BM] f32, written only after the last MMA has completed: it reuses the first stage of the ring (by then
    // every bulk copy has landed and every operand has been read), which keeps the CTA's footprint to the ring alone
    float* out_tile = reinterpret_cast<float*>(stage0);
    // split-K: receive slots [rank][this CTA's rows][BM] behind the ring (peers write here while this CTA's ring is
    // still in use, so they cannot share its memory)
    float* recv = reinterpret_cast<float*>(stage0 + (size_t)a.nstage * stage_bytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cs = CL ? a.ksplit : 1;
    const int nblk = blockIdx.x / cs;
    const int split = blockIdx.x - nblk * cs;
    const int kb_total = a.Kp / BK;
    const int kb_per = (kb_total + cs - 1) / cs;
    const int kb0 = split * kb_per, kb1 = min(kb_total, kb0 + kb_per);
    const int nkb = max(0, kb1 - kb0);
    const int nst = a.nstage;
    HM_TRACE(const bool tr = a.trace != nullptr && blockIdx.x == 0;)
    HM_TRACE(if (tr && tid == 0) a.trace[0] = global_timer();)
    HM_TRACE(if (a.trace && tid == 0) atomicMax(a.trace + 11, global_timer());)

    if (tid == 0) {
        for (int s = 0; s < nst; ++s) {
            mb_init(&sh.full[s], 1);
            mb_init(&sh.empty[s], 1);
        }
        mb_init(&sh.acc_full, 1);
        sh.abort_flag = 0;
        if (CL) {
            // the other ranks push their partial sums of this CTA's rows with asynchronous stores that count bytes
            // on this barrier: armed now, published by the cluster barrier below (both before the dependency wait)
            mb_init(&sh.rbar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            const int rows_per0 = (a.M + cs - 1) / cs;
            const int lo0 = min(a.M, split * rows_per0), hi0 = min(a.M, lo0 + rows_per0);
            mb_expect_tx(&sh.rbar, (uint32_t)(cs - 1) * (uint32_t)(hi0 - lo0) * (uint32_t)(BM * 4));
        } else {
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    if (CL) cluster_sync_all(); else
    __syncthreads();
    if (warp == 1) {  // TMEM: allocated and later freed by this warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&sh.tmem_base)), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sh.tmem_base;
    HM_TRACE(if (tr && tid == 0) a.trace[1] = global_timer();)

    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(a.W) + ((size_t)nblk * kb_total + kb0) * W_TILE;
            const unsigned char* xsrc = a.xp + (size_t)kb0 * x_tile;
            // weights never depend on the previous kernel: fill the ring with them first, then wait for
            // the packed activations
            const int pre = min(nkb, nst);
            for (int i = 0; i < pre; ++i) {
                mb_expect_tx(&sh.full[i], stage_bytes);
                bulk_copy(stage0 + (size_t)i * stage_bytes, wsrc + (size_t)i * W_TILE, W_TILE, &sh.full[i]);
            }
            pdl_wait();
            HM_TRACE(if (tr) a.trace[2] = global_timer();)
            for (int i = 0; i < pre; ++i) bulk_copy(stage0 + (size_t)i * stage_bytes + W_TILE, xsrc + (size_t)i * x_tile, x_tile, &sh.full[i]);
            for (int i = pre; i < nkb; ++i) {
                const int s = i % nst;
                const uint32_t par = ((i / nst) & 1u) ^ 1u;
                if (!mb_wait(&sh.empty[s], par, a.err_flag, &sh.abort_flag)) break;
                mb_expect_tx(&sh.full[s], stage_bytes);
                bulk_copy(stage0 + (size_t)s * stage_bytes, wsrc + (size_t)i * W_TILE, W_TILE, &sh.full[s]);
                bulk_copy(stage0 + (size_t)s * stage_bytes + W_TILE, xsrc + (size_t)i * x_tile, x_tile, &sh.full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(TERMS * mpad);
            for (int i = 0; i < nkb; ++i) {
                const int s = i % nst;
                const uint32_t par = (i / nst) & 1u;
                if (!mb_wait(&sh.full[s], par, a.err_flag, &sh.abort_flag)) break;
                HM_TRACE(if (tr && i == 0) a.trace[3] = global_timer();)
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t wa = s32(stage0 + (size_t)s * stage_bytes);
                const uint32_t xa = wa + W_TILE;
#pragma unroll
                for (int ks = 0; ks < BK / 16; ++ks)
                    umma_f16(tmem, umma_desc_k_sw128(wa + ks * 32), umma_desc_k_sw128(xa + ks * 32), idesc, (i > 0 || ks > 0) ? 1u : 0u);
                umma_commit(&sh.empty[s]);  // stage reusable once these MMAs have read it
            }
            umma_commit(&sh.acc_full);
            HM_TRACE(if (tr) a.trace[4] = global_timer();)
        }
    } else {
        // ---- accumulator -> registers (three terms summed) -> f32 tile in shared memory [m][128]
        if (a.epi == EPI_QKV_ROPE) {
            // positions and the page table were final before this pass began: fetched while the MMAs run
            for (int mm = tid - 64; mm < a.M; mm += 128) {
                const int pos = a.row_pos[mm], seq = a.row_seq ? a.row_seq[mm] : a.seq_base + mm;
                sh.pos[mm] = pos;
                sh.page[mm] = a.kv.page_table[(size_t)seq * a.kv.max_pages + pos / a.kv.page_tokens];
            }
        }
        if (a.ss_in) {
            // deferred RMSNorm: the row factors from the producer's partial sums of squares, while the MMAs run
            if (warp == 2) {
                pdl_wait();
                for (int m = lane; m < MR; m += 32) {
                    float ssum = 0.f;
                    for (int p = 0; p < a.ss_parts; ++p) ssum += ld_cg_f32(a.ss_in + p * MR + m);
                    sh.inv[m] = 1.0f / sqrtf(ssum / (float)a.K + a.eps);
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the four accumulator warps
        }
        const bool scale_rows = a.ss_in != nullptr;
        const bool acc_ok = __all_sync(0xffffffffu, mb_wait(&sh.acc_full, 0, a.err_flag, &sh.abort_flag));
        HM_TRACE(if (tr && tid == 64) a.trace[5] = global_timer();)
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int lane_base = (warp & 3) * 32;  // a warp may only touch its own quarter of the TMEM lanes
        const int n_local = lane_base + lane;   // output feature within the CTA's 128
        if (acc_ok && nkb > 0) {
            for (int c0 = 0; c0 < mpad; c0 += 16) {
                uint32_t r[TERMS][16];
#pragma unroll
                for (int t = 0; t < TERMS; ++t) {
                    const uint32_t taddr = tmem + ((uint32_t)lane_base << 16) + (uint32_t)(t * mpad + c0);
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                        : "=r"(r[t][0]), "=r"(r[t][1]), "=r"(r[t][2]), "=r"(r[t][3]), "=r"(r[t][4]), "=r"(r[t][5]), "=r"(r[t][6]), "=r"(r[t][7]), "=r"(r[t][8]), "=r"(r[t][9]),
                          "=r"(r[t][10]), "=r"(r[t][11]), "=r"(r[t][12]), "=r"(r[t][13]), "=r"(r[t][14]), "=r"(r[t][15])
                        : "r"(taddr));
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    // small terms first: lo + mid, then + hi
                    const float v = (__uint_as_float(r[2][j]) + __uint_as_float(r[1][j])) + __uint_as_float(r[0][j]);
                    out_tile[(c0 + j) * BM + n_local] = scale_rows ? v * sh.inv[c0 + j] : v;
                }
            }
        } else {
            for (int mm = 0; mm < mpad; ++mm) out_tile[mm * BM + n_local] = 0.f;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(a.tmem_cols) : "memory");

    // ---- with split-K the accumulators are first reduce-scattered by activation row: every CTA pushes the rows
    //      that belong to a peer into that peer's receive slot `rank` with 16-byte asynchronous stores that count
    //      bytes on the peer's mbarrier, waits (bounded) for its own rows from the other ranks, and adds them in
    //      rank order.  No cluster barrier after the dependency wait, and a CTA is free to exit once it has its rows.
    pdl_wait();
    HM_TRACE(if (tr && tid == 0) a.trace[6] = global_timer();)
    int m_lo = 0, m_hi = a.M;
    if (CL) {
        const int rows_per = (a.M + cs - 1) / cs;
        m_lo = min(a.M, split * rows_per);
        m_hi = min(a.M, m_lo + rows_per);
        for (int idx = tid; idx < a.M * (BM / 4); idx += TC_THREADS) {
            const int m = idx / (BM / 4), c = (idx % (BM / 4)) * 4;
            const int owner = m / rows_per;
            if (owner == split) continue;
            const float4 v = *reinterpret_cast<const float4*>(out_tile + m * BM + c);
            float* dst = recv + ((size_t)split * rows_per + (m - owner * rows_per)) * BM + c;
            st_async_f32x4(dsmem_addr(dst, (uint32_t)owner), v, dsmem_addr(&sh.rbar, (uint32_t)owner));
        }
        HM_TRACE(if (tr && tid == 0) a.trace[7] = global_timer();)
        const bool got = cs == 1 || mb_wait_cluster(&sh.rbar, 0, a.err_flag, &sh.abort_flag);
        if (got) {
            // four consecutive features per thread; every rank's piece is read before the first add
            for (int idx = tid; idx < (m_hi - m_lo) * (BM / 4); idx += TC_THREADS) {
                const int ml = idx / (BM / 4), c = (idx % (BM / 4)) * 4;
                float4 v[16];
#pragma unroll
                for (int r = 0; r < 16; ++r)
                    if (r < cs) v[r] = r == split ? *reinterpret_cast<const float4*>(out_tile + (m_lo + ml) * BM + c) : *reinterpret_cast<const float4*>(recv + ((size_t)r * rows_per + ml) * BM + c);
                float4 t = v[0];
#pragma unroll
                for (int r = 1; r < 16; ++r)
                    if (r < cs) { t.x += v[r].x; t.y += v[r].y; t.z += v[r].z; t.w += v[r].w; }
                *reinterpret_cast<float4*>(out_tile + (m_lo + ml) * BM + c) = t;
            }
        }
        __syncthreads();
    }
    HM_TRACE(if (tr && tid == 0) a.trace[8] = global_timer();)
    tc_epilogue(a, out_tile, m_lo, m_hi, nblk, tid, sh.pos, sh.page);
    HM_TRACE(if (tr && tid == 0) a.trace[9] = global_timer();)
    HM_TRACE(if (tr && tid == 0) a.trace[10] = global_timer();)
    HM_TRACE(if (a.trace && tid == 0) atomicMax(a.trace + 12, global_timer());)
}

}  // namespace

int tc_mpad(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : 64; }
// Stages of the ring.  Launches of one wave (at most one CTA per SM: every layer projection of the 0.5-1.5 B
// models) take the deep ring, because the main loop of a lone CTA is bound by the bytes it keeps in flight
// (measured on the 1.5 B x 64 step: 2.02 ms with 4 stages, 2.10 with 3, 2.30 with 2).  Launches of several
// waves (the LM head: 1187 blocks) take two stages, which lets two CTAs share an SM (81 KB and 256 TMEM columns
// each): the head and tail of one CTA overlap the main loop of the other (LM head 194 -> 152 us).
static int tc_nstage(int mpad, bool multi_wave) {
    if (mpad == 64) return multi_wave ? 2 : 4;
    return multi_wave ? 3 : 6;
}
static size_t tc_smem_for(int mpad, bool multi_wave) { return (size_t)tc_nstage(mpad, multi_wave) * (W_TILE + (size_t)TERMS * mpad * 128) + 1024; }
// receive slots of a split-K launch: one slot of ceil(M / ksplit) rows per rank
static size_t tc_recv_bytes(int M, int ksplit) { return (size_t)ksplit * ((M + ksplit - 1) / ksplit) * BM * 4; }
size_t tc_packed_elems(int K, int N) { return (size_t)((N + BM - 1) / BM) * ((K + BK - 1) / BK) * BM * BK; }
int tc_padded_k(int K) { return (K + BK - 1) / BK * BK; }
size_t tc_xpack_bytes(int M, int K) { return (size_t)(tc_padded_k(K) / BK) * TERMS * tc_mpad(M) * 128; }
int tc_pick_split(int K, int N, int sm_count) {
    const int nblk = (N + BM - 1) / BM, kb = (K + BK - 1) / BK;
    constexpr int cap = 8;  // measured on the 1.5 B x 64 step: 4 -> 2.26 ms, 6 -> 2.02, 8 -> 1.97, 12 (non-portable cluster size) -> 2.20
    int s = sm_count / nblk;  // CTAs per n-block that still fit one wave (1 CTA per SM)
    if (s > cap) s = cap;
    while (s > 1 && kb / s < 4) --s;  // keep at least 4 k-blocks per CTA
    return s < 1 ? 1 : s;
}

cudaError_t launch_tc_pack_x(const float* x, int ldx, int M, int K, const float* norm_w, float eps, void* xp, cudaStream_t st, bool pdl, unsigned long long* trace) {
    if (M < 1 || M > MR) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)tc_mpad(M));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, tc_pack_x_kernel, x, ldx, M, tc_mpad(M), K, tc_padded_k(K), norm_w, eps, (unsigned char*)xp, trace);
}

cudaError_t launch_gemm_tc(const TcArgs& a_in, cudaStream_t st, bool pdl) {
    TcArgs a = a_in;
    if (a.M < 1 || a.M > MR || a.Kp % BK != 0 || !a.xp) return cudaErrorInvalidValue;
    a.mpad = tc_mpad(a.M);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const bool multi_wave = (long)((a.N + BM - 1) / BM) * (a.ksplit > 1 ? a.ksplit : 1) >= 2L * sms;
    a.nstage = tc_nstage(a.mpad, multi_wave);
    a.tmem_cols = a.mpad == 16 ? 64 : a.mpad == 32 ? 128 : 256;  // power of two >= 3 * mpad
    const int nblk = (a.N + BM - 1) / BM;
    const bool cl = a.ksplit > 1;
    const size_t smem = tc_smem_for(a.mpad, multi_wave) + (cl ? tc_recv_bytes(a.M, a.ksplit) : 0);
    {
        const size_t mx = (tc_smem_for(64, false) > tc_smem_for(32, false) ? tc_smem_for(64, false) : tc_smem_for(32, false)) + (cl ? (size_t)(MR + 16) * BM * 4 : 0);
        cudaError_t e = cl ? ensure_dyn_smem(gemm_tc_kernel<true>, mx) : ensure_dyn_smem(gemm_tc_kernel<false>, mx);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(nblk * (cl ? a.ksplit : 1)));
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    int n = 0;
    if (pdl) {
        at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cl) {
        if (a.ksplit > 16) return cudaErrorInvalidValue;
        if (a.ksplit > 8) {  // clusters of 9..16 CTAs are allowed on request
            cudaError_t e = ensure_nonportable_clusters(gemm_tc_kernel<true>);
            if (e != cudaSuccess) return e;
        }
        at[n].id = cudaLaunchAttributeClusterDimension;
        at[n].val.clusterDim.x = (unsigned)a.ksplit;
        at[n].val.clusterDim.y = 1;
        at[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = at;
    cfg.numAttrs = n;
    return cl ? cudaLaunchKernelEx(&cfg, gemm_tc_kernel<true>, a) : cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false>, a);
}

// ---- weight packing: [N][K] (HF [out,in]) or [K][N] bf16 -> swizzled K-major tiles ----------
namespace {
__global__ void pack_tc_kernel(const uint16_t* __restrict__ src, int N, int K, int src_is_kn, uint16_t* __restrict__ dst, int n_off, int interleave_which) {
    const int kb_total = (K + BK - 1) / BK;
    const size_t total = (size_t)N * kb_total * BK;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int kk = (int)(i % BK);
        const int kb = (int)((i / BK) % kb_total);
        const int n = (int)(i / ((size_t)BK * kb_total));
        const int k = kb * BK + kk;
        const uint16_t v = k < K ? (src_is_kn ? src[(size_t)k * N + n] : src[(size_t)n * K + k]) : (uint16_t)0;
        const int no = interleave_which >= 0 ? (n / 64) * BM + interleave_which * 64 + (n % 64) : n + n_off;
        const int nb = no / BM, row = no % BM;
        const int chunk = kk >> 3, e = kk & 7;
        const size_t tile = ((size_t)nb * kb_total + kb) * (BM * BK);
        dst[tile + (size_t)row * BK + (size_t)((chunk ^ (row & 7)) << 3) + e] = v;
    }
}
}  // namespace

cudaError_t launch_pack_tc(const uint16_t* src, int N, int K, bool src_is_kn, uint16_t* dst, int n_off, int interleave_which, cudaStream_t st) {
    const size_t total = (size_t)N * ((K + BK - 1) / BK) * BK;
    size_t g = (total + 255) / 256;
    if (g > 148 * 32) g = 148 * 32;
    if (g < 1) g = 1;
    pack_tc_kernel<<<(unsigned)g, 256, 0, st>>>(src, N, K, src_is_kn ? 1 : 0, dst, n_off, interleave_which);
    return cudaGetLastError();
}

}  // namespace hm
