// GGUF block-quantised projections: Q8_0 (Homura's emit_dequant_matmul_q8_0,
// src/graph_builder/emit_quant.rs:30-142) and Q4_0 (no counterpart in Homura, which maps the
// type to no DType, src/gguf.rs:94-109; defined here from the public ggml block format:
// f16 scale d, 16 bytes, byte i = element i (low nibble) | element i+16 (high nibble),
// value = (nibble - 8) * d).
//
// GGUF stores blocks [N, K/32] of 34 (Q8_0) or 18 (Q4_0) bytes, which no 128-bit load can
// address.  At load the blocks are re-laid in tiles of 32 output rows (same bits, new order):
//   scales f16 [N/32][K/32][32 rows]
//   codes      [N/32][K/32][chunk][32 rows][16 B]   chunk = 2 halves of a Q8_0 block, 1 for Q4_0
// so that the 32 lanes of a warp, each owning one output row, read 512 contiguous bytes per
// load and all need the SAME 32 activations (one broadcast read from shared memory, no bank
// conflicts, no shuffle reduction).  A CTA's 8 warps take the k-blocks of its K range round-robin
// and are summed through shared memory in warp order; K may further be split over the CTAs of a
// thread-block cluster, summed in rank order through distributed shared memory.  Codes become
// f32 with a byte permute into the mantissa of 2^23 and one subtraction (exact).
#include <algorithm>

#include "common.cuh"
#include "launch_attrs.h"
#include "mbarrier.cuh"

namespace hm {


namespace {

constexpr int QT = 256;

// blocks: rows [0, n_part) of a projection part, stored at rows n_off.. of the tiled arrays.
// interleave_which 0 / 1: gate / up rows of a fused SwiGLU projection, 16 + 16 per 32-row tile.
__global__ void split_blocks_kernel(const uint8_t* __restrict__ blocks, size_t nblocks, int nb, int q4, int n_off, int interleave_which, uint16_t* __restrict__ scales, uint8_t* __restrict__ codes) {
    const int bsz = q4 ? 18 : 34;
    for (size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x; b < nblocks; b += (size_t)gridDim.x * blockDim.x) {
        const uint8_t* s = blocks + b * bsz;
        const int nl = (int)(b / nb), kb = (int)(b % nb);
        const int n = interleave_which >= 0 ? (nl >> 4) * 32 + interleave_which * 16 + (nl & 15) : n_off + nl;
        const size_t tk = (size_t)(n >> 5) * nb + kb;
        const int r = n & 31;
        scales[tk * 32 + r] = (uint16_t)(s[0] | (s[1] << 8));
        if (q4) {
            uint8_t* d = codes + (tk * 32 + r) * 16;
            for (int j = 0; j < 16; ++j) d[j] = s[2 + j];
        } else {
            for (int c = 0; c < 2; ++c) {
                uint8_t* d = codes + ((tk * 2 + c) * 32 + r) * 16;
                for (int j = 0; j < 16; ++j) d[j] = s[2 + c * 16 + j];
            }
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

// four packed codes -> f32, exact: the byte lands in the mantissa of 2^23, then 2^23 + bias is subtracted
__device__ __forceinline__ float code_f32(uint32_t w, int b, float magic) { return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u + b)) - magic; }

template <int M, bool Q4>
__device__ __forceinline__ void q_block(const uint4 (&c)[2], float d, const float* __restrict__ xb, int xstride, float (&acc)[M]) {
    float p[M];
#pragma unroll
    for (int m = 0; m < M; ++m) p[m] = 0.f;
    if (Q4) {
        // byte j = element j (low nibble) | element j + 16 (high nibble); value = nibble - 8
        const uint32_t w[4] = {c[0].x, c[0].y, c[0].z, c[0].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t lo = w[i] & 0x0F0F0F0Fu, hi = (w[i] >> 4) & 0x0F0F0F0Fu;
            float fl[4], fh[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                fl[b] = code_f32(lo, b, 8388616.0f);
                fh[b] = code_f32(hi, b, 8388616.0f);
            }
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float4 xl = *reinterpret_cast<const float4*>(xb + m * xstride + i * 4);
                const float4 xh = *reinterpret_cast<const float4*>(xb + m * xstride + 16 + i * 4);
                p[m] = fmaf(fl[0], xl.x, p[m]);
                p[m] = fmaf(fl[1], xl.y, p[m]);
                p[m] = fmaf(fl[2], xl.z, p[m]);
                p[m] = fmaf(fl[3], xl.w, p[m]);
                p[m] = fmaf(fh[0], xh.x, p[m]);
                p[m] = fmaf(fh[1], xh.y, p[m]);
                p[m] = fmaf(fh[2], xh.z, p[m]);
                p[m] = fmaf(fh[3], xh.w, p[m]);
            }
        }
    } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w[4] = {c[h].x, c[h].y, c[h].z, c[h].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t u = w[i] ^ 0x80808080u;  // int8 -> offset-128 byte
                float f[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) f[b] = code_f32(u, b, 8388736.0f);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float4 xv = *reinterpret_cast<const float4*>(xb + m * xstride + h * 16 + i * 4);
                    p[m] = fmaf(f[0], xv.x, p[m]);
                    p[m] = fmaf(f[1], xv.y, p[m]);
                    p[m] = fmaf(f[2], xv.z, p[m]);
                    p[m] = fmaf(f[3], xv.w, p[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = fmaf(d, p[m], acc[m]);
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
    float* xs = ST ? qsm + ((size_t)a.kb_per_split * (CHB + 64)) / 4 : qsm;  // [M][kspan]
    float* red = xs + M * kspan;            // [8 warps][M][32], then vals [M][32] at red[0..]
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
    const uint16_t* sbase = a.scales + ((size_t)tile * nb + kb0) * 32 + lane;

    pdl_launch_dependents();

    // weights never depend on a previous kernel: the whole slice into shared memory (ST), or the first batch of
    // streaming loads into registers, before the dependency wait
    uint4 c[QU][2];
    uint16_t sc[QU];
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
            sc[u] = ok ? sbase[(size_t)kb * 32] : (uint16_t)0;
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

    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
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
            }
            if (!ok) break;
            uint4 cc[2];
#pragma unroll
            for (int h = 0; h < CH; ++h) cc[h] = *reinterpret_cast<const uint4*>(codes_s + ((size_t)(kb * CH + h) * 32 + lane) * 16);
            q_block<M, Q4>(cc, f16_bits_to_f32(scales_s[kb * 32 + lane]), xs + kb * 32, kspan, acc);
        }
    } else
    for (int base = warp; base < nkb; base += 8 * QU) {
        // issue the next batch, then consume the current one
        uint4 cn[QU][2];
        uint16_t sn[QU];
#pragma unroll
        for (int u = 0; u < QU; ++u) {
            const int kb = base + 8 * (QU + u);
            const bool ok = kb < nkb;
#pragma unroll
            for (int h = 0; h < CH; ++h) cn[u][h] = ok ? ld_stream_u4(cbase + ((size_t)kb * CH + h) * 32) : make_uint4(0, 0, 0, 0);
            sn[u] = ok ? sbase[(size_t)kb * 32] : (uint16_t)0;
        }
#pragma unroll
        for (int u = 0; u < QU; ++u) {
            const int kb = base + 8 * u;
            if (kb < nkb) q_block<M, Q4>(c[u], f16_bits_to_f32(sc[u]), xs + kb * 32, kspan, acc);
        }
#pragma unroll
        for (int u = 0; u < QU; ++u) {
            c[u][0] = cn[u][0];
            if (!Q4) c[u][1] = cn[u][1];
            sc[u] = sn[u];
        }
    }

    // ---- sum the 8 warps (fixed order), then the cluster ranks (fixed order) ----
    __syncthreads();  // xs is dead; red aliases nothing of it but keep the phases apart
#pragma unroll
    for (int m = 0; m < M; ++m) red[(warp * M + m) * 32 + lane] = acc[m];
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
        if (split != 0) return;
        cluster_wait_acquire();
        if (tid < M * 32) {
            v = slots[tid];
            for (int r = 1; r < a.ksplit; ++r) v += slots[r * (M * 32) + tid];
        }
    }
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
    } else if (writer && tid < M * 32) {
        const int m = tid >> 5, n = tile * 32 + (tid & 31);
        if (m < a.m_valid && n < a.N) {
            if (a.bias) v += a.bias[n];
            if (a.resid) v = a.resid[(size_t)m * a.ldy + n] + v;
            a.y[(size_t)m * a.ldy + n] = v;
        }
    }
}

constexpr size_t QUANT_STAGE_MAX = 96 * 1024;  // largest weight slice staged in shared memory (two CTAs per SM stay resident)

template <int M, bool Q4, bool CL, bool ST>
cudaError_t launch_q4(const QuantArgs& a, size_t smem, cudaStream_t st, bool pdl);

template <int M, bool Q4, bool CL>
cudaError_t launch_q3(const QuantArgs& a, cudaStream_t st, bool pdl) {
    size_t smem = sizeof(float) * ((size_t)M * a.kb_per_split * 32 + 8 * M * 32 + (CL ? (size_t)a.ksplit * M * 32 : 0));
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

cudaError_t launch_split_blocks(const uint8_t* blocks, int n_rows, int K, int q4, int n_off, int interleave_which, uint16_t* scales, uint8_t* codes, cudaStream_t st) {
    const size_t nblocks = (size_t)n_rows * (K / 32);
    size_t g = (nblocks + 255) / 256;
    if (g > 148 * 32) g = 148 * 32;
    if (g < 1) g = 1;
    split_blocks_kernel<<<(unsigned)g, 256, 0, st>>>(blocks, nblocks, K / 32, q4, n_off, interleave_which, scales, codes);
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
