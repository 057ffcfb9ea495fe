// GGUF block-quantised projections: Q8_0 (Homura's emit_dequant_matmul_q8_0,
// src/graph_builder/emit_quant.rs:30-142) and Q4_0 (no counterpart in Homura, which maps the
// type to no DType, src/gguf.rs:94-109; defined here from the public ggml block format:
// f16 scale d, 16 bytes, byte i = element i (low nibble) | element i+16 (high nibble),
// value = (nibble - 8) * d).
//
// GGUF stores blocks [N, K/32] of 34 (Q8_0) or 18 (Q4_0) bytes, which no 128-bit load can
// address.  At load the blocks are split into two arrays (same bytes, same order):
//   scales f16 [N][K/32]    codes int8 [N][K]  (Q8_0)  or  nibble bytes [N][K/2]  (Q4_0)
// The GEMV is a row dot product per output: a warp owns an output row, every lane reads
// 16 bytes of codes per step (coalesced 512 B per warp), dequantises in registers
// (integer code -> f32, one multiply by the block scale) and the 32 lane partials are merged
// with xor shuffles.  Activations sit in shared memory as f32.
#include "common.cuh"

namespace hm {


namespace {

constexpr int QT = 256;

__global__ void split_blocks_kernel(const uint8_t* __restrict__ blocks, size_t nblocks, int q4, uint16_t* __restrict__ scales, uint8_t* __restrict__ codes) {
    const int bsz = q4 ? 18 : 34, csz = q4 ? 16 : 32;
    for (size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x; b < nblocks; b += (size_t)gridDim.x * blockDim.x) {
        const uint8_t* s = blocks + b * bsz;
        scales[b] = (uint16_t)(s[0] | (s[1] << 8));
        for (int j = 0; j < csz; ++j) codes[b * csz + j] = s[2 + j];
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

template <int M>
__global__ void __launch_bounds__(QT) gemv_quant_kernel(const QuantArgs a, int rows_per_warp) {
    extern __shared__ __align__(16) float xs[];  // [M][K]
    __shared__ double s_wsum[8][MAX_M];
    __shared__ float s_inv[MAX_M];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    pdl_wait();
    if (a.pro == PRO_RMSNORM) {
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
            const float* xr = a.x + (size_t)m * a.ldx;
            for (int k = tid; k < a.K; k += QT) xs[m * a.K + k] = (xr[k] * inv) * a.norm_w[k];
        }
    } else {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float* xr = a.x + (size_t)m * a.ldx;
            for (int k = tid; k < a.K; k += QT) xs[m * a.K + k] = xr[k];
        }
    }
    __syncthreads();

    const int nb = a.K / 32;
    const int row0 = (blockIdx.x * 8 + warp) * rows_per_warp;
    for (int r = 0; r < rows_per_warp; ++r) {
        const int n = row0 + r;
        if (n >= a.N) break;
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        if (a.q4) {
            // 16 bytes = one block of 32 values
            const uint4* cp = reinterpret_cast<const uint4*>(a.codes + (size_t)n * (a.K / 2));
            for (int c = lane; c < nb; c += 32) {
                const uint4 v = ld_stream_u4(cp + c);
                const float d = f16_bits_to_f32(a.scales[(size_t)n * nb + c]);
                const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float* xb = xs + m * a.K + c * 32;
                    float p = 0.f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            const uint32_t byte = (wv[i] >> (8 * b)) & 0xFFu;
                            const int j = i * 4 + b;
                            p = fmaf((float)((int)(byte & 0x0Fu) - 8), xb[j], p);
                            p = fmaf((float)((int)(byte >> 4) - 8), xb[j + 16], p);
                        }
                    }
                    acc[m] = fmaf(d, p, acc[m]);
                }
            }
        } else {
            // 16 bytes = half a block (16 values); two lanes share a scale
            const uint4* cp = reinterpret_cast<const uint4*>(a.codes + (size_t)n * a.K);
            for (int c = lane; c < nb * 2; c += 32) {
                const uint4 v = ld_stream_u4(cp + c);
                const float d = f16_bits_to_f32(a.scales[(size_t)n * nb + (c >> 1)]);
                const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float* xb = xs + m * a.K + c * 16;
                    float p = 0.f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            const int q = (int)(int8_t)((wv[i] >> (8 * b)) & 0xFFu);
                            p = fmaf((float)q, xb[i * 4 + b], p);
                        }
                    }
                    acc[m] = fmaf(d, p, acc[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = warp_sum(acc[m]);
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < M; ++m) {
                if (m < a.m_valid) {
                    float v = acc[m];
                    if (a.bias) v += a.bias[n];
                    if (a.resid) v = a.resid[(size_t)m * a.ldy + n] + v;
                    a.y[(size_t)m * a.ldy + n] = v;
                }
            }
        }
    }
}

template <int M>
cudaError_t launch_qm(const QuantArgs& a, int sm_count, cudaStream_t st, bool pdl) {
    const size_t smem = sizeof(float) * (size_t)M * a.K;
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    if (smem > 40 * 1024) {  // static shared memory counts against the 48 KB default too
        cudaError_t e = cudaFuncSetAttribute(gemv_quant_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    // about four CTAs per SM when the matrix is large enough, one row per warp at least
    int rpw = (a.N + sm_count * 4 * 8 - 1) / (sm_count * 4 * 8);
    if (rpw < 1) rpw = 1;
    const int grid = (a.N + 8 * rpw - 1) / (8 * rpw);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(QT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemv_quant_kernel<M>, a, rpw);
}

}  // namespace

cudaError_t launch_split_blocks(const uint8_t* blocks, size_t nblocks, int q4, uint16_t* scales, uint8_t* codes, cudaStream_t st) {
    size_t g = (nblocks + 255) / 256;
    if (g > 148 * 32) g = 148 * 32;
    if (g < 1) g = 1;
    split_blocks_kernel<<<(unsigned)g, 256, 0, st>>>(blocks, nblocks, q4, scales, codes);
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
