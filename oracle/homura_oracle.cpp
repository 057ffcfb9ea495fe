// homura_oracle.cpp -- CPU restatement of Homura's decoder-only RoPE transformer path.
//
// TEST INFRASTRUCTURE ONLY.  Nothing in the product (homura_b200/) links, imports or
// calls this file.  It is used by the tests as the checker, by the smoke check, and
// by the benchmark's CPU-baseline leg as "the reference's algorithm on host cores".
//
// Homura (Rust + MLIR/LLVM) cannot be built where this runs (no Rust toolchain, no
// patched LLVM 21), so this file restates the arithmetic that Homura's emitters
// generate, from its sources.  Each function cites the reference file:line it follows
// (paths are relative to the Homura repository root).
//
// Parity pins (reference tests whose expected values this file reproduces, checked by
// tests/test_oracle_golden.py):
//   KV cache append/view/multi-token/reset ...... src/runtime.rs:2228-2366
//   RoPE table values, duplication, slicing ...... src/hf/precompute.rs:108-131,163-179
//   causal mask prefill/decode ................... src/hf/precompute.rs:133-161
//   RMSNorm [1,2,3,4] ............................ src/graph_builder/mod.rs:3800-3825
//   SiLU, softmax known values ................... src/graph_builder/mod.rs:3773-3797,2942-2961
//   Q8_0 block dot = 528 ......................... src/graph_builder/emit_quant.rs:894-958
//   f16/bf16 -> f32 conversions .................. src/hf/safetensors.rs:195-237
//   greedy sample, min_p, RNG determinism ........ src/generate.rs:883-969
// PARITY UNPINNED (no runnable reference test or fixture exists): Q4_0 (absent from the
// reference; defined here from the public GGUF block format), emit_rope_half, the GQA
// floordiv QK/AV contraction, the mixed bf16 matmul and whole-model logits.  For those
// this restatement is the definition; tests cross-check it against an independent
// numpy float64 evaluation.
//
// Floating-point conventions restated from the sources: only the `contract` fast-math
// flag is set by the reference (src/graph_builder/mod.rs:889-896, src/compiler.rs:89-111),
// so reductions are never re-associated: every contraction is a single chain over the
// reduction index in ascending order, each step an FMA.  Sum-of-squares and softmax sums
// are sequential ascending; x*x is a separate multiply followed by an add.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <map>
#include <string>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------------------
// Scalar conversions
// ---------------------------------------------------------------------------------------

// src/gguf.rs:781-810 (also src/hf/safetensors.rs f16_to_f32): IEEE half bits -> f32.
ORC_API float orc_f16_to_f32(uint16_t bits) {
    uint32_t sign = (bits >> 15) & 1u;
    uint32_t exp = (bits >> 10) & 0x1Fu;
    uint32_t frac = bits & 0x3FFu;
    uint32_t out;
    if (exp == 0) {
        if (frac == 0) {
            out = sign << 31;
        } else {
            int e = 0;
            uint32_t f = frac;
            while ((f & 0x400u) == 0) {
                f <<= 1;
                e -= 1;
            }
            f &= 0x3FFu;
            uint32_t exp32 = (uint32_t)(127 - 15 + 1 + e);
            out = (sign << 31) | (exp32 << 23) | (f << 13);
        }
    } else if (exp == 31) {
        out = (sign << 31) | (0xFFu << 23) | (frac << 13);
    } else {
        uint32_t exp32 = (uint32_t)((int)exp - 15 + 127);
        out = (sign << 31) | (exp32 << 23) | (frac << 13);
    }
    float f;
    std::memcpy(&f, &out, 4);
    return f;
}

// src/hf/weights.rs:196-204: bf16 is the top 16 bits of an f32.
ORC_API float orc_bf16_to_f32(uint16_t bits) {
    uint32_t u = (uint32_t)bits << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// src/hf/weights.rs:207-214: f32 -> bf16 by truncation (used for the tied LM head).
ORC_API uint16_t orc_f32_to_bf16_trunc(float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    return (uint16_t)(u >> 16);
}

// ---------------------------------------------------------------------------------------
// RoPE table, causal mask  (src/hf/precompute.rs)
// ---------------------------------------------------------------------------------------

// src/hf/precompute.rs:10-40: angle in f64, cos/sin cast to f32, halves duplicated.
ORC_API void orc_rope_table(int head_dim, int max_pos, double theta, float* cos_out, float* sin_out) {
    int half = head_dim / 2;
    for (int pos = 0; pos < max_pos; ++pos) {
        for (int i = 0; i < half; ++i) {
            double freq = 1.0 / std::pow(theta, 2.0 * (double)i / (double)head_dim);
            double angle = (double)pos * freq;
            float c = (float)std::cos(angle);
            float s = (float)std::sin(angle);
            cos_out[(size_t)pos * head_dim + i] = c;
            cos_out[(size_t)pos * head_dim + half + i] = c;
            sin_out[(size_t)pos * head_dim + i] = s;
            sin_out[(size_t)pos * head_dim + half + i] = s;
        }
    }
}

// src/hf/precompute.rs:49-64: mask[i][j] = 0 if j <= i + past else -inf; shape [seq, seq+past].
ORC_API void orc_causal_mask(int seq, int past, float* out) {
    int total = seq + past;
    for (int i = 0; i < seq; ++i)
        for (int j = 0; j < total; ++j)
            out[(size_t)i * total + j] = (j > i + past) ? -std::numeric_limits<float>::infinity() : 0.0f;
}

// ---------------------------------------------------------------------------------------
// Elementwise / normalisation ops
// ---------------------------------------------------------------------------------------

// src/graph_builder/emit_linalg.rs:7-26: x * rsqrt(mean(x^2) + eps) * w.  mean = f32 sum
// (ascending) / count (emit_reduce_mean, emit_linalg.rs:379-498).  (x*inv)*w association.
ORC_API void orc_rms_norm(const float* x, const float* w, float eps, int rows, int n, float* out) {
    for (int r = 0; r < rows; ++r) {
        const float* xr = x + (size_t)r * n;
        float sum = 0.0f;
        for (int i = 0; i < n; ++i) {
            float sq = xr[i] * xr[i];
            sum = sum + sq;
        }
        float mean = sum / (float)n;
        float inv = 1.0f / std::sqrt(mean + eps);
        for (int i = 0; i < n; ++i) out[(size_t)r * n + i] = (xr[i] * inv) * w[i];
    }
}

// src/graph_builder/emit_linalg.rs:33-56: x*x in f32, widened to f64 for the sum, mean in
// f64 (sum / count), cast to f32, + eps, rsqrt.
ORC_API void orc_rms_norm_f64_accum(const float* x, const float* w, float eps, int rows, int n, float* out) {
    for (int r = 0; r < rows; ++r) {
        const float* xr = x + (size_t)r * n;
        double sum = 0.0;
        for (int i = 0; i < n; ++i) {
            float sq = xr[i] * xr[i];
            sum = sum + (double)sq;
        }
        float mean = (float)(sum / (double)n);
        float inv = 1.0f / std::sqrt(mean + eps);
        for (int i = 0; i < n; ++i) out[(size_t)r * n + i] = (xr[i] * inv) * w[i];
    }
}

// src/hf/emitter_quant.rs:713-791 (also :985-1071): x widened to f64 before squaring,
// mean = sum * (1/n) in f64, cast to f32, scale = 1 / sqrt(mean + eps), (x*scale)*w.
ORC_API void orc_rms_norm_quant_kernel(const float* x, const float* w, float eps, int rows, int n, float* out) {
    double inv_n = 1.0 / (double)n;
    for (int r = 0; r < rows; ++r) {
        const float* xr = x + (size_t)r * n;
        double sum = 0.0;
        for (int i = 0; i < n; ++i) {
            double v = (double)xr[i];
            sum = sum + v * v;
        }
        float mean = (float)(sum * inv_n);
        float rms = std::sqrt(mean + eps);
        float scale = 1.0f / rms;
        for (int i = 0; i < n; ++i) out[(size_t)r * n + i] = (xr[i] * scale) * w[i];
    }
}

// src/graph_builder/emit_arithmetic.rs:101-107: x / (1 + exp(-x)).
ORC_API void orc_silu(const float* x, int n, float* out) {
    for (int i = 0; i < n; ++i) out[i] = x[i] / (1.0f + std::exp(-x[i]));
}

// src/graph_builder/emit_linalg.rs:509-528 (f32 sum) and :534-555 (f64 sum).
ORC_API void orc_softmax(const float* x, int rows, int n, int f64_sum, float* out) {
    for (int r = 0; r < rows; ++r) {
        const float* xr = x + (size_t)r * n;
        float* o = out + (size_t)r * n;
        float mx = -std::numeric_limits<float>::infinity();
        for (int i = 0; i < n; ++i) mx = std::max(mx, xr[i]);
        if (f64_sum) {
            double s = 0.0;
            for (int i = 0; i < n; ++i) {
                o[i] = std::exp(xr[i] - mx);
                s += (double)o[i];
            }
            float sf = (float)s;
            for (int i = 0; i < n; ++i) o[i] = o[i] / sf;
        } else {
            float s = 0.0f;
            for (int i = 0; i < n; ++i) {
                o[i] = std::exp(xr[i] - mx);
                s += o[i];
            }
            for (int i = 0; i < n; ++i) o[i] = o[i] / s;
        }
    }
}

// src/graph_builder/emit_linalg.rs:315-342: out = x*cos + rotate_half(x)*sin with
// rotate_half(x) = cat(-x[hd/2:], x[:hd/2]).  x is [seq, heads, hd]; cos/sin are [seq, hd].
ORC_API void orc_rope_half(float* x, int seq, int heads, int hd, const float* cos_rows, const float* sin_rows) {
    int half = hd / 2;
    std::vector<float> tmp(hd);
    for (int s = 0; s < seq; ++s) {
        const float* c = cos_rows + (size_t)s * hd;
        const float* sn = sin_rows + (size_t)s * hd;
        for (int h = 0; h < heads; ++h) {
            float* v = x + ((size_t)s * heads + h) * hd;
            for (int d = 0; d < hd; ++d) {
                float rot = (d < half) ? -v[d + half] : v[d - half];
                tmp[d] = std::fma(rot, sn[d], v[d] * c[d]);
            }
            std::memcpy(v, tmp.data(), sizeof(float) * hd);
        }
    }
}

// ---------------------------------------------------------------------------------------
// Matmuls
// ---------------------------------------------------------------------------------------

// src/graph_builder/emit_linalg.rs:1928-2008,2224-2307 with the schedule of
// src/compiler.rs:1422-1682: y[m,n] = sum_k x[m,k] * f32(W[k,n]); f32 accumulator from 0,
// k ascending, one FMA per k.  Outer N tiles run as an OpenMP parallel-for, N innermost.
template <typename WT, typename CVT>
static void matmul_kn(const float* x, const WT* w, int M, int K, int N, float* y, CVT cvt) {
    const int NT = 128;
    int ntiles = (N + NT - 1) / NT;
#pragma omp parallel for schedule(static)
    for (int t = 0; t < ntiles; ++t) {
        int n0 = t * NT;
        int nw = std::min(NT, N - n0);
        float acc[NT];
        for (int m = 0; m < M; ++m) {
            for (int j = 0; j < nw; ++j) acc[j] = 0.0f;
            const float* xr = x + (size_t)m * K;
            for (int k = 0; k < K; ++k) {
                float xv = xr[k];
                const WT* wr = w + (size_t)k * N + n0;
                for (int j = 0; j < nw; ++j) acc[j] = std::fma(xv, cvt(wr[j]), acc[j]);
            }
            for (int j = 0; j < nw; ++j) y[(size_t)m * N + n0 + j] = acc[j];
        }
    }
}

ORC_API void orc_matmul_bf16(const float* x, const uint16_t* w, int M, int K, int N, float* y) {
    matmul_kn(x, w, M, K, N, y, [](uint16_t b) { return orc_bf16_to_f32(b); });
}

ORC_API void orc_matmul_f32(const float* x, const float* w, int M, int K, int N, float* y) {
    matmul_kn(x, w, M, K, N, y, [](float b) { return b; });
}

// src/gguf.rs:817-831: x[i] = (f32)q[i] * d.
ORC_API void orc_dequant_q8_0(const uint8_t* src, size_t nblocks, float* dst) {
    for (size_t b = 0; b < nblocks; ++b) {
        const uint8_t* blk = src + b * 34;
        float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int j = 0; j < 32; ++j) dst[b * 32 + j] = (float)(int8_t)blk[2 + j] * d;
    }
}

// Q4_0 is not implemented by the reference (src/gguf.rs:94-109 maps it to no DType; only
// its geometry, 32 values in 18 bytes, appears at src/gguf.rs:141).  Definition used here
// is the public GGUF/ggml block format: f16 scale d, then 16 bytes; byte i holds element i
// in its low nibble and element i+16 in its high nibble; value = (nibble - 8) * d.
ORC_API void orc_dequant_q4_0(const uint8_t* src, size_t nblocks, float* dst) {
    for (size_t b = 0; b < nblocks; ++b) {
        const uint8_t* blk = src + b * 18;
        float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int j = 0; j < 16; ++j) {
            int lo = blk[2 + j] & 0x0F;
            int hi = blk[2 + j] >> 4;
            dst[b * 32 + j] = (float)(lo - 8) * d;
            dst[b * 32 + j + 16] = (float)(hi - 8) * d;
        }
    }
}

// src/graph_builder/emit_quant.rs:30-142: weight blocks [N, K/32] x 34 bytes; per output:
// for each block: w_j = f32(q_j)*d, p_j = w_j*x_j, dot = ordered sum of the 32 p_j
// (vector.reduction <add>, sequential), acc = acc + dot.
ORC_API void orc_matmul_q8_0(const float* x, const uint8_t* w, int M, int K, int N, float* y) {
    int nb = K / 32;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            const float* xr = x + (size_t)m * K;
            float acc = 0.0f;
            for (int kb = 0; kb < nb; ++kb) {
                const uint8_t* blk = w + ((size_t)n * nb + kb) * 34;
                float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
                float dot = 0.0f;
                for (int j = 0; j < 32; ++j) {
                    float dq = (float)(int8_t)blk[2 + j] * d;
                    float p = dq * xr[kb * 32 + j];
                    dot = dot + p;
                }
                acc = acc + dot;
            }
            y[(size_t)m * N + n] = acc;
        }
    }
}

// Same accumulation structure as Q8_0 applied to the Q4_0 block format defined above.
ORC_API void orc_matmul_q4_0(const float* x, const uint8_t* w, int M, int K, int N, float* y) {
    int nb = K / 32;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            const float* xr = x + (size_t)m * K;
            float acc = 0.0f;
            for (int kb = 0; kb < nb; ++kb) {
                const uint8_t* blk = w + ((size_t)n * nb + kb) * 18;
                float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
                float wv[32];
                for (int j = 0; j < 16; ++j) {
                    wv[j] = (float)((blk[2 + j] & 0x0F) - 8) * d;
                    wv[j + 16] = (float)((blk[2 + j] >> 4) - 8) * d;
                }
                float dot = 0.0f;
                for (int j = 0; j < 32; ++j) {
                    float p = wv[j] * xr[kb * 32 + j];
                    dot = dot + p;
                }
                acc = acc + dot;
            }
            y[(size_t)m * N + n] = acc;
        }
    }
}

// ---------------------------------------------------------------------------------------
// K-quants: Q4_K and Q6_K super-blocks of 256 values.
//   dequantisation        src/gguf.rs:833-917 (embeddings and the LM head are widened to f32)
//   Q8_K activation quantisation + integer dot product
//                         src/graph_builder/emit_quant.rs:165-567 (Q4_K), 569-816 (Q6_K)
// ---------------------------------------------------------------------------------------

// get_scale_min_k4 as spelled out in src/gguf.rs:848-864.
static inline void orc_q4k_scales(const uint8_t* sr, uint8_t sc[8], uint8_t mn[8]) {
    for (int i = 0; i < 4; ++i) {
        sc[i] = sr[i] & 0x3F;
        mn[i] = sr[4 + i] & 0x3F;
    }
    for (int i = 0; i < 4; ++i) {
        sc[4 + i] = (uint8_t)((sr[8 + i] & 0x0F) | ((sr[i] >> 6) << 4));
        mn[4 + i] = (uint8_t)((sr[8 + i] >> 4) | ((sr[4 + i] >> 6) << 4));
    }
}

ORC_API void orc_dequant_q4_k(const uint8_t* src, size_t nblocks, float* dst) {
    for (size_t b = 0; b < nblocks; ++b) {
        const uint8_t* blk = src + b * 144;
        float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        float dmin = orc_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
        uint8_t sc[8], mn[8];
        orc_q4k_scales(blk + 4, sc, mn);
        const uint8_t* qs = blk + 16;
        for (int pair = 0; pair < 4; ++pair) {
            float scale0 = d * (float)sc[2 * pair], min0 = dmin * (float)mn[2 * pair];
            float scale1 = d * (float)sc[2 * pair + 1], min1 = dmin * (float)mn[2 * pair + 1];
            const uint8_t* q = qs + pair * 32;
            float* o = dst + b * 256 + pair * 64;
            for (int l = 0; l < 32; ++l) o[l] = (float)(q[l] & 0x0F) * scale0 - min0;
            for (int l = 0; l < 32; ++l) o[32 + l] = (float)(q[l] >> 4) * scale1 - min1;
        }
    }
}

// Signed 6-bit code of element e (0..255) of a Q6_K block (llama.cpp layout, src/gguf.rs:897-914).
static inline int orc_q6k_code(const uint8_t* blk, int e) {
    int chunk = e >> 7, r = e & 127, group = r >> 5, l = r & 31;
    uint8_t qlb = blk[chunk * 64 + (group & 1) * 32 + l];
    int lo = group >= 2 ? (qlb >> 4) : (qlb & 0x0F);
    int hi = (blk[128 + chunk * 32 + l] >> (group * 2)) & 3;
    return (lo | (hi << 4)) - 32;
}

ORC_API void orc_dequant_q6_k(const uint8_t* src, size_t nblocks, float* dst) {
    for (size_t b = 0; b < nblocks; ++b) {
        const uint8_t* blk = src + b * 210;
        float d = orc_f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
        for (int e = 0; e < 256; ++e) {
            float sc = (float)(int8_t)blk[192 + (e >> 4)];
            dst[b * 256 + e] = d * sc * (float)orc_q6k_code(blk, e);  // (d * sc) * q, as written in the reference
        }
    }
}

// Q8_K quantisation of one activation row (emit_quant.rs:409-460): per 256-value block
// act_d = amax / 127, iscale = 127 / amax (0 when amax == 0), q = clamp(roundeven(x * iscale), -127, 127),
// bsums[g] = sum of the 16 codes of group g.
ORC_API void orc_quantize_q8_k(const float* x, int K, int8_t* q8, float* act_d, int32_t* bsums) {
    int nb = K / 256;
    for (int kb = 0; kb < nb; ++kb) {
        const float* xb = x + kb * 256;
        float amax = 0.0f;
        for (int i = 0; i < 256; ++i) amax = std::fmax(amax, std::fabs(xb[i]));
        act_d[kb] = amax / 127.0f;
        float iscale = amax == 0.0f ? 0.0f : 127.0f / amax;
        for (int g = 0; g < 16; ++g) bsums[kb * 16 + g] = 0;
        for (int i = 0; i < 256; ++i) {
            float r = std::nearbyintf(xb[i] * iscale);  // round half to even (math.roundeven)
            r = std::fmin(r, 127.0f);
            r = std::fmax(r, -127.0f);
            int8_t q = (int8_t)(int32_t)r;
            q8[kb * 256 + i] = q;
            bsums[kb * 16 + (i >> 4)] += q;
        }
    }
}

ORC_API void orc_matmul_q4_k(const float* x, const uint8_t* w, int M, int K, int N, float* y) {
    int nb = K / 256;
    std::vector<int8_t> q8((size_t)M * K);
    std::vector<float> ad((size_t)M * nb);
    std::vector<int32_t> bs((size_t)M * nb * 16);
    for (int m = 0; m < M; ++m) orc_quantize_q8_k(x + (size_t)m * K, K, q8.data() + (size_t)m * K, ad.data() + (size_t)m * nb, bs.data() + (size_t)m * nb * 16);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int kb = 0; kb < nb; ++kb) {
                const uint8_t* blk = w + ((size_t)n * nb + kb) * 144;
                float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
                float dmin = orc_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
                uint8_t sc[8], mn[8];
                orc_q4k_scales(blk + 4, sc, mn);
                const int8_t* a = q8.data() + (size_t)m * K + kb * 256;
                int32_t scale_accum = 0;
                for (int sb = 0; sb < 8; ++sb) {
                    const uint8_t* q = blk + 16 + (sb / 2) * 32;
                    int32_t isum = 0;
                    for (int l = 0; l < 32; ++l) isum += (int32_t)((sb & 1) ? (q[l] >> 4) : (q[l] & 0x0F)) * (int32_t)a[sb * 32 + l];
                    scale_accum += (int32_t)sc[sb] * isum;
                }
                int32_t min_accum = 0;
                for (int g = 0; g < 16; ++g) min_accum += (int32_t)mn[g / 2] * bs[((size_t)m * nb + kb) * 16 + g];
                float act_d = ad[(size_t)m * nb + kb];
                float scale_part = (d * act_d) * (float)scale_accum;
                float min_part = (dmin * act_d) * (float)min_accum;
                acc = acc + (scale_part - min_part);
            }
            y[(size_t)m * N + n] = acc;
        }
    }
}

ORC_API void orc_matmul_q6_k(const float* x, const uint8_t* w, int M, int K, int N, float* y) {
    int nb = K / 256;
    std::vector<int8_t> q8((size_t)M * K);
    std::vector<float> ad((size_t)M * nb);
    std::vector<int32_t> bs((size_t)M * nb * 16);
    for (int m = 0; m < M; ++m) orc_quantize_q8_k(x + (size_t)m * K, K, q8.data() + (size_t)m * K, ad.data() + (size_t)m * nb, bs.data() + (size_t)m * nb * 16);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int kb = 0; kb < nb; ++kb) {
                const uint8_t* blk = w + ((size_t)n * nb + kb) * 210;
                float d = orc_f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
                const int8_t* a = q8.data() + (size_t)m * K + kb * 256;
                int32_t scale_accum = 0;
                for (int sb = 0; sb < 16; ++sb) {
                    int32_t isum = 0;
                    for (int j = 0; j < 16; ++j) isum += orc_q6k_code(blk, sb * 16 + j) * (int32_t)a[sb * 16 + j];
                    scale_accum += (int32_t)(int8_t)blk[192 + sb] * isum;
                }
                acc = acc + (d * ad[(size_t)m * nb + kb]) * (float)scale_accum;
            }
            y[(size_t)m * N + n] = acc;
        }
    }
}

// ---------------------------------------------------------------------------------------
// KV cache  (src/runtime.rs:375-650)
// ---------------------------------------------------------------------------------------

struct OrcKv {
    int layers, heads, max_len, hd;
    int current_len = 0, new_tokens = 0;
    std::vector<std::vector<float>> key, value;  // per layer [heads, max_len, hd]
};

ORC_API OrcKv* orc_kv_new(int layers, int heads, int max_len, int hd) {
    OrcKv* c = new OrcKv();
    c->layers = layers;
    c->heads = heads;
    c->max_len = max_len;
    c->hd = hd;
    c->key.assign(layers, std::vector<float>((size_t)heads * max_len * hd, 0.0f));
    c->value.assign(layers, std::vector<float>((size_t)heads * max_len * hd, 0.0f));
    return c;
}
ORC_API void orc_kv_free(OrcKv* c) { delete c; }

// src/runtime.rs:521-538 / :545-570: new rows [heads, new_seq, hd] copied to
// (h*max_len + current_len)*hd.  Returns 0, or 1 when the cache is full (the reference panics).
static int kv_append(OrcKv* c, std::vector<float>& dst, const float* src, int new_seq) {
    if (c->current_len + new_seq > c->max_len) return 1;
    c->new_tokens = new_seq;
    for (int h = 0; h < c->heads; ++h) {
        size_t d = ((size_t)h * c->max_len + c->current_len) * c->hd;
        size_t s = (size_t)h * new_seq * c->hd;
        std::memcpy(dst.data() + d, src + s, sizeof(float) * (size_t)new_seq * c->hd);
    }
    return 0;
}
ORC_API int orc_kv_append_key(OrcKv* c, int layer, const float* k, int new_seq) {
    return kv_append(c, c->key[layer], k, new_seq);
}
ORC_API int orc_kv_append_value(OrcKv* c, int layer, const float* v, int new_seq) {
    return kv_append(c, c->value[layer], v, new_seq);
}
// src/runtime.rs:625-634
ORC_API void orc_kv_advance_by(OrcKv* c, int n) {
    c->current_len += n;
    c->new_tokens = 0;
}
// src/runtime.rs:638-640
ORC_API void orc_kv_reset(OrcKv* c, int initial_len) { c->current_len = initial_len; }
ORC_API int orc_kv_current_len(const OrcKv* c) { return c->current_len; }
// src/runtime.rs:463-507: contiguous copy of [heads, 0..current_len, hd].
ORC_API void orc_kv_view(const OrcKv* c, int layer, float* k_out, float* v_out) {
    int len = c->current_len;
    for (int h = 0; h < c->heads; ++h)
        for (int s = 0; s < len; ++s) {
            size_t src = ((size_t)h * c->max_len + s) * c->hd;
            size_t dst = ((size_t)h * len + s) * c->hd;
            std::memcpy(k_out + dst, c->key[layer].data() + src, sizeof(float) * c->hd);
            std::memcpy(v_out + dst, c->value[layer].data() + src, sizeof(float) * c->hd);
        }
}

// ---------------------------------------------------------------------------------------
// GQA attention  (src/hf/emitter.rs:683-758; emit_linalg.rs:93-245)
// ---------------------------------------------------------------------------------------

// q [S, heads, hd]; k,v strided views [kv_heads, T, hd] with head stride `kv_head_stride`
// (elements) and token stride hd; mask [S, T] additive; out [S, heads*hd].
// s[h,m,n] = sum_d q[h,m,d]*k[h/g,n,d] (d ascending FMA); *scale; +mask; softmax;
// o[h,m,d] = sum_n p[h,m,n]*v[h/g,n,d] (n ascending FMA).
ORC_API void orc_gqa_attention(const float* q, const float* k, const float* v, const float* mask, int S, int T,
                               int heads, int kv_heads, int hd, size_t kv_head_stride, int f64_softmax_sum,
                               float* out) {
    int g = heads / kv_heads;
    float scale = (float)(1.0 / std::sqrt((double)hd));
#pragma omp parallel for schedule(static)
    for (int h = 0; h < heads; ++h) {
        std::vector<float> sc(T), p(T);
        const float* kh = k + (size_t)(h / g) * kv_head_stride;
        const float* vh = v + (size_t)(h / g) * kv_head_stride;
        for (int m = 0; m < S; ++m) {
            const float* qv = q + ((size_t)m * heads + h) * hd;
            for (int n = 0; n < T; ++n) {
                float acc = 0.0f;
                const float* kr = kh + (size_t)n * hd;
                for (int d = 0; d < hd; ++d) acc = std::fma(qv[d], kr[d], acc);
                float s = acc * scale;
                sc[n] = s + mask[(size_t)m * T + n];
            }
            orc_softmax(sc.data(), 1, T, f64_softmax_sum, p.data());
            float* o = out + ((size_t)m * heads + h) * hd;
            for (int d = 0; d < hd; ++d) o[d] = 0.0f;
            for (int n = 0; n < T; ++n) {
                float pv = p[n];
                const float* vr = vh + (size_t)n * hd;
                for (int d = 0; d < hd; ++d) o[d] = std::fma(pv, vr[d], o[d]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Sampler  (src/generate.rs)
// ---------------------------------------------------------------------------------------

// src/generate.rs:457-468 / :734-742: Iterator::max_by(partial_cmp, Equal on NaN) returns
// the LAST maximal element, so ties resolve to the highest index.
ORC_API uint32_t orc_argmax(const float* logits, int n) {
    if (n <= 0) return 0;
    int best = 0;
    for (int i = 1; i < n; ++i) {
        // max_by keeps `best` only when best > candidate (Ordering::Greater).
        if (!(logits[best] > logits[i])) best = i;
    }
    return (uint32_t)best;
}

// src/generate.rs:610-642: xorshift64 (13,7,17), seed|1, (state>>40)/2^24.
ORC_API uint64_t orc_rng_new(uint64_t seed) { return seed | 1ull; }
ORC_API float orc_rng_next_f32(uint64_t* state) {
    uint64_t s = *state;
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    *state = s;
    return (float)(s >> 40) / (float)(1ull << 24);
}

struct OrcSampling {
    float temperature, top_p, min_p, repetition_penalty, frequency_penalty, presence_penalty;
    int32_t top_k;
};

// src/generate.rs:698-801.  The reference sorts candidates with sort_unstable_by; equal
// probabilities may order differently here (std::stable_sort by descending probability).
ORC_API uint32_t orc_sample_token(const float* logits_in, int n, const OrcSampling* cfg, const uint32_t* generated,
                                  int ngen, uint64_t* rng_state) {
    std::vector<float> logits(logits_in, logits_in + n);
    if (cfg->repetition_penalty != 1.0f) {
        for (int i = 0; i < ngen; ++i) {
            size_t idx = generated[i];
            if (idx < (size_t)n) {
                if (logits[idx] > 0.0f)
                    logits[idx] /= cfg->repetition_penalty;
                else
                    logits[idx] *= cfg->repetition_penalty;
            }
        }
    }
    if (cfg->frequency_penalty != 0.0f || cfg->presence_penalty != 0.0f) {
        std::map<size_t, size_t> counts;
        for (int i = 0; i < ngen; ++i) counts[generated[i]] += 1;
        for (auto& kv : counts) {
            if (kv.first < (size_t)n) {
                logits[kv.first] -= cfg->frequency_penalty * (float)kv.second;
                logits[kv.first] -= cfg->presence_penalty;
            }
        }
    }
    if (cfg->temperature <= 0.0f) return orc_argmax(logits.data(), n);
    float inv_temp = 1.0f / cfg->temperature;
    for (auto& l : logits) l *= inv_temp;
    float mx = -std::numeric_limits<float>::infinity();
    for (float l : logits) mx = std::max(mx, l);
    std::vector<float> probs(n);
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) {
        probs[i] = std::exp(logits[i] - mx);
        sum += probs[i];
    }
    for (auto& p : probs) p /= sum;
    if (cfg->min_p > 0.0f) {
        float maxp = 0.0f;
        for (float p : probs) maxp = std::max(maxp, p);
        float thr = cfg->min_p * maxp;
        for (auto& p : probs)
            if (p < thr) p = 0.0f;
    }
    std::vector<std::pair<int, float>> idx(n);
    for (int i = 0; i < n; ++i) idx[i] = {i, probs[i]};
    std::stable_sort(idx.begin(), idx.end(),
                     [](const std::pair<int, float>& a, const std::pair<int, float>& b) { return a.second > b.second; });
    if (cfg->top_k > 0 && cfg->top_k < n) idx.resize(cfg->top_k);
    float cumulative = 0.0f;
    size_t cutoff = idx.size();
    for (size_t i = 0; i < idx.size(); ++i) {
        cumulative += idx[i].second;
        if (cumulative >= cfg->top_p) {
            cutoff = i + 1;
            break;
        }
    }
    float total = 0.0f;
    for (size_t i = 0; i < cutoff; ++i) total += idx[i].second;
    float r = orc_rng_next_f32(rng_state) * total;
    float accum = 0.0f;
    for (size_t i = 0; i < cutoff; ++i) {
        accum += idx[i].second;
        if (accum >= r) return (uint32_t)idx[i].first;
    }
    return cutoff ? (uint32_t)idx[cutoff - 1].first : 0u;
}

// ---------------------------------------------------------------------------------------
// Whole model: HfModel::{run, run_kv} (src/hf/model.rs:165-218) over the plans of
// src/hf/emitter.rs:902-1014 (bf16/f32 weights) and src/hf/emitter_quant.rs:1207-1440
// (GGUF block-quantised weights).
// ---------------------------------------------------------------------------------------

struct OrcConfig {
    int32_t hidden_size, intermediate_size, num_attention_heads, num_hidden_layers, num_key_value_heads, vocab_size,
        max_position_embeddings, head_dim, tie_word_embeddings;
    double rms_norm_eps, rope_theta;
};

enum { ORC_F32 = 0, ORC_BF16 = 1, ORC_F16 = 2, ORC_Q8_0 = 3, ORC_Q4_0 = 4, ORC_Q4_K = 5, ORC_Q6_K = 6 };

struct Linear {
    int K = 0, N = 0, kind = -1;
    std::vector<float> f32;      // [K,N]
    std::vector<uint16_t> bf16;  // [K,N]
    std::vector<uint8_t> q;      // GGUF blocks [N, K/32]
    void apply(const float* x, int M, float* y) const {
        switch (kind) {
            case ORC_F32: orc_matmul_f32(x, f32.data(), M, K, N, y); break;
            case ORC_BF16: orc_matmul_bf16(x, bf16.data(), M, K, N, y); break;
            case ORC_Q8_0: orc_matmul_q8_0(x, q.data(), M, K, N, y); break;
            case ORC_Q4_0: orc_matmul_q4_0(x, q.data(), M, K, N, y); break;
            case ORC_Q4_K: orc_matmul_q4_k(x, q.data(), M, K, N, y); break;
            case ORC_Q6_K: orc_matmul_q6_k(x, q.data(), M, K, N, y); break;
            default: std::fprintf(stderr, "oracle: linear not loaded\n"); std::abort();
        }
    }
};

struct Layer {
    std::vector<float> in_ln, post_ln, qb, kb, vb, qn, kn;
    Linear q, k, v, o, gate, up, down;
};

struct OrcModel {
    OrcConfig cfg;
    int heads, kvh, hd, g, qdim, kvdim;
    bool quant = false, has_bias = false, has_qk_norm = false;
    std::vector<float> embed;  // [V,H] f32 (src/hf/weights.rs:284-292: gather table is always f32)
    std::vector<float> final_norm;
    std::vector<Layer> layers;
    Linear lm_head;
    bool lm_head_loaded = false;
    std::vector<float> rope_cos, rope_sin;
    OrcKv* kv = nullptr;
    int max_seq_len = 0;
    int keep_bf16 = 1;
    std::string err;
};

ORC_API OrcModel* orc_model_new(const OrcConfig* cfg, int keep_bf16) {
    OrcModel* m = new OrcModel();
    m->cfg = *cfg;
    m->heads = cfg->num_attention_heads;
    m->kvh = cfg->num_key_value_heads > 0 ? cfg->num_key_value_heads : cfg->num_attention_heads;
    m->hd = cfg->head_dim > 0 ? cfg->head_dim : cfg->hidden_size / cfg->num_attention_heads;
    m->g = m->heads / m->kvh;
    m->qdim = m->heads * m->hd;
    m->kvdim = m->kvh * m->hd;
    m->keep_bf16 = keep_bf16;
    m->layers.resize(cfg->num_hidden_layers);
    // src/hf/model.rs:132-136: table over max_position_embeddings.
    m->rope_cos.resize((size_t)cfg->max_position_embeddings * m->hd);
    m->rope_sin.resize((size_t)cfg->max_position_embeddings * m->hd);
    orc_rope_table(m->hd, cfg->max_position_embeddings, cfg->rope_theta, m->rope_cos.data(), m->rope_sin.data());
    return m;
}

ORC_API void orc_model_free(OrcModel* m) {
    if (!m) return;
    if (m->kv) orc_kv_free(m->kv);
    delete m;
}

static void to_f32(const void* data, int dtype, size_t n, std::vector<float>& out) {
    out.resize(n);
    if (dtype == ORC_F32) {
        std::memcpy(out.data(), data, n * 4);
    } else if (dtype == ORC_BF16) {
        const uint16_t* p = (const uint16_t*)data;
        for (size_t i = 0; i < n; ++i) out[i] = orc_bf16_to_f32(p[i]);
    } else if (dtype == ORC_F16) {
        const uint16_t* p = (const uint16_t*)data;
        for (size_t i = 0; i < n; ++i) out[i] = orc_f16_to_f32(p[i]);
    } else if (dtype == ORC_Q8_0) {
        orc_dequant_q8_0((const uint8_t*)data, n / 32, out.data());
    } else if (dtype == ORC_Q4_0) {
        orc_dequant_q4_0((const uint8_t*)data, n / 32, out.data());
    } else if (dtype == ORC_Q4_K) {
        orc_dequant_q4_k((const uint8_t*)data, n / 256, out.data());
    } else if (dtype == ORC_Q6_K) {
        orc_dequant_q6_k((const uint8_t*)data, n / 256, out.data());
    }
}

// Linear from an HF tensor [out,in]: transposed to [in,out] at load (src/hf/weights.rs:304-381);
// bf16 is kept when keep_bf16, else widened to f32 (src/hf/safetensors.rs:76-82).
static void set_linear_hf(Linear& L, const void* data, int dtype, int out_f, int in_f, int keep_bf16) {
    L.K = in_f;
    L.N = out_f;
    if (dtype == ORC_BF16 && keep_bf16) {
        L.kind = ORC_BF16;
        L.bf16.resize((size_t)in_f * out_f);
        const uint16_t* p = (const uint16_t*)data;
        for (int r = 0; r < out_f; ++r)
            for (int c = 0; c < in_f; ++c) L.bf16[(size_t)c * out_f + r] = p[(size_t)r * in_f + c];
    } else {
        std::vector<float> tmp;
        to_f32(data, dtype, (size_t)in_f * out_f, tmp);
        L.kind = ORC_F32;
        L.f32.resize(tmp.size());
        for (int r = 0; r < out_f; ++r)
            for (int c = 0; c < in_f; ++c) L.f32[(size_t)c * out_f + r] = tmp[(size_t)r * in_f + c];
    }
}

// Linear from GGUF raw blocks [out, in/32] kept as-is (src/gguf.rs:594-612, weights.rs:190-194).
static void set_linear_gguf(Linear& L, const void* data, int dtype, int out_f, int in_f) {
    L.K = in_f;
    L.N = out_f;
    L.kind = dtype;
    size_t bytes = dtype == ORC_Q4_K   ? (size_t)out_f * (in_f / 256) * 144
                   : dtype == ORC_Q6_K ? (size_t)out_f * (in_f / 256) * 210
                                       : (size_t)out_f * (in_f / 32) * (dtype == ORC_Q8_0 ? 34 : 18);
    L.q.assign((const uint8_t*)data, (const uint8_t*)data + bytes);
}

static bool parse_layer(const std::string& name, const char* prefix, int* layer, std::string* rest) {
    size_t pl = std::strlen(prefix);
    if (name.compare(0, pl, prefix) != 0) return false;
    size_t dot = name.find('.', pl);
    if (dot == std::string::npos) return false;
    *layer = std::atoi(name.substr(pl, dot - pl).c_str());
    *rest = name.substr(dot + 1);
    return true;
}

// Accepts HF safetensors names (src/hf/weights.rs:267-417) and GGUF names
// (src/gguf.rs:589-708).  shape is outermost-first.  Returns 0 on success.
ORC_API int orc_model_set_tensor(OrcModel* m, const char* cname, int dtype, const int64_t* shape, int ndim,
                                 const void* data) {
    std::string name(cname);
    size_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= (size_t)shape[i];
    int layer;
    std::string rest;
    const int H = m->cfg.hidden_size;
    if (name == "model.embed_tokens.weight" || name == "token_embd.weight") {
        to_f32(data, dtype, n, m->embed);
        return 0;
    }
    if (name == "model.norm.weight" || name == "output_norm.weight") {
        to_f32(data, dtype, n, m->final_norm);
        return 0;
    }
    if (name == "lm_head.weight") {
        set_linear_hf(m->lm_head, data, dtype, (int)shape[0], (int)shape[1], m->keep_bf16);
        m->lm_head_loaded = true;
        return 0;
    }
    if (name == "output.weight") {
        // src/gguf.rs:695-700: always dequantised to f32; transposed to [hidden, vocab]
        // (src/hf/weights.rs:176-180).
        set_linear_hf(m->lm_head, data, dtype, (int)shape[0], (int)shape[1], 0);
        m->lm_head_loaded = true;
        m->quant = true;
        return 0;
    }
    if (parse_layer(name, "model.layers.", &layer, &rest)) {
        if (layer < 0 || layer >= (int)m->layers.size()) return 2;
        Layer& L = m->layers[layer];
        if (rest == "input_layernorm.weight") to_f32(data, dtype, n, L.in_ln);
        else if (rest == "post_attention_layernorm.weight") to_f32(data, dtype, n, L.post_ln);
        else if (rest == "self_attn.q_proj.weight") set_linear_hf(L.q, data, dtype, (int)shape[0], (int)shape[1], m->keep_bf16);
        else if (rest == "self_attn.k_proj.weight") set_linear_hf(L.k, data, dtype, (int)shape[0], (int)shape[1], m->keep_bf16);
        else if (rest == "self_attn.v_proj.weight") set_linear_hf(L.v, data, dtype, (int)shape[0], (int)shape[1], m->keep_bf16);
        else if (rest == "self_attn.o_proj.weight") set_linear_hf(L.o, data, dtype, (int)shape[0], (int)shape[1], m->keep_bf16);
        else if (rest == "mlp.gate_proj.weight") set_linear_hf(L.gate, data, dtype, (int)shape[0], (int)shape[1], m->keep_bf16);
        else if (rest == "mlp.up_proj.weight") set_linear_hf(L.up, data, dtype, (int)shape[0], (int)shape[1], m->keep_bf16);
        else if (rest == "mlp.down_proj.weight") set_linear_hf(L.down, data, dtype, (int)shape[0], (int)shape[1], m->keep_bf16);
        else if (rest == "self_attn.q_proj.bias") { to_f32(data, dtype, n, L.qb); m->has_bias = true; }
        else if (rest == "self_attn.k_proj.bias") to_f32(data, dtype, n, L.kb);
        else if (rest == "self_attn.v_proj.bias") to_f32(data, dtype, n, L.vb);
        else if (rest == "self_attn.q_norm.weight") { to_f32(data, dtype, n, L.qn); m->has_qk_norm = true; }
        else if (rest == "self_attn.k_norm.weight") to_f32(data, dtype, n, L.kn);
        else return 3;
        return 0;
    }
    if (parse_layer(name, "blk.", &layer, &rest)) {
        if (layer < 0 || layer >= (int)m->layers.size()) return 2;
        Layer& L = m->layers[layer];
        auto lin = [&](Linear& dst) {
            if (dtype == ORC_Q8_0 || dtype == ORC_Q4_0 || dtype == ORC_Q4_K || dtype == ORC_Q6_K) {
                set_linear_gguf(dst, data, dtype, (int)shape[0], (int)shape[1]);
                m->quant = true;
            } else {
                set_linear_hf(dst, data, dtype, (int)shape[0], (int)shape[1], m->keep_bf16);
            }
        };
        if (rest == "attn_norm.weight") to_f32(data, dtype, n, L.in_ln);
        else if (rest == "ffn_norm.weight") to_f32(data, dtype, n, L.post_ln);
        else if (rest == "attn_q.weight") lin(L.q);
        else if (rest == "attn_k.weight") lin(L.k);
        else if (rest == "attn_v.weight") lin(L.v);
        else if (rest == "attn_output.weight") lin(L.o);
        else if (rest == "ffn_gate.weight") lin(L.gate);
        else if (rest == "ffn_up.weight") lin(L.up);
        else if (rest == "ffn_down.weight") lin(L.down);
        else if (rest == "attn_q.bias") { to_f32(data, dtype, n, L.qb); m->has_bias = true; }
        else if (rest == "attn_k.bias") to_f32(data, dtype, n, L.kb);
        else if (rest == "attn_v.bias") to_f32(data, dtype, n, L.vb);
        else if (rest == "attn_q_norm.weight") { to_f32(data, dtype, n, L.qn); m->has_qk_norm = true; }
        else if (rest == "attn_k_norm.weight") to_f32(data, dtype, n, L.kn);
        else return 3;
        return 0;
    }
    (void)H;
    return 1;
}

// Tied LM head: transposed embedding, truncated to bf16 when projection weights are bf16
// (src/hf/weights.rs:101-113); f32 transposed copy on the quant path (weights.rs:176-180).
ORC_API int orc_model_finalize(OrcModel* m) {
    const int H = m->cfg.hidden_size, V = m->cfg.vocab_size;
    if (m->embed.size() != (size_t)V * H) return 1;
    if (!m->lm_head_loaded) {
        bool bf16 = !m->quant && m->layers[0].q.kind == ORC_BF16;
        m->lm_head.K = H;
        m->lm_head.N = V;
        if (bf16) {
            m->lm_head.kind = ORC_BF16;
            m->lm_head.bf16.resize((size_t)H * V);
            for (int v = 0; v < V; ++v)
                for (int h = 0; h < H; ++h)
                    m->lm_head.bf16[(size_t)h * V + v] = orc_f32_to_bf16_trunc(m->embed[(size_t)v * H + h]);
        } else {
            m->lm_head.kind = ORC_F32;
            m->lm_head.f32.resize((size_t)H * V);
            for (int v = 0; v < V; ++v)
                for (int h = 0; h < H; ++h) m->lm_head.f32[(size_t)h * V + v] = m->embed[(size_t)v * H + h];
        }
        m->lm_head_loaded = true;
    }
    return 0;
}

ORC_API void orc_model_reset(OrcModel* m) {
    if (m->kv) orc_kv_reset(m->kv, 0);
}
ORC_API int orc_model_kv_len(const OrcModel* m) { return m->kv ? m->kv->current_len : 0; }

// One pass over S new tokens with the persistent cache (ExecutionPlan::run_kv,
// src/runtime.rs:1580-1892; prefill with an empty cache is the same arithmetic,
// src/hf/model.rs:165-193 + src/runtime.rs:1898-1938).  logits_out: [S, V] when all_logits,
// else [V] for the last position.
static int forward(OrcModel* m, const int64_t* ids, int S, int max_seq_len, float* logits_out, int all_logits) {
    const OrcConfig& c = m->cfg;
    const int H = c.hidden_size, I = c.intermediate_size, V = c.vocab_size;
    const int heads = m->heads, kvh = m->kvh, hd = m->hd;
    const float eps = (float)c.rms_norm_eps;
    if (!m->kv) {
        m->kv = orc_kv_new(c.num_hidden_layers, kvh, max_seq_len, hd);
        m->max_seq_len = max_seq_len;
    }
    int past = m->kv->current_len;
    if (past + S > m->kv->max_len) return 3;  // "KV cache full" (src/runtime.rs:523-529)
    int T = past + S;
    for (int s = 0; s < S; ++s)
        if (ids[s] < 0 || ids[s] >= V) return 4;

    std::vector<float> h((size_t)S * H), normed((size_t)S * H), q((size_t)S * m->qdim), k((size_t)S * m->kvdim),
        v((size_t)S * m->kvdim), kt((size_t)S * m->kvdim), vt((size_t)S * m->kvdim), attn((size_t)S * m->qdim),
        attn_o((size_t)S * H), resid((size_t)S * H), gate((size_t)S * I), up((size_t)S * I), act((size_t)S * I),
        down((size_t)S * H), mask((size_t)S * T);
    // Embed (src/hf/emitter.rs:506-537): row gather from the f32 table.
    for (int s = 0; s < S; ++s) std::memcpy(&h[(size_t)s * H], &m->embed[(size_t)ids[s] * H], sizeof(float) * H);
    orc_causal_mask(S, past, mask.data());
    const float* cosr = m->rope_cos.data() + (size_t)past * hd;  // src/hf/precompute.rs:73-101
    const float* sinr = m->rope_sin.data() + (size_t)past * hd;

    for (int li = 0; li < c.num_hidden_layers; ++li) {
        Layer& L = m->layers[li];
        // --- QKV + RoPE (src/hf/emitter.rs:549-673 | quant: emitter_quant.rs:713-791, 800-905)
        if (m->quant)
            orc_rms_norm_quant_kernel(h.data(), L.in_ln.data(), eps, S, H, normed.data());
        else
            orc_rms_norm(h.data(), L.in_ln.data(), eps, S, H, normed.data());
        L.q.apply(normed.data(), S, q.data());
        L.k.apply(normed.data(), S, k.data());
        L.v.apply(normed.data(), S, v.data());
        if (m->has_bias) {
            for (int s = 0; s < S; ++s) {
                for (int i = 0; i < m->qdim; ++i) q[(size_t)s * m->qdim + i] += L.qb[i];
                for (int i = 0; i < m->kvdim; ++i) k[(size_t)s * m->kvdim + i] += L.kb[i];
                for (int i = 0; i < m->kvdim; ++i) v[(size_t)s * m->kvdim + i] += L.vb[i];
            }
        }
        if (m->has_qk_norm) {
            if (m->quant) {
                orc_rms_norm_f64_accum(q.data(), L.qn.data(), eps, S * heads, hd, q.data());
                orc_rms_norm_f64_accum(k.data(), L.kn.data(), eps, S * kvh, hd, k.data());
            } else {
                orc_rms_norm(q.data(), L.qn.data(), eps, S * heads, hd, q.data());
                orc_rms_norm(k.data(), L.kn.data(), eps, S * kvh, hd, k.data());
            }
        }
        orc_rope_half(q.data(), S, heads, hd, cosr, sinr);
        orc_rope_half(k.data(), S, kvh, hd, cosr, sinr);
        // BSHD -> BHSD for the cache concat (src/hf/emitter.rs:646-649).
        for (int s = 0; s < S; ++s)
            for (int hh = 0; hh < kvh; ++hh) {
                std::memcpy(&kt[((size_t)hh * S + s) * hd], &k[((size_t)s * kvh + hh) * hd], sizeof(float) * hd);
                std::memcpy(&vt[((size_t)hh * S + s) * hd], &v[((size_t)s * kvh + hh) * hd], sizeof(float) * hd);
            }
        // --- native KV concat intercepted by the cache (src/runtime.rs:1729-1755).
        orc_kv_append_key(m->kv, li, kt.data(), S);
        orc_kv_append_value(m->kv, li, vt.data(), S);
        // --- attention + O projection (src/hf/emitter.rs:683-758 | quant: emitter_quant.rs:915-975)
        orc_gqa_attention(q.data(), m->kv->key[li].data(), m->kv->value[li].data(), mask.data(), S, T, heads, kvh, hd,
                          (size_t)m->kv->max_len * hd, m->quant ? 1 : 0, attn.data());
        L.o.apply(attn.data(), S, attn_o.data());
        // --- residual + norm + SwiGLU + residual (src/hf/emitter.rs:767-822 | quant :985-1134)
        for (size_t i = 0; i < (size_t)S * H; ++i) resid[i] = h[i] + attn_o[i];
        if (m->quant)
            orc_rms_norm_quant_kernel(resid.data(), L.post_ln.data(), eps, S, H, normed.data());
        else
            orc_rms_norm(resid.data(), L.post_ln.data(), eps, S, H, normed.data());
        L.gate.apply(normed.data(), S, gate.data());
        L.up.apply(normed.data(), S, up.data());
        orc_silu(gate.data(), S * I, act.data());
        for (size_t i = 0; i < (size_t)S * I; ++i) act[i] = act[i] * up[i];
        L.down.apply(act.data(), S, down.data());
        for (size_t i = 0; i < (size_t)S * H; ++i) h[i] = resid[i] + down[i];
    }
    orc_kv_advance_by(m->kv, S);  // src/runtime.rs:1875-1880

    // --- final norm + LM head (src/hf/emitter.rs:828-862 | quant: emitter_quant.rs:1399-1440)
    int first = all_logits ? 0 : S - 1;
    int rows = S - first;
    std::vector<float> fin((size_t)rows * H);
    if (m->quant)
        orc_rms_norm_f64_accum(&h[(size_t)first * H], m->final_norm.data(), eps, rows, H, fin.data());
    else
        orc_rms_norm(&h[(size_t)first * H], m->final_norm.data(), eps, rows, H, fin.data());
    m->lm_head.apply(fin.data(), rows, logits_out);
    return 0;
}

// GenerativeModel::prefill (src/hf/model.rs:314-357): returns argmax at the last position.
ORC_API int orc_model_prefill(OrcModel* m, const int64_t* ids, int n, int max_seq_len, float* logits_last,
                              uint32_t* first_token) {
    std::vector<float> tmp;
    float* lo = logits_last;
    if (!lo) {
        tmp.resize(m->cfg.vocab_size);
        lo = tmp.data();
    }
    int rc = forward(m, ids, n, max_seq_len, lo, 0);
    if (rc) return rc;
    if (first_token) *first_token = orc_argmax(lo, m->cfg.vocab_size);
    return 0;
}

// GenerativeModel::decode_step (src/hf/model.rs:359-371): logits for one new token.
ORC_API int orc_model_decode_step(OrcModel* m, uint32_t token, float* logits) {
    int64_t id = (int64_t)token;
    return forward(m, &id, 1, m->max_seq_len, logits, 0);
}

// Multi-token run_kv returning logits for every new position (chat-delta prefill path,
// src/hf/model.rs:321-336); used to check batched / chunked GPU evaluation.
ORC_API int orc_model_forward_all(OrcModel* m, const int64_t* ids, int n, int max_seq_len, float* logits_all) {
    return forward(m, ids, n, max_seq_len, logits_all, 1);
}

// Read one layer's cache as the contiguous view [kv_heads, current_len, hd].
ORC_API int orc_model_kv_view(const OrcModel* m, int layer, float* k_out, float* v_out) {
    if (!m->kv) return 1;
    orc_kv_view(m->kv, layer, k_out, v_out);
    return 0;
}

ORC_API int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
