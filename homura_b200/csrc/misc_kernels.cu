// Small kernels around the projections: weight re-layout at load, embedding gather, argmax
// finish, standalone RMSNorm / QK-norm+RoPE, KV row access and dtype conversion.
#include "common.cuh"
#include "mbarrier.cuh"

namespace hm {
namespace {

// ---- weight re-layout -------------------------------------------------------------------
// Homura transposes every HF linear [out,in] to [in,out] at load (src/hf/weights.rs:304-381);
// the engine goes one step further and stores [in,out] in 128-column slabs,
// dst[slab][k][c] = W[n = slab*128 + c][k], so a CTA's share of a projection is one
// contiguous byte range.  Tile-transposed through shared memory: reads run along k,
// writes along c.
// interleave_which >= 0 selects the gate/up interleave: output j of gate (which = 0) or up
// (which = 1) lands in column (j/64)*128 + which*64 + j%64, so one slab holds 64 gate columns
// followed by the 64 matching up columns and the SwiGLU epilogue finds both in one CTA.
__global__ void pack_from_nk_kernel(const uint16_t* __restrict__ src, int N, int K, uint16_t* __restrict__ dst, int n_off, int interleave_which) {
    __shared__ uint16_t tile[32][33];
    const int n0 = blockIdx.y * 32, k0 = blockIdx.x * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int n = n0 + r, k = k0 + threadIdx.x;
        tile[r][threadIdx.x] = (n < N && k < K) ? src[(size_t)n * K + k] : (uint16_t)0;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int k = k0 + r, n = n0 + threadIdx.x;
        if (k < K && n < N) {
            const int no = interleave_which >= 0 ? (n / 64) * SLAB + interleave_which * 64 + (n % 64) : n + n_off;
            dst[((size_t)(no / SLAB) * K + k) * SLAB + (no % SLAB)] = tile[threadIdx.x][r];
        }
    }
}

__global__ void pack_from_kn_kernel(const uint16_t* __restrict__ src, int K, int N, uint16_t* __restrict__ dst) {
    const int nslabs = (N + SLAB - 1) / SLAB;
    const size_t total = (size_t)nslabs * K * SLAB;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % SLAB);
        const size_t r = i / SLAB;
        const int k = (int)(r % K);
        const int s = (int)(r / K);
        const int n = s * SLAB + c;
        dst[i] = n < N ? src[(size_t)k * N + n] : (uint16_t)0;
    }
}

// ---- embedding gather (src/hf/emitter.rs:506-537): hidden[m] = f32(table[token[m]]) -------
__global__ void embed_gather_kernel(const void* table, int dtype, const uint32_t* tokens, int H, int V, float* out, int* err_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    const uint32_t tok = tokens[m];
    if (tok >= (uint32_t)V) {
        if (threadIdx.x == 0 && err_flag) atomicExch(err_flag, 1);
        for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)m * H + i] = 0.f;
        return;
    }
    if (dtype == 1) {  // bf16 rows
        const uint16_t* row = reinterpret_cast<const uint16_t*>(table) + (size_t)tok * H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)m * H + i] = bf16_bits_to_f32(row[i]);
    } else {
        const float* row = reinterpret_cast<const float*>(table) + (size_t)tok * H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)m * H + i] = row[i];
    }
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i > bi); }

// ---- argmax finish: merge per-slab (value, index) pairs; ties go to the highest index ----
// (Iterator::max_by returns the last maximum, src/generate.rs:457-468).  Also feeds the token
// back as the next step's input, appends it to the sequence history and advances the
// sequence position (KvCache::advance_by, src/runtime.rs:1875-1880).
__global__ void argmax_finish_kernel(const float* amax_val, const int32_t* amax_idx, int nslabs, uint32_t* next_tok, uint32_t* feed_tok, int32_t* pos, uint32_t* hist, int hist_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    float bv = -INFINITY;
    int bi = -1;
    const float* row = amax_val + (size_t)m * nslabs;
    int done = 0;
    if (!amax_idx && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        // plain logits: 16-byte loads, four in flight per thread (a scalar loop pays one L2 round trip per element)
        const int n4 = nslabs >> 2;
        for (int b = threadIdx.x; b < n4; b += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = b + u * blockDim.x;
                v[u] = idx < n4 ? *reinterpret_cast<const float4*>(row + 4 * (size_t)idx) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = b + u * blockDim.x;
                if (idx < n4) {
                    const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (bi < 0 || better(e[k], 4 * idx + k, bv, bi)) { bv = e[k]; bi = 4 * idx + k; }
                }
            }
        }
        done = n4 << 2;
    }
    for (int s = done + threadIdx.x; s < nslabs; s += blockDim.x) {
        const float v = row[s];
        const int i = amax_idx ? amax_idx[(size_t)m * nslabs + s] : s;
        if (i >= 0 && (bi < 0 || better(v, i, bv, bi))) { bv = v; bi = i; }
    }
    __shared__ float sv[32];
    __shared__ int si[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            const uint32_t tok = bi < 0 ? 0u : (uint32_t)bi;
            next_tok[m] = tok;
            if (feed_tok) feed_tok[m] = tok;
            if (pos) {
                const int np = pos[m] + 1;
                pos[m] = np;
                if (hist) hist[(size_t)m * hist_stride + np] = tok;
            }
        }
    }
}

__global__ void argmax_rows_kernel(const float* logits, int n, uint32_t* out) {
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * n;
    float bv = -INFINITY;
    int bi = -1;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = row[i];
        if (bi < 0 || better(v, i, bv, bi)) { bv = v; bi = i; }
    }
    __shared__ float sv[32];
    __shared__ int si[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
        }
        if (lane == 0) out[r] = bi < 0 ? 0u : (uint32_t)bi;
    }
}

// ---- standalone RMSNorm (src/graph_builder/emit_linalg.rs:7-26) ---------------------------
__global__ void rms_norm_kernel(const float* x, const float* w, float eps, int n, float* out) {
    const int r = blockIdx.x;
    const float* xr = x + (size_t)r * n;
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s = fmaf(xr[i], xr[i], s);
    __shared__ float sw[32];
    __shared__ float s_inv;
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) sw[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += sw[i];
        s_inv = 1.0f / sqrtf(t / (float)n + eps);
    }
    __syncthreads();
    const float inv = s_inv;
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[(size_t)r * n + i] = (xr[i] * inv) * w[i];
}

// ---- standalone per-head QK-norm + RoPE half rotation (src/hf/emitter.rs:629-644) ---------
// One warp per (row, head); x [rows][heads][hd] in place; cos/sin rows [rows][hd].
__global__ void qknorm_rope_kernel(float* x, int rows, int heads, int hd, const float* norm_w, float eps, const float* cos_rows, const float* sin_rows) {
    const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (wid >= rows * heads) return;
    const int r = wid / heads;
    float* v = x + (size_t)wid * hd;
    const int per = hd / 32;  // hd in {64, 128}
    float val[4], oth[4];
    float s = 0.f;
    for (int e = 0; e < per; ++e) {
        val[e] = v[lane + 32 * e];
        s = fmaf(val[e], val[e], s);
    }
    if (norm_w) {
        s = warp_sum(s);
        const float inv = 1.0f / sqrtf(s / (float)hd + eps);
        for (int e = 0; e < per; ++e) val[e] = (val[e] * inv) * norm_w[lane + 32 * e];
    }
    const int half = hd / 2;
    // element d = lane + 32e pairs with d +- half, which lives in another register of the same
    // lane: (lane + 32e + half) % hd = lane + 32*((e + per/2) % per)
    for (int e = 0; e < per; ++e) {
        const int d = lane + 32 * e;
        const int eo = (e + per / 2) % per;
        oth[e] = d < half ? -val[eo] : val[eo];
    }
    for (int e = 0; e < per; ++e) {
        const int d = lane + 32 * e;
        v[d] = fmaf(oth[e], sin_rows[(size_t)r * hd + d], val[e] * cos_rows[(size_t)r * hd + d]);
    }
}

// ---- KV row access (KvCache::append_* / view, src/runtime.rs:463-570) ----------------------
__global__ void kv_write_rows_kernel(KvDesc kv, int seq, int pos0, const float* k_rows, const float* v_rows, int n_new) {
    const size_t total = (size_t)kv.kv_heads * n_new * kv.hd;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % kv.hd);
        const int s = (int)((i / kv.hd) % n_new);
        const int h = (int)(i / ((size_t)kv.hd * n_new));
        const int pos = pos0 + s;
        const int page = kv.page_table[(size_t)seq * kv.max_pages + pos / kv.page_tokens];
        const size_t tile = ((size_t)page * kv.kv_heads + h) * kv.page_tokens * kv.hd;
        const size_t ko = tile + k_tile_off(pos % kv.page_tokens, d), vo = tile + v_tile_off(pos % kv.page_tokens, d, kv.hd, kv.bf16);
        if (kv.bf16) {
            if (k_rows) reinterpret_cast<uint16_t*>(kv.k_pool)[ko] = f32_to_bf16_rne(k_rows[i]);
            if (v_rows) reinterpret_cast<uint16_t*>(kv.v_pool)[vo] = f32_to_bf16_rne(v_rows[i]);
        } else {
            if (k_rows) reinterpret_cast<float*>(kv.k_pool)[ko] = k_rows[i];
            if (v_rows) reinterpret_cast<float*>(kv.v_pool)[vo] = v_rows[i];
        }
    }
}

__global__ void kv_read_rows_kernel(KvDesc kv, int seq, int len, float* k_out, float* v_out) {
    const size_t total = (size_t)kv.kv_heads * len * kv.hd;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % kv.hd);
        const int pos = (int)((i / kv.hd) % len);
        const int h = (int)(i / ((size_t)kv.hd * len));
        const int page = kv.page_table[(size_t)seq * kv.max_pages + pos / kv.page_tokens];
        const size_t tile = ((size_t)page * kv.kv_heads + h) * kv.page_tokens * kv.hd;
        const size_t ko = tile + k_tile_off(pos % kv.page_tokens, d), vo = tile + v_tile_off(pos % kv.page_tokens, d, kv.hd, kv.bf16);
        if (kv.bf16) {
            k_out[i] = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(kv.k_pool)[ko]);
            v_out[i] = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(kv.v_pool)[vo]);
        } else {
            k_out[i] = reinterpret_cast<const float*>(kv.k_pool)[ko];
            v_out[i] = reinterpret_cast<const float*>(kv.v_pool)[vo];
        }
    }
}

// dtype codes follow hm_dtype: 0 f32, 1 bf16, 2 f16
__global__ void convert_to_f32_kernel(const void* src, int dtype, size_t n, float* dst) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        if (dtype == 0) dst[i] = reinterpret_cast<const float*>(src)[i];
        else if (dtype == 1) dst[i] = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(src)[i]);
        else dst[i] = f16_bits_to_f32(reinterpret_cast<const uint16_t*>(src)[i]);
    }
}

// ---- quant plan: PostQKV (src/hf/emitter_quant.rs:800-905) ---------------------------------
// qkv [M][q_dim + 2*kv_dim] already carries the bias.  One warp per (row, head): Q and K heads
// get the optional per-head RMSNorm (f64 sum of squares, emit_rms_norm_f64_accum) and the RoPE
// half rotation; Q goes to q_out, K and V go straight into the row's KV page slot.
__global__ void post_qkv_kernel(const float* qkv, int M, int heads, int kv_heads, int hd, int has_qk_norm, const float* q_norm_w, const float* k_norm_w, float eps,
                                const float* rope_cos, const float* rope_sin, const int32_t* row_pos, const int32_t* row_seq, KvDesc kv, float* q_out) {
    pdl_launch_dependents();
    pdl_wait();
    const int all = heads + 2 * kv_heads;
    const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (wid >= M * all) return;
    const int m = wid / all, h = wid % all;
    const int q_dim = heads * hd, kv_dim = kv_heads * hd;
    const float* v = qkv + (size_t)m * (q_dim + 2 * kv_dim) + (size_t)h * hd;
    const int per = hd / 32;
    const int pos = row_pos[m];
    float val[4], oth[4];
    for (int e = 0; e < per; ++e) val[e] = v[lane + 32 * e];
    const bool is_q = h < heads, is_k = !is_q && h < heads + kv_heads;
    if (is_q || is_k) {
        if (has_qk_norm) {
            double s = 0.0;
            for (int e = 0; e < per; ++e) s += (double)(val[e] * val[e]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            const float inv = 1.0f / sqrtf((float)(s / (double)hd) + eps);
            const float* nw = is_q ? q_norm_w : k_norm_w;
            for (int e = 0; e < per; ++e) val[e] = (val[e] * inv) * nw[lane + 32 * e];
        }
        const int half = hd / 2;
        for (int e = 0; e < per; ++e) {
            const int d = lane + 32 * e;
            const int eo = (e + per / 2) % per;
            oth[e] = d < half ? -val[eo] : val[eo];
        }
        for (int e = 0; e < per; ++e) {
            const int d = lane + 32 * e;
            val[e] = fmaf(oth[e], rope_sin[(size_t)pos * hd + d], val[e] * rope_cos[(size_t)pos * hd + d]);
        }
    }
    if (is_q) {
        for (int e = 0; e < per; ++e) q_out[(size_t)m * q_dim + (size_t)h * hd + lane + 32 * e] = val[e];
    } else {
        const int kvh = is_k ? h - heads : h - heads - kv_heads;
        const int seq = row_seq ? row_seq[m] : m;
        const int page = kv.page_table[(size_t)seq * kv.max_pages + pos / kv.page_tokens];
        const size_t tile = ((size_t)page * kv.kv_heads + kvh) * kv.page_tokens * hd;
        void* pool = is_k ? kv.k_pool : kv.v_pool;
        for (int e = 0; e < per; ++e) {
            const int d = lane + 32 * e;
            const size_t off = tile + (is_k ? k_tile_off(pos % kv.page_tokens, d) : v_tile_off(pos % kv.page_tokens, d, hd, kv.bf16));
            if (kv.bf16) reinterpret_cast<uint16_t*>(pool)[off] = f32_to_bf16_rne(val[e]);
            else reinterpret_cast<float*>(pool)[off] = val[e];
        }
    }
}

// ---- quant plan: SiLU(gate) * up (src/hf/emitter_quant.rs:1078-1099); gate_up [M][2I] ------
__global__ void silu_mul_kernel(const float* gate_up, int M, int I, float* act) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)M * I;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / I), j = (int)(i % I);
        const float g = gate_up[(size_t)m * 2 * I + j], u = gate_up[(size_t)m * 2 * I + I + j];
        act[i] = (g / (1.0f + expf(-g))) * u;
    }
}

inline unsigned grid_for(size_t n, int block) {
    size_t g = (n + block - 1) / block;
    return (unsigned)(g > 148u * 16u ? 148u * 16u : (g ? g : 1));
}

// hist[b][pos[b]] = tokens[b]: the token a host feeds into a decode step enters the sequence's history
// (the sampler's penalties count occurrences in it).
__global__ void hist_set_kernel(const uint32_t* tokens, const int32_t* pos, uint32_t* hist, int hist_stride, int batch) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch) hist[(size_t)b * hist_stride + pos[b]] = tokens[b];
}

// Self-test of the give-up path every bounded wait in this library takes.  One CTA: a real 16-byte bulk copy
// completes on barrier A (waited for, so nothing is in flight when the CTA returns); barrier B is armed for 16
// bytes that nobody sends, and its wait runs out after `limit` polls, raises the error word and returns.
__global__ void bounded_wait_probe_kernel(const void* src16, int* err_flag, unsigned long long limit, int* landed) {
    __shared__ __align__(16) unsigned char buf[16];
    __shared__ uint64_t bar_a, bar_b;
    __shared__ volatile int s_abort;
    if (threadIdx.x == 0) {
        mb_init(&bar_a, 1);
        mb_init(&bar_b, 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mb_expect_tx(&bar_a, 16);
        bulk_copy(buf, src16, 16, &bar_a);
        mb_expect_tx(&bar_b, 16);  // never completed
        const bool a_ok = mb_wait_limit(&bar_a, 0, nullptr, &s_abort, MB_SPIN_LIMIT);
        if (landed) *landed = a_ok ? 1 : 0;
        if (a_ok) mb_wait_limit(&bar_b, 0, err_flag, &s_abort, limit);
    }
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

}  // namespace

cudaError_t launch_pack_slabs_from_nk(const uint16_t* src_nk, int N, int K, uint16_t* dst, int n_off, int interleave_which, cudaStream_t st) {
    dim3 grid((K + 31) / 32, (N + 31) / 32), block(32, 8);
    pack_from_nk_kernel<<<grid, block, 0, st>>>(src_nk, N, K, dst, n_off, interleave_which);
    return cudaGetLastError();
}
cudaError_t launch_pack_slabs_from_kn(const uint16_t* src_kn, int K, int N, uint16_t* dst, cudaStream_t st) {
    const size_t total = (size_t)((N + SLAB - 1) / SLAB) * K * SLAB;
    pack_from_kn_kernel<<<grid_for(total, 256), 256, 0, st>>>(src_kn, K, N, dst);
    return cudaGetLastError();
}
cudaError_t launch_embed_gather(const void* table, int table_dtype, const uint32_t* tokens, int M, int H, int V, float* out, int* err_flag, cudaStream_t st, bool pdl) {
    return launch_pdl(embed_gather_kernel, dim3(M), dim3(256), st, pdl, table, table_dtype, tokens, H, V, out, err_flag);
}
cudaError_t launch_argmax_finish(const float* amax_val, const int32_t* amax_idx, int nslabs, int M, uint32_t* next_tok, uint32_t* feed_tok, int32_t* pos, uint32_t* hist, int hist_stride, cudaStream_t st, bool pdl) {
    return launch_pdl(argmax_finish_kernel, dim3(M), dim3(nslabs > 4096 ? 1024 : 256), st, pdl, amax_val, amax_idx, nslabs, next_tok, feed_tok, pos, hist, hist_stride);
}
cudaError_t launch_argmax_rows(const float* logits, int rows, int n, uint32_t* out, cudaStream_t st) {
    argmax_rows_kernel<<<rows, 1024, 0, st>>>(logits, n, out);
    return cudaGetLastError();
}
cudaError_t launch_rms_norm(const float* x, const float* w, float eps, int rows, int n, float* out, cudaStream_t st) {
    rms_norm_kernel<<<rows, 256, 0, st>>>(x, w, eps, n, out);
    return cudaGetLastError();
}
cudaError_t launch_qknorm_rope(float* x, int rows, int heads, int hd, const float* norm_w, float eps, const float* cos_rows, const float* sin_rows, cudaStream_t st) {
    if (hd != 64 && hd != 128) return cudaErrorInvalidValue;
    const int warps = rows * heads;
    qknorm_rope_kernel<<<(warps + 3) / 4, 128, 0, st>>>(x, rows, heads, hd, norm_w, eps, cos_rows, sin_rows);
    return cudaGetLastError();
}
cudaError_t launch_kv_write_rows(const KvDesc& kv, int seq, int pos0, const float* k_rows, const float* v_rows, int n_new, cudaStream_t st) {
    const size_t total = (size_t)kv.kv_heads * n_new * kv.hd;
    kv_write_rows_kernel<<<grid_for(total, 256), 256, 0, st>>>(kv, seq, pos0, k_rows, v_rows, n_new);
    return cudaGetLastError();
}
cudaError_t launch_kv_read_rows(const KvDesc& kv, int seq, int len, float* k_out, float* v_out, cudaStream_t st) {
    const size_t total = (size_t)kv.kv_heads * len * kv.hd;
    kv_read_rows_kernel<<<grid_for(total, 256), 256, 0, st>>>(kv, seq, len, k_out, v_out);
    return cudaGetLastError();
}
cudaError_t launch_convert_to_f32(const void* src, int dtype, size_t n, float* dst, cudaStream_t st) {
    convert_to_f32_kernel<<<grid_for(n, 256), 256, 0, st>>>(src, dtype, n, dst);
    return cudaGetLastError();
}

cudaError_t launch_post_qkv(const float* qkv, int M, int heads, int kv_heads, int hd, int has_qk_norm, const float* q_norm_w, const float* k_norm_w, float eps, const float* rope_cos, const float* rope_sin, const int32_t* row_pos, const int32_t* row_seq, const KvDesc& kv, float* q_out, cudaStream_t st, bool pdl) {
    if (hd != 64 && hd != 128) return cudaErrorInvalidValue;
    const int warps = M * (heads + 2 * kv_heads);
    return launch_pdl(post_qkv_kernel, dim3((warps + 3) / 4), dim3(128), st, pdl, qkv, M, heads, kv_heads, hd, has_qk_norm, q_norm_w, k_norm_w, eps, rope_cos, rope_sin, row_pos, row_seq, kv, q_out);
}
cudaError_t launch_hist_set(const uint32_t* tokens, const int32_t* pos, uint32_t* hist, int hist_stride, int batch, cudaStream_t st) {
    hist_set_kernel<<<(batch + 127) / 128, 128, 0, st>>>(tokens, pos, hist, hist_stride, batch);
    return cudaGetLastError();
}
cudaError_t launch_bounded_wait_probe(const void* src16, int* err_flag, unsigned long long limit, int* landed, cudaStream_t st) {
    bounded_wait_probe_kernel<<<1, 32, 0, st>>>(src16, err_flag, limit, landed);
    return cudaGetLastError();
}
cudaError_t launch_silu_mul(const float* gate_up, int M, int I, float* act, cudaStream_t st, bool pdl) {
    return launch_pdl(silu_mul_kernel, dim3(grid_for((size_t)M * I, 256)), dim3(256), st, pdl, gate_up, M, I, act);
}

}  // namespace hm
