// Shared device helpers and kernel-launch argument blocks (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hm {

constexpr int SLAB = 128;       // output columns per weight slab
constexpr int GEMV_THREADS = 256;
constexpr int ROWS_PER_PASS = 16;  // 256 threads x 16 B = 16 rows x 256 B
constexpr int MAX_M = 8;

// ---- programmatic dependent launch ----------------------------------------------------
// Kernels in the decode chain call pdl_launch_dependents() first (so the next kernel's CTAs
// may be placed and start fetching weights) and pdl_wait() before touching anything a
// previous kernel wrote.  Both are no-ops when the launch carries no programmatic edge.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- thread-block clusters / distributed shared memory ------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Full cluster barrier with release/acquire ordering of shared-memory writes.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of this CTA's shared-memory location `p` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t dsmem_addr(const void* p, uint32_t rank) {
    uint32_t local = (uint32_t)__cvta_generic_to_shared(p), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_dsmem_f32(uint32_t addr, float v) { asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
// Asynchronous store into another CTA's shared memory that also counts 4 bytes on an mbarrier of that CTA
// (both addresses are shared::cluster addresses of the same CTA): data and signal travel together, so the
// receiver waits on its own mbarrier and the sender needs no release fence and no cluster barrier.
__device__ __forceinline__ void st_async_f32(uint32_t addr, float v, uint32_t mbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(addr), "r"(__float_as_uint(v)), "r"(mbar) : "memory");
}
__device__ __forceinline__ void st_async_f32x2(uint32_t addr, float a, float b, uint32_t mbar) {  // addr 8-byte aligned, counts 8 bytes
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];" ::"r"(addr), "r"(__float_as_uint(a)), "r"(__float_as_uint(b)), "r"(mbar) : "memory");
}
__device__ __forceinline__ void st_async_f32x4(uint32_t addr, float4 v, uint32_t mbar) {  // addr 16-byte aligned, counts 16 bytes
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(addr), "r"(__float_as_uint(v.x)), "r"(__float_as_uint(v.y)),
                 "r"(__float_as_uint(v.z)), "r"(__float_as_uint(v.w)), "r"(mbar)
                 : "memory");
}
// not volatile: several of these may be in flight at once (callers order them with barriers)
__device__ __forceinline__ float4 ld_dsmem_f32x4(uint32_t addr) {
    float4 v;
    asm("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

// 128-bit streaming load of read-only weights: bypass L1 (each weight
// byte is used once per token and the working set is far larger than L2).
// Ask the L2 to fetch [base + off, base + off + bytes) from HBM; returns at once (fire and forget).
// Used to pull the weights of a LATER kernel of the decode chain into the L2 while the current,
// latency-bound kernel runs: weights never depend on activations, so the HBM stream can run ahead.
__device__ __forceinline__ void l2_prefetch_slice(const void* base, unsigned long long total, int part, int nparts, int tid) {
    constexpr unsigned long long CH = 8192;
    const unsigned long long per = ((total + nparts - 1) / nparts + CH - 1) / CH * CH;
    const unsigned long long lo = (unsigned long long)part * per;
    if (lo >= total) return;
    const unsigned long long hi = lo + per < total ? lo + per : total;
    for (unsigned long long o = lo + (unsigned long long)tid * CH; o < hi; o += 32ull * CH) {
        const unsigned long long n = (hi - o < CH ? hi - o : CH) & ~15ull;
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"((const char*)base + o), "r"((unsigned)n) : "memory");
    }
}

// Phase stamps (%globaltimer at the phase boundaries of a launch) exist only in builds with -DHM_PHASE_TRACE:
// the decode kernels are chains of instructions executed once, so even a predicated-off stamp costs time.
#ifdef HM_PHASE_TRACE
#define HM_TRACE(...) __VA_ARGS__
#else
#define HM_TRACE(...)
#endif
__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_u2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
// Loads that must observe other CTAs' writes of the same launch (split reductions).
__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 ld_cg_f32x4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// Cooperative copy of n floats written by a previous kernel into shared memory, NT threads, with up to
// four loads per thread in flight before the first use (a loop of load-then-use would pay one L2
// round trip per iteration).  128-bit loads when the pointers and n allow.  L2-only loads: the rows are
// rewritten by other SMs every launch.  Optionally multiplies by a per-element factor held in shared
// memory (mul), optionally only sums (STORE = false).  Returns this thread's share of the sum of squares
// of the loaded values (SQ).
template <int NT, bool SQ, bool STORE = true>
__device__ __forceinline__ float stage_row(const float* __restrict__ src, float* __restrict__ dst, int n, int tid, const float* __restrict__ mul = nullptr) {
    float s = 0.f;
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(mul)) & 15) == 0 && (n & 3) == 0) {
        const int n4 = n >> 2;
        for (int b = tid; b < n4; b += 4 * NT) {
            float4 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = b + i * NT;
                v[i] = idx < n4 ? ld_cg_f32x4(src + 4 * (size_t)idx) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = b + i * NT;
                if (idx < n4) {
                    if (SQ) s = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, s))));
                    if (STORE) {
                        if (mul) {
                            const float4 w = reinterpret_cast<const float4*>(mul)[idx];
                            v[i] = make_float4(v[i].x * w.x, v[i].y * w.y, v[i].z * w.z, v[i].w * w.w);
                        }
                        reinterpret_cast<float4*>(dst)[idx] = v[i];
                    }
                }
            }
        }
    } else {
        for (int b = tid; b < n; b += 4 * NT) {
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = b + i * NT;
                v[i] = idx < n ? ld_cg_f32(src + idx) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = b + i * NT;
                if (idx < n) {
                    if (SQ) s = fmaf(v[i], v[i], s);
                    if (STORE) dst[idx] = mul ? v[i] * mul[idx] : v[i];
                }
            }
        }
    }
    return s;
}

// The same for MR rows at once (row m at src + m * ld_src, stored at dst + m * ld_dst): the loads of all rows are
// issued before the first store, so that staging MR rows costs one L2 round trip, not MR.  Meant for slices of
// up to 4 * NT floats per row (one trip); longer rows take one trip per 4 * NT floats.
template <int NT, int MR>
__device__ __forceinline__ void stage_rows(const float* __restrict__ src, int ld_src, float* __restrict__ dst, int ld_dst, int n, int tid, const float* __restrict__ mul = nullptr) {
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(mul)) & 15) == 0 && ((n | ld_src | ld_dst) & 3) == 0) {
        const int n4 = n >> 2;
        for (int b = tid; b < n4; b += NT) {
            float4 v[MR];
#pragma unroll
            for (int m = 0; m < MR; ++m) v[m] = ld_cg_f32x4(src + (size_t)m * ld_src + 4 * (size_t)b);
            const float4 w = mul ? reinterpret_cast<const float4*>(mul)[b] : make_float4(1.f, 1.f, 1.f, 1.f);
#pragma unroll
            for (int m = 0; m < MR; ++m)
                *reinterpret_cast<float4*>(dst + (size_t)m * ld_dst + 4 * (size_t)b) = mul ? make_float4(v[m].x * w.x, v[m].y * w.y, v[m].z * w.z, v[m].w * w.w) : v[m];
        }
    } else {
        for (int b = tid; b < n; b += NT) {
            float v[MR];
#pragma unroll
            for (int m = 0; m < MR; ++m) v[m] = ld_cg_f32(src + (size_t)m * ld_src + b);
            const float w = mul ? mul[b] : 1.f;
#pragma unroll
            for (int m = 0; m < MR; ++m) dst[(size_t)m * ld_dst + b] = mul ? v[m] * w : v[m];
        }
    }
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
// f32 -> bf16 round-to-nearest-even (KV pages in bf16 mode).
__device__ __forceinline__ uint16_t f32_to_bf16_rne(float f) {
    uint32_t u = __float_as_uint(f);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
    float f;
    asm("{ .reg .b16 t; mov.b16 t, %1; cvt.f32.f16 %0, t; }" : "=f"(f) : "h"(h));
    return f;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- GEMV argument block ---------------------------------------------------------------
enum Prologue { PRO_PLAIN = 0, PRO_RMSNORM = 1 };
enum Epilogue { EPI_STORE = 0, EPI_QKV_ROPE = 1, EPI_SWIGLU = 2, EPI_LOGITS = 3 };

// Element offsets inside one [16 tokens][hd] page tile.  Chunk-major means: the chunk c of every token is stored
// together, so that the 16 tokens' copies of one chunk are one contiguous run; either way the tile is one
// contiguous block of the pool (one bulk copy).
//   K: chunks of 4 elements, K[d / 4][token][d % 4]: attention lanes that own one token each read a chunk
//      without bank conflicts while the matching query chunk is a broadcast.
//   V on bf16 pages: chunks of 8 elements, V[d / 8][token][d % 8]: a chunk is 16 bytes, so the eight rows of an
//      8x8 matrix that ldmatrix fetches for the P.V MMA (8 tokens of one chunk) are 128 contiguous bytes.
//   V on f32 pages: rows, V[token][d]: the CUDA-core kernels read one token's row with consecutive lanes.
__host__ __device__ __forceinline__ int k_tile_off(int t, int d) { return ((((d >> 2) << 4) + t) << 2) | (d & 3); }
__host__ __device__ __forceinline__ int v_tile_off(int t, int d, int hd, int bf16) { return bf16 ? (((((d >> 3) << 4) + t) << 3) | (d & 7)) : t * hd + d; }

// One activation value into the packed bf16 x 3 tile image the tensor-core GEMM copies in bulk
// (gemm_tc.cu: [k-block][term][mpad rows][64 k], rows of 128 B, 16-byte chunks XOR-swizzled by row & 7):
// lets a producer kernel hand its output to that GEMM without a packing launch in between.
__device__ __forceinline__ void tc_xpack_store(unsigned char* xp, int mpad, int m, int k, float v) {
    const uint16_t h = f32_to_bf16_rne(v);
    const float r1 = v - bf16_bits_to_f32(h);
    const uint16_t md = f32_to_bf16_rne(r1);
    const uint16_t lo = f32_to_bf16_rne(r1 - bf16_bits_to_f32(md));
    const int kb = k >> 6, kk = k & 63, chunk = kk >> 3, e = kk & 7;
    unsigned char* tile = xp + (size_t)kb * (3 * mpad * 128);
    const uint16_t term[3] = {h, md, lo};
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        const int row = t * mpad + m;
        *reinterpret_cast<uint16_t*>(tile + (size_t)row * 128 + ((chunk ^ (row & 7)) << 4) + e * 2) = term[t];
    }
}

// Eight consecutive activations (k0 a multiple of 8) as one 16-byte chunk per term.
__device__ __forceinline__ void tc_xpack_store8(unsigned char* xp, int mpad, int m, int k0, const float (&v)[8]) {
    uint32_t w[3][4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        uint16_t h[2], md[2], lo[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const float x = v[2 * e + u];
            h[u] = f32_to_bf16_rne(x);
            const float r1 = x - bf16_bits_to_f32(h[u]);
            md[u] = f32_to_bf16_rne(r1);
            lo[u] = f32_to_bf16_rne(r1 - bf16_bits_to_f32(md[u]));
        }
        w[0][e] = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
        w[1][e] = (uint32_t)md[0] | ((uint32_t)md[1] << 16);
        w[2][e] = (uint32_t)lo[0] | ((uint32_t)lo[1] << 16);
    }
    const int kb = k0 >> 6, chunk = (k0 & 63) >> 3;
    unsigned char* tile = xp + (size_t)kb * (3 * mpad * 128);
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        const int row = t * mpad + m;
        *reinterpret_cast<uint4*>(tile + (size_t)row * 128 + ((chunk ^ (row & 7)) << 4)) = make_uint4(w[t][0], w[t][1], w[t][2], w[t][3]);
    }
}

struct KvDesc {
    void* k_pool;            // this layer's K pages [n_pages][kv_heads][page_tokens][hd]
    void* v_pool;
    const int32_t* page_table;  // [n_seq][max_pages]
    int max_pages;
    int page_tokens;
    int kv_heads;
    int hd;
    int bf16;                // page element type: 0 = f32, 1 = bf16
};

// Fused-QKV epilogue of the 32-row-tile projections (Q8_0 / Q4_0 / K-quants; no QK-norm on this path).  The q and k rows
// of every head are stored so that a tile holds 16 dimensions of the head's first half followed by their 16 rotation
// partners (rope_tile_row); v rows keep their order.
struct RopeEpi {
    int q_dim, kv_dim, hd;
    const float* rope_cos;   // [max_pos][hd]
    const float* rope_sin;
    const int32_t* row_pos;  // [M] position of each row's token
    const int32_t* row_seq;  // [M] sequence of each row; null: row m is sequence seq_base + m
    int seq_base;
    KvDesc kv;
};

// row nl of a q or k part (rows n_off ..) -> its place in the tiled weight arrays
__host__ __device__ __forceinline__ int rope_tile_row(int nl, int n_off, int hd) {
    const int head = nl / hd, d = nl - head * hd, half = hd >> 1;
    const int hi = d >= half ? 1 : 0, dd = d - hi * half;
    return n_off + head * hd + (dd >> 4) * 32 + hi * 16 + (dd & 15);
}

// Bias, half rotation (src/hf/emitter.rs:560-640; the operation order of post_qkv_kernel) and the KV-page write for one
// value of a finished tile: vals = the tile's sums [M][32] in shared memory, v = vals[tid].
__device__ __forceinline__ void rope_tile_epilogue(const RopeEpi& r, const float* vals, float v, int tid, int tile, int m_valid, int N, const float* bias, float* y, int ldy) {
    const int m = tid >> 5, p = tid & 31, n0 = tile * 32;
    if (m >= m_valid || n0 >= N) return;
    const int pos = r.row_pos[m];
    const int seq = r.row_seq ? r.row_seq[m] : r.seq_base + m;
    const bool is_q = n0 < r.q_dim, is_k = !is_q && n0 < r.q_dim + r.kv_dim;
    const int part_off = is_q ? 0 : (is_k ? r.q_dim : r.q_dim + r.kv_dim);
    const int head = (n0 - part_off) / r.hd;
    int d;
    float val;
    if (is_q || is_k) {
        const int half = r.hd >> 1, hi = p >> 4;
        d = (((n0 - part_off) - head * r.hd) >> 5) * 16 + (p & 15) + hi * half;
        const int dp = hi ? d - half : d + half, base = part_off + head * r.hd;
        val = v;
        float oth = vals[tid ^ 16];
        if (bias) {
            val += bias[base + d];
            oth += bias[base + dp];
        }
        oth = hi ? oth : -oth;
        val = fmaf(oth, r.rope_sin[(size_t)pos * r.hd + d], val * r.rope_cos[(size_t)pos * r.hd + d]);
    } else {
        d = (n0 - part_off) - head * r.hd + p;
        val = bias ? v + bias[n0 + p] : v;
    }
    if (is_q) {
        y[(size_t)m * ldy + head * r.hd + d] = val;
    } else {
        const int page = r.kv.page_table[(size_t)seq * r.kv.max_pages + pos / r.kv.page_tokens];
        const size_t off = ((size_t)page * r.kv.kv_heads + head) * r.kv.page_tokens * r.hd +
                           (is_k ? k_tile_off(pos % r.kv.page_tokens, d) : v_tile_off(pos % r.kv.page_tokens, d, r.hd, r.kv.bf16));
        void* pool = is_k ? r.kv.k_pool : r.kv.v_pool;
        if (r.kv.bf16) reinterpret_cast<uint16_t*>(pool)[off] = f32_to_bf16_rne(val);
        else reinterpret_cast<float*>(pool)[off] = val;
    }
}

struct GemvArgs {
    int* err_flag;                 // optional: raised to 2 when the bounded wait for the staged weights runs out
    unsigned long long* trace;     // optional (HM_GEMV_TRACE=1): 8 %globaltimer stamps of CTA 0 of this launch
    const void* pf_ptr;            // optional: weights of a later kernel to pull into the L2 (see l2_prefetch_slice)
    unsigned long long pf_bytes;
    // weights: element (k, n) of slab s = n / 128 at byte  s*slab_stride + k*row_stride + (n%128)*2
    const uint16_t* W;
    long long slab_stride;  // bytes
    long long row_stride;   // bytes
    int K, N;
    int m_valid;            // rows >= m_valid are padding: computed, never stored
    int ksplit, rows_per_split;
    int cluster;            // > 1: the ksplit CTAs of a slab form one thread-block cluster and reduce through
                            // distributed shared memory (ksplit == cluster); else partial/tickets are used
    // input rows [M][ldx]
    const float* x;
    int ldx;
    int pro;
    const float* norm_w;
    float eps;
    // epilogue
    int epi;
    float* y;
    int ldy;
    const float* bias;   // [N] or null
    const float* resid;  // [M][ldy] or null (EPI_STORE: y = resid + acc)
    // EPI_QKV_ROPE
    int q_dim, kv_dim, hd, has_qk_norm;
    const float* q_norm_w;
    const float* k_norm_w;
    const float* rope_cos;  // [max_pos][hd]
    const float* rope_sin;
    const int32_t* row_pos;  // [M] position of each row's token
    const int32_t* row_seq;  // [M] sequence (page-table row) of each row; null: row m is sequence seq_base + m
    int seq_base;            // first row's sequence when row_seq is null (launches over a group of a larger batch)
    KvDesc kv;
    // EPI_LOGITS: per-slab argmax partials
    float* amax_val;     // [M][nslabs]
    int32_t* amax_idx;   // [M][nslabs]
    // EPI_LOGITS, optional: the CTA whose epilogue finishes last (a ticket over the slabs) also reduces the slab
    // partials to the greedy token of every row, stores it as the next step's input, advances the position and
    // appends to the history: what a separate argmax launch would do
    unsigned int* fin_ticket;  // one word, zero between launches
    uint32_t* next_tok;        // [M]
    uint32_t* feed_tok;        // [M] or null
    int32_t* pos;              // [M] or null
    uint32_t* hist;            // [M][hist_stride] or null
    int hist_stride;
    // split-K scratch
    float* partial;      // [nslabs*ksplit][M][128]
    unsigned int* tickets;  // [nslabs], zero between launches
};

struct AttnArgs {
    const void* pf_ptr;  // optional: weights of a later kernel to pull into the L2
    unsigned long long pf_bytes;
    unsigned char* xp_out;  // optional: write the output as packed tensor-core activations (tc_xpack_store) instead of `out`
    int xp_mpad;
    int early_pages;     // >= 1: every row is its own sequence (decode), so the pages below the one of the new token may be read before the dependency wait;
                         // 2: and every page of a split gets its own shared-memory slot (small launches, where latency counts and occupancy does not)
    int stream_pages;    // > 0: long contexts may use the bulk-copy ring variant (pages per CTA decided from max_pages / nsplit)
    int st_stages;       // stages of that variant's page ring, a multiple of its 8 consumer warps (filled in by the launcher)
    int* err_flag;       // raised to 2 when a bounded wait of that variant runs out
    unsigned long long* trace;  // optional (HM_GEMV_TRACE=1): 8 %globaltimer stamps of CTA (0,0,0) of the short-context kernel
    const float* q;       // [M][heads*hd]
    const void* k_pool;
    const void* v_pool;
    const int32_t* page_table;
    const int32_t* row_seq;  // null => row index
    const int32_t* row_pos;  // kv length - 1 per row (the row's own position); see kv_len
    const int32_t* kv_len;   // when non-null used instead of row_pos+1
    int max_pages, page_tokens, heads, kv_heads, hd, nsplit;
    int cluster;          // != 0: the nsplit CTAs of a (row, KV head) are one cluster and merge through DSMEM
    float scale;
    float* out;           // [M][heads*hd]
    float* part_acc;      // [M][heads][nsplit][hd]
    float* part_ml;       // [M][heads][nsplit][2]
    unsigned int* tickets;  // [M*kv_heads]
};

struct QuantArgs {
    int* err_flag;           // optional: raised to 2 when the bounded wait for the staged weights runs out
    unsigned long long* trace;  // optional, builds with -DHM_PHASE_TRACE: %globaltimer stamps of CTA 0 (indices as in GemvArgs; 7 = rows staged, before the digit pass)
    const uint16_t* scales;  // [N/32][K/32][32] f16 bits (launch_split_blocks)
    const uint8_t* codes;    // [N/32][K/32][chunk][32][16 B]: 2 chunks per Q8_0 block, 1 per Q4_0 block
    int q4;                  // 0 = Q8_0, 1 = Q4_0
    int K, N, m_valid;
    int ksplit, kb_per_split;  // filled in by launch_gemv_quant: CTAs per 32-row tile and k-blocks per CTA
    int from_regs;             // filled in by launch_gemv_quant: activation rows are read with 16-byte loads and never staged as f32
    int reg_tail;              // filled in by launch_gemv_quant: 1 = the last eight k-blocks of a staged slice are not staged (one per warp, from global memory)
    const float* x;
    int ldx;
    int pro;                 // PRO_PLAIN / PRO_RMSNORM (f64 sum of squares, emitter_quant.rs:713-791)
    const float* norm_w;
    float eps;
    int epi;                 // EPI_STORE, EPI_SWIGLU (gate/up rows interleaved 16 + 16 per tile, y = silu(gate) * up, [M][N/2]), or
                             // EPI_QKV_ROPE (q and k rows laid out by launch_split_blocks(rope_hd): y = rotated q [M][q_dim], k and v into the KV pages)
    float* y;
    int ldy;
    const float* bias;
    const float* resid;
    RopeEpi rope;            // EPI_QKV_ROPE
    // launch_gemm_quant: the rows as digit planes, written by its packing launch
    const uint32_t* img_in;  // [K/32][32 row pairs][64 words]
    const float* bs_in;      // [K/32][32 row pairs][2]
    int alias_slots;         // filled in by launch_gemm_quant: rank 0's split-K receive slots reuse the staged slice (one more cluster barrier)
};

// ---- launchers (defined in the .cu files) ----------------------------------------------
cudaError_t launch_gemv_bf16(const GemvArgs& a, int M, cudaStream_t st, bool pdl);

size_t gemv_partial_floats(int N, int ksplit, int M);
void gemv_pick_split(int K, int N, int M, int sm_count, int* ksplit, int* rows_per_split);
// Cluster variant: ksplit = cluster size (<= max_cluster), sized so that all CTAs are resident at once.
void gemv_pick_cluster(int K, int N, int M, int sm_count, int max_cluster, int* cluster, int* rows_per_split);
int gemv_max_cluster();  // largest cluster size the device schedules for the projection kernel (8 or 16)
cudaError_t launch_attn_decode(const AttnArgs& a, int M, bool kv_bf16, cudaStream_t st, bool pdl);
int attn_pick_nsplit(int M, int kv_heads, int max_pages, int sm_count, bool bf16_pages);
int attn_pick_cluster(int max_pages, int max_cluster);

cudaError_t launch_pack_slabs_from_nk(const uint16_t* src_nk, int N, int K, uint16_t* dst, int n_off, int interleave_which, cudaStream_t st);
cudaError_t launch_pack_slabs_from_kn(const uint16_t* src_kn, int K, int N, uint16_t* dst, cudaStream_t st);
cudaError_t launch_embed_gather(const void* table, int table_dtype, const uint32_t* tokens, int M, int H, int V, float* out, int* err_flag, cudaStream_t st, bool pdl);
cudaError_t launch_argmax_finish(const float* amax_val, const int32_t* amax_idx, int nslabs, int M, uint32_t* next_tok, uint32_t* feed_tok, int32_t* pos, uint32_t* hist, int hist_stride, cudaStream_t st, bool pdl);
cudaError_t launch_argmax_rows(const float* logits, int rows, int n, uint32_t* out, cudaStream_t st);
cudaError_t launch_rms_norm(const float* x, const float* w, float eps, int rows, int n, float* out, cudaStream_t st);
cudaError_t launch_qknorm_rope(float* x, int rows, int heads, int hd, const float* norm_w, float eps, const float* cos_rows, const float* sin_rows, cudaStream_t st);
cudaError_t launch_kv_write_rows(const KvDesc& kv, int seq, int pos0, const float* k_rows, const float* v_rows, int n_new, cudaStream_t st);
cudaError_t launch_kv_read_rows(const KvDesc& kv, int seq, int len, float* k_out, float* v_out, cudaStream_t st);
cudaError_t launch_convert_to_f32(const void* src, int dtype, size_t n, float* dst, cudaStream_t st);

// GGUF blocks of n_rows output rows (stored at rows n_off.. of the projection) -> the tiled arrays, which
// must hold quant_scale_elems / quant_code_bytes of the whole projection and start zeroed.
size_t quant_scale_elems(int K, int N);
size_t quant_code_bytes(int K, int N, int q4);
// rope_hd > 0 (q and k parts of a fused QKV projection whose epilogue rotates): the rows of every head are re-ordered so that a
// 32-row tile holds 16 dimensions of the head's first half followed by their 16 rotation partners (d + rope_hd / 2).
cudaError_t launch_split_blocks(const uint8_t* blocks, int n_rows, int K, int q4, int n_off, int interleave_which, uint16_t* scales, uint8_t* codes, cudaStream_t st, int rope_hd = 0);
cudaError_t launch_dequant(const uint8_t* blocks, size_t nblocks, int q4, float* out, cudaStream_t st);
cudaError_t launch_gemv_quant(const QuantArgs& a, int M, int sm_count, cudaStream_t st, bool pdl);
// Q8_0 / Q4_0 projection over up to 64 rows (a.m_valid): a packing launch (rows -> digit planes in img / bs) and the multiply.
size_t quant_rows_image_words(int K);
size_t quant_rows_scale_floats(int K);
bool quant_rows_supported(const QuantArgs& a);
cudaError_t launch_gemm_quant(const QuantArgs& a, uint32_t* img, float* bs, int sm_count, cudaStream_t st, bool pdl, int* launches);
// quant plan helpers: PostQKV (src/hf/emitter_quant.rs:800-905) and SiLU*Up (:1078-1099)
cudaError_t launch_post_qkv(const float* qkv, int M, int heads, int kv_heads, int hd, int has_qk_norm, const float* q_norm_w, const float* k_norm_w, float eps, const float* rope_cos, const float* rope_sin, const int32_t* row_pos, const int32_t* row_seq, const KvDesc& kv, float* q_out, cudaStream_t st, bool pdl);
cudaError_t launch_hist_set(const uint32_t* tokens, const int32_t* pos, uint32_t* hist, int hist_stride, int batch, cudaStream_t st);
// one-CTA kernel whose second mbarrier wait runs out after `limit` polls and raises *err_flag to 2 (self-test of the give-up path)
cudaError_t launch_bounded_wait_probe(const void* src16, int* err_flag, unsigned long long limit, int* landed, cudaStream_t st);
cudaError_t launch_silu_mul(const float* gate_up, int M, int I, float* act, cudaStream_t st, bool pdl);

}  // namespace hm
