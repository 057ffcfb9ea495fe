// Split-KV GQA decode attention over a paged KV cache (one new query token per row).
//
// Stands in for the attention body of Homura's Attn kernel (src/hf/emitter.rs:709-737):
// scores = (q . k) * 1/sqrt(hd) over the cached tokens, softmax, p . v, with the KV head of
// query head h given by h floordiv (heads / kv_heads) (src/graph_builder/emit_linalg.rs:
// 126,204).  The decode mask is all zeros (src/hf/precompute.rs:49-64), so only the length
// bound is applied.  The reference's cache is contiguous f32 [kv_heads, max_len, hd]
// (src/runtime.rs:375-385); here it is paged: page p of a layer holds
// [kv_heads][16 tokens][hd] in f32 or bf16, and a per-sequence page table maps token t to
// page_table[t / 16].
//
// One CTA = one (row, KV head, token split).  All g = heads/kv_heads query heads that share
// the KV head are processed together, so every K/V byte is read once per g heads.  A warp
// owns a page at a time: it stages the page's K and V tiles in shared memory with coalesced
// 128-bit loads, computes the 16 x g scores, folds them into running (max, sum, acc) state
// (online softmax), and accumulates p . v with each lane owning hd/32 output elements.
// Splits are merged by the CTA that arrives last at the (row, KV head) ticket, in split
// order; no CTA waits on another.
#include "common.cuh"

namespace hm {
namespace {

constexpr int PT = 16;      // tokens per page (the only supported page size)
constexpr int ATT_WARPS = 4;
constexpr int G_MAX = 8;    // query heads per KV head handled by one CTA

template <bool BF16>
struct KvElem;
template <>
struct KvElem<false> {
    using T = float;
    static constexpr int PER16 = 4;  // elements per 16-byte load
};
template <>
struct KvElem<true> {
    using T = uint16_t;
    static constexpr int PER16 = 8;
};

// Stage one [16][HD] page tile into shared memory as f32 rows of stride LD.
template <int HD, bool BF16, int LD>
__device__ __forceinline__ void load_tile(const void* src, float* dst, int lane) {
    constexpr int PER = KvElem<BF16>::PER16;
    constexpr int N16 = PT * HD / PER;  // 16-byte pieces in the tile
#pragma unroll
    for (int i = 0; i < N16 / 32; ++i) {
        const int piece = i * 32 + lane;
        const int e = piece * PER;
        const int t = e / HD, d = e % HD;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src) + piece);
        float* o = dst + t * LD + d;
        if (BF16) {
            o[0] = bf16_lo(v.x); o[1] = bf16_hi(v.x); o[2] = bf16_lo(v.y); o[3] = bf16_hi(v.y);
            o[4] = bf16_lo(v.z); o[5] = bf16_hi(v.z); o[6] = bf16_lo(v.w); o[7] = bf16_hi(v.w);
        } else {
            *reinterpret_cast<float4*>(o) = make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
        }
    }
}

template <int HD, bool BF16>
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_decode_kernel(const AttnArgs a) {
    constexpr int KLD = HD + 4;   // padded K row: lanes reading different tokens spread over banks
    constexpr int EPL = HD / 32;  // output elements per lane
    extern __shared__ __align__(16) float sm[];
    float* q_s = sm;                                   // [G_MAX][HD]
    float* k_s = q_s + G_MAX * HD;                     // [warps][16][KLD]
    float* v_s = k_s + ATT_WARPS * PT * KLD;           // [warps][16][HD]
    float* p_s = v_s + ATT_WARPS * PT * HD;            // [warps][G_MAX][16]
    float* w_m = p_s + ATT_WARPS * G_MAX * PT;         // [warps][G_MAX]
    float* w_l = w_m + ATT_WARPS * G_MAX;              // [warps][G_MAX]
    float* w_acc = w_l + ATT_WARPS * G_MAX;            // [warps][G_MAX][HD]
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
    const int g = a.heads / a.kv_heads;
    const int head0 = kvh * g;

    pdl_launch_dependents();
    pdl_wait();

    const int seq = a.row_seq ? a.row_seq[m] : m;
    const int kvlen = a.kv_len ? a.kv_len[m] : a.row_pos[m] + 1;
    const int npages = (kvlen + PT - 1) / PT;
    const int pps = (npages + a.nsplit - 1) / a.nsplit;
    const int p0 = split * pps, p1 = min(npages, p0 + pps);
    const int32_t* pt = a.page_table + (size_t)seq * a.max_pages;

    for (int i = tid; i < g * HD; i += ATT_WARPS * 32) q_s[i] = a.q[(size_t)m * a.heads * HD + head0 * HD + i];
    __syncthreads();

    float run_m[G_MAX], run_l[G_MAX], acc[G_MAX][EPL];
#pragma unroll
    for (int j = 0; j < G_MAX; ++j) {
        run_m[j] = -INFINITY;
        run_l[j] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[j][e] = 0.f;
    }

    float* kw = k_s + warp * PT * KLD;
    float* vw = v_s + warp * PT * HD;
    float* pw = p_s + warp * G_MAX * PT;
    const int t = lane & 15, hf = lane >> 4;
    using T = typename KvElem<BF16>::T;

    for (int p = p0 + warp; p < p1; p += ATT_WARPS) {
        const int page = pt[p];
        const size_t tile = ((size_t)page * a.kv_heads + kvh) * PT * HD;
        load_tile<HD, BF16, KLD>(reinterpret_cast<const T*>(a.k_pool) + tile, kw, lane);
        load_tile<HD, BF16, HD>(reinterpret_cast<const T*>(a.v_pool) + tile, vw, lane);
        __syncwarp();
        // scores: lane (t, hf) covers half of the head dim of token t for every head
        float s[G_MAX];
#pragma unroll
        for (int j = 0; j < G_MAX; ++j) s[j] = 0.f;
        const float* kr = kw + t * KLD + hf * (HD / 2);
#pragma unroll
        for (int dc = 0; dc < HD / 2; dc += 4) {
            const float4 kv4 = *reinterpret_cast<const float4*>(kr + dc);
#pragma unroll
            for (int j = 0; j < G_MAX; ++j) {
                if (j < g) {
                    const float4 q4 = *reinterpret_cast<const float4*>(q_s + j * HD + hf * (HD / 2) + dc);
                    s[j] = fmaf(q4.x, kv4.x, s[j]);
                    s[j] = fmaf(q4.y, kv4.y, s[j]);
                    s[j] = fmaf(q4.z, kv4.z, s[j]);
                    s[j] = fmaf(q4.w, kv4.w, s[j]);
                }
            }
        }
        const bool valid = (p * PT + t) < kvlen;
        float corr[G_MAX];
#pragma unroll
        for (int j = 0; j < G_MAX; ++j) {
            if (j < g) {
                float sc = s[j] + __shfl_xor_sync(0xffffffffu, s[j], 16);
                sc = valid ? sc * a.scale : -INFINITY;
                float mx = sc;
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float m_new = fmaxf(run_m[j], mx);
                const float pr = valid ? expf(sc - m_new) : 0.f;
                float ps = pr;
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
                corr[j] = expf(run_m[j] - m_new);  // exp(-inf) = 0 on the first page
                run_l[j] = run_l[j] * corr[j] + ps;
                run_m[j] = m_new;
                if (hf == 0) pw[j * PT + t] = pr;
            }
        }
        __syncwarp();
        // p . v : lane owns output elements [lane*EPL, lane*EPL + EPL)
#pragma unroll
        for (int j = 0; j < G_MAX; ++j) {
            if (j < g) {
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[j][e] *= corr[j];
            }
        }
#pragma unroll 4
        for (int tt = 0; tt < PT; ++tt) {
            float vv[EPL];
#pragma unroll
            for (int e = 0; e < EPL; ++e) vv[e] = vw[tt * HD + lane * EPL + e];
#pragma unroll
            for (int j = 0; j < G_MAX; ++j) {
                if (j < g) {
                    const float pr = pw[j * PT + tt];
#pragma unroll
                    for (int e = 0; e < EPL; ++e) acc[j][e] = fmaf(pr, vv[e], acc[j][e]);
                }
            }
        }
        __syncwarp();
    }

    // ---- merge the warps of this CTA ----
#pragma unroll
    for (int j = 0; j < G_MAX; ++j) {
        if (j < g) {
            if (lane == 0) {
                w_m[warp * G_MAX + j] = run_m[j];
                w_l[warp * G_MAX + j] = run_l[j];
            }
#pragma unroll
            for (int e = 0; e < EPL; ++e) w_acc[(warp * G_MAX + j) * HD + lane * EPL + e] = acc[j][e];
        }
    }
    __syncthreads();

    // thread -> (head j, element d); CTA-level (m, l, acc) for this split
    for (int i = tid; i < g * HD; i += ATT_WARPS * 32) {
        const int j = i / HD, d = i % HD;
        float M = -INFINITY;
#pragma unroll
        for (int wv = 0; wv < ATT_WARPS; ++wv) M = fmaxf(M, w_m[wv * G_MAX + j]);
        float l = 0.f, o = 0.f;
        if (M > -INFINITY) {
#pragma unroll
            for (int wv = 0; wv < ATT_WARPS; ++wv) {
                const float sc = expf(w_m[wv * G_MAX + j] - M);
                l = fmaf(w_l[wv * G_MAX + j], sc, l);
                o = fmaf(w_acc[(wv * G_MAX + j) * HD + d], sc, o);
            }
        }
        const int head = head0 + j;
        if (a.nsplit == 1) {
            a.out[(size_t)m * a.heads * HD + head * HD + d] = o / l;
        } else {
            const size_t pi = ((size_t)m * a.heads + head) * a.nsplit + split;
            a.part_acc[pi * HD + d] = o;
            if (d == 0) {
                a.part_ml[pi * 2 + 0] = M;
                a.part_ml[pi * 2 + 1] = l;
            }
        }
    }
    if (a.nsplit == 1) return;

    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int tk = atomicAdd(a.tickets + (m * a.kv_heads + kvh), 1u);
        s_last = (tk == (unsigned int)(a.nsplit - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int i = tid; i < g * HD; i += ATT_WARPS * 32) {
        const int j = i / HD, d = i % HD;
        const int head = head0 + j;
        const size_t base = ((size_t)m * a.heads + head) * a.nsplit;
        float M = -INFINITY;
        for (int s2 = 0; s2 < a.nsplit; ++s2) M = fmaxf(M, ld_cg_f32(a.part_ml + (base + s2) * 2));
        float l = 0.f, o = 0.f;
        for (int s2 = 0; s2 < a.nsplit; ++s2) {
            const float ms = ld_cg_f32(a.part_ml + (base + s2) * 2);
            if (ms > -INFINITY) {
                const float sc = expf(ms - M);
                l = fmaf(ld_cg_f32(a.part_ml + (base + s2) * 2 + 1), sc, l);
                o = fmaf(ld_cg_f32(a.part_acc + (base + s2) * HD + d), sc, o);
            }
        }
        a.out[(size_t)m * a.heads * HD + head * HD + d] = o / l;
    }
    if (tid == 0) a.tickets[m * a.kv_heads + kvh] = 0u;
}

template <int HD, bool BF16>
cudaError_t launch_t(const AttnArgs& a, int M, cudaStream_t st, bool pdl) {
    constexpr int KLD = HD + 4;
    const size_t smem = sizeof(float) * (G_MAX * HD + ATT_WARPS * PT * KLD + ATT_WARPS * PT * HD + ATT_WARPS * G_MAX * PT +
                                         2 * ATT_WARPS * G_MAX + ATT_WARPS * G_MAX * HD);
    if (smem > 40 * 1024) {  // static shared memory counts against the 48 KB default too
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)a.nsplit, (unsigned)a.kv_heads, (unsigned)M);
    cfg.blockDim = dim3(ATT_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, attn_decode_kernel<HD, BF16>, a);
}

}  // namespace

// Enough (row, KV head, split) CTAs to cover the SMs about twice, at least two pages each.
int attn_pick_nsplit(int M, int kv_heads, int max_pages, int sm_count) {
    int n = (2 * sm_count + M * kv_heads - 1) / (M * kv_heads);
    const int by_pages = (max_pages + 1) / 2;
    if (n > by_pages) n = by_pages;
    if (n > 64) n = 64;
    if (n < 1) n = 1;
    return n;
}

cudaError_t launch_attn_decode(const AttnArgs& a, int M, bool kv_bf16, cudaStream_t st, bool pdl) {
    if (a.page_tokens != PT || a.heads % a.kv_heads != 0 || a.heads / a.kv_heads > G_MAX) return cudaErrorInvalidValue;
    if (a.hd == 64) return kv_bf16 ? launch_t<64, true>(a, M, st, pdl) : launch_t<64, false>(a, M, st, pdl);
    if (a.hd == 128) return kv_bf16 ? launch_t<128, true>(a, M, st, pdl) : launch_t<128, false>(a, M, st, pdl);
    return cudaErrorInvalidValue;
}

}  // namespace hm
