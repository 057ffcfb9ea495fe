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
// One CTA = one (row, KV head, split) and 8 warps.  All g = heads/kv_heads query heads that
// share the KV head are served from the same K/V bytes: the CTA stages NSUB pages at a time in
// shared memory with coalesced 128-bit loads issued by all threads (the next group's loads are
// in flight while the current one is being used), and warp w works on query head w % g of page
// slot w / g: 16 x hd scores with lane (token, half of hd), an online-softmax update, and
// p . v with each lane owning hd/32 outputs.  Page slots are merged in shared memory; the
// splits of one (row, KV head) are either the CTAs of one thread-block cluster, merged by rank 0
// through distributed shared memory, or independent CTAs merged through global scratch by
// whichever arrives last at a ticket.  No CTA ever waits for another outside the hardware
// cluster barrier.
#include <type_traits>

#include <algorithm>

#include "common.cuh"
#include "launch_attrs.h"
#include "mbarrier.cuh"

namespace hm {
namespace {

constexpr int PT = 16;  // tokens per page (the only supported page size)
constexpr int ATT_WARPS = 8;
constexpr int ATT_THREADS = ATT_WARPS * 32;
constexpr int G_MAX = 8;   // query heads per KV head handled by one CTA
constexpr int MAXP = 4;    // 16-byte pieces of K (and of V) a thread may hold in flight
constexpr int ST_MIN_PAGES = 16;  // pages per CTA from which the streaming variant is used
constexpr int RES_MAX_PAGES = 8;  // decode launches with at most this many pages per CTA keep all of them in shared memory

template <int HD, bool BF16>
struct Tile {
    static constexpr int PER16 = BF16 ? 8 : 4;              // elements per 16-byte piece
    static constexpr int PIECES = PT * HD / PER16;          // 16-byte pieces per [16][HD] tile
    static constexpr int KLD = HD + 4;                      // padded K row stride (floats)
    static constexpr int SLOT_FLOATS = PT * KLD + PT * HD;  // K tile + V tile of one page slot
    static constexpr int MAX_NSUB = MAXP * ATT_THREADS / PIECES;
};

template <int HD, bool BF16>
__host__ __device__ inline int pick_nsub(int g) {
    int n = ATT_WARPS / g;
    if (n > Tile<HD, BF16>::MAX_NSUB) n = Tile<HD, BF16>::MAX_NSUB;
    return n < 1 ? 1 : n;
}

// Page slots of the short-context kernel: nsub slots reused group after group, or -- when a decode
// launch gives a CTA at most RES_MAX_PAGES pages -- one slot per page, so that every page that is
// final before the dependency wait is already in shared memory when the wait returns.
template <int HD, bool BF16>
__host__ __device__ inline int pick_nslots(int g, int early_pages, int max_pages, int nsplit) {
    const int nsub = pick_nsub<HD, BF16>(g);
    const int cap = (max_pages + nsplit - 1) / nsplit;
    if (early_pages < 2 || cap > RES_MAX_PAGES) return nsub;
    return (cap + nsub - 1) / nsub * nsub;
}

// Slots for the splits' (max, sum, acc) triples in rank 0 of a cluster are allocated in steps of 4 / 8 / 16,
// the unused ones hold neutral triples, and the merge loops run to that compile-time count with
// unconditional loads (a loop bounded by the run-time split count is compiled with one shared-memory round
// trip per iteration, which tripled the merge time).
__host__ __device__ inline int merge_slot_cap(int nsplit) { return nsplit <= 4 ? 4 : nsplit <= 8 ? 8 : 16; }

template <bool BF16>
__device__ __forceinline__ void unpack_store(float* o, const uint4& v) {
    if (BF16) {
        o[0] = bf16_lo(v.x); o[1] = bf16_hi(v.x); o[2] = bf16_lo(v.y); o[3] = bf16_hi(v.y);
        o[4] = bf16_lo(v.z); o[5] = bf16_hi(v.z); o[6] = bf16_lo(v.w); o[7] = bf16_hi(v.w);
    } else {
        *reinterpret_cast<float4*>(o) = make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
    }
}

// Merge the per-warp (max, sum, acc) triples of a CTA (warp = page slot * g + query head), then the
// splits of the (row, KV head): through the cluster (rank 0 reads its peers' shared memory in rank
// order), or through global scratch by whichever CTA arrives last at the ticket.
// Attention output of (row m, head, dim d): f32 [rows][heads * hd], or straight into the packed
// activation tiles of the O-projection's tensor-core GEMM.
template <int HD>
__device__ __forceinline__ void store_out(const AttnArgs& a, int m, int head, int d, float v) {
    if (a.xp_out) tc_xpack_store(a.xp_out, a.xp_mpad, m, head * HD + d, v);
    else a.out[(size_t)m * a.heads * HD + head * HD + d] = v;
}

// Rank 0 of a (row, KV head) cluster, after every split's (max, sum, acc) triple has landed in its
// shared memory: one scale factor per (split, head) first (g * nsplit exponentials instead of one per
// output element and split), then every output element is a short multiply-add over the splits.
template <int HD, int NS>
__device__ __forceinline__ void cluster_rank0_merge_n(const AttnArgs& a, int g, int head0, int m, float* scratch, const float* c_o, const float* c_ml) {
    const int tid = threadIdx.x, nthreads = blockDim.x;
    HM_TRACE(const bool tr = a.trace && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;)
    __syncthreads();  // rank 0's own triple and the neutral ones were written by its threads with plain stores
    HM_TRACE(if (tr) a.trace[4] = a.trace[5] = global_timer();)  // every split's triple has landed
    float* sc_s = scratch;               // [g][NS] scale of every slot's triple (zero for a neutral one)
    float* l_s = scratch + G_MAX * 16;   // [g] merged sums
    for (int i = tid; i < g * NS; i += nthreads) {
        const int jj = i / NS, r = i - jj * NS;
        float ms[NS];
#pragma unroll
        for (int r2 = 0; r2 < NS; ++r2) ms[r2] = c_ml[((size_t)r2 * g + jj) * 2];
        float M = ms[0];
#pragma unroll
        for (int r2 = 1; r2 < NS; ++r2) M = fmaxf(M, ms[r2]);
        const float mine = c_ml[((size_t)r * g + jj) * 2];
        sc_s[i] = mine > -INFINITY ? expf(mine - M) : 0.f;
    }
    __syncthreads();
    HM_TRACE(if (tr) a.trace[10] = global_timer();)
    if (tid < g) {
        float lv[NS];
#pragma unroll
        for (int r = 0; r < NS; ++r) lv[r] = c_ml[((size_t)r * g + tid) * 2 + 1] * sc_s[tid * NS + r];
        float l = 0.f;
#pragma unroll
        for (int r = 0; r < NS; ++r) l += lv[r];
        l_s[tid] = l;
    }
    float o[(G_MAX * HD + ATT_THREADS - 1) / ATT_THREADS];
#pragma unroll
    for (int k = 0; k < (G_MAX * HD + ATT_THREADS - 1) / ATT_THREADS; ++k) {
        const int i = tid + k * nthreads;
        float v = 0.f;
        if (i < g * HD) {
            const int jj = i / HD;
            float sc[NS], cv[NS];
#pragma unroll
            for (int r4 = 0; r4 < NS; r4 += 4) {
                const float4 t4 = *reinterpret_cast<const float4*>(sc_s + jj * NS + r4);
                sc[r4] = t4.x; sc[r4 + 1] = t4.y; sc[r4 + 2] = t4.z; sc[r4 + 3] = t4.w;
            }
#pragma unroll
            for (int r = 0; r < NS; ++r) cv[r] = c_o[(size_t)r * g * HD + i];
#pragma unroll
            for (int r = 0; r < NS; ++r) v = fmaf(cv[r], sc[r], v);
        }
        o[k] = v;
    }
    __syncthreads();
    HM_TRACE(if (tr) a.trace[11] = global_timer();)
#pragma unroll
    for (int k = 0; k < (G_MAX * HD + ATT_THREADS - 1) / ATT_THREADS; ++k) {
        const int i = tid + k * nthreads;
        if (i < g * HD) store_out<HD>(a, m, head0 + i / HD, i % HD, o[k] / l_s[i / HD]);
    }
    HM_TRACE(if (tr) a.trace[12] = global_timer();)
}

// Rank 0 of a (row, KV head) cluster, after every split's (max, sum, acc) triple has landed in its
// shared memory: one scale factor per (slot, head) first (exponentials per slot and head instead of per
// output element), then every output element is a short multiply-add over the slots.
template <int HD>
__device__ __forceinline__ void cluster_rank0_merge(const AttnArgs& a, int g, int head0, int m, float* scratch, const float* c_o, const float* c_ml) {
    const int cap = merge_slot_cap(a.nsplit);
    if (cap == 4) cluster_rank0_merge_n<HD, 4>(a, g, head0, m, scratch, c_o, c_ml);
    else if (cap == 8) cluster_rank0_merge_n<HD, 8>(a, g, head0, m, scratch, c_o, c_ml);
    else cluster_rank0_merge_n<HD, 16>(a, g, head0, m, scratch, c_o, c_ml);
}

// Neutral triples for the slots no split writes: [first, merge_slot_cap(nsplit)).  Rank 0 only, before its merge.
template <int HD>
__device__ __forceinline__ void fill_neutral_slots(const AttnArgs& a, int first, int g, float* c_o, float* c_ml) {
    const int cap = merge_slot_cap(a.nsplit);
    for (int i = first * g * HD + threadIdx.x; i < cap * g * HD; i += blockDim.x) c_o[i] = 0.f;
    for (int i = first * g + threadIdx.x; i < cap * g; i += blockDim.x) {
        c_ml[i * 2] = -INFINITY;
        c_ml[i * 2 + 1] = 0.f;
    }
}

template <int HD, bool CL>
__device__ __forceinline__ void merge_slots_and_write(const AttnArgs& a, int nsub, int g, int head0, int split, int kvh, int m, float* w_ml, float* w_acc, float* c_o, float* c_ml, int* s_last_p,
                                                      uint64_t* rbar = nullptr, volatile int* abortf = nullptr, int nact = -1);

// Cluster splits hand their triples to rank 0 either with plain remote stores followed by a cluster barrier
// (rbar == nullptr), or -- when rank 0 armed an mbarrier for them before the dependency wait -- with
// asynchronous stores that count bytes on that mbarrier, which takes the cluster barrier off the critical path.
__device__ __forceinline__ void push_f32(float* slot_in_rank0, float v, uint32_t rank, uint32_t rbar0) {
    if (rank == 0) *slot_in_rank0 = v;
    else if (rbar0) st_async_f32(dsmem_addr(slot_in_rank0, 0u), v, rbar0);
    else st_dsmem_f32(dsmem_addr(slot_in_rank0, 0u), v);
}
// after the pushes: false for the ranks that are done, true on rank 0 once every triple has landed
__device__ __forceinline__ bool pushes_landed(const AttnArgs& a, uint64_t* rbar, volatile int* abortf) {
    if (rbar) {
        if (cluster_ctarank() != 0) return false;
        return mb_wait_cluster(rbar, 0, a.err_flag, abortf);  // bounded (completes at once when no other split is active)
    }
    cluster_arrive_release();
    if (cluster_ctarank() != 0) return false;
    cluster_wait_acquire();
    return true;
}

// One-head-per-warp kernels: publish the warp's triple at entry (slot * g + head) = warp, then merge.
template <int HD, bool CL>
__device__ __forceinline__ void merge_and_write(const AttnArgs& a, bool active, float run_m, float run_l, const float (&acc)[HD / 32], int nsub, int g, int head0, int split, int kvh, int m, float* w_ml,
                                                float* w_acc, float* c_o, float* c_ml, int* s_last_p, uint64_t* rbar = nullptr, volatile int* abortf = nullptr, int nact = -1) {
    constexpr int EPL = HD / 32;
    if (nact < 0) nact = a.nsplit;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (CL && nsub == 1) {
        // one warp per query head and nothing to merge inside the CTA: every warp stores its triple straight
        // from registers into slot `rank` of rank 0's shared memory
        const uint32_t rank = cluster_ctarank();
        const uint32_t rbar0 = rbar ? dsmem_addr(rbar, 0u) : 0u;
        if (warp < g) {
            // four consecutive output dims per store: a lane's own (hd 128) or an even lane's and its neighbour's (hd 64)
            float4 v4;
            bool sender = true;
            int d0 = lane * EPL;
            if constexpr (EPL == 4) {
                v4 = make_float4(acc[0], acc[1], acc[2], acc[3]);
            } else {
                const float nx = __shfl_down_sync(0xffffffffu, acc[0], 1), ny = __shfl_down_sync(0xffffffffu, acc[EPL - 1], 1);
                v4 = make_float4(acc[0], acc[EPL - 1], nx, ny);
                sender = (lane & 1) == 0;
            }
            float* po = c_o + ((size_t)rank * g + warp) * HD + d0;
            float* pm = c_ml + ((size_t)rank * g + warp) * 2;
            if (rank == 0) {
                if (sender) *reinterpret_cast<float4*>(po) = v4;
                if (lane == 0) {
                    pm[0] = run_m;
                    pm[1] = run_l;
                }
            } else if (rbar0) {
                if (sender) st_async_f32x4(dsmem_addr(po, 0u), v4, rbar0);
                if (lane == 0) st_async_f32x2(dsmem_addr(pm, 0u), run_m, run_l, rbar0);
            } else {
#pragma unroll
                for (int e = 0; e < EPL; ++e) st_dsmem_f32(dsmem_addr(po + e, 0u), acc[e]);
                if (lane == 0) {
                    st_dsmem_f32(dsmem_addr(pm, 0u), run_m);
                    st_dsmem_f32(dsmem_addr(pm + 1, 0u), run_l);
                }
            }
        }
        if (!pushes_landed(a, rbar, abortf)) return;
        cluster_rank0_merge<HD>(a, g, head0, m, w_acc, c_o, c_ml);
        return;
    }
    if (warp < ATT_WARPS) {
        if (lane == 0) {
            w_ml[warp * 2 + 0] = active ? run_m : -INFINITY;
            w_ml[warp * 2 + 1] = active ? run_l : 0.f;
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) w_acc[warp * HD + lane * EPL + e] = active ? acc[e] : 0.f;
    }
    __syncthreads();
    merge_slots_and_write<HD, CL>(a, nsub, g, head0, split, kvh, m, w_ml, w_acc, c_o, c_ml, s_last_p, rbar, abortf, nact);
}

// Merge the (max, sum, acc) triples of nsub page slots per head (entry slot * g + head), then the
// splits of the (row, KV head): through the cluster (rank 0 reads its peers' shared memory in rank
// order), or through global scratch by whichever CTA arrives last at the ticket.
template <int HD, bool CL>
__device__ __forceinline__ void merge_slots_and_write(const AttnArgs& a, int nsub, int g, int head0, int split, int kvh, int m, float* w_ml, float* w_acc, float* c_o, float* c_ml, int* s_last_p, uint64_t* rbar,
                                                      volatile int* abortf, int nact) {
    if (nact < 0) nact = a.nsplit;
    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    int& s_last = *s_last_p;
    for (int i = tid; i < g * HD; i += nthreads) {
        const int jj = i / HD, d = i % HD;
        float M = -INFINITY;
        for (int sb = 0; sb < nsub; ++sb) M = fmaxf(M, w_ml[(sb * g + jj) * 2]);
        float l = 0.f, o = 0.f;
        if (M > -INFINITY) {
            for (int sb = 0; sb < nsub; ++sb) {
                const int w = sb * g + jj;
                const float ms = w_ml[w * 2];
                if (ms > -INFINITY) {
                    const float sc = expf(ms - M);
                    l = fmaf(w_ml[w * 2 + 1], sc, l);
                    o = fmaf(w_acc[w * HD + d], sc, o);
                }
            }
        }
        const int head = head0 + jj;
        if (CL) {
            // push this split's triple into slot `rank` of rank 0's shared memory
            const uint32_t rank = cluster_ctarank();
            const uint32_t rbar0 = rbar ? dsmem_addr(rbar, 0u) : 0u;
            push_f32(c_o + (size_t)rank * g * HD + i, o, rank, rbar0);
            if (d == 0) {
                float* pm = c_ml + ((size_t)rank * g + jj) * 2;
                push_f32(pm, M, rank, rbar0);
                push_f32(pm + 1, l, rank, rbar0);
            }
        } else if (a.nsplit == 1) {
            store_out<HD>(a, m, head, d, o / l);
        } else {
            const size_t pi = ((size_t)m * a.heads + head) * a.nsplit + split;
            a.part_acc[pi * HD + d] = o;
            if (d == 0) {
                a.part_ml[pi * 2 + 0] = M;
                a.part_ml[pi * 2 + 1] = l;
            }
        }
    }
    if (CL) {
        // The splits of one (row, KV head) are the CTAs of one cluster: every rank has pushed its
        // (max, sum, acc) triples into rank 0's shared memory; one barrier later rank 0 merges them in
        // rank order from its own memory and the other ranks are already gone.
        if (!pushes_landed(a, rbar, abortf)) return;
        cluster_rank0_merge<HD>(a, g, head0, m, w_acc, c_o, c_ml);
        return;
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
    for (int i = tid; i < g * HD; i += nthreads) {
        const int jj = i / HD, d = i % HD;
        const int head = head0 + jj;
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
        store_out<HD>(a, m, head, d, o / l);
    }
    if (tid == 0) a.tickets[m * a.kv_heads + kvh] = 0u;
}

template <int HD, bool BF16, bool CL>
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(const AttnArgs a) {
    using TL = Tile<HD, BF16>;
    using T = typename std::conditional<BF16, uint16_t, float>::type;
    constexpr int EPL = HD / 32;  // output elements per lane
    extern __shared__ __align__(16) float sm[];
    const int g = a.heads / a.kv_heads;
    const int nsub = pick_nsub<HD, BF16>(g);  // page slots worked on concurrently
    const int nslots = pick_nslots<HD, BF16>(g, a.early_pages, a.max_pages, a.nsplit);
    const bool resident = nslots * a.nsplit >= a.max_pages && a.early_pages >= 2;  // one slot per page of this CTA
    float* q_s = sm;                              // [G_MAX][HD]
    float* tiles = q_s + G_MAX * HD;              // [nslots][K tile | V tile]
    float* p_s = tiles + nslots * TL::SLOT_FLOATS;  // [ATT_WARPS][16]
    float* w_ml = p_s + ATT_WARPS * PT;           // [ATT_WARPS][2]
    float* w_acc = w_ml + ATT_WARPS * 2;          // [ATT_WARPS][HD]
    float* c_o = w_acc + ATT_WARPS * HD;          // cluster mode, rank 0: [nsplit][g][HD] triples pushed by the ranks
    float* c_ml = c_o + (CL ? merge_slot_cap(a.nsplit) : 1) * g * HD;  // [slots][g][2]
    __shared__ int s_last;
    __shared__ uint64_t s_rbar;  // cluster mode, rank 0: counts the bytes of the other splits' triples
    __shared__ volatile int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
    const int head0 = kvh * g;
    HM_TRACE(const bool tr = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tid == 0;)
    HM_TRACE(if (tr) a.trace[0] = global_timer();)  // CTA resident
    HM_TRACE(if (a.trace && tid == 0) atomicMax(a.trace + 8, global_timer());)  // the launch's last CTA to become resident

    pdl_launch_dependents();
    if (a.pf_bytes && tid < 32)
        l2_prefetch_slice(a.pf_ptr, a.pf_bytes, (int)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x), (int)(gridDim.x * gridDim.y * gridDim.z), tid);

    // Lengths, positions and the page table were written before the launch chain of this step began,
    // so the page range can be worked out before the dependency wait.  With early_pages set (decode:
    // one row per sequence) the pages BELOW the one that receives this step's token are final too and
    // are read now -- into their own slots when the CTA's pages all fit (resident), else only the
    // first group's loads are issued; the page of the new token (written by the preceding QKV kernel)
    // and the query are read after the wait.
    const int seq = a.row_seq ? a.row_seq[m] : m;
    const int kvlen = a.kv_len ? a.kv_len[m] : a.row_pos[m] + 1;
    const int npages = (kvlen + PT - 1) / PT;
    const int pps = (npages + a.nsplit - 1) / a.nsplit;
    const int p0 = split * pps, p1 = min(npages, p0 + pps);
    const int32_t* pt = a.page_table + (size_t)seq * a.max_pages;
    const T* kpool = reinterpret_cast<const T*>(a.k_pool);
    const T* vpool = reinterpret_cast<const T*>(a.v_pool);
    const int safe_end = a.early_pages ? min(p1, (kvlen - 1) / PT) : p0;  // pages [p0, safe_end) may be read early
    const int nact = pps > 0 ? (npages + pps - 1) / pps : 1;  // splits that have pages (known to every split: lengths are final before the chain starts)

    // cooperative tile loads: thread -> (slot, piece) pairs, the same mapping for every group
    const int total_pieces = nsub * TL::PIECES;  // per K (and per V), <= MAXP * ATT_THREADS
    uint4 kreg[MAXP], vreg[MAXP];
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
        kreg[i] = make_uint4(0, 0, 0, 0);
        vreg[i] = make_uint4(0, 0, 0, 0);
    }
    // loads the slots of the group starting at page pbase whose page lies in [lo, hi)
    auto issue_loads = [&](int pbase, int lo, int hi) {
#pragma unroll
        for (int i = 0; i < MAXP; ++i) {
            const int idx = tid + i * ATT_THREADS;
            if (idx < total_pieces) {
                const int slot = idx / TL::PIECES, piece = idx % TL::PIECES;
                const int p = pbase + slot;
                if (p >= lo && p < hi) {
                    const size_t tile = ((size_t)pt[p] * a.kv_heads + kvh) * PT * HD;
                    kreg[i] = __ldg(reinterpret_cast<const uint4*>(kpool + tile) + piece);
                    vreg[i] = __ldg(reinterpret_cast<const uint4*>(vpool + tile) + piece);
                }
            }
        }
    };
    // stores the group's registers into slots slot_base.., only the pages in [lo, hi)
    auto store_tiles = [&](int slot_base, int pbase, int lo, int hi) {
#pragma unroll
        for (int i = 0; i < MAXP; ++i) {
            const int idx = tid + i * ATT_THREADS;
            if (idx < total_pieces) {
                const int slot = idx / TL::PIECES, piece = idx % TL::PIECES;
                const int p = pbase + slot;
                if (p >= lo && p < hi) {
                    const int e = piece * TL::PER16;
                    float* base = tiles + (slot_base + slot) * TL::SLOT_FLOATS;
                    // K pages are chunk-major (k_tile_off) and stay so in shared memory: a straight copy;
                    // V pages (bf16: chunks of 8 elements, v_tile_off; f32: rows already) become rows [token][dim] here
                    const int vt_tok = BF16 ? (e >> 3) & (PT - 1) : e / HD, vd = BF16 ? ((e >> 7) << 3) | (e & 7) : e % HD;
                    unpack_store<BF16>(base + e, kreg[i]);
                    unpack_store<BF16>(base + PT * TL::KLD + vt_tok * HD + vd, vreg[i]);
                }
            }
        }
    };
    if (CL) {
        // arm rank 0's mbarrier for the triples of the other splits and publish it with a cluster barrier
        // that happens before the dependency wait, off the dependent-kernel chain
        if (tid == 0) {
            s_abort = 0;
            if (cluster_ctarank() == 0) {
                mb_init(&s_rbar, 1);
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                mb_expect_tx(&s_rbar, (uint32_t)(nact - 1) * (uint32_t)(g * (HD + 2)) * 4u);
            }
        }
        if (cluster_ctarank() == 0) fill_neutral_slots<HD>(a, nact, g, c_o, c_ml);  // slots no split will write
        cluster_arrive_release();
        cluster_wait_acquire();
        if (p0 >= p1 && cluster_ctarank() != 0) return;  // a split without pages sends nothing and is not waited for
    }
    if (resident) {
#pragma unroll 1
        for (int pb = p0; pb < safe_end; pb += nsub) {
            issue_loads(pb, pb, safe_end);
            store_tiles(pb - p0, pb, pb, safe_end);
        }
    } else if (p0 < safe_end) {
        issue_loads(p0, p0, safe_end);
    }
    pdl_wait();
    HM_TRACE(if (tr) a.trace[1] = global_timer();)  // predecessor complete

    const int late0 = max(p0, safe_end);  // [late0, p1): at most the page that holds the new token
    if (resident) {
        if (late0 < p1) {
            const int pb = p0 + (late0 - p0) / nsub * nsub;
            issue_loads(pb, late0, p1);
        }
    } else if (p0 < p1) {
        issue_loads(p0, late0, p1);
    }
    stage_row<ATT_THREADS, false>(a.q + (size_t)m * a.heads * HD + head0 * HD, q_s, g * HD, tid);

    const int j = warp % g, sub = warp / g;  // this warp's query head and page slot
    const bool active = sub < nsub;
    float run_m = -INFINITY, run_l = 0.f, acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
    const int t = lane & 15, hf = lane >> 4;
    float* pw = p_s + warp * PT;

    // one page of this warp's query head: 16 scores, online-softmax update, p . v
    auto page = [&](int p, const float* kt) {
        const float* vt = kt + PT * TL::KLD;
        const float* kr = kt + ((hf * (HD / 8) * PT + t) << 2);  // chunk-major: chunk c of token t at (c * 16 + t) * 4
        const float* qr = q_s + j * HD + hf * (HD / 2);
        float s = 0.f, s2 = 0.f;  // two chains: the dot product is latency, not throughput
#pragma unroll
        for (int dc = 0; dc < HD / 2; dc += 8) {
            const float4 k4 = *reinterpret_cast<const float4*>(kr + dc * PT);
            const float4 q4 = *reinterpret_cast<const float4*>(qr + dc);
            const float4 k5 = *reinterpret_cast<const float4*>(kr + (dc + 4) * PT);
            const float4 q5 = *reinterpret_cast<const float4*>(qr + dc + 4);
            s = fmaf(q4.x, k4.x, s);
            s2 = fmaf(q5.x, k5.x, s2);
            s = fmaf(q4.y, k4.y, s);
            s2 = fmaf(q5.y, k5.y, s2);
            s = fmaf(q4.z, k4.z, s);
            s2 = fmaf(q5.z, k5.z, s2);
            s = fmaf(q4.w, k4.w, s);
            s2 = fmaf(q5.w, k5.w, s2);
        }
        s += s2;
        s += __shfl_xor_sync(0xffffffffu, s, 16);
        const bool valid = (p * PT + t) < kvlen;
        const float sc = valid ? s * a.scale : -INFINITY;
        float mx = sc;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(run_m, mx);
        const float pr = valid ? expf(sc - m_new) : 0.f;
        float ps = pr;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        const float corr = expf(run_m - m_new);  // exp(-inf) = 0 on the first page
        run_l = run_l * corr + ps;
        run_m = m_new;
        if (hf == 0) pw[t] = pr;
        __syncwarp();
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] *= corr;
#pragma unroll
        for (int tt = 0; tt < PT; ++tt) {
            const float pv = pw[tt];
#pragma unroll
            for (int e = 0; e < EPL; ++e) acc[e] = fmaf(pv, vt[tt * HD + lane * EPL + e], acc[e]);
        }
        __syncwarp();
    };

    if (resident) {
        if (late0 < p1) {
            const int pb = p0 + (late0 - p0) / nsub * nsub;
            store_tiles(pb - p0, pb, late0, p1);
        }
        __syncthreads();  // every page of this CTA and the query are in shared memory
        HM_TRACE(if (tr) a.trace[2] = global_timer();)
        if (active)
            for (int p = p0 + sub; p < p1; p += nsub) page(p, tiles + (p - p0) * TL::SLOT_FLOATS);
    } else {
        for (int pb = p0; pb < p1; pb += nsub) {
            __syncthreads();  // previous group's tiles are no longer being read (also publishes q_s)
            store_tiles(0, pb, pb, p1);
            __syncthreads();
            if (pb + nsub < p1) issue_loads(pb + nsub, pb + nsub, p1);  // next group in flight during the math
            const int p = pb + sub;
            if (active && p < p1) page(p, tiles + sub * TL::SLOT_FLOATS);
        }
    }

    HM_TRACE(if (tr) a.trace[3] = global_timer();)  // this warp's pages done
    HM_TRACE(if (a.trace && tid == 0 && blockIdx.y == 0 && blockIdx.z == 0 && late0 < p1) a.trace[7] = global_timer();)  // the split that holds the new token is done
    merge_and_write<HD, CL>(a, active, run_m, run_l, acc, nsub, g, head0, split, kvh, m, w_ml, w_acc, c_o, c_ml, &s_last, CL ? &s_rbar : nullptr, &s_abort, CL ? nact : -1);
    HM_TRACE(if (tr) a.trace[6] = global_timer();)  // merged and stored (rank 0 of the cluster)
    HM_TRACE(if (a.trace && tid == 0) atomicMax(a.trace + 9, global_timer());)  // the launch's last rank 0 to finish
}

// ---- streaming variant for long contexts ---------------------------------------------------------
// Same (row, KV head, split) decomposition, but built for bandwidth: the pages arrive through a ring
// of shared-memory stages filled by cp.async.bulk (a K tile or a V tile of a page is one contiguous
// block of the pool, so the ninth warp's elected thread issues two bulk copies per page, up to
// ST_RING_BYTES ahead) and each of the eight consumer warps takes whole pages, round-robin, for ALL g
// query heads of the KV head: a K chunk is read from shared memory once and used g times (the
// chunk-major K tile makes that read conflict-free while the query chunk is a broadcast), and a V row
// is read once per token for g heads.  That cuts shared-memory traffic per page by about 3x against
// one-warp-per-head, which is what bounds the kernel above on long contexts.  Used when a CTA has at
// least ST_MIN_PAGES pages to read.
constexpr int ST_THREADS = ATT_THREADS + 32;
constexpr int ST_MAX_STAGES = 24;
constexpr int ST_RING_BYTES = 64 * 1024;  // per CTA; two CTAs per SM keep 128 KB of pages in flight
constexpr int ST_MAX_PT = 4096;  // page-table entries of one CTA staged in shared memory

template <int HD, bool BF16>
struct StTile {
    static constexpr int ESZ = BF16 ? 2 : 4;
    static constexpr int TILE_BYTES = PT * HD * ESZ;  // one K or V tile
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    // 64 KB of pages per CTA (two CTAs per SM); f32 pages of head_dim 128 get 128 KB so that eight warps
    // still have a stage each
    static constexpr int RING = STAGE_BYTES * ATT_WARPS > ST_RING_BYTES ? STAGE_BYTES * ATT_WARPS : ST_RING_BYTES;
    static constexpr int STAGES = (RING / STAGE_BYTES) < ST_MAX_STAGES ? (RING / STAGE_BYTES) : ST_MAX_STAGES;
    // Consumer warps that take pages round-robin.  Every phase of a stage must be consumed by the same
    // warp (a parity wait cannot tell phase k from phase k + 2), so the stage count is a multiple of it.
    static constexpr int CW = STAGES < ATT_WARPS ? STAGES : ATT_WARPS;
    static_assert(STAGES % CW == 0, "stage count must be a multiple of the consumer warp count");
};

template <bool BF16>
__device__ __forceinline__ float4 ld_chunk4(const void* tile, int elem) {  // 4 consecutive elements as f32
    if (BF16) {
        const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(tile) + elem);
        return make_float4(bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
    }
    return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(tile) + elem);
}

// ---- bf16 pages on the tensor cores ---------------------------------------------------------------
// With six or seven query heads per KV head the f32 FMAs of a page outweigh its bytes (6 flop per byte of bf16
// cache), so on bf16 pages the two contractions of a page run as warp-level MMAs (m16n8k16, f32 accumulate):
//   scores^T [16 tokens x 8 heads]  = K tile [16 tokens x hd]   . Q^T [hd x 8 heads]
//   out^T    [hd x 8 heads]        += V^T    [hd x 16 tokens]   . P^T [16 tokens x 8 heads]
// K and V are bf16 already; the f32 operands (Q, P) are split into three bf16 terms each (hi + mid + lo is
// exact to 2^-24), one MMA per term, so the products are the f32 x bf16 products of the reference and only
// the order of the f32 accumulation differs.  (The 8 heads of the MMA's N are the <= 8 query heads of the
// KV head: the floordiv head map again.)
__device__ __forceinline__ void mma_bf16_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// four 8x8 bf16 matrices, each delivered transposed (thread i supplies the address of row i % 8 of matrix i / 8)
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s32(row_addr)));
}
// two f32 values -> their three bf16 terms, packed (x low half, y high half)
__device__ __forceinline__ void split3_pack(float x, float y, uint32_t (&t)[3]) {
    const uint16_t hx = f32_to_bf16_rne(x), hy = f32_to_bf16_rne(y);
    const float rx = x - bf16_bits_to_f32(hx), ry = y - bf16_bits_to_f32(hy);
    const uint16_t mx = f32_to_bf16_rne(rx), my = f32_to_bf16_rne(ry);
    const uint16_t lx = f32_to_bf16_rne(rx - bf16_bits_to_f32(mx)), ly = f32_to_bf16_rne(ry - bf16_bits_to_f32(my));
    t[0] = (uint32_t)hx | ((uint32_t)hy << 16);
    t[1] = (uint32_t)mx | ((uint32_t)my << 16);
    t[2] = (uint32_t)lx | ((uint32_t)ly << 16);
}
__host__ __device__ constexpr size_t st_q_bytes(int hd) { return 3 * (size_t)(hd / 16) * 32 * 8 > (size_t)G_MAX * hd * 4 ? 3 * (size_t)(hd / 16) * 32 * 8 : (size_t)G_MAX * hd * 4; }

template <int HD, bool BF16, bool CL>
__global__ void __launch_bounds__(ST_THREADS, 2) attn_stream_kernel(const AttnArgs a) {
    using ST = StTile<HD, BF16>;
    using T = typename std::conditional<BF16, uint16_t, float>::type;
    constexpr int EPL = HD / 32;
    constexpr int NCH = HD / 8;  // 4-element chunks per half row (lane = token, half)
    extern __shared__ __align__(128) unsigned char st_sm[];
    unsigned char* ring = st_sm;                                                 // [STAGES][K tile | V tile]
    const int NST = a.st_stages;  // ST::STAGES, or more when the launch has an SM to itself per CTA (see launch_tc)
    float* q_s = reinterpret_cast<float*>(ring + NST * ST::STAGE_BYTES);  // f32 pages: [G_MAX][NCH][2 halves][4]; bf16 pages: MMA fragments [3 terms][HD/16][32 lanes] x 8 B
    float* p_s = q_s + st_q_bytes(HD) / 4;                                       // [ATT_WARPS][G_MAX][16]
    const int g_early = a.heads / a.kv_heads;
    float* c_o = p_s + ATT_WARPS * G_MAX * PT;                                   // cluster mode, rank 0: [nsplit][g][HD]
    float* c_ml = c_o + (CL ? merge_slot_cap(a.nsplit) : 1) * g_early * HD;     // [slots][g][2]
    // the per-warp results reuse the ring once every page has been consumed
    float* w_ml = reinterpret_cast<float*>(ring);                                // [ATT_WARPS * g][2]
    float* w_acc = w_ml + ATT_WARPS * G_MAX * 2;                                 // [ATT_WARPS * g][HD]
    static_assert(sizeof(float) * (ATT_WARPS * G_MAX * 2 + ATT_WARPS * G_MAX * HD) <= (size_t)ST::STAGES * ST::STAGE_BYTES, "ring too small for the merge scratch");
    int32_t* pt_s = reinterpret_cast<int32_t*>(c_ml + (CL ? merge_slot_cap(a.nsplit) : 1) * g_early * 2);  // [pages of this CTA]
    __shared__ uint64_t full[ST_MAX_STAGES], empty[ST_MAX_STAGES];
    __shared__ int s_last;
    __shared__ volatile int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
    const int g = a.heads / a.kv_heads;
    const int head0 = kvh * g;

    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mb_init(&full[s], 1);
            mb_init(&empty[s], 1);
        }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_launch_dependents();
    if (a.pf_bytes && tid < 32)
        l2_prefetch_slice(a.pf_ptr, a.pf_bytes, (int)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x), (int)(gridDim.x * gridDim.y * gridDim.z), tid);
    if (CL && cluster_ctarank() == 0) fill_neutral_slots<HD>(a, a.nsplit, g, c_o, c_ml);  // merge slots past the split count
    // Decode passes (one row per sequence, early_pages != 0): lengths and the page table were final before this
    // step's launches began, and every page below the one that receives the new token is complete, so the page
    // table is read and the first ring-full of those pages requested BEFORE the dependency wait.  Prefill chunks
    // (several rows of one sequence, pages being written by the launch before this one) wait first.
    const bool early = a.early_pages != 0;
    if (!early) pdl_wait();

    const int seq = a.row_seq ? a.row_seq[m] : m;
    const int kvlen = a.kv_len ? a.kv_len[m] : a.row_pos[m] + 1;
    const int npages = (kvlen + PT - 1) / PT;
    const int pps = (npages + a.nsplit - 1) / a.nsplit;
    const int p0 = split * pps, p1 = min(npages, p0 + pps);
    const int np = max(0, p1 - p0);
    const int32_t* pt = a.page_table + (size_t)seq * a.max_pages;
    for (int i = tid; i < np; i += ST_THREADS) pt_s[i] = pt[p0 + i];
    int n_pre = 0;  // pages requested before the dependency wait (producer thread only)
    if (early) {
        __syncthreads();
        if (warp == ATT_WARPS && lane == 0) {
            using TE = typename std::conditional<BF16, uint16_t, float>::type;
            const TE* kpool = reinterpret_cast<const TE*>(a.k_pool);
            const TE* vpool = reinterpret_cast<const TE*>(a.v_pool);
            const int new_page = (kvlen - 1) / PT;  // the page the new token's K/V are being written to
            while (n_pre < np && n_pre < NST && p0 + n_pre < new_page) {
                const size_t tile = ((size_t)pt_s[n_pre] * a.kv_heads + kvh) * PT * HD;
                unsigned char* dst = ring + (size_t)n_pre * ST::STAGE_BYTES;
                mb_expect_tx(&full[n_pre], ST::STAGE_BYTES);
                bulk_copy(dst, kpool + tile, ST::TILE_BYTES, &full[n_pre]);
                bulk_copy(dst + ST::TILE_BYTES, vpool + tile, ST::TILE_BYTES, &full[n_pre]);
                ++n_pre;
            }
        }
        pdl_wait();
    }
    if constexpr (BF16) {
        // B fragments of Q^T for every 16-dim step: lane (head = lane / 4, pair = lane % 4) holds dims 2*pair, 2*pair+1
        // (b0) and 2*pair+8, 2*pair+9 (b1) of its head, per bf16 term; heads beyond g are zero
        uint2* qf = reinterpret_cast<uint2*>(q_s);
        for (int i = tid; i < (HD / 16) * 32; i += ST_THREADS) {
            const int kt = i >> 5, ln = i & 31, hh = ln >> 2, d0 = kt * 16 + (ln & 3) * 2;
            uint32_t lo[3] = {0u, 0u, 0u}, hi[3] = {0u, 0u, 0u};
            if (hh < g) {
                const float* qr = a.q + (size_t)m * a.heads * HD + (size_t)(head0 + hh) * HD + d0;
                split3_pack(qr[0], qr[1], lo);
                split3_pack(qr[8], qr[9], hi);
            }
#pragma unroll
            for (int t3 = 0; t3 < 3; ++t3) qf[(t3 * (HD / 16) + kt) * 32 + ln] = make_uint2(lo[t3], hi[t3]);
        }
    } else {
        // query rows re-ordered so that the two halves' copies of chunk c are adjacent: q_s[j][c][half][4]
        for (int i = tid; i < g * HD; i += ST_THREADS) {
            const int jj = i / HD, d = i % HD;
            const int hfq = d / (HD / 2), c = (d % (HD / 2)) >> 2;
            q_s[jj * HD + (c * 2 + hfq) * 4 + (d & 3)] = a.q[(size_t)m * a.heads * HD + (head0 + jj) * HD + d];
        }
    }
    __syncthreads();

    // tensor-core path (bf16 pages): running state of heads 2 * (lane % 4) and 2 * (lane % 4) + 1, out^T accumulators
    float tm[2] = {-INFINITY, -INFINITY}, tl[2] = {0.f, 0.f};
    float to[BF16 ? HD / 16 : 1][4];
#pragma unroll
    for (int mt = 0; mt < (BF16 ? HD / 16 : 1); ++mt) to[mt][0] = to[mt][1] = to[mt][2] = to[mt][3] = 0.f;
    // per-warp running softmax state of every head; the page loop leaves warps with different maxima
    float run_m[G_MAX], run_l[G_MAX], acc[G_MAX][EPL];
#pragma unroll
    for (int jj = 0; jj < G_MAX; ++jj) {
        run_m[jj] = -INFINITY;
        run_l[jj] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[jj][e] = 0.f;
    }

    if (warp == ATT_WARPS) {
        // ---- producer: two bulk copies per page, as far ahead as the ring allows ----
        if (lane == 0) {
            const T* kpool = reinterpret_cast<const T*>(a.k_pool);
            const T* vpool = reinterpret_cast<const T*>(a.v_pool);
            // stage and phase advance with the page index (no division in the loop: the ring depth is a run-time value)
            int s = n_pre % NST;
            uint32_t par = ((n_pre / NST) & 1u) ^ 1u;
            for (int i = n_pre; i < np; ++i, ++s) {
                if (s == NST) {
                    s = 0;
                    par ^= 1u;
                }
                if (!mb_wait(&empty[s], par, a.err_flag, &s_abort)) break;
                const size_t tile = ((size_t)pt_s[i] * a.kv_heads + kvh) * PT * HD;
                unsigned char* dst = ring + (size_t)s * ST::STAGE_BYTES;
                mb_expect_tx(&full[s], ST::STAGE_BYTES);
                bulk_copy(dst, kpool + tile, ST::TILE_BYTES, &full[s]);
                bulk_copy(dst + ST::TILE_BYTES, vpool + tile, ST::TILE_BYTES, &full[s]);
            }
        }
    } else if (warp < ST::CW && BF16) {
        if constexpr (BF16) {
            const int gid = lane >> 2, tig = lane & 3;
            float* pw = p_s + warp * (G_MAX * PT);  // [8 heads][16 tokens]: the page's probabilities, transposed for the second MMA
            const uint2* qf = reinterpret_cast<const uint2*>(q_s);
            int s = warp;  // this warp's pages: i = warp, warp + 8, ...; their stages advance by 8 modulo the ring depth
            uint32_t par = 0u;
            for (int i = warp; i < np; i += ST::CW, s += ST::CW) {
                if (s >= NST) {
                    s -= NST;
                    par ^= 1u;
                }
                const bool ok = __all_sync(0xffffffffu, mb_wait(&full[s], par, a.err_flag, &s_abort));
                if (!ok) break;
                const uint32_t* kt32 = reinterpret_cast<const uint32_t*>(ring + (size_t)s * ST::STAGE_BYTES);
                const unsigned char* vt = ring + (size_t)s * ST::STAGE_BYTES + ST::TILE_BYTES;
                const int p = p0 + i;
                // ---- scores^T = K tile . Q^T ----
                float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int kt = 0; kt < HD / 16; ++kt) {
                    // chunk-major K tile: element (token, dim) at ((dim / 4) * 16 + token) * 4 + dim % 4
                    const int w0 = ((kt * 4 + (tig >> 1)) * 16 + gid) * 2 + (tig & 1);
                    const uint32_t a0 = kt32[w0], a1 = kt32[w0 + 16], a2 = kt32[w0 + 64], a3 = kt32[w0 + 80];
#pragma unroll
                    for (int t3 = 0; t3 < 3; ++t3) {
                        const uint2 b = qf[(t3 * (HD / 16) + kt) * 32 + lane];
                        mma_bf16_m16n8k16(sc, a0, a1, a2, a3, b.x, b.y);
                    }
                }
                // ---- online softmax: this thread follows heads 2*tig and 2*tig+1 (replicated over the 8 token lanes) ----
                const bool v0 = (p * PT + gid) < kvlen, v1 = (p * PT + gid + 8) < kvlen;
                float corr[2];
                float pr[4];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const float s0 = v0 ? sc[hh] * a.scale : -INFINITY, s1 = v1 ? sc[2 + hh] * a.scale : -INFINITY;
                    float mx = fmaxf(s0, s1);
#pragma unroll
                    for (int o = 4; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    const float m_new = fmaxf(tm[hh], mx);
                    const float p0v = v0 ? expf(s0 - m_new) : 0.f, p1v = v1 ? expf(s1 - m_new) : 0.f;
                    float ps = p0v + p1v;
#pragma unroll
                    for (int o = 4; o < 32; o <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
                    corr[hh] = expf(tm[hh] - m_new);  // exp(-inf) = 0 on the first page
                    tl[hh] = tl[hh] * corr[hh] + ps;
                    tm[hh] = m_new;
                    pr[hh] = p0v;
                    pr[2 + hh] = p1v;
                }
                pw[(tig * 2) * PT + gid] = pr[0];
                pw[(tig * 2 + 1) * PT + gid] = pr[1];
                pw[(tig * 2) * PT + gid + 8] = pr[2];
                pw[(tig * 2 + 1) * PT + gid + 8] = pr[3];
                __syncwarp();
                uint32_t b0[3], b1[3];  // P^T fragments: head = gid, tokens 2*tig, 2*tig+1 and +8
                {
                    const float2 x = *reinterpret_cast<const float2*>(pw + gid * PT + tig * 2), y = *reinterpret_cast<const float2*>(pw + gid * PT + tig * 2 + 8);
                    split3_pack(x.x, x.y, b0);
                    split3_pack(y.x, y.y, b1);
                }
                __syncwarp();
                // ---- out^T += V^T . P^T ----
                const int mj = lane >> 3, mr = lane & 7;  // ldmatrix: this lane addresses row mr of matrix mj
                // V tile: chunks of 8 dims, V[d / 8][token][d % 8]; matrix mj = tokens (mj / 2) * 8 .. + 7 of chunk 2 * mt + mj % 2
                const unsigned char* vrow = vt + ((size_t)((mj & 1) * PT + (mj >> 1) * 8 + mr) * 8) * 2;
#pragma unroll
                for (int mt = 0; mt < HD / 16; ++mt) {
                    to[mt][0] *= corr[0];
                    to[mt][1] *= corr[1];
                    to[mt][2] *= corr[0];
                    to[mt][3] *= corr[1];
                    uint32_t av[4];
                    ldmatrix_x4_trans(av, vrow + (size_t)mt * (2 * PT * 8 * 2));
#pragma unroll
                    for (int t3 = 0; t3 < 3; ++t3) mma_bf16_m16n8k16(to[mt], av[0], av[1], av[2], av[3], b0[t3], b1[t3]);
                }
                __syncwarp();
                if (lane == 0) mb_arrive(&empty[s]);  // the stage may be refilled
            }
        }
    } else if (warp < ST::CW) {
        const int t = lane & 15, hf = lane >> 4;
        float* pw = p_s + warp * (G_MAX * PT);
        int s = warp;  // this warp's pages and their stages, as above
        uint32_t par = 0u;
        for (int i = warp; i < np; i += ST::CW, s += ST::CW) {
            if (s >= NST) {
                s -= NST;
                par ^= 1u;
            }
            const bool ok = __all_sync(0xffffffffu, mb_wait(&full[s], par, a.err_flag, &s_abort));
            if (!ok) break;
            const unsigned char* kt = ring + (size_t)s * ST::STAGE_BYTES;
            const unsigned char* vt = kt + ST::TILE_BYTES;
            const int p = p0 + i;
            // ---- scores of the 16 tokens against all g heads: lane = (token, half of hd) ----
            // packed f32x2 FMAs: even and odd elements of a chunk accumulate in the two halves of a pair
            float2 sc2[G_MAX];
#pragma unroll
            for (int jj = 0; jj < G_MAX; ++jj) sc2[jj] = make_float2(0.f, 0.f);
#pragma unroll 4
            for (int c = 0; c < NCH; ++c) {
                const float4 k4 = ld_chunk4<BF16>(kt, (((hf * NCH + c) << 4) + t) << 2);  // chunk-major K tile
#pragma unroll
                for (int jj = 0; jj < G_MAX; ++jj) {
                    if (jj < g) {
                        const float4 q4 = *reinterpret_cast<const float4*>(q_s + jj * HD + (c * 2 + hf) * 4);
                        sc2[jj] = __ffma2_rn(make_float2(q4.x, q4.y), make_float2(k4.x, k4.y), sc2[jj]);
                        sc2[jj] = __ffma2_rn(make_float2(q4.z, q4.w), make_float2(k4.z, k4.w), sc2[jj]);
                    }
                }
            }
            float sc[G_MAX];
#pragma unroll
            for (int jj = 0; jj < G_MAX; ++jj) sc[jj] = sc2[jj].x + sc2[jj].y;
            const bool valid = (p * PT + t) < kvlen;
            float corr[G_MAX];
#pragma unroll
            for (int jj = 0; jj < G_MAX; ++jj) {
                if (jj < g) {
                    float sv = sc[jj] + __shfl_xor_sync(0xffffffffu, sc[jj], 16);
                    sv = valid ? sv * a.scale : -INFINITY;
                    float mx = sv;
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    const float m_new = fmaxf(run_m[jj], mx);
                    const float pr = valid ? expf(sv - m_new) : 0.f;
                    float ps = pr;
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
                    corr[jj] = expf(run_m[jj] - m_new);  // exp(-inf) = 0 on the first page
                    run_l[jj] = run_l[jj] * corr[jj] + ps;
                    run_m[jj] = m_new;
                    if (hf == 0) pw[jj * PT + t] = pr;
                }
            }
            __syncwarp();
            // ---- p . v: lane owns EPL output dims of every head; a V row is read once for all heads ----
#pragma unroll
            for (int jj = 0; jj < G_MAX; ++jj)
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[jj][e] *= (jj < g) ? corr[jj] : 1.f;
#pragma unroll
            for (int t4 = 0; t4 < PT; t4 += 4) {
                float vv[4][EPL];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (BF16) {
                        const uint16_t* vr = reinterpret_cast<const uint16_t*>(vt) + v_tile_off(t4 + u, lane * EPL, HD, BF16 ? 1 : 0);
#pragma unroll
                        for (int e = 0; e < EPL; ++e) vv[u][e] = bf16_bits_to_f32(vr[e]);
                    } else {
                        const float* vr = reinterpret_cast<const float*>(vt) + v_tile_off(t4 + u, lane * EPL, HD, BF16 ? 1 : 0);
#pragma unroll
                        for (int e = 0; e < EPL; ++e) vv[u][e] = vr[e];
                    }
                }
#pragma unroll
                for (int jj = 0; jj < G_MAX; ++jj) {
                    if (jj < g) {
                        const float4 p4 = *reinterpret_cast<const float4*>(pw + jj * PT + t4);  // broadcast
#pragma unroll
                        for (int e = 0; e < EPL; ++e) {
                            acc[jj][e] = fmaf(p4.x, vv[0][e], acc[jj][e]);
                            acc[jj][e] = fmaf(p4.y, vv[1][e], acc[jj][e]);
                            acc[jj][e] = fmaf(p4.z, vv[2][e], acc[jj][e]);
                            acc[jj][e] = fmaf(p4.w, vv[3][e], acc[jj][e]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mb_arrive(&empty[s]);  // the stage may be refilled
        }
    }
    __syncthreads();  // every page consumed: the ring becomes the merge scratch
    if (warp < ST::CW && BF16) {
        const int gid = lane >> 2, tig = lane & 3;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int jj = tig * 2 + hh;
            if (jj < g) {
                const int w = warp * g + jj;
                if (gid == 0) {
                    w_ml[w * 2 + 0] = tm[hh];
                    w_ml[w * 2 + 1] = tl[hh];
                }
#pragma unroll
                for (int mt = 0; mt < (BF16 ? HD / 16 : 1); ++mt) {
                    w_acc[w * HD + mt * 16 + gid] = to[mt][hh];
                    w_acc[w * HD + mt * 16 + gid + 8] = to[mt][2 + hh];
                }
            }
        }
    } else if (warp < ST::CW) {
        // publish this warp's state: slot = warp, entry (warp * g + head)
#pragma unroll
        for (int jj = 0; jj < G_MAX; ++jj) {
            if (jj < g) {
                const int w = warp * g + jj;
                if (lane == 0) {
                    w_ml[w * 2 + 0] = run_m[jj];
                    w_ml[w * 2 + 1] = run_l[jj];
                }
#pragma unroll
                for (int e = 0; e < EPL; ++e) w_acc[w * HD + lane * EPL + e] = acc[jj][e];
            }
        }
    }
    __syncthreads();
    merge_slots_and_write<HD, CL>(a, ST::CW, g, head0, split, kvh, m, w_ml, w_acc, c_o, c_ml, &s_last);
}

template <int HD, bool BF16>
size_t stream_smem_bytes(int pages_per_cta, int g, int slots, int stages) {
    using ST = StTile<HD, BF16>;
    return (size_t)stages * ST::STAGE_BYTES + st_q_bytes(HD) + sizeof(float) * (ATT_WARPS * G_MAX * PT + (size_t)slots * g * (HD + 2)) + (size_t)pages_per_cta * 4 + 128;
}

template <int HD, bool BF16>
size_t smem_bytes(int g, int slots, int nslots) {
    using TL = Tile<HD, BF16>;
    return sizeof(float) * ((size_t)G_MAX * HD + (size_t)nslots * TL::SLOT_FLOATS + ATT_WARPS * PT + ATT_WARPS * 2 + ATT_WARPS * HD + (size_t)slots * g * (HD + 2));
}

template <int HD, bool BF16, bool CL>
cudaError_t launch_tc(const AttnArgs& a, int M, cudaStream_t st, bool pdl) {
    const int g = a.heads / a.kv_heads;
    const int pages_per_cta = (a.max_pages + a.nsplit - 1) / a.nsplit;
    // long contexts: the bulk-copy ring; a slot layout needs ATT_WARPS / g >= 1 as in the kernel above
    const bool stream = a.stream_pages > 0 && pages_per_cta >= ST_MIN_PAGES && pages_per_cta <= ST_MAX_PT;
    const int slots = CL ? merge_slot_cap(a.nsplit) : 1;  // rank 0 of a cluster receives every split's triples
    // The ring bounds what one CTA keeps in flight (a warp asks for its next page only when it has freed a stage).
    // Launches that leave every CTA an SM to itself (64 sequences x 2 KV heads, one split: 128 CTAs) get as deep a
    // ring as shared memory holds, in multiples of the eight consumer warps; larger launches keep two CTAs per SM.
    using STT = StTile<HD, BF16>;
    int stages = STT::STAGES;
    if (stream) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if ((long)a.nsplit * a.kv_heads * M <= sms) {
            const int want = std::min(ST_MAX_STAGES, (pages_per_cta + ATT_WARPS - 1) / ATT_WARPS * ATT_WARPS);
            while (stages + ATT_WARPS <= want && stream_smem_bytes<HD, BF16>(pages_per_cta, g, slots, stages + ATT_WARPS) <= 216 * 1024) stages += ATT_WARPS;
        }
    }
    AttnArgs a2 = a;
    a2.st_stages = stages;
    const size_t smem = stream ? stream_smem_bytes<HD, BF16>(pages_per_cta, g, slots, stages) : smem_bytes<HD, BF16>(g, slots, pick_nslots<HD, BF16>(g, a.early_pages, a.max_pages, a.nsplit));
    // per device, and only ever raised: launches captured in a graph must stay valid after later calls
    {
        cudaError_t e = stream ? ensure_dyn_smem(attn_stream_kernel<HD, BF16, CL>, smem) : ensure_dyn_smem(attn_decode_kernel<HD, BF16, CL>, smem);
        if (e == cudaSuccess && CL && a.nsplit > 8) e = stream ? ensure_nonportable_clusters(attn_stream_kernel<HD, BF16, CL>) : ensure_nonportable_clusters(attn_decode_kernel<HD, BF16, CL>);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)a.nsplit, (unsigned)a.kv_heads, (unsigned)M);
    cfg.blockDim = dim3(stream ? ST_THREADS : ATT_THREADS);
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
        at[n].val.clusterDim.x = (unsigned)a.nsplit;
        at[n].val.clusterDim.y = 1;
        at[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = at;
    cfg.numAttrs = n;
    return stream ? cudaLaunchKernelEx(&cfg, attn_stream_kernel<HD, BF16, CL>, a2) : cudaLaunchKernelEx(&cfg, attn_decode_kernel<HD, BF16, CL>, a2);
}

template <int HD, bool BF16>
cudaError_t launch_t(const AttnArgs& a, int M, cudaStream_t st, bool pdl) {
    if (a.cluster) {
        if (a.nsplit < 1 || a.nsplit > 16) return cudaErrorInvalidValue;
        return launch_tc<HD, BF16, true>(a, M, st, pdl);
    }
    return launch_tc<HD, BF16, false>(a, M, st, pdl);
}

}  // namespace

// Enough (row, KV head, split) CTAs to cover the SMs about twice, at least two pages each.
int attn_pick_nsplit(int M, int kv_heads, int max_pages, int sm_count, bool bf16_pages) {
    // Splits per (row, KV head): minimise waves x (fixed cost per CTA + pages per CTA) + merge cost.
    // Units are "pages streamed by one CTA": the fixed cost (launch, query and page-table loads) is
    // worth about eight pages, merging one more partial about half a page.  The streaming variant
    // (>= ST_MIN_PAGES pages per CTA) keeps two CTAs per SM resident, the short-context kernel four.
    // max_pages is the capacity the launch is sized for (a captured graph cannot follow the length).
    const long pairs = (long)M * kv_heads;
    int cap = (max_pages + 1) / 2;  // at least two pages per split
    if (cap > sm_count) cap = sm_count;
    if (cap < 1) cap = 1;
    int best = 1;
    long best_cost = -1;
    for (int n = 1; n <= cap; ++n) {
        const int ppc = (max_pages + n - 1) / n;
        const bool streaming = ppc >= ST_MIN_PAGES;
        const long slots = (streaming ? 2L : 4L) * sm_count;
        const long waves = (pairs * n + slots - 1) / slots;
        // doubled so that the half page per partial stays an integer; a page costs the short-context
        // kernel about twice what it costs the streaming one (every query head re-reads the tile)
        // having any split at all costs a round trip of the partial triples through global memory, a ticket and a
        // second merge by the last CTA: about twenty pages' worth (64 sequences at 36 pages: one split 15.4 us, two 17.1)
        // a streaming launch that leaves every CTA an SM to itself gets the deep page ring (launch_tc), which about
        // halves what a page costs its CTA while the cache is short (measured on bf16 pages: 64 x 2 CTAs at 43 pages, one
        // split 11.9 us, two 18.7); on long caches two CTAs per SM stream faster than one with a deep ring, and on f32
        // pages fewer splits lost at every length
        const bool deep = streaming && bf16_pages && max_pages <= 64 && pairs * n <= sm_count;
        const long cost = 2 * waves * (8 + (streaming ? ppc : 2 * ppc)) / (deep ? 2 : 1) + (deep ? 8 : 0) + n + (n > 1 ? 40 : 0);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = n;
        }
    }
    return best;
}

// Cluster variant: the splits of a (row, KV head) form one cluster; one page per CTA when the
// context allows, at most max_cluster CTAs.
int attn_pick_cluster(int max_pages, int max_cluster) {
    int n = max_pages;
    if (n > max_cluster) n = max_cluster;
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
