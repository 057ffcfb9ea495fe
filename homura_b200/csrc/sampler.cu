// Device-side sample_token (src/generate.rs:698-801): repetition / frequency / presence penalties,
// temperature, softmax, min-p, descending sort, top-k, top-p, and the xorshift64 draw, one CTA per
// sequence, so that sampled generation (the reference's default: temperature 0.7, top-k 50, top-p 0.9,
// repetition penalty 1.1) never copies the logits to the host.
//
// The reference sorts the whole vocabulary and truncates to top_k; here the k-th largest scaled logit
// is found by a 4-pass radix select on the float's order-preserving bit pattern, the <= k survivors are
// gathered and sorted (probability descending, index ascending on ties -- the reference's unstable sort
// leaves ties unspecified), and one thread walks them exactly as the reference walks its sorted list.
// With 1 <= top_k <= SAMPLER_MAX_K that is the whole story.  With top-k disabled (0, or >= the vocabulary) or
// larger than SAMPLER_MAX_K the kernel still gathers the SAMPLER_MAX_K largest: when the top-p prefix ends
// inside them the result is what the reference's full sort gives; when it does not (a nearly flat
// distribution) the kernel raises the row's `overflow` word, leaves token and RNG untouched, and the host
// finishes that one token with the host sampler.
// temperature <= 0 is the reference's greedy mode: the penalties are applied, then argmax with ties to the
// highest index (src/generate.rs:707-745), and the RNG is not advanced.
//
// Exactness: the penalties, the maximum, the candidate order and the integer RNG are exact; the
// softmax denominator is a tree sum (the reference adds 151k terms in sequence) and expf differs from
// the host's in the last ulp, so a probability can differ in its last bits and the draw can land on
// the other side of a boundary in rare cases.

#include "common.cuh"
#include "launch_attrs.h"
#include "sampler.h"

namespace hm {
namespace {

constexpr int ST = 1024;  // threads per CTA

__device__ __forceinline__ uint32_t order_key(float f) {  // ascending uint order == ascending float order
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One shared-memory atomic per distinct bin of a warp instead of one per lane: in the first radix pass (sign and
// exponent bits) nearly every key of a row falls into two or three bins, and same-address atomics of a warp serialise.
__device__ __forceinline__ void hist_add(int* hist, bool act, uint32_t bin) {
    const unsigned am = __activemask();
    const unsigned peers = __match_any_sync(am, act ? bin : 0xFFFFFFFFu);
    if (act && (int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], __popc(peers));
}

__device__ __forceinline__ float block_max(float v, float* sw) {
    v = warp_max(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) sw[warp] = v;
    __syncthreads();
    float r = sw[0];
    for (int i = 1; i < ST / 32; ++i) r = fmaxf(r, sw[i]);  // every thread, same order
    __syncthreads();
    return r;
}

__device__ __forceinline__ float block_sum_fixed(float v, float* sw) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) sw[warp] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < ST / 32; ++i) r += sw[i];  // fixed order: the result does not depend on scheduling
    __syncthreads();
    return r;
}

// Visit every element of a row of n floats with f(index, value): 128-bit loads, four of them in flight per
// thread.  One CTA walks the vocabulary several times out of the L2; with one scalar load per iteration each
// pass costs an L2 round trip per element of a thread, which is what made the kernel take ~190 us.
template <typename F>
__device__ __forceinline__ void scan_row(const float* __restrict__ p, int n, int tid, F f) {
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
        const int n4 = n >> 2;
#pragma unroll 4
        for (int i = tid; i < n4; i += ST) {
            const float4 x = *reinterpret_cast<const float4*>(p + 4 * (size_t)i);
            f(4 * i, x.x);
            f(4 * i + 1, x.y);
            f(4 * i + 2, x.z);
            f(4 * i + 3, x.w);
        }
        done = n4 << 2;
    }
    for (int v = done + tid; v < n; v += ST) f(v, p[v]);
}

__global__ void __launch_bounds__(ST) sample_kernel(const SamplerArgs a) {
    __shared__ float sw[ST / 32];
    __shared__ int hist[256];
    __shared__ unsigned long long cand[SAMPLER_MAX_K];  // (order key << 32) | ~index: descending = prob desc, index asc
    __shared__ int tie_idx[SAMPLER_MAX_K];
    __shared__ int n_cand, n_tie, s_k, s_base;
    __shared__ int wcnt[ST / 32];
    __shared__ uint32_t s_prefix;

    const int b = blockIdx.x, tid = threadIdx.x;
    const int V = a.n;
    const float* logits = a.logits + (size_t)b * a.ld_logits;
    float* sl = a.scaled + (size_t)b * V;
    int* count = a.count + (size_t)b * V;
    const uint32_t* gen = a.hist ? a.hist + (size_t)b * a.hist_stride + a.gen_start[b] : a.generated;
    const int ngen = a.hist ? max(0, a.pos[b] - a.gen_start[b]) : a.n_generated;
    const bool pen = a.cfg.repetition_penalty != 1.0f || a.cfg.frequency_penalty != 0.0f || a.cfg.presence_penalty != 0.0f;

    // ---- occurrences of every generated token (the penalties apply per occurrence / per count) ----
    if (pen) {
        for (int i = tid; i < ngen; i += ST) {
            const uint32_t t = gen[i];
            if (t < (uint32_t)V) atomicAdd(count + t, 1);
        }
        __syncthreads();
    }

    // ---- penalties, temperature, maximum ----
    const bool greedy = !(a.cfg.temperature > 0.0f);
    const float inv_temp = greedy ? 1.0f : 1.0f / a.cfg.temperature;
    float mx = -INFINITY;
    auto adjust = [&](float l, int c) {  // penalties per occurrence / per count, then temperature
        if (c > 0) {
            if (a.cfg.repetition_penalty != 1.0f)
                for (int r = 0; r < c; ++r) l = l > 0.0f ? l / a.cfg.repetition_penalty : l * a.cfg.repetition_penalty;
            if (a.cfg.frequency_penalty != 0.0f || a.cfg.presence_penalty != 0.0f) {
                l -= a.cfg.frequency_penalty * (float)c;
                l -= a.cfg.presence_penalty;
            }
        }
        return greedy ? l : l * inv_temp;
    };
    int done = 0;
    if (((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(sl) | reinterpret_cast<uintptr_t>(count)) & 15) == 0) {
        const int V4 = V >> 2;
#pragma unroll 4
        for (int i = tid; i < V4; i += ST) {
            const float4 x = *reinterpret_cast<const float4*>(logits + 4 * (size_t)i);
            const int4 c = pen ? *reinterpret_cast<const int4*>(count + 4 * (size_t)i) : make_int4(0, 0, 0, 0);
            const float4 y = make_float4(adjust(x.x, c.x), adjust(x.y, c.y), adjust(x.z, c.z), adjust(x.w, c.w));
            *reinterpret_cast<float4*>(sl + 4 * (size_t)i) = y;
            mx = fmaxf(fmaxf(mx, fmaxf(y.x, y.y)), fmaxf(y.z, y.w));
        }
        done = V4 << 2;
    }
    for (int v = done + tid; v < V; v += ST) {
        const float l = adjust(logits[v], pen ? count[v] : 0);
        sl[v] = l;
        mx = fmaxf(mx, l);
    }
    __syncthreads();  // the passes below read sl with a different thread-to-element mapping than its stores (tail elements)
    mx = block_max(mx, sw);

    if (greedy) {
        // argmax of the penalised logits, ties to the highest index (Iterator::max_by keeps the last maximum)
        int bi = -1;
        scan_row(sl, V, tid, [&](int v, float l) {
            if (l == mx && v > bi) bi = v;
        });
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) bi = max(bi, __shfl_xor_sync(0xffffffffu, bi, o));
        if ((tid & 31) == 0) wcnt[tid >> 5] = bi;
        __syncthreads();
        if (tid == 0) {
            int best = -1;
            for (int i = 0; i < ST / 32; ++i) best = max(best, wcnt[i]);
            const uint32_t tok = best < 0 ? 0u : (uint32_t)best;
            a.next_tok[b] = tok;
            if (a.feed_tok) a.feed_tok[b] = tok;
            if (a.hist && a.pos) a.hist[(size_t)b * a.hist_stride + a.pos[b]] = tok;
        }
        if (pen) {
            __syncthreads();
            for (int i = tid; i < ngen; i += ST) {
                const uint32_t t = gen[i];
                if (t < (uint32_t)V) count[t] = 0;
            }
        }
        return;
    }

    // ---- softmax denominator ----
    float part = 0.f;
    scan_row(sl, V, tid, [&](int, float l) { part += expf(l - mx); });
    const float sum = block_sum_fixed(part, sw);

    // ---- radix select: order key of the k-th largest scaled logit ----
    // top-k outside 1..SAMPLER_MAX_K (disabled, or wider than the list): the SAMPLER_MAX_K largest are gathered and
    // the walk below decides whether they were enough
    const bool exact_k = (a.cfg.top_k >= 1 && a.cfg.top_k <= SAMPLER_MAX_K) || V <= SAMPLER_MAX_K;
    const int k = min(exact_k && a.cfg.top_k >= 1 ? a.cfg.top_k : SAMPLER_MAX_K, V);
    if (tid == 0) {
        s_prefix = 0u;
        s_k = k;
    }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        const uint32_t mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
        scan_row(sl, V, tid, [&](int, float l) {
            const uint32_t key = order_key(l);
            hist_add(hist, (key & mask) == prefix, (key >> shift) & 0xFFu);
        });
        __syncthreads();
        if (tid == 0) {
            int need = s_k, bin = 255;
            for (; bin > 0; --bin) {
                if (hist[bin] >= need) break;
                need -= hist[bin];
            }
            s_k = need;  // rank of the wanted key among those sharing the extended prefix
            s_prefix = prefix | ((uint32_t)bin << shift);
        }
        __syncthreads();
    }
    const uint32_t kth = s_prefix;  // full key of the k-th largest; s_k of the entries equal to it are wanted
    const int want_ties = s_k;

    // ---- gather: everything above the k-th key, then the lowest-index ties ----
    if (tid == 0) {
        n_cand = 0;
        n_tie = 0;
    }
    __syncthreads();
    scan_row(sl, V, tid, [&](int v, float l) {
        const uint32_t key = order_key(l);
        if (key > kth) {
            const int slot = atomicAdd(&n_cand, 1);
            if (slot < SAMPLER_MAX_K) cand[slot] = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)v);
        } else if (key == kth) {
            const int slot = atomicAdd(&n_tie, 1);
            if (slot < SAMPLER_MAX_K) tie_idx[slot] = v;
        }
    });
    __syncthreads();
    if (n_tie > SAMPLER_MAX_K) {
        // Degenerate rows (flat or masked logits) have more entries equal to the k-th key than the list holds, and
        // the slots above were handed out in arrival order.  Take the ties again in index order: chunks of ST
        // consecutive elements, every thread's rank from a ballot prefix count, until want_ties are found.
        if (tid == 0) s_base = 0;
        __syncthreads();
        for (int c0 = 0; c0 < V && s_base < want_ties; c0 += ST) {
            const int v = c0 + tid;
            const bool is = v < V && order_key(sl[v]) == kth;
            const unsigned bal = __ballot_sync(0xffffffffu, is);
            if ((tid & 31) == 0) wcnt[tid >> 5] = __popc(bal);
            __syncthreads();
            int before = 0, total = 0;
            for (int w = 0; w < ST / 32; ++w) {
                if (w < (tid >> 5)) before += wcnt[w];
                total += wcnt[w];
            }
            const int rank = s_base + before + __popc(bal & ((1u << (tid & 31)) - 1u));
            if (is && rank < SAMPLER_MAX_K) tie_idx[rank] = v;
            __syncthreads();
            if (tid == 0) s_base += total;
            __syncthreads();
        }
        if (tid == 0) n_tie = min(s_base, SAMPLER_MAX_K);
        __syncthreads();
    }
    if (tid == 0) {
        // ties: ascending index, the first want_ties of them (n_tie is tiny except for degenerate logits)
        const int nt = min(n_tie, SAMPLER_MAX_K);
        for (int i = 1; i < nt; ++i) {
            const int x = tie_idx[i];
            int j = i - 1;
            while (j >= 0 && tie_idx[j] > x) {
                tie_idx[j + 1] = tie_idx[j];
                --j;
            }
            tie_idx[j + 1] = x;
        }
        int nc = min(n_cand, SAMPLER_MAX_K);
        for (int i = 0; i < min(want_ties, nt) && nc < SAMPLER_MAX_K; ++i) cand[nc++] = ((unsigned long long)kth << 32) | (uint32_t)(~(uint32_t)tie_idx[i]);
        n_cand = nc;
    }
    __syncthreads();
    const int nc = n_cand;
    for (int i = nc + tid; i < SAMPLER_MAX_K; i += ST) cand[i] = 0ull;  // padding sorts last
    __syncthreads();

    // ---- bitonic sort, descending ----
    for (int size = 2; size <= SAMPLER_MAX_K; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < SAMPLER_MAX_K; i += ST) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool desc = (i & size) == 0;
                    const unsigned long long x = cand[i], y = cand[j];
                    if (desc ? (x < y) : (x > y)) {
                        cand[i] = y;
                        cand[j] = x;
                    }
                }
            }
            __syncthreads();
        }
    }

    // ---- min-p, top-p, draw: one thread walks the sorted list as the reference does ----
    // the candidates' probabilities in parallel (an exponential and a division each, and a load that may miss);
    // the walk itself is a few additions and comparisons per candidate
    float* probs = reinterpret_cast<float*>(tie_idx);  // reuse
    for (int i = tid; i < nc; i += ST) {
        const int v = (int)(~(uint32_t)(cand[i] & 0xFFFFFFFFull));
        probs[i] = expf(sl[v] - mx) / sum;
    }
    __syncthreads();
    if (tid == 0) {
        if (a.cfg.min_p > 0.0f && nc > 0) {
            const float thr = a.cfg.min_p * probs[0];  // the largest probability is the first of the sorted list
            for (int i = 0; i < nc; ++i)
                if (probs[i] < thr) probs[i] = 0.0f;
        }
        float cumulative = 0.0f;
        int cutoff = nc;
        for (int i = 0; i < nc; ++i) {
            cumulative += probs[i];
            if (cumulative >= a.cfg.top_p) {
                cutoff = i + 1;
                break;
            }
        }
        if (!exact_k && cutoff == nc && !(cumulative >= a.cfg.top_p)) {
            // the top-p prefix does not end inside the gathered candidates: this token is the host sampler's
            if (a.overflow) a.overflow[b] = 1;
            goto done_walk;
        }
        if (a.overflow) a.overflow[b] = 0;
        float total = 0.0f;
        for (int i = 0; i < cutoff; ++i) total += probs[i];
        unsigned long long s = a.rng[b];  // xorshift64 (13, 7, 17), src/generate.rs:634-641
        s ^= s << 13;
        s ^= s >> 7;
        s ^= s << 17;
        a.rng[b] = s;
        const float r = ((float)(s >> 40) / (float)(1ull << 24)) * total;
        float accum = 0.0f;
        int pick = cutoff ? cutoff - 1 : 0;
        for (int i = 0; i < cutoff; ++i) {
            accum += probs[i];
            if (accum >= r) {
                pick = i;
                break;
            }
        }
        const uint32_t tok = nc ? (uint32_t)(~(uint32_t)(cand[pick] & 0xFFFFFFFFull)) : 0u;
        a.next_tok[b] = tok;
        if (a.feed_tok) a.feed_tok[b] = tok;
        if (a.hist && a.pos) a.hist[(size_t)b * a.hist_stride + a.pos[b]] = tok;  // replaces the greedy token of this step
    }
done_walk:

    // ---- leave the occurrence counts clean for the next call ----
    if (pen) {
        __syncthreads();
        for (int i = tid; i < ngen; i += ST) {
            const uint32_t t = gen[i];
            if (t < (uint32_t)V) count[t] = 0;
        }
    }
}


// ---- the same algorithm over a thread-block cluster -------------------------------------------------------------
// One CTA walking a 151,936-entry row seven times out of the L2 takes ~115 us.  Here the SC CTAs of a cluster own one
// contiguous slice of the row each, read it from global memory once into shared memory, and exchange only scalars,
// 256-bin histograms and the <= SAMPLER_MAX_K candidates through distributed shared memory, a cluster barrier per
// exchange.  Every result that the single-CTA kernel defines (candidate set, ties to the lowest indices, order of the
// walk, RNG) is the same; the softmax denominator is summed per slice and then in rank order.
constexpr int SC = 8;  // CTAs per sequence (portable cluster size)

__device__ __forceinline__ void st_dsmem_u32(uint32_t addr, uint32_t v) { asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void st_dsmem_u64(uint32_t addr, unsigned long long v) { asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory"); }
__device__ __forceinline__ void red_dsmem_add_u32(uint32_t addr, uint32_t v) { asm volatile("red.shared::cluster.add.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_dsmem_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ float key_to_float(uint32_t key) { return __uint_as_float((key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key); }

__global__ void __launch_bounds__(ST) sample_cluster_kernel(const SamplerArgs a, int slice) {
    extern __shared__ __align__(16) float sl[];  // this CTA's slice of the scaled logits
    __shared__ float sw[ST / 32];
    __shared__ int wcnt[ST / 32];
    __shared__ float r_max[SC], r_sum[SC];
    __shared__ int r_arg[SC], r_above[SC], r_tie[SC];
    __shared__ int hist_all[4][256];  // rank 0: the cluster's histogram of every radix pass
    __shared__ int hist[256];         // this CTA's
    __shared__ unsigned long long cand[SAMPLER_MAX_K];  // rank 0: the gathered candidates; (order key << 32) | ~index
    __shared__ unsigned long long lcand[SAMPLER_MAX_K]; // this CTA's candidates above the k-th key
    __shared__ int tie_idx[SAMPLER_MAX_K];
    __shared__ int n_above, n_tie, s_k, s_base;
    __shared__ uint32_t s_prefix;

    const int b = blockIdx.y, tid = threadIdx.x;
    const uint32_t rank = cluster_ctarank();
    const int V = a.n;
    const int c0 = min(V, (int)rank * slice), nl = min(V, c0 + slice) - c0;  // slice is a multiple of 4
    const float* logits = a.logits + (size_t)b * a.ld_logits;
    int* count = a.count + (size_t)b * V;
    const uint32_t* gen = a.hist ? a.hist + (size_t)b * a.hist_stride + a.gen_start[b] : a.generated;
    const int ngen = a.hist ? max(0, a.pos[b] - a.gen_start[b]) : a.n_generated;
    const bool pen = a.cfg.repetition_penalty != 1.0f || a.cfg.frequency_penalty != 0.0f || a.cfg.presence_penalty != 0.0f;

    for (int i = tid; i < 4 * 256; i += ST) (&hist_all[0][0])[i] = 0;
    if (tid == 0) {
        n_above = 0;
        n_tie = 0;
    }
    // ---- occurrences of every generated token: the cluster shares the list, the counts meet in global memory ----
    if (pen) {
        for (int i = (int)rank * ST + tid; i < ngen; i += SC * ST) {
            const uint32_t t = gen[i];
            if (t < (uint32_t)V) atomicAdd(count + t, 1);
        }
    }
    cluster_sync_all();  // counts complete (and every CTA's shared memory initialised before a peer writes into it)

    // ---- penalties, temperature, maximum ----
    const bool greedy = !(a.cfg.temperature > 0.0f);
    const float inv_temp = greedy ? 1.0f : 1.0f / a.cfg.temperature;
    auto adjust = [&](float l, int c) {
        if (c > 0) {
            if (a.cfg.repetition_penalty != 1.0f)
                for (int r = 0; r < c; ++r) l = l > 0.0f ? l / a.cfg.repetition_penalty : l * a.cfg.repetition_penalty;
            if (a.cfg.frequency_penalty != 0.0f || a.cfg.presence_penalty != 0.0f) {
                l -= a.cfg.frequency_penalty * (float)c;
                l -= a.cfg.presence_penalty;
            }
        }
        return greedy ? l : l * inv_temp;
    };
    float mx = -INFINITY;
    {
        int done = 0;
        if (((reinterpret_cast<uintptr_t>(logits + c0) | reinterpret_cast<uintptr_t>(count + c0)) & 15) == 0) {
            const int n4 = nl >> 2;
#pragma unroll 4
            for (int i = tid; i < n4; i += ST) {
                const float4 x = __ldcg(reinterpret_cast<const float4*>(logits + c0) + i);
                const int4 c = pen ? __ldcg(reinterpret_cast<const int4*>(count + c0) + i) : make_int4(0, 0, 0, 0);
                const float4 y = make_float4(adjust(x.x, c.x), adjust(x.y, c.y), adjust(x.z, c.z), adjust(x.w, c.w));
                *reinterpret_cast<float4*>(sl + 4 * i) = y;
                mx = fmaxf(fmaxf(mx, fmaxf(y.x, y.y)), fmaxf(y.z, y.w));
            }
            done = n4 << 2;
        }
        for (int v = done + tid; v < nl; v += ST) {
            const float l = adjust(__ldcg(logits + c0 + v), pen ? __ldcg(count + c0 + v) : 0);
            sl[v] = l;
            mx = fmaxf(mx, l);
        }
    }
    __syncthreads();
    mx = block_max(mx, sw);
    if (tid < SC) st_dsmem_f32(dsmem_addr(&r_max[rank], (uint32_t)tid), mx);
    cluster_sync_all();
    mx = r_max[0];
    for (int r = 1; r < SC; ++r) mx = fmaxf(mx, r_max[r]);
    // every count has been read: leave them clean for the next call
    if (pen) {
        for (int i = (int)rank * ST + tid; i < ngen; i += SC * ST) {
            const uint32_t t = gen[i];
            if (t < (uint32_t)V) count[t] = 0;
        }
    }

    // visit the slice with f(global index, value)
    auto scan = [&](auto f) {
        const int n4 = nl >> 2;
#pragma unroll 4
        for (int i = tid; i < n4; i += ST) {
            const float4 x = *reinterpret_cast<const float4*>(sl + 4 * i);
            f(c0 + 4 * i, x.x);
            f(c0 + 4 * i + 1, x.y);
            f(c0 + 4 * i + 2, x.z);
            f(c0 + 4 * i + 3, x.w);
        }
        for (int v = (n4 << 2) + tid; v < nl; v += ST) f(c0 + v, sl[v]);
    };

    if (greedy) {
        // argmax of the penalised logits, ties to the highest index
        int bi = -1;
        scan([&](int v, float l) {
            if (l == mx && v > bi) bi = v;
        });
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) bi = max(bi, __shfl_xor_sync(0xffffffffu, bi, o));
        if ((tid & 31) == 0) wcnt[tid >> 5] = bi;
        __syncthreads();
        if (tid == 0) {
            int best = -1;
            for (int i = 0; i < ST / 32; ++i) best = max(best, wcnt[i]);
            st_dsmem_u32(dsmem_addr(&r_arg[rank], 0u), (uint32_t)best);
        }
        cluster_arrive_release();
        if (rank != 0) return;
        cluster_wait_acquire();
        if (tid == 0) {
            int best = -1;
            for (int r = 0; r < SC; ++r) best = max(best, r_arg[r]);
            const uint32_t tok = best < 0 ? 0u : (uint32_t)best;
            a.next_tok[b] = tok;
            if (a.feed_tok) a.feed_tok[b] = tok;
            if (a.hist && a.pos) a.hist[(size_t)b * a.hist_stride + a.pos[b]] = tok;
        }
        return;
    }

    // ---- softmax denominator: per slice in a fixed order, then the slices in rank order ----
    // (summed during the first radix pass, which visits every element anyway; that pass's barrier publishes r_sum)
    float part = 0.f;

    // ---- radix select over the cluster: order key of the k-th largest scaled logit ----
    const bool exact_k = (a.cfg.top_k >= 1 && a.cfg.top_k <= SAMPLER_MAX_K) || V <= SAMPLER_MAX_K;
    const int k = min(exact_k && a.cfg.top_k >= 1 ? a.cfg.top_k : SAMPLER_MAX_K, V);
    if (tid == 0) {
        s_prefix = 0u;
        s_k = k;
    }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        const uint32_t mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
        if (pass == 0) {
            scan([&](int, float l) {
                part += expf(l - mx);
                hist_add(hist, true, order_key(l) >> 24);
            });
            part = block_sum_fixed(part, sw);
            if (tid < SC) st_dsmem_f32(dsmem_addr(&r_sum[rank], (uint32_t)tid), part);
        } else {
            scan([&](int, float l) {
                const uint32_t key = order_key(l);
                hist_add(hist, (key & mask) == prefix, (key >> shift) & 0xFFu);
            });
        }
        __syncthreads();
        if (tid < 256 && hist[tid]) red_dsmem_add_u32(dsmem_addr(&hist_all[pass][tid], 0u), (uint32_t)hist[tid]);
        cluster_sync_all();
        if (tid < 256) hist[tid] = (int)ld_dsmem_u32(dsmem_addr(&hist_all[pass][tid], 0u));
        __syncthreads();
        if (tid < 32) {
            // every CTA takes the same decision from the same numbers: lane l owns bins 8l .. 8l + 7; the wanted bin is
            // in the lane whose suffix count reaches the rank while the next lane's does not
            int mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) mine += hist[8 * tid + j];
            int suffix = mine;  // bins >= 8 * tid
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_down_sync(0xffffffffu, suffix, o);
                if (tid + o < 32) suffix += up;
            }
            const int above = suffix - mine;  // bins >= 8 * (tid + 1)
            const int need0 = s_k;
            if (above < need0 && (suffix >= need0 || tid == 0)) {
                int need = need0 - above, bin = 8 * tid + 7;
                for (; bin > 8 * tid; --bin) {
                    if (hist[bin] >= need) break;
                    need -= hist[bin];
                }
                s_k = need;
                s_prefix = prefix | ((uint32_t)bin << shift);
            }
        }
        __syncthreads();
    }
    const uint32_t kth = s_prefix;
    const int want_ties = s_k;
    float sum = 0.f;
    for (int r = 0; r < SC; ++r) sum += r_sum[r];

    // ---- gather: this slice's keys above the k-th, and its lowest-index ties ----
    scan([&](int v, float l) {
        const uint32_t key = order_key(l);
        if (key > kth) {
            const int slot = atomicAdd(&n_above, 1);
            if (slot < SAMPLER_MAX_K) lcand[slot] = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)v);
        } else if (key == kth) {
            const int slot = atomicAdd(&n_tie, 1);
            if (slot < SAMPLER_MAX_K) tie_idx[slot] = v;
        }
    });
    __syncthreads();
    if (n_tie > 32) {
        // many ties (flat or masked logits): take them again in index order, chunks of ST consecutive elements, every
        // thread's rank from a ballot prefix count, until the list is full or the slice ends
        if (tid == 0) s_base = 0;
        __syncthreads();
        for (int v0 = 0; v0 < nl && s_base < SAMPLER_MAX_K; v0 += ST) {
            const int v = v0 + tid;
            const bool is = v < nl && order_key(sl[v]) == kth;
            const unsigned bal = __ballot_sync(0xffffffffu, is);
            if ((tid & 31) == 0) wcnt[tid >> 5] = __popc(bal);
            __syncthreads();
            int before = 0, total = 0;
            for (int w = 0; w < ST / 32; ++w) {
                if (w < (tid >> 5)) before += wcnt[w];
                total += wcnt[w];
            }
            const int rk = s_base + before + __popc(bal & ((1u << (tid & 31)) - 1u));
            if (is && rk < SAMPLER_MAX_K) tie_idx[rk] = c0 + v;
            __syncthreads();
            if (tid == 0) s_base += total;
            __syncthreads();
        }
    } else if (tid == 0) {
        for (int i = 1; i < n_tie; ++i) {  // ascending index
            const int x = tie_idx[i];
            int j = i - 1;
            while (j >= 0 && tie_idx[j] > x) {
                tie_idx[j + 1] = tie_idx[j];
                --j;
            }
            tie_idx[j + 1] = x;
        }
    }
    __syncthreads();
    if (tid < SC) {
        st_dsmem_u32(dsmem_addr(&r_above[rank], (uint32_t)tid), (uint32_t)n_above);
        st_dsmem_u32(dsmem_addr(&r_tie[rank], (uint32_t)tid), (uint32_t)n_tie);
    }
    cluster_sync_all();
    // slices are contiguous index ranges in rank order: the lowest-index ties are those of the lowest ranks
    int above_before = 0, above_total = 0, ties_before = 0;
    for (int r = 0; r < SC; ++r) {
        if (r < (int)rank) {
            above_before += r_above[r];
            ties_before += r_tie[r];
        }
        above_total += r_above[r];
    }
    const int take = max(0, min(min(n_tie, SAMPLER_MAX_K), want_ties - ties_before));
    int taken_before = 0;
    {
        int tb = 0;
        for (int r = 0; r < (int)rank; ++r) {
            const int t = max(0, min(min(r_tie[r], SAMPLER_MAX_K), want_ties - tb));
            taken_before += t;
            tb += r_tie[r];
        }
    }
    for (int i = tid; i < min(n_above, SAMPLER_MAX_K); i += ST) {
        const int slot = above_before + i;
        if (slot < SAMPLER_MAX_K) st_dsmem_u64(dsmem_addr(&cand[slot], 0u), lcand[i]);
    }
    for (int i = tid; i < take; i += ST) {
        const int slot = above_total + taken_before + i;
        if (slot < SAMPLER_MAX_K) st_dsmem_u64(dsmem_addr(&cand[slot], 0u), ((unsigned long long)kth << 32) | (uint32_t)(~(uint32_t)tie_idx[i]));
    }
    cluster_arrive_release();
    if (rank != 0) return;
    cluster_wait_acquire();

    int ties_total = 0;
    {
        int tb = 0;
        for (int r = 0; r < SC; ++r) {
            ties_total += max(0, min(min(r_tie[r], SAMPLER_MAX_K), want_ties - tb));
            tb += r_tie[r];
        }
    }
    const int nc = min(above_total + ties_total, SAMPLER_MAX_K);
    // descending order by rank: the entries are distinct (they carry their index), so every entry's rank is the number
    // of larger ones; no barrier per step, and the usual few dozen candidates cost a few dozen compares per thread
    __syncthreads();
    for (int i = tid; i < nc; i += ST) {
        const unsigned long long x = cand[i];
        int rk = 0;
        for (int j = 0; j < nc; ++j) rk += cand[j] > x ? 1 : 0;
        lcand[rk] = x;
    }
    __syncthreads();
    for (int i = tid; i < nc; i += ST) cand[i] = lcand[i];
    __syncthreads();

    // ---- min-p, top-p, draw: one thread walks the sorted list as the reference does ----
    float* probs = reinterpret_cast<float*>(tie_idx);  // reuse
    for (int i = tid; i < nc; i += ST) probs[i] = expf(key_to_float((uint32_t)(cand[i] >> 32)) - mx) / sum;
    __syncthreads();
    if (tid == 0) {
        if (a.cfg.min_p > 0.0f && nc > 0) {
            const float thr = a.cfg.min_p * probs[0];
            for (int i = 0; i < nc; ++i)
                if (probs[i] < thr) probs[i] = 0.0f;
        }
        float cumulative = 0.0f;
        int cutoff = nc;
        for (int i = 0; i < nc; ++i) {
            cumulative += probs[i];
            if (cumulative >= a.cfg.top_p) {
                cutoff = i + 1;
                break;
            }
        }
        if (!exact_k && cutoff == nc && !(cumulative >= a.cfg.top_p)) {
            if (a.overflow) a.overflow[b] = 1;  // this token is the host sampler's
            return;
        }
        if (a.overflow) a.overflow[b] = 0;
        float total = 0.0f;
        for (int i = 0; i < cutoff; ++i) total += probs[i];
        unsigned long long s = a.rng[b];  // xorshift64 (13, 7, 17), src/generate.rs:634-641
        s ^= s << 13;
        s ^= s >> 7;
        s ^= s << 17;
        a.rng[b] = s;
        const float r = ((float)(s >> 40) / (float)(1ull << 24)) * total;
        float accum = 0.0f;
        int pick = cutoff ? cutoff - 1 : 0;
        for (int i = 0; i < cutoff; ++i) {
            accum += probs[i];
            if (accum >= r) {
                pick = i;
                break;
            }
        }
        const uint32_t tok = nc ? (uint32_t)(~(uint32_t)(cand[pick] & 0xFFFFFFFFull)) : 0u;
        a.next_tok[b] = tok;
        if (a.feed_tok) a.feed_tok[b] = tok;
        if (a.hist && a.pos) a.hist[(size_t)b * a.hist_stride + a.pos[b]] = tok;
    }
}

}  // namespace

cudaError_t launch_sample(const SamplerArgs& a, int batch, cudaStream_t st) {
    const bool exact_k = (a.cfg.top_k >= 1 && a.cfg.top_k <= SAMPLER_MAX_K) || a.n <= SAMPLER_MAX_K;
    if (a.cfg.temperature > 0.f && !exact_k && !a.overflow) return cudaErrorInvalidValue;  // the caller must be able to learn that a row needs the host sampler
    // rows of a real vocabulary: one cluster per sequence, the row split over its CTAs' shared memory
    const int slice = ((a.n + SC - 1) / SC + 3) & ~3;
    const size_t smem = (size_t)slice * sizeof(float);
    if (a.n >= 16384 && smem <= 160 * 1024) {
        cudaError_t e = ensure_dyn_smem(sample_cluster_kernel, smem);
        if (e != cudaSuccess) return e;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(SC, (unsigned)batch);
        cfg.blockDim = dim3(ST);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = SC;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, sample_cluster_kernel, a, slice);
    }
    sample_kernel<<<batch, ST, 0, st>>>(a);
    return cudaGetLastError();
}

}  // namespace hm
