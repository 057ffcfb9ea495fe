// Persistent decode kernel: one cooperative launch runs a whole decode step (batch 1, bf16
// weights) -- embedding, 24 x {QKV+RoPE+KV write, attention, O, gate/up+SwiGLU, down}, final norm,
// LM head and argmax -- with one CTA per SM.
//
// It computes what the chain of per-projection kernels computes (same reference anchors:
// src/hf/emitter.rs:506-862 for the fused kernels, src/runtime.rs:1729-1755 for the KV append,
// src/generate.rs:457-468 for the argmax), restructured around two facts about batch-1 decode
// on a B200: the weights never depend on activations, and every phase is a latency chain.
//
//   * The last warp of every CTA is a producer.  It walks the CTA's static schedule of weight tiles
//     for the WHOLE step and streams them with bulk async copies (cp.async.bulk, completion on
//     an mbarrier, no multicast) into a ring of 16 KB shared-memory stages, as far ahead as the
//     ring allows.  It never looks at a grid barrier, so HBM keeps streaming while the consumer
//     warps sit in a phase boundary.
//   * The other eight warps are consumers.  A phase is a list of (128-column slab, K-split) items dealt
//     round-robin to the CTAs.  An item multiplies its K-slice of the input vector with its
//     tile out of the ring and writes a 128-float PARTIAL to global scratch.  Nobody reduces
//     partials at the producing side: the next phase's items add, in split order, just the
//     partials of the K-slice they need while they build their input slice (so the sum is
//     deterministic and there are no atomics).  RMSNorm's 1/rms is deferred the same way: an
//     item multiplies with x*w, publishes its slice's sum of squares, and the consumer of the
//     partials applies the scalar.
//   * There is no grid barrier.  Everything one CTA hands to another (partials, sums of squares,
//     residual slices, attention chunk results, argmax candidates) is an 8-byte {value,
//     generation} pair written with one 64-bit store; the reader polls the pair until the
//     generation is the current step's, so readiness and data arrive in the same L2 round trip
//     and an item waits only for the items it really depends on.  Every layer has its own
//     exchange buffers, so nothing is overwritten within a step.  The launch is cooperative (all
//     CTAs resident, phases processed in order, so dependencies always make progress); every
//     poll is bounded: on overrun the error flag is raised, all later waits give up at once, and
//     the kernel returns.
#include <cooperative_groups.h>

#include "common.cuh"
#include "persistent.h"

namespace hm {
namespace {

constexpr int CONSUMERS = 256;            // 8 warps (16 warps measured slower: more pollers, register spills)
constexpr int NW = CONSUMERS / 32;
constexpr int RL = CONSUMERS / 16;          // row lanes: threads per 128-column row group
constexpr int MK_THREADS = CONSUMERS + 32;  // + producer warp
constexpr int CH = 64;                     // rows per ring stage (64 x 256 B = 16 KB)
constexpr int STAGE_BYTES = CH * SLAB * 2;
constexpr int NSTAGE = 10;
constexpr int XS_MAX = 2048;               // longest input slice an item may need (floats)
constexpr int PTK = 16;                    // tokens per KV page
constexpr unsigned long long SPIN_LIMIT = 4000000ULL;

// ---- mbarrier / bulk copy -----------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(b)), "r"(parity)
        : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> this CTA's shared memory; completion is signalled on `bar`.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes),
                 "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory"); }

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned int ld_cg_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// {value, generation} exchanged between CTAs with single 64-bit accesses.
// One naturally aligned 64-bit scalar access each way: single-copy atomic, coherent at GPU scope.
__device__ __forceinline__ void ll_store(LL* p, float v, uint32_t gen) {
    const unsigned long long w = (unsigned long long)__float_as_uint(v) | ((unsigned long long)gen << 32);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ll_load(const LL* p, float& v, uint32_t& gen) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    v = __uint_as_float((uint32_t)w);
    gen = (uint32_t)(w >> 32);
}

struct Shared {
    uint64_t full[NSTAGE];
    uint64_t empty[NSTAGE];
    volatile int abort;
    int pos, token;
    alignas(16) float red[2][NW][SLAB];  // double-buffered by item parity; written with 128-bit stores
    float wsum[NW];
    int widx[NW];
};

struct Ctx {
    const MkArgs& a;
    Shared& sh;
    unsigned char* ring;
    float* xs;     // [XS_MAX]
    float* att;    // attention scratch (see attention_item)
    int cta, nb, tid, lane, warp;
    uint32_t g;    // chunks consumed (consumer) / issued (producer)
    uint32_t gen;  // generation of this step (launch index + 1)
    int phase_idx;
    int item_parity;
};

__device__ __forceinline__ bool wait_bounded(Ctx& c, uint64_t* bar, uint32_t parity) {
    unsigned long long it = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (c.sh.abort) return false;
        if (++it > SPIN_LIMIT) {
            c.sh.abort = 1;
            atomicExch(c.a.err_flag, 2);
            return false;
        }
    }
    return true;
}

// ---- producer -------------------------------------------------------------------------------
__device__ __forceinline__ void produce_item(Ctx& c, const uint16_t* W, int K, int slab, int k0, int nrows) {
    const char* src = reinterpret_cast<const char*>(W) + ((size_t)slab * K + k0) * (SLAB * 2);
    for (int r = 0; r < nrows; r += CH) {
        const int rows = min(CH, nrows - r);
        const int stage = c.g % NSTAGE;
        const uint32_t par = ((c.g / NSTAGE) & 1u) ^ 1u;
        if (!wait_bounded(c, &c.sh.empty[stage], par)) return;
        mbar_arrive_expect_tx(&c.sh.full[stage], (uint32_t)rows * SLAB * 2);
        bulk_g2s(c.ring + (size_t)stage * STAGE_BYTES, src + (size_t)r * SLAB * 2, (uint32_t)rows * SLAB * 2, &c.sh.full[stage]);
        ++c.g;
    }
}

__device__ void produce_phase(Ctx& c, const uint16_t* W, int K, int nslabs, int S, int R) {
    const int nitems = nslabs * S;
    for (int i = c.cta; i < nitems; i += c.nb) {
        if (c.sh.abort) return;
        const int slab = i / S, split = i - slab * S;
        const int k0 = split * R;
        const int nrows = max(0, min(K, k0 + R) - k0);
        produce_item(c, W, K, slab, k0, nrows);
    }
}

__device__ void producer(Ctx& c) {
    const MkArgs& a = c.a;
    for (int l = 0; l < a.L; ++l) {
        const MkLayer& w = a.layers[l];
        produce_phase(c, w.wqkv, a.H, a.slabs_qkv, a.S1, a.R1);
        produce_phase(c, w.wo, a.qdim, a.slabs_h, a.S3, a.R3);
        produce_phase(c, w.wgu, a.H, a.slabs_gu, a.S4, a.R4);
        produce_phase(c, w.wdown, a.I, a.slabs_h, a.S5, a.R5);
    }
    produce_phase(c, a.wlm, a.H, a.slabs_v, 1, a.H);
}

// ---- consumer helpers -------------------------------------------------------------------------
// Poll limit shared by all flag waits of a thread.
__device__ __forceinline__ bool poll_overrun(Ctx& c, unsigned long long& it) {
    if (c.sh.abort) return true;
    if ((++it & 255ULL) == 0 && ld_cg_u32((const unsigned int*)c.a.err_flag) == 2u) {
        c.sh.abort = 1;
        return true;
    }
    if (it > SPIN_LIMIT) {
        c.sh.abort = 1;
        atomicExch(c.a.err_flag, 2);
        return true;
    }
    return false;
}

// Sum of up to MAX_SPLITS exchanged values base[s * stride], s ascending, once all of them carry
// this step's generation.  All loads of a round are issued before any is inspected, so a round
// costs one L2 round trip.
constexpr int MAX_SPLITS = 24;
__device__ __forceinline__ float ll_sum(Ctx& c, const LL* base, size_t stride, int S, const LL* extra = nullptr) {
    float v[MAX_SPLITS];
    float ev = 0.f;
    unsigned long long it = 0;
    while (true) {
        bool ready = true;
        if (extra) {
            uint32_t gen;
            ll_load(extra, ev, gen);
            ready = gen == c.gen;
        }
#pragma unroll
        for (int s = 0; s < MAX_SPLITS; ++s) {
            v[s] = 0.f;
            if (s < S) {
                uint32_t gen;
                ll_load(base + (size_t)s * stride, v[s], gen);
                ready = ready && gen == c.gen;
            }
        }
        if (ready || poll_overrun(c, it)) break;
    }
    float t = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_SPLITS; ++s) t += v[s];
    return extra ? ev + t : t;
}
__device__ __forceinline__ LL* lay(const MkArgs& a, int layer, size_t off) { return a.ll + (size_t)layer * a.layer_stride + off; }
__device__ __forceinline__ float ll_get(Ctx& c, const LL* p) {
    float v;
    uint32_t gen;
    unsigned long long it = 0;
    while (true) {
        ll_load(p, v, gen);
        if (gen == c.gen || poll_overrun(c, it)) break;
    }
    return v;
}

// Optional sub-phase stamp k (0..2) of the current phase for CTA 0 (after slices built, after tiles multiplied).
__device__ __forceinline__ void sub_mark(Ctx& c, int k) {
    if (c.a.trace && c.cta == 0 && c.tid == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        c.a.trace[c.a.barriers_per_launch + 1 + c.phase_idx * 2 + k] = t;
    }
}

__device__ __forceinline__ void phase_mark(Ctx& c) {
    ++c.phase_idx;
    if (c.a.trace && c.cta == 0 && c.tid == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        c.a.trace[c.phase_idx] = t;
    }
}

// Multiply the item's tile (streamed through the ring) with xs[0..nrows): thread (rl, cg) owns
// rows rl, rl+16, ... of every chunk and 8 columns.  Returns, in threads 0..127, the sum of
// column `tid` of the slab.  sh.red is double-buffered by item parity, so one barrier per item
// is enough.
__device__ __forceinline__ float run_item(Ctx& c, const float* xs, int nrows) {
    const int cg = c.tid & 15, rl = c.tid >> 4;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r = 0; r < nrows; r += CH) {
        const int rows = min(CH, nrows - r);
        const int stage = c.g % NSTAGE;
        const uint32_t par = (c.g / NSTAGE) & 1u;
        const bool ok = wait_bounded(c, &c.sh.full[stage], par);
        if (ok) {
            const uint4* tile = reinterpret_cast<const uint4*>(c.ring + (size_t)stage * STAGE_BYTES);
#pragma unroll
            for (int i = 0; i < CH / RL; ++i) {
                const int rr = rl + RL * i;
                if (rr < rows) {
                    const uint4 w = tile[rr * 16 + cg];
                    const float xv = xs[r + rr];
                    acc[0] = fmaf(xv, bf16_lo(w.x), acc[0]); acc[1] = fmaf(xv, bf16_hi(w.x), acc[1]);
                    acc[2] = fmaf(xv, bf16_lo(w.y), acc[2]); acc[3] = fmaf(xv, bf16_hi(w.y), acc[3]);
                    acc[4] = fmaf(xv, bf16_lo(w.z), acc[4]); acc[5] = fmaf(xv, bf16_hi(w.z), acc[5]);
                    acc[6] = fmaf(xv, bf16_lo(w.w), acc[6]); acc[7] = fmaf(xv, bf16_hi(w.w), acc[7]);
                }
            }
        }
        __syncwarp();
        if (c.lane == 0 && ok) mbar_arrive(&c.sh.empty[stage]);
        ++c.g;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 16);
    float(*red)[SLAB] = c.sh.red[c.item_parity];
    c.item_parity ^= 1;
    if (c.lane < 16) {
        float4* dst = reinterpret_cast<float4*>(&red[c.warp][cg * 8]);
        dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    consumer_sync();
    float v = 0.f;
    if (c.tid < SLAB) {
#pragma unroll
        for (int wv = 0; wv < NW; ++wv) v += red[wv][c.tid];
    }
    return v;
}

// Deterministic block sum (consumer threads).
__device__ __forceinline__ float block_sum(Ctx& c, float v) {
    v = warp_sum(v);
    consumer_sync();
    if (c.lane == 0) c.sh.wsum[c.warp] = v;
    consumer_sync();
    float t = 0.f;
#pragma unroll
    for (int wv = 0; wv < NW; ++wv) t += c.sh.wsum[wv];
    return t;
}

__device__ __forceinline__ float inv_rms_from(Ctx& c, const LL* ss, int n, int H, float eps) {
    return 1.0f / sqrtf(ll_sum(c, ss, 1, n) / (float)H + eps);
}

// ---- phases -----------------------------------------------------------------------------------
// Every projection phase runs in two passes over the CTA's items: first all input slices are
// built side by side in xs (their global loads overlap), then the tiles are multiplied.

// P1 / P4: input slice of the residual stream = previous residual buffer + the partials of the
// projection that was added to it; publishes the new residual and the slice's sum of squares.
__device__ void phase_norm_proj(Ctx& c, int layer, bool is_qkv) {
    const MkArgs& a = c.a;
    const MkLayer& w = a.layers[layer];
    const int S = is_qkv ? a.S1 : a.S4, R = is_qkv ? a.R1 : a.R4;
    const int nslabs = is_qkv ? a.slabs_qkv : a.slabs_gu;
    const int Sprev = is_qkv ? a.S5 : a.S3;
    const LL* part_prev = is_qkv ? lay(a, layer - 1, a.o_pdown) : lay(a, layer, a.o_po);  // (layer 0 reads the embedding instead)
    const LL* h_prev = is_qkv ? lay(a, layer - 1, a.o_hmid) : lay(a, layer, a.o_hcur);
    LL* h_out = is_qkv ? lay(a, layer, a.o_hcur) : lay(a, layer, a.o_hmid);
    const float* norm_w = is_qkv ? w.in_ln : w.post_ln;
    LL* part_out = is_qkv ? lay(a, layer, a.o_pqkv) : lay(a, layer, a.o_pgu);
    LL* ss_out = is_qkv ? lay(a, layer, a.o_ssin) : lay(a, layer, a.o_sspost);
    const int ld_out = nslabs * SLAB;
    const int nitems = nslabs * S;
    const bool from_embed = is_qkv && layer == 0;
    if (c.cta >= nitems) return;
    int off = 0;
    for (int i = c.cta; i < nitems; i += c.nb) {
        const int slab = i / S, split = i - slab * S;
        const int k0 = split * R;
        const int nrows = max(0, min(a.H, k0 + R) - k0);
        float ssq = 0.f;
        for (int r = c.tid; r < nrows; r += CONSUMERS) {
            const int k = k0 + r;
            float h;
            if (from_embed) {
                h = a.embed_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(a.embed)[(size_t)c.sh.token * a.H + k])
                                 : reinterpret_cast<const float*>(a.embed)[(size_t)c.sh.token * a.H + k];
            } else {
                h = ll_sum(c, part_prev + k, (size_t)a.slabs_h * SLAB, Sprev, h_prev + k);
            }
            c.xs[off + r] = h * __ldg(norm_w + k);
            ssq = fmaf(h, h, ssq);
            if (slab == 0) ll_store(h_out + k, h, c.gen);
        }
        if (slab == 0) {  // uniform per CTA: the slab-0 item of a split publishes the slice's sum of squares
            ssq = block_sum(c, ssq);
            if (c.tid == 0) ll_store(ss_out + split, ssq, c.gen);
        }
        off += nrows;
    }
    consumer_sync();
    sub_mark(c, 0);
    off = 0;
    for (int i = c.cta; i < nitems; i += c.nb) {
        const int slab = i / S, split = i - slab * S;
        const int k0 = split * R;
        const int nrows = max(0, min(a.H, k0 + R) - k0);
        const float v = run_item(c, c.xs + off, nrows);
        if (c.tid < SLAB) ll_store(part_out + (size_t)split * ld_out + slab * SLAB + c.tid, v, c.gen);
        off += nrows;
    }
}

// P3: input slice = attention output, merged over the page chunks.
__device__ void phase_o_proj(Ctx& c, int layer, int nc) {
    const MkArgs& a = c.a;
    const int g = a.heads / a.kvh;
    const int nitems = a.slabs_h * a.S3;
    if (c.cta >= nitems) return;
    int off = 0;
    for (int i = c.cta; i < nitems; i += c.nb) {
        const int slab = i / a.S3, split = i - slab * a.S3;
        const int k0 = split * a.R3;
        const int nrows = max(0, min(a.qdim, k0 + a.R3) - k0);
        for (int r = c.tid; r < nrows; r += CONSUMERS) {
            const int k = k0 + r;
            const int head = k / a.hd, d = k - head * a.hd;
            const int kh = head / g, j = head - kh * g;
            const LL* ml = lay(a, layer, a.o_attml) + ((size_t)kh * a.att_cap) * g * 2 + j * 2;
            const LL* ac = lay(a, layer, a.o_attacc) + ((size_t)kh * a.att_cap) * g * a.hd + (size_t)j * a.hd + d;
            // merge the page chunks in order, eight at a time (24 loads in flight per round trip)
            float M = -INFINITY, num = 0.f, den = 0.f;
            for (int c0 = 0; c0 < nc; c0 += 8) {
                float ms[8], ls[8], as[8];
                unsigned long long it = 0;
                while (true) {
                    bool ready = true;
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        ms[u] = -INFINITY;
                        ls[u] = 0.f;
                        as[u] = 0.f;
                        if (c0 + u < nc) {
                            uint32_t g0, g1, g2;
                            ll_load(ml + (size_t)(c0 + u) * g * 2, ms[u], g0);
                            ll_load(ml + (size_t)(c0 + u) * g * 2 + 1, ls[u], g1);
                            ll_load(ac + (size_t)(c0 + u) * g * a.hd, as[u], g2);
                            ready = ready && g0 == c.gen && g1 == c.gen && g2 == c.gen;
                        }
                    }
                    if (ready || poll_overrun(c, it)) break;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (ms[u] > -INFINITY) {
                        const float mn = fmaxf(M, ms[u]);
                        const float so = expf(M - mn), sn = expf(ms[u] - mn);
                        num = num * so + as[u] * sn;
                        den = den * so + ls[u] * sn;
                        M = mn;
                    }
                }
            }
            c.xs[off + r] = num / den;
        }
        off += nrows;
    }
    consumer_sync();
    sub_mark(c, 0);
    off = 0;
    for (int i = c.cta; i < nitems; i += c.nb) {
        const int slab = i / a.S3, split = i - slab * a.S3;
        const int k0 = split * a.R3;
        const int nrows = max(0, min(a.qdim, k0 + a.R3) - k0);
        const float v = run_item(c, c.xs + off, nrows);
        if (c.tid < SLAB) ll_store(lay(a, layer, a.o_po) + (size_t)split * a.slabs_h * SLAB + slab * SLAB + c.tid, v, c.gen);
        off += nrows;
    }
}

// P5: input slice = SiLU(gate) * up from the gate/up partials (1/rms applied here).
__device__ void phase_down(Ctx& c, int layer) {
    const MkArgs& a = c.a;
    const int nitems = a.slabs_h * a.S5;
    if (c.cta >= nitems) return;
    const float inv = inv_rms_from(c, lay(a, layer, a.o_sspost), a.S4, a.H, a.eps);
    const LL* p_gu = lay(a, layer, a.o_pgu);
    const int ld_gu = a.slabs_gu * SLAB;
    int off = 0;
    for (int i = c.cta; i < nitems; i += c.nb) {
        const int slab = i / a.S5, split = i - slab * a.S5;
        const int k0 = split * a.R5;
        const int nrows = max(0, min(a.I, k0 + a.R5) - k0);
        for (int r = c.tid; r < nrows; r += CONSUMERS) {
            const int k = k0 + r;
            const int col = (k >> 6) * SLAB + (k & 63);
            const float gsum = ll_sum(c, p_gu + col, (size_t)ld_gu, a.S4);
            const float usum = ll_sum(c, p_gu + col + 64, (size_t)ld_gu, a.S4);
            const float gt = gsum * inv, up = usum * inv;
            c.xs[off + r] = (gt / (1.0f + expf(-gt))) * up;
        }
        off += nrows;
    }
    consumer_sync();
    sub_mark(c, 0);
    off = 0;
    for (int i = c.cta; i < nitems; i += c.nb) {
        const int slab = i / a.S5, split = i - slab * a.S5;
        const int k0 = split * a.R5;
        const int nrows = max(0, min(a.I, k0 + a.R5) - k0);
        const float v = run_item(c, c.xs + off, nrows);
        if (c.tid < SLAB) ll_store(lay(a, layer, a.o_pdown) + (size_t)split * a.slabs_h * SLAB + slab * SLAB + c.tid, v, c.gen);
        off += nrows;
    }
}

// P2: attention items (KV head, page chunk).  Every item rebuilds q (g heads), k and v of the new
// token from the QKV partials (1/rms, bias, QK-norm, RoPE); the item whose chunk holds the new
// position also appends k and v to the cache page.  The K/V tile of the first page is requested
// before anything else so that its latency overlaps the partial sums.
__device__ void phase_attention(Ctx& c, int layer, int npages, int ppc, int nc) {
    const MkArgs& a = c.a;
    const MkLayer& w = a.layers[layer];
    const int g = a.heads / a.kvh, hd = a.hd, half = hd >> 1;
    const int nitems = a.kvh * nc;
    if (c.cta >= nitems) return;
    const int pos = c.sh.pos;
    const int kvlen = pos + 1;
    const int KLD = hd + 4;
    float* raw = c.att;                       // [(g+2)][hd]  q heads, k, v before RoPE
    float* q_s = raw + (G_MAX_MK + 2) * 128;  // [g][hd]
    float* kn = q_s + G_MAX_MK * 128;         // [hd] new k (after RoPE)
    float* vn = kn + 128;                     // [hd] new v
    float* kt = vn + 128;                     // [16][KLD]
    float* vt = kt + PTK * (128 + 4);         // [16][hd]
    float* p_s = vt + PTK * 128;              // [8][16]
    const int ld_qkv = a.slabs_qkv * SLAB;
    const int32_t* pt = a.page_table;
    const int per16 = a.kv_bf16 ? 8 : 4;
    const int pieces = PTK * hd / per16;  // 16-byte pieces per tile: <= 512, two per thread at most
    for (int i = c.cta; i < nitems; i += c.nb) {
        const int kh = i / nc, cc = i - kh * nc;
        const int p0 = cc * ppc, p1 = min(npages, p0 + ppc);
        const int pnew = pos / PTK;
        // tile registers of the current page (loads in flight while q/k/v are being rebuilt)
        uint4 kq[2], vq[2];
        auto issue_tile = [&](int p) {
            const size_t tile_b = (((size_t)pt[p] * a.kvh + kh) * PTK * hd) * (a.kv_bf16 ? 2 : 4);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int pc = c.tid + u * CONSUMERS;
                if (pc < pieces) {
                    kq[u] = *(reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(w.k_pool) + tile_b) + pc);
                    vq[u] = *(reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(w.v_pool) + tile_b) + pc);
                }
            }
        };
        auto store_tile = [&]() {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int pc = c.tid + u * CONSUMERS;
                if (pc < pieces) {
                    const int e = pc * per16, tt = e / hd, d = e - tt * hd;
                    float* vo = vt + tt * hd + d;
                    // K pages are chunk-major (k_tile_off): a 16-byte piece is one 4-element chunk of one
                    // token (f32) or of two neighbouring tokens (bf16)
                    const int kc = e >> 6, ktok = (e >> 2) & 15;
                    float* ko = kt + ktok * KLD + kc * 4;
                    if (a.kv_bf16) {
                        ko[0] = bf16_lo(kq[u].x); ko[1] = bf16_hi(kq[u].x); ko[2] = bf16_lo(kq[u].y); ko[3] = bf16_hi(kq[u].y);
                        ko[KLD + 0] = bf16_lo(kq[u].z); ko[KLD + 1] = bf16_hi(kq[u].z); ko[KLD + 2] = bf16_lo(kq[u].w); ko[KLD + 3] = bf16_hi(kq[u].w);
                        vo[0] = bf16_lo(vq[u].x); vo[1] = bf16_hi(vq[u].x); vo[2] = bf16_lo(vq[u].y); vo[3] = bf16_hi(vq[u].y);
                        vo[4] = bf16_lo(vq[u].z); vo[5] = bf16_hi(vq[u].z); vo[6] = bf16_lo(vq[u].w); vo[7] = bf16_hi(vq[u].w);
                    } else {
                        *reinterpret_cast<float4*>(ko) = make_float4(__uint_as_float(kq[u].x), __uint_as_float(kq[u].y), __uint_as_float(kq[u].z), __uint_as_float(kq[u].w));
                        *reinterpret_cast<float4*>(vo) = make_float4(__uint_as_float(vq[u].x), __uint_as_float(vq[u].y), __uint_as_float(vq[u].z), __uint_as_float(vq[u].w));
                    }
                }
            }
        };
        if (p0 < p1) issue_tile(p0);
        // ---- q / k / v of the new token: all partial loads of up to three elements in flight ----
        {
            const int total = (g + 2) * hd;  // <= 1280: at most five elements per thread
            const float inv = inv_rms_from(c, lay(a, layer, a.o_ssin), a.S1, a.H, a.eps);
            const LL* p_qkv = lay(a, layer, a.o_pqkv);
            for (int base = 0; base < total; base += 2 * CONSUMERS) {
                float vals[2];
                int ns[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int idx = base + c.tid + u * CONSUMERS;
                    vals[u] = 0.f;
                    ns[u] = -1;
                    if (idx < total) {
                        const int part = idx / hd, d = idx - part * hd;
                        ns[u] = part < g ? (kh * g + part) * hd + d : (part == g ? a.qdim + kh * hd + d : a.qdim + a.kvdim + kh * hd + d);
                        vals[u] = ll_sum(c, p_qkv + ns[u], (size_t)ld_qkv, a.S1);
                    }
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int idx = base + c.tid + u * CONSUMERS;
                    if (idx < total) {
                        float v = vals[u] * inv;
                        if (w.qkv_bias) v += __ldg(w.qkv_bias + ns[u]);
                        raw[idx] = v;
                    }
                }
            }
        }
        consumer_sync();
        if (a.has_qk_norm) {
            for (int p = c.warp; p < g + 1; p += NW) {  // q heads and k
                float* v = raw + p * hd;
                float s = 0.f;
                for (int d = c.lane; d < hd; d += 32) s = fmaf(v[d], v[d], s);
                s = warp_sum(s);
                const float iv = 1.0f / sqrtf(s / (float)hd + a.eps);
                const float* nw = p < g ? w.q_norm : w.k_norm;
                for (int d = c.lane; d < hd; d += 32) v[d] = (v[d] * iv) * __ldg(nw + d);
            }
            consumer_sync();
        }
        for (int idx = c.tid; idx < (g + 2) * hd; idx += CONSUMERS) {
            const int part = idx / hd, d = idx - part * hd;
            float v = raw[idx];
            if (part <= g) {
                const float other = d < half ? -raw[idx + half] : raw[idx - half];
                v = fmaf(other, __ldg(a.rope_sin + (size_t)pos * hd + d), v * __ldg(a.rope_cos + (size_t)pos * hd + d));
            }
            if (a.kv_bf16 && part >= g) v = bf16_bits_to_f32(f32_to_bf16_rne(v));
            if (part < g) q_s[part * hd + d] = v;
            else if (part == g) kn[d] = v;
            else vn[d] = v;
        }
        consumer_sync();
        if (pnew >= p0 && pnew < p1) {  // append to the cache (KvCache::append_*, src/runtime.rs:521-570)
            const size_t tile = ((size_t)pt[pnew] * a.kvh + kh) * PTK * hd;
            for (int d = c.tid; d < hd; d += CONSUMERS) {
                const size_t ko = tile + k_tile_off(pos % PTK, d), vo = tile + v_tile_off(pos % PTK, d, hd);
                if (a.kv_bf16) {
                    reinterpret_cast<uint16_t*>(w.k_pool)[ko] = f32_to_bf16_rne(kn[d]);
                    reinterpret_cast<uint16_t*>(w.v_pool)[vo] = f32_to_bf16_rne(vn[d]);
                } else {
                    reinterpret_cast<float*>(w.k_pool)[ko] = kn[d];
                    reinterpret_cast<float*>(w.v_pool)[vo] = vn[d];
                }
            }
        }
        // ---- pages of this chunk: warp j <-> query head j ----
        const int j = c.warp;
        const int t = c.lane & 15, hf = c.lane >> 4;
        const int epl = hd >> 5;
        float run_m = -INFINITY, run_l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int p = p0; p < p1; ++p) {
            store_tile();
            if (p == pnew) {
                consumer_sync();  // tile rows are in place before the new token's row replaces its slot
                for (int d = c.tid; d < hd; d += CONSUMERS) {
                    kt[(pos % PTK) * KLD + d] = kn[d];
                    vt[(pos % PTK) * hd + d] = vn[d];
                }
            }
            consumer_sync();
            if (p + 1 < p1) issue_tile(p + 1);
            if (j < g) {
                const float* kr = kt + t * KLD + hf * half;
                const float* qr = q_s + j * hd + hf * half;
                float s = 0.f;
                for (int dc = 0; dc < half; dc += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(kr + dc);
                    const float4 q4 = *reinterpret_cast<const float4*>(qr + dc);
                    s = fmaf(q4.x, k4.x, s);
                    s = fmaf(q4.y, k4.y, s);
                    s = fmaf(q4.z, k4.z, s);
                    s = fmaf(q4.w, k4.w, s);
                }
                s += __shfl_xor_sync(0xffffffffu, s, 16);
                const bool valid = (p * PTK + t) < kvlen;
                const float sc = valid ? s * a.scale : -INFINITY;
                float mx = sc;
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float m_new = fmaxf(run_m, mx);
                const float pr = valid ? expf(sc - m_new) : 0.f;
                float ps = pr;
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
                const float corr = expf(run_m - m_new);
                run_l = run_l * corr + ps;
                run_m = m_new;
                float* pw = p_s + j * PTK;
                if (hf == 0) pw[t] = pr;
                __syncwarp();
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] *= corr;
                for (int tt = 0; tt < PTK; ++tt) {
                    const float pv = pw[tt];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (e < epl) acc[e] = fmaf(pv, vt[tt * hd + c.lane * epl + e], acc[e]);
                }
                __syncwarp();
            }
            consumer_sync();  // tiles free for the next page
        }
        if (j < g) {
            const size_t base = ((size_t)kh * a.att_cap + cc) * g + j;
            if (c.lane == 0) {
                ll_store(lay(a, layer, a.o_attml) + base * 2 + 0, run_m, c.gen);
                ll_store(lay(a, layer, a.o_attml) + base * 2 + 1, run_l, c.gen);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (e < epl) ll_store(lay(a, layer, a.o_attacc) + base * hd + c.lane * epl + e, acc[e], c.gen);
        }
    }
}

// Final norm + LM head + argmax partials.
__device__ void phase_lm_head(Ctx& c) {
    const MkArgs& a = c.a;
    float ssq = 0.f;
    for (int k = c.tid; k < a.H; k += CONSUMERS) {
        const float h = ll_sum(c, lay(a, a.L - 1, a.o_pdown) + k, (size_t)a.slabs_h * SLAB, a.S5, lay(a, a.L - 1, a.o_hmid) + k);
        c.xs[k] = h * __ldg(a.final_norm + k);
        ssq = fmaf(h, h, ssq);
    }
    ssq = block_sum(c, ssq);
    const float inv = 1.0f / sqrtf(ssq / (float)a.H + a.eps);
    float bv = -INFINITY;
    int bi = -1;
    for (int slab = c.cta; slab < a.slabs_v; slab += c.nb) {
        const float s = run_item(c, c.xs, a.H);
        if (c.tid < SLAB) {
            const int n = slab * SLAB + c.tid;
            if (n < a.V) {
                const float v = s * inv;
                a.logits[n] = v;
                if (bi < 0 || v > bv || (v == bv && n > bi)) { bv = v; bi = n; }
            }
        }
    }
    // block argmax (ties to the highest index), threads >= 128 hold (-inf, -1)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi > bi))) { bv = ov; bi = oi; }
    }
    consumer_sync();
    if (c.lane == 0) {
        c.sh.wsum[c.warp] = bv;
        c.sh.widx[c.warp] = bi;
    }
    consumer_sync();
    if (c.tid == 0) {
        for (int wv = 1; wv < NW; ++wv) {
            const float ov = c.sh.wsum[wv];
            const int oi = c.sh.widx[wv];
            if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi > bi))) { bv = ov; bi = oi; }
        }
        ll_store(a.amax_v + c.cta, bv, c.gen);
        ll_store(a.amax_i + c.cta, __int_as_float(bi), c.gen);
    }
}

__global__ void __launch_bounds__(MK_THREADS, 1) decode_persistent_kernel(const MkArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ Shared sh;
    Ctx c{a, sh, smem_raw, nullptr, nullptr, (int)blockIdx.x, (int)gridDim.x, (int)threadIdx.x, (int)(threadIdx.x & 31), (int)(threadIdx.x >> 5), 0u, 0u, 0, 0};
    c.xs = reinterpret_cast<float*>(smem_raw + (size_t)NSTAGE * STAGE_BYTES);
    c.att = c.xs + XS_MAX;
    if (c.tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&sh.full[s], 1);
            mbar_init(&sh.empty[s], NW);
        }
        sh.abort = 0;
        const int pos = *reinterpret_cast<volatile const int32_t*>(a.pos);
        unsigned int tok = *reinterpret_cast<volatile const uint32_t*>(a.token);
        if (tok >= (unsigned int)a.V) {
            atomicExch(a.err_flag, 1);
            tok = 0;
        }
        sh.pos = pos;
        sh.token = (int)tok;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (c.warp == NW) {
        if (c.lane == 0) producer(c);
        return;
    }
    if (a.trace && c.cta == 0 && c.tid == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        a.trace[0] = t;
    }
    const unsigned int launch = ld_cg_u32(a.launch_idx);
    c.gen = launch + 1u;  // never 0: the exchange buffers start zeroed
    const int pos = sh.pos;
    const int npages = pos / PTK + 1;
    const int ppc = (npages + a.att_cap - 1) / a.att_cap;
    const int nc = (npages + ppc - 1) / ppc;

    for (int l = 0; l < a.L; ++l) {
        phase_norm_proj(c, l, true);
        phase_mark(c);
        phase_attention(c, l, npages, ppc, nc);
        phase_mark(c);
        phase_o_proj(c, l, nc);
        phase_mark(c);
        phase_norm_proj(c, l, false);
        phase_mark(c);
        phase_down(c, l);
        phase_mark(c);
    }
    phase_lm_head(c);
    phase_mark(c);
    if (c.cta == 0 && c.warp == 0) {
        float bv = -INFINITY;
        int bi = -1;
        for (int i = c.lane; i < c.nb; i += 32) {
            const float v = ll_get(c, a.amax_v + i);
            const int ix = __float_as_int(ll_get(c, a.amax_i + i));
            if (ix >= 0 && (bi < 0 || v > bv || (v == bv && ix > bi))) { bv = v; bi = ix; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi > bi))) { bv = ov; bi = oi; }
        }
        if (c.lane == 0) {
            const uint32_t tok = bi < 0 ? 0u : (uint32_t)bi;
            a.next_tok[0] = tok;
            a.feed_tok[0] = tok;
            const int np = pos + 1;
            a.pos[0] = np;
            a.hist[np] = tok;
            *a.launch_idx = launch + 1;  // every CTA read it before the first barrier
        }
    }
}

}  // namespace

size_t mk_smem_bytes() { return (size_t)NSTAGE * STAGE_BYTES + sizeof(float) * (XS_MAX + MK_ATT_FLOATS); }
int mk_threads() { return MK_THREADS; }
int mk_xs_max() { return XS_MAX; }

cudaError_t mk_prepare(int* max_ctas_per_sm) {
    cudaError_t e = cudaFuncSetAttribute(decode_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mk_smem_bytes());
    if (e != cudaSuccess) return e;
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(max_ctas_per_sm, decode_persistent_kernel, MK_THREADS, mk_smem_bytes());
}

cudaError_t launch_decode_persistent(const MkArgs& a, int nb, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)nb);
    cfg.blockDim = dim3(MK_THREADS);
    cfg.dynamicSmemBytes = mk_smem_bytes();
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_persistent_kernel, a);
}

}  // namespace hm
