// Weight-streaming bf16 GEMV / skinny GEMM (M <= 8 rows of f32 activations).
//
// Stands in for Homura's mixed bf16 x f32 -> f32 matmul (src/graph_builder/emit_linalg.rs:
// 1928-2008, 2224-2307) on every projection of the decode step, fused with the work the
// reference puts in the same compiled kernel:
//   prologue  RMSNorm of the input row            (src/hf/emitter.rs:601,790,845)
//   epilogue  bias + QK-norm + RoPE + KV append   (src/hf/emitter.rs:604-649, src/runtime.rs:1729-1755)
//             residual add                        (src/hf/emitter.rs:787,804)
//             SiLU(gate) * up                     (src/hf/emitter.rs:794-799)
//             logits + per-slab argmax            (src/hf/emitter.rs:845-846, src/generate.rs:457-468)
//
// HBM-bound by design: a CTA streams one contiguous run of a 128-column weight slab with
// 128-bit loads (thread t always reads bytes [16t, 16t+16) of each 4 KB pass, so a warp
// covers 512 contiguous bytes), keeps 8 column accumulators per thread in f32, and never
// re-reads a weight byte.  K is split across CTAs so that even the 1.6 MB projections put
// work on every SM; partial sums go through global scratch and the CTA that arrives last at
// the slab's ticket adds them in split order (deterministic, no float atomics) and runs the
// epilogue.  Nothing here spins: a CTA that is not last simply exits.
#include <atomic>
#include <mutex>

#include "../../include/homura_b200.h"
#include <cstdlib>

#include "common.cuh"
#include "launch_attrs.h"
#include "mbarrier.cuh"

namespace hm {

namespace {

constexpr int U = 8;  // 128-bit loads in flight per thread

// One weight row segment (8 bf16 columns) times the M activation values of that row.  The accumulators are
// pairs, so that one packed FMA (two independent IEEE FMAs, same bits as two scalar ones) serves two columns:
// the multiply of the staged kernels is bound by instruction issue, not by shared-memory bandwidth.
template <int M>
__device__ __forceinline__ void fma_row(float2 (&acc)[M][4], const uint4& w, const float* __restrict__ xs, int rps, int row) {
    const float2 f0 = make_float2(bf16_lo(w.x), bf16_hi(w.x));
    const float2 f1 = make_float2(bf16_lo(w.y), bf16_hi(w.y));
    const float2 f2 = make_float2(bf16_lo(w.z), bf16_hi(w.z));
    const float2 f3 = make_float2(bf16_lo(w.w), bf16_hi(w.w));
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float xv = xs[m * rps + row];
        const float2 x2 = make_float2(xv, xv);
        acc[m][0] = __ffma2_rn(x2, f0, acc[m][0]);
        acc[m][1] = __ffma2_rn(x2, f1, acc[m][1]);
        acc[m][2] = __ffma2_rn(x2, f2, acc[m][2]);
        acc[m][3] = __ffma2_rn(x2, f3, acc[m][3]);
    }
}

// Sum of NS partials `stride` floats apart, in slot order, with every load issued before the first add (a loop
// bounded by a run-time count is compiled with one shared-memory round trip per iteration).
template <int NS>
__device__ __forceinline__ float sum_slots(const float* s, int stride) {
    float v[NS];
#pragma unroll
    for (int r = 0; r < NS; ++r) v[r] = s[r * stride];
    float t = v[0];
#pragma unroll
    for (int r = 1; r < NS; ++r) t += v[r];
    return t;
}
__device__ __forceinline__ float sum_slots_any(const float* s, int stride, int n) {
    switch (n) {
        case 2: return sum_slots<2>(s, stride);
        case 3: return sum_slots<3>(s, stride);
        case 4: return sum_slots<4>(s, stride);
        case 5: return sum_slots<5>(s, stride);
        case 6: return sum_slots<6>(s, stride);
        case 7: return sum_slots<7>(s, stride);
        case 8: return sum_slots<8>(s, stride);
        case 10: return sum_slots<10>(s, stride);
        case 12: return sum_slots<12>(s, stride);
        case 14: return sum_slots<14>(s, stride);
        case 16: return sum_slots<16>(s, stride);
    }
    float t = s[0];
    for (int r = 1; r < n; ++r) t += s[r * stride];
    return t;
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i > bi); }

// The unsplit M = 1 variant (LM head: one long stream per CTA) runs three CTAs per SM (<= 85
// registers) to keep ~96 KB of weight loads in flight per SM; measured 5.0 -> 5.3 TB/s.  The
// clustered one-row variants are latency chains and were slower under a tighter register budget.  The
// 2- and 4-row variants (split or not) are held to 128 registers so that two CTAs stay resident per SM:
// wide projections launch more CTAs than there are SMs.
// ST (with CL): the CTA's whole weight slice (rows [k0, k0+nrows) of its slab, one contiguous byte range of
// at most GEMV_STAGE_MAX bytes) is pulled into shared memory by bulk copies issued BEFORE the dependency
// wait, so that by the time the predecessor has finished the multiply runs out of shared memory and HBM
// latency is off the critical path of the dependent-kernel chain.
template <int M, bool CL, bool ST>
__global__ void __launch_bounds__(GEMV_THREADS, CL ? (M <= 4 ? 2 : 1) : (M == 1 ? 3 : (M <= 4 ? 2 : 1))) gemv_bf16_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) float smem_raw[];
    const int rps = a.rows_per_split;
    // staged weights first (bulk copies want 16-byte aligned destinations), then the f32 scratch
    float* smem = ST ? smem_raw + (size_t)rps * (SLAB * 2 / 4) : smem_raw;
    const uint4* wst = reinterpret_cast<const uint4*>(smem_raw);  // [nrows][16] x 16 B
    __shared__ uint64_t s_wbar, s_rbar;  // staged weights; split-K partials pushed into rank 0
    __shared__ volatile int s_abort;
    float* xs = smem;                 // [M][rps]
    float* red = smem + M * rps;      // [8][M][128], later vals[M][128]
    float* slots = red + 8 * M * SLAB;  // cluster variant, rank 0: [ksplit][M][128] partials pushed by the ranks
    // values that do not depend on the previous kernel, fetched before the dependency wait:
    float* nws = CL ? slots + a.ksplit * M * SLAB : slots;  // [rps] RMSNorm weights of this CTA's K range
    float* cs_s = nws + rps;                        // [M][128] RoPE cos, [M][128] sin of this slab's columns (QKV epilogue)
    float* sn_s = cs_s + M * SLAB;
    float* bias_s = sn_s + M * SLAB;                // [128] bias of this slab's columns (QKV epilogue with bias)
    __shared__ int s_page[MAX_M], s_pos[MAX_M];     // page and position of every row's new token
    __shared__ float s_inv[MAX_M];
    __shared__ float s_warp[8][MAX_M];
    __shared__ int s_last;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int slab = blockIdx.x / a.ksplit;
    const int split = blockIdx.x - slab * a.ksplit;
    const int k0 = split * rps;
    const int nrows = max(0, min(a.K, k0 + rps) - k0);
    const int cg = tid & 15, rl = tid >> 4;
    const int niter = (nrows + ROWS_PER_PASS - 1) / ROWS_PER_PASS;
    const bool col_ok = (slab * SLAB + cg * 8) < a.N;
    const char* wbase = (const char*)a.W + (long long)slab * a.slab_stride + (long long)(k0 + rl) * a.row_stride + cg * 16;
    const long long pass_stride = (long long)ROWS_PER_PASS * a.row_stride;

    HM_TRACE(const bool tr = a.trace != nullptr && blockIdx.x == 0 && tid == 0;)
    HM_TRACE(if (tr) a.trace[0] = global_timer();)  // CTA resident
    HM_TRACE(if (a.trace && tid == 0) atomicMax(a.trace + 8, global_timer());)  // the launch's last CTA to become resident
    pdl_launch_dependents();
    if (a.pf_bytes && tid < 32) l2_prefetch_slice(a.pf_ptr, a.pf_bytes, blockIdx.x, gridDim.x, tid);

    // Weights never depend on a previous kernel, so they are requested before the dependency wait:
    // the whole slice into shared memory (ST), or the first batch of streaming loads into registers.
    uint4 w[U];
    if (ST) {
        if (tid == 0) {
            mb_init(&s_wbar, 1);
            s_abort = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            const uint32_t bytes = (uint32_t)nrows * (SLAB * 2);
            if (bytes) {
                mb_expect_tx(&s_wbar, bytes);
                const char* src = (const char*)a.W + (long long)slab * a.slab_stride + (long long)k0 * a.row_stride;
                for (uint32_t o = 0; o < bytes; o += 16384u) bulk_copy((char*)smem_raw + o, src + o, min(16384u, bytes - o), &s_wbar);
            }
        }
    } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool ok = col_ok && (u * ROWS_PER_PASS + rl) < nrows;
            w[u] = ok ? ld_stream_u4(wbase + u * pass_stride) : make_uint4(0, 0, 0, 0);
        }
    }

    if (CL) {
        // Rank 0 of the cluster receives every other rank's partial by asynchronous stores that count bytes on
        // its mbarrier; the barrier is armed here and published by a cluster barrier that costs nothing on the
        // dependent-kernel chain because it happens before the dependency wait.
        if (tid == 0) {
            if (!ST) s_abort = 0;
            if (cluster_ctarank() == 0) {
                mb_init(&s_rbar, 1);
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                mb_expect_tx(&s_rbar, (uint32_t)(a.ksplit - 1) * (uint32_t)(M * SLAB) * 4u);
            }
        }
        cluster_arrive_release();
        cluster_wait_acquire();
    }
    if (a.pro == PRO_RMSNORM)
        for (int r = tid; r < nrows; r += GEMV_THREADS) nws[r] = __ldg(a.norm_w + k0 + r);
    if (a.epi == EPI_QKV_ROPE) {
        // positions, the RoPE table and the page table were final before this step's launches began
        const int n0e = slab * SLAB;
        for (int idx = tid; idx < M * SLAB; idx += GEMV_THREADS) {
            const int m = idx / SLAB, c = idx % SLAB;
            if (m < a.m_valid && n0e + c < a.q_dim + a.kv_dim) {  // V columns are not rotated
                const int pos = a.row_pos[m], d = c % a.hd;
                cs_s[idx] = __ldg(a.rope_cos + (size_t)pos * a.hd + d);
                sn_s[idx] = __ldg(a.rope_sin + (size_t)pos * a.hd + d);
            }
        }
        if (tid < M && tid < a.m_valid) {
            const int pos = a.row_pos[tid], seq = a.row_seq ? a.row_seq[tid] : a.seq_base + tid;
            s_pos[tid] = pos;
            s_page[tid] = a.kv.page_table[(size_t)seq * a.kv.max_pages + pos / a.kv.page_tokens];
        }
        if (a.bias && tid < SLAB) bias_s[tid] = n0e + tid < a.N ? __ldg(a.bias + n0e + tid) : 0.f;
    }

    pdl_wait();
    // the RMSNorm weights fetched above are read below by other threads than those that stored them (a CTA that
    // became resident just before its dependency resolved may still have those loads in flight)
    if (CL && a.pro == PRO_RMSNORM) __syncthreads();
    HM_TRACE(if (tr) a.trace[1] = global_timer();)  // predecessor complete

    // the residual element this thread adds in the epilogue (known epilogue CTA only): requested now, used after the reduction
    float resid_v = 0.f;
    const bool resid_early = a.epi == EPI_STORE && a.resid && tid < M * SLAB && (CL ? cluster_ctarank() == 0 : a.ksplit == 1);
    if (resid_early) {
        const int m = tid / SLAB, n = slab * SLAB + (tid % SLAB);
        if (n < a.N && m < a.m_valid) resid_v = ld_cg_f32(a.resid + (size_t)m * a.ldy + n);
    }

    // ---- prologue: activation slice [k0, k0+nrows) of every row into shared memory ----
    // Cluster launches apply the RMSNorm row factor AFTER the split-K sum: y = inv * sum_k W[k][n] * (x[k] * w[k]).
    // Every rank stages its slice of x * w at once; only rank 0 reads the whole rows for their sums of squares,
    // while the multiply is already running, and scales the reduced sums.  (The unsplit and ticket variants
    // keep the reference's order, (x * inv) * w before the product.)
    const bool defer_norm = CL && a.pro == PRO_RMSNORM && a.K <= 4096 && (a.K & 3) == 0 && (a.ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0;
    const bool norm_rank0 = defer_norm && cluster_ctarank() == 0;
    float4 rowv[CL ? M : 1][4];
    if (defer_norm) {
        stage_rows<GEMV_THREADS, M>(a.x + k0, a.ldx, xs, rps, nrows, tid, nws);
        // rank 0: the whole rows are requested now (up to four 16-byte loads per thread and row) and squared
        // after the multiply, so that their latency and the reduction overlap it
        if (norm_rank0) {
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int idx = tid + i * GEMV_THREADS;
                    rowv[m][i] = idx < (a.K >> 2) ? ld_cg_f32x4(a.x + (size_t)m * a.ldx + 4 * (size_t)idx) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
        }
    } else if (a.pro == PRO_RMSNORM) {
        float ss[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float s = 0.f;
            const float* xr = a.x + (size_t)m * a.ldx;
#pragma unroll 4
            for (int k = tid; k < a.K; k += GEMV_THREADS) {
                float v = __ldg(xr + k);
                s = fmaf(v, v, s);
            }
            ss[m] = warp_sum(s);
        }
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < M; ++m) s_warp[warp][m] = ss[m];
        }
        __syncthreads();
        if (tid < M) {
            float s = 0.f;
#pragma unroll
            for (int wv = 0; wv < 8; ++wv) s += s_warp[wv][tid];
            s_inv[tid] = 1.0f / sqrtf(s / (float)a.K + a.eps);
        }
        __syncthreads();
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float inv = s_inv[m];
            const float* xr = a.x + (size_t)m * a.ldx + k0;
            for (int r = tid; r < nrows; r += GEMV_THREADS) xs[m * rps + r] = (__ldg(xr + r) * inv) * nws[r];
        }
    } else {
        stage_rows<GEMV_THREADS, M>(a.x + k0, a.ldx, xs, rps, nrows, tid);
    }
    __syncthreads();
    __syncthreads();
    HM_TRACE(if (tr) a.trace[2] = global_timer();)  // activations in shared memory

    // ---- main loop: stream the slab run, 8 column accumulators per row per thread ----
    float2 acc[M][4];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[m][j] = make_float2(0.f, 0.f);

    if (ST) {
        // every thread waits (bounded) for the bulk copies, then multiplies out of shared memory
        const bool ok = nrows == 0 || mb_wait(&s_wbar, 0, a.err_flag, &s_abort);
        if (ok) {
#pragma unroll 4
            for (int row = rl; row < nrows; row += ROWS_PER_PASS) fma_row<M>(acc, wst[row * 16 + cg], xs, rps, row);
        }
    } else
    for (int it = 0; it < niter; it += U) {
        uint4 cur[U];
#pragma unroll
        for (int u = 0; u < U; ++u) cur[u] = w[u];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int p = it + U + u;
            const bool ok = col_ok && p < niter && (p * ROWS_PER_PASS + rl) < nrows;
            w[u] = ok ? ld_stream_u4(wbase + (long long)p * pass_stride) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int row = (it + u) * ROWS_PER_PASS + rl;
            if (row < nrows) fma_row<M>(acc, cur[u], xs, rps, row);
        }
    }

    HM_TRACE(if (tr) a.trace[3] = global_timer();)  // weights multiplied
    if (norm_rank0) {  // sums of squares of the whole rows, published by the barrier of the reduction below
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) s = fmaf(rowv[m][i].x, rowv[m][i].x, fmaf(rowv[m][i].y, rowv[m][i].y, fmaf(rowv[m][i].z, rowv[m][i].z, fmaf(rowv[m][i].w, rowv[m][i].w, s))));
            s = warp_sum(s);
            if (lane == 0) s_warp[warp][m] = s;
        }
    }
    // ---- reduce the 16 row lanes: xor-16 shuffle, then across the 8 warps in smem ----
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[m][j].x += __shfl_xor_sync(0xffffffffu, acc[m][j].x, 16);
            acc[m][j].y += __shfl_xor_sync(0xffffffffu, acc[m][j].y, 16);
        }
    if (lane < 16) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float4* dst = reinterpret_cast<float4*>(red + ((warp * M + m) * SLAB + cg * 8));
            dst[0] = make_float4(acc[m][0].x, acc[m][0].y, acc[m][1].x, acc[m][1].y);
            dst[1] = make_float4(acc[m][2].x, acc[m][2].y, acc[m][3].x, acc[m][3].y);
        }
    }
    __syncthreads();
    if (norm_rank0 && tid < M) {  // read by the rank-order sum, two barriers later
        float s = 0.f;
#pragma unroll
        for (int wv = 0; wv < 8; ++wv) s += s_warp[wv][tid];
        s_inv[tid] = 1.0f / sqrtf(s / (float)a.K + a.eps);
    }
    float mine[(M * SLAB + GEMV_THREADS - 1) / GEMV_THREADS];
    float4 mine4 = make_float4(0.f, 0.f, 0.f, 0.f);  // cluster variant: four consecutive columns per thread, sent as one 16-byte store
    if (CL) {
        if (tid < M * SLAB / 4) {
#pragma unroll
            for (int wv = 0; wv < 8; ++wv) {
                const float4 v = *reinterpret_cast<const float4*>(red + wv * M * SLAB + tid * 4);
                mine4.x += v.x; mine4.y += v.y; mine4.z += v.z; mine4.w += v.w;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < (M * SLAB + GEMV_THREADS - 1) / GEMV_THREADS; ++i) {
            const int idx = tid + i * GEMV_THREADS;
            float v = 0.f;
            if (idx < M * SLAB) {
#pragma unroll
                for (int wv = 0; wv < 8; ++wv) v += red[wv * M * SLAB + idx];
            }
            mine[i] = v;
        }
    }
    __syncthreads();
    float* vals = red;  // [M][128]
    if (CL) {
        // The CTAs of one cluster hold the K-splits of this slab.  Every rank but 0 sends its partial into
        // slot `rank` of rank 0's shared memory with asynchronous 16-byte stores that count bytes on rank 0's
        // mbarrier, and is done; rank 0 waits (bounded) for the byte count and adds the slots in rank order
        // from its own shared memory.  No cluster barrier and no remote load on the critical path.
        constexpr int PER = (M * SLAB + GEMV_THREADS - 1) / GEMV_THREADS;
        const uint32_t rank = cluster_ctarank();
        if (tid < M * SLAB / 4) {
            if (rank == 0) *reinterpret_cast<float4*>(slots + tid * 4) = mine4;
            else st_async_f32x4(dsmem_addr(slots + rank * (M * SLAB) + tid * 4, 0u), mine4, dsmem_addr(&s_rbar, 0u));
        }
        if (rank != 0) return;  // nothing reads this CTA's shared memory; its stores are on their way
        __syncthreads();        // rank 0's own slot is read by other threads than those that wrote it
        if (a.ksplit > 1 && !mb_wait_cluster(&s_rbar, 0, a.err_flag, &s_abort)) return;  // bounded
        HM_TRACE(if (tr) a.trace[4] = global_timer();)  // all ranks' partials have landed
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int idx = tid + i * GEMV_THREADS;
            if (idx < M * SLAB) {
                const float v = sum_slots_any(slots + idx, M * SLAB, a.ksplit);
                vals[idx] = defer_norm ? v * s_inv[idx / SLAB] : v;
            }
        }
    } else if (a.ksplit == 1) {
#pragma unroll
        for (int i = 0; i < (M * SLAB + GEMV_THREADS - 1) / GEMV_THREADS; ++i) {
            const int idx = tid + i * GEMV_THREADS;
            if (idx < M * SLAB) vals[idx] = mine[i];
        }
    } else {
        float* part = a.partial + (size_t)(slab * a.ksplit + split) * (M * SLAB);
#pragma unroll
        for (int i = 0; i < (M * SLAB + GEMV_THREADS - 1) / GEMV_THREADS; ++i) {
            const int idx = tid + i * GEMV_THREADS;
            if (idx < M * SLAB) part[idx] = mine[i];
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned int t = atomicAdd(a.tickets + slab, 1u);
            s_last = (t == (unsigned int)(a.ksplit - 1));
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        const float* pbase = a.partial + (size_t)slab * a.ksplit * (M * SLAB);
        for (int idx = tid; idx < M * SLAB; idx += GEMV_THREADS) {
            float v = 0.f;
            for (int s = 0; s < a.ksplit; ++s) v += ld_cg_f32(pbase + (size_t)s * (M * SLAB) + idx);
            vals[idx] = v;
        }
        if (tid == 0) a.tickets[slab] = 0u;  // leave the ticket clean for the next launch
    }
    __syncthreads();

    HM_TRACE(if (tr) a.trace[5] = global_timer();)  // split-K reduced
    // ---- epilogues on vals[M][128] (columns n0 .. n0+127 of the output) ----
    const int n0 = slab * SLAB;
    if (a.epi == EPI_STORE) {
        for (int idx = tid; idx < M * SLAB; idx += GEMV_THREADS) {
            const int m = idx / SLAB, n = n0 + (idx % SLAB);
            if (n < a.N && m < a.m_valid) {
                float v = vals[idx];
                if (a.bias) v += __ldg(a.bias + n);
                if (a.resid) v = (resid_early && idx == tid ? resid_v : a.resid[(size_t)m * a.ldy + n]) + v;
                a.y[(size_t)m * a.ldy + n] = v;
            }
        }
    } else if (a.epi == EPI_SWIGLU) {
        // slab = 64 gate columns followed by the 64 matching up columns
        for (int idx = tid; idx < M * 64; idx += GEMV_THREADS) {
            const int m = idx / 64, c = idx % 64;
            const int j = slab * 64 + c;
            if (j < a.N / 2 && m < a.m_valid) {
                const float g = vals[m * SLAB + c], u = vals[m * SLAB + 64 + c];
                const float act = g / (1.0f + expf(-g));
                a.y[(size_t)m * a.ldy + j] = act * u;
            }
        }
    } else if (a.epi == EPI_LOGITS) {
        if (warp < M && warp < a.m_valid) {
            const int m = warp;
            float bv = -INFINITY;
            int bi = -1;
#pragma unroll
            for (int i = 0; i < SLAB / 32; ++i) {
                const int c = lane + i * 32;
                const int n = n0 + c;
                if (n < a.N) {
                    const float v = vals[m * SLAB + c];
                    if (bi < 0 || better(v, n, bv, bi)) { bv = v; bi = n; }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi >= 0 && (bi < 0 || better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
            }
            if (lane == 0) {
                const int nslabs = (a.N + SLAB - 1) / SLAB;
                a.amax_val[m * nslabs + slab] = bv;
                a.amax_idx[m * nslabs + slab] = bi;
            }
        }
        if (a.fin_ticket) {
            // last epilogue of the launch: every slab's partial is in place, reduce them (ties to the higher index)
            const int nslabs = (a.N + SLAB - 1) / SLAB;
            __threadfence();
            __syncthreads();
            if (tid == 0) s_last = atomicAdd(a.fin_ticket, 1u) == (unsigned int)(nslabs - 1);
            __syncthreads();
            if (s_last) {
                __threadfence();
                float* rv = red + M * SLAB;                       // [8 warps] values, reused per row (behind vals, which is stored below)
                int* ri = reinterpret_cast<int*>(rv + 8);         // [8 warps] indices
                for (int m = 0; m < a.m_valid; ++m) {
                    float bv = -INFINITY;
                    int bi = -1;
                    for (int sidx = tid; sidx < nslabs; sidx += GEMV_THREADS) {
                        const float v = ld_cg_f32(a.amax_val + (size_t)m * nslabs + sidx);
                        const int i = __ldcg(a.amax_idx + (size_t)m * nslabs + sidx);
                        if (i >= 0 && (bi < 0 || better(v, i, bv, bi))) { bv = v; bi = i; }
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                        if (oi >= 0 && (bi < 0 || better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
                    }
                    __syncthreads();
                    if (lane == 0) { rv[warp] = bv; ri[warp] = bi; }
                    __syncthreads();
                    if (tid == 0) {
                        for (int w = 0; w < 8; ++w)
                            if (ri[w] >= 0 && (bi < 0 || better(rv[w], ri[w], bv, bi))) { bv = rv[w]; bi = ri[w]; }
                        const uint32_t tok = bi < 0 ? 0u : (uint32_t)bi;
                        a.next_tok[m] = tok;
                        if (a.feed_tok) a.feed_tok[m] = tok;
                        if (a.pos) {
                            const int np = a.pos[m] + 1;
                            a.pos[m] = np;
                            if (a.hist) a.hist[(size_t)m * a.hist_stride + np] = tok;
                        }
                    }
                }
                if (tid == 0) *a.fin_ticket = 0u;  // clean for the next launch
            }
        }
        // the rows themselves go out last: when they go to mapped host memory, the fence in front of the ticket must not wait
        // for them to cross PCIe
        for (int idx = tid; idx < M * SLAB; idx += GEMV_THREADS) {
            const int m = idx / SLAB, n = n0 + (idx % SLAB);
            if (n < a.N && m < a.m_valid) a.y[(size_t)m * a.ldy + n] = vals[idx];
        }
    } else {  // EPI_QKV_ROPE
        const int hd = a.hd, half = hd >> 1, hps = SLAB / hd;
        // head_dim and the page size are powers of two in every supported model: shifts instead of divisions
        // (an integer division is ~20 instructions, and every instruction of this one-shot code is on the chain)
        const bool p2 = (hd & (hd - 1)) == 0 && (a.kv.page_tokens & (a.kv.page_tokens - 1)) == 0;
        const int hs = 31 - __clz(hd);
        // bias: folded into the rotation below unless QK-norm needs the biased values first
        const bool bias_late = a.bias && !a.has_qk_norm;
        if (a.bias && !bias_late) {
            for (int idx = tid; idx < M * SLAB; idx += GEMV_THREADS) vals[idx] += bias_s[idx % SLAB];
            __syncthreads();
        }
        // per-head RMSNorm of Q and K heads (Qwen3), before the rotation
        if (a.has_qk_norm) {
            for (int p = warp; p < M * hps; p += 8) {
                const int m = p / hps, hh = p % hps;
                const int nh = n0 + hh * hd;
                if (nh >= a.q_dim + a.kv_dim || nh >= a.N) continue;  // V heads are not normalised
                float* v = vals + m * SLAB + hh * hd;
                float s = 0.f;
                for (int d = lane; d < hd; d += 32) s = fmaf(v[d], v[d], s);
                s = warp_sum(s);
                const float inv = 1.0f / sqrtf(s / (float)hd + a.eps);
                const float* nw = (nh < a.q_dim) ? a.q_norm_w : a.k_norm_w;
                for (int d = lane; d < hd; d += 32) v[d] = (v[d] * inv) * __ldg(nw + d);
            }
            __syncthreads();
        }
        for (int idx = tid; idx < M * SLAB; idx += GEMV_THREADS) {
            const int m = idx / SLAB, c = idx % SLAB;
            const int n = n0 + c;
            if (n >= a.N || m >= a.m_valid) continue;
            const int hh = p2 ? c >> hs : c / hd, d = p2 ? c & (hd - 1) : c % hd;
            const int nh = n0 + hh * hd;
            const int pos = s_pos[m];
            float v = vals[idx];
            if (bias_late) v += bias_s[c];
            if (nh < a.q_dim + a.kv_dim) {
                const int oc = d < half ? half : -half;
                float o = vals[idx + oc];
                if (bias_late) o += bias_s[c + oc];
                const float other = d < half ? -o : o;
                v = fmaf(other, sn_s[idx], v * cs_s[idx]);
            }
            if (nh < a.q_dim) {
                a.y[(size_t)m * a.ldy + n] = v;
            } else {
                const bool is_k = nh < a.q_dim + a.kv_dim;
                const int rel = nh - a.q_dim - (is_k ? 0 : a.kv_dim);
                const int kvh = p2 ? rel >> hs : rel / hd;
                const int page = s_page[m];
                const int tok = p2 ? pos & (a.kv.page_tokens - 1) : pos % a.kv.page_tokens;
                const size_t off = ((size_t)page * a.kv.kv_heads + kvh) * a.kv.page_tokens * hd + (is_k ? k_tile_off(tok, d) : v_tile_off(tok, d, hd, a.kv.bf16));
                void* pool = is_k ? a.kv.k_pool : a.kv.v_pool;
                if (a.kv.bf16)
                    reinterpret_cast<uint16_t*>(pool)[off] = f32_to_bf16_rne(v);
                else
                    reinterpret_cast<float*>(pool)[off] = v;
            }
        }
    }
    HM_TRACE(if (tr) a.trace[6] = global_timer();)  // epilogue stored
    HM_TRACE(if (a.trace && tid == 0) atomicMax(a.trace + 9, global_timer());)  // the launch's last CTA to finish
}

constexpr size_t GEMV_STAGE_MAX = 80 * 1024;  // largest weight slice staged in shared memory (two CTAs per SM stay resident)

template <int M, bool CL, bool ST>
cudaError_t launch_mcs(const GemvArgs& a, size_t smem, int nslabs, cudaStream_t st, bool pdl) {
    {
        cudaError_t e = ensure_dyn_smem(gemv_bf16_kernel<M, CL, ST>, smem);
        if (e == cudaSuccess && CL && a.cluster > 8) e = ensure_nonportable_clusters(gemv_bf16_kernel<M, CL, ST>);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(nslabs * a.ksplit));
    cfg.blockDim = dim3(GEMV_THREADS);
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
        at[n].val.clusterDim.x = (unsigned)a.cluster;
        at[n].val.clusterDim.y = 1;
        at[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = at;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, gemv_bf16_kernel<M, CL, ST>, a);
}

template <int M, bool CL>
cudaError_t launch_mc(const GemvArgs& a_in, cudaStream_t st, bool pdl) {
    GemvArgs a = a_in;
    const int nslabs = (a.N + SLAB - 1) / SLAB;
    size_t floats = (size_t)M * a.rows_per_split + 8 * (size_t)M * SLAB + (CL ? (size_t)a.ksplit * M * SLAB : 0);
    floats += (size_t)a.rows_per_split;                            // pre-fetched RMSNorm weights
    if (a.epi == EPI_QKV_ROPE) floats += 2 * (size_t)M * SLAB + SLAB;  // pre-fetched RoPE rows and bias
    size_t smem = sizeof(float) * floats;
    // cluster launches over the slab layout whose slice fits: weights staged in shared memory before the dependency wait
    const size_t slice = (size_t)a.rows_per_split * SLAB * 2;
    if (CL && a.row_stride == SLAB * 2 && slice <= GEMV_STAGE_MAX && ((uintptr_t)a.W & 15) == 0) {
        smem += slice;
        return launch_mcs<M, true, true>(a, smem, nslabs, st, pdl);
    }
    return launch_mcs<M, CL, false>(a, smem, nslabs, st, pdl);
}

template <int M>
cudaError_t launch_m(const GemvArgs& a, cudaStream_t st, bool pdl) {
    if (a.cluster > 1) {
        if (a.cluster != a.ksplit || a.cluster > 16) return cudaErrorInvalidValue;
        return launch_mc<M, true>(a, st, pdl);
    }
    return launch_mc<M, false>(a, st, pdl);
}

}  // namespace

size_t gemv_partial_floats(int N, int ksplit, int M) {
    const int nslabs = (N + SLAB - 1) / SLAB;
    return ksplit > 1 ? (size_t)nslabs * ksplit * M * SLAB : 0;
}

// Split K so that roughly two CTAs land on every SM, each streaming at least 32 rows, with
// the activation slice of all M rows fitting 48 KB of shared memory.
void gemv_pick_split(int K, int N, int M, int sm_count, int* ksplit, int* rows_per_split) {
    const int nslabs = (N + SLAB - 1) / SLAB;
    const int target = 2 * sm_count;
    int ks = (target + nslabs - 1) / nslabs;
    const int max_by_rows = K / 32 > 0 ? K / 32 : 1;
    if (ks > max_by_rows) ks = max_by_rows;
    if (ks < 1) ks = 1;
    int rps = ((K + ks - 1) / ks + ROWS_PER_PASS - 1) / ROWS_PER_PASS * ROWS_PER_PASS;
    const int max_rps = (12288 / M) / ROWS_PER_PASS * ROWS_PER_PASS;
    if (rps > max_rps) rps = max_rps;
    ks = (K + rps - 1) / rps;
    *ksplit = ks;
    *rows_per_split = rps;
}

// Cluster split: as many K-splits per slab as keep every CTA resident in one wave, at most
// max_cluster, at least 32 rows each.
void gemv_pick_cluster(int K, int N, int M, int sm_count, int max_cluster, int* cluster, int* rows_per_split) {
    const int nslabs = (N + SLAB - 1) / SLAB;
    int cs = (2 * sm_count) / nslabs;  // two CTAs per SM resident at once (one per SM measured 1.5x slower on the widest projection)
    if (cs > max_cluster) cs = max_cluster;
    if (cs < 1) cs = 1;
    while (cs > 1 && K / cs < 32) --cs;
    int rps = ((K + cs - 1) / cs + ROWS_PER_PASS - 1) / ROWS_PER_PASS * ROWS_PER_PASS;
    const int max_rps = (12288 / M) / ROWS_PER_PASS * ROWS_PER_PASS;
    if (rps > max_rps) {  // activation slice would not fit: fall back to no split-limit via more, smaller clusters is impossible, so cap
        rps = max_rps;
    }
    cs = (K + rps - 1) / rps;
    *cluster = cs;
    *rows_per_split = rps;
}

// Asked of the current device every time (an occupancy query, no launch): engines on different GPUs of one
// process each get their own answer.
int gemv_max_cluster() {
    if (ensure_nonportable_clusters(gemv_bf16_kernel<1, true, false>) != cudaSuccess) {
        cudaGetLastError();
        return 8;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(16);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = 8 * 1024;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 16;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemv_bf16_kernel<1, true, false>, &cfg);
    if (e != cudaSuccess) cudaGetLastError();
    return (e == cudaSuccess && n >= 4) ? 16 : 8;
}

cudaError_t launch_gemv_bf16(const GemvArgs& a, int M, cudaStream_t st, bool pdl) {
    switch (M) {
        case 1: return launch_m<1>(a, st, pdl);
        case 2: return launch_m<2>(a, st, pdl);
        case 4: return launch_m<4>(a, st, pdl);
        case 8: return launch_m<8>(a, st, pdl);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace hm

// ---- projection without any allocation -----------------------------------------------------
//
// hm_gemv_bf16 borrows split-K scratch from a lazily grown cudaMalloc'd buffer.  Some callers
// must never reach an allocator from the token path: a host that drives kernels the way
// Homura's ExecutionPlan does hands each kernel nothing but memory it already owns, and a
// serving loop with a latency budget cannot take the device-wide synchronisation (and the
// unbounded time) that cudaMalloc / cudaFree may cost.  For them the same kernel runs here
// with its partial sums and slab tickets in a fixed array that is part of the library image:
// every GPU that loads the library holds kNoAllocBytes of it until the process exits.
namespace hm {
int set_global_error(int code, const char* msg);  // capi.cu
}

namespace {
constexpr size_t kNoAllocPartialBytes = 4u << 20;  // split-K partial sums
constexpr int kNoAllocMaxSlabs = 4096;             // one ticket per 128-column slab: N <= 524288
constexpr size_t kNoAllocBytes = kNoAllocPartialBytes + kNoAllocMaxSlabs * sizeof(unsigned int);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address; the
// address on each device comes from cudaGetSymbolAddress, asked once per device.
constexpr int kNoAllocMaxDevices = 64;
void* g_noalloc_addr[kNoAllocMaxDevices];
std::atomic<int> g_noalloc_ready[kNoAllocMaxDevices];
std::mutex g_noalloc_mu;

// Device (or managed) memory that the GPU `dev` can dereference: a buffer that lives on another GPU is
// refused, because the kernel would read it without peer access.
bool on_device(const void* p, int dev) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (at.type == cudaMemoryTypeManaged) return true;
    return at.type == cudaMemoryTypeDevice && at.device == dev;
}
}  // namespace

extern "C" HM_API int hm_gemv_bf16_noalloc(const float* x, const void* w_bf16, int layout, int M, int K, int N, float* y, void* stream) {
    using namespace hm;
    if (!x || !w_bf16 || !y || K < 1 || N < 1) return set_global_error(HM_ERR_INVALID, "hm_gemv_bf16_noalloc: null pointer or non-positive size");
    if (M != 1 && M != 2 && M != 4 && M != 8 && M != 16)
        return set_global_error(HM_ERR_UNSUPPORTED, "hm_gemv_bf16_noalloc: M must be 1, 2, 4, 8 or 16 (other row counts need a padded copy of x, which this entry point cannot allocate)");
    if (layout != HM_LAYOUT_KN && layout != HM_LAYOUT_SLAB128) return set_global_error(HM_ERR_INVALID, "hm_gemv_bf16_noalloc: unknown layout");
    if (layout == HM_LAYOUT_KN && N % 8 != 0) return set_global_error(HM_ERR_UNSUPPORTED, "hm_gemv_bf16_noalloc: row-major [K,N] needs N to be a multiple of 8");
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return set_global_error(HM_ERR_CUDA, "hm_gemv_bf16_noalloc: no CUDA device available");
    if (dev < 0 || dev >= kNoAllocMaxDevices) return set_global_error(HM_ERR_UNSUPPORTED, "hm_gemv_bf16_noalloc: device index beyond 63");
    if (!on_device(x, dev) || !on_device(w_bf16, dev) || !on_device(y, dev))
        return set_global_error(HM_ERR_INVALID, "hm_gemv_bf16_noalloc: x, w and y must be device pointers on the current device (staging host buffers would need an allocation)");

    const int nslabs = (N + SLAB - 1) / SLAB;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int mp = M >= MAX_M ? MAX_M : M;
    int ksplit = 1, rps = 0;
    gemv_pick_split(K, N, mp, sms, &ksplit, &rps);
    const size_t need = gemv_partial_floats(N, ksplit, mp) * sizeof(float);
    if (nslabs > kNoAllocMaxSlabs || need > kNoAllocPartialBytes)
        return set_global_error(HM_ERR_UNSUPPORTED,
                                "hm_gemv_bf16_noalloc: this shape needs more split-K scratch than the built-in 4 MiB + 4096 tickets; use hm_gemv_bf16");

    // One-time set-up per device (with that device current): resolve the array's address.
    if (!g_noalloc_ready[dev].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (!g_noalloc_ready[dev].load(std::memory_order_relaxed)) {
            void* p = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) {
                cudaGetLastError();
                return set_global_error(HM_ERR_CUDA, "hm_gemv_bf16_noalloc: cudaGetSymbolAddress failed for the built-in scratch array");
            }
            g_noalloc_addr[dev] = p;
            g_noalloc_ready[dev].store(1, std::memory_order_release);
        }
    }
    unsigned char* base = static_cast<unsigned char*>(g_noalloc_addr[dev]);
    float* partial = reinterpret_cast<float*>(base);
    unsigned int* tickets = reinterpret_cast<unsigned int*>(base + kNoAllocPartialBytes);
    cudaStream_t st = (cudaStream_t)stream;
    // The array keeps whatever the previous call left.  Partials are fully rewritten before they
    // are read; the tickets must start at zero, so they are cleared on the caller's stream.
    cudaError_t ce = ksplit > 1 ? cudaMemsetAsync(tickets, 0, (size_t)nslabs * sizeof(unsigned int), st) : cudaSuccess;
    for (int m0 = 0; m0 < M && ce == cudaSuccess; m0 += MAX_M) {
        GemvArgs a{};
        a.W = static_cast<const uint16_t*>(w_bf16);
        if (layout == HM_LAYOUT_KN) {
            a.slab_stride = SLAB * 2;
            a.row_stride = (long long)N * 2;
        } else {
            a.slab_stride = (long long)K * SLAB * 2;
            a.row_stride = SLAB * 2;
        }
        a.K = K;
        a.N = N;
        a.m_valid = mp;
        a.ksplit = ksplit;
        a.rows_per_split = rps;
        a.x = x + (size_t)m0 * K;
        a.ldx = K;
        a.pro = PRO_PLAIN;
        a.epi = EPI_STORE;
        a.y = y + (size_t)m0 * N;
        a.ldy = N;
        a.partial = partial;
        a.tickets = tickets;
        ce = launch_gemv_bf16(a, mp, st, false);
    }
    if (ce != cudaSuccess) return set_global_error(HM_ERR_CUDA, cudaGetErrorString(ce));
    return HM_OK;
}
