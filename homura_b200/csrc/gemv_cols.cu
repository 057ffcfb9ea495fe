// Column-group bf16 GEMV for the layer projections of a decode step (M <= 8 rows of f32 activations):
// every CTA owns whole output columns, so no partial sum ever crosses a CTA.
//
// Same arithmetic as gemv_bf16.cu (Homura's mixed bf16 x f32 -> f32 matmul,
// src/graph_builder/emit_linalg.rs:1928-2008, with the RMSNorm prologue and the bias / RoPE /
// KV-append / residual / SwiGLU epilogues of src/hf/emitter.rs:601-649,787-804), different
// decomposition.  A layer projection of a small model is 1.6 - 17 MB: far too short to be
// bandwidth-bound, so what a launch costs is its chain of dependent latencies.  Splitting K over a
// cluster puts a cluster barrier (about 1 us) on that chain; here the weights are stored at load as
// GROUPS of 8 output columns, group g = [K][8] bf16 = 16*K contiguous bytes, a CTA takes a contiguous
// run of groups (all groups spread evenly over at most one CTA per SM), pulls its whole run into
// shared memory with bulk copies BEFORE the dependency wait, and after the wait only has to fetch
// the activation rows, multiply out of shared memory and reduce inside the CTA.
//
// Which 8 columns make a group depends on the epilogue, so that everything an epilogue needs is in
// the group (cols_group_col below): 8 consecutive outputs for a plain store; 4 gate columns and
// their 4 up columns for SwiGLU; 4 columns d..d+3 of a head and their rotation partners
// d+hd/2..d+hd/2+3 for the Q and K heads of the fused QKV projection (V columns are consecutive).
// QK-norm needs a whole head's sum of squares and stays on the slab kernel.
#include "common.cuh"
#include "mbarrier.cuh"

namespace hm {

namespace {

constexpr int CW = COLS_THREADS / 32;  // warps per CTA

template <int M>
__device__ __forceinline__ void fma_row8(float (&acc)[M][8], const uint4& w, const float* __restrict__ xs, int K, int row) {
    float f[8];
    f[0] = bf16_lo(w.x); f[1] = bf16_hi(w.x);
    f[2] = bf16_lo(w.y); f[3] = bf16_hi(w.y);
    f[4] = bf16_lo(w.z); f[5] = bf16_hi(w.z);
    f[6] = bf16_lo(w.w); f[7] = bf16_hi(w.w);
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float xv = xs[m * K + row];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[m][j] = fmaf(xv, f[j], acc[m][j]);
    }
}

// Sum 8 values over the 32 lanes of a warp with 9 shuffles: three halving exchanges (each lane keeps
// half of what it held and receives the partner's matching half), then two full exchanges.  Returns the
// total of column c = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1), the same on
// the four lanes that share c.
__device__ __forceinline__ float warp_sum8(const float (&v)[8], int lane) {
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
    float h4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float send = b4 ? v[i] : v[i + 4];
        const float keep = b4 ? v[i + 4] : v[i];
        h4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
    float h2[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float send = b3 ? h4[i] : h4[i + 2];
        const float keep = b3 ? h4[i + 2] : h4[i];
        h2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    const float send = b2 ? h2[0] : h2[1];
    const float keep = b2 ? h2[1] : h2[0];
    float r = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    r += __shfl_xor_sync(0xffffffffu, r, 2);
    r += __shfl_xor_sync(0xffffffffu, r, 1);
    return r;
}

template <int M>
__global__ void __launch_bounds__(COLS_THREADS, 1) gemv_cols_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) unsigned char cols_smem[];
    const int K = a.K;
    // group run of this CTA: the groups are spread evenly, the first `extra` CTAs take one more
    const int base = a.n_groups / (int)gridDim.x, extra = a.n_groups % (int)gridDim.x;
    const int bid = blockIdx.x;
    const int G = base + (bid < extra ? 1 : 0);
    const int g0 = bid * base + min(bid, extra);
    const int gmax = base + (extra ? 1 : 0);

    const uint4* wst = reinterpret_cast<const uint4*>(cols_smem);               // [G][K] x 16 B
    float* xs = reinterpret_cast<float*>(cols_smem + (size_t)gmax * K * 16);     // [M][K]
    float* nws = xs + (size_t)M * K;                                             // [K] RMSNorm weights (PRO_RMSNORM)
    float* part = nws + (a.pro == PRO_RMSNORM ? K : 0);                          // [CW][M][8]
    float* vals = part + CW * M * 8;                                             // [gmax][M][8]
    float* cs_s = vals + gmax * M * 8;                                           // [gmax][M][8] RoPE cos / sin (QKV epilogue)
    float* sn_s = cs_s + gmax * M * 8;
    float* b_s = sn_s + gmax * M * 8;                                            // [gmax][8] bias of this CTA's columns
    __shared__ uint64_t s_wbar;
    __shared__ volatile int s_abort;
    __shared__ int s_page[MAX_M], s_pos[MAX_M];
    __shared__ float s_warp[CW][MAX_M];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool tr = a.trace != nullptr && bid == 0 && tid == 0;
    if (tr) a.trace[0] = global_timer();  // CTA resident
    if (a.trace && tid == 0) atomicMax(a.trace + 8, global_timer());  // the launch's last CTA to become resident
    pdl_launch_dependents();
    if (a.pf_bytes && tid < 32) l2_prefetch_slice(a.pf_ptr, a.pf_bytes, bid, gridDim.x, tid);

    // ---- everything that does not depend on the previous kernel ----
    if (tid == 0) {
        mb_init(&s_wbar, 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const uint32_t bytes = (uint32_t)G * (uint32_t)K * 16u;
        if (bytes) {
            mb_expect_tx(&s_wbar, bytes);
            const char* src = (const char*)a.W + (size_t)g0 * K * 16;
            for (uint32_t o = 0; o < bytes; o += 16384u) bulk_copy(cols_smem + o, src + o, min(16384u, bytes - o), &s_wbar);
        }
    }
    if (a.pro == PRO_RMSNORM)
        for (int k = tid; k < K; k += COLS_THREADS) nws[k] = __ldg(a.norm_w + k);
    if (a.bias && a.epi != EPI_SWIGLU) {
        for (int idx = tid; idx < G * 8; idx += COLS_THREADS) {
            const int n = cols_group_col(a.epi, g0 + idx / 8, idx % 8, a.q_dim, a.kv_dim, a.hd, a.N);
            b_s[idx] = n < a.N ? __ldg(a.bias + n) : 0.f;
        }
    }
    if (a.epi == EPI_QKV_ROPE) {
        for (int idx = tid; idx < G * M * 8; idx += COLS_THREADS) {
            const int grp = idx / (M * 8), m = (idx / 8) % M, c = idx % 8;
            const int n = cols_group_col(EPI_QKV_ROPE, g0 + grp, c, a.q_dim, a.kv_dim, a.hd, a.N);
            if (m < a.m_valid && n < a.q_dim + a.kv_dim) {  // V columns are not rotated
                const int pos = a.row_pos[m], d = n % a.hd;
                cs_s[idx] = __ldg(a.rope_cos + (size_t)pos * a.hd + d);
                sn_s[idx] = __ldg(a.rope_sin + (size_t)pos * a.hd + d);
            }
        }
        if (tid < M && tid < a.m_valid) {
            const int pos = a.row_pos[tid], seq = a.row_seq ? a.row_seq[tid] : a.seq_base + tid;
            s_pos[tid] = pos;
            s_page[tid] = a.kv.page_table[(size_t)seq * a.kv.max_pages + pos / a.kv.page_tokens];
        }
    }

    pdl_wait();
    if (tr) a.trace[1] = global_timer();  // predecessor complete

    // the residual element this thread will add in the epilogue: requested now, used after the reduction
    float resid_v = 0.f;
    if (a.epi == EPI_STORE && a.resid && tid < G * M * 8) {
        const int gi = tid / (M * 8), m = (tid / 8) % M, n = (g0 + gi) * 8 + (tid % 8);
        if (m < a.m_valid && n < a.N) resid_v = ld_cg_f32(a.resid + (size_t)m * a.ldy + n);
    }

    // ---- activation rows into shared memory (every CTA needs all K of them) ----
    if (a.pro == PRO_RMSNORM) {
        float ss[M];
#pragma unroll
        for (int m = 0; m < M; ++m) ss[m] = warp_sum(stage_row<COLS_THREADS, true>(a.x + (size_t)m * a.ldx, xs + m * K, K, tid));
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < M; ++m) s_warp[warp][m] = ss[m];
        }
        __syncthreads();  // also publishes the raw rows and the RMSNorm weights
        // every thread sums the warps' shares in the same order (no second barrier for a broadcast)
        float inv[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float s = 0.f;
#pragma unroll
            for (int wv = 0; wv < CW; ++wv) s += s_warp[wv][m];
            inv[m] = 1.0f / sqrtf(s / (float)K + a.eps);
        }
        // scale in place; the thread -> element mapping of this pass is free (everything is published)
#pragma unroll
        for (int m = 0; m < M; ++m)
            for (int k = tid; k < K; k += COLS_THREADS) xs[m * K + k] = (xs[m * K + k] * inv[m]) * nws[k];
    } else {
#pragma unroll
        for (int m = 0; m < M; ++m) stage_row<COLS_THREADS, false>(a.x + (size_t)m * a.ldx, xs + m * K, K, tid);
    }
    __syncthreads();
    if (tr) a.trace[2] = global_timer();  // activations in shared memory

    // ---- multiply: wpg warps per group, lane rl of a group's warps takes rows rl, rl + RL, ... ----
    const int wpg = G > 0 ? max(1, CW / G) : 1;
    const int grp = warp / wpg, sub = warp - grp * wpg;
    const bool busy = grp < G;
    float acc[M][8];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[m][j] = 0.f;
    const bool ok = G == 0 || mb_wait(&s_wbar, 0, a.err_flag, &s_abort);  // bounded; every thread waits
    if (ok && busy) {
        const uint4* wg = wst + (size_t)grp * K;
        const int RL = wpg * 32;
#pragma unroll 4
        for (int row = sub * 32 + lane; row < K; row += RL) fma_row8<M>(acc, wg[row], xs, K, row);
    }
    if (tr) a.trace[3] = global_timer();  // weights multiplied

    // ---- reduce inside the CTA: lanes by shuffles, the warps of a group through shared memory ----
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float r = warp_sum8(acc[m], lane);
        if ((lane & 3) == 0) part[(warp * M + m) * 8 + (lane >> 2)] = r;
    }
    __syncthreads();
    for (int idx = tid; idx < G * M * 8; idx += COLS_THREADS) {
        const int gi = idx / (M * 8), rem = idx - gi * (M * 8);
        float v = 0.f;
        for (int s = 0; s < wpg; ++s) v += part[(gi * wpg + s) * M * 8 + rem];
        vals[idx] = v;
    }
    __syncthreads();
    if (tr) {
        a.trace[4] = a.trace[3];  // no barrier between CTAs
        a.trace[5] = global_timer();  // reduced
    }

    // ---- epilogues on vals[G][M][8] ----
    for (int idx = tid; idx < G * M * 8; idx += COLS_THREADS) {
        const int gi = idx / (M * 8), m = (idx / 8) % M, c = idx % 8;
        if (m >= a.m_valid) continue;
        const int gidx = g0 + gi;
        if (a.epi == EPI_STORE) {
            const int n = gidx * 8 + c;
            if (n < a.N) {
                float v = vals[idx];
                if (a.bias) v += b_s[gi * 8 + c];
                if (a.resid) v = (idx == tid ? resid_v : ld_cg_f32(a.resid + (size_t)m * a.ldy + n)) + v;
                a.y[(size_t)m * a.ldy + n] = v;
            }
        } else if (a.epi == EPI_SWIGLU) {
            const int j = gidx * 4 + c;  // gate column j, its up column 4 slots further in the group
            if (c < 4 && j < a.N / 2) {
                const float g = vals[idx], u = vals[idx + 4];
                const float act = g / (1.0f + expf(-g));
                a.y[(size_t)m * a.ldy + j] = act * u;
            }
        } else {  // EPI_QKV_ROPE (no QK-norm)
            const int hd = a.hd;
            const int n = cols_group_col(EPI_QKV_ROPE, gidx, c, a.q_dim, a.kv_dim, hd, a.N);
            if (n >= a.N) continue;
            float v = vals[idx];
            if (a.bias) v += b_s[gi * 8 + c];
            const int nh = n - n % hd, d = n % hd;
            if (nh < a.q_dim + a.kv_dim) {
                const int pidx = c < 4 ? idx + 4 : idx - 4;  // rotation partner: column d +- hd/2 of the same head, 4 positions away in the group
                float o = vals[pidx];
                if (a.bias) o += b_s[gi * 8 + (c ^ 4)];
                const float other = c < 4 ? -o : o;
                v = fmaf(other, sn_s[idx], v * cs_s[idx]);
            }
            if (nh < a.q_dim) {
                a.y[(size_t)m * a.ldy + n] = v;
            } else {
                const bool is_k = nh < a.q_dim + a.kv_dim;
                const int kvh = (nh - a.q_dim - (is_k ? 0 : a.kv_dim)) / hd;
                const int tok = s_pos[m] % a.kv.page_tokens;
                const size_t off = ((size_t)s_page[m] * a.kv.kv_heads + kvh) * a.kv.page_tokens * hd + (is_k ? k_tile_off(tok, d) : v_tile_off(tok, d, hd));
                void* pool = is_k ? a.kv.k_pool : a.kv.v_pool;
                if (a.kv.bf16)
                    reinterpret_cast<uint16_t*>(pool)[off] = f32_to_bf16_rne(v);
                else
                    reinterpret_cast<float*>(pool)[off] = v;
            }
        }
    }
    if (tr) a.trace[6] = global_timer();  // epilogue stored
    if (a.trace && tid == 0) atomicMax(a.trace + 9, global_timer());  // the launch's last CTA to finish
}

// Re-layout at load: slab layout (element (k, n) of slab n / 128 at [slab][k][n % 128]) -> column groups.
__global__ void pack_cols_kernel(const uint16_t* __restrict__ slabs, int K, int N, int epi, int q_dim, int kv_dim, int hd, int n_groups, uint16_t* __restrict__ dst) {
    const size_t total = (size_t)n_groups * K;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int g = (int)(i / K), k = (int)(i % K);
        uint16_t v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            // position of the column in the slab layout (gate/up slabs hold 64 gate + 64 up columns)
            int n;
            if (epi == EPI_SWIGLU) {
                const int j = g * 4 + (c & 3);
                n = j < N / 2 ? (j / 64) * SLAB + (c >> 2) * 64 + (j % 64) : N;
            } else {
                n = cols_group_col(epi, g, c, q_dim, kv_dim, hd, N);
            }
            v[c] = n < N ? slabs[((size_t)(n / SLAB) * K + k) * SLAB + (n % SLAB)] : (uint16_t)0;
        }
        uint4 o;
        o.x = v[0] | ((uint32_t)v[1] << 16);
        o.y = v[2] | ((uint32_t)v[3] << 16);
        o.z = v[4] | ((uint32_t)v[5] << 16);
        o.w = v[6] | ((uint32_t)v[7] << 16);
        reinterpret_cast<uint4*>(dst)[i] = o;
    }
}

template <int M>
cudaError_t launch_cols_m(const GemvArgs& a, int grid, size_t smem, cudaStream_t st, bool pdl) {
    static size_t opted = 40 * 1024;  // only ever raised: launches captured in a graph stay valid
    if (smem > opted) {
        cudaError_t e = cudaFuncSetAttribute(gemv_cols_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        opted = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(COLS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    int n = 0;
    if (pdl) {
        at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = at;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, gemv_cols_kernel<M>, a);
}

}  // namespace

int cols_groups(int epi, int N) { return epi == EPI_SWIGLU ? (N / 2 + 3) / 4 : (N + 7) / 8; }

// CTAs and shared memory of a launch; false when the shape does not fit one CTA per SM.
bool gemv_cols_plan(int epi, int pro, int K, int N, int M, int sm_count, int* grid, size_t* smem) {
    if (epi != EPI_STORE && epi != EPI_SWIGLU && epi != EPI_QKV_ROPE) return false;
    if (epi == EPI_SWIGLU && (N % 8) != 0) return false;
    const int ng = cols_groups(epi, N);
    const int g = ng < sm_count ? ng : sm_count;
    const int gmax = (ng + g - 1) / g;
    const size_t bytes = (size_t)gmax * K * 16 + sizeof(float) * ((size_t)M * K + (pro == PRO_RMSNORM ? K : 0) + (size_t)CW * M * 8 + 3 * (size_t)gmax * M * 8 + (size_t)gmax * 8) + 128;
    if (gmax > CW || bytes > COLS_SMEM_MAX) return false;
    *grid = g;
    *smem = bytes;
    return true;
}

cudaError_t launch_pack_cols(const uint16_t* slabs, int K, int N, int epi, int q_dim, int kv_dim, int hd, uint16_t* dst, cudaStream_t st) {
    const int ng = cols_groups(epi, N);
    const size_t total = (size_t)ng * K;
    const unsigned grid = (unsigned)std::min<size_t>((total + 255) / 256, 65535);
    pack_cols_kernel<<<grid, 256, 0, st>>>(slabs, K, N, epi, q_dim, kv_dim, hd, ng, dst);
    return cudaGetLastError();
}

cudaError_t launch_gemv_cols(const GemvArgs& a_in, int M, int sm_count, cudaStream_t st, bool pdl) {
    GemvArgs a = a_in;
    int grid = 0;
    size_t smem = 0;
    if (a.has_qk_norm && a.epi == EPI_QKV_ROPE) return cudaErrorInvalidValue;
    if (!gemv_cols_plan(a.epi, a.pro, a.K, a.N, M, sm_count, &grid, &smem)) return cudaErrorInvalidValue;
    a.n_groups = cols_groups(a.epi, a.N);
    switch (M) {
        case 1: return launch_cols_m<1>(a, grid, smem, st, pdl);
        case 2: return launch_cols_m<2>(a, grid, smem, st, pdl);
        case 4: return launch_cols_m<4>(a, grid, smem, st, pdl);
        case 8: return launch_cols_m<8>(a, grid, smem, st, pdl);
    }
    return cudaErrorInvalidValue;
}

}  // namespace hm
