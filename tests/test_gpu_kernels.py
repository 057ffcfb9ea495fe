"""Kernel-level parity on a B200: every CUDA kernel is called through the C ABI and compared
with the CPU oracle on the same seeded inputs.  Integer/byte work is bit-exact; floating point
differs from the oracle only by summation order (and expf/rsqrt last-ulp), tolerances below."""
import numpy as np
import pytest

from homura_b200 import synth

pytestmark = pytest.mark.gpu

# (K, N) of the projection sweep; the vocab-sized shape is cut down for the CPU oracle
SWEEP = [(896, 1152), (896, 9728), (4864, 896), (1536, 17920), (8960, 1536), (1024, 151936 // 16)]


def rel_err(got, want):
    return float(np.abs(got - want).max() / (np.abs(want).max() + 1e-30))


@pytest.mark.parametrize("K,N", SWEEP)
@pytest.mark.parametrize("M", [1, 4, 16])
def test_gemv_bf16_matches_oracle(hm, oracle, K, N, M):
    rng = np.random.default_rng(K * 31 + N + M)
    w = synth.f32_to_bf16_rne(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02))
    x = rng.standard_normal((M, K), dtype=np.float32)
    want = oracle.matmul_bf16(x, w)
    got_kn = hm.gemv_bf16(x, w, hm.LAYOUT_KN)
    slabs = hm.pack_bf16_slabs(w)
    got_slab = hm.gemv_bf16(x, slabs, hm.LAYOUT_SLAB128, K=K, N=N)
    # f32 accumulation in a different order: a few ulp of the sum of |terms|
    assert rel_err(got_kn, want) < 2e-5
    assert rel_err(got_slab, want) < 2e-5
    # both layouts run the same kernel in the same order: identical bits
    np.testing.assert_array_equal(got_kn, got_slab)
    # deterministic across launches (fixed-order split-K reduction)
    np.testing.assert_array_equal(got_kn, hm.gemv_bf16(x, w, hm.LAYOUT_KN))


def test_gemv_bf16_ragged_shapes(hm, oracle):
    # N not a multiple of 128, K not a multiple of 16, odd M
    for (M, K, N) in [(3, 200, 136), (5, 48, 8), (7, 1000, 1000), (1, 16, 128), (12, 96, 264)]:
        rng = np.random.default_rng(M + K + N)
        w = synth.f32_to_bf16_rne(rng.standard_normal((K, N), dtype=np.float32))
        x = rng.standard_normal((M, K), dtype=np.float32)
        assert rel_err(hm.gemv_bf16(x, w, hm.LAYOUT_KN), oracle.matmul_bf16(x, w)) < 2e-5
        slabs = hm.pack_bf16_slabs(w)
        assert rel_err(hm.gemv_bf16(x, slabs, hm.LAYOUT_SLAB128, K=K, N=N), oracle.matmul_bf16(x, w)) < 2e-5
    with pytest.raises(hm.HomuraError):
        hm.gemv_bf16(np.ones((1, 16), np.float32), np.ones((16, 12), np.uint16), hm.LAYOUT_KN)  # N % 8 != 0
    with pytest.raises(hm.HomuraError):
        hm.gemv_bf16(np.ones((17, 16), np.float32), np.ones((16, 16), np.uint16), hm.LAYOUT_KN)  # M > 16


def test_gemv_is_linear(hm):
    # size-independent property at full vocab width: W(a*x + b*y) == a*Wx + b*Wy
    K, N = 1024, 151936
    rng = np.random.default_rng(9)
    w = synth.f32_to_bf16_rne(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02))
    x, y = rng.standard_normal((2, K), dtype=np.float32)
    wx, wy = hm.gemv_bf16(x[None], w), hm.gemv_bf16(y[None], w)
    wz = hm.gemv_bf16((2 * x - 3 * y)[None], w)
    assert rel_err(wz, 2 * wx - 3 * wy) < 1e-5


@pytest.mark.parametrize("kind,dt", [("q8_0", "Q8_0"), ("q4_0", "Q4_0")])
def test_dequant_is_bit_exact(hm, oracle, kind, dt):
    gt = synth.GGML_Q8_0 if kind == "q8_0" else synth.GGML_Q4_0
    blocks = synth.quant_blocks(5, "t", 64, 2048, gt)
    np.testing.assert_array_equal(hm.dequant(blocks, hm.DType[dt]), oracle.dequant(blocks, kind))
    # every code value and a spread of scales, including subnormal / large f16
    bsz = 34 if kind == "q8_0" else 18
    scales = np.array([0x0001, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0x8400, 0xBC00, 0x2E66], np.uint16)
    blk = np.zeros((len(scales) * 8, bsz), np.uint8)
    rng = np.random.default_rng(1)
    blk[:, 2:] = rng.integers(0, 256, size=(blk.shape[0], bsz - 2), dtype=np.uint8)
    blk[:, 0:2] = np.repeat(scales, 8).view(np.uint8).reshape(-1, 2)
    np.testing.assert_array_equal(hm.dequant(blk.ravel(), hm.DType[dt]), oracle.dequant(blk.ravel(), kind))


def test_q8_0_block_dot_528(hm):
    # emit_q8_0_correctness, src/graph_builder/emit_quant.rs:894-958
    K, N = 32, 4
    blk = np.zeros((N, 34), np.uint8)
    blk[:, 1] = 0x3C
    blk[:, 2:] = np.arange(1, 33, dtype=np.uint8)
    y = hm.gemv_quant(np.ones((1, K), np.float32), blk.ravel(), hm.DType.Q8_0, N)
    np.testing.assert_array_equal(y, np.full((1, N), 528.0, np.float32))


@pytest.mark.parametrize("kind,dt", [("q8_0", "Q8_0"), ("q4_0", "Q4_0")])
@pytest.mark.parametrize("M,K,N", [(1, 2048, 2048), (1, 5632, 2048), (4, 2048, 512), (8, 256, 40), (1, 32, 1)])
def test_gemv_quant_matches_oracle(hm, oracle, kind, dt, M, K, N):
    gt = synth.GGML_Q8_0 if kind == "q8_0" else synth.GGML_Q4_0
    blocks = synth.quant_blocks(7, f"w{K}x{N}", N, K, gt)
    x = np.random.default_rng(K + N).standard_normal((M, K), dtype=np.float32)
    want = oracle.matmul_q(x, blocks, N, kind)
    got = hm.gemv_quant(x, blocks, hm.DType[dt], N)
    assert rel_err(got, want) < 2e-5


@pytest.mark.parametrize("kind,dt", [("q8_0", "Q8_0"), ("q4_0", "Q4_0")])
def test_gemv_quant_wide_dynamic_range(hm, oracle, kind, dt):
    # The projection rewrites every 32-element block of a row as one power-of-two scale and 31-bit integers: rows whose
    # blocks differ by many orders of magnitude, all-zero blocks, a lone outlier inside a block and exact powers of two.
    gt = synth.GGML_Q8_0 if kind == "q8_0" else synth.GGML_Q4_0
    M, K, N = 4, 2048, 512
    blocks = synth.quant_blocks(11, f"w{K}x{N}", N, K, gt)
    rng = np.random.default_rng(17)
    x = rng.standard_normal((M, K), dtype=np.float32)
    x[0] *= np.exp(6.0 * rng.standard_normal(K)).astype(np.float32)         # element-wise spread of e^+-18
    x[1].reshape(-1, 32)[::3] = 0.0                                           # zero blocks
    x[1] *= np.repeat(np.exp(10.0 * rng.standard_normal(K // 32)), 32).astype(np.float32)  # block-wise spread
    x[2] *= 1e-3
    x[2, 5::64] = 1e4                                                         # outliers: the rest of their blocks keeps 2^-30 of them
    x[3] = np.ldexp(1.0, rng.integers(-20, 20, K)).astype(np.float32) * rng.choice([-1.0, 1.0], K).astype(np.float32)
    want = oracle.matmul_q(x, blocks, N, kind)
    got = hm.gemv_quant(x, blocks, hm.DType[dt], N)
    for m in range(M):
        assert rel_err(got[m], want[m]) < 2e-5, m


def test_rms_norm_and_rope(hm, oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 896), dtype=np.float32)
    w = (1 + 0.1 * rng.standard_normal(896)).astype(np.float32)
    np.testing.assert_allclose(hm.rms_norm(x, w, 1e-6), oracle.rms_norm(x, w, 1e-6), rtol=2e-6, atol=1e-7)
    # rms_norm_basic, src/graph_builder/mod.rs:3800-3825
    np.testing.assert_allclose(hm.rms_norm(np.array([[1, 2, 3, 4]], np.float32), np.ones(4, np.float32), 1e-6).ravel(), np.array([1, 2, 3, 4]) / np.sqrt(7.5), atol=1e-4)
    for hd in (64, 128):
        cos, sin = oracle.rope_table(hd, 64, 1e6)
        q = rng.standard_normal((3, 4, hd), dtype=np.float32)
        pos = [5, 17, 63]
        want = oracle.rope_half(q, cos[pos], sin[pos])
        np.testing.assert_allclose(hm.qknorm_rope(q, cos[pos], sin[pos]), want, rtol=0, atol=2e-6)
        nw = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
        qn = oracle.rms_norm(q, nw, 1e-6)
        np.testing.assert_allclose(hm.qknorm_rope(q, cos[pos], sin[pos], nw, 1e-6), oracle.rope_half(qn, cos[pos], sin[pos]), rtol=0, atol=4e-6)


def test_argmax_ties_resolve_to_highest_index(hm, oracle):
    rng = np.random.default_rng(4)
    lg = rng.standard_normal((3, 151936), dtype=np.float32)
    lg[0, [7, 90000, 151935]] = 9.0
    lg[1, [0, 5]] = 8.0
    got = hm.argmax(lg)
    assert got.tolist() == [151935, 5, int(np.argmax(lg[2]))]
    for r in range(3):
        assert got[r] == oracle.argmax(lg[r])
    assert hm.argmax(np.array([[0.0, 1.0, 0.5, 0.2]], np.float32))[0] == 1  # src/generate.rs:892-900


def _paged(rng, B, kvh, hd, lens, bf16, hm):
    """Random K/V for each sequence scattered into a shuffled page pool."""
    PT = 16
    max_pages = max((l + PT - 1) // PT for l in lens)
    n_pages = B * max_pages
    perm = rng.permutation(n_pages).astype(np.int32).reshape(B, max_pages)
    esz = 2 if bf16 else 4
    kpool = np.zeros((n_pages, kvh, PT, hd), np.uint16 if bf16 else np.float32)
    vpool = np.zeros_like(kpool)
    ks, vs = [], []
    for b, L in enumerate(lens):
        k = rng.standard_normal((kvh, L, hd), dtype=np.float32)
        v = rng.standard_normal((kvh, L, hd), dtype=np.float32)
        if bf16:
            kb, vb = synth.f32_to_bf16_rne(k), synth.f32_to_bf16_rne(v)
            k, v = synth.bf16_to_f32(kb), synth.bf16_to_f32(vb)
        for t in range(L):
            pg = perm[b, t // PT]
            kpool[pg, :, t % PT] = kb[:, t] if bf16 else k[:, t]
            vpool[pg, :, t % PT] = vb[:, t] if bf16 else v[:, t]
        ks.append(k)
        vs.append(v)
    kd, vd = hm.DeviceBuffer(kpool.nbytes), hm.DeviceBuffer(vpool.nbytes)
    # K tiles are stored chunk-major inside a page, [hd/4][16 tokens][4]; V tiles are rows [16 tokens][hd] on f32 pages
    # and chunk-major [hd/8][16 tokens][8] on bf16 pages
    kd.upload(np.ascontiguousarray(kpool.reshape(n_pages, kvh, PT, hd // 4, 4).transpose(0, 1, 3, 2, 4)))
    vd.upload(np.ascontiguousarray(vpool.reshape(n_pages, kvh, PT, hd // 8, 8).transpose(0, 1, 3, 2, 4)) if bf16 else vpool)
    return kd, vd, perm, max_pages, ks, vs


@pytest.mark.parametrize("heads,kvh,hd", [(16, 8, 128), (14, 2, 64), (32, 4, 64), (12, 2, 128), (4, 4, 64)])
@pytest.mark.parametrize("bf16", [False, True])
def test_attention_matches_oracle(hm, oracle, heads, kvh, hd, bf16):
    rng = np.random.default_rng(heads * 7 + hd + bf16)
    lens = [1, 15, 16, 17, 300, 1024]
    B = len(lens)
    kd, vd, perm, max_pages, ks, vs = _paged(rng, B, kvh, hd, lens, bf16, hm)
    q = rng.standard_normal((B, heads, hd), dtype=np.float32)
    got = hm.attn_decode_paged(q, kd, vd, hm.DType.BF16 if bf16 else hm.DType.F32, perm, lens, heads, kvh, hd, max_pages)
    for b, L in enumerate(lens):
        want = oracle.gqa_attention(q[b : b + 1], ks[b], vs[b], np.zeros((1, L), np.float32), heads, kvh)
        # online softmax vs two-pass softmax: same math, different rounding order
        np.testing.assert_allclose(got[b], want[0], rtol=0, atol=3e-6 * max(1.0, float(np.abs(want).max())))


@pytest.mark.parametrize("heads,kvh,hd", [(14, 2, 64), (12, 2, 128), (16, 8, 128), (4, 4, 64), (32, 4, 64), (8, 1, 64)])
@pytest.mark.parametrize("bf16", [False, True])
def test_attention_streaming_variant_matches_oracle(hm, oracle, heads, kvh, hd, bf16):
    # contexts of thousands of tokens and enough sequences that every CTA owns >= 8 pages: the
    # bulk-copy ring kernel; ragged lengths leave some CTAs with a partial or empty page range
    rng = np.random.default_rng(heads * 5 + hd + 3 * bf16)
    lens = [4096, 2500, 4000, 17, 3333, 4096, 1, 2049]
    B = len(lens)
    kd, vd, perm, max_pages, ks, vs = _paged(rng, B, kvh, hd, lens, bf16, hm)
    q = rng.standard_normal((B, heads, hd), dtype=np.float32)
    got = hm.attn_decode_paged(q, kd, vd, hm.DType.BF16 if bf16 else hm.DType.F32, perm, lens, heads, kvh, hd, max_pages)
    for b, L in enumerate(lens):
        want = oracle.gqa_attention(q[b : b + 1], ks[b], vs[b], np.zeros((1, L), np.float32), heads, kvh)
        np.testing.assert_allclose(got[b], want[0], rtol=0, atol=3e-6 * max(1.0, float(np.abs(want).max())))
    # deterministic: same bits on a second launch
    again = hm.attn_decode_paged(q, kd, vd, hm.DType.BF16 if bf16 else hm.DType.F32, perm, lens, heads, kvh, hd, max_pages)
    np.testing.assert_array_equal(got, again)


def test_attention_long_context_property(hm):
    # KV length 32768: all keys equal => output is the mean of V exactly up to rounding
    heads, kvh, hd, L, PT = 16, 8, 128, 32768, 16
    rng = np.random.default_rng(11)
    pages = L // PT
    perm = rng.permutation(pages).astype(np.int32).reshape(1, pages)
    k = np.ones((pages, kvh, PT, hd), np.float32)
    v = rng.standard_normal((pages, kvh, PT, hd), dtype=np.float32)
    kd, vd = hm.DeviceBuffer(k.nbytes), hm.DeviceBuffer(v.nbytes)
    kd.upload(k)  # all ones: any layout
    vd.upload(v)  # f32 pages: V tiles are rows
    q = rng.standard_normal((1, heads, hd), dtype=np.float32)
    got = hm.attn_decode_paged(q, kd, vd, hm.DType.F32, perm, [L], heads, kvh, hd, pages).reshape(heads, hd)
    mean_v = v.astype(np.float64).mean(axis=(0, 2))  # [kvh, hd]
    for h in range(heads):
        np.testing.assert_allclose(got[h], mean_v[h // 2], atol=2e-5)


def _attention_oracle_rows(oracle, q, k, v, heads, kvh, head_list):
    """oracle.gqa_attention for the KV heads that serve `head_list`, returned as {head: row}."""
    g = heads // kvh
    out = {}
    for kh in sorted({h // g for h in head_list}):
        # a one-KV-head problem with that head's g query heads: same floordiv map, 1/kvh of the work
        want = oracle.gqa_attention(q[None, kh * g : (kh + 1) * g], k[kh : kh + 1], v[kh : kh + 1], np.zeros((1, k.shape[1]), np.float32), g, 1)
        for h in head_list:
            if h // g == kh:
                out[h] = want[0].reshape(g, -1)[h - kh * g]
    return out


@pytest.mark.parametrize("B,L,bf16", [(1, 32768, True), (1, 32768, False), (64, 4096, True)])
def test_attention_full_size_against_oracle(hm, oracle, B, L, bf16):
    # the attention configuration at its real sizes (16/8 heads, head_dim 128, page 16): KV length 32768 for
    # one sequence, and 64 sequences of 4096; compared with the oracle on a sample of (sequence, head)
    heads, kvh, hd, PT = 16, 8, 128, 16
    rng = np.random.default_rng(B * 7 + L + bf16)
    pages = L // PT
    n_pages = B * pages
    perm = rng.permutation(n_pages).astype(np.int32).reshape(B, pages)
    dt = np.uint16 if bf16 else np.float32
    kpool = np.empty((n_pages, kvh, PT, hd), dt)
    vpool = np.empty_like(kpool)
    sample = sorted({0, B - 1, B // 2, B // 3})  # sequences whose K/V are kept for the oracle
    keep = {}
    for b in range(B):
        k = rng.standard_normal((kvh, L, hd), dtype=np.float32)
        v = rng.standard_normal((kvh, L, hd), dtype=np.float32)
        if bf16:
            kb, vb = synth.f32_to_bf16_rne(k), synth.f32_to_bf16_rne(v)
            k, v = synth.bf16_to_f32(kb), synth.bf16_to_f32(vb)
        else:
            kb, vb = k, v
        # logical page p of sequence b lives at physical page perm[b, p]
        kpool[perm[b]] = kb.reshape(kvh, pages, PT, hd).transpose(1, 0, 2, 3)
        vpool[perm[b]] = vb.reshape(kvh, pages, PT, hd).transpose(1, 0, 2, 3)
        if b in sample:
            keep[b] = (k, v)
    kd, vd = hm.DeviceBuffer(kpool.nbytes), hm.DeviceBuffer(vpool.nbytes)
    kd.upload(np.ascontiguousarray(kpool.reshape(n_pages, kvh, PT, hd // 4, 4).transpose(0, 1, 3, 2, 4)))  # K tiles: chunks of 4
    vd.upload(np.ascontiguousarray(vpool.reshape(n_pages, kvh, PT, hd // 8, 8).transpose(0, 1, 3, 2, 4)) if bf16 else vpool)  # V tiles: chunks of 8 on bf16 pages
    del kpool, vpool
    q = rng.standard_normal((B, heads, hd), dtype=np.float32)
    got = hm.attn_decode_paged(q, kd, vd, hm.DType.BF16 if bf16 else hm.DType.F32, perm, [L] * B, heads, kvh, hd, pages).reshape(B, heads, hd)
    for b in sample:
        head_list = [0, 5, 15] if B > 1 else list(range(heads))
        want = _attention_oracle_rows(oracle, q[b], keep[b][0], keep[b][1], heads, kvh, head_list)
        for h, row in want.items():
            np.testing.assert_allclose(got[b, h], row, rtol=0, atol=3e-6 * max(1.0, float(np.abs(row).max())))


def test_attention_rejects_bad_arguments(hm):
    d = hm.DeviceBuffer(16 * 64 * 4 * 2)
    q = np.zeros((1, 2, 64), np.float32)
    with pytest.raises(hm.HomuraError):
        hm.attn_decode_paged(q, d, d, hm.DType.F32, [[0]], [0], 2, 2, 64, 1)  # empty sequence
    with pytest.raises(hm.HomuraError):
        hm.attn_decode_paged(q, d, d, hm.DType.F32, [[0]], [17], 2, 2, 64, 1)  # longer than its pages
    with pytest.raises(hm.HomuraError):
        hm.attn_decode_paged(q, d, d, hm.DType.F32, [[0]], [1], 2, 2, 64, 1, page_tokens=32)


# ---- K-quants (Q4_K / Q6_K): dequantisation bit-exact, Q8_K integer-dot projections ------------


@pytest.mark.parametrize("kind,dt,gt", [("q4_k", "Q4_K", synth.GGML_Q4_K), ("q6_k", "Q6_K", synth.GGML_Q6_K)])
def test_kquant_dequant_is_bit_exact(hm, oracle, kind, dt, gt):
    blocks = synth.quant_blocks(5, "t", 48, 1024, gt)
    np.testing.assert_array_equal(hm.dequant(blocks, hm.DType[dt]), oracle.dequant(blocks, kind))


def test_kquant_known_answers(hm):
    # emit_q4_k_correctness (src/graph_builder/emit_quant.rs:993-1100): d = 1, sc[0..3] = 1, nibbles 1, x = 1 -> 128
    b4 = np.zeros((4, 144), np.uint8)
    b4[:, 1] = 0x3C
    b4[:, 4:8] = 1
    b4[:, 16:] = 0x11
    np.testing.assert_array_equal(hm.gemv_quant(np.ones((1, 256), np.float32), b4.ravel(), hm.DType.Q4_K, 4), np.full((1, 4), 128.0, np.float32))
    # emit_q6_k_correctness (emit_quant.rs:1285-1360): d = 1, sc = 1, low nibbles 1, high bits 0 -> 256 * (1 - 32)
    b6 = np.zeros((4, 210), np.uint8)
    b6[:, 209] = 0x3C
    b6[:, 192:208] = 1
    b6[:, 0:128] = 0x11
    np.testing.assert_array_equal(hm.gemv_quant(np.ones((1, 256), np.float32), b6.ravel(), hm.DType.Q6_K, 4), np.full((1, 4), -7936.0, np.float32))


@pytest.mark.parametrize("kind,dt,gt", [("q4_k", "Q4_K", synth.GGML_Q4_K), ("q6_k", "Q6_K", synth.GGML_Q6_K)])
@pytest.mark.parametrize("M,K,N", [(1, 2048, 2048), (1, 5632, 2048), (4, 2048, 512), (8, 256, 40), (2, 1024, 33), (1, 256, 1)])
def test_kquant_gemv_matches_oracle(hm, oracle, kind, dt, gt, M, K, N):
    blocks = synth.quant_blocks(7, f"w{K}x{N}", N, K, gt)
    x = np.random.default_rng(K + N).standard_normal((M, K), dtype=np.float32)
    want = oracle.matmul_q(x, blocks, N, kind)
    got = hm.gemv_quant(x, blocks, hm.DType[dt], N)
    # integer dot products are exact; only the f32 sum over super-blocks is in a different order
    assert rel_err(got, want) < 1e-5
    if K == 256:  # one super-block per row: no reordering at all
        np.testing.assert_array_equal(got, want)
