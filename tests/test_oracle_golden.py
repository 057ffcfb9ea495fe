"""Pins the CPU oracle to the known-answer vectors held by Homura's own unit tests.

Each test names the reference test (file:line in the Homura repository) whose inputs and
expected values it restates.  These run without a GPU.
"""
import math

import numpy as np
import pytest


# ---- KV cache: src/runtime.rs:2228-2366 -------------------------------------------------


def test_kv_cache_append_and_view(oracle):
    # src/runtime.rs:2228-2280 (kv_cache_append_and_view): 1 layer, 2 heads, max 4, hd 3
    c = oracle.KvCache(1, 2, 4, 3)
    assert c.current_len() == 0
    k0 = np.array([1, 2, 3, 4, 5, 6], np.float32).reshape(1, 2, 1, 3)
    v0 = np.array([10, 20, 30, 40, 50, 60], np.float32).reshape(1, 2, 1, 3)
    c.append_key(0, k0)
    c.append_value(0, v0)
    c.advance_by(1)
    assert c.current_len() == 1
    kv, vv = c.view(0)
    assert kv.shape == (1, 2, 1, 3)
    assert kv.ravel().tolist() == [1, 2, 3, 4, 5, 6]
    assert vv.ravel().tolist() == [10, 20, 30, 40, 50, 60]
    k1 = np.array([7, 8, 9, 0.1, 0.2, 0.3], np.float32).reshape(1, 2, 1, 3)
    v1 = np.array([70, 80, 90, 0.4, 0.5, 0.6], np.float32).reshape(1, 2, 1, 3)
    c.append_key(0, k1)
    c.append_value(0, v1)
    c.advance_by(1)
    assert c.current_len() == 2
    kv, vv = c.view(0)
    assert kv.shape == (1, 2, 2, 3)
    np.testing.assert_array_equal(kv.ravel(), np.array([1, 2, 3, 7, 8, 9, 4, 5, 6, 0.1, 0.2, 0.3], np.float32))
    np.testing.assert_array_equal(vv.ravel(), np.array([10, 20, 30, 70, 80, 90, 40, 50, 60, 0.4, 0.5, 0.6], np.float32))


def test_kv_cache_multi_token_append(oracle):
    # src/runtime.rs:2282-2351 (kv_cache_multi_token_append)
    c = oracle.KvCache(1, 2, 8, 3)
    k = np.arange(1, 19, dtype=np.float32).reshape(1, 2, 3, 3)
    v = np.array([91, 92, 93, 94, 95, 96, 97, 98, 99, 81, 82, 83, 84, 85, 86, 87, 88, 89], np.float32).reshape(1, 2, 3, 3)
    c.append_key(0, k)
    c.append_value(0, v)
    c.advance_by(3)
    assert c.current_len() == 3
    kv, vv = c.view(0)
    assert kv.shape == (1, 2, 3, 3) and vv.shape == (1, 2, 3, 3)
    np.testing.assert_array_equal(kv.ravel(), np.arange(1, 19, dtype=np.float32))
    k1 = np.array([20, 21, 22, 30, 31, 32], np.float32).reshape(1, 2, 1, 3)
    v1 = np.array([40, 41, 42, 50, 51, 52], np.float32).reshape(1, 2, 1, 3)
    c.append_key(0, k1)
    c.append_value(0, v1)
    c.advance_by(1)
    assert c.current_len() == 4
    kv, _ = c.view(0)
    assert kv.shape == (1, 2, 4, 3)
    exp = [1, 2, 3, 4, 5, 6, 7, 8, 9, 20, 21, 22, 10, 11, 12, 13, 14, 15, 16, 17, 18, 30, 31, 32]
    np.testing.assert_array_equal(kv.ravel(), np.array(exp, np.float32))


def test_kv_cache_reset_and_full(oracle):
    # src/runtime.rs:2353-2366 (kv_cache_reset); overflow is a panic at src/runtime.rs:523-529
    c = oracle.KvCache(2, 1, 2, 4)
    k = np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 1, 4)
    assert c.append_key(0, k) == 0
    c.append_value(0, k)
    c.advance_by(1)
    assert c.current_len() == 1
    c.reset(0)
    assert c.current_len() == 0
    c.advance_by(2)
    assert c.append_key(0, k) == 1  # full


# ---- RoPE table / mask: src/hf/precompute.rs:108-179 ------------------------------------


def test_rope_basic_values(oracle):
    # src/hf/precompute.rs:108-131 (rope_basic_values): theta=1e4, hd=4, 3 positions
    cos, sin = oracle.rope_table(4, 3, 10000.0)
    assert cos.shape == (3, 4)
    c, s = cos.ravel(), sin.ravel()
    assert abs(c[0] - 1.0) < 1e-5 and abs(c[1] - 1.0) < 1e-5
    assert c[0] == c[2] and c[1] == c[3]
    assert abs(c[4] - 0.5403023) < 1e-4 and abs(c[5] - 0.99995) < 1e-4
    assert c[4] == c[6] and c[5] == c[7]
    assert abs(s[0]) < 1e-5 and abs(s[4] - 0.8414709) < 1e-4


def test_rope_table_matches_f64_formula(oracle):
    # definition at src/hf/precompute.rs:10-40, evaluated independently in numpy float64
    for hd, theta in ((64, 1e6), (128, 1e6), (64, 1e4)):
        cos, sin = oracle.rope_table(hd, 300, theta)
        i = np.arange(hd // 2, dtype=np.float64)
        freq = 1.0 / np.power(theta, 2.0 * i / hd)
        ang = np.arange(300, dtype=np.float64)[:, None] * freq[None, :]
        ec = np.cos(ang).astype(np.float32)
        es = np.sin(ang).astype(np.float32)
        # libm vs numpy may differ by one f32 ulp after the cast
        np.testing.assert_allclose(cos[:, : hd // 2], ec, rtol=0, atol=1.2e-7)
        np.testing.assert_allclose(sin[:, : hd // 2], es, rtol=0, atol=1.2e-7)
        np.testing.assert_array_equal(cos[:, : hd // 2], cos[:, hd // 2 :])
        np.testing.assert_array_equal(sin[:, : hd // 2], sin[:, hd // 2 :])


def test_causal_mask(oracle):
    # src/hf/precompute.rs:133-161 (causal_mask_prefill, causal_mask_decode)
    m = oracle.causal_mask(3, 0)
    assert m.shape == (3, 3)
    d = m.ravel()
    assert d[0] == 0 and np.isneginf(d[1]) and np.isneginf(d[2])
    assert d[3] == 0 and d[4] == 0 and np.isneginf(d[5])
    assert d[6] == 0 and d[7] == 0 and d[8] == 0
    m = oracle.causal_mask(1, 5)
    assert m.shape == (1, 6) and np.all(m == 0)


# ---- op known values: src/graph_builder/mod.rs -------------------------------------------


def test_rms_norm_basic(oracle):
    # src/graph_builder/mod.rs:3800-3825 (rms_norm_basic): [1,2,3,4] with unit weight -> x/sqrt(7.5)
    x = np.array([[1, 2, 3, 4]], np.float32)
    w = np.ones(4, np.float32)
    for variant in ("f32", "f64_accum", "quant_kernel"):
        y = oracle.rms_norm(x, w, 1e-6, variant)
        np.testing.assert_allclose(y.ravel(), x.ravel() / math.sqrt(7.5), atol=1e-4)


def test_silu_values(oracle):
    # src/graph_builder/mod.rs:3773-3797 (silu_basic), tolerance 1e-5
    x = np.array([0.0, 1.0, -1.0, 2.0], np.float32)
    y = oracle.silu(x)
    exp = x.astype(np.float64) / (1.0 + np.exp(-x.astype(np.float64)))
    np.testing.assert_allclose(y, exp, atol=1e-5)
    assert abs(y[1] - 0.7310586) < 1e-5 and y[0] == 0.0


def test_softmax_static(oracle):
    # src/graph_builder/mod.rs:2942-2961 (softmax_static): [1,2,3], tol 1e-3, sum 1e-5
    for f64 in (False, True):
        y = oracle.softmax(np.array([[1.0, 2.0, 3.0]], np.float32), f64).ravel()
        np.testing.assert_allclose(y, [0.09003057, 0.24472848, 0.66524094], atol=1e-3)
        assert abs(y.sum() - 1.0) < 1e-5


def test_matmul_known_values(oracle):
    # src/graph_builder/mod.rs:2562 (matmul_2d_known_values): [[1,2],[3,4]] @ [[5,6],[7,8]]
    y = oracle.matmul_f32(np.array([[1, 2], [3, 4]], np.float32), np.array([[5, 6], [7, 8]], np.float32))
    np.testing.assert_array_equal(y, np.array([[19, 22], [43, 50]], np.float32))


# ---- Q8_0: src/graph_builder/emit_quant.rs:894-958 ---------------------------------------


def test_q8_0_block_dot_528(oracle):
    # emit_q8_0_correctness: scale 1.0 (f16 0x3C00), q = 1..32, activations 1 -> 528 per row
    K, N = 32, 4
    blk = np.zeros((N, 34), np.uint8)
    blk[:, 0], blk[:, 1] = 0x00, 0x3C
    blk[:, 2:] = np.arange(1, 33, dtype=np.uint8)
    y = oracle.matmul_q(np.ones((1, K), np.float32), blk.ravel(), N, "q8_0")
    np.testing.assert_array_equal(y, np.full((1, N), 528.0, np.float32))
    # and the CPU dequant of src/gguf.rs:817-831
    np.testing.assert_array_equal(oracle.dequant(blk[0], "q8_0"), np.arange(1, 33, dtype=np.float32))


def test_q8_0_negative_codes_and_scale(oracle):
    blk = np.zeros(34, np.uint8)
    blk[0:2] = np.array([0.5], np.float16).view(np.uint8)
    blk[2:] = np.arange(-16, 16, dtype=np.int8).view(np.uint8)
    np.testing.assert_array_equal(oracle.dequant(blk, "q8_0"), np.arange(-16, 16, dtype=np.float32) * 0.5)


def test_q4_0_public_block_format(oracle):
    # Not in the reference (src/gguf.rs:94-109,141 give geometry only): public ggml layout --
    # byte i = element i (low nibble) | element i+16 (high nibble), value = (nibble-8)*d.
    blk = np.zeros(18, np.uint8)
    blk[0:2] = np.array([2.0], np.float16).view(np.uint8)
    lo = np.arange(16, dtype=np.uint8)
    hi = (15 - np.arange(16)).astype(np.uint8)
    blk[2:] = lo | (hi << 4)
    got = oracle.dequant(blk, "q4_0")
    exp = np.concatenate([(lo.astype(np.float32) - 8) * 2, (hi.astype(np.float32) - 8) * 2])
    np.testing.assert_array_equal(got, exp)
    y = oracle.matmul_q(np.ones((1, 32), np.float32), blk, 1, "q4_0")
    assert y[0, 0] == exp.sum()


def test_block_byte_sizes():
    # src/gguf.rs:1175-1182 (ggml_type_byte_sizes), src/dtype.rs:128-155
    from homura_b200 import synth

    assert synth.quant_blocks(1, "t", 2, 64, synth.GGML_Q8_0).size == 2 * 2 * 34
    assert synth.quant_blocks(1, "t", 2, 64, synth.GGML_Q4_0).size == 2 * 2 * 18


# ---- scalar conversions: src/hf/safetensors.rs:195-237 ------------------------------------


def test_f16_bf16_conversions(oracle):
    L = oracle.lib()
    assert L.orc_bf16_to_f32(0x3F80) == 1.0 and L.orc_bf16_to_f32(0xC000) == -2.0
    assert L.orc_f16_to_f32(0x3C00) == 1.0 and L.orc_f16_to_f32(0xBC00) == -1.0
    assert L.orc_f16_to_f32(0x0000) == 0.0
    assert math.isinf(L.orc_f16_to_f32(0x7C00)) and math.isnan(L.orc_f16_to_f32(0x7E00))
    for v in (1.0, -0.5, 0.0, 2.0):
        assert L.orc_bf16_to_f32(L.orc_f32_to_bf16_trunc(v)) == v
    # every f16 bit pattern against numpy's converter (subnormals included)
    bits = np.arange(65536, dtype=np.uint16)
    exp = bits.view(np.float16).astype(np.float32)
    got = np.array([L.orc_f16_to_f32(int(b)) for b in bits[::7]], np.float32)
    e = exp[::7]
    ok = (got == e) | (np.isnan(got) & np.isnan(e))
    assert ok.all()


# ---- sampler: src/generate.rs:883-969 ------------------------------------------------------


def test_rng_is_deterministic(oracle):
    a, b = oracle.Rng(42), oracle.Rng(42)
    va = [a.next_f32() for _ in range(10)]
    assert va == [b.next_f32() for _ in range(10)]
    assert all(0.0 <= v < 1.0 for v in va)
    # xorshift64 (13,7,17) restated in python ints (src/generate.rs:634-641)
    s = 42 | 1
    mask = (1 << 64) - 1
    exp = []
    for _ in range(10):
        s ^= (s << 13) & mask
        s ^= s >> 7
        s ^= (s << 17) & mask
        exp.append(np.float32(s >> 40) / np.float32(1 << 24))
    assert va == [float(e) for e in exp]


def test_sample_token_greedy(oracle):
    # src/generate.rs:892-900
    r = oracle.Rng(1)
    assert oracle.sample_token([0.0, 1.0, 0.5, 0.2], r, temperature=0.0) == 1


def test_greedy_ties_resolve_to_last_index(oracle):
    # Iterator::max_by returns the last maximum (src/generate.rs:457-468, 734-742)
    assert oracle.argmax([1.0, 3.0, 3.0, 2.0]) == 2
    assert oracle.argmax([5.0, 5.0, 5.0]) == 2
    assert oracle.argmax([-1.0]) == 0


def test_min_p_filters_low_prob(oracle):
    # src/generate.rs:953-969
    r = oracle.Rng(42)
    for _ in range(10):
        assert oracle.sample_token([10.0, 0, 0, 0], r, temperature=1.0, min_p=0.5, top_k=0, top_p=1.0, repetition_penalty=1.0) == 0


def test_repetition_penalty_applied_before_greedy(oracle):
    # src/generate.rs:707-718: positive logits divided, negative multiplied
    r = oracle.Rng(1)
    assert oracle.sample_token([1.0, 0.95], r, generated=[0], temperature=0.0, repetition_penalty=1.1) == 1
    assert oracle.sample_token([-1.0, -1.05], r, generated=[0], temperature=0.0, repetition_penalty=1.1) == 1


# ---- unpinned pieces: checked against an independent float64 evaluation --------------------


def test_rope_half_against_numpy(oracle):
    rng = np.random.default_rng(0)
    S, Hh, hd = 3, 2, 8
    x = rng.standard_normal((S, Hh, hd)).astype(np.float32)
    cos, sin = oracle.rope_table(hd, 16, 1e4)
    y = oracle.rope_half(x, cos[5:8], sin[5:8])
    rot = np.concatenate([-x[..., hd // 2 :], x[..., : hd // 2]], -1).astype(np.float64)
    exp = x.astype(np.float64) * cos[5:8, None, :] + rot * sin[5:8, None, :]
    np.testing.assert_allclose(y, exp, atol=1e-6)


def test_gqa_attention_against_numpy(oracle):
    rng = np.random.default_rng(1)
    S, T, heads, kvh, hd = 2, 7, 6, 2, 16
    q = rng.standard_normal((S, heads, hd)).astype(np.float32)
    k = rng.standard_normal((kvh, T, hd)).astype(np.float32)
    v = rng.standard_normal((kvh, T, hd)).astype(np.float32)
    mask = oracle.causal_mask(S, T - S)
    out = oracle.gqa_attention(q, k, v, mask, heads, kvh).reshape(S, heads, hd)
    g = heads // kvh
    for h in range(heads):
        sc = q[:, h].astype(np.float64) @ k[h // g].astype(np.float64).T / math.sqrt(hd) + mask
        p = np.exp(sc - sc.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        np.testing.assert_allclose(out[:, h], p @ v[h // g].astype(np.float64), atol=2e-6)


def test_matmul_bf16_against_numpy(oracle):
    from homura_b200 import synth

    rng = np.random.default_rng(2)
    x = rng.standard_normal((3, 96)).astype(np.float32)
    wb = synth.f32_to_bf16_rne(rng.standard_normal((96, 200)).astype(np.float32) * 0.02)
    y = oracle.matmul_bf16(x, wb)
    exp = x.astype(np.float64) @ synth.bf16_to_f32(wb).astype(np.float64)
    np.testing.assert_allclose(y, exp, atol=1e-5)


def test_bf16_rne():
    from homura_b200 import synth

    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 0.0], np.float32)  # 1+2^-8 ties to even
    b = synth.f32_to_bf16_rne(x)
    assert b[0] == 0x3F80 and b[1] == 0x3F80 and b[2] == 0x3F82 and b[4] == 0
    import torch

    t = torch.randn(4096, dtype=torch.float32)
    exp = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    np.testing.assert_array_equal(synth.f32_to_bf16_rne(t.numpy()), exp)


# ---- K-quants: the reference's own known-answer tests -------------------------------------------


def test_q4_k_matmul_known_answer(oracle):
    # emit_q4_k_correctness, src/graph_builder/emit_quant.rs:993-1100: d = 1.0, dmin = 0, sc[0..3] = 1,
    # sc[4..7] = 0, every nibble 1, activation 1.0 -> 4 sub-blocks x 32 = 128 per output
    blk = np.zeros((4, 144), np.uint8)
    blk[:, 1] = 0x3C
    blk[:, 4:8] = 1
    blk[:, 16:] = 0x11
    np.testing.assert_array_equal(oracle.matmul_q(np.ones((1, 256), np.float32), blk.ravel(), 4, "q4_k"), np.full((1, 4), 128.0, np.float32))


def test_q6_k_matmul_known_answer(oracle):
    # emit_q6_k_correctness, emit_quant.rs:1285-1360: d = 1.0, every sub-block scale 1, low nibbles 1,
    # high bits 0 -> code 1 - 32 = -31, 256 of them
    blk = np.zeros((4, 210), np.uint8)
    blk[:, 209] = 0x3C
    blk[:, 192:208] = 1
    blk[:, 0:128] = 0x11
    np.testing.assert_array_equal(oracle.matmul_q(np.ones((1, 256), np.float32), blk.ravel(), 4, "q6_k"), np.full((1, 4), -7936.0, np.float32))


def test_k_quant_geometry_and_dequant_layout(oracle):
    # type sizes pinned by src/gguf.rs:1175-1182
    assert oracle.QUANT_BLOCK["q4_k"] == (144, 256) and oracle.QUANT_BLOCK["q6_k"] == (210, 256)
    # Q4_K: sub-block sb uses the low (even sb) or high (odd sb) nibbles of bytes [16 + (sb/2)*32, +32)
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(2.0).tobytes(), np.uint8)   # d
    blk[2:4] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)   # dmin
    blk[4] = 3       # sc[0] = 3
    blk[8] = 2       # mn[0] = 2
    blk[16] = 0x0A   # element 0 = low nibble 10, element 32 = high nibble 0
    out = oracle.dequant(blk, "q4_k")
    assert out[0] == 10 * (2.0 * 3) - 0.5 * 2 and out[1] == -1.0 and out[32] == 0.0
    # Q6_K: element l of group 0 takes ql[l] low nibble and qh[l] bits 0-1; scale index e / 16
    b6 = np.zeros(210, np.uint8)
    b6[208:210] = np.frombuffer(np.float16(0.25).tobytes(), np.uint8)
    b6[192] = np.uint8(np.int8(-3).view(np.uint8))
    b6[0] = 0x05
    b6[128] = 0x02
    o6 = oracle.dequant(b6, "q6_k")
    assert o6[0] == 0.25 * -3 * ((5 | (2 << 4)) - 32) and o6[1] == 0.25 * -3 * (0 - 32) and o6[16] == 0.0


def test_q8_k_activation_quantisation(oracle):
    # emit_quant.rs:409-460: act_d = amax / 127, codes roundeven(x * 127 / amax), sums of 16
    x = np.zeros(256, np.float32)
    x[0], x[1], x[2], x[17] = 127.0, 0.5, 1.5, -2.5   # halves round to even: 0, 2, -2
    q8, d, bs = oracle.quantize_q8_k(x)
    assert d[0] == 1.0 and list(q8[:3]) == [127, 0, 2] and q8[17] == -2
    assert bs[0] == 129 and bs[1] == -2 and int(bs.sum()) == 127
    q8z, dz, _ = oracle.quantize_q8_k(np.zeros(256, np.float32))
    assert dz[0] == 0.0 and not q8z.any()
