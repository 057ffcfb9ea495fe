"""Whole-model checks of the CPU oracle (no GPU).

* against float32 logits of the `transformers` Qwen2 / Llama / Qwen3 implementations on the
  same seeded tiny weights (tests/golden/hf_xcheck.npz, made by tests/golden/make_hf_xcheck.py);
* incremental decode through the persistent cache equals one full pass;
* the GGUF (block-quantised) plan against a float64 numpy evaluation of dequantised weights.
"""
import os
import tempfile

import numpy as np
import pytest

from homura_b200 import synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hf_xcheck.npz")
CASES = {
    "qwen2": dict(),
    "llama": dict(qkv_bias=False, tie_word_embeddings=False, rope_theta=1e4, num_attention_heads=8, num_key_value_heads=2, rms_norm_eps=1e-5),
    "qwen3": dict(qkv_bias=False, qk_norm=True, head_dim=128, num_attention_heads=4, num_key_value_heads=2),
}


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_transformers_fp32(oracle, name):
    gold = np.load(GOLD)
    cfg = synth.tiny_config(**CASES[name])
    d = tempfile.mkdtemp()
    synth.write_hf_model(d, cfg, seed=7, norm_jitter=0.1)
    ids = gold[name + "_ids"]
    np.testing.assert_array_equal(ids, synth.prompt_ids(3, 12, cfg.vocab_size))
    om = oracle.OracleModel.from_hf_dir(d)
    lo = om.forward_all(ids)
    # f32 evaluation orders differ between the two implementations: 1e-5 on logits of order 1
    np.testing.assert_allclose(lo[[3, 11]], gold[name + "_logits"], atol=1e-5, rtol=0)


def test_incremental_decode_equals_full_pass(oracle):
    cfg = synth.tiny_config()
    d = tempfile.mkdtemp()
    synth.write_hf_model(d, cfg, seed=11)
    om = oracle.OracleModel.from_hf_dir(d)
    ids = synth.prompt_ids(5, 10, cfg.vocab_size)
    full = om.forward_all(ids)
    om.reset()
    tok, lg = om.prefill(ids[:6])
    np.testing.assert_array_equal(lg, full[5])
    assert tok == oracle.argmax(full[5])
    for i in range(6, 10):
        np.testing.assert_array_equal(om.decode_step(int(ids[i])), full[i])
    assert om.kv_len() == 10


@pytest.mark.parametrize("gt,kind", [(synth.GGML_Q8_0, "q8_0"), (synth.GGML_Q4_0, "q4_0"), (synth.GGML_Q4_K, "q4_k"), (synth.GGML_Q6_K, "q6_k")])
def test_gguf_plan_against_float64(oracle, gt, kind):
    # K-quant projections multiply Q8_K-quantised activations (8-bit codes per 256 values), so against an evaluation
    # with exact activations they carry that quantisation's noise; the block formats with f32 activations do not
    kq = kind in ("q4_k", "q6_k")
    cfg = synth.tiny_config(qkv_bias=False, tie_word_embeddings=False, rope_theta=1e4, rms_norm_eps=1e-5, intermediate_size=768 if kq else 640)
    path = os.path.join(tempfile.mkdtemp(), "m.gguf")
    synth.write_gguf_model(path, cfg, seed=5, ggml_type=gt, norm_jitter=0.1)
    om = oracle.OracleModel.from_gguf(path)
    ids = synth.prompt_ids(9, 6, cfg.vocab_size)
    got = om.forward_all(ids)

    # independent float64 evaluation from the dequantised tensors
    md, T = synth.read_gguf(path)
    H, hd, heads, kvh = cfg.hidden_size, cfg.hd, cfg.num_attention_heads, cfg.num_key_value_heads

    def lin(name):
        shape, g, raw = T[name]
        tkind = {synth.GGML_Q8_0: "q8_0", synth.GGML_Q4_0: "q4_0", synth.GGML_Q4_K: "q4_k", synth.GGML_Q6_K: "q6_k"}[g]
        return oracle.dequant(np.array(raw), tkind).reshape(shape).astype(np.float64).T  # [in,out]

    def vec(name):
        return synth.bf16_to_f32(np.array(T[name][2]).view(np.uint16)).astype(np.float64)

    def rms(x, w, eps):
        return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w

    emb = synth.bf16_to_f32(np.array(T["token_embd.weight"][2]).view(np.uint16)).reshape(cfg.vocab_size, H).astype(np.float64)
    S = len(ids)
    h = emb[ids]
    i = np.arange(hd // 2)
    ang = np.arange(S)[:, None] / np.power(cfg.rope_theta, 2.0 * i / hd)[None]
    cos = np.concatenate([np.cos(ang)] * 2, -1)[:, None]
    sin = np.concatenate([np.sin(ang)] * 2, -1)[:, None]
    rot = lambda x: np.concatenate([-x[..., hd // 2 :], x[..., : hd // 2]], -1)
    mask = np.triu(np.full((S, S), -np.inf), 1)
    for l in range(cfg.num_hidden_layers):
        p = f"blk.{l}."
        n = rms(h, vec(p + "attn_norm.weight"), cfg.rms_norm_eps)
        q = (n @ lin(p + "attn_q.weight")).reshape(S, heads, hd)
        k = (n @ lin(p + "attn_k.weight")).reshape(S, kvh, hd)
        v = (n @ lin(p + "attn_v.weight")).reshape(S, kvh, hd)
        q = q * cos + rot(q) * sin
        k = k * cos + rot(k) * sin
        o = np.zeros((S, heads, hd))
        for hh in range(heads):
            sc = q[:, hh] @ k[:, hh // (heads // kvh)].T / np.sqrt(hd) + mask
            pr = np.exp(sc - sc.max(-1, keepdims=True))
            pr /= pr.sum(-1, keepdims=True)
            o[:, hh] = pr @ v[:, hh // (heads // kvh)]
        r = h + o.reshape(S, -1) @ lin(p + "attn_output.weight")
        n = rms(r, vec(p + "ffn_norm.weight"), cfg.rms_norm_eps)
        g = n @ lin(p + "ffn_gate.weight")
        u = n @ lin(p + "ffn_up.weight")
        h = r + (g / (1 + np.exp(-g)) * u) @ lin(p + "ffn_down.weight")
    exp = rms(h, vec("output_norm.weight"), cfg.rms_norm_eps) @ lin("output.weight")
    scale = np.abs(exp).max()
    assert np.abs(got - exp).max() <= (3e-2 if kq else 2e-5) * scale
