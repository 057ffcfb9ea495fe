"""Generates tests/golden/hf_xcheck.npz: logits of three tiny seeded decoders (Qwen2-, Llama-
and Qwen3-shaped) evaluated in float32 by the `transformers` reference implementations.

The CPU oracle is checked against these vectors (tests/test_oracle_model.py), which guards the
parts of the restatement that no Homura unit test pins (RoPE half rotation, GQA head mapping,
QK-norm, bias, tied head).  Run:  python tests/golden/make_hf_xcheck.py
"""
import os
import sys
import tempfile

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from homura_b200 import synth  # noqa: E402

CASES = {
    "qwen2": dict(),
    "llama": dict(qkv_bias=False, tie_word_embeddings=False, rope_theta=1e4, num_attention_heads=8, num_key_value_heads=2, rms_norm_eps=1e-5),
    "qwen3": dict(qkv_bias=False, qk_norm=True, head_dim=128, num_attention_heads=4, num_key_value_heads=2),
}
SEED, PROMPT_SEED, NTOK, JITTER = 7, 3, 12, 0.1


def hf_model(cfg, d):
    from transformers import LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM, Qwen3Config, Qwen3ForCausalLM

    common = dict(
        hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, num_attention_heads=cfg.num_attention_heads,
        num_hidden_layers=cfg.num_hidden_layers, num_key_value_heads=cfg.num_key_value_heads, vocab_size=cfg.vocab_size,
        rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta, max_position_embeddings=cfg.max_position_embeddings,
        tie_word_embeddings=cfg.tie_word_embeddings,
    )
    if cfg.qk_norm:
        m = Qwen3ForCausalLM(Qwen3Config(head_dim=cfg.hd, **common))
    elif cfg.qkv_bias:
        m = Qwen2ForCausalLM(Qwen2Config(**common))
    else:
        m = LlamaForCausalLM(LlamaConfig(**common))
    sd = {}
    for name, (_, shape, arr) in synth.read_safetensors(os.path.join(d, "model.safetensors")).items():
        sd[name] = torch.from_numpy(synth.bf16_to_f32(np.array(arr)).reshape(shape).copy())
    if cfg.tie_word_embeddings:
        sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    res = m.load_state_dict(sd, strict=False)
    assert not res.missing_keys and not res.unexpected_keys, res
    return m.float().eval()


def main():
    out = {}
    for name, kw in CASES.items():
        cfg = synth.tiny_config(**kw)
        d = tempfile.mkdtemp()
        synth.write_hf_model(d, cfg, seed=SEED, norm_jitter=JITTER)
        ids = synth.prompt_ids(PROMPT_SEED, NTOK, cfg.vocab_size)
        with torch.no_grad():
            logits = hf_model(cfg, d)(torch.from_numpy(ids)[None]).logits[0].numpy()
        out[name + "_ids"] = ids
        out[name + "_logits"] = logits[[3, NTOK - 1]].astype(np.float32)  # two positions keep the file small
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "hf_xcheck.npz"), **out)


if __name__ == "__main__":
    main()
