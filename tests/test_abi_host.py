"""Host-side checks of the C ABI library that need no GPU: it loads, exports every symbol the
header declares, parses checkpoints the way Homura's loaders do, samples like sample_token,
and fails loudly (no CPU fallback) when asked to compute without a device."""
import json
import os
import re
import struct
import tempfile

import numpy as np
import pytest

from homura_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "homura_b200.h")).read()
    return sorted(set(re.findall(r"HM_API[^;(]*?\b(hm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(hm):
    lib = hm.load_library()
    names = declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/homura_b200.h but not exported"
    assert sorted(hm.SIGNATURES) == names, "python binding and header disagree"
    assert b"sm_100a" in lib.hm_version()


def test_config_json_parsing_matches_reference_cases(hm):
    # the three configs of src/hf/config.rs:80-150
    cases = [
        ({"architectures": ["Qwen2ForCausalLM"], "hidden_size": 896, "intermediate_size": 4864, "num_attention_heads": 14, "num_hidden_layers": 24,
          "num_key_value_heads": 2, "vocab_size": 151936, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 32768,
          "tie_word_embeddings": True, "eos_token_id": 151643, "bos_token_id": 151643},
         dict(num_key_value_heads=2, head_dim=64, tie_word_embeddings=True, eos_token_id=151643, rope_theta=1e6, max_position_embeddings=32768)),
        ({"hidden_size": 4096, "intermediate_size": 11008, "num_attention_heads": 32, "num_hidden_layers": 32, "vocab_size": 32000, "rope_theta": 10000.0},
         dict(num_key_value_heads=32, head_dim=128, tie_word_embeddings=False, rope_theta=1e4, rms_norm_eps=1e-6, max_position_embeddings=2048, eos_token_id=-1)),
        ({"architectures": ["Qwen3ForCausalLM"], "hidden_size": 1024, "intermediate_size": 3072, "num_attention_heads": 16, "num_hidden_layers": 28,
          "num_key_value_heads": 8, "vocab_size": 151936, "head_dim": 128, "rope_theta": 1000000, "tie_word_embeddings": True, "eos_token_id": 151645},
         dict(num_key_value_heads=8, head_dim=128, tie_word_embeddings=True, eos_token_id=151645)),
    ]
    for js, expect in cases:
        d = tempfile.mkdtemp()
        json.dump(js, open(os.path.join(d, "config.json"), "w"))
        # a minimal safetensors file: one F32 tensor "x" = [1, 2]  (src/hf/safetensors.rs:240-264)
        header = b'{"x":{"dtype":"F32","shape":[2],"data_offsets":[0,8]}}'
        with open(os.path.join(d, "model.safetensors"), "wb") as f:
            f.write(struct.pack("<Q", len(header)) + header + struct.pack("<ff", 1.0, 2.0))
        info = hm.checkpoint_info(d)
        for k, v in expect.items():
            assert info["config"][k] == v, (k, info["config"][k], v)
        assert info["tensors"] == [{"name": "x", "dtype": "F32", "shape": [2], "nbytes": 8, "fnv1a": info["tensors"][0]["fnv1a"]}]


def fnv1a(b: bytes) -> str:
    h = 1469598103934665603
    for x in b:
        h = ((h ^ x) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return f"{h:016x}"


def test_safetensors_listing_matches_writer(hm):
    cfg = synth.tiny_config(num_hidden_layers=1, vocab_size=64, hidden_size=64, intermediate_size=64, num_attention_heads=1, num_key_value_heads=1)
    d = synth.write_hf_model(tempfile.mkdtemp(), cfg, seed=3)
    info = hm.checkpoint_info(d)
    assert info["format"] == "safetensors"
    want = synth.read_safetensors(os.path.join(d, "model.safetensors"))
    got = {t["name"]: t for t in info["tensors"]}
    assert set(got) == set(want)
    for name, (dt, shape, arr) in want.items():
        assert got[name]["dtype"] == dt and tuple(got[name]["shape"]) == shape
        assert got[name]["fnv1a"] == fnv1a(np.array(arr).tobytes())


def test_sharded_safetensors_index_is_followed(hm):
    # src/hf/model.rs:86-127: without model.safetensors the loader reads model.safetensors.index.json and
    # loads every shard its weight_map names, each once
    cfg = synth.tiny_config(num_hidden_layers=2, vocab_size=64, hidden_size=64, intermediate_size=64, num_attention_heads=1, num_key_value_heads=1)
    d = synth.write_hf_model(tempfile.mkdtemp(), cfg, seed=3)
    whole = {t["name"]: t for t in hm.checkpoint_info(d)["tensors"]}
    for n_shards in (2, 3):
        sd = synth.shard_hf_model(d, tempfile.mkdtemp(), n_shards)
        assert not os.path.exists(os.path.join(sd, "model.safetensors"))
        info = hm.checkpoint_info(sd)
        got = {t["name"]: t for t in info["tensors"]}
        assert len(info["tensors"]) == len(whole) and got == whole  # same names, dtypes, shapes, bytes (fnv1a)
        assert info["config"] == hm.checkpoint_info(d)["config"]
    # an index that names a missing shard, and an index without weight_map
    os.remove(os.path.join(sd, "model-00002-of-00003.safetensors"))
    with pytest.raises(hm.HomuraError) as e:
        hm.checkpoint_info(sd)
    assert e.value.status == hm.HM_ERR_IO
    json.dump({"metadata": {}}, open(os.path.join(sd, "model.safetensors.index.json"), "w"))
    with pytest.raises(hm.HomuraError) as e:
        hm.checkpoint_info(sd)
    assert "weight_map" in e.value.message


def test_gguf_listing_matches_writer(hm):
    # container rules of src/gguf.rs:1055-1172: dims reversed to outermost-first, aligned data
    cfg = synth.tiny_config(num_hidden_layers=1, vocab_size=64, hidden_size=64, intermediate_size=64, num_attention_heads=1, num_key_value_heads=1,
                            qkv_bias=False, tie_word_embeddings=False, rope_theta=1e4, rms_norm_eps=1e-5)
    for gt, name in ((synth.GGML_Q8_0, "Q8_0"), (synth.GGML_Q4_0, "Q4_0")):
        p = os.path.join(tempfile.mkdtemp(), "m.gguf")
        synth.write_gguf_model(p, cfg, seed=4, ggml_type=gt)
        info = hm.checkpoint_info(p)
        assert info["format"] == "gguf"
        c = info["config"]
        assert (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["vocab_size"], c["tie_word_embeddings"]) == (64, 1, 1, 64, False)
        assert c["rope_theta"] == 1e4 and abs(c["rms_norm_eps"] - 1e-5) < 1e-12
        md, tensors = synth.read_gguf(p)
        got = {t["name"]: t for t in info["tensors"]}
        assert set(got) == set(tensors)
        for nm, (shape, g, raw) in tensors.items():
            assert tuple(got[nm]["shape"]) == shape
            assert got[nm]["fnv1a"] == fnv1a(np.array(raw).tobytes())
        assert got["blk.0.attn_q.weight"]["dtype"] == name
        assert got["blk.0.attn_q.weight"]["nbytes"] == 64 * 2 * (34 if name == "Q8_0" else 18)


def test_malformed_checkpoints_are_reported(hm):
    d = tempfile.mkdtemp()
    with pytest.raises(hm.HomuraError) as e:
        hm.checkpoint_info(d)
    assert e.value.status == hm.HM_ERR_IO
    json.dump({"hidden_size": 8}, open(os.path.join(d, "config.json"), "w"))
    with pytest.raises(hm.HomuraError) as e:
        hm.checkpoint_info(d)
    assert "missing field" in e.value.message
    p = os.path.join(d, "bad.gguf")
    open(p, "wb").write(b"NOPE" + b"\0" * 32)
    with pytest.raises(hm.HomuraError) as e:
        hm.checkpoint_info(p)
    assert "magic" in e.value.message
    # truncated safetensors header (src/hf/safetensors.rs:44-56)
    cfg = synth.tiny_config(num_hidden_layers=1, vocab_size=64, hidden_size=64, intermediate_size=64, num_attention_heads=1, num_key_value_heads=1)
    d2 = synth.write_hf_model(tempfile.mkdtemp(), cfg, seed=3)
    raw = open(os.path.join(d2, "model.safetensors"), "rb").read()
    open(os.path.join(d2, "model.safetensors"), "wb").write(raw[: len(raw) // 2])
    with pytest.raises(hm.HomuraError) as e:
        hm.checkpoint_info(d2)
    assert e.value.status == hm.HM_ERR_IO


def test_host_sampler_matches_oracle(hm, oracle):
    rng = np.random.default_rng(0)
    logits = rng.standard_normal(500).astype(np.float32) * 3
    gen = [3, 7, 7, 20]
    for kw in (dict(temperature=0.0, repetition_penalty=1.0), dict(temperature=0.0, repetition_penalty=1.1), dict(),
               dict(temperature=1.3, top_k=0, top_p=1.0, min_p=0.05, frequency_penalty=0.3, presence_penalty=0.2)):
        cfg = hm.SamplingConfig(**kw)
        r = oracle.Rng(42)
        state = 42 | 1
        for _ in range(20):
            want = oracle.sample_token(logits, r, gen, **{k: getattr(cfg, k) for k in ("temperature", "top_k", "top_p", "min_p", "repetition_penalty", "frequency_penalty", "presence_penalty")})
            got, state = hm.sample_token(logits, cfg, gen, state)
            assert got == want
    # sample_token_greedy, src/generate.rs:892-900
    tok, _ = hm.sample_token([0.0, 1.0, 0.5, 0.2], hm.SamplingConfig(temperature=0.0), [], 1)
    assert tok == 1


def test_no_cpu_fallback_without_device(hm):
    if hm.device_count() > 0:
        pytest.skip("a GPU is present")
    d = synth.write_hf_model(tempfile.mkdtemp(), synth.tiny_config(), seed=1)
    with pytest.raises(hm.HomuraError) as e:
        hm.HfModel.load(d)
    assert e.value.status == hm.HM_ERR_CUDA and "no CPU fallback" in e.value.message
    with pytest.raises(hm.HomuraError) as e:
        hm.rms_norm(np.ones((1, 8), np.float32), np.ones(8, np.float32), 1e-6)
    assert e.value.status == hm.HM_ERR_CUDA
