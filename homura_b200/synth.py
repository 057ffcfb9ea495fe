"""Seeded synthetic checkpoints in the two container formats Homura loads.

There are no real checkpoints where this code runs, so tests and the benchmark write
random-initialised models of the named architectures from a seed:

* ``write_hf_model``  -> ``config.json`` + ``model.safetensors`` with the HuggingFace tensor
  names that Homura's loader expects (src/hf/weights.rs:267-417 in the Homura repository):
  linears stored ``[out, in]`` in bf16 ~N(0, 0.02) rounded to nearest even, norms = 1,
  biases ~N(0, 0.02).
* ``write_gguf_model`` -> a GGUF v3 file with ``blk.N.*`` tensors (src/gguf.rs:589-708):
  Q8_0 or Q4_0 blocks for all linears (f16 scale = |N(0, 0.01)|, codes uniform), bf16
  embedding and norms.

Every tensor draws from its own PCG64 stream keyed by (seed, crc32(name)), so the bytes do
not depend on generation order.
"""
from __future__ import annotations

import json
import os
import struct
import zlib
from dataclasses import dataclass, asdict
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np

GGUF_MAGIC = 0x46554747  # "GGUF" little-endian
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0, GGML_BF16 = 0, 1, 2, 8, 30
GGML_Q4_K, GGML_Q6_K = 12, 14


@dataclass
class DecoderConfig:
    """Mirror of Homura's TransformerConfig (src/hf/config.rs:11-38)."""

    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_hidden_layers: int
    num_key_value_heads: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 2048
    tie_word_embeddings: bool = False
    head_dim: Optional[int] = None
    # model-shape facts Homura infers from tensor names, not from config.json
    qkv_bias: bool = False
    qk_norm: bool = False

    @property
    def hd(self) -> int:
        return self.head_dim or self.hidden_size // self.num_attention_heads

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.hd

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.hd


# Architectures named by the benchmark configurations.
QWEN25_05B = DecoderConfig(896, 4864, 14, 24, 2, 151936, 1e-6, 1e6, 2048, True, None, True, False)
QWEN25_15B = DecoderConfig(1536, 8960, 12, 28, 2, 151936, 1e-6, 1e6, 2048, True, None, True, False)
QWEN3_06B = DecoderConfig(1024, 3072, 16, 28, 8, 151936, 1e-6, 1e6, 2048, True, 128, False, True)
TINYLLAMA_11B = DecoderConfig(2048, 5632, 32, 22, 4, 32000, 1e-5, 1e4, 2048, False, None, False, False)


def tiny_config(**kw) -> DecoderConfig:
    """A small Qwen2-shaped model for tests that the CPU oracle runs in milliseconds."""
    base = dict(
        hidden_size=256,
        intermediate_size=640,
        num_attention_heads=4,
        num_hidden_layers=3,
        num_key_value_heads=2,
        vocab_size=1024,
        rms_norm_eps=1e-6,
        rope_theta=1e6,
        max_position_embeddings=256,
        tie_word_embeddings=True,
        head_dim=None,
        qkv_bias=True,
        qk_norm=False,
    )
    base.update(kw)
    return DecoderConfig(**base)


def _rng(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64([seed, zlib.crc32(name.encode())]))


def f32_to_bf16_rne(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def normal_bf16(seed: int, name: str, shape: Tuple[int, ...], std: float = 0.02) -> np.ndarray:
    g = _rng(seed, name)
    n = int(np.prod(shape))
    out = np.empty(n, dtype=np.uint16)
    step = 1 << 24
    for i in range(0, n, step):
        m = min(step, n - i)
        v = g.standard_normal(m, dtype=np.float32)
        v *= np.float32(std)
        out[i : i + m] = f32_to_bf16_rne(v)
    return out.reshape(shape)


def ones_bf16(shape) -> np.ndarray:
    return np.full(shape, 0x3F80, dtype=np.uint16)


def hf_tensor_specs(cfg: DecoderConfig) -> List[Tuple[str, Tuple[int, ...], str]]:
    """(name, shape, kind) in file order; kind in {'w','one','bias'}."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    specs: List[Tuple[str, Tuple[int, ...], str]] = [("model.embed_tokens.weight", (V, H), "w")]
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        specs.append((p + "input_layernorm.weight", (H,), "one"))
        for nm, out_f in (("q", cfg.q_dim), ("k", cfg.kv_dim), ("v", cfg.kv_dim)):
            specs.append((p + f"self_attn.{nm}_proj.weight", (out_f, H), "w"))
            if cfg.qkv_bias:
                specs.append((p + f"self_attn.{nm}_proj.bias", (out_f,), "bias"))
        if cfg.qk_norm:
            specs.append((p + "self_attn.q_norm.weight", (cfg.hd,), "one"))
            specs.append((p + "self_attn.k_norm.weight", (cfg.hd,), "one"))
        specs.append((p + "self_attn.o_proj.weight", (H, cfg.q_dim), "w"))
        specs.append((p + "post_attention_layernorm.weight", (H,), "one"))
        specs.append((p + "mlp.gate_proj.weight", (I, H), "w"))
        specs.append((p + "mlp.up_proj.weight", (I, H), "w"))
        specs.append((p + "mlp.down_proj.weight", (H, I), "w"))
    specs.append(("model.norm.weight", (H,), "one"))
    if not cfg.tie_word_embeddings:
        specs.append(("lm_head.weight", (V, H), "w"))
    return specs


def config_json(cfg: DecoderConfig) -> dict:
    d = {
        "hidden_size": cfg.hidden_size,
        "intermediate_size": cfg.intermediate_size,
        "num_attention_heads": cfg.num_attention_heads,
        "num_hidden_layers": cfg.num_hidden_layers,
        "num_key_value_heads": cfg.num_key_value_heads,
        "vocab_size": cfg.vocab_size,
        "rms_norm_eps": cfg.rms_norm_eps,
        "rope_theta": cfg.rope_theta,
        "max_position_embeddings": cfg.max_position_embeddings,
        "tie_word_embeddings": cfg.tie_word_embeddings,
    }
    if cfg.head_dim is not None:
        d["head_dim"] = cfg.head_dim
    # eos_token_id is left out on purpose: it then resolves to u32::MAX in Homura
    # (src/hf/model.rs:373-377) and a random-weight run never stops early.
    return d


def write_hf_model(model_dir: str, cfg: DecoderConfig, seed: int, norm_jitter: float = 0.0) -> str:
    """Write config.json + model.safetensors (all tensors bf16).  Returns model_dir.

    ``norm_jitter`` > 0 perturbs the norm weights around 1 so tests can tell a missing
    norm multiply from a present one; the benchmark models use exactly 1.
    """
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config_json(cfg), f, indent=1)
    specs = hf_tensor_specs(cfg)
    header: Dict[str, dict] = {}
    off = 0
    for name, shape, _ in specs:
        nbytes = int(np.prod(shape)) * 2
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    path = os.path.join(model_dir, "model.safetensors")

    def make(spec):
        name, shape, kind = spec
        if kind in ("w", "bias"):
            return normal_bf16(seed, name, shape, 0.02)
        if norm_jitter > 0:
            v = 1.0 + norm_jitter * _rng(seed, name).standard_normal(shape, dtype=np.float32)
            return f32_to_bf16_rne(v)
        return ones_bf16(shape)

    # every tensor has its own generator (seed, name), so they can be drawn by several threads (numpy's
    # generators release the GIL) and still be written in file order
    from concurrent.futures import ThreadPoolExecutor

    with open(path, "wb") as f, ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as pool:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        window = 32
        futs = [pool.submit(make, sp) for sp in specs[:window]]
        for i in range(len(specs)):
            arr = futs[i].result()
            futs[i] = None
            if i + window < len(specs):
                futs.append(pool.submit(make, specs[i + window]))
            f.write(arr.tobytes())
    return model_dir


def shard_hf_model(src_dir: str, dst_dir: str, n_shards: int = 2) -> str:
    """Rewrite a single-file checkpoint as `n_shards` safetensors files plus model.safetensors.index.json,
    the layout HfModel::load_with_dtype falls back to (src/hf/model.rs:86-127).  Tensors are dealt out
    round-robin, so every shard holds pieces of every layer."""
    os.makedirs(dst_dir, exist_ok=True)
    with open(os.path.join(src_dir, "config.json")) as f, open(os.path.join(dst_dir, "config.json"), "w") as g:
        g.write(f.read())
    tensors = read_safetensors(os.path.join(src_dir, "model.safetensors"))
    names = list(tensors)
    weight_map = {}
    for sh in range(n_shards):
        fname = f"model-{sh + 1:05d}-of-{n_shards:05d}.safetensors"
        mine = names[sh::n_shards]
        header, off = {}, 0
        for name in mine:
            dt, shape, arr = tensors[name]
            header[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [off, off + arr.nbytes]}
            off += arr.nbytes
            weight_map[name] = fname
        hjson = json.dumps(header, separators=(",", ":")).encode()
        hjson += b" " * ((8 - len(hjson) % 8) % 8)
        with open(os.path.join(dst_dir, fname), "wb") as f:
            f.write(struct.pack("<Q", len(hjson)))
            f.write(hjson)
            for name in mine:
                f.write(np.ascontiguousarray(tensors[name][2]).tobytes())
    with open(os.path.join(dst_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": sum(t[2].nbytes for t in tensors.values())}, "weight_map": weight_map}, f)
    return dst_dir


def read_safetensors(path: str) -> Dict[str, Tuple[str, Tuple[int, ...], np.ndarray]]:
    """name -> (dtype string, shape, raw array view).  BF16/F16 come back as uint16 bits."""
    raw = np.memmap(path, dtype=np.uint8, mode="r")
    (hlen,) = struct.unpack("<Q", raw[:8].tobytes())
    header = json.loads(raw[8 : 8 + hlen].tobytes())
    base = 8 + hlen
    np_of = {"BF16": np.uint16, "F16": np.uint16, "F32": np.float32, "F64": np.float64, "I32": np.int32, "I64": np.int64}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        arr = raw[base + b : base + e].view(np_of[info["dtype"]]).reshape(info["shape"])
        out[name] = (info["dtype"], tuple(info["shape"]), arr)
    return out


# ----------------------------------------------------------------------------------------
# GGUF
# ----------------------------------------------------------------------------------------


def quant_blocks(seed: int, name: str, n_out: int, n_in: int, ggml_type: int) -> np.ndarray:
    """Random blocks [n_out, n_in/32] in GGUF byte order: f16 scale |N(0,0.01)| + codes
    (Q8_0 / Q4_0), or super-blocks [n_out, n_in/256] of 144 (Q4_K) / 210 (Q6_K) bytes."""
    assert n_in % 32 == 0
    g = _rng(seed, name)
    if ggml_type in (GGML_Q4_K, GGML_Q6_K):
        assert n_in % 256 == 0, "K-quants need in_features to be a multiple of 256"
        nsb = n_out * (n_in // 256)
        if ggml_type == GGML_Q4_K:
            blk = g.integers(0, 256, size=(nsb, 144), dtype=np.uint8)  # packed 6-bit scales/mins and nibbles: any byte is valid
            d = np.abs(g.standard_normal(nsb, dtype=np.float32) * np.float32(4e-4)).astype(np.float16)
            dmin = np.abs(g.standard_normal(nsb, dtype=np.float32) * np.float32(1e-4)).astype(np.float16)
            blk[:, 0:2] = d.view(np.uint8).reshape(nsb, 2)
            blk[:, 2:4] = dmin.view(np.uint8).reshape(nsb, 2)
        else:
            blk = g.integers(0, 256, size=(nsb, 210), dtype=np.uint8)
            blk[:, 192:208] = g.integers(-64, 64, size=(nsb, 16), dtype=np.int8).view(np.uint8)  # i8 sub-block scales
            d = np.abs(g.standard_normal(nsb, dtype=np.float32) * np.float32(2e-5)).astype(np.float16)
            blk[:, 208:210] = d.view(np.uint8).reshape(nsb, 2)
        return blk.reshape(-1)
    nb = n_out * (n_in // 32)
    scale = np.abs(g.standard_normal(nb, dtype=np.float32) * np.float32(0.01)).astype(np.float16)
    if ggml_type == GGML_Q8_0:
        codes = g.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
        blk = np.empty((nb, 34), dtype=np.uint8)
    elif ggml_type == GGML_Q4_0:
        nib = g.integers(0, 16, size=(nb, 32), dtype=np.uint8)
        codes = (nib[:, :16] | (nib[:, 16:] << 4)).astype(np.uint8)
        blk = np.empty((nb, 18), dtype=np.uint8)
    else:
        raise ValueError(ggml_type)
    blk[:, 0:2] = scale.view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = codes
    return blk.reshape(-1)


def _gguf_str(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _gguf_kv(key: str, val) -> bytes:
    out = _gguf_str(key)
    if isinstance(val, str):
        out += struct.pack("<I", 8) + _gguf_str(val)
    elif isinstance(val, bool):
        out += struct.pack("<IB", 7, int(val))
    elif isinstance(val, float):
        out += struct.pack("<If", 6, val)
    elif isinstance(val, int):
        out += struct.pack("<II", 4, val)
    else:
        raise TypeError(type(val))
    return out


def write_gguf(path: str, metadata: Dict[str, object], tensors: Iterable[Tuple[str, Tuple[int, ...], int, np.ndarray]], alignment: int = 32) -> None:
    """tensors: (name, logical shape outermost-first, ggml type, raw bytes as uint8/uint16 array)."""
    tensors = list(tensors)
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(metadata))
    for k, v in metadata.items():
        head += _gguf_kv(k, v)
    infos = b""
    off = 0
    offsets = []
    for name, shape, gt, data in tensors:
        nbytes = data.nbytes
        infos += _gguf_str(name) + struct.pack("<I", len(shape))
        for d in reversed(shape):  # GGUF stores dims innermost-first (src/gguf.rs:412-417)
            infos += struct.pack("<Q", d)
        infos += struct.pack("<IQ", gt, off)
        offsets.append(off)
        off += (nbytes + alignment - 1) // alignment * alignment
    pre = head + infos
    pad = (alignment - len(pre) % alignment) % alignment
    with open(path, "wb") as f:
        f.write(pre + b"\0" * pad)
        for (name, shape, gt, data), o in zip(tensors, offsets):
            b = data.tobytes()
            f.write(b)
            f.write(b"\0" * ((alignment - len(b) % alignment) % alignment))


def gguf_metadata(cfg: DecoderConfig, arch: str = "llama") -> Dict[str, object]:
    md: Dict[str, object] = {
        "general.architecture": arch,
        f"{arch}.embedding_length": cfg.hidden_size,
        f"{arch}.feed_forward_length": cfg.intermediate_size,
        f"{arch}.attention.head_count": cfg.num_attention_heads,
        f"{arch}.block_count": cfg.num_hidden_layers,
        f"{arch}.attention.head_count_kv": cfg.num_key_value_heads,
        f"{arch}.vocab_size": cfg.vocab_size,
        f"{arch}.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps),
        f"{arch}.rope.freq_base": float(cfg.rope_theta),
        f"{arch}.context_length": cfg.max_position_embeddings,
    }
    if cfg.head_dim is not None:
        md[f"{arch}.attention.key_length"] = cfg.head_dim
    return md


def write_gguf_model(path: str, cfg: DecoderConfig, seed: int, ggml_type: int, quant_lm_head: bool = True, norm_jitter: float = 0.0, k_mix: bool = False, quant_embed: bool = False) -> str:
    """GGUF file: all linears in ``ggml_type`` blocks, bf16 embedding/norms, optional biases (f32).
    ``k_mix`` writes attn_v, ffn_down and output as Q6_K beside Q4_K elsewhere (the mix of a Q4_K_M
    file); ``quant_embed`` quantises token_embd too (Q6_K, or ``ggml_type`` for the 32-value formats)."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q6_names = ("attn_v.weight", "ffn_down.weight", "output.weight") if k_mix else ()

    def norm(name, n):
        if norm_jitter > 0:
            v = 1.0 + norm_jitter * _rng(seed, name).standard_normal(n, dtype=np.float32)
            return (name, (n,), GGML_BF16, f32_to_bf16_rne(v))
        return (name, (n,), GGML_BF16, ones_bf16((n,)))

    def lin(name, out_f, in_f):
        gt = GGML_Q6_K if name.endswith(q6_names) and q6_names else ggml_type
        return (name, (out_f, in_f), gt, quant_blocks(seed, name, out_f, in_f, gt))

    def gen():
        if quant_embed:
            gt = GGML_Q6_K if ggml_type in (GGML_Q4_K, GGML_Q6_K) else ggml_type
            yield ("token_embd.weight", (V, H), gt, quant_blocks(seed, "token_embd.weight", V, H, gt))
        else:
            yield ("token_embd.weight", (V, H), GGML_BF16, normal_bf16(seed, "token_embd.weight", (V, H)))
        for i in range(cfg.num_hidden_layers):
            p = f"blk.{i}."
            yield norm(p + "attn_norm.weight", H)
            for nm, out_f in (("q", cfg.q_dim), ("k", cfg.kv_dim), ("v", cfg.kv_dim)):
                yield lin(p + f"attn_{nm}.weight", out_f, H)
                if cfg.qkv_bias:
                    b = _rng(seed, p + f"attn_{nm}.bias").standard_normal(out_f, dtype=np.float32) * np.float32(0.02)
                    yield (p + f"attn_{nm}.bias", (out_f,), GGML_F32, b)
            if cfg.qk_norm:
                yield norm(p + "attn_q_norm.weight", cfg.hd)
                yield norm(p + "attn_k_norm.weight", cfg.hd)
            yield lin(p + "attn_output.weight", H, cfg.q_dim)
            yield norm(p + "ffn_norm.weight", H)
            yield lin(p + "ffn_gate.weight", I, H)
            yield lin(p + "ffn_up.weight", I, H)
            yield lin(p + "ffn_down.weight", H, I)
        yield norm("output_norm.weight", H)
        if not cfg.tie_word_embeddings:
            if quant_lm_head:
                yield lin("output.weight", V, H)
            else:
                yield ("output.weight", (V, H), GGML_BF16, normal_bf16(seed, "output.weight", (V, H)))

    write_gguf(path, gguf_metadata(cfg), gen())
    return path


def read_gguf(path: str):
    """Minimal GGUF v2/v3 reader: returns (metadata dict, {name: (shape, ggml_type, uint8 view)})."""
    raw = np.memmap(path, dtype=np.uint8, mode="r")
    pos = 0

    def rd(fmt):
        nonlocal pos
        sz = struct.calcsize(fmt)
        v = struct.unpack("<" + fmt, raw[pos : pos + sz].tobytes())
        pos += sz
        return v if len(v) > 1 else v[0]

    def rstr():
        nonlocal pos
        n = rd("Q")
        s = raw[pos : pos + n].tobytes().decode()
        pos += n
        return s

    magic, version = rd("II")
    assert magic == GGUF_MAGIC and version in (2, 3)
    nt, nkv = (rd("QQ") if version >= 3 else rd("II"))
    scalar = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "B", 10: "Q", 11: "q", 12: "d"}

    def rval(t):
        if t == 8:
            return rstr()
        if t == 9:
            et = rd("I")
            n = rd("Q")
            return [rval(et) for _ in range(n)]
        v = rd(scalar[t])
        return bool(v) if t == 7 else v

    md = {}
    for _ in range(nkv):
        k = rstr()
        t = rd("I")
        md[k] = rval(t)
    align = int(md.get("general.alignment", 32))
    infos = []
    for _ in range(nt):
        name = rstr()
        nd = rd("I")
        dims = [rd("Q") for _ in range(nd)]
        dims.reverse()
        gt = rd("I")
        off = rd("Q")
        infos.append((name, tuple(dims), gt, off))
    data0 = (pos + align - 1) // align * align
    bpe = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2), GGML_Q8_0: (32, 34), GGML_Q4_0: (32, 18), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210)}
    tensors = {}
    for name, shape, gt, off in infos:
        bs, ts = bpe[gt]
        nbytes = int(np.prod(shape)) // bs * ts
        tensors[name] = (shape, gt, raw[data0 + off : data0 + off + nbytes])
    return md, tensors


def prompt_ids(seed: int, n: int, vocab: int) -> np.ndarray:
    """Prompt token ids uniform in [0, vocab)."""
    return _rng(seed, "prompt").integers(0, vocab, size=n, dtype=np.int64)
