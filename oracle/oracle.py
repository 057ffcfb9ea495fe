"""ctypes front end of the CPU oracle (oracle/homura_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's
CPU-baseline leg.  The product package never imports this module.

The checkpoint readers used here are independent numpy parsers (homura_b200.synth), not
the product's native loaders, so a loader bug in the product shows up as a parity failure.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libhomura_oracle.so")

ORC_F32, ORC_BF16, ORC_F16, ORC_Q8_0, ORC_Q4_0, ORC_Q4_K, ORC_Q6_K = 0, 1, 2, 3, 4, 5, 6


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "homura_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B" if force else "-s"])
    return _LIB_PATH


def build_native() -> str:
    """The same source built -march=native on the machine that runs it (the benchmark's CPU arm).  Falls back
    to the portable build when the host has no compiler."""
    path = os.path.join(_HERE, "libhomura_oracle_native.so")
    try:
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "native"])
        return path
    except Exception:
        return build()


def use_native_build():
    """Call before the first use of the library: load the -march=native build (timing runs only)."""
    global _LIB_PATH
    if _lib is not None:
        raise RuntimeError("oracle library already loaded")
    _LIB_PATH = build_native()


class OrcConfig(C.Structure):
    _fields_ = [
        ("hidden_size", C.c_int32),
        ("intermediate_size", C.c_int32),
        ("num_attention_heads", C.c_int32),
        ("num_hidden_layers", C.c_int32),
        ("num_key_value_heads", C.c_int32),
        ("vocab_size", C.c_int32),
        ("max_position_embeddings", C.c_int32),
        ("head_dim", C.c_int32),
        ("tie_word_embeddings", C.c_int32),
        ("rms_norm_eps", C.c_double),
        ("rope_theta", C.c_double),
    ]


class OrcSampling(C.Structure):
    _fields_ = [
        ("temperature", C.c_float),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("repetition_penalty", C.c_float),
        ("frequency_penalty", C.c_float),
        ("presence_penalty", C.c_float),
        ("top_k", C.c_int32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.endswith("_native.so"):
        build()
    L = C.CDLL(_LIB_PATH)
    f32p, u8p, u16p, i64p, u32p, vp = (C.POINTER(C.c_float), C.POINTER(C.c_uint8), C.POINTER(C.c_uint16), C.POINTER(C.c_int64), C.POINTER(C.c_uint32), C.c_void_p)
    sig = {
        "orc_f16_to_f32": (C.c_float, [C.c_uint16]),
        "orc_bf16_to_f32": (C.c_float, [C.c_uint16]),
        "orc_f32_to_bf16_trunc": (C.c_uint16, [C.c_float]),
        "orc_rope_table": (None, [C.c_int, C.c_int, C.c_double, vp, vp]),
        "orc_causal_mask": (None, [C.c_int, C.c_int, vp]),
        "orc_rms_norm": (None, [vp, vp, C.c_float, C.c_int, C.c_int, vp]),
        "orc_rms_norm_f64_accum": (None, [vp, vp, C.c_float, C.c_int, C.c_int, vp]),
        "orc_rms_norm_quant_kernel": (None, [vp, vp, C.c_float, C.c_int, C.c_int, vp]),
        "orc_silu": (None, [vp, C.c_int, vp]),
        "orc_softmax": (None, [vp, C.c_int, C.c_int, C.c_int, vp]),
        "orc_rope_half": (None, [vp, C.c_int, C.c_int, C.c_int, vp, vp]),
        "orc_matmul_bf16": (None, [vp, vp, C.c_int, C.c_int, C.c_int, vp]),
        "orc_matmul_f32": (None, [vp, vp, C.c_int, C.c_int, C.c_int, vp]),
        "orc_matmul_q8_0": (None, [vp, vp, C.c_int, C.c_int, C.c_int, vp]),
        "orc_matmul_q4_0": (None, [vp, vp, C.c_int, C.c_int, C.c_int, vp]),
        "orc_dequant_q8_0": (None, [vp, C.c_size_t, vp]),
        "orc_dequant_q4_0": (None, [vp, C.c_size_t, vp]),
        "orc_matmul_q4_k": (None, [vp, vp, C.c_int, C.c_int, C.c_int, vp]),
        "orc_matmul_q6_k": (None, [vp, vp, C.c_int, C.c_int, C.c_int, vp]),
        "orc_dequant_q4_k": (None, [vp, C.c_size_t, vp]),
        "orc_dequant_q6_k": (None, [vp, C.c_size_t, vp]),
        "orc_quantize_q8_k": (None, [vp, C.c_int, vp, vp, vp]),
        "orc_kv_new": (vp, [C.c_int, C.c_int, C.c_int, C.c_int]),
        "orc_kv_free": (None, [vp]),
        "orc_kv_append_key": (C.c_int, [vp, C.c_int, vp, C.c_int]),
        "orc_kv_append_value": (C.c_int, [vp, C.c_int, vp, C.c_int]),
        "orc_kv_advance_by": (None, [vp, C.c_int]),
        "orc_kv_reset": (None, [vp, C.c_int]),
        "orc_kv_current_len": (C.c_int, [vp]),
        "orc_kv_view": (None, [vp, C.c_int, vp, vp]),
        "orc_gqa_attention": (None, [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_int, vp]),
        "orc_argmax": (C.c_uint32, [vp, C.c_int]),
        "orc_rng_new": (C.c_uint64, [C.c_uint64]),
        "orc_rng_next_f32": (C.c_float, [C.POINTER(C.c_uint64)]),
        "orc_sample_token": (C.c_uint32, [vp, C.c_int, C.POINTER(OrcSampling), vp, C.c_int, C.POINTER(C.c_uint64)]),
        "orc_model_new": (vp, [C.POINTER(OrcConfig), C.c_int]),
        "orc_model_free": (None, [vp]),
        "orc_model_set_tensor": (C.c_int, [vp, C.c_char_p, C.c_int, i64p, C.c_int, vp]),
        "orc_model_finalize": (C.c_int, [vp]),
        "orc_model_reset": (None, [vp]),
        "orc_model_kv_len": (C.c_int, [vp]),
        "orc_model_prefill": (C.c_int, [vp, vp, C.c_int, C.c_int, vp, u32p]),
        "orc_model_decode_step": (C.c_int, [vp, C.c_uint32, vp]),
        "orc_model_forward_all": (C.c_int, [vp, vp, C.c_int, C.c_int, vp]),
        "orc_model_kv_view": (C.c_int, [vp, C.c_int, vp, vp]),
        "orc_num_threads": (C.c_int, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- thin numpy wrappers around the op-level functions ---------------------------------


def rope_table(head_dim, max_pos, theta):
    cos = np.empty((max_pos, head_dim), np.float32)
    sin = np.empty((max_pos, head_dim), np.float32)
    lib().orc_rope_table(head_dim, max_pos, float(theta), _p(cos), _p(sin))
    return cos, sin


def causal_mask(seq, past):
    m = np.empty((seq, seq + past), np.float32)
    lib().orc_causal_mask(seq, past, _p(m))
    return m


def rms_norm(x, w, eps, variant="f32"):
    x = _f32(x)
    w = _f32(w)
    out = np.empty_like(x)
    n = x.shape[-1]
    fn = {"f32": lib().orc_rms_norm, "f64_accum": lib().orc_rms_norm_f64_accum, "quant_kernel": lib().orc_rms_norm_quant_kernel}[variant]
    fn(_p(x), _p(w), float(eps), x.size // n, n, _p(out))
    return out


def silu(x):
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_silu(_p(x), x.size, _p(out))
    return out


def softmax(x, f64_sum=False):
    x = _f32(x)
    out = np.empty_like(x)
    n = x.shape[-1]
    lib().orc_softmax(_p(x), x.size // n, n, int(f64_sum), _p(out))
    return out


def rope_half(x, cos_rows, sin_rows):
    """x [seq, heads, hd]; cos/sin rows [seq, hd]."""
    x = _f32(x).copy()
    s, h, d = x.shape
    lib().orc_rope_half(_p(x), s, h, d, _p(_f32(cos_rows)), _p(_f32(sin_rows)))
    return x


def matmul_bf16(x, w_bits):
    x = _f32(x)
    M, K = x.shape
    N = w_bits.shape[1]
    w_bits = np.ascontiguousarray(w_bits, dtype=np.uint16)
    y = np.empty((M, N), np.float32)
    lib().orc_matmul_bf16(_p(x), _p(w_bits), M, K, N, _p(y))
    return y


def matmul_f32(x, w):
    x = _f32(x)
    w = _f32(w)
    M, K = x.shape
    N = w.shape[1]
    y = np.empty((M, N), np.float32)
    lib().orc_matmul_f32(_p(x), _p(w), M, K, N, _p(y))
    return y


def matmul_q(x, blocks, N, kind):
    x = _f32(x)
    M, K = x.shape
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    y = np.empty((M, N), np.float32)
    fn = getattr(lib(), "orc_matmul_" + kind)  # q8_0, q4_0, q4_k, q6_k
    fn(_p(x), _p(blocks), M, K, N, _p(y))
    return y


QUANT_BLOCK = {"q8_0": (34, 32), "q4_0": (18, 32), "q4_k": (144, 256), "q6_k": (210, 256)}  # bytes, values


def quantize_q8_k(x):
    """Q8_K activation quantisation of one row: (int8 codes [K], f32 scales [K/256], int32 group sums [K/16])."""
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    K = x.size
    q8 = np.empty(K, np.int8)
    d = np.empty(K // 256, np.float32)
    bs = np.empty(K // 16, np.int32)
    lib().orc_quantize_q8_k(_p(x), K, _p(q8), _p(d), _p(bs))
    return q8, d, bs


def dequant(blocks, kind):
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    bsz, vals = QUANT_BLOCK[kind]
    nb = blocks.size // bsz
    out = np.empty(nb * vals, np.float32)
    getattr(lib(), "orc_dequant_" + kind)(_p(blocks), nb, _p(out))
    return out


def gqa_attention(q, k, v, mask, heads, kv_heads, f64_softmax_sum=False):
    """q [S, heads, hd]; k, v [kv_heads, T, hd] contiguous; mask [S, T] -> [S, heads*hd]."""
    q, k, v, mask = _f32(q), _f32(k), _f32(v), _f32(mask)
    S, _, hd = q.shape
    T = k.shape[1]
    out = np.empty((S, heads * hd), np.float32)
    lib().orc_gqa_attention(_p(q), _p(k), _p(v), _p(mask), S, T, heads, kv_heads, hd, T * hd, int(f64_softmax_sum), _p(out))
    return out


def argmax(logits) -> int:
    logits = _f32(logits)
    return int(lib().orc_argmax(_p(logits), logits.size))


class Rng:
    def __init__(self, seed: int):
        self.state = C.c_uint64(lib().orc_rng_new(seed))

    def next_f32(self) -> float:
        return float(lib().orc_rng_next_f32(C.byref(self.state)))


def sample_token(logits, rng: Rng, generated=(), temperature=0.7, top_k=50, top_p=0.9, min_p=0.0, repetition_penalty=1.1, frequency_penalty=0.0, presence_penalty=0.0) -> int:
    logits = _f32(logits)
    cfg = OrcSampling(temperature, top_p, min_p, repetition_penalty, frequency_penalty, presence_penalty, top_k)
    gen = np.ascontiguousarray(generated, dtype=np.uint32)
    return int(lib().orc_sample_token(_p(logits), logits.size, C.byref(cfg), _p(gen), gen.size, C.byref(rng.state)))


class KvCache:
    """Mirror of runtime::KvCache for the indexing known-answer tests."""

    def __init__(self, layers, heads, max_len, hd):
        self.p = lib().orc_kv_new(layers, heads, max_len, hd)
        self.heads, self.hd = heads, hd

    def __del__(self):
        if getattr(self, "p", None) and _lib is not None:
            _lib.orc_kv_free(self.p)
            self.p = None

    def append_key(self, layer, k):
        k = _f32(k)
        return lib().orc_kv_append_key(self.p, layer, _p(k), k.shape[-2])

    def append_value(self, layer, v):
        v = _f32(v)
        return lib().orc_kv_append_value(self.p, layer, _p(v), v.shape[-2])

    def advance_by(self, n):
        lib().orc_kv_advance_by(self.p, n)

    def reset(self, n=0):
        lib().orc_kv_reset(self.p, n)

    def current_len(self):
        return lib().orc_kv_current_len(self.p)

    def view(self, layer):
        n = self.current_len()
        k = np.empty((1, self.heads, n, self.hd), np.float32)
        v = np.empty_like(k)
        lib().orc_kv_view(self.p, layer, _p(k), _p(v))
        return k, v


# ---- whole-model oracle ------------------------------------------------------------------

_GGML_TO_ORC = {0: ORC_F32, 1: ORC_F16, 30: ORC_BF16, 8: ORC_Q8_0, 2: ORC_Q4_0, 12: ORC_Q4_K, 14: ORC_Q6_K}
_ST_TO_ORC = {"F32": ORC_F32, "BF16": ORC_BF16, "F16": ORC_F16}


class OracleModel:
    """HfModel + HfGenerationContext restated on the CPU (src/hf/model.rs:37-382)."""

    def __init__(self, cfg_dict: dict, keep_bf16: bool = True):
        c = OrcConfig()
        c.hidden_size = cfg_dict["hidden_size"]
        c.intermediate_size = cfg_dict["intermediate_size"]
        c.num_attention_heads = cfg_dict["num_attention_heads"]
        c.num_hidden_layers = cfg_dict["num_hidden_layers"]
        c.num_key_value_heads = cfg_dict.get("num_key_value_heads") or cfg_dict["num_attention_heads"]
        c.vocab_size = cfg_dict["vocab_size"]
        c.max_position_embeddings = cfg_dict.get("max_position_embeddings", 2048)
        c.head_dim = cfg_dict.get("head_dim") or 0
        c.tie_word_embeddings = int(bool(cfg_dict.get("tie_word_embeddings", False)))
        c.rms_norm_eps = cfg_dict.get("rms_norm_eps", 1e-6)
        c.rope_theta = cfg_dict.get("rope_theta", 10000.0)
        self.cfg = c
        self.vocab = c.vocab_size
        self.layers = c.num_hidden_layers
        self.kv_heads = c.num_key_value_heads
        self.hd = c.head_dim or c.hidden_size // c.num_attention_heads
        self.p = lib().orc_model_new(C.byref(c), int(keep_bf16))
        self.max_seq_len = c.max_position_embeddings

    def __del__(self):
        if getattr(self, "p", None) and _lib is not None:
            _lib.orc_model_free(self.p)
            self.p = None

    def set_tensor(self, name: str, dtype: int, shape, data: np.ndarray):
        shp = (C.c_int64 * len(shape))(*shape)
        data = np.ascontiguousarray(data)
        rc = lib().orc_model_set_tensor(self.p, name.encode(), dtype, shp, len(shape), _p(data))
        if rc:
            raise ValueError(f"oracle: set_tensor({name}) -> {rc}")

    def finalize(self):
        rc = lib().orc_model_finalize(self.p)
        if rc:
            raise ValueError(f"oracle: finalize -> {rc}")

    @classmethod
    def from_hf_dir(cls, model_dir: str, keep_bf16: bool = True, max_seq_len: Optional[int] = None) -> "OracleModel":
        import json

        from homura_b200 import synth

        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        m = cls(cfg, keep_bf16)
        for name, (dt, shape, arr) in synth.read_safetensors(os.path.join(model_dir, "model.safetensors")).items():
            m.set_tensor(name, _ST_TO_ORC[dt], shape, arr)
        m.finalize()
        if max_seq_len:
            m.max_seq_len = max_seq_len
        return m

    @classmethod
    def from_gguf(cls, path: str, max_seq_len: Optional[int] = None) -> "OracleModel":
        from homura_b200 import synth

        md, tensors = synth.read_gguf(path)
        arch = md["general.architecture"]
        cfg = {
            "hidden_size": md[f"{arch}.embedding_length"],
            "intermediate_size": md[f"{arch}.feed_forward_length"],
            "num_attention_heads": md[f"{arch}.attention.head_count"],
            "num_hidden_layers": md[f"{arch}.block_count"],
            "num_key_value_heads": md.get(f"{arch}.attention.head_count_kv"),
            "vocab_size": md[f"{arch}.vocab_size"],
            # src/gguf.rs:519-523: float metadata is read as f32 then widened
            "rms_norm_eps": float(np.float32(md.get(f"{arch}.attention.layer_norm_rms_epsilon", 1e-6))),
            "rope_theta": float(np.float32(md.get(f"{arch}.rope.freq_base", 10000.0))),
            "max_position_embeddings": md.get(f"{arch}.context_length", 2048),
            "tie_word_embeddings": "output.weight" not in tensors,
            "head_dim": md.get(f"{arch}.attention.key_length"),
        }
        m = cls(cfg, keep_bf16=False)
        for name, (shape, gt, raw) in tensors.items():
            m.set_tensor(name, _GGML_TO_ORC[gt], shape, raw)
        m.finalize()
        if max_seq_len:
            m.max_seq_len = max_seq_len
        return m

    # -- GenerativeModel --
    def prefill(self, ids, want_logits=True):
        ids = np.ascontiguousarray(ids, dtype=np.int64)
        logits = np.empty(self.vocab, np.float32)
        tok = C.c_uint32(0)
        rc = lib().orc_model_prefill(self.p, _p(ids), ids.size, self.max_seq_len, _p(logits), C.byref(tok))
        if rc:
            raise RuntimeError(f"oracle prefill -> {rc}")
        return int(tok.value), logits

    def decode_step(self, token: int) -> np.ndarray:
        logits = np.empty(self.vocab, np.float32)
        rc = lib().orc_model_decode_step(self.p, int(token), _p(logits))
        if rc:
            raise RuntimeError(f"oracle decode_step -> {rc}")
        return logits

    def forward_all(self, ids) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int64)
        logits = np.empty((ids.size, self.vocab), np.float32)
        rc = lib().orc_model_forward_all(self.p, _p(ids), ids.size, self.max_seq_len, _p(logits))
        if rc:
            raise RuntimeError(f"oracle forward_all -> {rc}")
        return logits

    def reset(self):
        lib().orc_model_reset(self.p)

    def kv_len(self) -> int:
        return lib().orc_model_kv_len(self.p)

    def kv_view(self, layer):
        n = self.kv_len()
        k = np.empty((self.kv_heads, n, self.hd), np.float32)
        v = np.empty_like(k)
        lib().orc_model_kv_view(self.p, layer, _p(k), _p(v))
        return k, v

    def generate_greedy(self, prompt, max_new_tokens, return_logits=False):
        """generate_streaming_core with temperature 0 and all penalties neutral
        (src/generate.rs:100-315): 1 token from prefill + (max_new_tokens-1) decode steps."""
        tok, lg = self.prefill(prompt)
        out = [tok]
        all_logits = [lg] if return_logits else None
        pos = len(prompt)
        for _ in range(1, max_new_tokens):
            if pos >= self.max_seq_len:
                break
            lg = self.decode_step(out[-1])
            pos += 1
            out.append(argmax(lg))
            if return_logits:
                all_logits.append(lg)
        return (out, all_logits) if return_logits else out


def num_threads() -> int:
    return lib().orc_num_threads()
