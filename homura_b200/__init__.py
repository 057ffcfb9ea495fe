"""homura_b200 -- Python front end of the B200 decode engine (libhomura_b200.so).

The names mirror Homura's own interface on this path so that a test written against the
reference reads the same here (file:line in the Homura repository):

    HfModel.load / load_with_dtype / load_gguf      src/hf/model.rs:37-145
    HfModel.run_kv-style decode, kv_cache_len, ...   src/hf/model.rs:198-249
    HfGenerationContext.prefill / decode_step        src/hf/model.rs:301-382
    SamplingConfig                                   src/generate.rs:648-683
    DType                                            src/dtype.rs:8-26

Everything computes on the GPU through the C ABI of include/homura_b200.h; there is no CPU
path.  Importing this package does not load the library -- the first call does, and it
raises if the library is missing or cannot be loaded.
"""
from __future__ import annotations

import ctypes as C
import enum
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhomura_b200.so")

HM_OK, HM_ERR_INVALID, HM_ERR_CUDA, HM_ERR_KV_FULL, HM_ERR_IO, HM_ERR_UNSUPPORTED, HM_ERR_TIMEOUT, HM_ERR_STATE = range(8)
LAYOUT_KN, LAYOUT_SLAB128 = 0, 1


class DType(enum.IntEnum):
    F32 = 0
    BF16 = 1
    F16 = 2
    Q8_0 = 3
    Q4_0 = 4
    I64 = 5
    I32 = 6
    U8 = 7
    Q4_K = 8
    Q6_K = 9


class HomuraError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[status {status}] {message}")
        self.status = status
        self.message = message


class KvCacheFull(HomuraError):
    pass


class _Config(C.Structure):
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
        ("has_qkv_bias", C.c_int32),
        ("has_qk_norm", C.c_int32),
        ("weight_dtype", C.c_int32),
        ("eos_token_id", C.c_uint32),
        ("bos_token_id", C.c_uint32),
        ("rms_norm_eps", C.c_double),
        ("rope_theta", C.c_double),
    ]


class _Sampling(C.Structure):
    _fields_ = [
        ("temperature", C.c_float),
        ("top_k", C.c_int32),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("repetition_penalty", C.c_float),
        ("frequency_penalty", C.c_float),
        ("presence_penalty", C.c_float),
        ("seed_set", C.c_int32),
        ("seed", C.c_uint64),
    ]


class _KernelStat(C.Structure):
    _fields_ = [("name", C.c_char * 32), ("launches_per_step", C.c_int32), ("ms_per_step", C.c_float), ("bytes_per_step", C.c_uint64)]


_vp, _i32, _u32p, _i32p, _f32p, _i64p = C.c_void_p, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_int32), C.POINTER(C.c_float), C.POINTER(C.c_int64)

# name -> (restype, argtypes); every symbol include/homura_b200.h declares
SIGNATURES = {
    "hm_version": (C.c_char_p, []),
    "hm_device_count": (_i32, []),
    "hm_last_error_global": (C.c_char_p, []),
    "hm_model_load": (_i32, [C.c_char_p, _i32, _i32, C.POINTER(_vp)]),
    "hm_model_load_gguf": (_i32, [C.c_char_p, _i32, C.POINTER(_vp)]),
    "hm_engine_create": (_i32, [C.POINTER(_Config), _i32, C.POINTER(_vp)]),
    "hm_load_tensor": (_i32, [_vp, C.c_char_p, _i32, _i64p, _i32, _vp, C.c_size_t]),
    "hm_finalize_weights": (_i32, [_vp]),
    "hm_engine_destroy": (None, [_vp]),
    "hm_last_error": (C.c_char_p, [_vp]),
    "hm_get_config": (_i32, [_vp, C.POINTER(_Config)]),
    "hm_weight_bytes": (_i32, [_vp, C.POINTER(C.c_uint64)]),
    "hm_checkpoint_info": (_i32, [C.c_char_p, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "hm_kv_alloc": (_i32, [_vp, _i32, _i32, _i32, _i32]),
    "hm_kv_free": (_i32, [_vp]),
    "hm_kv_reset": (_i32, [_vp, _i32]),
    "hm_kv_len": (_i32, [_vp, _i32, _i32p]),
    "hm_kv_append": (_i32, [_vp, _i32, _i32, _vp, _vp, _i32, _i32]),
    "hm_kv_view": (_i32, [_vp, _i32, _i32, _vp, _vp]),
    "hm_prefill": (_i32, [_vp, _i32, _vp, _i32, _vp, _u32p]),
    "hm_decode_step": (_i32, [_vp, _vp, _vp, _vp]),
    "hm_decode_step_sampled": (_i32, [_vp, _vp, C.POINTER(_Sampling), _vp, _vp, _vp]),
    "hm_generate": (_i32, [_vp, _i32, _vp, _i32, _i32, C.POINTER(_Sampling), _vp, _i32p]),
    "hm_decode_greedy_n": (_i32, [_vp, _vp, _i32, _vp]),
    "hm_sample_token": (_i32, [_vp, _i32, C.POINTER(_Sampling), _vp, _i32, C.POINTER(C.c_uint64), _u32p]),
    "hm_sample_token_device": (_i32, [_vp, _i32, C.POINTER(_Sampling), _vp, _i32, C.POINTER(C.c_uint64), _u32p]),
    "hm_time_decode": (_i32, [_vp, _i32, _i32, _f32p]),
    "hm_profile_decode": (_i32, [_vp, _i32, C.POINTER(_KernelStat), _i32, _i32p]),
    "hm_selftest_expire_wait": (_i32, [_vp]),
    "hm_engine_stream": (_vp, [_vp]),
    "hm_launches_per_step": (_i32, [_vp, _i32p]),
    "hm_gemv_bf16": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "hm_gemv_bf16_noalloc": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "hm_pack_bf16_slabs": (_i32, [_vp, _i32, _i32, _vp, _vp]),
    "hm_gemm_bf16_tc": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "hm_tc_packed_elems": (C.c_size_t, [_i32, _i32]),
    "hm_pack_bf16_tc": (_i32, [_vp, _i32, _i32, _vp, _vp]),
    "hm_gemv_quant": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "hm_dequant": (_i32, [_vp, _i32, C.c_size_t, _vp, _vp]),
    "hm_rms_norm": (_i32, [_vp, _vp, C.c_float, _i32, _i32, _vp, _vp]),
    "hm_qknorm_rope": (_i32, [_vp, _i32, _i32, _i32, _vp, C.c_float, _vp, _vp, _vp]),
    "hm_attn_decode_paged": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "hm_argmax": (_i32, [_vp, _i32, _i32, _vp, _vp]),
    "hm_dev_alloc": (_i32, [C.c_size_t, C.POINTER(_vp)]),
    "hm_dev_free": (_i32, [_vp]),
    "hm_dev_copy": (_i32, [_vp, _vp, C.c_size_t]),
    "hm_dev_sync": (_i32, []),
    "hm_dev_set": (_i32, [_i32]),
    "hm_dev_mem_info": (_i32, [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
}

_lib = None


def load_library() -> C.CDLL:
    """Load libhomura_b200.so.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("HOMURA_B200_LIB") or LIB_PATH  # e.g. the phase-trace build of `python -m homura_b200.build --trace`
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: build it with `python -m homura_b200.build` (nvcc, sm_100a)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _ptr(a) -> C.c_void_p:
    """numpy array, int device address or None -> void*."""
    if a is None:
        return C.c_void_p(None)
    if isinstance(a, np.ndarray):
        return a.ctypes.data_as(C.c_void_p)
    return C.c_void_p(int(a))


def _check(rc: int, handle=None):
    if rc == HM_OK:
        return
    lib = load_library()
    msg = (lib.hm_last_error(handle) if handle else lib.hm_last_error_global()) or b""
    cls = KvCacheFull if rc == HM_ERR_KV_FULL else HomuraError
    raise cls(rc, msg.decode(errors="replace"))


def device_count() -> int:
    return load_library().hm_device_count()


def checkpoint_info(path: str) -> dict:
    """Parse a model directory or .gguf file with the library's own loaders (host only)."""
    import json

    lib = load_library()
    need = C.c_size_t(0)
    rc = lib.hm_checkpoint_info(os.fsencode(path), None, 0, C.byref(need))
    if rc != HM_ERR_INVALID or need.value == 0:
        _check(rc)
    buf = C.create_string_buffer(need.value)
    _check(lib.hm_checkpoint_info(os.fsencode(path), buf, need.value, None))
    return json.loads(buf.value.decode())


# ---- TransformerConfig / SamplingConfig ---------------------------------------------------


@dataclass
class TransformerConfig:
    """src/hf/config.rs:11-73"""

    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_hidden_layers: int
    num_key_value_heads: Optional[int]
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 2048
    tie_word_embeddings: bool = False
    head_dim: Optional[int] = None
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    has_qkv_bias: bool = False
    has_qk_norm: bool = False
    weight_dtype: Optional[DType] = None

    def kv_heads(self) -> int:
        return self.num_key_value_heads or self.num_attention_heads

    def get_head_dim(self) -> int:
        return self.head_dim or self.hidden_size // self.num_attention_heads

    def gqa_repeat(self) -> int:
        return self.num_attention_heads // self.kv_heads()

    def _to_c(self) -> _Config:
        c = _Config()
        c.hidden_size, c.intermediate_size = self.hidden_size, self.intermediate_size
        c.num_attention_heads, c.num_hidden_layers = self.num_attention_heads, self.num_hidden_layers
        c.num_key_value_heads = self.kv_heads()
        c.vocab_size, c.max_position_embeddings = self.vocab_size, self.max_position_embeddings
        c.head_dim = self.get_head_dim()
        c.tie_word_embeddings = int(self.tie_word_embeddings)
        c.eos_token_id = 0xFFFFFFFF if self.eos_token_id is None else self.eos_token_id
        c.bos_token_id = 0xFFFFFFFF if self.bos_token_id is None else self.bos_token_id
        c.rms_norm_eps, c.rope_theta = self.rms_norm_eps, self.rope_theta
        return c

    @classmethod
    def _from_c(cls, c: _Config) -> "TransformerConfig":
        return cls(
            c.hidden_size, c.intermediate_size, c.num_attention_heads, c.num_hidden_layers, c.num_key_value_heads, c.vocab_size,
            c.rms_norm_eps, c.rope_theta, c.max_position_embeddings, bool(c.tie_word_embeddings), c.head_dim,
            None if c.eos_token_id == 0xFFFFFFFF else c.eos_token_id, None if c.bos_token_id == 0xFFFFFFFF else c.bos_token_id,
            bool(c.has_qkv_bias), bool(c.has_qk_norm), DType(c.weight_dtype) if c.weight_dtype >= 0 else None,
        )


@dataclass
class SamplingConfig:
    """src/generate.rs:648-683 (defaults included)."""

    temperature: float = 0.7
    top_k: int = 50
    top_p: float = 0.9
    min_p: float = 0.0
    repetition_penalty: float = 1.1
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    stop_sequences: List[str] = field(default_factory=list)
    seed: Optional[int] = None

    @classmethod
    def greedy(cls) -> "SamplingConfig":
        """temperature 0 with every penalty neutral: plain argmax."""
        return cls(temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0)

    def _to_c(self) -> _Sampling:
        return _Sampling(self.temperature, self.top_k, self.top_p, self.min_p, self.repetition_penalty, self.frequency_penalty, self.presence_penalty, int(self.seed is not None), self.seed or 0)


def sample_token(logits, config: SamplingConfig, generated_ids: Sequence[int], rng_state: int):
    """sample_token of src/generate.rs:698-801 on host logits.  Returns (token, new rng state)."""
    lib = load_library()
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    gen = np.ascontiguousarray(generated_ids, dtype=np.uint32)
    st = C.c_uint64(rng_state)
    out = C.c_uint32(0)
    cfg = config._to_c()
    _check(lib.hm_sample_token(_ptr(lg), lg.size, C.byref(cfg), _ptr(gen), gen.size, C.byref(st), C.byref(out)))
    return int(out.value), int(st.value)


def sample_token_device(logits, config: SamplingConfig, generated_ids: Sequence[int], rng_state: int):
    """The same sampler as one GPU kernel, every setting.  Returns (token, new rng state)."""
    lib = load_library()
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    gen = np.ascontiguousarray(generated_ids, dtype=np.uint32)
    st = C.c_uint64(rng_state)
    out = C.c_uint32(0)
    cfg = config._to_c()
    _check(lib.hm_sample_token_device(_ptr(lg), lg.size, C.byref(cfg), _ptr(gen) if gen.size else None, gen.size, C.byref(st), C.byref(out)))
    return int(out.value), int(st.value)


# ---- HfModel ----------------------------------------------------------------------------------


class HfModel:
    """A decoder-only RoPE transformer resident on one B200 (src/hf/model.rs:17-267)."""

    def __init__(self, handle: int):
        self._h = C.c_void_p(handle)
        self._lib = load_library()
        c = _Config()
        _check(self._lib.hm_get_config(self._h, C.byref(c)), self._h)
        self._config = TransformerConfig._from_c(c)
        self.batch = 0
        self.max_seq_len = 0

    # -- construction --
    @classmethod
    def load(cls, model_dir: str, device: int = 0) -> "HfModel":
        return cls.load_with_dtype(model_dir, DType.BF16, device)

    @classmethod
    def load_with_dtype(cls, model_dir: str, weight_dtype: DType = DType.BF16, device: int = 0) -> "HfModel":
        lib = load_library()
        h = C.c_void_p()
        _check(lib.hm_model_load(os.fsencode(model_dir), int(weight_dtype), device, C.byref(h)))
        return cls(h.value)

    @classmethod
    def load_gguf(cls, gguf_path: str, device: int = 0) -> "HfModel":
        lib = load_library()
        h = C.c_void_p()
        _check(lib.hm_model_load_gguf(os.fsencode(gguf_path), device, C.byref(h)))
        return cls(h.value)

    @classmethod
    def from_tensors(cls, config: TransformerConfig, tensors, device: int = 0) -> "HfModel":
        """tensors: iterable of (name, DType, shape, numpy array of raw bytes/values)."""
        lib = load_library()
        h = C.c_void_p()
        cc = config._to_c()
        _check(lib.hm_engine_create(C.byref(cc), device, C.byref(h)))
        try:
            for name, dt, shape, arr in tensors:
                arr = np.ascontiguousarray(arr)
                shp = (C.c_int64 * len(shape))(*shape)
                _check(lib.hm_load_tensor(h, name.encode(), int(dt), shp, len(shape), _ptr(arr), arr.nbytes), h)
            _check(lib.hm_finalize_weights(h), h)
        except Exception:
            lib.hm_engine_destroy(h)
            raise
        return cls(h.value)

    def close(self):
        if self._h:
            self._lib.hm_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- accessors --
    def config(self) -> TransformerConfig:
        return self._config

    def weight_bytes(self) -> int:
        v = C.c_uint64(0)
        _check(self._lib.hm_weight_bytes(self._h, C.byref(v)), self._h)
        return int(v.value)

    def launches_per_step(self) -> int:
        v = C.c_int(0)
        _check(self._lib.hm_launches_per_step(self._h, C.byref(v)), self._h)
        return v.value

    # -- KV cache --
    def init_kv_cache(self, max_seq_len: int, batch: int = 1, kv_dtype: DType = DType.F32, page_tokens: int = 16):
        """init_kv_cache (src/hf/model.rs:221-229).  Calling it again replaces the cache."""
        if self.batch:
            _check(self._lib.hm_kv_free(self._h), self._h)
            self.batch = 0
        _check(self._lib.hm_kv_alloc(self._h, batch, max_seq_len, page_tokens, int(kv_dtype)), self._h)
        self.batch, self.max_seq_len = batch, max_seq_len

    def reset_kv_cache(self, seq: int = -1):
        _check(self._lib.hm_kv_reset(self._h, seq), self._h)

    def kv_cache_len(self, seq: int = 0) -> int:
        v = C.c_int(0)
        _check(self._lib.hm_kv_len(self._h, seq, C.byref(v)), self._h)
        return v.value

    def kv_append(self, layer: int, k_rows, v_rows, seq: int = 0, advance: bool = False):
        """KvCache::append_key / append_value: rows [1, kv_heads, n_new, head_dim] f32."""
        k = None if k_rows is None else np.ascontiguousarray(k_rows, dtype=np.float32)
        v = None if v_rows is None else np.ascontiguousarray(v_rows, dtype=np.float32)
        n_new = (k if k is not None else v).shape[-2]
        _check(self._lib.hm_kv_append(self._h, seq, layer, _ptr(k), _ptr(v), n_new, int(advance)), self._h)

    def kv_advance_by(self, n: int, seq: int = 0):
        _check(self._lib.hm_kv_append(self._h, seq, 0, None, None, n, 1), self._h)

    def kv_view(self, layer: int, seq: int = 0):
        c = self._config
        n = self.kv_cache_len(seq)
        k = np.zeros((1, c.kv_heads(), n, c.get_head_dim()), np.float32)
        v = np.zeros_like(k)
        _check(self._lib.hm_kv_view(self._h, seq, layer, _ptr(k), _ptr(v)), self._h)
        return k, v

    # -- GenerativeModel --
    def prefill(self, token_ids, seq: int = 0, want_logits: bool = False):
        ids = np.ascontiguousarray(token_ids, dtype=np.int64)
        logits = np.empty(self._config.vocab_size, np.float32) if want_logits else None
        tok = C.c_uint32(0)
        _check(self._lib.hm_prefill(self._h, seq, _ptr(ids), ids.size, _ptr(logits), C.byref(tok)), self._h)
        return (int(tok.value), logits) if want_logits else int(tok.value)

    def decode_step(self, tokens, want_logits: bool = True):
        """One token per sequence in; ([batch, vocab] logits or None, greedy next tokens) out."""
        # the per-token call: addresses go in as plain integers (a few microseconds less than building ctypes pointers)
        t = tokens if (type(tokens) is np.ndarray and tokens.dtype == np.uint32 and tokens.ndim == 1 and tokens.flags.c_contiguous) else np.ascontiguousarray(np.atleast_1d(tokens), dtype=np.uint32)
        if t.size != self.batch:
            raise HomuraError(HM_ERR_INVALID, f"decode_step wants {self.batch} tokens, got {t.size}")
        logits = np.empty((self.batch, self._config.vocab_size), np.float32) if want_logits else None
        nxt = np.empty(self.batch, np.uint32)
        rc = self._lib.hm_decode_step(self._h, t.ctypes.data, logits.ctypes.data if want_logits else None, nxt.ctypes.data)
        if rc != HM_OK:
            _check(rc, self._h)
        return logits, nxt

    def decode_step_sampled(self, tokens, sampling: "SamplingConfig", rng_states, want_logits: bool = False):
        """decode_step + sample_token for every sequence.  rng_states: one xorshift64 word per sequence
        (numpy uint64 array, updated in place).  Returns ([batch, vocab] logits or None, sampled tokens)."""
        t = np.ascontiguousarray(np.atleast_1d(tokens), dtype=np.uint32)
        if t.size != self.batch or rng_states.size != self.batch or rng_states.dtype != np.uint64:
            raise HomuraError(HM_ERR_INVALID, f"decode_step_sampled wants {self.batch} tokens and uint64 RNG words")
        logits = np.empty((self.batch, self._config.vocab_size), np.float32) if want_logits else None
        nxt = np.empty(self.batch, np.uint32)
        sc = sampling._to_c()
        _check(self._lib.hm_decode_step_sampled(self._h, _ptr(t), C.byref(sc), _ptr(rng_states), _ptr(logits), _ptr(nxt)), self._h)
        return logits, nxt

    def decode_greedy_n(self, first_tokens, steps: int) -> np.ndarray:
        t = None if first_tokens is None else np.ascontiguousarray(np.atleast_1d(first_tokens), dtype=np.uint32)
        out = np.empty((self.batch, steps), np.uint32)
        _check(self._lib.hm_decode_greedy_n(self._h, _ptr(t), steps, _ptr(out)), self._h)
        return out

    def generate_ids(self, prompt_ids, max_new_tokens: int, sampling: Optional[SamplingConfig] = None, seq: int = 0) -> List[int]:
        """generate_streaming_core on token ids (src/generate.rs:100-315)."""
        ids = np.ascontiguousarray(prompt_ids, dtype=np.int64)
        out = np.empty(max(max_new_tokens, 1), np.uint32)
        n = C.c_int(0)
        sc = (sampling or SamplingConfig())._to_c()
        _check(self._lib.hm_generate(self._h, seq, _ptr(ids), ids.size, max_new_tokens, C.byref(sc), _ptr(out), C.byref(n)), self._h)
        return out[: n.value].tolist()

    def profile_decode(self, steps: int):
        """Per-kernel-class device time of the decode step (the HOMURA_PROFILE=1 table)."""
        arr = (_KernelStat * 16)()
        n = C.c_int(0)
        _check(self._lib.hm_profile_decode(self._h, steps, arr, 16, C.byref(n)), self._h)
        return [dict(name=arr[i].name.decode(), launches_per_step=arr[i].launches_per_step, ms_per_step=arr[i].ms_per_step, bytes_per_step=arr[i].bytes_per_step) for i in range(n.value)]

    def selftest_expire_wait(self):
        """Queue the bounded-wait probe: the next pass on this model raises HomuraError(HM_ERR_TIMEOUT)."""
        _check(self._lib.hm_selftest_expire_wait(self._h), self._h)

    def time_decode(self, warmup: int, steps: int) -> float:
        ms = C.c_float(0)
        _check(self._lib.hm_time_decode(self._h, warmup, steps, C.byref(ms)), self._h)
        return float(ms.value)


class HfGenerationContext:
    """trait GenerativeModel as implemented for HfModel (src/hf/model.rs:301-382), on token ids."""

    def __init__(self, model: HfModel, max_seq_len: int, eos_override: Optional[int] = None, kv_dtype: DType = DType.F32):
        self.model = model
        self._max_seq_len = max_seq_len
        self.eos_override = eos_override
        if model.batch == 0:
            model.init_kv_cache(max_seq_len, 1, kv_dtype)

    def prefill(self, token_ids):
        prior = self.model.kv_cache_len(0)
        first = self.model.prefill(token_ids, 0)
        return {"first_token": first, "prompt_len": len(token_ids), "real_pos": prior + len(token_ids)}

    def decode_step(self, token: int, real_pos: int = 0) -> np.ndarray:
        logits, _ = self.model.decode_step([token], want_logits=True)
        return logits[0]

    def eos_token_id(self) -> int:
        if self.eos_override is not None:
            return self.eos_override
        e = self.model.config().eos_token_id
        return 0xFFFFFFFF if e is None else e

    def max_seq_len(self) -> int:
        return self._max_seq_len


# ---- standalone kernels (numpy in, numpy out; device addresses accepted where noted) ---------


def gemv_bf16(x, w_bits, layout: int = LAYOUT_KN, K: Optional[int] = None, N: Optional[int] = None, y=None, stream=None):
    """y[M,N] = x[M,K] @ W.  Host mode: x float32 [M,K], w_bits uint16 ([K,N] or slab layout with
    K, N given).  Device mode: pass integer device addresses for x, w_bits, y and M, K, N via x=(addr, M)."""
    lib = load_library()
    if isinstance(x, tuple):
        (xa, M) = x
        _check(lib.hm_gemv_bf16(_ptr(xa), _ptr(w_bits), layout, M, K, N, _ptr(y), _ptr(stream)))
        return None
    x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
    M, Kx = x.shape
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    if layout == LAYOUT_KN:
        K, N = w.shape
    assert K == Kx
    out = np.empty((M, N), np.float32)
    _check(lib.hm_gemv_bf16(_ptr(x), _ptr(w), layout, M, K, N, _ptr(out), _ptr(stream)))
    return out


def gemv_bf16_noalloc(x_addr: int, w_addr: int, layout: int, M: int, K: int, N: int, y_addr: int, stream=None):
    """The projection for callers that may not allocate: device addresses only, scratch built
    into the library (see hm_gemv_bf16_noalloc in include/homura_b200.h for the limits)."""
    lib = load_library()
    _check(lib.hm_gemv_bf16_noalloc(_ptr(x_addr), _ptr(w_addr), layout, M, K, N, _ptr(y_addr), _ptr(stream)))


def pack_bf16_slabs(w_bits) -> np.ndarray:
    lib = load_library()
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    K, N = w.shape
    out = np.empty(((N + 127) // 128, K, 128), np.uint16)
    _check(lib.hm_pack_bf16_slabs(_ptr(w), K, N, _ptr(out), None))
    return out


def pack_bf16_tc(w_bits) -> np.ndarray:
    """Row-major [K, N] bf16 bit patterns -> the tensor-core tile layout (flat uint16 array)."""
    lib = load_library()
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    K, N = w.shape
    out = np.empty(int(lib.hm_tc_packed_elems(K, N)), np.uint16)
    _check(lib.hm_pack_bf16_tc(_ptr(w), K, N, _ptr(out), None))
    return out


def gemm_bf16_tc(x, w_tc, N: int, ksplit: int = 0, K: Optional[int] = None, y=None, stream=None):
    """y = x @ W for 1..64 rows on the tcgen05 path; `w_tc` comes from pack_bf16_tc.
    Device mode (asynchronous): x=(addr, M), w_tc and y integer device addresses, K given."""
    lib = load_library()
    if isinstance(x, tuple):
        (xa, M) = x
        _check(lib.hm_gemm_bf16_tc(_ptr(xa), _ptr(w_tc), M, K, N, int(ksplit), _ptr(y), _ptr(stream)))
        return None
    x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
    M, K = x.shape
    w = np.ascontiguousarray(w_tc, dtype=np.uint16)
    if w.size != int(lib.hm_tc_packed_elems(K, N)):
        raise ValueError("w_tc does not match a packed [K, N] weight")
    out = np.empty((M, N), np.float32)
    _check(lib.hm_gemm_bf16_tc(_ptr(x), _ptr(w), M, K, N, int(ksplit), _ptr(out), None))
    return out


def gemv_quant(x, blocks, dtype: DType, N: int):
    lib = load_library()
    x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
    M, K = x.shape
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.empty((M, N), np.float32)
    _check(lib.hm_gemv_quant(_ptr(x), _ptr(b), int(dtype), M, K, N, _ptr(out), None))
    return out


def dequant(blocks, dtype: DType) -> np.ndarray:
    lib = load_library()
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    bsz, vals = {DType.Q8_0: (34, 32), DType.Q4_0: (18, 32), DType.Q4_K: (144, 256), DType.Q6_K: (210, 256)}[DType(dtype)]
    nb = b.size // bsz
    out = np.empty(nb * vals, np.float32)
    _check(lib.hm_dequant(_ptr(b), int(dtype), nb, _ptr(out), None))
    return out


def rms_norm(x, w, eps: float) -> np.ndarray:
    lib = load_library()
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    n = x.shape[-1]
    out = np.empty_like(x)
    _check(lib.hm_rms_norm(_ptr(x), _ptr(w), eps, x.size // n, n, _ptr(out), None))
    return out


def qknorm_rope(x, cos_rows, sin_rows, norm_w=None, eps: float = 1e-6) -> np.ndarray:
    """x [rows, heads, hd] -> per-head RMSNorm (when norm_w is given) then RoPE half rotation."""
    lib = load_library()
    x = np.ascontiguousarray(x, dtype=np.float32).copy()
    rows, heads, hd = x.shape
    c = np.ascontiguousarray(cos_rows, dtype=np.float32)
    s = np.ascontiguousarray(sin_rows, dtype=np.float32)
    nw = None if norm_w is None else np.ascontiguousarray(norm_w, dtype=np.float32)
    _check(lib.hm_qknorm_rope(_ptr(x), rows, heads, hd, _ptr(nw), eps, _ptr(c), _ptr(s), None))
    return x


def argmax(logits) -> np.ndarray:
    lib = load_library()
    lg = np.ascontiguousarray(np.atleast_2d(logits), dtype=np.float32)
    out = np.empty(lg.shape[0], np.uint32)
    _check(lib.hm_argmax(_ptr(lg), lg.shape[0], lg.shape[1], _ptr(out), None))
    return out


class DeviceBuffer:
    """A raw device allocation (hm_dev_alloc) for HBM-resident measurements."""

    def __init__(self, nbytes: int):
        self._lib = load_library()
        p = C.c_void_p()
        _check(self._lib.hm_dev_alloc(nbytes, C.byref(p)))
        self.ptr = p.value
        self.nbytes = nbytes

    def upload(self, arr: np.ndarray, offset: int = 0):
        arr = np.ascontiguousarray(arr)
        _check(self._lib.hm_dev_copy(C.c_void_p(self.ptr + offset), _ptr(arr), arr.nbytes))

    def download(self, dtype, count: int, offset: int = 0) -> np.ndarray:
        out = np.empty(count, dtype)
        _check(self._lib.hm_dev_copy(_ptr(out), C.c_void_p(self.ptr + offset), out.nbytes))
        return out

    def free(self):
        if self.ptr:
            self._lib.hm_dev_free(C.c_void_p(self.ptr))
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def attn_decode_paged(q, k_pages: DeviceBuffer, v_pages: DeviceBuffer, kv_dtype: DType, page_table, kv_len, heads: int, kv_heads: int, hd: int, max_pages: int, page_tokens: int = 16) -> np.ndarray:
    lib = load_library()
    q = np.ascontiguousarray(q, dtype=np.float32)
    B = q.shape[0]
    pt = np.ascontiguousarray(page_table, dtype=np.int32)
    kl = np.ascontiguousarray(kv_len, dtype=np.int32)
    out = np.empty((B, heads * hd), np.float32)
    _check(lib.hm_attn_decode_paged(_ptr(q), C.c_void_p(k_pages.ptr), C.c_void_p(v_pages.ptr), int(kv_dtype), _ptr(pt), _ptr(kl), B, heads, kv_heads, hd, page_tokens, max_pages, _ptr(out), None))
    return out


def dev_sync():
    _check(load_library().hm_dev_sync())


def dev_set(device: int):
    """Make `device` current on this thread for DeviceBuffer and the standalone kernels."""
    _check(load_library().hm_dev_set(device))


def dev_mem_info():
    """(free, total) bytes of the current device."""
    f, t = C.c_size_t(0), C.c_size_t(0)
    _check(load_library().hm_dev_mem_info(C.byref(f), C.byref(t)))
    return int(f.value), int(t.value)
