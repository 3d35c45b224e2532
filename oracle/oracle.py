"""ctypes binding of the CPU oracle (``libyule_oracle.so``) — TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this module;
the shipped package never does.  Each wrapper forwards to the C function of the same name, whose
header comment cites the Yule source lines it restates.
"""

from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build_oracle as _build

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K = 0, 1, 2, 8, 12, 14
SCALAR, AVX2, AVX2_ASM = 0, 1, 2

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)


class ModelConfig(C.Structure):
    _fields_ = [
        ("dim", C.c_uint32), ("n_layers", C.c_uint32), ("n_heads", C.c_uint32),
        ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("vocab_size", C.c_uint32),
        ("ff_dim", C.c_uint32), ("max_seq_len", C.c_uint32),
        ("norm_eps", C.c_float), ("rope_freq_base", C.c_float),
        ("mod_enabled", C.c_int32), ("simd", C.c_int32), ("n_threads", C.c_int32),
        ("rotary_dim", C.c_uint32), ("sliding_window", C.c_uint32), ("attn_logit_softcap", C.c_float),
        ("logit_softcap", C.c_float), ("norm_weight_offset", C.c_float), ("geglu", C.c_int32),
        ("n_experts", C.c_uint32), ("n_experts_used", C.c_uint32),
    ]


def _load() -> C.CDLL:
    so = _build.build_oracle()
    lib = C.CDLL(so)
    lib.yo_f16_to_f32.restype = C.c_float
    lib.yo_f16_to_f32.argtypes = [C.c_uint16]
    for name in ("q4_0", "q8_0", "q4_k", "q6_k", "q4_1", "q5_0", "q5_1", "q8_1", "q2_k", "q3_k", "q5_k"):
        f = getattr(lib, "yo_vec_dot_" + name)
        f.restype = C.c_float
        f.argtypes = [_u8p, _f32p]
        g = getattr(lib, "yo_dequant_" + name)
        g.restype = None
        g.argtypes = [_u8p, _f32p]
    for name in ("yo_vec_dot_q8_0_avx2", "yo_vec_dot_q4_0_avx2", "yo_vec_dot_q4_k_avx2_rust",
                 "yo_vec_dot_q6_k_avx2"):
        f = getattr(lib, name)
        f.restype = C.c_float
        f.argtypes = [_u8p, _f32p]
    lib.yo_extract_q4k_scales_mins.argtypes = [_u8p, _u8p, _u8p]
    lib.yo_dequant_tensor.argtypes = [C.c_int, _u8p, C.c_size_t, _f32p]
    lib.yo_vec_dot_block.argtypes = [C.c_int, _u8p, _f32p, C.c_int, _f32p]
    lib.yo_qmv.argtypes = [C.c_int, _u8p, _f32p, _f32p, C.c_size_t, C.c_size_t, C.c_int, C.c_int]
    lib.yo_rms_norm.argtypes = [_f32p, _f32p, C.c_size_t, C.c_float, C.c_float, _f32p]
    lib.yo_rms_norm.restype = None
    lib.yo_rope_table.argtypes = [C.c_size_t, C.c_size_t, C.c_float, _f32p, _f32p]
    lib.yo_rope_table.restype = None
    lib.yo_apply_rope.argtypes = [_f32p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, _f32p, _f32p]
    lib.yo_apply_rope.restype = None
    lib.yo_softmax.argtypes = [_f32p, C.c_size_t]
    lib.yo_softmax.restype = None
    lib.yo_attention.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p] + [C.c_size_t] * 4
    lib.yo_attention.restype = None
    lib.yo_attention_ex.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p] + [C.c_size_t] * 5 + [C.c_float]
    lib.yo_attention_ex.restype = None
    lib.yo_ct_gte.argtypes = [C.c_float, C.c_float]
    lib.yo_ct_gte.restype = C.c_float
    lib.yo_sample_ct.argtypes = [_f32p, C.c_size_t, C.c_float]
    lib.yo_sample_ct.restype = C.c_uint32
    lib.yo_sample.argtypes = [_f32p, C.c_size_t, C.c_float, C.c_float, C.c_uint32, C.c_float, C.c_float,
                              C.POINTER(C.c_uint32), C.c_size_t, C.c_float]
    lib.yo_sample.restype = C.c_int64
    lib.yo_gelu.argtypes = [C.c_float]
    lib.yo_gelu.restype = C.c_float
    lib.yo_moe_route.argtypes = [_f32p, C.c_size_t, C.c_size_t, C.POINTER(C.c_uint32), _f32p]
    lib.yo_moe_route.restype = None
    lib.yo_swiglu.argtypes = [_f32p, _f32p, C.c_size_t]
    lib.yo_swiglu.restype = None
    lib.yo_argmax.argtypes = [_f32p, C.c_size_t]
    lib.yo_argmax.restype = C.c_uint32
    lib.yo_set_q4k_asm.argtypes = [C.c_void_p]
    lib.yo_set_q4k_asm.restype = None
    lib.yo_model_create.argtypes = [C.POINTER(ModelConfig)]
    lib.yo_model_create.restype = C.c_void_p
    lib.yo_model_destroy.argtypes = [C.c_void_p]
    lib.yo_model_destroy.restype = None
    lib.yo_model_set_tensor.argtypes = [C.c_void_p, C.c_char_p, _u8p, C.c_size_t, C.c_int]
    lib.yo_model_forward.argtypes = [C.c_void_p, C.c_uint32, _f32p]
    lib.yo_model_reset.argtypes = [C.c_void_p]
    lib.yo_model_reset.restype = None
    lib.yo_model_pos.argtypes = [C.c_void_p]
    lib.yo_model_pos.restype = C.c_uint32
    lib.yo_model_layers_skipped.argtypes = [C.c_void_p]
    lib.yo_model_layers_skipped.restype = C.c_uint64
    lib.yo_model_hidden.argtypes = [C.c_void_p]
    lib.yo_model_hidden.restype = _f32p
    lib.yo_model_k_cache.argtypes = [C.c_void_p, C.c_uint32]
    lib.yo_model_k_cache.restype = _f32p
    lib.yo_model_v_cache.argtypes = [C.c_void_p, C.c_uint32]
    lib.yo_model_v_cache.restype = _f32p
    return lib


lib = _load()
_ref_lib = None


def load_reference_asm() -> bool:
    """Load Yule's own q4k_gemv_avx2 object from ``oracle/_ref`` and register it with the oracle.

    Returns False when the object is not there (no Yule checkout was reachable at build time).
    """
    global _ref_lib
    if _ref_lib is not None:
        return True
    so = _build.build_ref()
    if so is None or not os.path.exists(so) or not lib.yo_have_avx2():
        return False
    _ref_lib = C.CDLL(so)
    _ref_lib.yule_q4k_gemv_avx2.restype = C.c_float
    _ref_lib.yule_q4k_gemv_avx2.argtypes = [_u8p, _f32p]
    lib.yo_set_q4k_asm(C.cast(_ref_lib.yule_q4k_gemv_avx2, C.c_void_p))
    return True


def reference_q4k_asm(block: np.ndarray, act: np.ndarray) -> float:
    """Call Yule's assembly kernel directly on one 144-byte block and 256 activations."""
    assert load_reference_asm()
    block = np.ascontiguousarray(block, dtype=np.uint8)
    act = np.ascontiguousarray(act, dtype=np.float32)
    assert block.size >= 144 and act.size >= 256
    return float(_ref_lib.yule_q4k_gemv_avx2(_u8(block), _f32(act)))


def _u8(a: np.ndarray):
    return a.ctypes.data_as(_u8p)


def _f32(a: np.ndarray):
    return a.ctypes.data_as(_f32p)


def block_size(t: int) -> int:
    return lib.yo_block_size(t)


def block_bytes(t: int) -> int:
    return lib.yo_block_bytes(t)


def f16_to_f32(bits: int) -> np.float32:
    return np.float32(lib.yo_f16_to_f32(bits))


def extract_q4k_scales_mins(q12: np.ndarray):
    q12 = np.ascontiguousarray(q12, dtype=np.uint8)
    sc = np.zeros(8, np.uint8)
    mn = np.zeros(8, np.uint8)
    lib.yo_extract_q4k_scales_mins(_u8(q12), _u8(sc), _u8(mn))
    return sc, mn


def dequant(t: int, data: np.ndarray) -> np.ndarray:
    """Dequantise a whole tensor of raw GGUF blocks to f32 (dequant_block per block)."""
    data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    bb, bs = block_bytes(t), block_size(t)
    assert bb and data.size % bb == 0
    n = data.size // bb
    out = np.empty(n * bs, np.float32)
    assert lib.yo_dequant_tensor(t, _u8(data), n, _f32(out)) == 0
    return out


def vec_dot(t: int, block: np.ndarray, act: np.ndarray, simd: int = SCALAR) -> np.float32:
    block = np.ascontiguousarray(block, dtype=np.uint8)
    act = np.ascontiguousarray(act, dtype=np.float32)
    out = C.c_float()
    assert lib.yo_vec_dot_block(t, _u8(block), _f32(act), simd, C.byref(out)) == 0
    return np.float32(out.value)


def qmv(t: int, w: np.ndarray, x: np.ndarray, n_rows: int, n_cols: int, simd: int = SCALAR,
        n_threads: int = 0) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    assert x.size == n_cols and w.size == n_rows * (n_cols // block_size(t)) * block_bytes(t)
    out = np.empty(n_rows, np.float32)
    assert lib.yo_qmv(t, _u8(w), _f32(x), _f32(out), n_rows, n_cols, n_threads, simd) == 0
    return out


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float, offset: float = 0.0) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    out = np.empty_like(x)
    lib.yo_rms_norm(_f32(x), _f32(w), x.size, eps, offset, _f32(out))
    return out


def rope_table(max_seq_len: int, rotary_dim: int, freq_base: float):
    half = rotary_dim // 2
    cos = np.empty(max_seq_len * half, np.float32)
    sin = np.empty(max_seq_len * half, np.float32)
    lib.yo_rope_table(max_seq_len, rotary_dim, freq_base, _f32(cos), _f32(sin))
    return cos, sin


def apply_rope(vec: np.ndarray, pos: int, head_dim: int, cos: np.ndarray, sin: np.ndarray,
               rotary_dim: int = 0) -> np.ndarray:
    """``rotary_dim`` (0 = head_dim) is the dimension the table was built for: only that prefix of each head turns."""
    out = np.array(vec, dtype=np.float32, copy=True)
    lib.yo_apply_rope(_f32(out), out.size, pos, head_dim, (rotary_dim or head_dim) // 2, _f32(cos), _f32(sin))
    return out


def softmax(s: np.ndarray) -> np.ndarray:
    out = np.array(s, dtype=np.float32, copy=True)
    lib.yo_softmax(_f32(out), out.size)
    return out


def attention(q, k_cache, v_cache, n_heads, n_kv_heads, head_dim, seq_len, sliding_window: int = 0,
              softcap: float = 0.0) -> np.ndarray:
    q = np.ascontiguousarray(q, np.float32)
    k_cache = np.ascontiguousarray(k_cache, np.float32)
    v_cache = np.ascontiguousarray(v_cache, np.float32)
    out = np.zeros(n_heads * head_dim, np.float32)
    scratch = np.zeros(max(seq_len, 1), np.float32)
    lib.yo_attention_ex(_f32(q), _f32(k_cache), _f32(v_cache), _f32(out), _f32(scratch), n_heads,
                        n_kv_heads, head_dim, seq_len, sliding_window, softcap)
    return out


def ct_gte(a: float, b: float) -> float:
    return float(lib.yo_ct_gte(a, b))


def sample_ct(probs: np.ndarray, r: float) -> int:
    probs = np.ascontiguousarray(probs, np.float32)
    return int(lib.yo_sample_ct(_f32(probs), probs.size, r))


def sample(logits: np.ndarray, r: float, temperature: float = 0.7, top_p: float = 0.9, top_k: int = 40,
           min_p: float = 0.05, repetition_penalty: float = 1.1, previous=()) -> int:
    """Sampler::sample_with_history with the random value ``r`` given (defaults: SamplingParams::default,
    yule-infer/src/lib.rs:74-84)."""
    logits = np.ascontiguousarray(logits, np.float32)
    prev = np.ascontiguousarray(previous, np.uint32)
    return int(lib.yo_sample(_f32(logits), logits.size, temperature, top_p, top_k, min_p, repetition_penalty,
                             prev.ctypes.data_as(C.POINTER(C.c_uint32)), prev.size, r))


def gelu(x: float) -> float:
    return float(lib.yo_gelu(x))


def moe_route(logits, n_used: int):
    """Router of the mixture-of-experts FFN (model_runner.rs:827-854): returns (probabilities, selected experts in
    order of decreasing probability, their renormalised weights)."""
    probs = np.ascontiguousarray(logits, dtype=np.float32).copy()
    sel = np.empty(n_used, np.uint32)
    w = np.empty(n_used, np.float32)
    lib.yo_moe_route(_f32(probs), probs.size, n_used, sel.ctypes.data_as(C.POINTER(C.c_uint32)), _f32(w))
    return probs, sel, w


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    out = np.array(gate, dtype=np.float32, copy=True)
    up = np.ascontiguousarray(up, np.float32)
    lib.yo_swiglu(_f32(out), _f32(up), out.size)
    return out


def argmax(v: np.ndarray) -> int:
    v = np.ascontiguousarray(v, np.float32)
    return int(lib.yo_argmax(_f32(v), v.size))


class Model:
    """TransformerRunner restated (forward / prefill / decode_step / reset)."""

    def __init__(self, *, dim, n_layers, n_heads, n_kv_heads, head_dim, vocab_size, ff_dim,
                 max_seq_len, norm_eps=1e-5, rope_freq_base=10000.0, mod_enabled=-1, simd=SCALAR,
                 n_threads=0, rotary_dim=0, sliding_window=0, attn_logit_softcap=0.0, logit_softcap=0.0,
                 norm_weight_offset=0.0, geglu=False, n_experts=0, n_experts_used=0):
        if simd == AVX2_ASM and not load_reference_asm():
            simd = AVX2
        self.simd = simd
        self.cfg = ModelConfig(dim, n_layers, n_heads, n_kv_heads, head_dim, vocab_size, ff_dim,
                               max_seq_len, norm_eps, rope_freq_base, mod_enabled, simd, n_threads,
                               rotary_dim, sliding_window, attn_logit_softcap, logit_softcap, norm_weight_offset,
                               1 if geglu else 0, n_experts, n_experts_used)
        self._m = lib.yo_model_create(C.byref(self.cfg))
        self._keep = {}

    def set_tensor(self, name: str, data: np.ndarray, t: int) -> None:
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        self._keep[name] = data
        rc = lib.yo_model_set_tensor(self._m, name.encode(), _u8(data), data.size, t)
        if rc != 0:
            raise KeyError(name)

    def forward(self, token: int) -> np.ndarray:
        logits = np.empty(self.cfg.vocab_size, np.float32)
        rc = lib.yo_model_forward(self._m, token, _f32(logits))
        if rc == -2:
            raise RuntimeError("context length exceeded")
        if rc != 0:
            raise RuntimeError("oracle forward failed (missing tensor?)")
        return logits

    def prefill(self, tokens) -> np.ndarray:
        logits = None
        for t in tokens:
            logits = self.forward(int(t))
        return logits

    decode_step = forward

    def reset(self) -> None:
        lib.yo_model_reset(self._m)

    @property
    def pos(self) -> int:
        return lib.yo_model_pos(self._m)

    @property
    def layers_skipped(self) -> int:
        return lib.yo_model_layers_skipped(self._m)

    def hidden(self) -> np.ndarray:
        return np.ctypeslib.as_array(lib.yo_model_hidden(self._m), (self.cfg.dim,)).copy()

    def k_cache(self, layer: int, n_pos: int) -> np.ndarray:
        n = n_pos * self.cfg.n_kv_heads * self.cfg.head_dim
        return np.ctypeslib.as_array(lib.yo_model_k_cache(self._m, layer), (n,)).copy()

    def v_cache(self, layer: int, n_pos: int) -> np.ndarray:
        n = n_pos * self.cfg.n_kv_heads * self.cfg.head_dim
        return np.ctypeslib.as_array(lib.yo_model_v_cache(self._m, layer), (n,)).copy()

    def __del__(self):
        if getattr(self, "_m", None):
            lib.yo_model_destroy(self._m)
            self._m = None
