"""Seeded synthetic tensors: random-field blocks for matvec sweeps and quantised N(0, σ) models.

No model file can be fetched offline and Yule has no quantiser, so every benchmark and test input is
generated here (``csrc/synth.cpp``).  Each value is a pure function of ``(seed, index)``.
"""

from __future__ import annotations

import ctypes as C
import zlib

import numpy as np

from . import _lib
from .dtype import DType
from .runner import ModelConfig

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)

# Shapes of the configs in BASELINE.json: Llama-architecture shapes only; weights are random.
TINYLLAMA = ModelConfig(dim=2048, n_layers=22, n_heads=32, n_kv_heads=4, head_dim=64, vocab_size=32000,
                        ff_dim=5632, max_seq_len=4096, norm_eps=1e-5, rope_freq_base=10000.0)
LLAMA3_8B = ModelConfig(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, head_dim=128, vocab_size=128256,
                        ff_dim=14336, max_seq_len=4096, norm_eps=1e-5, rope_freq_base=500000.0)
LLAMA3_70B = ModelConfig(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, head_dim=128, vocab_size=128256,
                         ff_dim=28672, max_seq_len=4096, norm_eps=1e-5, rope_freq_base=500000.0)


def tensor_seed(seed: int, name: str) -> int:
    """One 64-bit seed per tensor: a hash of (run seed, tensor name)."""
    return ((seed & 0xFFFFFFFF) << 32) | zlib.crc32(name.encode())


def normal(seed: int, n: int, mean: float = 0.0, std: float = 1.0, n_threads: int = 0) -> np.ndarray:
    out = np.empty(n, np.float32)
    _lib.synth_lib().ys_fill_normal(seed, mean, std, out.ctypes.data_as(_f32p), n, n_threads)
    return out


def tokens(seed: int, n: int, vocab: int) -> np.ndarray:
    out = np.empty(n, np.uint32)
    _lib.synth_lib().ys_fill_tokens(seed, vocab, out.ctypes.data_as(C.POINTER(C.c_uint32)), n)
    return out


def random_blocks(dtype: DType, seed: int, n_blocks: int, scale_std: float = 0.002, n_threads: int = 0) -> np.ndarray:
    """Blocks with random fields: f16 d (and dmin) = |N(0, scale_std)|, every other byte uniform 0..255."""
    out = np.empty(n_blocks * dtype.size_of_block, np.uint8)
    rc = _lib.synth_lib().ys_random_blocks(int(dtype), seed, scale_std, out.ctypes.data_as(_u8p), n_blocks, n_threads)
    assert rc == 0
    return out


def quantize(dtype: DType, x: np.ndarray, n_threads: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    assert x.size % dtype.block_size == 0
    out = np.empty(x.size // dtype.block_size * dtype.size_of_block, np.uint8)
    rc = _lib.synth_lib().ys_quantize(int(dtype), x.ctypes.data_as(_f32p), x.size, out.ctypes.data_as(_u8p), n_threads)
    assert rc == 0
    return out


def random_quantized(dtype: DType, seed: int, n_weights: int, std: float = 0.02, n_threads: int = 0,
                     first_weight: int = 0) -> np.ndarray:
    """N(0, std) weights quantised to ``dtype`` (generated block by block, no f32 copy kept): the weights at
    positions ``[first_weight, first_weight + n_weights)`` of the stream that ``seed`` defines, so a row shard
    generated on its own equals those rows of the whole tensor."""
    assert n_weights % dtype.block_size == 0 and first_weight % dtype.block_size == 0
    out = np.empty(n_weights // dtype.block_size * dtype.size_of_block, np.uint8)
    rc = _lib.synth_lib().ys_random_quantized_at(int(dtype), seed, std, out.ctypes.data_as(_u8p), first_weight,
                                                  n_weights, n_threads)
    assert rc == 0
    return out


ROW_SHARDED = ("attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight", "ffn_gate.weight",
               "ffn_up.weight", "ffn_down.weight", "output.weight")


def synthetic_model(cfg: ModelConfig, seed: int = 0, linear: DType = DType.Q4_K, ffn_down: DType | None = None,
                    output: DType | None = None, token_embd: DType | None = None, std: float = 0.02,
                    norm_dtype: DType = DType.F32, rank: int = 0, world: int = 1, packed_experts: bool = True,
                    router: DType = DType.F32) -> dict:
    """Random-init N(0, std) Llama-architecture weights as a GGUF-name → (bytes, DType) map.

    Norm weights are 1.0.  ``ffn_down`` / ``output`` / ``token_embd`` default to ``linear``.  With ``world`` > 1
    only this rank's output rows of every linear are generated (the same bytes as those rows of the
    ``world`` = 1 model); the embedding table and the norms are whole.
    """
    ffn_down = ffn_down or linear
    output = output or linear
    token_embd = token_embd or linear
    weights = {}
    for name, (rows, cols) in cfg.tensor_shapes(packed_experts).items():
        if name.endswith("ffn_gate_inp.weight"):
            # the router of a mixture-of-experts layer: F32 / F16 in model files (or any block format); a larger
            # spread than the linears so that the expert probabilities differ
            if router in (DType.F32, DType.F16):
                vals = normal(tensor_seed(seed, name), rows * cols) * np.float32(0.5)
                data = vals.view(np.uint8) if router == DType.F32 else vals.astype(np.float16).view(np.uint8)
                weights[name] = (data, router)
            else:
                weights[name] = (random_quantized(router, tensor_seed(seed, name), rows * cols, 0.5), router)
            continue
        if name == "token_embd.weight":
            dt = token_embd
        elif name == "output.weight":
            dt = output
        elif name.endswith("ffn_down.weight") or name.endswith("ffn_down_exps.weight") or ".ffn_down." in name:
            dt = ffn_down
        else:
            dt = linear
        if world > 1 and name.endswith(ROW_SHARDED):
            assert rows % world == 0
            local = rows // world
            weights[name] = (random_quantized(dt, tensor_seed(seed, name), local * cols, std, first_weight=rank * local * cols), dt)
        else:
            weights[name] = (random_quantized(dt, tensor_seed(seed, name), rows * cols, std), dt)
    for name in cfg.norm_names():
        ones = np.ones(cfg.dim, np.float32)
        if norm_dtype == DType.F16:
            weights[name] = (ones.astype(np.float16).view(np.uint8), DType.F16)
        else:
            weights[name] = (ones.view(np.uint8), DType.F32)
    return weights
