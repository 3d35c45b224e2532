"""Host-side mirror of Yule's GPU forward-pass runner over the C ABI.

``CudaTransformerRunner`` plays the part of ``GpuTransformerRunner`` (yule-infer/src/gpu_runner.rs:72-720)
behind the ``ModelRunner`` trait (yule-infer/src/model_runner.rs:12-17): it uploads every tensor as raw
GGUF bytes (gpu_runner.rs:171-254) and exposes ``prefill`` / ``decode_step`` / ``reset``.  The forward
pass itself runs inside ``libyule_cuda.so``.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from .backend import BufferHandle, CudaB200Backend, _check
from .dtype import DType


@dataclass(frozen=True)
class ModelConfig:
    """The fields of ``GpuConfig`` (yule-infer/src/gpu_runner.rs:13-25) the Llama path uses."""
    dim: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    vocab_size: int
    ff_dim: int
    max_seq_len: int = 4096
    norm_eps: float = 1e-5
    rope_freq_base: float = 10000.0
    # architecture variants of the CPU runner's dense path (yule-infer/src/model_runner.rs:417-460); zero = Llama
    rotary_dim: int = 0
    sliding_window: int = 0
    attn_logit_softcap: float = 0.0
    logit_softcap: float = 0.0
    norm_weight_offset: float = 0.0
    geglu: bool = False
    # mixture of experts (model_runner.rs:395-397, 813-958): experts per layer (0 = dense FFN), experts used per token
    n_experts: int = 0
    n_experts_used: int = 0

    def tensor_shapes(self, packed_experts: bool = True) -> dict[str, tuple[int, int]]:
        """GGUF tensor name → (rows, cols) for every matrix the runner reads (gpu_runner.rs:213-222); for a
        mixture-of-experts model the router and the experts, packed (one tensor per projection holding all experts'
        rows) or one tensor per expert (weight_loader.rs:222-260)."""
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        shapes = {"token_embd.weight": (self.vocab_size, self.dim), "output.weight": (self.vocab_size, self.dim)}
        for l in range(self.n_layers):
            p = f"blk.{l}."
            shapes[p + "attn_q.weight"] = (q, self.dim)
            shapes[p + "attn_k.weight"] = (kv, self.dim)
            shapes[p + "attn_v.weight"] = (kv, self.dim)
            shapes[p + "attn_output.weight"] = (self.dim, q)
            if self.n_experts == 0:
                shapes[p + "ffn_gate.weight"] = (self.ff_dim, self.dim)
                shapes[p + "ffn_up.weight"] = (self.ff_dim, self.dim)
                shapes[p + "ffn_down.weight"] = (self.dim, self.ff_dim)
            else:
                shapes[p + "ffn_gate_inp.weight"] = (self.n_experts, self.dim)
                if packed_experts:
                    shapes[p + "ffn_gate_exps.weight"] = (self.n_experts * self.ff_dim, self.dim)
                    shapes[p + "ffn_up_exps.weight"] = (self.n_experts * self.ff_dim, self.dim)
                    shapes[p + "ffn_down_exps.weight"] = (self.n_experts * self.dim, self.ff_dim)
                else:
                    for e in range(self.n_experts):
                        shapes[p + f"ffn_gate.{e}.weight"] = (self.ff_dim, self.dim)
                        shapes[p + f"ffn_up.{e}.weight"] = (self.ff_dim, self.dim)
                        shapes[p + f"ffn_down.{e}.weight"] = (self.dim, self.ff_dim)
        return shapes

    def norm_names(self) -> list[str]:
        names = ["output_norm.weight"]
        for l in range(self.n_layers):
            names += [f"blk.{l}.attn_norm.weight", f"blk.{l}.ffn_norm.weight"]
        return names


class CudaTransformerRunner:
    """``ModelRunner`` over the CUDA backend.

    ``weights`` maps GGUF tensor names to ``(bytes-like or uint8/float array, DType)``.  ``fused=False``
    issues one kernel per reference dispatch; ``fused=True`` replays fused kernels from a CUDA graph; ``fused=2``
    additionally runs the token step as one persistent kernel where the model allows it (``step_kind`` tells).
    """

    def __init__(self, backend: CudaB200Backend, config: ModelConfig, weights: dict, fused: bool = True):
        self.backend = backend
        self.config = config
        self._lib = _lib.cuda_lib()
        cfg = _lib.RunnerConfig(config.dim, config.n_layers, config.n_heads, config.n_kv_heads, config.head_dim,
                                config.vocab_size, config.ff_dim, config.max_seq_len, config.norm_eps,
                                config.rope_freq_base, int(fused), config.rotary_dim, config.sliding_window,
                                config.attn_logit_softcap, config.logit_softcap, config.norm_weight_offset,
                                1 if config.geglu else 0, config.n_experts, config.n_experts_used)
        r = C.c_void_p()
        _check(self._lib.yule_cuda_runner_create(backend._ctx, C.byref(cfg), C.byref(r)))
        self._r = r
        backend._runners.add(self)
        self._handles: dict[str, BufferHandle] = {}
        self.weight_bytes = 0
        for name, (data, dtype) in weights.items():
            arr = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
            h = backend.allocate(arr.nbytes)
            backend.copy_to_device(arr, h)
            self._handles[name] = h
            self.weight_bytes += arr.nbytes
            _check(self._lib.yule_cuda_runner_set_tensor(self._r, name.encode(), h.id, int(dtype)))
        backend.synchronize()

    def close(self) -> None:
        r, self._r = getattr(self, "_r", None), None  # at most one destroy, whatever the frees below raise
        if r:
            handles, self._handles = self._handles, {}
            if getattr(self.backend, "_ctx", None):  # the context takes its runners with it (backend.close)
                self._lib.yule_cuda_runner_destroy(r)
                for h in handles.values():
                    self.backend.free(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ── ModelRunner ────────────────────────────────────────────────────────────────────────
    def prefill(self, tokens) -> np.ndarray:
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits = np.empty(self.config.vocab_size, np.float32)
        _check(self._lib.yule_cuda_runner_prefill(self._r, toks.ctypes.data_as(C.POINTER(C.c_uint32)), toks.size,
                                                  logits.ctypes.data_as(C.POINTER(C.c_float))))
        return logits

    def decode_step(self, token: int, out: np.ndarray | None = None) -> np.ndarray:
        logits = out if out is not None else np.empty(self.config.vocab_size, np.float32)
        _check(self._lib.yule_cuda_runner_decode_step(self._r, int(token), logits.ctypes.data_as(C.POINTER(C.c_float))))
        return logits

    def reset(self) -> None:
        _check(self._lib.yule_cuda_runner_reset(self._r))

    # ── additive ───────────────────────────────────────────────────────────────────────────
    @property
    def pos(self) -> int:
        p = C.c_uint32()
        _check(self._lib.yule_cuda_runner_position(self._r, C.byref(p)))
        return p.value

    @property
    def step_kind(self) -> int:
        """0: one kernel per dispatch; 1: fused kernels in a CUDA graph; 2: one persistent kernel per token."""
        k = C.c_uint32()
        _check(self._lib.yule_cuda_runner_step_kind(self._r, C.byref(k)))
        return k.value

    def selftest_bounded_wait(self, budget_cycles: int = 0) -> int:
        """Runs the persistent token kernel once with waits that cannot be satisfied; returns the error code
        (``YULE_ERR_DEVICE_STATUS`` is the expected one).  Reset the runner afterwards."""
        return int(self._lib.yule_cuda_runner_selftest_bounded_wait(self._r, int(budget_cycles)))

    def generate_greedy(self, prompt, n_generate: int) -> np.ndarray:
        """Feed ``prompt`` (may be empty to continue), then emit ``n_generate`` greedy tokens on the device."""
        toks = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.empty(max(n_generate, 1), np.uint32)
        _check(self._lib.yule_cuda_runner_generate_greedy(
            self._r, toks.ctypes.data_as(C.POINTER(C.c_uint32)), toks.size, n_generate,
            out.ctypes.data_as(C.POINTER(C.c_uint32))))
        return out[:n_generate]

    def generate_sampled(self, prompt, n_generate: int, seed: int, *, temperature: float = 0.7, top_p: float = 0.9,
                         top_k: int = 40, repetition_penalty: float = 1.1, min_p: float = 0.05) -> np.ndarray:
        """Feed ``prompt`` (the runner must be at position 0), then emit ``n_generate`` tokens picked by the
        device sampler; pick ``g`` uses ``random_value(seed, g)``."""
        toks = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.empty(max(n_generate, 1), np.uint32)
        params = _lib.SamplingParams(temperature, top_p, top_k, repetition_penalty, min_p)
        _check(self._lib.yule_cuda_runner_generate_sampled(
            self._r, toks.ctypes.data_as(C.POINTER(C.c_uint32)), toks.size, n_generate, C.byref(params), seed,
            out.ctypes.data_as(C.POINTER(C.c_uint32))))
        return out[:n_generate]

    @staticmethod
    def random_value(seed: int, index: int) -> float:
        return float(_lib.cuda_lib().yule_cuda_sampling_random_value(seed, index))

    # ── batched decode: independent sequences advancing together ───────────────────────────
    def decode_batch(self, tokens) -> np.ndarray:
        """One new token for each of ``len(tokens)`` sequences (each with its own KV caches and position);
        returns the logits ``[batch][vocab_size]``.  The first call fixes the batch size."""
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits = np.empty((toks.size, self.config.vocab_size), np.float32)
        _check(self._lib.yule_cuda_runner_decode_batch(self._r, toks.ctypes.data_as(C.POINTER(C.c_uint32)), toks.size,
                                                       logits.ctypes.data_as(C.POINTER(C.c_float))))
        return logits

    def reset_batch(self) -> None:
        _check(self._lib.yule_cuda_runner_reset_batch(self._r))

    def generate_greedy_batch(self, prompts, n_generate: int) -> np.ndarray:
        """``prompts`` is ``[batch][n_prompt]`` (equal lengths); returns ``[batch][n_generate]`` greedy tokens,
        picked on the device."""
        p = np.ascontiguousarray(prompts, dtype=np.uint32)
        assert p.ndim == 2
        out = np.empty((p.shape[0], max(n_generate, 1)), np.uint32)
        _check(self._lib.yule_cuda_runner_generate_greedy_batch(
            self._r, p.ctypes.data_as(C.POINTER(C.c_uint32)), p.shape[0], p.shape[1], n_generate,
            out.ctypes.data_as(C.POINTER(C.c_uint32))))
        return out[:, :n_generate] if n_generate else out[:, :0]

    def buffer(self, which: str, layer: int = 0) -> BufferHandle:
        sel = {"hidden": 0, "k_cache": 1, "v_cache": 2, "logits": 3}[which]
        h = C.c_uint64()
        _check(self._lib.yule_cuda_runner_buffer(self._r, sel, layer, C.byref(h)))
        return BufferHandle(h.value)
