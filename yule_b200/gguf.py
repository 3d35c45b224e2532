"""GGUF v3 files over the C ABI: the reader (``yule_gguf_*``) and the loader that puts a model file's
tensors into HBM and returns a runner (``yule_cuda_runner_load_gguf``).

Mirrors ``GgufParser`` / ``GgufFile`` (yule-core/src/gguf.rs:240-620) and the weight upload of
``GpuTransformerRunner::new`` (yule-infer/src/gpu_runner.rs:86-254).  Parsing needs no GPU.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from .backend import CudaB200Backend, _check
from .dtype import DType
from .runner import CudaTransformerRunner, ModelConfig


@dataclass(frozen=True)
class GgufTensor:
    name: str
    shape: tuple[int, ...]   # GGUF order: shape[0] is the row length
    gguf_type: int
    offset: int              # from the start of the data section
    size_bytes: int


class GgufFile:
    """A parsed GGUF file.  ``GgufFile.open(path)`` maps the file; ``GgufFile.parse(bytes)`` parses an image."""

    def __init__(self, handle, keep_alive=None):
        self._lib = _lib.cuda_lib()
        self._g = handle
        self._keep = keep_alive
        ver, nt, nkv, off, al = C.c_uint32(), C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_uint64()
        _check(self._lib.yule_gguf_summary(self._g, C.byref(ver), C.byref(nt), C.byref(nkv), C.byref(off), C.byref(al)))
        self.version, self.n_tensors, self.n_kv = ver.value, nt.value, nkv.value
        self.data_offset, self.alignment = off.value, al.value

    @classmethod
    def open(cls, path: str) -> "GgufFile":
        g = C.c_void_p()
        _check(_lib.cuda_lib().yule_gguf_open(str(path).encode(), C.byref(g)))
        return cls(g)

    @classmethod
    def parse(cls, image) -> "GgufFile":
        buf = np.frombuffer(bytes(image), np.uint8).copy()  # kept alive with the object
        g = C.c_void_p()
        _check(_lib.cuda_lib().yule_gguf_parse(buf.ctypes.data_as(C.c_void_p), buf.size, C.byref(g)))
        return cls(g, keep_alive=buf)

    def close(self) -> None:
        if getattr(self, "_g", None):
            self._lib.yule_gguf_close(self._g)
            self._g = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensor(self, index: int) -> GgufTensor:
        info = _lib.GgufTensorInfo()
        _check(self._lib.yule_gguf_tensor(self._g, index, C.byref(info)))
        return GgufTensor(info.name.decode(), tuple(info.shape[i] for i in range(info.n_dims)), info.gguf_type,
                          info.offset, info.size_bytes)

    def tensors(self) -> list[GgufTensor]:
        return [self.tensor(i) for i in range(self.n_tensors)]

    def tensor_bytes(self, name: str) -> np.ndarray:
        """A copy of the tensor's raw bytes (``GgufFile::tensor_data``, gguf.rs:589-606)."""
        idx = C.c_uint64()
        _check(self._lib.yule_gguf_find_tensor(self._g, name.encode(), C.byref(idx)))
        info = _lib.GgufTensorInfo()
        _check(self._lib.yule_gguf_tensor(self._g, idx.value, C.byref(info)))
        return np.ctypeslib.as_array(C.cast(info.data, C.POINTER(C.c_uint8)), shape=(info.size_bytes,)).copy()

    def get_u32(self, key: str):
        v = C.c_uint32()
        return v.value if self._lib.yule_gguf_meta_u32(self._g, key.encode(), C.byref(v)) == 0 else None

    def get_f64(self, key: str):
        v = C.c_double()
        return v.value if self._lib.yule_gguf_meta_f64(self._g, key.encode(), C.byref(v)) == 0 else None

    def get_str(self, key: str):
        v = C.c_char_p()
        return v.value.decode() if self._lib.yule_gguf_meta_str(self._g, key.encode(), C.byref(v)) == 0 else None

    def model_config(self, max_seq_len: int = 0) -> ModelConfig:
        cfg = _lib.RunnerConfig()
        _check(self._lib.yule_gguf_runner_config(self._g, max_seq_len, C.byref(cfg)))
        return ModelConfig(dim=cfg.dim, n_layers=cfg.n_layers, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads,
                           head_dim=cfg.head_dim, vocab_size=cfg.vocab_size, ff_dim=cfg.ff_dim,
                           max_seq_len=cfg.max_seq_len, norm_eps=cfg.norm_eps, rope_freq_base=cfg.rope_freq_base,
                           rotary_dim=cfg.rotary_dim, sliding_window=cfg.sliding_window,
                           attn_logit_softcap=cfg.attn_logit_softcap, logit_softcap=cfg.logit_softcap,
                           norm_weight_offset=cfg.norm_weight_offset, geglu=bool(cfg.geglu),
                           n_experts=cfg.n_experts, n_experts_used=cfg.n_experts_used)


def load_runner(backend: CudaB200Backend, gguf: GgufFile, max_seq_len: int = 0, fused: bool = True) -> CudaTransformerRunner:
    """A runner whose weights come straight from the file image (pinned staging, asynchronous copies)."""
    r = C.c_void_p()
    _check(_lib.cuda_lib().yule_cuda_runner_load_gguf(backend._ctx, gguf._g, max_seq_len, 1 if fused else 0, C.byref(r)))
    run = CudaTransformerRunner.__new__(CudaTransformerRunner)
    run.backend = backend
    run.config = gguf.model_config(max_seq_len)
    run._lib = _lib.cuda_lib()
    run._r = r
    run._handles = {}  # the device buffers belong to the native runner
    run.weight_bytes = sum(t.size_bytes for t in gguf.tensors())
    backend.synchronize()
    return run


__all__ = ["GgufFile", "GgufTensor", "load_runner", "DType"]
