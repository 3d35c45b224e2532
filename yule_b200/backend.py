"""Host-side mirror of Yule's ``ComputeBackend`` trait (yule-gpu/src/lib.rs:21-132) over the C ABI.

Method names, argument order and meaning follow the trait; failures raise :class:`YuleGpuError`
(the counterpart of ``YuleError::Gpu(String)``, yule-core/src/error.rs:44).  Buffers are opaque
:class:`BufferHandle` values exactly as in lib.rs:135.  Host data crosses as ``bytes``-like objects
or numpy arrays.  All compute runs in ``libyule_cuda.so``; nothing here computes on the CPU.
"""

from __future__ import annotations

import ctypes as C
import weakref
from dataclasses import dataclass

import numpy as np

from . import _lib
from .dtype import DType


class YuleGpuError(RuntimeError):
    """``YuleError::Gpu`` — carries the library's status code and message."""

    def __init__(self, code: int, message: str):
        super().__init__(f"GPU error: {message}")
        self.code = code
        self.message = message


@dataclass(frozen=True)
class BufferHandle:
    """``BufferHandle(pub u64)`` (yule-gpu/src/lib.rs:135)."""
    id: int


@dataclass(frozen=True)
class DeviceInfo:
    """``DeviceInfo`` (yule-gpu/src/lib.rs:138-143)."""
    name: str
    backend: str
    memory_bytes: int
    compute_units: int


def is_available() -> bool:
    """``CudaBackend::is_available`` (yule-gpu/src/cuda/mod.rs:39-41)."""
    return bool(_lib.cuda_lib().yule_cuda_is_available())


def _check(rc: int) -> None:
    if rc != 0:
        msg = _lib.cuda_lib().yule_cuda_last_error()
        raise YuleGpuError(rc, msg.decode("utf-8", "replace") if msg else f"status {rc}")


def _host_ptr(data) -> tuple[C.c_void_p, int, object]:
    """(pointer, byte length, keep-alive) of a bytes-like object or numpy array."""
    if isinstance(data, np.ndarray):
        arr = np.ascontiguousarray(data)
        return C.c_void_p(arr.ctypes.data), arr.nbytes, arr
    mv = memoryview(data)
    arr = np.frombuffer(mv, dtype=np.uint8)
    return C.c_void_p(arr.ctypes.data), arr.nbytes, arr


class CudaB200Backend:
    """``impl ComputeBackend for CudaBackend`` (yule-gpu/src/cuda/mod.rs:43-329), B200 edition."""

    def __init__(self, device: int = 0):
        self._lib = _lib.cuda_lib()
        ctx = C.c_void_p()
        _check(self._lib.yule_cuda_create(device, C.byref(ctx)))
        self._ctx = ctx
        self._runners = weakref.WeakSet()  # runners created on this context: destroyed before it

    def close(self) -> None:
        if getattr(self, "_ctx", None):
            # A runner holds a pointer to the context: one left open (an exception between its creation and its
            # close) must not outlive it.
            for run in list(self._runners):
                run.close()
            self._lib.yule_cuda_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ── trait methods ──────────────────────────────────────────────────────────────────────
    def name(self) -> str:
        return "cuda"

    def device_info(self) -> DeviceInfo:
        buf = C.create_string_buffer(256)
        mem, cu = C.c_uint64(), C.c_uint32()
        _check(self._lib.yule_cuda_device_info(self._ctx, buf, 256, C.byref(mem), C.byref(cu)))
        return DeviceInfo(buf.value.decode(), "Cuda", mem.value, cu.value)

    def allocate(self, size_bytes: int) -> BufferHandle:
        h = C.c_uint64()
        _check(self._lib.yule_cuda_allocate(self._ctx, size_bytes, C.byref(h)))
        return BufferHandle(h.value)

    def free(self, handle: BufferHandle) -> None:
        _check(self._lib.yule_cuda_free(self._ctx, handle.id))

    def matmul(self, a: BufferHandle, b: BufferHandle, out: BufferHandle, m: int, n: int, k: int) -> None:
        _check(self._lib.yule_cuda_matmul(self._ctx, a.id, b.id, out.id, m, n, k))

    def softmax(self, input: BufferHandle, output: BufferHandle, size: int) -> None:
        _check(self._lib.yule_cuda_softmax(self._ctx, input.id, output.id, size))

    def rms_norm(self, input: BufferHandle, weight: BufferHandle, output: BufferHandle, size: int, eps: float) -> None:
        _check(self._lib.yule_cuda_rms_norm(self._ctx, input.id, weight.id, output.id, size, eps))

    def rope(self, q: BufferHandle, k: BufferHandle, pos: int, head_dim: int, freq_base: float, n_heads_q: int,
             n_heads_k: int) -> None:
        _check(self._lib.yule_cuda_rope(self._ctx, q.id, k.id, pos, head_dim, freq_base, n_heads_q, n_heads_k))

    def silu(self, input: BufferHandle, output: BufferHandle, size: int) -> None:
        _check(self._lib.yule_cuda_silu(self._ctx, input.id, output.id, size))

    def element_mul(self, a: BufferHandle, b: BufferHandle, output: BufferHandle, size: int) -> None:
        _check(self._lib.yule_cuda_element_mul(self._ctx, a.id, b.id, output.id, size))

    def add(self, a: BufferHandle, b: BufferHandle, output: BufferHandle, size: int) -> None:
        _check(self._lib.yule_cuda_add(self._ctx, a.id, b.id, output.id, size))

    def copy_to_device(self, data, handle: BufferHandle) -> None:
        ptr, n, keep = _host_ptr(data)
        _check(self._lib.yule_cuda_copy_to_device(self._ctx, ptr, n, handle.id))
        del keep

    def copy_from_device(self, handle: BufferHandle, data) -> None:
        """Fills ``data`` (a writable bytes-like object or numpy array) from the buffer."""
        if isinstance(data, np.ndarray):
            assert data.flags["C_CONTIGUOUS"] and data.flags["WRITEABLE"]
            ptr, n = C.c_void_p(data.ctypes.data), data.nbytes
        else:
            arr = np.frombuffer(memoryview(data), dtype=np.uint8)
            ptr, n = C.c_void_p(arr.ctypes.data), arr.nbytes
        _check(self._lib.yule_cuda_copy_from_device(self._ctx, handle.id, ptr, n))

    def copy_buffer(self, src: BufferHandle, dst: BufferHandle, size: int) -> None:
        _check(self._lib.yule_cuda_copy_buffer(self._ctx, src.id, dst.id, size))

    def copy_buffer_offset(self, src: BufferHandle, dst: BufferHandle, src_offset: int, dst_offset: int,
                           size: int) -> None:
        _check(self._lib.yule_cuda_copy_buffer_offset(self._ctx, src.id, dst.id, src_offset, dst_offset, size))

    def synchronize(self) -> None:
        _check(self._lib.yule_cuda_synchronize(self._ctx))

    def set_wait_budget(self, cycles: int) -> None:
        """Budget (SM clock cycles) of the bounded device-side waits launched afterwards; 0 = default."""
        _check(self._lib.yule_cuda_set_wait_budget(self._ctx, cycles))

    def selftest_bounded_wait(self, which: int, budget_cycles: int) -> None:
        """Runs a kernel whose wait cannot be satisfied; raises ``YuleGpuError`` (code 7, device status) when the
        give-up path works, which is the expected outcome."""
        _check(self._lib.yule_cuda_selftest_bounded_wait(self._ctx, which, budget_cycles))

    def sample(self, logits: BufferHandle, n: int, random_value: float, *, temperature: float = 0.7, top_p: float = 0.9,
               top_k: int = 40, repetition_penalty: float = 1.1, min_p: float = 0.05,
               previous: BufferHandle | None = None, n_previous: int = 0) -> int:
        """``Sampler::sample_with_history`` (yule-infer/src/sampler.rs:17-136) on the device; defaults are
        ``SamplingParams::default`` (yule-infer/src/lib.rs:74-84)."""
        params = _lib.SamplingParams(temperature, top_p, top_k, repetition_penalty, min_p)
        out = C.c_uint32()
        _check(self._lib.yule_cuda_sample(self._ctx, logits.id, n, C.byref(params), previous.id if previous else 0,
                                          n_previous, random_value, C.byref(out)))
        return out.value

    def attn_score(self, q: BufferHandle, k_cache: BufferHandle, scores: BufferHandle, head_dim: int, seq_len: int,
                   head_offset: int, kv_offset: int, kv_stride: int) -> None:
        _check(self._lib.yule_cuda_attn_score(self._ctx, q.id, k_cache.id, scores.id, head_dim, seq_len,
                                              head_offset, kv_offset, kv_stride))

    def attn_value(self, weights: BufferHandle, v_cache: BufferHandle, output: BufferHandle, head_dim: int,
                   seq_len: int, kv_offset: int, kv_stride: int, out_offset: int) -> None:
        _check(self._lib.yule_cuda_attn_value(self._ctx, weights.id, v_cache.id, output.id, head_dim, seq_len,
                                              kv_offset, kv_stride, out_offset))

    def quantized_matmul(self, weights: BufferHandle, input: BufferHandle, output: BufferHandle, n_rows: int,
                         n_cols: int, dtype: DType) -> None:
        _check(self._lib.yule_cuda_quantized_matmul(self._ctx, weights.id, input.id, output.id, n_rows, n_cols,
                                                    int(dtype)))

    # ── additive entry points ──────────────────────────────────────────────────────────────
    def quantized_matmul_batched(self, weights: BufferHandle, input: BufferHandle, output: BufferHandle,
                                 n_rows: int, n_cols: int, dtype: DType, batch: int, x_stride: int | None = None,
                                 out_stride: int | None = None) -> None:
        _check(self._lib.yule_cuda_quantized_matmul_batched(
            self._ctx, weights.id, input.id, output.id, n_rows, n_cols, int(dtype), batch,
            n_cols if x_stride is None else x_stride, n_rows if out_stride is None else out_stride))

    def quantized_matmul_at(self, weights: BufferHandle, weight_offset: int, input: BufferHandle,
                            output: BufferHandle, n_rows: int, n_cols: int, dtype: DType) -> None:
        _check(self._lib.yule_cuda_quantized_matmul_at(self._ctx, weights.id, weight_offset, input.id, output.id,
                                                       n_rows, n_cols, int(dtype)))

    def prepare_weights(self, weights: BufferHandle, dtype: DType, n_rows: int, n_cols: int) -> None:
        """Optional, once per tensor: lets the library keep a device copy in its fastest layout."""
        _check(self._lib.yule_cuda_prepare_weights(self._ctx, weights.id, int(dtype), n_rows, n_cols))

    def dequantize(self, weights: BufferHandle, dtype: DType, n_blocks: int, out_f32: BufferHandle) -> None:
        _check(self._lib.yule_cuda_dequantize(self._ctx, weights.id, int(dtype), n_blocks, out_f32.id))

    def multihead_attention(self, q: BufferHandle, k_cache: BufferHandle, v_cache: BufferHandle, out: BufferHandle,
                            head_dim: int, seq_len: int, n_heads: int, n_kv_heads: int, kv_stride: int) -> None:
        _check(self._lib.yule_cuda_multihead_attention(self._ctx, q.id, k_cache.id, v_cache.id, out.id, head_dim,
                                                       seq_len, n_heads, n_kv_heads, kv_stride))

    def multihead_attention_static(self, q: BufferHandle, k_cache: BufferHandle, v_cache: BufferHandle,
                                   out: BufferHandle, head_dim: int, seq_len: int, n_heads: int, n_kv_heads: int,
                                   kv_stride: int) -> None:
        """``multihead_attention`` without any device allocation: the split scratch is a fixed array
        inside the library (at most 128 heads, head_dim <= 256).  For hosts that cannot call the
        device allocator once inference has started."""
        _check(self._lib.yule_cuda_multihead_attention_static(self._ctx, q.id, k_cache.id, v_cache.id, out.id,
                                                              head_dim, seq_len, n_heads, n_kv_heads, kv_stride))

    def embed_gather(self, table: BufferHandle, dtype: DType, dim: int, token: int, out: BufferHandle) -> None:
        _check(self._lib.yule_cuda_embed_gather(self._ctx, table.id, int(dtype), dim, token, out.id))

    # ── tensor parallelism (one process per GPU) ───────────────────────────────────────────
    @staticmethod
    def tp_unique_id() -> bytes:
        """Rendezvous id created by rank 0; carry it to the other ranks (e.g. torch.distributed broadcast)."""
        lib = _lib.cuda_lib()
        buf = (C.c_uint8 * 128)()
        _check(lib.yule_cuda_tp_unique_id(buf))
        return bytes(buf)

    def tp_init(self, rank: int, world: int, unique_id: bytes) -> None:
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        _check(self._lib.yule_cuda_tp_init(self._ctx, rank, world, buf))

    def tp_all_gather(self, buffer: BufferHandle, count_per_rank: int) -> None:
        _check(self._lib.yule_cuda_tp_all_gather(self._ctx, buffer.id, count_per_rank))

    # ── graph capture / replay (begin_batch / submit_batch of the Vulkan runner, in CUDA terms) ──
    def graph_begin(self) -> None:
        _check(self._lib.yule_cuda_graph_begin(self._ctx))

    def graph_end(self) -> int:
        g = C.c_uint32()
        _check(self._lib.yule_cuda_graph_end(self._ctx, C.byref(g)))
        return g.value

    def graph_launch(self, graph_id: int) -> None:
        _check(self._lib.yule_cuda_graph_launch(self._ctx, graph_id))

    def graph_destroy(self, graph_id: int) -> None:
        _check(self._lib.yule_cuda_graph_destroy(self._ctx, graph_id))

    # ── timing / bookkeeping ───────────────────────────────────────────────────────────────
    def event_record(self) -> int:
        e = C.c_uint32()
        _check(self._lib.yule_cuda_event_record(self._ctx, C.byref(e)))
        return e.value

    def event_elapsed_ms(self, start: int, end: int) -> float:
        ms = C.c_float()
        _check(self._lib.yule_cuda_event_elapsed_ms(self._ctx, start, end, C.byref(ms)))
        return ms.value

    def event_reset(self) -> None:
        _check(self._lib.yule_cuda_event_reset(self._ctx))

    def flush_l2(self) -> None:
        _check(self._lib.yule_cuda_flush_l2(self._ctx))

    def launch_count(self) -> int:
        n = C.c_uint64()
        _check(self._lib.yule_cuda_launch_count(self._ctx, C.byref(n)))
        return n.value

    # ── conveniences for tests (upload / download numpy) ───────────────────────────────────
    def upload(self, array: np.ndarray) -> BufferHandle:
        array = np.ascontiguousarray(array)
        h = self.allocate(max(array.nbytes, 1))
        if array.nbytes:
            self.copy_to_device(array, h)
        return h

    def download(self, handle: BufferHandle, count: int, dtype=np.float32) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        self.copy_from_device(handle, out)
        return out
