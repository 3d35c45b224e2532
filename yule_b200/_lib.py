"""Loader of the package's native libraries.  There is no fallback: a missing library is an error."""

from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
CUDA_SO = os.path.join(HERE, "libyule_cuda.so")
SYNTH_SO = os.path.join(HERE, "libyule_synth.so")

_cuda = None
_synth = None

u64, u32, i32, f32, size_t = C.c_uint64, C.c_uint32, C.c_int32, C.c_float, C.c_size_t
vp = C.c_void_p


class RunnerConfig(C.Structure):
    """``yule_runner_config`` of include/yule_cuda.h."""
    _fields_ = [("dim", u32), ("n_layers", u32), ("n_heads", u32), ("n_kv_heads", u32), ("head_dim", u32),
                ("vocab_size", u32), ("ff_dim", u32), ("max_seq_len", u32), ("norm_eps", f32),
                ("rope_freq_base", f32), ("fused", u32), ("rotary_dim", u32), ("sliding_window", u32),
                ("attn_logit_softcap", f32), ("logit_softcap", f32), ("norm_weight_offset", f32), ("geglu", u32),
                ("n_experts", u32), ("n_experts_used", u32)]


class SamplingParams(C.Structure):
    """``yule_sampling_params`` of include/yule_cuda.h (SamplingParams, yule-infer/src/lib.rs:65-84)."""
    _fields_ = [("temperature", f32), ("top_p", f32), ("top_k", u32), ("repetition_penalty", f32), ("min_p", f32)]


class GgufTensorInfo(C.Structure):
    """``yule_gguf_tensor_info`` of include/yule_cuda.h."""
    _fields_ = [("name", C.c_char_p), ("n_dims", u32), ("shape", u64 * 8), ("gguf_type", u32), ("offset", u64),
                ("size_bytes", u64), ("data", vp)]


# name → argtypes; every entry returns int32 status unless listed in _RESTYPES.
_SIGNATURES = {
    "yule_cuda_is_available": [],
    "yule_cuda_create": [i32, C.POINTER(vp)],
    "yule_cuda_destroy": [vp],
    "yule_cuda_device_info": [vp, C.c_char_p, size_t, C.POINTER(u64), C.POINTER(u32)],
    "yule_cuda_allocate": [vp, size_t, C.POINTER(u64)],
    "yule_cuda_free": [vp, u64],
    "yule_cuda_copy_to_device": [vp, vp, size_t, u64],
    "yule_cuda_copy_from_device": [vp, u64, vp, size_t],
    "yule_cuda_copy_buffer": [vp, u64, u64, size_t],
    "yule_cuda_copy_buffer_offset": [vp, u64, u64, size_t, size_t, size_t],
    "yule_cuda_synchronize": [vp],
    "yule_cuda_set_wait_budget": [vp, u64],
    "yule_cuda_selftest_bounded_wait": [vp, u32, u64],
    "yule_cuda_matmul": [vp, u64, u64, u64, u32, u32, u32],
    "yule_cuda_softmax": [vp, u64, u64, u32],
    "yule_cuda_rms_norm": [vp, u64, u64, u64, u32, f32],
    "yule_cuda_rope": [vp, u64, u64, u32, u32, f32, u32, u32],
    "yule_cuda_silu": [vp, u64, u64, u32],
    "yule_cuda_element_mul": [vp, u64, u64, u64, u32],
    "yule_cuda_add": [vp, u64, u64, u64, u32],
    "yule_cuda_attn_score": [vp, u64, u64, u64, u32, u32, u32, u32, u32],
    "yule_cuda_attn_value": [vp, u64, u64, u64, u32, u32, u32, u32, u32],
    "yule_cuda_quantized_matmul": [vp, u64, u64, u64, u32, u32, u32],
    "yule_cuda_quantized_matmul_batched": [vp, u64, u64, u64, u32, u32, u32, u32, u32, u32],
    "yule_cuda_quantized_matmul_at": [vp, u64, size_t, u64, u64, u32, u32, u32],
    "yule_cuda_prepare_weights": [vp, u64, u32, u32, u32],
    "yule_cuda_dequantize": [vp, u64, u32, u64, u64],
    "yule_cuda_multihead_attention": [vp, u64, u64, u64, u64, u32, u32, u32, u32, u32],
    "yule_cuda_multihead_attention_static": [vp, u64, u64, u64, u64, u32, u32, u32, u32, u32],
    "yule_cuda_embed_gather": [vp, u64, u32, u32, u32, u64],
    "yule_cuda_graph_begin": [vp],
    "yule_cuda_graph_end": [vp, C.POINTER(u32)],
    "yule_cuda_graph_launch": [vp, u32],
    "yule_cuda_graph_destroy": [vp, u32],
    "yule_cuda_event_record": [vp, C.POINTER(u32)],
    "yule_cuda_event_elapsed_ms": [vp, u32, u32, C.POINTER(f32)],
    "yule_cuda_event_reset": [vp],
    "yule_cuda_flush_l2": [vp],
    "yule_cuda_launch_count": [vp, C.POINTER(u64)],
    "yule_cuda_tp_unique_id": [C.POINTER(C.c_uint8)],
    "yule_cuda_tp_init": [vp, u32, u32, C.POINTER(C.c_uint8)],
    "yule_cuda_tp_all_gather": [vp, u64, size_t],
    "yule_cuda_tp_exchange_layout": [C.POINTER(RunnerConfig), C.POINTER(u64)],
    "yule_cuda_runner_create": [vp, C.POINTER(RunnerConfig), C.POINTER(vp)],
    "yule_cuda_runner_destroy": [vp],
    "yule_cuda_runner_set_tensor": [vp, C.c_char_p, u64, u32],
    "yule_cuda_runner_prefill": [vp, C.POINTER(u32), u32, C.POINTER(f32)],
    "yule_cuda_runner_decode_step": [vp, u32, C.POINTER(f32)],
    "yule_cuda_runner_reset": [vp],
    "yule_cuda_runner_position": [vp, C.POINTER(u32)],
    "yule_cuda_runner_step_kind": [vp, C.POINTER(u32)],
    "yule_cuda_runner_selftest_bounded_wait": [vp, C.c_uint64],
    "yule_cuda_runner_generate_greedy": [vp, C.POINTER(u32), u32, u32, C.POINTER(u32)],
    "yule_cuda_runner_buffer": [vp, u32, u32, C.POINTER(u64)],
    "yule_cuda_sample": [vp, u64, u32, C.POINTER(SamplingParams), u64, u32, f32, C.POINTER(u32)],
    "yule_cuda_runner_generate_sampled": [vp, C.POINTER(u32), u32, u32, C.POINTER(SamplingParams), u64, C.POINTER(u32)],
    "yule_cuda_runner_decode_batch": [vp, C.POINTER(u32), u32, C.POINTER(f32)],
    "yule_cuda_runner_reset_batch": [vp],
    "yule_cuda_runner_generate_greedy_batch": [vp, C.POINTER(u32), u32, u32, u32, C.POINTER(u32)],
    "yule_gguf_open": [C.c_char_p, C.POINTER(vp)],
    "yule_gguf_parse": [vp, size_t, C.POINTER(vp)],
    "yule_gguf_close": [vp],
    "yule_gguf_summary": [vp, C.POINTER(u32), C.POINTER(u64), C.POINTER(u64), C.POINTER(u64), C.POINTER(u64)],
    "yule_gguf_tensor": [vp, u64, C.POINTER(GgufTensorInfo)],
    "yule_gguf_find_tensor": [vp, C.c_char_p, C.POINTER(u64)],
    "yule_gguf_meta_u32": [vp, C.c_char_p, C.POINTER(u32)],
    "yule_gguf_meta_f64": [vp, C.c_char_p, C.POINTER(C.c_double)],
    "yule_gguf_meta_str": [vp, C.c_char_p, C.POINTER(C.c_char_p)],
    "yule_gguf_runner_config": [vp, u32, C.POINTER(RunnerConfig)],
    "yule_cuda_runner_load_gguf": [vp, vp, u32, u32, C.POINTER(vp)],
}
_RESTYPES = {"yule_cuda_last_error": C.c_char_p, "yule_cuda_sampling_random_value": f32}

EXPORTS = tuple(sorted(list(_SIGNATURES) + list(_RESTYPES)))


def cuda_lib() -> C.CDLL:
    """``libyule_cuda.so`` with typed entry points.  Raises when the library has not been built."""
    global _cuda
    if _cuda is None:
        if not os.path.exists(CUDA_SO):
            raise RuntimeError(f"{CUDA_SO} is missing: build it with `python -m yule_b200.build` "
                               "(this package has no CPU fallback)")
        lib = C.CDLL(CUDA_SO)
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = i32
        lib.yule_cuda_last_error.argtypes = []
        lib.yule_cuda_last_error.restype = C.c_char_p
        lib.yule_cuda_sampling_random_value.argtypes = [u64, u32]
        lib.yule_cuda_sampling_random_value.restype = f32
        _cuda = lib
    return _cuda


def synth_lib() -> C.CDLL:
    """``libyule_synth.so`` — host-side synthetic tensor generator."""
    global _synth
    if _synth is None:
        if not os.path.exists(SYNTH_SO):
            raise RuntimeError(f"{SYNTH_SO} is missing: build it with `python -m yule_b200.build`")
        lib = C.CDLL(SYNTH_SO)
        lib.ys_fill_normal.argtypes = [u64, f32, f32, C.POINTER(f32), u64, C.c_int]
        lib.ys_fill_normal.restype = None
        lib.ys_fill_tokens.argtypes = [u64, u32, C.POINTER(u32), u64]
        lib.ys_fill_tokens.restype = None
        lib.ys_random_blocks.argtypes = [C.c_int, u64, f32, C.POINTER(C.c_uint8), u64, C.c_int]
        lib.ys_quantize.argtypes = [C.c_int, C.POINTER(f32), u64, C.POINTER(C.c_uint8), C.c_int]
        lib.ys_random_quantized.argtypes = [C.c_int, u64, f32, C.POINTER(C.c_uint8), u64, C.c_int]
        lib.ys_random_quantized_at.argtypes = [C.c_int, u64, f32, C.POINTER(C.c_uint8), u64, u64, C.c_int]
        lib.ys_f32_to_f16.argtypes = [f32]
        lib.ys_f32_to_f16.restype = C.c_uint16
        _synth = lib
    return _synth
