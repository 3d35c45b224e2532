"""The C-ABI library loads and exports every symbol include/yule_cuda.h declares (no compute calls)."""

import ctypes
import os
import re

from yule_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "yule_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(yule_(?:cuda|gguf)_\w+)\s*\(", text)))


def test_header_symbols_are_exported(native_libs):
    lib = ctypes.CDLL(_lib.CUDA_SO)
    names = declared_symbols()
    assert len(names) >= 40
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/yule_cuda.h but not exported"


def test_python_mirror_covers_the_header(native_libs):
    assert set(declared_symbols()) == set(_lib.EXPORTS)


def test_every_trait_method_has_an_entry_point():
    """The 19 methods of ComputeBackend (yule-gpu/src/lib.rs:21-132); name() is a constant in the shim."""
    trait = ["device_info", "allocate", "free", "matmul", "softmax", "rms_norm", "rope", "silu", "element_mul",
             "add", "copy_to_device", "copy_from_device", "copy_buffer", "copy_buffer_offset", "synchronize",
             "attn_score", "attn_value", "quantized_matmul"]
    names = declared_symbols()
    for m in trait:
        assert f"yule_cuda_{m}" in names


def test_status_and_error_text_without_a_device(native_libs):
    """Argument errors are reported before any CUDA work, so they can be checked on a CPU-only host."""
    lib = _lib.cuda_lib()
    assert lib.yule_cuda_synchronize(None) != 0
    assert b"null context" in lib.yule_cuda_last_error()
    assert lib.yule_cuda_create(0, None) != 0
    assert lib.yule_cuda_is_available() in (0, 1)


def test_no_cpu_fallback_when_no_device(native_libs):
    lib = _lib.cuda_lib()
    if lib.yule_cuda_is_available():
        return
    ctx = ctypes.c_void_p()
    assert lib.yule_cuda_create(0, ctypes.byref(ctx)) != 0
    assert b"no CUDA device" in lib.yule_cuda_last_error()
