"""Launcher of Yule's own CUDA matvec kernels (``oracle/_ref/qmv_*.cubin``, built by ``build_oracle.build_ref_cuda``
from ``yule-gpu/kernels/cuda/qmv_*.cu`` where they lie in a Yule checkout).

TEST INFRASTRUCTURE ONLY: a second pin of the oracle (the reference's GPU arithmetic on the same bytes) and the
"reference kernel on this GPU" leg of ``bench.py``.  Nothing in the shipped package loads this module.

The launch shape is the reference's (``yule-gpu/src/cuda/kernels.rs:236-243`` ``launch_config_per_row``: one block
of 256 threads per output row, 1 KB of dynamic shared memory) and the arguments those of
``yule-gpu/src/cuda/mod.rs:289-328``: weights, input, out, n_rows, n_cols, blocks_per_row.
Device memory and streams come from torch; the kernels are loaded with the CUDA driver API (cuda-python).
"""

from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build_oracle as _build

_KERNELS = {2: ("qmv_q4_0", 32), 8: ("qmv_q8_0", 32), 12: ("qmv_q4_k", 256), 14: ("qmv_q6_k", 256)}  # GGUF type → (file, block size)
_funcs: dict[int, object] = {}


def available(gguf_type: int) -> bool:
    name = _KERNELS.get(gguf_type, (None,))[0]
    return name is not None and os.path.exists(os.path.join(_build.REF_DIR, name + ".cubin"))


def _function(gguf_type: int):
    from cuda.bindings import driver
    import torch
    if gguf_type in _funcs:
        return _funcs[gguf_type]
    torch.cuda.init()
    torch.zeros(1, device="cuda")  # makes torch's primary context current
    name = _KERNELS[gguf_type][0]
    with open(os.path.join(_build.REF_DIR, name + ".cubin"), "rb") as f:
        image = f.read()
    err, module = driver.cuModuleLoadData(image)
    if err != driver.CUresult.CUDA_SUCCESS:
        raise RuntimeError(f"cuModuleLoadData({name}.cubin): {err}")
    err, fn = driver.cuModuleGetFunction(module, (name + "_kernel").encode())
    if err != driver.CUresult.CUDA_SUCCESS:
        raise RuntimeError(f"cuModuleGetFunction({name}_kernel): {err}")
    _funcs[gguf_type] = fn
    return fn


def launch(gguf_type: int, w_ptr: int, x_ptr: int, out_ptr: int, n_rows: int, n_cols: int, stream: int) -> None:
    """One launch of the reference kernel on raw device pointers, on CUDA stream handle ``stream``."""
    from cuda.bindings import driver
    fn = _function(gguf_type)
    bpr = n_cols // _KERNELS[gguf_type][1]
    args = [C.c_void_p(w_ptr), C.c_void_p(x_ptr), C.c_void_p(out_ptr), C.c_uint32(n_rows), C.c_uint32(n_cols), C.c_uint32(bpr)]
    arr = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
    (err,) = driver.cuLaunchKernel(fn, n_rows, 1, 1, 256, 1, 1, 256 * 4, stream, C.addressof(arr), 0)
    if err != driver.CUresult.CUDA_SUCCESS:
        raise RuntimeError(f"cuLaunchKernel: {err}")


def qmv(gguf_type: int, w: np.ndarray, x: np.ndarray, n_rows: int, n_cols: int) -> np.ndarray:
    """out = W·x through the reference's kernel (host arrays in, host array out)."""
    import torch
    wt = torch.from_numpy(np.ascontiguousarray(w).view(np.uint8).reshape(-1)).cuda()
    xt = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()
    ot = torch.empty(n_rows, dtype=torch.float32, device="cuda")
    launch(gguf_type, wt.data_ptr(), xt.data_ptr(), ot.data_ptr(), n_rows, n_cols, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return ot.cpu().numpy()


def time_ring(gguf_type: int, ring: np.ndarray, per_bytes: int, copies: int, x: np.ndarray, n_rows: int, n_cols: int,
              launches: int, reps: int = 3) -> float:
    """Microseconds per launch over a ring of weight copies (each launch a different copy), CUDA-event timed on
    torch's stream; the launches are captured once into a CUDA graph so that host launch cost stays out."""
    import torch
    wt = torch.from_numpy(np.ascontiguousarray(ring).view(np.uint8).reshape(-1)).cuda()
    xt = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()
    ot = torch.empty(n_rows, dtype=torch.float32, device="cuda")
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        launch(gguf_type, wt.data_ptr(), xt.data_ptr(), ot.data_ptr(), n_rows, n_cols, side.cuda_stream)  # loads the module
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for i in range(launches):
                launch(gguf_type, wt.data_ptr() + (i % copies) * per_bytes, xt.data_ptr(), ot.data_ptr(), n_rows, n_cols,
                       side.cuda_stream)
        best = None
        for _ in range(reps + 1):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            graph.replay()
            e1.record(side)
            e1.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None or ms < best else best
    return best * 1e3 / launches
