"""Matvec micro-benchmark over the C ABI: one dtype and shape, CUDA-event timed.

    python -m yule_b200.microbench --dtype Q4_K --rows 5632 --cols 2048 [--batch 1] [--iters 200] [--ring]

Without ``--ring`` the weight tensor is read again and again (small tensors stay in L2 — that number is
labelled ``l2_resident``).  With ``--ring`` the launches rotate over copies of the tensor that together
exceed twice the L2 capacity, so every launch streams from HBM.  Launches are captured into one CUDA
graph and replayed; the time per launch is the graph time divided by the launch count.
"""

from __future__ import annotations

import argparse
import json
import statistics

import numpy as np

from . import CudaB200Backend, DType, matvec_bytes, synth


def run(backend, dtype: DType, rows: int, cols: int, batch: int, iters: int, ring: bool, reps: int = 5,
        prepare: bool = True) -> dict:
    per = dtype.tensor_bytes(rows, cols)
    copies = max(1, -(-2 * 2 * 126 * 2 ** 20 // per)) if ring else 1  # ≥ 4 x L2 in total
    copies = min(copies, max(1, (24 << 30) // per))
    base = synth.random_blocks(dtype, 1, rows * cols // dtype.block_size)
    # one buffer per copy, so that each can carry its own prepared layout
    whs = [backend.upload(base) for _ in range(copies)]
    if prepare:
        for h in whs:
            backend.prepare_weights(h, dtype, rows, cols)
    xh = backend.upload(synth.normal(2, batch * cols))
    oh = backend.allocate(batch * rows * 4)
    if batch > 1:  # scratch of the batched paths is sized outside the capture
        backend.quantized_matmul_batched(whs[0], xh, oh, rows, cols, dtype, batch)
    backend.graph_begin()
    for i in range(iters):
        if batch == 1:
            backend.quantized_matmul(whs[i % copies], xh, oh, rows, cols, dtype)
        else:
            backend.quantized_matmul_batched(whs[i % copies], xh, oh, rows, cols, dtype, batch)
    graph = backend.graph_end()
    for _ in range(3):
        backend.graph_launch(graph)
    backend.synchronize()
    times = []
    for _ in range(reps):
        backend.event_reset()
        e0 = backend.event_record()
        backend.graph_launch(graph)
        e1 = backend.event_record()
        times.append(backend.event_elapsed_ms(e0, e1))
    y = backend.download(oh, batch * rows)
    backend.graph_destroy(graph)
    for h in whs + [xh, oh]:
        backend.free(h)
    us = statistics.median(times) * 1e3 / iters
    nbytes = matvec_bytes(dtype, rows, cols, batch)
    return {"dtype": dtype.name, "rows": rows, "cols": cols, "batch": batch, "mode": "hbm_ring" if ring else "l2_resident",
            "copies": copies, "prepared": prepare, "us_per_launch": round(us, 3), "bytes_per_launch": nbytes,
            "gbs": round(nbytes / us / 1e3, 1),
            "tflops": round(2.0 * rows * cols * batch / us / 1e6, 2), "nan_outputs": int(np.isnan(y).sum())}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="Q4_K")
    ap.add_argument("--rows", type=int, default=5632)
    ap.add_argument("--cols", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--ring", action="store_true")
    ap.add_argument("--raw", action="store_true", help="do not call prepare_weights (raw GGUF layout only)")
    ap.add_argument("--sweep", action="store_true",
                    help="the format x shape x batch grid of the matvec sweep (4 formats, 5 shapes, batch 1/4/16), "
                         "weights streamed from HBM; prints one JSON line per case")
    ap.add_argument("--formats", default="Q4_0,Q8_0,Q4_K,Q6_K", help="comma-separated formats of --sweep")
    args = ap.parse_args()
    backend = CudaB200Backend(0)
    if args.sweep:
        shapes = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]
        for dt in [DType[n] for n in args.formats.split(",")]:
            for rows, cols in shapes:
                for batch in (1, 4, 16):
                    iters = 20 if rows * cols > 10 ** 8 else 100
                    print(json.dumps(run(backend, dt, rows, cols, batch, iters, True, reps=3)), flush=True)
        backend.close()
        return
    print(json.dumps(run(backend, DType[args.dtype], args.rows, args.cols, args.batch, args.iters, args.ring,
                         prepare=not args.raw)))
    backend.close()


if __name__ == "__main__":
    main()
