"""Two contexts on two GPUs in one process, which the C ABI allows (`yule_cuda_create(device)`): per-device state of
the library — the opt-in for large dynamic shared memory is a per-device attribute of every kernel, tensor maps are
cached per address — must not leak from one device to the other.  No peer memory is involved.  Skipped with fewer
than two GPUs."""

import numpy as np
import pytest

from conftest import REL_TOL, guarded_rel_err
from test_gpu_tp import _gpu_count
from yule_b200 import CudaB200Backend, DType, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [DType.Q4_K, DType.Q6_K, DType.Q8_0], ids=lambda d: d.name)
def test_matvec_on_both_devices(backend, oracle, dtype):
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    n_rows, n_cols = 512, 4096  # a 4096-column image of x needs more than 48 KB of shared memory
    w = synth.random_blocks(dtype, 5, n_rows * n_cols // dtype.block_size)
    x = synth.normal(6, n_cols)
    want = oracle.qmv(int(dtype), w, x, n_rows, n_cols)
    other = CudaB200Backend(1)
    try:
        for b in (backend, other, backend):  # device 0, then 1, then 0 again
            wh, xh, oh = b.upload(w), b.upload(x), b.allocate(n_rows * 4)
            b.prepare_weights(wh, dtype, n_rows, n_cols)
            for _ in range(2):  # the second call is an independent one: the ring kernel
                b.quantized_matmul(wh, xh, oh, n_rows, n_cols, dtype)
            y = b.download(oh, n_rows)
            b.synchronize()
            for h in (wh, xh, oh):
                b.free(h)
            assert guarded_rel_err(y, want) <= REL_TOL
    finally:
        other.close()
