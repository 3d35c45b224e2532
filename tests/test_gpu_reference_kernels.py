"""Yule's own CUDA matvec kernels (yule-gpu/kernels/cuda/qmv_*.cu, compiled unmodified into oracle/_ref/ by
oracle/build_oracle.py) run on this GPU with the reference's launch shape, against the oracle and against this
library: the reference's GPU arithmetic, the CPU restatement and the B200 kernels agree on the same bytes.
This is a second pin of the oracle (the first is the reference's AVX2 assembly kernel for Q4_K blocks)."""

import numpy as np
import pytest

from conftest import REL_TOL, guarded_rel_err
from yule_b200 import DType, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [DType.Q4_K, DType.Q6_K, DType.Q4_0, DType.Q8_0])
@pytest.mark.parametrize("n_rows,n_cols", [(33, 512), (512, 2048), (300, 5632)])
def test_reference_cuda_kernel_agrees_with_oracle_and_library(backend, oracle, dtype, n_rows, n_cols):
    from oracle import ref_cuda
    if not ref_cuda.available(int(dtype)):
        pytest.skip("oracle/_ref holds no compiled reference kernel (no Yule checkout was reachable at build time)")
    w = synth.random_blocks(dtype, 500 + n_rows, n_rows * (n_cols // dtype.block_size))
    x = synth.normal(501, n_cols)
    ref_gpu = ref_cuda.qmv(int(dtype), w, x, n_rows, n_cols)
    ref_cpu = oracle.qmv(int(dtype), w, x, n_rows, n_cols, simd=oracle.SCALAR)
    assert guarded_rel_err(ref_gpu, ref_cpu) <= 3e-4  # same per-block arithmetic; the block sums are added in tree order
    wh, xh, oh = backend.upload(w), backend.upload(x), backend.allocate(n_rows * 4)
    backend.quantized_matmul(wh, xh, oh, n_rows, n_cols, dtype)
    ours = backend.download(oh, n_rows)
    for h in (wh, xh, oh):
        backend.free(h)
    assert guarded_rel_err(ours, ref_gpu) <= REL_TOL
