"""Tensor-core GEMM path of quantized_matmul_batched (eight or more activation rows) against the
scalar CPU restatement of Yule's per-row dot product (yule-gpu/src/cpu.rs:149-175), row by row."""

import numpy as np
import pytest

from yule_b200 import DType, synth

from conftest import REL_TOL, guarded_rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def gemm_for_small_batches(monkeypatch):
    """By default the GEMM takes over from 16 (Q4_K) or 32 (other formats) activation rows; these tests
    want it from 8, its smallest tile."""
    monkeypatch.setenv("YULE_GEMM_MIN_BATCH", "8")


def run(backend, w, x, n_rows, n_cols, batch, x_stride=None, out_stride=None, dtype=DType.Q4_K):
    x_stride = x_stride or n_cols
    out_stride = out_stride or n_rows
    xs = np.zeros((batch, x_stride), np.float32)
    xs[:, :n_cols] = x.reshape(batch, n_cols)
    wh, xh = backend.upload(w), backend.upload(xs.reshape(-1))
    oh = backend.upload(np.full(batch * out_stride, 7.0, np.float32))
    backend.quantized_matmul_batched(wh, xh, oh, n_rows, n_cols, dtype, batch, x_stride, out_stride)
    backend.synchronize()
    y = backend.download(oh, batch * out_stride).reshape(batch, out_stride)
    for h in (wh, xh, oh):
        backend.free(h)
    return y


@pytest.mark.parametrize("n_rows,n_cols,batch", [
    (128, 256, 8),        # one tile, one super-block per row
    (256, 512, 32),       # a full 32-row activation tile
    (1000, 1024, 33),     # ragged rows and one activation row past a tile
    (513, 2048, 64),
    (300, 2048, 200),     # two 128-row activation tiles, the second padded
    (4096, 4096, 128),
    (2048, 5632, 16),     # the TinyLlama down-projection shape
])
def test_gemm_matches_scalar_reference(backend, oracle, n_rows, n_cols, batch):
    w = synth.random_blocks(DType.Q4_K, 300 + n_rows, n_rows * (n_cols // 256))
    x = synth.normal(301 + batch, batch * n_cols)
    y = run(backend, w, x, n_rows, n_cols, batch)
    worst = 0.0
    for b in range(0, batch, max(1, batch // 24)):  # up to ~24 activation rows, spread over the tiles
        ref = oracle.qmv(int(DType.Q4_K), w, x[b * n_cols:(b + 1) * n_cols], n_rows, n_cols)
        worst = max(worst, guarded_rel_err(y[b], ref))
    assert worst <= REL_TOL
    # Against an exact (float64) product of the dequantised weights the error stays near the fp32
    # accumulation floor: the fp16 hi/lo split keeps 22 bits, the tensor core truncates its fp32 sums.
    W = oracle.dequant(int(DType.Q4_K), w).astype(np.float64).reshape(n_rows, n_cols)
    X = x.astype(np.float64).reshape(batch, n_cols)
    scale = np.sqrt((X ** 2).sum(1))[:, None] * np.sqrt((W ** 2).sum(1))[None, :]
    assert (np.abs(y - X @ W.T) / scale).max() <= 4e-6


def test_gemm_strides_and_untouched_padding(backend, oracle):
    n_rows, n_cols, batch = 200, 512, 9
    w = synth.random_blocks(DType.Q4_K, 41, n_rows * (n_cols // 256))
    x = synth.normal(42, batch * n_cols)
    y = run(backend, w, x, n_rows, n_cols, batch, x_stride=n_cols + 64, out_stride=n_rows + 24)
    for b in range(batch):
        ref = oracle.qmv(int(DType.Q4_K), w, x[b * n_cols:(b + 1) * n_cols], n_rows, n_cols)
        assert guarded_rel_err(y[b, :n_rows], ref) <= REL_TOL
    assert np.all(y[:, n_rows:] == 7.0)  # the gap between output rows is not written


def test_gemm_rows_with_very_different_magnitudes(backend, oracle):
    """Every activation row gets its own power-of-two scale: tiny, huge and zero rows in one tile."""
    n_rows, n_cols, batch = 256, 1024, 12
    w = synth.random_quantized(DType.Q4_K, 43, n_rows * n_cols)
    x = synth.normal(44, batch * n_cols).reshape(batch, n_cols)
    x[1] *= 1e-6
    x[2] *= 1e5
    x[3] = 0.0
    x[4, 5] = 3e4  # one outlier far above the rest of its row
    y = run(backend, w, x.reshape(-1), n_rows, n_cols, batch)
    for b in range(batch):
        ref = oracle.qmv(int(DType.Q4_K), w, x[b], n_rows, n_cols)
        assert guarded_rel_err(y[b], ref) <= REL_TOL
    assert np.all(y[3] == 0.0)


def test_gemm_equals_matvec_path(backend):
    """Batch 8 (GEMM) and batch 4 + 4 (tensor-pipe matvec) agree to the parity tolerance."""
    n_rows, n_cols = 1024, 2048
    w = synth.random_quantized(DType.Q4_K, 45, n_rows * n_cols)
    x = synth.normal(46, 8 * n_cols)
    y8 = run(backend, w, x, n_rows, n_cols, 8)
    y4 = np.concatenate([run(backend, w, x[:4 * n_cols], n_rows, n_cols, 4),
                         run(backend, w, x[4 * n_cols:], n_rows, n_cols, 4)])
    assert guarded_rel_err(y8.reshape(-1), y4.reshape(-1)) <= REL_TOL


@pytest.mark.parametrize("dtype", [DType.Q6_K, DType.Q8_0, DType.Q4_0, DType.Q4_K, DType.Q5_K, DType.Q5_0, DType.Q4_1, DType.Q5_1,
                                   DType.Q8_1, DType.Q3_K, DType.Q2_K])
@pytest.mark.parametrize("n_rows,n_cols,batch", [(200, 512, 9), (513, 2048, 64), (1024, 1024, 200)])
def test_generic_format_gemm(backend, oracle, monkeypatch, dtype, n_rows, n_cols, batch):
    """Every format but Q4_K (and Q4_K when forced) goes through the kernel whose producers dequantise with the
    bit-exact per-element routine and split the weight into fp16 hi + lo."""
    monkeypatch.setenv("YULE_GEMM_GENERIC", "1")
    w = synth.random_blocks(dtype, 500 + n_rows, n_rows * (n_cols // dtype.block_size))
    x = synth.normal(501 + batch, batch * n_cols)
    y = run(backend, w, x, n_rows, n_cols, batch, dtype=dtype)
    W = oracle.dequant(int(dtype), w).astype(np.float64).reshape(n_rows, n_cols)
    X = x.astype(np.float64).reshape(batch, n_cols)
    scale = np.sqrt((X ** 2).sum(1))[:, None] * np.sqrt((W ** 2).sum(1))[None, :]
    assert (np.abs(y - X @ W.T) / scale).max() <= 4e-6
    for b in range(0, batch, max(1, batch // 8)):
        ref = oracle.qmv(int(dtype), w, x[b * n_cols:(b + 1) * n_cols], n_rows, n_cols)
        assert guarded_rel_err(y[b], ref) <= REL_TOL


@pytest.mark.parametrize("dtype", [DType.Q4_K, DType.Q8_0, DType.Q6_K])
@pytest.mark.parametrize("n_rows,n_cols,batch,forced", [
    (256, 4096, 32, None),    # two tiles, sixteen super-blocks: four parts of four
    (200, 2816, 16, None),    # eleven super-blocks: parts of six and five, ragged rows
    (1280, 8192, 32, None),   # the Q/K/V slice of a 70B-class layer on eight GPUs
    (2560, 2048, 24, 8),      # 160 work items: some CTAs take two
])
def test_column_split(backend, oracle, monkeypatch, dtype, n_rows, n_cols, batch, forced):
    """With few row tiles and long rows the columns of a tile are split over several CTAs; the warp that stores its
    part last adds the parts in their order.  Same result as the unsplit kernel to fp32 rounding, the same bits on
    every launch (the tickets return to zero), parity with the scalar reference."""
    w = synth.random_blocks(dtype, 700 + n_rows, n_rows * (n_cols // dtype.block_size))
    x = synth.normal(701 + batch, batch * n_cols)
    if forced:
        monkeypatch.setenv("YULE_GEMM_KSPLIT", str(forced))
    y = run(backend, w, x, n_rows, n_cols, batch, dtype=dtype)
    again = run(backend, w, x, n_rows, n_cols, batch, dtype=dtype)
    assert np.array_equal(y, again)
    monkeypatch.setenv("YULE_GEMM_KSPLIT", "1")
    whole = run(backend, w, x, n_rows, n_cols, batch, dtype=dtype)
    assert not np.array_equal(y, whole), "the split did not take place"
    assert np.abs(y - whole).max() <= 4e-6 * np.abs(whole).max()
    for b in (0, batch // 2, batch - 1):
        ref = oracle.qmv(int(dtype), w, x[b * n_cols:(b + 1) * n_cols], n_rows, n_cols)
        assert guarded_rel_err(y[b], ref) <= REL_TOL
