"""Fused dequant-matvec (ComputeBackend::quantized_matmul, yule-gpu/src/lib.rs:119) against the
scalar fused dots of yule-core/src/dequant.rs:902-1207 driven by qmv (yule-infer/src/model_runner.rs:152)."""

import numpy as np
import pytest

from conftest import REL_TOL, guarded_rel_err
from yule_b200 import DType, YuleGpuError, synth
from yule_b200.dtype import EXTRA_QUANTIZED

pytestmark = pytest.mark.gpu

FORMATS = [DType.Q4_0, DType.Q8_0, DType.Q4_K, DType.Q6_K] + list(EXTRA_QUANTIZED)


def gpu_qmv(backend, dtype, w, x, n_rows, n_cols, batch=1):
    wh = backend.upload(w)
    xh = backend.upload(x)
    oh = backend.allocate(batch * n_rows * 4)
    if batch == 1:
        backend.quantized_matmul(wh, xh, oh, n_rows, n_cols, dtype)
    else:
        backend.quantized_matmul_batched(wh, xh, oh, n_rows, n_cols, dtype, batch)
    y = backend.download(oh, batch * n_rows)
    for h in (wh, xh, oh):
        backend.free(h)
    return y


def case(dtype, n_rows, n_cols, seed, batch=1):
    w = synth.random_blocks(dtype, seed, n_rows * (n_cols // dtype.block_size))
    x = synth.normal(seed + 1, batch * n_cols)
    return w, x


@pytest.mark.parametrize("dtype", FORMATS)
@pytest.mark.parametrize("n_rows,blocks_per_row", [(1, 1), (7, 2), (129, 22), (5632, 8), (2048, 22), (300, 56)])
def test_matches_scalar_reference(backend, oracle, dtype, n_rows, blocks_per_row):
    n_cols = blocks_per_row * 256  # a multiple of every format's block size
    w, x = case(dtype, n_rows, n_cols, seed=100 + n_rows)
    y = gpu_qmv(backend, dtype, w, x, n_rows, n_cols)
    ref = oracle.qmv(int(dtype), w, x, n_rows, n_cols, simd=oracle.SCALAR)
    assert guarded_rel_err(y, ref) <= REL_TOL


@pytest.mark.parametrize("dtype", [DType.Q4_0, DType.Q8_0, DType.Q4_1, DType.Q5_0, DType.Q5_1, DType.Q8_1])
def test_small_block_formats_odd_columns(backend, oracle, dtype):
    """32-weight blocks with a column count that is not a multiple of 256."""
    n_rows, n_cols = 33, 32 * 5
    w, x = case(dtype, n_rows, n_cols, seed=9)
    y = gpu_qmv(backend, dtype, w, x, n_rows, n_cols)
    ref = oracle.qmv(int(dtype), w, x, n_rows, n_cols)
    assert guarded_rel_err(y, ref) <= REL_TOL


@pytest.mark.parametrize("dtype", FORMATS)
@pytest.mark.parametrize("batch", [2, 4, 5, 16])
def test_batched_equals_per_vector(backend, oracle, dtype, batch):
    n_rows, n_cols = 513, 2048
    w, x = case(dtype, n_rows, n_cols, seed=77, batch=batch)
    y = gpu_qmv(backend, dtype, w, x, n_rows, n_cols, batch=batch).reshape(batch, n_rows)
    for b in range(batch):
        ref = oracle.qmv(int(dtype), w, x[b * n_cols:(b + 1) * n_cols], n_rows, n_cols)
        assert guarded_rel_err(y[b], ref) <= REL_TOL


@pytest.mark.parametrize("dtype,n_rows,n_cols,batch", [
    (DType.Q8_0, 16, 256, 2),        # one tile, one group of columns
    (DType.Q8_0, 1000, 4096, 3),     # three vectors, ragged last tile, four stages per tile
    (DType.Q4_0, 1000, 4096, 4),
    (DType.Q8_0, 300, 8192, 7),      # three vectors per pass fit beside the ring: 3 + 3 + 1
    (DType.Q4_0, 129, 14336, 4),     # rows longer than one launch's image: three launches over a part of the columns each
    (DType.Q8_0, 200, 14336, 3),
    (DType.Q8_0, 64, 28672, 2),
    (DType.Q4_0, 40, 512, 6),
    (DType.Q8_0, 4096, 4096, 4),
])
def test_q8_0_q4_0_several_vectors_per_pass(backend, oracle, dtype, n_rows, n_cols, batch):
    """Q8_0 / Q4_0 with two to four activation vectors per pass of the ring kernel (one MMA column pair per vector),
    vectors of very different magnitudes (each has its own power-of-two scale), strides wider than the data."""
    w = synth.random_blocks(dtype, 400 + n_rows, n_rows * (n_cols // 32))
    x = synth.normal(401 + batch, batch * n_cols).reshape(batch, n_cols)
    x *= np.float32(10.0) ** np.arange(-3, -3 + batch, dtype=np.float32)[:, None]
    x_stride, out_stride = n_cols + 64, n_rows + 5
    xs = np.zeros((batch, x_stride), np.float32)
    xs[:, :n_cols] = x
    wh, xh = backend.upload(w), backend.upload(xs.reshape(-1))
    oh = backend.upload(np.full(batch * out_stride, 7.0, np.float32))
    backend.quantized_matmul_batched(wh, xh, oh, n_rows, n_cols, dtype, batch, x_stride, out_stride)
    y = backend.download(oh, batch * out_stride).reshape(batch, out_stride)
    for h in (wh, xh, oh):
        backend.free(h)
    assert np.all(y[:, n_rows:] == 7.0)
    for b in range(batch):
        ref = oracle.qmv(int(dtype), w, x[b], n_rows, n_cols)
        assert guarded_rel_err(y[b, :n_rows], ref) <= REL_TOL, f"vector {b}"


@pytest.mark.parametrize("dtype,n_rows,n_cols,batch", [
    (DType.Q4_K, 16, 256, 2),        # one tile, one super-block
    (DType.Q6_K, 16, 256, 2),
    (DType.Q4_K, 1000, 4096, 3),     # three vectors, ragged last tile, two stages per tile
    (DType.Q6_K, 1000, 4096, 4),
    (DType.Q4_K, 300, 8192, 7),
    (DType.Q6_K, 300, 8192, 5),      # two or three vectors per pass fit beside the ring
    (DType.Q4_K, 129, 14336, 4),     # rows longer than one launch's image: three launches over a part of the columns each
    (DType.Q6_K, 129, 14336, 4),
    (DType.Q4_K, 64, 28672, 3),
    (DType.Q6_K, 40, 768, 6),        # three super-blocks: five of a stage's eight warps idle
    (DType.Q4_K, 5632, 2048, 4),
    (DType.Q6_K, 4096, 4096, 4),
    (DType.Q4_K, 1000, 2048, 8),     # two passes of four
    (DType.Q6_K, 300, 2048, 8),
    (DType.Q4_K, 64, 4096, 8),
    (DType.Q6_K, 2048, 5632, 6),
    (DType.Q4_K, 5632, 2048, 9),     # two passes of four, and one vector through the one-vector kernel
])
def test_q4_k_q6_k_several_vectors_per_pass(backend, oracle, dtype, n_rows, n_cols, batch):
    """Q4_K and Q6_K (prepared: row-planar copy) with two to four activation vectors per pass of the batched ring
    kernel, vectors of very different magnitudes, strides wider than the data."""
    w = synth.random_blocks(dtype, 600 + n_rows, n_rows * (n_cols // 256))
    x = synth.normal(601 + batch, batch * n_cols).reshape(batch, n_cols)
    x *= np.float32(10.0) ** np.arange(-3, -3 + batch, dtype=np.float32)[:, None]
    x_stride, out_stride = n_cols + 64, n_rows + 5
    xs = np.zeros((batch, x_stride), np.float32)
    xs[:, :n_cols] = x
    wh, xh = backend.upload(w), backend.upload(xs.reshape(-1))
    backend.prepare_weights(wh, dtype, n_rows, n_cols)
    oh = backend.upload(np.full(batch * out_stride, 7.0, np.float32))
    backend.quantized_matmul_batched(wh, xh, oh, n_rows, n_cols, dtype, batch, x_stride, out_stride)
    y = backend.download(oh, batch * out_stride).reshape(batch, out_stride)
    for h in (wh, xh, oh):
        backend.free(h)
    assert np.all(y[:, n_rows:] == 7.0)
    for b in range(batch):
        ref = oracle.qmv(int(dtype), w, x[b], n_rows, n_cols)
        assert guarded_rel_err(y[b, :n_rows], ref) <= REL_TOL, f"vector {b}"


def test_config0_shape_quantised_gaussian(backend, oracle):
    """The TinyLlama FFN-up shape of the headline matvec: 5632 x 2048 Q4_K."""
    n_rows, n_cols = 5632, 2048
    w = synth.random_quantized(DType.Q4_K, 5, n_rows * n_cols)
    x = synth.normal(6, n_cols)
    y = gpu_qmv(backend, DType.Q4_K, w, x, n_rows, n_cols)
    ref = oracle.qmv(int(DType.Q4_K), w, x, n_rows, n_cols)
    assert guarded_rel_err(y, ref) <= REL_TOL


def test_q4_0_kat_from_cpu_backend_tests(backend):
    """yule-gpu/src/cpu.rs:991-1076: two rows of 32 weights that all dequantise to 1.0."""
    w = np.zeros(36, np.uint8)
    w[0:2] = (0x00, 0x3C)
    w[2:18] = 0x99
    w[18:20] = (0x00, 0x38)
    w[20:36] = 0xAA
    y = gpu_qmv(backend, DType.Q4_0, w, np.ones(32, np.float32), 2, 32)
    assert abs(y[0] - 32.0) < 1e-4 and abs(y[1] - 32.0) < 1e-4


def test_linearity_at_full_size(backend):
    """Size-independent property at a large shape: W(ax + by) = a Wx + b Wy within fp32 noise."""
    dtype, n_rows, n_cols = DType.Q4_K, 14336, 4096
    w = synth.random_blocks(dtype, 21, n_rows * (n_cols // 256))
    x1, x2 = synth.normal(1, n_cols), synth.normal(2, n_cols)
    y1 = gpu_qmv(backend, dtype, w, x1, n_rows, n_cols)
    y2 = gpu_qmv(backend, dtype, w, x2, n_rows, n_cols)
    y3 = gpu_qmv(backend, dtype, w, (2 * x1 - 3 * x2).astype(np.float32), n_rows, n_cols)
    assert guarded_rel_err(y3, 2 * y1.astype(np.float64) - 3 * y2.astype(np.float64)) <= REL_TOL


def test_weight_offset_view(backend, oracle):
    """A tensor that starts inside a larger buffer (row shard / ring slot)."""
    dtype, n_rows, n_cols = DType.Q4_K, 64, 512
    w = synth.random_blocks(dtype, 4, 3 * n_rows * 2)
    x = synth.normal(8, n_cols)
    per = n_rows * 2 * 144
    wh, xh, oh = backend.upload(w), backend.upload(x), backend.allocate(n_rows * 4)
    backend.quantized_matmul_at(wh, 2 * per, xh, oh, n_rows, n_cols, dtype)
    y = backend.download(oh, n_rows)
    ref = oracle.qmv(int(dtype), w[2 * per:], x, n_rows, n_cols)
    assert guarded_rel_err(y, ref) <= REL_TOL
    with pytest.raises(YuleGpuError):
        backend.quantized_matmul_at(wh, 2 * per + 144, xh, oh, n_rows, n_cols, dtype)  # runs off the end
    for h in (wh, xh, oh):
        backend.free(h)


@pytest.mark.parametrize("shift", [0, 6])
def test_q5k_any_two_byte_offset(backend, oracle, shift):
    """Q5_K at a 16-byte-aligned offset (vectorised kernel) and at an odd one (element-wise kernel)."""
    dtype, n_rows, n_cols = DType.Q5_K, 70, 1024
    blocks = synth.random_blocks(dtype, 21, n_rows * 4)
    w = np.concatenate([np.zeros(176 + shift, np.uint8), blocks])
    x = synth.normal(8, n_cols)
    wh, xh, oh = backend.upload(w), backend.upload(x), backend.allocate(n_rows * 4)
    backend.quantized_matmul_at(wh, 176 + shift, xh, oh, n_rows, n_cols, dtype)
    y = backend.download(oh, n_rows)
    assert guarded_rel_err(y, oracle.qmv(int(dtype), blocks, x, n_rows, n_cols)) <= REL_TOL
    for h in (wh, xh, oh):
        backend.free(h)


def test_error_paths(backend):
    w = backend.allocate(144 * 4)
    x = backend.allocate(256 * 4)
    o = backend.allocate(16)
    with pytest.raises(YuleGpuError) as e:
        backend.quantized_matmul(w, x, o, 4, 256, 16)  # IQ2_XXS: unsupported dtype for CUDA qmv
    assert "unsupported dtype" in str(e.value)
    with pytest.raises(YuleGpuError):
        backend.quantized_matmul(w, x, o, 4, 200, DType.Q4_K)  # not a block multiple
    with pytest.raises(YuleGpuError):
        backend.quantized_matmul(w, x, o, 5, 256, DType.Q4_K)  # weights too small
    from yule_b200 import BufferHandle
    with pytest.raises(YuleGpuError) as e:
        backend.quantized_matmul(BufferHandle(987654), x, o, 4, 256, DType.Q4_K)
    assert "unknown buffer" in str(e.value)
    backend.quantized_matmul(w, x, o, 0, 256, DType.Q4_K)  # zero rows: nothing to do
    for h in (w, x, o):
        backend.free(h)


@pytest.mark.parametrize("n_rows,blocks_per_row", [(1, 1), (7, 2), (129, 22), (2048, 22), (300, 56), (4736, 8), (32000, 8)])
def test_prepared_q6k_matches_scalar_reference(backend, oracle, n_rows, blocks_per_row):
    """prepare_weights keeps a planar device copy of a Q6_K tensor; the matvec that reads it must
    give the same numbers as the scalar reference (and as the raw-layout kernel)."""
    dtype, n_cols = DType.Q6_K, blocks_per_row * 256
    w, x = case(dtype, n_rows, n_cols, seed=300 + n_rows)
    wh, xh, oh = backend.upload(w), backend.upload(x), backend.allocate(n_rows * 4)
    backend.quantized_matmul(wh, xh, oh, n_rows, n_cols, dtype)
    raw = backend.download(oh, n_rows)
    backend.prepare_weights(wh, dtype, n_rows, n_cols)
    backend.quantized_matmul(wh, xh, oh, n_rows, n_cols, dtype)
    y = backend.download(oh, n_rows)
    ref = oracle.qmv(int(dtype), w, x, n_rows, n_cols)
    assert guarded_rel_err(y, ref) <= REL_TOL and guarded_rel_err(raw, ref) <= REL_TOL
    # writing to the buffer drops the prepared copy: results follow the new bytes
    w2 = synth.random_blocks(dtype, 999, n_rows * blocks_per_row)
    backend.copy_to_device(w2, wh)
    backend.quantized_matmul(wh, xh, oh, n_rows, n_cols, dtype)
    assert guarded_rel_err(backend.download(oh, n_rows), oracle.qmv(int(dtype), w2, x, n_rows, n_cols)) <= REL_TOL
    for h in (wh, xh, oh):
        backend.free(h)


def test_prepare_weights_is_a_noop_for_other_formats(backend):
    for dt in (DType.Q4_K, DType.Q8_0, DType.Q4_0):
        w = backend.upload(synth.random_blocks(dt, 1, 8 * (256 // dt.block_size)))
        backend.prepare_weights(w, dt, 8, 256)
        with pytest.raises(YuleGpuError):
            backend.prepare_weights(w, dt, 9, 256)  # tensor larger than the buffer
        backend.free(w)


def test_dependent_chain_of_matvecs(backend, oracle):
    """Consecutive trait calls are chained with programmatic dependent launch (weights fetched before the
    previous kernel ends, activations after): y1 = W1 x, y2 = W2 y1, y3 = W3 y2 must still see each other's
    results, and a buffer written by one call may be the next call's weights."""
    n = 512
    ws = [synth.random_blocks(DType.Q4_K, 40 + i, n * n // 256, scale_std=0.02) for i in range(3)]
    x = synth.normal(50, n)
    whs = [backend.upload(w) for w in ws]
    bufs = [backend.upload(x)] + [backend.allocate(n * 4) for _ in range(3)]
    for rep in range(3):
        for i in range(3):
            backend.quantized_matmul(whs[i], bufs[i], bufs[i + 1], n, n, DType.Q4_K)
    y = backend.download(bufs[3], n)
    ref = x
    for w in ws:
        ref = oracle.qmv(int(DType.Q4_K), w, ref, n, n)
    assert guarded_rel_err(y, ref) <= REL_TOL
    # a matvec whose "weights" are the bytes the previous call just wrote: no early read may happen
    big = backend.allocate(16 * 144)
    raw = synth.random_blocks(DType.Q4_K, 60, 16)
    src = backend.upload(np.frombuffer(raw.tobytes(), np.float32).copy())
    ident = backend.upload(x[:256])
    backend.quantized_matmul(whs[0], bufs[0], bufs[1], n, n, DType.Q4_K)
    backend.copy_buffer(src, big, 16 * 144)
    out = backend.allocate(16 * 4)
    backend.quantized_matmul(big, ident, out, 16, 256, DType.Q4_K)
    got = backend.download(out, 16)
    assert guarded_rel_err(got, oracle.qmv(int(DType.Q4_K), raw, x[:256], 16, 256)) <= REL_TOL
    for h in whs + bufs + [big, src, ident, out]:
        backend.free(h)


@pytest.mark.parametrize("dtype", [DType.Q4_K, DType.Q6_K])
@pytest.mark.parametrize("kernel", ["ring", "stream"])
@pytest.mark.parametrize("n_rows,blocks_per_row", [(1, 1), (7, 2), (129, 22), (5632, 8), (2048, 22), (300, 56), (40000, 16)])
def test_both_q4k_q6k_kernels(backend, oracle, monkeypatch, dtype, kernel, n_rows, blocks_per_row):
    """The shared-memory-ring kernel (independent calls) and the register-streaming kernel (dependent chains)
    are picked by what a call depends on; here each is forced in turn on the same inputs, prepared weights."""
    monkeypatch.setenv("YULE_QMV_RING", "1" if kernel == "ring" else "0")
    n_cols = blocks_per_row * 256
    w, x = case(dtype, n_rows, n_cols, seed=300 + n_rows)
    wh, xh, oh = backend.upload(w), backend.upload(x), backend.allocate(n_rows * 4)
    backend.prepare_weights(wh, dtype, n_rows, n_cols)
    for _ in range(3):  # the second and third calls are chained to their predecessor (late wait)
        backend.quantized_matmul(wh, xh, oh, n_rows, n_cols, dtype)
    y = backend.download(oh, n_rows)
    for h in (wh, xh, oh):
        backend.free(h)
    ref = oracle.qmv(int(dtype), w, x, n_rows, n_cols, simd=oracle.SCALAR)
    assert guarded_rel_err(y, ref) <= REL_TOL


def test_independent_calls_share_inputs(backend, oracle):
    """Q, K, V style: three matrices, one input vector, three outputs, issued back to back twice; then a call
    that consumes one of the outputs (it must wait for it)."""
    n = 2048
    ws = [synth.random_blocks(DType.Q4_K, 70 + i, n * n // 256, scale_std=0.02) for i in range(3)]
    w6 = synth.random_blocks(DType.Q6_K, 75, n * n // 256, scale_std=0.02)
    x = synth.normal(76, n)
    whs = [backend.upload(w) for w in ws]
    w6h = backend.upload(w6)
    backend.prepare_weights(w6h, DType.Q6_K, n, n)
    xh = backend.upload(x)
    outs = [backend.allocate(n * 4) for _ in range(4)]
    for rep in range(2):
        for i in range(3):
            backend.quantized_matmul(whs[i], xh, outs[i], n, n, DType.Q4_K)
        backend.quantized_matmul(w6h, outs[1], outs[3], n, n, DType.Q6_K)  # depends on the second output
    refs = [oracle.qmv(int(DType.Q4_K), w, x, n, n) for w in ws]
    for i in range(3):
        assert guarded_rel_err(backend.download(outs[i], n), refs[i]) <= REL_TOL
    assert guarded_rel_err(backend.download(outs[3], n), oracle.qmv(int(DType.Q6_K), w6, refs[1], n, n)) <= REL_TOL
    for h in whs + [w6h, xh] + outs:
        backend.free(h)
