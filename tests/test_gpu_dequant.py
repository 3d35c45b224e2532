"""Dequantised weights must be bit-identical to yule-core's scalar dequantisers
(yule-core/src/dequant.rs:77-165, :196-372), checked through the C ABI."""

import numpy as np
import pytest

from yule_b200 import DType, synth
from yule_b200.dtype import EXTRA_QUANTIZED

pytestmark = pytest.mark.gpu

FORMATS = [DType.Q4_0, DType.Q8_0, DType.Q4_K, DType.Q6_K] + list(EXTRA_QUANTIZED)
QUANTISABLE = [d for d in FORMATS if d not in (DType.Q8_1, DType.Q2_K, DType.Q3_K)]


def gpu_dequant(backend, dtype, data):
    n_blocks = data.size // dtype.size_of_block
    w = backend.upload(data)
    out = backend.allocate(n_blocks * dtype.block_size * 4)
    backend.dequantize(w, dtype, n_blocks, out)
    res = backend.download(out, n_blocks * dtype.block_size)
    backend.free(w)
    backend.free(out)
    return res


@pytest.mark.parametrize("dtype", FORMATS)
def test_random_field_blocks_bit_exact(backend, oracle, dtype):
    data = synth.random_blocks(dtype, seed=11 + int(dtype), n_blocks=4096)
    got = gpu_dequant(backend, dtype, data)
    ref = oracle.dequant(int(dtype), data)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), "f32 bit mismatch"


@pytest.mark.parametrize("dtype", QUANTISABLE)
def test_quantised_gaussian_bit_exact(backend, oracle, dtype):
    data = synth.random_quantized(dtype, seed=3, n_weights=256 * 2048, std=0.02)
    got = gpu_dequant(backend, dtype, data)
    ref = oracle.dequant(int(dtype), data)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_every_f16_scale_pattern(backend, oracle):
    """All 65 536 half patterns as the Q8_0 scale with quant 1: the output is f16_to_f32(bits)
    (yule-core/src/dequant.rs:20-49).  NaN payloads are compared as 'both NaN'."""
    blocks = np.zeros((65536, 34), np.uint8)
    bits = np.arange(65536, dtype=np.uint16)
    blocks[:, 0] = bits & 0xFF
    blocks[:, 1] = bits >> 8
    blocks[:, 2] = 1
    data = blocks.reshape(-1)
    got = gpu_dequant(backend, DType.Q8_0, data).reshape(65536, 32)[:, 0]
    ref = oracle.dequant(int(DType.Q8_0), data).reshape(65536, 32)[:, 0]
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), ref[~nan].view(np.uint32))


def test_reference_kats(backend):
    """The hand-built blocks of yule-core's own tests (dequant.rs:1309-1359)."""
    b = np.zeros(18, np.uint8)
    b[1] = 0x3C
    b[2:] = 0x88
    assert np.all(gpu_dequant(backend, DType.Q4_0, b) == 0.0)
    b = np.zeros(18, np.uint8)
    b[1] = 0x3C
    b[2] = 0xF0
    out = gpu_dequant(backend, DType.Q4_0, b)
    assert out[0] == -8.0 and out[1] == 7.0
    b = np.zeros(34, np.uint8)
    b[1] = 0x3C
    b[2] = 127
    b[3] = 0x80
    out = gpu_dequant(backend, DType.Q8_0, b)
    assert out[0] == 127.0 and out[1] == -128.0


def test_reference_kats_other_formats(backend):
    """The hand-built blocks of yule-core's tests for Q4_1, Q5_0, Q3_K, Q5_K and Q8_1
    (dequant.rs:1405-1426, :1444-1474, :1490-1527, :1530-1563, :1598-1611)."""
    b = np.zeros(20, np.uint8)
    b[1] = b[3] = 0x3C
    b[4] = 0xF0
    out = gpu_dequant(backend, DType.Q4_1, b)
    assert out[0] == 1.0 and out[1] == 16.0 and out[2] == 1.0
    b = np.zeros(22, np.uint8)
    b[1] = 0x3C
    b[2] = 0x02
    b[6] = 0x5A
    out = gpu_dequant(backend, DType.Q5_0, b)
    assert out[0] == -6.0 and out[1] == 5.0
    b = np.zeros(110, np.uint8)
    b[109] = 0x3C
    b[96], b[104], b[32] = 0x01, 0x02, 0x01
    assert gpu_dequant(backend, DType.Q3_K, b)[0] == -3.0
    b[0] = 0x01
    assert gpu_dequant(backend, DType.Q3_K, b)[0] == 1.0
    b = np.zeros(176, np.uint8)
    b[1] = 0x3C
    b[4], b[48] = 0x01, 0x05
    assert gpu_dequant(backend, DType.Q5_K, b)[0] == 5.0
    b[16] = 0x01
    assert gpu_dequant(backend, DType.Q5_K, b)[0] == 21.0
    b = np.zeros(36, np.uint8)
    b[1] = 0x3C
    b[4], b[5] = 42, 0x80
    out = gpu_dequant(backend, DType.Q8_1, b)
    assert out[0] == 42.0 and out[1] == -128.0


def test_empty_and_errors(backend):
    from yule_b200 import YuleGpuError
    w = backend.allocate(144)
    out = backend.allocate(256 * 4)
    backend.dequantize(w, DType.Q4_K, 0, out)  # nothing to do
    with pytest.raises(YuleGpuError):
        backend.dequantize(w, DType.Q4_K, 2, out)  # reads past the weight buffer
    with pytest.raises(YuleGpuError):
        backend.dequantize(w, 16, 1, out)  # IQ2_XXS: no kernel reads it
    backend.free(w)
    backend.free(out)
