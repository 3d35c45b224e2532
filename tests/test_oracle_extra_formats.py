"""The CPU restatement of Yule's remaining block formats (Q4_1, Q5_0, Q5_1, Q8_1, Q2_K, Q3_K, Q5_K)
pinned to the known-answer tests of yule-core/src/dequant.rs:1405-1565 and :1598-1611, and checked
for self-consistency where the reference holds no vector (Q5_1, Q2_K)."""

import numpy as np
import pytest

from yule_b200 import DType, synth
from yule_b200.dtype import EXTRA_QUANTIZED


def one(value=0x3C):
    return value  # high byte of f16 1.0


def test_q4_1_kats(oracle):
    b = np.zeros(20, np.uint8)
    b[1] = b[3] = one()
    b[4] = 0xF0
    out = oracle.dequant(int(DType.Q4_1), b)
    assert out[0] == 1.0 and out[1] == 16.0 and out[2] == 1.0
    b[4] = 0
    assert abs(oracle.vec_dot(int(DType.Q4_1), b, np.ones(32, np.float32)) - 32.0) < 1e-4


def test_q5_0_kats(oracle):
    b = np.zeros(22, np.uint8)
    b[1] = one()
    b[2] = 0x01
    out = oracle.dequant(int(DType.Q5_0), b)
    assert out[0] == 0.0 and out[1] == -16.0
    b[6], b[2] = 0x5A, 0x02
    out = oracle.dequant(int(DType.Q5_0), b)
    assert out[0] == -6.0 and out[1] == 5.0
    b = np.zeros(22, np.uint8)
    b[1] = one()
    assert abs(oracle.vec_dot(int(DType.Q5_0), b, np.ones(32, np.float32)) + 512.0) < 1e-4


def test_q3_k_kats(oracle):
    b = np.zeros(110, np.uint8)
    b[109] = one()
    b[96], b[104], b[32] = 0x01, 0x02, 0x01  # scale[0] = 33 - 32 = 1, first weight's low bits = 1
    assert oracle.dequant(int(DType.Q3_K), b)[0] == -3.0
    b[0] = 0x01  # high bit of weight 0
    assert oracle.dequant(int(DType.Q3_K), b)[0] == 1.0


def test_q5_k_kats(oracle):
    b = np.zeros(176, np.uint8)
    b[1] = one()
    b[4], b[48] = 0x01, 0x05
    assert oracle.dequant(int(DType.Q5_K), b)[0] == 5.0
    b[16] = 0x01
    assert oracle.dequant(int(DType.Q5_K), b)[0] == 21.0


def test_q8_1_kats(oracle):
    b = np.zeros(36, np.uint8)
    b[1] = one()
    b[4], b[5] = 42, 0x80
    out = oracle.dequant(int(DType.Q8_1), b)
    assert out[0] == 42.0 and out[1] == -128.0


def test_q5_1_and_q2_k_by_hand(oracle):
    """No vector in the reference: the formulas of dequant.rs:124-138 and :196-214 on hand-built blocks."""
    b = np.zeros(24, np.uint8)
    b[1] = one()          # d = 1
    b[3] = 0x40           # m = 2
    b[4] = 0x01           # high bit of weight 0
    b[8] = 0x73           # weight 0 low nibble 3, weight 1 nibble 7
    out = oracle.dequant(int(DType.Q5_1), b)
    assert out[0] == 19.0 + 2.0 and out[1] == 7.0 + 2.0 and out[2] == 2.0
    b = np.zeros(84, np.uint8)
    b[81] = one()         # d = 1
    b[83] = 0x38          # dmin = 0.5
    b[0] = 0x23           # sub-block 0: scale 3, min 2
    b[16] = 0b11_10_01_00
    out = oracle.dequant(int(DType.Q2_K), b)
    assert list(out[:4]) == [-1.0, 2.0, 5.0, 8.0]
    assert np.all(out[16:] == 0.0)


@pytest.mark.parametrize("dtype", EXTRA_QUANTIZED)
def test_fused_dot_equals_dequantised_dot(oracle, dtype):
    """vec_dot (dequant.rs:1013-1207) against Σ dequant(w)·x in float64 on random-field blocks."""
    data = synth.random_blocks(dtype, seed=5 + int(dtype), n_blocks=64)
    bs, bb = dtype.block_size, dtype.size_of_block
    w = oracle.dequant(int(dtype), data).reshape(64, bs).astype(np.float64)
    x = synth.normal(9, bs)
    for i in range(64):
        got = float(oracle.vec_dot(int(dtype), data[i * bb:(i + 1) * bb], x))
        want = float(w[i] @ x.astype(np.float64))
        assert abs(got - want) <= 1e-4 * (np.abs(w[i]) @ np.abs(x)) + 1e-6


@pytest.mark.parametrize("dtype,levels", [(DType.Q4_1, 15), (DType.Q5_0, 31), (DType.Q5_1, 31), (DType.Q5_K, 31)])
def test_quantiser_round_trip(oracle, dtype, levels):
    """The synthetic-model quantisers write blocks the reference layout reads back within one step."""
    x = synth.normal(3, 256 * 64, std=0.05)
    back = oracle.dequant(int(dtype), synth.quantize(dtype, x))
    step = (x.max() - x.min()) / levels
    assert np.max(np.abs(back - x)) <= 0.75 * step
    assert np.corrcoef(back, x)[0, 1] > 0.995
