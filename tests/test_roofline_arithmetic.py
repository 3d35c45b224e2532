"""The algorithmic byte counts the roofline figures are built on: one matvec reads its weight tensor once plus x and
writes y; a decode token reads every matrix once.  The expected numbers are worked out here from the block sizes of
yule-core/src/dtype.rs:62-118 and the shapes of the three model architectures, independently of the helpers."""

import pytest

from yule_b200 import DType, synth
from yule_b200.dtype import matvec_bytes

BLOCK = {DType.Q4_0: (32, 18), DType.Q8_0: (32, 34), DType.Q4_K: (256, 144), DType.Q6_K: (256, 210)}


def by_hand(dt, rows, cols, batch=1):
    weights_per_block, block_bytes = BLOCK[dt]
    return rows * (cols // weights_per_block) * block_bytes + 4 * batch * cols + 4 * batch * rows


def test_the_headline_matvec():
    assert matvec_bytes(DType.Q4_K, 5632, 2048) == 6_488_064 + 8_192 + 22_528 == 6_518_784


@pytest.mark.parametrize("dt", list(BLOCK))
@pytest.mark.parametrize("shape", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336), (128256, 4096)])
@pytest.mark.parametrize("batch", [1, 4, 16])
def test_sweep_shapes(dt, shape, batch):
    assert matvec_bytes(dt, *shape, batch) == by_hand(dt, *shape, batch)


def test_weight_tensors_of_the_sweep():
    assert DType.Q4_K.tensor_bytes(4096, 4096) == DType.Q4_0.tensor_bytes(4096, 4096) == 9_437_184
    assert DType.Q6_K.tensor_bytes(4096, 4096) == 13_762_560
    assert DType.Q8_0.tensor_bytes(4096, 4096) == 17_825_792
    assert DType.Q4_K.tensor_bytes(128256, 4096) == 295_501_824
    assert DType.Q6_K.tensor_bytes(128256, 4096) == 430_940_160


def matrices_per_token(cfg, linear, ffn_down, output):
    """Bytes of every matrix a decode token reads once (the embedding table is read one row at a time)."""
    total = 0
    for name, (rows, cols) in cfg.tensor_shapes().items():
        if name == "token_embd.weight":
            continue
        dt = output if name == "output.weight" else (ffn_down if name.endswith("ffn_down.weight") else linear)
        total += dt.tensor_bytes(rows, cols)
    return total


def test_weight_bytes_per_decode_token():
    # TinyLlama architecture, Q4_K linears with Q6_K ffn_down and output: 22 layers of 27 746 304 B + 53 760 000 B
    assert matrices_per_token(synth.TINYLLAMA, DType.Q4_K, DType.Q6_K, DType.Q6_K) == 22 * 27_746_304 + 53_760_000 == 664_178_688
    # Llama-3-8B architecture, Q4_K linears, Q6_K output
    assert matrices_per_token(synth.LLAMA3_8B, DType.Q4_K, DType.Q4_K, DType.Q6_K) == 32 * 122_683_392 + 430_940_160 == 4_356_808_704
    # Llama-3-70B architecture, all Q4_K
    assert matrices_per_token(synth.LLAMA3_70B, DType.Q4_K, DType.Q4_K, DType.Q4_K) == 80 * 481_296_384 + 591_003_648 == 39_094_714_368
