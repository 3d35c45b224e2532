"""Generates ``q4k_reference_asm.npz``: outputs of Yule's own hand-written AVX2 kernel
(yule-core/src/kernels/q4k_gemv_avx2.S, assembled unmodified into oracle/_ref/) on seeded Q4_K blocks.

Two groups of inputs:
* ``recipe_*`` — the block/activation recipe of Yule's AVX2-vs-scalar test (yule-core/src/simd/avx2.rs:409-440:
  xorshift seed 777, d = 0x3800, dmin = 0x2E66, scale bytes % 64, activations (r % 1000)/500 - 1);
* ``field_*``  — random-field blocks as the benchmarks use them (f16 d, dmin = |N(0, 0.002)|, all other
  bytes uniform) with N(0, 1) activations.

The fixture travels with the repository; this script only runs where a Yule checkout was reachable when
the oracle was built (it needs oracle/_ref/libyule_ref_q4k.so).  Run: ``python tests/golden/make_golden.py``.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as o  # noqa: E402
from yule_b200 import DType, synth  # noqa: E402

MASK = (1 << 64) - 1


def xorshift(s: int) -> int:
    s ^= (s << 13) & MASK
    s ^= s >> 7
    s ^= (s << 17) & MASK
    return s


def recipe_blocks(n: int):
    s = 777
    blocks, acts = np.zeros((n, 144), np.uint8), np.zeros((n, 256), np.float32)
    for k in range(n):
        b = blocks[k]
        b[0:4] = (0x00, 0x38, 0x66, 0x2E)
        for i in range(4, 144):
            s = xorshift(s)
            b[i] = s & 0xFF
        for i in range(4, 16):
            s = xorshift(s)
            b[i] = s % 64
        for i in range(256):
            s = xorshift(s)
            acts[k, i] = np.float32(s % 1000) / np.float32(500.0) - np.float32(1.0)
    return blocks, acts


def main() -> None:
    assert o.load_reference_asm(), "oracle/_ref/libyule_ref_q4k.so is missing"
    rb, ra = recipe_blocks(64)
    ry = np.array([o.reference_q4k_asm(rb[k], ra[k]) for k in range(64)], np.float32)
    fb = synth.random_blocks(DType.Q4_K, 4242, 64).reshape(64, 144)
    fa = synth.normal(4243, 64 * 256).reshape(64, 256)
    fy = np.array([o.reference_q4k_asm(fb[k], fa[k]) for k in range(64)], np.float32)
    np.savez_compressed(os.path.join(HERE, "q4k_reference_asm.npz"), recipe_blocks=rb, recipe_acts=ra,
                        recipe_out=ry, field_blocks=fb, field_acts=fa, field_out=fy)
    print("wrote q4k_reference_asm.npz", ry[:3], fy[:3])


if __name__ == "__main__":
    main()
