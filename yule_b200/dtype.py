"""GGML tensor types the kernels read — the subset of Yule's ``DType`` (yule-core/src/dtype.rs:13-58)
whose discriminant is the GGUF type id that crosses the C ABI."""

from __future__ import annotations

import enum


class DType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14

    @property
    def block_size(self) -> int:
        """Weights per block (yule-core/src/dtype.rs:99-118)."""
        return 1 if self in (DType.F32, DType.F16) else 256 if self.name.endswith("_K") else 32

    @property
    def size_of_block(self) -> int:
        """Bytes per block (yule-core/src/dtype.rs:62-96)."""
        return {DType.F32: 4, DType.F16: 2, DType.Q4_0: 18, DType.Q4_1: 20, DType.Q5_0: 22, DType.Q5_1: 24,
                DType.Q8_0: 34, DType.Q8_1: 36, DType.Q2_K: 84, DType.Q3_K: 110, DType.Q4_K: 144, DType.Q5_K: 176,
                DType.Q6_K: 210}[self]

    def tensor_bytes(self, n_rows: int, n_cols: int) -> int:
        assert n_cols % self.block_size == 0
        return n_rows * (n_cols // self.block_size) * self.size_of_block


QUANTIZED = (DType.Q4_0, DType.Q8_0, DType.Q4_K, DType.Q6_K)
# Formats served by the element-wise matvec (no tuned kernel, no tensor-core GEMM).
EXTRA_QUANTIZED = (DType.Q4_1, DType.Q5_0, DType.Q5_1, DType.Q8_1, DType.Q2_K, DType.Q3_K, DType.Q5_K)


def matvec_bytes(dtype: DType, n_rows: int, n_cols: int, batch: int = 1) -> int:
    """Algorithmic bytes of one dequant-matvec: the weight tensor once, x in, y out."""
    return dtype.tensor_bytes(n_rows, n_cols) + 4 * batch * n_cols + 4 * batch * n_rows
