"""GGML tensor types on the hot path — the subset of Yule's ``DType`` (yule-core/src/dtype.rs:13-58)
whose discriminant is the GGUF type id that crosses the C ABI."""

from __future__ import annotations

import enum


class DType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q8_0 = 8
    Q4_K = 12
    Q6_K = 14

    @property
    def block_size(self) -> int:
        """Weights per block (yule-core/src/dtype.rs:99-118)."""
        return {DType.F32: 1, DType.F16: 1, DType.Q4_0: 32, DType.Q8_0: 32, DType.Q4_K: 256, DType.Q6_K: 256}[self]

    @property
    def size_of_block(self) -> int:
        """Bytes per block (yule-core/src/dtype.rs:62-96)."""
        return {DType.F32: 4, DType.F16: 2, DType.Q4_0: 18, DType.Q8_0: 34, DType.Q4_K: 144, DType.Q6_K: 210}[self]

    def tensor_bytes(self, n_rows: int, n_cols: int) -> int:
        assert n_cols % self.block_size == 0
        return n_rows * (n_cols // self.block_size) * self.size_of_block


QUANTIZED = (DType.Q4_0, DType.Q8_0, DType.Q4_K, DType.Q6_K)


def matvec_bytes(dtype: DType, n_rows: int, n_cols: int, batch: int = 1) -> int:
    """Algorithmic bytes of one dequant-matvec: the weight tensor once, x in, y out."""
    return dtype.tensor_bytes(n_rows, n_cols) + 4 * batch * n_cols + 4 * batch * n_rows
