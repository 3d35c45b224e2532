"""Output-row tensor parallelism for quantized linears: the host-side partitioning logic.

Every quantized linear computes ``out[row] = dot(dequant(W[row, :]), x)``, so its rows are independent:
rank ``r`` of ``N`` owns rows ``[r*n/N, (r+1)*n/N)`` — a contiguous byte slice of the raw GGUF tensor, no
repacking — and the full output is the concatenation (all-gather) of the ranks' slices.  Q/K/V row shards
coincide with head shards (``n_heads`` and ``n_kv_heads`` must be multiples of ``N``), so RoPE, the KV cache
and attention stay rank-local.  Yule itself has no multi-device code; this layer has no counterpart there.
"""

from __future__ import annotations

import numpy as np

from .dtype import DType
from .runner import ModelConfig


def row_range(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Rows owned by ``rank``: an even split (``n_rows`` must be a multiple of ``world``)."""
    if n_rows % world:
        raise ValueError(f"{n_rows} rows do not split evenly over {world} ranks")
    per = n_rows // world
    return rank * per, (rank + 1) * per


def shard_rows(data, dtype: DType, n_rows: int, n_cols: int, rank: int, world: int) -> np.ndarray:
    """The raw bytes of this rank's rows of a ``[n_rows][n_cols]`` quantized tensor (a view, not a copy)."""
    raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    row_bytes = dtype.tensor_bytes(1, n_cols)
    if raw.size != n_rows * row_bytes:
        raise ValueError("tensor size does not match its shape")
    lo, hi = row_range(n_rows, rank, world)
    return raw[lo * row_bytes:hi * row_bytes]


# Which matrices are sharded by output rows, and what their input is.
_ROW_SHARDED = ("attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight", "ffn_gate.weight",
                "ffn_up.weight", "ffn_down.weight")


def local_config(cfg: ModelConfig, world: int) -> ModelConfig:
    """Per-rank view of the attention shape: each rank holds ``n_heads/world`` query and ``n_kv_heads/world`` KV heads."""
    if cfg.n_heads % world or cfg.n_kv_heads % world or cfg.ff_dim % world or cfg.dim % world or cfg.vocab_size % world:
        raise ValueError(f"model dimensions do not split evenly over {world} ranks")
    return cfg


def shard_model(cfg: ModelConfig, weights: dict, rank: int, world: int) -> dict:
    """Per-rank weights: every matrix cut by output rows, norms and the embedding table replicated."""
    local_config(cfg, world)
    shapes = cfg.tensor_shapes()
    out = {}
    for name, (data, dt) in weights.items():
        if name == "output.weight" or name.endswith(_ROW_SHARDED):
            rows, cols = shapes[name]
            out[name] = (shard_rows(data, dt, rows, cols, rank, world), dt)
        else:
            out[name] = (data, dt)  # token_embd.weight and the norm vectors are replicated
    return out


def all_gather_rows(local: np.ndarray, world: int, group=None) -> np.ndarray:
    """Concatenate the ranks' output slices in rank order (``torch.distributed`` all-gather)."""
    import torch
    import torch.distributed as dist
    t = torch.from_numpy(np.ascontiguousarray(local))
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t, group=group)
    return torch.cat(parts).numpy()
