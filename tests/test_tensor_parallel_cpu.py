"""Row-sharded tensor parallelism, host logic only: two gloo ranks on the CPU each run the oracle's matvec
on their byte slice of the raw tensor; the all-gathered result must equal the unsharded one bit for bit
(row sharding does not change any row's summation order)."""

import os
import socket
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from oracle import oracle as o
    from yule_b200 import DType, parallel, synth
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    ok = True
    for dt in (DType.Q4_K, DType.Q6_K, DType.Q8_0, DType.Q4_0):
        n_rows, n_cols = 64, 512  # 64 rows split over 2, 4 or 8 ranks
        w = synth.random_blocks(dt, 7, n_rows * n_cols // dt.block_size)
        x = synth.normal(8, n_cols)
        mine = parallel.shard_rows(w, dt, n_rows, n_cols, rank, world)
        lo, hi = parallel.row_range(n_rows, rank, world)
        y_local = o.qmv(int(dt), mine, x, hi - lo, n_cols, n_threads=1)
        y = parallel.all_gather_rows(y_local, world)
        full = o.qmv(int(dt), w, x, n_rows, n_cols, n_threads=1)
        ok = ok and np.array_equal(y, full)
    # a whole sharded model keeps replicated tensors whole and cuts matrices by rows
    from yule_b200 import ModelConfig
    cfg = ModelConfig(dim=256, n_layers=1, n_heads=16, n_kv_heads=8, head_dim=16, vocab_size=512, ff_dim=512, max_seq_len=8)
    weights = synth.synthetic_model(cfg, seed=1, linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K)
    local = parallel.shard_model(cfg, weights, rank, world)
    ok = ok and local["blk.0.attn_q.weight"][0].size * world == weights["blk.0.attn_q.weight"][0].size
    ok = ok and local["token_embd.weight"][0].size == weights["token_embd.weight"][0].size
    ok = ok and local["blk.0.attn_norm.weight"][0].size == weights["blk.0.attn_norm.weight"][0].size
    # a shard generated on its own equals the slice of the whole model
    direct = synth.synthetic_model(cfg, seed=1, linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K, rank=rank, world=world)
    ok = ok and all(np.array_equal(np.asarray(local[k][0]), np.asarray(direct[k][0])) for k in local)
    open(os.path.join(out_dir, f"rank{rank}"), "w").write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_sharded_matvec_equals_full(native_libs, tmp_path, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}").read() == "ok"


def test_row_ranges_and_errors():
    from yule_b200 import parallel
    assert [parallel.row_range(128, r, 4) for r in range(4)] == [(0, 32), (32, 64), (64, 96), (96, 128)]
    with pytest.raises(ValueError):
        parallel.row_range(10, 0, 4)
    from yule_b200 import ModelConfig
    with pytest.raises(ValueError):
        parallel.local_config(ModelConfig(dim=256, n_layers=1, n_heads=6, n_kv_heads=2, head_dim=64, vocab_size=512,
                                          ff_dim=512), 4)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_exchange_region_layout(native_libs, world):
    """The offsets of the tensor-parallel exchange region at the 70B-class shapes: the gathered vectors and
    their (value, epoch) pair copies do not overlap, the pair copies are 16-byte aligned (they are read two
    pairs per 16-byte load), and the ranks' slices tile every vector exactly."""
    import ctypes as C
    from yule_b200 import _lib, synth
    cfg = synth.LLAMA3_70B
    rc = _lib.RunnerConfig(cfg.dim, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.vocab_size, cfg.ff_dim,
                           cfg.max_seq_len, cfg.norm_eps, cfg.rope_freq_base, 1)
    off = (C.c_uint64 * 8)()
    assert _lib.cuda_lib().yule_cuda_tp_exchange_layout(C.byref(rc), off) == 0
    qdim = cfg.n_heads * cfg.head_dim
    sizes = [qdim, cfg.dim, cfg.ff_dim, cfg.vocab_size, 2 * cfg.dim, 2 * cfg.ff_dim, 2 * qdim]
    regions = sorted((off[i], off[i] + sizes[i]) for i in range(7))
    for (a0, a1), (b0, b1) in zip(regions, regions[1:]):
        assert a1 <= b0
    assert regions[-1][1] <= off[7]
    for i in (4, 5, 6):
        assert off[i] % 4 == 0
    for n in (qdim, cfg.dim, cfg.ff_dim, cfg.vocab_size):
        assert n % world == 0
        per = n // world
        assert per % 8 == 0  # consumers read eight elements (four 16-byte pair loads) at a time
        assert [(r * per, (r + 1) * per) for r in range(world)][-1][1] == n
