"""Benchmark of the quantized-decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[1]): TinyLlama-1.1B-architecture decode — 22 layers, hidden 2048, 32 query /
4 KV heads (head_dim 64), SwiGLU FFN 5632, vocab 32000; random-init N(0, 0.02) weights quantised to
Q4_K (output and ffn_down Q6_K), fp32 KV cache, batch 1, 32-token random prompt, 128 greedy tokens.
One *step* is one such job.  The metric is decode tokens per second (the 128 generated tokens; the
prompt pass is timed separately).

`value`  — inputs resident in HBM: prompt feed and greedy loop run on the device (argmax included),
           timed with CUDA events on the library's stream.
`e2e`    — the same job through the reference-facing ModelRunner calls (prefill / decode_step) with
           host buffers: every step uploads the token and position and downloads the vocab-sized logits, and the
           argmax runs on the host.
`roofline` — the Q4_K dequant-matvec kernel at the TinyLlama FFN-up shape (BASELINE.json configs[0]:
           5632x2048, 1000 launches) over a ring of weight copies larger than L2, replayed from a
           CUDA graph and timed with CUDA events; achieved = algorithmic bytes per launch / average
           launch duration, peak = measured copy bandwidth of this pool's B200s.
`cpu_baseline` — the CPU restatement of the reference's runner (its own AVX2 Q4_K assembly kernel where
           built) on the host cores, on a bounded sample of the same job.

With --gpus N > 1 (launched under torchrun, one rank per GPU) every rank decodes its own independent
sequence with its own replica of the model — batch-1 decode of a model that fits one GPU has no
exchange step — and `value` is the sum over ranks divided by the slowest rank's time (weak scaling).

`tp` — measured in the same run at every N: batch-1 decode of the Llama-3-70B-architecture model
       (BASELINE.json configs[4], every linear Q4_K, ~39 GB) with the output rows of every linear sharded over
       the N GPUs and the activations exchanged over NVLink peer memory (strong scaling: one sequence, N GPUs).
       Carries ms/token, tokens/s, the per-GPU fraction of the HBM roofline, and `tp_check`: a two-layer model
       of the same layer shapes run on N GPUs and on one, logits compared bit for bit and greedy tokens compared.

`--impl reference` — the CPU runner (the oracle's restatement of the reference, its own Q4_K assembly kernel
       where built) on the same job: the same 32-token prompt, then greedy tokens until 128 or a time budget.
"""

from __future__ import annotations

import argparse
import faulthandler
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_PROMPT, N_GEN = 32, 128
# DRAM bytes of one 5632x2048 launch of the ring kernel, from the ncu capture summarised in the named file
RING_TRAFFIC_BYTES = 6534144
RING_TRAFFIC_SOURCE = "profiles/qmv_q4k_ring_5632x2048.md (dram__bytes_read.sum + dram__bytes_write.sum of one launch, ncu capture)"
METRIC = "batch-1 decode tokens/s; Q4_K matvec achieved HBM GB/s vs B200 peak"
UNIT = "tokens/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def host_argmax_last(logits: np.ndarray) -> int:
    """argmax with ties to the highest index (yule-infer/src/sampler.rs:150-163)."""
    return int(logits.size - 1 - np.argmax(logits[::-1]))


def build_model_70b(rank: int, world: int, which: str = "c4"):
    """BASELINE.json configs[4]: Llama-3-70B architecture, every linear Q4_K (~39 GB), row-sharded over `world` ranks;
    configs[3]: Llama-3-8B architecture, Q4_K linears with a Q6_K output matrix.
    To bound host time the quantised N(0, 0.02) tensors of one layer are generated once and uploaded for all
    the layers (distinct device buffers, so HBM traffic is that of different layers)."""
    from yule_b200 import DType, parallel, synth
    cfg = synth.LLAMA3_70B if which == "c4" else synth.LLAMA3_8B
    one = synth.synthetic_model(ModelConfigOneLayer(cfg), seed=70, linear=DType.Q4_K,
                                output=DType.Q4_K if which == "c4" else DType.Q6_K, token_embd=DType.Q4_K)
    weights = {}
    for name, val in one.items():
        if name.startswith("blk.0."):
            for l in range(cfg.n_layers):
                weights[name.replace("blk.0.", f"blk.{l}.")] = val
        else:
            weights[name] = val
    if which == "c4":
        weights["token_embd.weight"] = weights["output.weight"]  # same bytes: only one row per token is read
    if world > 1:
        weights = parallel.shard_model(cfg, weights, rank, world)
    prompt = synth.tokens(7, N_PROMPT, cfg.vocab_size)
    return cfg, weights, prompt


def ModelConfigOneLayer(cfg):
    import dataclasses
    return dataclasses.replace(cfg, n_layers=1)


def build_model(rank: int, linear: str = "Q4_K"):
    from yule_b200 import DType, synth
    cfg = synth.TINYLLAMA
    weights = synth.synthetic_model(cfg, seed=2024, linear=DType[linear], ffn_down=DType.Q6_K, output=DType.Q6_K)
    prompt = synth.tokens(99 + rank, N_PROMPT, cfg.vocab_size)
    return cfg, weights, prompt


def small_batch_decode(backend, cfg, weights, n_prompt: int = 8, n_gen: int = 64):
    """The same model serving a few independent sequences per step (own KV caches and positions, device picks):
    every linear reads its weights once per step for up to four sequences (batched matvec kernels) or for all of
    them (GEMM, from thirteen sequences).  Device time per step over `n_prompt + n_gen` steps, tokens/s over all sequences."""
    from yule_b200 import CudaTransformerRunner, synth
    out = {}
    for batch in (4, 8, 12, 16):
        run = CudaTransformerRunner(backend, cfg, weights, fused=1)
        prompts = synth.tokens(7 + batch, batch * n_prompt, cfg.vocab_size).reshape(batch, n_prompt)
        run.generate_greedy_batch(prompts, 4)  # warm-up: buffers, graph
        run.reset_batch()
        backend.synchronize()
        backend.event_reset()
        e0 = backend.event_record()
        run.generate_greedy_batch(prompts, n_gen)  # the prompt tokens are steps of the same kind
        e1 = backend.event_record()
        ms = backend.event_elapsed_ms(e0, e1)
        steps = n_prompt + n_gen
        out[f"batch_{batch}"] = {"steps": steps, "ms_per_step": round(ms / steps, 4),
                                 "tokens_per_s": round(batch * steps / (ms * 1e-3), 1),
                                 "linears": "batched matvec kernels" if batch <= 12 else "tcgen05 GEMM"}
        run.close()
    return out


def decode_bytes_per_token(cfg, weights, pos: int, tp_world: int = 1) -> int:
    """Algorithmic HBM bytes one GPU reads per decode token: every matrix (shard) once, the embedding row,
    and this GPU's KV rows of positions [0, pos] for every layer (K and V)."""
    total = 0
    for name, (data, dt) in weights.items():
        if name == "token_embd.weight":
            total += data.size // cfg.vocab_size
        else:
            total += data.size
    total += 2 * cfg.n_layers * (pos + 1) * (cfg.n_kv_heads // tp_world) * cfg.head_dim * 4
    return total


def matvec_ring_roofline(backend, peaks, peak_kind, iters: int = 1000) -> dict:
    """configs[0]: Q4_K 5632x2048 matvec, `iters` launches rotating over copies that together exceed
    twice the L2, captured once into a CUDA graph and replayed; CUDA-event time / launches."""
    from yule_b200 import DType, matvec_bytes, synth
    n_rows, n_cols, dt = 5632, 2048, DType.Q4_K
    per = dt.tensor_bytes(n_rows, n_cols)
    copies = 80  # 80 x 6.49 MB = 519 MB > 2 x 126 MB L2
    ring = np.concatenate([synth.random_blocks(dt, 1000 + c, n_rows * n_cols // 256) for c in range(8)])
    ring = np.tile(ring, copies // 8)
    wh = backend.upload(ring)
    xh = backend.upload(synth.normal(7, n_cols))
    oh = backend.allocate(n_rows * 4)
    backend.graph_begin()
    for i in range(iters):
        backend.quantized_matmul_at(wh, (i % copies) * per, xh, oh, n_rows, n_cols, dt)
    graph = backend.graph_end()
    for _ in range(3):
        backend.graph_launch(graph)
    backend.synchronize()
    times = []
    for _ in range(5):
        backend.event_reset()
        e0 = backend.event_record()
        backend.graph_launch(graph)
        e1 = backend.event_record()
        times.append(backend.event_elapsed_ms(e0, e1))
    backend.graph_destroy(graph)
    for h in (wh, xh, oh):
        backend.free(h)
    ms = statistics.median(times)
    bytes_per_launch = matvec_bytes(dt, n_rows, n_cols)
    achieved = bytes_per_launch * iters / (ms * 1e-3) / 1e9
    peak = float(peaks["hbm_gbs"])
    return {"bound": "hbm", "kernel": "qmv_q4k_ring_kernel",
            "workload": "Q4_K 5632x2048 matvec x1000 over an 80-copy ring (519 MB); the launches are independent calls of the "
                        "trait method (same input vector), so each overlaps with its predecessor and only its stores wait for it",
            "achieved": round(achieved, 1), "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
            "frac": round(achieved / peak, 4), "bytes_per_launch": bytes_per_launch,
            "us_per_launch": round(ms * 1e3 / iters, 3),
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch in the committed ncu capture: not measured
            # in this run
            "traffic": RING_TRAFFIC_BYTES, "traffic_source": RING_TRAFFIC_SOURCE}


def reference_cuda_kernel_leg(peaks) -> dict:
    """The reference's own CUDA kernel for the same matvec (yule-gpu/kernels/cuda/qmv_q4_k.cu, compiled unmodified
    for sm_100a into oracle/_ref/ and launched with its launch shape, yule-gpu/src/cuda/kernels.rs:236-243: one
    256-thread block per row) on the same 5632x2048 ring: what a recompile of the reference gives on this GPU."""
    try:
        from oracle import ref_cuda
        from yule_b200 import DType, matvec_bytes, synth
        if not ref_cuda.available(int(DType.Q4_K)):
            return {"unavailable": "oracle/_ref holds no compiled reference kernel (no Yule checkout was reachable at build time)"}
        n_rows, n_cols, dt = 5632, 2048, DType.Q4_K
        per, copies = dt.tensor_bytes(n_rows, n_cols), 80
        ring = np.concatenate([synth.random_blocks(dt, 1000 + c, n_rows * n_cols // 256) for c in range(8)])
        ring = np.tile(ring, copies // 8)
        us = ref_cuda.time_ring(int(dt), ring, per, copies, synth.normal(7, n_cols), n_rows, n_cols, launches=200)
        nbytes = matvec_bytes(dt, n_rows, n_cols)
        gbs = nbytes / us / 1e3
        return {"kernel": "qmv_q4_k_kernel (reference, one block per row)", "workload": "Q4_K 5632x2048 matvec x200 over the same 80-copy ring",
                "us_per_launch": round(us, 3), "achieved": round(gbs, 1), "unit": "GB/s", "frac": round(gbs / float(peaks["hbm_gbs"]), 4)}
    except Exception as e:  # a missing driver binding or module must not take the bench line down
        return {"unavailable": f"{type(e).__name__}: {e}"}


def large_shape_rooflines(backend, peaks) -> dict:
    """The same matvec kernels on shapes large enough to be bandwidth-bound (BASELINE.json configs[2]'s 128256x4096,
    Q4_K and Q6_K, batch 1) and the tcgen05 GEMM on a prefill-sized problem: what the kernels do when launch
    and dependency latency do not dominate.  Weights stream from HBM over a ring of copies."""
    from yule_b200 import DType, microbench
    out = {}
    peak = float(peaks["hbm_gbs"])
    for dt in (DType.Q4_K, DType.Q6_K):
        r = microbench.run(backend, dt, 128256, 4096, 1, 20, True, reps=3)
        out[f"{dt.name}_128256x4096_batch1"] = {"bound": "hbm", "achieved": r["gbs"], "peak": peak, "unit": "GB/s",
                                                "frac": round(r["gbs"] / peak, 4), "us_per_launch": r["us_per_launch"]}
    r = microbench.run(backend, DType.Q4_K, 4096, 14336, 512, 10, True, reps=3)
    tpeak = float(peaks.get("bf16_tflops", 0) or 0)
    out["Q4_K_gemm_4096x14336_x512"] = {"bound": "tensor", "achieved": r["tflops"], "peak": tpeak, "unit": "TFLOP/s",
                                        "frac": round(r["tflops"] / tpeak, 4) if tpeak else None,
                                        "us_per_launch": r["us_per_launch"],
                                        "note": "useful FLOPs; the kernel issues two MMAs per product (fp16 hi/lo activations)"}
    return out


def cpu_forward_tokens_per_s(cfg, weights, prompt, budget_s: float, max_tokens: int):
    """Decode tokens/s of the CPU runner restated in the oracle, all host threads, on a bounded sample of the
    same job: the same prompt token by token (untimed, as the prompt pass of the GPU arm), then greedy decode
    steps until `budget_s` seconds or `max_tokens` tokens."""
    from oracle import oracle as o
    have_asm = o.load_reference_asm()
    simd = o.AVX2_ASM if have_asm else (o.AVX2 if o.lib.yo_have_avx2() else o.SCALAR)
    m = o.Model(dim=cfg.dim, n_layers=cfg.n_layers, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads,
                head_dim=cfg.head_dim, vocab_size=cfg.vocab_size, ff_dim=cfg.ff_dim, max_seq_len=cfg.max_seq_len,
                norm_eps=cfg.norm_eps, rope_freq_base=cfg.rope_freq_base, simd=simd, n_threads=0)
    for name, (data, dt) in weights.items():
        m.set_tensor(name, data, int(dt))
    logits = m.prefill(prompt)
    n, t0 = 0, time.perf_counter()
    while n < max_tokens and (time.perf_counter() - t0) < budget_s:
        logits = m.decode_step(o.argmax(logits))
        n += 1
    dt_s = time.perf_counter() - t0
    cores = o.lib.yo_hardware_threads()
    kind = "port"
    sample = (f"{n} of the {max_tokens} greedy decode tokens after the same {len(prompt)}-token prompt (time-bounded), "
              f"TinyLlama-arch Q4_K/Q6_K, {'reference q4k_gemv_avx2.S for Q4_K blocks, ' if have_asm else ''}"
              f"{'AVX2' if simd != o.SCALAR else 'scalar'} fused dots, one thread per row chunk per matvec")
    return n / dt_s, cores, kind, sample, n, dt_s


WORKLOAD_C1 = ("configs[1] TinyLlama-1.1B-arch decode, {linear} linears, Q6_K output+ffn_down, fp32 KV, batch 1, "
               "{n_prompt}-token prompt + {n_gen} greedy tokens per step")


def run_reference(args, rank: int, world: int) -> int:
    if rank != 0:
        return 0
    cfg, weights, prompt = build_model(0)
    total_tokens, total_s = 0, 0.0
    cores = kind = sample = None
    for _ in range(args.warmup):
        cpu_forward_tokens_per_s(cfg, weights, prompt[:2], budget_s=0.5, max_tokens=2)
    for _ in range(args.steps):
        tps, cores, kind, sample, n, dt_s = cpu_forward_tokens_per_s(cfg, weights, prompt, budget_s=4.0, max_tokens=N_GEN)
        total_tokens += n
        total_s += dt_s
    value = total_tokens / total_s
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * total_s / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_C1.format(linear="Q4_K", n_prompt=N_PROMPT, n_gen=N_GEN),
                       "parallelism": "host cores of rank 0 (the reference has no multi-device path)",
                       "sample": sample},
            "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)
    return 0


def measure_tp(args, rank: int, world: int, local_rank: int, dist, peaks) -> dict | None:
    """configs[4] at world size N: batch-1 decode of the Llama-3-70B-architecture model, output rows of every
    linear sharded over the N GPUs (one layer's tensors generated once and uploaded for all 80 layers, each
    rank generating only its own rows).  Before the timing, a two-layer model of the same layer shapes is run
    on N GPUs and (on rank 0) on one GPU: logits compared bit for bit, greedy tokens compared."""
    import dataclasses
    from yule_b200 import CudaB200Backend, CudaTransformerRunner, DType, YuleGpuError, synth

    def gather_max(v: float) -> float:
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    n_prompt, n_gen = (8, 8) if args.small else (args.tp_prompt, args.tp_gen)
    full = synth.LLAMA3_70B
    out = {"workload": f"configs[4] Llama-3-70B-arch decode, all linears Q4_K (one layer's tensors repeated for the "
                       f"{full.n_layers} layers), fp32 KV, batch 1, {n_prompt}-token prompt + {n_gen} greedy tokens",
           "world": world, "scaling": "strong",
           "exchange": ("none (one GPU)" if world == 1 else
                        "(value, epoch) pairs stored into every rank's peer-mapped buffer from the producer's epilogue, "
                        "polled by the consumer; logits through the exchange kernel; NVLS/multimem not used")}
    tpb = CudaB200Backend(local_rank)
    try:
        if world > 1:
            ids = [CudaB200Backend.tp_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            tpb.tp_init(rank, world, ids[0])
            tpb.set_wait_budget(600_000_000)  # ~0.3 s: a lost peer ends the step quickly with a status, not a stall
        # ── parity: two layers, N GPUs against one ────────────────────────────────────────────────
        small = dataclasses.replace(full, n_layers=2, vocab_size=8192, max_seq_len=64)
        w_loc = synth.synthetic_model(small, seed=71, linear=DType.Q4_K, rank=rank, world=world)
        prompt = synth.tokens(11, 6, small.vocab_size)
        run = CudaTransformerRunner(tpb, small, w_loc, fused=True)
        logits_tp = run.prefill(prompt).copy()
        run.reset()
        toks_tp = run.generate_greedy(prompt, 12)
        run.close()
        if world > 1 and rank == 0:
            one = CudaB200Backend(local_rank)
            w_all = synth.synthetic_model(small, seed=71, linear=DType.Q4_K)
            run1 = CudaTransformerRunner(one, small, w_all, fused=True)
            logits_1 = run1.prefill(prompt).copy()
            run1.reset()
            toks_1 = run1.generate_greedy(prompt, 12)
            run1.close()
            one.close()
            scale = float(np.abs(logits_1).max())
            out["tp_check"] = {"world": world, "layers": 2,
                               "logits_bit_identical": bool(np.array_equal(logits_tp.view(np.uint32), logits_1.view(np.uint32))),
                               "logits_max_rel_diff": float(np.abs(logits_tp - logits_1).max() / max(scale, 1e-30)),
                               "greedy_identical": bool(np.array_equal(toks_tp, toks_1))}
        elif world == 1:
            out["tp_check"] = {"world": 1, "note": "the one-GPU run is the reference of the check"}
        del w_loc
        # ── timing: the 80-layer model ────────────────────────────────────────────────────────────
        # 1024 positions suffice for the prompt + generated tokens and bound the KV caches of the 32-sequence batch
        cfg = dataclasses.replace(full, max_seq_len=1024) if not args.small else dataclasses.replace(full, n_layers=4, max_seq_len=256)
        one_layer = synth.synthetic_model(dataclasses.replace(cfg, n_layers=1), seed=70, linear=DType.Q4_K, rank=rank, world=world)
        weights = {}
        for name, val in one_layer.items():
            if name.startswith("blk.0."):
                for l in range(cfg.n_layers):
                    weights[name.replace("blk.0.", f"blk.{l}.")] = val
            elif name != "token_embd.weight":
                weights[name] = val
        # the embedding table is replicated and only one row per token is read: a sixteenth of it is generated
        # and repeated (rows are self-contained runs of blocks)
        part = synth.random_quantized(DType.Q4_K, synth.tensor_seed(70, "token_embd.weight"), cfg.vocab_size // 16 * cfg.dim)
        weights["token_embd.weight"] = (np.tile(part, 16), DType.Q4_K)
        prompt = synth.tokens(7, n_prompt, cfg.vocab_size)
        run = CudaTransformerRunner(tpb, cfg, weights, fused=True)

        def job():
            run.reset()
            e0 = tpb.event_record()
            run.generate_greedy(prompt, 0)
            e1 = tpb.event_record()
            toks = run.generate_greedy([], n_gen)
            e2 = tpb.event_record()
            return tpb.event_elapsed_ms(e0, e1), tpb.event_elapsed_ms(e1, e2), toks

        job()
        tpb.synchronize()
        tpb.event_reset()
        if dist is not None:
            dist.barrier()
        reps = 1 if args.small else 2
        pre_ms = dec_ms = 0.0
        for _ in range(reps):
            p_ms, d_ms, _ = job()
            pre_ms += p_ms
            dec_ms += d_ms
        tpb.synchronize()
        dec_ms = gather_max(dec_ms)
        pre_ms = gather_max(pre_ms)
        bpt = decode_bytes_per_token(cfg, weights, n_prompt + n_gen // 2, tp_world=world)
        ms_tok = dec_ms / (reps * n_gen)
        gbs = bpt / (ms_tok * 1e-3) / 1e9
        out.update({"ms_per_token": round(ms_tok, 4), "tokens_per_s": round(1e3 / ms_tok, 2),
                    "prefill_tokens_per_s": round(n_prompt * reps / (pre_ms * 1e-3), 1),
                    "hbm_bytes_per_token_per_gpu": bpt, "achieved_gbs_per_gpu": round(gbs, 1),
                    "frac_of_peak_per_gpu": round(gbs / float(peaks["hbm_gbs"]), 4),
                    "dominant_kernel": "qmv_q4k_mma_kernel (Q4_K matvec, about 95 % of the token step; attention and the "
                                       "logits exchange are the rest)"})
        # ── configs[4] batch 32: 32 independent sequences decoded together, every linear one GEMM per step ──
        nb, bp, bg = (8, 4, 4) if args.small else (32, args.tp_prompt, args.tp_gen // 2)
        prompts = synth.tokens(17, nb * bp, cfg.vocab_size).reshape(nb, bp)
        run.generate_greedy_batch(prompts, bg)  # warm-up: allocations, graph capture
        tpb.synchronize()
        tpb.event_reset()
        if dist is not None:
            dist.barrier()
        e0 = tpb.event_record()
        run.generate_greedy_batch(prompts, bg)
        e1 = tpb.event_record()
        b_ms = gather_max(tpb.event_elapsed_ms(e0, e1))
        steps = bp + bg
        step_ms = b_ms / steps
        kv_bytes = 2 * cfg.n_layers * nb * (bp + bg // 2) * (cfg.n_kv_heads // world) * cfg.head_dim * 4
        wbytes = decode_bytes_per_token(cfg, weights, 0, tp_world=world)
        out["batch32"] = {"sequences": nb, "prompt_tokens": bp, "generated_tokens": bg, "ms_per_step": round(step_ms, 4),
                          "tokens_per_s": round(nb * 1e3 / step_ms, 1),
                          "weight_bytes_per_step_per_gpu": wbytes,
                          "achieved_gbs_per_gpu": round((wbytes + kv_bytes) / (step_ms * 1e-3) / 1e9, 1),
                          "frac_of_peak_per_gpu": round((wbytes + kv_bytes) / (step_ms * 1e-3) / 1e9 / float(peaks["hbm_gbs"]), 4),
                          "path": "tcgen05 GEMM per linear over the 32 rows (prompt positions are steps of the same kind)"}
        run.close()
    except YuleGpuError as e:
        out["error"] = f"{e.code}: {e.message}"
    finally:
        tpb.close()
    return out if rank == 0 else None


def run_ours(args, rank: int, world: int, local_rank: int) -> int:
    import ctypes as C
    from yule_b200 import CudaB200Backend, CudaTransformerRunner

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v: float) -> float:
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    backend = CudaB200Backend(local_rank)
    tp = args.workload in ("c3", "c4")
    if tp:
        if world > 1:
            ids = [CudaB200Backend.tp_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            backend.tp_init(rank, world, ids[0])
        cfg, weights, prompt = build_model_70b(rank, world, args.workload)
    else:
        cfg, weights, prompt = build_model(rank, args.linear)
    runner = CudaTransformerRunner(backend, cfg, weights, fused=1 if ((tp and world > 1) or args.step == "graph") else 2)
    step_kind = runner.step_kind

    def job():
        """One configs[1] job on the device; returns (prefill ms, decode ms, tokens)."""
        runner.reset()
        e0 = backend.event_record()
        runner.generate_greedy(prompt, 0)
        e1 = backend.event_record()
        toks = runner.generate_greedy([], N_GEN)
        e2 = backend.event_record()
        return backend.event_elapsed_ms(e0, e1), backend.event_elapsed_ms(e1, e2), toks

    for _ in range(max(args.warmup, 3)):
        job()
    backend.synchronize()
    backend.event_reset()
    launches0 = backend.launch_count()
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    backend.synchronize()
    prefill_ms, decode_ms = 0.0, 0.0
    first_tokens = None
    for _ in range(args.steps):
        p, d, toks = job()
        prefill_ms += p
        decode_ms += d
        first_tokens = toks if first_tokens is None else first_tokens
    backend.synchronize()
    barrier()
    launches = backend.launch_count() - launches0

    # end-to-end through prefill / decode_step with host logits and host argmax
    logits = np.empty(cfg.vocab_size, np.float32)
    e2e_ms = 0.0
    e2e_tokens_match = True
    for it in range(args.steps):
        runner.reset()
        lg = runner.prefill(prompt)
        backend.event_reset()
        e0 = backend.event_record()
        toks = []
        for _ in range(N_GEN):
            t = host_argmax_last(lg)
            toks.append(t)
            lg = runner.decode_step(t, out=logits)
        e1 = backend.event_record()
        e2e_ms += backend.event_elapsed_ms(e0, e1)
        if it == 0:
            e2e_tokens_match = bool(np.array_equal(np.array(toks, np.uint32), first_tokens))
    clocks = sampler.stop()

    decode_ms_max = max_over_ranks(decode_ms)
    e2e_ms_max = max_over_ranks(e2e_ms)
    # replicas: every rank decodes its own sequence; tensor parallelism: all ranks decode one sequence
    total_tokens = N_GEN * args.steps * (1 if tp else world)
    value = total_tokens / (decode_ms_max * 1e-3)
    e2e_value = total_tokens / (e2e_ms_max * 1e-3)

    peaks, peak_kind = measured_peaks()
    tp_obj = None
    if not tp and not args.no_tp:
        tp_obj = measure_tp(args, rank, world, local_rank, dist, peaks)

    small_batch = None
    if rank == 0 and not tp and not args.small:
        small_batch = small_batch_decode(backend, cfg, weights)

    if rank == 0:
        roof = matvec_ring_roofline(backend, peaks, peak_kind, iters=20 if args.small else 1000)
        roof_large = None if (args.small or world > 1 or args.workload != "c1") else large_shape_rooflines(backend, peaks)
        ref_kernel = None if (args.small or world > 1 or args.workload != "c1") else reference_cuda_kernel_leg(peaks)
        mid_pos = N_PROMPT + N_GEN // 2
        bpt = decode_bytes_per_token(cfg, weights, mid_pos, tp_world=world if tp else 1)
        per_gpu_tok_s = N_GEN * args.steps / (decode_ms * 1e-3)
        decode_gbs = bpt * per_gpu_tok_s / 1e9
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            tps, cores, kind, sample, _, _ = cpu_forward_tokens_per_s(cfg, weights, prompt, budget_s=10.0, max_tokens=N_GEN)
            cpu = {"value": round(tps, 3), "unit": UNIT, "cores": cores, "kind": kind, "sample": sample}
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "warmup_requested": args.warmup, "ms_per_step": round((prefill_ms + decode_ms) / args.steps, 3),
            "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": ({"workload": ("configs[4] Llama-3-70B-arch decode, all linears Q4_K" if args.workload == "c4" else
                                     "configs[3] Llama-3-8B-arch, Q4_K linears, Q6_K output, prompt through the chunked GEMM prefill on one GPU") +
                                    f" (one layer's tensors repeated for the {cfg.n_layers} layers), fp32 KV, batch 1, "
                                    f"{N_PROMPT}-token prompt + {N_GEN} greedy tokens per step",
                        "parallelism": f"tp{world}: output rows of every linear sharded over {world} GPU(s), "
                                       "NCCL all-gather of activations",
                        "l2": "weights read per token per GPU (GBs) exceed the 126 MB L2; no flush needed"}
                       if tp else
                       {"workload": WORKLOAD_C1.format(linear=args.linear, n_prompt=N_PROMPT, n_gen=N_GEN),
                        "parallelism": f"{world} independent replica(s), one sequence per GPU",
                        "l2": f"weights read per token ({bpt / 1e6:.0f} MB) exceed the 126 MB L2; no flush needed"}),
            "decode": {"token_step": {1: "fused kernels replayed from a CUDA graph", 2: "one persistent kernel per token"}[step_kind],
                       "ms_per_token": round(decode_ms / (N_GEN * args.steps), 4),
                       "prefill_tokens_per_s": round(N_PROMPT * args.steps / (prefill_ms * 1e-3), 1),
                       "hbm_bytes_per_token": bpt, "achieved_gbs": round(decode_gbs, 1),
                       "frac_of_peak": round(decode_gbs / float(peaks["hbm_gbs"]), 4),
                       "greedy_stream_matches_host_argmax_path": e2e_tokens_match,
                       "several_sequences": small_batch},
            "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": 8 * N_GEN,
                    "d2h_bytes_per_step": 4 * cfg.vocab_size * N_GEN,
                    "path": "ModelRunner prefill/decode_step over the C ABI, host logits + host argmax"},
            "gpu_launches": int(launches), "roofline": roof, "roofline_large_shapes": roof_large, "reference_cuda_kernel": ref_kernel,
            "cpu_baseline": cpu,
            "clocks": clocks, "tp": tp_obj,
        }
        print(json.dumps(line), flush=True)
    runner.close()
    backend.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main() -> int:
    faulthandler.enable()  # a crash in native code leaves the Python stack on stderr
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["c1", "c3", "c4"], default="c1",
                    help="c1: TinyLlama-arch decode, one replica per GPU (default).  c3: Llama-3-8B-arch, 2048-token "
                         "prompt + 256 tokens.  c4: Llama-3-70B-arch decode (512-token prompt + "
                         "256 tokens).  c3/c4 shard the output rows of every linear over the GPUs (tensor parallelism)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--step", choices=["persistent", "graph"], default="persistent",
                    help="token step of the configs[1] runner: one persistent kernel (default) or the multi-kernel CUDA graph")
    ap.add_argument("--no-tp", action="store_true", help="leave out the `tp` object (the 70B-arch tensor-parallel decode)")
    ap.add_argument("--tp-prompt", type=int, default=64, help="prompt tokens of the `tp` measurement")
    ap.add_argument("--tp-gen", type=int, default=128, help="generated tokens of the `tp` measurement")
    ap.add_argument("--small", action="store_true",
                    help="profiling-sized run: 4-token prompt + 4 tokens, 20 ring launches, no CPU leg")
    ap.add_argument("--linear", default="Q4_K", choices=["Q4_K", "Q5_K", "Q8_0", "Q4_0", "Q5_0"],
                    help="diagnostic: block format of the c1 workload's linears (the metric is quoted on Q4_K)")
    ap.add_argument("--prompt-tokens", type=int, default=0, help="diagnostic: override the workload's prompt length")
    ap.add_argument("--gen-tokens", type=int, default=0, help="diagnostic: override the workload's generated tokens")
    args = ap.parse_args()
    global N_PROMPT, N_GEN
    if args.workload == "c4":
        N_PROMPT, N_GEN = 512, 256
        args.no_cpu_baseline = True  # the CPU runner needs seconds per token at this size
    if args.workload == "c3":
        N_PROMPT, N_GEN = 2048, 256
        args.no_cpu_baseline = True
    if args.small:
        N_PROMPT, N_GEN = 4, 4
        args.no_cpu_baseline = True
    N_PROMPT, N_GEN = args.prompt_tokens or N_PROMPT, args.gen_tokens or N_GEN
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    return run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    sys.exit(main())
