"""Batched decode (several independent sequences per step, every linear one GEMM over the batch) against
the same sequences run one by one: on separate batch-1 runners of this library and on the CPU runner
restated in the oracle.  The reference serves one sequence per runner (yule-infer/src/lib.rs:169-216)."""

import numpy as np
import pytest

from conftest import REL_TOL
from test_gpu_runner import PREFILL_CFG, greedy_reference, guarded_rel_err, make_oracle_model
from yule_b200 import CudaTransformerRunner, DType, YuleGpuError, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,mix", [(12, "q4k"), (3, "q4k"), (32, "q4k_q6k"), (9, "q8_0"),
                                       (4, "q4k_q6k"), (7, "q4k_q6k"), (2, "q8_0")])  # up to eight rows: the batched matvec kernels
def test_batch_matches_independent_sequences(backend, oracle, batch, mix):
    kw = {"q4k": dict(linear=DType.Q4_K), "q4k_q6k": dict(linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K),
          "q8_0": dict(linear=DType.Q8_0)}[mix]
    cfg = PREFILL_CFG
    weights = synth.synthetic_model(cfg, seed=41, std=0.05, **kw)
    n_steps = 7
    toks = synth.tokens(43, batch * n_steps, cfg.vocab_size).reshape(batch, n_steps)  # a different stream per sequence
    run = CudaTransformerRunner(backend, cfg, weights, fused=True)
    got = [run.decode_batch(toks[:, i]) for i in range(n_steps)]  # [step][batch][vocab]
    # (a) the same sequences on a batch-1 runner of this library, one after the other
    single = CudaTransformerRunner(backend, cfg, weights, fused=True)
    ref = make_oracle_model(oracle, cfg, weights)
    for b in (0, batch // 2, batch - 1):
        single.reset()
        ref.reset()
        for i in range(n_steps):
            want_gpu = single.decode_step(int(toks[b, i]))
            want_cpu = ref.decode_step(int(toks[b, i]))
            assert guarded_rel_err(got[i][b], want_gpu) <= REL_TOL
            assert guarded_rel_err(got[i][b], want_cpu) <= REL_TOL
    # (b) rewinding starts every sequence again
    run.reset_batch()
    again = run.decode_batch(toks[:, 0])
    assert guarded_rel_err(again, got[0]) <= 1e-6
    # a different batch size on the same runner is refused
    with pytest.raises(YuleGpuError):
        run.decode_batch(toks[: batch - 1, 0])
    single.close()
    run.close()


def test_batch_greedy_streams(backend, oracle):
    cfg = PREFILL_CFG
    weights = synth.synthetic_model(cfg, seed=47, std=0.05, linear=DType.Q4_K)
    batch, n_prompt, n_gen = 10, 9, 20
    prompts = synth.tokens(49, batch * n_prompt, cfg.vocab_size).reshape(batch, n_prompt)
    run = CudaTransformerRunner(backend, cfg, weights, fused=True)
    got = run.generate_greedy_batch(prompts, n_gen)
    assert got.shape == (batch, n_gen)
    ref = make_oracle_model(oracle, cfg, weights)
    for b in (0, 4, 9):
        ref.reset()
        want, margin = greedy_reference(oracle, ref, prompts[b], n_gen)
        if margin > 1e-4:  # a near-tie may legitimately flip under re-ordered fp32 sums
            assert np.array_equal(got[b], want), f"sequence {b}: first mismatch at {np.argmax(got[b] != want)}"
        else:
            assert got[b][0] == want[0]
    run.close()
