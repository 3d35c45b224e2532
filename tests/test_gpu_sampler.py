"""The device sampler (Sampler::sample_with_history, yule-infer/src/sampler.rs:17-136) against its CPU
restatement in the oracle, on the same logits and the same random values.  Sums are trees on the device and
left-to-right on the CPU, so a pick may differ only when the random value lies within rounding distance of a
boundary of the cumulative distribution: such draws are recognised (float64 recomputation) and skipped."""

import numpy as np
import pytest

from test_gpu_runner import SMALL, make_oracle_model
from yule_b200 import CudaTransformerRunner, DType, YuleGpuError, synth

pytestmark = pytest.mark.gpu

CASES = {
    "defaults": dict(temperature=0.7, top_p=0.9, top_k=40, repetition_penalty=1.1, min_p=0.05),
    "plain": dict(temperature=1.0, top_p=1.0, top_k=0, repetition_penalty=1.0, min_p=0.0),
    "top_k_only": dict(temperature=1.0, top_p=1.0, top_k=7, repetition_penalty=1.0, min_p=0.0),
    "top_p_only": dict(temperature=1.3, top_p=0.6, top_k=0, repetition_penalty=1.0, min_p=0.0),
    "min_p_only": dict(temperature=0.5, top_p=1.0, top_k=0, repetition_penalty=1.0, min_p=0.2),
    "penalty": dict(temperature=1.0, top_p=1.0, top_k=0, repetition_penalty=1.7, min_p=0.0),
}


def near_boundary(oracle, logits, r, kw, previous, eps=5e-5):
    """True when moving r by eps changes the CPU pick: the draw sits on a boundary of the distribution."""
    picks = {oracle.sample(logits, float(np.clip(r + d, 0.0, 0.99999)), previous=previous, **kw) for d in (-eps, 0.0, eps)}
    return len(picks) > 1


@pytest.mark.parametrize("case", list(CASES))
@pytest.mark.parametrize("n", [4, 1000, 32000, 128256])
def test_device_sampler_matches_cpu(backend, oracle, case, n):
    kw = CASES[case]
    # peaked enough that the cumulative distribution has steps wider than the rounding of a vocabulary-long sum
    logits = ((3.0 if n <= 1000 else 8.0) * synth.normal(900 + n, n)).astype(np.float32)
    previous = synth.tokens(7, 50, n) if kw["repetition_penalty"] != 1.0 else np.zeros(0, np.uint32)
    if previous.size:
        previous[10:14] = previous[3]  # a token seen several times is penalised once per occurrence
    lh = backend.upload(logits)
    ph = backend.upload(previous) if previous.size else None
    checked = 0
    rs = np.random.default_rng(n).random(24).astype(np.float32)
    for r in rs:
        r = float(min(r, 0.999999))
        if near_boundary(oracle, logits, r, kw, previous):
            continue
        got = backend.sample(lh, n, r, previous=ph, n_previous=previous.size, **kw)
        want = oracle.sample(logits, r, previous=previous, **kw)
        assert got == want, f"r={r}"
        checked += 1
    assert checked >= 12
    backend.free(lh)
    if ph:
        backend.free(ph)


def test_degenerate_inputs(backend, oracle):
    # all the mass on one token; a single-token vocabulary; ties at the top-k threshold
    for logits in (np.array([0.0, 50.0, 0.0, 0.0], np.float32), np.array([1.5], np.float32),
                   np.array([1.0, 2.0, 2.0, 2.0, 0.5, 2.0], np.float32)):
        lh = backend.upload(logits)
        for r in (0.001, 0.37, 0.73, 0.99):
            kw = dict(temperature=1.0, top_p=0.95, top_k=2, repetition_penalty=1.0, min_p=0.01)
            assert backend.sample(lh, logits.size, r, **kw) == oracle.sample(logits, r, **kw)
        backend.free(lh)
    lh = backend.upload(np.zeros(4, np.float32))
    with pytest.raises(YuleGpuError):
        backend.sample(lh, 0, 0.5)  # empty logits (sampler.rs:19-21)
    with pytest.raises(YuleGpuError):
        backend.sample(lh, 4, 1.0)  # the random value lies in [0, 1)
    backend.free(lh)


def test_sampled_generation_feeds_picks_back(backend, oracle):
    """generate_sampled against the CPU runner driven by the oracle's sampler with the same random values."""
    cfg = SMALL
    weights = synth.synthetic_model(cfg, seed=61, std=0.05, linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K)
    prompt = synth.tokens(63, 8, cfg.vocab_size)
    kw = dict(temperature=0.9, top_p=0.95, top_k=20, repetition_penalty=1.2, min_p=0.02)
    run = CudaTransformerRunner(backend, cfg, weights, fused=True)
    seed, n_gen = 1234, 24
    got = run.generate_sampled(prompt, n_gen, seed, **kw)
    assert np.array_equal(got, run_again(run, prompt, n_gen, seed, kw))  # equal seeds, equal streams
    ref = make_oracle_model(oracle, cfg, weights)
    logits = ref.prefill(prompt)
    seq = list(prompt)
    for g in range(n_gen):
        r = CudaTransformerRunner.random_value(seed, g)
        if near_boundary(oracle, logits, r, kw, np.array(seq, np.uint32), eps=1e-3):
            break  # the streams may part here for a legitimate reason; everything before must agree
        want = oracle.sample(logits, r, previous=np.array(seq, np.uint32), **kw)
        assert got[g] == want, f"pick {g}"
        seq.append(want)
        logits = ref.decode_step(want)
    assert g >= 4
    run.close()


def run_again(run, prompt, n_gen, seed, kw):
    run.reset()
    return run.generate_sampled(prompt, n_gen, seed, **kw)
