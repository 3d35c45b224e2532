"""The oracle's sampler against the known answers of the reference's own tests
(yule-infer/src/sampler.rs:224-301) and against the definition of each step."""

import numpy as np

from yule_b200 import synth


def test_ct_gte_basic(oracle):  # sampler.rs:229-234
    assert oracle.ct_gte(1.0, 0.5) == 1.0
    assert oracle.ct_gte(0.5, 1.0) == 0.0
    assert oracle.ct_gte(1.0, 1.0) == 1.0


def test_argmax_finds_max(oracle):  # sampler.rs:236-240
    assert oracle.argmax(np.array([0.1, 0.3, 0.9, 0.2], np.float32)) == 2


def test_sample_ct_deterministic(oracle):  # sampler.rs:242-251
    probs = np.array([0.25, 0.25, 0.25, 0.25], np.float32)
    assert oracle.sample_ct(probs, 0.01) == 0
    assert oracle.sample_ct(probs, 0.3) == 1
    assert oracle.sample_ct(probs, 0.99) == 3


def test_sampler_returns_valid_token(oracle):  # sampler.rs:261-274
    logits = np.array([0.1, 5.0, 0.2, 0.3], np.float32)
    for r in np.linspace(0.0, 0.999, 50):
        tok = oracle.sample(logits, float(r), temperature=1.0, top_p=0.9, top_k=10, min_p=0.05, repetition_penalty=1.0)
        assert 0 <= tok < 4


def test_near_greedy_picks_max(oracle):  # sampler.rs:276-300
    logits = np.array([0.1, 0.2, 10.0, 0.3], np.float32)
    picks = [oracle.sample(logits, float(r), temperature=0.0001, top_p=1.0, top_k=0, min_p=0.0, repetition_penalty=1.0)
             for r in np.linspace(0.0, 0.999, 100)]
    assert picks.count(2) > 90


def test_steps_follow_their_definitions(oracle):
    logits = synth.normal(5, 200)
    # top-k keeps the entries >= sorted[k] of the descending order: k + 1 candidates without ties (sampler.rs:58-70)
    seen = {oracle.sample(logits, float(r), temperature=1.0, top_p=1.0, top_k=3, min_p=0.0, repetition_penalty=1.0)
            for r in np.linspace(0.0005, 0.9999, 400)}
    assert seen <= set(np.argsort(-logits)[:4].tolist()) and len(seen) >= 3
    # a repetition penalty pushes a positive logit down once per occurrence (sampler.rs:26-38)
    top = int(np.argmax(logits))
    base = sum(oracle.sample(logits, float(r), temperature=1.0, top_p=1.0, top_k=0, min_p=0.0, repetition_penalty=1.0) == top
               for r in np.linspace(0.0005, 0.9999, 400))
    pen = sum(oracle.sample(logits, float(r), temperature=1.0, top_p=1.0, top_k=0, min_p=0.0, repetition_penalty=2.0,
                            previous=[top, top]) == top for r in np.linspace(0.0005, 0.9999, 400))
    assert pen < base
    # top-p: the nucleus is the shortest descending prefix whose mass reaches top_p (sampler.rs:83-118)
    p = np.exp(logits - logits.max())
    p /= p.sum()
    order = np.argsort(-p)
    n_in = int(np.searchsorted(np.cumsum(p[order]), 0.5) + 1)
    seen = {oracle.sample(logits, float(r), temperature=1.0, top_p=0.5, top_k=0, min_p=0.0, repetition_penalty=1.0)
            for r in np.linspace(0.0005, 0.9999, 800)}
    assert seen <= set(order[:n_in].tolist())
