"""The oracle's mixture-of-experts FFN (yule-infer/src/model_runner.rs:813-958) on the CPU: the router against the
reference's own test (:1138-1186) and its definition, the expert sum against the dense FFN it must reduce to, the two
namings of the expert tensors against each other."""

import dataclasses

import numpy as np
import pytest

from test_gpu_runner import make_oracle_model
from yule_b200 import DType, ModelConfig, synth

CFG = ModelConfig(dim=256, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=32, vocab_size=256, ff_dim=512, max_seq_len=32,
                  n_experts=4, n_experts_used=2)


def moe_model(oracle, cfg, weights):
    m = oracle.Model(dim=cfg.dim, n_layers=cfg.n_layers, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                     vocab_size=cfg.vocab_size, ff_dim=cfg.ff_dim, max_seq_len=cfg.max_seq_len, norm_eps=cfg.norm_eps,
                     rope_freq_base=cfg.rope_freq_base, simd=oracle.SCALAR, n_experts=cfg.n_experts,
                     n_experts_used=cfg.n_experts_used)
    for name, (data, dt) in weights.items():
        m.set_tensor(name, data, int(dt))
    return m


def test_router_known_answer(oracle):
    """model_runner.rs:1138-1186: eight logits, two experts used → experts 2 and 4, weights that sum to 1."""
    probs, sel, w = oracle.moe_route([0.1, 0.05, 0.8, 0.02, 0.5, 0.03, 0.01, 0.3], 2)
    assert list(sel) == [2, 4]
    assert abs(float(w[0] + w[1]) - 1.0) < 1e-6 and w[0] > w[1] > 0
    assert abs(float(probs.sum()) - 1.0) < 1e-6


def test_router_definition_and_tie_order(oracle):
    logits = synth.normal(3, 16)
    probs, sel, w = oracle.moe_route(logits, 4)
    e = np.exp(logits.astype(np.float64) - logits.max())
    want = e / e.sum()
    assert np.allclose(probs, want, rtol=1e-6)
    order = np.argsort(-want, kind="stable")[:4]
    assert list(sel) == list(order)
    assert np.allclose(w, want[order] / want[order].sum(), rtol=1e-6)
    # equal probabilities keep index order (the CPU runner's sort is stable)
    _, sel, w = oracle.moe_route([0.5, 0.5, 0.5, 0.1], 2)
    assert list(sel) == [0, 1] and abs(float(w[0]) - 0.5) < 1e-6


def test_identical_experts_reduce_to_the_dense_ffn(oracle):
    """With every expert holding the same matrices the weighted sum of the chosen experts is the dense FFN's output
    (the weights sum to 1), whatever the router says."""
    dense_cfg = dataclasses.replace(CFG, n_experts=0, n_experts_used=0)
    dense = synth.synthetic_model(dense_cfg, seed=3, std=0.05, linear=DType.Q8_0)
    moe = {n: t for n, t in dense.items() if ".ffn_gate." not in n and ".ffn_up." not in n and ".ffn_down." not in n}
    for l in range(CFG.n_layers):
        router = synth.normal(40 + l, CFG.n_experts * CFG.dim)
        moe[f"blk.{l}.ffn_gate_inp.weight"] = (router.view(np.uint8), DType.F32)
        for proj in ("gate", "up", "down"):
            one = np.asarray(dense[f"blk.{l}.ffn_{proj}.weight"][0]).view(np.uint8)
            moe[f"blk.{l}.ffn_{proj}_exps.weight"] = (np.tile(one, CFG.n_experts), DType.Q8_0)
    a, b = make_oracle_model(oracle, dense_cfg, dense), moe_model(oracle, CFG, moe)
    for tok in (5, 77, 200):
        la, lb = a.decode_step(tok), b.decode_step(tok)
        assert np.abs(la - lb).max() <= 2e-5 * np.abs(la).max()


def test_packed_and_per_expert_tensors_agree(oracle):
    packed = synth.synthetic_model(CFG, seed=9, std=0.05, linear=DType.Q4_K, router=DType.F16)
    per_expert = synth.synthetic_model(CFG, seed=9, std=0.05, linear=DType.Q4_K, router=DType.F16, packed_experts=False)
    ff, dim = CFG.ff_dim, CFG.dim
    # the same expert matrices under the other naming: slices of the packed tensors
    for l in range(CFG.n_layers):
        for proj, rows, cols in (("gate", ff, dim), ("up", ff, dim), ("down", dim, ff)):
            whole = np.asarray(packed[f"blk.{l}.ffn_{proj}_exps.weight"][0]).view(np.uint8)
            per = whole.size // CFG.n_experts
            for e in range(CFG.n_experts):
                per_expert[f"blk.{l}.ffn_{proj}.{e}.weight"] = (whole[e * per:(e + 1) * per].copy(), DType.Q4_K)
        per_expert[f"blk.{l}.ffn_gate_inp.weight"] = packed[f"blk.{l}.ffn_gate_inp.weight"]
    a, b = moe_model(oracle, CFG, packed), moe_model(oracle, CFG, per_expert)
    for tok in (1, 2, 3, 250):
        assert np.array_equal(a.decode_step(tok), b.decode_step(tok))


def test_expert_choice_matters(oracle):
    """Different experts, and the router decides: swapping the router rows of two experts changes the logits."""
    w = synth.synthetic_model(CFG, seed=11, std=0.05, linear=DType.Q8_0)
    a = moe_model(oracle, CFG, w)
    la = a.decode_step(9)
    swapped = dict(w)
    r = np.asarray(w["blk.0.ffn_gate_inp.weight"][0]).view(np.float32).reshape(CFG.n_experts, CFG.dim).copy()
    r = r[::-1].copy()
    swapped["blk.0.ffn_gate_inp.weight"] = (r.reshape(-1).view(np.uint8), DType.F32)
    b = moe_model(oracle, CFG, swapped)
    assert not np.allclose(la, b.decode_step(9), rtol=1e-4)


def test_bad_expert_counts_fail(oracle):
    w = synth.synthetic_model(CFG, seed=11, std=0.05, linear=DType.Q8_0)
    m = moe_model(oracle, dataclasses.replace(CFG, n_experts_used=5), w)
    with pytest.raises(RuntimeError):
        m.decode_step(1)
