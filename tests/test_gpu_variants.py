"""Architecture variants of the dense forward pass that Yule's CPU runner handles and its GPU runner drops
(yule-infer/src/model_runner.rs: Q/K/V bias :640-651, sliding window :688-696, partial RoPE :78-99 + :430-434,
attention / final logit softcaps :716-721 + :1027-1032, Gemma norm offset and embedding scale :246-275 + :568-574,
GeGLU :974-978, post-attention / post-FFN norms :764-779 + :985-999): the CUDA runner against the CPU runner
restated in the oracle, logits within 1e-3 and identical greedy tokens, in both runner modes."""

import dataclasses

import numpy as np
import pytest

from conftest import REL_TOL
from test_gpu_runner import greedy_reference, guarded_rel_err, make_oracle_model
from yule_b200 import CudaTransformerRunner, DType, ModelConfig, synth

pytestmark = pytest.mark.gpu

BASE = ModelConfig(dim=256, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=32, vocab_size=512, ff_dim=768, max_seq_len=64)


def with_extras(cfg, weights, *, bias=False, post_norms=False, seed=0):
    """Adds the optional tensors of a variant: Q/K/V biases (F32, one layer F16) and Gemma2's post-norm weights."""
    w = dict(weights)
    q, kv = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    for l in range(cfg.n_layers):
        if bias:
            for name, n in (("attn_q.bias", q), ("attn_k.bias", kv), ("attn_v.bias", kv)):
                b = synth.normal(seed + 17 * l + n, n, std=0.2)
                if l == 1:
                    w[f"blk.{l}.{name}"] = (b.astype(np.float16).view(np.uint8), DType.F16)
                else:
                    w[f"blk.{l}.{name}"] = (b.view(np.uint8), DType.F32)
        if post_norms:
            for name in ("attn_post_norm.weight", "ffn_post_norm.weight"):
                g = (0.1 * synth.normal(seed + 31 * l + len(name), cfg.dim)).astype(np.float32)
                w[f"blk.{l}.{name}"] = (g.view(np.uint8), DType.F32)
    return w


VARIANTS = {
    "qkv_bias": (dict(), dict(bias=True)),
    "sliding_window": (dict(sliding_window=5), dict()),
    "partial_rope": (dict(rotary_dim=16), dict()),
    "attn_softcap": (dict(attn_logit_softcap=2.0), dict()),
    "logit_softcap": (dict(logit_softcap=3.0), dict()),
    "gemma": (dict(norm_weight_offset=1.0, geglu=True, attn_logit_softcap=50.0, logit_softcap=30.0, norm_eps=1e-6),
              dict(post_norms=True)),
    "everything": (dict(norm_weight_offset=1.0, geglu=True, attn_logit_softcap=4.0, logit_softcap=8.0, sliding_window=6,
                        rotary_dim=8), dict(bias=True, post_norms=True)),
}


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("variant", list(VARIANTS))
@pytest.mark.parametrize("mix", ["q4k_q6k", "q8_0"])
def test_variant_matches_cpu_runner(backend, oracle, variant, fused, mix):
    cfg_kw, extra_kw = VARIANTS[variant]
    cfg = dataclasses.replace(BASE, **cfg_kw)
    kw = dict(linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K) if mix == "q4k_q6k" else dict(linear=DType.Q8_0)
    std = 0.02 if cfg.norm_weight_offset else 0.05  # Gemma's sqrt(dim) embedding scale keeps the activations in range
    weights = with_extras(cfg, synth.synthetic_model(cfg, seed=11, std=std, **kw), seed=5, **extra_kw)
    ref = make_oracle_model(oracle, cfg, weights)
    run = CudaTransformerRunner(backend, cfg, weights, fused=fused)
    prompt = synth.tokens(13, 12, cfg.vocab_size)  # longer than the windows above
    got, want = run.prefill(prompt), ref.prefill(prompt)
    assert guarded_rel_err(got, want) <= REL_TOL
    for tok in (5, 499, 17, 230):
        got, want = run.decode_step(tok), ref.decode_step(tok)
        assert guarded_rel_err(got, want) <= REL_TOL
    kv = cfg.n_kv_heads * cfg.head_dim
    assert guarded_rel_err(backend.download(run.buffer("k_cache", 1), 16 * kv), ref.k_cache(1, 16)) <= REL_TOL
    if fused:
        run.reset()
        ref.reset()
        want_toks, margin = greedy_reference(oracle, ref, prompt, 16)
        got_toks = run.generate_greedy(prompt, 16)
        assert np.array_equal(got_toks, want_toks), f"first mismatch at {np.argmax(got_toks != want_toks)}; min margin {margin:g}"
    run.close()


def test_long_prompt_with_window_uses_token_path(backend, oracle):
    """A prompt long enough for the chunked tensor-core prefill: a variant model must not take it (that path
    implements the Llama op sequence only) and still match."""
    cfg = dataclasses.replace(BASE, sliding_window=7)
    weights = synth.synthetic_model(cfg, seed=21, std=0.05, linear=DType.Q4_K)
    ref = make_oracle_model(oracle, cfg, weights)
    run = CudaTransformerRunner(backend, cfg, weights, fused=True)
    prompt = synth.tokens(23, 40, cfg.vocab_size)
    assert guarded_rel_err(run.prefill(prompt), ref.prefill(prompt)) <= REL_TOL
    run.close()
