"""The mixture-of-experts FFN (yule-infer/src/model_runner.rs:813-958), which Yule's GPU runner does not implement:
the CUDA runner against the CPU runner restated in the oracle — logits within 1e-3, the same greedy tokens — for
packed and per-expert tensors, F32 / F16 / block-quantised routers, and a model loaded from a GGUF image."""

import numpy as np
import pytest

from conftest import REL_TOL
from test_gpu_runner import guarded_rel_err
from test_oracle_moe import moe_model
from yule_b200 import CudaTransformerRunner, DType, ModelConfig, synth

pytestmark = pytest.mark.gpu

CFG = ModelConfig(dim=256, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=32, vocab_size=512, ff_dim=768, max_seq_len=64,
                  n_experts=8, n_experts_used=2)

CASES = {
    "packed_q4k_f32_router": dict(linear=DType.Q4_K, router=DType.F32),
    "packed_q6k_down_f16_router": dict(linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K, router=DType.F16),
    "per_expert_q8_0": dict(linear=DType.Q8_0, router=DType.F32, packed_experts=False),
    "quantised_router": dict(linear=DType.Q4_K, router=DType.Q8_0),
}


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("case", list(CASES))
def test_moe_matches_cpu_runner(backend, oracle, case, fused):
    weights = synth.synthetic_model(CFG, seed=23, std=0.05, **CASES[case])
    ref = moe_model(oracle, CFG, weights)
    run = CudaTransformerRunner(backend, CFG, weights, fused=fused)
    assert run.step_kind == 0  # the expert choice passes through the host: one kernel per dispatch
    prompt = synth.tokens(5, 6, CFG.vocab_size)
    got, want = run.prefill(prompt), ref.prefill(prompt)
    assert guarded_rel_err(got, want) <= REL_TOL
    tok = int(np.argmax(want))
    for _ in range(6):
        got, want = run.decode_step(tok), ref.decode_step(tok)
        assert guarded_rel_err(got, want) <= REL_TOL
        assert int(np.argmax(got)) == int(np.argmax(want))
        tok = int(np.argmax(want))
    run.reset()
    ref.reset()
    assert guarded_rel_err(run.prefill(prompt), ref.prefill(prompt)) <= REL_TOL
    run.close()


def test_three_of_five_experts(backend, oracle):
    cfg = ModelConfig(dim=256, n_layers=2, n_heads=4, n_kv_heads=4, head_dim=64, vocab_size=300, ff_dim=512, max_seq_len=32,
                      n_experts=5, n_experts_used=3)
    weights = synth.synthetic_model(cfg, seed=29, std=0.05, linear=DType.Q4_0)
    ref = moe_model(oracle, cfg, weights)
    run = CudaTransformerRunner(backend, cfg, weights, fused=False)
    for tok in (3, 299, 17):
        assert guarded_rel_err(run.decode_step(tok), ref.decode_step(tok)) <= REL_TOL
    run.close()


def test_moe_model_from_a_gguf_image(backend, oracle, tmp_path):
    import gguf_writer as gw
    from yule_b200.gguf import GgufFile, load_runner
    cfg = ModelConfig(dim=256, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=32, vocab_size=256, ff_dim=512, max_seq_len=32,
                      n_experts=4, n_experts_used=2)
    for packed in (True, False):
        weights = synth.synthetic_model(cfg, seed=31, std=0.05, linear=DType.Q4_K, packed_experts=packed)
        path = tmp_path / f"moe_{int(packed)}.gguf"
        path.write_bytes(gw.model_file(cfg, weights))
        g = GgufFile.open(str(path))
        got_cfg = g.model_config()
        assert (got_cfg.n_experts, got_cfg.n_experts_used, got_cfg.ff_dim) == (4, 2, 512)
        run = load_runner(backend, g)
        ref = moe_model(oracle, cfg, weights)
        for tok in (1, 100, 255):
            assert guarded_rel_err(run.decode_step(tok), ref.decode_step(tok)) <= REL_TOL
        run.close()
        g.close()


def test_refusals(backend):
    from yule_b200 import YuleGpuError
    weights = synth.synthetic_model(CFG, seed=23, std=0.05, linear=DType.Q4_K)
    import dataclasses
    with pytest.raises(YuleGpuError):
        CudaTransformerRunner(backend, dataclasses.replace(CFG, n_experts_used=9), weights)
    # a layer without its router
    partial = {n: t for n, t in weights.items() if n != "blk.1.ffn_gate_inp.weight"}
    run = CudaTransformerRunner(backend, CFG, partial, fused=False)
    with pytest.raises(YuleGpuError, match="ffn_gate_inp"):
        run.decode_step(1)
    run.close()
    # the device loop entry points need the graph modes
    run = CudaTransformerRunner(backend, CFG, weights, fused=True)
    with pytest.raises(YuleGpuError):
        run.generate_greedy([1, 2, 3], 4)
    run.close()
