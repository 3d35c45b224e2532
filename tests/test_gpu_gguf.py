"""A model file → HBM → logits: the loader (yule_cuda_runner_load_gguf) gives the same runner as uploading
the same tensors by hand (GpuTransformerRunner::upload_weights, yule-infer/src/gpu_runner.rs:171-254)."""

import numpy as np
import pytest

from yule_b200 import CudaTransformerRunner, DType, GgufFile, ModelConfig, YuleGpuError, load_runner, synth

import gguf_writer as gw
from test_gpu_runner import guarded_rel_err, make_oracle_model
from conftest import REL_TOL

pytestmark = pytest.mark.gpu

CFG = ModelConfig(dim=256, n_layers=3, n_heads=4, n_kv_heads=2, head_dim=64, vocab_size=512, ff_dim=768, max_seq_len=96)


@pytest.mark.parametrize("mix", ["q4k_q6k_f16norm", "q8_0_tied", "q5k_q6k", "q5_0_q4_1"])
def test_loaded_runner_equals_hand_built_runner(backend, oracle, tmp_path, mix):
    if mix == "q4k_q6k_f16norm":
        weights = synth.synthetic_model(CFG, seed=21, std=0.05, linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K,
                                        norm_dtype=DType.F16)
    elif mix == "q5k_q6k":  # the layout of a Q5_K_M file: formats Yule's own GPU backends refuse
        weights = synth.synthetic_model(CFG, seed=25, std=0.05, linear=DType.Q5_K, ffn_down=DType.Q6_K, output=DType.Q6_K)
    elif mix == "q5_0_q4_1":
        weights = synth.synthetic_model(CFG, seed=26, std=0.05, linear=DType.Q5_0, ffn_down=DType.Q4_1, token_embd=DType.Q5_1)
    else:
        weights = synth.synthetic_model(CFG, seed=22, std=0.05, linear=DType.Q8_0)
        del weights["output.weight"]  # tied embedding: the loader falls back to token_embd (gpu_runner.rs:209-210)
    path = tmp_path / "model.gguf"
    path.write_bytes(gw.model_file(CFG, weights))
    g = GgufFile.open(str(path))
    run = load_runner(backend, g, fused=True)
    assert run.config.dim == CFG.dim and run.config.ff_dim == CFG.ff_dim and run.config.max_seq_len == CFG.max_seq_len
    hand = CudaTransformerRunner(backend, CFG, weights, fused=True)
    prompt = synth.tokens(23, 20, CFG.vocab_size)
    a, b = run.prefill(prompt), hand.prefill(prompt)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))  # same bytes, same kernels
    ref = make_oracle_model(oracle, CFG, weights)
    assert guarded_rel_err(a, ref.prefill(prompt)) <= REL_TOL
    assert np.array_equal(run.generate_greedy([], 8), hand.generate_greedy([], 8))
    run.close()
    hand.close()
    g.close()


def test_missing_tensor_and_unsupported_format_are_refused(backend, tmp_path):
    weights = synth.synthetic_model(CFG, seed=24, std=0.05, linear=DType.Q4_K)
    broken = dict(weights)
    del broken["blk.1.ffn_up.weight"]
    g = GgufFile.parse(gw.model_file(CFG, broken))
    with pytest.raises(YuleGpuError) as e:
        load_runner(backend, g)
    assert "tensor not found: blk.1.ffn_up.weight" in str(e.value)
    # a format the kernels do not read (IQ2_XXS, id 16, 66 bytes per 256): parsed, but refused at load with the reference's words
    shapes = CFG.tensor_shapes()
    tensors = {n: (d, int(t), (shapes[n][1], shapes[n][0]) if n in shapes else (CFG.dim,)) for n, (d, t) in weights.items()}
    rows, cols = shapes["blk.0.attn_q.weight"]
    tensors["blk.0.attn_q.weight"] = (np.zeros(rows * cols // 256 * 66, np.uint8), 16, (cols, rows))
    g2 = GgufFile.parse(gw.build(gw.llama_metadata(CFG), tensors))
    with pytest.raises(YuleGpuError) as e:
        load_runner(backend, g2)
    assert "unsupported dtype" in str(e.value)
