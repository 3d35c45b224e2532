"""Parity at the layer shapes of the Llama-3-8B and Llama-3-70B architectures (two layers each, so the
CPU runner finishes in seconds; mixture-of-depths needs 32 layers, yule-infer/src/model_runner.rs:463,
and stays off): logits within 1e-3 and the first greedy tokens identical, on the token-by-token path
and on the chunked tensor-core prefill.  Plus the largest matvec of those models against the threaded
qmv of yule-infer/src/model_runner.rs:152-244."""

import numpy as np
import pytest

from conftest import REL_TOL, guarded_rel_err as elementwise_rel_err
from test_gpu_runner import greedy_reference, guarded_rel_err, make_oracle_model
from yule_b200 import CudaTransformerRunner, DType, ModelConfig, synth

pytestmark = pytest.mark.gpu

# hidden 4096, 32 query / 8 KV heads of 128, FFN 14336, vocabulary 128256, Q4_K linears with a Q6_K output matrix
SHAPE_8B = ModelConfig(dim=4096, n_layers=2, n_heads=32, n_kv_heads=8, head_dim=128, vocab_size=128256, ff_dim=14336,
                       max_seq_len=64, rope_freq_base=500000.0)
# hidden 8192, 64 query / 8 KV heads of 128, FFN 28672, all Q4_K; a short vocabulary keeps the CPU side quick
SHAPE_70B = ModelConfig(dim=8192, n_layers=2, n_heads=64, n_kv_heads=8, head_dim=128, vocab_size=4096, ff_dim=28672,
                        max_seq_len=64, rope_freq_base=500000.0)

CASES = {"8b": (SHAPE_8B, dict(linear=DType.Q4_K, output=DType.Q6_K)), "70b": (SHAPE_70B, dict(linear=DType.Q4_K))}


@pytest.fixture(scope="module", params=["8b", "70b"])
def shaped_model(request, oracle):
    cfg, kw = CASES[request.param]
    weights = synth.synthetic_model(cfg, seed=31, std=0.02, **kw)
    return cfg, weights, make_oracle_model(oracle, cfg, weights)


def test_token_path_logits_and_greedy(backend, oracle, shaped_model):
    cfg, weights, ref = shaped_model
    ref.reset()
    prompt = synth.tokens(41, 4, cfg.vocab_size)
    want, margin = greedy_reference(oracle, ref, prompt, 8)
    ref.reset()
    want_logits = ref.prefill(prompt)
    run = CudaTransformerRunner(backend, cfg, weights, fused=True)
    got_logits = run.prefill(prompt)  # fewer than 16 tokens: one token step each
    assert guarded_rel_err(got_logits, want_logits) <= REL_TOL
    run.reset()
    got = run.generate_greedy(prompt, 8)
    assert np.array_equal(got, want), f"first mismatch at {np.argmax(got != want)}; min margin {margin:g}"
    run.close()


def test_chunked_prefill_logits_and_greedy(backend, oracle, shaped_model):
    cfg, weights, ref = shaped_model
    ref.reset()
    prompt = synth.tokens(43, 20, cfg.vocab_size)
    want, margin = greedy_reference(oracle, ref, prompt, 8)
    ref.reset()
    want_logits = ref.prefill(prompt)
    run = CudaTransformerRunner(backend, cfg, weights, fused=True)
    got_logits = run.prefill(prompt)  # 19 tokens through the tcgen05 GEMM, the last through the token step
    assert guarded_rel_err(got_logits, want_logits) <= REL_TOL
    run.reset()
    got = run.generate_greedy(prompt, 8)
    assert np.array_equal(got, want), f"first mismatch at {np.argmax(got != want)}; min margin {margin:g}"
    run.close()


@pytest.mark.parametrize("dtype", [DType.Q4_K, DType.Q6_K, DType.Q8_0, DType.Q4_0])
@pytest.mark.parametrize("batch", [1, 4, 7])
def test_vocabulary_matvec_against_threaded_qmv(backend, oracle, dtype, batch):
    """128256 x 4096 (the Llama-3 output matrix): the matvec's shared-memory ring wraps many times per CTA; one
    vector, four vectors in one pass of the batched kernels, seven as a pass of four and one of three."""
    n_rows, n_cols = 128256, 4096
    w = synth.random_blocks(dtype, 7, n_rows * n_cols // dtype.block_size)
    x = synth.normal(8, batch * n_cols)
    wh, xh, oh = backend.upload(w), backend.upload(x), backend.allocate(batch * n_rows * 4)
    backend.prepare_weights(wh, dtype, n_rows, n_cols)
    if batch == 1:
        backend.quantized_matmul(wh, xh, oh, n_rows, n_cols, dtype)
    else:
        backend.quantized_matmul_batched(wh, xh, oh, n_rows, n_cols, dtype, batch)
    y = backend.download(oh, batch * n_rows).reshape(batch, n_rows)
    for h in (wh, xh, oh):
        backend.free(h)
    for b in range(batch):
        ref = oracle.qmv(int(dtype), w, x[b * n_cols:(b + 1) * n_cols], n_rows, n_cols, simd=oracle.SCALAR, n_threads=0)
        assert elementwise_rel_err(y[b], ref) <= REL_TOL
