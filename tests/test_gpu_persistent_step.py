"""The token step as one persistent kernel (``fused=2``): same contract as the multi-kernel runner — logits within
1e-3 of the CPU runner restated in the oracle (yule-infer/src/model_runner.rs:533-1036), identical greedy
streams — on every head shape the kernel is instantiated for, on both format mixes it covers, through short and
long contexts (one split, several splits with a merge), and its bounded waits give up cleanly."""

import time

import numpy as np
import pytest

from conftest import REL_TOL
from test_gpu_runner import greedy_reference, guarded_rel_err, make_oracle_model
from yule_b200 import CudaTransformerRunner, DType, ModelConfig, synth

pytestmark = pytest.mark.gpu

YULE_ERR_DEVICE_STATUS = 7

# grouped-query shape (group, head_dim) = (4, 64); vocabulary not a multiple of 16 (ragged last tile)
SMALL = ModelConfig(dim=512, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=64, vocab_size=1000, ff_dim=1024,
                    max_seq_len=160)
MIXES = {"q4k_q6k": dict(linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K),
         "q4k": dict(linear=DType.Q4_K),
         "q4k_o_q6k": dict(linear=DType.Q4_K, output=DType.Q6_K)}


def persistent_runner(backend, cfg, weights):
    run = CudaTransformerRunner(backend, cfg, weights, fused=2)
    assert run.step_kind == 2, "the persistent kernel does not cover a model it should cover"
    return run


@pytest.mark.parametrize("mix", list(MIXES))
def test_logits_match_cpu_runner(backend, oracle, mix):
    weights = synth.synthetic_model(SMALL, seed=11, std=0.05, **MIXES[mix])
    ref = make_oracle_model(oracle, SMALL, weights)
    run = persistent_runner(backend, SMALL, weights)
    prompt = synth.tokens(3, 9, SMALL.vocab_size)
    assert guarded_rel_err(run.prefill(prompt), ref.prefill(prompt)) <= REL_TOL
    for tok in (5, 999, 17, 0):
        assert guarded_rel_err(run.decode_step(tok), ref.decode_step(tok)) <= REL_TOL
    assert run.pos == ref.pos == 13
    kv = SMALL.n_kv_heads * SMALL.head_dim
    for layer in (0, 2):
        assert guarded_rel_err(backend.download(run.buffer("k_cache", layer), 13 * kv), ref.k_cache(layer, 13)) <= REL_TOL
    run.reset()
    ref.reset()
    assert guarded_rel_err(run.prefill(prompt), ref.prefill(prompt)) <= REL_TOL
    run.close()


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 1, 64), (4, 4, 64), (8, 1, 128), (8, 2, 128), (4, 4, 128)],
                         ids=["g8_hd64", "g1_hd64", "g8_hd128", "g4_hd128", "g1_hd128"])
def test_head_shapes(backend, oracle, heads, kv_heads, head_dim):
    cfg = ModelConfig(dim=512, n_layers=2, n_heads=heads, n_kv_heads=kv_heads, head_dim=head_dim, vocab_size=512,
                      ff_dim=768, max_seq_len=96)
    weights = synth.synthetic_model(cfg, seed=13, std=0.05, linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K)
    ref = make_oracle_model(oracle, cfg, weights)
    run = persistent_runner(backend, cfg, weights)
    prompt = synth.tokens(5, 40, cfg.vocab_size)  # head_dim 128: the attention unit needs two passes from position 32 on
    assert guarded_rel_err(run.prefill(prompt), ref.prefill(prompt)) <= REL_TOL
    for tok in (1, 2, 3):
        assert guarded_rel_err(run.decode_step(tok), ref.decode_step(tok)) <= REL_TOL
    run.close()


@pytest.mark.parametrize("ff_dim,down", [(4608, DType.Q6_K), (4096, DType.Q4_K)], ids=["three_chunks_q6k", "two_chunks_q4k"])
def test_rows_wider_than_a_stage(backend, oracle, ff_dim, down):
    """A down projection with more than 2048 columns is several stages per tile; with few tiles the two groups of a CTA
    share a tile, take half of the stages each and add their partial sums in shared memory."""
    cfg = ModelConfig(dim=512, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=64, vocab_size=1000, ff_dim=ff_dim, max_seq_len=64)
    weights = synth.synthetic_model(cfg, seed=17, std=0.05, linear=DType.Q4_K, ffn_down=down, output=DType.Q6_K)
    ref = make_oracle_model(oracle, cfg, weights)
    run = persistent_runner(backend, cfg, weights)
    prompt = synth.tokens(4, 6, cfg.vocab_size)
    assert guarded_rel_err(run.prefill(prompt), ref.prefill(prompt)) <= REL_TOL
    for tok in (11, 12, 13):
        assert guarded_rel_err(run.decode_step(tok), ref.decode_step(tok)) <= REL_TOL
    run.close()


def test_greedy_stream_identical(backend, oracle):
    weights = synth.synthetic_model(SMALL, seed=5, std=0.05, linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K)
    ref = make_oracle_model(oracle, SMALL, weights)
    prompt = synth.tokens(6, 8, SMALL.vocab_size)
    want, margin = greedy_reference(oracle, ref, prompt, 60)
    run = persistent_runner(backend, SMALL, weights)
    got = run.generate_greedy(prompt, 60)
    assert np.array_equal(got, want), f"first mismatch at {np.argmax(got != want)}; min margin {margin:g}"
    more = run.generate_greedy([], 10)  # continues from the pick held on the device
    run.reset()
    again = run.generate_greedy(prompt, 70)
    assert np.array_equal(again[:60], want) and np.array_equal(again[60:], more)
    run.close()


def test_long_context_uses_several_passes_and_splits(backend, oracle):
    """A unit of the attention phase takes its positions 64 at a time (head_dim 64) with a running soft-max, and past
    256 positions a KV head is split over several CTAs whose partial results the last one to finish merges.  The
    prompt goes through the chunked prefill, which shares the KV caches with the persistent kernel."""
    cfg = ModelConfig(dim=512, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=64, vocab_size=1000, ff_dim=1024, max_seq_len=640)
    weights = synth.synthetic_model(cfg, seed=21, std=0.05, linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K)
    ref = make_oracle_model(oracle, cfg, weights)
    run = persistent_runner(backend, cfg, weights)
    prompt = synth.tokens(9, 130, cfg.vocab_size)  # positions 129..: three passes of one unit
    assert guarded_rel_err(run.prefill(prompt), ref.prefill(prompt)) <= REL_TOL
    for tok in (7, 8):
        assert guarded_rel_err(run.decode_step(tok), ref.decode_step(tok)) <= REL_TOL
    more = synth.tokens(10, 400, cfg.vocab_size)  # on to position 532: three splits of three passes each, merged
    got, want = run.prefill(more), ref.prefill(more)
    assert guarded_rel_err(got, want) <= REL_TOL
    for tok in (9, 10, 11):
        assert guarded_rel_err(run.decode_step(tok), ref.decode_step(tok)) <= REL_TOL
    run.close()


def test_tinyllama_shape_against_the_multi_kernel_step(backend):
    """Two layers of the configs[1] architecture: the persistent kernel against the multi-kernel graph on the
    same weights (the oracle comparison at this size is the job of test_gpu_layer_shapes)."""
    cfg = ModelConfig(dim=2048, n_layers=2, n_heads=32, n_kv_heads=4, head_dim=64, vocab_size=32000, ff_dim=5632,
                      max_seq_len=256)
    weights = synth.synthetic_model(cfg, seed=31, linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K)
    a = persistent_runner(backend, cfg, weights)
    b = CudaTransformerRunner(backend, cfg, weights, fused=1)
    assert b.step_kind == 1
    prompt = synth.tokens(2, 12, cfg.vocab_size)
    assert guarded_rel_err(a.prefill(prompt), b.prefill(prompt)) <= REL_TOL
    ga, gb = a.generate_greedy([], 48), b.generate_greedy([], 48)
    assert np.array_equal(ga, gb), f"first mismatch at {np.argmax(ga != gb)}"
    a.close()
    b.close()


def test_models_it_does_not_cover_keep_the_graph(backend, oracle):
    weights = synth.synthetic_model(SMALL, seed=3, std=0.05, linear=DType.Q8_0)
    ref = make_oracle_model(oracle, SMALL, weights)
    run = CudaTransformerRunner(backend, SMALL, weights, fused=2)
    assert run.step_kind == 1
    prompt = synth.tokens(3, 6, SMALL.vocab_size)
    assert guarded_rel_err(run.prefill(prompt), ref.prefill(prompt)) <= REL_TOL
    run.close()


def test_waits_run_out_and_report(backend, oracle):
    """Every consumer of the kernel waits for an epoch that nothing writes: the first wait to run out of its
    (tiny) budget records the status word, the others return at once, the kernel ends by itself and the host
    sees YULE_ERR_DEVICE_STATUS.  The runner then works again."""
    weights = synth.synthetic_model(SMALL, seed=11, std=0.05, linear=DType.Q4_K, ffn_down=DType.Q6_K, output=DType.Q6_K)
    ref = make_oracle_model(oracle, SMALL, weights)
    run = persistent_runner(backend, SMALL, weights)
    prompt = synth.tokens(3, 9, SMALL.vocab_size)
    want = ref.prefill(prompt)
    assert guarded_rel_err(run.prefill(prompt), want) <= REL_TOL
    backend.synchronize()
    t0 = time.time()
    assert run.selftest_bounded_wait(2_000_000) == YULE_ERR_DEVICE_STATUS  # about a millisecond of SM clock
    assert time.time() - t0 < 5.0  # one budget, not one per wait
    backend.synchronize()  # the report cleared the status word
    run.reset()
    assert guarded_rel_err(run.prefill(prompt), want) <= REL_TOL
    run.close()
