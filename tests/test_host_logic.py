"""Host-side logic that needs no GPU: format registry, synthetic generator, quantisers, byte models."""

import numpy as np

from yule_b200 import DType, matvec_bytes, synth


def test_dtype_registry():
    assert [int(d) for d in (DType.F32, DType.F16, DType.Q4_0, DType.Q8_0, DType.Q4_K, DType.Q6_K)] == [0, 1, 2, 8, 12, 14]
    assert DType.Q4_K.size_of_block == 144 and DType.Q6_K.size_of_block == 210
    assert DType.Q4_0.size_of_block == 18 and DType.Q8_0.size_of_block == 34
    assert DType.Q4_K.tensor_bytes(5632, 2048) == 6_488_064
    assert matvec_bytes(DType.Q4_K, 5632, 2048) == 6_518_784


def test_generator_is_seeded_and_thread_independent(native_libs):
    a = synth.normal(7, 10_000, n_threads=1)
    b = synth.normal(7, 10_000, n_threads=4)
    assert np.array_equal(a, b) and not np.array_equal(a, synth.normal(8, 10_000))
    assert abs(a.mean()) < 0.05 and abs(a.std() - 1) < 0.05
    for dt in (DType.Q4_0, DType.Q8_0, DType.Q4_K, DType.Q6_K):
        x = synth.random_blocks(dt, 3, 200, n_threads=1)
        assert np.array_equal(x, synth.random_blocks(dt, 3, 200, n_threads=3))
        q1 = synth.random_quantized(dt, 5, 256 * 40, n_threads=1)
        assert np.array_equal(q1, synth.random_quantized(dt, 5, 256 * 40, n_threads=2))
    t = synth.tokens(1, 1000, 32000)
    assert t.max() < 32000 and np.array_equal(t, synth.tokens(1, 1000, 32000))


def test_quantisers_round_trip_through_the_oracle(oracle):
    """f32 → blocks → dequant: error bounded by half a quantisation step of each format."""
    x = synth.normal(11, 256 * 64, std=0.02)
    bounds = {DType.Q8_0: 0.02 * 5 / 127, DType.Q4_0: 0.02 * 5 / 7, DType.Q4_K: 0.02 * 8 / 15, DType.Q6_K: 0.02 * 5 / 31}
    for dt, bound in bounds.items():
        y = oracle.dequant(int(dt), synth.quantize(dt, x))
        assert np.abs(y - x).max() <= bound
        assert np.sqrt(np.mean((y - x) ** 2)) < 0.12 * x.std()


def test_random_field_scales_follow_the_spec(oracle):
    """configs[0]: f16 d and dmin drawn as |N(0, 0.002)|; some of them are f16-subnormal (< 6.1e-5)."""
    b = synth.random_blocks(DType.Q4_K, 1, 20000).reshape(-1, 144)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(-1)
    assert (d >= 0).all() and abs(np.sqrt(np.mean(d ** 2)) - 0.002) < 2e-4
    assert 0.005 < np.mean(d < 6.1e-5) < 0.06


def test_model_shapes_and_bytes():
    cfg = synth.TINYLLAMA
    shapes = cfg.tensor_shapes()
    per_layer = sum(DType.Q6_K.tensor_bytes(*s) if n.endswith("ffn_down.weight") else DType.Q4_K.tensor_bytes(*s)
                    for n, s in shapes.items() if n.startswith("blk.0."))
    assert per_layer == 27_746_304
    assert 22 * per_layer + DType.Q6_K.tensor_bytes(32000, 2048) == 664_178_688
