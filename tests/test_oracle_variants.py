"""The oracle's architecture variants against what the reference's own tests fix
(yule-infer/src/model_runner.rs:1099-1135: GELU values, the sliding-window mask, the softcap bound)
and against their definitions, on the CPU."""

import numpy as np

from yule_b200 import synth


def test_gelu_values(oracle):  # model_runner.rs:1100-1104
    assert abs(oracle.gelu(0.0)) < 1e-6
    assert abs(oracle.gelu(1.0) - 0.8413) < 1e-3
    assert abs(oracle.gelu(-1.0) + 0.1587) < 1e-3


def test_sliding_window_masks_positions_before_pos_minus_window(oracle):
    """model_runner.rs:1107-1123: pos = 8, window = 4 → positions 0..3 carry no weight, 4..8 are visible.
    A masked position contributes exp(-inf) = 0, so the result equals attention over the visible suffix."""
    hd, n_heads, n_kv = 8, 4, 2
    seq = 9  # pos = 8
    q = synth.normal(1, n_heads * hd)
    k = synth.normal(2, seq * n_kv * hd)
    v = synth.normal(3, seq * n_kv * hd)
    got = oracle.attention(q, k, v, n_heads, n_kv, hd, seq, sliding_window=4)
    stride = n_kv * hd
    want = oracle.attention(q, k[4 * stride:], v[4 * stride:], n_heads, n_kv, hd, seq - 4)
    assert np.array_equal(got, want)
    # before the window fills (pos < window) nothing is masked
    assert np.array_equal(oracle.attention(q, k, v, n_heads, n_kv, hd, 4, sliding_window=4),
                          oracle.attention(q, k, v, n_heads, n_kv, hd, 4))


def test_attention_softcap_is_bounded_and_monotone(oracle):
    """model_runner.rs:1125-1135: cap * tanh(x / cap) stays within the cap and keeps 0 at 0; with a huge cap
    the attention output approaches the uncapped one."""
    hd, n_heads, n_kv, seq = 8, 2, 1, 6
    q = 10.0 * synth.normal(4, n_heads * hd)
    k = 10.0 * synth.normal(5, seq * n_kv * hd)
    v = synth.normal(6, seq * n_kv * hd)
    plain = oracle.attention(q, k, v, n_heads, n_kv, hd, seq)
    assert np.allclose(oracle.attention(q, k, v, n_heads, n_kv, hd, seq, softcap=1e6), plain, rtol=1e-4, atol=1e-5)
    capped = oracle.attention(q, k, v, n_heads, n_kv, hd, seq, softcap=0.5)
    # scores squeezed into [-0.5, 0.5] make the softmax nearly uniform: the output nears the mean of V
    mean_v = v.reshape(seq, hd).mean(axis=0)
    assert np.abs(capped.reshape(n_heads, hd) - mean_v).max() < np.abs(plain.reshape(n_heads, hd) - mean_v).max()


def test_partial_rope_leaves_the_tail_of_each_head(oracle):
    """model_runner.rs:78-99 with rotary_dim < head_dim: pairs beyond rotary_dim/2 are untouched, and the
    frequencies are formed over rotary_dim."""
    hd, rot, pos = 16, 8, 5
    cos, sin = oracle.rope_table(8, rot, 10000.0)
    x = synth.normal(7, 2 * hd)
    y = oracle.apply_rope(x, pos, hd, cos, sin, rotary_dim=rot)
    for h in range(2):
        assert np.array_equal(y[h * hd + rot:(h + 1) * hd], x[h * hd + rot:(h + 1) * hd])
        for i in range(rot // 2):
            theta = np.float32(pos) * np.float32(1.0 / np.float32(10000.0) ** np.float32(2.0 * i / rot))
            c, s = np.cos(theta, dtype=np.float32), np.sin(theta, dtype=np.float32)
            x0, x1 = x[h * hd + 2 * i], x[h * hd + 2 * i + 1]
            assert abs(y[h * hd + 2 * i] - (x0 * c - x1 * s)) < 1e-5 and abs(y[h * hd + 2 * i + 1] - (x0 * s + x1 * c)) < 1e-5


def test_window_and_softcap_together_leave_masked_positions_a_weight(oracle):
    """model_runner.rs:688-721 masks first and caps second: cap * tanh(-inf / cap) is -cap, a finite score, so
    with both options on the positions before the window are not excluded from the softmax.  The restatement
    keeps that order."""
    hd, n_heads, n_kv, seq = 8, 2, 1, 9
    q = synth.normal(11, n_heads * hd)
    k = synth.normal(12, seq * n_kv * hd)
    v = synth.normal(13, seq * n_kv * hd)
    both = oracle.attention(q, k, v, n_heads, n_kv, hd, seq, sliding_window=4, softcap=1.0)
    stride = n_kv * hd
    suffix_only = oracle.attention(q, k[4 * stride:], v[4 * stride:], n_heads, n_kv, hd, seq - 4, softcap=1.0)
    assert not np.allclose(both, suffix_only, rtol=1e-3, atol=1e-4)
