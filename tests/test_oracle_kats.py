"""Pins the CPU oracle against every known-answer vector Yule's own tests hold for this path, against
Yule's own Q4_K assembly kernel (outputs committed under tests/golden/), and against an independent
numpy decoding of the block layouts."""

import math
import os

import numpy as np
import pytest

from yule_b200 import DType, synth

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "q4k_reference_asm.npz")
MASK = (1 << 64) - 1


def xorshift(s):  # yule-core/src/simd/avx2.rs:347-352
    s ^= (s << 13) & MASK
    s ^= s >> 7
    s ^= (s << 17) & MASK
    return s


def test_f16_kats(oracle):  # yule-core/src/dequant.rs:1289-1298
    assert oracle.f16_to_f32(0x3C00) == 1.0
    assert oracle.f16_to_f32(0xBC00) == -1.0
    assert oracle.f16_to_f32(0x0000) == 0.0
    assert oracle.f16_to_f32(0x3800) == 0.5


def test_f16_all_patterns_match_ieee(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(b)) for b in bits], np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_q4_0_kats(oracle):  # dequant.rs:1309-1345, :1362-1375
    b = np.zeros(18, np.uint8)
    b[1] = 0x3C
    b[2:] = 0x88
    assert np.all(oracle.dequant(oracle.Q4_0, b) == 0.0)
    b[2:] = 0
    b[2] = 0xF0
    out = oracle.dequant(oracle.Q4_0, b)
    assert out[0] == -8.0 and out[1] == 7.0  # low nibble first, then high nibble of the same byte
    b[2:] = 0x99
    assert abs(oracle.vec_dot(oracle.Q4_0, b, np.ones(32, np.float32)) - 32.0) < 1e-4


def test_q8_0_kats(oracle):  # dequant.rs:1347-1359, :1393-1402
    b = np.zeros(34, np.uint8)
    b[1] = 0x3C
    b[2], b[3] = 127, 0x80
    out = oracle.dequant(oracle.Q8_0, b)
    assert out[0] == 127.0 and out[1] == -128.0
    b[2] = 42
    assert oracle.dequant(oracle.Q8_0, b)[0] == 42.0


def test_block_sizes(oracle):  # yule-core/src/dtype.rs:62-118
    for dt in DType:
        assert oracle.block_size(int(dt)) == dt.block_size
        assert oracle.block_bytes(int(dt)) == dt.size_of_block


def numpy_dequant_q4k(block):
    """Independent decoding from the format description (ggml get_scale_min_k4 layout)."""
    d = block[0:2].view(np.float16).astype(np.float32)[0]
    dmin = block[2:4].view(np.float16).astype(np.float32)[0]
    q = block[4:16].astype(np.uint32)
    sc, mn = np.zeros(8, np.uint32), np.zeros(8, np.uint32)
    for j in range(8):
        if j < 4:
            sc[j], mn[j] = q[j] & 63, q[j + 4] & 63
        else:
            sc[j] = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)
            mn[j] = (q[j + 4] >> 4) | ((q[j] >> 6) << 4)
    qs = block[16:144]
    out = np.zeros(256, np.float32)
    for j in range(4):
        lo = (qs[32 * j:32 * j + 32] & 0xF).astype(np.float32)
        hi = (qs[32 * j:32 * j + 32] >> 4).astype(np.float32)
        out[64 * j:64 * j + 32] = lo * (d * np.float32(sc[2 * j])) - dmin * np.float32(mn[2 * j])
        out[64 * j + 32:64 * j + 64] = hi * (d * np.float32(sc[2 * j + 1])) - dmin * np.float32(mn[2 * j + 1])
    return out, sc, mn


def numpy_dequant_q6k(block):
    d = block[208:210].view(np.float16).astype(np.float32)[0]
    sc = block[192:208].view(np.int8).astype(np.float32)
    ql, qh = block[0:128].astype(np.int32), block[128:192].astype(np.int32)
    out = np.zeros(256, np.float32)
    for c in range(256):
        h, r = divmod(c, 128)
        g, l = divmod(r, 32)
        low4 = (ql[64 * h + l + 32 * (g & 1)] >> (4 * (g >> 1))) & 0xF
        high2 = (qh[32 * h + l] >> (2 * g)) & 3
        qv = np.float32((low4 | (high2 << 4)) - 32)
        out[c] = (d * sc[8 * h + l // 16 + 2 * g]) * qv
    return out


def test_q4k_q6k_dequant_against_independent_decoder(oracle):
    for seed in range(8):
        b = synth.random_blocks(DType.Q4_K, seed, 1)
        want, sc, mn = numpy_dequant_q4k(b)
        osc, omn = oracle.extract_q4k_scales_mins(b[4:16])
        assert np.array_equal(osc, sc) and np.array_equal(omn, mn)
        assert np.array_equal(oracle.dequant(oracle.Q4_K, b).view(np.uint32), want.view(np.uint32))
        b6 = synth.random_blocks(DType.Q6_K, seed, 1)
        assert np.array_equal(oracle.dequant(oracle.Q6_K, b6).view(np.uint32), numpy_dequant_q6k(b6).view(np.uint32))


@pytest.mark.parametrize("name,typ,nbytes,seed,iters,tol", [
    ("q8_0", 8, 34, 42, 2000, 1e-2), ("q4_0", 2, 18, 123, 2000, 1e-2)])
def test_avx2_vs_scalar_recipe_small_blocks(oracle, name, typ, nbytes, seed, iters, tol):
    """yule-core/src/simd/avx2.rs:355-406 (the reference runs 10 000 iterations; 2 000 keep this fast)."""
    if not oracle.lib.yo_have_avx2():
        pytest.skip("no AVX2")
    s = seed
    for _ in range(iters):
        b = np.zeros(nbytes, np.uint8)
        b[1] = 0x38
        for i in range(nbytes - 2):
            s = xorshift(s)
            b[2 + i] = s & 0xFF
        act = np.zeros(32, np.float32)
        for i in range(32):
            s = xorshift(s)
            act[i] = np.float32(s % 1000) / np.float32(500.0) - np.float32(1.0)
        assert abs(oracle.vec_dot(typ, b, act, oracle.SCALAR) - oracle.vec_dot(typ, b, act, oracle.AVX2)) < tol


def test_q6k_recipe_scalar_vs_dequant_dot(oracle):
    """avx2.rs:544-573 recipe (seed 999, scales % 20): fused dot equals dequantise-then-dot."""
    s = 999
    for _ in range(200):
        b = np.zeros(210, np.uint8)
        for i in range(210):
            s = xorshift(s)
            b[i] = s & 0xFF
        b[208], b[209] = 0x00, 0x38
        for i in range(192, 208):
            s = xorshift(s)
            b[i] = s % 20
        act = np.zeros(256, np.float32)
        for i in range(256):
            s = xorshift(s)
            act[i] = np.float32(s % 1000) / np.float32(500.0) - np.float32(1.0)
        fused = oracle.vec_dot(oracle.Q6_K, b, act, oracle.SCALAR)
        simd = oracle.vec_dot(oracle.Q6_K, b, act, oracle.AVX2)
        ref = float(np.dot(oracle.dequant(oracle.Q6_K, b).astype(np.float64), act.astype(np.float64)))
        assert abs(fused - simd) < 1e-1 and abs(fused - ref) < 1e-2 * max(1.0, abs(ref))


def test_q4k_against_reference_assembly_golden(oracle):
    """Outputs of Yule's own q4k_gemv_avx2.S (tests/golden/make_golden.py) vs the scalar restatement and
    the intrinsic restatement, within the reference test's own bound (avx2.rs:434-438: 1e-1)."""
    g = np.load(GOLDEN)
    for blocks, acts, outs in ((g["recipe_blocks"], g["recipe_acts"], g["recipe_out"]),
                               (g["field_blocks"], g["field_acts"], g["field_out"])):
        for k in range(blocks.shape[0]):
            sc = oracle.vec_dot(oracle.Q4_K, blocks[k], acts[k], oracle.SCALAR)
            av = oracle.vec_dot(oracle.Q4_K, blocks[k], acts[k], oracle.AVX2)
            assert abs(sc - outs[k]) < 1e-1 and abs(av - outs[k]) < 1e-1
            assert abs(sc - outs[k]) <= 2e-5 * max(1.0, np.abs(oracle.dequant(oracle.Q4_K, blocks[k]) * acts[k]).sum())


def test_reference_assembly_live_when_built(oracle):
    """Where oracle/_ref holds the freshly assembled kernel, it reproduces the committed fixture bit for bit."""
    if not oracle.load_reference_asm():
        pytest.skip("oracle/_ref not built (no Yule checkout reachable)")
    g = np.load(GOLDEN)
    for k in range(16):
        assert np.float32(oracle.reference_q4k_asm(g["recipe_blocks"][k], g["recipe_acts"][k])) == g["recipe_out"][k]
        assert oracle.vec_dot(oracle.Q4_K, g["field_blocks"][k], g["field_acts"][k], oracle.AVX2_ASM) == g["field_out"][k]


def test_trait_level_kats_on_oracle(oracle):
    """yule-gpu/src/cpu.rs:612-790, :906-988 expressed on the oracle's functions."""
    r = oracle.softmax(np.array([1, 2, 3, 4], np.float32))
    assert abs(r.sum() - 1) < 1e-5 and r[3] > r[2] > r[1] > r[0]
    r = oracle.rms_norm(np.array([1, 2, 3, 4], np.float32), np.ones(4, np.float32), 1e-6)
    rms = math.sqrt(7.5 + 1e-6)
    assert abs(r[0] - 1 / rms) < 1e-4 and abs(r[3] - 4 / rms) < 1e-4
    cos, sin = oracle.rope_table(6, 4, 10000.0)
    q = oracle.apply_rope(np.array([1, 0, 1, 0], np.float32), 5, 4, cos, sin)
    assert abs(q[0] - math.cos(5.0)) < 1e-4 and abs(q[1] - math.sin(5.0)) < 1e-4
    assert np.array_equal(oracle.apply_rope(np.array([1, 0, 1, 0], np.float32), 0, 4, cos, sin),
                          np.array([1, 0, 1, 0], np.float32))
    # attention: Q=[1,0], K rows [1,0],[0,1],[1,1], V rows [10,20],[30,40],[50,60]
    out = oracle.attention(np.array([1, 0], np.float32), np.array([1, 0, 0, 1, 1, 1], np.float32),
                           np.array([10, 20, 30, 40, 50, 60], np.float32), 1, 1, 2, 3)
    s = np.array([1, 0, 1]) / math.sqrt(2)
    w = np.exp(s - s.max())
    w /= w.sum()
    assert abs(out[0] - (w * [10, 30, 50]).sum()) < 1e-3 and abs(out[1] - (w * [20, 40, 60]).sum()) < 1e-3
    # GQA 2:1 (cpu.rs:1079-1156)
    out = oracle.attention(np.array([1, 0, 0, 1], np.float32), np.array([1, 0, 0, 1], np.float32),
                           np.array([10, 20, 30, 40], np.float32), 2, 1, 2, 2)
    assert out[0] < 25 and out[1] < 35 and out[2] > 15 and out[3] > 25
    sw = oracle.swiglu(np.array([0, 1, -1], np.float32), np.ones(3, np.float32))
    assert abs(sw[0]) < 1e-6 and abs(sw[1] - 0.7311) < 1e-3 and abs(sw[2] + 0.2689) < 1e-3


def test_argmax_ties_go_to_last(oracle):  # yule-infer/src/sampler.rs:150-163
    assert oracle.argmax(np.array([1, 3, 3, 2], np.float32)) == 2
    assert oracle.argmax(np.array([5, 5, 5], np.float32)) == 2
    assert oracle.argmax(np.array([-1, -7], np.float32)) == 0


def test_qmv_threaded_equals_sequential(oracle):
    """model_runner.rs:152-244: row partitioning must not change any row's value."""
    for dt in (DType.Q4_K, DType.Q6_K, DType.Q4_0, DType.Q8_0):
        w = synth.random_blocks(dt, 5, 300 * 4 * (256 // dt.block_size))
        x = synth.normal(6, 1024)
        a = oracle.qmv(int(dt), w, x, 300, 1024, n_threads=1)
        b = oracle.qmv(int(dt), w, x, 300, 1024, n_threads=5)
        assert np.array_equal(a, b)
        deq = oracle.dequant(int(dt), w).reshape(300, 1024).astype(np.float64)
        assert np.allclose(a, deq @ x.astype(np.float64), rtol=0, atol=1e-4 * np.abs(a).max())


def test_forward_mod_switch(oracle):
    """Mixture-of-Depths turns on at >= 32 layers (model_runner.rs:463) and skips low-norm layers after
    10 tokens (mixture_of_depths.rs:82-111); below 32 layers nothing is skipped."""
    from yule_b200 import ModelConfig
    for n_layers, expect_skips in ((4, False), (32, True)):
        cfg = ModelConfig(dim=64, n_layers=n_layers, n_heads=2, n_kv_heads=1, head_dim=32, vocab_size=64,
                          ff_dim=256, max_seq_len=16)
        weights = synth.synthetic_model(cfg, seed=3, std=0.02, linear=DType.Q8_0)
        m = oracle.Model(dim=64, n_layers=n_layers, n_heads=2, n_kv_heads=1, head_dim=32, vocab_size=64, ff_dim=256,
                         max_seq_len=16)
        for name, (data, dt) in weights.items():
            m.set_tensor(name, data, int(dt))
        for t in range(12):
            logits = m.forward(t)
        assert np.isfinite(logits).all()
        assert (m.layers_skipped > 0) == expect_skips
        with pytest.raises(RuntimeError):
            for t in range(8):
                m.forward(1)
