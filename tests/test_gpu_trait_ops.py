"""The trait-level known-answer tests of yule-gpu/src/cpu.rs:612-1157, replayed through the C ABI with
the semantics of the reference's GPU backends (silu / element_mul / matmul differ from the CPU
backend: yule-gpu/src/cuda/mod.rs:95-208), plus comparisons with the oracle on random inputs."""

import math

import numpy as np
import pytest

from conftest import REL_TOL, guarded_rel_err
from yule_b200 import YuleGpuError, synth

pytestmark = pytest.mark.gpu


def f32(*v):
    return np.array(v, np.float32)


def test_softmax(backend, oracle):  # cpu.rs:612-629
    i, o = backend.upload(f32(1, 2, 3, 4)), backend.allocate(16)
    backend.softmax(i, o, 4)
    r = backend.download(o, 4)
    assert abs(r.sum() - 1.0) < 1e-5 and r[3] > r[2] > r[1] > r[0]
    x = synth.normal(3, 3000, std=3.0)
    i2, o2 = backend.upload(x), backend.allocate(x.nbytes)
    backend.softmax(i2, o2, x.size)
    assert guarded_rel_err(backend.download(o2, x.size), oracle.softmax(x)) <= REL_TOL
    backend.softmax(i2, i2, x.size)  # in place, as attention uses it (cpu.rs:937)
    assert guarded_rel_err(backend.download(i2, x.size), oracle.softmax(x)) <= REL_TOL


def test_rms_norm(backend, oracle):  # cpu.rs:632-649
    i, w, o = backend.upload(f32(1, 2, 3, 4)), backend.upload(f32(1, 1, 1, 1)), backend.allocate(16)
    backend.rms_norm(i, w, o, 4, 1e-6)
    r = backend.download(o, 4)
    rms = math.sqrt(7.5 + 1e-6)
    assert abs(r[0] - 1 / rms) < 1e-4 and abs(r[3] - 4 / rms) < 1e-4
    x, g = synth.normal(1, 2048), synth.normal(2, 2048, mean=1.0, std=0.1)
    i, w, o = backend.upload(x), backend.upload(g), backend.allocate(x.nbytes)
    backend.rms_norm(i, w, o, 2048, 1e-5)
    assert guarded_rel_err(backend.download(o, 2048), oracle.rms_norm(x, g, 1e-5)) <= 1e-5


def test_silu_is_silu_times_output(backend):
    """GPU semantics: output = SiLU(input) * output (cuda/mod.rs:173-188), not the CPU backend's plain SiLU."""
    i, o = backend.upload(f32(0, 1, -1)), backend.upload(f32(2, 2, 2))
    backend.silu(i, o, 3)
    r = backend.download(o, 3)
    assert abs(r[0]) < 1e-6 and abs(r[1] - 2 * 0.7310586) < 1e-5 and abs(r[2] + 2 * 0.2689414) < 1e-5


def test_element_mul_is_silu_a_times_b(backend, oracle):
    """GPU semantics: out = SiLU(a) * b (cuda/mod.rs:190-208) — the SiluMul dispatch of the runner."""
    g, u = synth.normal(4, 5632), synth.normal(5, 5632)
    a, b, o = backend.upload(g), backend.upload(u), backend.allocate(g.nbytes)
    backend.element_mul(a, b, o, g.size)
    assert guarded_rel_err(backend.download(o, g.size), oracle.swiglu(g, u)) <= 1e-5


def test_add(backend):  # cpu.rs:688-703
    a, b, o = backend.upload(f32(1, 2, 3)), backend.upload(f32(4, 5, 6)), backend.allocate(12)
    backend.add(a, b, o, 3)
    assert np.array_equal(backend.download(o, 3), f32(5, 7, 9))


def test_matmul_is_per_row_matvec(backend):
    """CUDA semantics (kernels/cuda/matmul.cu:4-32): out[row] = dot(A[row, :k], b); n is ignored."""
    A = synth.normal(7, 37 * 300).reshape(37, 300)
    v = synth.normal(8, 300)
    a, b, o = backend.upload(A), backend.upload(v), backend.allocate(37 * 4)
    backend.matmul(a, b, o, 37, 1, 300)
    assert guarded_rel_err(backend.download(o, 37), A.astype(np.float64) @ v.astype(np.float64)) <= REL_TOL


def test_rope_pos0_and_multi_head(backend):  # cpu.rs:734-768
    q, k = backend.upload(f32(1, 0, 1, 0, 0, 1, 0, 1)), backend.upload(f32(1, 0, 1, 0))
    backend.rope(q, k, 0, 4, 10000.0, 2, 1)
    assert np.array_equal(backend.download(q, 8), f32(1, 0, 1, 0, 0, 1, 0, 1))
    assert np.array_equal(backend.download(k, 4), f32(1, 0, 1, 0))


def test_rope_pos5(backend, oracle):  # cpu.rs:771-790
    q, k = backend.upload(f32(1, 0, 1, 0)), backend.upload(f32(1, 0, 1, 0))
    backend.rope(q, k, 5, 4, 10000.0, 1, 1)
    r = backend.download(q, 4)
    assert abs(r[0] - math.cos(5.0)) < 1e-4 and abs(r[1] - math.sin(5.0)) < 1e-4
    # bit-exact with the CPU runner's table recipe (model_runner.rs:78-99, :277-293)
    hd, nq, nk, pos = 64, 32, 4, 137
    qv, kv = synth.normal(1, nq * hd), synth.normal(2, nk * hd)
    cos, sin = oracle.rope_table(pos + 1, hd, 10000.0)
    qh, kh = backend.upload(qv), backend.upload(kv)
    backend.rope(qh, kh, pos, hd, 10000.0, nq, nk)
    assert np.array_equal(backend.download(qh, qv.size), oracle.apply_rope(qv, pos, hd, cos, sin))
    assert np.array_equal(backend.download(kh, kv.size), oracle.apply_rope(kv, pos, hd, cos, sin))


def test_copy_buffer_and_offset(backend):  # cpu.rs:793-857
    src, dst = backend.upload(f32(10, 20, 30, 40)), backend.allocate(32)
    backend.copy_buffer_offset(src, dst, 4, 8, 8)
    assert np.array_equal(backend.download(dst, 8), f32(0, 0, 20, 30, 0, 0, 0, 0))
    d2 = backend.allocate(16)
    backend.copy_buffer(src, d2, 16)
    assert np.array_equal(backend.download(d2, 4), f32(10, 20, 30, 40))
    # KV-cache pattern: one position's row written at pos * kv_stride * 4
    kv_stride, max_seq = 8, 4
    k_tmp = backend.upload(np.arange(1, kv_stride + 1, dtype=np.float32))
    cache = backend.allocate(max_seq * kv_stride * 4)
    backend.copy_buffer_offset(k_tmp, cache, 0, 2 * kv_stride * 4, kv_stride * 4)
    c = backend.download(cache, max_seq * kv_stride).reshape(max_seq, kv_stride)
    assert np.all(c[[0, 1, 3]] == 0) and np.array_equal(c[2], np.arange(1, 9, dtype=np.float32))
    with pytest.raises(YuleGpuError):
        backend.copy_buffer_offset(k_tmp, cache, 0, max_seq * kv_stride * 4 - 4, 8)  # past the end
    with pytest.raises(YuleGpuError):
        backend.copy_buffer_offset(k_tmp, cache, 30, 0, 8)


def test_attn_score_value_and_manual_pipeline(backend):  # cpu.rs:860-988
    hd, seq = 2, 3
    q = backend.upload(f32(1, 0, 0, 1, 1, 1, .5, .5))
    kc = backend.upload(f32(1, 0, 0, 1, 0, 1, 1, 0, 1, 1, .5, .5))
    vc = backend.upload(f32(10, 20, 30, 40, 50, 60, 70, 80, 90, 100, 110, 120))
    s, o = backend.allocate(seq * 4), backend.allocate(8 * 4)
    backend.attn_score(q, kc, s, hd, seq, 0, 0, 4)
    sc = backend.download(s, 3)
    scale = 1 / math.sqrt(2)
    assert abs(sc[0] - scale) < 1e-5 and abs(sc[1]) < 1e-5 and abs(sc[2] - scale) < 1e-5
    backend.softmax(s, s, seq)
    w = backend.download(s, 3)
    backend.attn_value(s, vc, o, hd, seq, 0, 4, 0)
    r = backend.download(o, 2)
    V = np.array([[10, 20], [50, 60], [90, 100]], np.float64)
    assert np.allclose(r, w.astype(np.float64) @ V, rtol=1e-5)


@pytest.mark.parametrize("n_heads,n_kv,hd,seq", [(2, 1, 2, 2), (32, 4, 64, 1), (32, 4, 64, 160), (32, 8, 128, 777),
                                                (8, 8, 96, 33),
                                                # grouped-query kernel (from 512 positions): every group size, both
                                                # head sizes, a length whose last split is empty (2049 over 64 splits)
                                                (32, 4, 64, 2049), (64, 8, 128, 1500), (8, 8, 128, 600), (16, 8, 64, 513),
                                                (16, 4, 128, 4100), (4, 4, 64, 512), (8, 2, 64, 999), (16, 8, 128, 640)])
def test_multihead_attention_vs_oracle(backend, oracle, n_heads, n_kv, hd, seq):
    """GQA: head h reads kv head h / (n_heads / n_kv) (cpu.rs:1079-1156, gpu_runner.rs:477-499)."""
    kv_stride = n_kv * hd
    q = synth.normal(1, n_heads * hd)
    K, V = synth.normal(2, seq * kv_stride), synth.normal(3, seq * kv_stride)
    qh, kh, vh, oh = backend.upload(q), backend.upload(K), backend.upload(V), backend.allocate(q.nbytes)
    backend.multihead_attention(qh, kh, vh, oh, hd, seq, n_heads, n_kv, kv_stride)
    ref = oracle.attention(q, K, V, n_heads, n_kv, hd, seq)
    assert guarded_rel_err(backend.download(oh, q.size), ref) <= REL_TOL


def test_gqa_kat(backend):  # cpu.rs:1079-1156
    q, kc, vc = backend.upload(f32(1, 0, 0, 1)), backend.upload(f32(1, 0, 0, 1)), backend.upload(f32(10, 20, 30, 40))
    o = backend.allocate(16)
    backend.multihead_attention(q, kc, vc, o, 2, 2, 2, 1, 2)
    r = backend.download(o, 4)
    assert r[0] < 25 and r[1] < 35 and r[2] > 15 and r[3] > 25


def test_embed_gather(backend, oracle):
    from yule_b200 import DType
    vocab, dim = 50, 512
    for dt in (DType.Q4_K, DType.Q6_K, DType.Q8_0, DType.Q4_0):
        table = synth.random_quantized(dt, 9, vocab * dim)
        th, oh = backend.upload(table), backend.allocate(dim * 4)
        backend.embed_gather(th, dt, dim, 37, oh)
        row_bytes = dim // dt.block_size * dt.size_of_block
        ref = oracle.dequant(int(dt), table[37 * row_bytes:38 * row_bytes])
        assert np.array_equal(backend.download(oh, dim).view(np.uint32), ref.view(np.uint32))
        with pytest.raises(YuleGpuError):
            backend.embed_gather(th, dt, dim, vocab, oh)


def test_allocations_are_zeroed_and_handles_checked(backend):
    from yule_b200 import BufferHandle
    h = backend.allocate(1000)
    assert not backend.download(h, 250).any()
    backend.free(h)
    with pytest.raises(YuleGpuError):
        backend.free(h)
    with pytest.raises(YuleGpuError):
        backend.copy_to_device(b"abcd", BufferHandle(123456789))
    info = backend.device_info()
    assert backend.name() == "cuda" and info.compute_units > 0 and info.memory_bytes > 0
