"""The allocation-free attention entry point (``yule_cuda_multihead_attention_static``).

Some embedders cannot allocate device memory once inference is running — a sandboxed Yule process whose
driver requests are filtered, or a host with a fixed memory budget — so this variant keeps its split-KV
scratch in a fixed array inside the library.  It must give the same numbers as the regular entry point,
call after call (the array is shared and keeps the previous call's contents), and refuse shapes that do
not fit the array.  Collected last on purpose: a run that stops at the first failure has then already run
every other test.
"""

import numpy as np
import pytest

from conftest import REL_TOL, guarded_rel_err
from yule_b200 import YuleGpuError, synth

pytestmark = pytest.mark.gpu


def _attend(backend, fn, q, K, V, hd, seq, n_heads, n_kv):
    qh, kh, vh, oh = backend.upload(q), backend.upload(K), backend.upload(V), backend.allocate(q.nbytes)
    fn(qh, kh, vh, oh, hd, seq, n_heads, n_kv, n_kv * hd)
    out = backend.download(oh, q.size)
    for h in (qh, kh, vh, oh):
        backend.free(h)
    return out


@pytest.mark.parametrize("n_heads,n_kv,hd,seq", [(32, 4, 64, 160), (32, 8, 128, 2300), (8, 2, 32, 700)])
def test_matches_regular_entry_point_twice_in_a_row(backend, oracle, n_heads, n_kv, hd, seq):
    for call in range(2):  # second call finds the first call's partial sums in the shared array
        q = synth.normal(10 + call, n_heads * hd)
        K = synth.normal(20 + call, seq * n_kv * hd)
        V = synth.normal(30 + call, seq * n_kv * hd)
        ref = _attend(backend, backend.multihead_attention, q, K, V, hd, seq, n_heads, n_kv)
        got = _attend(backend, backend.multihead_attention_static, q, K, V, hd, seq, n_heads, n_kv)
        assert guarded_rel_err(got, ref) <= REL_TOL
        assert guarded_rel_err(got, oracle.attention(q, K, V, n_heads, n_kv, hd, seq)) <= REL_TOL


def test_shapes_beyond_the_built_in_scratch_are_refused(backend):
    hd, seq = 64, 8
    for n_heads in (256, 129):
        q = backend.allocate(n_heads * hd * 4)
        kv = backend.allocate(seq * n_heads * hd * 4)
        with pytest.raises(YuleGpuError) as e:
            backend.multihead_attention_static(q, kv, kv, q, hd, seq, n_heads, n_heads, n_heads * hd)
        assert "exceeds the built-in scratch" in str(e.value)
        backend.free(q)
        backend.free(kv)
    q = backend.allocate(8 * 96 * 4)
    kv = backend.allocate(4 * 8 * 96 * 4)
    with pytest.raises(YuleGpuError):  # head_dim 96: 256 % 24 != 0
        backend.multihead_attention_static(q, kv, kv, q, 96, 4, 8, 8, 8 * 96)
    backend.free(q)
    backend.free(kv)
