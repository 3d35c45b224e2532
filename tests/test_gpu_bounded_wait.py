"""The give-up path of the bounded device-side waits, exercised without a peer and without a fault: a kernel
polls memory that nothing writes, runs out of its (tiny) budget, records the status word and returns; the host
sees YULE_ERR_DEVICE_STATUS and the context keeps working.  The reference synchronises on the host only
(yule-gpu/src/cuda/mod.rs), so these waits have no counterpart there."""

import time

import numpy as np
import pytest

from conftest import REL_TOL, guarded_rel_err
from yule_b200 import DType, YuleGpuError, synth

pytestmark = pytest.mark.gpu

YULE_ERR_DEVICE_STATUS = 7


@pytest.mark.parametrize("which", [0, 1], ids=["matvec_waits_for_pairs", "exchange_waits_for_flag"])
def test_wait_runs_out_and_reports(backend, oracle, which):
    backend.synchronize()
    t0 = time.time()
    with pytest.raises(YuleGpuError) as err:
        backend.selftest_bounded_wait(which, 2_000_000)  # about a millisecond of SM clock
    assert err.value.code == YULE_ERR_DEVICE_STATUS
    assert time.time() - t0 < 5.0  # one budget, not one per wait
    # the status word was cleared by the report and the context is intact: a matvec still matches the oracle
    backend.synchronize()
    n_rows, n_cols = 64, 512
    w = synth.random_blocks(DType.Q4_K, 3, n_rows * n_cols // 256)
    x = synth.normal(4, n_cols)
    wh, xh, oh = backend.upload(w), backend.upload(x), backend.allocate(n_rows * 4)
    backend.quantized_matmul(wh, xh, oh, n_rows, n_cols, DType.Q4_K)
    y = backend.download(oh, n_rows)
    backend.synchronize()
    for h in (wh, xh, oh):
        backend.free(h)
    assert guarded_rel_err(y, oracle.qmv(int(DType.Q4_K), w, x, n_rows, n_cols)) <= REL_TOL


def test_wait_budget_setter(backend):
    backend.set_wait_budget(123456)
    with pytest.raises(YuleGpuError) as err:
        backend.selftest_bounded_wait(0, 0)  # 0: the context's budget
    assert err.value.code == YULE_ERR_DEVICE_STATUS
    backend.set_wait_budget(0)  # back to the default
    backend.synchronize()
