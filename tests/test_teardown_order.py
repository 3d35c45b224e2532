"""Teardown order of the Python mirror of the runner and the backend: a runner holds a pointer to its context, so the
context destroys the runners still open on it first, a runner is destroyed at most once whatever its frees raise, and
a runner that outlived its context does not touch it.  Fakes stand in for the C library: no GPU needed."""

import weakref

import pytest

from yule_b200.backend import CudaB200Backend, YuleGpuError
from yule_b200.runner import CudaTransformerRunner


class FakeLib:
    def __init__(self):
        self.calls = []

    def yule_cuda_runner_destroy(self, r):
        self.calls.append(("runner_destroy", r))

    def yule_cuda_destroy(self, ctx):
        self.calls.append(("ctx_destroy", ctx))


def fake_backend(lib, free_raises=False):
    b = CudaB200Backend.__new__(CudaB200Backend)
    b._lib = lib
    b._ctx = "ctx"
    b._runners = weakref.WeakSet()

    def free(h):
        lib.calls.append(("free", h))
        if free_raises:
            raise YuleGpuError(7, "device status")
    b.free = free
    return b


def fake_runner(lib, backend, handles=("a", "b")):
    r = CudaTransformerRunner.__new__(CudaTransformerRunner)
    r._lib = lib
    r.backend = backend
    r._r = "runner"
    r._handles = {h: h for h in handles}
    backend._runners.add(r)
    return r


def test_runner_is_destroyed_once():
    lib = FakeLib()
    b = fake_backend(lib)
    r = fake_runner(lib, b)
    r.close()
    r.close()
    assert lib.calls == [("runner_destroy", "runner"), ("free", "a"), ("free", "b")]


def test_a_failing_free_does_not_lead_to_a_second_destroy():
    lib = FakeLib()
    b = fake_backend(lib, free_raises=True)
    r = fake_runner(lib, b)
    with pytest.raises(YuleGpuError):
        r.close()
    r.close()  # what __del__ would do later
    assert [c for c in lib.calls if c[0] == "runner_destroy"] == [("runner_destroy", "runner")]


def test_context_takes_its_open_runners_with_it():
    lib = FakeLib()
    b = fake_backend(lib)
    r = fake_runner(lib, b, handles=("w",))
    b.close()
    assert lib.calls == [("runner_destroy", "runner"), ("free", "w"), ("ctx_destroy", "ctx")]
    r.close()
    b.close()
    assert len(lib.calls) == 3


def test_runner_that_outlived_its_context_leaves_it_alone():
    lib = FakeLib()
    b = fake_backend(lib)
    r = fake_runner(lib, b)
    b._runners.discard(r)  # as if created before the registry existed
    b.close()
    r.close()
    assert lib.calls == [("ctx_destroy", "ctx")]
