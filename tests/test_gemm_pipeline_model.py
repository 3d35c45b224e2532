"""The hand-off protocol of the tcgen05 GEMM kernel (yule_b200/csrc/qgemm_tc.cu) checked on a model under random
interleavings: the ring sizes the kernel is built with, a sweep around them, and two variants that are known to be
broken, which the model must catch (so that a green run means something)."""

import pytest

from gemm_pipeline_model import Config, ProtocolViolation, run

# (stages, accumulator sets, raw boxes, stages per super-block) as instantiated: 32 rows with two column groups per
# stage; 32 rows with one; 64 rows; 128 rows
KERNEL_RINGS = {"rows32_wide": (3, 4, 3, 2), "rows32_narrow": (5, 4, 4, 4), "rows64": (3, 2, 4, 4), "rows128": (3, 3, 2, 4)}


def failures(cfg: Config, seeds) -> list:
    bad = []
    for seed in seeds:
        try:
            run(cfg, seed)
        except ProtocolViolation as e:
            bad.append((seed, str(e)))
    return bad


@pytest.mark.parametrize("name", list(KERNEL_RINGS))
def test_protocol_holds_at_the_kernel_ring_sizes(name):
    stages, nbuf, raw, spu = KERNEL_RINGS[name]
    cfg = Config(stages=stages, nbuf=nbuf, raw_slots=raw, stages_per_unit=spu, units=9)
    assert failures(cfg, range(150)) == []


def test_protocol_holds_around_them():
    for stages in (2, 3, 4, 6):
        for nbuf in (2, 3, 4):
            for raw in (2, 4):
                cfg = Config(stages=stages, nbuf=nbuf, raw_slots=raw, stages_per_unit=2, units=6)
                assert failures(cfg, range(12)) == [], (stages, nbuf, raw)


def test_full_size_warp_counts():
    assert failures(Config(producer_warps=8, drain_warps=8, units=5), range(40)) == []


def test_teams_on_alternate_stages_are_caught():
    """Two teams of unpacking warps on alternate stages wait on every other phase of a stage's `empty` barrier; a
    parity wait cannot tell phase k from phase k - 2, so a team that is ahead passes its wait early and overwrites a
    slab that has not been read."""
    bad = failures(Config(teams=True), range(40))
    assert bad, "the model no longer finds the overwrite"
    assert any("has not read slot" in msg or "beyond the count" in msg for _, msg in bad)


def test_missing_progress_guard_is_caught():
    """Without the check that the other MMA thread has seen the previous phase of a `full` barrier, a thread can ask
    for a phase two ahead of the barrier's and run on incomplete operands."""
    bad = failures(Config(progress_guard=False), range(200))
    assert bad, "the model no longer finds the early MMA"
