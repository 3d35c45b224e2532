"""A model of the hand-offs inside the tcgen05 GEMM kernel (yule_b200/csrc/qgemm_tc.cu), for checking the protocol on the
CPU under many interleavings.  It models what the kernel's roles do to the mbarriers and to the buffers they guard,
nothing of the arithmetic:

* operand stages (ring of ``stages``): filled by the unpacking warps (W slab) and by the loader's bulk copy (x slabs),
  read by the MMAs of that stage, released by ``tcgen05.commit`` on the stage's ``empty`` barrier;
* raw boxes (ring of ``raw_slots``): filled by the tiled TMA load of one super-block, read by every unpacking warp;
* accumulator sets (ring of ``nbuf``): written by the MMAs of a stage, read by every drain warp;
* two MMA threads issuing alternate stages, each committing only its own MMAs.

An mbarrier here is what the hardware gives: an arrival count per phase, an optional transaction count, and a wait
that knows only the PARITY of the phase it wants, so it cannot tell phase k from phase k - 2.  The checks: no arrival
beyond a phase's count, no buffer written before its last reader is done, no buffer read before its writers are
done, and no deadlock.  The scheduler resumes one runnable agent at a time, chosen at random with per-agent speeds
drawn per run, so slow and fast roles of every kind occur.

Variants: ``teams`` lets two teams of unpacking warps take alternate stages (each waits on every other phase of a
stage's ``empty`` barrier), ``progress_guard=False`` removes the MMA threads' check that the other thread has seen the
previous phase of a ``full`` barrier.  Both are broken; the tests show that the model finds it."""

from __future__ import annotations

import random
from dataclasses import dataclass, field


class ProtocolViolation(AssertionError):
    pass


class Barrier:
    """Phase k is in progress; phases 0 .. k-1 are complete.  ``test(parity)`` is mbarrier.try_wait.parity: true when
    the phase with that parity is not the one in progress."""

    def __init__(self, name: str, count: int):
        self.name, self.count = name, count
        self.pending, self.tx, self.phase = count, 0, 0

    def _maybe_complete(self):
        if self.pending == 0 and self.tx == 0:
            self.phase += 1
            self.pending = self.count

    def arrive(self):
        if self.pending == 0:
            raise ProtocolViolation(f"{self.name}: arrival beyond the count of phase {self.phase}")
        self.pending -= 1
        self._maybe_complete()

    def arrive_expect_tx(self):
        self.tx += 1
        self.arrive()

    def complete_tx(self):
        if self.tx == 0:
            raise ProtocolViolation(f"{self.name}: transaction bytes nobody announced")
        self.tx -= 1
        self._maybe_complete()

    def test(self, parity: int) -> bool:
        return (self.phase & 1) != parity


@dataclass
class Config:
    stages: int = 3
    nbuf: int = 4
    raw_slots: int = 3
    stages_per_unit: int = 2      # stages per super-block
    units: int = 9                # super-blocks this CTA walks through
    producer_warps: int = 4
    drain_warps: int = 2
    teams: bool = False
    progress_guard: bool = True


@dataclass
class State:
    cfg: Config
    full: list = field(default_factory=list)
    empty: list = field(default_factory=list)
    acc_full: list = field(default_factory=list)
    acc_empty: list = field(default_factory=list)
    raw_full: list = field(default_factory=list)
    raw_empty: list = field(default_factory=list)

    def __post_init__(self):
        c = self.cfg
        writers = c.producer_warps // 2 if c.teams else c.producer_warps
        self.full = [Barrier(f"full[{s}]", writers + 1) for s in range(c.stages)]
        self.empty = [Barrier(f"empty[{s}]", 1) for s in range(c.stages)]
        self.acc_full = [Barrier(f"acc_full[{b}]", 1) for b in range(c.nbuf)]
        self.acc_empty = [Barrier(f"acc_empty[{b}]", c.drain_warps) for b in range(c.nbuf)]
        self.raw_full = [Barrier(f"raw_full[{r}]", 1) for r in range(c.raw_slots)]
        self.raw_empty = [Barrier(f"raw_empty[{r}]", c.producer_warps) for r in range(c.raw_slots)]
        n = c.units * c.stages_per_unit
        self.n_stages = n
        self.w_written = [set() for _ in range(n)]   # per stage use j: the warps that wrote its W slab
        self.x_landed = [False] * n
        self.mma_done = [False] * n
        self.drained = [set() for _ in range(n)]     # per stage use j: the drain warps that read its accumulator
        self.raw_landed = [False] * c.units
        self.raw_read = [set() for _ in range(c.units)]
        self.mma_progress = [0, 0]
        self.pipe = [[], []]                         # per MMA thread: issued, not yet executed ("mma", j) / ("commit", bars)
        self.copies = []                             # bulk copies in flight: callables that land them

    def writers_of(self, j: int):
        c = self.cfg
        if not c.teams:
            return set(range(c.producer_warps))
        half = c.producer_warps // 2
        team = j % 2
        return set(range(team * half, team * half + half))


def wait(bar: Barrier, parity: int):
    return lambda: bar.test(parity)


def loader(st: State):
    """One thread: the x slabs of every stage (waits for the stage to be free, announces the bytes, issues the copy)."""
    c = st.cfg
    for j in range(st.n_stages):
        s, ph = j % c.stages, (j // c.stages) & 1
        yield wait(st.empty[s], ph ^ 1)
        if j >= c.stages and not st.mma_done[j - c.stages]:
            raise ProtocolViolation(f"loader: x slab of stage {j} requested while MMA {j - c.stages} has not read slot {s}")
        st.full[s].arrive_expect_tx()

        def land(j=j, s=s):
            st.x_landed[j] = True
            st.full[s].complete_tx()
        st.copies.append(land)
        yield None


def raw_loader(st: State):
    c = st.cfg
    for u in range(c.units):
        r, ph = u % c.raw_slots, (u // c.raw_slots) & 1
        yield wait(st.raw_empty[r], ph ^ 1)
        if u >= c.raw_slots and len(st.raw_read[u - c.raw_slots]) != c.producer_warps:
            raise ProtocolViolation(f"raw loader: box {r} refilled for unit {u} before every warp read unit {u - c.raw_slots}")
        st.raw_full[r].arrive_expect_tx()

        def land(u=u, r=r):
            st.raw_landed[u] = True
            st.raw_full[r].complete_tx()
        st.copies.append(land)
        yield None


def copy_engine(st: State):
    """Lands the bulk copies in flight, in any order."""
    while True:
        yield lambda: bool(st.copies) or st.finished_issuers
        if not st.copies:
            return
        st.copies.pop(st.rng.randrange(len(st.copies)))()
        yield None


def producer(st: State, warp: int):
    c = st.cfg
    half = c.producer_warps // 2
    team = warp // half if c.teams else 0
    for u in range(c.units):
        r, ph = u % c.raw_slots, (u // c.raw_slots) & 1
        yield wait(st.raw_full[r], ph)
        if not st.raw_landed[u]:
            raise ProtocolViolation(f"warp {warp}: read raw box {r} for unit {u} before it landed")
        st.raw_read[u].add(warp)
        yield None
        for g in range(c.stages_per_unit):
            if c.teams and g % 2 != team:
                continue
            j = u * c.stages_per_unit + g
            s, sph = j % c.stages, (j // c.stages) & 1
            yield wait(st.empty[s], sph ^ 1)
            if j >= c.stages and not st.mma_done[j - c.stages]:
                raise ProtocolViolation(f"warp {warp}: W slab of stage {j} written while MMA {j - c.stages} has not read slot {s}")
            st.w_written[j].add(warp)
            yield None
            st.full[s].arrive()
            yield None
        st.raw_empty[r].arrive()
        yield None


def mma_thread(st: State, t: int):
    c = st.cfg
    for j in range(st.n_stages):
        if j % 2 != t:
            continue
        s, ph = j % c.stages, (j // c.stages) & 1
        buf, aph = j % c.nbuf, (j // c.nbuf) & 1
        yield wait(st.acc_empty[buf], aph ^ 1)
        if c.progress_guard and j >= c.stages and (j - c.stages) % 2 != t:
            yield lambda j=j: st.mma_progress[t ^ 1] >= j - c.stages + 1
        yield wait(st.full[s], ph)
        st.mma_progress[t] = j + 1
        st.pipe[t].append(("mma", j))
        st.pipe[t].append(("commit", (st.empty[s], st.acc_full[buf])))
        yield None


def tensor_pipe(st: State):
    """Executes each thread's MMAs in its issue order, the two threads' in any order; a commit arrives when the MMAs
    its thread issued before it are done."""
    c = st.cfg
    while True:
        yield lambda: any(st.pipe) or st.finished_issuers
        ready = [t for t in (0, 1) if st.pipe[t]]
        if not ready:
            return
        t = st.rng.choice(ready)
        kind, arg = st.pipe[t].pop(0)
        if kind == "mma":
            j = arg
            if st.w_written[j] != st.writers_of(j) or not st.x_landed[j]:
                raise ProtocolViolation(f"MMA {j} ran before its operands were complete")
            if j >= c.nbuf and len(st.drained[j - c.nbuf]) != c.drain_warps:
                raise ProtocolViolation(f"MMA {j} overwrote accumulator {j % c.nbuf} before stage {j - c.nbuf} was drained")
            st.mma_done[j] = True
        else:
            for bar in arg:
                bar.arrive()
        yield None


def drain(st: State, warp: int):
    c = st.cfg
    for j in range(st.n_stages):
        buf, aph = j % c.nbuf, (j // c.nbuf) & 1
        yield wait(st.acc_full[buf], aph)
        if not st.mma_done[j]:
            raise ProtocolViolation(f"drain warp {warp}: read accumulator {buf} for stage {j} before its MMAs ran")
        st.drained[j].add(warp)
        yield None
        st.acc_empty[buf].arrive()
        yield None


def run(cfg: Config, seed: int, max_steps: int = 200000) -> None:
    """One random interleaving to completion.  Raises ProtocolViolation on a broken invariant or a deadlock."""
    rng = random.Random(seed)
    st = State(cfg)
    st.rng = rng
    st.finished_issuers = False
    issuers = {"loader": loader(st), "raw": raw_loader(st), "mma0": mma_thread(st, 0), "mma1": mma_thread(st, 1)}
    for w in range(cfg.producer_warps):
        issuers[f"prod{w}"] = producer(st, w)
    for w in range(cfg.drain_warps):
        issuers[f"drain{w}"] = drain(st, w)
    engines = {"copy": copy_engine(st), "pipe": tensor_pipe(st)}
    agents = {**issuers, **engines}
    speed = {name: rng.choice((1, 1, 2, 4, 16)) for name in agents}  # some roles much slower than others, per run
    blocked = {name: None for name in agents}  # the condition an agent waits for, or None if it can go on
    for _ in range(max_steps):
        st.finished_issuers = all(name not in agents for name in issuers)
        runnable = [n for n in agents if blocked[n] is None or blocked[n]()]
        if not runnable:
            if not agents:
                return
            raise ProtocolViolation(f"deadlock: {sorted(agents)} wait forever")
        name = rng.choices(runnable, weights=[1.0 / speed[n] for n in runnable])[0]
        try:
            blocked[name] = next(agents[name])
        except StopIteration:
            del agents[name]
            blocked.pop(name)
    raise ProtocolViolation("no completion within the step budget")
