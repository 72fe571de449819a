"""The prefill kernel's host-checkable arithmetic, restated in Python and checked without a GPU:

* the closed-form lists of KV blocks a 256-row super-tile loads and each of its two 128-row tiles takes part in
  (``tile_blocks`` / ``tile_seen`` in moa_b200/csrc/prefill.cu) against the block layout of the oracle;
* the hand-off protocol between the TMA producer and the two MMA issuers over the K and V rings (what each
  waits for and releases, in the order the kernel does it), simulated with every MMA completing at once:
  no schedule may end with somebody still waiting.
"""
import numpy as np
import pytest

from oracle import moa_oracle as orc

STAGES = 4


def tile_blocks(t_lo, t_hi, nb, sink_b, local_b):
    hi = min(2 * t_hi + 2, nb)
    n_a = max(0, min(sink_b, hi))
    b_b = max(n_a, 2 * t_lo + 1 - local_b)
    return n_a, b_b, max(0, hi - b_b)


def tile_seen(exists, t, tb, nb, local_b):
    n_a, b_b, n_b = tb
    hi, lo = min(2 * t + 2, nb), 2 * t + 1 - local_b
    s_end = min(n_a, hi) if exists else 0
    b_begin = n_a + max(lo, b_b) - b_b
    b_end = n_a + min(hi, b_b + n_b) - b_b
    if not exists or n_b == 0 or b_end < b_begin:
        b_end = b_begin
    return [i if i < s_end else b_begin + (i - s_end) for i in range(s_end + b_end - b_begin)]


def block_of(tb, u):
    n_a, b_b, _ = tb
    return u if u < n_a else b_b + (u - n_a)


def lists(n, sink_b, local_b, st):
    nb = -(-n // 64)
    t0, t1 = 2 * st, 2 * st + 1
    active1 = t1 * 128 < n
    tb = tile_blocks(t0, t1 if active1 else t0, nb, sink_b, local_b)
    return tb, [tile_seen(True, t0, tb, nb, local_b), tile_seen(active1, t1, tb, nb, local_b)], tb[0] + tb[2]


CASES = [(n, s, l) for n in (64, 200, 256, 1000, 2048, 4096, 5000) for s in (0, 1, 2, 3) for l in (1, 2, 3, 7, 16, 40, 100)]


@pytest.mark.parametrize("n,sink_b,local_b", CASES)
def test_tile_lists_are_exactly_the_blocks_the_tile_rows_see(n, sink_b, local_b):
    nb = -(-n // 64)
    layout = orc.block_layout(nb, sink_b, local_b)          # [query block, kv block]
    for st in range(-(-n // 256)):
        tb, seen, nkv = lists(n, sink_b, local_b, st)
        loaded = [block_of(tb, u) for u in range(nkv)]
        assert loaded == sorted(set(loaded)) and all(0 <= b < nb for b in loaded)
        for x in range(2):
            qblocks = [qb for qb in (2 * (2 * st + x), 2 * (2 * st + x) + 1) if qb < nb]
            want = sorted({int(j) for qb in qblocks for j in np.nonzero(layout[qb])[0]})
            got = [block_of(tb, u) for u in seen[x]]
            assert got == want, (st, x)
            assert set(got) <= set(loaded)


def simulate(n, sink_b, local_b, st):
    """Producer and the two issuers as generators that yield what they wait for; returns None when everyone
    finishes, or the pending waits on a deadlock."""
    tb, seen, nkv = lists(n, sink_b, local_b, st)
    kfull, vfull = [0] * STAGES, [0] * STAGES
    kempty, vempty = [[0] * STAGES for _ in range(2)], [[0] * STAGES for _ in range(2)]

    def producer():
        for u in range(nkv + 1):
            if u < nkv:
                yield ("kempty", u % STAGES, u // STAGES)
                kfull[u % STAGES] += 1
            if u >= 1:
                uv = u - 1
                yield ("vempty", uv % STAGES, uv // STAGES)
                vfull[uv % STAGES] += 1

    def issuer(x):
        sn, total = seen[x], len(seen[x])

        def skip_k(a, b):
            for w in range(a, b):
                yield ("kfull", w % STAGES, w // STAGES + 1)
                kempty[x][w % STAGES] += 1

        def skip_v(a, b):
            for w in range(a, b):
                yield ("vfull", w % STAGES, w // STAGES + 1)
                vempty[x][w % STAGES] += 1

        def skip_both(a, b):
            for w in range(a, b):
                yield from skip_k(w, w + 1)
                yield from skip_v(w, w + 1)

        def qk(j):
            u = sn[j]
            yield ("kfull", u % STAGES, u // STAGES + 1)
            kempty[x][u % STAGES] += 1

        if total == 0:
            yield from skip_both(0, nkv)
            return
        yield from skip_both(0, sn[0])
        yield from qk(0)
        if total > 1:
            yield from skip_k(sn[0] + 1, sn[1])
            yield from qk(1)
        u_prev, u, u1 = -1, sn[0], (sn[1] if total > 1 else -1)
        for i in range(total):
            ahead = i + 2 < total
            u2 = sn[i + 2] if ahead else -1
            if i > 0 and u != u_prev + 1:
                yield from skip_v(u_prev + 1, u)
            if ahead and u2 != u1 + 1:
                yield from skip_k(u1 + 1, u2)
            yield ("vfull", u % STAGES, u // STAGES + 1)
            if ahead:
                yield ("kfull", u2 % STAGES, u2 // STAGES + 1)
            vempty[x][u % STAGES] += 1          # commit after O += P V
            if ahead:
                kempty[x][u2 % STAGES] += 1     # commit after the S two steps ahead
            u_prev, u, u1 = u, u1, u2
        yield from skip_both(sn[-1] + 1, nkv)

    def ready(req):
        kind, s, need = req
        if kind == "kempty":
            return kempty[0][s] >= need and kempty[1][s] >= need
        if kind == "vempty":
            return vempty[0][s] >= need and vempty[1][s] >= need
        return (kfull if kind == "kfull" else vfull)[s] >= need

    agents = {"producer": producer(), "issuer A": issuer(0), "issuer B": issuer(1)}
    pending = {}
    for name, g in agents.items():
        pending[name] = next(g, None)
    while True:
        progressed = False
        for name, g in agents.items():
            while pending[name] is not None and ready(pending[name]):
                pending[name] = next(g, None)
                progressed = True
        if all(v is None for v in pending.values()):
            return None
        if not progressed:
            return dict(pending)


@pytest.mark.parametrize("n,sink_b,local_b", CASES)
def test_ring_protocol_never_deadlocks(n, sink_b, local_b):
    for st in range(-(-n // 256)):
        assert simulate(n, sink_b, local_b, st) is None, (st,)


# ---------------------------------------------------------------------------------------------------
# Barrier phases.  An mbarrier wait only sees the parity of the phase it waits for, so a barrier whose
# signaller can complete phase n+1 before the waiter has looked at phase n reads as "phase n not complete"
# for ever.  The model below runs producer, issuers and softmax groups under random schedules and checks, at
# every look at a barrier, that it is at most the awaited phase ahead -- never one more.
# ---------------------------------------------------------------------------------------------------
class Barrier:
    def __init__(self, name):
        self.name, self.done = name, 0          # number of completed phases

    def look(self, need):
        """True when phase number ``need`` (1-based) is complete; asserts the parity wait is unambiguous."""
        assert self.done <= need, f"{self.name}: {self.done} phases complete while phase {need} is awaited"
        return self.done >= need


def simulate_phases(n, sink_b, local_b, st, rng, p_barriers_per_tile):
    tb, seen, nkv = lists(n, sink_b, local_b, st)
    kfull = [Barrier(f"k_full[{s}]") for s in range(STAGES)]
    vfull = [Barrier(f"v_full[{s}]") for s in range(STAGES)]
    kempty = [[Barrier(f"k_empty[{x}][{s}]") for s in range(STAGES)] for x in range(2)]
    vempty = [[Barrier(f"v_empty[{x}][{s}]") for s in range(STAGES)] for x in range(2)]
    sfull = [[Barrier(f"s_full[{x}][{b}]") for b in range(2)] for x in range(2)]
    pfull = [[Barrier(f"p_full[{x}][{b}]") for b in range(p_barriers_per_tile)] for x in range(2)]

    def p_of(x, i):      # barrier and phase number of "P(i) is ready"
        return (pfull[x][i & 1], (i >> 1) + 1) if p_barriers_per_tile == 2 else (pfull[x][0], i + 1)

    def producer():
        for u in range(nkv + 1):
            if u < nkv:
                s, need = u % STAGES, u // STAGES
                while not (kempty[0][s].look(need) and kempty[1][s].look(need)):
                    yield
                kfull[s].done += 1
            if u >= 1:
                s, need = (u - 1) % STAGES, (u - 1) // STAGES
                while not (vempty[0][s].look(need) and vempty[1][s].look(need)):
                    yield
                vfull[s].done += 1

    def issuer(x):
        sn, total = seen[x], len(seen[x])

        def wait(bar, need):
            while not bar.look(need):
                yield

        def skip(kind, a, b):
            for w in range(a, b):
                full, empty = (kfull, kempty) if kind == "k" else (vfull, vempty)
                yield from wait(full[w % STAGES], w // STAGES + 1)
                empty[x][w % STAGES].done += 1

        def skip_both(a, b):
            for w in range(a, b):
                yield from skip("k", w, w + 1)
                yield from skip("v", w, w + 1)

        def qk(j):
            u = sn[j]
            yield from wait(kfull[u % STAGES], u // STAGES + 1)
            sfull[x][j & 1].done += 1
            kempty[x][u % STAGES].done += 1

        if total == 0:
            yield from skip_both(0, nkv)
            return
        yield from skip_both(0, sn[0])
        yield from qk(0)
        if total > 1:
            yield from skip("k", sn[0] + 1, sn[1])
            yield from qk(1)
        u_prev, u, u1 = -1, sn[0], (sn[1] if total > 1 else -1)
        for i in range(total):
            ahead = i + 2 < total
            u2 = sn[i + 2] if ahead else -1
            if i > 0 and u != u_prev + 1:
                yield from skip("v", u_prev + 1, u)
            if ahead and u2 != u1 + 1:
                yield from skip("k", u1 + 1, u2)
            yield from wait(vfull[u % STAGES], u // STAGES + 1)
            if ahead:
                yield from wait(kfull[u2 % STAGES], u2 // STAGES + 1)
            bar, need = p_of(x, i)
            yield from wait(bar, need)
            vempty[x][u % STAGES].done += 1
            if ahead:
                sfull[x][i & 1].done += 1
                kempty[x][u2 % STAGES].done += 1
            u_prev, u, u1 = u, u1, u2
        yield from skip_both(sn[-1] + 1, nkv)

    def softmax(x):
        total = len(seen[x])
        for i in range(total):
            while not sfull[x][i & 1].look((i >> 1) + 1):
                yield
            if 0 < i < total - 1 and rng.randint(3) == 0:
                # a rescale of O: "S(i+1) complete" stands for "P.V(i-1) complete"
                while not sfull[x][(i + 1) & 1].look(((i + 1) >> 1) + 1):
                    yield
            p_of(x, i)[0].done += 1

    agents = [producer(), issuer(0), issuer(1), softmax(0), softmax(1)]
    alive = list(range(len(agents)))
    idle_rounds = 0
    while alive:
        k = alive[rng.randint(len(alive))]
        before = _snapshot(kfull, vfull, kempty, vempty, sfull, pfull)
        try:
            next(agents[k])
        except StopIteration:
            alive.remove(k)
        idle_rounds = idle_rounds + 1 if _snapshot(kfull, vfull, kempty, vempty, sfull, pfull) == before else 0
        assert idle_rounds < 4000, "nobody makes progress"


def _snapshot(*groups):
    out = []
    for g in groups:
        for item in g:
            out.extend(b.done for b in item) if isinstance(item, list) else out.append(item.done)
    return out


@pytest.mark.parametrize("n,sink_b,local_b", [(4096, 1, 100), (4096, 1, 7), (2048, 2, 3), (1000, 0, 2), (5000, 3, 16)])
def test_no_barrier_runs_two_phases_ahead_under_random_schedules(n, sink_b, local_b):
    for seed in range(6):
        rng = np.random.RandomState(seed)
        for st in range(0, -(-n // 256), 3):
            simulate_phases(n, sink_b, local_b, st, rng, p_barriers_per_tile=2)


def test_the_model_catches_a_single_p_barrier():
    """With one "P is ready" barrier per tile the softmax group can complete two phases while the issuer waits
    for TMA data: the model must notice (this is the stall the kernel once had)."""
    caught = 0
    for seed in range(20):
        try:
            simulate_phases(4096, 1, 100, 8, np.random.RandomState(seed), p_barriers_per_tile=1)
        except AssertionError as exc:
            caught += "p_full" in str(exc)
    assert caught > 0


# ---------------------------------------------------------------------------------------------------
# The persistent form: one block works through a sequence of super-tiles.  Every role keeps running counts
# (ring entries, S/P buffers, phases of the per-super-tile barriers), the producer publishes the next
# super-tile through a two-entry ring and runs ahead.  Same model as above, over a whole sequence, with the
# barriers that only exist across super-tiles (tile_full / tile_empty, q_full / q_empty, pv_done, o_full).
# ---------------------------------------------------------------------------------------------------
class CountBarrier(Barrier):
    def __init__(self, name, count):
        super().__init__(name)
        self.count, self.pending = count, 0

    def arrive(self):
        self.pending += 1
        if self.pending == self.count:
            self.pending, self.done = 0, self.done + 1


def simulate_persistent(units, rng, q_empty_per_issuer=True, q_wait_first=True, q_load_every_unit=False):
    """units: [(n, sink_b, local_b, st), ...] in the order one block receives them.

    The producer's bulk copies are modelled as what they are: the producer *arms* a "full" barrier (expect-tx)
    and the copy lands at some later, random time.  A barrier may only be armed when its previous phase has
    completed, and no copy may be in flight when the block's roles have all finished."""

    def hand_back(bar):
        if isinstance(bar, CountBarrier):
            bar.arrive()
        else:
            bar.done += 1

    work = [lists(n, s, l, st) for n, s, l, st in units]
    kfull = [Barrier(f"k_full[{s}]") for s in range(STAGES)]
    vfull = [Barrier(f"v_full[{s}]") for s in range(STAGES)]
    kempty = [[Barrier(f"k_empty[{x}][{s}]") for s in range(STAGES)] for x in range(2)]
    vempty = [[Barrier(f"v_empty[{x}][{s}]") for s in range(STAGES)] for x in range(2)]
    sfull = [[Barrier(f"s_full[{x}][{b}]") for b in range(2)] for x in range(2)]
    pfull = [[Barrier(f"p_full[{x}][{b}]") for b in range(2)] for x in range(2)]
    pvdone = [Barrier(f"pv_done[{x}]") for x in range(2)]
    ofull = [Barrier(f"o_full[{x}]") for x in range(2)]
    qfull = Barrier("q_full")
    qempty = [Barrier(f"q_empty[{x}]") for x in range(2)] if q_empty_per_issuer else [CountBarrier("q_empty", 2)] * 2
    tfull = [Barrier(f"tile_full[{s}]") for s in range(2)]
    tempty = [CountBarrier(f"tile_empty[{s}]", 4) for s in range(2)]     # 2 issuers + 2 softmax groups
    slot_value = [None, None]
    finished = {"o_read": [0, 0], "o_written_first": [0, 0]}

    in_flight = []
    armed = {}

    def arm(bar):
        assert armed.get(bar.name, 0) == bar.done, f"{bar.name} armed again before its previous phase completed"
        armed[bar.name] = bar.done + 1
        in_flight.append(bar)

    def copies():
        while True:
            if in_flight and rng.randint(3) == 0:
                in_flight.pop(rng.randint(len(in_flight))).done += 1
            yield

    def wait(bar, need):
        while not bar.look(need):
            yield

    def producer():
        ring = 0
        for n in range(len(units) + 1):
            unit = n if n < len(units) else -1
            slot = n & 1
            if n > 0 and q_wait_first:                           # both issuers are done with the previous Q
                while not (qempty[0].look(n) and qempty[1].look(n)):
                    yield
            yield from wait(tempty[slot], n >> 1)                # phase (n >> 1) of the slot's "empty" complete
            slot_value[slot] = unit
            tfull[slot].done += 1
            if unit < 0:
                return
            nkv = work[unit][2]
            if n > 0 and not q_wait_first:
                while not (qempty[0].look(n) and qempty[1].look(n)):
                    yield
            if nkv > 0 or q_load_every_unit:
                arm(qfull)
            for u in range(nkv + 1):
                if u < nkv:
                    g = ring + u
                    while not (kempty[0][g % STAGES].look(g // STAGES) and kempty[1][g % STAGES].look(g // STAGES)):
                        yield
                    arm(kfull[g % STAGES])
                if u >= 1:
                    g = ring + u - 1
                    while not (vempty[0][g % STAGES].look(g // STAGES) and vempty[1][g % STAGES].look(g // STAGES)):
                        yield
                    arm(vfull[g % STAGES])
            ring += nkv

    def take_unit(n):
        slot = n & 1
        yield from wait(tfull[slot], (n >> 1) + 1)
        unit = slot_value[slot]
        tempty[slot].arrive()
        return unit

    def issuer(x):
        ring = sbase = q_loads = 0
        n = 0
        while True:
            unit = yield from take_unit(n)
            if unit < 0:
                return
            tb, seen, nkv = work[unit]
            sn, total = seen[x], len(seen[x])

            def skip(kind, a, b):
                for e in range(a, b):
                    g = ring + e
                    full, empty = (kfull, kempty) if kind == "k" else (vfull, vempty)
                    yield from wait(full[g % STAGES], g // STAGES + 1)
                    empty[x][g % STAGES].done += 1

            def skip_both(a, b):
                for e in range(a, b):
                    yield from skip("k", e, e + 1)
                    yield from skip("v", e, e + 1)

            def qk_mmas(j, g):
                gs = sbase + j
                sfull[x][gs & 1].done += 1
                kempty[x][g % STAGES].done += 1
                if j == total - 1:
                    hand_back(qempty[x])

            def issue_qk(j):
                g = ring + sn[j]
                yield from wait(kfull[g % STAGES], g // STAGES + 1)
                qk_mmas(j, g)

            if total > 0:
                yield from skip_both(0, sn[0])
                yield from wait(qfull, (n if q_load_every_unit else q_loads) + 1)
                yield from issue_qk(0)
                if total > 1:
                    yield from skip("k", sn[0] + 1, sn[1])
                    yield from issue_qk(1)
            else:
                hand_back(qempty[x])
                yield from skip_both(0, nkv)
            u_prev, u, u1 = -1, (sn[0] if total > 0 else -1), (sn[1] if total > 1 else -1)
            for i in range(total):
                ahead = i + 2 < total
                u2 = sn[i + 2] if ahead else -1
                if i > 0 and u != u_prev + 1:
                    yield from skip("v", u_prev + 1, u)
                if ahead and u2 != u1 + 1:
                    yield from skip("k", u1 + 1, u2)
                gv = ring + u
                yield from wait(vfull[gv % STAGES], gv // STAGES + 1)
                if ahead:
                    gk = ring + u2
                    yield from wait(kfull[gk % STAGES], gk // STAGES + 1)
                gs = sbase + i
                yield from wait(pfull[x][gs & 1], (gs >> 1) + 1)
                if i == 0:
                    # the first O += P V of a super-tile overwrites O: the previous epilogue must have read it
                    assert finished["o_read"][x] == finished["o_written_first"][x], "O overwritten before it was read"
                    finished["o_written_first"][x] += 1
                if i + 2 == total:
                    pvdone[x].done += 1
                vempty[x][gv % STAGES].done += 1
                if ahead:
                    qk_mmas(i + 2, ring + u2)
                u_prev, u, u1 = u, u1, u2
            if total > 0:
                ofull[x].done += 1
                yield from skip_both(sn[-1] + 1, nkv)
            ring += nkv
            sbase += total
            q_loads += 1 if nkv > 0 else 0
            n += 1

    def softmax(x):
        sbase = n_pv = n_o = 0
        n = 0
        while True:
            unit = yield from take_unit(n)
            if unit < 0:
                return
            total = len(work[unit][1][x])
            for i in range(total):
                gs = sbase + i
                yield from wait(sfull[x][gs & 1], (gs >> 1) + 1)
                if i > 0 and rng.randint(3) == 0:
                    if i + 1 < total:
                        yield from wait(sfull[x][(gs + 1) & 1], ((gs + 1) >> 1) + 1)
                    else:
                        yield from wait(pvdone[x], n_pv + 1)
                pfull[x][gs & 1].done += 1
            if total > 0:
                yield from wait(ofull[x], n_o + 1)
                finished["o_read"][x] += 1
            sbase += total
            n_pv += 1 if total >= 2 else 0
            n_o += 1 if total > 0 else 0
            n += 1

    agents = [producer(), issuer(0), issuer(1), softmax(0), softmax(1), copies()]
    alive = list(range(len(agents)))
    everything = (kfull, vfull, kempty, vempty, sfull, pfull, [pvdone], [ofull], [[qfull] + qempty], [tfull], [tempty])
    idle_rounds = 0
    while alive != [5]:                       # until every role of the block has finished
        k = alive[rng.randint(len(alive))]
        before = _snapshot(*everything)
        try:
            next(agents[k])
        except StopIteration:
            alive.remove(k)
        idle_rounds = idle_rounds + 1 if _snapshot(*everything) == before else 0
        assert idle_rounds < 20000, "nobody makes progress"
    assert not in_flight, f"{in_flight[0].name}: a copy is still in flight when the block ends"
    assert finished["o_read"] == finished["o_written_first"]


def test_persistent_sequence_of_super_tiles_keeps_every_barrier_unambiguous():
    """Random sequences of super-tiles of different heads and lengths through one block, under random schedules:
    no wait may ever be ambiguous (a barrier two phases ahead of its waiter), nobody may stall, and O is never
    overwritten before the previous epilogue has read it.  Includes super-tiles in which one tile or both see
    nothing, single-entry tiles, and ragged last super-tiles."""
    shapes = [(4096, 1, 100), (4096, 1, 7), (2048, 2, 3), (1000, 0, 2), (5000, 3, 16), (200, 1, 1), (64, 0, 0),
              (700, 0, 0), (300, 1, 0), (129, 1, 1), (256, 1, 40), (513, 0, 0), (17, 0, 0)]
    for seed in range(12):
        rng = np.random.RandomState(100 + seed)
        units = []
        for _ in range(int(rng.randint(2, 9))):
            n, s, l = shapes[rng.randint(len(shapes))]
            units.append((n, s, l, int(rng.randint(-(-n // 256)))))
        simulate_persistent(units, rng)


def test_the_persistent_model_catches_a_shared_q_hand_back_barrier():
    """With one "Q is free" barrier of count 2 shared by the two issuers, an issuer that has nothing to do in the
    next super-tile arrives twice in a row and completes the phase on its own; the producer then overwrites Q
    (and completes a second phase of q_full, or sees q_empty two phases on) while the other issuer still waits for
    the first (when, in addition, the next super-tile is published before the hand-back has been seen).  The model
    must notice."""
    units = [(700, 0, 0, 1), (64, 0, 0, 0), (2048, 2, 3, 4), (2048, 2, 3, 1)]
    caught = 0
    for seed in range(40):
        try:
            simulate_persistent(units, np.random.RandomState(seed), q_empty_per_issuer=False, q_wait_first=False)
        except AssertionError as exc:
            caught += "q_full" in str(exc) or "q_empty" in str(exc)
    assert caught > 0


def test_the_persistent_model_catches_a_q_load_nobody_waits_for():
    """A super-tile that visits no KV block (no sink, no window, at most 64 rows at the ragged end) has no reader of
    Q.  Loading its Q all the same leaves a copy in flight when the block ends, or has q_full armed a second time
    inside one phase when another super-tile follows at once.  The model must notice both; the kernel therefore
    loads Q only for super-tiles that visit something and counts q_full's phases by those."""
    in_flight = armed_twice = 0
    for seed in range(40):
        for units in ([(2048, 2, 3, 4), (64, 0, 0, 0)], [(64, 0, 0, 0), (513, 0, 0, 2), (2048, 2, 3, 1)]):
            try:
                simulate_persistent(units, np.random.RandomState(seed), q_load_every_unit=True)
            except AssertionError as exc:
                in_flight += "in flight" in str(exc)
                armed_twice += "armed again" in str(exc)
            simulate_persistent(units, np.random.RandomState(seed))          # the kernel's rule passes
    assert in_flight > 0 and armed_twice > 0


def test_the_persistent_model_catches_publishing_before_q_is_handed_back():
    """If the producer published the next super-tile before it has seen "Q is free" for the previous one, an
    issuer with nothing to do in the next one would hand Q back a second time first, and the producer's wait
    would see a barrier two phases on.  The model must notice — this fixes the order in the kernel."""
    units = [(4096, 1, 7, 9), (64, 0, 0, 0), (300, 1, 0, 0), (5000, 3, 16, 16)]
    caught = 0
    for seed in range(40):
        try:
            simulate_persistent(units, np.random.RandomState(seed), q_wait_first=False)
        except AssertionError as exc:
            caught += "q_empty" in str(exc)
    assert caught > 0


def tile_coord(unit, B, H, nsuper, chunk):
    """The kernel's unit -> (batch, head, super-tile) map (``tile_coord`` in moa_b200/csrc/prefill.cu)."""
    heads = B * H
    per_chunk, full = heads * chunk, nsuper // chunk
    k, width, r = unit // per_chunk, chunk, unit % per_chunk
    if k >= full:
        k, width, r = full, nsuper - full * chunk, unit - full * per_chunk
    bh, j = r // width, r % width
    return bh // H, bh % H, nsuper - 1 - k * chunk - j


@pytest.mark.parametrize("B,H,nsuper,chunk", [(1, 32, 8, 1), (2, 3, 7, 3), (1, 32, 64, 4), (1, 5, 10, 10), (3, 2, 9, 4),
                                              (1, 1, 1, 1), (1, 4, 5, 5), (2, 2, 6, 2), (1, 3, 11, 16 // 2)])
def test_unit_order_covers_every_super_tile_once_heaviest_chunk_first(B, H, nsuper, chunk):
    units = [tile_coord(u, B, H, nsuper, chunk) for u in range(B * H * nsuper)]
    assert sorted(units) == sorted((b, h, st) for b in range(B) for h in range(H) for st in range(nsuper))
    # chunks are handed out from the end of the sequence backwards: the chunk index never decreases ...
    chunk_of = [(nsuper - 1 - st) // chunk for _, _, st in units]
    assert chunk_of == sorted(chunk_of)
    # ... and inside a chunk a head's super-tiles are consecutive and descending
    for i in range(1, len(units)):
        if units[i][:2] == units[i - 1][:2] and chunk_of[i] == chunk_of[i - 1]:
            assert units[i][2] == units[i - 1][2] - 1
