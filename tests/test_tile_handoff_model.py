"""Discrete model of the tiled GEMV's producer/consumer hand-off (cogni_ml_b200/csrc/gemv_imma.cu).

It models the protocol, not the CUDA code: four producer warps that fill a ring of S stages chunk
by chunk (one arrival per producer warp on the stage's `full` barrier, whose phase parity the
consumers test), NW consumer warps that take the items of one ordered sequence round-robin (per
tile: one item per superblock pair, then the fold of the previous tile), the monotone count of
armed chunks that a consumer checks before it trusts a phase parity, and the monotone counters
that hand tile buffers from block items to the fold and back.  Warps are scheduled at random with
weights that make some of them lag badly.  Asserted: the run ends (no deadlock), no barrier is
arrived on more often than it expects, a consumer never passes the wait of a stage before the fill
it waits for, and every tile is folded exactly once with all its partial sums present.

A parity-only variant of the same protocol (no armed-chunk counter, tile buffers handed over by
mbarrier parity) deadlocks in this model when a warp's consecutive items lie more than a ring
apart, e.g. 48 superblocks per row, 8 per stage, 4 stages.
"""
import random

import pytest


class Bar:
    def __init__(self, n, prog):
        self.init, self.pend, self.phase, self.prog = n, n, 0, prog

    def arrive(self, k=1):
        self.pend -= k
        self.prog[0] += 1
        assert self.pend >= 0, "over-arrival"
        if self.pend == 0:
            self.phase += 1
            self.pend = self.init

    def test(self, parity):  # has the phase with this parity completed?
        return (self.phase & 1) != parity


def simulate(nitems, kb, stages, ntiles, nw=16, fold_bufs=4, pw=4, seed=0):
    """nitems work items per tile, kb of them per stage (the last stage of a tile may be short)."""
    rnd = random.Random(seed)
    nch = (nitems + kb - 1) // kb
    per = nitems + 1
    prog = [0]
    full = [Bar(pw, prog) for _ in range(stages)]
    empty = [Bar(kb, prog) for _ in range(stages)]
    issued, arrivals, folded = [0], [0] * fold_bufs, [0] * fold_bufs
    done = set()

    def producer(w):
        s, par, cc = 0, 1, 0
        for _tile in range(ntiles):
            for _c in range(nch):
                while not empty[s].test(par):
                    yield
                yield
                full[s].arrive()
                cc += 1
                if w == 0:
                    issued[0] = cc
                    prog[0] += 1
                s += 1
                if s == stages:
                    s, par = 0, par ^ 1

    def consumer(w):
        li, e = divmod(w, per)
        step_li, step_e = divmod(nw, per)
        while True:
            if li > ntiles or (li == ntiles and e > 0):
                return
            if e < nitems and li < ntiles:
                c, bi = divmod(e, kb)
                cc = li * nch + c
                s, par = cc % stages, (cc // stages) & 1
                while issued[0] < cc + 1:
                    yield
                while not full[s].test(par):
                    yield
                assert full[s].phase == cc // stages + 1, "stage read before its awaited fill"
                yield
                tb = li % fold_bufs
                while folded[tb] < li // fold_bufs:
                    yield
                assert folded[tb] == li // fold_bufs
                nb = min(kb, nitems - c * kb)
                empty[s].arrive(kb - nb + 1 if bi == nb - 1 else 1)
                arrivals[tb] += 1
                prog[0] += 1
            elif li > 0:
                fl = li - 1
                tb = fl % fold_bufs
                while arrivals[tb] < (fl // fold_bufs + 1) * nitems:
                    yield
                assert arrivals[tb] == (fl // fold_bufs + 1) * nitems
                yield
                folded[tb] = fl // fold_bufs + 1
                prog[0] += 1
                assert fl not in done
                done.add(fl)
            e += step_e
            li += step_li
            if e >= per:
                e -= per
                li += 1

    gens = [producer(i) for i in range(pw)] + [consumer(w) for w in range(nw)]
    alive = list(range(len(gens)))
    weights = [rnd.choice([1, 1, 1, 20, 0.05]) for _ in gens]
    idle = 0
    while alive:
        i = rnd.choices(alive, [weights[a] for a in alive])[0]
        before = prog[0]
        try:
            next(gens[i])
            idle += 1
        except StopIteration:
            alive.remove(i)
            idle = 0
        if prog[0] != before:
            idle = 0
        assert idle < 50000, f"no progress: deadlock with {len(alive)} warps alive"
    assert done == set(range(ntiles))


@pytest.mark.parametrize("nitems,kb,stages,ntiles,nw", [
    (8, 8, 4, 28, 16),     # Q4_K 4096 columns, pairs
    (16, 16, 5, 12, 24),   # Q4_K 4096 columns, single superblocks
    (48, 8, 4, 3, 20),     # Q6_K 12288 columns
    (16, 4, 5, 14, 16),    # Q6_K 8192 columns, pairs
    (1, 16, 8, 40, 16),    # one superblock per row
    (2, 8, 8, 30, 16),
    (32, 4, 3, 4, 16),     # long rows, minimum ring
    (3, 16, 3, 17, 20),
    (10, 4, 3, 9, 16),     # short final stage
])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_hand_off_is_live_and_ordered(nitems, kb, stages, ntiles, nw, seed):
    simulate(nitems, kb, stages, ntiles, nw=nw, seed=seed)
