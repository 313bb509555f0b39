"""Host simulation of the mbarrier protocol of `cross_tc_kernel` (csrc/hz_cross_tc.cuh).

The kernel's roles (TMA producer, UMMA issuer, rewriters, two consumer groups) are run as
coroutines under a random scheduler with the kernel's own index arithmetic: which barrier a role
waits on, with which parity, and which buffer it then touches. A parity wait returns as soon as
the barrier's phase differs from the one asked for, so a waiter that skipped a phase would pass
early; the simulation checks that every role always finds the unit it expects in the operand
buffer, accumulator, scale slot and ring stage it reads, and that nothing deadlocks."""
import random

import pytest


class Barrier:
    def __init__(self, count=1):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def done(self, parity):
        return (self.phase & 1) != parity


def simulate(n_units, chunks, ring, seed):
    rnd = random.Random(seed)
    conv, afree = [Barrier(), Barrier()], [Barrier(), Barrier()]
    tfull, tfree = [Barrier() for _ in range(4)], [Barrier() for _ in range(4)]
    jfull, jfree = [Barrier() for _ in range(2 * ring)], [Barrier() for _ in range(2 * ring)]
    operand, acc, stage, scale = [None, None], [None, None], [None] * (2 * ring), [None] * 4
    errors = []

    def producer():
        for i in range(n_units):
            g, lu = (i >> 1) & 1, (i >> 2) * 2 + (i & 1)
            for ch in range(chunks):
                lidx = lu * chunks + ch
                slot = g * ring + lidx % ring
                if lidx >= ring:
                    while not jfree[slot].done((lidx // ring - 1) & 1):
                        yield
                stage[slot] = (i, ch)
                jfull[slot].arrive()
                yield

    def issuer():
        for i in range(n_units):
            buf, g = i & 1, (i >> 1) & 1
            while not conv[buf].done((i >> 1) & 1):
                yield
            if i >= 2:
                while not tfree[(g ^ 1) * 2 + buf].done(((i - 2) >> 2) & 1):
                    yield
            if operand[buf] != i:
                errors.append(("operand", i, operand[buf]))
            yield
            acc[buf] = i
            tfull[g * 2 + buf].arrive()
            afree[buf].arrive()
            yield

    def rewriter():
        for i in range(n_units):
            buf = i & 1
            if i >= 2:
                while not afree[buf].done(((i >> 1) - 1) & 1):
                    yield
            scale[i & 3] = i
            operand[buf] = i
            yield
            conv[buf].arrive()
            yield

    def consumer(group):
        i = 2 * group
        while i < n_units:
            for s in range(2):
                ii = i + s
                if ii >= n_units:
                    continue
                buf = ii & 1
                while not tfull[group * 2 + buf].done((ii >> 2) & 1):
                    yield
                if scale[ii & 3] != ii:
                    errors.append(("scale", ii, scale[ii & 3]))
                for ch in range(chunks):
                    lidx = ((ii >> 2) * 2 + s) * chunks + ch
                    slot = group * ring + lidx % ring
                    if acc[buf] != ii:
                        errors.append(("accumulator", ii, acc[buf]))
                    while not jfull[slot].done((lidx // ring) & 1):
                        yield
                    if ch == chunks - 1:
                        tfree[group * 2 + buf].arrive()
                    if stage[slot] != (ii, ch):
                        errors.append(("stage", ii, ch, stage[slot]))
                    yield
                    jfree[slot].arrive()
            for _ in range(rnd.randint(0, 6)):      # the contraction with T_i
                yield
            i += 4

    alive = [producer(), issuer(), rewriter(), consumer(0), consumer(1)]
    for _ in range(200000):
        if not alive:
            return errors
        t = rnd.choice(alive)
        try:
            next(t)
        except StopIteration:
            alive.remove(t)
    return errors + [("deadlock",)]


@pytest.mark.parametrize("chunks,ring", [(1, 2), (2, 2), (3, 2), (6, 2), (1, 3), (3, 4)])
def test_every_role_sees_its_own_unit_and_nothing_deadlocks(chunks, ring):
    for n_units in range(0, 19):
        for seed in range(12):
            assert simulate(n_units, chunks, ring, seed) == [], (n_units, chunks, ring, seed)


def test_shared_barriers_between_the_consumer_groups_would_pass_early():
    """The variant that was rejected: one tfull barrier per accumulator for both groups. The second
    group's first wait (parity 1 on a barrier still in phase 0) passes before the unit exists."""
    b = Barrier()
    assert b.done(1)            # phase 0, parity 1 asked: reads as complete
    assert not b.done(0)
