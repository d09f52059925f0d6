"""Host-side model of the hand-off protocol of the TMA-fed convolution kernel
(deep-learning-framework_b200/csrc/kai_conv_igemm_tma.cu): one producer, several MMA-issuing warps that own
alternate accumulation chunks, and the accumulate warps, synchronised by phase-parity barriers.

An mbarrier parity wait only knows "the phase with this parity is over": it also passes on a barrier that is two
phases behind.  The model runs the roles under many interleavings and checks, at every wait that passes, the fact the
kernel relies on there (the stage is loaded and still in its slot, the accumulator was read, ...), and that nothing
deadlocks.  It also shows why every issuer needs its own "stage loaded" barriers: with one shared ring the same
model finds a wait that passes too early.
"""
import random

import pytest


class Barrier:
    def __init__(self, count):
        self.count, self.pending, self.done = count, count, 0      # done = completed phases

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.pending, self.done = self.count, self.done + 1

    def passed(self, parity):
        """mbarrier.try_wait.parity: true when the phase with this parity is not the one in progress."""
        return (self.done & 1) != parity


class Model:
    def __init__(self, tiles, k_stages, chunk_stages, slots, issuers, acc_bufs, own_full_barriers):
        self.S, self.NI, self.B = slots, issuers, acc_bufs
        self.own = own_full_barriers
        # the stage sequence: (global stage g, chunk c, last stage of its chunk)
        self.stages, c = [], 0
        for _ in range(tiles):
            ks = 0
            while ks < k_stages:
                n = min(chunk_stages, k_stages - ks)
                for i in range(n):
                    self.stages.append((len(self.stages), c, i == n - 1))
                ks += n
                c += 1
        self.n_chunks = c
        self.full = [[Barrier(1) for _ in range(slots)] for _ in range(issuers if own_full_barriers else 1)]
        self.empty = [Barrier(1) for _ in range(slots)]
        self.tmem_full = [Barrier(1) for _ in range(acc_bufs)]
        self.tmem_empty = [Barrier(1) for _ in range(acc_bufs)]
        self.slot_holds = [None] * slots          # which stage's data is in the slot
        self.consumed = set()
        self.mma_done = set()
        self.acc_read = set()
        self.errors = []

    # Each role is a generator that yields (barrier, parity, check) before every wait and resumes once it passed.
    def producer(self):
        given = [0] * self.NI
        for g, c, _ in self.stages:
            slot = g % self.S
            yield self.empty[slot], ((g // self.S) & 1) ^ 1, (lambda g=g: g < self.S or (g - self.S) in self.consumed)
            self.slot_holds[slot] = g
            owner = c % self.NI
            if self.own:
                self.full[owner][given[owner] % self.S].arrive()
                given[owner] += 1
            else:
                self.full[0][slot].arrive()

    def issuer(self, me):
        j = 0
        for g, c, last in self.stages:
            if c % self.NI != me:
                continue
            first = g == 0 or self.stages[g - 1][1] != c
            if first:
                yield (self.tmem_empty[c % self.B], ((c // self.B) & 1) ^ 1,
                       (lambda c=c: c < self.B or (c - self.B) in self.acc_read))
            slot = g % self.S
            if self.own:
                bar, parity = self.full[me][j % self.S], (j // self.S) & 1
            else:
                bar, parity = self.full[0][slot], (g // self.S) & 1
            yield bar, parity, (lambda g=g, slot=slot: self.slot_holds[slot] == g)
            j += 1
            self.consumed.add(g)
            self.empty[slot].arrive()
            if last:
                self.mma_done.add(c)
                self.tmem_full[c % self.B].arrive()

    def accumulate(self):
        for c in range(self.n_chunks):
            yield self.tmem_full[c % self.B], (c // self.B) & 1, (lambda c=c: c in self.mma_done)
            self.acc_read.add(c)
            self.tmem_empty[c % self.B].arrive()

    def run(self, pick):
        roles = [self.producer()] + [self.issuer(i) for i in range(self.NI)] + [self.accumulate()]
        waiting = [next(r, None) for r in roles]
        while any(w is not None for w in waiting):
            ready = [i for i, w in enumerate(waiting) if w is not None and w[0].passed(w[1])]
            if not ready:
                self.errors.append("deadlock")
                return
            i = pick(ready)
            if not waiting[i][2]():
                self.errors.append(f"role {i}: a wait passed before its condition held")
                return
            waiting[i] = next(roles[i], None)


# (slots, issuers, accumulator buffers) of the two instantiations: 64 and 128 output channels
CONFIGS = [(4, 4, 8), (3, 4, 4)]


@pytest.mark.parametrize("slots,issuers,bufs", CONFIGS)
@pytest.mark.parametrize("chunk_stages", [1, 2])
@pytest.mark.parametrize("k_stages", [1, 2, 5, 18])
def test_own_barriers_never_pass_early(slots, issuers, bufs, chunk_stages, k_stages):
    rng = random.Random(slots * 1000 + issuers * 100 + chunk_stages * 10 + k_stages)
    picks = [lambda r: r[0], lambda r: r[-1]] + [lambda r: rng.choice(r)] * 30
    for pick in picks:
        m = Model(7, k_stages, chunk_stages, slots, issuers, bufs, own_full_barriers=True)
        m.run(pick)
        assert m.errors == []
        assert len(m.acc_read) == m.n_chunks and len(m.consumed) == len(m.stages)


def test_shared_full_barriers_can_pass_early():
    """Three issuers on a shared ring of three "stage loaded" barriers: the issuer of the third chunk asks for the
    second phase of a barrier whose first phase has not happened yet, and the parity test lets it through."""
    m = Model(2, 12, 2, 3, 3, 4, own_full_barriers=False)
    m.run(lambda r: r[-1])          # always run the role furthest down the list that can move
    assert m.errors and "before its condition" in m.errors[0]
