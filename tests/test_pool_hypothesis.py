"""Property tests of the native page pool and batch bookkeeping (hypothesis state machine, CPU).

Invariants checked after every step, whatever the interleaving of admissions, decode steps, filters, merges and
clears: no page is owned twice, the pool's accounting equals the pages the live requests hold, every live request
has exactly the pages its length needs, and finished or dropped requests give everything back.
"""
import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import settings, strategies as st  # noqa: E402
from hypothesis.stateful import RuleBasedStateMachine, invariant, precondition, rule  # noqa: E402

from blitz_scale_b200.runtime import core  # noqa: E402

PAGES, PS = 64, 16


class PoolMachine(RuleBasedStateMachine):
    def __init__(self):
        super().__init__()
        self.pool = core.PagePool(PAGES, PS)
        self.batches = []
        self.next_req = 0
        self.next_batch = 0

    @rule(lens=st.lists(st.integers(1, 70), min_size=1, max_size=4), max_new=st.integers(1, 6))
    def admit(self, lens, max_new):
        b = core.Batch(self.next_batch, self.pool)
        self.next_batch += 1
        specs = [core.SeqSpec(self.next_req + i, list(range(n)), max_new) for i, n in enumerate(lens)]
        need = sum((n + 1 + PS - 1) // PS for n in lens)
        free = self.pool.free_pages
        ok = b.add_prompts(specs)
        assert ok == (need <= free)
        if ok:
            self.next_req += len(lens)
            b.mark_prefilled()
            self.batches.append(b)
        else:
            assert self.pool.free_pages == free          # all-or-nothing

    @precondition(lambda self: self.batches)
    @rule(i=st.integers(0, 1000), count_cached=st.booleans())
    def step(self, i, count_cached):
        b = self.batches[i % len(self.batches)]
        if b.size == 0:
            return
        b.append_tokens([7] * b.size, count_cached)
        b.filter(b.unfinished_ids())
        if b.size == 0:
            self.batches.remove(b)

    @precondition(lambda self: len(self.batches) >= 2)
    @rule(i=st.integers(0, 1000), j=st.integers(0, 1000))
    def merge(self, i, j):
        a, b = self.batches[i % len(self.batches)], self.batches[j % len(self.batches)]
        if a is b:
            return
        n = a.size + b.size
        a.extend(b)
        assert a.size == n and b.size == 0
        self.batches.remove(b)

    @precondition(lambda self: self.batches)
    @rule(i=st.integers(0, 1000), k=st.integers(0, 3))
    def drop_some(self, i, k):
        b = self.batches[i % len(self.batches)]
        keep = [s.spec.id for s in b.seqs][k:]
        b.filter(keep)
        if b.size == 0:
            self.batches.remove(b)

    @precondition(lambda self: self.batches)
    @rule(i=st.integers(0, 1000))
    def clear(self, i):
        b = self.batches.pop(i % len(self.batches))
        b.clear()
        assert b.size == 0

    @invariant()
    def accounting(self):
        owned = [p for b in self.batches for s in b.seqs for p in s.pages]
        assert len(owned) == len(set(owned)), "a page is owned twice"
        assert self.pool.used_pages == len(owned) and self.pool.free_pages == PAGES - len(owned)
        assert all(self.pool.is_used(p) for p in owned)
        for b in self.batches:
            for s in b.seqs:
                if s.finish < 0:
                    assert len(s.pages) * PS >= s.total_len()      # a live request always owns the page of its next position

    def teardown(self):
        for b in self.batches:
            b.clear()
        assert self.pool.used_pages == 0


PoolMachine.TestCase.settings = settings(max_examples=60, stateful_step_count=40, deadline=None)
TestPool = PoolMachine.TestCase
