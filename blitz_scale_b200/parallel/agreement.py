"""Agreement among the tensor-parallel shards of one replica on how much of the model is loaded.

While parameters stream in, every shard of a replica learns about arrived units from its own flag pad, at its
own pace.  A layer may only run once *all* shards hold it (its collectives involve every shard), so each shard
publishes its count of arrived units into a word of every peer's flag pad and everybody acts on the minimum.
The counts only grow during a transfer, hence the minimum any shard computes never exceeds the true minimum:
no shard starts a layer another one lacks, and all of them get there without a barrier.  This replaces the
reference's step lockers (an MPI barrier plus an allgather of loaded-layer counts per step,
src/include/step_locker.hpp:65-79,137-145).

Unit numbering follows the weight segment: unit 0 = embedding, units 1..L = layers, unit L+1 = final norm + head.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple


class LoadAgreement:
    def __init__(self, fabric, tp_ranks: Sequence[int], my_rank: int, flag0: int, layers: int):
        self.fabric, self.ranks, self.flag0, self.layers = fabric, list(tp_ranks), flag0, layers
        self.index = self.ranks.index(my_rank)
        self.published = -1

    def publish(self, units_ready: int) -> None:
        """Tell every shard (this one included) that `units_ready` units have fully arrived here."""
        if units_ready == self.published:
            return
        for r in self.ranks:
            self.fabric.set_flag(r, self.flag0 + self.index, units_ready, add=False)
        self.published = units_ready

    def agreed_units(self) -> int:
        return min(self.fabric.read_flags(self.flag0, len(self.ranks)))

    def agreed_state(self) -> Tuple[bool, int, bool]:
        """(embedding ready, layers ready, head ready) that every shard can rely on."""
        n = self.agreed_units()
        return n >= 1, max(0, min(self.layers, n - 1)), n >= self.layers + 2


class StepLog:
    """Order of live-execution steps within one tensor-parallel replica.

    Every step of a layer-interleaved prefill contains collectives, so all shards must run the same steps of the
    same tasks in the same order, although requests, relay calls and parameter units reach them at different times.
    The leading shard (index 0) alone decides; it publishes each decision as one word into a small ring in every
    other shard's flag pad before it acts, and the others execute what they read, in order.  The reference reaches
    the same agreement with a barrier and an allgather among the shards before every step
    (src/include/step_locker.hpp:100-198); here a shard never waits for more than the word it needs next.

    Word layout: bits 0-1 kind (STEP, RELAY, RELAY_NONE), 2-4 step code, 5-12 layer (+1 for a relay: 0 means "not
    embedded yet"), 13-15 activation slot, 16-23 task sequence number mod 256, 24-30 position in the log + 1 mod 128.
    The ring has 16 entries and the leader is never more than a step and a relay ahead (a step cannot finish before
    every shard has joined its collectives), so an entry is always read before its place is reused.
    """
    STEP, RELAY, RELAY_NONE = 0, 1, 2

    def __init__(self, fabric, tp_ranks: Sequence[int], my_rank: int, flag0: int, ring: int):
        self.fabric, self.ranks, self.flag0, self.ring = fabric, list(tp_ranks), flag0, ring
        self.index = self.ranks.index(my_rank)
        self.leader = self.index == 0
        self.pos = 0           # entries published (leader) or consumed (others)

    @staticmethod
    def pack(pos: int, kind: int, step: int = 0, layer: int = 0, slot: int = 0, seq_num: int = 0) -> int:
        return (kind & 3) | ((step & 7) << 2) | ((layer & 0xFF) << 5) | ((slot & 7) << 13) | ((seq_num & 0xFF) << 16) | \
            (((pos + 1) & 0x7F) << 24)

    @staticmethod
    def unpack(word: int) -> dict:
        return {"kind": word & 3, "step": (word >> 2) & 7, "layer": (word >> 5) & 0xFF, "slot": (word >> 13) & 7,
                "seq_num": (word >> 16) & 0xFF, "tag": (word >> 24) & 0x7F}

    def publish(self, kind: int, step: int = 0, layer: int = 0, slot: int = 0, seq_num: int = 0) -> None:
        assert self.leader
        word = self.pack(self.pos, kind, step, layer, slot, seq_num)
        for r in self.ranks[1:]:
            self.fabric.set_flag(r, self.flag0 + self.pos % self.ring, word, add=False)
        self.pos += 1

    def peek(self) -> Optional[dict]:
        """The next unread entry, or None if the leader has not published it yet.  `consume()` moves on."""
        word = self.fabric.read_flags(self.flag0 + self.pos % self.ring, 1)[0]
        e = self.unpack(word)
        return e if e["tag"] == ((self.pos + 1) & 0x7F) else None

    def consume(self) -> None:
        self.pos += 1
