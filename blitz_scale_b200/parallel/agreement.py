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

from typing import Sequence, Tuple


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
