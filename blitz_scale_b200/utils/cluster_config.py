"""The cluster description shared by workers and router: `{"init_states": [...], "machines": [...], "replicas": [...]}`,
one entry per rank (src/server/disaggregate.cc:31-50, 97-120)."""
from __future__ import annotations

from typing import List

STATES = ("Prefill", "Decode", "Normal", "Inactive")


def check_cluster(cluster, tp: int) -> List[str]:
    """Return the per-rank initial states, or raise ValueError with the mistake in words."""
    states = cluster.get("init_states") if isinstance(cluster, dict) else None
    if not isinstance(states, list) or not states or not all(s in STATES for s in states):
        raise ValueError(f"cluster config: `init_states` must be a non-empty list of {STATES} with one entry per rank")
    if tp < 1 or len(states) % tp:
        raise ValueError(f"cluster config: {len(states)} ranks cannot be split into replicas of {tp} tensor-parallel ranks")
    for r0 in range(0, len(states), tp):
        if len(set(states[r0:r0 + tp])) != 1:
            raise ValueError(f"cluster config: ranks {r0}..{r0 + tp - 1} form one replica and must share a state, "
                             f"got {states[r0:r0 + tp]}")
    machines = cluster.get("machines")
    if machines is not None and (not isinstance(machines, list) or len(machines) != len(states)):
        raise ValueError("cluster config: `machines` must name one machine per rank")
    return list(states)
