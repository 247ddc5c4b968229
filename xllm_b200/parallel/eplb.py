"""Expert-parallel load balancing: measure per-expert load, re-place (and replicate) experts.

Parity: `EplbManager`, `EplbPolicy`, `EplbExecutor` (xllm/core/framework/eplb/eplb_manager.cpp,
eplb_policy.cpp, eplb_executor.cpp; engine side llm_engine.cpp:224-237, 1259-1302): workers report
how many tokens each expert received, the manager aggregates the counts, a policy computes a new
placement with `num_redundant` extra replicas of the hottest experts, and layers switch to it one at
a time (prepare the weights of the new placement in a spare buffer, then activate) so that serving
never stops.

Placement of one layer: `slots[rank][j]` = logical expert held in physical slot j of that rank;
every rank has the same number of slots.  Tokens routed to a replicated expert are spread over its
replicas round-robin (`replica_table`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np


def balanced_placement(load: Sequence[float], n_ranks: int, n_redundant: int = 0) -> List[List[int]]:
    """Greedy placement: replicate the experts with the highest load per replica until the spare
    slots are used, then assign replicas to ranks heaviest-first onto the least loaded rank that has
    a free slot and does not already hold that expert."""
    load = np.asarray(load, dtype=np.float64)
    E = len(load)
    total = E + n_redundant
    assert total % n_ranks == 0, "slots must divide evenly over the ranks"
    per_rank = total // n_ranks
    replicas = np.ones(E, dtype=np.int64)
    for _ in range(n_redundant):
        replicas[int(np.argmax(load / replicas))] += 1
    items = [(load[e] / replicas[e], e) for e in range(E) for _ in range(replicas[e])]
    items.sort(key=lambda t: (-t[0], t[1]))
    slots: List[List[int]] = [[] for _ in range(n_ranks)]
    rank_load = np.zeros(n_ranks)
    for w, e in items:
        order = np.argsort(rank_load, kind="stable")
        pick = next((r for r in order if len(slots[r]) < per_rank and e not in slots[r]), None)
        if pick is None:  # every rank with room already holds e: allow a second copy there
            pick = next(r for r in order if len(slots[r]) < per_rank)
        slots[pick].append(e)
        rank_load[pick] += w
    return slots


def replica_table(slots: List[List[int]], n_experts: int):
    """expert -> list of (rank, slot) holding it."""
    tab: Dict[int, List[tuple]] = {e: [] for e in range(n_experts)}
    for r, row in enumerate(slots):
        for j, e in enumerate(row):
            tab[e].append((r, j))
    return tab


def rank_loads(slots, load):
    tab = replica_table(slots, len(load))
    out = np.zeros(len(slots))
    for e, reps in tab.items():
        for r, _ in reps:
            out[r] += load[e] / max(len(reps), 1)
    return out


@dataclass
class LayerState:
    slots: List[List[int]]
    pending: Optional[List[List[int]]] = None   # prepared, not yet active
    prepared_ranks: set = field(default_factory=set)


class EplbManager:
    """Aggregates expert loads and walks layers through prepare -> activate."""

    def __init__(self, n_layers: int, n_experts: int, n_ranks: int, n_redundant: int = 0, decay: float = 0.5,
                 min_gain: float = 0.05):
        self.L, self.E, self.R, self.red = n_layers, n_experts, n_ranks, n_redundant
        self.decay, self.min_gain = decay, min_gain
        self.load = np.zeros((n_layers, n_experts))
        base = balanced_placement(np.ones(n_experts), n_ranks, n_redundant)
        self.layers = [LayerState([list(r) for r in base]) for _ in range(n_layers)]
        self.version = 0

    # workers call this every step (or every few steps) with their local counts
    def report(self, layer: int, counts: Sequence[float]):
        self.load[layer] = self.decay * self.load[layer] + (1 - self.decay) * np.asarray(counts, dtype=np.float64)

    def imbalance(self, layer: int, slots=None) -> float:
        rl = rank_loads(slots or self.layers[layer].slots, self.load[layer])
        return float(rl.max() / rl.mean()) if rl.mean() > 0 else 1.0

    def plan(self, layer: int) -> Optional[List[List[int]]]:
        """New placement for `layer` if it lowers the max/mean rank load by at least `min_gain`."""
        st = self.layers[layer]
        if st.pending is not None or self.load[layer].sum() == 0:
            return None
        new = balanced_placement(self.load[layer], self.R, self.red)
        if self.imbalance(layer) - self.imbalance(layer, new) < self.min_gain:
            return None
        st.pending = new
        st.prepared_ranks = set()
        return new

    def moves(self, layer: int, rank: int):
        """(slot, expert) pairs whose weights `rank` has to load for the pending placement."""
        st = self.layers[layer]
        if st.pending is None:
            return []
        cur = st.slots[rank]
        return [(j, e) for j, e in enumerate(st.pending[rank]) if j >= len(cur) or cur[j] != e]

    def prepared(self, layer: int, rank: int) -> bool:
        """A rank reports its spare buffer loaded; True once every rank has: time to activate."""
        st = self.layers[layer]
        st.prepared_ranks.add(rank)
        return len(st.prepared_ranks) == self.R

    def activate(self, layer: int):
        st = self.layers[layer]
        assert st.pending is not None and len(st.prepared_ranks) == self.R
        st.slots, st.pending = st.pending, None
        st.prepared_ranks = set()
        self.version += 1
        return st.slots


class EplbExecutor:
    """Worker side: double-buffered expert weights of one layer on one rank."""

    def __init__(self, fetch_expert, n_slots: int):
        """fetch_expert(expert_id) -> weights of that logical expert (any object)."""
        self.fetch = fetch_expert
        self.active: List = [None] * n_slots
        self.spare: List = [None] * n_slots

    def prepare(self, moves, current):
        self.spare = list(current)
        for slot, e in moves:
            if slot >= len(self.spare):
                self.spare.extend([None] * (slot + 1 - len(self.spare)))
            self.spare[slot] = self.fetch(e)

    def activate(self):
        self.active, self.spare = self.spare, self.active
        return self.active
