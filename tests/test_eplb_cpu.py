"""EPLB: placement quality, replication of hot experts, and the prepare/activate state machine."""
import numpy as np

from xllm_b200.parallel.eplb import EplbExecutor, EplbManager, balanced_placement, rank_loads, replica_table


def test_placement_balances_and_replicates_hot_experts():
    rng = np.random.default_rng(0)
    load = rng.zipf(1.5, 64).astype(float)
    load[7] = load.sum()                      # one very hot expert
    slots = balanced_placement(load, 8, n_redundant=8)
    assert all(len(r) == 9 for r in slots)
    tab = replica_table(slots, 64)
    assert all(len(v) >= 1 for v in tab.values())
    assert len(tab[7]) > 1 and len({r for r, _ in tab[7]}) == len(tab[7])   # replicas on distinct ranks
    naive = [list(range(r * 8, r * 8 + 8)) for r in range(8)]
    rl_new, rl_old = rank_loads(slots, load), rank_loads(naive, load)
    assert rl_new.max() / rl_new.mean() < 0.5 * rl_old.max() / rl_old.mean()


def test_manager_state_machine():
    m = EplbManager(n_layers=2, n_experts=16, n_ranks=4, n_redundant=4, decay=0.0)
    assert m.plan(0) is None                  # no load seen yet
    counts = np.ones(16)
    counts[3] = 200
    m.report(0, counts)
    before = m.imbalance(0)
    new = m.plan(0)
    assert new is not None and m.plan(0) is None          # one pending placement at a time
    store = {}
    execs = [EplbExecutor(lambda e: ("w", e), 5) for _ in range(4)]
    for r in range(4):
        cur = [("w", e) for e in m.layers[0].slots[r]]
        execs[r].prepare(m.moves(0, r), cur)
        done = m.prepared(0, r)
        assert done == (r == 3)
    active = m.activate(0)
    assert active == new and m.version == 1 and m.imbalance(0) < before
    for r in range(4):
        assert execs[r].activate() == [("w", e) for e in new[r]]
    assert m.layers[1].pending is None        # other layers untouched
