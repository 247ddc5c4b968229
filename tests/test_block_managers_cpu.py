"""Sliding-window, composite, embedding and concurrent block managers of the C++ runtime."""
import threading

from xllm_b200 import _rt


def test_sliding_window_manager_bounds_a_sequence_and_returns_dead_blocks():
    bm = _rt.SlidingWindowBlockManager(num_blocks=8, block_size=16, window=40)
    assert bm.max_blocks_per_sequence == 4
    table = []
    peak = 0
    for n in range(1, 400):
        ok, table = bm.grow(table, n)
        assert ok
        live = [b for b in table if b > 0]
        peak = max(peak, len(live))
        assert len(table) == (n + 15) // 16
        first_needed = max(0, n - 40 + 1) // 16
        assert all(b == 0 for b in table[:first_needed]) and all(b > 0 for b in table[first_needed:])
    assert peak <= 4 and bm.num_used_blocks == len([b for b in table if b > 0])
    bm.release(table)
    assert bm.num_used_blocks == 0
    # a long prompt arriving at once only takes the blocks inside its window
    ok, t2 = bm.grow([], 300)
    assert ok and sum(b > 0 for b in t2) <= 4 and len(t2) == 19
    # the pool is finite: two more such sequences fit, a third does not (7 usable blocks)
    ok3, t3 = bm.grow([], 300)
    ok4, t4 = bm.grow([], 300)
    assert ok3 and not ok4 and t4 == []


def test_composite_manager_allocates_in_all_pools_or_none():
    cm = _rt.CompositeBlockManager()
    cm.add_pool("full", 10, 16, True)
    cm.add_pool("swa", 4, 16, False)
    assert sorted(cm.names()) == ["full", "swa"]
    a = cm.allocate({"full": 3, "swa": 2})
    assert len(a["full"]) == 3 and len(a["swa"]) == 2
    before = (cm.pool("full").num_free_blocks, cm.pool("swa").num_free_blocks)
    assert cm.allocate({"full": 2, "swa": 2}) == {}          # swa has one usable block left: nothing is taken
    assert (cm.pool("full").num_free_blocks, cm.pool("swa").num_free_blocks) == before
    assert cm.utilization > 0.6
    cm.free(a)
    assert cm.pool("full").num_used_blocks == 0 and cm.pool("swa").num_used_blocks == 0


def test_embedding_manager_counts_requests_in_flight():
    em = _rt.EmbeddingBlockManager(2)
    assert em.allocate("a") and em.allocate("b") and not em.allocate("c") and not em.allocate("a")
    assert em.num_in_flight == 2 and em.free("a") and not em.free("a") and em.allocate("c")


def test_concurrent_manager_survives_threads():
    bm = _rt.ConcurrentBlockManager(257, 16, True)
    errors = []

    def worker(seed):
        try:
            for i in range(300):
                got = bm.allocate(1 + (seed + i) % 4)
                bm.match_prefix(list(range(seed, seed + 40)))
                bm.free(got)
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    ts = [threading.Thread(target=worker, args=(s,)) for s in range(8)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errors and bm.num_used_blocks == 0 and bm.num_free_blocks == 256
